// Gated linear attention: a linear recurrence whose decay is computed for every token and key channel.
//
//     alpha_t = sigmoid(z_t)^(1/tau),  z_t = W_a2 a_t + b      (a_t: a low-rank projection of the input; heads x d)
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T       (S [d, dv] per request and head, 32-bit, zero before the first token)
//     o_t = S_t^T q_t;   out_t = o_t / sqrt(mean(o_t^2) + eps) * w * silu(g_t)      (per head over its dv elements, w [dv])
//
// The step's rows come from one product as [q: H d | k: H d | v: H dv | g: H dv | a: rank] in 32-bit.
//  * `gla_encode` multiplies q by `q_scale` in place and writes L_t = log2(alpha_t) = -softplus(-z_t) / (tau ln 2) for
//    every key channel (the small product W_a2 a_t is taken here, in 32-bit).
//  * Single tokens (`gla_single`): one CTA per (token, head) updates the state in place and forms o from it.  In a step of
//    single tokens alone it also does what `gla_encode` does, for its own token and head, with the same sums in the same
//    order: such a step has no encoding launch.
//  * Prompt portions are cut into chunks of CHUNK tokens that run side by side, in three launches; with
//    C_t = L_1 + ... + L_t inside the chunk (per channel, so every exponent below is <= 0 and nothing overflows):
//      sums    U_c = sum_j diag(2^(C_len - C_j)) k_j v_j^T of each chunk, from zero, and C_len beside it;
//      carry   along each portion: the state that each chunk starts from takes U_c's place in scratch,
//              S <- diag(2^C_len) S + U_c, and the last S goes back to the request's state;
//      output  o_t = S_in^T (q_t * 2^C_t) + sum_(j<=t) (sum_i q_t[i] k_j[i] 2^(C_t[i] - C_j[i])) v_j, then the head's norm,
//              its weight and the gate.
//    The recurrence is linear in the state, so this is the recurrence itself in another order of additions.
// Everything is 32-bit (decays, their logarithms and powers, the state, every sum); only `out` has the compute element
// type.  A row whose slot is negative belongs to nobody and is skipped.
#include "common.cuh"
#include "linear_recurrence.cuh"

namespace {
constexpr int GLA_THREADS = 256;
constexpr int GLA_MAX = 256;                  // largest head size of keys and of values

// 2^x for x <= 0 by the hardware's exponential (relative error about 2^-22, results below the smallest normal number are
// zero): for the powers inside a chunk, which multiply a term once.  What multiplies the state again and again (a single
// token's decay, a chunk's whole decay in the carry) takes exp2f, whose error has no side.
__device__ __forceinline__ float pow2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ENCODE_TOKENS tokens a CTA: a decay weight is read once for all of them (prompt portions); 1 for a few single tokens
template <typename TW, int ENCODE_TOKENS>
__global__ void gla_encode_kernel(float* __restrict__ rows, long long ld, const TW* __restrict__ w_a2,
                                  const float* __restrict__ bias, float* __restrict__ log_decay,
                                  const int* __restrict__ slots, int n_tokens, int heads, int d, int dv, int rank,
                                  float q_scale, float inv_tau) {
    extern __shared__ float encode_shared[];              // a [ENCODE_TOKENS][rank]
    pdl_launch_dependents();
    pdl_wait();
    const int first = blockIdx.x * ENCODE_TOKENS;
    const int count = min(ENCODE_TOKENS, n_tokens - first);
    for (int e = threadIdx.x; e < ENCODE_TOKENS * rank; e += blockDim.x) {
        const int t = e / rank, r = e - t * rank;
        encode_shared[e] = t < count ? rows[(size_t)(first + t) * ld + (size_t)2 * heads * (d + dv) + r] : 0.f;
    }
    __syncthreads();
    const int channels = heads * d;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const TW* w = w_a2 + (size_t)c * rank;
        float z[ENCODE_TOKENS];
        const float b = bias ? bias[c] : 0.f;
#pragma unroll
        for (int t = 0; t < ENCODE_TOKENS; ++t) z[t] = b;
        for (int r = 0; r < rank; ++r) {                 // (a token's sum runs over r in ascending order whatever else is in the batch)
            const float wr = to_float(w[r]);
#pragma unroll
            for (int t = 0; t < ENCODE_TOKENS; ++t) z[t] = fmaf(wr, encode_shared[t * rank + r], z[t]);
        }
#pragma unroll
        for (int t = 0; t < ENCODE_TOKENS; ++t) {
            if (t >= count || slots[first + t] < 0) continue;
            rows[(size_t)(first + t) * ld + c] *= q_scale;
            // log(sigmoid(z)) = -softplus(-z) = -(max(-z, 0) + log1p(exp(-|z|)))
            const float log_sigmoid = -(fmaxf(-z[t], 0.f) + log1pf(expf(-fabsf(z[t]))));
            log_decay[(size_t)(first + t) * channels + c] = log_sigmoid * inv_tau * 1.4426950408889634f;
        }
    }
}

// What `gla_encode` does for a token, done by the single-token kernel itself for its own head when `w_a2` is given
// (steps of single tokens alone then need no encoding launch): the rows are as the product left them.
struct InlineEncode {
    const void* w_a2;                // [heads d, rank], bfloat16 or 32-bit; null: the rows and log_decay are encoded already
    const float* bias;               // [heads d] or null
    int w_bf16, rank;
    float q_scale, inv_tau;
};

template <typename TO>
__global__ void __launch_bounds__(GLA_THREADS)
gla_single_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ log_decay,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ single_rows,
                  const int* __restrict__ slots, const float* __restrict__ norm_weight, TO* __restrict__ out, int heads,
                  int d, int dv, float eps, InlineEncode enc) {
    extern __shared__ float single_shared[];              // q [d], k [d], alpha [d], partial sums [max(GLA_THREADS, dv)]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = single_rows[blockIdx.x];
    const int h = blockIdx.y;
    if (t < 0) return;
    const int slot = slots[t];
    if (slot < 0) return;
    float* qs = single_shared;
    float* ks = qs + d;
    float* as = ks + d;
    float* partial = as + d;
    const float* row = rows + (size_t)t * ld;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const int c = h * d + i;
        ks[i] = row[(size_t)(heads + h) * d + i];
        if (enc.w_a2) {
            // z = W_a2 a + b over r in ascending order, as the encoding kernel sums it
            const float* a = row + (size_t)2 * heads * (d + dv);
            float z = enc.bias ? enc.bias[c] : 0.f;
            if (enc.w_bf16) {
                const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(enc.w_a2) + (size_t)c * enc.rank;
                for (int r = 0; r < enc.rank; ++r) z = fmaf(to_float(w[r]), a[r], z);
            } else {
                const float* w = reinterpret_cast<const float*>(enc.w_a2) + (size_t)c * enc.rank;
                for (int r = 0; r < enc.rank; ++r) z = fmaf(w[r], a[r], z);
            }
            const float log_sigmoid = -(fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z))));
            as[i] = exp2f(log_sigmoid * enc.inv_tau * 1.4426950408889634f);
            qs[i] = row[c] * enc.q_scale;
        } else {
            as[i] = exp2f(log_decay[(size_t)t * heads * d + c]);
            qs[i] = row[c];
        }
    }
    __syncthreads();
    const float* v = row + (size_t)2 * heads * d + (size_t)h * dv;
    const float* g = row + (size_t)2 * heads * d + (size_t)(heads + h) * dv;
    float* S = state + (size_t)slot * state_stride + (size_t)h * d * dv;
    // `lanes` threads side by side over the value's columns, `groups` of them over the key's rows
    int lanes = 32;
    while (lanes < dv && lanes < GLA_THREADS) lanes <<= 1;
    const int groups = GLA_THREADS / lanes;
    const int lane = threadIdx.x % lanes, group = threadIdx.x / lanes;
    for (int j = lane; j < dv; j += lanes) {
        const float vj = v[j];
        float acc = 0.f;
        // (eight rows of the state at a time: their loads are in flight together; the sums keep their order)
        constexpr int AHEAD = 8;
        for (int i0 = group; i0 < d; i0 += groups * AHEAD) {
            float held[AHEAD];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                const int i = i0 + k * groups;
                held[k] = i < d ? S[(size_t)i * dv + j] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                const int i = i0 + k * groups;
                if (i < d) {
                    const float s = fmaf(as[i], held[k], ks[i] * vj);
                    S[(size_t)i * dv + j] = s;
                    acc = fmaf(s, qs[i], acc);
                }
            }
        }
        if (groups > 1) partial[group * lanes + lane] = acc;       // (groups > 1 only when dv <= lanes: one j a lane)
        else partial[j] = acc;
    }
    __syncthreads();
    float sum = 0.f;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
        float o = partial[j];
        for (int gr = 1; gr < groups; ++gr) o += partial[gr * lanes + j];
        partial[j] = o;                                            // (j < dv <= lanes: only this thread touches it)
        sum = fmaf(o, o, sum);
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)dv + eps);
    TO* dst = out + (size_t)t * heads * dv + (size_t)h * dv;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
        const float z = g[j];
        dst[j] = from_float<TO>(partial[j] * inv * (norm_weight ? norm_weight[j] : 1.f) * (z / (1.0f + expf(-z))));
    }
}

// C [CHUNK][stride]: the running sums of a chunk's log2 decays, C_t = L_0 + ... + L_t per channel (rows behind `len` repeat
// the last one); a thread a channel
__device__ __forceinline__ void running_logs(float* __restrict__ C, int stride, int dp, const float* __restrict__ L,
                                             long long ld_l, int len, int d) {
    for (int i = threadIdx.x; i < stride; i += blockDim.x) {
        float sum = 0.f;
        constexpr int AHEAD = 8;                            // (eight of a channel's loads are in flight together)
        for (int t0 = 0; t0 < CHUNK; t0 += AHEAD) {
            float held[AHEAD];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) held[k] = (t0 + k < len && i < d) ? L[(size_t)(t0 + k) * ld_l + i] : 0.f;
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                sum += held[k];
                C[(t0 + k) * stride + i] = sum;
            }
        }
    }
}

// U [chunk, head, d, dv] = sum_j diag(2^(C_len - C_j)) k_j v_j^T;  totals [chunk, head, d] = C_len
__global__ void __launch_bounds__(GLA_THREADS)
gla_sums_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ log_decay,
                const int* __restrict__ segments, int n_segments, float* __restrict__ sums, float* __restrict__ totals,
                int heads, int d, int dv, int vec) {
    extern __shared__ float sums_shared[];                // k [CHUNK][dp] weighted, v [CHUNK][dvp], C [CHUNK][dp]
    pdl_launch_dependents();
    pdl_wait();
    int first, len, segment, chunk;
    if (!find_chunk(segments, n_segments, blockIdx.x, &first, &len, &segment, &chunk)) return;
    const int h = blockIdx.y;
    const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
    float* ks = sums_shared;
    float* vs = ks + CHUNK * dp;
    float* C = vs + CHUNK * dvp;
    const float* chunk_rows = rows + (size_t)first * ld;
    load_chunk(ks, dp, chunk_rows + (size_t)(heads + h) * d, ld, len, d, vec, false, 0.f);
    load_chunk(vs, dvp, chunk_rows + (size_t)2 * heads * d + (size_t)h * dv, ld, len, dv, vec, false, 0.f);
    running_logs(C, dp, dp, log_decay + (size_t)first * heads * d + (size_t)h * d, (long long)heads * d, len, d);
    __syncthreads();
    for (int e = threadIdx.x; e < len * dp; e += blockDim.x) {
        const int t = e / dp, i = e - t * dp;
        ks[e] *= pow2(C[(len - 1) * dp + i] - C[t * dp + i]);
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) totals[((size_t)blockIdx.x * heads + h) * d + i] = C[(len - 1) * dp + i];
    __syncthreads();
    float* U = sums + ((size_t)blockIdx.x * heads + h) * d * dv;
    const int tiles_j = dvp / 4, tiles = (dp / 4) * tiles_j;
    for (int tile = threadIdx.x; tile < tiles; tile += blockDim.x) {
        const int i0 = (tile / tiles_j) * 4, j0 = (tile % tiles_j) * 4;
        float acc[4][4] = {};
        for (int t = 0; t < len; ++t) {
            const float4 a = *reinterpret_cast<const float4*>(ks + t * dp + i0);
            const float4 b = *reinterpret_cast<const float4*>(vs + t * dvp + j0);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y)
                if (i0 + x < d && j0 + y < dv) U[(size_t)(i0 + x) * dv + j0 + y] = acc[x][y];
    }
}

// along each portion: scratch[c] <- the state chunk c starts from; S <- diag(2^C_len) S + U_c; state <- the last S
__global__ void __launch_bounds__(GLA_THREADS)
gla_carry_kernel(const int* __restrict__ segments, int n_segments, const int* __restrict__ slots, float* __restrict__ sums,
                 const float* __restrict__ totals, float* __restrict__ state, long long state_stride, int heads, int d,
                 int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    if (s >= n_segments) return;
    const int first = segments[3 * s], count = segments[3 * s + 2];
    const int slot = slots[first];
    if (slot < 0) return;
    int before = 0;
    for (int p = 0; p < s; ++p) before += (segments[3 * p + 2] + CHUNK - 1) / CHUNK;
    const int chunks = (count + CHUNK - 1) / CHUNK;
    const int size = d * dv;
    float* S = state + (size_t)slot * state_stride + (size_t)h * size;
    const size_t chunk_stride = (size_t)heads * size;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < size; e += gridDim.z * blockDim.x) {
        const int i = e / dv;
        float value = S[e];
        float* U = sums + ((size_t)before * heads + h) * size + e;
        const float* total = totals + ((size_t)before * heads + h) * d + i;
        // (a thread walks its element's chunks eight at a time: the loads are in flight together)
        constexpr int AHEAD = 8;
        for (int c0 = 0; c0 < chunks; c0 += AHEAD) {
            float u[AHEAD], a[AHEAD];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                u[k] = c0 + k < chunks ? U[(size_t)(c0 + k) * chunk_stride] : 0.f;
                a[k] = c0 + k < chunks ? total[(size_t)(c0 + k) * heads * d] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < AHEAD; ++k)
                if (c0 + k < chunks) {
                    U[(size_t)(c0 + k) * chunk_stride] = value;
                    value = fmaf(exp2f(a[k]), value, u[k]);
                }
        }
        S[e] = value;
    }
}

template <typename TO>
__global__ void __launch_bounds__(GLA_THREADS, 3)
gla_output_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ log_decay,
                  const int* __restrict__ segments, int n_segments, const float* __restrict__ sums,
                  const float* __restrict__ norm_weight, TO* __restrict__ out, int heads, int d, int dv, float eps, int vec) {
    // q [CHUNK][ds], k [CHUNK][ds], C [CHUNK][ds], v [CHUNK][dvp], A [CHUNK][CHUNK], o [CHUNK][dvp]; ds = dp + 4: rows four
    // floats apart from a multiple of 32, so that 32 lanes reading four floats each of 32 different rows meet no bank twice
    extern __shared__ float out_shared[];
    pdl_launch_dependents();
    pdl_wait();
    int first, len, segment, chunk;
    if (!find_chunk(segments, n_segments, blockIdx.x, &first, &len, &segment, &chunk)) return;
    const int h = blockIdx.y;
    const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3, ds = dp + 4;
    float* qs = out_shared;
    float* ks = qs + CHUNK * ds;
    float* C = ks + CHUNK * ds;
    float* vs = C + CHUNK * ds;
    float* A = vs + CHUNK * dvp;
    // (the outputs take the keys' room where they fit: the keys are done with once A is made)
    float* os = dvp <= ds ? ks : A + CHUNK * CHUNK;
    const float* chunk_rows = rows + (size_t)first * ld;
    load_chunk(qs, ds, chunk_rows + (size_t)h * d, ld, len, d, vec, false, 0.f);
    load_chunk(ks, ds, chunk_rows + (size_t)(heads + h) * d, ld, len, d, vec, false, 0.f);
    load_chunk(vs, dvp, chunk_rows + (size_t)2 * heads * d + (size_t)h * dv, ld, len, dv, vec, false, 0.f);
    running_logs(C, ds, dp, log_decay + (size_t)first * heads * d + (size_t)h * d, (long long)heads * d, len, d);
    __syncthreads();
    // A[t][j] = sum_i q_t[i] k_j[i] 2^(C_t[i] - C_j[i]) for j <= t: a thread a pair, a warp one key j and 32 queries t
    // (the key's row is read by all lanes at once, the queries' rows are `ds` apart), four channels at a time
    for (int e = threadIdx.x; e < CHUNK * CHUNK; e += blockDim.x) {
        const int j = e / CHUNK, t = e - j * CHUNK;
        float acc = 0.f;
        if (j <= t && t < len) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + t * ds);
            const float4* ct4 = reinterpret_cast<const float4*>(C + t * ds);
            const float4* k4 = reinterpret_cast<const float4*>(ks + j * ds);
            const float4* cj4 = reinterpret_cast<const float4*>(C + j * ds);
            for (int i = 0; i < dp / 4; ++i) {
                const float4 q = q4[i], ct = ct4[i], k = k4[i], cj = cj4[i];
                acc = fmaf(q.x * k.x, pow2(ct.x - cj.x), acc);
                acc = fmaf(q.y * k.y, pow2(ct.y - cj.y), acc);
                acc = fmaf(q.z * k.z, pow2(ct.z - cj.z), acc);
                acc = fmaf(q.w * k.w, pow2(ct.w - cj.w), acc);
            }
        }
        A[t * CHUNK + j] = acc;
    }
    __syncthreads();
    // the queries take their decay from the chunk's start: q_t * 2^C_t
    for (int e = threadIdx.x; e < CHUNK * ds; e += blockDim.x) qs[e] *= pow2(C[e]);
    __syncthreads();
    // o[t][j] = sum_i (q_t 2^C_t)[i] S_in[i][j] + sum_j' A[t][j'] v_j'[j]: a thread owns four tokens and four columns
    const float* S = sums + ((size_t)blockIdx.x * heads + h) * d * dv;
    const int tiles_j = dvp / 4, tiles = (CHUNK / 4) * tiles_j;
    for (int tile = threadIdx.x; tile < tiles; tile += blockDim.x) {
        const int t0 = (tile / tiles_j) * 4, j0 = (tile % tiles_j) * 4;
        float acc[4][4] = {};
        const bool aligned = (dv & 3) == 0 && vec;
#pragma unroll 8
        for (int i = 0; i < d; ++i) {
            float bv[4];
            if (aligned) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(S + (size_t)i * dv + j0));
                bv[0] = b.x, bv[1] = b.y, bv[2] = b.z, bv[3] = b.w;
            } else {
#pragma unroll
                for (int y = 0; y < 4; ++y) bv[y] = j0 + y < dv ? __ldg(S + (size_t)i * dv + j0 + y) : 0.f;
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float a = qs[(t0 + x) * ds + i];
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(a, bv[y], acc[x][y]);
            }
        }
        for (int jj = 0; jj < len; ++jj) {
            const float4 b = *reinterpret_cast<const float4*>(vs + jj * dvp + j0);
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float w = A[(t0 + x) * CHUNK + jj];
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(w, bv[y], acc[x][y]);
            }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) os[(t0 + x) * dvp + j0 + y] = acc[x][y];
    }
    __syncthreads();
    // the head's norm over its dv elements, its weight and the gate: a warp a token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < len; t += GLA_THREADS / 32) {
        float sum = 0.f;
        for (int j = lane; j < dv; j += 32) sum = fmaf(os[t * dvp + j], os[t * dvp + j], sum);
        sum = warp_sum(sum);
        const float inv = 1.0f / sqrtf(sum / (float)dv + eps);
        const float* g = rows + (size_t)(first + t) * ld + (size_t)2 * heads * d + (size_t)(heads + h) * dv;
        TO* dst = out + (size_t)(first + t) * heads * dv + (size_t)h * dv;
        for (int j = lane; j < dv; j += 32) {
            const float z = g[j];
            dst[j] = from_float<TO>(os[t * dvp + j] * inv * (norm_weight ? norm_weight[j] : 1.f) * (z / (1.0f + expf(-z))));
        }
    }
}

size_t gla_output_shared_bytes(int d, int dv) {
    const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
    return ((size_t)3 * CHUNK * (dp + 4) + (size_t)(dvp <= dp + 4 ? 1 : 2) * CHUNK * dvp + CHUNK * CHUNK) * sizeof(float);
}
}  // namespace

// Words of 32-bit scratch for `chunks` chunks (the chunks' sums and, behind them, their summed log decays).
LIA_EXPORT long long lia_gla_scratch_floats(int chunks, int heads, int d, int dv) {
    return (long long)chunks * heads * d * (dv + 1);
}

// rows [n, ld] 32-bit, [q | k | v | g | a] with a [rank] behind the 2 heads (d + dv) elements ahead of it: q is multiplied
// by q_scale in place; log_decay [n, heads d] 32-bit receives log2(sigmoid(W_a2 a + bias)) / tau.  w_a2 [heads d, rank]
// of `w_dtype`, bias [heads d] 32-bit or null.
LIA_EXPORT int lia_gla_encode(float* rows, long long ld, const void* w_a2, int w_dtype, const float* bias, float* log_decay,
                              const int* slots, int n_tokens, int heads, int d, int dv, int rank, float q_scale, float tau,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || rank <= 0 || rank > 8192 || !(tau > 0.f) ||
        ld < (long long)2 * heads * (d + dv) + rank)
        return LIA_ERR_SIZE;
    const int per_cta = n_tokens >= 1024 ? 8 : 1;
    const size_t bytes = (size_t)per_cta * rank * sizeof(float);
    const dim3 grid((n_tokens + per_cta - 1) / per_cta);
#define LIA_ENCODE(TW, TOKENS)                                                                                     \
    return lia_launch(gla_encode_kernel<TW, TOKENS>, grid, dim3(256), bytes, stream, rows, ld, (const TW*)w_a2, bias, \
                      log_decay, slots, n_tokens, heads, d, dv, rank, q_scale, 1.0f / tau)
    if (w_dtype == LIA_BF16) {
        if (per_cta == 8) LIA_ENCODE(__nv_bfloat16, 8);
        LIA_ENCODE(__nv_bfloat16, 1);
    }
    if (w_dtype == LIA_F32) {
        if (per_cta == 8) LIA_ENCODE(float, 8);
        LIA_ENCODE(float, 1);
    }
#undef LIA_ENCODE
    return LIA_ERR_DTYPE;
}

// The step's runs: `segments` [n_segments, 3] int32 (first batch index, first position, count) are the portions of
// several tokens, `single_rows` [n_single] the batch indices of the single tokens.  rows [n, ld] 32-bit and log_decay
// [n, heads d] as `gla_encode` left them; norm_weight [dv] 32-bit or null; state [slots, heads, d, dv] 32-bit with slot
// stride `state_stride`; out [n, heads dv] of `out_dtype`; scratch: `lia_gla_scratch_floats(max_chunks, ...)` words.
// With `w_a2` (a step of single tokens alone) the rows are as the product left them and `log_decay` is not read: the
// kernel encodes each token's head itself (w_a2, bias, rank, q_scale, tau as for `lia_gla_encode`).
LIA_EXPORT int lia_gla(const float* rows, long long ld, const float* log_decay, float* state, long long state_stride,
                       const int* segments, int n_segments, int max_chunks, const int* single_rows, int n_single,
                       const int* slots, const float* norm_weight, void* out, int out_dtype, int heads, int d, int dv,
                       float eps, float* scratch, long long scratch_floats, const void* w_a2, int w_dtype, const float* bias,
                       int rank, float q_scale, float tau, cudaStream_t stream) {
    if (heads <= 0 || d <= 0 || dv <= 0 || d > GLA_MAX || dv > GLA_MAX || ld < (long long)2 * heads * (d + dv) ||
        state_stride < (long long)heads * d * dv)
        return LIA_ERR_SIZE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    InlineEncode enc = {};
    if (w_a2) {
        // the single tokens' rows are not encoded yet: only a step without portions may ask for that
        if (n_segments > 0 || rank <= 0 || !(tau > 0.f) || ld < (long long)2 * heads * (d + dv) + rank) return LIA_ERR_SIZE;
        if (w_dtype != LIA_F32 && w_dtype != LIA_BF16) return LIA_ERR_DTYPE;
        enc.w_a2 = w_a2; enc.bias = bias; enc.w_bf16 = w_dtype == LIA_BF16; enc.rank = rank; enc.q_scale = q_scale;
        enc.inv_tau = 1.0f / tau;
    } else if (!log_decay) {
        return LIA_ERR_SIZE;
    }
    int code = LIA_OK;
    if (n_segments > 0) {
        if (max_chunks <= 0 || !scratch || scratch_floats < lia_gla_scratch_floats(max_chunks, heads, d, dv))
            return LIA_ERR_SIZE;
        float* totals = scratch + (size_t)max_chunks * heads * d * dv;
        const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
        const int vec = ((d | dv) & 3) == 0 && (ld & 3) == 0 && (((uintptr_t)rows | (uintptr_t)scratch) & 15u) == 0 ? 1 : 0;
        const size_t sums_bytes = (size_t)CHUNK * (2 * dp + dvp) * sizeof(float);
        const size_t out_bytes = gla_output_shared_bytes(d, dv);
        static bool raised = false;
        if (!raised) {
            cudaFuncSetAttribute(gla_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            cudaFuncSetAttribute(gla_output_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            cudaFuncSetAttribute(gla_output_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            raised = true;
        }
        code = lia_launch(gla_sums_kernel, dim3(max_chunks, heads), dim3(GLA_THREADS), sums_bytes, stream, rows, ld, log_decay,
                          segments, n_segments, scratch, totals, heads, d, dv, vec);
        if (code != LIA_OK) return code;
        const int parts = (d * dv + GLA_THREADS - 1) / GLA_THREADS;          // one element a thread
        code = lia_launch(gla_carry_kernel, dim3(n_segments, heads, parts), dim3(GLA_THREADS), 0, stream, segments,
                          n_segments, slots, scratch, (const float*)totals, state, state_stride, heads, d, dv);
        if (code != LIA_OK) return code;
        if (out_dtype == LIA_F32)
            code = lia_launch(gla_output_kernel<float>, dim3(max_chunks, heads), dim3(GLA_THREADS), out_bytes, stream, rows,
                              ld, log_decay, segments, n_segments, (const float*)scratch, norm_weight, (float*)out, heads, d,
                              dv, eps, vec);
        else
            code = lia_launch(gla_output_kernel<__nv_bfloat16>, dim3(max_chunks, heads), dim3(GLA_THREADS), out_bytes, stream,
                              rows, ld, log_decay, segments, n_segments, (const float*)scratch, norm_weight,
                              (__nv_bfloat16*)out, heads, d, dv, eps, vec);
        if (code != LIA_OK) return code;
    }
    if (n_single > 0) {
        const size_t bytes = ((size_t)3 * d + (dv > GLA_THREADS ? dv : GLA_THREADS)) * sizeof(float);
        if (out_dtype == LIA_F32)
            code = lia_launch(gla_single_kernel<float>, dim3(n_single, heads), dim3(GLA_THREADS), bytes, stream, rows, ld,
                              log_decay, state, state_stride, single_rows, slots, norm_weight, (float*)out, heads, d, dv, eps, enc);
        else
            code = lia_launch(gla_single_kernel<__nv_bfloat16>, dim3(n_single, heads), dim3(GLA_THREADS), bytes, stream, rows,
                              ld, log_decay, state, state_stride, single_rows, slots, norm_weight, (__nv_bfloat16*)out, heads,
                              d, dv, eps, enc);
    }
    return code;
}
