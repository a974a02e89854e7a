// Retention: linear attention with one fixed decay per head, no softmax and no denominator.
//
//     S_t = decay_h S_(t-1) + k_t v_t^T        (S [d, dv] per request and head, 32-bit, zero before the first token)
//     o_t = S_t^T q_t;   out_t = o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)      (per head, over its dv elements)
//
// The step's rows come from one product as [q: H d | k: H d | v: H dv | g: H dv] in 32-bit.
//  * `retention_encode` rotates q and k in place (element i of a head with i + rot_dims/2 over the first rot_dims
//    elements, angle float(position) * freq[i]) and multiplies k by d^(-1/2) after the rotation.
//  * Single tokens (`retention_single`): one CTA per (token, head) updates the state in place and forms o from it.
//  * Prompt portions are cut into chunks of CHUNK tokens that run side by side, in three launches:
//      sums    U_c = sum_j decay^(len-1-j) k_j v_j^T of each chunk, from zero;
//      carry   along each portion: the state that each chunk starts from takes U_c's place in scratch,
//              S <- decay^len S + U_c, and the last S goes back to the request's state;
//      output  o_t = decay^(t+1) S_in^T q_t + sum_(j<=t) decay^(t-j) (q_t . k_j) v_j  (t counted inside the chunk), then
//              the head's norm and the gate.
//    The recurrence is linear in the state, so this is the recurrence itself in another order of additions.
// Everything is 32-bit (decays, their powers, the state, every sum); only `out` has the compute element type.  A row whose
// slot is negative belongs to nobody and is skipped.
#include "common.cuh"
#include "linear_recurrence.cuh"

namespace {
constexpr int RET_THREADS = 256;
constexpr int RET_MAX = 256;                  // largest head size of keys and of values

__global__ void retention_encode_kernel(float* __restrict__ rows, long long ld, const float* __restrict__ freq,
                                        int rot_dims, const int* __restrict__ positions, const int* __restrict__ slots,
                                        int n_tokens, int heads, int d, float k_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens || slots[t] < 0) return;
    const float pos = (float)positions[t];
    float* q = rows + (size_t)t * ld;
    float* k = q + (size_t)heads * d;
    const int half = rot_dims / 2;
    const int plain = d - rot_dims;
    // the rotated pairs of q and k
    for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        float s, c;
        sincosf(pos * freq[i], &s, &c);
        float* qh = q + (size_t)h * d;
        float* kh = k + (size_t)h * d;
        const float qu = qh[i], qv = qh[half + i], ku = kh[i], kv = kh[half + i];
        qh[i] = qu * c - qv * s;
        qh[half + i] = qv * c + qu * s;
        kh[i] = (ku * c - kv * s) * k_scale;
        kh[half + i] = (kv * c + ku * s) * k_scale;
    }
    // the elements of k that pass unrotated are scaled too
    for (int e = threadIdx.x; e < heads * plain; e += blockDim.x) {
        const int h = e / plain, i = rot_dims + (e - h * plain);
        k[(size_t)h * d + i] *= k_scale;
    }
}

template <typename TO>
__global__ void __launch_bounds__(RET_THREADS)
retention_single_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ decay,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ single_rows,
                        const int* __restrict__ slots, TO* __restrict__ out, int heads, int d, int dv, float eps) {
    extern __shared__ float single_shared[];              // q [d], k [d], partial sums [max(RET_THREADS, dv)]
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
    float* partial = ks + d;
    const float* row = rows + (size_t)t * ld;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        qs[i] = row[(size_t)h * d + i];
        ks[i] = row[(size_t)(heads + h) * d + i];
    }
    __syncthreads();
    const float* v = row + (size_t)2 * heads * d + (size_t)h * dv;
    const float* g = row + (size_t)2 * heads * d + (size_t)(heads + h) * dv;
    float* S = state + (size_t)slot * state_stride + (size_t)h * d * dv;
    const float a = decay[h];
    // `lanes` threads side by side over the value's columns, `groups` of them over the key's rows
    int lanes = 32;
    while (lanes < dv && lanes < RET_THREADS) lanes <<= 1;
    const int groups = RET_THREADS / lanes;
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
                    const float s = fmaf(a, held[k], ks[i] * vj);
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
        dst[j] = from_float<TO>(partial[j] * inv * (z / (1.0f + expf(-z))));
    }
}

// U [chunk, head, d, dv] = sum_j decay^(len-1-j) k_j v_j^T
__global__ void __launch_bounds__(RET_THREADS)
retention_sums_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ decay,
                      const int* __restrict__ segments, int n_segments, float* __restrict__ sums, int heads, int d, int dv,
                      int vec) {
    extern __shared__ float sums_shared[];                // k [CHUNK][dp] weighted, v [CHUNK][dvp]
    pdl_launch_dependents();
    pdl_wait();
    int first, len, segment, chunk;
    if (!find_chunk(segments, n_segments, blockIdx.x, &first, &len, &segment, &chunk)) return;
    const int h = blockIdx.y;
    const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
    float* ks = sums_shared;
    float* vs = ks + CHUNK * dp;
    const float log_a = log2f(decay[h]);
    const float* chunk_rows = rows + (size_t)first * ld;
    load_chunk(ks, dp, chunk_rows + (size_t)(heads + h) * d, ld, len, d, vec, true, log_a);
    load_chunk(vs, dvp, chunk_rows + (size_t)2 * heads * d + (size_t)h * dv, ld, len, dv, vec, false, 0.f);
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
        if (vec) {                                          // (d and dv multiples of four: whole rows of four)
#pragma unroll
            for (int x = 0; x < 4; ++x)
                *reinterpret_cast<float4*>(U + (size_t)(i0 + x) * dv + j0) = make_float4(acc[x][0], acc[x][1], acc[x][2], acc[x][3]);
            continue;
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y)
                if (i0 + x < d && j0 + y < dv) U[(size_t)(i0 + x) * dv + j0 + y] = acc[x][y];
    }
}

// along each portion: scratch[c] <- the state chunk c starts from; S <- decay^len S + U_c; state <- the last S
__global__ void __launch_bounds__(RET_THREADS)
retention_carry_kernel(const float* __restrict__ decay, const int* __restrict__ segments, int n_segments,
                       const int* __restrict__ slots, float* __restrict__ sums, float* __restrict__ state,
                       long long state_stride, int heads, int d, int dv) {
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
    const float log_a = log2f(decay[h]);
    const float full = exp2f((float)CHUNK * log_a);
    const float last = exp2f((float)(count - (chunks - 1) * CHUNK) * log_a);
    const int size = d * dv;
    float* S = state + (size_t)slot * state_stride + (size_t)h * size;
    // (a thread walks its element's chunks eight at a time: the eight loads are in flight together)
    constexpr int AHEAD = 8;
    const size_t chunk_stride = (size_t)heads * size;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < size; e += gridDim.z * blockDim.x) {
        float value = S[e];
        float* U = sums + ((size_t)before * heads + h) * size + e;
        for (int c0 = 0; c0 < chunks; c0 += AHEAD) {
            float u[AHEAD];
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) u[k] = c0 + k < chunks ? U[(size_t)(c0 + k) * chunk_stride] : 0.f;
#pragma unroll
            for (int k = 0; k < AHEAD; ++k)
                if (c0 + k < chunks) {
                    U[(size_t)(c0 + k) * chunk_stride] = value;
                    value = fmaf(c0 + k + 1 < chunks ? full : last, value, u[k]);
                }
        }
        S[e] = value;
    }
}

template <typename TO>
__global__ void __launch_bounds__(RET_THREADS)
retention_output_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ decay,
                        const int* __restrict__ segments, int n_segments, const float* __restrict__ sums,
                        TO* __restrict__ out, int heads, int d, int dv, float eps, int vec) {
    extern __shared__ float out_shared[];  // qT [dp][CHUNK] (decayed), k [CHUNK][dp], v [CHUNK][dvp], A [CHUNK][CHUNK], o [CHUNK][dvp], powers [CHUNK + 1]
    pdl_launch_dependents();
    pdl_wait();
    int first, len, segment, chunk;
    if (!find_chunk(segments, n_segments, blockIdx.x, &first, &len, &segment, &chunk)) return;
    const int h = blockIdx.y;
    const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
    float* qT = out_shared;
    float* ks = qT + dp * CHUNK;
    float* vs = ks + CHUNK * dp;
    float* A = vs + CHUNK * dvp;
    float* os = A + CHUNK * CHUNK;
    float* powers = os + CHUNK * dvp;
    const float log_a = log2f(decay[h]);
    for (int i = threadIdx.x; i <= CHUNK; i += blockDim.x) powers[i] = exp2f((float)i * log_a);
    const float* chunk_rows = rows + (size_t)first * ld;
    if (vec) {
        // the queries transposed: a lane a token (its stores fall into 32 banks), a warp four elements of the head
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 4
        for (int i0 = 4 * warp; i0 < d; i0 += 4 * (RET_THREADS / 32)) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (lane < len) v = *reinterpret_cast<const float4*>(chunk_rows + (size_t)lane * ld + (size_t)h * d + i0);
            qT[(i0 + 0) * CHUNK + lane] = v.x;
            qT[(i0 + 1) * CHUNK + lane] = v.y;
            qT[(i0 + 2) * CHUNK + lane] = v.z;
            qT[(i0 + 3) * CHUNK + lane] = v.w;
        }
    } else {
        for (int e = threadIdx.x; e < CHUNK * dp; e += blockDim.x) {
            const int t = e / dp, i = e - t * dp;
            qT[i * CHUNK + t] = (t < len && i < d) ? chunk_rows[(size_t)t * ld + (size_t)h * d + i] : 0.f;
        }
    }
    load_chunk(ks, dp, chunk_rows + (size_t)(heads + h) * d, ld, len, d, vec, false, 0.f);
    load_chunk(vs, dvp, chunk_rows + (size_t)2 * heads * d + (size_t)h * dv, ld, len, dv, vec, false, 0.f);
    __syncthreads();
    // A[t][j] = decay^(t-j) q_t . k_j for j <= t
    for (int e = threadIdx.x; e < CHUNK * CHUNK; e += blockDim.x) {
        const int j = e / CHUNK, t = e - j * CHUNK;          // a warp shares the key and reads neighbouring queries
        float acc = 0.f;
        if (j <= t && t < len) {
            for (int i = 0; i < d; ++i) acc = fmaf(qT[i * CHUNK + t], ks[j * dp + i], acc);
            acc *= powers[t - j];
        }
        A[t * CHUNK + j] = acc;
    }
    __syncthreads();
    // o[t][j] = decay^(t+1) sum_i q_t[i] S_in[i][j] + sum_j' A[t][j'] v_j'[j]: a thread owns four tokens and four columns
    const float* S = sums + ((size_t)blockIdx.x * heads + h) * d * dv;
    const int tiles_j = dvp / 4, tiles = (CHUNK / 4) * tiles_j;
    const bool aligned = (dv & 3) == 0;
    // When every thread has at most one tile, the incoming state goes through shared memory CHUNK rows at a time (in the
    // room of `os`, which is written only afterwards): every warp reads all of it, and the SM's L1 does not hold it.
    const bool staged = tiles <= (int)blockDim.x;
    for (int tile = threadIdx.x; tile < (staged ? (int)blockDim.x : tiles); tile += blockDim.x) {
        const bool active = tile < tiles;
        const int t0 = active ? (tile / tiles_j) * 4 : 0, j0 = active ? (tile % tiles_j) * 4 : 0;
        float acc[4][4] = {};
        if (staged) {
            for (int i0 = 0; i0 < d; i0 += CHUNK) {
                const int rows_now = min(CHUNK, d - i0);
                if (aligned) {
                    const int w4 = dv / 4;
#pragma unroll 4
                    for (int e = threadIdx.x; e < rows_now * w4; e += blockDim.x) {
                        const int r = e / w4, c4 = e - r * w4;
                        *reinterpret_cast<float4*>(os + r * dvp + 4 * c4) =
                            __ldg(reinterpret_cast<const float4*>(S + (size_t)(i0 + r) * dv + 4 * c4));
                    }
                } else {
                    for (int e = threadIdx.x; e < rows_now * dvp; e += blockDim.x) {
                        const int r = e / dvp, c = e - r * dvp;
                        os[e] = c < dv ? S[(size_t)(i0 + r) * dv + c] : 0.f;
                    }
                }
                __syncthreads();
                if (active) {
#pragma unroll 8
                    for (int ii = 0; ii < rows_now; ++ii) {
                        const float4 a = *reinterpret_cast<const float4*>(qT + (i0 + ii) * CHUNK + t0);
                        const float4 b = *reinterpret_cast<const float4*>(os + ii * dvp + j0);
                        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                        for (int x = 0; x < 4; ++x)
#pragma unroll
                            for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
                    }
                }
                __syncthreads();
            }
            if (!active) continue;
        } else {
#pragma unroll 8
            for (int i = 0; i < d; ++i) {
                const float4 a = *reinterpret_cast<const float4*>(qT + i * CHUNK + t0);
                float bv[4];
                if (aligned) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(S + (size_t)i * dv + j0));
                    bv[0] = b.x, bv[1] = b.y, bv[2] = b.z, bv[3] = b.w;
                } else {
#pragma unroll
                    for (int y = 0; y < 4; ++y) bv[y] = j0 + y < dv ? S[(size_t)i * dv + j0 + y] : 0.f;
                }
                const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
            }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) acc[x][y] *= powers[t0 + x + 1];
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
    // the head's norm over its dv elements and the gate: a warp a token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < len; t += RET_THREADS / 32) {
        float sum = 0.f;
        for (int j = lane; j < dv; j += 32) sum = fmaf(os[t * dvp + j], os[t * dvp + j], sum);
        sum = warp_sum(sum);
        const float inv = 1.0f / sqrtf(sum / (float)dv + eps);
        const float* g = rows + (size_t)(first + t) * ld + (size_t)2 * heads * d + (size_t)(heads + h) * dv;
        TO* dst = out + (size_t)(first + t) * heads * dv + (size_t)h * dv;
        for (int j = lane; j < dv; j += 32) {
            const float z = g[j];
            dst[j] = from_float<TO>(os[t * dvp + j] * inv * (z / (1.0f + expf(-z))));
        }
    }
}

size_t output_shared_bytes(int d, int dv) {
    const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
    return ((size_t)2 * CHUNK * dp + (size_t)2 * CHUNK * dvp + CHUNK * CHUNK + CHUNK + 1) * sizeof(float);
}
}  // namespace

// Most chunks that the portions of a step with `portion_tokens` tokens in `n_segments` portions are cut into.
LIA_EXPORT int lia_retention_chunks(int portion_tokens, int n_segments) {
    return n_segments > 0 ? portion_tokens / CHUNK + n_segments : 0;
}

// Words of 32-bit scratch for `chunks` chunks.
LIA_EXPORT long long lia_retention_scratch_floats(int chunks, int heads, int d, int dv) {
    return (long long)chunks * heads * d * dv;
}

// rows [n, ld] 32-bit: q and k (heads x d each) are rotated and k scaled in place.
LIA_EXPORT int lia_retention_encode(float* rows, long long ld, const float* freq, int rot_dims, const int* positions,
                                    const int* slots, int n_tokens, int heads, int d, float k_scale, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (heads <= 0 || d <= 0 || rot_dims < 0 || rot_dims > d || (rot_dims & 1) || (rot_dims > 0 && !freq) ||
        ld < (long long)2 * heads * d)
        return LIA_ERR_SIZE;
    return lia_launch(retention_encode_kernel, dim3(n_tokens), dim3(128), 0, stream, rows, ld, freq, rot_dims, positions,
                      slots, n_tokens, heads, d, k_scale);
}

// The step's runs: `segments` [n_segments, 3] int32 (first batch index, first position, count) are the portions of
// several tokens, `single_rows` [n_single] the batch indices of the single tokens.  rows [n, ld] 32-bit as
// `retention_encode` left them; decay [heads] 32-bit; state [slots, heads, d, dv] 32-bit with slot stride
// `state_stride`; out [n, heads dv] of `out_dtype`; scratch: `lia_retention_scratch_floats(max_chunks, ...)` words.
LIA_EXPORT int lia_retention(const float* rows, long long ld, const float* decay, float* state, long long state_stride,
                             const int* segments, int n_segments, int max_chunks, const int* single_rows, int n_single,
                             const int* slots, void* out, int out_dtype, int heads, int d, int dv, float eps,
                             float* scratch, long long scratch_floats, cudaStream_t stream) {
    if (heads <= 0 || d <= 0 || dv <= 0 || d > RET_MAX || dv > RET_MAX || ld < (long long)2 * heads * (d + dv) ||
        state_stride < (long long)heads * d * dv)
        return LIA_ERR_SIZE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    int code = LIA_OK;
    if (n_segments > 0) {
        if (max_chunks <= 0 || !scratch || scratch_floats < lia_retention_scratch_floats(max_chunks, heads, d, dv))
            return LIA_ERR_SIZE;
        const int dp = (d + 3) & ~3, dvp = (dv + 3) & ~3;
        const int vec = ((d | dv) & 3) == 0 && (ld & 3) == 0 && (((uintptr_t)rows | (uintptr_t)scratch) & 15u) == 0 ? 1 : 0;
        const size_t sums_bytes = (size_t)CHUNK * (dp + dvp) * sizeof(float);
        const size_t out_bytes = output_shared_bytes(d, dv);
        static bool raised = false;
        if (!raised) {
            cudaFuncSetAttribute(retention_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            cudaFuncSetAttribute(retention_output_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            cudaFuncSetAttribute(retention_output_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            raised = true;
        }
        code = lia_launch(retention_sums_kernel, dim3(max_chunks, heads), dim3(RET_THREADS), sums_bytes, stream, rows, ld,
                          decay, segments, n_segments, scratch, heads, d, dv, vec);
        if (code != LIA_OK) return code;
        const int parts = (d * dv + RET_THREADS - 1) / RET_THREADS;          // one element a thread
        code = lia_launch(retention_carry_kernel, dim3(n_segments, heads, parts), dim3(RET_THREADS), 0, stream, decay,
                          segments, n_segments, slots, scratch, state, state_stride, heads, d, dv);
        if (code != LIA_OK) return code;
        if (out_dtype == LIA_F32)
            code = lia_launch(retention_output_kernel<float>, dim3(max_chunks, heads), dim3(RET_THREADS), out_bytes, stream,
                              rows, ld, decay, segments, n_segments, (const float*)scratch, (float*)out, heads, d, dv, eps, vec);
        else
            code = lia_launch(retention_output_kernel<__nv_bfloat16>, dim3(max_chunks, heads), dim3(RET_THREADS), out_bytes,
                              stream, rows, ld, decay, segments, n_segments, (const float*)scratch, (__nv_bfloat16*)out,
                              heads, d, dv, eps, vec);
        if (code != LIA_OK) return code;
    }
    if (n_single > 0) {
        const size_t bytes = ((size_t)2 * d + (dv > RET_THREADS ? dv : RET_THREADS)) * sizeof(float);
        if (out_dtype == LIA_F32)
            code = lia_launch(retention_single_kernel<float>, dim3(n_single, heads), dim3(RET_THREADS), bytes, stream, rows,
                              ld, decay, state, state_stride, single_rows, slots, (float*)out, heads, d, dv, eps);
        else
            code = lia_launch(retention_single_kernel<__nv_bfloat16>, dim3(n_single, heads), dim3(RET_THREADS), bytes, stream,
                              rows, ld, decay, state, state_stride, single_rows, slots, (__nv_bfloat16*)out, heads, d, dv, eps);
    }
    return code;
}
