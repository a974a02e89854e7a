// A mixture of gated feed-forward experts: each token goes to the `top` experts with the largest router scores.
//
//  * `moe_route`: z = W_router x in 32-bit (W_router 32-bit, x in the compute element type), s = softmax(z) over all
//    router outputs, the `top` outputs with the largest choice score chosen (the lower index wins a tie), their
//    weights s_e * scale, or with `renormalise` s_e / (sum of the chosen s + 1e-20) * scale.  The choice score is s, or
//    s + correction with a 32-bit `correction` per output; with `groups` > 1 the outputs form that many equal groups
//    of neighbours, a group's score is its largest choice score, and only outputs of the `keep` best groups can be
//    chosen.  Outputs from `experts` on name no expert (their pairs belong to no row of the products; `moe_combine`
//    adds the token's own input for them).  An optional extra row of the router matrix gives one more logit a token,
//    whose logistic function is the gate of a shared expert.
//  * `moe_plan`: the (token, choice) pairs grouped by expert: where each expert's rows begin, which pair each sorted row
//    is, where each pair went, and the list of (expert, first row, rows) tiles of `tile_rows` rows that the products run
//    over.  With `pad` every expert's group begins at a multiple of `tile_rows` (rows in between belong to no pair), so
//    that a tile of the tensor-core product (csrc/gemm_tc.cu, grouped) never holds rows of two experts.
//    Which pair gets which row inside an expert's group is not fixed, and does not matter: every row of a product is
//    computed for itself, its sum over K in ascending order.
//  * `moe_gather`: the sorted rows' inputs side by side (rows of no pair are zero), for the tensor-core product.
//  * `moe_gemm`: for every tile, rows x W_e^T with the expert's own matrix, on the 32-bit pipes (the 32-bit path, and
//    sizes that TMA cannot address): mode 1 reads token rows through the sorted list and writes up * silu(gate)
//    of [W_gate; W_up]; mode 2 reads them likewise and writes relu(W_up x)^2; mode 0 reads the sorted rows and writes
//    32-bit rows.
//  * `moe_combine`: residual (+)= alpha * (sum_c weight_c y[row of (t, c)] + gate_t shared_t), the choices added in
//    their order, so a token's result does not depend on what else is in the batch; a choice without a row (an
//    identity output) adds weight_c x_t.
#include "common.cuh"

namespace {
constexpr int TILE_M = 32, TILE_N = 64, TILE_K = 32;
constexpr int MOE_MAX_EXPERTS = 1024, MOE_MAX_TOP = 32;

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, long long ld, const float* __restrict__ router, int hidden,
                                 int experts, int top, float scale, int extra, const float* __restrict__ correction,
                                 int groups, int keep, int renormalise, int* __restrict__ ids,
                                 float* __restrict__ weights, float* __restrict__ shared_gate) {
    extern __shared__ __align__(16) float route_shared[];  // x [hidden], z [experts + extra], choice scores [experts]
    __shared__ int picked[MOE_MAX_TOP];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    float* xs = route_shared;
    float* z = xs + hidden;
    float* choice = z + experts + extra;
    const T* row = x + (size_t)t * ld;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = to_float(row[i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    // (four elements a lane and step where the rows allow it; the order of a score's additions depends on `hidden` alone)
    const bool by_fours = (hidden & 3) == 0 && ((uintptr_t)router & 15u) == 0;
    for (int e = warp; e < experts + extra; e += warps) {
        const float* w = router + (size_t)e * hidden;
        float acc = 0.f;
        if (by_fours) {
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 4
            for (int i = lane; i < hidden / 4; i += 32) {
                const float4 a = x4[i], b = __ldg(w4 + i);
                acc = fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, acc))));
            }
        } else {
            for (int i = lane; i < hidden; i += 32) acc = fmaf(xs[i], w[i], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    float largest = -INFINITY;
    for (int e = 0; e < experts; ++e) largest = fmaxf(largest, z[e]);
    float total = 0.f;
    for (int e = 0; e < experts; ++e) {
        z[e] = expf(z[e] - largest);
        total += z[e];
    }
    const float inv = 1.0f / total;
    for (int e = 0; e < experts; ++e) {
        z[e] *= inv;                                       // the score s_e
        choice[e] = z[e] + (correction ? correction[e] : 0.f);
    }
    if (groups > 1) {
        // the `keep` groups with the largest best choice score stay (the lower group wins a tie); the others' outputs
        // cannot be chosen
        const int size = experts / groups;
        for (int g = 0; g < groups; ++g) {
            float best = -INFINITY;
            for (int e = g * size; e < (g + 1) * size; ++e) best = fmaxf(best, choice[e]);
            int ahead = 0;
            for (int o = 0; o < groups; ++o) {
                if (o == g) continue;
                float other = -INFINITY;
                for (int e = o * size; e < (o + 1) * size; ++e) other = fmaxf(other, choice[e]);
                if (other > best || (other == best && o < g)) ++ahead;
            }
            if (ahead >= keep) {
                // NaN marks an output that is out of the choice (a choice score may be any number, minus infinity too)
                for (int e = g * size; e < (g + 1) * size; ++e) choice[e] = __int_as_float(0x7fc00000);
            }
        }
    }
    float chosen_sum = 0.f;
    for (int c = 0; c < top; ++c) {
        int best = -1;
        float value = 0.f;
        for (int e = 0; e < experts; ++e) {
            const float v = choice[e];
            if (v != v) continue;                          // taken, or of a group that is out
            if (best < 0 || v > value) value = v, best = e;
        }
        if (best < 0) best = 0;                            // (fewer outputs left than `top`: the launcher refuses that)
        picked[c] = best;
        chosen_sum += z[best];
        choice[best] = __int_as_float(0x7fc00000);
    }
    const float factor = renormalise ? scale / (chosen_sum + 1e-20f) : scale;
    for (int c = 0; c < top; ++c) {
        ids[(size_t)t * top + c] = picked[c];
        weights[(size_t)t * top + c] = z[picked[c]] * factor;
    }
    if (extra) shared_gate[t] = 1.0f / (1.0f + expf(-z[experts]));
}

__global__ void moe_plan_kernel(const int* __restrict__ ids, int pairs, int experts, int tile_rows, int pad, int rows_cap,
                                int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ inverse,
                                int* __restrict__ tiles, int* __restrict__ n_tiles) {
    __shared__ int counts[MOE_MAX_EXPERTS], starts[MOE_MAX_EXPERTS + 1], tile_starts[MOE_MAX_EXPERTS + 1];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    if (pad)
        for (int r = threadIdx.x; r < rows_cap; r += blockDim.x) order[r] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < experts; ++e) {
            if (pad) at = tile * tile_rows;
            starts[e] = at;
            tile_starts[e] = tile;
            at += counts[e];
            tile += (counts[e] + tile_rows - 1) / tile_rows;
        }
        starts[experts] = at;
        tile_starts[experts] = tile;
        *n_tiles = tile;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = starts[e];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        for (int k = tile_starts[e]; k < tile_starts[e + 1]; ++k) {
            const int first = (k - tile_starts[e]) * tile_rows;
            tiles[3 * k] = e;
            tiles[3 * k + 1] = starts[e] + first;
            tiles[3 * k + 2] = min(tile_rows, counts[e] - first);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e < 0 || e >= experts) {
            inverse[p] = -1;                                // a pair of no expert has no row
            continue;
        }
        const int r = starts[e] + atomicAdd(&counts[e], 1);
        order[r] = p;
        inverse[p] = r;
    }
}

// dst[r] = src[order[r] / top] (zero where order[r] < 0); rows of `width` elements, a multiple of 8.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ src, long long ld, const int* __restrict__ order, int top,
                                  __nv_bfloat16* __restrict__ dst, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = order[blockIdx.x];
    const uint4* from = p >= 0 ? reinterpret_cast<const uint4*>(src + (size_t)(p / top) * ld) : nullptr;
    uint4* to = reinterpret_cast<uint4*>(dst + (size_t)blockIdx.x * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) to[i] = from ? from[i] : make_uint4(0, 0, 0, 0);
}

// MODE 0: out[r, n] = sum_k a[r, k] w_e[n, k] (32-bit out).  MODE 1: out[r, n] = u * silu(g), g = a . w_e[n], u = a . w_e[N + n].
// MODE 2: out[r, n] = relu(a . w_e[n])^2.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ a, long long lda, const int* __restrict__ order, int top,
                const T* __restrict__ w, long long expert_stride, void* __restrict__ out_raw, long long ldo,
                const int* __restrict__ tiles, const int* __restrict__ n_tiles, int N, int K) {
    __shared__ float as[TILE_K][TILE_M + 1];
    __shared__ __align__(16) float ws[MODE == 1 ? 2 : 1][TILE_K][TILE_N];
    __shared__ int source[TILE_M];
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
    const int n0 = blockIdx.y * TILE_N;
    const T* we = w + (size_t)e * expert_stride;
    if (threadIdx.x < TILE_M) {
        int src = -1;
        if ((int)threadIdx.x < rows) src = order ? order[row0 + threadIdx.x] / top : row0 + threadIdx.x;
        source[threadIdx.x] = src;
    }
    __syncthreads();
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;      // rows 2 ty, 2 ty + 1; columns 4 tx .. 4 tx + 3
    float acc[MODE == 1 ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < K; k0 += TILE_K) {
        for (int idx = threadIdx.x; idx < TILE_M * TILE_K; idx += 256) {
            const int r = idx / TILE_K, kk = idx % TILE_K;
            const int src = source[r];
            as[kk][r] = (src >= 0 && k0 + kk < K) ? to_float(a[(size_t)src * lda + k0 + kk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < TILE_N * TILE_K; idx += 256) {
            const int n = idx / TILE_K, kk = idx % TILE_K;
            const bool in = n0 + n < N && k0 + kk < K;
            ws[0][kk][n] = in ? to_float(we[(size_t)(n0 + n) * K + k0 + kk]) : 0.f;
            if (MODE == 1) ws[1][kk][n] = in ? to_float(we[(size_t)(N + n0 + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TILE_K; ++kk) {
            const float a0 = as[kk][2 * ty], a1 = as[kk][2 * ty + 1];
#pragma unroll
            for (int m = 0; m < (MODE == 1 ? 2 : 1); ++m) {
                const float4 b = *reinterpret_cast<const float4*>(&ws[m][kk][4 * tx]);
                acc[m][0][0] = fmaf(a0, b.x, acc[m][0][0]);
                acc[m][0][1] = fmaf(a0, b.y, acc[m][0][1]);
                acc[m][0][2] = fmaf(a0, b.z, acc[m][0][2]);
                acc[m][0][3] = fmaf(a0, b.w, acc[m][0][3]);
                acc[m][1][0] = fmaf(a1, b.x, acc[m][1][0]);
                acc[m][1][1] = fmaf(a1, b.y, acc[m][1][1]);
                acc[m][1][2] = fmaf(a1, b.z, acc[m][1][2]);
                acc[m][1][3] = fmaf(a1, b.w, acc[m][1][3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int r = 2 * ty + x;
        if (r >= rows) continue;
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int n = n0 + 4 * tx + y;
            if (n >= N) continue;
            if (MODE == 1) {
                const float g = acc[0][x][y], u = acc[MODE == 1 ? 1 : 0][x][y];
                reinterpret_cast<T*>(out_raw)[(size_t)(row0 + r) * ldo + n] = from_float<T>(u * (g / (1.0f + expf(-g))));
            } else if (MODE == 2) {
                const float g = fmaxf(acc[0][x][y], 0.f);
                reinterpret_cast<T*>(out_raw)[(size_t)(row0 + r) * ldo + n] = from_float<T>(g * g);
            } else {
                reinterpret_cast<float*>(out_raw)[(size_t)(row0 + r) * ldo + n] = acc[0][x][y];
            }
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ residual, const float* __restrict__ y,
                                   const int* __restrict__ inverse, const float* __restrict__ weights,
                                   const float* __restrict__ shared_y, const float* __restrict__ shared_gate,
                                   const T* __restrict__ x, long long ld_x, int hidden, int top, float alpha, int store) {
    __shared__ int rows[MOE_MAX_TOP];
    __shared__ float w[MOE_MAX_TOP];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if ((int)threadIdx.x < top) {
        rows[threadIdx.x] = inverse[(size_t)t * top + threadIdx.x];
        w[threadIdx.x] = weights[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    const float gate = shared_y ? shared_gate[t] : 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < top; ++c) {
            // a choice without a row is an identity output: the token's own input
            const float v = rows[c] >= 0 ? y[(size_t)rows[c] * hidden + i] : (x ? to_float(x[(size_t)t * ld_x + i]) : 0.f);
            acc = fmaf(w[c], v, acc);
        }
        if (shared_y) acc = fmaf(gate, shared_y[(size_t)t * hidden + i], acc);
        float* dst = residual + (size_t)t * hidden + i;
        *dst = store ? alpha * acc : fmaf(alpha, acc, *dst);
    }
}
}  // namespace

LIA_EXPORT int lia_moe_tile_rows() { return TILE_M; }

// x [n, ld] of `dtype`; router [experts + extra, hidden] 32-bit; ids, weights [n, top]; shared_gate [n] (extra = 1);
// correction [experts] 32-bit or null; groups (0 or 1: none) divides experts, 1 <= keep <= groups, and the kept groups
// hold at least `top` outputs.  `experts` counts every router output, also those that name no expert.
LIA_EXPORT int lia_moe_route(const void* x, int dtype, long long ld, const float* router, int n, int hidden, int experts,
                             int top, float scale, int extra, const float* correction, int groups, int keep,
                             int renormalise, int* ids, float* weights, float* shared_gate, cudaStream_t stream) {
    if (n <= 0) return LIA_OK;
    if (hidden <= 0 || experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts || top > MOE_MAX_TOP ||
        extra < 0 || extra > 1 || (extra && !shared_gate) || ld < hidden || (size_t)(hidden + 2 * experts + 1) * 4 > 200 * 1024)
        return LIA_ERR_SIZE;
    if (groups > 1 && (experts % groups || keep < 1 || keep > groups || (long long)keep * (experts / groups) < top))
        return LIA_ERR_SIZE;
    const size_t bytes = (size_t)(hidden + 2 * experts + extra) * sizeof(float);
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    if (dtype == LIA_F32)
        return lia_launch(moe_route_kernel<float>, dim3(n), dim3(256), bytes, stream, (const float*)x, ld, router, hidden,
                          experts, top, scale, extra, correction, groups, keep, renormalise, ids, weights, shared_gate);
    if (dtype == LIA_BF16)
        return lia_launch(moe_route_kernel<__nv_bfloat16>, dim3(n), dim3(256), bytes, stream, (const __nv_bfloat16*)x, ld,
                          router, hidden, experts, top, scale, extra, correction, groups, keep, renormalise, ids, weights,
                          shared_gate);
    return LIA_ERR_DTYPE;
}

// ids [pairs]; offsets [experts + 1]; order [pairs, or rows_cap with pad]; inverse [pairs]; tiles [3 * (pairs / tile_rows +
// min(experts, pairs))]; n_tiles [1].  pad: every expert's rows begin at a multiple of tile_rows, and `order` is -1 on the
// rows of no pair, up to rows_cap = tile_rows * the most tiles.
LIA_EXPORT int lia_moe_plan(const int* ids, int pairs, int experts, int tile_rows, int pad, int rows_cap, int* offsets,
                            int* order, int* inverse, int* tiles, int* n_tiles, cudaStream_t stream) {
    if (pairs <= 0) return LIA_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || tile_rows <= 0) return LIA_ERR_SIZE;
    if (pad && rows_cap < (pairs / tile_rows + min(experts, pairs)) * tile_rows) return LIA_ERR_SIZE;
    return lia_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, ids, pairs, experts, tile_rows, pad, rows_cap, offsets,
                      order, inverse, tiles, n_tiles);
}

// dst [rows, width] bf16 = src[order[r] / top] (zero where order[r] < 0); width a multiple of 8, 16-byte aligned rows.
LIA_EXPORT int lia_moe_gather(const void* src, long long ld, const int* order, int top, void* dst, int rows, int width,
                              cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (width <= 0 || width % 8 || ld % 8 || top <= 0) return LIA_ERR_SIZE;
    if (((uintptr_t)src & 15u) || ((uintptr_t)dst & 15u)) return LIA_ERR_ALIGN;
    return lia_launch(moe_gather_kernel, dim3(rows), dim3(width >= 2048 ? 256 : 128), 0, stream, (const __nv_bfloat16*)src, ld,
                      order, top, (__nv_bfloat16*)dst, width);
}

// mode 1: a = the tokens' rows [n, lda] read through `order` (pair -> token pair / top), w [experts, 2 N, K], out
// [pairs, ldo] of `dtype`.  mode 2: the same rows, w [experts, N, K], out = relu(.)^2 of `dtype`.  mode 0: a = sorted rows
// [pairs, lda], w [experts, N, K], out [pairs, ldo] 32-bit.
// `max_tiles`: pairs / TILE_M + min(experts, pairs), the most tiles the plan can list (planned with TILE_M rows a tile).
LIA_EXPORT int lia_moe_gemm(int mode, const void* a, int dtype, long long lda, const int* order, int top, const void* w,
                            void* out, long long ldo, const int* tiles, const int* n_tiles, int max_tiles, int N, int K,
                            cudaStream_t stream) {
    if (max_tiles <= 0) return LIA_OK;
    if (N <= 0 || K <= 0 || lda < K || ldo < N || top <= 0 || mode < 0 || mode > 2 || (mode != 0 && !order))
        return LIA_ERR_SIZE;
    const dim3 grid(max_tiles, (N + TILE_N - 1) / TILE_N);
    const long long stride = (long long)(mode == 1 ? 2 : 1) * N * K;
#define LIA_MOE(T, MODE)                                                                                              \
    return lia_launch(moe_gemm_kernel<T, MODE>, grid, dim3(256), 0, stream, (const T*)a, lda, order, top, (const T*)w, \
                      stride, out, ldo, tiles, n_tiles, N, K)
    if (dtype == LIA_F32) {
        if (mode == 1) LIA_MOE(float, 1);
        if (mode == 2) LIA_MOE(float, 2);
        LIA_MOE(float, 0);
    }
    if (dtype == LIA_BF16) {
        if (mode == 1) LIA_MOE(__nv_bfloat16, 1);
        if (mode == 2) LIA_MOE(__nv_bfloat16, 2);
        LIA_MOE(__nv_bfloat16, 0);
    }
#undef LIA_MOE
    return LIA_ERR_DTYPE;
}

// residual [n, hidden] 32-bit (+)= alpha * (sum_c weights[t, c] y[inverse[t, c]] + shared_gate[t] shared_y[t]); where
// inverse[t, c] < 0 the term is weights[t, c] x[t] (x [n, ld_x] of `x_dtype`; null: such terms are zero).
LIA_EXPORT int lia_moe_combine(float* residual, const float* y, const int* inverse, const float* weights,
                               const float* shared_y, const float* shared_gate, const void* x, int x_dtype, long long ld_x,
                               int n, int hidden, int top, float alpha, int store, cudaStream_t stream) {
    if (n <= 0) return LIA_OK;
    if (hidden <= 0 || top <= 0 || top > MOE_MAX_TOP || (shared_y && !shared_gate) || (x && ld_x < hidden)) return LIA_ERR_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (x && x_dtype == LIA_BF16)
        return lia_launch(moe_combine_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, residual, y, inverse, weights,
                          shared_y, shared_gate, (const __nv_bfloat16*)x, ld_x, hidden, top, alpha, store);
    if (x && x_dtype != LIA_F32) return LIA_ERR_DTYPE;
    return lia_launch(moe_combine_kernel<float>, dim3(n), dim3(threads), 0, stream, residual, y, inverse, weights, shared_y,
                      shared_gate, (const float*)x, ld_x, hidden, top, alpha, store);
}
