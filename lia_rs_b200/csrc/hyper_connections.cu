// A residual stream kept as several copies ("streams") that every sublayer reads through one weighted sum and writes
// back through a mixing matrix (hyper-connections), and the small row-wise steps that decoders of this kind need
// around their products.
//
//  * `embedding_streams`: x_s[t] = table[token_t] * scale for every stream s (all streams start as the embedding
//    output).  A token's streams lie side by side in one row: x [tokens, streams * hidden].
//  * `hyper_step`: for every token, in one pass over its row,
//        (1) with y (a sublayer's output): x_t <- sum_s mix[s, t] x_s + out[t] y   for all streams t at once
//            (mix is indexed [from, to]);
//        (2) with u: u = sum_s in[s] x_s (in absent: the plain sum), from the new streams, and optionally
//            normed = u / sqrt(mean(u^2) + eps) * w in the compute element type (the next sublayer's input).
//    Either half may be left out.  `rows_index` (only without y) gathers: output row r is computed from row
//    rows_index[r] of x.
//  * `softcap_rows`: z <- cap * tanh(z / cap), in place on 32-bit rows.
//  * `gate_rows`: o <- o * f(g), f the logistic function or SiLU, g 32-bit rows of any stride; one gate element for
//    every `span` neighbouring elements of o (span 1: element by element; span = a head's size: one gate a head).
//
// Everything is 32-bit but the normed rows and the gated rows.  The order of a row's additions depends on the width
// and the number of streams alone.
#include "common.cuh"

namespace {
constexpr int MAX_STREAMS = 8;

template <typename TW>
__global__ void embedding_streams_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                         float* __restrict__ out, int n_tokens, int hidden, int streams, int vocab,
                                         float scale, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int token = tokens[t];
    const bool ok = token >= 0 && token < vocab;
    if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
    const TW* row = table + (size_t)(ok ? token : 0) * hidden;
    float* dst = out + (size_t)t * hidden * streams;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = ok ? to_float(row[i]) * scale : 0.f;
        for (int s = 0; s < streams; ++s) dst[(size_t)s * hidden + i] = v;
    }
}

template <typename TO>
__global__ void hyper_step_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                                  const float* __restrict__ out_w, const float* __restrict__ in_w,
                                  const int* __restrict__ rows_index, float* __restrict__ u,
                                  const float* __restrict__ norm_w, TO* __restrict__ normed, int rows, int hidden,
                                  int streams, float eps) {
    __shared__ float coefficients[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    float* m = coefficients;
    float* ow = coefficients + MAX_STREAMS * MAX_STREAMS;
    float* iw = ow + MAX_STREAMS;
    for (int i = threadIdx.x; i < streams * streams; i += blockDim.x) m[i] = mix ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < streams; i += blockDim.x) {
        ow[i] = out_w ? out_w[i] : 0.f;
        iw[i] = in_w ? in_w[i] : 1.f;
    }
    __syncthreads();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int source = rows_index ? rows_index[r] : r;
    float* xr = x + (size_t)(source < 0 ? 0 : source) * hidden * streams;
    const float* yr = y ? y + (size_t)r * hidden : nullptr;
    float* ur = u ? u + (size_t)r * hidden : nullptr;
    float sum = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float xs[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) xs[s] = (s < streams && source >= 0) ? xr[(size_t)s * hidden + i] : 0.f;
        if (yr) {
            const float yi = yr[i];
            float next[MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < streams && t < streams) acc = fmaf(m[s * streams + t], xs[s], acc);
                next[t] = fmaf(ow[t < streams ? t : 0], yi, acc);
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t)
                if (t < streams) {
                    xs[t] = next[t];
                    xr[(size_t)t * hidden + i] = next[t];
                }
        }
        if (ur) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < streams) acc = fmaf(iw[s], xs[s], acc);
            ur[i] = acc;
            sum = fmaf(acc, acc, sum);
        }
    }
    if (!normed) return;
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
    TO* nr = normed + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)            // (each thread reads back what it wrote itself)
        nr[i] = from_float<TO>(ur[i] * inv * norm_w[i]);
}

// The same step four elements at a time: hidden a multiple of 4, every row 16-byte aligned, at most VEC_ITERS * blockDim
// groups of four a row, so that a thread keeps its part of u in registers between the sum and the norm.
constexpr int VEC_ITERS = 4;

__device__ __forceinline__ float4 fma4(float a, float4 b, float4 c) {
    return make_float4(fmaf(a, b.x, c.x), fmaf(a, b.y, c.y), fmaf(a, b.z, c.z), fmaf(a, b.w, c.w));
}
__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename TO>
__global__ void __launch_bounds__(512) hyper_step_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                                      const float* __restrict__ out_w, const float* __restrict__ in_w,
                                      const int* __restrict__ rows_index, float* __restrict__ u,
                                      const float* __restrict__ norm_w, TO* __restrict__ normed, int rows, int hidden,
                                      int streams, float eps) {
    __shared__ float coefficients[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    float* m = coefficients;
    float* ow = coefficients + MAX_STREAMS * MAX_STREAMS;
    float* iw = ow + MAX_STREAMS;
    for (int i = threadIdx.x; i < streams * streams; i += blockDim.x) m[i] = mix ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < streams; i += blockDim.x) {
        ow[i] = out_w ? out_w[i] : 0.f;
        iw[i] = in_w ? in_w[i] : 1.f;
    }
    float4 weight[VEC_ITERS];
    const int quads = hidden / 4;
    if (normed) {                                           // (the norm's weights do not depend on the kernel ahead)
#pragma unroll
        for (int it = 0; it < VEC_ITERS; ++it) {
            const int i = threadIdx.x + it * blockDim.x;
            if (i < quads) weight[it] = reinterpret_cast<const float4*>(norm_w)[i];
        }
    }
    __syncthreads();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int source = rows_index ? rows_index[r] : r;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)(source < 0 ? 0 : source) * hidden * streams);
    const float4* yr = y ? reinterpret_cast<const float4*>(y + (size_t)r * hidden) : nullptr;
    float4* ur = u ? reinterpret_cast<float4*>(u + (size_t)r * hidden) : nullptr;
    float4 keep[VEC_ITERS];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < VEC_ITERS; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i >= quads) break;
        float4 xs[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
            xs[s] = (s < streams && source >= 0) ? xr[(size_t)s * quads + i] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (yr) {
            const float4 yi = yr[i];
            float4 next[MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < streams && t < streams) acc = fma4(m[s * streams + t], xs[s], acc);
                next[t] = fma4(ow[t < streams ? t : 0], yi, acc);
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t)
                if (t < streams) {
                    xs[t] = next[t];
                    xr[(size_t)t * quads + i] = next[t];
                }
        }
        if (ur) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < streams) acc = fma4(iw[s], xs[s], acc);
            ur[i] = acc;
            keep[it] = acc;
            sum = fmaf(acc.x, acc.x, fmaf(acc.y, acc.y, fmaf(acc.z, acc.z, fmaf(acc.w, acc.w, sum))));
        }
    }
    if (!normed) return;
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
    TO* nr = normed + (size_t)r * hidden;
#pragma unroll
    for (int it = 0; it < VEC_ITERS; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i >= quads) break;
        const float4 v = keep[it], w = weight[it];
        store4(nr + 4 * (size_t)i, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
    }
}

__global__ void softcap_rows_kernel(float* __restrict__ z, long long ld, int rows, int width, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)rows * width;
    const float inv = 1.0f / cap;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / width;
        float* p = z + r * ld + (e - r * width);
        *p = cap * tanhf(*p * inv);
    }
}

template <typename T, int ACT>
__global__ void gate_rows_kernel(T* __restrict__ o, long long ld_o, const float* __restrict__ g, long long ld_g, int rows,
                                 int width, int span) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)rows * width;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / width;
        const int i = (int)(e - r * width);
        const float z = g[r * ld_g + i / span];
        const float s = 1.0f / (1.0f + expf(-z));
        const float f = ACT == 2 ? z * s : s;
        o[r * ld_o + i] = from_float<T>(to_float(o[r * ld_o + i]) * f);
    }
}

int grid_for(long long total) {
    const long long blocks = (total + 255) / 256;
    return (int)(blocks < 8192 ? blocks : 8192);
}
}  // namespace

// out [n, streams * hidden] 32-bit: every stream of token t is table[tokens[t]] * scale.
LIA_EXPORT int lia_embedding_streams(const int* tokens, const void* table, int table_dtype, float* out, int n_tokens,
                                     int hidden, int streams, int vocab, float scale, int* error_flag,
                                     cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (hidden <= 0 || vocab <= 0 || streams <= 0 || streams > MAX_STREAMS) return LIA_ERR_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == LIA_BF16)
        return lia_launch(embedding_streams_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                          (const __nv_bfloat16*)table, out, n_tokens, hidden, streams, vocab, scale, error_flag);
    if (table_dtype == LIA_F32)
        return lia_launch(embedding_streams_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                          (const float*)table, out, n_tokens, hidden, streams, vocab, scale, error_flag);
    return LIA_ERR_DTYPE;
}

// x [.., streams * hidden] 32-bit, changed in place when y [rows, hidden] is given (mix [streams, streams] indexed
// [from, to], out_w [streams]); u [rows, hidden] 32-bit receives sum_s in_w[s] x_s (in_w null: all ones) when given,
// and normed [rows, hidden] of `normed_dtype` its RMS norm with norm_w [hidden] (32-bit).  rows_index: only without y.
LIA_EXPORT int lia_hyper_step(float* x, const float* y, const float* mix, const float* out_w, const float* in_w,
                              const int* rows_index, float* u, const float* norm_w, void* normed, int normed_dtype,
                              int rows, int hidden, int streams, float eps, cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (hidden <= 0 || streams <= 0 || streams > MAX_STREAMS || (y && (!mix || !out_w || rows_index)) ||
        (normed && (!u || !norm_w)) || (!y && !u))
        return LIA_ERR_SIZE;
    const auto aligned = [](const void* p) { return ((uintptr_t)p & 15u) == 0; };
    if (hidden % 4 == 0 && hidden <= 4 * VEC_ITERS * 512 && aligned(x) && aligned(y) && aligned(u) && aligned(norm_w) &&
        (normed_dtype == LIA_F32 ? aligned(normed) : ((uintptr_t)normed & 7u) == 0)) {
        // four elements a thread and step: as many threads as a row has groups of four, 64 to 512
        const int quads = hidden / 4;
        const int vec_threads = quads >= 512 ? 512 : quads <= 64 ? 64 : (quads + 31) / 32 * 32;
        if (!normed || normed_dtype == LIA_F32)
            return lia_launch(hyper_step_vec_kernel<float>, dim3(rows), dim3(vec_threads), 0, stream, x, y, mix, out_w, in_w,
                              rows_index, u, norm_w, (float*)normed, rows, hidden, streams, eps);
        if (normed_dtype == LIA_BF16)
            return lia_launch(hyper_step_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(vec_threads), 0, stream, x, y, mix, out_w,
                              in_w, rows_index, u, norm_w, (__nv_bfloat16*)normed, rows, hidden, streams, eps);
        return LIA_ERR_DTYPE;
    }
    const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
    if (!normed || normed_dtype == LIA_F32)
        return lia_launch(hyper_step_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, y, mix, out_w, in_w,
                          rows_index, u, norm_w, (float*)normed, rows, hidden, streams, eps);
    if (normed_dtype == LIA_BF16)
        return lia_launch(hyper_step_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, y, mix, out_w, in_w,
                          rows_index, u, norm_w, (__nv_bfloat16*)normed, rows, hidden, streams, eps);
    return LIA_ERR_DTYPE;
}

// z [rows, width] 32-bit with row stride ld, in place: z <- cap * tanh(z / cap).
LIA_EXPORT int lia_softcap_rows(float* z, long long ld, int rows, int width, float cap, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return LIA_OK;
    if (ld < width || !(cap > 0.f)) return LIA_ERR_SIZE;
    return lia_launch(softcap_rows_kernel, dim3(grid_for((long long)rows * width)), dim3(256), 0, stream, z, ld, rows,
                      width, cap);
}

// o [rows, width] of `dtype` with row stride ld_o, in place: o[r, i] <- o[r, i] * f(g[r, i / span]), g 32-bit with row
// stride ld_g; act 1: the logistic function, 2: SiLU.
LIA_EXPORT int lia_gate_rows(void* o, int dtype, long long ld_o, const float* g, long long ld_g, int rows, int width,
                             int act, int span, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return LIA_OK;
    if (span <= 0 || ld_o < width || ld_g < (width + span - 1) / span || act < 1 || act > 2) return LIA_ERR_SIZE;
    const int blocks = grid_for((long long)rows * width);
#define LIA_GATE(T, ACT)                                                                                             \
    return lia_launch(gate_rows_kernel<T, ACT>, dim3(blocks), dim3(256), 0, stream, (T*)o, ld_o, g, ld_g, rows, width, span)
    if (dtype == LIA_F32) {
        if (act == 1) LIA_GATE(float, 1);
        LIA_GATE(float, 2);
    }
    if (dtype == LIA_BF16) {
        if (act == 1) LIA_GATE(__nv_bfloat16, 1);
        LIA_GATE(__nv_bfloat16, 2);
    }
#undef LIA_GATE
    return LIA_ERR_DTYPE;
}
