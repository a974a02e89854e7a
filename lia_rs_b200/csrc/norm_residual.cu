// What a layer with a norm on both sides of each sublayer needs on the 32-bit residual stream:
//  * residual[r] += rms(y[r] + bias) * w        (the sublayer's output y, normed, joins the stream), and in the same
//    pass, optionally, next[r] = rms(residual[r]) * w2 in the compute element type (the input of the sublayer that
//    follows), so that the stream is read once between two sublayers;
//  * out[r, :] = act(in[r, :]) for 32-bit rows with any row stride: the activation between the two products of a dense
//    feed-forward (tanh form of GELU), SiLU, or a plain change of element type of some columns.
// Sums of squares, means and reciprocal roots are 32-bit; the order of a row's additions depends on the width alone.
#include "common.cuh"

namespace {
template <typename TO>
__global__ void norm_residual_kernel(const float* __restrict__ y, const float* __restrict__ bias,
                                     const float* __restrict__ weight, float* __restrict__ residual,
                                     const float* __restrict__ next_weight, TO* __restrict__ next, int rows, int hidden,
                                     float eps, float next_eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const float* yr = y + (size_t)r * hidden;
    float* xr = residual + (size_t)r * hidden;
    float sum = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = yr[i] + (bias ? bias[i] : 0.f);
        sum = fmaf(v, v, sum);
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
    float sum2 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = yr[i] + (bias ? bias[i] : 0.f);
        const float x = xr[i] + v * inv * weight[i];
        xr[i] = x;
        sum2 = fmaf(x, x, sum2);
    }
    if (!next) return;
    sum2 = block_sum(sum2, scratch);
    const float inv2 = 1.0f / sqrtf(sum2 / (float)hidden + next_eps);
    TO* nr = next + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)          // (each thread reads back what it wrote itself)
        nr[i] = from_float<TO>(xr[i] * inv2 * next_weight[i]);
}

// 0.5 z (1 + tanh(u)), u = sqrt(2/pi) (z + 0.044715 z^3), written as z / (1 + exp(-2u)): the same function, one exponential
__device__ __forceinline__ float gelu_tanh(float z) {
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return z / (1.0f + expf(-2.0f * u));
}

// act: 0 identity, 1 GELU (tanh form), 2 SiLU, 3 the square of ReLU, 4 ReLU
__device__ __forceinline__ float activate(int act, float z) {
    if (act == 1) return gelu_tanh(z);
    if (act == 2) return z / (1.0f + expf(-z));
    if (act == 3) { const float r = fmaxf(z, 0.f); return r * r; }
    if (act == 4) return fmaxf(z, 0.f);
    return z;
}

template <typename TO> __device__ __forceinline__ void store_four(TO* dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store_four<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store_four<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
}

// four elements a thread: rows whose width and strides are multiples of 4 from 16-byte aligned bases.  `gated`: the
// row holds `width` gate elements and then `width` more, out = act(gate) * the other.
template <typename TO>
__global__ void activation_rows4_kernel(const float* __restrict__ in, long long ld_in, TO* __restrict__ out,
                                        long long ld_out, int rows, int quads, int act, int gated) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)rows * quads;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / quads;
        const int i = (int)(e - r * quads) * 4;
        const float4 z = *reinterpret_cast<const float4*>(in + r * ld_in + i);
        float4 u = make_float4(1.f, 1.f, 1.f, 1.f);
        if (gated) u = *reinterpret_cast<const float4*>(in + r * ld_in + 4 * quads + i);
        store_four<TO>(out + r * ld_out + i, activate(act, z.x) * u.x, activate(act, z.y) * u.y, activate(act, z.z) * u.z,
                       activate(act, z.w) * u.w);
    }
}

template <typename TO>
__global__ void activation_rows_kernel(const float* __restrict__ in, long long ld_in, TO* __restrict__ out,
                                       long long ld_out, int rows, int width, int act, int gated) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)rows * width;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / width;
        const int i = (int)(e - r * width);
        const float u = gated ? in[r * ld_in + width + i] : 1.f;
        out[r * ld_out + i] = from_float<TO>(activate(act, in[r * ld_in + i]) * u);
    }
}
}  // namespace

// residual [rows, hidden] += rms(y [rows, hidden] + bias [hidden] or nothing) * weight [hidden]; with `next`
// (next_dtype) also next = rms(residual) * next_weight.  Everything but `next` is 32-bit.
LIA_EXPORT int lia_norm_residual(const float* y, const float* bias, const float* weight, float* residual,
                                 const float* next_weight, void* next, int next_dtype, int rows, int hidden, float eps,
                                 float next_eps, cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (hidden <= 0 || (next && !next_weight)) return LIA_ERR_SIZE;
    const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
    if (!next || next_dtype == LIA_F32)
        return lia_launch(norm_residual_kernel<float>, dim3(rows), dim3(threads), 0, stream, y, bias, weight, residual,
                          next_weight, (float*)next, rows, hidden, eps, next_eps);
    if (next_dtype == LIA_BF16)
        return lia_launch(norm_residual_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, y, bias, weight,
                          residual, next_weight, (__nv_bfloat16*)next, rows, hidden, eps, next_eps);
    return LIA_ERR_DTYPE;
}

// out[r, i] = act(in[r, i]), i < width, or with `gated` act(in[r, i]) * in[r, width + i]; act: 0 identity, 1 GELU
// (tanh form), 2 SiLU, 3 the square of ReLU, 4 ReLU.  Row strides in elements.
LIA_EXPORT int lia_activation_rows(const float* in, long long ld_in, void* out, int out_dtype, long long ld_out,
                                   int rows, int width, int act, int gated, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return LIA_OK;
    if (ld_in < (gated ? 2 : 1) * (long long)width || ld_out < width || act < 0 || act > 4) return LIA_ERR_SIZE;
    const bool four = width % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && ((uintptr_t)in & 15u) == 0 && ((uintptr_t)out & 15u) == 0;
    const long long total = four ? (long long)rows * (width / 4) : (long long)rows * width;
    const int blocks = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
#define LIA_ACT(TO)                                                                                                      \
    {                                                                                                                    \
        if (four)                                                                                                        \
            return lia_launch(activation_rows4_kernel<TO>, dim3(blocks), dim3(256), 0, stream, in, ld_in, (TO*)out,     \
                              ld_out, rows, width / 4, act, gated);                                                      \
        return lia_launch(activation_rows_kernel<TO>, dim3(blocks), dim3(256), 0, stream, in, ld_in, (TO*)out,          \
                          ld_out, rows, width, act, gated);                                                              \
    }
    if (out_dtype == LIA_F32) LIA_ACT(float)
    if (out_dtype == LIA_BF16) LIA_ACT(__nv_bfloat16)
#undef LIA_ACT
    return LIA_ERR_DTYPE;
}
