// What the chunked kernels of the linear recurrences share (retention with one fixed decay a head, gated linear
// attention with a decay per token and key channel): the chunk's length, how a CTA finds its chunk among a step's
// portions, and how a chunk's rows come into shared memory.
#pragma once
#include "common.cuh"

namespace {
constexpr int CHUNK = 32;

__device__ __forceinline__ float4 scaled(float4 v, float w) { return make_float4(v.x * w, v.y * w, v.z * w, v.w * w); }

// [CHUNK][width] of a chunk's rows into shared memory (row stride `stride`, zero behind `len` rows), each row times
// weight^(len - 1 - t) when weight_log2 is given; four elements at a time (`vec`: width and ld multiples of four, the
// base 16-byte aligned), several loads in flight.
__device__ __forceinline__ void load_chunk(float* __restrict__ dst, int stride, const float* __restrict__ src, long long ld,
                                           int len, int width, bool vec, bool weighted, float weight_log2) {
    if (vec) {
        const int w4 = width / 4;
#pragma unroll 4
        for (int e = threadIdx.x; e < CHUNK * w4; e += blockDim.x) {
            const int t = e / w4, i4 = e - t * w4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < len) v = *reinterpret_cast<const float4*>(src + (size_t)t * ld + 4 * i4);
            if (weighted) v = scaled(v, exp2f((float)(len - 1 - t) * weight_log2));
            *reinterpret_cast<float4*>(dst + t * stride + 4 * i4) = v;
        }
        return;
    }
    const int padded = (width + 3) & ~3;
    for (int e = threadIdx.x; e < CHUNK * padded; e += blockDim.x) {
        const int t = e / padded, i = e - t * padded;
        float value = 0.f;
        if (t < len && i < width) value = src[(size_t)t * ld + i] * (weighted ? exp2f((float)(len - 1 - t) * weight_log2) : 1.0f);
        dst[t * stride + i] = value;
    }
}

// which portion and which of its chunks the CTA `index` serves: false when there is none
__device__ __forceinline__ bool find_chunk(const int* __restrict__ segments, int n_segments, int index, int* first_row,
                                           int* length, int* segment, int* chunk) {
    for (int s = 0; s < n_segments; ++s) {
        const int count = segments[3 * s + 2];
        const int chunks = (count + CHUNK - 1) / CHUNK;
        if (index < chunks) {
            *first_row = segments[3 * s] + index * CHUNK;
            *length = min(CHUNK, count - index * CHUNK);
            *segment = s;
            *chunk = index;
            return true;
        }
        index -= chunks;
    }
    return false;
}
}  // namespace
