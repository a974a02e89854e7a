// What happens to a step's projected rows between the product and the attention, for two kinds of attention whose
// queries and keys are more than a product's output:
//
//  * `qkv_prepare`: rows [q heads | k heads | v heads] (keys of size d, values of size dv) get, in this order, a bias
//    (the projection's), an RMS norm per head of q and of k with a weight of size d shared by the heads, the
//    rotate-half encoding over the first `rot_dims` elements of every q and k head (element i with i + rot_dims/2,
//    angle position * freq[i]), and a mixing of the values with those that an earlier layer left for the same token,
//    v <- (1 - lambda) v + lambda v_first (mode 2; mode 1 leaves v for later layers; mode 0 neither).  q goes out in the
//    compute element type, k and the mixed v are appended to the pages.
//  * `latent_prepare`: attention through a latent.  The query rows hold, per head, `d` unrotated elements and then
//    `dr` rotated ones; the shared row holds `rank` latent elements and then `dr` elements of a rotated key part that
//    all heads share.  The latent is RMS-normed (weight of size rank) and appended to the first pages, the key part is
//    encoded and appended to the second pages; the queries' unrotated parts go out head by head in planes of their own
//    ([heads, tokens, d]: each head's rows are then a matrix for the product with that head's share of the key
//    expansion), the rotated parts encoded as [tokens, heads, dr].
//
// Everything is computed in 32-bit: bias, sums of squares, angles (float(position) * freq[i]), sines and cosines.  A
// token whose slot is negative belongs to nobody and is skipped; a position without a page raises error flag 2.
#include "common.cuh"

namespace {
constexpr int PREP_WARPS = 4;

// page row (in units of cache rows) of `pos` for `slot`, or -1 with the flag raised
__device__ __forceinline__ long long page_row(const int* __restrict__ block_table, int table_stride, int slot, int pos,
                                              int page_size, int num_pages, int* __restrict__ error_flag) {
    const int page = block_table[(size_t)slot * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
        return -1;
    }
    return (long long)page * page_size + pos % page_size;
}

// One warp norms (optionally) and rotates one head that lies in `h` (shared memory, 32-bit, `d` elements; the rotated
// span begins at `offset` and is `rot_dims` long), in place.
__device__ __forceinline__ void norm_and_rotate(float* h, int d, const float* __restrict__ norm_weight, float eps,
                                                int offset, int rot_dims, const float* rotation, int lane,
                                                bool pairs = false) {
    if (norm_weight) {
        float sum = 0.f;
        for (int i = lane; i < d; i += 32) sum = fmaf(h[i], h[i], sum);
        sum = warp_sum(sum);
        const float inv = 1.0f / sqrtf(sum / (float)d + eps);
        for (int i = lane; i < d; i += 32) h[i] = h[i] * inv * norm_weight[i];
        __syncwarp();
    }
    const int half = rot_dims / 2;
    for (int i = lane; i < half; i += 32) {
        const float c = rotation[i], s = rotation[half + i];
        const int a = offset + (pairs ? 2 * i : i), b = offset + (pairs ? 2 * i + 1 : half + i);
        const float u = h[a], v = h[b];
        h[a] = u * c - v * s;
        h[b] = v * c + u * s;
    }
    __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
qkv_prepare_kernel(const float* __restrict__ rows, long long ld, const float* __restrict__ bias,
                   const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                   const float* __restrict__ freq, int rot_dims, int vmix_mode, float lambda,
                   float* __restrict__ v_first, const int* __restrict__ positions, const int* __restrict__ slots,
                   const int* __restrict__ block_table, int table_stride, T* __restrict__ q_out,
                   T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int nq, int nkv, int d, int dv,
                   int page_size, int num_pages, int write_kv, int norm_whole, int* __restrict__ error_flag) {
    extern __shared__ float prep_shared[];                 // [rot_dims] cosines then sines, then [PREP_WARPS][d]
    __shared__ float whole_scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = rot_dims / 2;
    float* rotation = prep_shared;
    float* heads = prep_shared + rot_dims;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * freq[i], &rotation[half + i], &rotation[i]);
    __syncthreads();
    const long long cache_row = write_kv ? page_row(block_table, table_stride, slot, pos, page_size, num_pages, error_flag) : -1;
    const float* row = rows + (size_t)t * ld;
    float* h = heads + (size_t)warp * d;
    // norm_whole: one root mean square over all of q's elements (bias added) and one over all of k's, weights of those sizes
    float whole_inv[2] = {1.f, 1.f};
    if (norm_whole) {
        for (int part = 0; part < 2; ++part) {
            const int first = part ? nq * d : 0, width = part ? nkv * d : nq * d;
            float sum = 0.f;
            for (int i = threadIdx.x; i < width; i += blockDim.x) {
                const float v = row[first + i] + (bias ? bias[first + i] : 0.f);
                sum = fmaf(v, v, sum);
            }
            sum = block_sum(sum, whole_scratch);
            whole_inv[part] = 1.0f / sqrtf(sum / (float)width + eps);
        }
    }
    for (int head = warp; head < nq + nkv; head += PREP_WARPS) {
        const bool is_q = head < nq;
        for (int i = lane; i < d; i += 32) h[i] = row[head * d + i] + (bias ? bias[head * d + i] : 0.f);
        if (norm_whole) {
            const float* w = is_q ? q_norm + (size_t)head * d : k_norm + (size_t)(head - nq) * d;
            for (int i = lane; i < d; i += 32) h[i] = h[i] * whole_inv[is_q ? 0 : 1] * w[i];
        }
        __syncwarp();
        norm_and_rotate(h, d, norm_whole ? nullptr : (is_q ? q_norm : k_norm), eps, 0, rot_dims, rotation, lane);
        if (is_q) {
            T* dst = q_out + ((size_t)t * nq + head) * d;
            for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(h[i]);
        } else if (cache_row >= 0) {
            T* dst = k_pages + ((size_t)cache_row * nkv + (head - nq)) * d;
            for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(h[i]);
        }
        __syncwarp();
    }
    const int v_width = nkv * dv;
    const float* v = row + (size_t)(nq + nkv) * d;
    const float* v_bias = bias ? bias + (size_t)(nq + nkv) * d : nullptr;
    for (int i = threadIdx.x; i < v_width; i += blockDim.x) {
        float x = v[i] + (v_bias ? v_bias[i] : 0.f);
        if (vmix_mode == 1) v_first[(size_t)t * v_width + i] = x;
        if (vmix_mode == 2) x = (1.0f - lambda) * x + lambda * v_first[(size_t)t * v_width + i];
        if (cache_row >= 0) v_pages[(size_t)cache_row * v_width + i] = from_float<T>(x);
    }
}

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
latent_prepare_kernel(const float* __restrict__ q_rows, long long ld_q, const float* __restrict__ shared_rows,
                      long long ld_s, const float* __restrict__ latent_norm, float eps, const float* __restrict__ freq,
                      int rot_dims, const int* __restrict__ positions, const int* __restrict__ slots,
                      const int* __restrict__ block_table, int table_stride, T* __restrict__ q_plain,
                      T* __restrict__ q_rotated, T* __restrict__ latent_pages, T* __restrict__ key_pages, int n_tokens,
                      int heads, int d, int dr, int rank, int page_size, int num_pages, int write_kv, int pairs,
                      int* __restrict__ error_flag) {
    extern __shared__ float prep_shared[];                 // [rot_dims] cosines then sines, then [PREP_WARPS][dr]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = rot_dims / 2;
    float* rotation = prep_shared;
    float* parts = prep_shared + rot_dims;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * freq[i], &rotation[half + i], &rotation[i]);
    __syncthreads();
    const long long cache_row = (write_kv && shared_rows)
                                    ? page_row(block_table, table_stride, slot, pos, page_size, num_pages, error_flag) : -1;
    // the queries: unrotated parts into the head's plane, rotated parts encoded
    const float* q = q_rows + (size_t)t * ld_q;
    float* part = parts + (size_t)warp * dr;
    for (int head = warp; head < heads; head += PREP_WARPS) {
        const float* src = q + (size_t)head * (d + dr);
        T* plain = q_plain + ((size_t)head * n_tokens + t) * d;
        for (int i = lane; i < d; i += 32) plain[i] = from_float<T>(src[i]);
        for (int i = lane; i < dr; i += 32) part[i] = src[d + i];
        __syncwarp();
        norm_and_rotate(part, dr, nullptr, 0.f, 0, rot_dims, rotation, lane, pairs != 0);
        T* rotated = q_rotated + ((size_t)t * heads + head) * dr;
        for (int i = lane; i < dr; i += 32) rotated[i] = from_float<T>(part[i]);
        __syncwarp();
    }
    // the latent, normed over its own length, and the shared key part, encoded (a layer that reads another layer's
    // pages has neither)
    if (!shared_rows) return;
    const float* s = shared_rows + (size_t)t * ld_s;
    float sum = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) sum = fmaf(s[i], s[i], sum);
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)rank + eps);
    if (cache_row >= 0) {
        T* dst = latent_pages + (size_t)cache_row * rank;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(s[i] * inv * latent_norm[i]);
    }
    __syncthreads();                                       // every warp is done with its `part`
    if (warp == 0) {
        for (int i = lane; i < dr; i += 32) parts[i] = s[rank + i];
        __syncwarp();
        norm_and_rotate(parts, dr, nullptr, 0.f, 0, rot_dims, rotation, lane, pairs != 0);
        if (cache_row >= 0) {
            T* dst = key_pages + (size_t)cache_row * dr;
            for (int i = lane; i < dr; i += 32) dst[i] = from_float<T>(parts[i]);
        }
    }
}
}  // namespace

// rows [n, ld] 32-bit: nq heads of d, nkv heads of d, nkv heads of dv.  bias (32-bit, the rows' layout) or null;
// q_norm, k_norm (32-bit [d]; with `norm_whole` [nq d] and [nkv d]: one norm over all of q and one over all of k) or
// null; freq (32-bit [rot_dims / 2]; rot_dims 0: no encoding).  vmix_mode 1 writes,
// 2 reads v_first (32-bit [n, nkv dv]).  q_out [n, nq d], k_pages [pages, page_size, nkv, d], v_pages [.., nkv, dv].
LIA_EXPORT int lia_qkv_prepare(const float* rows, long long ld, const float* bias, const float* q_norm,
                               const float* k_norm, float eps, const float* freq, int rot_dims, int vmix_mode,
                               float lambda, float* v_first, const int* positions, const int* slots,
                               const int* block_table, int table_stride, void* q_out, void* k_pages, void* v_pages,
                               int dtype, int n_tokens, int nq, int nkv, int d, int dv, int page_size, int num_pages,
                               int write_kv, int norm_whole, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (norm_whole && (!q_norm || !k_norm)) return LIA_ERR_SIZE;
    if (nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || rot_dims < 0 || rot_dims > d || (rot_dims & 1) ||
        (rot_dims > 0 && !freq) || ld < (long long)(nq + nkv) * d + (long long)nkv * dv || vmix_mode < 0 || vmix_mode > 2 ||
        (vmix_mode && !v_first) || d > 4096)
        return LIA_ERR_SIZE;
    const size_t smem = ((size_t)rot_dims + (size_t)PREP_WARPS * d) * sizeof(float);
#define LIA_PREP(T)                                                                                                   \
    return lia_launch(qkv_prepare_kernel<T>, dim3(n_tokens), dim3(PREP_WARPS * 32), smem, stream, rows, ld, bias,     \
                      q_norm, k_norm, eps, freq, rot_dims, vmix_mode, lambda, v_first, positions, slots, block_table, \
                      table_stride, (T*)q_out, (T*)k_pages, (T*)v_pages, n_tokens, nq, nkv, d, dv, page_size,         \
                      num_pages, write_kv, norm_whole, error_flag)
    if (dtype == LIA_BF16) LIA_PREP(__nv_bfloat16);
    if (dtype == LIA_F32) LIA_PREP(float);
#undef LIA_PREP
    return LIA_ERR_DTYPE;
}

// q_rows [n, ld_q] 32-bit: per head d unrotated then dr rotated elements; shared_rows [n, ld_s] 32-bit: rank latent
// elements then dr of the shared key part.  q_plain [heads, n, d], q_rotated [n, heads, dr], latent_pages [pages,
// page_size, rank], key_pages [pages, page_size, dr], all of `dtype`.  `pairs`: the rotation pairs element 2i with 2i+1
// (0: i with i + rot_dims/2).  shared_rows null: only the queries are prepared (the pages are another layer's).
LIA_EXPORT int lia_latent_prepare(const float* q_rows, long long ld_q, const float* shared_rows, long long ld_s,
                                  const float* latent_norm, float eps, const float* freq, int rot_dims,
                                  const int* positions, const int* slots, const int* block_table, int table_stride,
                                  void* q_plain, void* q_rotated, void* latent_pages, void* key_pages, int dtype,
                                  int n_tokens, int heads, int d, int dr, int rank, int page_size, int num_pages,
                                  int write_kv, int pairs, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (heads <= 0 || d <= 0 || dr <= 0 || rank <= 0 || page_size <= 0 || rot_dims < 0 || rot_dims > dr || (rot_dims & 1) ||
        (rot_dims > 0 && !freq) || ld_q < (long long)heads * (d + dr) || (shared_rows && (ld_s < rank + dr || !latent_norm)) ||
        dr > 4096)
        return LIA_ERR_SIZE;
    const size_t smem = ((size_t)rot_dims + (size_t)PREP_WARPS * dr) * sizeof(float);
#define LIA_PREP(T)                                                                                                  \
    return lia_launch(latent_prepare_kernel<T>, dim3(n_tokens), dim3(PREP_WARPS * 32), smem, stream, q_rows, ld_q,   \
                      shared_rows, ld_s, latent_norm, eps, freq, rot_dims, positions, slots, block_table,            \
                      table_stride, (T*)q_plain, (T*)q_rotated, (T*)latent_pages, (T*)key_pages, n_tokens, heads, d, \
                      dr, rank, page_size, num_pages, write_kv, pairs, error_flag)
    if (dtype == LIA_BF16) LIA_PREP(__nv_bfloat16);
    if (dtype == LIA_F32) LIA_PREP(float);
#undef LIA_PREP
    return LIA_ERR_DTYPE;
}
