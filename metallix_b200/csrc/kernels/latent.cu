// Helpers of attention through a latent: what is cached per position is one
// normalised latent vector c (width `rank`) followed by one rotated key part
// (width `rot`), shared by all heads. Queries meet it as
// [q_absorbed (rank) | q_rotated (rot)] per head, so that a head's score is one
// dot product over rank + rot values and its output a mixture of latents.
//
// latent_cache_kernel: one block per token. c = x[:rank] / rms(x[:rank]) * w
// (float32 inside), the last `rot` values rotated by the token's position,
// both stored at the token's slot of a one-plane page pool
// [pages, 1, 1, page_tokens, rank + rot].
// rotate_into_kernel: for every (token, head) the `rot` values at
// src[token, src_off + head * src_step ...] rotated by the position and
// written to dst[token, head, dst_off ...] (rows of dst hold heads * dst_step).
// Pairs are (2i, 2i + 1) when interleaved, else (i, i + rotary_dim / 2); values
// beyond rotary_dim pass unchanged. cos/sin: float32 [positions, rotary_dim / 2].
#include "common.cuh"

namespace mxb {

template <typename T>
__device__ __forceinline__ float rotated_value(const T* src, int i, int rotary_dim, int interleaved,
                                               const float* cos_row, const float* sin_row) {
  if (i >= rotary_dim) return to_float(src[i]);
  const int half = rotary_dim / 2;
  int pair, first;
  if (interleaved) { pair = i >> 1; first = (i & 1) == 0; }
  else { pair = i < half ? i : i - half; first = i < half; }
  const int other = interleaved ? (first ? i + 1 : i - 1) : (first ? i + half : i - half);
  const float c = cos_row[pair], s = sin_row[pair];
  const float mine = to_float(src[i]), theirs = to_float(src[other]);
  return first ? mine * c - theirs * s : mine * c + theirs * s;
}

template <typename T>
__global__ void latent_cache_kernel(const T* __restrict__ x, long long ld, const float* __restrict__ w, float eps,
                                    int rank, int rot, int rotary_dim, int interleaved,
                                    const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                    int table_positions, const int* __restrict__ positions,
                                    const int* __restrict__ slots, T* __restrict__ cache, int page_tokens,
                                    int num_pages, int* status) {
  chain_release();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int slot = slots != nullptr ? slots[t] : t;   // without slots: row t of a plain [tokens, rank + rot] buffer
  if (slot < 0) return;   // a padding row of a captured step
  const int pos = positions[t];
  if (slot >= num_pages * page_tokens || pos < 0 || (rotary_dim > 0 && pos >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  const T* row = x + static_cast<long long>(t) * ld;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(row[i]);
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float scale = rsqrtf(sum / static_cast<float>(rank) + eps);
  T* dst = cache + static_cast<long long>(slot) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]) * scale * w[i]);
  const float* cos_row = cos_table + static_cast<long long>(pos) * (rotary_dim / 2);
  const float* sin_row = sin_table + static_cast<long long>(pos) * (rotary_dim / 2);
  for (int i = threadIdx.x; i < rot; i += blockDim.x)
    dst[rank + i] = from_float<T>(rotated_value(row + rank, i, rotary_dim, interleaved, cos_row, sin_row));
}

template <typename T>
__global__ void rotate_into_kernel(const T* __restrict__ src, long long ld_src, int src_off, int src_step,
                                   T* __restrict__ dst, int dst_off, int dst_step, int heads, int rot, int rotary_dim,
                                   int interleaved, const float* __restrict__ cos_table,
                                   const float* __restrict__ sin_table, int table_positions,
                                   const int* __restrict__ positions, int* status) {
  chain_release();
  const int t = blockIdx.x;
  int pos = positions[t];
  if (pos < 0 || (rotary_dim > 0 && pos >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    pos = 0;
  }
  const float* cos_row = cos_table + static_cast<long long>(pos) * (rotary_dim / 2);
  const float* sin_row = sin_table + static_cast<long long>(pos) * (rotary_dim / 2);
  for (int e = threadIdx.x; e < heads * rot; e += blockDim.x) {
    const int h = e / rot, i = e - h * rot;
    const T* from = src + static_cast<long long>(t) * ld_src + src_off + h * src_step;
    dst[(static_cast<long long>(t) * heads + h) * dst_step + dst_off + i] =
        from_float<T>(rotated_value(from, i, rotary_dim, interleaved, cos_row, sin_row));
  }
}

// The other way to cache the same attention: per head, whole key and value rows. For every token, head h:
//   q_heads[t, h] = [q_u (D) | rot(q_r) (R) | 0 ...]                       (width `hd`)
//   K row at the token's slot = [k_h (D) | rotated shared key part (R) | 0 ...]
//   V row                      = [v_h (V) | 0 ...]
// q: [tokens, heads * (D + R)] with the rotated part still unrotated; up: [tokens, heads * D + heads * V], the
// keys then the values that the latent was widened to; shared: [tokens, ...] holding the ALREADY rotated shared
// key part from column shared_off on. The pool is [pages, 2, heads, page_tokens, hd].
template <typename T>
__global__ void latent_heads_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ up, long long ld_up,
                                    const T* __restrict__ shared_part, long long ld_shared, int shared_off,
                                    T* __restrict__ q_heads, T* __restrict__ cache, const int* __restrict__ slots,
                                    const int* __restrict__ positions, const float* __restrict__ cos_table,
                                    const float* __restrict__ sin_table, int table_positions, int rotary_dim,
                                    int interleaved, int heads, int D, int R, int V, int hd, int page_tokens,
                                    int num_pages, int* status) {
  chain_release();
  const int t = blockIdx.x;
  int pos = positions[t];
  if (pos < 0 || (rotary_dim > 0 && pos >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    pos = 0;
  }
  const float* cos_row = cos_table + static_cast<long long>(pos) * (rotary_dim / 2);
  const float* sin_row = sin_table + static_cast<long long>(pos) * (rotary_dim / 2);
  const T* q_row = q + static_cast<long long>(t) * ld_q;
  for (int e = threadIdx.x; e < heads * hd; e += blockDim.x) {
    const int h = e / hd, i = e - h * hd;
    float v = 0.0f;
    if (i < D) v = to_float(q_row[h * (D + R) + i]);
    else if (i < D + R) v = rotated_value(q_row + h * (D + R) + D, i - D, rotary_dim, interleaved, cos_row, sin_row);
    q_heads[static_cast<long long>(t) * heads * hd + e] = from_float<T>(v);
  }
  const int slot = slots != nullptr ? slots[t] : -1;
  if (slot < 0) return;
  if (slot >= num_pages * page_tokens) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  const int page = slot / page_tokens, in_page = slot - page * page_tokens;
  const T* up_row = up + static_cast<long long>(t) * ld_up;
  const T* shared_row = shared_part + static_cast<long long>(t) * ld_shared + shared_off;
  for (int e = threadIdx.x; e < heads * hd; e += blockDim.x) {
    const int h = e / hd, i = e - h * hd;
    T key = from_float<T>(0.0f), value = from_float<T>(0.0f);
    if (i < D) key = up_row[h * D + i];
    else if (i < D + R) key = shared_row[i - D];
    if (i < V) value = up_row[heads * D + h * V + i];
    const long long at = ((static_cast<long long>(page) * 2 * heads + h) * page_tokens + in_page) * hd + i;
    cache[at] = key;
    cache[at + static_cast<long long>(heads) * page_tokens * hd] = value;
  }
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_latent_heads(const void* q, long long ld_q, const void* up, long long ld_up, const void* shared_part,
                             long long ld_shared, int shared_off, void* q_heads, void* cache, const int* slots,
                             const int* positions, const float* cos_table, const float* sin_table, int table_positions,
                             int rotary_dim, int interleaved, int heads, int D, int R, int V, int hd, int page_tokens,
                             int num_pages, int tokens, int dtype, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || D + R > hd || V > hd || rotary_dim > R || rotary_dim % 2) return static_cast<int>(cudaErrorInvalidValue);
  if (dtype == kF32)
    latent_heads_kernel<float><<<tokens, 256, 0, stream>>>(
        static_cast<const float*>(q), ld_q, static_cast<const float*>(up), ld_up, static_cast<const float*>(shared_part),
        ld_shared, shared_off, static_cast<float*>(q_heads), static_cast<float*>(cache), slots, positions, cos_table,
        sin_table, table_positions, rotary_dim, interleaved, heads, D, R, V, hd, page_tokens, num_pages, status);
  else if (dtype == kBF16)
    latent_heads_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), ld_q, static_cast<const __nv_bfloat16*>(up), ld_up,
        static_cast<const __nv_bfloat16*>(shared_part), ld_shared, shared_off, static_cast<__nv_bfloat16*>(q_heads),
        static_cast<__nv_bfloat16*>(cache), slots, positions, cos_table, sin_table, table_positions, rotary_dim,
        interleaved, heads, D, R, V, hd, page_tokens, num_pages, status);
  else return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_latent_cache(const void* x, long long ld, const float* w, float eps, int rank, int rot, int rotary_dim,
                             int interleaved, const float* cos_table, const float* sin_table, int table_positions,
                             const int* positions, const int* slots, void* cache, int page_tokens, int num_pages,
                             int tokens, int dtype, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rank <= 0 || rot < 0 || rotary_dim > rot || rotary_dim % 2) return static_cast<int>(cudaErrorInvalidValue);
  const int threads = rank >= 256 ? 256 : 128;
  if (dtype == kF32)
    latent_cache_kernel<float><<<tokens, threads, 0, stream>>>(
        static_cast<const float*>(x), ld, w, eps, rank, rot, rotary_dim, interleaved, cos_table, sin_table,
        table_positions, positions, slots, static_cast<float*>(cache), page_tokens, num_pages, status);
  else if (dtype == kBF16)
    latent_cache_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ld, w, eps, rank, rot, rotary_dim, interleaved, cos_table, sin_table,
        table_positions, positions, slots, static_cast<__nv_bfloat16*>(cache), page_tokens, num_pages, status);
  else return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_rotate_into(const void* src, long long ld_src, int src_off, int src_step, void* dst, int dst_off,
                            int dst_step, int heads, int rot, int rotary_dim, int interleaved, const float* cos_table,
                            const float* sin_table, int table_positions, const int* positions, int tokens, int dtype,
                            int* status, cudaStream_t stream) {
  if (tokens <= 0 || heads <= 0 || rot <= 0) return 0;
  if (rotary_dim > rot || rotary_dim % 2) return static_cast<int>(cudaErrorInvalidValue);
  if (dtype == kF32)
    rotate_into_kernel<float><<<tokens, 128, 0, stream>>>(
        static_cast<const float*>(src), ld_src, src_off, src_step, static_cast<float*>(dst), dst_off, dst_step, heads,
        rot, rotary_dim, interleaved, cos_table, sin_table, table_positions, positions, status);
  else if (dtype == kBF16)
    rotate_into_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), ld_src, src_off, src_step, static_cast<__nv_bfloat16*>(dst), dst_off,
        dst_step, heads, rot, rotary_dim, interleaved, cos_table, sin_table, table_positions, positions, status);
  else return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}
