// A sublayer whose output passes a norm of its own before it joins the
// residual stream ("sandwich" norms: one norm ahead of the sublayer, one
// behind it):
//
//   x <- x + RMSNorm(d) * w_post;   y = RMSNorm(x) * w_next
//
// in one pass over the row: the sublayer's output d is read once, the
// residual stream x (float32) is read and written once, and the input y of
// the next sublayer leaves in the compute type. Both sums of squares and both
// scales are float32. d may be a sum that its producer left in parts
// ([parts, rows, size] float32: the output projection of a decode step taken
// head by head); the parts are added up in their order first. Without w_next
// only the residual sum is made (the last sublayer of a model).
//
// A row's values stay in shared memory as float32 between the passes; every
// thread touches its own elements only, so the block meets just for the two
// sums.
#include "common.cuh"

namespace mxb {

template <typename TDelta, typename TOut>
__global__ void __launch_bounds__(256)
postnorm_add_rmsnorm_kernel(float* __restrict__ x, const TDelta* __restrict__ delta, int parts, size_t part_stride,
                            const float* __restrict__ w_post, float eps_post, TOut* __restrict__ y,
                            const float* __restrict__ w_next, float eps_next, int size) {
  extern __shared__ float held[];   // the row: first d, then x + norm(d)
  __shared__ float scratch[33];
  chain_release();
  const size_t base = static_cast<size_t>(blockIdx.x) * size;
  chain_wait();
  float* row = behind_wait(x) + base;            // both written by kernels ahead of this one
  const TDelta* d_row = behind_wait(delta) + base;

  float sum = 0.0f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    float d = 0.0f;
    for (int part = 0; part < parts; ++part) d += to_float(d_row[part * part_stride + i]);
    held[i] = d;
    sum += d * d;
  }
  sum = block_sum(sum, scratch);
  const float scale_post = rsqrtf(sum / static_cast<float>(size) + eps_post);
  sum = 0.0f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float v = row[i] + held[i] * scale_post * w_post[i];
    row[i] = v;
    held[i] = v;
    sum += v * v;
  }
  if (y == nullptr) return;   // the same for every thread of the launch
  sum = block_sum(sum, scratch);
  const float scale_next = rsqrtf(sum / static_cast<float>(size) + eps_next);
  TOut* dst = y + base;
  for (int i = threadIdx.x; i < size; i += blockDim.x) dst[i] = from_float<TOut>(held[i] * scale_next * w_next[i]);
}

// out[t, i] = a[t, i] * sigmoid(g[t, i]): an output gate over the
// concatenated heads, sigmoid and product in float32. Rows of `a`, `g` and
// `out` may be strided (g is a column range of a wider product).
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ g,
                                    long long out_stride, long long a_stride, long long g_stride, int width,
                                    long long count) {
  chain_release();
  chain_wait();
  a = behind_wait(a);
  g = behind_wait(g);
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= count) return;
  const long long t = index / width;
  const int i = static_cast<int>(index - t * width);
  const float gate = 1.0f / (1.0f + expf(-to_float(g[t * g_stride + i])));
  out[t * out_stride + i] = from_float<T>(to_float(a[t * a_stride + i]) * gate);
}

// x[i] = cap * tanh(x[i] / cap) in place: logits bounded to (-cap, cap).
__global__ void softcap_kernel(float* __restrict__ x, float cap, long long count) {
  chain_release();
  chain_wait();
  x = behind_wait(x);
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace mxb

using namespace mxb;

// delta: [rows, size] of delta_dtype, or (parts > 1, float32 only) [parts, rows, size].
// y / w_next may both be null: only x is updated.
MXB_API int mxb_postnorm_add_rmsnorm(float* x, const void* delta, int delta_dtype, int parts, const float* w_post,
                                     float eps_post, void* y, int y_dtype, const float* w_next, float eps_next,
                                     int rows, int size, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (size <= 0 || parts < 1 || (parts > 1 && delta_dtype != kF32) || (y != nullptr && w_next == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  int threads = 32;
  while (threads < size && threads < 256) threads <<= 1;   // a fixed block size per row width: one order of additions
  const size_t shared = static_cast<size_t>(size) * sizeof(float);
  const size_t part_stride = static_cast<size_t>(rows) * size;
  cudaError_t e = cudaSuccess;
#define LAUNCH(TD, TO) do { \
    auto kernel = postnorm_add_rmsnorm_kernel<TD, TO>; \
    if (shared > 48 * 1024) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)); \
    if (e == cudaSuccess) e = launch_chained(kernel, dim3(rows), dim3(threads), shared, stream, x, static_cast<const TD*>(delta), \
                                             parts, part_stride, w_post, eps_post, static_cast<TO*>(y), w_next, eps_next, size); } while (0)
  const bool out_bf16 = y != nullptr && y_dtype == kBF16;
  if (y != nullptr && y_dtype != kBF16 && y_dtype != kF32) return static_cast<int>(cudaErrorInvalidValue);
  if (delta_dtype == kF32) { if (out_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float); }
  else if (delta_dtype == kBF16) { if (out_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float); }
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(e);
}

MXB_API int mxb_sigmoid_gate(void* out, const void* a, const void* g, long long out_stride, long long a_stride,
                             long long g_stride, int rows, int width, int dtype, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  const long long count = static_cast<long long>(rows) * width;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((count + threads - 1) / threads);
  if (dtype == kF32)
    return static_cast<int>(launch_chained(sigmoid_gate_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
                                           static_cast<float*>(out), static_cast<const float*>(a),
                                           static_cast<const float*>(g), out_stride, a_stride, g_stride, width, count));
  if (dtype == kBF16)
    return static_cast<int>(launch_chained(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
                                           static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(a),
                                           static_cast<const __nv_bfloat16*>(g), out_stride, a_stride, g_stride,
                                           width, count));
  return static_cast<int>(cudaErrorInvalidValue);
}

MXB_API int mxb_softcap(float* x, float cap, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!(cap > 0.0f)) return static_cast<int>(cudaErrorInvalidValue);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((count + threads - 1) / threads);
  return static_cast<int>(launch_chained(softcap_kernel, dim3(blocks), dim3(threads), 0, stream, x, cap, count));
}
