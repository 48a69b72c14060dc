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

// V values per access: 4 where rows are a multiple of four wide and start on
// 16-byte boundaries (8 for a bfloat16 delta), else 1.
__device__ __forceinline__ float4 sn_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 sn_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void sn_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void sn_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&lo);
  raw.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// PARTS: the delta comes in parts (their loads in flight together take
// registers that the common case, a whole delta, leaves to more resident blocks).
template <typename TDelta, typename TOut, bool VEC4, bool PARTS>
__global__ void __launch_bounds__(256)
postnorm_add_rmsnorm_kernel(float* __restrict__ x, const TDelta* __restrict__ delta, int parts, size_t part_stride,
                            const float* __restrict__ w_post, float eps_post, TOut* __restrict__ y,
                            const float* __restrict__ w_next, float eps_next, int size) {
  extern __shared__ __align__(16) float held[];   // the row: first d, then x + norm(d)
  __shared__ float scratch[33];
  constexpr int V = VEC4 ? 4 : 1;
  constexpr int BATCH = 16;   // parts whose loads are on their way before the first of them is added
  chain_release();
  const size_t base = static_cast<size_t>(blockIdx.x) * size;
  const int first = threadIdx.x * V, step = blockDim.x * V;
  // The norms' weights for the thread's first values are fetched before the
  // wait for the kernel that produces the delta (for rows up to 4 * blockDim.x
  // wide that is all of them).
  float4 first_post = make_float4(0.0f, 0.0f, 0.0f, 0.0f), first_next = first_post;
  if (VEC4 && first < size) {
    first_post = sn_load4(w_post + first);
    if (y != nullptr) first_next = sn_load4(w_next + first);
  }
  chain_wait();
  float* row = behind_wait(x) + base;            // both written by kernels ahead of this one
  const TDelta* d_row = behind_wait(delta) + base;

  float sum = 0.0f;
  for (int i = first; i < size; i += step) {
    if (VEC4) {
      prefetch_line(row + i);   // the second pass reads it
      float4 d = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (!PARTS) {
        d = sn_load4(d_row + i);
      } else {
        // a loop of one load and one add would make a trip to memory per part
        for (int part = 0; part < parts; part += BATCH) {
          float4 more[BATCH];
#pragma unroll
          for (int j = 0; j < BATCH; ++j) more[j] = sn_load4(d_row + min(part + j, parts - 1) * part_stride + i);
#pragma unroll
          for (int j = 0; j < BATCH; ++j)
            if (part + j < parts) { d.x += more[j].x; d.y += more[j].y; d.z += more[j].z; d.w += more[j].w; }
        }
      }
      *reinterpret_cast<float4*>(held + i) = d;
      sum += d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w;
    } else {
      float d = 0.0f;
      for (int part = 0; part < (PARTS ? parts : 1); ++part) d += to_float(d_row[part * part_stride + i]);
      held[i] = d;
      sum += d * d;
    }
  }
  sum = block_sum(sum, scratch);
  const float scale_post = rsqrtf(sum / static_cast<float>(size) + eps_post);
  sum = 0.0f;
  for (int i = first; i < size; i += step) {
    if (VEC4) {
      const float4 d = *reinterpret_cast<const float4*>(held + i), g = i == first ? first_post : sn_load4(w_post + i);
      float4 v = sn_load4(row + i);
      v.x += d.x * scale_post * g.x; v.y += d.y * scale_post * g.y;
      v.z += d.z * scale_post * g.z; v.w += d.w * scale_post * g.w;
      sn_store4(row + i, v);
      *reinterpret_cast<float4*>(held + i) = v;
      sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      const float v = row[i] + held[i] * scale_post * w_post[i];
      row[i] = v;
      held[i] = v;
      sum += v * v;
    }
  }
  if (y == nullptr) return;   // the same for every thread of the launch
  sum = block_sum(sum, scratch);
  const float scale_next = rsqrtf(sum / static_cast<float>(size) + eps_next);
  TOut* dst = y + base;
  for (int i = first; i < size; i += step) {
    if (VEC4) {
      const float4 v = *reinterpret_cast<const float4*>(held + i), g = i == first ? first_next : sn_load4(w_next + i);
      sn_store4(dst + i, make_float4(v.x * scale_next * g.x, v.y * scale_next * g.y, v.z * scale_next * g.z,
                                     v.w * scale_next * g.w));
    } else {
      dst[i] = from_float<TOut>(held[i] * scale_next * w_next[i]);
    }
  }
}

// out[t, i] = a[t, i] * sigmoid(g[t, i]): an output gate over the
// concatenated heads, sigmoid and product in float32. Rows of `a`, `g` and
// `out` may be strided (g is a column range of a wider product). V values per
// thread, one access of V * sizeof(T) bytes each way where rows allow it.
template <typename T, int V>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ g,
                                    long long out_stride, long long a_stride, long long g_stride, int width,
                                    long long count) {
  struct alignas(sizeof(T) * V) Values { T v[V]; };
  chain_release();
  chain_wait();
  a = behind_wait(a);
  g = behind_wait(g);
  const long long index = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
  if (index >= count) return;
  const long long t = index / width;
  const int i = static_cast<int>(index - t * width);   // V divides width: a vector stays in its row
  const Values av = *reinterpret_cast<const Values*>(a + t * a_stride + i);
  const Values gv = *reinterpret_cast<const Values*>(g + t * g_stride + i);
  Values ov;
#pragma unroll
  for (int j = 0; j < V; ++j)
    ov.v[j] = from_float<T>(to_float(av.v[j]) * (1.0f / (1.0f + expf(-to_float(gv.v[j])))));
  *reinterpret_cast<Values*>(out + t * out_stride + i) = ov;
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
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  // four values per access: rows a multiple of four wide (eight for a bfloat16 delta or output, whose four
  // values are eight bytes) on 16-byte boundaries
  const bool narrow = delta_dtype == kBF16 || (y != nullptr && y_dtype == kBF16);
  const bool vec4 = size % (narrow ? 8 : 4) == 0 && aligned(x) && aligned(delta) && aligned(w_post) &&
                    aligned(y) && aligned(w_next);
  if (vec4) {
    threads = 32;
    while (threads * 4 < size && threads < 256) threads <<= 1;
  }
#define LAUNCH(TD, TO) do { \
    if (vec4) { if (parts > 1) LAUNCH_AS(TD, TO, true, true); else LAUNCH_AS(TD, TO, true, false); } \
    else { if (parts > 1) LAUNCH_AS(TD, TO, false, true); else LAUNCH_AS(TD, TO, false, false); } } while (0)
#define LAUNCH_AS(TD, TO, VEC, MANY) do { \
    auto kernel = postnorm_add_rmsnorm_kernel<TD, TO, VEC, MANY>; \
    if (shared > 48 * 1024) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)); \
    if (e == cudaSuccess) e = launch_chained(kernel, dim3(rows), dim3(threads), shared, stream, x, static_cast<const TD*>(delta), \
                                             parts, part_stride, w_post, eps_post, static_cast<TO*>(y), w_next, eps_next, size); } while (0)
  const bool out_bf16 = y != nullptr && y_dtype == kBF16;
  if (y != nullptr && y_dtype != kBF16 && y_dtype != kF32) return static_cast<int>(cudaErrorInvalidValue);
  if (delta_dtype == kF32) { if (out_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float); }
  else if (delta_dtype == kBF16) { if (out_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float); }
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
#undef LAUNCH_AS
  return static_cast<int>(e);
}

MXB_API int mxb_sigmoid_gate(void* out, const void* a, const void* g, long long out_stride, long long a_stride,
                             long long g_stride, int rows, int width, int dtype, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (dtype != kF32 && dtype != kBF16) return static_cast<int>(cudaErrorInvalidValue);
  const long long count = static_cast<long long>(rows) * width;
  const int element = dtype == kF32 ? 4 : 2, vector = 16 / element;
  auto fits = [&](const void* p, long long stride) {
    return reinterpret_cast<uintptr_t>(p) % 16 == 0 && (stride * element) % 16 == 0;
  };
  const bool wide = width % vector == 0 && fits(out, out_stride) && fits(a, a_stride) && fits(g, g_stride);
  const int threads = 256;
  const long long items = wide ? count / vector : count;
  const unsigned blocks = static_cast<unsigned>((items + threads - 1) / threads);
#define GATE(T, V) return static_cast<int>(launch_chained(sigmoid_gate_kernel<T, V>, dim3(blocks), dim3(threads), 0, stream, \
      static_cast<T*>(out), static_cast<const T*>(a), static_cast<const T*>(g), out_stride, a_stride, g_stride, width, count))
  if (dtype == kF32) { if (wide) GATE(float, 4); GATE(float, 1); }
  if (wide) GATE(__nv_bfloat16, 8);
  GATE(__nv_bfloat16, 1);
#undef GATE
}

MXB_API int mxb_softcap(float* x, float cap, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!(cap > 0.0f)) return static_cast<int>(cudaErrorInvalidValue);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((count + threads - 1) / threads);
  return static_cast<int>(launch_chained(softcap_kernel, dim3(blocks), dim3(threads), 0, stream, x, cap, count));
}

MXB_TIMELINE_EXPORT(mxb_timeline_sandwich_norms)
