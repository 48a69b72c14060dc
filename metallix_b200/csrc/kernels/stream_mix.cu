// Several residual streams (hyper-connections) and the Dynamic Tanh norm.
//
// A model may carry s copies of the residual stream, x[token, stream, :] in
// float32. A sublayer reads one mixture of them, u = sum_s in[s] x_s, and its
// result y is written back to all of them at once:
//   x_t <- sum_s mix[s, t] x_s + out[t] * (scale ⊙ y)
// with `scale` an optional per-channel factor (layer scale) and y = a * y_a +
// b * y_b the weighted sum of up to two results (two mixers side by side).
// Both halves are one pass over the row here: the write of the sublayer that
// has just finished, then the read (and the norm) for the one that follows,
// the way add_rmsnorm folds a residual sum into the next norm. With s = 1,
// mix = out = in = 1 this is the ordinary residual sum.
//
// The norm that follows the read is elementwise, so nothing is reduced over a
// row: Dynamic Tanh, y = tanh(alpha * u) * w + b (alpha a scalar), or none (u
// itself leaves, for a norm part that runs afterwards). Sums, tanh and the
// streams are float32 in both precisions.
#include "common.cuh"

namespace mxb {

constexpr int kMaxStreams = 8;
constexpr int kMixThreads = 256;

struct StreamMixArgs {
  float* streams;            // [tokens, s, width], updated in place when a result is given
  const void* result_a;      // [tokens, width] rows of stride lda, or null: nothing is written back
  const void* result_b;      // second result or null
  long long lda, ldb;
  float weight_a, weight_b;
  const float* channel_scale;  // [width] or null
  const float* mix;            // [s, s] indexed [from, to]
  const float* out_weights;    // [s]
  const float* in_weights;     // [s] or null: the plain sum of the streams is read
  const float* alpha;          // Dynamic Tanh: scalar on the device; null: no norm, u leaves as it is
  const float* norm_weight;    // [width]
  const float* norm_bias;      // [width] or null
  void* normed;                // [rows, width] or null: nothing is read
  const int* rows_index;       // optional: only these rows (of tokens) are worked on
  int rows, width, count;      // count = s
  int keep_streams;            // 0: the streams are not written (the last read of a step)
};

template <typename TResult, typename TOut>
__global__ void __launch_bounds__(kMixThreads) stream_mix_kernel(StreamMixArgs a) {
  chain_release();   // the kernel behind may start and fetch what no kernel writes (its weights) meanwhile
  __shared__ float s_mix[kMaxStreams * kMaxStreams], s_out[kMaxStreams], s_in[kMaxStreams];
  const int s = a.count;
  if (threadIdx.x < s * s) s_mix[threadIdx.x] = a.mix != nullptr ? a.mix[threadIdx.x] : 0.0f;
  if (threadIdx.x < s) {
    s_out[threadIdx.x] = a.out_weights != nullptr ? a.out_weights[threadIdx.x] : 0.0f;
    s_in[threadIdx.x] = a.in_weights != nullptr ? a.in_weights[threadIdx.x] : 1.0f;
  }
  __syncthreads();
  const float alpha = a.alpha != nullptr ? a.alpha[0] : 0.0f;
  const long long total = static_cast<long long>(a.rows) * a.width;
  for (long long i = static_cast<long long>(blockIdx.x) * kMixThreads + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kMixThreads) {
    const int r = static_cast<int>(i / a.width), c = static_cast<int>(i - static_cast<long long>(r) * a.width);
    const long long token = a.rows_index != nullptr ? a.rows_index[r] : r;
    float* x = a.streams + (token * s) * a.width + c;
    float v[kMaxStreams];
#pragma unroll
    for (int j = 0; j < kMaxStreams; ++j) v[j] = j < s ? x[static_cast<long long>(j) * a.width] : 0.0f;
    if (a.result_a != nullptr) {
      float y = a.weight_a * to_float(static_cast<const TResult*>(a.result_a)[token * a.lda + c]);
      if (a.result_b != nullptr) y += a.weight_b * to_float(static_cast<const TResult*>(a.result_b)[token * a.ldb + c]);
      if (a.channel_scale != nullptr) y *= a.channel_scale[c];
      float w[kMaxStreams];
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < kMaxStreams; ++j)
          if (j < s && t < s) sum = fmaf(s_mix[j * s + t], v[j], sum);
        w[t] = t < s ? fmaf(s_out[t], y, sum) : 0.0f;
      }
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        v[t] = w[t];
        if (t < s && a.keep_streams) x[static_cast<long long>(t) * a.width] = w[t];
      }
    }
    if (a.normed != nullptr) {
      float u = 0.0f;
#pragma unroll
      for (int j = 0; j < kMaxStreams; ++j)
        if (j < s) u = fmaf(s_in[j], v[j], u);
      if (a.alpha != nullptr) {
        u = tanhf(alpha * u) * a.norm_weight[c];
        if (a.norm_bias != nullptr) u += a.norm_bias[c];
      }
      static_cast<TOut*>(a.normed)[static_cast<long long>(r) * a.width + c] = from_float<TOut>(u);
    }
  }
}

// Four columns per thread at a time, for widths that are multiples of 4 and rows that start on 16-byte
// boundaries (8 for bfloat16): 16-byte loads and stores of the streams.
__device__ __forceinline__ float4 read4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 read4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void write4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void write4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// SM bounds the number of streams (1, 2, 4 or 8), so that a model with few of them holds few registers.
template <typename TResult, typename TOut, int SM>
__global__ void __launch_bounds__(kMixThreads) stream_mix_by4_kernel(StreamMixArgs a) {
  chain_release();   // the kernel behind may start and fetch what no kernel writes (its weights) meanwhile
  __shared__ float s_mix[kMaxStreams * kMaxStreams], s_out[kMaxStreams], s_in[kMaxStreams];
  const int s = a.count;
  if (threadIdx.x < s * s) s_mix[threadIdx.x] = a.mix != nullptr ? a.mix[threadIdx.x] : 0.0f;
  if (threadIdx.x < s) {
    s_out[threadIdx.x] = a.out_weights != nullptr ? a.out_weights[threadIdx.x] : 0.0f;
    s_in[threadIdx.x] = a.in_weights != nullptr ? a.in_weights[threadIdx.x] : 1.0f;
  }
  __syncthreads();
  const float alpha = a.alpha != nullptr ? a.alpha[0] : 0.0f;
  const int quads = a.width / 4;
  const long long total = static_cast<long long>(a.rows) * quads;
  for (long long i = static_cast<long long>(blockIdx.x) * kMixThreads + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kMixThreads) {
    const int r = static_cast<int>(i / quads), c = 4 * static_cast<int>(i - static_cast<long long>(r) * quads);
    const long long token = a.rows_index != nullptr ? a.rows_index[r] : r;
    float* x = a.streams + (token * s) * a.width + c;
    float v[SM][4];
#pragma unroll
    for (int j = 0; j < SM; ++j) {
      const float4 q = j < s ? read4(x + static_cast<long long>(j) * a.width) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[j][0] = q.x; v[j][1] = q.y; v[j][2] = q.z; v[j][3] = q.w;
    }
    if (a.result_a != nullptr) {
      const float4 ya = read4(static_cast<const TResult*>(a.result_a) + token * a.lda + c);
      float y[4] = {a.weight_a * ya.x, a.weight_a * ya.y, a.weight_a * ya.z, a.weight_a * ya.w};
      if (a.result_b != nullptr) {
        const float4 yb = read4(static_cast<const TResult*>(a.result_b) + token * a.ldb + c);
        y[0] += a.weight_b * yb.x; y[1] += a.weight_b * yb.y; y[2] += a.weight_b * yb.z; y[3] += a.weight_b * yb.w;
      }
      if (a.channel_scale != nullptr) {
        const float4 g = read4(a.channel_scale + c);
        y[0] *= g.x; y[1] *= g.y; y[2] *= g.z; y[3] *= g.w;
      }
      float w[SM][4];
#pragma unroll
      for (int t = 0; t < SM; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float sum = 0.0f;
#pragma unroll
          for (int j = 0; j < SM; ++j)
            if (j < s && t < s) sum = fmaf(s_mix[j * s + t], v[j][e], sum);
          w[t][e] = t < s ? fmaf(s_out[t], y[e], sum) : 0.0f;
        }
      }
#pragma unroll
      for (int t = 0; t < SM; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[t][e] = w[t][e];
        if (t < s && a.keep_streams)
          write4(x + static_cast<long long>(t) * a.width, make_float4(w[t][0], w[t][1], w[t][2], w[t][3]));
      }
    }
    if (a.normed != nullptr) {
      float u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < SM; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (j < s) u[e] = fmaf(s_in[j], v[j][e], u[e]);
      }
      if (a.alpha != nullptr) {
        const float4 g = read4(a.norm_weight + c);
        const float4 b = a.norm_bias != nullptr ? read4(a.norm_bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        u[0] = tanhf(alpha * u[0]) * g.x + b.x;
        u[1] = tanhf(alpha * u[1]) * g.y + b.y;
        u[2] = tanhf(alpha * u[2]) * g.z + b.z;
        u[3] = tanhf(alpha * u[3]) * g.w + b.w;
      }
      write4(static_cast<TOut*>(a.normed) + static_cast<long long>(r) * a.width + c, make_float4(u[0], u[1], u[2], u[3]));
    }
  }
}

// out[r, c] = a * x[r, c] + b * y[r, c] in float32 (rows may be strided).
template <typename T>
__global__ void __launch_bounds__(kMixThreads) weighted_sum_kernel(float* __restrict__ out, const T* __restrict__ x,
                                                                   const T* __restrict__ y, long long ldx, long long ldy,
                                                                   float a, float b, int rows, int width) {
  chain_release();
  const long long total = static_cast<long long>(rows) * width;
  for (long long i = static_cast<long long>(blockIdx.x) * kMixThreads + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kMixThreads) {
    const long long r = i / width, c = i - r * width;
    out[i] = a * to_float(x[r * ldx + c]) + b * to_float(y[r * ldy + c]);
  }
}

}  // namespace mxb

using namespace mxb;

// See StreamMixArgs. result_dtype: element type of the results; out_dtype: of `normed`.
MXB_API int mxb_stream_mix(float* streams, const void* result_a, const void* result_b, long long lda, long long ldb,
                           float weight_a, float weight_b, int result_dtype, const float* channel_scale,
                           const float* mix, const float* out_weights, const float* in_weights, const float* alpha,
                           const float* norm_weight, const float* norm_bias, void* normed, int out_dtype,
                           const int* rows_index, int rows, int width, int count, int keep_streams,
                           cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (count <= 0 || count > kMaxStreams) return static_cast<int>(cudaErrorInvalidValue);
  StreamMixArgs a{streams, result_a, result_b, lda, ldb, weight_a, weight_b, channel_scale, mix, out_weights,
                  in_weights, alpha, norm_weight, norm_bias, normed, rows_index, rows, width, count, keep_streams};
  // four columns per thread where every row of everything starts on a boundary of four values
  const size_t result_bytes = result_dtype == kF32 ? 4 : 2, out_bytes = out_dtype == kF32 ? 4 : 2;
  auto aligned = [](const void* p, size_t bytes) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % bytes == 0; };
  const bool by4 = width % 4 == 0 && aligned(streams, 16) && aligned(result_a, 4 * result_bytes) &&
                   aligned(result_b, 4 * result_bytes) && lda % 4 == 0 && ldb % 4 == 0 && aligned(channel_scale, 16) &&
                   aligned(norm_weight, 16) && aligned(norm_bias, 16) && aligned(normed, 4 * out_bytes);
  const long long total = static_cast<long long>(rows) * (by4 ? width / 4 : width);
  long long blocks = (total + kMixThreads - 1) / kMixThreads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  const dim3 grid(static_cast<unsigned>(blocks));
#define LAUNCH(TR, TO)                                                                              \
  if (by4 && count == 1) stream_mix_by4_kernel<TR, TO, 1><<<grid, kMixThreads, 0, stream>>>(a);      \
  else if (by4 && count == 2) stream_mix_by4_kernel<TR, TO, 2><<<grid, kMixThreads, 0, stream>>>(a); \
  else if (by4 && count <= 4) stream_mix_by4_kernel<TR, TO, 4><<<grid, kMixThreads, 0, stream>>>(a); \
  else if (by4) stream_mix_by4_kernel<TR, TO, 8><<<grid, kMixThreads, 0, stream>>>(a);               \
  else stream_mix_kernel<TR, TO><<<grid, kMixThreads, 0, stream>>>(a)
  if (result_dtype == kF32 && out_dtype == kF32) { LAUNCH(float, float); }
  else if (result_dtype == kF32 && out_dtype == kBF16) { LAUNCH(float, __nv_bfloat16); }
  else if (result_dtype == kBF16 && out_dtype == kF32) { LAUNCH(__nv_bfloat16, float); }
  else if (result_dtype == kBF16 && out_dtype == kBF16) { LAUNCH(__nv_bfloat16, __nv_bfloat16); }
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_weighted_sum(float* out, const void* x, const void* y, long long ldx, long long ldy, float a, float b,
                             int rows, int width, int dtype, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  const long long total = static_cast<long long>(rows) * width;
  long long blocks = (total + kMixThreads - 1) / kMixThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == kF32)
    weighted_sum_kernel<float><<<static_cast<unsigned>(blocks), kMixThreads, 0, stream>>>(
        out, static_cast<const float*>(x), static_cast<const float*>(y), ldx, ldy, a, b, rows, width);
  else if (dtype == kBF16)
    weighted_sum_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), kMixThreads, 0, stream>>>(
        out, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), ldx, ldy, a, b, rows, width);
  else return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}
