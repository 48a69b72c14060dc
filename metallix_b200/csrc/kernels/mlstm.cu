// The matrix-memory recurrence (mLSTM) with its state in the cache's slots.
//
// Per head, with key width D and value width V, a request carries a matrix
// C [D, V], a vector n [D] and a running maximum m, all float32, zero at the
// start of a sequence. A token brings q (already to be scaled by D^-1/2), k, v
// and two gate pre-activations; with a cap c on the gates
//   i = c tanh((gi + bi) / c),   f = logsigmoid(c tanh((gf + bf) / c)),
//   m' = max(f + m, i),  a = exp(f + m - m'),  b = exp(i - m'),
//   C' = a C + b k v^T,  n' = a n + b k,
//   o  = C'^T q / (max(|n' . q|, exp(-m')) + 1e-6).
// Everything here is float32 whatever the projections' type.
//
// One block owns a slice of 32 value columns of one head of one request and
// walks that request's tokens of the step in order, its slice of C in shared
// memory; a decode step and a portion of a prompt are the same kernel, and a
// position's output does not depend on how the tokens were cut into steps
// (the state that is carried is exact). Each slice keeps n and m for itself
// (they are a few values), so that no block reads what another one writes.
// State of one slot: per head [C: D * V][n: slices * D][m: slices]. Key widths up to 256 run a form that
// keeps C in registers and fetches a token ahead; wider ones the form with C in shared memory.
//
// The second kernel is what follows the recurrence: each head's output over
// its root mean square, times a weight over all heads, times sigmoid of a
// gate taken from the projections.
#include "common.cuh"

namespace mxb {

constexpr int kSliceColumns = 32;
constexpr int kScanParts = 4;
constexpr int kScanThreads = kSliceColumns * kScanParts;

__device__ __forceinline__ float log_sigmoid(float z) {
  return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
mlstm_scan_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int i_off, int f_off,
                  const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                  float* __restrict__ state, long long slot_stride, int num_slots,
                  const int* __restrict__ row_start, const int* __restrict__ row_length,
                  const int* __restrict__ request_slots, float* __restrict__ out, int heads, int dim, int vdim,
                  int* status) {
  extern __shared__ float shared[];
  float* sC = shared;                         // [dim][32]
  float* sn = sC + dim * kSliceColumns;       // [dim]
  float* sq = sn + dim;                       // [dim]
  float* sk = sq + dim;                       // [dim]
  float* red = sk + dim;                      // [parts][32]
  float* red_nq = red + kScanParts * kSliceColumns;   // [parts]

  const int row = blockIdx.x, head = blockIdx.y, slice = blockIdx.z;
  const int length = row_length[row];
  if (length <= 0) return;
  const int slot = request_slots[row];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  const int first = row_start[row];
  const int slices = (vdim + kSliceColumns - 1) / kSliceColumns;
  const int col = threadIdx.x & (kSliceColumns - 1), part = threadIdx.x / kSliceColumns;
  const int j = slice * kSliceColumns + col;
  const bool col_ok = j < vdim;
  const long long head_stride = static_cast<long long>(dim) * vdim + static_cast<long long>(slices) * (dim + 1);
  float* C = state + slot * slot_stride + head * head_stride;
  float* n_state = C + static_cast<long long>(dim) * vdim + static_cast<long long>(slice) * dim;
  float* m_state = C + static_cast<long long>(dim) * vdim + static_cast<long long>(slices) * dim + slice;

  for (int d = part; d < dim; d += kScanParts)
    sC[d * kSliceColumns + col] = col_ok ? C[static_cast<long long>(d) * vdim + j] : 0.0f;
  for (int d = threadIdx.x; d < dim; d += kScanThreads) sn[d] = n_state[d];
  float m = m_state[0];
  const float bi = i_bias[head], bf = f_bias[head];
  const int out_width = heads * vdim;

  for (int t = 0; t < length; ++t) {
    const T* x = proj + static_cast<long long>(first + t) * ld;
    __syncthreads();   // the token before is done with sq, sk, sn and red
    for (int d = threadIdx.x; d < dim; d += kScanThreads) {
      sq[d] = to_float(x[q_off + head * dim + d]) * q_scale;
      sk[d] = to_float(x[k_off + head * dim + d]);
    }
    const float ig = cap * tanhf((to_float(x[i_off + head]) + bi) / cap);
    const float fg = log_sigmoid(cap * tanhf((to_float(x[f_off + head]) + bf) / cap));
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), b = expf(ig - m_new);
    m = m_new;
    const float bv = col_ok ? b * to_float(x[v_off + head * vdim + j]) : 0.0f;
    __syncthreads();
    float acc = 0.0f, nq = 0.0f;
    for (int d = part; d < dim; d += kScanParts) {
      const float kd = sk[d], qd = sq[d];
      const float c = fmaf(a, sC[d * kSliceColumns + col], kd * bv);
      sC[d * kSliceColumns + col] = c;
      acc = fmaf(c, qd, acc);
      const float nn = fmaf(a, sn[d], b * kd);   // the same in all 32 lanes of this warp
      __syncwarp();
      if (col == 0) sn[d] = nn;
      nq = fmaf(nn, qd, nq);
    }
    red[part * kSliceColumns + col] = acc;
    if (col == 0) red_nq[part] = nq;
    __syncthreads();
    if (part == 0 && col_ok) {
      float num = 0.0f, dot = 0.0f;
#pragma unroll
      for (int p = 0; p < kScanParts; ++p) {
        num += red[p * kSliceColumns + col];
        dot += red_nq[p];
      }
      const float den = fmaxf(fabsf(dot), expf(-m)) + 1.0e-6f;
      out[static_cast<long long>(first + t) * out_width + head * vdim + j] = num / den;
    }
  }
  __syncthreads();
  for (int d = part; d < dim; d += kScanParts)
    if (col_ok) C[static_cast<long long>(d) * vdim + j] = sC[d * kSliceColumns + col];
  for (int d = threadIdx.x; d < dim; d += kScanThreads) n_state[d] = sn[d];
  if (threadIdx.x == 0) m_state[0] = m;
}

// The same walk for key widths up to 4 * R (R a template parameter, up to 64): this thread's rows of its
// column of C stay in registers, the inputs of the next token are asked for while the current one is worked
// on, and what the threads share of a token (q, k, the partial sums) has two copies used in turn, so that a
// token costs two barriers.
template <typename T, int R>
__global__ void __launch_bounds__(kScanThreads)
mlstm_scan_registers_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int i_off,
                            int f_off, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                            float q_scale, float* __restrict__ state, long long slot_stride, int num_slots,
                            const int* __restrict__ row_start, const int* __restrict__ row_length,
                            const int* __restrict__ request_slots, float* __restrict__ out, int heads, int dim, int vdim,
                            int* status) {
  constexpr int kMaxDim = 4 * R;
  __shared__ float sq[2][kMaxDim], sk[2][kMaxDim], sn[kMaxDim];
  __shared__ float red[2][kScanParts * kSliceColumns], red_nq[2][kScanParts];
  const int row = blockIdx.x, head = blockIdx.y, slice = blockIdx.z;
  const int length = row_length[row];
  if (length <= 0) return;
  const int slot = request_slots[row];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  const int first = row_start[row];
  const int slices = (vdim + kSliceColumns - 1) / kSliceColumns;
  const int col = threadIdx.x & (kSliceColumns - 1), part = threadIdx.x / kSliceColumns;
  const int j = slice * kSliceColumns + col;
  const bool col_ok = j < vdim;
  const long long head_stride = static_cast<long long>(dim) * vdim + static_cast<long long>(slices) * (dim + 1);
  float* C = state + slot * slot_stride + head * head_stride;
  float* n_state = C + static_cast<long long>(dim) * vdim + static_cast<long long>(slice) * dim;
  float* m_state = C + static_cast<long long>(dim) * vdim + static_cast<long long>(slices) * dim + slice;

  float c[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = part + kScanParts * r;
    c[r] = d < dim && col_ok ? C[static_cast<long long>(d) * vdim + j] : 0.0f;
  }
  for (int d = threadIdx.x; d < dim; d += kScanThreads) sn[d] = n_state[d];
  float m = m_state[0];
  const float bi = i_bias[head], bf = f_bias[head];
  const int out_width = heads * vdim;
  const int d0 = threadIdx.x, d1 = threadIdx.x + kScanThreads;   // the values of q and k this thread stages

  // inputs of a token, fetched one token ahead
  float nq0 = 0.0f, nq1 = 0.0f, nk0 = 0.0f, nk1 = 0.0f, nv = 0.0f, ni = 0.0f, nf = 0.0f;
  auto fetch = [&](int t) {
    const T* x = proj + static_cast<long long>(first + t) * ld;
    if (d0 < dim) { nq0 = to_float(x[q_off + head * dim + d0]); nk0 = to_float(x[k_off + head * dim + d0]); }
    if (d1 < dim) { nq1 = to_float(x[q_off + head * dim + d1]); nk1 = to_float(x[k_off + head * dim + d1]); }
    nv = col_ok ? to_float(x[v_off + head * vdim + j]) : 0.0f;
    ni = to_float(x[i_off + head]);
    nf = to_float(x[f_off + head]);
  };
  fetch(0);
  for (int t = 0; t < length; ++t) {
    const int turn = t & 1;
    if (d0 < dim) { sq[turn][d0] = nq0 * q_scale; sk[turn][d0] = nk0; }
    if (d1 < dim) { sq[turn][d1] = nq1 * q_scale; sk[turn][d1] = nk1; }
    const float ig = cap * tanhf((ni + bi) / cap);
    const float fg = log_sigmoid(cap * tanhf((nf + bf) / cap));
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), b = expf(ig - m_new);
    m = m_new;
    const float bv = b * nv;
    __syncthreads();   // q and k of this token are staged; the token before is done with sn and the other copies
    if (t + 1 < length) fetch(t + 1);
    float acc = 0.0f, nq = 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = part + kScanParts * r;
      if (d < dim) {
        const float kd = sk[turn][d], qd = sq[turn][d];
        c[r] = fmaf(a, c[r], kd * bv);
        acc = fmaf(c[r], qd, acc);
        const float nn = fmaf(a, sn[d], b * kd);   // the same in all 32 lanes of this warp
        __syncwarp();
        if (col == 0) sn[d] = nn;
        nq = fmaf(nn, qd, nq);
      }
    }
    red[turn][part * kSliceColumns + col] = acc;
    if (col == 0) red_nq[turn][part] = nq;
    __syncthreads();
    if (part == 0 && col_ok) {
      float num = 0.0f, dot = 0.0f;
#pragma unroll
      for (int p = 0; p < kScanParts; ++p) {
        num += red[turn][p * kSliceColumns + col];
        dot += red_nq[turn][p];
      }
      const float den = fmaxf(fabsf(dot), expf(-m)) + 1.0e-6f;
      out[static_cast<long long>(first + t) * out_width + head * vdim + j] = num / den;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = part + kScanParts * r;
    if (d < dim && col_ok) C[static_cast<long long>(d) * vdim + j] = c[r];
  }
  for (int d = threadIdx.x; d < dim; d += kScanThreads) n_state[d] = sn[d];
  if (threadIdx.x == 0) m_state[0] = m;
}

// y[t, h, :] = x[t, h, :] * rsqrt(mean_v(x^2) + eps) * w[h, :] * sigmoid(g[t, h, :]); one warp per (t, h).
template <typename TGate, typename TOut>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, const TGate* __restrict__ gate,
                      long long ldg, TOut* __restrict__ y, int pairs, int heads, int vdim, float eps) {
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= pairs) return;
  const int t = pair / heads, h = pair - t * heads;
  const float* row = x + static_cast<long long>(pair) * vdim;
  float sum = 0.0f;
  for (int j = lane; j < vdim; j += 32) sum = fmaf(row[j], row[j], sum);
  sum = warp_sum(sum);
  const float scale = rsqrtf(sum / static_cast<float>(vdim) + eps);
  const TGate* g = gate != nullptr ? gate + static_cast<long long>(t) * ldg + h * vdim : nullptr;
  TOut* dst = y + static_cast<long long>(pair) * vdim;
  for (int j = lane; j < vdim; j += 32) {
    float v = row[j] * scale * w[h * vdim + j];
    if (g != nullptr) v *= sigmoid_of(to_float(g[j]));
    dst[j] = from_float<TOut>(v);
  }
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_mlstm_state_values(int heads, int dim, int vdim) {
  const int slices = (vdim + kSliceColumns - 1) / kSliceColumns;
  return heads * (dim * vdim + slices * (dim + 1));
}

// proj: [tokens, ld] of `dtype` holding q, k (heads * dim each), v (heads * vdim) and the two gates (heads each)
// at the given column offsets. rows: requests of the step; row r brings row_length[r] tokens (0: a padding row,
// nothing is read or written) from packed token row_start[r] on. out: float32 [tokens, heads * vdim].
MXB_API int mxb_mlstm_scan(const void* proj, long long ld, int q_off, int k_off, int v_off, int i_off, int f_off,
                           const float* i_bias, const float* f_bias, float cap, float q_scale, float* state,
                           long long slot_stride, int num_slots, const int* row_start, const int* row_length,
                           const int* request_slots, float* out, int rows, int heads, int dim, int vdim, int dtype,
                           int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || !(cap > 0.0f)) return static_cast<int>(cudaErrorInvalidValue);
  const int slices = (vdim + kSliceColumns - 1) / kSliceColumns;
  const size_t shared = sizeof(float) * (static_cast<size_t>(dim) * kSliceColumns + 3 * static_cast<size_t>(dim) +
                                         kScanParts * kSliceColumns + kScanParts);
  const dim3 grid(rows, heads, slices);
#define REGISTERS(T, R)                                                                                            \
  mlstm_scan_registers_kernel<T, R><<<grid, kScanThreads, 0, stream>>>(                                            \
      static_cast<const T*>(proj), ld, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, q_scale, state,      \
      slot_stride, num_slots, row_start, row_length, request_slots, out, heads, dim, vdim, status)
#define LAUNCH(T)                                                                                                  \
  if (dim <= 32) REGISTERS(T, 8);                                                                                  \
  else if (dim <= 64) REGISTERS(T, 16);                                                                            \
  else if (dim <= 128) REGISTERS(T, 32);                                                                           \
  else if (dim <= 256) REGISTERS(T, 64);                                                                           \
  else {                                                                                                           \
    auto kernel = mlstm_scan_kernel<T>;                                                                            \
    if (shared > 48 * 1024) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)); \
      if (e != cudaSuccess) return static_cast<int>(e);                                                            \
    }                                                                                                              \
    kernel<<<grid, kScanThreads, shared, stream>>>(static_cast<const T*>(proj), ld, q_off, k_off, v_off, i_off, f_off, \
                                                   i_bias, f_bias, cap, q_scale, state, slot_stride, num_slots,    \
                                                   row_start, row_length, request_slots, out, heads, dim, vdim,    \
                                                   status);                                                        \
  }
  if (dtype == kF32) { LAUNCH(float) }
  else if (dtype == kBF16) { LAUNCH(__nv_bfloat16) }
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
#undef REGISTERS
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_head_norm_gate(const float* x, const float* w, const void* gate, long long ldg, int gate_dtype, void* y,
                               int out_dtype, int tokens, int heads, int vdim, float eps, cudaStream_t stream) {
  const int pairs = tokens * heads;
  if (pairs <= 0) return 0;
  const dim3 grid((pairs + 3) / 4);
#define LAUNCH(TG, TO)                                                                                         \
  head_norm_gate_kernel<TG, TO><<<grid, 128, 0, stream>>>(x, w, static_cast<const TG*>(gate), ldg,              \
                                                          static_cast<TO*>(y), pairs, heads, vdim, eps)
  if (gate_dtype == kF32 && out_dtype == kF32) LAUNCH(float, float);
  else if (gate_dtype == kF32 && out_dtype == kBF16) LAUNCH(float, __nv_bfloat16);
  else if (gate_dtype == kBF16 && out_dtype == kF32) LAUNCH(__nv_bfloat16, float);
  else if (gate_dtype == kBF16 && out_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}
