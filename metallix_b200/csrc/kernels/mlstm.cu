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
  chain_release();   // the kernel behind may start and fetch its weights meanwhile
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
  chain_release();   // the kernel behind may start and fetch its weights meanwhile
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

// Portions of prompts: the same recurrence, a chunk of up to 16 tokens at a time. With the chunk's first
// state (C0, n0, m0), F_t the sum of the log forget gates up to token t of the chunk and i_s the log input
// gates, unrolling the recurrence gives, exactly,
//   m_t = max(f_t + m_(t-1), i_t)                                     (a scalar walk over the chunk)
//   C_t = e^(F_t + m0 - m_t) C0 + sum_(s <= t) e^(F_t - F_s + i_s - m_t) k_s v_s^T,  n_t likewise,
// every exponent at most 0. So the chunk's outputs are
//   C_t^T q_t = e^(F_t + m0 - m_t) (C0^T q_t) + sum_(s <= t) w_ts (k_s . q_t) v_s,   w_ts = e^(F_t - F_s + i_s - m_t)
// and the state moves once a chunk: C <- e^(F_L + m0 - m_L) C0 + sum_s w_Ls k_s v_s^T. The tokens of a chunk
// are worked on side by side (a few barriers a chunk instead of two a token), all in float32; the sums run in
// another order than token by token, so the two forms agree to rounding.
constexpr int kChunk = 16;
constexpr int kChunkFrom = 8;   // steps whose longest row brings at least this many tokens take the chunkwise form

template <typename T, int R, int PARTS>
__global__ void __launch_bounds__(kSliceColumns * PARTS)
mlstm_chunk_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int i_off, int f_off,
                   const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                   float* __restrict__ state, long long slot_stride, int num_slots, const int* __restrict__ row_start,
                   const int* __restrict__ row_length, const int* __restrict__ request_slots, float* __restrict__ out,
                   int heads, int dim, int vdim, int* status) {
  chain_release();   // the kernel behind may start and fetch its weights meanwhile
  constexpr int THREADS = kSliceColumns * PARTS;
  extern __shared__ float shared[];
  const int pitch = dim + 1;                          // rows of q and k a bank apart
  float* sq = shared;                                 // [16][dim + 1]
  float* sk = sq + kChunk * pitch;                    // [16][dim + 1]
  float* sn = sk + kChunk * pitch;                    // [dim]
  float* sv = sn + dim;                               // [16][32]
  float* sw = sv + kChunk * kSliceColumns;            // [16][16]: w_ts, then w_ts (k_s . q_t)
  float* red = sw + kChunk * kChunk;                  // [PARTS][16][32]
  float* s_i = red + PARTS * kChunk * kSliceColumns;  // [16] log input gates
  float* s_F = s_i + kChunk;                          // [16] sums of log forget gates
  float* s_m = s_F + kChunk;                          // [16] running maxima
  float* s_decay = s_m + kChunk;                      // [16] e^(F_t + m0 - m_t)
  float* s_n0q = s_decay + kChunk;                    // [16] n0 . q_t
  float* s_take = s_n0q + kChunk;                     // [16] e^(F_L - F_s + i_s - m_L): what the state takes of token s
  float* s_m0 = s_take + kChunk;                      // [1]

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
    const int d = part + PARTS * r;
    c[r] = d < dim && col_ok ? C[static_cast<long long>(d) * vdim + j] : 0.0f;
  }
  for (int d = threadIdx.x; d < dim; d += THREADS) sn[d] = n_state[d];
  for (int e = threadIdx.x; e < kChunk * pitch; e += THREADS) sk[e] = 0.0f;   // rows no token has filled yet count as zeros
  if (threadIdx.x == 0) s_m0[0] = m_state[0];
  const float bi = i_bias[head], bf = f_bias[head];
  const int out_width = heads * vdim;

  for (int begin = 0; begin < length; begin += kChunk) {
    const int len = min(kChunk, length - begin);
    const T* x0 = proj + static_cast<long long>(first + begin) * ld;
    __syncthreads();   // the chunk before is done with everything shared
    // ---- this chunk's q (scaled), k, v and gates
    for (int e = threadIdx.x; e < len * dim; e += THREADS) {
      const int t = e / dim, d = e - t * dim;
      const T* x = x0 + static_cast<long long>(t) * ld;
      sq[t * pitch + d] = to_float(x[q_off + head * dim + d]) * q_scale;
      sk[t * pitch + d] = to_float(x[k_off + head * dim + d]);
    }
    for (int e = threadIdx.x; e < len * kSliceColumns; e += THREADS) {
      const int t = e / kSliceColumns, cc = e - t * kSliceColumns;
      const int jj = slice * kSliceColumns + cc;
      sv[e] = jj < vdim ? to_float(x0[static_cast<long long>(t) * ld + v_off + head * vdim + jj]) : 0.0f;
    }
    if (threadIdx.x < len) {
      const T* x = x0 + static_cast<long long>(threadIdx.x) * ld;
      s_i[threadIdx.x] = cap * tanhf((to_float(x[i_off + head]) + bi) / cap);
      s_F[threadIdx.x] = log_sigmoid(cap * tanhf((to_float(x[f_off + head]) + bf) / cap));   // f_t for now
    }
    __syncthreads();
    // ---- the scalar walk: sums of log forget gates, running maxima
    if (threadIdx.x == 0) {
      float m = s_m0[0], F = 0.0f;
      for (int t = 0; t < len; ++t) {
        const float f = s_F[t];
        m = fmaxf(f + m, s_i[t]);
        F += f;
        s_F[t] = F;
        s_m[t] = m;
      }
    }
    __syncthreads();
    const int last = len - 1;
    if (threadIdx.x < len) {
      s_decay[threadIdx.x] = expf(s_F[threadIdx.x] + s_m0[0] - s_m[threadIdx.x]);
      s_take[threadIdx.x] = expf(s_F[last] - s_F[threadIdx.x] + s_i[threadIdx.x] - s_m[last]);
    }
    // ---- w_ts (k_s . q_t) for s <= t, and n0 . q_t
    for (int e = threadIdx.x; e < len * len; e += THREADS) {
      const int t = e / len, u = e - t * len;
      float value = 0.0f;
      if (u <= t) {
        const float* qr = sq + t * pitch;
        const float* kr = sk + u * pitch;
        float dot = 0.0f;
        for (int d = 0; d < dim; ++d) dot = fmaf(qr[d], kr[d], dot);
        value = expf(s_F[t] - s_F[u] + s_i[u] - s_m[t]) * dot;
      }
      sw[t * kChunk + u] = value;
    }
    for (int t = part; t < len; t += PARTS) {   // a warp a token
      float dot = 0.0f;
      for (int d = col; d < dim; d += kSliceColumns) dot = fmaf(sn[d], sq[t * pitch + d], dot);
      dot = warp_sum(dot);
      if (col == 0) s_n0q[t] = dot;
    }
    // ---- C0^T q_t: this thread's rows of its column, for every token of the chunk
    for (int t = 0; t < len; ++t) {
      const float* qr = sq + t * pitch;
      float acc = 0.0f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = part + PARTS * r;
        if (d < dim) acc = fmaf(c[r], qr[d], acc);
      }
      red[(part * kChunk + t) * kSliceColumns + col] = acc;
    }
    __syncthreads();
    // ---- outputs: tokens shared out among the parts
    for (int t = part; t < len; t += PARTS) {
      float inter = 0.0f;
#pragma unroll
      for (int p = 0; p < PARTS; ++p) inter += red[(p * kChunk + t) * kSliceColumns + col];
      float num = s_decay[t] * inter, dot = s_decay[t] * s_n0q[t];
      for (int u = 0; u <= t; ++u) {
        const float a = sw[t * kChunk + u];
        num = fmaf(a, sv[u * kSliceColumns + col], num);
        dot += a;
      }
      const float den = fmaxf(fabsf(dot), expf(-s_m[t])) + 1.0e-6f;
      if (col_ok) out[static_cast<long long>(first + begin + t) * out_width + head * vdim + j] = num / den;
    }
    // ---- the state behind the chunk
    const float keep = s_decay[last];
    float taken[kChunk];   // what the state takes of each token's value in this thread's column
#pragma unroll
    for (int u = 0; u < kChunk; ++u) taken[u] = u < len ? s_take[u] * sv[u * kSliceColumns + col] : 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = part + PARTS * r;
      if (d < dim) {
        float sum = 0.0f;
#pragma unroll
        for (int u = 0; u < kChunk; ++u) sum = fmaf(taken[u], sk[u * pitch + d], sum);   // rows past len hold old values times 0
        c[r] = fmaf(keep, c[r], sum);
      }
    }
    __syncthreads();   // n0 . q_t and m0 have been read by all; n and m0 may move
    for (int d = threadIdx.x; d < dim; d += THREADS) {
      float sum = 0.0f;
      for (int u = 0; u < len; ++u) sum = fmaf(s_take[u], sk[u * pitch + d], sum);
      sn[d] = fmaf(keep, sn[d], sum);
    }
    if (threadIdx.x == 0) s_m0[0] = s_m[last];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = part + PARTS * r;
    if (d < dim && col_ok) C[static_cast<long long>(d) * vdim + j] = c[r];
  }
  for (int d = threadIdx.x; d < dim; d += THREADS) n_state[d] = sn[d];
  if (threadIdx.x == 0) m_state[0] = s_m0[0];
}

// y[t, h, :] = x[t, h, :] * rsqrt(mean_v(x^2) + eps) * w[h, :] * sigmoid(g[t, h, :]); one warp per (t, h).
template <typename TGate, typename TOut>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, const TGate* __restrict__ gate,
                      long long ldg, TOut* __restrict__ y, int pairs, int heads, int vdim, float eps) {
  chain_release();
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
                           int longest, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || !(cap > 0.0f)) return static_cast<int>(cudaErrorInvalidValue);
  const int slices = (vdim + kSliceColumns - 1) / kSliceColumns;
  const size_t shared = sizeof(float) * (static_cast<size_t>(dim) * kSliceColumns + 3 * static_cast<size_t>(dim) +
                                         kScanParts * kSliceColumns + kScanParts);
  const dim3 grid(rows, heads, slices);
  // A step in which some request brings a portion of a prompt (`longest`, the most tokens of any row, at least
  // kChunkFrom) runs the chunkwise form for all its rows; steps of single tokens the token-by-token form.
  if (longest >= kChunkFrom && dim <= 256) {
    constexpr int parts = 16;   // sixteen warps share a chunk: each holds a sixteenth of the rows of C
    const size_t bytes = sizeof(float) * (2 * static_cast<size_t>(kChunk) * (dim + 1) + dim + kChunk * kSliceColumns +
                                          kChunk * kChunk + static_cast<size_t>(parts) * kChunk * kSliceColumns +
                                          6 * kChunk + 1);
#define CHUNKS(T, R, PARTS)                                                                                          \
  {                                                                                                                  \
    auto kernel = mlstm_chunk_kernel<T, R, PARTS>;                                                                   \
    if (bytes > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)); \
      if (e != cudaSuccess) return static_cast<int>(e);                                                              \
    }                                                                                                                \
    kernel<<<grid, kSliceColumns * PARTS, bytes, stream>>>(                                                          \
        static_cast<const T*>(proj), ld, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, q_scale, state,      \
        slot_stride, num_slots, row_start, row_length, request_slots, out, heads, dim, vdim, status);                 \
  }
#define BY_DIM(T)                                    \
  if (dim <= 32) CHUNKS(T, 2, 16)                    \
  else if (dim <= 64) CHUNKS(T, 4, 16)               \
  else if (dim <= 128) CHUNKS(T, 8, 16)              \
  else CHUNKS(T, 16, 16)
    if (dtype == kF32) { BY_DIM(float) }
    else if (dtype == kBF16) { BY_DIM(__nv_bfloat16) }
    else return static_cast<int>(cudaErrorInvalidValue);
#undef BY_DIM
#undef CHUNKS
    return static_cast<int>(cudaGetLastError());
  }
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
