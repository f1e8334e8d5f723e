// Recurrent mixers that carry a matrix per head or a vector per layer from token to token: what lies between their input
// projections and their output projection.
//
//   ms_unit_norm_heads        every head's vector becomes scale * v / sqrt(sum v^2 + eps), in place
//   ms_exponential_gates      log gates with a soft cap, a running maximum carried by the request, and the three factors
//                             (keep, write, floor) that a matrix memory with exponential gating needs per token and head
//   ms_decay_gates            decay exp(-exp(A_log) softplus(a + dt_bias)) and write strength sigmoid(b) per token and head
//   ms_matrix_scan            the recurrence over a dim x vdim matrix per head, in two forms:
//                               memory: S = keep S + write k v^T, n = keep n + write k, y = S^T q, bottom = max(|n.q|, floor) + 1e-6
//                               delta:  S = decay S, u = beta (v - S^T k), S = S + k u^T, y = S^T q
//                               decay:  S = decay_h S + k v^T with a constant per head, y = S^T q (q, k, v through SiLU if asked)
//                               channel delta: the delta form with one decay per head and key channel (rows of S)
//   ms_low_rank_expand        the second product of a two-step (low-rank) projection, as it is, or turned into decays
//   ms_head_norm_gate         y / bottom, divided by its root mean square per head, times a weight, times sigmoid or SiLU of a gate
//   ms_gated_recurrence_scan  S = a S + sqrt(1 - a^2) i u per channel with a = exp(rate sigmoid(.)), times gelu_tanh of a branch
//
// Everything here is float32 arithmetic on float32 state; only the projections that the kernels read and the last kernels'
// outputs are in the model's compute type.  A request's tokens are walked in order and every sum has a fixed order, so a
// position's result depends on the tokens before it alone, not on how they were cut into steps, on what else is in the
// batch or on which state slot the request holds.
#include "common.cuh"

namespace ms {

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float log_sigmoid_f(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// One warp per (token, head) of x[n, ld]: the head's dim entries from column col + head dim.
__global__ void unit_norm_heads_kernel(float* __restrict__ x, int ld, int col, int heads, int dim, float eps, float scale,
                                       int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)n_tokens * heads) return;
  float* v = x + (size_t)(item / heads) * ld + col + (size_t)(item % heads) * dim;
  float sum_sq = 0.f;
  for (int c = lane; c < dim; c += 32) sum_sq += v[c] * v[c];
  const float factor = scale / sqrtf(warp_sum(sum_sq) + eps);
  for (int c = lane; c < dim; c += 32) v[c] *= factor;
}

// One warp per (request, head).  logits [tokens, 2 heads] = [input | forget].  Lane l squashes the logits of token l of a
// chunk of 32; the running maximum then walks the chunk's tokens in order (values handed round by shuffles), and each lane
// writes its token's three factors.  The request's maximum is read from and left in states[slot, offset + head].
__global__ void exponential_gates_kernel(const float* __restrict__ logits, float cap, float* __restrict__ states,
                                         long long state_stride, int state_offset, const int* __restrict__ state_slots,
                                         const int* __restrict__ query_start, int heads, float* __restrict__ gates) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * warps + warp, request = blockIdx.y;
  if (head >= heads) return;
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  if (q_len <= 0) return;
  float* kept = states + (long long)state_slots[request] * state_stride + state_offset + head;
  float peak = *kept;
  for (int t0 = 0; t0 < q_len; t0 += 32) {
    const int t = t0 + lane;
    float log_i = 0.f, log_f = 0.f;
    if (t < q_len) {
      const float* row = logits + (size_t)(q0 + t) * 2 * heads;
      log_i = cap * tanhf(row[head] / cap);
      log_f = log_sigmoid_f(cap * tanhf(row[heads + head] / cap));
    }
    float before = 0.f, mine = 0.f;
    const int count = min(32, q_len - t0);
    for (int j = 0; j < count; ++j) {
      const float fj = __shfl_sync(0xffffffffu, log_f, j), ij = __shfl_sync(0xffffffffu, log_i, j);
      const float next = fmaxf(fj + peak, ij);
      if (lane == j) { before = peak; mine = next; }
      peak = next;
    }
    if (t < q_len) {
      float* out = gates + ((size_t)(q0 + t) * heads + head) * 3;
      out[0] = expf(log_f + before - mine);
      out[1] = expf(log_i - mine);
      out[2] = expf(-mine);
    }
  }
  if (lane == 0) *kept = peak;
}

// logits [tokens, 2 heads] = [b | a]; gates [tokens, heads, 2] = (decay, beta).
__global__ void decay_gates_kernel(const float* __restrict__ logits, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias, float* __restrict__ gates, int n_tokens, int heads) {
  grid_dependency_wait();
  grid_dependency_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_tokens * heads) return;
  const int head = (int)(i % heads);
  const float* row = logits + (size_t)(i / heads) * 2 * heads;
  gates[2 * i] = expf(-expf(a_log[head]) * softplus_f(row[heads + head] + dt_bias[head]));
  gates[2 * i + 1] = sigmoid_f(row[head]);
}

// The matrix recurrence.  grid (column tiles, heads, requests); a block of 256 threads owns 256 / LPC columns of one head's
// matrix for one request, LPC lanes (a power of two) a column: lane `sub` holds the column's entries sub R .. sub R + R - 1
// (zero beyond dim) in registers, so that a token's key and query reach it as 16-byte reads of shared memory (the rows
// there give every lane's piece four floats of padding: the pieces of the lanes that read together lie in different banks).
// With few lanes a column a token costs a lane 2 R multiply-adds (3 R in the delta form) against R / 2 reads and a
// butterfly of log2 LPC steps.  In the memory form the matrix has one more column, n, whose "value" is 1 and whose read-out
// n . q gives the token's divisor.  The tokens' keys, queries (times q_scale), values and gates pass through shared memory
// in chunks of `tok` tokens; a column's sums are the lane's own entries in four interleaved partial sums of ascending
// order, then a butterfly over its LPC lanes, whatever the chunk.  While a chunk is walked, the next one is already on its
// way from memory into registers (kScanFetch keys, queries and values a thread: a chunk holds at most 256 kScanFetch of
// each), so that the walk waits for memory once a request and not once a chunk.
constexpr int kScanThreads = 256, kScanShift = 8;
constexpr int kModeMemory = 0, kModeDelta = 1, kModeDecay = 2, kModeChannelDelta = 3;
constexpr int kPiecePad = 4;
constexpr int kScanFetch = 8;

// The sum over the 2^shift lanes of a column (a butterfly from the widest step down; `shift` is the same in the whole block).
__device__ __forceinline__ float column_sum(float v, int shift) {
  if (shift > 4) v += __shfl_xor_sync(0xffffffffu, v, 16);
  if (shift > 3) v += __shfl_xor_sync(0xffffffffu, v, 8);
  if (shift > 2) v += __shfl_xor_sync(0xffffffffu, v, 4);
  if (shift > 1) v += __shfl_xor_sync(0xffffffffu, v, 2);
  if (shift > 0) v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

template <typename T, int R, int MODE>
__global__ void __launch_bounds__(kScanThreads)
matrix_scan_kernel(const T* __restrict__ q, int q_ld, int q_col, const T* __restrict__ k, int k_ld, int k_col,
                   const T* __restrict__ v, int v_ld, int v_col, float q_scale, const float* __restrict__ gates,
                   float* __restrict__ states, long long state_stride, int state_offset,
                   const int* __restrict__ state_slots, const int* __restrict__ query_start, int heads, int kv_heads, int dim,
                   int vdim, int lpc_shift, int tok, float* __restrict__ y, float* __restrict__ bottom, int gate_ld,
                   int gate_col, const float* __restrict__ channel_decay, int input_act) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ __align__(16) float matrix_smem[];
  // numbers of `gates` a token and head has: (keep, write, floor), (decay, beta), none (the decay is the head's constant:
  // gates [heads]), or one logit whose sigmoid is beta (gates: rows of gate_ld numbers, the heads' logits from gate_col)
  constexpr int G = MODE == kModeMemory ? 3 : MODE == kModeDelta ? 2 : MODE == kModeDecay ? 0 : 1;
  constexpr bool CHANNEL = MODE == kModeChannelDelta;
  constexpr int PIECE = R + kPiecePad;
  const int LPC = 1 << lpc_shift, cols_per_block = kScanThreads >> lpc_shift;
  const int row = LPC * PIECE;                                // floats of a token's key (or query) in shared memory
  const int columns = MODE == kModeMemory ? vdim + 1 : vdim;
  const int tid = threadIdx.x, cc = tid >> lpc_shift, sub = tid & (LPC - 1);
  const int col = blockIdx.x * cols_per_block + cc;
  const bool active = col < columns;
  const int head = blockIdx.y, request = blockIdx.z;
  const int kv_head = head / (heads / kv_heads);
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  if (q_len <= 0) return;                                    // (the whole block)
  float* ks = matrix_smem;                                    // [tok][row]
  float* qs = ks + tok * row;                                 // [tok][row]
  float* vs = qs + tok * row;                                 // [tok][cols_per_block]
  float* gs = vs + tok * cols_per_block;                      // [tok][4]
  float* ds = gs + tok * 4;                                   // [tok][row]: the key channels' decays (channel delta only)
  const float head_decay = MODE == kModeDecay ? gates[head] : 1.f;
  float* kept = states + (long long)state_slots[request] * state_stride + state_offset + ((size_t)head * columns + (active ? col : 0)) * dim;
  float s[R];
  // (a lane's piece as 16-byte accesses where it lies so: a column is `dim` floats, the state's row may start anywhere)
  const bool wide = (dim & 3) == 0 && (reinterpret_cast<size_t>(kept) & 15) == 0;
  if (wide) {
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      const int i = sub * R + r;
      const float4 piece = (active && i < dim) ? *reinterpret_cast<const float4*>(kept + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s[r] = piece.x, s[r + 1] = piece.y, s[r + 2] = piece.z, s[r + 3] = piece.w;
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = sub * R + r;
      s[r] = (active && i < dim) ? kept[i] : 0.f;
    }
  }
  constexpr int LOG_R = R == 4 ? 2 : R == 8 ? 3 : R == 16 ? 4 : 5;
  const int dim_shift = LOG_R + lpc_shift, dim_pad = 1 << dim_shift, col_shift = kScanShift - lpc_shift;
  const T* k_head = k + k_col + kv_head * dim;
  const T* q_head = q + q_col + kv_head * dim;
  const T* v_head = v + v_col + head * vdim + blockIdx.x * cols_per_block;
  const int cols_here = min(cols_per_block, vdim - (int)blockIdx.x * cols_per_block);      // value columns of this block (n is none)
  // where this lane writes: a value column's read-out into y, the column n's into the tokens' divisors; one step a token
  const bool is_n = MODE == kModeMemory && col == vdim;
  float* out_at = (sub == 0 && active) ? (is_n ? bottom + (size_t)q0 * heads + head : y + ((size_t)q0 * heads + head) * vdim + col) : nullptr;
  const size_t out_step = is_n ? (size_t)heads : (size_t)heads * vdim;
  T next_k[kScanFetch], next_q[kScanFetch], next_v[kScanFetch];
  float next_d[CHANNEL ? kScanFetch : 1];
  const float* d_head = CHANNEL ? channel_decay + (size_t)head * dim : nullptr;
  const int d_ld = heads * dim;
  float next_g = 0.f;
  auto fetch = [&](int t0) {
    const int len = min(tok, q_len - t0);
    const size_t first = (size_t)(q0 + t0);
#pragma unroll
    for (int j = 0; j < kScanFetch; ++j) {
      const int idx = tid + kScanThreads * j, tt = idx >> dim_shift, i = idx & (dim_pad - 1);
      const bool real = tt < len && i < dim;
      next_k[j] = real ? k_head[(first + tt) * k_ld + i] : from_float<T>(0.f);
      next_q[j] = real ? q_head[(first + tt) * q_ld + i] : from_float<T>(0.f);
      if (CHANNEL) next_d[j] = real ? d_head[(first + tt) * d_ld + i] : 1.f;
    }
#pragma unroll
    for (int j = 0; j < kScanFetch; ++j) {
      const int idx = tid + kScanThreads * j, tt = idx >> col_shift, c = idx & (cols_per_block - 1);
      next_v[j] = (tt < len && c < cols_here) ? v_head[(first + tt) * v_ld + c] : from_float<T>(1.f);      // (the column n)
    }
    if (CHANNEL) {
      if (tid < len) next_g = sigmoid_f(gates[(first + tid) * gate_ld + gate_col + head]);
    } else if (G > 0) {
      if (tid < len * G) next_g = gates[((first + tid / (G > 0 ? G : 1)) * heads + head) * G + tid % (G > 0 ? G : 1)];
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < q_len; t0 += tok) {
    const int len = min(tok, q_len - t0);
    __syncthreads();                                          // the chunk before has been read
#pragma unroll
    for (int j = 0; j < kScanFetch; ++j) {
      const int idx = tid + kScanThreads * j, tt = idx >> dim_shift, i = idx & (dim_pad - 1);
      if (tt < len) {
        const int at = tt * row + (i >> LOG_R) * PIECE + (i & (R - 1));
        float key = to_float(next_k[j]), query = to_float(next_q[j]);
        if (input_act) key *= sigmoid_f(key), query *= sigmoid_f(query);
        ks[at] = key;
        qs[at] = q_scale * query;
        if (CHANNEL) ds[at] = next_d[j];
      }
    }
#pragma unroll
    for (int j = 0; j < kScanFetch; ++j) {
      const int idx = tid + kScanThreads * j;
      if ((idx >> col_shift) < len) {
        float value = to_float(next_v[j]);
        if (input_act) value *= sigmoid_f(value);
        vs[idx] = value;
      }
    }
    if (CHANNEL) {
      if (tid < len) gs[tid * 4 + 1] = next_g;
    } else if (G > 0) {
      if (tid < len * G) gs[(tid / (G > 0 ? G : 1)) * 4 + tid % (G > 0 ? G : 1)] = next_g;
    }
    __syncthreads();
    if (t0 + tok < q_len) fetch(t0 + tok);
#pragma unroll 4
    for (int tt = 0; tt < len; ++tt) {
      const float4* kk = reinterpret_cast<const float4*>(ks + tt * row + sub * PIECE);
      const float4* qq = reinterpret_cast<const float4*>(qs + tt * row + sub * PIECE);
      const float value = vs[tt * cols_per_block + cc];
      const float4 gate = reinterpret_cast<const float4*>(gs)[tt];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (MODE == kModeMemory || MODE == kModeDecay) {
        const float keep = MODE == kModeDecay ? head_decay : gate.x, write = MODE == kModeDecay ? value : gate.y * value;
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = kk[r >> 2], qv = qq[r >> 2];
          s[r] = keep * s[r] + write * kv.x;
          s[r + 1] = keep * s[r + 1] + write * kv.y;
          s[r + 2] = keep * s[r + 2] + write * kv.z;
          s[r + 3] = keep * s[r + 3] + write * kv.w;
          acc[0] += s[r] * qv.x;
          acc[1] += s[r + 1] * qv.y;
          acc[2] += s[r + 2] * qv.z;
          acc[3] += s[r + 3] * qv.w;
        }
      } else {
        const float decay = gate.x, beta = gate.y;
        const float4* dd = reinterpret_cast<const float4*>(ds + tt * row + sub * PIECE);
        float seen[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = kk[r >> 2];
          const float4 dv = CHANNEL ? dd[r >> 2] : make_float4(decay, decay, decay, decay);
          s[r] *= dv.x;
          s[r + 1] *= dv.y;
          s[r + 2] *= dv.z;
          s[r + 3] *= dv.w;
          seen[0] += s[r] * kv.x;
          seen[1] += s[r + 1] * kv.y;
          seen[2] += s[r + 2] * kv.z;
          seen[3] += s[r + 3] * kv.w;
        }
        float total = (seen[0] + seen[1]) + (seen[2] + seen[3]);
        total = column_sum(total, lpc_shift);
        const float u = beta * (value - total);
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 kv = kk[r >> 2], qv = qq[r >> 2];
          s[r] += kv.x * u;
          s[r + 1] += kv.y * u;
          s[r + 2] += kv.z * u;
          s[r + 3] += kv.w * u;
          acc[0] += s[r] * qv.x;
          acc[1] += s[r + 1] * qv.y;
          acc[2] += s[r + 2] * qv.z;
          acc[3] += s[r + 3] * qv.w;
        }
      }
      float read = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      read = column_sum(read, lpc_shift);
      if (out_at != nullptr) {
        *out_at = is_n ? fmaxf(fabsf(read), gate.z) + 1e-6f : read;
        out_at += out_step;
      }
    }
  }
  if (active && wide) {
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      const int i = sub * R + r;
      if (i < dim) *reinterpret_cast<float4*>(kept + i) = make_float4(s[r], s[r + 1], s[r + 2], s[r + 3]);
    }
  } else if (active) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = sub * R + r;
      if (i < dim) kept[i] = s[r];
    }
  }
}

// The second product of a projection made in two steps through `rank` numbers: value[n, r] = sum_j mid[n, col + j] w[r, j]
// with mid float32 (rows of ld numbers) and w float32 [rows, rank].  decay == 0: out[n, r] = value in the type T.
// decay != 0 (T float): out[n, r] = exp(-exp(a_log[r / per_head]) softplus(value + bias[r])), a decay per head and channel.
template <typename T>
__global__ void low_rank_expand_kernel(const float* __restrict__ mid, int ld, int col, int rank, const float* __restrict__ w,
                                       int rows, int decay, const float* __restrict__ a_log, const float* __restrict__ bias,
                                       int per_head, T* __restrict__ out, long long total) {
  grid_dependency_wait();
  grid_dependency_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int r = (int)(i % rows);
  const float* row = mid + (size_t)(i / rows) * ld + col;
  float sum = 0.f;
  if (w == nullptr) {
    sum = row[r];                                             // (no second matrix: the numbers themselves)
  } else {
    const float* wr = w + (size_t)r * rank;
    for (int j = 0; j < rank; ++j) sum += row[j] * wr[j];
  }
  if (decay) sum = expf(-expf(a_log[r / per_head]) * softplus_f(sum + bias[r]));
  out[i] = from_float<T>(sum);
}

// The same product for many results: a block of 256 threads owns 256 results (consecutive r) of kExpandTokens tokens.  The
// tokens' `rank` numbers lie in shared memory (every thread reads the same one at a time), the second matrix is given
// TRANSPOSED, wt [rank, rows], so that the threads of a warp read consecutive numbers, and each of its numbers feeds
// kExpandTokens multiply-adds.  A result's sum runs over j in ascending order whatever the tile.
constexpr int kExpandTokens = 8;

template <typename T>
__global__ void __launch_bounds__(256)
low_rank_expand_tiled_kernel(const float* __restrict__ mid, int ld, int col, int rank, const float* __restrict__ wt, int rows,
                             int decay, const float* __restrict__ a_log, const float* __restrict__ bias, int per_head,
                             T* __restrict__ out, int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float expand_smem[];                      // [kExpandTokens][rank]
  const int t0 = blockIdx.y * kExpandTokens;
  const int len = min(kExpandTokens, n_tokens - t0);
  for (int i = threadIdx.x; i < kExpandTokens * rank; i += blockDim.x) {
    const int t = i / rank, j = i % rank;
    expand_smem[i] = t < len ? mid[(size_t)(t0 + t) * ld + col + j] : 0.f;
  }
  __syncthreads();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float acc[kExpandTokens];
#pragma unroll
  for (int t = 0; t < kExpandTokens; ++t) acc[t] = 0.f;
  for (int j = 0; j < rank; ++j) {
    const float w = wt[(size_t)j * rows + r];
#pragma unroll
    for (int t = 0; t < kExpandTokens; ++t) acc[t] += expand_smem[t * rank + j] * w;
  }
  float rate = 0.f, b = 0.f;
  if (decay) rate = -expf(a_log[r / per_head]), b = bias[r];
#pragma unroll
  for (int t = 0; t < kExpandTokens; ++t) {
    if (t < len) out[(size_t)(t0 + t) * rows + r] = from_float<T>(decay ? expf(rate * softplus_f(acc[t] + b)) : acc[t]);
  }
}

// One warp per (token, head): v = y / bottom, v / sqrt(mean(v^2) + eps) * weight * act(gate).  Where a head's row is
// at most 512 numbers, a multiple of four, and lies on 16-byte boundaries in all four arrays (`wide`), a lane keeps its
// four-number pieces in registers between the sum and the output and every access is one piece; otherwise number by number.
template <typename T> struct alignas(sizeof(T) * 4) Four { T v[4]; };
constexpr int kHeadPieces = 4;                               // pieces of four numbers a lane

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ y, const float* __restrict__ bottom,
                                      const float* __restrict__ weight, int weight_per_head, const T* __restrict__ gate,
                                      int gate_ld, int gate_col, int activation, float eps, T* __restrict__ out, int n_tokens,
                                      int heads, int vdim, int wide) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long items = (long long)n_tokens * heads;
  for (long long item = (long long)blockIdx.x * warps + warp; item < items; item += (long long)gridDim.x * warps) {
    const size_t token = (size_t)(item / heads);
    const int head = (int)(item % heads);
    const float* row = y + (size_t)item * vdim;
    const float divisor = bottom ? bottom[item] : 1.f;
    const float* w = weight + (weight_per_head ? (size_t)head * vdim : 0);
    const T* z = gate + token * gate_ld + gate_col + (size_t)head * vdim;
    T* dst = out + (token * heads + head) * vdim;
    if (wide) {
      const int pieces = vdim >> 2;
      float4 value[kHeadPieces];
      Four<T> g[kHeadPieces];
      float sum_sq = 0.f;
#pragma unroll
      for (int j = 0; j < kHeadPieces; ++j) {
        const int at = lane + 32 * j;
        value[j] = at < pieces ? reinterpret_cast<const float4*>(row)[at] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (at < pieces) g[j] = reinterpret_cast<const Four<T>*>(z)[at];
      }
#pragma unroll
      for (int j = 0; j < kHeadPieces; ++j) {
        value[j].x /= divisor, value[j].y /= divisor, value[j].z /= divisor, value[j].w /= divisor;
        sum_sq += (value[j].x * value[j].x + value[j].y * value[j].y) + (value[j].z * value[j].z + value[j].w * value[j].w);
      }
      const float inv = 1.0f / sqrtf(warp_sum(sum_sq) / (float)vdim + eps);
#pragma unroll
      for (int j = 0; j < kHeadPieces; ++j) {
        const int at = lane + 32 * j;
        if (at < pieces) {
          const float4 scale = reinterpret_cast<const float4*>(w)[at];
          const float v4[4] = {value[j].x * inv * scale.x, value[j].y * inv * scale.y, value[j].z * inv * scale.z, value[j].w * inv * scale.w};
          Four<T> o;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float gv = to_float(g[j].v[e]);
            o.v[e] = from_float<T>(v4[e] * (activation ? gv * sigmoid_f(gv) : sigmoid_f(gv)));
          }
          reinterpret_cast<Four<T>*>(dst)[at] = o;
        }
      }
      continue;
    }
    float sum_sq = 0.f;
    for (int c = lane; c < vdim; c += 32) {
      const float value = row[c] / divisor;
      sum_sq += value * value;
    }
    const float inv = 1.0f / sqrtf(warp_sum(sum_sq) / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) {
      const float g = to_float(z[c]);
      const float factor = activation ? g * sigmoid_f(g) : sigmoid_f(g);
      dst[c] = from_float<T>((row[c] / divisor) * inv * w[c] * factor);
    }
  }
}

// The same for long rows (all heads normed together: one "head" of thousands of numbers): a block of 256 threads a (token,
// head), the sum of squares over the block in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_block_kernel(const float* __restrict__ y, const float* __restrict__ bottom, const float* __restrict__ weight,
                            int weight_per_head, const T* __restrict__ gate, int gate_ld, int gate_col, int activation, float eps,
                            T* __restrict__ out, int heads, int vdim) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const long long item = blockIdx.x;
  const size_t token = (size_t)(item / heads);
  const int head = (int)(item % heads);
  const float* row = y + (size_t)item * vdim;
  const float divisor = bottom ? bottom[item] : 1.f;
  const float* w = weight + (weight_per_head ? (size_t)head * vdim : 0);
  const T* z = gate + token * gate_ld + gate_col + (size_t)head * vdim;
  T* dst = out + (token * heads + head) * vdim;
  float sum_sq = 0.f;
  for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
    const float value = row[c] / divisor;
    sum_sq += value * value;
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)vdim + eps);
  for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
    const float g = to_float(z[c]);
    const float factor = activation ? g * sigmoid_f(g) : sigmoid_f(g);
    dst[c] = from_float<T>((row[c] / divisor) * inv * w[c] * factor);
  }
}

// grid (channel blocks, requests); a block of sixteen warps owns 32 channels (a lane a channel) and walks the request's tokens
// in tiles of 64, four tokens a warp, whose loads are issued together, a tile ahead of the walk.  What does not depend
// on the state (both gates, the decay a, the token's input b = sqrt(1 - a^2) i u and the gelu branch) is computed by all
// warps; a and b go to shared memory, where one warp walks the tile with S = a S + b, one fused multiply-add a token, whatever
// the tile (so a sequence whole or in portions gives the same bits); all warps then multiply by their branch and store.
constexpr int kRecChannels = 32, kRecTile = 64, kRecWarps = 16, kRecEach = kRecTile / kRecWarps;

template <typename T>
__global__ void __launch_bounds__(kRecWarps * 32)
gated_recurrence_scan_kernel(const float* __restrict__ u, const float* __restrict__ pre, const float* __restrict__ gate_bias,
                             const float* __restrict__ rate, const T* __restrict__ proj, int ld, int y_col,
                             const float* __restrict__ y_bias, float* __restrict__ states, long long state_stride,
                             int state_offset, const int* __restrict__ state_slots, const int* __restrict__ query_start,
                             int width, int n_tokens, T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float decay[kRecTile][kRecChannels];
  __shared__ float carried[kRecTile][kRecChannels];           // b on the way in, S on the way out
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * kRecChannels + lane, request = blockIdx.y;
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  if (q_len <= 0) return;                                     // (the whole block)
  const bool real = c < width;
  const int cc = real ? c : 0;
  float* kept = states + (long long)state_slots[request] * state_stride + state_offset + cc;
  const float r_bias = gate_bias[cc], i_bias = gate_bias[width + cc], slope = rate[cc], branch_bias = y_bias ? y_bias[cc] : 0.f;
  const float* pre_r = pre + (size_t)q0 * width + cc;
  const float* pre_i = pre + ((size_t)n_tokens + q0) * width + cc;
  const float* input = u + (size_t)q0 * width + cc;
  const T* branch = proj + (size_t)q0 * ld + y_col + cc;
  T* dst = out + (size_t)q0 * width + cc;
  float state = warp == 0 ? *kept : 0.f;
  float pr[kRecEach], pi[kRecEach], in[kRecEach];           // the next tile's inputs, on their way (as loaded: no
  T br[kRecEach];                                             // arithmetic waits for them before the walk)
  auto fetch = [&](int t0) {
    const int len = min(kRecTile, q_len - t0);
#pragma unroll
    for (int e = 0; e < kRecEach; ++e) {                      // (a token beyond the tile reads the tile's first again)
      const int tt = warp + e * kRecWarps;
      const size_t t = (size_t)(t0 + (tt < len ? tt : 0));
      pr[e] = pre_r[t * width], pi[e] = pre_i[t * width], in[e] = input[t * width], br[e] = branch[t * ld];
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < q_len; t0 += kRecTile) {
    const int len = min(kRecTile, q_len - t0);
    float gelu[kRecEach];
#pragma unroll
    for (int e = 0; e < kRecEach; ++e) {
      const int tt = warp + e * kRecWarps;
      const float r = sigmoid_f(pr[e] + r_bias);
      const float gate_in = sigmoid_f(pi[e] + i_bias);
      const float log_a = slope * r;
      const float spread = sqrtf(-expm1f(2.f * log_a));       // sqrt(1 - a^2) without cancellation
      decay[tt][lane] = expf(log_a);
      carried[tt][lane] = spread * (gate_in * in[e]);
      gelu[e] = gelu_tanh_f(to_float(br[e]) + branch_bias);
    }
    __syncthreads();
    if (t0 + kRecTile < q_len) fetch(t0 + kRecTile);
    if (warp == 0) {
#pragma unroll 8
      for (int tt = 0; tt < len; ++tt) {
        state = fmaf(decay[tt][lane], state, carried[tt][lane]);
        carried[tt][lane] = state;
      }
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < kRecEach; ++e) {
      const int tt = warp + e * kRecWarps;
      if (real && tt < len) dst[(size_t)(t0 + tt) * width] = from_float<T>(carried[tt][lane] * gelu[e]);
    }
    __syncthreads();                                          // the next tile writes what this one read
  }
  if (warp == 0 && real) *kept = state;
}

}  // namespace ms

using namespace ms;

#define MS_REC_DISPATCH(dtype, ...)                              \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// x float32 [n_tokens, ld], in place.
MS_EXPORT int ms_unit_norm_heads(float* x, int ld, int col, int heads, int dim, float eps, float scale, int n_tokens,
                                 cudaStream_t stream) {
  if (n_tokens == 0 || heads == 0) return 0;
  MS_REQUIRE(dim > 0 && col >= 0 && col + heads * dim <= ld, "unit_norm_heads: %d heads of %d from column %d of rows of %d", heads, dim, col, ld);
  const int warps = 4;
  const long long blocks = ((long long)n_tokens * heads + warps - 1) / warps;
  MS_REQUIRE(blocks < 2147483647LL, "unit_norm_heads: %lld heads in one launch is too many", (long long)n_tokens * heads);
  ms::launch(unit_norm_heads_kernel, (unsigned)blocks, warps * 32, 0, stream, x, ld, col, heads, dim, eps, scale, n_tokens);
  MS_CHECK_LAUNCH("unit_norm_heads");
  return 0;
}

// logits float32 [tokens, 2 heads]; states float32 rows of state_stride numbers, the heads' maxima at state_offset;
// gates float32 [tokens, heads, 3].
MS_EXPORT int ms_exponential_gates(const float* logits, float cap, float* states, long long state_stride, int state_offset,
                                   const int* state_slots, const int* query_start, int n_requests, int heads, float* gates,
                                   cudaStream_t stream) {
  if (n_requests == 0 || heads == 0) return 0;
  MS_REQUIRE(cap > 0.f && n_requests <= 65535, "exponential_gates: cap %f, %d requests", cap, n_requests);
  const int warps = heads >= 4 ? 4 : heads;
  dim3 grid((heads + warps - 1) / warps, n_requests);
  ms::launch(exponential_gates_kernel, grid, warps * 32, 0, stream, logits, cap, states, state_stride, state_offset, state_slots,
             query_start, heads, gates);
  MS_CHECK_LAUNCH("exponential_gates");
  return 0;
}

MS_EXPORT int ms_decay_gates(const float* logits, const float* a_log, const float* dt_bias, float* gates, int n_tokens,
                             int heads, cudaStream_t stream) {
  const long long total = (long long)n_tokens * heads;
  if (total == 0) return 0;
  ms::launch(decay_gates_kernel, (unsigned)((total + 127) / 128), 128, 0, stream, logits, a_log, dt_bias, gates, n_tokens, heads);
  MS_CHECK_LAUNCH("decay_gates");
  return 0;
}

static int scan_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    count = sms;
  }
  return count;
}

// mode 0 (memory): gates [tokens, heads, 3], state [heads, vdim + 1, dim] per slot, bottom [tokens, heads];
// mode 1 (delta): gates [tokens, heads, 2], state [heads, vdim, dim], bottom unused.  q, k, v: rows of q_ld, k_ld, v_ld
// numbers of type `dtype`; y float32 [tokens, heads, vdim].  max_query_len: an upper bound of the tokens a request brings.
// mode 2 (decay): gates [heads], the heads' constant decays; state [heads, vdim, dim].  mode 3 (channel delta): gates are rows
// of gate_ld float32 numbers whose columns gate_col .. gate_col + heads hold the logits of beta; channel_decay float32
// [tokens, heads, dim]; state [heads, vdim, dim].  input_act != 0: q, k and v pass SiLU as they are read.
MS_EXPORT int ms_matrix_scan(int mode, const void* q, int q_ld, int q_col, const void* k, int k_ld, int k_col, const void* v,
                             int v_ld, int v_col, int dtype, float q_scale, const float* gates, float* states,
                             long long state_stride, int state_offset, const int* state_slots, const int* query_start,
                             int n_requests, int max_query_len, int heads, int kv_heads, int dim, int vdim, float* y,
                             float* bottom, int gate_ld, int gate_col, const float* channel_decay, int input_act,
                             cudaStream_t stream) {
  if (n_requests == 0 || max_query_len <= 0 || heads == 0) return 0;
  MS_REQUIRE(mode >= kModeMemory && mode <= kModeChannelDelta, "matrix_scan: mode %d", mode);
  MS_REQUIRE(mode != kModeChannelDelta || (channel_decay != nullptr && gate_col >= 0 && gate_col + heads <= gate_ld),
             "matrix_scan: the channel form needs the channels' decays and the heads' logits (columns %d.. of %d)", gate_col, gate_ld);
  MS_REQUIRE(kv_heads > 0 && heads % kv_heads == 0 && dim >= 1 && dim <= 512 && vdim >= 1, "matrix_scan: %d/%d heads of %d/%d",
             heads, kv_heads, dim, vdim);
  MS_REQUIRE(mode != kModeMemory || bottom != nullptr, "matrix_scan: the memory form writes the tokens' divisors");
  MS_REQUIRE(heads <= 65535 && n_requests <= 65535, "matrix_scan: grid %d x %d exceeds the launch limits", heads, n_requests);
  // lanes per column: at least as many as hold the column in 32 entries a lane, the lane's piece rounded up to 4, 8, 16 or 32
  // (one more doubling of the lanes where that wastes less).  Few lanes a column make the most of a token's key and query
  // in shared memory, and suit a launch that fills the GPU anyway (many requests).  A launch of few requests is a chain of
  // tokens whose length is what a warp does for one token: there the lanes are doubled (shorter pieces, more warps) while
  // the launch stays under eight warps a multiprocessor.
  int lpc_shift = 0;
  while (lpc_shift < 5 && (dim + (1 << lpc_shift) - 1) / (1 << lpc_shift) > 32) ++lpc_shift;
  auto piece = [&](int shift) {
    const int per_lane = (dim + (1 << shift) - 1) >> shift;
    return per_lane <= 4 ? 4 : per_lane <= 8 ? 8 : per_lane <= 16 ? 16 : 32;
  };
  while (lpc_shift < 3 && (piece(lpc_shift + 1) << (lpc_shift + 1)) < (piece(lpc_shift) << lpc_shift)) ++lpc_shift;
  const long long all_columns = (long long)(mode == kModeMemory ? vdim + 1 : vdim);
  auto warps_of = [&](int shift) {
    const int per_block = kScanThreads >> shift;
    return (long long)n_requests * heads * ((all_columns + per_block - 1) / per_block) * (kScanThreads / 32);
  };
  const long long room = 8LL * scan_sm_count();
  while (lpc_shift < 5 && piece(lpc_shift) > 4 && warps_of(lpc_shift + 1) <= room) ++lpc_shift;
  const int r = piece(lpc_shift);
  const int cols_per_block = kScanThreads >> lpc_shift;
  const int columns = mode == kModeMemory ? vdim + 1 : vdim;
  const int row_floats = (mode == kModeChannelDelta ? 3 : 2) * ((r + kPiecePad) << lpc_shift) + cols_per_block + 4;
  // a chunk: at most 16 tokens, kScanThreads kScanFetch keys and as many values (what the threads hold of the next chunk)
  // and 40 KB of shared memory
  int tok = max_query_len < 16 ? max_query_len : 16;
  while (tok > 1 && ((size_t)tok * row_floats * sizeof(float) > 40 * 1024 || (tok * r << lpc_shift) > kScanThreads * kScanFetch ||
                     tok * cols_per_block > kScanThreads * kScanFetch)) tok >>= 1;
  MS_REQUIRE((tok * r << lpc_shift) <= kScanThreads * kScanFetch && tok * cols_per_block <= kScanThreads * kScanFetch,
             "matrix_scan: a chunk of %d tokens of %d entries does not fit the threads' registers", tok, r << lpc_shift);
  const size_t smem = (size_t)tok * row_floats * sizeof(float);
  dim3 grid((columns + cols_per_block - 1) / cols_per_block, heads, n_requests);
#define MS_MATRIX_SCAN(R, MODE)                                                                                               \
  MS_REC_DISPATCH(dtype, (ms::launch(matrix_scan_kernel<T, R, MODE>, grid, kScanThreads, smem, stream, (const T*)q, q_ld, q_col, \
                                     (const T*)k, k_ld, k_col, (const T*)v, v_ld, v_col, q_scale, gates, states, state_stride,  \
                                     state_offset, state_slots, query_start, heads, kv_heads, dim, vdim, lpc_shift, tok, y,     \
                                     bottom, gate_ld, gate_col, channel_decay, input_act)))
  if (mode == kModeMemory) {
    if (r == 4) { MS_MATRIX_SCAN(4, kModeMemory); } else if (r == 8) { MS_MATRIX_SCAN(8, kModeMemory); }
    else if (r == 16) { MS_MATRIX_SCAN(16, kModeMemory); } else { MS_MATRIX_SCAN(32, kModeMemory); }
  } else if (mode == kModeDecay) {
    if (r == 4) { MS_MATRIX_SCAN(4, kModeDecay); } else if (r == 8) { MS_MATRIX_SCAN(8, kModeDecay); }
    else if (r == 16) { MS_MATRIX_SCAN(16, kModeDecay); } else { MS_MATRIX_SCAN(32, kModeDecay); }
  } else if (mode == kModeChannelDelta) {
    if (r == 4) { MS_MATRIX_SCAN(4, kModeChannelDelta); } else if (r == 8) { MS_MATRIX_SCAN(8, kModeChannelDelta); }
    else if (r == 16) { MS_MATRIX_SCAN(16, kModeChannelDelta); } else { MS_MATRIX_SCAN(32, kModeChannelDelta); }
  } else {
    if (r == 4) { MS_MATRIX_SCAN(4, kModeDelta); } else if (r == 8) { MS_MATRIX_SCAN(8, kModeDelta); }
    else if (r == 16) { MS_MATRIX_SCAN(16, kModeDelta); } else { MS_MATRIX_SCAN(32, kModeDelta); }
  }
#undef MS_MATRIX_SCAN
  MS_CHECK_LAUNCH("matrix_scan");
  return 0;
}

// mid float32 rows of ld numbers (the first product's results from column col); wt float32 [rank, rows], the second matrix
// TRANSPOSED; out [tokens, rows] of type `dtype`, or, decay != 0, float32 decays exp(-exp(a_log[row / per_head]) softplus(. +
// bias[row])).  wt null (rank == rows): the numbers of mid themselves take the place of the product.
MS_EXPORT int ms_low_rank_expand(const float* mid, int ld, int col, int rank, const float* wt, int rows, int decay,
                                 const float* a_log, const float* bias, int per_head, void* out, int dtype, int n_tokens,
                                 cudaStream_t stream) {
  const long long total = (long long)n_tokens * rows;
  if (total == 0) return 0;
  MS_REQUIRE(rank >= 1 && col >= 0 && col + rank <= ld, "low_rank_expand: %d numbers from column %d of rows of %d", rank, col, ld);
  MS_REQUIRE(wt != nullptr || rank == rows, "low_rank_expand: without a second matrix the %d numbers are the %d results", rank, rows);
  MS_REQUIRE(!decay || (a_log && bias && per_head >= 1 && rows % per_head == 0 && dtype == MS_F32),
             "low_rank_expand: decays are float32 and need A_log, a bias and the heads' size (%d rows, %d a head)", rows, per_head);
  if (wt != nullptr) {
    const size_t smem = (size_t)kExpandTokens * rank * sizeof(float);
    MS_REQUIRE(smem <= 48 * 1024, "low_rank_expand: %d numbers a token do not fit the shared memory", rank);
    const int token_tiles = (n_tokens + kExpandTokens - 1) / kExpandTokens;
    MS_REQUIRE(token_tiles <= 65535, "low_rank_expand: %d tokens in one launch is too many", n_tokens);
    dim3 grid((rows + 255) / 256, token_tiles);
    MS_REC_DISPATCH(dtype, (ms::launch(low_rank_expand_tiled_kernel<T>, grid, 256, smem, stream, mid, ld, col, rank, wt, rows, decay,
                                       a_log, bias, per_head, (T*)out, n_tokens)));
    MS_CHECK_LAUNCH("low_rank_expand");
    return 0;
  }
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "low_rank_expand: %lld numbers in one launch is too many", total);
  MS_REC_DISPATCH(dtype, (ms::launch(low_rank_expand_kernel<T>, (unsigned)blocks, 256, 0, stream, mid, ld, col, rank, wt, rows, decay,
                                     a_log, bias, per_head, (T*)out, total)));
  MS_CHECK_LAUNCH("low_rank_expand");
  return 0;
}

// y float32 [tokens, heads, vdim]; bottom float32 [tokens, heads] or null; weight float32 [heads * vdim] (weight_per_head) or
// [vdim]; gate rows of gate_ld numbers of type `dtype`; activation 0: sigmoid, 1: SiLU; out [tokens, heads * vdim].
MS_EXPORT int ms_head_norm_gate(const float* y, const float* bottom, const float* weight, int weight_per_head, const void* gate,
                                int dtype, int gate_ld, int gate_col, int activation, float eps, void* out, int n_tokens,
                                int heads, int vdim, cudaStream_t stream) {
  if (n_tokens == 0 || heads == 0 || vdim == 0) return 0;
  MS_REQUIRE(activation == 0 || activation == 1, "head_norm_gate: activation code %d", activation);
  if (vdim > 128 * kHeadPieces) {
    const long long rows_ = (long long)n_tokens * heads;
    MS_REQUIRE(rows_ < 2147483647LL, "head_norm_gate: %lld rows in one launch is too many", rows_);
    MS_REC_DISPATCH(dtype, (ms::launch(head_norm_gate_block_kernel<T>, (unsigned)rows_, 256, 0, stream, y, bottom, weight, weight_per_head,
                                       (const T*)gate, gate_ld, gate_col, activation, eps, (T*)out, heads, vdim)));
    MS_CHECK_LAUNCH("head_norm_gate");
    return 0;
  }
  // blocks of eight warps that walk the (token, head) pairs with the grid's stride: at most sixteen blocks a multiprocessor
  const int warps = 8;
  long long blocks = ((long long)n_tokens * heads + warps - 1) / warps;
  if (blocks > 16LL * scan_sm_count()) blocks = 16LL * scan_sm_count();
  const size_t element = dtype == MS_F32 ? 4 : 2;
  const int wide = vdim % 4 == 0 && vdim <= 128 * kHeadPieces && gate_ld % 4 == 0 && gate_col % 4 == 0 &&
                   reinterpret_cast<size_t>(y) % 16 == 0 && reinterpret_cast<size_t>(weight) % 16 == 0 &&
                   reinterpret_cast<size_t>(gate) % (4 * element) == 0 && reinterpret_cast<size_t>(out) % (4 * element) == 0;
  MS_REC_DISPATCH(dtype, (ms::launch(head_norm_gate_kernel<T>, (unsigned)blocks, warps * 32, 0, stream, y, bottom, weight,
                                     weight_per_head, (const T*)gate, gate_ld, gate_col, activation, eps, (T*)out, n_tokens,
                                     heads, vdim, wide)));
  MS_CHECK_LAUNCH("head_norm_gate");
  return 0;
}

// u float32 [tokens, width]; pre float32 [2, tokens, width]; gate_bias float32 [2, width]; rate float32 [width]; proj rows of ld
// numbers of type `dtype` (the gated branch at y_col); y_bias float32 [width] or null; the state [width] at state_offset of a
// slot's row; out [tokens, width] of type `dtype`.
MS_EXPORT int ms_gated_recurrence_scan(const float* u, const float* pre, const float* gate_bias, const float* rate,
                                       const void* proj, int dtype, int ld, int y_col, const float* y_bias, float* states,
                                       long long state_stride, int state_offset, const int* state_slots,
                                       const int* query_start, int n_requests, int n_tokens, int width, void* out,
                                       cudaStream_t stream) {
  if (n_requests == 0 || n_tokens == 0 || width == 0) return 0;
  MS_REQUIRE(n_requests <= 65535, "gated_recurrence_scan: %d requests exceed the launch limits", n_requests);
  dim3 grid((width + kRecChannels - 1) / kRecChannels, n_requests);
  MS_REC_DISPATCH(dtype, (ms::launch(gated_recurrence_scan_kernel<T>, grid, kRecWarps * 32, 0, stream, u, pre, gate_bias, rate, (const T*)proj,
                                     ld, y_col, y_bias, states, state_stride, state_offset, state_slots, query_start, width,
                                     n_tokens, (T*)out)));
  MS_CHECK_LAUNCH("gated_recurrence_scan");
  return 0;
}
