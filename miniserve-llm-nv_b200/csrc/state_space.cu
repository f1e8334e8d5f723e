// The selective state-space mixer: what lies between its input projection and its output projection.
//
//   ms_causal_conv        per channel a causal convolution of a few taps with a bias, then SiLU (or nothing), over the tokens
//                         of every request in the batch; the request's last (taps - 1) inputs are kept in its state vector
//   ms_selective_scan     per head S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T and y_t = S_t^T C_t + D x_t with
//                         dt_t = softplus(dt_t + dt_bias), walked token by token from the state the request's slot holds
//   ms_gated_group_norm   out = weight * (y silu(z)) / rms(y silu(z)), the root mean square taken per group of channels
//
// Everything here is float32 arithmetic on float32 state; only the projection that the kernels read (z, the
// convolution's inputs, dt) and the last kernel's output are in the model's compute type.  A request's tokens are
// walked in order and every sum has a fixed order, so a position's result depends on the tokens before it alone, not
// on how they were cut into steps, on what else is in the batch or on which state slot the request holds.
//
// A request's state vector: [taps - 1][channels] convolution inputs, oldest first, then [heads][P][N] head states
// (zero at admission: the zeros before a sequence's start and the empty state are the same thing).
#include "common.cuh"
#include "elementwise_vec.cuh"

namespace ms {

constexpr int kConvTokens = 16;      // tokens of a request that one thread walks
constexpr int kMaxTaps = 8;

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// grid (channel blocks, token chunks, requests); a thread owns one channel and walks kConvTokens tokens with the last
// inputs in registers.  The block of a request's FIRST chunk also writes the request's new convolution state: it is the
// only block that reads the old one (into registers, before anything is written), so nothing races.
// `in_bias` (or null) is added to every input read from `proj` (the bias of the projection that made it; the state keeps
// inputs with it, and the zeros before a sequence's start stay zeros); `bias` (or null) is the convolution's own.
template <typename T, typename U>
__global__ void __launch_bounds__(128)
causal_conv_silu_kernel(const T* __restrict__ proj, int ld, int col, int channels, int taps,
                        const float* __restrict__ weight, const float* __restrict__ bias,
                        const float* __restrict__ in_bias, int activation, float* __restrict__ states,
                        long long state_stride, int state_offset, const int* __restrict__ state_slots,
                        const int* __restrict__ query_start, U* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int request = blockIdx.z;
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  const int t0 = blockIdx.y * kConvTokens;
  if (c >= channels || t0 >= q_len) return;
  float* state = states + (long long)state_slots[request] * state_stride + state_offset;     // [taps - 1][channels]
  const int keep = taps - 1;
  float w[kMaxTaps], window[kMaxTaps];       // window[k]: the input that tap k meets at the current token
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) w[k] = k < taps ? weight[(size_t)c * taps + k] : 0.f;
  const float b = bias ? bias[c] : 0.f;
  const float ib = in_bias ? in_bias[c] : 0.f;
  // inputs before token t0: from the batch where the request's portion reaches back that far, else from the state
  // (the input at local index i < 0 is state[keep + i])
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) window[k] = 0.f;
#pragma unroll
  for (int k = 0; k + 1 < kMaxTaps; ++k) {
    if (k + 1 < taps) {                      // slots 1 .. taps - 1 hold inputs t0 - keep + k .. ; slot 0 is shifted out first
      const int i = t0 - keep + k;
      window[k + 1] = i >= 0 ? to_float(proj[(size_t)(q0 + i) * ld + col + c]) + ib : state[(size_t)(keep + i) * channels + c];
    }
  }
  if (t0 == 0) {
    // new state: the last `keep` inputs of (old state, this portion)
    for (int j = 0; j < keep; ++j) {
      const int i = q_len - keep + j;        // local index of the input that becomes state[j]
      float v = 0.f;
      if (i >= 0) {
        v = to_float(proj[(size_t)(q0 + i) * ld + col + c]) + ib;
      } else {
#pragma unroll
        for (int k = 1; k < kMaxTaps; ++k)
          if (k == 1 + keep + i) v = window[k];      // = old state[keep + i], read above, before this write
      }
      state[(size_t)j * channels + c] = v;
    }
  }
  const int t_end = min(q_len, t0 + kConvTokens);
#pragma unroll 4
  for (int t = t0; t < t_end; ++t) {
#pragma unroll
    for (int k = 0; k + 1 < kMaxTaps; ++k) window[k] = window[k + 1];
    // after the shift the newest input belongs at index taps - 1
    const float u = to_float(proj[(size_t)(q0 + t) * ld + col + c]) + ib;
    float sum = b;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k == taps - 1) window[k] = u;
      if (k < taps) sum += w[k] * window[k];
    }
    out[(size_t)(q0 + t) * channels + c] = from_float<U>(activation ? silu_f(sum) : sum);
  }
}

// The recurrence.  grid (column blocks of a head, heads, requests); a block of four warps owns 4 * CP channels (columns p)
// of one head of one request, a warp CP of them, with the 32 lanes along the state: lane j holds the entries n = j,
// j + 32, ... (R of them) of each of its columns in registers.  The tokens' B, C and x pass through shared memory in chunks
// of `tok` tokens (at most TOK; fewer where no request of the step brings that many, so that a step of single tokens
// holds next to no shared memory and more of its blocks are resident), two chunks deep: the asynchronous copies of the next chunk run while this one is multiplied, so the trip to
// the second-level cache is paid once per kernel, not once per token.  Step sizes and decays (a softplus and two
// exponentials per token and head) are computed for a chunk at a time, lane l taking token l, and handed round by shuffles.
// y_t[p] for the warp's CP columns is reduced across the lanes in one butterfly that halves the number of values a lane
// carries at each of its first steps (six shuffles for four columns, not twenty); the order of every sum is fixed.
constexpr int kScanWarps = 4;

__device__ __forceinline__ void scan_copy(float* dst, const float* src, bool valid, bool wide) {
  const unsigned to = (unsigned)__cvta_generic_to_shared(dst);
  if (wide) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(to), "l"(src), "r"(valid ? 16 : 0));
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(to), "l"(src), "r"(valid ? 4 : 0));
  }
}

// FULL: the state is a multiple of 32 numbers and the head's channels a multiple of the block's (no lane or column is idle,
// and no bound is tested per token).
// SHORT: no request of the step brings TOK tokens, and the chunks are as long as the longest portion (a run-time number).
template <typename T, int R, int CP, int TOK, bool FULL, bool SHORT>
__global__ void __launch_bounds__(kScanWarps * 32)
selective_scan_kernel(const float* __restrict__ conv, int conv_ld, const T* __restrict__ proj, int ld, int dt_col,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      float* __restrict__ states, long long state_stride, int state_offset,
                      const int* __restrict__ state_slots, const int* __restrict__ query_start, int heads, int P, int N,
                      int groups, float* __restrict__ y, int wide, int short_tok) {
  grid_dependency_wait();
  grid_dependency_launch();
  constexpr int COLS = kScanWarps * CP;
  const int tok = SHORT ? short_tok : TOK;
  extern __shared__ __align__(16) float scan_smem[];
  const int n_pad = (N + 3) & ~3;                           // a token's B (or C) row in shared memory
  const int stage_floats = tok * (2 * n_pad + COLS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y, request = blockIdx.z;
  const int block_p0 = blockIdx.x * COLS, p0 = block_p0 + warp * CP;
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  if (q_len <= 0) return;                                   // (the whole block)
  const int group = head / (heads / groups);
  const int inner = heads * P;
  const float* conv_x = conv + (size_t)q0 * conv_ld + head * P + block_p0;
  const float* conv_b = conv + (size_t)q0 * conv_ld + inner + group * N;
  const float* conv_c = conv_b + (size_t)groups * N;
  float* y_row = y + (size_t)q0 * inner + head * P + p0;
  float* state = states + (long long)state_slots[request] * state_stride + state_offset + ((size_t)head * P + p0) * N;

  // one chunk's copies: rows of B and C (n_pad floats each, in pieces of four floats or single floats) and COLS values of x
  auto fetch = [&](int chunk, int stage) {
    float* b_s = scan_smem + stage * stage_floats;
    float* c_s = b_s + tok * n_pad;
    float* x_s = c_s + tok * n_pad;
    const int t0 = chunk * tok;
    if (wide) {
      const int pieces = n_pad / 4;
      for (int i = tid; i < tok * pieces; i += kScanWarps * 32) {
        const int t = i / pieces, piece = (i % pieces) * 4;
        const bool valid = t0 + t < q_len;
        const size_t row = valid ? (size_t)(t0 + t) * conv_ld : 0;
        scan_copy(b_s + t * n_pad + piece, conv_b + row + piece, valid, true);
        scan_copy(c_s + t * n_pad + piece, conv_c + row + piece, valid, true);
      }
    } else {
      for (int i = tid; i < tok * N; i += kScanWarps * 32) {
        const int t = i / N, n = i % N;
        const bool valid = t0 + t < q_len;
        const size_t row = valid ? (size_t)(t0 + t) * conv_ld : 0;
        scan_copy(b_s + t * n_pad + n, conv_b + row + n, valid, false);
        scan_copy(c_s + t * n_pad + n, conv_c + row + n, valid, false);
      }
    }
    for (int i = tid; i < tok * COLS; i += kScanWarps * 32) {
      const int t = i / COLS, col = i % COLS;
      const bool valid = t0 + t < q_len && block_p0 + col < P;
      scan_copy(x_s + i, conv_x + (valid ? (size_t)(t0 + t) * conv_ld + col : 0), valid, false);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  const int chunks = (q_len + tok - 1) / tok;
  fetch(0, 0);
  float s[CP][R];
#pragma unroll
  for (int cp = 0; cp < CP; ++cp)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int n = lane + 32 * r;
      s[cp][r] = (p0 + cp < P && n < N) ? state[(size_t)cp * N + n] : 0.f;
    }
  const float a = -expf(a_log[head]);
  const float bias = dt_bias[head], skip = d_skip[head];
  auto raw_step = [&](int chunk) {                          // the step-size logit of token chunk * tok + lane
    const int t = chunk * tok + lane;
    return (lane < tok && t < q_len) ? to_float(proj[(size_t)(q0 + t) * ld + dt_col + head]) : 0.f;
  };
  float raw_next = raw_step(0);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const float raw = raw_next + bias;
    if (chunk + 1 < chunks) {
      fetch(chunk + 1, (chunk + 1) & 1);
      raw_next = raw_step(chunk + 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float my_step = raw > 20.f ? raw : log1pf(expf(raw));         // softplus; above 20 the two agree in float32
    const float my_decay = expf(a * my_step);
    const float* b_s = scan_smem + (chunk & 1) * stage_floats;
    const float* c_s = b_s + tok * n_pad;
    const float* x_s = c_s + tok * n_pad + warp * CP;
    const int t0 = chunk * tok, count = min(tok, q_len - t0);
    if (p0 < P) {
      float* y_at = y_row + (size_t)t0 * inner;
#pragma unroll 4
      for (int u = 0; u < count; ++u, y_at += inner) {
        float b[R], c[R], x[CP];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int n = lane + 32 * r;
          b[r] = (FULL || n < N) ? b_s[u * n_pad + n] : 0.f;
          c[r] = (FULL || n < N) ? c_s[u * n_pad + n] : 0.f;
        }
        if constexpr (CP == 4) {                            // (16-byte aligned: COLS and CP are multiples of four)
          const float4 four = *reinterpret_cast<const float4*>(x_s + u * COLS);
          x[0] = four.x, x[1] = four.y, x[2] = four.z, x[3] = four.w;
        } else {
#pragma unroll
          for (int cp = 0; cp < CP; ++cp) x[cp] = x_s[u * COLS + cp];
        }
        const float step = __shfl_sync(0xffffffffu, my_step, u), decay = __shfl_sync(0xffffffffu, my_decay, u);
        float partial[CP];
#pragma unroll
        for (int cp = 0; cp < CP; ++cp) {
          const float in = step * x[cp];
          float sum = 0.f;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            s[cp][r] = decay * s[cp][r] + in * b[r];
            sum += s[cp][r] * c[r];
          }
          partial[cp] = sum;
        }
        // butterfly: the upper half of the lanes goes on with the upper half of the columns, and so on; the lanes
        // 0, 32 / CP, 2 * 32 / CP, ... end up with the totals of columns 0, 1, 2, ...
        float value, mine_x;
        if constexpr (CP == 4) {
          const bool upper = lane & 16;
          const float keep0 = upper ? partial[2] : partial[0], keep1 = upper ? partial[3] : partial[1];
          const float give0 = upper ? partial[0] : partial[2], give1 = upper ? partial[1] : partial[3];
          const float v0 = keep0 + __shfl_xor_sync(0xffffffffu, give0, 16), v1 = keep1 + __shfl_xor_sync(0xffffffffu, give1, 16);
          const bool second = lane & 8;
          value = (second ? v1 : v0) + __shfl_xor_sync(0xffffffffu, second ? v0 : v1, 8);
          value += __shfl_xor_sync(0xffffffffu, value, 4);
          mine_x = upper ? (second ? x[3] : x[2]) : (second ? x[1] : x[0]);
        } else {
          const bool upper = lane & 16;
          value = (upper ? partial[CP - 1] : partial[0]) + __shfl_xor_sync(0xffffffffu, upper ? partial[0] : partial[CP - 1], 16);
          value += __shfl_xor_sync(0xffffffffu, value, 8);
          value += __shfl_xor_sync(0xffffffffu, value, 4);
          mine_x = upper ? x[CP - 1] : x[0];
        }
        value += __shfl_xor_sync(0xffffffffu, value, 2);
        value += __shfl_xor_sync(0xffffffffu, value, 1);
        const int column = lane / (32 / CP);
        if ((lane & (32 / CP - 1)) == 0 && (FULL || p0 + column < P)) y_at[column] = value + skip * mine_x;
      }
    }
    __syncthreads();                                        // the stage may be refilled
  }
  if (p0 < P) {
#pragma unroll
    for (int cp = 0; cp < CP; ++cp)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int n = lane + 32 * r;
        if (p0 + cp < P && n < N) state[(size_t)cp * N + n] = s[cp][r];
      }
  }
}

// One block per (token, group), sixteen-byte loads and stores, the group's values in registers between the two passes: each
// thread keeps up to CHUNKS runs of eight numbers.  Group size, row lengths and z's column multiples of eight.
template <typename T, int CHUNKS>
__global__ void gated_group_norm_vec_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col,
                                            const float* __restrict__ weight, int groups, int inner, float eps,
                                            T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t token = blockIdx.x;
  const int size = inner / groups, c0 = blockIdx.y * size;
  Vec8 v[CHUNKS];
  float sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < size) {
      v[i] = load8(y + token * inner + c0 + c);
      const Vec8 z = load8(proj + token * ld + z_col + c0 + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[i].v[e] *= silu_f(z.v[e]);
        sum_sq += v[i].v[e] * v[i].v[e];
      }
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)size + eps);
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < size) {
      const Vec8 w = load8(weight + c0 + c);
      Vec8 r;
#pragma unroll
      for (int e = 0; e < 8; ++e) r.v[e] = v[i].v[e] * inv * w.v[e];
      store8(out + token * inner + c0 + c, r);
    }
  }
}

// One block per (token, group) with the group's values in registers between the two passes (groups of up to 16 numbers per
// thread): the row is read once.
constexpr int kGroupNormPerThread = 16;

template <typename T>
__global__ void gated_group_norm_once_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col,
                                             const float* __restrict__ weight, int groups, int inner, float eps,
                                             T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t token = blockIdx.x;
  const int size = inner / groups, c0 = blockIdx.y * size;
  float v[kGroupNormPerThread];
  float sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < kGroupNormPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < size ? y[token * inner + c0 + c] * silu_f(to_float(proj[token * ld + z_col + c0 + c])) : 0.f;
    sum_sq += v[i] * v[i];
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)size + eps);
#pragma unroll
  for (int i = 0; i < kGroupNormPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < size) out[token * inner + c0 + c] = from_float<T>(v[i] * inv * weight[c0 + c]);
  }
}

// One block per (token, group): v = y * silu(z); out = weight * v / sqrt(mean(v^2) + eps).
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col,
                                        const float* __restrict__ weight, int groups, int inner, float eps,
                                        T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t token = blockIdx.x;
  const int size = inner / groups, c0 = blockIdx.y * size;
  float sum_sq = 0.f;
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    const float v = y[token * inner + c0 + c] * silu_f(to_float(proj[token * ld + z_col + c0 + c]));
    sum_sq += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)size + eps);
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    const float v = y[token * inner + c0 + c] * silu_f(to_float(proj[token * ld + z_col + c0 + c]));
    out[token * inner + c0 + c] = from_float<T>(v * inv * weight[c0 + c]);
  }
}

// The same with one warp per (token, group) and the group's values in registers (a group of up to 32 * PER numbers): the
// row is read once.
template <typename T, int PER>
__global__ void gated_group_norm_warp_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col,
                                             const float* __restrict__ weight, int groups, int inner, float eps,
                                             T* __restrict__ out, long long items) {
  grid_dependency_wait();
  grid_dependency_launch();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const size_t token = item / groups;
  const int size = inner / groups, c0 = (int)(item % groups) * size;
  float v[PER];
  float sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = lane + 32 * i;
    v[i] = c < size ? y[token * inner + c0 + c] * silu_f(to_float(proj[token * ld + z_col + c0 + c])) : 0.f;
    sum_sq += v[i] * v[i];
  }
  const float inv = 1.0f / sqrtf(warp_sum(sum_sq) / (float)size + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = lane + 32 * i;
    if (c < size) out[token * inner + c0 + c] = from_float<T>(v[i] * inv * weight[c0 + c]);
  }
}

}  // namespace ms

using namespace ms;

#define MS_SS_DISPATCH(dtype, ...)                               \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// proj [tokens, ld]: the convolution's inputs are its columns col .. col + channels; weight float32 [channels, taps] (the
// last tap is the current token's), bias float32 [channels] or null; in_bias float32 [channels] or null (added to the inputs
// as they are read); activation 0: none, 1: SiLU; states float32, one row of state_stride numbers per slot, the
// convolution's part at state_offset; out [tokens, channels], float32 or (out_like_proj != 0) of proj's type.
MS_EXPORT int ms_causal_conv(const void* proj, int dtype, int ld, int col, int channels, int taps, const float* weight,
                             const float* bias, const float* in_bias, int activation, float* states, long long state_stride,
                             int state_offset, const int* state_slots, const int* query_start, int n_requests,
                             int max_query_len, void* out, int out_like_proj, cudaStream_t stream) {
  if (n_requests == 0 || max_query_len == 0 || channels == 0) return 0;
  MS_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal_conv: %d taps outside 1..%d", taps, kMaxTaps);
  MS_REQUIRE(activation == 0 || activation == 1, "causal_conv: activation code %d", activation);
  const int chunks = (max_query_len + kConvTokens - 1) / kConvTokens;
  MS_REQUIRE(chunks <= 65535 && n_requests <= 65535, "causal_conv: grid %d x %d exceeds the launch limits", chunks, n_requests);
  dim3 grid((channels + 127) / 128, chunks, n_requests);
  if (out_like_proj) {
    MS_SS_DISPATCH(dtype, (ms::launch(causal_conv_silu_kernel<T, T>, grid, 128, 0, stream, (const T*)proj, ld, col, channels, taps,
                                      weight, bias, in_bias, activation, states, state_stride, state_offset, state_slots,
                                      query_start, (T*)out)));
  } else {
    MS_SS_DISPATCH(dtype, (ms::launch(causal_conv_silu_kernel<T, float>, grid, 128, 0, stream, (const T*)proj, ld, col, channels, taps,
                                      weight, bias, in_bias, activation, states, state_stride, state_offset, state_slots,
                                      query_start, (float*)out)));
  }
  MS_CHECK_LAUNCH("causal_conv");
  return 0;
}

constexpr int kScanMaxState = 256;      // 32 lanes with up to eight entries each

MS_EXPORT int ms_scan_max_state() { return kScanMaxState; }

// conv float32 [tokens, conv_ld] = [x: heads * P | B: groups * N | C: groups * N]; dt is column dt_col + head of proj;
// dt_bias, a_log, d float32 [heads]; the heads' states [heads][P][N] at state_offset of a slot's row; y float32
// [tokens, heads * P].  max_query_len: an upper bound of the tokens a request brings (it sizes the chunks).
MS_EXPORT int ms_selective_scan(const float* conv, int conv_ld, const void* proj, int dtype, int ld, int dt_col,
                                const float* dt_bias, const float* a_log, const float* d, float* states,
                                long long state_stride, int state_offset, const int* state_slots, const int* query_start,
                                int n_requests, int max_query_len, int heads, int p, int n_state, int groups, float* y,
                                cudaStream_t stream) {
  if (n_requests == 0 || max_query_len <= 0) return 0;
  MS_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "selective_scan: %d heads in %d groups", heads, groups);
  MS_REQUIRE(n_state >= 1 && n_state <= kScanMaxState, "selective_scan: a state of %d numbers per channel outside 1..%d",
             n_state, kScanMaxState);
  MS_REQUIRE(heads <= 65535 && n_requests <= 65535, "selective_scan: grid exceeds the launch limits");
  const int per_lane = (n_state + 31) / 32;
  // the copies into shared memory move four floats at a time where every row of B and C starts on a 16-byte boundary
  const int inner = heads * p;
  const int wide = (n_state % 4 == 0 && conv_ld % 4 == 0 && inner % 4 == 0 && (reinterpret_cast<uintptr_t>(conv) & 15) == 0) ? 1 : 0;
  const int full = (n_state % 32 == 0 && p % (kScanWarps * (per_lane <= 4 ? 4 : 2)) == 0) ? 1 : 0;
  // columns per warp: four where a lane holds few entries (more products per load), two where it holds many
#define MS_SCAN(R, CP, TOK)                                                                                                    \
  {                                                                                                                            \
    dim3 grid((p + kScanWarps * CP - 1) / (kScanWarps * CP), heads, n_requests);                                              \
    const int tok = max_query_len < TOK ? max_query_len : TOK;                                                                \
    const size_t smem = (size_t)2 * tok * (2 * ((n_state + 3) & ~3) + kScanWarps * CP) * sizeof(float);                        \
    MS_SS_DISPATCH(dtype, {                                                                                                    \
      const bool brief = tok < TOK;                                                                                            \
      auto kernel = brief ? (full ? selective_scan_kernel<T, R, CP, TOK, true, true> : selective_scan_kernel<T, R, CP, TOK, false, true>)  \
                          : (full ? selective_scan_kernel<T, R, CP, TOK, true, false> : selective_scan_kernel<T, R, CP, TOK, false, false>); \
      static bool configured[4] = {false, false, false, false};                                                                                          \
      if (!configured[full + 2 * brief]) {                                                                                     \
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * TOK * (2 * 32 * R + kScanWarps * CP) * 4); \
        if (e != cudaSuccess) MS_FAIL("selective_scan: shared memory refused: %s", cudaGetErrorString(e));                     \
        configured[full + 2 * brief] = true;                                                                                   \
      }                                                                                                                        \
      ms::launch(kernel, grid, kScanWarps * 32, smem, stream, conv, conv_ld, (const T*)proj, ld, dt_col, dt_bias, a_log, d,    \
                 states, state_stride, state_offset, state_slots, query_start, heads, p, n_state, groups, y, wide, tok);       \
    })                                                                                                                         \
  }
  if (per_lane <= 1) MS_SCAN(1, 4, 32) else if (per_lane <= 2) MS_SCAN(2, 4, 32) else if (per_lane <= 4) MS_SCAN(4, 4, 32) else MS_SCAN(8, 2, 16)
#undef MS_SCAN
  MS_CHECK_LAUNCH("selective_scan");
  return 0;
}

// y float32 [tokens, inner]; z is columns z_col .. z_col + inner of proj [tokens, ld]; weight float32 [inner];
// out [tokens, inner] in proj's type.
MS_EXPORT int ms_gated_group_norm(const float* y, const void* proj, int dtype, int ld, int z_col, const float* weight,
                                  int groups, int inner, float eps, void* out, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || inner == 0) return 0;
  MS_REQUIRE(groups > 0 && inner % groups == 0 && groups <= 65535, "gated_group_norm: %d channels in %d groups", inner, groups);
  const int size = inner / groups;
  if (size % 8 == 0 && ld % 8 == 0 && z_col % 8 == 0 && size >= 256 && size <= 8192) {
    const int runs = size / 8;
    const int vec_threads = runs >= 256 ? 256 : ((runs + 31) / 32) * 32;
    const int chunks = (runs + vec_threads - 1) / vec_threads;
    dim3 vec_grid(n_tokens, groups);
#define MS_GROUP_NORM_VEC(C)                                                                                                  \
  MS_SS_DISPATCH(dtype, (ms::launch(gated_group_norm_vec_kernel<T, C>, vec_grid, vec_threads, 0, stream, y, (const T*)proj, ld,     \
                                    z_col, weight, groups, inner, eps, (T*)out)))
    if (chunks == 1) { MS_GROUP_NORM_VEC(1); } else if (chunks == 2) { MS_GROUP_NORM_VEC(2); } else { MS_GROUP_NORM_VEC(4); }
#undef MS_GROUP_NORM_VEC
    MS_CHECK_LAUNCH("gated_group_norm");
    return 0;
  }
  if (size <= 128) {
    const long long items = (long long)n_tokens * groups;
    const long long blocks = (items + 3) / 4;
    MS_REQUIRE(blocks < 2147483647LL, "gated_group_norm: %lld groups in one launch is too many", items);
#define MS_GROUP_NORM(PER)                                                                                                   \
  MS_SS_DISPATCH(dtype, (ms::launch(gated_group_norm_warp_kernel<T, PER>, (unsigned)blocks, 128, 0, stream, y, (const T*)proj, ld, \
                                    z_col, weight, groups, inner, eps, (T*)out, items)))
    MS_GROUP_NORM(4);
#undef MS_GROUP_NORM
    MS_CHECK_LAUNCH("gated_group_norm");
    return 0;
  }
  dim3 grid(n_tokens, groups);
  if (size <= 256 * kGroupNormPerThread) {
    const int once_threads = size >= 2048 ? 256 : (size >= 512 ? 128 : 64);
    MS_SS_DISPATCH(dtype, (ms::launch(gated_group_norm_once_kernel<T>, grid, once_threads, 0, stream, y, (const T*)proj, ld, z_col,
                                      weight, groups, inner, eps, (T*)out)));
    MS_CHECK_LAUNCH("gated_group_norm");
    return 0;
  }
  const int threads = 256;
  MS_SS_DISPATCH(dtype, (ms::launch(gated_group_norm_kernel<T>, grid, threads, 0, stream, y, (const T*)proj, ld, z_col, weight,
                                    groups, inner, eps, (T*)out)));
  MS_CHECK_LAUNCH("gated_group_norm");
  return 0;
}
