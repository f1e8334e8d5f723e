// A feed-forward of routed experts, on the device from the router to the weighted sum, so that a step never waits
// for the host to learn which experts were chosen (and a captured decode step can hold it):
//
//   ms_router_topk      float32 router logits W x + b of every token (one kernel), the `top` largest and the softmax
//                       over those alone (a second)
//   ms_expert_route     sorts the (token, choice) pairs by expert: segment offsets, the pairs in sorted order and
//                       each pair's place in that order
//   ms_expert_linear    one product per expert over its segment of rows (rows gathered from the tokens for the first
//                       product of an expert), optional squared-ReLU on the results
//   ms_expert_combine   out[token] = sum over its choices of weight * result row (+ a shared expert's output)
//   ms_relu_square      x = max(x, 0)^2 in place
//   ms_router_choose    another way to route: scores are the softmax over ALL router outputs, a correction is added for the
//                       choice only, the outputs form groups of which only the best can be chosen from, and the weights are
//                       the chosen scores as they are
//   ms_clamped_glu      out = g sigmoid(1.702 g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit) for
//                       alternating (gate, up) columns; the same activation is an epilogue of ms_expert_linear
//
// An expert id at or above the number of experts with weights stands for an identity expert (its output is its input):
// ms_expert_route sorts such pairs behind the others, ms_expert_linear is given the smaller expert count and never
// touches them, and ms_expert_combine reads the token's own row for them.
//
// The products accumulate in float32.  The float32 form has one thread per output element summing k in ascending order;
// the bfloat16 form runs on the tensor cores.  In both a row's result depends on the row and its expert alone, not on
// what else is in the batch or on where the row was sorted to.
#include "common.cuh"
#include "mma_common.cuh"

namespace ms {

// Router logits, float32: logits[n][e] = sum_c x_n[c] W[e, c] + b[e].  A block of eight warps holds the rows of RT
// tokens in shared memory (in their stored type: the conversion is exact) and takes `per_block` experts, warp w the
// experts w, w + 8, ... of them: it reads an expert's weight row once, sixteen bytes per lane and two such loads
// ahead of the sums, and forms the RT tokens' logits beside one another.  A logit is the fixed tree over the lanes'
// sums of their own pieces in ascending order, so it does not depend on the token's neighbours or on the grid.
template <typename T, int RT>
__global__ void __launch_bounds__(256)
router_logits_kernel(const T* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ bias,
                     int width, int experts, int per_block, float* __restrict__ logits, int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ __align__(16) unsigned char router_smem[];
  T* xs = reinterpret_cast<T*>(router_smem);          // [RT][width]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * RT;
  constexpr int VEC = 16 / sizeof(T);                 // elements per 16-byte load
  if (width % VEC == 0) {
    const int per_row = width / VEC;
#pragma unroll 4
    for (int i = threadIdx.x; i < RT * per_row; i += blockDim.x) {
      const int t = i / per_row, c = (i % per_row) * VEC;
      const uint4 v = n0 + t < n_tokens ? *reinterpret_cast<const uint4*>(x + (size_t)(n0 + t) * width + c) : make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(xs + t * width + c) = v;
    }
  } else {
    for (int i = threadIdx.x; i < RT * width; i += blockDim.x) {
      const int t = i / width, c = i % width;
      xs[i] = n0 + t < n_tokens ? x[(size_t)(n0 + t) * width + c] : from_float<T>(0.f);
    }
  }
  __syncthreads();
  const int e_end = min(experts, (blockIdx.y + 1) * per_block);
  for (int e = blockIdx.y * per_block + warp; e < e_end; e += 8) {
    const float* w = weight + (size_t)e * width;
    float sum[RT];
#pragma unroll
    for (int t = 0; t < RT; ++t) sum[t] = 0.f;
    if ((width & 3) == 0) {
      for (int c = lane * 4; c < width; c += 256) {
        const float4 w0 = *reinterpret_cast<const float4*>(w + c);
        const bool more = c + 128 < width;
        const float4 w1 = more ? *reinterpret_cast<const float4*>(w + c + 128) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int t = 0; t < RT; ++t) {
          const T* row = xs + t * width + c;
          sum[t] += to_float(row[0]) * w0.x;
          sum[t] += to_float(row[1]) * w0.y;
          sum[t] += to_float(row[2]) * w0.z;
          sum[t] += to_float(row[3]) * w0.w;
        }
        if (more) {
#pragma unroll
          for (int t = 0; t < RT; ++t) {
            const T* row = xs + t * width + c + 128;
            sum[t] += to_float(row[0]) * w1.x;
            sum[t] += to_float(row[1]) * w1.y;
            sum[t] += to_float(row[2]) * w1.z;
            sum[t] += to_float(row[3]) * w1.w;
          }
        }
      }
    } else {
      for (int c = lane; c < width; c += 32) {
        const float wc = w[c];
#pragma unroll
        for (int t = 0; t < RT; ++t) sum[t] += to_float(xs[t * width + c]) * wc;
      }
    }
#pragma unroll
    for (int t = 0; t < RT; ++t) {
      const float total = warp_sum(sum[t]);
      if (lane == 0 && n0 + t < n_tokens) logits[(size_t)(n0 + t) * experts + e] = total + (bias ? bias[e] : 0.f);
    }
  }
}

// One warp per token: the `top` largest of its logits one after the other (ties: the lower index); weights are
// exp(l - l_max) / sum over the taken.
__global__ void router_select_kernel(const float* __restrict__ all_logits, int experts, int top, int* __restrict__ ids,
                                     float* __restrict__ weights, int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float select_smem[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* logits = select_smem + (size_t)warp * (experts + top);
  float* taken = logits + experts;
  const int n = blockIdx.x * warps + warp;
  if (n >= n_tokens) return;
  for (int e = lane; e < experts; e += 32) logits[e] = all_logits[(size_t)n * experts + e];
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = logits[e];
      if (v > best) { best = v; best_e = e; }       // ascending e: the lower index wins a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (lane == 0) {
      taken[k] = best;
      ids[(size_t)n * top + k] = best_e;
      logits[best_e] = -INFINITY;
    }
    __syncwarp();
  }
  const float peak = taken[0];
  float total = 0.f;
  for (int k = 0; k < top; ++k) total += expf(taken[k] - peak);
  for (int k = lane; k < top; k += 32) weights[(size_t)n * top + k] = expf(taken[k] - peak) / total;
}

// One warp per token.  scores = softmax over the first `total` logits of the row; choice = score + correction; the
// outputs form `group_count` equal groups of neighbours, a group's score is its largest choice score, and only members of
// the `group_keep` best groups (ties: the lower group) can be chosen; the `top` largest choice scores among those are
// taken one after the other (ties: the lower index); weights are the taken outputs' scores, not renormalised.  A choice
// score that is not a number counts as the smallest, so that every id written is a valid one.
__global__ void router_choose_kernel(const float* __restrict__ all_logits, int ld, int total, int top,
                                     const float* __restrict__ correction, int group_count, int group_keep,
                                     int* __restrict__ ids, float* __restrict__ weights, int n_tokens, int sigmoid_scores) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float select_smem[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* score = select_smem + (size_t)warp * (2 * total + group_count);
  float* choice = score + total;
  float* group_best = choice + total;
  const int n = blockIdx.x * warps + warp;
  if (n >= n_tokens) return;
  const float* logits = all_logits + (size_t)n * ld;
  float peak = -INFINITY;
  for (int e = lane; e < total; e += 32) peak = fmaxf(peak, logits[e]);
  peak = warp_max(peak);
  float sum = 0.f;
  for (int e = lane; e < total; e += 32) {
    const float v = expf(logits[e] - peak);
    score[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < total; e += 32) {
    // scores: the softmax over all outputs, or the sigmoid of every output on its own
    const float v = sigmoid_scores ? 1.f / (1.f + expf(-logits[e])) : score[e] / sum;
    score[e] = v;
    float c = v + (correction ? correction[e] : 0.f);
    if (!(c == c)) c = -3.0e38f;
    choice[e] = fmaxf(c, -3.0e38f);
  }
  __syncwarp();
  const int per_group = total / group_count;
  if (group_keep < group_count) {
    for (int g = lane; g < group_count; g += 32) {
      float best = -INFINITY;
      for (int i = 0; i < per_group; ++i) best = fmaxf(best, choice[g * per_group + i]);
      group_best[g] = best;
    }
    __syncwarp();
    // a group is kept if fewer than `group_keep` groups come before it (a larger score, or the same with a lower index)
    for (int g = lane; g < group_count; g += 32) {
      const float mine = group_best[g];
      int before = 0;
      for (int o = 0; o < group_count; ++o) before += (group_best[o] > mine || (group_best[o] == mine && o < g)) ? 1 : 0;
      if (before >= group_keep)
        for (int i = 0; i < per_group; ++i) choice[g * per_group + i] = -INFINITY;
    }
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < total; e += 32) {
      const float v = choice[e];
      if (v > best) { best = v; best_e = e; }       // ascending e: the lower index wins a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (lane == 0) {
      ids[(size_t)n * top + k] = best_e;
      weights[(size_t)n * top + k] = score[best_e];
      choice[best_e] = -INFINITY;
    }
    __syncwarp();
  }
}

// One block.  offsets[e] .. offsets[e + 1] is expert e's segment of the sorted order; order[i] is the pair (token * top
// + choice) at place i, place[pair] its place.  Within a segment the order is arbitrary: rows are computed independently.
__global__ void expert_route_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ offsets,
                                    int* __restrict__ order, int* __restrict__ place) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ int route_smem[];
  int* counts = route_smem;              // [experts]
  int* cursor = route_smem + experts;    // [experts]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int running = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = running;
      cursor[e] = running;
      running += counts[e];
    }
    offsets[experts] = running;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int at = atomicAdd(&cursor[ids[i]], 1);
    order[at] = i;
    place[i] = at;
  }
}

constexpr int EBM = 64, EBN = 64, EBK = 16, ETM = 4, ETN = 4;

// epilogues of the experts' products
enum : int { kActNone = 0, kActReluSquare = 1, kActClampedGlu = 2, kActSiluGlu = 3 };

// silu(s gate) (s up): the gated expert computed on s times its input (its first products are linear)
__device__ __forceinline__ float silu_glu(float gate, float up, float s) {
  const float g = s * gate;
  return g / (1.f + expf(-g)) * (s * up);
}

// g = min(gate, limit), u = clamp(up, -limit, limit); g sigmoid(1.702 g) (u + 1)
__device__ __forceinline__ float clamped_glu(float gate, float up, float limit) {
  const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
  return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
}

// C[i, :] = act(A[src(i), :] W_e^T) for every place i of expert e's segment; W [experts, N, K].  blockIdx.y walks the
// row tiles of all segments one after the other (a segment's last tile may be partial); tiles beyond the last do nothing.
// src(i) = order[i] / top with `order` (rows gathered from the tokens), else i.
template <typename T>
__global__ void __launch_bounds__(256)
expert_linear_kernel(const T* __restrict__ A, int lda, const int* __restrict__ order, int top, const T* __restrict__ W,
                     T* __restrict__ C, int ldc, const int* __restrict__ offsets, int experts, int N, int K, int activation,
                     float limit, const float* __restrict__ pair_scale) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float As[EBK][EBM + 4];
  __shared__ float Ws[EBK][EBN + 4];
  __shared__ int src_row[EBM];
  int tile = blockIdx.y, expert = 0, first = 0, end = 0;
  for (; expert < experts; ++expert) {
    first = offsets[expert];
    end = offsets[expert + 1];
    const int tiles = (end - first + EBM - 1) / EBM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (expert == experts) return;
  const int m0 = first + tile * EBM, n0 = blockIdx.x * EBN;
  const int tid = threadIdx.x;
  if (tid < EBM) {
    const int i = m0 + tid;
    src_row[tid] = i < end ? (order ? order[i] / top : i) : -1;
  }
  __syncthreads();
  const T* We = W + (size_t)expert * N * K;
  const int tx = tid % 16, ty = tid / 16;
  const int load_row = tid / 4, load_k = (tid % 4) * 4;
  const int a_row = src_row[load_row];
  float acc[ETM][ETN] = {};
  for (int k0 = 0; k0 < K; k0 += EBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + load_k + i;
      const int wn = n0 + load_row;
      As[load_k + i][load_row] = (a_row >= 0 && k < K) ? to_float(A[(size_t)a_row * lda + k]) : 0.f;
      Ws[load_k + i][load_row] = (wn < N && k < K) ? to_float(We[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < EBK; ++k) {
      float a[ETM], w[ETN];
#pragma unroll
      for (int i = 0; i < ETM; ++i) a[i] = As[k][ty * ETM + i];
#pragma unroll
      for (int j = 0; j < ETN; ++j) w[j] = Ws[k][tx * ETN + j];
#pragma unroll
      for (int i = 0; i < ETM; ++i)
#pragma unroll
        for (int j = 0; j < ETN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < ETM; ++i) {
    const int m = m0 + ty * ETM + i;
    if (m >= end) continue;
    if (activation >= kActClampedGlu) {           // columns alternate (gate, up): two of them give one result
      const float s = (activation == kActSiluGlu && pair_scale) ? pair_scale[order[m]] : 1.f;
#pragma unroll
      for (int j = 0; j < ETN; j += 2) {
        const int n = n0 + tx * ETN + j;
        if (n + 1 < N)
          C[(size_t)m * ldc + n / 2] = from_float<T>(activation == kActSiluGlu ? silu_glu(acc[i][j], acc[i][j + 1], s)
                                                                                  : clamped_glu(acc[i][j], acc[i][j + 1], limit));
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < ETN; ++j) {
      const int n = n0 + tx * ETN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (activation == kActReluSquare) { v = fmaxf(v, 0.f); v *= v; }
      C[(size_t)m * ldc + n] = from_float<T>(v);
    }
  }
}

// The same product on the tensor cores (bfloat16, mma.sync.m16n8k16, float32 sums): tiles of 64 rows x 128 columns, k in
// steps of GBK through GSTAGES cp.async stages; eight warps, each 32 x 32 of the tile.  Rows of A are gathered through
// `order` as above (a row's address is looked up once).  Inner size and column count multiples of 8.  (Measured against k
// steps of 32 in three stages, which fit three blocks on a multiprocessor instead of two: steps of few rows, which only
// stream the experts' weights, 25 -> 19 us per launch, half the barriers and twice the bytes on their way; prompt steps
// 155 -> 147 us.)
// Where the segments are long (prompt steps) the tiles have 128 rows, so that every weight fragment a warp fetches from shared
// memory feeds four products instead of two (three stages then, two blocks a multiprocessor as before).
constexpr int GBN = 128, GBK = 64;

template <int GBM, int GSTAGES>
__global__ void __launch_bounds__(256)
expert_linear_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ order, int top,
                         const __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ C, int ldc,
                         const int* __restrict__ offsets, int experts, int N, int K, int activation, float limit,
                         const float* __restrict__ pair_scale) {
  grid_dependency_wait();
  grid_dependency_launch();
  constexpr int GLD = GBK + 8;          // elements between the rows of a stage
  constexpr int CPR = GBK / 8;          // 16-byte pieces per row of a stage
  extern __shared__ __align__(16) unsigned char expert_smem[];
  typedef __nv_bfloat16 (*StageA)[GBM][GLD];
  typedef __nv_bfloat16 (*StageB)[GBN][GLD];
  StageA As = reinterpret_cast<StageA>(expert_smem);
  StageB Bs = reinterpret_cast<StageB>(expert_smem + sizeof(__nv_bfloat16) * GSTAGES * GBM * GLD);
  __shared__ int src_row[GBM];
  int tile = blockIdx.y, expert = 0, first = 0, end = 0;
  for (; expert < experts; ++expert) {
    first = offsets[expert];
    end = offsets[expert + 1];
    const int tiles = (end - first + GBM - 1) / GBM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (expert == experts) return;
  const int m0 = first + tile * GBM, n0 = blockIdx.x * GBN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < GBM) {
    const int i = m0 + tid;
    src_row[tid] = i < end ? (order ? order[i] / top : i) : -1;
  }
  __syncthreads();
  const __nv_bfloat16* We = W + (size_t)expert * N * K;
  auto load_stage = [&](int stage, int k0) {
#pragma unroll
    for (int i = 0; i < GBM * CPR / 256; ++i) {                    // the A tile: its rows' addresses were looked up above
      const int piece = tid + i * 256, r = piece / CPR, c = (piece % CPR) * 8;
      const int src = src_row[r];
      cp_async_16(&As[stage][r][c], A + (size_t)(src < 0 ? 0 : src) * lda + k0 + c, src >= 0 && k0 + c < K);
    }
#pragma unroll
    for (int i = 0; i < GBN * CPR / 256; ++i) {
      const int piece = tid + i * 256, r = piece / CPR, c = (piece % CPR) * 8;
      const bool valid = n0 + r < N && k0 + c < K;
      cp_async_16(&Bs[stage][r][c], We + (size_t)(valid ? n0 + r : 0) * K + (valid ? k0 + c : 0), valid);
    }
  };
  const int k_tiles = (K + GBK - 1) / GBK;
#pragma unroll
  for (int s = 0; s < GSTAGES - 1; ++s) {
    if (s < k_tiles) load_stage(s, s * GBK);
    cp_async_commit();
  }
  const int warp_m = warp >> 2, warp_n = warp & 3;
  constexpr int MI = GBM / 32;          // 16-row pieces of a warp's rows
  float acc[MI][4][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  for (int kt = 0; kt < k_tiles; ++kt) {
    cp_async_wait<GSTAGES - 2>();
    __syncthreads();
    const int next = kt + GSTAGES - 1;
    if (next < k_tiles) load_stage(next % GSTAGES, next * GBK);
    cp_async_commit();
    const int stage = kt % GSTAGES;
#pragma unroll
    for (int kk = 0; kk < GBK / 16; ++kk) {
      unsigned a[MI][4], b[2][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        ldmatrix_x4(a[mi], &As[stage][warp_m * (GBM / 2) + mi * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int np = 0; np < 2; ++np)
        ldmatrix_x4(b[np], &Bs[stage][warp_n * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8][kk * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          mma_bf16(acc[mi][2 * np], a[mi], b[np][0], b[np][1]);
          mma_bf16(acc[mi][2 * np + 1], a[mi], b[np][2], b[np][3]);
        }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const int n = n0 + warp_n * 32 + ni * 8 + (lane & 3) * 2;
      if (n >= N) continue;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp_m * (GBM / 2) + mi * 16 + (lane >> 2) + half * 8;
        if (m >= end) continue;
        float v0 = acc[mi][ni][2 * half], v1 = acc[mi][ni][2 * half + 1];
        if (activation == kActClampedGlu) {         // (v0, v1) are a feature's gate and up sums
          C[(size_t)m * ldc + n / 2] = __float2bfloat16_rn(clamped_glu(v0, v1, limit));
          continue;
        }
        if (activation == kActSiluGlu) {
          C[(size_t)m * ldc + n / 2] = __float2bfloat16_rn(silu_glu(v0, v1, pair_scale ? pair_scale[order[m]] : 1.f));
          continue;
        }
        if (activation == kActReluSquare) {
          v0 = fmaxf(v0, 0.f);
          v1 = fmaxf(v1, 0.f);
          v0 *= v0;
          v1 *= v1;
        }
        *reinterpret_cast<__nv_bfloat162*>(C + (size_t)m * ldc + n) = __floats2bfloat162_rn(v0, v1);
      }
    }
}

// One block per token: out[n, c] = sum_k weights[n, k] * Y[place[n * top + k], c] (+ shared[n, c]), k ascending, float32.
// With `ids`, a choice whose id is first_identity or more stands for an identity expert: its row is x[n] instead.  With
// `shared_gate` the shared expert's output is multiplied by sigmoid(shared_gate[n * shared_gate_ld]).
template <typename T>
__global__ void expert_combine_kernel(const T* __restrict__ Y, int ldy, const int* __restrict__ place,
                                      const float* __restrict__ weights, int top, const T* __restrict__ shared,
                                      T* __restrict__ out, int width, const int* __restrict__ ids, int first_identity,
                                      const T* __restrict__ x, const float* __restrict__ shared_gate, int shared_gate_ld) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t n = blockIdx.x;
  const float share = shared_gate ? 1.f / (1.f + expf(-shared_gate[n * shared_gate_ld])) : 1.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const bool identity = ids && ids[n * top + k] >= first_identity;
      const float v = identity ? to_float(x[n * width + c]) : to_float(Y[(size_t)place[n * top + k] * ldy + c]);
      sum += weights ? weights[n * top + k] * v : v;       // (no weights: the experts' inputs carried them)
    }
    if (shared) sum += share * to_float(shared[n * width + c]);
    out[n * width + c] = from_float<T>(sum);
  }
}

// out[n, j] = clamped_glu(both[n, 2 j], both[n, 2 j + 1])
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ both, T* __restrict__ out, size_t total, float limit) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  out[i] = from_float<T>(clamped_glu(to_float(both[2 * i]), to_float(both[2 * i + 1]), limit));
}

template <typename T>
__global__ void relu_square_kernel(T* __restrict__ x, size_t total) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = fmaxf(to_float(x[i]), 0.f);
  x[i] = from_float<T>(v * v);
}

}  // namespace ms

using namespace ms;

#define MS_EXP_DISPATCH(dtype, ...)                              \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

namespace ms {

// Launches the logits kernel: logits[n, e] for the `experts` rows of `weight`.
static int launch_router_logits(const void* x, int dtype, const float* weight, const float* bias, int width, int experts,
                                float* logits, int n_tokens, cudaStream_t stream) {
  MS_REQUIRE(dtype == MS_F32 || dtype == MS_BF16, "router: unknown element type code %d", dtype);
  const size_t element = dtype == MS_F32 ? 4 : 2;
  MS_REQUIRE((size_t)width * element <= 48 * 1024, "router: a row of %d numbers does not fit the shared memory", width);
  int rt = 8;                              // tokens per block: as many rows as 32 KB hold, at most eight
  while (rt > 1 && (size_t)rt * width * element > 32 * 1024) rt >>= 1;
  const int token_tiles = (n_tokens + rt - 1) / rt;
  // few token tiles (decode steps): the experts are spread over blocks too, one per warp, so that every weight row has a warp of its own
  const int per_block = token_tiles >= 128 ? experts : 8;
  dim3 grid(token_tiles, (experts + per_block - 1) / per_block);
  const size_t smem = (size_t)rt * width * element;
#define MS_ROUTER_LOGITS(RT)                                                                                                \
  MS_EXP_DISPATCH(dtype, (ms::launch(router_logits_kernel<T, RT>, grid, 256, smem, stream, (const T*)x, weight, bias, width, \
                                     experts, per_block, logits, n_tokens)))
  if (rt == 8) { MS_ROUTER_LOGITS(8); } else if (rt == 4) { MS_ROUTER_LOGITS(4); } else if (rt == 2) { MS_ROUTER_LOGITS(2); }
  else { MS_ROUTER_LOGITS(1); }
#undef MS_ROUTER_LOGITS
  MS_CHECK_LAUNCH("router: logits");
  return 0;
}

}  // namespace ms

// x [n_tokens, width]; weight float32 [experts, width]; bias float32 [experts] or null; logits float32 [n_tokens, experts]
// (scratch, left holding the logits); ids int32 and weights float32 [n_tokens, top].
MS_EXPORT int ms_router_topk(const void* x, int dtype, const float* weight, const float* bias, int width, int experts,
                             int top, float* logits, int* ids, float* weights, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(experts > 0 && top > 0 && top <= experts, "router_topk: %d of %d experts", top, experts);
  if (launch_router_logits(x, dtype, weight, bias, width, experts, logits, n_tokens, stream)) return 1;
  const int warps = 4;
  const size_t select_smem = (size_t)warps * (experts + top) * sizeof(float);
  MS_REQUIRE(select_smem <= 48 * 1024, "router_topk: %d experts need %zu bytes of shared memory", experts, select_smem);
  ms::launch(router_select_kernel, (n_tokens + warps - 1) / warps, warps * 32, select_smem, stream, (const float*)logits, experts,
             top, ids, weights, n_tokens);
  MS_CHECK_LAUNCH("router_topk: selection");
  return 0;
}

// The router whose scores are the softmax over all outputs (sigmoid_scores: the sigmoid of each output).  weight float32 [rows, width] with rows >= total: the first
// `total` rows are the router's outputs, further rows ride along (their logits are left in `logits` for the caller);
// bias [rows] or null; correction float32 [total] or null; logits float32 [n_tokens, rows]; ids, weights [n_tokens, top].
MS_EXPORT int ms_router_choose(const void* x, int dtype, const float* weight, const float* bias, int width, int rows,
                               int total, int top, const float* correction, int group_count, int group_keep, float* logits,
                               int* ids, float* weights, int n_tokens, int sigmoid_scores, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(total > 0 && rows >= total, "router_choose: %d outputs in %d rows", total, rows);
  MS_REQUIRE(group_count > 0 && total % group_count == 0 && group_keep >= 1 && group_keep <= group_count,
             "router_choose: %d outputs in %d groups of which %d are kept", total, group_count, group_keep);
  MS_REQUIRE(top > 0 && top <= group_keep * (total / group_count), "router_choose: %d of %d outputs (%d of %d groups kept)", top,
             total, group_keep, group_count);
  if (launch_router_logits(x, dtype, weight, bias, width, rows, logits, n_tokens, stream)) return 1;
  const int warps = 4;
  const size_t smem = (size_t)warps * (2 * total + group_count) * sizeof(float);
  MS_REQUIRE(smem <= 48 * 1024, "router_choose: %d outputs need %zu bytes of shared memory", total, smem);
  ms::launch(router_choose_kernel, (n_tokens + warps - 1) / warps, warps * 32, smem, stream, (const float*)logits, rows, total, top,
             correction, group_count, group_keep, ids, weights, n_tokens, sigmoid_scores);
  MS_CHECK_LAUNCH("router_choose: selection");
  return 0;
}

// out[n, r] = x[n] . weight[r] + bias[r] in float32: the router's logits kernel for any float32 weight of few rows (the gate
// logits of a recurrence).  x [n_tokens, width] of type `dtype`; weight float32 [rows, width]; bias float32 [rows] or null.
MS_EXPORT int ms_small_linear_f32(const void* x, int dtype, const float* weight, const float* bias, int width, int rows,
                                  float* out, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || rows == 0) return 0;
  return launch_router_logits(x, dtype, weight, bias, width, rows, out, n_tokens, stream);
}

// ids [pairs] (each in 0 .. experts - 1); offsets [experts + 1]; order, place [pairs].
MS_EXPORT int ms_expert_route(const int* ids, int pairs, int experts, int* offsets, int* order, int* place,
                              cudaStream_t stream) {
  MS_REQUIRE(experts > 0 && experts <= 4096, "expert_route: %d experts outside 1..4096", experts);
  ms::launch(expert_route_kernel, 1, 1024, (size_t)2 * experts * sizeof(int), stream, ids, pairs, experts, offsets, order, place);
  MS_CHECK_LAUNCH("expert_route");
  return 0;
}

// A rows of K numbers (row stride lda); order null or [pairs]; W [experts, N, K]; C [pairs, ldc].  activation: 0 none,
// 1 squared ReLU, 2 the clamped gated one (the rows of W alternate gate, up; C then has N / 2 columns), 3 the silu-gated one
// (the same layout; pair_scale float32 [pairs] or null, indexed by order[i]: the factor on the expert's input).
MS_EXPORT int ms_expert_linear(const void* A, int dtype, int lda, const int* order, int top, const void* W, void* C, int ldc,
                               const int* offsets, int experts, int pairs, int N, int K, int activation, float limit,
                               const float* pair_scale, cudaStream_t stream) {
  if (pairs == 0 || N == 0 || experts == 0) return 0;
  MS_REQUIRE(K > 0 && top > 0, "expert_linear: inner size %d and choices %d must be positive", K, top);
  MS_REQUIRE(activation >= kActNone && activation <= kActSiluGlu && (activation < kActClampedGlu || N % 2 == 0),
             "expert_linear: activation %d with %d columns", activation, N);
  MS_REQUIRE(pair_scale == nullptr || (activation == kActSiluGlu && order != nullptr),
             "expert_linear: a scale per pair goes with the silu-gated activation and gathered rows");
  const int row_tiles = (pairs + EBM - 1) / EBM + experts;      // every segment may end in a partial tile
  MS_REQUIRE(row_tiles <= 65535, "expert_linear: %d rows in one launch is too many", pairs);
  if (dtype == MS_BF16 && K % 8 == 0 && N % 8 == 0 && lda % 8 == 0 && (ldc % 2 == 0 || activation >= kActClampedGlu)) {
    // long segments (256 rows an expert on average, or more): tiles of 128 rows; else tiles of 64
    const bool tall = pairs >= 256 * experts;
    const int rows = tall ? 128 : 64, stages = tall ? 3 : 4;
    dim3 mma_grid((N + GBN - 1) / GBN, (pairs + rows - 1) / rows + experts);
    const size_t smem = sizeof(__nv_bfloat16) * stages * (rows + GBN) * (GBK + 8);
    auto kernel = tall ? expert_linear_mma_kernel<128, 3> : expert_linear_mma_kernel<64, 4>;
    static bool allowed[2] = {false, false};
    if (!allowed[tall]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) MS_FAIL("expert_linear: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      allowed[tall] = true;
    }
    ms::launch(kernel, mma_grid, 256, smem, stream, (const __nv_bfloat16*)A, lda, order, top,
               (const __nv_bfloat16*)W, (__nv_bfloat16*)C, ldc, offsets, experts, N, K, activation, limit, pair_scale);
    MS_CHECK_LAUNCH("expert_linear (tensor cores)");
    return 0;
  }
  dim3 grid((N + EBN - 1) / EBN, row_tiles);
  MS_EXP_DISPATCH(dtype, (ms::launch(expert_linear_kernel<T>, grid, 256, 0, stream, (const T*)A, lda, order, top, (const T*)W,
                                     (T*)C, ldc, offsets, experts, N, K, activation, limit, pair_scale)));
  MS_CHECK_LAUNCH("expert_linear");
  return 0;
}

// Y [pairs, ldy]; place [n_tokens * top]; weights float32 [n_tokens, top]; shared [n_tokens, width] or null; out [n_tokens, width].
// ids [n_tokens * top] or null: a choice with ids >= first_identity adds weight * x[token] (x [n_tokens, width]) instead of a
// row of Y.  shared_gate float32 or null: the logit at shared_gate[token * shared_gate_ld] gates the shared expert's output.
MS_EXPORT int ms_expert_combine(const void* Y, int dtype, int ldy, const int* place, const float* weights, int top,
                                const void* shared, void* out, int width, int n_tokens, const int* ids, int first_identity,
                                const void* x, const float* shared_gate, int shared_gate_ld, cudaStream_t stream) {
  if (n_tokens == 0 || width == 0) return 0;
  MS_REQUIRE(ids == nullptr || x != nullptr, "expert_combine: identity experts need the tokens' rows");
  MS_EXP_DISPATCH(dtype, (ms::launch(expert_combine_kernel<T>, n_tokens, 256, 0, stream, (const T*)Y, ldy, place, weights, top,
                                     (const T*)shared, (T*)out, width, ids, first_identity, (const T*)x, shared_gate,
                                     shared_gate_ld)));
  MS_CHECK_LAUNCH("expert_combine");
  return 0;
}

namespace ms {
// Sixteen bytes a thread (four float32 or eight bfloat16 numbers); `pieces` such pieces, the array on a 16-byte boundary.
template <typename T>
__global__ void relu_square_wide_kernel(T* __restrict__ x, size_t pieces) {
  grid_dependency_wait();
  grid_dependency_launch();
  constexpr int PER = 16 / sizeof(T);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (size_t)gridDim.x * blockDim.x) {
    uint4 raw = reinterpret_cast<uint4*>(x)[i];
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const float f = fmaxf(to_float(v[e]), 0.f);
      v[e] = from_float<T>(f * f);
    }
    reinterpret_cast<uint4*>(x)[i] = raw;
  }
}
}  // namespace ms

MS_EXPORT int ms_relu_square(void* x, int dtype, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  const long long per = dtype == MS_F32 ? 4 : 8;
  if (total % per == 0 && reinterpret_cast<size_t>(x) % 16 == 0) {
    const long long pieces = total / per;
    long long wide_blocks = (pieces + 255) / 256;
    if (wide_blocks > 148 * 16) wide_blocks = 148 * 16;
    MS_EXP_DISPATCH(dtype, (ms::launch(relu_square_wide_kernel<T>, (unsigned)wide_blocks, 256, 0, stream, (T*)x, (size_t)pieces)));
    MS_CHECK_LAUNCH("relu_square");
    return 0;
  }
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "relu_square: %lld elements in one launch is too many", total);
  MS_EXP_DISPATCH(dtype, (ms::launch(relu_square_kernel<T>, (unsigned)blocks, 256, 0, stream, (T*)x, (size_t)total)));
  MS_CHECK_LAUNCH("relu_square");
  return 0;
}

namespace ms {
// Eight results per thread: two sixteen-byte loads of (gate, up) pairs, one store (bfloat16; total % 8 == 0).
__global__ void clamped_glu_vec_kernel(const __nv_bfloat16* __restrict__ both, __nv_bfloat16* __restrict__ out, size_t groups,
                                       float limit) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  const uint4 lo = *reinterpret_cast<const uint4*>(both + 16 * i), hi = *reinterpret_cast<const uint4*>(both + 16 * i + 8);
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&lo);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&hi);
  uint4 packed;
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float2 p0 = __bfloat1622float2(a[2 * e]), p1 = __bfloat1622float2(a[2 * e + 1]);
    const float2 q0 = __bfloat1622float2(b[2 * e]), q1 = __bfloat1622float2(b[2 * e + 1]);
    o[e] = __floats2bfloat162_rn(clamped_glu(p0.x, p0.y, limit), clamped_glu(p1.x, p1.y, limit));
    o[2 + e] = __floats2bfloat162_rn(clamped_glu(q0.x, q0.y, limit), clamped_glu(q1.x, q1.y, limit));
  }
  *reinterpret_cast<uint4*>(out + 8 * i) = packed;
}
}  // namespace ms

// both [n_tokens, 2 * inter] with alternating (gate, up) columns; out [n_tokens, inter].
MS_EXPORT int ms_clamped_glu(const void* both, int dtype, void* out, int n_tokens, int inter, float limit, cudaStream_t stream) {
  const long long total = (long long)n_tokens * inter;
  if (total <= 0) return 0;
  if (dtype == MS_BF16 && total % 8 == 0) {
    const long long groups = total / 8;
    ms::launch(clamped_glu_vec_kernel, (unsigned)((groups + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)both, (__nv_bfloat16*)out,
               (size_t)groups, limit);
    MS_CHECK_LAUNCH("clamped_glu");
    return 0;
  }
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "clamped_glu: %lld elements in one launch is too many", total);
  MS_EXP_DISPATCH(dtype, (ms::launch(clamped_glu_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)both, (T*)out, (size_t)total, limit)));
  MS_CHECK_LAUNCH("clamped_glu");
  return 0;
}
