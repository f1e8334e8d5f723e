// More memory-bound kernels between the matrix products, for blocks and mixers whose forms elementwise.cu does not cover:
//
//   ms_postnorm_add_rmsnorm   a sublayer's output is RMS-normed with a weight of its own, added (times a constant) to the
//                             float32 residual stream, and the stream is RMS-normed for the next sublayer, or handed on as
//                             it is where the next sublayer reads the stream itself: one kernel, one pass over the row
//   ms_silu_mul_bias, ms_add_bias, ms_scaled_sum   a gated activation and an output with biases; a weighted sum of two outputs
//   ms_qkv_prepare            per-head norm, partial half-split rotation and paged append for a projection whose columns are
//                             laid out freely: query heads of d numbers, key heads of d, value heads of dv (another size),
//                             or queries alone (a layer that reads another layer's keys and values)
//
// All arithmetic is float32; storage is float32 or bfloat16.
#include "common.cuh"
#include "elementwise_vec.cuh"

namespace ms {

// For output row k (source row r = rows ? rows[k] : k):
//   a = post_scale * post_weight * delta[r] / sqrt(mean(delta[r]^2) + post_eps)      (delta null: a = 0;
//       post_eps < 0: no division, a = post_scale * post_weight * delta[r], a scale per channel)
//   x = residual[r] + a            (float32; written back to residual unless rows are gathered)
//   out[k] = weight * x / sqrt(mean(x^2) + eps)     rounded once to T      (weight null: out[k] = x)
// The row (width <= blockDim.x * kPostNormPerThread) stays in registers between the passes.
constexpr int kPostNormPerThread = 16;

template <typename T>
__global__ void postnorm_add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                            const void* __restrict__ post_weight, int post_weight_dtype, float post_eps,
                                            float post_scale, const void* __restrict__ weight, int weight_dtype, float eps,
                                            const int* __restrict__ rows, T* __restrict__ out, int hidden) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t k = blockIdx.x;
  const size_t r = rows ? (size_t)rows[k] : k;
  float* res = residual + r * hidden;
  const T* del = delta + r * hidden;
  float v[kPostNormPerThread];
  float sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < kPostNormPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = (delta && c < hidden) ? to_float(del[c]) : 0.f;
    sum_sq += v[i] * v[i];
  }
  float inv_delta = 0.f;
  if (delta) inv_delta = post_eps < 0.f ? post_scale : post_scale / sqrtf(block_sum(sum_sq, scratch) / (float)hidden + post_eps);
  sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < kPostNormPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < hidden) {
      if (delta) {
        v[i] = res[c] + load_as_float(post_weight, post_weight_dtype, c) * (v[i] * inv_delta);
        if (rows == nullptr) res[c] = v[i];
      } else {
        v[i] = res[c];
      }
      sum_sq += v[i] * v[i];
    }
  }
  float inv = 1.f;
  if (weight) inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)hidden + eps);
  T* dst = out + k * hidden;
#pragma unroll
  for (int i = 0; i < kPostNormPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < hidden) dst[c] = from_float<T>(weight ? load_as_float(weight, weight_dtype, c) * (v[i] * inv) : v[i]);
  }
}

// The same with sixteen-byte loads and stores: each thread keeps up to CHUNKS groups of eight elements in registers, so
// every row is read once.  Requires hidden % 8 == 0 and hidden <= 8 * blockDim.x * CHUNKS.
template <typename T, int CHUNKS>
__global__ void postnorm_add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                                const void* __restrict__ post_weight, int post_weight_dtype, float post_eps,
                                                float post_scale, const void* __restrict__ weight, int weight_dtype, float eps,
                                                const int* __restrict__ rows, T* __restrict__ out, int hidden) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t k = blockIdx.x;
  const size_t r = rows ? (size_t)rows[k] : k;
  float* res = residual + r * hidden;
  const T* del = delta + r * hidden;
  Vec8 v[CHUNKS], x[CHUNKS];
  float sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      if (delta) v[i] = load8(del + c);
      x[i] = load8(res + c);                               // (on its way while the first sum is formed)
      if (delta) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sum_sq += v[i].v[e] * v[i].v[e];
      }
    }
  }
  float inv_delta = 0.f;
  if (delta) inv_delta = post_eps < 0.f ? post_scale : post_scale / sqrtf(block_sum(sum_sq, scratch) / (float)hidden + post_eps);
  sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      if (delta) {
        const Vec8 w = load8_any(post_weight, post_weight_dtype, c);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[i].v[e] += w.v[e] * (v[i].v[e] * inv_delta);
        if (rows == nullptr) store8(res + c, x[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sum_sq += x[i].v[e] * x[i].v[e];
    }
  }
  float inv = 1.f;
  if (weight) inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)hidden + eps);
  T* dst = out + k * hidden;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      Vec8 y = x[i];
      if (weight) {
        const Vec8 w = load8_any(weight, weight_dtype, c);
#pragma unroll
        for (int e = 0; e < 8; ++e) y.v[e] = w.v[e] * (x[i].v[e] * inv);
      }
      store8(dst + c, y);
    }
  }
}

// One warp per (token, head) of proj[n, ld]: query head h at columns q_col + h d, key head g at k_col + g d, value head
// g at v_col + g dv (k_col < 0: the projection holds no keys and values).
//   q heads: optional RMS norm over d (weight float32), rotation, written to q_out[n, h, :]
//   k heads: the same with their own weight, written to the key pool [page, kv_head, page_size, d] at the token's slot
//   v heads: copied to the value pool [page, kv_head, page_size, dv]
// Rotation: the first rotary_dim entries of a head, entry i paired with entry i + rotary_dim / 2 (interleaved: entry 2i with
// entry 2i + 1); the pair (u, v)
// becomes (u cos - v sin, v cos + u sin) with (cos, sin) = cos_sin[n, i].  A negative slot skips the writes.
// bias (null: none): float32 [ld], the projection's bias column by column, added in float32 to every head as it is read.
// value_heads: the projection and the value pool [page, value_heads, page_size, dv] hold that many value heads (a divisor of
// n_kv: key heads that share values).
template <typename T>
__global__ void qkv_prepare_kernel(const T* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int n_q, int n_kv,
                                   int d, int dv, const int* __restrict__ slots, const float* __restrict__ q_weight,
                                   const float* __restrict__ k_weight, float eps, const float2* __restrict__ cos_sin,
                                   int rotary_dim, T* __restrict__ k_pool, T* __restrict__ v_pool, int page_size,
                                   T* __restrict__ q_out, int n_tokens, int interleaved, const float* __restrict__ bias,
                                   int value_heads) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float prepare_smem[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = n_q + (k_col >= 0 ? n_kv + value_heads : 0);
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)n_tokens * heads) return;
  const int n = (int)(item / heads), head = (int)(item % heads);
  const T* row = proj + (size_t)n * ld;
  float* x = prepare_smem + warp * d;

  const T* src;
  T* dst;
  const float* weight;
  if (head < n_q) {
    src = row + q_col + head * d;
    dst = q_out + ((size_t)n * n_q + head) * d;
    weight = q_weight;
  } else {
    const int slot = slots[n];
    if (slot < 0) return;
    const int page = slot / page_size, offset = slot % page_size;
    if (head >= n_q + n_kv) {
      const int g = head - n_q - n_kv;
      src = row + v_col + g * dv;                        // (value_heads of them: key head g reads value head g % value_heads)
      dst = v_pool + (((size_t)page * value_heads + g) * page_size + offset) * dv;
      if (bias) {
        const float* b = bias + v_col + g * dv;
        for (int c = lane; c < dv; c += 32) dst[c] = from_float<T>(to_float(src[c]) + b[c]);
      } else {
        for (int c = lane; c < dv; c += 32) dst[c] = src[c];
      }
      return;
    }
    const int g = head - n_q;
    src = row + k_col + g * d;
    dst = k_pool + (((size_t)page * n_kv + g) * page_size + offset) * d;
    weight = k_weight;
  }
  float sum_sq = 0.f;
  const float* head_bias = bias ? bias + (src - row) : nullptr;      // (the projection's bias lies by its columns)
  for (int c = lane; c < d; c += 32) {
    const float v = to_float(src[c]) + (head_bias ? head_bias[c] : 0.f);
    x[c] = v;
    sum_sq += v * v;
  }
  float inv = 1.f;
  if (weight) inv = 1.0f / sqrtf(warp_sum(sum_sq) / (float)d + eps);
  __syncwarp();
  const int half = rotary_dim >> 1;
  const float2* table = cos_sin ? cos_sin + (size_t)n * half : nullptr;
  for (int c = lane; c < d; c += 32) {
    float v = x[c] * inv;
    if (weight) v *= weight[c];
    if (table && c < rotary_dim) {
      // the pair's first entry is c (partner behind it) or its second; half-split: (j, j + half), interleaved: (2j, 2j + 1)
      const bool first = interleaved ? (c & 1) == 0 : c < half;
      const int j = interleaved ? c >> 1 : (c < half ? c : c - half);
      const int partner = interleaved ? c ^ 1 : (c < half ? c + half : c - half);
      float other = x[partner] * inv;
      if (weight) other *= weight[partner];
      const float2 cs = table[j];
      v = first ? v * cs.x - other * cs.y : v * cs.x + other * cs.y;
    }
    dst[c] = from_float<T>(v);
  }
}

}  // namespace ms

using namespace ms;

#define MS_EG_DISPATCH(dtype, ...)                               \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// residual float32 [rows, hidden]; delta [rows, hidden] and out [n_out, hidden] of type `dtype`; the two weights [hidden]
// in their own types; rows int32 [n_out] or null (then n_out rows in place, and the residual receives the sum).
// delta null: nothing is added (post_weight is not read); weight null: out is the stream itself, rounded once.
MS_EXPORT int ms_postnorm_add_rmsnorm(float* residual, const void* delta, int dtype, const void* post_weight,
                                      int post_weight_dtype, float post_eps, float post_scale, const void* weight,
                                      int weight_dtype, float eps, const int* rows, void* out, int n_out, int hidden,
                                      cudaStream_t stream) {
  if (n_out == 0) return 0;
  MS_REQUIRE(hidden > 0 && hidden <= 1024 * kPostNormPerThread, "postnorm_add_rmsnorm: width %d outside 1..%d", hidden,
             1024 * kPostNormPerThread);
  if (hidden % 8 == 0 && hidden <= 8192) {
    const int groups = hidden / 8;
    const int vec_threads = groups >= 256 ? 256 : ((groups + 31) / 32) * 32;
    const int chunks = (groups + vec_threads - 1) / vec_threads;
#define MS_POSTNORM_VEC(C)                                                                                                   \
  MS_EG_DISPATCH(dtype, (ms::launch(postnorm_add_rmsnorm_vec_kernel<T, C>, n_out, vec_threads, 0, stream, residual,          \
                                    (const T*)delta, post_weight, post_weight_dtype, post_eps, post_scale, weight,           \
                                    weight_dtype, eps,                                                                       \
                                    rows, (T*)out, hidden)))
    if (chunks == 1) { MS_POSTNORM_VEC(1); } else if (chunks == 2) { MS_POSTNORM_VEC(2); } else { MS_POSTNORM_VEC(4); }
#undef MS_POSTNORM_VEC
    MS_CHECK_LAUNCH("postnorm_add_rmsnorm");
    return 0;
  }
  int threads = ((hidden + kPostNormPerThread - 1) / kPostNormPerThread + 31) / 32 * 32;
  if (threads < 128 && hidden >= 128) threads = 128;
  if (hidden >= 2048 && threads < 256) threads = 256;
  MS_EG_DISPATCH(dtype, (ms::launch(postnorm_add_rmsnorm_kernel<T>, n_out, threads, 0, stream, residual, (const T*)delta,
                                    post_weight, post_weight_dtype, post_eps, post_scale, weight, weight_dtype, eps, rows, (T*)out,
                                    hidden)));
  MS_CHECK_LAUNCH("postnorm_add_rmsnorm");
  return 0;
}

MS_EXPORT int ms_qkv_prepare(const void* proj, int dtype, int ld, int q_col, int k_col, int v_col, int n_q, int n_kv, int d,
                             int dv, const int* slots, const float* q_weight, const float* k_weight, float eps,
                             const float* cos_sin, int rotary_dim, void* k_pool, void* v_pool, int page_size, void* q_out,
                             int n_tokens, int interleaved, const float* bias, int value_heads, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(d > 0 && d <= 1024 && dv > 0, "qkv_prepare: head sizes %d and %d", d, dv);
  MS_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
             "qkv_prepare: rotary size %d must be even and at most the head size %d", rotary_dim, d);
  MS_REQUIRE(page_size > 0, "qkv_prepare: page size must be positive, got %d", page_size);
  MS_REQUIRE(k_col < 0 || (v_col >= 0 && slots && k_pool && v_pool), "qkv_prepare: keys and values need their columns, slots and pools");
  MS_REQUIRE(k_col < 0 || (value_heads >= 1 && n_kv % value_heads == 0), "qkv_prepare: %d value heads for %d key heads", value_heads, n_kv);
  const int warps = 4;
  const long long items = (long long)n_tokens * (n_q + (k_col >= 0 ? n_kv + (value_heads > 0 ? value_heads : n_kv) : 0));
  const long long blocks = (items + warps - 1) / warps;
  MS_REQUIRE(blocks < 2147483647LL, "qkv_prepare: %lld heads in one launch is too many", items);
  const size_t smem = (size_t)warps * d * sizeof(float);
  MS_EG_DISPATCH(dtype, (ms::launch(qkv_prepare_kernel<T>, (unsigned)blocks, warps * 32, smem, stream, (const T*)proj, ld, q_col,
                                    k_col, v_col, n_q, n_kv, d, dv, slots, q_weight, k_weight, eps, (const float2*)cos_sin,
                                    rotary_dim, (T*)k_pool, (T*)v_pool, page_size, (T*)q_out, n_tokens, interleaved, bias, value_heads > 0 ? value_heads : n_kv)));
  MS_CHECK_LAUNCH("qkv_prepare");
  return 0;
}

namespace ms {

// out[n, c] = silu(gate_up[n, c] + bias[c]) * (gate_up[n, I + c] + bias[I + c])
template <typename T>
__global__ void silu_mul_bias_kernel(const T* __restrict__ gate_up, const float* __restrict__ bias, T* __restrict__ out,
                                     size_t total, int inter) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t n = i / inter;
  const int c = (int)(i % inter);
  const float g = to_float(gate_up[n * 2 * inter + c]) + bias[c];
  const float u = to_float(gate_up[n * 2 * inter + inter + c]) + bias[inter + c];
  out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// The same, four numbers a thread in 16-byte (8-byte for bfloat16) accesses, where `inter` is a multiple of four and
// the arrays lie on such boundaries.
template <typename T> struct alignas(sizeof(T) * 4) Quad { T v[4]; };

template <typename T>
__global__ void silu_mul_bias_quad_kernel(const T* __restrict__ gate_up, const float* __restrict__ bias, T* __restrict__ out,
                                          size_t quads, int inter) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= quads) return;
  const int per_row = inter >> 2;
  const size_t n = i / per_row;
  const int c = (int)(i % per_row) * 4;
  const Quad<T> gate = *reinterpret_cast<const Quad<T>*>(gate_up + n * 2 * inter + c);
  const Quad<T> up = *reinterpret_cast<const Quad<T>*>(gate_up + n * 2 * inter + inter + c);
  const float4 gate_bias = *reinterpret_cast<const float4*>(bias + c), up_bias = *reinterpret_cast<const float4*>(bias + inter + c);
  const float gb[4] = {gate_bias.x, gate_bias.y, gate_bias.z, gate_bias.w}, ub[4] = {up_bias.x, up_bias.y, up_bias.z, up_bias.w};
  Quad<T> result;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float g = to_float(gate.v[e]) + gb[e];
    const float u = to_float(up.v[e]) + ub[e];
    result.v[e] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
  *reinterpret_cast<Quad<T>*>(out + i * 4) = result;
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, size_t total, int width) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  x[i] = from_float<T>(to_float(x[i]) + bias[i % width]);
}

template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float a_scale, const T* __restrict__ b, float b_scale,
                                  T* __restrict__ out, size_t total) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  out[i] = from_float<T>(a_scale * to_float(a[i]) + b_scale * to_float(b[i]));
}

// out[n] = a_scale * a_weight * a[n] / rms(a[n]) + b_scale * b_weight * b[n] / rms(b[n]): two outputs, each normed over the
// row with a weight of its own, summed.  One block a row.
template <typename T>
__global__ void normed_sum_kernel(const T* __restrict__ a, const float* __restrict__ a_weight, float a_scale,
                                  const T* __restrict__ b, const float* __restrict__ b_weight, float b_scale, float eps,
                                  T* __restrict__ out, int hidden) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const T* ar = a + (size_t)blockIdx.x * hidden;
  const T* br = b + (size_t)blockIdx.x * hidden;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float x = to_float(ar[c]), y = to_float(br[c]);
    sa += x * x;
    sb += y * y;
  }
  const float inv_a = a_scale / sqrtf(block_sum(sa, scratch) / (float)hidden + eps);
  const float inv_b = b_scale / sqrtf(block_sum(sb, scratch) / (float)hidden + eps);
  T* dst = out + (size_t)blockIdx.x * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    dst[c] = from_float<T>(a_weight[c] * (to_float(ar[c]) * inv_a) + b_weight[c] * (to_float(br[c]) * inv_b));
}

// out[n, c] = x[n, c] * sigmoid(gate[n, gate_col + c]): a gate per entry on the concatenated heads.
template <typename T>
__global__ void sigmoid_gate_mul_kernel(const T* __restrict__ x, const T* __restrict__ gate, int gate_ld, int gate_col,
                                        T* __restrict__ out, size_t total, int width) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float g = to_float(gate[(i / width) * gate_ld + gate_col + i % width]);
  out[i] = from_float<T>(to_float(x[i]) / (1.f + expf(-g)));
}

// One warp per (token, head): o = first - lambda second with first = a[n, head], second = a[n, heads + head] (the outputs of
// two score maps over the same values), o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate[n, gate_col + head dv + c]).
// `wide`: dv is a multiple of four, at most 512, and every row lies on a boundary of four numbers: a lane keeps its pieces of
// four in registers between the sum and the output.
template <typename T>
__global__ void differential_combine_kernel(const T* __restrict__ a, int heads, int dv, float lambda, float eps,
                                            float out_scale, const T* __restrict__ gate, int gate_ld, int gate_col,
                                            T* __restrict__ out, long long items, int wide) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= items) return;
  const size_t n = (size_t)(item / heads);
  const int head = (int)(item % heads);
  const T* first = a + (n * 2 * heads + head) * dv;
  const T* second = a + (n * 2 * heads + heads + head) * dv;
  const T* g = gate ? gate + n * gate_ld + gate_col + (size_t)head * dv : nullptr;
  T* dst = out + (n * heads + head) * dv;
  if (wide) {
    constexpr int PIECES = 4;
    const int pieces = dv >> 2;
    float o[PIECES][4];
    Quad<T> gates[PIECES];
    float sum_sq = 0.f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
      const int at = lane + 32 * j;
      if (at < pieces) {
        const Quad<T> x = reinterpret_cast<const Quad<T>*>(first)[at], y = reinterpret_cast<const Quad<T>*>(second)[at];
        if (g) gates[j] = reinterpret_cast<const Quad<T>*>(g)[at];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[j][e] = to_float(x.v[e]) - lambda * to_float(y.v[e]);
          sum_sq += o[j][e] * o[j][e];
        }
      }
    }
    const float inv = out_scale / sqrtf(warp_sum(sum_sq) / (float)dv + eps);
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
      const int at = lane + 32 * j;
      if (at < pieces) {
        Quad<T> result;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = o[j][e] * inv;
          if (g) v /= 1.f + expf(-to_float(gates[j].v[e]));
          result.v[e] = from_float<T>(v);
        }
        reinterpret_cast<Quad<T>*>(dst)[at] = result;
      }
    }
    return;
  }
  float sum_sq = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float o = to_float(first[c]) - lambda * to_float(second[c]);
    sum_sq += o * o;
  }
  const float inv = out_scale / sqrtf(warp_sum(sum_sq) / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    float o = (to_float(first[c]) - lambda * to_float(second[c])) * inv;
    if (g) o /= 1.f + expf(-to_float(g[c]));
    dst[c] = from_float<T>(o);
  }
}

}  // namespace ms

// a, b, out [rows, hidden] of type `dtype`; the weights float32 [hidden].
MS_EXPORT int ms_normed_sum(const void* a, const float* a_weight, float a_scale, const void* b, const float* b_weight,
                            float b_scale, float eps, void* out, int dtype, int rows, int hidden, cudaStream_t stream) {
  if (rows == 0 || hidden == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  MS_EG_DISPATCH(dtype, (ms::launch(normed_sum_kernel<T>, rows, threads, 0, stream, (const T*)a, a_weight, a_scale, (const T*)b,
                                    b_weight, b_scale, eps, (T*)out, hidden)));
  MS_CHECK_LAUNCH("normed_sum");
  return 0;
}

// x, out [rows, width]; gate rows of gate_ld numbers, the logits from column gate_col; all of type `dtype` (out may be x).
MS_EXPORT int ms_sigmoid_gate_mul(const void* x, const void* gate, int gate_ld, int gate_col, void* out, int dtype, int rows,
                                  int width, cudaStream_t stream) {
  const long long total = (long long)rows * width;
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "sigmoid_gate_mul: %lld elements in one launch is too many", total);
  MS_EG_DISPATCH(dtype, (ms::launch(sigmoid_gate_mul_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)x, (const T*)gate, gate_ld,
                                    gate_col, (T*)out, (size_t)total, width)));
  MS_CHECK_LAUNCH("sigmoid_gate_mul");
  return 0;
}

// a [tokens, 2 heads, dv] (the first map's heads, then the second's); gate rows of gate_ld numbers (null: no gate); out
// [tokens, heads, dv]; all of type `dtype`.
MS_EXPORT int ms_differential_combine(const void* a, int heads, int dv, float lambda, float eps, float out_scale,
                                      const void* gate, int gate_ld, int gate_col, void* out, int dtype, int n_tokens,
                                      cudaStream_t stream) {
  const long long items = (long long)n_tokens * heads;
  if (items == 0 || dv == 0) return 0;
  const long long blocks = (items + 3) / 4;
  MS_REQUIRE(blocks < 2147483647LL, "differential_combine: %lld heads in one launch is too many", items);
  const size_t four = dtype == MS_F32 ? 16 : 8;
  const int wide = dv % 4 == 0 && dv <= 512 && reinterpret_cast<size_t>(a) % four == 0 && reinterpret_cast<size_t>(out) % four == 0 &&
                   (gate == nullptr || (reinterpret_cast<size_t>(gate) % four == 0 && gate_ld % 4 == 0 && gate_col % 4 == 0));
  MS_EG_DISPATCH(dtype, (ms::launch(differential_combine_kernel<T>, (unsigned)blocks, 128, 0, stream, (const T*)a, heads, dv, lambda,
                                    eps, out_scale, (const T*)gate, gate_ld, gate_col, (T*)out, items, wide)));
  MS_CHECK_LAUNCH("differential_combine");
  return 0;
}

// gate_up [n_tokens, 2 inter] (gate columns, then up columns); bias float32 [2 inter]; out [n_tokens, inter].
MS_EXPORT int ms_silu_mul_bias(const void* gate_up, int dtype, const float* bias, void* out, int n_tokens, int inter,
                               cudaStream_t stream) {
  const long long total = (long long)n_tokens * inter;
  if (total == 0) return 0;
  const size_t four = dtype == MS_F32 ? 16 : 8;
  if (inter % 4 == 0 && reinterpret_cast<size_t>(gate_up) % four == 0 && reinterpret_cast<size_t>(out) % four == 0 &&
      reinterpret_cast<size_t>(bias) % 16 == 0) {
    const long long quads = total / 4, quad_blocks = (quads + 255) / 256;
    MS_REQUIRE(quad_blocks < 2147483647LL, "silu_mul_bias: %lld elements in one launch is too many", total);
    MS_EG_DISPATCH(dtype, (ms::launch(silu_mul_bias_quad_kernel<T>, (unsigned)quad_blocks, 256, 0, stream, (const T*)gate_up, bias,
                                      (T*)out, (size_t)quads, inter)));
    MS_CHECK_LAUNCH("silu_mul_bias");
    return 0;
  }
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "silu_mul_bias: %lld elements in one launch is too many", total);
  MS_EG_DISPATCH(dtype, (ms::launch(silu_mul_bias_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)gate_up, bias, (T*)out,
                                    (size_t)total, inter)));
  MS_CHECK_LAUNCH("silu_mul_bias");
  return 0;
}

// x [rows, width] in place; bias float32 [width].
MS_EXPORT int ms_add_bias(void* x, int dtype, const float* bias, int rows, int width, cudaStream_t stream) {
  const long long total = (long long)rows * width;
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "add_bias: %lld elements in one launch is too many", total);
  MS_EG_DISPATCH(dtype, (ms::launch(add_bias_kernel<T>, (unsigned)blocks, 256, 0, stream, (T*)x, bias, (size_t)total, width)));
  MS_CHECK_LAUNCH("add_bias");
  return 0;
}

// out = a_scale * a + b_scale * b over `total` elements (out may be a or b).
MS_EXPORT int ms_scaled_sum(const void* a, float a_scale, const void* b, float b_scale, void* out, int dtype, long long total,
                            cudaStream_t stream) {
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "scaled_sum: %lld elements in one launch is too many", total);
  MS_EG_DISPATCH(dtype, (ms::launch(scaled_sum_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)a, a_scale, (const T*)b,
                                    b_scale, (T*)out, (size_t)total)));
  MS_CHECK_LAUNCH("scaled_sum");
  return 0;
}
