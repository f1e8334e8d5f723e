// Kernels that look one token back along a sequence, across the steps that a request is cut into: what the last token of a
// portion leaves is kept in the request's state slot and read by the first token of its next portion.
//
//   ms_token_shift       out[t] = x[t] + (x[t - 1] - x[t]) * shift per channel; x[-1] of a sequence is zero
//   ms_pair_embedding    residual[t] += table[(token[t - 1] * mul_prev + token[t] * mul_cur) mod buckets]; the first token of a
//                        sequence takes row `buckets`
//
// The block that handles a request's first token of the step reads the slot and then writes what the request's last token of
// the step leaves there; no other block touches the slot, and the inputs are not written, so the order of blocks is free.
// (The padding rows of a captured decode step all name the scratch slot and race for it; no request ever reads that slot.)
#include "common.cuh"
#include "elementwise_vec.cuh"

namespace ms {

// grid (tokens); x, out [tokens, hidden]; state: float32 [hidden] at state_offset of the slot's row (zero at admission).
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ x, const float* __restrict__ shift, float* __restrict__ states,
                                   long long state_stride, int state_offset, const int* __restrict__ state_slots,
                                   const int* __restrict__ query_start, const int* __restrict__ request_of_token,
                                   T* __restrict__ out, int hidden) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t t = blockIdx.x;
  const int request = request_of_token[t];
  const int first = query_start[request], last = query_start[request + 1] - 1;
  const T* row = x + t * hidden;
  T* dst = out + t * hidden;
  if ((int)t != first) {
    const T* before = row - hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float h = to_float(row[c]);
      dst[c] = from_float<T>(h + (to_float(before[c]) - h) * shift[c]);
    }
    return;
  }
  float* kept = states + (long long)state_slots[request] * state_stride + state_offset;
  const T* leaves = x + (size_t)last * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float h = to_float(row[c]);
    const float before = kept[c];
    kept[c] = to_float(leaves[c]);
    dst[c] = from_float<T>(h + (before - h) * shift[c]);
  }
}

// The same in pieces of eight numbers (hidden a multiple of eight, rows on 16-byte boundaries): every access is sixteen bytes
// (thirty-two for float32).
template <typename T>
__global__ void token_shift_wide_kernel(const T* __restrict__ x, const float* __restrict__ shift, float* __restrict__ states,
                                        long long state_stride, int state_offset, const int* __restrict__ state_slots,
                                        const int* __restrict__ query_start, const int* __restrict__ request_of_token,
                                        T* __restrict__ out, int hidden) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t t = blockIdx.x;
  const int request = request_of_token[t];
  const int first = query_start[request], last = query_start[request + 1] - 1;
  const T* row = x + t * hidden;
  T* dst = out + t * hidden;
  const bool from_state = (int)t == first;
  float* kept = states + (long long)state_slots[request] * state_stride + state_offset;
  const T* leaves = x + (size_t)last * hidden;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    const Vec8 h = load8(row + c), s = load8(shift + c);
    Vec8 before;
    if (from_state) {
      before = load8(kept + c);
      store8(kept + c, load8(leaves + c));
    } else {
      before = load8(row - hidden + c);
    }
    Vec8 result;
#pragma unroll
    for (int e = 0; e < 8; ++e) result.v[e] = h.v[e] + (before.v[e] - h.v[e]) * s.v[e];
    store8(dst + c, result);
  }
}

// grid (tokens); the slot's state is one int32: the request's last token + 1 (0 at admission: no token yet).
template <typename T>
__global__ void pair_embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table, int buckets,
                                      long long mul_prev, long long mul_cur, int* __restrict__ states, long long state_stride,
                                      int state_offset, const int* __restrict__ state_slots,
                                      const int* __restrict__ query_start, const int* __restrict__ request_of_token,
                                      float* __restrict__ residual, int hidden) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ int before_s;
  const size_t t = blockIdx.x;
  const int request = request_of_token[t];
  const int first = query_start[request], last = query_start[request + 1] - 1;
  if (threadIdx.x == 0) {
    if ((int)t != first) {
      before_s = tokens[t - 1];
    } else {
      int* kept = states + (long long)state_slots[request] * state_stride + state_offset;
      before_s = *kept - 1;
      *kept = tokens[last] + 1;
    }
  }
  __syncthreads();
  const long long before = before_s;
  const long long row = before < 0 ? (long long)buckets : (before * mul_prev + (long long)tokens[t] * mul_cur) % buckets;
  const T* src = table + (size_t)row * hidden;
  float* dst = residual + t * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] += to_float(src[c]);
}

}  // namespace ms

using namespace ms;

#define MS_SEQ_DISPATCH(dtype, ...)                              \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// x, out [n_tokens, hidden] of type `dtype` (out is not x); shift float32 [hidden]; states float32 rows of state_stride numbers.
MS_EXPORT int ms_token_shift(const void* x, int dtype, const float* shift, float* states, long long state_stride,
                             int state_offset, const int* state_slots, const int* query_start, const int* request_of_token,
                             void* out, int n_tokens, int hidden, cudaStream_t stream) {
  if (n_tokens == 0 || hidden == 0) return 0;
  MS_REQUIRE(x != out, "token_shift: the output must not be the input (a token reads the one before it)");
  const int threads = hidden >= 1024 ? 256 : 128;
  const size_t state_base = reinterpret_cast<size_t>(states) + (size_t)state_offset * sizeof(float);
  if (hidden % 8 == 0 && reinterpret_cast<size_t>(x) % 16 == 0 && reinterpret_cast<size_t>(out) % 16 == 0 &&
      reinterpret_cast<size_t>(shift) % 16 == 0 && state_base % 16 == 0 && state_stride % 4 == 0) {
    const int wide_threads = hidden >= 2048 ? 256 : hidden >= 512 ? 64 : 32;
    MS_SEQ_DISPATCH(dtype, (ms::launch(token_shift_wide_kernel<T>, n_tokens, wide_threads, 0, stream, (const T*)x, shift, states,
                                       state_stride, state_offset, state_slots, query_start, request_of_token, (T*)out, hidden)));
    MS_CHECK_LAUNCH("token_shift");
    return 0;
  }
  MS_SEQ_DISPATCH(dtype, (ms::launch(token_shift_kernel<T>, n_tokens, threads, 0, stream, (const T*)x, shift, states, state_stride,
                                     state_offset, state_slots, query_start, request_of_token, (T*)out, hidden)));
  MS_CHECK_LAUNCH("token_shift");
  return 0;
}

// tokens int32 [n_tokens]; table [buckets + 1, hidden] of type `dtype`; states int32 rows of state_stride numbers; residual
// float32 [n_tokens, hidden], added to.
MS_EXPORT int ms_pair_embedding(const int* tokens, const void* table, int dtype, int buckets, long long mul_prev, long long mul_cur,
                                int* states, long long state_stride, int state_offset, const int* state_slots,
                                const int* query_start, const int* request_of_token, float* residual, int n_tokens, int hidden,
                                cudaStream_t stream) {
  if (n_tokens == 0 || hidden == 0) return 0;
  MS_REQUIRE(buckets >= 1 && mul_prev >= 0 && mul_cur >= 0 && mul_prev < (1LL << 31) && mul_cur < (1LL << 31),
             "pair_embedding: %d buckets, factors %lld and %lld (0 .. 2^31 - 1: the hash is formed in 64 bits)", buckets, mul_prev, mul_cur);
  const int threads = hidden >= 1024 ? 256 : 128;
  MS_SEQ_DISPATCH(dtype, (ms::launch(pair_embedding_kernel<T>, n_tokens, threads, 0, stream, tokens, (const T*)table, buckets,
                                     mul_prev, mul_cur, states, state_stride, state_offset, state_slots,
                                     query_start, request_of_token, residual, hidden)));
  MS_CHECK_LAUNCH("pair_embedding");
  return 0;
}
