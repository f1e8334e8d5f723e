// Paged grouped-query attention on the tensor cores for head sizes that attention_mma.cu is not built for: query and key
// heads of d entries and value heads of dv entries, both any multiple of 16 up to 128 and not necessarily the same, with
// the two options of the other kernels (a sink in the softmax's denominator, a gate per head on the output).
//
// The scheme is attention_mma.cu's: one thread block per (request, key/value head, tile of query rows, split of the keys);
// the rows of a tile are the pairs (token, query head of the kv head's group), token-major; W warps of 16 rows each; key and
// value tiles of BN keys gathered from the pages by 16-byte asynchronous copies into two buffers; S = Q K^T and O += P V
// by mma.m16n8k16 with ldmatrix fragments, the softmax online in float32 with the scale folded into exp2.  What differs: the
// head sizes are run-time numbers, so the tiles' rows are padded by 16 bytes instead of swizzled (a row of d + 8 elements:
// eight consecutive rows still fall into different banks because (d + 8) / 8 is odd), the loops over a head's 16-entry
// pieces have run-time bounds, and the output accumulator is sized for 128 value entries whatever dv is.
#include "mma_common.cuh"

namespace ms {

constexpr int kAnyMax = 128;      // largest head size (d and dv)

template <int W, int BN>
__global__ void __launch_bounds__(W * 32)
attention_mma_any_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_tables, int table_stride,
                         const int* __restrict__ query_start, const int* __restrict__ context_lens, int page_size, int n_q,
                         int n_kv, int d, int dv, float scale_log2, int window, __nv_bfloat16* __restrict__ out,
                         float* __restrict__ part_o, float* __restrict__ part_lse, int num_splits, int sink,
                         const __nv_bfloat16* __restrict__ gate, int gate_ld, int chunk, int n_v) {
  grid_dependency_wait();
  grid_dependency_launch();
  constexpr int BM = 16 * W, THREADS = 32 * W;
  const int ks = d + 8, vs = dv + 8;                    // elements between the rows of a tile
  const int k_chunks = d / 8, v_chunks = dv / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [BM][ks]
  __nv_bfloat16* k_s = q_s + BM * ks;                                       // [2][BN][ks]
  __nv_bfloat16* v_s = k_s + 2 * BN * ks;                                   // [2][BN][vs]
  long long* row_index = reinterpret_cast<long long*>(v_s + 2 * BN * vs);   // [2][BN] row of a key in the key pool, -1: none
  long long* value_index = row_index + 2 * BN;                              // [2][BN] its row in the value pool (n_v heads)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv_head = blockIdx.y;
  const int request = blockIdx.z / num_splits, split = blockIdx.z % num_splits;
  const int group = n_q / n_kv;
  const int q0 = query_start[request];
  const int q_len = query_start[request + 1] - q0;
  const int ctx = context_lens[request];
  const int rows_total = q_len * group;
  const int row0 = ((rows_total + BM - 1) / BM - 1 - (int)blockIdx.x) * BM;      // the last tiles (most keys) first
  if (row0 < 0) return;
  const int first_pos = ctx - q_len;
  const int t_lo = row0 / group;
  const int last_row = min(rows_total, row0 + BM) - 1;
  const int t_hi = last_row / group;
  int key_begin = 0;
  if (window > 0) key_begin = max(0, first_pos + t_lo - window + 1);
  if (chunk > 0) key_begin = max(key_begin, (first_pos + t_lo) - (first_pos + t_lo) % chunk);      // the lowest row's chunk
  const int key_end = first_pos + t_hi + 1;
  const int tile_begin = (key_begin / BN) * BN;
  const int n_tiles = (key_end - tile_begin + BN - 1) / BN;
  const int tiles_per_split = (n_tiles + num_splits - 1) / num_splits;
  const int tile_lo = split * tiles_per_split;
  const int tile_hi = min(n_tiles, tile_lo + tiles_per_split);
  const int* table = block_tables + (size_t)request * table_stride;
  const int quad_row = lane >> 2, quad_col = lane & 3;
  const int warp_row0 = row0 + warp * 16;
  auto thread_row = [&](int half) { return warp_row0 + quad_row + half * 8; };
  auto index_of = [&](int row) { return (size_t)(q0 + row / group) * n_q + kv_head * group + row % group; };

  if (tile_lo >= tile_hi) {                               // nothing to do for this split
    if (num_splits > 1 && quad_col == 0) {
      for (int half = 0; half < 2; ++half) {
        const int row = thread_row(half);
        if (row >= rows_total) continue;
        const size_t index = index_of(row);
        if (sink && split == 0) {                         // the sink alone: a result of zeros with weight 1
          float* dst = part_o + index * num_splits * dv;
          for (int c = 0; c < dv; ++c) dst[c] = 0.f;
          part_lse[index * num_splits] = 0.f;
        } else {
          part_lse[index * num_splits + split] = -INFINITY;
        }
      }
    }
    return;
  }

  auto find_rows = [&](int tile, int buffer) {
    const int key0 = tile_begin + tile * BN;
    for (int r = tid; r < BN; r += THREADS) {
      const int key = key0 + r;
      long long index = -1, value = -1;
      if (tile < tile_hi && key < key_end) {
        const int page = table[key / page_size];
        index = ((long long)page * n_kv + kv_head) * page_size + key % page_size;
        value = ((long long)page * n_v + kv_head % n_v) * page_size + key % page_size;
      }
      row_index[buffer * BN + r] = index;
      value_index[buffer * BN + r] = value;
    }
  };
  auto load_tile = [&](int stage) {
    __nv_bfloat16* kt = k_s + stage * BN * ks;
    __nv_bfloat16* vt = v_s + stage * BN * vs;
    const long long* rows = row_index + stage * BN;
    for (int i = tid; i < BN * k_chunks; i += THREADS) {
      const int r = i / k_chunks, c = i % k_chunks;
      const long long at = rows[r];
      cp_async_16(kt + r * ks + c * 8, k_pool + (at < 0 ? 0 : at * d + c * 8), at >= 0);
    }
    const long long* value_rows = value_index + stage * BN;
    for (int i = tid; i < BN * v_chunks; i += THREADS) {
      const int r = i / v_chunks, c = i % v_chunks;
      const long long at = value_rows[r];
      cp_async_16(vt + r * vs + c * 8, v_pool + (at < 0 ? 0 : at * dv + c * 8), at >= 0);
    }
  };

  find_rows(tile_lo, 0);
  find_rows(tile_lo + 1, 1);
  __syncthreads();
  load_tile(0);
  for (int i = tid; i < BM * k_chunks; i += THREADS) {       // the query tile
    const int r = i / k_chunks, c = i % k_chunks;
    const int row = row0 + r;
    const bool valid = row < rows_total;
    cp_async_16(q_s + r * ks + c * 8, valid ? q + index_of(row) * d + c * 8 : q, valid);
  }
  cp_async_commit();

  float acc_o[kAnyMax / 8][4];
#pragma unroll
  for (int n = 0; n < kAnyMax / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc_o[n][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  int pos[2];
  for (int half = 0; half < 2; ++half) pos[half] = first_pos + thread_row(half) / group;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 < tile_hi) load_tile(stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    find_rows(tile + 2, stage);          // this tile's copies have landed; its rows are no longer needed
    const __nv_bfloat16* kt = k_s + stage * BN * ks;
    const __nv_bfloat16* vt = v_s + stage * BN * vs;
    const int key0 = tile_begin + tile * BN;

    // ---- S = Q K^T
    float acc_s[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc_s[n][e] = 0.f;
    for (int kk = 0; kk < d / 16; ++kk) {
      unsigned a[4];
      ldmatrix_x4(a, q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ks + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        unsigned b[4];
        ldmatrix_x4(b, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ks + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(acc_s[2 * np], a, b[0], b[1]);
        mma_bf16(acc_s[2 * np + 1], a, b[2], b[3]);
      }
    }

    // ---- mask and online softmax (scores are scaled inside the exponent)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + n * 8 + quad_col * 2 + (e & 1);
        const int p = pos[e >> 1];
        const bool visible = key <= p && (window <= 0 || key > p - window) && (chunk <= 0 || key >= p - p % chunk);
        if (!visible) acc_s[n][e] = -INFINITY;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], acc_s[n][e]);
      }
    float base[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float v = tile_max[half];
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
      const float updated = fmaxf(m_run[half], v);
      base[half] = updated == -INFINITY ? 0.f : updated * scale_log2;
      corr[half] = exp2f(m_run[half] * scale_log2 - base[half]);      // m == -inf gives 0
      m_run[half] = updated;
    }
#pragma unroll
    for (int n = 0; n < BN / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc_s[n][e] = exp2f(acc_s[n][e] * scale_log2 - base[e >> 1]);
        sum[e >> 1] += acc_s[n][e];
      }
#pragma unroll
    for (int half = 0; half < 2; ++half) l_run[half] = l_run[half] * corr[half] + sum[half];
#pragma unroll
    for (int n = 0; n < kAnyMax / 8; ++n) {
      acc_o[n][0] *= corr[0];
      acc_o[n][1] *= corr[0];
      acc_o[n][2] *= corr[1];
      acc_o[n][3] *= corr[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kp = 0; kp < BN / 16; ++kp) {
      unsigned p[4];
      p[0] = pack_bf16(acc_s[2 * kp][0], acc_s[2 * kp][1]);
      p[1] = pack_bf16(acc_s[2 * kp][2], acc_s[2 * kp][3]);
      p[2] = pack_bf16(acc_s[2 * kp + 1][0], acc_s[2 * kp + 1][1]);
      p[3] = pack_bf16(acc_s[2 * kp + 1][2], acc_s[2 * kp + 1][3]);
#pragma unroll
      for (int np = 0; np < kAnyMax / 16; ++np) {
        if (np < dv / 16) {
          unsigned b[4];
          ldmatrix_x4_trans(b, vt + (kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vs + np * 16 + (lane >> 4) * 8);
          mma_bf16(acc_o[2 * np], p, b[0], b[1]);
          mma_bf16(acc_o[2 * np + 1], p, b[2], b[3]);
        }
      }
    }
    __syncthreads();       // all warps are done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- finish: row sums across the quad, the sink, normalise, the gate, store
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float l = l_run[half];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = thread_row(half);
    if (row >= rows_total) continue;
    const float m = m_run[half];
    if (sink && split == 0) l += m == -INFINITY ? 1.f : exp2f(-m * scale_log2);
    float inv = l > 0.f ? 1.f / l : 0.f;
    const size_t index = index_of(row);
    if (num_splits == 1) {
      if (gate != nullptr) inv /= 1.f + __expf(-__bfloat162float(gate[(size_t)(q0 + row / group) * gate_ld + kv_head * group + row % group]));
      __nv_bfloat16* dst = out + index * dv;
#pragma unroll
      for (int n = 0; n < kAnyMax / 8; ++n)
        if (n < dv / 8)
          *reinterpret_cast<unsigned*>(dst + n * 8 + quad_col * 2) = pack_bf16(acc_o[n][2 * half] * inv, acc_o[n][2 * half + 1] * inv);
    } else {
      float* dst = part_o + (index * num_splits + split) * dv;
#pragma unroll
      for (int n = 0; n < kAnyMax / 8; ++n)
        if (n < dv / 8)
          *reinterpret_cast<float2*>(dst + n * 8 + quad_col * 2) = make_float2(acc_o[n][2 * half] * inv, acc_o[n][2 * half + 1] * inv);
      if (quad_col == 0)
        part_lse[index * num_splits + split] = l > 0.f ? (m == -INFINITY ? 0.f : m * scale_log2) + log2f(l) : -INFINITY;
    }
  }
}

// Merges the key splits of one (token, head) for any dv: out = sum_s w_s O_s / sum_s w_s with w_s = 2^(lse_s - max lse), splits
// added in ascending order; one warp per item.
__global__ void attention_combine_any_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                             __nv_bfloat16* __restrict__ out, int num_splits, int dv, int n_items,
                                             const __nv_bfloat16* __restrict__ gate, int gate_ld, int n_q) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const float* lse = part_lse + (size_t)item * num_splits;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, lse[s]);
  float total = 0.f;
  for (int s = 0; s < num_splits; ++s) total += lse[s] == -INFINITY ? 0.f : exp2f(lse[s] - m);
  float inv = total > 0.f ? 1.f / total : 0.f;
  if (gate != nullptr) inv /= 1.f + __expf(-__bfloat162float(gate[(size_t)(item / n_q) * gate_ld + item % n_q]));
  for (int c = lane; c < dv; c += 32) {
    float sum = 0.f;
    for (int s = 0; s < num_splits; ++s)
      if (lse[s] != -INFINITY) sum += exp2f(lse[s] - m) * part_o[((size_t)item * num_splits + s) * dv + c];
    out[(size_t)item * dv + c] = __float2bfloat16_rn(sum * inv);
  }
}

template <int W, int BN>
int launch_attention_any(const void* q, const void* k_pool, const void* v_pool, const int* block_tables, int table_stride,
                         const int* query_start, const int* context_lens, int page_size, int n_q, int n_kv, int d, int dv,
                         float scale, int window, void* out, float* part_o, float* part_lse, int num_splits, int n_requests,
                         int max_query_len, int n_tokens, int sink, const void* gate, int gate_ld, int first_token,
                         int chunk, int n_v, cudaStream_t stream) {
  constexpr int BM = 16 * W;
  const size_t smem = (size_t)(BM * (d + 8) + 2 * BN * (d + 8) + 2 * BN * (dv + 8)) * sizeof(__nv_bfloat16) + 4 * BN * sizeof(long long);
  auto kernel = attention_mma_any_kernel<W, BN>;
  static bool configured = false;
  if (!configured) {
    const size_t most = (size_t)(BM + 4 * BN) * (kAnyMax + 8) * sizeof(__nv_bfloat16) + 4 * BN * sizeof(long long);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e != cudaSuccess) MS_FAIL("attention (any head size): cannot reserve %zu bytes of shared memory: %s", most, cudaGetErrorString(e));
    configured = true;
  }
  const int group = n_q / n_kv;
  const long long tiles = ((long long)max_query_len * group + BM - 1) / BM;
  MS_REQUIRE(tiles <= 2147483647LL && (long long)n_requests * num_splits <= 65535 && n_kv <= 65535,
             "attention (any head size): grid %lld x %d x %lld exceeds the launch limits", tiles, n_kv, (long long)n_requests * num_splits);
  dim3 grid((unsigned)tiles, n_kv, n_requests * num_splits);
  ms::launch(kernel, grid, W * 32, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
             block_tables, table_stride, query_start, context_lens, page_size, n_q, n_kv, d, dv, scale * 1.4426950408889634f, window,
             (__nv_bfloat16*)out, part_o, part_lse, num_splits, sink, (const __nv_bfloat16*)gate, gate_ld, chunk, n_v);
  MS_CHECK_LAUNCH("attention_mma_any");
  if (num_splits > 1) {
    const size_t skip = (size_t)first_token * n_q;
    const int items = (n_tokens - first_token) * n_q;
    const __nv_bfloat16* gates = gate ? (const __nv_bfloat16*)gate + (size_t)first_token * gate_ld : nullptr;
    ms::launch(attention_combine_any_kernel, (items + 3) / 4, 128, 0, stream, (const float*)(part_o + skip * num_splits * dv),
               (const float*)(part_lse + skip * num_splits), (__nv_bfloat16*)out + skip * dv, num_splits, dv, items, gates, gate_ld, n_q);
    MS_CHECK_LAUNCH("attention_combine_any");
  }
  return 0;
}

}  // namespace ms

using namespace ms;

// Head sizes this kernel takes (the sizes attention_mma.cu is built for should go there: its loops are unrolled).
MS_EXPORT int ms_attention_mma_any_supports(int d, int dv) {
  return d >= 16 && d <= kAnyMax && d % 16 == 0 && dv >= 16 && dv <= kAnyMax && dv % 16 == 0;
}

// In how many parts the keys of a step of few rows per request should be cut (1 for anything else): as many as give every
// multiprocessor about two blocks, each part keeping 128 keys or more, at most 32.
MS_EXPORT int ms_attention_mma_any_splits(int n_requests, int n_kv, int n_q, int max_query_len, int max_context_len) {
  if (n_kv <= 0 || (long long)max_query_len * (n_q / n_kv) > 16) return 1;
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int base = n_requests * n_kv;
  int splits = (2 * sms + base - 1) / (base > 0 ? base : 1);
  const int limit = max_context_len / 128;
  if (splits > limit) splits = limit;
  if (splits > 32) splits = 32;
  return splits < 1 ? 1 : splits;
}

// Arguments as ms_paged_attention_mma, with the value heads' size dv: q [n_tokens, n_q, d], key pool [pages, n_kv, page_size, d],
// value pool [pages, n_v, page_size, dv] (n_v a divisor of n_kv: key head g reads value head g % n_v), out [n_tokens, n_q, dv];
// part_o [n_tokens * n_q * num_splits * dv].
MS_EXPORT int ms_paged_attention_mma_any(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                         int table_stride, const int* query_start, const int* context_lens, int page_size,
                                         int n_q, int n_kv, int d, int dv, float scale, int window, void* out, float* part_o,
                                         float* part_lse, int num_splits, int n_requests, int max_query_len, int n_tokens,
                                         int sink, const void* gate, int gate_ld, int first_token, int chunk, int n_v, cudaStream_t stream) {
  if (n_tokens == 0 || n_requests == 0) return 0;
  MS_REQUIRE(ms_attention_mma_any_supports(d, dv), "attention (any head size): sizes %d and %d are not multiples of 16 up to %d", d, dv, kAnyMax);
  MS_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention: %d query heads are not a multiple of %d key/value heads", n_q, n_kv);
  MS_REQUIRE(page_size > 0 && max_query_len > 0, "attention: page size %d, longest portion %d", page_size, max_query_len);
  MS_REQUIRE(num_splits >= 1 && num_splits <= 64 && (num_splits == 1 || (part_o && part_lse)), "attention: %d splits (1..64) need scratch", num_splits);
  MS_REQUIRE(first_token >= 0 && first_token < n_tokens, "attention: first row %d of %d", first_token, n_tokens);
  MS_REQUIRE(n_v > 0 && n_kv % n_v == 0, "attention: %d value heads for %d key heads", n_v, n_kv);
  const bool small = (long long)max_query_len * (n_q / n_kv) <= 16;
  if (small)
    return launch_attention_any<1, 32>(q, k_pool, v_pool, block_tables, table_stride, query_start, context_lens, page_size, n_q, n_kv, d,
                                       dv, scale, window, out, part_o, part_lse, num_splits, n_requests, max_query_len, n_tokens, sink,
                                       gate, gate_ld, first_token, chunk, n_v, stream);
  return launch_attention_any<4, 64>(q, k_pool, v_pool, block_tables, table_stride, query_start, context_lens, page_size, n_q, n_kv, d, dv,
                                     scale, window, out, part_o, part_lse, num_splits, n_requests, max_query_len, n_tokens, sink, gate,
                                     gate_ld, first_token, chunk, n_v, stream);
}
