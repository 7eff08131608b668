// Attention over the paged cache, generic form: any head_dim, any number of query heads per kv
// head, any page size, optional window, optional sink per query head, values as wide as the keys or
// narrower, 32-bit arithmetic throughout.  T is the storage type of q, the pages and the
// output.  It is the whole attention of the 32-bit path and the fallback of the bfloat16
// path for sizes its tensor-core kernels refuse.
//
// Formula (crates/sglang-kernel/src/cpu.rs:475-517): kv head = q head / (n_q / n_kv);
// s_t = (q . k_t) * scale over the keys the row may see; softmax with the maximum
// subtracted; o = sum_t p_t v_t.  The mask is by length only: a row at position pos sees
// keys max(0, pos - window + 1) .. pos (crates/sglang-srt/src/cuda_attention.rs:285-297 for
// the causal length).  The running maximum and denominator follow the online form of
// cuda_attention.rs:137-151.
//
// Two terms that other designs add, both off by default:
//  * a sink: `sinks` holds one float per query head; exp(sink_h) is added to the softmax's denominator and to nothing
//    else.  It belongs to no key, gets no share of the values, is taken as it is (the score scale does not apply), and is
//    added exactly one time per row, also when the row's keys are split over several blocks (the merge adds it);
//  * a gate: `gates` holds one float per (row, query head) that multiplies the head's result (a mixer's output gate,
//    already passed through its sigmoid), applied where the result is normalised and written;
//  * values of another width than the keys: the output and the value rows are `value_dim` wide.  With
//    `shared_values` the value of a key is the first `value_dim` entries of its key row (a cache that
//    keeps one latent row per token serves as key and as value), and v_pool is not read.
//
// Work split: one block per (row, kv head and chunk of its query heads, split); the block's warp w
// owns query head kv_head * G + chunk * heads_per_block + w (at most 32 warps, so more than 32 query
// heads per kv head go in several chunks).  Keys are visited in blocks of 32 aligned to absolute multiples of 32,
// and a split covers `split_size` keys aligned to absolute multiples of split_size, so a
// row's arithmetic depends on its own position only, never on how the step was cut or
// what else is in the batch.  With split_size == 0 the block walks all keys and writes
// the output; otherwise it writes an unnormalised partial (acc, m, l) to scratch memory
// and srb_attention_combine merges the partials in split order.
#pragma once
#include "common.cuh"
#include <math.h>

#define KEY_BLOCK 32

struct AttnParams {
  const int* positions;      // [rows] position of the row in its sequence
  const int* row_request;    // [rows] index of the row's request in the block table
  const int* block_table;    // [requests, table_stride] page ids, -1 where none
  int table_stride;
  int n_q, n_kv, head_dim, page_size, num_pages;
  int window;                // 0 = all keys
  int chunk;                 // > 0: a row sees only the keys of its own chunk of `chunk` positions, counted from position 0
  int split_size;            // 0 = no split
  int max_splits;
  float scale;
  int* error_word;
  const float* sinks;        // [n_q] or null
  int value_dim;             // width of a value row and of the output
  int shared_values;         // 1: values are the first value_dim entries of the key rows
  int head_chunks;           // blocks per (row, kv head, split) along the query heads
  int heads_per_block;
  const float* gates = nullptr;   // [rows, n_q] or null: a factor on the result of every (row, query head)
};

// The first key that a row at `pos` may see: the start of its window, or of its chunk of positions, whichever is later.
// It never falls as pos grows, so the first row of a tile has the lowest first key of the tile.
__host__ __device__ __forceinline__ int srb_first_visible(int pos, int window, int chunk) {
  int begin = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  if (chunk > 0) {
    const int start = pos / chunk * chunk;
    begin = begin > start ? begin : start;
  }
  return begin;
}

__device__ __forceinline__ void row_key_range(const AttnParams& p, int pos, int split, int& lo, int& hi) {
  const int begin = srb_first_visible(pos, p.window, p.chunk);
  const int end = pos + 1;
  if (p.split_size == 0) {
    lo = begin;
    hi = end;
    return;
  }
  const int first = begin / p.split_size;
  lo = max(begin, (first + split) * p.split_size);
  hi = min(end, (first + split + 1) * p.split_size);
}

__device__ __forceinline__ int row_split_count(const AttnParams& p, int pos) {
  if (p.split_size == 0) return 1;
  const int begin = srb_first_visible(pos, p.window, p.chunk);
  return pos / p.split_size - begin / p.split_size + 1;
}

template <typename T, int DIM_PER_LANE>
__global__ void paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                       const T* __restrict__ v_pool, T* __restrict__ out,
                                       float* __restrict__ part_acc, float* __restrict__ part_ml,
                                       AttnParams p) {
  extern __shared__ float smem[];
  const int d = p.head_dim, vd = p.value_dim;
  const int groups = p.n_q / p.n_kv;
  float* k_tile = smem;                                  // [32][d + 1]
  float* v_tile = k_tile + KEY_BLOCK * (d + 1);          // [32][vd], or the key tile itself
  float* q_tile = v_tile + (p.shared_values ? 0 : KEY_BLOCK * vd);   // [heads_per_block][d]
  const int v_stride = p.shared_values ? d + 1 : vd;
  if (p.shared_values) v_tile = k_tile;
  __shared__ long long key_offset[KEY_BLOCK];            // element offset of each key's row, -1 = masked

  const int row = blockIdx.z, kv_head = blockIdx.y / p.head_chunks, chunk = blockIdx.y % p.head_chunks;
  const int split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[row];
  int lo, hi;
  row_key_range(p, pos, split, lo, hi);
  if (lo >= hi) return;
  const int request = p.row_request[row];
  const int first_head = chunk * p.heads_per_block;      // within the kv head's group
  const int here = min(p.heads_per_block, groups - first_head);
  const bool live = warp < here;                         // a warp beyond the group's heads only helps to load
  const int q_head = kv_head * groups + first_head + (live ? warp : 0);

  for (int i = threadIdx.x; i < here * d; i += blockDim.x)
    q_tile[i] = srb_to_float(q[((size_t)row * p.n_q + (size_t)kv_head * groups + first_head) * d + i]);

  float m = -INFINITY, l = 0.f;
  float acc[DIM_PER_LANE];
#pragma unroll
  for (int j = 0; j < DIM_PER_LANE; ++j) acc[j] = 0.f;

  for (int base = lo & ~(KEY_BLOCK - 1); base < hi; base += KEY_BLOCK) {
    __syncthreads();                                     // previous tile fully consumed
    if (threadIdx.x < KEY_BLOCK) {
      const int key = base + threadIdx.x;
      long long offset = -1;
      if (key >= lo && key < hi) {
        const int page = p.block_table[(size_t)request * p.table_stride + key / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          atomicOr(p.error_word, SRB_FLAG_BAD_PAGE);
        } else {
          offset = (((long long)page * p.n_kv + kv_head) * p.page_size + key % p.page_size) * d;
        }
      }
      key_offset[threadIdx.x] = offset;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < KEY_BLOCK * d; i += blockDim.x) {
      const int key = i / d, e = i - key * d;
      const long long offset = key_offset[key];
      k_tile[key * (d + 1) + e] = offset < 0 ? 0.f : srb_to_float(k_pool[offset + e]);
    }
    if (!p.shared_values) {
      for (int i = threadIdx.x; i < KEY_BLOCK * vd; i += blockDim.x) {
        const int key = i / vd, e = i - key * vd;
        const long long offset = key_offset[key];          // in elements of a key row: rows are d or vd wide
        v_tile[key * vd + e] = offset < 0 ? 0.f : srb_to_float(v_pool[offset / d * vd + e]);
      }
    }
    __syncthreads();

    // one key per lane: the dot product runs over the head in index order
    float s = 0.f;
    const float* qv = q_tile + (live ? warp : 0) * d;
    const float* kv = k_tile + lane * (d + 1);
    for (int e = 0; e < d; ++e) s += qv[e] * kv[e];
    s = key_offset[lane] < 0 ? -INFINITY : s * p.scale;

    const float m_new = fmaxf(m, srb_warp_max(s));       // finite: the tile holds a visible key
    const float correction = expf(m - m_new);            // exp(-inf) = 0 on the first tile
    const float prob = expf(s - m_new);                  // 0 for masked keys
    l = l * correction + srb_warp_sum(prob);
    m = m_new;
#pragma unroll
    for (int j = 0; j < DIM_PER_LANE; ++j) acc[j] *= correction;
    for (int key = 0; key < KEY_BLOCK; ++key) {
      const float pk = __shfl_sync(0xffffffffu, prob, key);
#pragma unroll
      for (int j = 0; j < DIM_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (e < vd) acc[j] += pk * v_tile[key * v_stride + e];
      }
    }
  }
  if (!live) return;

  if (p.split_size == 0) {
    if (p.sinks) {
      // the sink joins the denominator as one more term: exp(sink - M) with M the larger maximum
      const float sink = p.sinks[q_head];
      const float m_new = fmaxf(m, sink);
      const float correction = expf(m - m_new);
      l = l * correction + expf(sink - m_new);
#pragma unroll
      for (int j = 0; j < DIM_PER_LANE; ++j) acc[j] *= correction;
    }
    const float inv = p.gates ? p.gates[(size_t)row * p.n_q + q_head] / l : 1.0f / l;
#pragma unroll
    for (int j = 0; j < DIM_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < vd) out[((size_t)row * p.n_q + q_head) * vd + e] = srb_from_float<T>(acc[j] * inv);
    }
  } else {
    const size_t slot = ((size_t)row * p.n_q + q_head) * p.max_splits + split;
#pragma unroll
    for (int j = 0; j < DIM_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < vd) part_acc[slot * vd + e] = acc[j];
    }
    if (lane == 0) {
      part_ml[slot * 2] = m;
      part_ml[slot * 2 + 1] = l;
    }
  }
}

// Merges a row's partials in split order: M = max m_s, out = sum acc_s e^(m_s - M) / sum l_s e^(m_s - M).
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                         T* __restrict__ out, AttnParams p) {
  const int row = blockIdx.x, q_head = blockIdx.y;
  const int pos = p.positions[row];
  if (pos < 0) return;                                   // a padding row: no block wrote partials for it
  const int wanted = row_split_count(p, pos);
  if (wanted > p.max_splits) {
    // the launch has too few blocks along the splits for this row: its newest keys were left out
    if (q_head == 0 && threadIdx.x == 0 && p.error_word) atomicOr(p.error_word, SRB_FLAG_TOO_FEW_SPLITS);
  }
  const int count = min(wanted, p.max_splits);
  const size_t first = ((size_t)row * p.n_q + q_head) * p.max_splits;
  float m = p.sinks ? p.sinks[q_head] : -INFINITY;
  for (int s = 0; s < count; ++s) m = fmaxf(m, part_ml[(first + s) * 2]);
  float l = p.sinks ? expf(p.sinks[q_head] - m) : 0.f;   // the sink counts once, whatever the number of splits
  for (int s = 0; s < count; ++s) l += part_ml[(first + s) * 2 + 1] * expf(part_ml[(first + s) * 2] - m);
  const float inv = p.gates ? p.gates[(size_t)row * p.n_q + q_head] / l : 1.0f / l;
  for (int e = threadIdx.x; e < p.value_dim; e += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < count; ++s)
      acc += part_acc[(first + s) * p.value_dim + e] * expf(part_ml[(first + s) * 2] - m);
    out[((size_t)row * p.n_q + q_head) * p.value_dim + e] = srb_from_float<T>(acc * inv);
  }
}

template <typename T, int DIM_PER_LANE>
static int launch_attention(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_acc,
                            float* part_ml, const AttnParams& p, int rows, cudaStream_t s) {
  const size_t smem = ((size_t)KEY_BLOCK * (p.head_dim + 1) + (p.shared_values ? 0 : (size_t)KEY_BLOCK * p.value_dim) +
                       (size_t)p.heads_per_block * p.head_dim) * sizeof(float);
  if (smem > 227 * 1024) SRB_FAIL("paged_attention: %zu bytes of shared memory exceed 232448", smem);
  if (smem > 48 * 1024)
    SRB_CUDA_CALL(cudaFuncSetAttribute(paged_attention_kernel<T, DIM_PER_LANE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(p.split_size == 0 ? 1 : p.max_splits, p.n_kv * p.head_chunks, rows);
  if (grid.y > 65535) SRB_FAIL("paged_attention: %d blocks along the heads exceed 65535", (int)grid.y);
  paged_attention_kernel<T, DIM_PER_LANE><<<grid, p.heads_per_block * 32, smem, s>>>(
      (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, part_acc, part_ml, p);
  SRB_LAUNCH_CHECK("paged_attention");
  if (p.split_size != 0) {
    dim3 cgrid(rows, p.n_q);
    attention_combine_kernel<T><<<cgrid, 64, 0, s>>>(part_acc, part_ml, (T*)out, p);
    SRB_LAUNCH_CHECK("attention_combine");
  }
  return SRB_OK;
}

// Checks the sizes and launches; shared by every entry point.  Scratch (only when split_size > 0):
// part_acc holds rows * n_q * max_splits * value_dim floats and part_ml rows * n_q * max_splits * 2.
// `sinks` null: no sink.  `value_dim` 0: as wide as the keys.  `v_pool` null: the values are the first
// value_dim entries of the key rows.
// `chunk` > 0: a row sees only keys of its own chunk of positions (see AttnParams).
static int paged_attention_dispatch_masked(const void* q, const void* k_pool, const void* v_pool, void* out,
                                           float* part_acc, float* part_ml, const int* positions,
                                           const int* row_request, const int* block_table, int table_stride, int rows,
                                           int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                           int chunk, int split_size, int max_splits, float scale, int* error_word,
                                           int dtype, const float* sinks, int value_dim, void* stream,
                                           const float* gates = nullptr) {
  if (rows <= 0) return SRB_OK;
  if (chunk < 0) SRB_FAIL("paged_attention: the chunk size must be non-negative");
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0)
    SRB_FAIL("paged_attention: %d query heads are not a multiple of %d kv heads", n_q, n_kv);
  if (head_dim <= 0) SRB_FAIL("paged_attention: head_dim %d must be positive", head_dim);
  if (value_dim == 0) value_dim = head_dim;
  if (value_dim < 0 || value_dim > 1024 || (!v_pool && value_dim > head_dim))
    SRB_FAIL("paged_attention: values of %d entries must be positive, at most 1024 and, if they are the head of the key "
             "rows (%d entries), no wider than those", value_dim, head_dim);
  if (page_size <= 0 || num_pages <= 0 || table_stride <= 0)
    SRB_FAIL("paged_attention: page size, page count and table stride must be positive");
  if (window < 0 || split_size < 0) SRB_FAIL("paged_attention: window and split size must be non-negative");
  if (split_size != 0 && (max_splits <= 0 || !part_acc || !part_ml))
    SRB_FAIL("paged_attention: a split run needs scratch memory and max_splits > 0");
  if (rows > 65535) {
    // grid.z is limited to 65535 blocks
    SRB_FAIL("paged_attention: %d rows exceed 65535 in one launch", rows);
  }
  AttnParams p;
  p.positions = positions; p.row_request = row_request; p.block_table = block_table;
  p.table_stride = table_stride; p.n_q = n_q; p.n_kv = n_kv; p.head_dim = head_dim;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.chunk = chunk; p.split_size = split_size;
  p.max_splits = split_size == 0 ? 1 : max_splits; p.scale = scale; p.error_word = error_word;
  p.sinks = sinks; p.value_dim = value_dim; p.shared_values = v_pool == nullptr; p.gates = gates;
  const int groups = n_q / n_kv;
  p.head_chunks = (groups + 31) / 32;
  p.heads_per_block = (groups + p.head_chunks - 1) / p.head_chunks;
  cudaStream_t s = (cudaStream_t)stream;
  const int per_lane = (value_dim + 31) / 32;
#define SRB_ATTN_CASE(T, N) \
  return launch_attention<T, N>(q, k_pool, v_pool, out, part_acc, part_ml, p, rows, s)
#define SRB_ATTN_DISPATCH(T)                        \
  if (per_lane <= 1) { SRB_ATTN_CASE(T, 1); }       \
  else if (per_lane <= 2) { SRB_ATTN_CASE(T, 2); }  \
  else if (per_lane <= 4) { SRB_ATTN_CASE(T, 4); }  \
  else if (per_lane <= 8) { SRB_ATTN_CASE(T, 8); }  \
  else if (per_lane <= 16) { SRB_ATTN_CASE(T, 16); } \
  else { SRB_ATTN_CASE(T, 32); }
  if (dtype == SRB_DTYPE_F32) { SRB_ATTN_DISPATCH(float) }
  if (dtype == SRB_DTYPE_BF16) { SRB_ATTN_DISPATCH(__nv_bfloat16) }
  SRB_FAIL("paged_attention: unknown dtype %d", dtype);
}

static int paged_attention_dispatch_ex(const void* q, const void* k_pool, const void* v_pool, void* out,
                                       float* part_acc, float* part_ml, const int* positions,
                                       const int* row_request, const int* block_table, int table_stride, int rows,
                                       int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                       int split_size, int max_splits, float scale, int* error_word, int dtype,
                                       const float* sinks, int value_dim, void* stream) {
  return paged_attention_dispatch_masked(q, k_pool, v_pool, out, part_acc, part_ml, positions, row_request, block_table,
                                         table_stride, rows, n_q, n_kv, head_dim, page_size, num_pages, window, 0,
                                         split_size, max_splits, scale, error_word, dtype, sinks, value_dim, stream);
}

static int paged_attention_dispatch(const void* q, const void* k_pool, const void* v_pool, void* out,
                                   float* part_acc, float* part_ml, const int* positions,
                                   const int* row_request, const int* block_table, int table_stride, int rows,
                                   int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                   int split_size, int max_splits, float scale, int* error_word, int dtype,
                                   void* stream) {
  if (!v_pool) SRB_FAIL("paged_attention: the value pool is missing");
  return paged_attention_dispatch_ex(q, k_pool, v_pool, out, part_acc, part_ml, positions, row_request, block_table,
                                     table_stride, rows, n_q, n_kv, head_dim, page_size, num_pages, window, split_size,
                                     max_splits, scale, error_word, dtype, nullptr, 0, stream);
}
