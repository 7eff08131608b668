// Attention over cache rows that serve as key and as value, on the tensor cores (bfloat16): every query head
// reads the same row per token (one "kv head"); the key is the whole row (d entries), the value its first vd
// entries; optional sink per head.  This is the shape that attention through latents gives once the queries
// are carried into the latent space (parts/latent_attention.py).  The generic kernel (attention_kernels.cuh)
// computes the same in 32-bit arithmetic for every size and dtype; this one takes d % 16 == 0, vd % 32 == 0,
// vd <= 512.
//
// A block owns 16 query slots: `heads_per_block` heads of one row, or, when there are fewer than 16 heads, the
// heads of several consecutive rows of one request (each row masked by its own position), and walks the keys
// 64 at a time.  Its warps (eight when the value columns divide among them in whole 8-column tiles, else four)
// share every step: for the scores each warp takes its share of the 64 keys (mma.sync m16n8k16, the row of
// queries against the key rows in shared memory, two chains of accumulators so that consecutive products do not
// wait for each other); maxima and sums of the softmax are exchanged through shared memory, in 32-bit; the weights
// go to shared memory as bfloat16 and each warp multiplies them with its share of the value columns, which it keeps
// in registers (32-bit).
// Key tiles are aligned to absolute positions (multiples of 64), so a row's arithmetic depends on its own
// position only, however the step was cut.  Two ways of launching:
//   * tiles (prompt portions): int32 [n, 4] = (first row, rows <= 64, request, first position); a block takes
//     rows_per_block consecutive rows of a tile and all keys up to them, and writes the output;
//   * split rows (decoded tokens): one block per (row, head group, split of `split_size` keys); partial results
//     go to scratch memory in the generic kernel's layout and its merge kernel finishes them (with the sink).
#include "attention_kernels.cuh"
#include "mma_helpers.cuh"

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define LA_KEYS 64
#define LA_SLOTS 16
#define LA_PAD 8

struct LaParams {
  const __nv_bfloat16* q;      // [rows, n_q, d]
  const __nv_bfloat16* pool;   // [pages, 1, page_size, d]
  __nv_bfloat16* out;          // [rows, n_q, vd]
  float* part_acc;
  float* part_ml;
  const int* positions;
  const int* row_request;
  const int* block_table;
  const int* tiles;
  const float* sinks;
  int* error_word;
  int table_stride, n_q, d, vd, page_size, num_pages;
  int split_size, max_splits;
  int window;                  // a row sees itself and the window - 1 keys before it; 0: every earlier key
  int heads_per_block, rows_per_block, units_per_tile;
  float scale;
};

template <int NT_MAX, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(LaParams p) {
  constexpr int THREADS = WARPS * 32;
  constexpr int KEYS_PER_WARP = LA_KEYS / WARPS;          // 16 (two 8-key tiles) or 8 (one)
  constexpr int ST = KEYS_PER_WARP / 8;
  extern __shared__ __align__(16) unsigned char la_smem[];
  const int d = p.d, vd = p.vd, pitch = d + LA_PAD;
  __nv_bfloat16* k_tile = reinterpret_cast<__nv_bfloat16*>(la_smem);             // [64][pitch]
  __nv_bfloat16* q_tile = k_tile + LA_KEYS * pitch;                              // [16][pitch]
  __nv_bfloat16* p_tile = q_tile + LA_SLOTS * pitch;                             // [16][72]
  float* warp_max = reinterpret_cast<float*>(p_tile + LA_SLOTS * (LA_KEYS + LA_PAD));   // [WARPS][16]
  float* warp_sum = warp_max + WARPS * LA_SLOTS;                                 // [WARPS][16]
  long long* key_offset = reinterpret_cast<long long*>(warp_sum + WARPS * LA_SLOTS);   // [64]
  srb_launch_dependents();
  srb_grid_dependency_wait();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, group = blockIdx.y;
  int first_row, n_rows, request, first_pos;
  if (p.split_size == 0) {
    const int* t = p.tiles + 4 * (blockIdx.z / p.units_per_tile);
    const int sub = (blockIdx.z % p.units_per_tile) * p.rows_per_block;
    first_row = t[0] + sub;
    n_rows = min(p.rows_per_block, t[1] - sub);
    request = t[2];
    first_pos = t[3] + sub;
    if (n_rows <= 0) return;
  } else {
    first_row = blockIdx.z;
    n_rows = 1;
    request = p.row_request[first_row];
    first_pos = p.positions[first_row];
    if (first_pos < 0) return;                      // a padding row
  }
  // the block's first row sees the earliest key of all its rows; splits are counted from that row's first split on
  const int earliest = srb_first_visible(first_pos, p.window, 0);
  const int lo = p.split_size == 0 ? earliest : max(earliest, (earliest / p.split_size + split) * p.split_size);
  const int hi = p.split_size == 0 ? first_pos + n_rows : min((earliest / p.split_size + split + 1) * p.split_size, first_pos + 1);
  if (lo >= hi) return;
  const int hg = p.heads_per_block;
  const int head0 = group * hg;

  // the queries: slot m = (row m / hg of the block, head head0 + m % hg)
  const int chunks = d / 8;
  for (int i = tid; i < LA_SLOTS * chunks; i += THREADS) {
    const int m = i / chunks, c = i - m * chunks;
    const int r = m / hg, head = head0 + m % hg;
    const bool valid = r < n_rows && head < p.n_q;
    const __nv_bfloat16* src = valid ? p.q + ((size_t)(first_row + r) * p.n_q + head) * d + c * 8 : p.q;
    cp_async_16(q_tile + m * pitch + c * 8, src, valid ? 16 : 0);
  }
  cp_async_commit();

  // the two slots whose scores and sums this thread holds
  const int m_a = lane >> 2, m_b = m_a + 8;
  const int r_a = m_a / hg, r_b = m_b / hg;
  const bool valid_a = r_a < n_rows && head0 + m_a % hg < p.n_q;
  const bool valid_b = r_b < n_rows && head0 + m_b % hg < p.n_q;
  const int limit_a = valid_a ? min(hi - 1, first_pos + r_a) : -1;      // the last key the slot sees
  const int limit_b = valid_b ? min(hi - 1, first_pos + r_b) : -1;
  const int from_a = valid_a ? max(lo, srb_first_visible(first_pos + r_a, p.window, 0)) : 0;   // the first key it sees
  const int from_b = valid_b ? max(lo, srb_first_visible(first_pos + r_b, p.window, 0)) : 0;
  float max_a = -INFINITY, max_b = -INFINITY, sum_a = 0.f, sum_b = 0.f;
  const int cols_per_warp = vd / WARPS, nt = cols_per_warp / 8;
  float acc[NT_MAX][4];
#pragma unroll
  for (int j = 0; j < NT_MAX; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;

  for (int base = lo & ~(LA_KEYS - 1); base < hi; base += LA_KEYS) {
    if (tid < LA_KEYS) {
      const int key = base + tid;
      long long offset = -1;
      if (key >= lo && key < hi) {
        const int page = p.block_table[(size_t)request * p.table_stride + key / p.page_size];
        if (page < 0 || page >= p.num_pages)
          atomicOr(p.error_word, SRB_FLAG_BAD_PAGE);
        else
          offset = ((long long)page * p.page_size + key % p.page_size) * d;
      }
      key_offset[tid] = offset;
    }
    __syncthreads();
    for (int i = tid; i < LA_KEYS * chunks; i += THREADS) {
      const int key = i / chunks, c = i - key * chunks;
      const long long offset = key_offset[key];
      cp_async_16(k_tile + key * pitch + c * 8, offset < 0 ? p.pool : p.pool + offset + c * 8, offset < 0 ? 0 : 16);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // scores of this warp's keys; even and odd steps along the row add into chains of their own
    float s[ST][4] = {}, s_odd[ST][4] = {};
    const __nv_bfloat16* q_at = q_tile + (lane & 15) * pitch + (lane >> 4) * 8;
    const __nv_bfloat16* k_at = ST == 2
        ? k_tile + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * pitch + ((lane >> 3) & 1) * 8
        : k_tile + (warp * 8 + (lane & 7)) * pitch + ((lane >> 3) & 1) * 8;
    auto step = [&](int kk, float (&into)[ST][4]) {
      unsigned a[4], b0, b1, b2, b3;
      ldmatrix_x4(a[0], a[1], a[2], a[3], q_at + kk);
      if (ST == 2) {
        ldmatrix_x4(b0, b1, b2, b3, k_at + kk);
        mma_bf16(into[0], a, b0, b1);
        mma_bf16(into[ST - 1], a, b2, b3);
      } else {
        ldmatrix_x2(b0, b1, k_at + kk);
        mma_bf16(into[0], a, b0, b1);
      }
    };
    int kk = 0;
#pragma unroll 2
    for (; kk + 32 <= d; kk += 32) {
      step(kk, s);
      step(kk + 16, s_odd);
    }
    if (kk < d) step(kk, s);
#pragma unroll
    for (int t = 0; t < ST; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[t][c] += s_odd[t][c];
    float tile_max_a = -INFINITY, tile_max_b = -INFINITY;
#pragma unroll
    for (int t = 0; t < ST; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = base + warp * KEYS_PER_WARP + t * 8 + (lane & 3) * 2 + (c & 1);
        const bool seen = key >= ((c >> 1) ? from_b : from_a) && key <= ((c >> 1) ? limit_b : limit_a);
        s[t][c] = seen ? s[t][c] * p.scale : -INFINITY;
        if (c >> 1) tile_max_b = fmaxf(tile_max_b, s[t][c]); else tile_max_a = fmaxf(tile_max_a, s[t][c]);
      }
    tile_max_a = fmaxf(tile_max_a, __shfl_xor_sync(0xffffffffu, tile_max_a, 1));
    tile_max_a = fmaxf(tile_max_a, __shfl_xor_sync(0xffffffffu, tile_max_a, 2));
    tile_max_b = fmaxf(tile_max_b, __shfl_xor_sync(0xffffffffu, tile_max_b, 1));
    tile_max_b = fmaxf(tile_max_b, __shfl_xor_sync(0xffffffffu, tile_max_b, 2));
    if ((lane & 3) == 0) {
      warp_max[warp * LA_SLOTS + m_a] = tile_max_a;
      warp_max[warp * LA_SLOTS + m_b] = tile_max_b;
    }
    __syncthreads();
    float new_a = max_a, new_b = max_b;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      new_a = fmaxf(new_a, warp_max[w * LA_SLOTS + m_a]);
      new_b = fmaxf(new_b, warp_max[w * LA_SLOTS + m_b]);
    }
    const float safe_a = new_a == -INFINITY ? 0.f : new_a, safe_b = new_b == -INFINITY ? 0.f : new_b;
    const float corr_a = expf(max_a - safe_a), corr_b = expf(max_b - safe_b);     // exp(-inf) = 0 before the first key
    float part_a = 0.f, part_b = 0.f;
#pragma unroll
    for (int t = 0; t < ST; ++t) {
      const float p0 = expf(s[t][0] - safe_a), p1 = expf(s[t][1] - safe_a);
      const float p2 = expf(s[t][2] - safe_b), p3 = expf(s[t][3] - safe_b);
      part_a += p0 + p1;
      part_b += p2 + p3;
      const int col = warp * KEYS_PER_WARP + t * 8 + (lane & 3) * 2;
      *reinterpret_cast<unsigned*>(p_tile + m_a * (LA_KEYS + LA_PAD) + col) = pack_bf16(p0, p1);
      *reinterpret_cast<unsigned*>(p_tile + m_b * (LA_KEYS + LA_PAD) + col) = pack_bf16(p2, p3);
    }
    part_a += __shfl_xor_sync(0xffffffffu, part_a, 1);
    part_a += __shfl_xor_sync(0xffffffffu, part_a, 2);
    part_b += __shfl_xor_sync(0xffffffffu, part_b, 1);
    part_b += __shfl_xor_sync(0xffffffffu, part_b, 2);
    if ((lane & 3) == 0) {
      warp_sum[warp * LA_SLOTS + m_a] = part_a;
      warp_sum[warp * LA_SLOTS + m_b] = part_b;
    }
#pragma unroll
    for (int j = 0; j < NT_MAX; ++j) {
      acc[j][0] *= corr_a; acc[j][1] *= corr_a;
      acc[j][2] *= corr_b; acc[j][3] *= corr_b;
    }
    max_a = new_a;
    max_b = new_b;
    __syncthreads();
    float tile_sum_a = 0.f, tile_sum_b = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {                     // in warp order: the same sum in every thread
      tile_sum_a += warp_sum[w * LA_SLOTS + m_a];
      tile_sum_b += warp_sum[w * LA_SLOTS + m_b];
    }
    sum_a = sum_a * corr_a + tile_sum_a;
    sum_b = sum_b * corr_b + tile_sum_b;

    // weights times this warp's value columns
    const __nv_bfloat16* p_at = p_tile + (lane & 15) * (LA_KEYS + LA_PAD) + (lane >> 4) * 8;
    const __nv_bfloat16* v_at = k_tile + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + warp * cols_per_warp + (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < LA_KEYS; kk += 16) {
      unsigned a[4];
      ldmatrix_x4(a[0], a[1], a[2], a[3], p_at + kk);
#pragma unroll
      for (int jj = 0; jj < (NT_MAX + 1) / 2; ++jj) {
        if (2 * jj < nt) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, v_at + kk * pitch + jj * 16);
          mma_bf16(acc[2 * jj], a, b0, b1);
          if (2 * jj + 1 < nt) mma_bf16(acc[2 * jj + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();                               // the tile and the weights are consumed
  }

  // results of the two slots of this thread
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const bool valid = half ? valid_b : valid_a;
    if (!valid) continue;
    const int m = half ? m_b : m_a;
    const int row = first_row + m / hg, head = head0 + m % hg;
    const float top = half ? max_b : max_a, sum = half ? sum_b : sum_a;
    if (p.split_size == 0) {
      float factor = 1.0f / sum;
      if (p.sinks) {
        // the sink joins the denominator as one more term
        const float sink = p.sinks[head];
        const float all = fmaxf(top, sink);
        factor = expf(top - all) / (sum * expf(top - all) + expf(sink - all));
      }
      __nv_bfloat16* dst = p.out + ((size_t)row * p.n_q + head) * vd + warp * cols_per_warp + (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < NT_MAX; ++j)
        if (j < nt)
          *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(acc[j][half * 2] * factor, acc[j][half * 2 + 1] * factor);
    } else {
      const size_t slot = ((size_t)row * p.n_q + head) * p.max_splits + split;
      float* dst = p.part_acc + slot * vd + warp * cols_per_warp + (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < NT_MAX; ++j)
        if (j < nt) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(acc[j][half * 2], acc[j][half * 2 + 1]);
      if (warp == 0 && (lane & 3) == 0) {
        p.part_ml[slot * 2] = top;
        p.part_ml[slot * 2 + 1] = sum;
      }
    }
  }
}

extern "C" int srb_latent_attention_supports(int d, int vd) {
  return d > 0 && d % 16 == 0 && vd > 0 && vd % 32 == 0 && vd <= 512 && vd <= d;
}

template <int NT_MAX, int WARPS>
static int launch_latent_attention(const LaParams& p, dim3 grid, size_t smem, cudaStream_t s) {
  if (smem > 48 * 1024)
    SRB_CUDA_CALL(cudaFuncSetAttribute(latent_attention_kernel<NT_MAX, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  SRB_CUDA_CALL(srb_launch(latent_attention_kernel<NT_MAX, WARPS>, grid, dim3(WARPS * 32), smem, s, p));
  SRB_LAUNCH_CHECK("latent_attention");
  return SRB_OK;
}

// tiles null: rows are split rows (one block per row, head group and split; partial results merged by the generic
// kernel's merge, scratch as there).  tiles given: prompt portions, unsplit (split_size is taken as 0).
// `window` > 0: a row sees itself and the window - 1 keys before it.
extern "C" int srb_latent_attention_masked(const void* q, const void* pool, void* out, float* part_acc, float* part_ml,
                                           const int* positions, const int* row_request, const int* block_table, int table_stride,
                                           int rows, int n_q, int d, int vd, int page_size, int num_pages, int split_size,
                                           int max_splits, const int* tiles, int num_tiles, float scale, const float* sinks,
                                           int window, int* error_word, void* stream) {
  if (window < 0) SRB_FAIL("latent_attention: a window of %d keys", window);
  if (!srb_latent_attention_supports(d, vd)) SRB_FAIL("latent_attention: rows of %d entries with values of %d are not taken", d, vd);
  if (n_q <= 0 || page_size <= 0 || num_pages <= 0 || table_stride <= 0) SRB_FAIL("latent_attention: sizes must be positive");
  LaParams p;
  p.q = (const __nv_bfloat16*)q; p.pool = (const __nv_bfloat16*)pool; p.out = (__nv_bfloat16*)out;
  p.part_acc = part_acc; p.part_ml = part_ml; p.positions = positions; p.row_request = row_request;
  p.block_table = block_table; p.tiles = tiles; p.sinks = sinks; p.error_word = error_word;
  p.table_stride = table_stride; p.n_q = n_q; p.d = d; p.vd = vd; p.page_size = page_size; p.num_pages = num_pages;
  p.scale = scale; p.window = window;
  p.heads_per_block = n_q < LA_SLOTS ? n_q : LA_SLOTS;
  const int groups = (n_q + p.heads_per_block - 1) / p.heads_per_block;
  dim3 grid;
  if (tiles) {
    if (num_tiles <= 0) return SRB_OK;
    p.split_size = 0; p.max_splits = 1;
    p.rows_per_block = LA_SLOTS / p.heads_per_block;
    p.units_per_tile = (64 + p.rows_per_block - 1) / p.rows_per_block;
    grid = dim3(1, groups, (unsigned)num_tiles * p.units_per_tile);
  } else {
    if (rows <= 0) return SRB_OK;
    if (split_size <= 0 || split_size % LA_KEYS || max_splits <= 0 || !part_acc || !part_ml)
      SRB_FAIL("latent_attention: split rows need a split size that is a multiple of %d, and scratch memory", LA_KEYS);
    p.split_size = split_size; p.max_splits = max_splits;
    p.rows_per_block = 1; p.units_per_tile = 1;
    grid = dim3(max_splits, groups, rows);
  }
  if (grid.y > 65535 || grid.z > 65535) SRB_FAIL("latent_attention: too many blocks for one launch");
  const size_t pitch = d + LA_PAD;
  const int warps = vd % 64 == 0 ? 8 : 4;                 // every warp gets whole 8-column tiles of the values
  const size_t smem = (LA_KEYS + LA_SLOTS) * pitch * 2 + LA_SLOTS * (LA_KEYS + LA_PAD) * 2 + 2 * warps * LA_SLOTS * 4 + LA_KEYS * 8;
  if (smem > 227 * 1024) SRB_FAIL("latent_attention: %zu bytes of shared memory exceed 232448", smem);
  cudaStream_t s = (cudaStream_t)stream;
  const int nt = vd / (8 * warps);
  int status;
  if (warps == 8) status = nt <= 4 ? launch_latent_attention<4, 8>(p, grid, smem, s) : launch_latent_attention<8, 8>(p, grid, smem, s);
  else if (nt <= 4) status = launch_latent_attention<4, 4>(p, grid, smem, s);
  else if (nt <= 8) status = launch_latent_attention<8, 4>(p, grid, smem, s);
  else status = launch_latent_attention<16, 4>(p, grid, smem, s);
  if (status != SRB_OK || tiles) return status;
  AttnParams m = {};
  m.positions = positions; m.n_q = n_q; m.n_kv = 1; m.head_dim = d; m.window = window; m.split_size = split_size;
  m.max_splits = max_splits; m.error_word = error_word; m.sinks = sinks; m.value_dim = vd;
  attention_combine_kernel<__nv_bfloat16><<<dim3(rows, n_q), 64, 0, s>>>(part_acc, part_ml, (__nv_bfloat16*)out, m);
  SRB_LAUNCH_CHECK("attention_combine");
  return SRB_OK;
}

extern "C" int srb_latent_attention(const void* q, const void* pool, void* out, float* part_acc, float* part_ml,
                                    const int* positions, const int* row_request, const int* block_table, int table_stride,
                                    int rows, int n_q, int d, int vd, int page_size, int num_pages, int split_size,
                                    int max_splits, const int* tiles, int num_tiles, float scale, const float* sinks,
                                    int* error_word, void* stream) {
  return srb_latent_attention_masked(q, pool, out, part_acc, part_ml, positions, row_request, block_table, table_stride, rows,
                                     n_q, d, vd, page_size, num_pages, split_size, max_splits, tiles, num_tiles, scale, sinks, 0,
                                     error_word, stream);
}
