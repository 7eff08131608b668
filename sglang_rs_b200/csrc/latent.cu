// Kernels of attention through latents: queries and keys/values are projected down to narrow rows
// ("latents"), normalised, and projected up again head by head.  Only the key/value latent and one
// rotated key part that all heads share are kept per token, in one page pool whose rows are
// [latent | rotated part].
//
//   srb_latent_prepare   per row: RMS norm of the query latent -> its own tensor; RMS norm of the
//                        key/value latent and rotation of the shared key part -> the row's cache slot
//   srb_rope_slice       rotates a slice of every head of a [rows, heads, *] tensor into another tensor
//   srb_head_linear      out[r, h, :] = W_h x[r, h, :] for every head h (one weight matrix per head), with
//                        an optional sigmoid gate per (row, head) or per (row, head, entry) on the result
//
// Norms, angles and the rotation are 32-bit; T is the storage type (float or bfloat16).  The rotation
// pairs entry i with entry i + dims/2 of the slice ("rotate half") or, with `interleaved`, entry 2i with entry 2i + 1:
// (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * inv_freq[i], cosines and sines times `magnitude`;
// entries of the slice behind `rotary_dim` pass unchanged.
#include "common.cuh"
#include "tile_mma.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, size_t pitch, int q_rank, int kv_rank, int rot_dim,
                                      const float* __restrict__ q_weight, const float* __restrict__ kv_weight,
                                      float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                      int rotary_dim, T* __restrict__ q_latent, T* __restrict__ pool,
                                      const int* __restrict__ slots, long long pool_rows, int* error_word,
                                      int interleaved, float magnitude) {
  __shared__ float scratch[33];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const T* src = proj + (size_t)row * pitch;
  // the query latent
  if (q_rank > 0) {
    float partial = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
      const float v = srb_to_float(src[i]);
      partial += v * v;
    }
    const float inv = 1.0f / sqrtf(srb_block_sum(partial, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      q_latent[(size_t)row * q_rank + i] = srb_from_float<T>(srb_to_float(src[i]) * inv * q_weight[i]);
  }
  if (!slots) return;
  const long long slot = slots[row];
  if (slot < 0 || slot >= pool_rows) {
    if (threadIdx.x == 0) atomicOr(error_word, SRB_FLAG_BAD_SLOT);
    return;
  }
  T* dst = pool + (size_t)slot * (kv_rank + rot_dim);
  const T* kv = src + q_rank;
  float partial = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float v = srb_to_float(kv[i]);
    partial += v * v;
  }
  const float inv = 1.0f / sqrtf(srb_block_sum(partial, scratch) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    dst[i] = srb_from_float<T>(srb_to_float(kv[i]) * inv * kv_weight[i]);
  // the rotated part that all heads share: not normed
  const T* shared_key = kv + kv_rank;
  const int half = rotary_dim / 2;
  const float position = (float)positions[row];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sine, cosine;
    sincosf(position * inv_freq[i], &sine, &cosine);
    sine *= magnitude; cosine *= magnitude;
    const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
    const float u = srb_to_float(shared_key[ia]), v = srb_to_float(shared_key[ib]);
    dst[kv_rank + ia] = srb_from_float<T>(u * cosine - v * sine);
    dst[kv_rank + ib] = srb_from_float<T>(v * cosine + u * sine);
  }
  for (int i = rotary_dim + threadIdx.x; i < rot_dim; i += blockDim.x) dst[kv_rank + i] = shared_key[i];
}

// proj: [rows, pitch] with the query latent in columns [0, q_rank), the key/value latent behind it and the
// shared key part behind that.  pool: [pool_rows, kv_rank + rot_dim]; slots null: nothing is stored.
// `interleaved`: the rotation pairs entry 2i with entry 2i + 1 instead of i with i + dims/2; `magnitude` multiplies
// every cosine and sine.
extern "C" int srb_latent_prepare_ex(const void* proj, long long pitch, int rows, int q_rank, int kv_rank, int rot_dim,
                                     const float* q_weight, const float* kv_weight, float eps, const int* positions,
                                     const float* inv_freq, int rotary_dim, void* q_latent, void* pool, const int* slots,
                                     long long pool_rows, int* error_word, int dtype, int interleaved, float magnitude,
                                     void* stream) {
  if (rows <= 0) return SRB_OK;
  if (q_rank < 0 || kv_rank <= 0 || rot_dim < 0) SRB_FAIL("latent_prepare: sizes %d, %d, %d do not describe latents", q_rank, kv_rank, rot_dim);
  if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > rot_dim)
    SRB_FAIL("latent_prepare: %d rotated entries must be even and at most the shared key part (%d)", rotary_dim, rot_dim);
  if (pitch < (long long)q_rank + kv_rank + rot_dim) SRB_FAIL("latent_prepare: rows of the projection are too short");
  if (rotary_dim > 0 && (!inv_freq || !positions)) SRB_FAIL("latent_prepare: a rotation without positions or frequencies");
  if (!(eps >= 0.f)) SRB_FAIL("latent_prepare: eps must be finite and non-negative");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(latent_prepare_kernel<float>, dim3(rows), dim3(128), 0, s, (const float*)proj, (size_t)pitch,
                             q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, positions, inv_freq, rotary_dim,
                             (float*)q_latent, (float*)pool, slots, pool_rows, error_word, interleaved, magnitude));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, s,
                             (const __nv_bfloat16*)proj, (size_t)pitch, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps,
                             positions, inv_freq, rotary_dim, (__nv_bfloat16*)q_latent, (__nv_bfloat16*)pool, slots,
                             pool_rows, error_word, interleaved, magnitude));
  else
    SRB_FAIL("latent_prepare: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("latent_prepare");
  return SRB_OK;
}

extern "C" int srb_latent_prepare(const void* proj, long long pitch, int rows, int q_rank, int kv_rank, int rot_dim,
                                  const float* q_weight, const float* kv_weight, float eps, const int* positions,
                                  const float* inv_freq, int rotary_dim, void* q_latent, void* pool, const int* slots,
                                  long long pool_rows, int* error_word, int dtype, void* stream) {
  return srb_latent_prepare_ex(proj, pitch, rows, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, positions, inv_freq,
                               rotary_dim, q_latent, pool, slots, pool_rows, error_word, dtype, 0, 1.0f, stream);
}

// out[r, h, out_offset + i] = rotated(x[r, h, in_offset + i]) for i < width; entries from rotary_dim on are copied.
template <typename T>
__global__ void rope_slice_kernel(const T* __restrict__ x, size_t x_row, size_t x_head, int in_offset,
                                  T* __restrict__ out, size_t out_row, size_t out_head, int out_offset, int heads,
                                  int width, int rotary_dim, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int interleaved, float magnitude) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const int half = rotary_dim / 2;
  const float position = (float)positions[row];
  const int pairs_and_rest = half + (width - rotary_dim);
  for (int item = threadIdx.x; item < heads * pairs_and_rest; item += blockDim.x) {
    const int head = item / pairs_and_rest, i = item % pairs_and_rest;
    const T* src = x + (size_t)row * x_row + (size_t)head * x_head + in_offset;
    T* dst = out + (size_t)row * out_row + (size_t)head * out_head + out_offset;
    if (i < half) {
      float sine, cosine;
      sincosf(position * inv_freq[i], &sine, &cosine);
      sine *= magnitude; cosine *= magnitude;
      const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
      const float u = srb_to_float(src[ia]), v = srb_to_float(src[ib]);
      dst[ia] = srb_from_float<T>(u * cosine - v * sine);
      dst[ib] = srb_from_float<T>(v * cosine + u * sine);
    } else {
      dst[rotary_dim + i - half] = src[rotary_dim + i - half];
    }
  }
}

extern "C" int srb_rope_slice_ex(const void* x, long long x_row, long long x_head, int in_offset, void* out,
                                 long long out_row, long long out_head, int out_offset, int rows, int heads, int width,
                                 int rotary_dim, const int* positions, const float* inv_freq, int dtype, int interleaved,
                                 float magnitude, void* stream) {
  if (rows <= 0 || heads <= 0 || width <= 0) return SRB_OK;
  if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > width)
    SRB_FAIL("rope_slice: %d rotated entries must be even and at most the slice (%d)", rotary_dim, width);
  if (rotary_dim > 0 && (!inv_freq || !positions)) SRB_FAIL("rope_slice: a rotation without positions or frequencies");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(rope_slice_kernel<float>, dim3(rows), dim3(256), 0, s, (const float*)x, (size_t)x_row,
                             (size_t)x_head, in_offset, (float*)out, (size_t)out_row, (size_t)out_head, out_offset, heads,
                             width, rotary_dim, positions, inv_freq, interleaved, magnitude));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(rope_slice_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, (const __nv_bfloat16*)x,
                             (size_t)x_row, (size_t)x_head, in_offset, (__nv_bfloat16*)out, (size_t)out_row,
                             (size_t)out_head, out_offset, heads, width, rotary_dim, positions, inv_freq, interleaved,
                             magnitude));
  else
    SRB_FAIL("rope_slice: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("rope_slice");
  return SRB_OK;
}

extern "C" int srb_rope_slice(const void* x, long long x_row, long long x_head, int in_offset, void* out,
                              long long out_row, long long out_head, int out_offset, int rows, int heads, int width,
                              int rotary_dim, const int* positions, const float* inv_freq, int dtype, void* stream) {
  return srb_rope_slice_ex(x, x_row, x_head, in_offset, out, out_row, out_head, out_offset, rows, heads, width, rotary_dim,
                           positions, inv_freq, dtype, 0, 1.0f, stream);
}

// ---- one matrix per head ------------------------------------------------------------------------------
// out[r, h, o] = sum_i x[r, h, i] * w[h, o, i], accumulated in 32-bit over i in index order by one thread, so
// a row's result does not depend on the other rows.  Tiles of 64 rows x 64 outputs, 16 inputs at a time.
#define HL_TILE 64
#define HL_K 16

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, size_t x_row, size_t x_head, const T* __restrict__ w, T* __restrict__ out,
                   size_t out_row, size_t out_head, int rows, int n_in, int n_out, const T* __restrict__ gate,
                   size_t gate_row, int gate_head, int gate_col) {
  __shared__ float x_tile[HL_K][HL_TILE + 4];
  __shared__ float w_tile[HL_K][HL_TILE + 4];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int head = blockIdx.z;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * HL_TILE, col0 = blockIdx.x * HL_TILE;
  const T* xh = x + (size_t)head * x_head;
  const T* wh = w + (size_t)head * n_out * n_in;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < n_in; k0 += HL_K) {
    for (int i = threadIdx.x; i < HL_TILE * HL_K; i += 256) {
      const int r = i / HL_K, kk = i % HL_K;
      const int gk = k0 + kk;
      x_tile[kk][r] = (row0 + r < rows && gk < n_in) ? srb_to_float(xh[(size_t)(row0 + r) * x_row + gk]) : 0.f;
      w_tile[kk][r] = (col0 + r < n_out && gk < n_in) ? srb_to_float(wh[(size_t)(col0 + r) * n_in + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_K; ++kk) {
      float xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = x_tile[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_tile[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= n_out) continue;
      float g = 1.f;
      if (gate) g = 1.0f / (1.0f + expf(-srb_to_float(gate[(size_t)r * gate_row + (size_t)head * gate_head + (size_t)c * gate_col])));
      out[(size_t)r * out_row + (size_t)head * out_head + c] = srb_from_float<T>(acc[i][j] * g);
    }
  }
}

// The same on the tensor cores (bfloat16): tile_mma.cuh.
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, size_t x_row, size_t x_head, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ out, size_t out_row, size_t out_head, int rows, int n_in, int n_out,
                       const __nv_bfloat16* __restrict__ gate, size_t gate_row, int gate_head, int gate_col) {
  __shared__ __align__(16) TileMmaSmem s;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int head = blockIdx.z, row0 = blockIdx.y * TM_TILE, col0 = blockIdx.x * TM_TILE;
  const int t = threadIdx.x;
  if (t < TM_TILE) s.a_row[t] = row0 + t < rows ? x + (size_t)(row0 + t) * x_row + (size_t)head * x_head : nullptr;
  __syncthreads();
  const __nv_bfloat16* const bases[1] = {w + (size_t)head * n_out * n_in + (size_t)col0 * n_in};
  float acc[1][2][4][4];
  tile_mma_64x64<1>(s, bases, n_out - col0, n_in, acc);
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {
      const int r = row0 + tile_mma_row(i, c2 * 2);
      if (r >= rows) continue;
      float g = 1.f;
      if (gate && !gate_col) g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * gate_row + (size_t)head * gate_head])));
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c1 = 0; c1 < 2; ++c1) {
          const int col = col0 + tile_mma_col(j, c1);
          if (col >= n_out) continue;
          if (gate && gate_col)
            g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * gate_row + (size_t)head * gate_head + (size_t)col * gate_col])));
          out[(size_t)r * out_row + (size_t)head * out_head + col] = __float2bfloat16_rn(acc[0][i][j][c2 * 2 + c1] * g);
        }
    }
}

// Tiles of 128 rows with operands through a ring of asynchronous copies, for rows on 16-byte boundaries.
__global__ void __launch_bounds__(256)
head_linear_async_kernel(const __nv_bfloat16* __restrict__ x, size_t x_row, size_t x_head, const __nv_bfloat16* __restrict__ w,
                         __nv_bfloat16* __restrict__ out, size_t out_row, size_t out_head, int rows, int n_in, int n_out,
                         const __nv_bfloat16* __restrict__ gate, size_t gate_row, int gate_head, int gate_col) {
  extern __shared__ __align__(16) unsigned char hl_smem[];
  TileAsyncSmem<1>& s = *reinterpret_cast<TileAsyncSmem<1>*>(hl_smem);
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int head = blockIdx.z, row0 = blockIdx.y * TA_ROWS, col0 = blockIdx.x * TA_COLS;
  const int t = threadIdx.x;
  if (t < TA_ROWS) s.a_row[t] = row0 + t < rows ? x + (size_t)(row0 + t) * x_row + (size_t)head * x_head : nullptr;
  __syncthreads();
  const __nv_bfloat16* const bases[1] = {w + (size_t)head * n_out * n_in + (size_t)col0 * n_in};
  float acc[1][2][4][4];
  tile_mma_128x64_async<1>(s, bases, n_out - col0, rows - row0, n_in, acc);
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {
      const int r = row0 + tile_async_row(i, c2 * 2);
      if (r >= rows) continue;
      float g = 1.f;
      if (gate && !gate_col) g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * gate_row + (size_t)head * gate_head])));
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c1 = 0; c1 < 2; ++c1) {
          const int col = col0 + tile_async_col(j, c1);
          if (col >= n_out) continue;
          if (gate && gate_col)
            g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * gate_row + (size_t)head * gate_head + (size_t)col * gate_col])));
          out[(size_t)r * out_row + (size_t)head * out_head + col] = __float2bfloat16_rn(acc[0][i][j][c2 * 2 + c1] * g);
        }
    }
}

// x: rows x_row elements apart, heads x_head apart; w: [heads, n_out, n_in]; out likewise by out_row / out_head.
// gate (optional): gate[r * gate_row + h * gate_head + o * gate_col] is a logit; the result out[r, h, o] is multiplied by
// its sigmoid (gate_head 1, gate_col 0: one gate per head; gate_head n_out, gate_col 1: one per entry).
extern "C" int srb_head_linear_ex(const void* x, long long x_row, long long x_head, const void* w, void* out,
                                  long long out_row, long long out_head, int rows, int heads, int n_in, int n_out,
                                  const void* gate, long long gate_row, int gate_head, int gate_col, int dtype, void* stream) {
  if (rows <= 0 || heads <= 0 || n_out <= 0) return SRB_OK;
  if (n_in <= 0) SRB_FAIL("head_linear: inner size %d must be positive", n_in);
  dim3 grid((n_out + HL_TILE - 1) / HL_TILE, (rows + HL_TILE - 1) / HL_TILE, heads);
  if (grid.y > 65535 || grid.z > 65535) SRB_FAIL("head_linear: %d rows or %d heads exceed one launch", rows, heads);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(head_linear_kernel<float>, grid, dim3(256), 0, s, (const float*)x, (size_t)x_row,
                             (size_t)x_head, (const float*)w, (float*)out, (size_t)out_row, (size_t)out_head, rows, n_in,
                             n_out, (const float*)gate, (size_t)gate_row, gate_head, gate_col));
  else if (dtype == SRB_DTYPE_BF16 && n_in % 8 == 0 && x_row % 8 == 0 && x_head % 8 == 0 &&
           (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
    grid.y = (rows + TA_ROWS - 1) / TA_ROWS;
    SRB_CUDA_CALL(cudaFuncSetAttribute(head_linear_async_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)sizeof(TileAsyncSmem<1>)));
    SRB_CUDA_CALL(srb_launch(head_linear_async_kernel, grid, dim3(256), sizeof(TileAsyncSmem<1>), s, (const __nv_bfloat16*)x,
                             (size_t)x_row, (size_t)x_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (size_t)out_row,
                             (size_t)out_head, rows, n_in, n_out, (const __nv_bfloat16*)gate, (size_t)gate_row, gate_head, gate_col));
  } else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(head_linear_mma_kernel, grid, dim3(128), 0, s, (const __nv_bfloat16*)x,
                             (size_t)x_row, (size_t)x_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (size_t)out_row,
                             (size_t)out_head, rows, n_in, n_out, (const __nv_bfloat16*)gate, (size_t)gate_row, gate_head, gate_col));
  else
    SRB_FAIL("head_linear: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("head_linear");
  return SRB_OK;
}

extern "C" int srb_head_linear(const void* x, long long x_row, long long x_head, const void* w, void* out,
                               long long out_row, long long out_head, int rows, int heads, int n_in, int n_out,
                               const void* gate, long long gate_row, int dtype, void* stream) {
  return srb_head_linear_ex(x, x_row, x_head, w, out, out_row, out_head, rows, heads, n_in, n_out, gate, gate_row, 1, 0, dtype,
                            stream);
}
