// Linear attention with one fixed decay per head ("lightning attention") over a state of fixed size per request.
//
// Per head, with q_t, k_t (dim entries) and v_t (vdim entries) the SiLU of the row's projections:
//     S_t = decay * S_(t-1) + k_t v_t^T          S: [dim, vdim] 32-bit floats, zero before a sequence's first token
//     o_t = S_t^T q_t
// The rows of a request in one step (a prompt portion, or one decoded token) are walked in chunks of LA_CHUNK
// tokens.  Inside a chunk that starts from state S and holds tokens 0 .. n-1:
//     A[t, j] = (q_t . k_j) decay^(t - j)                              for j <= t
//     o_t     = sum_(j <= t) A[t, j] v_j + decay^(t+1) S^T q_t
//     S      <- decay^n S + sum_j decay^(n-1-j) k_j v_j^T
// Powers of the decay are products of 32-bit floats, never quotients, so nothing overflows however small the
// decay is.  Scores, weights, sums and the state are 32-bit in both dtypes; T is the type of the projections.
//
//   srb_lightning_scan       the recurrence: reads q, k, v from the rows of the stacked projection, updates the
//                            requests' states in place, writes o as float [rows, heads * vdim]
//   srb_lightning_gate_norm  out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g), over all heads of a row together
#include "common.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define LA_CHUNK 32
#define LA_THREADS 256
#define LA_SLICE 64          // value columns that one block owns at most

struct LightningArgs {
  const void* proj;          // T [rows, pitch]
  long long pitch;
  int q_offset, k_offset, v_offset;
  const int* cu_rows;        // [requests + 1]
  const int* positions;      // [rows]
  const int* state_slots;    // [requests]
  float* state;              // [slots, heads, dim, vdim]
  const float* decay;        // [heads]
  float* out;                // [rows, heads * vdim]
  int heads, dim, vdim, slices, slice_width, read_only;
};

__device__ __forceinline__ float la_silu(float x) { return x / (1.0f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(LA_THREADS) lightning_scan_kernel(LightningArgs a) {
  extern __shared__ float smem[];
  srb_launch_dependents();
  const int head = blockIdx.x / a.slices, slice = blockIdx.x % a.slices;
  const int request = blockIdx.y;
  const int dim = a.dim, c0 = slice * a.slice_width;
  const int vs = min(a.slice_width, a.vdim - c0);
  const int qk_pitch = dim + 1;
  float* S = smem;                                  // [dim][slice_width]
  float* Q = S + dim * a.slice_width;               // [LA_CHUNK][dim + 1]
  float* K = Q + LA_CHUNK * qk_pitch;               // [LA_CHUNK][dim + 1]
  float* V = K + LA_CHUNK * qk_pitch;               // [LA_CHUNK][slice_width]
  float* A = V + LA_CHUNK * a.slice_width;          // [LA_CHUNK][LA_CHUNK + 1]
  float* power = A + LA_CHUNK * (LA_CHUNK + 1);     // [LA_CHUNK + 1]: decay^n
  if (vs <= 0) return;
  if (threadIdx.x == 0) {
    const float decay = a.decay[head];
    float p = 1.f;
    for (int n = 0; n <= LA_CHUNK; ++n) {
      power[n] = p;
      p *= decay;
    }
  }
  srb_grid_dependency_wait();
  const int row_begin = a.cu_rows[request], row_end = a.cu_rows[request + 1];
  if (row_end <= row_begin) return;
  float* state = a.state + (((size_t)a.state_slots[request] * a.heads + head) * dim) * a.vdim + c0;
  const bool fresh = a.positions[row_begin] == 0;    // a sequence's first token starts from the zero state
  for (int e = threadIdx.x; e < dim * vs; e += LA_THREADS) {
    const int d = e / vs, c = e - d * vs;
    S[d * a.slice_width + c] = fresh ? 0.f : state[(size_t)d * a.vdim + c];
  }
  const T* proj = reinterpret_cast<const T*>(a.proj);
  const int out_pitch = a.heads * a.vdim;
  for (int row0 = row_begin; row0 < row_end; row0 += LA_CHUNK) {
    const int n = min(LA_CHUNK, row_end - row0);
    __syncthreads();                                 // the chunk before is done with Q, K, V, A; S is updated
    for (int e = threadIdx.x; e < n * dim; e += LA_THREADS) {
      const int t = e / dim, d = e - t * dim;
      const T* row = proj + (size_t)(row0 + t) * a.pitch + (size_t)head * dim + d;
      Q[t * qk_pitch + d] = la_silu(srb_to_float(row[a.q_offset]));
      K[t * qk_pitch + d] = la_silu(srb_to_float(row[a.k_offset]));
    }
    for (int e = threadIdx.x; e < n * vs; e += LA_THREADS) {
      const int t = e / vs, c = e - t * vs;
      V[t * a.slice_width + c] =
          la_silu(srb_to_float(proj[(size_t)(row0 + t) * a.pitch + a.v_offset + (size_t)head * a.vdim + c0 + c]));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * LA_CHUNK; e += LA_THREADS) {
      const int t = e / LA_CHUNK, j = e - t * LA_CHUNK;
      float s = 0.f;
      if (j <= t) {
        const float* q = Q + t * qk_pitch;
        const float* k = K + j * qk_pitch;
        for (int d = 0; d < dim; ++d) s = fmaf(q[d], k[d], s);
        s *= power[t - j];
      }
      A[t * (LA_CHUNK + 1) + j] = s;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * vs; e += LA_THREADS) {
      const int t = e / vs, c = e - t * vs;
      float inside = 0.f, carried = 0.f;
      for (int j = 0; j <= t; ++j) inside = fmaf(A[t * (LA_CHUNK + 1) + j], V[j * a.slice_width + c], inside);
      const float* q = Q + t * qk_pitch;
      for (int d = 0; d < dim; ++d) carried = fmaf(q[d], S[d * a.slice_width + c], carried);
      a.out[(size_t)(row0 + t) * out_pitch + (size_t)head * a.vdim + c0 + c] = fmaf(power[t + 1], carried, inside);
    }
    __syncthreads();                                 // every read of the old state is done
    for (int e = threadIdx.x; e < dim * vs; e += LA_THREADS) {
      const int d = e / vs, c = e - d * vs;
      float add = 0.f;
      for (int j = 0; j < n; ++j) add = fmaf(power[n - 1 - j] * K[j * qk_pitch + d], V[j * a.slice_width + c], add);
      S[d * a.slice_width + c] = fmaf(power[n], S[d * a.slice_width + c], add);
    }
  }
  __syncthreads();
  if (a.read_only) return;
  for (int e = threadIdx.x; e < dim * vs; e += LA_THREADS) {
    const int d = e / vs, c = e - d * vs;
    state[(size_t)d * a.vdim + c] = S[d * a.slice_width + c];
  }
}

extern "C" int srb_lightning_scan(const void* proj, long long pitch, int q_offset, int k_offset, int v_offset,
                                  const int* cu_rows, const int* positions, const int* state_slots, float* state,
                                  const float* decay, float* out, int requests, int heads, int dim, int vdim,
                                  int read_only, int dtype, void* stream) {
  if (requests <= 0) return SRB_OK;
  if (heads <= 0 || dim <= 0 || vdim <= 0) SRB_FAIL("lightning_scan: heads, dim and vdim must be positive");
  if (requests > 65535) SRB_FAIL("lightning_scan: %d requests exceed one launch", requests);
  LightningArgs a;
  a.proj = proj; a.pitch = pitch; a.q_offset = q_offset; a.k_offset = k_offset; a.v_offset = v_offset;
  a.cu_rows = cu_rows; a.positions = positions; a.state_slots = state_slots; a.state = state; a.decay = decay; a.out = out;
  a.heads = heads; a.dim = dim; a.vdim = vdim; a.read_only = read_only;
  a.slices = (vdim + LA_SLICE - 1) / LA_SLICE;
  a.slice_width = (vdim + a.slices - 1) / a.slices;
  const size_t smem = ((size_t)dim * a.slice_width + 2 * (size_t)LA_CHUNK * (dim + 1) + (size_t)LA_CHUNK * a.slice_width +
                       (size_t)LA_CHUNK * (LA_CHUNK + 1) + LA_CHUNK + 1) * sizeof(float);
  if (smem > 220 * 1024) SRB_FAIL("lightning_scan: a state of %d x %d per head does not fit a block's shared memory", dim, vdim);
  dim3 grid(heads * a.slices, requests);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32) {
    SRB_CUDA_CALL(cudaFuncSetAttribute(lightning_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(lightning_scan_kernel<float>, grid, dim3(LA_THREADS), smem, s, a));
  } else if (dtype == SRB_DTYPE_BF16) {
    SRB_CUDA_CALL(cudaFuncSetAttribute(lightning_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(lightning_scan_kernel<__nv_bfloat16>, grid, dim3(LA_THREADS), smem, s, a));
  } else {
    SRB_FAIL("lightning_scan: unknown dtype %d", dtype);
  }
  SRB_LAUNCH_CHECK("lightning_scan");
  return SRB_OK;
}

// Steps of decoded tokens (every request brings one row): S <- decay S + k v^T and o = S^T q in one pass over the
// state.  A block owns 32 value columns of one (request, head); its eight warps share the rows of the state (dim / 8
// each, all of a thread's loads in flight together) and add their parts of o through shared memory in warp order.
#define LD_COLUMNS 32
#define LD_WARPS 8
template <typename T>
__global__ void __launch_bounds__(LD_COLUMNS * LD_WARPS) lightning_decode_kernel(LightningArgs a) {
  extern __shared__ float ld_smem[];                 // q [dim], k [dim], partial results [LD_WARPS][LD_COLUMNS]
  srb_launch_dependents();
  const int head = blockIdx.x, request = blockIdx.y, c0 = blockIdx.z * LD_COLUMNS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dim = a.dim;
  float* q = ld_smem;
  float* k = q + dim;
  float* part = k + dim;
  const float decay = a.decay[head];
  srb_grid_dependency_wait();
  const int row = a.cu_rows[request];
  if (a.cu_rows[request + 1] != row + 1) return;      // (the launcher is only used for steps of single rows)
  const T* proj = reinterpret_cast<const T*>(a.proj) + (size_t)row * a.pitch;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    q[d] = la_silu(srb_to_float(proj[a.q_offset + head * dim + d]));
    k[d] = la_silu(srb_to_float(proj[a.k_offset + head * dim + d]));
  }
  const int c = c0 + lane;
  const bool live = c < a.vdim;
  const float v = live ? la_silu(srb_to_float(proj[a.v_offset + head * a.vdim + c])) : 0.f;
  const bool fresh = a.positions[row] == 0;           // a sequence's first token starts from the zero state
  float* state = a.state + (((size_t)a.state_slots[request] * a.heads + head) * dim) * a.vdim + c;
  __syncthreads();
  const int per_warp = (dim + LD_WARPS - 1) / LD_WARPS;
  const int d_begin = warp * per_warp, d_end = min(dim, d_begin + per_warp);
  float acc = 0.f;
  for (int d0 = d_begin; d0 < d_end; d0 += 8) {
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = (live && !fresh && d0 + i < d_end) ? state[(size_t)(d0 + i) * a.vdim] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (d0 + i < d_end) {
        const float next = fmaf(decay, s[i], k[d0 + i] * v);
        acc = fmaf(q[d0 + i], next, acc);
        if (live && !a.read_only) state[(size_t)(d0 + i) * a.vdim] = next;
      }
    }
  }
  part[warp * LD_COLUMNS + lane] = acc;
  __syncthreads();
  if (warp == 0 && live) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < LD_WARPS; ++w) total += part[w * LD_COLUMNS + lane];
    a.out[(size_t)row * a.heads * a.vdim + (size_t)head * a.vdim + c] = total;
  }
}

// `single_rows` of srb_lightning_scan_step: every request of the step brings exactly one row.
static int launch_lightning_decode(const LightningArgs& a, int requests, int dtype, cudaStream_t s) {
  dim3 grid(a.heads, requests, (a.vdim + LD_COLUMNS - 1) / LD_COLUMNS);
  if (grid.z > 65535 || a.heads > 65535) SRB_FAIL("lightning_scan: %d heads or %d value columns exceed one launch", a.heads, a.vdim);
  const size_t smem = ((size_t)2 * a.dim + LD_WARPS * LD_COLUMNS) * sizeof(float);
  if (smem > 48 * 1024) SRB_FAIL("lightning_scan: heads of %d entries do not fit", a.dim);
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(lightning_decode_kernel<float>, grid, dim3(LD_COLUMNS * LD_WARPS), smem, s, a));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(lightning_decode_kernel<__nv_bfloat16>, grid, dim3(LD_COLUMNS * LD_WARPS), smem, s, a));
  else
    SRB_FAIL("lightning_scan: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("lightning_decode");
  return SRB_OK;
}

// srb_lightning_scan for a step in which every request brings exactly one row (decoded tokens; the caller knows it
// from the step's shape, so nothing is decided from device memory).
extern "C" int srb_lightning_scan_single(const void* proj, long long pitch, int q_offset, int k_offset, int v_offset,
                                         const int* cu_rows, const int* positions, const int* state_slots, float* state,
                                         const float* decay, float* out, int requests, int heads, int dim, int vdim,
                                         int read_only, int dtype, void* stream) {
  if (requests <= 0) return SRB_OK;
  if (heads <= 0 || dim <= 0 || vdim <= 0) SRB_FAIL("lightning_scan: heads, dim and vdim must be positive");
  if (requests > 65535) SRB_FAIL("lightning_scan: %d requests exceed one launch", requests);
  LightningArgs a;
  a.proj = proj; a.pitch = pitch; a.q_offset = q_offset; a.k_offset = k_offset; a.v_offset = v_offset;
  a.cu_rows = cu_rows; a.positions = positions; a.state_slots = state_slots; a.state = state; a.decay = decay; a.out = out;
  a.heads = heads; a.dim = dim; a.vdim = vdim; a.read_only = read_only; a.slices = 1; a.slice_width = vdim;
  return launch_lightning_decode(a, requests, dtype, (cudaStream_t)stream);
}

// One block per row: the heads' results are normed together, scaled, gated and rounded.
template <typename T>
__global__ void lightning_gate_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, long long pitch,
                                           int g_offset, const float* __restrict__ weight, float eps, int width,
                                           T* __restrict__ out) {
  __shared__ float reduce[33];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const float* src = o + (size_t)row * width;
  float squares = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) squares = fmaf(src[i], src[i], squares);
  const float inv = rsqrtf(srb_block_sum(squares, reduce) / (float)width + eps);
  const T* gate = proj + (size_t)row * pitch + g_offset;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float g = srb_to_float(gate[i]);
    out[(size_t)row * width + i] = srb_from_float<T>(src[i] * inv * weight[i] * (1.0f / (1.0f + expf(-g))));
  }
}

extern "C" int srb_lightning_gate_norm(const float* o, const void* proj, long long pitch, int g_offset, const float* weight,
                                       float eps, int rows, int width, void* out, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0) SRB_FAIL("lightning_gate_norm: width %d must be positive", width);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(lightning_gate_norm_kernel<float>, dim3(rows), dim3(256), 0, s, o, (const float*)proj, pitch,
                             g_offset, weight, eps, width, (float*)out));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(lightning_gate_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, o,
                             (const __nv_bfloat16*)proj, pitch, g_offset, weight, eps, width, (__nv_bfloat16*)out));
  else
    SRB_FAIL("lightning_gate_norm: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("lightning_gate_norm");
  return SRB_OK;
}

// ---- prompt portions in bfloat16: chunks in parallel, products on the tensor cores -------------------------------
// The rows of every request are cut into chunks of LC_TOKENS (128) tokens (from the request's first row of the step).  Three
// kernels behind one pass that replaces the q, k and v columns of the projection by their SiLU (rounded to bfloat16):
//   1. per (chunk, head) the chunk's own contribution to the state, U = sum_j decay^(n-1-j) k_j v_j^T        (parallel)
//   2. per (request, head, entry) the states before every chunk, S_(c+1) = decay^(n_c) S_c + U_c, walking the
//      request's chunks in order; U_c is replaced by S_c, and the request's slot receives the last state     (cheap)
//   3. per (chunk, head) the results o_t = decay^(t+1) S_c^T q_t + sum_(j<=t) decay^(t-j) (q_t . k_j) v_j    (parallel)
// q, k, v are the SiLU of the projections rounded to bfloat16 (mma.sync m16n8k16, 32-bit accumulation).  Rows come in
// by 16-byte loads, all of a thread's loads in flight before the first is used.  Whatever is
// 32-bit by the design and has to be an operand of a product (keys times powers of the decay, decayed scores, the
// state) goes in as the sum of two bfloat16 numbers, its rounding and the rounding of the rest, in two products: 16
// bits of mantissa survive.  Operands lie in shared memory with the contraction index contiguous and rows padded by
// 16 bytes, so a fragment is four (or two) conflict-free 32-bit loads.
#include "chunk_helpers.cuh"
#define LC_THREADS 128
#define LC_OUT_THREADS (LC_TOKENS * 2)      // the results kernel: a warp per sixteen rows of the chunk

struct LightningChunkArgs {
  const __nv_bfloat16* proj;
  long long pitch;
  int q_offset, k_offset, v_offset;
  const int* cu_rows;
  const int* positions;
  const int* state_slots;
  float* state;              // [slots, heads, dim, vdim]
  const float* decay;
  float* chunk_states;       // [chunks, heads, dim, vdim]: U of a chunk, then the state before it
  float* out;                // [rows, heads * vdim]
  int requests, heads, read_only;
};

// the request and the chunk of it that block `index` works on; false: there is no such chunk
__device__ __forceinline__ bool lc_find(const LightningChunkArgs& a, int index, int& request, int& row0, int& n) {
  int first = 0;
  for (request = 0; request < a.requests; ++request) {
    const int begin = a.cu_rows[request], rows = a.cu_rows[request + 1] - begin;
    const int chunks = (rows + LC_TOKENS - 1) / LC_TOKENS;
    if (index < first + chunks) {
      row0 = begin + (index - first) * LC_TOKENS;
      n = min(LC_TOKENS, begin + rows - row0);
      return true;
    }
    first += chunks;
  }
  return false;
}

__device__ __forceinline__ void lc_powers(float* power, float decay) {     // power[m] = decay^m, m = 0 .. LC_TOKENS
  if (threadIdx.x == 0) {
    float p = 1.f;
    for (int m = 0; m <= LC_TOKENS; ++m) {
      power[m] = p;
      p *= decay;
    }
  }
}

// columns [begin, begin + count) of every row: x <- SiLU(x), rounded once; eight values a thread
__global__ void lightning_activate_kernel(__nv_bfloat16* proj, long long pitch, int rows, int begin0, int count0, int begin1,
                                          int count1, int begin2, int count2) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int per_row = (count0 + count1 + count2) / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / per_row);
    int at = (int)(i - (long long)row * per_row) * 8;
    int column;
    if (at < count0) column = begin0 + at;
    else if (at < count0 + count1) column = begin1 + at - count0;
    else column = begin2 + at - count0 - count1;
    __nv_bfloat16* p = proj + (size_t)row * pitch + column;
    Bf16x8 x = lc_load8(p, true);
#pragma unroll
    for (int k = 0; k < 8; ++k) x.v[k] = __float2bfloat16_rn(la_silu(__bfloat162float(x.v[k])));
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(x.v);
  }
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(LC_THREADS) lightning_chunk_states_kernel(LightningChunkArgs a) {
  constexpr int TP = LC_TOKENS + LC_PAD;
  extern __shared__ __align__(16) unsigned char lc_smem[];
  __nv_bfloat16* kt_hi = reinterpret_cast<__nv_bfloat16*>(lc_smem);      // [DIM][TP]: decay^(n-1-j) k_j[d], rounded
  __nv_bfloat16* kt_lo = kt_hi + DIM * TP;                               // ... and what the rounding left
  __nv_bfloat16* vt = kt_lo + DIM * TP;                                  // [VDIM][TP]
  __shared__ float power[LC_TOKENS + 1];
  srb_launch_dependents();
  const int head = blockIdx.y;
  lc_powers(power, a.decay[head]);
  srb_grid_dependency_wait();
  int request, row0, n;
  if (!lc_find(a, blockIdx.x, request, row0, n)) return;
  __syncthreads();
  lc_load_transposed<DIM, LC_THREADS>(a.proj + (size_t)row0 * a.pitch + a.k_offset + head * DIM, a.pitch, n, power, n - 1, -1, kt_hi, kt_lo);
  lc_load_transposed<VDIM, LC_THREADS>(a.proj + (size_t)row0 * a.pitch + a.v_offset + head * VDIM, a.pitch, n, nullptr, 0, 0, vt, nullptr);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int MT = DIM / 64;                 // m16 tiles per warp: the warp owns DIM / 4 rows of U
  constexpr int NT = VDIM / 8;
  float acc[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[m][nt][0] = acc[m][nt][1] = acc[m][nt][2] = acc[m][nt][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < LC_TOKENS / 16; ++kk) {
    unsigned ah[MT][4], al[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int row = warp * (DIM / 4) + m * 16 + g, col = kk * 16 + 2 * t;
      ah[m][0] = lc_word(kt_hi + row * TP + col);       al[m][0] = lc_word(kt_lo + row * TP + col);
      ah[m][1] = lc_word(kt_hi + (row + 8) * TP + col); al[m][1] = lc_word(kt_lo + (row + 8) * TP + col);
      ah[m][2] = lc_word(kt_hi + row * TP + col + 8);   al[m][2] = lc_word(kt_lo + row * TP + col + 8);
      ah[m][3] = lc_word(kt_hi + (row + 8) * TP + col + 8); al[m][3] = lc_word(kt_lo + (row + 8) * TP + col + 8);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const __nv_bfloat16* b = vt + (nt * 8 + g) * TP + kk * 16 + 2 * t;
      const unsigned b0 = lc_word(b), b1 = lc_word(b + 8);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        mma_bf16(acc[m][nt], ah[m], b0, b1);
        mma_bf16(acc[m][nt], al[m], b0, b1);
      }
    }
  }
  float* u = a.chunk_states + ((size_t)blockIdx.x * a.heads + head) * DIM * VDIM;
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int row = warp * (DIM / 4) + m * 16 + g, col = nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(u + (size_t)row * VDIM + col) = make_float2(acc[m][nt][0], acc[m][nt][1]);
      *reinterpret_cast<float2*>(u + (size_t)(row + 8) * VDIM + col) = make_float2(acc[m][nt][2], acc[m][nt][3]);
    }
}

// One thread per entry of a head's state: the request's chunks in order.
__global__ void lightning_chunk_prefix_kernel(LightningChunkArgs a, int entries) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x, head = blockIdx.y, request = blockIdx.z;
  if (e >= entries) return;
  int first = 0;
  for (int r = 0; r < request; ++r) first += (a.cu_rows[r + 1] - a.cu_rows[r] + LC_TOKENS - 1) / LC_TOKENS;
  const int begin = a.cu_rows[request], rows = a.cu_rows[request + 1] - begin;
  if (rows <= 0) return;
  const float decay = a.decay[head];
  float whole = 1.f;                                   // decay^LC_TOKENS, as the other kernels' tables have it
  for (int m = 0; m < LC_TOKENS; ++m) whole *= decay;
  float* state = a.state + ((size_t)a.state_slots[request] * a.heads + head) * entries + e;
  float s = a.positions[begin] == 0 ? 0.f : *state;
  const int chunks = (rows + LC_TOKENS - 1) / LC_TOKENS;
  const size_t step = (size_t)a.heads * entries;
  float* u = a.chunk_states + ((size_t)first * a.heads + head) * entries + e;
  for (int c0 = 0; c0 < chunks; c0 += 8) {
    float own[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (c0 + k < chunks) own[k] = u[(size_t)(c0 + k) * step];       // eight loads in flight
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = c0 + k;
      if (c >= chunks) break;
      const int n = min(LC_TOKENS, rows - c * LC_TOKENS);
      float factor = whole;
      if (n < LC_TOKENS) {
        factor = 1.f;
        for (int m = 0; m < n; ++m) factor *= decay;
      }
      u[(size_t)c * step] = s;
      s = fmaf(factor, s, own[k]);
    }
  }
  if (!a.read_only) *state = s;
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(LC_OUT_THREADS) lightning_chunk_outputs_kernel(LightningChunkArgs a) {
  constexpr int DP = DIM + LC_PAD, TP = LC_TOKENS + LC_PAD;
  extern __shared__ __align__(16) unsigned char lc_smem[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(lc_smem);          // [LC_TOKENS][DP]
  __nv_bfloat16* ks = qs + LC_TOKENS * DP;                                // [LC_TOKENS][DP]
  __nv_bfloat16* vt = ks + LC_TOKENS * DP;                                // [VDIM][TP]
  __nv_bfloat16* st_hi = vt + VDIM * TP;                                  // [VDIM][DP]: the state before the chunk, transposed
  __nv_bfloat16* st_lo = st_hi + VDIM * DP;
  __shared__ float power[LC_TOKENS + 1];
  srb_launch_dependents();
  const int head = blockIdx.y;
  lc_powers(power, a.decay[head]);
  srb_grid_dependency_wait();
  int request, row0, n;
  if (!lc_find(a, blockIdx.x, request, row0, n)) return;
  {
    // q and k as they lie: 16-byte pieces, a row's pieces in consecutive lanes
    constexpr int PIECES = LC_TOKENS * DIM / 8, PER = PIECES / LC_OUT_THREADS;
    Bf16x8 xq[PER], xk[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int piece = threadIdx.x + i * LC_OUT_THREADS, j = piece / (DIM / 8), d0 = piece % (DIM / 8) * 8;
      const __nv_bfloat16* row = a.proj + (size_t)(row0 + j) * a.pitch + head * DIM + d0;
      xq[i] = lc_load8(row + a.q_offset, j < n);
      xk[i] = lc_load8(row + a.k_offset, j < n);
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int piece = threadIdx.x + i * LC_OUT_THREADS, j = piece / (DIM / 8), d0 = piece % (DIM / 8) * 8;
      *reinterpret_cast<uint4*>(qs + j * DP + d0) = *reinterpret_cast<const uint4*>(xq[i].v);
      *reinterpret_cast<uint4*>(ks + j * DP + d0) = *reinterpret_cast<const uint4*>(xk[i].v);
    }
  }
  lc_load_transposed<VDIM, LC_OUT_THREADS>(a.proj + (size_t)row0 * a.pitch + a.v_offset + head * VDIM, a.pitch, n, nullptr, 0, 0, vt, nullptr);
  {
    // the state before the chunk, [d][c] floats, into [c][d] as two bfloat16 numbers: consecutive lanes take
    // consecutive d, four columns each
    const float* before = a.chunk_states + ((size_t)blockIdx.x * a.heads + head) * DIM * VDIM;
    constexpr int ITEMS = DIM * VDIM / 4, BATCH = 8;
    for (int first = 0; first < ITEMS; first += BATCH * LC_OUT_THREADS) {
      float4 x[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int item = first + threadIdx.x + i * LC_OUT_THREADS, d = item % DIM, c0 = item / DIM * 4;
        x[i] = item < ITEMS ? *reinterpret_cast<const float4*>(before + (size_t)d * VDIM + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int item = first + threadIdx.x + i * LC_OUT_THREADS, d = item % DIM, c0 = item / DIM * 4;
        if (item >= ITEMS) continue;
        const float v[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          __nv_bfloat16 hi, lo;
          lc_split(v[k], hi, lo);
          st_hi[(c0 + k) * DP + d] = hi;
          st_lo[(c0 + k) * DP + d] = lo;
        }
      }
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int NT = VDIM / 8, ST = LC_TOKENS / 8;
  const int r0 = warp * 16 + g, r1 = r0 + 8;              // this thread's two rows (tokens) of the chunk
  // what the state before the chunk gives: q_t S, then times decay^(t+1)
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  float score[ST][4];
#pragma unroll
  for (int nt = 0; nt < ST; ++nt) score[nt][0] = score[nt][1] = score[nt][2] = score[nt][3] = 0.f;
#pragma unroll 2
  for (int kk = 0; kk < DIM / 16; ++kk) {
    unsigned qa[4];
    const int col = kk * 16 + 2 * t;
    qa[0] = lc_word(qs + r0 * DP + col);
    qa[1] = lc_word(qs + r1 * DP + col);
    qa[2] = lc_word(qs + r0 * DP + col + 8);
    qa[3] = lc_word(qs + r1 * DP + col + 8);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int at = (nt * 8 + g) * DP + col;
      mma_bf16(acc[nt], qa, lc_word(st_hi + at), lc_word(st_hi + at + 8));
      mma_bf16(acc[nt], qa, lc_word(st_lo + at), lc_word(st_lo + at + 8));
    }
#pragma unroll
    for (int nt = 0; nt < ST; ++nt) {
      const int at = (nt * 8 + g) * DP + col;
      mma_bf16(score[nt], qa, lc_word(ks + at), lc_word(ks + at + 8));
    }
  }
  const float carry0 = power[min(r0, LC_TOKENS - 1) + 1], carry1 = power[min(r1, LC_TOKENS - 1) + 1];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    acc[nt][0] *= carry0; acc[nt][1] *= carry0;
    acc[nt][2] *= carry1; acc[nt][3] *= carry1;
  }
  // the chunk's own tokens: decayed scores of the keys up to the row's own, as two bfloat16 operands
#pragma unroll
  for (int kj = 0; kj < LC_TOKENS / 16; ++kj) {
    unsigned hi[4], lo[4];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int nt = 2 * kj + half, j0 = nt * 8 + 2 * t;
      float v[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = c < 2 ? r0 : r1, j = j0 + (c & 1);
        v[c] = (j <= r && r < n) ? score[nt][c] * power[r - j] : 0.f;
      }
      __nv_bfloat16 h[4], l[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) lc_split(v[c], h[c], l[c]);
      hi[half * 2] = pack_bf16(__bfloat162float(h[0]), __bfloat162float(h[1]));
      hi[half * 2 + 1] = pack_bf16(__bfloat162float(h[2]), __bfloat162float(h[3]));
      lo[half * 2] = pack_bf16(__bfloat162float(l[0]), __bfloat162float(l[1]));
      lo[half * 2 + 1] = pack_bf16(__bfloat162float(l[2]), __bfloat162float(l[3]));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const __nv_bfloat16* b = vt + (nt * 8 + g) * TP + kj * 16 + 2 * t;
      const unsigned b0 = lc_word(b), b1 = lc_word(b + 8);
      mma_bf16(acc[nt], hi, b0, b1);
      mma_bf16(acc[nt], lo, b0, b1);
    }
  }
  const int out_pitch = a.heads * VDIM;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = head * VDIM + nt * 8 + 2 * t;
    if (r0 < n) *reinterpret_cast<float2*>(a.out + (size_t)(row0 + r0) * out_pitch + col) = make_float2(acc[nt][0], acc[nt][1]);
    if (r1 < n) *reinterpret_cast<float2*>(a.out + (size_t)(row0 + r1) * out_pitch + col) = make_float2(acc[nt][2], acc[nt][3]);
  }
}

template <int DIM, int VDIM>
static int launch_lightning_chunks(const LightningChunkArgs& a, int rows, int chunks, cudaStream_t s) {
  const size_t smem1 = (size_t)(2 * DIM + VDIM) * (LC_TOKENS + LC_PAD) * 2;
  const size_t smem3 = ((size_t)2 * LC_TOKENS * (DIM + LC_PAD) + (size_t)VDIM * (LC_TOKENS + LC_PAD) + (size_t)2 * VDIM * (DIM + LC_PAD)) * 2;
  SRB_CUDA_CALL(cudaFuncSetAttribute(lightning_chunk_states_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
  SRB_CUDA_CALL(cudaFuncSetAttribute(lightning_chunk_outputs_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3));
  SRB_CUDA_CALL(srb_launch(lightning_activate_kernel, dim3(srb_sm_count() * 8), dim3(256), 0, s, const_cast<__nv_bfloat16*>(a.proj),
                           a.pitch, rows, a.q_offset, a.heads * DIM, a.k_offset, a.heads * DIM, a.v_offset, a.heads * VDIM));
  SRB_LAUNCH_CHECK("lightning_activate");
  SRB_CUDA_CALL(srb_launch(lightning_chunk_states_kernel<DIM, VDIM>, dim3(chunks, a.heads), dim3(LC_THREADS), smem1, s, a));
  SRB_LAUNCH_CHECK("lightning_chunk_states");
  const int entries = DIM * VDIM;
  SRB_CUDA_CALL(srb_launch(lightning_chunk_prefix_kernel, dim3((entries + 255) / 256, a.heads, a.requests), dim3(256), 0, s, a, entries));
  SRB_LAUNCH_CHECK("lightning_chunk_prefix");
  SRB_CUDA_CALL(srb_launch(lightning_chunk_outputs_kernel<DIM, VDIM>, dim3(chunks, a.heads), dim3(LC_OUT_THREADS), smem3, s, a));
  SRB_LAUNCH_CHECK("lightning_chunk_outputs");
  return SRB_OK;
}

// Tokens of a chunk, and whether these sizes are taken (bfloat16; dim and vdim 64 or 128 each).
extern "C" int srb_lightning_chunk_tokens() { return LC_TOKENS; }
extern "C" int srb_lightning_chunks_supports(int dim, int vdim, int dtype) {
  return dtype == SRB_DTYPE_BF16 && (dim == 64 || dim == 128) && (vdim == 64 || vdim == 128);
}

// `chunks`: at least the number of chunks of the step, sum over the requests of ceil(rows / srb_lightning_chunk_tokens());
// `chunk_states`: chunks * heads * dim * vdim floats of scratch.  The rest as for srb_lightning_scan, but: the q, k and v
// columns of `proj` (`rows` rows) are replaced by their SiLU, and rows and column offsets lie on 16-byte borders.
extern "C" int srb_lightning_chunks(void* proj, int rows, long long pitch, int q_offset, int k_offset, int v_offset,
                                    const int* cu_rows, const int* positions, const int* state_slots, float* state,
                                    const float* decay, float* chunk_states, float* out, int requests, int chunks, int heads,
                                    int dim, int vdim, int read_only, void* stream) {
  if (requests <= 0 || chunks <= 0) return SRB_OK;
  if (!srb_lightning_chunks_supports(dim, vdim, SRB_DTYPE_BF16))
    SRB_FAIL("lightning_chunks: a state of %d x %d per head is not taken (64 or 128 each)", dim, vdim);
  if (heads <= 0 || heads > 65535 || requests > 65535) SRB_FAIL("lightning_chunks: %d heads or %d requests exceed one launch", heads, requests);
  if (((pitch | q_offset | k_offset | v_offset) & 7) || ((uintptr_t)proj & 15))
    SRB_FAIL("lightning_chunks: rows and the q, k, v columns must start on 16-byte borders");
  if (rows <= 0) return SRB_OK;
  LightningChunkArgs a;
  a.proj = (const __nv_bfloat16*)proj; a.pitch = pitch; a.q_offset = q_offset; a.k_offset = k_offset; a.v_offset = v_offset;
  a.cu_rows = cu_rows; a.positions = positions; a.state_slots = state_slots; a.state = state; a.decay = decay;
  a.chunk_states = chunk_states; a.out = out; a.requests = requests; a.heads = heads; a.read_only = read_only;
  cudaStream_t s = (cudaStream_t)stream;
  if (dim == 64 && vdim == 64) return launch_lightning_chunks<64, 64>(a, rows, chunks, s);
  if (dim == 64) return launch_lightning_chunks<64, 128>(a, rows, chunks, s);
  if (vdim == 64) return launch_lightning_chunks<128, 64>(a, rows, chunks, s);
  return launch_lightning_chunks<128, 128>(a, rows, chunks, s);
}
