// A state-space mixer with a scalar decay per head and step ("Mamba-2"), over a state of fixed size per request.
//
// A row of the in-projection is [z: inner | x: inner | B: groups * N | C: groups * N | dt: heads] with inner =
// heads * P.  x, B and C (the `channels` = inner + 2 * groups * N middle entries) pass a causal convolution per
// channel over the last `taps` tokens and SiLU.  Per head h (its B and C are those of group h / (heads / groups)):
//
//   dt_t = softplus(dt_t + dt_bias_h)                       a_t = exp(-exp(A_log_h) * dt_t)
//   S_t  = a_t S_(t-1) + dt_t B_t x_t^T     (S is N x P)     y_t = S_t^T C_t + D_h x_t
//
// A request's slot of state holds, in 32-bit floats, the last taps - 1 inputs of the convolution
// [taps - 1][channels] (oldest first) followed by S as [heads][P][N] (a column's N entries together).  Kernels:
//
//   srb_mamba_conv        the convolution + SiLU of every row of the step (32-bit result, or rounded to bfloat16 for the
//                         chunk kernels), reading earlier rows of the
//                         same request from the step and, before the step's first row, from the slot; then the slot's
//                         inputs are replaced by the last taps - 1 of the sequence (a second launch: rows read the old ones)
//   srb_mamba_scan        the recurrence, token by token: a block owns a head's N x PB slice of the state in registers
//                         (PB columns, N cut over the lanes beside each column), stages 16 tokens' B, C, x, dt at a time in
//                         shared memory and walks them; decoded tokens and prompt portions take the same arithmetic, so a
//                         row's result does not depend on how the sequence was cut
//   srb_mamba_chunks      the same recurrence for prompt portions in bfloat16, in chunks of 128 tokens that run in parallel
//                         on the tensor cores (described above those kernels)
//   srb_mamba_gate_norm   y * silu(z), RMS norm in `norm_groups` equal parts, times the weight, rounded
//
// Decays, step sizes, the state, the sums and the norm are 32-bit in both dtypes.  A request whose first row of the step
// is at position 0 starts from zero whatever its slot holds; rows at negative positions pad a captured step and are skipped.
#include "common.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define MAMBA_MAX_TAPS 16
#define MAMBA_TOKENS 16        // tokens staged in shared memory at a time
#define MAMBA_CONV_ROWS 8      // rows of the step that one thread of the convolution takes
#define MAMBA_THREADS 256

struct MambaShape {
  int heads, vdim, nstate, groups, taps;
  int inner, channels;            // heads * vdim; inner + 2 * groups * nstate
  long long proj_pitch;           // elements between rows of the in-projection
  long long slot_floats;          // floats of state per request
  int conv_floats;                // (taps - 1) * channels
};

__device__ __forceinline__ float mamba_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float mamba_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// SiLU of the convolution's sum as the result's type: a bfloat16 result keeps 8 bits of mantissa, so the quick exponential
// and quotient (about 22 bits) round to the same number but for ties
template <typename O> __device__ __forceinline__ O mamba_conv_result(float acc);
template <> __device__ __forceinline__ float mamba_conv_result<float>(float acc) { return mamba_silu(acc); }
template <> __device__ __forceinline__ __nv_bfloat16 mamba_conv_result<__nv_bfloat16>(float acc) {
  return __float2bfloat16_rn(__fdividef(acc, 1.0f + __expf(-acc)));
}

// grid (channel blocks, ceil(rows / ROWS)), so that blocks that run together read neighbouring pieces of the same rows:
// a thread takes one channel of ROWS consecutive rows (MAMBA_CONV_ROWS in steps
// of many rows, so that the filter is read once and the rows' loads are in flight together; 1 in steps of few rows).
// TAPS: the filter's length, or 0 for any.
template <typename T, typename O, int TAPS, int ROWS>
__global__ void mamba_conv_kernel(const T* __restrict__ proj, const float* __restrict__ weight, const float* __restrict__ bias,
                                  const int* __restrict__ positions, const int* __restrict__ row_request,
                                  const int* __restrict__ cu_rows, const int* __restrict__ state_slots,
                                  const float* __restrict__ state, O* __restrict__ out, int rows, MambaShape s) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= s.channels) return;
  const int taps = TAPS > 0 ? TAPS : s.taps;
  constexpr int HELD = TAPS > 0 ? TAPS : 1;
  float w[HELD];
  if (TAPS > 0) {
#pragma unroll
    for (int j = 0; j < HELD; ++j) w[j] = weight[(size_t)c * TAPS + j];
  }
  const float b = bias[c];
  const int row0 = blockIdx.y * ROWS;
  // what the rows need to know, all loads in flight together: position, rows of the request before it, the slot
  int pos[ROWS], ahead[ROWS], slot[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const bool live = row0 + r < rows;
    pos[r] = live ? positions[row0 + r] : -1;
    ahead[r] = live ? row_request[row0 + r] : 0;
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int request = ahead[r];
    ahead[r] = row0 + r - cu_rows[request];
    slot[r] = state_slots[request];
  }
  if constexpr (TAPS > 0) {
    // the inputs of rows row0 - (TAPS - 1) .. row0 + ROWS - 1 of the step, whichever request they belong to
    float u[ROWS + HELD - 1];
#pragma unroll
    for (int k = 0; k < ROWS + HELD - 1; ++k) {
      const int row = row0 + k - (HELD - 1);
      u[k] = (row >= 0 && row < rows) ? srb_to_float(proj[(size_t)row * s.proj_pitch + s.inner + c]) : 0.f;
    }
    // rows in the middle of a request's rows of the step: every input is one of the step's
    bool inside = row0 + ROWS <= rows;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) inside = inside && pos[r] >= HELD - 1 && ahead[r] >= HELD - 1;
    if (inside) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        float acc = b;
#pragma unroll
        for (int j = 0; j < HELD; ++j) acc = fmaf(w[j], u[r + j], acc);
        out[(size_t)(row0 + r) * s.channels + c] = mamba_conv_result<O>(acc);
      }
      return;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (row0 + r >= rows) break;
      O* dst = out + (size_t)(row0 + r) * s.channels + c;
      if (pos[r] < 0) { *dst = srb_from_float<O>(0.f); continue; }
      const float* kept = state + (size_t)slot[r] * s.slot_floats;
      float acc = b;
#pragma unroll
      for (int j = 0; j < HELD; ++j) {
        const int back = HELD - 1 - j;
        if (pos[r] - back < 0) continue;                   // zeros before the start of the sequence
        const float v = back <= ahead[r] ? u[r + j] : kept[(size_t)(HELD - 1 - (back - ahead[r])) * s.channels + c];
        acc = fmaf(w[j], v, acc);
      }
      *dst = mamba_conv_result<O>(acc);
    }
  } else {
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = row0 + r;
    if (row >= rows) break;
    O* dst = out + (size_t)row * s.channels + c;
    if (pos[r] < 0) { *dst = srb_from_float<O>(0.f); continue; }
    const float* kept = state + (size_t)slot[r] * s.slot_floats;
    float acc = b;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      if (pos[r] - back < 0) continue;                     // zeros before the start of the sequence
      float v;
      if (back <= ahead[r])
        v = srb_to_float(proj[(size_t)(row - back) * s.proj_pitch + s.inner + c]);
      else
        v = kept[(size_t)(taps - 1 - (back - ahead[r])) * s.channels + c];
      acc = fmaf(weight[(size_t)c * taps + j], v, acc);
    }
    *dst = mamba_conv_result<O>(acc);
  }
  }
}

// One thread per (request, channel): the slot's inputs become the last taps - 1 of the sequence after this step.
template <typename T>
__global__ void mamba_conv_keep_kernel(const T* __restrict__ proj, const int* __restrict__ positions,
                                       const int* __restrict__ cu_rows, const int* __restrict__ state_slots,
                                       float* __restrict__ state, MambaShape s) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int request = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= s.channels) return;
  const int first = cu_rows[request], count = cu_rows[request + 1] - first;
  if (count <= 0) return;
  const int start = positions[first];
  if (start < 0) return;
  float* kept = state + (size_t)state_slots[request] * s.slot_floats;
  const int keep = s.taps - 1;
  float fresh[MAMBA_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < MAMBA_MAX_TAPS; ++k) {
    if (k >= keep) break;
    const int at = start + count - keep + k;           // position in the sequence of the k-th kept input
    float v = 0.f;
    if (at >= start) v = srb_to_float(proj[(size_t)(first + at - start) * s.proj_pitch + s.inner + c]);
    else if (at >= 0) v = kept[(size_t)(at - start + keep) * s.channels + c];
    fresh[k] = v;
  }
#pragma unroll
  for (int k = 0; k < MAMBA_MAX_TAPS; ++k) {
    if (k >= keep) break;
    kept[(size_t)k * s.channels + c] = fresh[k];
  }
}

// grid (heads * column blocks, requests); NS lanes share a column of the state, each with NR of its N entries
template <typename T, int NS, int NR>
__global__ void __launch_bounds__(MAMBA_THREADS)
mamba_scan_kernel(const T* __restrict__ proj, const float* __restrict__ xbc, const float* __restrict__ a_log,
                  const float* __restrict__ d_skip, const float* __restrict__ dt_bias, const int* __restrict__ positions,
                  const int* __restrict__ cu_rows, const int* __restrict__ state_slots, float* __restrict__ state,
                  float* __restrict__ y, int write_state, MambaShape s) {
  constexpr int PB = MAMBA_THREADS / NS;
  extern __shared__ float mamba_smem[];
  const int N = s.nstate, P = s.vdim;
  float* b_s = mamba_smem;                              // [MAMBA_TOKENS][N]
  float* c_s = b_s + MAMBA_TOKENS * N;                  // [MAMBA_TOKENS][N]
  float* x_s = c_s + MAMBA_TOKENS * N;                  // [MAMBA_TOKENS][PB]
  float* dt_s = x_s + MAMBA_TOKENS * PB;                // [MAMBA_TOKENS]
  float* da_s = dt_s + MAMBA_TOKENS;                    // [MAMBA_TOKENS]
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int column_blocks = (P + PB - 1) / PB;
  const int head = blockIdx.x / column_blocks, p0 = (blockIdx.x % column_blocks) * PB;
  const int request = blockIdx.y;
  const int first = cu_rows[request], count = cu_rows[request + 1] - first;
  if (count <= 0) return;
  const int start = positions[first];
  if (start < 0) return;
  const int tid = threadIdx.x, ns = tid % NS, pl = tid / NS, p = p0 + pl;
  const bool active = p < P;
  float* mine = state + (size_t)state_slots[request] * s.slot_floats + s.conv_floats + (size_t)head * N * P;
  float st[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int n = ns + i * NS;
    st[i] = (active && n < N && start > 0) ? mine[(size_t)p * N + n] : 0.f;
  }
  const int group = head / (s.heads / s.groups);
  const float a = -expf(a_log[head]), skip = d_skip[head], bias = dt_bias[head];
  const int b_at = s.inner + group * N, c_at = s.inner + s.groups * N + group * N;
  const int dt_at = s.inner + s.channels + head;
  for (int t0 = 0; t0 < count; t0 += MAMBA_TOKENS) {
    const int tc = min(MAMBA_TOKENS, count - t0);
    for (int i = tid; i < tc * N; i += MAMBA_THREADS) {
      const int t = i / N, n = i - t * N;
      const float* src = xbc + (size_t)(first + t0 + t) * s.channels;
      b_s[t * N + n] = src[b_at + n];
      c_s[t * N + n] = src[c_at + n];
    }
    for (int i = tid; i < tc * PB; i += MAMBA_THREADS) {
      const int t = i / PB, q = i - t * PB;
      x_s[t * PB + q] = p0 + q < P ? xbc[(size_t)(first + t0 + t) * s.channels + head * P + p0 + q] : 0.f;
    }
    if (tid < tc) {
      const float dt = mamba_softplus(srb_to_float(proj[(size_t)(first + t0 + tid) * s.proj_pitch + dt_at]) + bias);
      dt_s[tid] = dt;
      da_s[tid] = expf(a * dt);
    }
    __syncthreads();
    for (int t = 0; t < tc; ++t) {
      const float x = x_s[t * PB + pl], decay = da_s[t], dx = dt_s[t] * x;
      float partial = 0.f;
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int n = ns + i * NS;
        if (n < N) {
          st[i] = fmaf(decay, st[i], dx * b_s[t * N + n]);
          partial = fmaf(st[i], c_s[t * N + n], partial);
        }
      }
#pragma unroll
      for (int offset = NS / 2; offset > 0; offset >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, offset);
      if (ns == 0 && active) y[(size_t)(first + t0 + t) * s.inner + head * P + p] = fmaf(skip, x, partial);
    }
    __syncthreads();
  }
  if (!write_state || !active) return;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int n = ns + i * NS;
    if (n < N) mine[(size_t)p * N + n] = st[i];
  }
}

// grid (rows * norm groups), a row's parts in neighbouring blocks: out = rms_part(y * silu(z)) * weight
template <typename T>
__global__ void mamba_gate_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, long long proj_pitch,
                                       const float* __restrict__ weight, float eps, int inner, int part,
                                       T* __restrict__ out) {
  extern __shared__ float gate_smem[];                  // part floats, then 33 of scratch
  float* scratch = gate_smem + part;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int parts = inner / part, row = blockIdx.x / parts, base = (blockIdx.x % parts) * part;
  float partial = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float z = srb_to_float(proj[(size_t)row * proj_pitch + base + i]);
    const float v = y[(size_t)row * inner + base + i] * mamba_silu(z);
    gate_smem[i] = v;
    partial += v * v;
  }
  const float inv = 1.0f / sqrtf(srb_block_sum(partial, scratch) / (float)part + eps);
  for (int i = threadIdx.x; i < part; i += blockDim.x)
    out[(size_t)row * inner + base + i] = srb_from_float<T>(gate_smem[i] * inv * weight[base + i]);
}

__device__ __forceinline__ float4 mamba_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 mamba_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void mamba_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void mamba_store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&a);
  raw.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same with four consecutive entries a thread (parts, rows and pointers on 16-byte borders of floats).
template <typename T>
__global__ void mamba_gate_norm_vec_kernel(const float* __restrict__ y, const T* __restrict__ proj, long long proj_pitch,
                                           const float* __restrict__ weight, float eps, int inner, int part,
                                           T* __restrict__ out) {
  extern __shared__ __align__(16) float gate_vec_smem[];    // part floats, then 33 of scratch
  float* scratch = gate_vec_smem + part;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int parts = inner / part, row = blockIdx.x / parts, base = (blockIdx.x % parts) * part;
  float partial = 0.f;
  for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
    const float4 z = mamba_load4(proj + (size_t)row * proj_pitch + base + i);
    float4 v = mamba_load4(y + (size_t)row * inner + base + i);
    v.x *= mamba_silu(z.x); v.y *= mamba_silu(z.y); v.z *= mamba_silu(z.z); v.w *= mamba_silu(z.w);
    *reinterpret_cast<float4*>(gate_vec_smem + i) = v;
    partial += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  const float inv = 1.0f / sqrtf(srb_block_sum(partial, scratch) / (float)part + eps);
  for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(gate_vec_smem + i), w = mamba_load4(weight + base + i);
    mamba_store4(out + (size_t)row * inner + base + i, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
  }
}

static int mamba_shape(MambaShape& s, int heads, int vdim, int nstate, int groups, int taps, long long proj_pitch,
                       long long slot_floats) {
  if (heads <= 0 || vdim <= 0 || nstate <= 0 || groups <= 0 || heads % groups) SRB_FAIL("mamba: %d heads of %d columns, %d state entries and %d groups do not fit", heads, vdim, nstate, groups);
  if (taps < 1 || taps > MAMBA_MAX_TAPS) SRB_FAIL("mamba: a convolution over %d tokens is outside 1 .. %d", taps, MAMBA_MAX_TAPS);
  if (nstate > 256) SRB_FAIL("mamba: a state of %d entries per column exceeds 256", nstate);
  s.heads = heads; s.vdim = vdim; s.nstate = nstate; s.groups = groups; s.taps = taps;
  s.inner = heads * vdim; s.channels = s.inner + 2 * groups * nstate;
  s.proj_pitch = proj_pitch; s.conv_floats = (taps - 1) * s.channels;
  s.slot_floats = slot_floats;
  if (proj_pitch < (long long)s.inner + s.channels + heads) SRB_FAIL("mamba: rows of the in-projection are too short");
  if (slot_floats < (long long)s.conv_floats + (long long)heads * nstate * vdim) SRB_FAIL("mamba: a slot of %lld floats is too small", slot_floats);
  return SRB_OK;
}

extern "C" long long srb_mamba_slot_floats(int heads, int vdim, int nstate, int groups, int taps) {
  return (long long)(taps - 1) * (heads * vdim + 2 * groups * nstate) + (long long)heads * nstate * vdim;
}

template <typename T, typename O>
static int launch_mamba_conv(const void* proj, const float* weight, const float* bias, const int* positions,
                             const int* row_request, const int* cu_rows, const int* state_slots, float* state, void* out,
                             int rows, int requests, int write_state, const MambaShape& s, cudaStream_t st) {
  const int block = 128;
  const bool many = rows >= 64 * MAMBA_CONV_ROWS;
  const int per = many ? MAMBA_CONV_ROWS : 1;
  const dim3 grid((s.channels + block - 1) / block, (rows + per - 1) / per);
  if (grid.y > 65535) SRB_FAIL("mamba_conv: %d rows exceed one launch", rows);
  const dim3 keep_grid((s.channels + block - 1) / block, requests);
#define MAMBA_CONV_LAUNCH(TAPS, ROWS)                                                                                        \
  SRB_CUDA_CALL(srb_launch(mamba_conv_kernel<T, O, TAPS, ROWS>, grid, dim3(block), 0, st, (const T*)proj, weight, bias,     \
                           positions, row_request, cu_rows, state_slots, (const float*)state, (O*)out, rows, s))
  if (s.taps == 4 && many) MAMBA_CONV_LAUNCH(4, MAMBA_CONV_ROWS);
  else if (s.taps == 4) MAMBA_CONV_LAUNCH(4, 1);
  else if (s.taps == 3 && many) MAMBA_CONV_LAUNCH(3, MAMBA_CONV_ROWS);
  else if (s.taps == 2 && many) MAMBA_CONV_LAUNCH(2, MAMBA_CONV_ROWS);
  else if (many) MAMBA_CONV_LAUNCH(0, MAMBA_CONV_ROWS);
  else MAMBA_CONV_LAUNCH(0, 1);
#undef MAMBA_CONV_LAUNCH
  if (write_state && s.taps > 1)
    SRB_CUDA_CALL(srb_launch(mamba_conv_keep_kernel<T>, keep_grid, dim3(block), 0, st, (const T*)proj, positions, cu_rows,
                             state_slots, state, s));
  SRB_LAUNCH_CHECK("mamba_conv");
  return SRB_OK;
}

// proj: [rows, pitch]; weight [channels, taps], bias [channels] (float); out: [rows, channels] of `out_dtype` (float,
// or bfloat16 beside a bfloat16 projection: what the chunk kernels read)
extern "C" int srb_mamba_conv(const void* proj, long long proj_pitch, const float* weight, const float* bias,
                              const int* positions, const int* row_request, const int* cu_rows, const int* state_slots,
                              float* state, long long slot_floats, void* out, int rows, int requests, int heads, int vdim,
                              int nstate, int groups, int taps, int write_state, int dtype, int out_dtype, void* stream) {
  if (rows <= 0 || requests <= 0) return SRB_OK;
  MambaShape s;
  if (mamba_shape(s, heads, vdim, nstate, groups, taps, proj_pitch, slot_floats) != SRB_OK) return SRB_ERR_INVALID;
  if (requests > 65535) SRB_FAIL("mamba_conv: %d requests exceed one launch", requests);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32 && out_dtype == SRB_DTYPE_F32)
    return launch_mamba_conv<float, float>(proj, weight, bias, positions, row_request, cu_rows, state_slots, state, out, rows,
                                           requests, write_state, s, st);
  if (dtype == SRB_DTYPE_BF16 && out_dtype == SRB_DTYPE_F32)
    return launch_mamba_conv<__nv_bfloat16, float>(proj, weight, bias, positions, row_request, cu_rows, state_slots, state, out,
                                                   rows, requests, write_state, s, st);
  if (dtype == SRB_DTYPE_BF16 && out_dtype == SRB_DTYPE_BF16)
    return launch_mamba_conv<__nv_bfloat16, __nv_bfloat16>(proj, weight, bias, positions, row_request, cu_rows, state_slots, state,
                                                           out, rows, requests, write_state, s, st);
  SRB_FAIL("mamba_conv: a projection of dtype %d with a result of dtype %d is not taken", dtype, out_dtype);
}

template <typename T>
static int launch_mamba_scan(const void* proj, const float* xbc, const float* a_log, const float* d_skip, const float* dt_bias,
                             const int* positions, const int* cu_rows, const int* state_slots, float* state, float* y,
                             int requests, int write_state, const MambaShape& s, cudaStream_t st) {
  const bool wide = s.nstate > 128;
  const int pb = MAMBA_THREADS / (wide ? 32 : 16);
  const dim3 grid(s.heads * ((s.vdim + pb - 1) / pb), requests);
  const size_t smem = (size_t)(2 * MAMBA_TOKENS * s.nstate + MAMBA_TOKENS * pb + 2 * MAMBA_TOKENS) * sizeof(float);
  if (wide)
    SRB_CUDA_CALL(srb_launch(mamba_scan_kernel<T, 32, 8>, grid, dim3(MAMBA_THREADS), smem, st, (const T*)proj, xbc, a_log, d_skip,
                             dt_bias, positions, cu_rows, state_slots, state, y, write_state, s));
  else
    SRB_CUDA_CALL(srb_launch(mamba_scan_kernel<T, 16, 8>, grid, dim3(MAMBA_THREADS), smem, st, (const T*)proj, xbc, a_log, d_skip,
                             dt_bias, positions, cu_rows, state_slots, state, y, write_state, s));
  SRB_LAUNCH_CHECK("mamba_scan");
  return SRB_OK;
}

// xbc: float [rows, channels] (what srb_mamba_conv wrote); y: float [rows, inner]
extern "C" int srb_mamba_scan(const void* proj, long long proj_pitch, const float* xbc, const float* a_log, const float* d_skip,
                              const float* dt_bias, const int* positions, const int* cu_rows, const int* state_slots,
                              float* state, long long slot_floats, float* y, int rows, int requests, int heads, int vdim,
                              int nstate, int groups, int taps, int write_state, int dtype, void* stream) {
  if (rows <= 0 || requests <= 0) return SRB_OK;
  MambaShape s;
  if (mamba_shape(s, heads, vdim, nstate, groups, taps, proj_pitch, slot_floats) != SRB_OK) return SRB_ERR_INVALID;
  if (requests > 65535) SRB_FAIL("mamba_scan: %d requests exceed one launch", requests);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    return launch_mamba_scan<float>(proj, xbc, a_log, d_skip, dt_bias, positions, cu_rows, state_slots, state, y, requests,
                                    write_state, s, st);
  if (dtype == SRB_DTYPE_BF16)
    return launch_mamba_scan<__nv_bfloat16>(proj, xbc, a_log, d_skip, dt_bias, positions, cu_rows, state_slots, state, y,
                                            requests, write_state, s, st);
  SRB_FAIL("mamba_scan: unknown dtype %d", dtype);
}

// y: float [rows, inner]; z = the first `inner` entries of proj's rows; out: [rows, inner] of proj's type
extern "C" int srb_mamba_gate_norm(const float* y, const void* proj, long long proj_pitch, const float* weight, float eps,
                                   int rows, int inner, int norm_groups, void* out, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (inner <= 0 || norm_groups <= 0 || inner % norm_groups) SRB_FAIL("mamba_gate_norm: %d entries do not split into %d equal parts", inner, norm_groups);
  if (!(eps >= 0.f)) SRB_FAIL("mamba_gate_norm: eps must be finite and non-negative");
  if ((long long)rows * norm_groups > 0x7fffffffLL) SRB_FAIL("mamba_gate_norm: %d rows of %d parts exceed one launch", rows, norm_groups);
  const int part = inner / norm_groups;
  const size_t smem = (size_t)(part + 33) * sizeof(float);
  if (smem > 227 * 1024) SRB_FAIL("mamba_gate_norm: a part of %d entries needs %zu bytes of shared memory (limit 232448)", part, smem);
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = part % 4 == 0 && proj_pitch % 4 == 0 && !(((uintptr_t)y | (uintptr_t)proj | (uintptr_t)weight | (uintptr_t)out) & 15);
  if (vec) {
    const int vblock = part >= 2048 ? 256 : (part >= 512 ? 128 : 64);
    if (dtype == SRB_DTYPE_F32) {
      if (smem > 48 * 1024) SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_gate_norm_vec_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      SRB_CUDA_CALL(srb_launch(mamba_gate_norm_vec_kernel<float>, dim3((unsigned)rows * norm_groups), dim3(vblock), smem, st, y, (const float*)proj,
                               proj_pitch, weight, eps, inner, part, (float*)out));
    } else if (dtype == SRB_DTYPE_BF16) {
      if (smem > 48 * 1024) SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_gate_norm_vec_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      SRB_CUDA_CALL(srb_launch(mamba_gate_norm_vec_kernel<__nv_bfloat16>, dim3((unsigned)rows * norm_groups), dim3(vblock), smem, st, y,
                               (const __nv_bfloat16*)proj, proj_pitch, weight, eps, inner, part, (__nv_bfloat16*)out));
    } else {
      SRB_FAIL("mamba_gate_norm: unknown dtype %d", dtype);
    }
    SRB_LAUNCH_CHECK("mamba_gate_norm");
    return SRB_OK;
  }
  const int block = part >= 2048 ? 512 : (part >= 512 ? 256 : 128);
  if (dtype == SRB_DTYPE_F32) {
    if (smem > 48 * 1024) SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_gate_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(mamba_gate_norm_kernel<float>, dim3((unsigned)rows * norm_groups), dim3(block), smem, st, y, (const float*)proj,
                             proj_pitch, weight, eps, inner, part, (float*)out));
  } else if (dtype == SRB_DTYPE_BF16) {
    if (smem > 48 * 1024) SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_gate_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(mamba_gate_norm_kernel<__nv_bfloat16>, dim3((unsigned)rows * norm_groups), dim3(block), smem, st, y,
                             (const __nv_bfloat16*)proj, proj_pitch, weight, eps, inner, part, (__nv_bfloat16*)out));
  } else {
    SRB_FAIL("mamba_gate_norm: unknown dtype %d", dtype);
  }
  SRB_LAUNCH_CHECK("mamba_gate_norm");
  return SRB_OK;
}

// ---- prompt portions in bfloat16: chunks in parallel, products on the tensor cores -------------------------------
// The rows of every request are cut into chunks of LC_TOKENS (128) tokens (from the request's first row of the step).
// With c_t = sum_(i <= t) -exp(A_log) dt_i taken inside the chunk (never positive, so no exponential exceeds 1), a
// chunk that starts from state S and holds tokens 0 .. n-1 has
//     y_t = exp(c_t) S^T C_t + sum_(j <= t) exp(c_t - c_j) dt_j (C_t . B_j) x_j + D x_t
//     S  <- exp(c_(n-1)) S + sum_j exp(c_(n-1) - c_j) dt_j B_j x_j^T
// Three kernels behind the convolution (which here rounds its result to bfloat16):
//   1. per (chunk, head) the chunk's own contribution to the state, U, and exp(c_(n-1))                   (parallel)
//   2. per (request, head, entry) the states before every chunk, walking the request's chunks in order; U is replaced
//      by the state before the chunk, and the request's slot receives the last state                      (cheap)
//   3. per (chunk, head) the results                                                                       (parallel)
// x, B and C go in as bfloat16 (mma.sync m16n8k16, 32-bit accumulation); step sizes, sums of logarithms of decays and
// exponentials are 32-bit; whatever is 32-bit by the design and has to be an operand of a product (B times its factor,
// decayed scores, the state) goes in as the sum of two bfloat16 numbers in two products.  The state and U lie as
// [heads][P][N], as in a request's slot.
#include "chunk_helpers.cuh"
#define MC_THREADS 128
#define MC_OUT_THREADS (LC_TOKENS * 2)      // the results kernel: a warp per sixteen rows of the chunk

struct MambaChunkArgs {
  const __nv_bfloat16* proj;   // [rows, pitch]: the dt entries are read
  const __nv_bfloat16* xbc;    // [rows, channels]: what the convolution wrote
  const float* a_log;
  const float* d_skip;
  const float* dt_bias;
  const int* cu_rows;
  const int* positions;
  const int* state_slots;
  float* state;
  float* chunk_states;         // [chunks, heads, P, N]: U of a chunk, then the state before it
  float* chunk_decay;          // [chunks, heads]: exp(c_(n-1))
  float* y;                    // [rows, inner]
  int requests, write_state;
  MambaShape s;
};

// the request and the chunk of it that block `index` works on; false: there is no such chunk
__device__ __forceinline__ bool mc_find(const MambaChunkArgs& a, int index, int& request, int& row0, int& n) {
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

// dt_s[j] = softplus(dt_j + bias) and cum_s[j] = c_j for the chunk's tokens (beyond the n-th: 0, and c stays); every
// thread of the block comes here, and the block has at least LC_TOKENS threads
__device__ __forceinline__ void mc_steps(const MambaChunkArgs& a, int head, int row0, int n, float* dt_s, float* cum_s) {
  const int tid = threadIdx.x;
  if (tid < LC_TOKENS) {
    float dt = 0.f;
    if (tid < n) {
      const size_t at = (size_t)(row0 + tid) * a.s.proj_pitch + a.s.inner + a.s.channels + head;
      dt = mamba_softplus(__bfloat162float(a.proj[at]) + a.dt_bias[head]);
    }
    dt_s[tid] = dt;
    cum_s[tid] = -expf(a.a_log[head]) * dt;
  }
  __syncthreads();
  if (tid < 32) {                      // a lane sums four consecutive tokens, the lanes' totals are scanned
    float part[LC_TOKENS / 32], sum = 0.f;
#pragma unroll
    for (int k = 0; k < LC_TOKENS / 32; ++k) {
      sum += cum_s[tid * (LC_TOKENS / 32) + k];
      part[k] = sum;
    }
    float total = sum;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const float other = __shfl_up_sync(0xffffffffu, total, offset);
      if (tid >= offset) total += other;
    }
    float before = __shfl_up_sync(0xffffffffu, total, 1);
    if (tid == 0) before = 0.f;
#pragma unroll
    for (int k = 0; k < LC_TOKENS / 32; ++k) cum_s[tid * (LC_TOKENS / 32) + k] = before + part[k];
  }
  __syncthreads();
}

template <int N, int P>
__global__ void __launch_bounds__(MC_THREADS) mamba_chunk_states_kernel(MambaChunkArgs a) {
  constexpr int TP = LC_TOKENS + LC_PAD;
  extern __shared__ __align__(16) unsigned char mc_smem[];
  __nv_bfloat16* xt = reinterpret_cast<__nv_bfloat16*>(mc_smem);         // [P][TP]
  __nv_bfloat16* bt_hi = xt + P * TP;                                    // [N][TP]: exp(c_(n-1) - c_j) dt_j B_j, rounded
  __nv_bfloat16* bt_lo = bt_hi + N * TP;                                 // ... and what the rounding left
  __shared__ float dt_s[LC_TOKENS], cum_s[LC_TOKENS], w_s[LC_TOKENS];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int head = blockIdx.y;
  int request, row0, n;
  if (!mc_find(a, blockIdx.x, request, row0, n)) return;
  mc_steps(a, head, row0, n, dt_s, cum_s);
  if (threadIdx.x < LC_TOKENS) w_s[threadIdx.x] = threadIdx.x < n ? expf(cum_s[n - 1] - cum_s[threadIdx.x]) * dt_s[threadIdx.x] : 0.f;
  __syncthreads();
  const int group = head / (a.s.heads / a.s.groups);
  const __nv_bfloat16* rows = a.xbc + (size_t)row0 * a.s.channels;
  lc_load_transposed<P, MC_THREADS>(rows + head * P, a.s.channels, n, nullptr, 0, 0, xt, nullptr);
  lc_load_transposed<N, MC_THREADS>(rows + a.s.inner + group * N, a.s.channels, n, w_s, 0, 1, bt_hi, bt_lo);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int MT = P / 64;                   // m16 tiles per warp: the warp owns P / 4 rows of U
  constexpr int NT = N / 8;
  float acc[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[m][nt][0] = acc[m][nt][1] = acc[m][nt][2] = acc[m][nt][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < LC_TOKENS / 16; ++kk) {
    unsigned ax[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int row = warp * (P / 4) + m * 16 + g, col = kk * 16 + 2 * t;
      ax[m][0] = lc_word(xt + row * TP + col);
      ax[m][1] = lc_word(xt + (row + 8) * TP + col);
      ax[m][2] = lc_word(xt + row * TP + col + 8);
      ax[m][3] = lc_word(xt + (row + 8) * TP + col + 8);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int at = (nt * 8 + g) * TP + kk * 16 + 2 * t;
      const unsigned h0 = lc_word(bt_hi + at), h1 = lc_word(bt_hi + at + 8);
      const unsigned l0 = lc_word(bt_lo + at), l1 = lc_word(bt_lo + at + 8);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        mma_bf16(acc[m][nt], ax[m], h0, h1);
        mma_bf16(acc[m][nt], ax[m], l0, l1);
      }
    }
  }
  float* u = a.chunk_states + ((size_t)blockIdx.x * a.s.heads + head) * N * P;
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int row = warp * (P / 4) + m * 16 + g, col = nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(u + (size_t)row * N + col) = make_float2(acc[m][nt][0], acc[m][nt][1]);
      *reinterpret_cast<float2*>(u + (size_t)(row + 8) * N + col) = make_float2(acc[m][nt][2], acc[m][nt][3]);
    }
  if (threadIdx.x == 0) a.chunk_decay[(size_t)blockIdx.x * a.s.heads + head] = expf(cum_s[n - 1]);
}

// One thread per entry of a head's state: the request's chunks in order.
__global__ void mamba_chunk_prefix_kernel(MambaChunkArgs a, int entries) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x, head = blockIdx.y, request = blockIdx.z;
  if (e >= entries) return;
  int first = 0;
  for (int r = 0; r < request; ++r) first += (a.cu_rows[r + 1] - a.cu_rows[r] + LC_TOKENS - 1) / LC_TOKENS;
  const int begin = a.cu_rows[request], rows = a.cu_rows[request + 1] - begin;
  if (rows <= 0) return;
  const int start = a.positions[begin];
  if (start < 0) return;
  float* state = a.state + (size_t)a.state_slots[request] * a.s.slot_floats + a.s.conv_floats + (size_t)head * entries + e;
  float s = start == 0 ? 0.f : *state;
  const int chunks = (rows + LC_TOKENS - 1) / LC_TOKENS;
  const size_t step = (size_t)a.s.heads * entries;
  float* u = a.chunk_states + ((size_t)first * a.s.heads + head) * entries + e;
  const float* decay = a.chunk_decay + (size_t)first * a.s.heads + head;
  for (int c0 = 0; c0 < chunks; c0 += 8) {
    float own[8], factor[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (c0 + k < chunks) {                                           // the loads of eight chunks in flight
        own[k] = u[(size_t)(c0 + k) * step];
        factor[k] = decay[(size_t)(c0 + k) * a.s.heads];
      }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = c0 + k;
      if (c >= chunks) break;
      u[(size_t)c * step] = s;
      s = fmaf(factor[k], s, own[k]);
    }
  }
  if (a.write_state) *state = s;
}

template <int N, int P>
__global__ void __launch_bounds__(MC_OUT_THREADS) mamba_chunk_outputs_kernel(MambaChunkArgs a) {
  constexpr int DP = N + LC_PAD, TP = LC_TOKENS + LC_PAD;
  extern __shared__ __align__(16) unsigned char mc_smem[];
  __nv_bfloat16* cs = reinterpret_cast<__nv_bfloat16*>(mc_smem);          // [LC_TOKENS][DP]: C_t
  __nv_bfloat16* bs = cs + LC_TOKENS * DP;                                // [LC_TOKENS][DP]: B_j
  __nv_bfloat16* xt = bs + LC_TOKENS * DP;                                // [P][TP]
  __nv_bfloat16* st_hi = xt + P * TP;                                     // [P][DP]: the state before the chunk
  __nv_bfloat16* st_lo = st_hi + P * DP;
  __shared__ float dt_s[LC_TOKENS], cum_s[LC_TOKENS];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int head = blockIdx.y;
  int request, row0, n;
  if (!mc_find(a, blockIdx.x, request, row0, n)) return;
  mc_steps(a, head, row0, n, dt_s, cum_s);
  const int group = head / (a.s.heads / a.s.groups);
  const __nv_bfloat16* rows = a.xbc + (size_t)row0 * a.s.channels;
  {
    // B and C as they lie: 16-byte pieces, a row's pieces in consecutive lanes
    constexpr int PIECES = LC_TOKENS * N / 8, PER = PIECES / MC_OUT_THREADS;
    const int c_from_b = a.s.groups * N;
    Bf16x8 xc[PER], xb[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int piece = threadIdx.x + i * MC_OUT_THREADS, j = piece / (N / 8), d0 = piece % (N / 8) * 8;
      const __nv_bfloat16* row = rows + (size_t)j * a.s.channels + a.s.inner + group * N + d0;
      xb[i] = lc_load8(row, j < n);
      xc[i] = lc_load8(row + c_from_b, j < n);
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int piece = threadIdx.x + i * MC_OUT_THREADS, j = piece / (N / 8), d0 = piece % (N / 8) * 8;
      *reinterpret_cast<uint4*>(cs + j * DP + d0) = *reinterpret_cast<const uint4*>(xc[i].v);
      *reinterpret_cast<uint4*>(bs + j * DP + d0) = *reinterpret_cast<const uint4*>(xb[i].v);
    }
  }
  lc_load_transposed<P, MC_OUT_THREADS>(rows + head * P, a.s.channels, n, nullptr, 0, 0, xt, nullptr);
  {
    // the state before the chunk, [p][n] floats, as two bfloat16 numbers: four entries of a column a thread
    const float* before = a.chunk_states + ((size_t)blockIdx.x * a.s.heads + head) * N * P;
    constexpr int ITEMS = N * P / 4, BATCH = 8;
    for (int first = 0; first < ITEMS; first += BATCH * MC_OUT_THREADS) {
      float4 x[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int item = first + threadIdx.x + i * MC_OUT_THREADS;
        x[i] = item < ITEMS ? *reinterpret_cast<const float4*>(before + (size_t)item * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int item = first + threadIdx.x + i * MC_OUT_THREADS, p = item / (N / 4), n0 = item % (N / 4) * 4;
        if (item >= ITEMS) continue;
        const float v[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
        __nv_bfloat16 hi[4], lo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) lc_split(v[k], hi[k], lo[k]);
        *reinterpret_cast<uint2*>(st_hi + p * DP + n0) = *reinterpret_cast<const uint2*>(hi);
        *reinterpret_cast<uint2*>(st_lo + p * DP + n0) = *reinterpret_cast<const uint2*>(lo);
      }
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int NT = P / 8, ST = LC_TOKENS / 8;
  const int r0 = warp * 16 + g, r1 = r0 + 8;              // this thread's two rows (tokens) of the chunk
  // what the state before the chunk gives: C_t S, then times exp(c_t)
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  float score[ST][4];
#pragma unroll
  for (int nt = 0; nt < ST; ++nt) score[nt][0] = score[nt][1] = score[nt][2] = score[nt][3] = 0.f;
#pragma unroll 2
  for (int kk = 0; kk < N / 16; ++kk) {
    unsigned qa[4];
    const int col = kk * 16 + 2 * t;
    qa[0] = lc_word(cs + r0 * DP + col);
    qa[1] = lc_word(cs + r1 * DP + col);
    qa[2] = lc_word(cs + r0 * DP + col + 8);
    qa[3] = lc_word(cs + r1 * DP + col + 8);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int at = (nt * 8 + g) * DP + col;
      mma_bf16(acc[nt], qa, lc_word(st_hi + at), lc_word(st_hi + at + 8));
      mma_bf16(acc[nt], qa, lc_word(st_lo + at), lc_word(st_lo + at + 8));
    }
#pragma unroll
    for (int nt = 0; nt < ST; ++nt) {
      const int at = (nt * 8 + g) * DP + col;
      mma_bf16(score[nt], qa, lc_word(bs + at), lc_word(bs + at + 8));
    }
  }
  const float cum0 = cum_s[r0], cum1 = cum_s[r1];
  const float carry0 = expf(cum0), carry1 = expf(cum1);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    acc[nt][0] *= carry0; acc[nt][1] *= carry0;
    acc[nt][2] *= carry1; acc[nt][3] *= carry1;
  }
  // the chunk's own tokens: decayed scores of the tokens up to the row's own, times their steps, as two bfloat16 operands
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
        v[c] = (j <= r && r < n) ? score[nt][c] * (expf((c < 2 ? cum0 : cum1) - cum_s[j]) * dt_s[j]) : 0.f;
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
      const __nv_bfloat16* b = xt + (nt * 8 + g) * TP + kj * 16 + 2 * t;
      const unsigned b0 = lc_word(b), b1 = lc_word(b + 8);
      mma_bf16(acc[nt], hi, b0, b1);
      mma_bf16(acc[nt], lo, b0, b1);
    }
  }
  const float skip = a.d_skip[head];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int c = nt * 8 + 2 * t;
    float* out = a.y + (size_t)row0 * a.s.inner + head * P + c;
    if (r0 < n)
      *reinterpret_cast<float2*>(out + (size_t)r0 * a.s.inner) =
          make_float2(fmaf(skip, __bfloat162float(xt[c * TP + r0]), acc[nt][0]), fmaf(skip, __bfloat162float(xt[(c + 1) * TP + r0]), acc[nt][1]));
    if (r1 < n)
      *reinterpret_cast<float2*>(out + (size_t)r1 * a.s.inner) =
          make_float2(fmaf(skip, __bfloat162float(xt[c * TP + r1]), acc[nt][2]), fmaf(skip, __bfloat162float(xt[(c + 1) * TP + r1]), acc[nt][3]));
  }
}

template <int N, int P>
static int launch_mamba_chunks(const MambaChunkArgs& a, int chunks, cudaStream_t st) {
  const size_t smem1 = (size_t)(2 * N + P) * (LC_TOKENS + LC_PAD) * 2;
  const size_t smem3 = ((size_t)2 * LC_TOKENS * (N + LC_PAD) + (size_t)P * (LC_TOKENS + LC_PAD) + (size_t)2 * P * (N + LC_PAD)) * 2;
  SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_chunk_states_kernel<N, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
  SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_chunk_outputs_kernel<N, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3));
  SRB_CUDA_CALL(srb_launch(mamba_chunk_states_kernel<N, P>, dim3(chunks, a.s.heads), dim3(MC_THREADS), smem1, st, a));
  SRB_LAUNCH_CHECK("mamba_chunk_states");
  const int entries = N * P;
  SRB_CUDA_CALL(srb_launch(mamba_chunk_prefix_kernel, dim3((entries + 255) / 256, a.s.heads, a.requests), dim3(256), 0, st, a, entries));
  SRB_LAUNCH_CHECK("mamba_chunk_prefix");
  SRB_CUDA_CALL(srb_launch(mamba_chunk_outputs_kernel<N, P>, dim3(chunks, a.s.heads), dim3(MC_OUT_THREADS), smem3, st, a));
  SRB_LAUNCH_CHECK("mamba_chunk_outputs");
  return SRB_OK;
}

// Tokens of a chunk, and whether these sizes are taken (bfloat16; N and P 64 or 128 each).
extern "C" int srb_mamba_chunk_tokens() { return LC_TOKENS; }
extern "C" int srb_mamba_chunks_supports(int vdim, int nstate, int dtype) {
  return dtype == SRB_DTYPE_BF16 && (nstate == 64 || nstate == 128) && (vdim == 64 || vdim == 128);
}

// What srb_mamba_scan computes, for prompt portions in bfloat16.  `xbc`: bfloat16 [rows, channels] (srb_mamba_conv with a
// bfloat16 result); `chunks`: at least the number of chunks of the step, sum over the requests of ceil(rows /
// srb_mamba_chunk_tokens()); `scratch`: chunks * heads * (N * P + 1) floats.
extern "C" int srb_mamba_chunks(const void* proj, long long proj_pitch, const void* xbc, const float* a_log, const float* d_skip,
                                const float* dt_bias, const int* positions, const int* cu_rows, const int* state_slots,
                                float* state, long long slot_floats, float* scratch, float* y, int rows, int requests, int chunks,
                                int heads, int vdim, int nstate, int groups, int taps, int write_state, void* stream) {
  if (rows <= 0 || requests <= 0 || chunks <= 0) return SRB_OK;
  MambaChunkArgs a;
  if (mamba_shape(a.s, heads, vdim, nstate, groups, taps, proj_pitch, slot_floats) != SRB_OK) return SRB_ERR_INVALID;
  if (!srb_mamba_chunks_supports(vdim, nstate, SRB_DTYPE_BF16))
    SRB_FAIL("mamba_chunks: a state of %d x %d per head is not taken (64 or 128 each)", nstate, vdim);
  if (heads > 65535 || requests > 65535) SRB_FAIL("mamba_chunks: %d heads or %d requests exceed one launch", heads, requests);
  if (((uintptr_t)xbc & 15) || ((uintptr_t)scratch & 15)) SRB_FAIL("mamba_chunks: the convolved inputs and the scratch must start on 16-byte borders");
  a.proj = (const __nv_bfloat16*)proj; a.xbc = (const __nv_bfloat16*)xbc; a.a_log = a_log; a.d_skip = d_skip; a.dt_bias = dt_bias;
  a.cu_rows = cu_rows; a.positions = positions; a.state_slots = state_slots; a.state = state;
  a.chunk_states = scratch; a.chunk_decay = scratch + (size_t)chunks * heads * nstate * vdim; a.y = y;
  a.requests = requests; a.write_state = write_state;
  cudaStream_t st = (cudaStream_t)stream;
  if (nstate == 64 && vdim == 64) return launch_mamba_chunks<64, 64>(a, chunks, st);
  if (nstate == 64) return launch_mamba_chunks<64, 128>(a, chunks, st);
  if (vdim == 64) return launch_mamba_chunks<128, 64>(a, chunks, st);
  return launch_mamba_chunks<128, 128>(a, chunks, st);
}
