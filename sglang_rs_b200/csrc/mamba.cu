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
//   srb_mamba_conv        the convolution + SiLU of every row of the step (32-bit result), reading earlier rows of the
//                         same request from the step and, before the step's first row, from the slot; then the slot's
//                         inputs are replaced by the last taps - 1 of the sequence (a second launch: rows read the old ones)
//   srb_mamba_scan        the recurrence, token by token: a block owns a head's N x PB slice of the state in registers
//                         (PB columns, N cut over the lanes beside each column), stages 16 tokens' B, C, x, dt at a time in
//                         shared memory and walks them; decoded tokens and prompt portions take the same arithmetic, so a
//                         row's result does not depend on how the sequence was cut
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

template <typename T>
__global__ void mamba_conv_kernel(const T* __restrict__ proj, const float* __restrict__ weight, const float* __restrict__ bias,
                                  const int* __restrict__ positions, const int* __restrict__ row_request,
                                  const int* __restrict__ cu_rows, const int* __restrict__ state_slots,
                                  const float* __restrict__ state, float* __restrict__ out, MambaShape s) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= s.channels) return;
  const int pos = positions[row];
  float* dst = out + (size_t)row * s.channels + c;
  if (pos < 0) { *dst = 0.f; return; }
  const int request = row_request[row];
  const int ahead = row - cu_rows[request];            // rows of this request before this one in the step
  const float* kept = state + (size_t)state_slots[request] * s.slot_floats;
  float acc = bias[c];
  for (int j = 0; j < s.taps; ++j) {
    const int back = s.taps - 1 - j;
    if (pos - back < 0) continue;                      // zeros before the start of the sequence
    float u;
    if (back <= ahead)
      u = srb_to_float(proj[(size_t)(row - back) * s.proj_pitch + s.inner + c]);
    else
      u = kept[(size_t)(s.taps - 1 - (back - ahead)) * s.channels + c];
    acc = fmaf(weight[(size_t)c * s.taps + j], u, acc);
  }
  *dst = mamba_silu(acc);
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

// grid (rows, norm groups): out = rms_part(y * silu(z)) * weight
template <typename T>
__global__ void mamba_gate_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, long long proj_pitch,
                                       const float* __restrict__ weight, float eps, int inner, int part,
                                       T* __restrict__ out) {
  extern __shared__ float gate_smem[];                  // part floats, then 33 of scratch
  float* scratch = gate_smem + part;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x, base = blockIdx.y * part;
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

// proj: [rows, pitch]; weight [channels, taps], bias [channels] (float); out: float [rows, channels]
extern "C" int srb_mamba_conv(const void* proj, long long proj_pitch, const float* weight, const float* bias,
                              const int* positions, const int* row_request, const int* cu_rows, const int* state_slots,
                              float* state, long long slot_floats, float* out, int rows, int requests, int heads, int vdim,
                              int nstate, int groups, int taps, int write_state, int dtype, void* stream) {
  if (rows <= 0 || requests <= 0) return SRB_OK;
  MambaShape s;
  if (mamba_shape(s, heads, vdim, nstate, groups, taps, proj_pitch, slot_floats) != SRB_OK) return SRB_ERR_INVALID;
  if (requests > 65535) SRB_FAIL("mamba_conv: %d requests exceed one launch", requests);
  cudaStream_t st = (cudaStream_t)stream;
  const int block = 128;
  const dim3 grid(rows, (s.channels + block - 1) / block), keep_grid((s.channels + block - 1) / block, requests);
  if (dtype == SRB_DTYPE_F32) {
    SRB_CUDA_CALL(srb_launch(mamba_conv_kernel<float>, grid, dim3(block), 0, st, (const float*)proj, weight, bias, positions,
                             row_request, cu_rows, state_slots, (const float*)state, out, s));
    if (write_state && taps > 1)
      SRB_CUDA_CALL(srb_launch(mamba_conv_keep_kernel<float>, keep_grid, dim3(block), 0, st, (const float*)proj, positions,
                               cu_rows, state_slots, state, s));
  } else if (dtype == SRB_DTYPE_BF16) {
    SRB_CUDA_CALL(srb_launch(mamba_conv_kernel<__nv_bfloat16>, grid, dim3(block), 0, st, (const __nv_bfloat16*)proj, weight,
                             bias, positions, row_request, cu_rows, state_slots, (const float*)state, out, s));
    if (write_state && taps > 1)
      SRB_CUDA_CALL(srb_launch(mamba_conv_keep_kernel<__nv_bfloat16>, keep_grid, dim3(block), 0, st,
                               (const __nv_bfloat16*)proj, positions, cu_rows, state_slots, state, s));
  } else {
    SRB_FAIL("mamba_conv: unknown dtype %d", dtype);
  }
  SRB_LAUNCH_CHECK("mamba_conv");
  return SRB_OK;
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
  if (norm_groups > 65535) SRB_FAIL("mamba_gate_norm: %d parts exceed one launch", norm_groups);
  const int part = inner / norm_groups;
  const size_t smem = (size_t)(part + 33) * sizeof(float);
  if (smem > 227 * 1024) SRB_FAIL("mamba_gate_norm: a part of %d entries needs %zu bytes of shared memory (limit 232448)", part, smem);
  const int block = part >= 2048 ? 512 : (part >= 512 ? 256 : 128);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32) {
    if (smem > 48 * 1024) SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_gate_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(mamba_gate_norm_kernel<float>, dim3(rows, norm_groups), dim3(block), smem, st, y, (const float*)proj,
                             proj_pitch, weight, eps, inner, part, (float*)out));
  } else if (dtype == SRB_DTYPE_BF16) {
    if (smem > 48 * 1024) SRB_CUDA_CALL(cudaFuncSetAttribute(mamba_gate_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(mamba_gate_norm_kernel<__nv_bfloat16>, dim3(rows, norm_groups), dim3(block), smem, st, y,
                             (const __nv_bfloat16*)proj, proj_pitch, weight, eps, inner, part, (__nv_bfloat16*)out));
  } else {
    SRB_FAIL("mamba_gate_norm: unknown dtype %d", dtype);
  }
  SRB_LAUNCH_CHECK("mamba_gate_norm");
  return SRB_OK;
}
