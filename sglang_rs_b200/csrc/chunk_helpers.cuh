// Shared by the kernels that walk a sequence in chunks of LC_TOKENS tokens on the tensor cores (linear attention with a
// fixed decay, the state-space mixer): 16-byte loads of bfloat16 rows, the transposed copy of a chunk's slice into
// shared memory, and the split of a 32-bit number into two bfloat16 operands (its rounding and the rounding of the
// rest: 16 bits of mantissa survive two products).
#pragma once
#include "mma_helpers.cuh"

#define LC_TOKENS 128
#define LC_PAD 8

__device__ __forceinline__ unsigned lc_word(const __nv_bfloat16* p) { return *reinterpret_cast<const unsigned*>(p); }

__device__ __forceinline__ void lc_split(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(v);
  lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

struct Bf16x8 { __nv_bfloat16 v[8]; };
__device__ __forceinline__ Bf16x8 lc_load8(const __nv_bfloat16* p, bool live) {
  Bf16x8 r;
  uint4 raw = make_uint4(0u, 0u, 0u, 0u);
  if (live) raw = *reinterpret_cast<const uint4*>(p);
  *reinterpret_cast<uint4*>(r.v) = raw;
  return r;
}

// Loads a [LC_TOKENS, WIDTH] slice of the (activated) projection, transposed, into `dst` [WIDTH][TP]: consecutive lanes
// take consecutive tokens, so the 2-byte stores of a warp fall into consecutive words.  `scale` (or null) gives a
// factor per token, token j's at scale[scale_first + scale_step * j]; with it the product goes in as two bfloat16 numbers
// (dst, dst_lo).
template <int WIDTH, int THREADS>
__device__ __forceinline__ void lc_load_transposed(const __nv_bfloat16* src, long long pitch, int n, const float* scale,
                                                   int scale_first, int scale_step, __nv_bfloat16* dst, __nv_bfloat16* dst_lo) {
  constexpr int TP = LC_TOKENS + LC_PAD, ITEMS = LC_TOKENS * WIDTH / 8, PER = ITEMS / THREADS, BATCH = PER < 8 ? PER : 8;
#pragma unroll 1
  for (int first = 0; first < PER; first += BATCH) {          // eight loads of a thread in flight at a time
    Bf16x8 x[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int item = threadIdx.x + (first + i) * THREADS, j = item % LC_TOKENS, d0 = item / LC_TOKENS * 8;
      x[i] = lc_load8(src + (size_t)j * pitch + d0, j < n);
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int item = threadIdx.x + (first + i) * THREADS, j = item % LC_TOKENS, d0 = item / LC_TOKENS * 8;
      const float factor = (scale && j < n) ? scale[scale_first + scale_step * j] : 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (scale) {
          __nv_bfloat16 hi, lo;
          lc_split(factor * __bfloat162float(x[i].v[k]), hi, lo);
          dst[(d0 + k) * TP + j] = hi;
          dst_lo[(d0 + k) * TP + j] = lo;
        } else {
          dst[(d0 + k) * TP + j] = x[i].v[k];
        }
      }
    }
  }
}

