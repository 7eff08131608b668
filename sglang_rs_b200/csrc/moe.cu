// A feed-forward of routed experts: every row goes through `top` of `experts` small gated feed-forwards
// and their results are summed with the router's weights.
//
//   srb_moe_route     logits = router . h in 32-bit, scores = softmax over all experts, the `top` largest are
//                     chosen (ties: the lower index); weights are the chosen scores, or those divided by their
//                     sum if `renormalize`
//   srb_moe_plan      groups the (row, choice) entries by expert: a slot for each entry, the row of each slot, the
//                     first slot of each expert, and the list of row tiles that the two products walk
//   srb_moe_gated_up  act[slot, :] = activation(W_gate[e] h[row]) * (W_up[e] h[row])   for the slot's expert and row
//   srb_moe_act_up    act[slot, :] = activation(W_up[e] h[row])                        (experts without a gate)
//   srb_moe_down      y[slot, :]   = W_down[e] act[slot]                              (32-bit result)
//   srb_moe_combine   out[row, :]  = sum over the row's choices, in their order, of weight * y[slot]   (32-bit)
//
// The router may have more outputs than there are experts with matrices (srb_moe_route / srb_moe_select are then called
// with the number of outputs, srb_moe_plan and the products with the number of experts): a choice beyond the experts gets
// no slot, the products never see it, and srb_moe_combine_identity adds weight * h[row] for it: an expert that returns
// its input.
//
// Nothing here is decided on the host: counts, offsets and tiles stay on the device, the products are
// launched for the largest number of tiles the step can need, and blocks without a tile leave at once.
// Every output element is accumulated in 32-bit over the inner index in order by one thread, so a row's
// result depends neither on the slot it got nor on the rows beside it.
#include "common.cuh"
#include "activations.cuh"
#include "tile_mma.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define MOE_ROWS 128     // rows of a tile of the plan: slots of one expert that one block (or two) takes
#define MOE_FEW_ROWS 32  // ... when the step's choices are few per expert (decoded tokens): tiles are then almost empty,
                         // and the products' blocks trade the rows of the A buffer for stages of weights in flight
#define MOE_FEW_STAGES 4

// The tile size is a function of the step's shape only, so every launch of a step agrees on it.
static inline int moe_tile_rows(int rows, int top, int experts) {
  return (long long)rows * top <= 8LL * experts ? MOE_FEW_ROWS : MOE_ROWS;
}
#define MOE_TILE 64      // rows that the smaller kernels take at a time (half a tile), and output columns of a block
#define MOE_K 16
#define MOE_MAX_EXPERTS 1024

// How the router's logits become a choice and weights.  `scoring` 0: scores are a softmax over all experts; 1: each
// expert's score is the sigmoid of its logit.  `choice_bias` (one float per expert, or null) is added to the scores for
// the choice only; the weights are the chosen experts' scores without it, divided by their sum plus `norm_eps` if
// `renormalize`, then multiplied by `scale`.
struct RouteRule {
  int scoring;
  int renormalize;
  const float* choice_bias;
  float scale;
  float norm_eps;
};
#define MOE_SCORE_SOFTMAX 0
#define MOE_SCORE_SIGMOID 1

// One warp.  `score` holds the row's logits on entry; `pick` is scratch of the same length.  The `top` experts with
// the largest choice scores are taken (ties: the lower index).
__device__ __forceinline__ void moe_choose(float* score, float* pick, int experts, int top, const RouteRule& rule, int lane,
                                           int* __restrict__ chosen, float* __restrict__ weights) {
  float sum = 1.f;
  if (rule.scoring == MOE_SCORE_SIGMOID) {
    for (int e = lane; e < experts; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
  } else {
    float top_logit = -INFINITY;
    for (int e = lane; e < experts; e += 32) top_logit = fmaxf(top_logit, score[e]);
    top_logit = srb_warp_max(top_logit);
    sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
      const float p = expf(score[e] - top_logit);
      score[e] = p;
      sum += p;
    }
    sum = srb_warp_sum(sum);
  }
  for (int e = lane; e < experts; e += 32) pick[e] = rule.choice_bias ? score[e] / sum + rule.choice_bias[e] : score[e];
  __syncwarp();
  float kept = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_index = experts;
    for (int e = lane; e < experts; e += 32)
      if (pick[e] > best) { best = pick[e]; best_index = e; }          // the first of equals within a lane
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
      if (other > best || (other == best && other_index < best_index)) { best = other; best_index = other_index; }
    }
    if (best_index >= experts) best_index = 0;                          // only if every score left is not a number
    const float weight = score[best_index] / sum;
    if (lane == 0) {
      chosen[k] = best_index;
      weights[k] = weight;
      pick[best_index] = -INFINITY;                                     // never chosen again
    }
    kept += weight;
    __syncwarp();
  }
  if (lane < top) {
    float w = weights[lane];
    if (rule.renormalize) w /= kept + rule.norm_eps;
    weights[lane] = w * rule.scale;
  }
}

// One block per row.  Warps share the experts' dot products; warp 0 then picks the largest scores.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const T* __restrict__ router, int width, int experts, int top,
                                 RouteRule rule, int* __restrict__ chosen, float* __restrict__ weights) {
  __shared__ float score[MOE_MAX_EXPERTS];
  __shared__ float pick[MOE_MAX_EXPERTS];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* x = h + (size_t)row * width;
  if (sizeof(T) == 2 && width % 8 == 0 && (((uintptr_t)h | (uintptr_t)router) & 15) == 0) {
    // 16-byte loads: a lane's pieces of the row stay in registers for every expert of its warp (up to 4 pieces:
    // widths to 1024; wider rows read the later pieces again per expert)
    const int pieces = width / 8;
    uint4 mine[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      mine[j] = lane + 32 * j < pieces ? *reinterpret_cast<const uint4*>(x + (size_t)(lane + 32 * j) * 8) : make_uint4(0u, 0u, 0u, 0u);
    for (int e = warp; e < experts; e += warps) {
      const T* w = router + (size_t)e * width;
      float partial = 0.f;
      for (int piece = lane, j = 0; piece < pieces; piece += 32, ++j) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + (size_t)piece * 8);
        const uint4 xv = j < 4 ? mine[j < 4 ? j : 0] : *reinterpret_cast<const uint4*>(x + (size_t)piece * 8);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 a = __bfloat1622float2(x2[q]), b = __bfloat1622float2(w2[q]);
          partial = fmaf(a.x, b.x, partial);
          partial = fmaf(a.y, b.y, partial);
        }
      }
      partial = srb_warp_sum(partial);
      if (lane == 0) score[e] = partial;
    }
  } else {
    for (int e = warp; e < experts; e += warps) {
      const T* w = router + (size_t)e * width;
      float partial = 0.f;
      for (int i = lane; i < width; i += 32) partial += srb_to_float(x[i]) * srb_to_float(w[i]);
      partial = srb_warp_sum(partial);
      if (lane == 0) score[e] = partial;
    }
  }
  __syncthreads();
  if (warp != 0) return;
  moe_choose(score, pick, experts, top, rule, lane, chosen + (size_t)row * top, weights + (size_t)row * top);
}

extern "C" int srb_moe_route_ex(const void* h, const void* router, int rows, int width, int experts, int top, int renormalize,
                                int scoring, const float* choice_bias, float scale, float norm_eps, int* chosen, float* weights,
                                int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (scoring != MOE_SCORE_SOFTMAX && scoring != MOE_SCORE_SIGMOID) SRB_FAIL("moe_route: unknown scoring %d", scoring);
  const RouteRule rule{scoring, renormalize, choice_bias, scale, norm_eps};
  if (experts <= 0 || experts > MOE_MAX_EXPERTS) SRB_FAIL("moe_route: %d experts are outside 1 .. %d", experts, MOE_MAX_EXPERTS);
  if (top <= 0 || top > experts || top > 32) SRB_FAIL("moe_route: %d chosen experts are outside 1 .. min(%d, 32)", top, experts);
  if (width <= 0) SRB_FAIL("moe_route: width %d must be positive", width);
  cudaStream_t s = (cudaStream_t)stream;
  const int block = experts >= 32 ? 1024 : 32 * experts;          // a warp per expert, up to 32 warps
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(moe_route_kernel<float>, dim3(rows), dim3(block), 0, s, (const float*)h, (const float*)router,
                             width, experts, top, rule, chosen, weights));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(moe_route_kernel<__nv_bfloat16>, dim3(rows), dim3(block), 0, s, (const __nv_bfloat16*)h,
                             (const __nv_bfloat16*)router, width, experts, top, rule, chosen, weights));
  else
    SRB_FAIL("moe_route: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("moe_route");
  return SRB_OK;
}

extern "C" int srb_moe_route(const void* h, const void* router, int rows, int width, int experts, int top, int renormalize,
                             int* chosen, float* weights, int dtype, void* stream) {
  return srb_moe_route_ex(h, router, rows, width, experts, top, renormalize, MOE_SCORE_SOFTMAX, nullptr, 1.0f, 0.0f, chosen,
                          weights, dtype, stream);
}

// The choice alone, from logits that a product kernel made (float [rows, experts], `pitch` floats apart): a warp per
// row does the softmax over all experts and picks the `top` largest as moe_route_kernel does.
__global__ void moe_select_kernel(const float* __restrict__ logits, size_t pitch, int rows, int experts, int top,
                                  RouteRule rule, int* __restrict__ chosen, float* __restrict__ weights) {
  extern __shared__ float select_scores[];                  // [warps of the block][2][experts]
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  float* score = select_scores + (size_t)warp * 2 * experts;
  const float* z = logits + (size_t)row * pitch;
  for (int e = lane; e < experts; e += 32) score[e] = z[e];
  moe_choose(score, score + experts, experts, top, rule, lane, chosen + (size_t)row * top, weights + (size_t)row * top);
}

extern "C" int srb_moe_select_ex(const float* logits, long long pitch, int rows, int experts, int top, int renormalize,
                                 int scoring, const float* choice_bias, float scale, float norm_eps, int* chosen,
                                 float* weights, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (scoring != MOE_SCORE_SOFTMAX && scoring != MOE_SCORE_SIGMOID) SRB_FAIL("moe_select: unknown scoring %d", scoring);
  const RouteRule rule{scoring, renormalize, choice_bias, scale, norm_eps};
  if (experts <= 0 || experts > MOE_MAX_EXPERTS) SRB_FAIL("moe_select: %d experts are outside 1 .. %d", experts, MOE_MAX_EXPERTS);
  if (top <= 0 || top > experts || top > 32) SRB_FAIL("moe_select: %d chosen experts are outside 1 .. min(%d, 32)", top, experts);
  if (pitch < experts) SRB_FAIL("moe_select: rows of the logits overlap");
  const int warps = 4;
  SRB_CUDA_CALL(srb_launch(moe_select_kernel, dim3((rows + warps - 1) / warps), dim3(32 * warps), (size_t)warps * experts * 8,
                           (cudaStream_t)stream, logits, (size_t)pitch, rows, experts, top, rule, chosen, weights));
  SRB_LAUNCH_CHECK("moe_select");
  return SRB_OK;
}

extern "C" int srb_moe_select(const float* logits, long long pitch, int rows, int experts, int top, int renormalize,
                              int* chosen, float* weights, void* stream) {
  return srb_moe_select_ex(logits, pitch, rows, experts, top, renormalize, MOE_SCORE_SOFTMAX, nullptr, 1.0f, 0.0f, chosen,
                           weights, stream);
}

// One block.  plan: [0] number of tiles, then offsets[experts + 1], then per tile (expert, first slot).
// slot_row[slot]: the row whose entry sits in the slot; entry_slot[row * top + k]: the slot of that entry.
__global__ void moe_plan_kernel(const int* __restrict__ chosen, int entries, int top, int experts, int max_tiles,
                                int tile_rows, int* __restrict__ plan, int* __restrict__ slot_row, int* __restrict__ entry_slot,
                                int* error_word) {
  __shared__ int count[MOE_MAX_EXPERTS];
  __shared__ int first[MOE_MAX_EXPERTS + 1];
  __shared__ int tile_first[MOE_MAX_EXPERTS + 1];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int slots = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = slots;
      tile_first[e] = tiles;
      slots += count[e];
      tiles += (count[e] + tile_rows - 1) / tile_rows;
    }
    first[experts] = slots;
    tile_first[experts] = tiles;
    plan[0] = tiles <= max_tiles ? tiles : max_tiles;
    if (tiles > max_tiles) atomicOr(error_word, SRB_FLAG_BAD_SLOT);
  }
  __syncthreads();
  int* offsets = plan + 1;
  int* tiles = plan + 1 + experts + 1;
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = first[e];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = tile_first[e + 1] - tile_first[e];
    for (int t = 0; t < n; ++t) {
      const int at = tile_first[e] + t;
      if (at < max_tiles) {
        tiles[2 * at] = e;
        tiles[2 * at + 1] = first[e] + t * tile_rows;
      }
    }
    count[e] = 0;                       // becomes the number of the expert's slots handed out so far
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = chosen[i];
    if (e < 0 || e >= experts) { entry_slot[i] = -1; continue; }
    const int slot = first[e] + atomicAdd(&count[e], 1);
    slot_row[slot] = i / top;
    entry_slot[i] = slot;
  }
}

extern "C" int srb_moe_plan_ints(int rows, int top, int experts) {
  const int max_tiles = (rows * top) / moe_tile_rows(rows, top, experts) + experts;
  return 1 + experts + 1 + 2 * max_tiles;
}

// The same plan with tiles of a size that the caller names (a product kernel with tiles of its own, e.g. 256 slots);
// the products of this file do not read such a plan.
extern "C" int srb_moe_plan_ints_of(int rows, int top, int experts, int tile_rows) {
  return 1 + experts + 1 + 2 * ((rows * top) / tile_rows + experts);
}
extern "C" int srb_moe_max_tiles_of(int rows, int top, int experts, int tile_rows) { return (rows * top) / tile_rows + experts; }
extern "C" int srb_moe_plan_of(const int* chosen, int rows, int top, int experts, int tile_rows, int* plan, int* slot_row,
                               int* entry_slot, int* error_word, void* stream);

extern "C" int srb_moe_max_tiles(int rows, int top, int experts) {
  return (rows * top) / moe_tile_rows(rows, top, experts) + experts;
}

extern "C" int srb_moe_plan_of(const int* chosen, int rows, int top, int experts, int tile_rows, int* plan, int* slot_row,
                               int* entry_slot, int* error_word, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || tile_rows <= 0)
    SRB_FAIL("moe_plan: %d experts, %d chosen, tiles of %d", experts, top, tile_rows);
  SRB_CUDA_CALL(srb_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, chosen, rows * top, top, experts,
                           (rows * top) / tile_rows + experts, tile_rows, plan, slot_row, entry_slot, error_word));
  SRB_LAUNCH_CHECK("moe_plan");
  return SRB_OK;
}

extern "C" int srb_moe_plan(const int* chosen, int rows, int top, int experts, int* plan, int* slot_row, int* entry_slot,
                            int* error_word, void* stream) {
  return srb_moe_plan_of(chosen, rows, top, experts, moe_tile_rows(rows, top, experts), plan, slot_row, entry_slot, error_word,
                         stream);
}

// Half a tile (up to 64 slots of one expert; blockIdx.z names the half) times 64 output columns.  GATED: two weight matrices (gate, up), rows of
// x gathered through slot_row, result act(gate) * up in T.  Otherwise one matrix, rows of x are the slots
// themselves, result in float.  MODE: MOE_DOWN (one matrix, rows are the slots, float result), MOE_GATED (two matrices,
// rows gathered, act(gate) * up in T), MOE_ACT (one matrix, rows gathered, act(product) in T).
#define MOE_DOWN 0
#define MOE_GATED 1
#define MOE_ACT 2
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_product_kernel(const T* __restrict__ x, const T* __restrict__ w_a, const T* __restrict__ w_b,
                   const int* __restrict__ plan, const int* __restrict__ slot_row, int experts, int n_in, int n_out,
                   int activation, float act_param, T* __restrict__ out_t, float* __restrict__ out_f, int tile_rows, size_t expert_stride) {
  constexpr bool GATED = MODE == MOE_GATED, GATHER = MODE != MOE_DOWN;
  __shared__ float x_tile[MOE_K][MOE_TILE + 4];
  __shared__ float a_tile[MOE_K][MOE_TILE + 4];
  __shared__ float b_tile[GATED ? MOE_K : 1][MOE_TILE + 4];
  __shared__ int tile_row[MOE_TILE];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* offsets = plan + 1;
  const int* tiles = plan + 1 + experts + 1;
  const int expert = tiles[2 * tile], first = tiles[2 * tile + 1] + MOE_TILE * blockIdx.z;
  const int count = min(min(MOE_TILE, tile_rows - MOE_TILE * (int)blockIdx.z), offsets[expert + 1] - first);
  if (count <= 0) return;
  const int t = threadIdx.x;
  if (t < MOE_TILE) tile_row[t] = t < count ? (GATHER ? slot_row[first + t] : first + t) : -1;
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int col0 = blockIdx.x * MOE_TILE;
  const T* wa = w_a + (size_t)expert * expert_stride;
  const T* wb = GATED ? w_b + (size_t)expert * expert_stride : nullptr;
  float acc_a[4][4] = {}, acc_b[GATED ? 4 : 1][4] = {};
  for (int k0 = 0; k0 < n_in; k0 += MOE_K) {
    for (int i = threadIdx.x; i < MOE_TILE * MOE_K; i += 256) {
      const int r = i / MOE_K, kk = i % MOE_K;
      const int gk = k0 + kk;
      const int source = tile_row[r];
      x_tile[kk][r] = (source >= 0 && gk < n_in) ? srb_to_float(x[(size_t)source * n_in + gk]) : 0.f;
      const bool inside = col0 + r < n_out && gk < n_in;
      a_tile[kk][r] = inside ? srb_to_float(wa[(size_t)(col0 + r) * n_in + gk]) : 0.f;
      if (GATED) b_tile[kk][r] = inside ? srb_to_float(wb[(size_t)(col0 + r) * n_in + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MOE_K; ++kk) {
      float xv[4], av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = x_tile[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        av[j] = a_tile[kk][tx * 4 + j];
        if (GATED) bv[j] = b_tile[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc_a[i][j] = fmaf(xv[i], av[j], acc_a[i][j]);
          if (GATED) acc_b[i][j] = fmaf(xv[i], bv[j], acc_b[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= count) continue;
    const size_t slot = (size_t)first + r;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= n_out) continue;
      if (GATED)
        out_t[slot * n_out + c] = srb_from_float<T>(srb_gated<true>(activation, acc_a[i][j], acc_b[i][j], act_param));
      else if (MODE == MOE_ACT)
        out_t[slot * n_out + c] = srb_from_float<T>(srb_gated<true>(activation, acc_a[i][j], 1.0f, act_param));
      else
        out_f[slot * n_out + c] = acc_a[i][j];
    }
  }
}

// The same tile on the tensor cores (bfloat16): tile_mma.cuh.
template <int MODE>
__global__ void __launch_bounds__(128)
moe_product_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_a,
                       const __nv_bfloat16* __restrict__ w_b, const int* __restrict__ plan,
                       const int* __restrict__ slot_row, int experts, int n_in, int n_out, int activation, float act_param,
                       __nv_bfloat16* __restrict__ out_t, float* __restrict__ out_f, int tile_rows, size_t expert_stride) {
  constexpr bool GATED = MODE == MOE_GATED, GATHER = MODE != MOE_DOWN;
  __shared__ __align__(16) TileMmaSmem s;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* offsets = plan + 1;
  const int* tiles = plan + 1 + experts + 1;
  const int expert = tiles[2 * tile], first = tiles[2 * tile + 1] + MOE_TILE * blockIdx.z;
  const int count = min(min(MOE_TILE, tile_rows - MOE_TILE * (int)blockIdx.z), offsets[expert + 1] - first);
  if (count <= 0) return;
  const int t = threadIdx.x;
  if (t < MOE_TILE) s.a_row[t] = t < count ? x + (size_t)(GATHER ? slot_row[first + t] : first + t) * n_in : nullptr;
  __syncthreads();
  const int col0 = blockIdx.x * MOE_TILE;
  const size_t matrix = (size_t)expert * expert_stride + (size_t)col0 * n_in;
  constexpr int NW = GATED ? 2 : 1;
  float acc[NW][2][4][4];
  if (GATED) {
    const __nv_bfloat16* const bases[2] = {w_a + matrix, w_b + matrix};
    tile_mma_64x64<NW>(s, reinterpret_cast<const __nv_bfloat16* const(&)[NW]>(bases), n_out - col0, n_in, acc);
  } else {
    const __nv_bfloat16* const bases[2] = {w_a + matrix, nullptr};
    tile_mma_64x64<NW>(s, reinterpret_cast<const __nv_bfloat16* const(&)[NW]>(bases), n_out - col0, n_in, acc);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = tile_mma_row(i, c), col = col0 + tile_mma_col(j, c);
        if (r >= count || col >= n_out) continue;
        const size_t at = ((size_t)first + r) * n_out + col;
        if (GATED)
          out_t[at] = __float2bfloat16_rn(srb_gated<true>(activation, acc[0][i][j][c], acc[NW - 1][i][j][c], act_param));
        else if (MODE == MOE_ACT)
          out_t[at] = __float2bfloat16_rn(srb_gated<true>(activation, acc[0][i][j][c], 1.0f, act_param));
        else
          out_f[at] = acc[0][i][j][c];
      }
}

// A whole tile (up to 128 slots) times 64 output columns, operands through a ring of asynchronous copies
// (tile_mma.cuh); for rows that start on 16-byte boundaries.
template <int MODE, int ROWS, int STAGES>
__global__ void __launch_bounds__(256)
moe_product_async_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_a,
                         const __nv_bfloat16* __restrict__ w_b, const int* __restrict__ plan,
                         const int* __restrict__ slot_row, int experts, int n_in, int n_out, int activation, float act_param,
                         __nv_bfloat16* __restrict__ out_t, float* __restrict__ out_f, size_t expert_stride) {
  constexpr bool GATED = MODE == MOE_GATED, GATHER = MODE != MOE_DOWN;
  constexpr int NW = GATED ? 2 : 1;
  extern __shared__ __align__(16) unsigned char moe_smem[];
  TileAsyncSmem<NW, ROWS, STAGES>& s = *reinterpret_cast<TileAsyncSmem<NW, ROWS, STAGES>*>(moe_smem);
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* offsets = plan + 1;
  const int* tiles = plan + 1 + experts + 1;
  const int expert = tiles[2 * tile], first = tiles[2 * tile + 1];
  const int count = min(ROWS, offsets[expert + 1] - first);
  const int t = threadIdx.x;
  if (t < ROWS) s.a_row[t] = t < count ? x + (size_t)(GATHER ? slot_row[first + t] : first + t) * n_in : nullptr;
  __syncthreads();
  const int col0 = blockIdx.x * TA_COLS;
  const size_t matrix = (size_t)expert * expert_stride + (size_t)col0 * n_in;
  float acc[NW][2][4][4];
  if (GATED) {
    const __nv_bfloat16* const bases[2] = {w_a + matrix, w_b + matrix};
    tile_mma_128x64_async<NW, ROWS, STAGES>(s, reinterpret_cast<const __nv_bfloat16* const(&)[NW]>(bases), n_out - col0, count, n_in, acc);
  } else {
    const __nv_bfloat16* const bases[2] = {w_a + matrix, nullptr};
    tile_mma_128x64_async<NW, ROWS, STAGES>(s, reinterpret_cast<const __nv_bfloat16* const(&)[NW]>(bases), n_out - col0, count, n_in, acc);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; c += 2) {
        const int r = tile_async_row(i, c), col = col0 + tile_async_col(j, c);      // columns col and col + 1
        if (r >= count || col >= n_out) continue;
        const size_t at = ((size_t)first + r) * n_out + col;
        const bool pair = col + 1 < n_out;
        if (MODE != MOE_DOWN) {
          const float lo = srb_gated<true>(activation, acc[0][i][j][c], GATED ? acc[NW - 1][i][j][c] : 1.0f, act_param);
          const float hi = srb_gated<true>(activation, acc[0][i][j][c + 1], GATED ? acc[NW - 1][i][j][c + 1] : 1.0f, act_param);
          if (pair && (at & 1) == 0) {
            *reinterpret_cast<unsigned*>(out_t + at) = pack_bf16(lo, hi);
          } else {
            out_t[at] = __float2bfloat16_rn(lo);
            if (pair) out_t[at + 1] = __float2bfloat16_rn(hi);
          }
        } else if (pair && (at & 1) == 0) {
          *reinterpret_cast<float2*>(out_f + at) = make_float2(acc[0][i][j][c], acc[0][i][j][c + 1]);
        } else {
          out_f[at] = acc[0][i][j][c];
          if (pair) out_f[at + 1] = acc[0][i][j][c + 1];
        }
      }
}

template <typename T>
static int launch_moe_products(int mode, const void* x, const void* w_a, const void* w_b, const int* plan,
                               const int* slot_row, int rows, int top, int experts, int n_in, int n_out, int activation, float act_param,
                               void* out_t, float* out_f, size_t expert_stride, cudaStream_t s) {
  const int tile_rows = moe_tile_rows(rows, top, experts);
  dim3 grid((n_out + MOE_TILE - 1) / MOE_TILE, srb_moe_max_tiles(rows, top, experts), (tile_rows + MOE_TILE - 1) / MOE_TILE);
  if (grid.y > 65535) SRB_FAIL("moe product: %d tiles exceed one launch", (int)grid.y);
  if (sizeof(T) == 2 && n_in % 8 == 0 && (((uintptr_t)x | (uintptr_t)w_a | (uintptr_t)w_b) & 15) == 0) {
    // bfloat16 rows on 16-byte boundaries: whole tiles, operands by asynchronous copies
    grid.z = 1;
#define MOE_ASYNC_LAUNCH(MODE, ROWS, STAGES)                                                                           \
  do {                                                                                                                 \
    const size_t smem = sizeof(TileAsyncSmem<(MODE) == MOE_GATED ? 2 : 1, ROWS, STAGES>);                              \
    SRB_CUDA_CALL(cudaFuncSetAttribute(moe_product_async_kernel<MODE, ROWS, STAGES>,                                   \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                       \
    SRB_CUDA_CALL(srb_launch(moe_product_async_kernel<MODE, ROWS, STAGES>, grid, dim3(256), smem, s,                   \
                             (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_a, (const __nv_bfloat16*)w_b, plan,      \
                             slot_row, experts, n_in, n_out, activation, act_param, (__nv_bfloat16*)out_t, out_f, expert_stride)); \
  } while (0)
    if (tile_rows == MOE_FEW_ROWS) {
      if (mode == MOE_GATED) MOE_ASYNC_LAUNCH(MOE_GATED, MOE_FEW_ROWS, MOE_FEW_STAGES);
      else if (mode == MOE_ACT) MOE_ASYNC_LAUNCH(MOE_ACT, MOE_FEW_ROWS, MOE_FEW_STAGES);
      else MOE_ASYNC_LAUNCH(MOE_DOWN, MOE_FEW_ROWS, MOE_FEW_STAGES);
    } else {
      if (mode == MOE_GATED) MOE_ASYNC_LAUNCH(MOE_GATED, MOE_ROWS, TA_STAGES);
      else if (mode == MOE_ACT) MOE_ASYNC_LAUNCH(MOE_ACT, MOE_ROWS, TA_STAGES);
      else MOE_ASYNC_LAUNCH(MOE_DOWN, MOE_ROWS, TA_STAGES);
    }
#undef MOE_ASYNC_LAUNCH
    SRB_LAUNCH_CHECK("moe product");
    return SRB_OK;
  }
  if (sizeof(T) == 2) {
    // bfloat16: the tensor cores
#define MOE_MMA_LAUNCH(MODE)                                                                                             \
  SRB_CUDA_CALL(srb_launch(moe_product_mma_kernel<MODE>, grid, dim3(128), 0, s, (const __nv_bfloat16*)x,                 \
                           (const __nv_bfloat16*)w_a, (const __nv_bfloat16*)w_b, plan, slot_row, experts, n_in, n_out,   \
                           activation, act_param, (__nv_bfloat16*)out_t, out_f, tile_rows, expert_stride))
    if (mode == MOE_GATED) MOE_MMA_LAUNCH(MOE_GATED);
    else if (mode == MOE_ACT) MOE_MMA_LAUNCH(MOE_ACT);
    else MOE_MMA_LAUNCH(MOE_DOWN);
#undef MOE_MMA_LAUNCH
    SRB_LAUNCH_CHECK("moe product");
    return SRB_OK;
  }
#define MOE_PLAIN_LAUNCH(MODE)                                                                                           \
  SRB_CUDA_CALL(srb_launch(moe_product_kernel<T, MODE>, grid, dim3(256), 0, s, (const T*)x, (const T*)w_a, (const T*)w_b, \
                           plan, slot_row, experts, n_in, n_out, activation, act_param, (T*)out_t, out_f, tile_rows, expert_stride))
  if (mode == MOE_GATED) MOE_PLAIN_LAUNCH(MOE_GATED);
  else if (mode == MOE_ACT) MOE_PLAIN_LAUNCH(MOE_ACT);
  else MOE_PLAIN_LAUNCH(MOE_DOWN);
#undef MOE_PLAIN_LAUNCH
  SRB_LAUNCH_CHECK("moe product");
  return SRB_OK;
}

// h: [rows, width]; w_gate, w_up: expert e's [inner, width] matrix starts expert_stride elements after expert e - 1's
// (the two may be halves of one stacked tensor); act: [rows * top, inner]
extern "C" int srb_moe_gated_up(const void* h, const void* w_gate, const void* w_up, long long expert_stride, const int* plan,
                                const int* slot_row, int rows, int top, int experts, int width, int inner, int activation, float act_param,
                                void* act, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0 || inner <= 0) SRB_FAIL("moe_gated_up: sizes %d, %d must be positive", width, inner);
  if (activation < 0 || activation >= SRB_ACT_COUNT) SRB_FAIL("moe_gated_up: unknown activation %d", activation);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    return launch_moe_products<float>(MOE_GATED, h, w_gate, w_up, plan, slot_row, rows, top, experts, width, inner, activation, act_param, act, nullptr, (size_t)expert_stride, s);
  if (dtype == SRB_DTYPE_BF16)
    return launch_moe_products<__nv_bfloat16>(MOE_GATED, h, w_gate, w_up, plan, slot_row, rows, top, experts, width, inner, activation, act_param, act, nullptr, (size_t)expert_stride, s);
  SRB_FAIL("moe_gated_up: unknown dtype %d", dtype);
}

// The first product of experts without a gate: act[slot, :] = activation(W_up[e] h[row]); w_up: [experts, inner, width].
extern "C" int srb_moe_act_up(const void* h, const void* w_up, const int* plan, const int* slot_row, int rows, int top,
                              int experts, int width, int inner, int activation, float act_param, void* act, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0 || inner <= 0) SRB_FAIL("moe_act_up: sizes %d, %d must be positive", width, inner);
  if (activation < 0 || activation >= SRB_ACT_COUNT) SRB_FAIL("moe_act_up: unknown activation %d", activation);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t stride = (size_t)inner * width;
  if (dtype == SRB_DTYPE_F32)
    return launch_moe_products<float>(MOE_ACT, h, w_up, nullptr, plan, slot_row, rows, top, experts, width, inner, activation, act_param, act, nullptr, stride, s);
  if (dtype == SRB_DTYPE_BF16)
    return launch_moe_products<__nv_bfloat16>(MOE_ACT, h, w_up, nullptr, plan, slot_row, rows, top, experts, width, inner, activation, act_param, act, nullptr, stride, s);
  SRB_FAIL("moe_act_up: unknown dtype %d", dtype);
}

// act: [rows * top, inner]; w_down: [experts, width, inner]; y: float [rows * top, width]
extern "C" int srb_moe_down(const void* act, const void* w_down, const int* plan, int rows, int top, int experts, int width,
                            int inner, float* y, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0 || inner <= 0) SRB_FAIL("moe_down: sizes %d, %d must be positive", width, inner);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    return launch_moe_products<float>(MOE_DOWN, act, w_down, nullptr, plan, nullptr, rows, top, experts, inner, width, 0, 0.f, nullptr, y, (size_t)width * inner, s);
  if (dtype == SRB_DTYPE_BF16)
    return launch_moe_products<__nv_bfloat16>(MOE_DOWN, act, w_down, nullptr, plan, nullptr, rows, top, experts, inner, width, 0, 0.f, nullptr, y, (size_t)width * inner, s);
  SRB_FAIL("moe_down: unknown dtype %d", dtype);
}

// `base` (float [rows, width], or null): a term that every row gets beside its experts' (an expert that all rows share);
// it is the first term of the sum.  `chosen` and `input` (both or neither): a choice whose number is `experts` or more
// names an expert that returns its input, so its term is weight * input[row] (such choices have no slot in the plan).
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ entry_slot,
                                   const float* __restrict__ weights, int top, int width, float* __restrict__ out,
                                   const float* __restrict__ base, const int* __restrict__ chosen, int experts,
                                   const T* __restrict__ input) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float sum = base ? base[(size_t)row * width + i] : 0.f;
    for (int k = 0; k < top; ++k) {
      const int slot = entry_slot[(size_t)row * top + k];
      if (slot >= 0) sum += weights[(size_t)row * top + k] * y[(size_t)slot * width + i];
      else if (input && chosen[(size_t)row * top + k] >= experts)
        sum += weights[(size_t)row * top + k] * srb_to_float(input[(size_t)row * width + i]);
    }
    out[(size_t)row * width + i] = sum;
  }
}

extern "C" int srb_moe_combine_identity(const float* y, const int* entry_slot, const float* weights, int rows, int top,
                                        int width, float* out, const float* base, const int* chosen, int experts,
                                        const void* input, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if ((chosen == nullptr) != (input == nullptr)) SRB_FAIL("moe_combine: the choices and the experts' input come together");
  const dim3 block(width >= 1024 ? 256 : 128);
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(moe_combine_kernel<float>, dim3(rows), block, 0, (cudaStream_t)stream, y, entry_slot, weights, top,
                             width, out, base, chosen, experts, (const float*)input));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(moe_combine_kernel<__nv_bfloat16>, dim3(rows), block, 0, (cudaStream_t)stream, y, entry_slot,
                             weights, top, width, out, base, chosen, experts, (const __nv_bfloat16*)input));
  else
    SRB_FAIL("moe_combine: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("moe_combine");
  return SRB_OK;
}

extern "C" int srb_moe_combine_onto(const float* y, const int* entry_slot, const float* weights, int rows, int top, int width,
                                    float* out, const float* base, void* stream) {
  return srb_moe_combine_identity(y, entry_slot, weights, rows, top, width, out, base, nullptr, 0, nullptr, SRB_DTYPE_F32, stream);
}

extern "C" int srb_moe_combine(const float* y, const int* entry_slot, const float* weights, int rows, int top, int width,
                               float* out, void* stream) {
  return srb_moe_combine_onto(y, entry_slot, weights, rows, top, width, out, nullptr, stream);
}

// rows of h in slot order: out[slot, :] = h[slot_row[slot], :] (16 bytes a thread where the rows allow it), for
// products that take their operands as whole tiles of consecutive rows.  `used` (or null) points at the number of slots
// that the plan handed out (its last offset): choices without a slot leave the slots behind it without a row.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ slot_row, int width, T* __restrict__ out,
                                  const int* __restrict__ used) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int slot = blockIdx.x;
  if (used && slot >= *used) return;
  const T* src = h + (size_t)slot_row[slot] * width;
  T* dst = out + (size_t)slot * width;
  if ((width * sizeof(T)) % 16 == 0 && (((uintptr_t)h | (uintptr_t)out) & 15) == 0) {
    const int pieces = width * sizeof(T) / 16;
    for (int i = threadIdx.x; i < pieces; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

extern "C" int srb_moe_gather_used(const void* h, const int* slot_row, int slots, int width, void* out, const int* used,
                                   int dtype, void* stream);
extern "C" int srb_moe_gather(const void* h, const int* slot_row, int slots, int width, void* out, int dtype, void* stream) {
  return srb_moe_gather_used(h, slot_row, slots, width, out, nullptr, dtype, stream);
}

extern "C" int srb_moe_gather_used(const void* h, const int* slot_row, int slots, int width, void* out, const int* used,
                                   int dtype, void* stream) {
  if (slots <= 0 || width <= 0) return SRB_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(moe_gather_kernel<float>, dim3(slots), dim3(128), 0, s, (const float*)h, slot_row, width, (float*)out, used));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(moe_gather_kernel<__nv_bfloat16>, dim3(slots), dim3(128), 0, s, (const __nv_bfloat16*)h, slot_row,
                             width, (__nv_bfloat16*)out, used));
  else
    SRB_FAIL("moe_gather: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("moe_gather");
  return SRB_OK;
}

extern "C" int srb_moe_tile_rows(int rows, int top, int experts) { return moe_tile_rows(rows, top, experts); }
