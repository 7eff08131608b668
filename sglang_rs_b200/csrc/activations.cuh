// The activation of a gated feed-forward, act(gate) * up, as a number that the part chooses: the
// epilogues of the two tcgen05 products and the stand-alone kernel all call srb_gated().  Another
// activation is one more case here and one more name in parts/mlp.py; no kernel changes.
//
//   SRB_ACT_SILU       g / (1 + exp(-g))                     (crates/sglang-kernel/src/cpu.rs:119-123)
//   SRB_ACT_GELU_TANH  g/2 * (1 + tanh(sqrt(2/pi) * (g + 0.044715 g^3)))
//   SRB_ACT_RELU2      max(g, 0)^2
//   SRB_ACT_SWIGLU_CLAMP  g' sigmoid(1.702 g') * (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit); the
//                      limit is the activation's parameter (`param`), which the other activations ignore
//
// A feed-forward without a gate calls the same function with u = 1.
//
// EXACT selects the full-precision exponential and division (the 32-bit path and epilogues whose
// result stays 32-bit); without it the hardware's approximations are used, which is exact enough for
// a result that is rounded to bfloat16.
#pragma once

#define SRB_ACT_SILU 0
#define SRB_ACT_GELU_TANH 1
#define SRB_ACT_RELU2 2
#define SRB_ACT_SWIGLU_CLAMP 3
#define SRB_ACT_COUNT 4

template <bool EXACT>
__device__ __forceinline__ float srb_gated(int activation, float g, float u, float param = 0.f) {
  if (activation == SRB_ACT_SWIGLU_CLAMP) {
    g = fminf(g, param);
    u = fminf(fmaxf(u, -param), param);
    const float s = EXACT ? 1.0f / (1.0f + expf(-1.702f * g)) : __fdividef(1.0f, 1.0f + __expf(-1.702f * g));
    return g * s * (u + 1.0f);
  }
  if (activation == SRB_ACT_RELU2) {
    const float r = fmaxf(g, 0.f);
    return r * r * u;
  }
  if (activation == SRB_ACT_GELU_TANH) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    // tanh(x) = 1 - 2 / (exp(2x) + 1): finite for every x
    const float t = EXACT ? 1.0f - 2.0f / (expf(2.0f * inner) + 1.0f) : 1.0f - __fdividef(2.0f, __expf(2.0f * inner) + 1.0f);
    return 0.5f * g * (1.0f + t) * u;
  }
  return (EXACT ? g / (1.0f + expf(-g)) : __fdividef(g, 1.0f + __expf(-g))) * u;
}
