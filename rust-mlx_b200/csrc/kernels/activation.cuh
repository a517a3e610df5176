// The pointwise part of a gated feed-forward, out = f(gate, up), in float.
//
//   act 0  silu:          gate / (1 + exp(-gate)) * up
//   act 1  gelu (tanh):   0.5 gate (1 + tanh(sqrt(2/pi) (gate + 0.044715 gate^3))) * up
//   act 2  clamped swish: g = min(gate, limit), u = clamp(up, -limit, limit);  g * sigmoid(alpha * g) * (u + 1)
//
// `limit` and `alpha` are read by act 2 only.  The `_fast` forms use the fast exponential and division (about two
// units in the last place of a float) and serve kernels whose result is rounded to bfloat16.
#pragma once
#include "common.cuh"

enum { RMX_ACT_SILU = 0, RMX_ACT_GELU_TANH = 1, RMX_ACT_SWISH_CLAMP = 2, RMX_ACT_RELU2 = 3, RMX_ACT_TANH = 4 };

// One-argument activations, out = f(x):  act 3  squared relu: max(x, 0)^2 (a feed-forward without a gate);  act 4  tanh.
__device__ __forceinline__ float unary_act(float x, int act) {
    if (act == RMX_ACT_TANH) return tanhf(x);
    const float r = fmaxf(x, 0.f);
    return act == RMX_ACT_RELU2 ? r * r : x;
}

__device__ __forceinline__ float gated_act(float g, float u, int act, float limit, float alpha) {
    if (act == RMX_ACT_GELU_TANH) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.f + tanhf(inner)) * u;
    }
    if (act == RMX_ACT_SWISH_CLAMP) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.f + expf(-alpha * g)) * (u + 1.f);
    }
    return g / (1.f + expf(-g)) * u;
}

__device__ __forceinline__ float gated_act_fast(float g, float u, int act, float limit, float alpha) {
    if (act == RMX_ACT_GELU_TANH) {
        // tanh(y) = 1 - 2 / (1 + exp(2y)), so 0.5 g (1 + tanh(y)) = g / (1 + exp(-2y)): the same fast pieces as silu
        const float y2 = 1.5957691216057308f * (g + 0.044715f * g * g * g);
        return __fdividef(g, 1.f + __expf(-y2)) * u;
    }
    if (act == RMX_ACT_SWISH_CLAMP) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fdividef(g, 1.f + __expf(-alpha * g)) * (u + 1.f);
    }
    return __fdividef(g, 1.f + __expf(-g)) * u;
}
