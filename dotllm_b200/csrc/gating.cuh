// The gatings of a feed-forward's two products g (gate) and u (up), float32 arithmetic:
//   GATE_SILU             g sigmoid(g) u
//   GATE_GELU_TANH        gelu_tanh(g) u,  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   GATE_CLAMPED_SIGMOID  g' sigmoid(alpha g') (u' + 1)  with g' = min(g, limit), u' = clamp(u, -limit, limit)
//   GATE_RELU2            relu(u)^2: an activation of ONE product (a feed-forward without a gate); g is not read
#pragma once
#include "common.cuh"

enum { GATE_SILU = 0, GATE_GELU_TANH = 1, GATE_CLAMPED_SIGMOID = 2, GATE_RELU2 = 3, GATE_KINDS = 4 };

// Does the activation read two products (gate and up) or one?
__host__ __device__ __forceinline__ bool dl_gate_is_gated(int kind) { return kind != GATE_RELU2; }

__device__ __forceinline__ float dl_gate_value(int kind, float g, float u, float limit, float alpha) {
    if (kind == GATE_RELU2) {
        const float r = fmaxf(u, 0.f);
        return r * r;
    }
    if (kind == GATE_GELU_TANH) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    if (kind == GATE_CLAMPED_SIGMOID) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
    }
    return g * (1.0f / (1.0f + expf(-g))) * u;
}

