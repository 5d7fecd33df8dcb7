// Activation functions of the GEMM epilogues, on packed fp32 pairs (shared by the one-block and the two-block GEMM kernel).
#pragma once
#include "stof_ptx.cuh"

namespace stof {

// erf-form GELU on a packed pair: x * Phi(x) with Phi(x) - 0.5 = x * g(x^2), g a degree-8 polynomial fitted on |x| <= 4.5
// (|error of Phi| < 2.4e-5, of the GELU value < 1.1e-4, below half an fp16 step of any output above 0.1); x^2 is capped at 4.5^2
// and 0.5 + x g saturates to [0, 1], so the tails are exactly 0 and x.  Ten packed FMAs / products and four scalar
// instructions per pair, where an erf by the 7.1.28 rational form of Abramowitz & Stegun took about twice as many.
__device__ __forceinline__ float2 gelu_erf2(float2 x2) {
    float x0, x1, u0, u1;
    upk2(x2, x0, x1);
    upk2(mul2(x2, x2), u0, u1);
    const float2 u = pk2(fminf(u0, 20.25f), fminf(u1, 20.25f));
    float2 g = fma2(pk2(3.805775833e-11f, 3.805775833e-11f), u, pk2(-4.002384202e-09f, -4.002384202e-09f));
    g = fma2(g, u, pk2(1.846188695e-07f, 1.846188695e-07f));
    g = fma2(g, u, pk2(-4.959777016e-06f, -4.959777016e-06f));
    g = fma2(g, u, pk2(8.727704699e-05f, 8.727704699e-05f));
    g = fma2(g, u, pk2(-1.076741493e-03f, -1.076741493e-03f));
    g = fma2(g, u, pk2(9.729498066e-03f, 9.729498066e-03f));
    g = fma2(g, u, pk2(-6.624044478e-02f, -6.624044478e-02f));
    g = fma2(g, u, pk2(3.988665044e-01f, 3.988665044e-01f));
    float g0, g1;
    upk2(g, g0, g1);
    return mul2(x2, pk2(__saturatef(fmaf(x0, g0, 0.5f)), __saturatef(fmaf(x1, g1, 0.5f))));
}
// tanh-form GELU: 0.5 x (1 + tanh(u)) = x * sigmoid(2u), u = 0.79788456 (x + 0.044715 x^3)
__device__ __forceinline__ float2 gelu_tanh2(float2 x2) {
    const float2 xx = mul2(x2, x2);
    const float2 inner = fma2(xx, pk2(0.044715f * 0.7978845608028654f, 0.044715f * 0.7978845608028654f),
                                pk2(0.7978845608028654f, 0.7978845608028654f));
    float u0, u1, x0, x1;
    upk2(mul2(inner, x2), u0, u1);
    upk2(x2, x0, x1);
    // sigmoid(2u) = 1 / (1 + 2^(-2u log2 e))
    const float s0 = __fdividef(1.0f, 1.0f + fast_exp2(-2.8853900817779268f * u0));
    const float s1 = __fdividef(1.0f, 1.0f + fast_exp2(-2.8853900817779268f * u1));
    return pk2(x0 * s0, x1 * s1);
}

}  // namespace stof
