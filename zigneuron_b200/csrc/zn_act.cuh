// gelu, leaky_relu and elu of src/activation.zig:128-185, shared by the GEMM epilogues and the row-wise
// kernels.  Every product and sum is a separate rounding (no FMA contraction), in the reference's order.
#pragma once

// geluForward, src/activation.zig:128-134 (tanh approximation).
__device__ __forceinline__ float zn_gelu_fwd(float x) {
    const float c = 0.7978845608f, k = 0.044715f;
    const float x3 = __fmul_rn(__fmul_rn(x, x), x);
    const float inner = __fmul_rn(c, __fadd_rn(x, __fmul_rn(k, x3)));
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner)));
}

// geluBackward, src/activation.zig:139-150: the derivative formula evaluated at the ACTIVATED output
// (the reference takes x ~= y), times the incoming gradient (:44).
__device__ __forceinline__ float zn_gelu_bwd(float y, float g) {
    const float c = 0.7978845608f, k = 0.044715f;
    const float x = y;
    const float x3 = __fmul_rn(__fmul_rn(x, x), x);
    const float inner = __fmul_rn(c, __fadd_rn(x, __fmul_rn(k, x3)));
    const float t = tanhf(inner);
    const float sech2 = __fsub_rn(1.0f, __fmul_rn(t, t));
    const float left = __fmul_rn(0.5f, __fadd_rn(1.0f, t));
    const float poly = __fadd_rn(1.0f, __fmul_rn(__fmul_rn(__fmul_rn(3.0f, k), x), x));
    const float right = __fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(0.5f, x), sech2), c), poly);
    return __fmul_rn(__fadd_rn(left, right), g);
}

// leakyReluForward / Backward, src/activation.zig:155-167 (alpha 0.01).
__device__ __forceinline__ float zn_leaky_fwd(float x) { return x > 0.f ? x : __fmul_rn(0.01f, x); }
__device__ __forceinline__ float zn_leaky_bwd(float y, float g) { return __fmul_rn(y > 0.f ? 1.0f : 0.01f, g); }

// eluForward / Backward, src/activation.zig:171-184 (alpha 1).
__device__ __forceinline__ float zn_elu_fwd(float x) { return x > 0.f ? x : __fsub_rn(expf(x), 1.0f); }
__device__ __forceinline__ float zn_elu_bwd(float y, float g) { return __fmul_rn(y > 0.f ? 1.0f : __fadd_rn(y, 1.0f), g); }
