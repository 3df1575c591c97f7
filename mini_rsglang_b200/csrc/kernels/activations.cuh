// The activations that kernels apply to a product's float32 sums, by number: 0 gelu with the error function, 1 gelu with
// tanh, 2 silu, 3 relu, 4 the square of relu.  Exact float32 forms.
#pragma once

__device__ __forceinline__ float mrs_activate(float z, int kind) {
    if (kind == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));
    if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    if (kind == 3) return fmaxf(z, 0.0f);
    if (kind == 4) return fmaxf(z, 0.0f) * fmaxf(z, 0.0f);
    return z / (1.0f + expf(-z));
}
