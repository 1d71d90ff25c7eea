// A soft cap on an attention score: c tanh(x / c) for c > 0 (inv_c = 1 / c), with tanh(y) = 1 - 2 / (e^(2y) + 1)
// from the fast exponential and division (absolute error about 1e-7 c).  The kernels that hold unscaled scores pass
// c = cap / scale, so that the scale they apply afterwards gives cap tanh(scale x / cap).  The cap is applied before
// the mask: a masked score stays the most negative number.
#pragma once

__device__ __forceinline__ float ri_softcap(float x, float c, float inv_c) {
    float e;
    const float y = fminf(x * inv_c * 2.8853900817779268f, 64.0f);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y));
    return c * (1.0f - __fdividef(2.0f, e + 1.0f));
}
