// Reproducible fp32 transcendentals shared by the CUDA kernels and the CPU oracle.
//
// The reference evaluates softplus / sigmoid / the small-point layer factor with CUDA's expf and
// logf (src/lib/rendering/RenderForward.cu:154-159, RenderBackward.cu:71-83, PointBlending.h:106).
// Those library routines are not bit-reproducible on a CPU, and the quantities they feed (projected
// point size -> pyramid layer count, alpha -> transmittance cut-off) decide which fragments exist.
// Both sides therefore evaluate exp and log with the routines below, which use only IEEE fp32
// add / mul / div and integer bit operations. Compiled without FMA contraction (nvcc -fmad=false,
// gcc -ffp-contract=off) they return identical bits on host and device; accuracy is ~1 ulp.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define TM_HD __host__ __device__ __forceinline__
#else
#define TM_HD inline
#endif

TM_HD float tm_bits_to_float(uint32_t u)
{
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

TM_HD uint32_t tm_float_to_bits(float f)
{
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

// floor for |x| < 2^23 without calling libm (keeps host/device identical and inlineable).
TM_HD float tm_floorf(float x)
{
    float t = (float)(int)x;  // truncation toward zero
    return (t > x) ? t - 1.0f : t;
}

// exp(x), x clamped to [-87, 88].
TM_HD float tm_expf(float x)
{
    if (x < -87.0f) x = -87.0f;
    if (x > 88.0f) x = 88.0f;
    float kf = tm_floorf(x * 1.44269504088896341f + 0.5f);
    // Cody-Waite: ln2 = hi + lo, hi has 11 trailing zero bits so kf*hi is exact for |kf| < 2^11
    float r = x - kf * 0.693145751953125f;
    r       = r - kf * 1.42860682030941723e-6f;
    float p = 1.98412698412698413e-4f;  // 1/5040
    p       = p * r + 1.38888888888888894e-3f;  // 1/720
    p       = p * r + 8.33333333333333322e-3f;  // 1/120
    p       = p * r + 4.16666666666666644e-2f;  // 1/24
    p       = p * r + 1.66666666666666657e-1f;  // 1/6
    p       = p * r + 0.5f;
    p       = p * r + 1.0f;
    p       = p * r + 1.0f;
    int k   = (int)kf;  // in [-126, 127]
    float s = tm_bits_to_float((uint32_t)(k + 127) << 23);
    return p * s;
}

// log(y) for finite y > 0 (normal numbers; denormals are treated as the smallest normal).
TM_HD float tm_logf(float y)
{
    uint32_t b = tm_float_to_bits(y);
    if (b < 0x00800000u) b = 0x00800000u;
    int e      = (int)(b >> 23) - 127;
    float m    = tm_bits_to_float((b & 0x007fffffu) | 0x3f800000u);  // [1, 2)
    if (m > 1.41421356237309515f)
    {
        m = m * 0.5f;
        e = e + 1;
    }
    float s  = (m - 1.0f) / (m + 1.0f);
    float s2 = s * s;
    float p  = 2.22222222222222210e-1f;  // 2/9
    p        = p * s2 + 2.85714285714285698e-1f;  // 2/7
    p        = p * s2 + 0.4f;                     // 2/5
    p        = p * s2 + 6.66666666666666630e-1f;  // 2/3
    p        = p * s2 + 2.0f;
    p        = p * s;
    float ef = (float)e;
    return ef * 0.693145751953125f + (p + ef * 1.42860682030941723e-6f);
}

// softplus with beta = 1, threshold = 20 (RenderForward.cu:154-159): x > 20 ? x : log(1 + exp(x)).
TM_HD float tm_softplus(float x)
{
    if (x > 20.0f) return x;
    return tm_logf(1.0f + tm_expf(x));
}

// derivative of softplus (RenderBackward.cu:71-83): y > 20 ? 1 : e^y / (e^y + 1).
TM_HD float tm_softplus_grad(float y)
{
    if (y > 20.0f) return 1.0f;
    float z = tm_expf(y);
    return z / (z + 1.0f);
}

// logistic function 1 / (1 + e^-x), the activation of the per-point confidence (NeuralTexture.h:40-43)
TM_HD float tm_sigmoid(float x) { return 1.0f / (1.0f + tm_expf(-x)); }

// Exact floor(log2(x)) and ceil(log2(x)) for finite normal x > 0, from the exponent / mantissa bits.
// The reference takes floor / ceil of log2f(x) (RenderForward.cu:345, PointBlending.h:83-90); the two
// agree except where log2f rounds a value a few ulp above a power of two down to that integer.
TM_HD int tm_floor_log2(float x)
{
    uint32_t b = tm_float_to_bits(x);
    return (int)(b >> 23) - 127;
}
TM_HD int tm_ceil_log2(float x)
{
    uint32_t b = tm_float_to_bits(x);
    return (int)(b >> 23) - 127 + ((b & 0x007fffffu) ? 1 : 0);
}
