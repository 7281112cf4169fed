// Rotary position embedding on one [seq, dim] matrix (reference: rope_kernel / rope_neox_kernel,
// src/rope.cu:39-92): row r has absolute position m = r + pos_offset, pair j is rotated by the angle
// m * theta^(-2j/dim); interleaved pairs (2j, 2j+1) or NeoX pairs (j, j + dim/2). The rotation itself is
// float32; the angle is formed and reduced to [-pi, pi] in double (see rope_cs_from_freq), which keeps the result within
// 1e-4 of the reference's CPU statement (src/rope.cu:95-146) at any position. HBM-bound: 2 * seq * dim *
// sizeof bytes per call.
//
// One thread rotates two pairs: four consecutive elements (interleaved), or two consecutive elements in each
// half (NeoX), so every access is 8 bytes (bf16) or 16 / 8 bytes (float32) wide and coalesced. Rows whose
// width is not a multiple of 4 take the one-pair-per-thread path.
#pragma once

#include "common.cuh"

namespace ftk {

struct RopeParams {
    const void* x;
    void* y;
    long long seq;
    int dim;
    int pos_offset;
    int neox;
    double log2_theta;
    double ratio;          // theta^(-2/dim): frequency of pair j + 1 over that of pair j
};

template <typename T> __device__ __forceinline__ float rope_ld(const T* p) { return (float)*p; }
template <> __device__ __forceinline__ float rope_ld<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}
template <typename T> __device__ __forceinline__ void rope_st(T* p, float v) { *p = (T)v; }
template <> __device__ __forceinline__ void rope_st<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}
template <typename T> __device__ __forceinline__ float2 rope_ld2(const T* p);
template <> __device__ __forceinline__ float2 rope_ld2<float>(const float* p) {
    return *reinterpret_cast<const float2*>(p);
}
template <> __device__ __forceinline__ float2 rope_ld2<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void rope_st2(T* p, float a, float b);
template <> __device__ __forceinline__ void rope_st2<float>(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <> __device__ __forceinline__ void rope_st2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// The angle is formed in double: at position m the float32 product m * freq is only good to m * 2^-24 radians
// (1e-3 at m = 4096, 1e-2 at m = 100000), which the reference's double-precision CPU statement does not suffer.
// Only the product and its reduction to [-pi, pi] need double (two fused multiply-adds against a two-term 2*pi);
// the sine and cosine of the reduced angle are float32 (2 ulp), which keeps the result within 1e-6 of the double
// statement at any position and the kernel's latency short (no double-precision sincos).
__device__ __forceinline__ void rope_cs_from_freq(double freq, int m, float& c, float& s) {
    const double a = (double)m * freq;
    const double k = rint(a * 0.15915494309189535);          // a / (2 pi)
    double r = fma(-k, 6.283185307179586, a);                 // a - k * 2 pi, high part
    r = fma(-k, 2.4492935982947064e-16, r);                   // ... low part
    sincosf((float)r, &s, &c);
}
__device__ __forceinline__ void rope_cs(int j, int dim, int m, double log2_theta, float& c, float& s) {
    rope_cs_from_freq(exp2(-(2.0 * j / dim) * log2_theta), m, c, s);
}
// Pairs j and j + 1: the second frequency is the first times theta^(-2/dim) (`ratio`, from the host).
__device__ __forceinline__ void rope_cs2(int j, int dim, int m, double log2_theta, double ratio, float& c0, float& s0,
                                         float& c1, float& s1) {
    const double f0 = exp2(-(2.0 * j / dim) * log2_theta);
    rope_cs_from_freq(f0, m, c0, s0);
    rope_cs_from_freq(f0 * ratio, m, c1, s1);
}

// VEC: two pairs per thread (dim % 4 == 0 and 8-byte aligned rows), else one pair per thread.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) rope_kernel(const RopeParams p) {
    const T* x = static_cast<const T*>(p.x);
    T* y = static_cast<T*>(p.y);
    const int half = p.dim >> 1;
    const int per_row = VEC ? half >> 1 : half;
    const long long total = p.seq * per_row;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (long long)gridDim.x * blockDim.x) {
        const long long row = t / per_row;
        const int u = (int)(t - row * per_row);
        const int m = (int)row + p.pos_offset;
        const long long base = row * p.dim;
        if (VEC) {
            const int j = 2 * u;
            float c0, s0, c1, s1;
            rope_cs2(j, p.dim, m, p.log2_theta, p.ratio, c0, s0, c1, s1);
            if (p.neox) {
                const float2 a = rope_ld2<T>(x + base + j), b = rope_ld2<T>(x + base + half + j);
                rope_st2<T>(y + base + j, a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
                rope_st2<T>(y + base + half + j, a.x * s0 + b.x * c0, a.y * s1 + b.y * c1);
            } else {
                const float2 a = rope_ld2<T>(x + base + 2 * j), b = rope_ld2<T>(x + base + 2 * j + 2);
                rope_st2<T>(y + base + 2 * j, a.x * c0 - a.y * s0, a.x * s0 + a.y * c0);
                rope_st2<T>(y + base + 2 * j + 2, b.x * c1 - b.y * s1, b.x * s1 + b.y * c1);
            }
        } else {
            float c, s;
            rope_cs(u, p.dim, m, p.log2_theta, c, s);
            const long long ia = p.neox ? base + u : base + 2 * u;
            const long long ib = p.neox ? ia + half : ia + 1;
            const float xa = rope_ld<T>(x + ia), xb = rope_ld<T>(x + ib);
            rope_st<T>(y + ia, xa * c - xb * s);
            rope_st<T>(y + ib, xa * s + xb * c);
        }
    }
}

}  // namespace ftk
