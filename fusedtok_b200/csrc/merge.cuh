// Cross-GPU log-sum-exp merge: merge_parts_kernel folds n whole-batch triples
// (one per GPU of a KV-length split, as laid out by an all-gather) into the
// normalised output, one warp per (sequence, query head), with the reference's
// rule (attn_reduce_kernel, src/attention.cu:503-548): partials with l <= 0
// skipped, first live partial adopted verbatim, later ones max-rescaled.
// (Within one GPU the same fold runs inside the partial kernels: merge_unit in
// common.cuh.)
#pragma once

#include "common.cuh"

namespace ftk {

constexpr int MERGE_WARPS = 4;
constexpr int MAX_LANE_CHUNKS = 4;      // head dim <= 512

// parts: n blocks of [rows*2 (m,l), padded to a multiple of 4 | rows*D acc] floats, rows = B*Hq.
template <typename T>
__global__ void __launch_bounds__(MERGE_WARPS * 32)
merge_parts_kernel(const float* __restrict__ parts, int n, T* __restrict__ out, long long rows, int D) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * MERGE_WARPS + warp;
    if (r >= rows) return;
    const int chunks = D >> 2;
    const size_t acc_off = triple_acc_offset(rows);
    const size_t block = acc_off + (size_t)rows * D;
    float4 o[MAX_LANE_CHUNKS];
#pragma unroll
    for (int j = 0; j < MAX_LANE_CHUNKS; ++j) o[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    float m = -INFINITY, l = 0.0f;
    for (int s = 0; s < n; ++s) {
        const float* base = parts + (size_t)s * block;
        const float2 ml = *reinterpret_cast<const float2*>(base + (size_t)r * 2);
        if (ml.y <= 0.0f) continue;
        const float* a = base + acc_off + (size_t)r * D;
        if (l == 0.0f) {
            m = ml.x;
            l = ml.y;
#pragma unroll
            for (int j = 0; j < MAX_LANE_CHUNKS; ++j) {
                const int cc = lane + 32 * j;
                if (cc < chunks) o[j] = *reinterpret_cast<const float4*>(a + cc * 4);
            }
            continue;
        }
        const float m_new = fmaxf(m, ml.x);
        const float r_old = expf(m - m_new), r_new = expf(ml.x - m_new);
        l = lse_fold(l, r_old, ml.y, r_new);
#pragma unroll
        for (int j = 0; j < MAX_LANE_CHUNKS; ++j) {
            const int cc = lane + 32 * j;
            if (cc < chunks) {
                const float4 x = *reinterpret_cast<const float4*>(a + cc * 4);
                o[j].x = lse_fold(o[j].x, r_old, x.x, r_new);
                o[j].y = lse_fold(o[j].y, r_old, x.y, r_new);
                o[j].z = lse_fold(o[j].z, r_old, x.z, r_new);
                o[j].w = lse_fold(o[j].w, r_old, x.w, r_new);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)r * D;
#pragma unroll
    for (int j = 0; j < MAX_LANE_CHUNKS; ++j) {
        const int cc = lane + 32 * j;
        if (cc < chunks) {
            float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
            if (l > 0.0f) y = make_float4(o[j].x / l, o[j].y / l, o[j].z / l, o[j].w / l);
            Store<T>::st4(orow + cc * 4, y);
        }
    }
}

// Triple of an empty cache: (m, l, acc) = (-inf, 0, 0) for every row.
__global__ void fill_empty_triple_kernel(float* ml, float* acc, long long rows, int D) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) {
        ml[i * 2] = -INFINITY;
        ml[i * 2 + 1] = 0.0f;
    }
    if (i < rows * D) acc[i] = 0.0f;
}

// Measurement aid for the benchmark's roofline: reads `n16` 16-byte words once, as fast as plain loads go
// (8 independent streaming loads in flight per thread), and does nothing with them - the read-only
// counterpart of a copy bandwidth. `sink` is written only if the XOR of everything read hits one value.
__global__ void __launch_bounds__(256) read_stream_kernel(const uint4* __restrict__ src, size_t n16, unsigned int* sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint4 acc = make_uint4(0u, 0u, 0u, 0u);
    for (; i + 7 * stride < n16; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc.x ^= v[j].x; acc.y ^= v[j].y; acc.z ^= v[j].z; acc.w ^= v[j].w;
        }
    }
    for (; i < n16; i += stride) {
        const uint4 v = __ldcs(src + i);
        acc.x ^= v.x; acc.y ^= v.y; acc.z ^= v.z; acc.w ^= v.w;
    }
    if ((acc.x ^ acc.y ^ acc.z ^ acc.w) == 0x9e3779b9u && sink) *sink = 1u;
}

}  // namespace ftk
