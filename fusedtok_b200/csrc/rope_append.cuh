// One launch for the three elementwise steps that precede a decode-attention call in the serving loop
// (reference: rope on q and on k_new, src/rope.cu:39-92, then kv_append / kv_append_paged,
// src/attention.cu:1753-1782 - three to four launches there):
//   * q[b, h, :]      is rotated to position lens[b] + pos_offset and written to q_out (which may be q),
//   * k_new[b, kv, :] is rotated to the same position and written straight into the cache row lens[b]
//                     (contiguous row, or block table[b][lens[b] / P] at offset lens[b] % P),
//   * v_new[b, kv, :] is copied into the same row of the V cache.
// The rotated key never makes a round trip through HBM between the two steps. The rotation is the one of
// rope.cuh (same rope_cs, float32 arithmetic, angle in double), so q_out is bit-identical to rope_kernel run on
// each head as a one-row matrix at pos_offset = lens[b], and the cache rows are bit-identical to rope followed
// by kv_append. Launch-bound at decode sizes: (Hq + 2 Hkv) * D * sizeof bytes read and written per sequence.
//
// A thread handles two pairs of one row: four consecutive elements (interleaved) or two consecutive elements in
// each half (NeoX); V rows are copied with the same indexing, which covers every element exactly once.
// A position outside the cache skips the K/V writes (as kv_append does); q is rotated regardless.
#pragma once

#include <cuda_fp16.h>

#include <type_traits>

#include "rope.cuh"

namespace ftk {

template <> __device__ __forceinline__ float2 rope_ld2<__half>(const __half* p) {
    return __half22float2(*reinterpret_cast<const __half2*>(p));
}
template <> __device__ __forceinline__ void rope_st2<__half>(__half* p, float a, float b) {
    *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
}

struct RopeAppendParams {
    const void* q;        // [B, Hq, D]
    void* q_out;          // [B, Hq, D], may alias q
    const void* k_new;    // [B, Hkv, D]
    const void* v_new;
    void* k_dst;          // contiguous [B, Hkv, T, D] or pool [Nb, Hkv, P, D]
    void* v_dst;
    const int* lens;      // [B] write position = rotary position - pos_offset
    const int* table;     // [B, tbl_width] or null (contiguous)
    int B, Hq, Hkv, D;
    int rows;             // cache rows T (contiguous) or page size P (paged)
    int tbl_width;
    int pos_offset;
    int neox;
    double log2_theta;
    double ratio;         // theta^(-2/D)
};

template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendParams p) {
    // launched with programmatic stream serialization: the launch overlaps the previous kernel's
    // tail and the decode kernel that follows may set itself up while this one runs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x;
    const int half = p.D >> 1;
    const int per_row = half >> 1;                       // threads per row: two pairs each (D % 4 == 0)
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;
    const int nrows = p.Hq + 2 * p.Hkv;
    if (idx >= nrows * per_row) return;
    const int r = idx / per_row, u = idx - r * per_row;
    const int j = 2 * u;
    const int pos = __ldg(p.lens + b);

    // element offsets of the two 2-element accesses inside a row
    const int e0 = p.neox ? j : 2 * j;
    const int e1 = p.neox ? half + j : 2 * j + 2;

    const T* src;
    T* dst;
    bool rotate = true;
    if (r < p.Hq) {
        const size_t row = ((size_t)b * p.Hq + r) * p.D;
        src = static_cast<const T*>(p.q) + row;
        dst = static_cast<T*>(p.q_out) + row;
    } else {
        const bool is_v = r >= p.Hq + p.Hkv;
        const int h = r - p.Hq - (is_v ? p.Hkv : 0);
        size_t dst_row;
        if (p.table) {
            if (pos < 0 || pos >= p.tbl_width * p.rows) return;
            const int blk = __ldg(p.table + (size_t)b * p.tbl_width + pos / p.rows);
            dst_row = ((size_t)blk * p.Hkv + h) * p.rows + pos % p.rows;
        } else {
            if (pos < 0 || pos >= p.rows) return;
            dst_row = ((size_t)b * p.Hkv + h) * p.rows + pos;
        }
        src = static_cast<const T*>(is_v ? p.v_new : p.k_new) + ((size_t)b * p.Hkv + h) * p.D;
        dst = static_cast<T*>(is_v ? p.v_dst : p.k_dst) + dst_row * p.D;
        rotate = !is_v;
    }
    if (!rotate) {                                       // V: plain copy in the storage type
        using W = typename std::conditional<sizeof(T) == 4, float2, unsigned>::type;
        *reinterpret_cast<W*>(dst + e0) = *reinterpret_cast<const W*>(src + e0);
        *reinterpret_cast<W*>(dst + e1) = *reinterpret_cast<const W*>(src + e1);
        return;
    }
    const int m = pos + p.pos_offset;
    float c0, s0, c1, s1;
    rope_cs2(j, p.D, m, p.log2_theta, p.ratio, c0, s0, c1, s1);
    const float2 a = rope_ld2<T>(src + e0), bb = rope_ld2<T>(src + e1);
    if (p.neox) {
        rope_st2<T>(dst + e0, a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
        rope_st2<T>(dst + e1, a.x * s0 + bb.x * c0, a.y * s1 + bb.y * c1);
    } else {
        rope_st2<T>(dst + e0, a.x * c0 - a.y * s0, a.x * s0 + a.y * c0);
        rope_st2<T>(dst + e1, bb.x * c1 - bb.y * s1, bb.x * s1 + bb.y * c1);
    }
}

}  // namespace ftk
