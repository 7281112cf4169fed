// kv-cache append: scatter ONE fresh token's K and V rows per sequence into the
// cache at position lens[b] - the write side of the decode loop. Counterpart
// of the reference's kv_append_kernel<PAGED, T> (src/attention.cu:1753-1782).
//
// It is a byte copy, so one kernel serves every storage type: a thread moves
// one VEC-byte chunk of the [Hkv, D] row pair (16 bytes where the row length
// allows, 8 otherwise; D % 4 == 0 makes every row a multiple of 8 bytes).
// HBM-bound in principle (2 * B * Hkv * D * sizeof read + the same written),
// launch-bound in practice: 262 KB for configuration 2.
// Positions outside the cache (device lens are trusted, never read back) are
// skipped rather than written.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ftk {

struct AppendParams {
    const uint8_t* k_new;   // [B, Hkv, D] storage type
    const uint8_t* v_new;
    uint8_t* k_dst;         // contiguous [B, Hkv, T, D] or pool [Nb, Hkv, P, D]
    uint8_t* v_dst;
    const int* lens;        // [B] write positions
    const int* table;       // [B, tbl_width] or null (contiguous)
    int B, Hkv;
    int row_bytes;          // D * sizeof(storage)
    int rows;               // cache rows T (contiguous) or page size P (paged)
    int tbl_width;
};

template <typename V>
__global__ void __launch_bounds__(256) kv_append_kernel(const AppendParams p) {
    // launched with programmatic stream serialization: the launch overlaps the previous kernel's
    // tail and the decode kernel that follows may set itself up while this one runs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x;
    const int chunks_per_row = p.row_bytes / (int)sizeof(V);
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;
    if (idx >= p.Hkv * chunks_per_row) return;
    const int h = idx / chunks_per_row, c = idx % chunks_per_row;
    const int pos = __ldg(p.lens + b);
    size_t dst_row;
    if (p.table) {
        if (pos < 0 || pos >= p.tbl_width * p.rows) return;
        const int blk = __ldg(p.table + (size_t)b * p.tbl_width + pos / p.rows);
        dst_row = ((size_t)blk * p.Hkv + h) * p.rows + pos % p.rows;
    } else {
        if (pos < 0 || pos >= p.rows) return;
        dst_row = ((size_t)b * p.Hkv + h) * p.rows + pos;
    }
    const size_t src = ((size_t)b * p.Hkv + h) * p.row_bytes + (size_t)c * sizeof(V);
    const size_t dst = dst_row * p.row_bytes + (size_t)c * sizeof(V);
    *reinterpret_cast<V*>(p.k_dst + dst) = *reinterpret_cast<const V*>(p.k_new + src);
    *reinterpret_cast<V*>(p.v_dst + dst) = *reinterpret_cast<const V*>(p.v_new + src);
}

}  // namespace ftk
