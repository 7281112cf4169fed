// Shared device-side pieces of the decode-attention kernels: launch
// parameters, the tile scheduler, storage-type conversion and the one place
// where a finished (m, l, acc) state leaves a kernel.
//
// Work decomposition (all kernels): a UNIT is one (sequence b, kv head,
// head chunk) triple - the query heads of one GQA group (at most GC of them)
// that share the same K/V rows. A unit with len_b valid rows has
// ceil(len_b / TILE) TILES of TILE cache rows. All tiles of all units, in
// (b, kv, chunk, tile) order, form one linear sequence; CTA c of n owns the
// contiguous range [c*total/n, (c+1)*total/n). A CTA therefore walks through
// a few SEGMENTS (maximal runs of tiles of one unit). A segment that covers
// its whole unit is finished in place; otherwise its (m, l, acc) goes to the
// workspace slot c + unit (unique, because both indices only grow along the
// walk), the CTA bumps the unit's arrival counter, and whichever CTA arrives
// last folds the unit's slots - always in CTA order, so the result does not
// depend on who was last. The split depends only on (lens, n): results are
// bit-identical from call to call. (Counterpart of the reference's workspace +
// attn_reduce_kernel, src/attention.cu:434-463 and :478-549, without the
// second launch.)
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace ftk {

constexpr int TILE = 64;            // cache rows per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// device status word values (0 = ok)
enum : int {
    ST_OK = 0,
    ST_WAIT_FULL_TIMEOUT = 1,    // a consumer gave up waiting for a K/V tile
    ST_WAIT_EMPTY_TIMEOUT = 2,   // the producer gave up waiting for a free stage
    ST_SMEM_MISALIGNED = 3,
    ST_DRAIN_TIMEOUT = 4,
};

struct DecodeParams {
    const void* q;        // [B, Hq, D] storage type
    const void* k;        // contiguous [B, Hkv, T, D] or pool [Nb, Hkv, P, D]
    const void* v;
    void* out;            // [B, Hq, D] storage type (unused when triple != 0)
    const int* lens;      // [B] or null
    const int* table;     // [B, tbl_width] block ids, null for contiguous
    float* ws_ml;         // [slots][GC][2]  (m natural-log units, l)
    float* ws_acc;        // [slots][GC][D]  unnormalised
    int* counters;        // [units] arrival counters, zero between launches (the last arriver resets)
    int* status;          // device status word
    float* triple_ml;     // when non-null: emit raw triples instead of `out`: one block
                          // [B*Hq*2 (m, l), padded | B*Hq*D unnormalised acc] starting here ...
    size_t triple_acc_off;  // ... with the acc part at this float offset
    // KV-length split with direct peer exchange: when n_peers > 0 the triple block is written
    // into EVERY rank's exchange buffer (plain stores over NVLink) instead of triple_ml.
    float* peer_blocks[16];          // data region of each rank's exchange buffer (own included)
    const unsigned int* peer_epoch;  // this rank's count of completed exchange steps
    int n_peers, peer_rank;
    long long peer_nf;               // floats per triple block
    int B, Hq, Hkv, G;    // G = Hq / Hkv
    int GC, NCH;          // heads per unit, units per (b, kv)
    int T;                // cache rows (contiguous) or tbl_width * page
    int D;
    int page, tbl_width;
    int box_rows, box_shift;   // rows per TMA box (a power of two) and its log2 (tensor-core kernel)
    int ncta;
    float scale;          // 1/sqrt(D)
};

// Float offset of the acc block inside a triple buffer of `rows` (b, h) rows:
// the (m, l) block padded so that the acc rows stay 16-byte aligned.
__host__ __device__ __forceinline__ size_t triple_acc_offset(long long rows) {
    return ((size_t)rows * 2 + 3) & ~(size_t)3;
}

constexpr int MAX_PEERS = 16;

// Where destination j of a raw triple block lives. Exchange buffers are double-buffered by the
// parity of the step number, so a rank that runs one step ahead never overwrites a block its
// peer is still merging.
__device__ __forceinline__ float* triple_block(const struct DecodeParams& p, int j);

// ---- storage types ---------------------------------------------------------
template <typename T> struct Store;
template <> struct Store<float> {
    static __device__ __forceinline__ float4 ld4(const float* p) {
        return *reinterpret_cast<const float4*>(p);
    }
    static __device__ __forceinline__ void st4(float* p, float4 v) {
        *reinterpret_cast<float4*>(p) = v;
    }
    static __device__ __forceinline__ void st2(float* p, float a, float b) {
        *reinterpret_cast<float2*>(p) = make_float2(a, b);
    }
};
template <> struct Store<__nv_bfloat16> {
    static __device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    static __device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    }
    static __device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    }
};
template <> struct Store<__half> {
    static __device__ __forceinline__ float4 ld4(const __half* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    static __device__ __forceinline__ void st4(__half* p, float4 v) {
        __half2 lo = __floats2half2_rn(v.x, v.y);
        __half2 hi = __floats2half2_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    }
    static __device__ __forceinline__ void st2(__half* p, float a, float b) {
        *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
    }
};

__device__ __forceinline__ float* triple_block(const DecodeParams& p, int j) {
    if (!p.n_peers) return p.triple_ml;
    const unsigned int parity = (__ldg(p.peer_epoch) + 1u) & 1u;
    return p.peer_blocks[j] + ((size_t)parity * p.n_peers + p.peer_rank) * (size_t)p.peer_nf;
}

// ---- scheduler -------------------------------------------------------------
__device__ __forceinline__ int seq_len(const DecodeParams& p, int b) {
    if (!p.lens) return p.T;
    const int l = __ldg(p.lens + b);
    return l < 0 ? 0 : (l > p.T ? p.T : l);   // device lens are trusted; the clamp only keeps addresses in range
}
__device__ __forceinline__ int tiles_of(int len) { return (len + TILE - 1) / TILE; }

// a / b for non-negative operands; 32-bit hardware path when both fit (a 64-bit divide is a
// long subroutine on the GPU and these sit on every CTA's start-up path)
__device__ __forceinline__ long long qdiv(long long a, long long b) {
    if (((unsigned long long)a | (unsigned long long)b) >> 32) return a / b;
    return (long long)((unsigned int)a / (unsigned int)b);
}

struct SchedShared {
    long long total;     // tiles in the whole launch
    long long red[33];   // block-reduction scratch
    long long pb;        // tiles (per unit-of-b) before sequence b_start
    int b_start;
    int found;
};

// Position of one walker inside the linear tile sequence.
struct Walker {
    long long g, end;    // current / one-past-last global tile index
    int b, ub, ti;       // sequence, unit within the sequence, tile within the unit
    int nt, len;         // tiles and valid rows of sequence b
};

__device__ __forceinline__ long long block_sum(long long v, long long* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    long long s = 0;
    for (int w = 0; w < nwarp; ++w) s += red[w];
    return s;
}

// Zero row for an empty sequence (len == 0): the reference's convention
// (src/attention.cu:211-216). One thread writes the whole [Hq, D] row.
template <typename T>
__device__ void zero_rows(const DecodeParams& p, int b) {
    if (p.triple_ml) {
        const int nd = p.n_peers ? p.n_peers : 1;
        for (int j = 0; j < nd; ++j) {
            float* blk = triple_block(p, j);
            for (int h = 0; h < p.Hq; ++h) {
                const size_t r = (size_t)b * p.Hq + h;
                blk[r * 2] = -INFINITY;
                blk[r * 2 + 1] = 0.0f;
                for (int d = 0; d < p.D; d += 4)
                    *reinterpret_cast<float4*>(blk + p.triple_acc_off + r * p.D + d) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        return;
    }
    T* o = reinterpret_cast<T*>(p.out) + (size_t)b * p.Hq * p.D;
    const int n = p.Hq * p.D;
    for (int i = 0; i < n; i += 4) Store<T>::st4(o + i, make_float4(0.f, 0.f, 0.f, 0.f));
}

// Block-wide: total tile count, this CTA's range and its starting position.
// Every thread of the block must call it. Returns false for an empty range.
// Also writes the zero rows of empty sequences (sequence b is handled by the
// CTA with b % ncta == blockIdx.x).
template <typename T>
__device__ bool sched_init(const DecodeParams& p, SchedShared* sh, Walker& w) {
    const int upb = p.Hkv * p.NCH;
    const int c = blockIdx.x;
    long long total_nt;
    if (!p.lens) {
        total_nt = (long long)p.B * tiles_of(p.T);
    } else {
        long long loc = 0;
        for (int b = threadIdx.x; b < p.B; b += blockDim.x) {
            const int len = seq_len(p, b);
            loc += tiles_of(len);
            if (len == 0 && (b % p.ncta) == c) zero_rows<T>(p, b);
        }
        total_nt = block_sum(loc, sh->red);
    }
    const long long total = total_nt * upb;
    const long long start = qdiv(total * c, p.ncta);
    const long long end = qdiv(total * (c + 1), p.ncta);
    if (start >= end) return false;
    const long long x = qdiv(start, upb);    // tiles-per-unit prefix we look for
    int b0;
    long long pb;
    if (!p.lens) {
        const int nt = tiles_of(p.T);
        b0 = (int)qdiv(x, nt);
        pb = (long long)b0 * nt;
    } else {
        // chunked block scan over tiles_of(len_b) to find P_b <= x < P_{b+1}
        if (threadIdx.x == 0) sh->found = 0;
        long long running = 0;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int nwarp = (blockDim.x + 31) >> 5;
        for (int base = 0; base < p.B; base += blockDim.x) {
            const int b = base + threadIdx.x;
            const long long v = (b < p.B) ? tiles_of(seq_len(p, b)) : 0;
            long long inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            __syncthreads();
            if (lane == 31) sh->red[warp] = inc;
            __syncthreads();
            long long before = running;
            for (int i = 0; i < warp; ++i) before += sh->red[i];
            long long chunk = 0;
            for (int i = 0; i < nwarp; ++i) chunk += sh->red[i];
            const long long excl = before + inc - v;
            if (v > 0 && excl <= x && x < excl + v) {
                sh->b_start = b;
                sh->pb = excl;
                sh->found = 1;
            }
            running += chunk;
            __syncthreads();
            if (sh->found) break;
        }
        b0 = sh->b_start;
        pb = sh->pb;
    }
    w.g = start;
    w.end = end;
    w.b = b0;
    w.len = seq_len(p, b0);
    w.nt = tiles_of(w.len);
    const long long rem = start - pb * upb;
    w.ub = (int)qdiv(rem, w.nt);
    w.ti = (int)(rem - (long long)w.ub * w.nt);
    if (threadIdx.x == 0) sh->total = total;
    __syncthreads();
    return true;
}

// Step to the next tile (skipping empty sequences).
__device__ __forceinline__ void walker_advance(const DecodeParams& p, Walker& w) {
    ++w.g;
    if (++w.ti < w.nt) return;
    w.ti = 0;
    if (++w.ub < p.Hkv * p.NCH) return;
    w.ub = 0;
    if (w.g >= w.end) return;          // nothing follows in this CTA's range
    do {
        ++w.b;
        w.len = seq_len(p, w.b);
        w.nt = tiles_of(w.len);
    } while (w.nt == 0 && w.b + 1 < p.B);
}

// CTA that owns global tile x when `total` tiles are split over n CTAs.
__device__ __forceinline__ int owner_of(long long x, long long total, int n) {
    return (int)qdiv((x + 1) * n - 1, total);
}

// Where a finished segment goes.
struct SegDest {
    bool whole;          // the segment covers its whole unit: finish in place
    size_t slot;         // workspace slot otherwise
    long long unit;      // global unit index
    int b, h0;           // sequence and first query head of the unit
    int gvalid;          // query heads in this unit
    int c_first, c_last; // CTAs holding the unit's first and last tile
    int nparts;          // CTAs that deliver a partial for this unit
};

__device__ __forceinline__ bool cta_range_empty(long long total, int n, int c) {
    return qdiv(total * c, n) == qdiv(total * (c + 1), n);
}

__device__ __forceinline__ SegDest seg_dest(const DecodeParams& p, const Walker& w, long long total,
                                            long long seg_first_g) {
    SegDest d;
    const int upb = p.Hkv * p.NCH;
    d.unit = (long long)w.b * upb + w.ub;
    const long long u_start = w.g - w.ti;            // global index of the unit's tile 0
    const long long u_end = u_start + w.nt;
    const int kv = w.ub / p.NCH, ch = w.ub % p.NCH;
    d.b = w.b;
    d.h0 = kv * p.G + ch * p.GC;
    d.gvalid = min(p.GC, p.G - ch * p.GC);
    d.whole = (seg_first_g == u_start) && (w.g + 1 == u_end);
    d.slot = (size_t)blockIdx.x + (size_t)d.unit;
    d.c_first = d.c_last = (int)blockIdx.x;
    d.nparts = 1;
    if (!d.whole) {
        d.c_first = owner_of(u_start, total, p.ncta);
        d.c_last = owner_of(u_end - 1, total, p.ncta);
        d.nparts = d.c_last - d.c_first + 1;
        if (p.ncta > total)                          // more CTAs than tiles: some ranges are empty
            for (int c = d.c_first + 1; c < d.c_last; ++c)
                if (cta_range_empty(total, p.ncta, c)) --d.nparts;
    }
    return d;
}

// Final store of two adjacent elements (d, d+1) of head h of sequence b:
// normalised output in the storage type, or the raw triple for the
// multi-GPU layer.
template <typename T>
__device__ __forceinline__ void emit_final2(const DecodeParams& p, int b, int h, int d, float m_nat,
                                            float l, float a0, float a1, bool write_ml) {
    const size_t r = (size_t)b * p.Hq + h;
    if (p.triple_ml) {
        const int nd = p.n_peers ? p.n_peers : 1;
        for (int j = 0; j < nd; ++j) {
            float* blk = triple_block(p, j);
            *reinterpret_cast<float2*>(blk + p.triple_acc_off + r * p.D + d) = make_float2(a0, a1);
            if (write_ml) *reinterpret_cast<float2*>(blk + r * 2) = make_float2(m_nat, l);
        }
    } else {
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        Store<T>::st2(reinterpret_cast<T*>(p.out) + r * p.D + d, a0 * inv, a1 * inv);
    }
}

// Fold the workspace slots of a split unit into its final rows. Called by all
// `nthreads` threads (index `tid`) of the CTA that delivered the last partial.
// The reference's rule (attn_reduce_kernel, src/attention.cu:503-548):
// partials with l <= 0 are skipped, the first live one is adopted verbatim,
// later ones are max-rescaled, then the row is divided by l.
template <typename T>
__device__ __forceinline__ void merge_unit(const DecodeParams& p, const SegDest& d, long long total, int tid,
                                           int nthreads) {
    constexpr int BATCH = 8;                      // slots fetched together: one L2 round trip per batch
    const int D = p.D, halfd = D >> 1;
    const bool sparse = p.ncta > total;
    for (int e = tid; e < d.gvalid * halfd; e += nthreads) {
        const int g = e / halfd, dd = (e % halfd) * 2;
        float m = -INFINITY, l = 0.0f, a0 = 0.0f, a1 = 0.0f;
        for (int c0 = d.c_first; c0 <= d.c_last; c0 += BATCH) {
            float2 ml[BATCH], x[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int c = c0 + j;
                ml[j] = make_float2(0.0f, 0.0f);
                x[j] = make_float2(0.0f, 0.0f);
                if (c <= d.c_last && !(sparse && cta_range_empty(total, p.ncta, c))) {
                    const size_t pr = ((size_t)c + (size_t)d.unit) * p.GC + g;
                    ml[j] = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + pr * 2));
                    x[j] = __ldcg(reinterpret_cast<const float2*>(p.ws_acc + pr * D + dd));
                }
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                if (ml[j].y <= 0.0f) continue;
                if (l == 0.0f) {
                    m = ml[j].x; l = ml[j].y; a0 = x[j].x; a1 = x[j].y;
                    continue;
                }
                const float m_new = fmaxf(m, ml[j].x);
                const float r_old = expf(m - m_new), r_new = expf(ml[j].x - m_new);
                l = l * r_old + ml[j].y * r_new;
                a0 = a0 * r_old + x[j].x * r_new;
                a1 = a1 * r_old + x[j].y * r_new;
                m = m_new;
            }
        }
        emit_final2<T>(p, d.b, d.h0 + g, dd, m, l, a0, a1, dd == 0);
    }
}

// One thread per CTA calls this after every thread of the CTA has written and
// fenced its part of the partial. Returns true if this CTA delivered the last
// partial of the unit and must therefore merge it.
__device__ __forceinline__ bool deliver_partial(const DecodeParams& p, const SegDest& d) {
    const int old = atomicAdd(p.counters + d.unit, 1);
    const bool last = old == d.nparts - 1;
    if (last) p.counters[d.unit] = 0;          // ready for the next launch
    return last;
}

}  // namespace ftk
