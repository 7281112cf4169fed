// Shared device-side pieces of the decode-attention kernels: launch
// parameters, the tile scheduler, storage-type conversion and the one place
// where a finished (m, l, acc) state leaves a kernel.
//
// Work decomposition (all kernels): a UNIT is one (sequence b, kv head,
// head chunk) triple - the query heads of one GQA group (at most GC of them)
// that share the same K/V rows. A unit with len_b valid rows has
// ceil(len_b / TILE) TILES of TILE cache rows. All tiles of all units, in
// (b, kv, chunk, tile) order, form one linear sequence, which a PLAN cuts into
// RANGES whose boundaries are a pure function of (lens, number of CTAs):
//   * equal split: range c = [c*total/n, (c+1)*total/n), one per CTA;
//   * static + dynamic (large launches, tensor-core kernel): the sequence is cut
//     into one block per CTA; CTA c first takes the static range at the head
//     of block c; the last few tiles of every block are cut into small ranges
//     of `chunk` tiles that the CTAs take from an atomic counter as they run
//     dry, so that SMs which stream faster do more of them.
// A range crosses unit boundaries; each maximal run of its tiles inside one
// unit is a SEGMENT. A segment that covers its whole unit is finished in
// place; otherwise its (m, l, acc) goes to the workspace slot range + unit
// (unique, because both indices only grow along the tile sequence), the CTA
// bumps the unit's arrival counter, and whichever CTA arrives last folds the
// unit's slots - always in range order. WHICH CTA computes a tail range varies
// from launch to launch; what is computed and the order in which it is merged
// do not, so results are bit-identical from call to call. (Counterpart of the
// reference's workspace + attn_reduce_kernel, src/attention.cu:434-463 and
// :478-549, without the second launch, and of its capacity-based equal slice
// counts, src/attention.cu:1819-1821.)
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
    ST_PEER_TIMEOUT = 5,         // a peer's block of the KV-length split never arrived
    ST_WAIT_RANGE_TIMEOUT = 7,   // a consumer gave up waiting for the producer's next range
    ST_BOUNDS = 8,               // self-checking build: a computed cache row, partial slot or counter index was out of range
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
    int* counters;        // [units] arrival counters, zero between launches (the last arriver resets);
                          // counters[units] hands out the tail ranges of a launch (reset by the last taker)
    int* status;          // device status word
    float* triple_ml;     // when non-null: emit raw triples instead of `out`: one block
                          // [B*Hq*2 (m, l), padded | B*Hq*D unnormalised acc] starting here ...
    size_t triple_acc_off;  // ... with the acc part at this float offset
    // KV-length split with direct peer exchange: when n_peers > 0 the rows of every finished unit
    // are written into EVERY rank's exchange buffer (plain stores over NVLink) instead of
    // triple_ml, a per-(unit, rank) flag is raised there, and at its end every CTA folds the n
    // blocks of its share of the rows into `out` (peer_fold).
    float* peer_blocks[16];          // data region of each rank's exchange buffer (own included)
    unsigned int* peer_hdr[16];      // header of each rank's exchange buffer
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
    int dyn_chunk;        // tiles per tail range of the static + dynamic plan; 0 = equal split only
    int dyn_tail_max;     // most tiles per CTA that go to the dynamic tail
    int sched_table;      // lens given and the per-sequence tile prefix sums fit the kernel's table
    int cost_split;       // cut the ranges at equal cost (tiles + unit ends) instead of equal tile counts
    int cost_a, cost_b;   // ... a tile counts cost_a, a unit end cost_b
    int unit_split;       // generic kernel only: CTA c takes unit c whole (ncta == units); no workspace, no counters
    float scale;          // 1/sqrt(D)
    // What the launch may touch, for the self-checking build (-DFTK_BOUNDS); 0 = not known, not checked.
    unsigned long long bound_rows;    // rows of the K (and V) array: B*Hkv*T, or pool blocks * Hkv * page
    unsigned int bound_slots;         // partial slots of the workspace
    unsigned int bound_words;         // arrival counters
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
__device__ __forceinline__ float* triple_block(const struct DecodeParams& p, int j, unsigned int step);

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

// acc * r_old + x * r_new with the rounding spelled out (one rounded product, one fused multiply-add),
// so that every place that folds partials - inside a kernel, across kernels, across GPUs - produces the
// same bits whatever the compiler would otherwise choose to contract.
// ---- self-checking build (-DFTK_BOUNDS): the stand-in for a memory checker ----------------------------
// Every cache row a kernel is about to read and every workspace slot / arrival counter it is about to
// touch is compared with what the host said the launch owns; a value out of range is recorded in the
// status word (ST_BOUNDS) and the access is redirected (row 0) or left out, so the build reports the
// mistake instead of faulting. The product build compiles all of it away.
#ifdef FTK_BOUNDS
__device__ __forceinline__ bool bounds_ok(const DecodeParams& p, bool ok) {
    if (!ok && p.status) atomicCAS(p.status, ST_OK, ST_BOUNDS);
    return ok;
}
#define FTK_ROW_OK(p, row) bounds_ok(p, (p).bound_rows == 0 || (unsigned long long)(row) < (p).bound_rows)
#define FTK_SLOT_OK(p, slot, unit)                                                             \
    bounds_ok(p, ((p).bound_slots == 0 || (unsigned long long)(slot) < (p).bound_slots) &&    \
                     ((p).bound_words == 0 || (unsigned long long)(unit) < (p).bound_words))
#else
#define FTK_ROW_OK(p, row) true
#define FTK_SLOT_OK(p, slot, unit) true
#endif

__device__ __forceinline__ float lse_fold(float acc, float r_old, float x, float r_new) {
    return fmaf(acc, r_old, __fmul_rn(x, r_new));
}

// Step number of this launch of a peer-exchange kernel (0 otherwise). Read once per thread, right after
// the dependency wait, from L2 (the word changes between launches, so no read-only cache).
__device__ __forceinline__ unsigned int peer_step(const DecodeParams& p) {
    return p.n_peers ? __ldcg(p.peer_epoch) + 1u : 0u;
}
__device__ __forceinline__ float* triple_block(const DecodeParams& p, int j, unsigned int step) {
    if (!p.n_peers) return p.triple_ml;
    return p.peer_blocks[j] + ((size_t)(step & 1u) * p.n_peers + p.peer_rank) * (size_t)p.peer_nf;
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

constexpr int SCHED_MAX_B = 2048;   // sequences whose tile prefix sums fit the shared-memory table
constexpr int DYN_MIN_PER = 24;     // tiles per CTA below which a launch keeps the equal split

struct SchedShared {
    long long total;     // tiles in the whole launch
    long long red[33];   // block-reduction scratch
    long long pb;        // tiles (per unit-of-b) before sequence b_start
    int b_start;
    int found;
};

// How the tile sequence of a launch is cut into ranges. Under the static + dynamic plan the sequence is
// cut into ncta equal blocks of `per` tiles; block c is the static range of CTA c (its first S tiles)
// followed by nd dynamic ranges of `chunk` tiles; what is left over after the ncta blocks (fewer than ncta
// tiles) forms a few more dynamic ranges. Ranges are numbered in tile order (which is the order partials
// are merged in); the dynamic ones are handed out round-robin over the blocks (dyn_range).
struct Plan {
    long long total;     // tiles in the launch
    long long per;       // tiles per block; 0 = equal split
    int S;               // tiles of a block's static range
    int chunk;           // tiles per dynamic range
    int nd;              // dynamic ranges per block
    int nstat;           // ranges inside the blocks: ncta * (1 + nd)
    int ndyn;            // dynamic ranges in all: ncta * nd + those of the leftover
    int R;               // ranges (equal split: one per CTA, some possibly empty)
    int ncta;
    // Cost-weighted equal split (tensor-core kernel): a unit of nt tiles counts ka * nt + kb (nt + 1 unless
    // overridden) - every unit that ENDS inside a range costs its CTA a fold and a fresh set of query fragments,
    // about one tile's worth of streaming (measured: 1 : 1 and 2 : 3 do best on ragged batches, 2 : 1 and 1 : 2
    // within 0.5 % of them) - and the ranges are cut at equal cost instead of equal tile counts, so that a CTA
    // whose range is full of short sequences is given fewer tiles. ctot == 0: off.
    long long ctot;                 // cost of the whole launch
    const unsigned int* pre;        // per sequence: tiles before it (units of one kv head); null without lens
    const unsigned int* zpre;       // per sequence: non-empty sequences before it; null without lens
    int upb, nt_uniform;            // units per sequence; tiles per unit when every sequence has p.T rows
    int ka, kb;                     // cost of a tile and of a unit end
};

// dyn_chunk == 0: equal split. Otherwise a block keeps all but min(per / 6, dyn_tail_max) of its
// per = total / ncta tiles static (the rest rounded to whole dynamic ranges of dyn_chunk tiles),
// provided per >= DYN_MIN_PER.
__device__ __forceinline__ Plan make_plan(long long total, int ncta, int dyn_chunk, int dyn_tail_max) {
    Plan pl;
    pl.total = total;
    pl.per = 0;
    pl.S = 0;
    pl.chunk = 1;
    pl.nd = 0;
    pl.nstat = ncta;
    pl.ndyn = 0;
    pl.R = ncta;
    pl.ncta = ncta;
    pl.ctot = 0;
    pl.pre = pl.zpre = nullptr;
    pl.upb = pl.nt_uniform = 0;
    pl.ka = 1;
    pl.kb = 1;
    if (dyn_chunk > 0) {
        const long long per = qdiv(total, ncta);
        if (per >= DYN_MIN_PER && per < (1ll << 30)) {
            int td = (int)(per / 6);
            if (td > dyn_tail_max) td = dyn_tail_max;
            const int nd = td / dyn_chunk;
            if (nd > 0) {
                pl.per = per;
                pl.chunk = dyn_chunk;
                pl.nd = nd;
                pl.S = (int)per - nd * dyn_chunk;
                pl.nstat = ncta * (1 + nd);
                const int left = (int)(total - per * ncta);          // < ncta
                const int nl = (left + dyn_chunk - 1) / dyn_chunk;
                pl.ndyn = ncta * nd + nl;
                pl.R = pl.nstat + nl;
            }
        }
    }
    return pl;
}
// first tile of range r (r == R gives the end of the sequence)
__device__ __forceinline__ long long range_start(const Plan& pl, int r) {
    if (!pl.per) return qdiv(pl.total * r, pl.ncta);
    if (r < pl.nstat) {
        const int c = (int)((unsigned)r / (unsigned)(1 + pl.nd)), k = r - c * (1 + pl.nd);
        return (long long)c * pl.per + (k ? pl.S + (k - 1) * pl.chunk : 0);
    }
    const long long x = pl.per * pl.ncta + (long long)(r - pl.nstat) * pl.chunk;
    return x < pl.total ? x : pl.total;
}
// range that holds tile x
__device__ __forceinline__ int range_of(const Plan& pl, long long x) {
    if (!pl.per) return (int)qdiv((x + 1) * pl.ncta - 1, pl.total);
    const long long blocks_end = pl.per * pl.ncta;
    if (x < blocks_end) {
        const int c = (int)qdiv(x, pl.per);
        const int off = (int)(x - (long long)c * pl.per);
        return c * (1 + pl.nd) + (off < pl.S ? 0 : 1 + (off - pl.S) / pl.chunk);
    }
    return pl.nstat + (int)qdiv(x - blocks_end, pl.chunk);
}
__device__ __forceinline__ bool range_empty(const Plan& pl, int r) {
    return !pl.per && !pl.ctot && qdiv(pl.total * r, pl.ncta) == qdiv(pl.total * (r + 1), pl.ncta);
}
// ---- cost-weighted equal split
// Switch it on for a launch of `total_nt` tiles per kv-head unit row and `nonempty` non-empty sequences (only
// when every range is then certain to hold a tile: at least 4 cost units per range).
__device__ __forceinline__ void plan_enable_cost(Plan& pl, long long total_nt, long long nonempty, int upb,
                                                 const unsigned int* pre, const unsigned int* zpre, int nt_uniform,
                                                 int ka, int kb) {
    // (tiles sit ka apart in cost, ka + kb across a unit end: ranges of at least ka + kb + 1 always hold a tile)
    const long long ctot = (ka * total_nt + kb * nonempty) * upb;
    if (pl.per || ka < 1 || kb < 0 || ctot < (long long)(ka + kb + 1) * pl.ncta) return;
    pl.ka = ka;
    pl.kb = kb;
    pl.ctot = ctot;
    pl.pre = pre;
    pl.zpre = zpre;
    pl.upb = upb;
    pl.nt_uniform = nt_uniform;
}
// cost position of tile 0 of unit (b, ub); nt = tiles of sequence b
__device__ __forceinline__ long long cost_of_unit(const Plan& pl, int b, int ub, int nt) {
    const long long pb = pl.pre ? (long long)pl.pre[b] : (long long)b * pl.nt_uniform;
    const long long zb = pl.zpre ? (long long)pl.zpre[b] : (long long)b;
    return (pl.ka * pb + pl.kb * zb) * pl.upb + (long long)ub * (pl.ka * nt + pl.kb);
}
__device__ __forceinline__ long long cost_start(const Plan& pl, int r) { return qdiv(pl.ctot * r, pl.ncta); }
__device__ __forceinline__ int cost_owner(const Plan& pl, long long c) { return (int)qdiv((c + 1) * pl.ncta - 1, pl.ctot); }
// static range of CTA c, and the i-th dynamic range in hand-out order
__device__ __forceinline__ int static_range(const Plan& pl, int c) { return pl.per ? c * (1 + pl.nd) : c; }
__device__ __forceinline__ int dyn_range(const Plan& pl, int i) {
    const int in_blocks = pl.ncta * pl.nd;
    if (i < in_blocks) {
        const int round = (int)((unsigned)i / (unsigned)pl.ncta), c = i - round * pl.ncta;
        return c * (1 + pl.nd) + 1 + round;
    }
    return pl.nstat + (i - in_blocks);
}

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

// ---- direct peer exchange (KV-length split) -----------------------------------
// Exchange buffer of one rank (allocated by the library, mapped into every peer
// through CUDA IPC): a header of 32-bit words - [0] steps completed (epoch),
// [1] count of warps that have finished the current step - and, from byte
// XCHG_DATA_BYTES on, the blocks gather[2][n][nf], double-buffered by step
// parity. A block carries one rank's raw triples with the step number riding
// beside every value: per (sequence, query head) row one 16-byte word
// {m, step, l, step}, then per row D/2 words {acc[d], step, acc[d+1], step}.
// Every 8-byte half is written by one store and validates itself, so the
// reader needs no separate flag and the writer no fence: it polls the data
// until the step number in it is the current one.
constexpr int XCHG_DATA_BYTES = 1024;
constexpr unsigned long long XCHG_WAIT_NS = 2000000000ull;      // bounded wait: 2 s
// floats per block and offset of its acc part
__host__ __device__ __forceinline__ size_t xchg_acc_off(long long rows) { return (size_t)rows * 4; }
__host__ __device__ __forceinline__ size_t xchg_block_floats(long long rows, int dim) {
    return (size_t)rows * 4 + (size_t)rows * dim * 2;
}
// 16-byte load that bypasses L1 (the words are written by other GPUs)
__device__ __forceinline__ uint4 ld_peer16(const float* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Zero row for an empty sequence (len == 0): the reference's convention
// (src/attention.cu:211-216). One thread writes the whole [Hq, D] row.
template <typename T>
__device__ void zero_rows(const DecodeParams& p, int b, unsigned int step) {
    if (p.n_peers) {
        const float e = __uint_as_float(step);
        for (int j = 0; j < p.n_peers; ++j) {
            float* blk = triple_block(p, j, step);
            for (int h = 0; h < p.Hq; ++h) {
                const size_t r = (size_t)b * p.Hq + h;
                *reinterpret_cast<float4*>(blk + r * 4) = make_float4(-INFINITY, e, 0.0f, e);
                for (int d = 0; d < p.D; d += 2)
                    *reinterpret_cast<float4*>(blk + p.triple_acc_off + (r * p.D + d) * 2) = make_float4(0.f, e, 0.f, e);
            }
        }
        return;
    }
    if (p.triple_ml) {
        float* blk = p.triple_ml;
        for (int h = 0; h < p.Hq; ++h) {
            const size_t r = (size_t)b * p.Hq + h;
            blk[r * 2] = -INFINITY;
            blk[r * 2 + 1] = 0.0f;
            for (int d = 0; d < p.D; d += 4)
                *reinterpret_cast<float4*>(blk + p.triple_acc_off + r * p.D + d) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    T* o = reinterpret_cast<T*>(p.out) + (size_t)b * p.Hq * p.D;
    const int n = p.Hq * p.D;
    for (int i = 0; i < n; i += 4) Store<T>::st4(o + i, make_float4(0.f, 0.f, 0.f, 0.f));
}

// Block-wide: total tile count, this CTA's range under the equal split and its
// starting position. Every thread of the block must call it. Returns false for
// an empty range. Also writes the zero rows of empty sequences (sequence b is
// handled by the CTA with b % ncta == blockIdx.x).
template <typename T>
__device__ bool sched_init(const DecodeParams& p, SchedShared* sh, Walker& w, unsigned int step) {
    const int upb = p.Hkv * p.NCH;
    const int c = blockIdx.x;
    if (p.unit_split) {
        // one CTA per (sequence, kv head, head chunk) unit, every unit whole: each segment is final, so
        // neither the partial slots nor the arrival counters are touched (the launch that needs no
        // workspace: a first call that arrives inside a stream capture, where nothing may be allocated)
        const int b = c / upb;
        const int len = seq_len(p, b);
        if (threadIdx.x == 0) sh->total = 1;
        __syncthreads();
        if (len == 0) {
            if (c == b * upb && threadIdx.x == 0) zero_rows<T>(p, b, step);
            return false;
        }
        w.b = b;
        w.ub = c - b * upb;
        w.ti = 0;
        w.len = len;
        w.nt = tiles_of(len);
        w.g = 0;
        w.end = w.nt;
        return true;
    }
    long long total_nt;
    if (!p.lens) {
        total_nt = (long long)p.B * tiles_of(p.T);
    } else {
        long long loc = 0;
        for (int b = threadIdx.x; b < p.B; b += blockDim.x) {
            const int len = seq_len(p, b);
            loc += tiles_of(len);
            if (len == 0 && (b % p.ncta) == c) zero_rows<T>(p, b, step);
        }
        total_nt = block_sum(loc, sh->red);
    }
    const long long total = total_nt * upb;
    if (threadIdx.x == 0) sh->total = total;
    __syncthreads();
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
    return true;
}

// Block-wide, for launches with lens and at most SCHED_MAX_B sequences: exclusive prefix sums of
// tiles_of(len_b) into prefix[0 .. B] (prefix[B] = the total), so that afterwards ONE thread can
// locate any range (walker_locate). Also writes the zero rows of empty sequences, like sched_init.
// Returns the number of tiles of the launch.
template <typename T>
__device__ long long sched_prefix(const DecodeParams& p, SchedShared* sh, unsigned int* prefix, unsigned int* zprefix,
                                  unsigned int step) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    unsigned int running = 0, zrunning = 0;
    for (int base = 0; base < p.B; base += blockDim.x) {
        const int b = base + threadIdx.x;
        unsigned int v = 0;
        if (b < p.B) {
            const int len = seq_len(p, b);
            v = (unsigned int)tiles_of(len);
            if (len == 0 && (b % p.ncta) == (int)blockIdx.x) zero_rows<T>(p, b, step);
        }
        // two scans at once: tiles in the low half of a 64-bit word, non-empty sequences in the high half
        const unsigned long long both = (unsigned long long)v | ((unsigned long long)(v > 0 ? 1u : 0u) << 32);
        unsigned long long inc = both;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        __syncthreads();
        if (lane == 31) sh->red[warp] = (long long)inc;
        __syncthreads();
        unsigned long long before = 0, chunk = 0;
        for (int i = 0; i < nwarp; ++i) {
            const unsigned long long t = (unsigned long long)sh->red[i];
            if (i < warp) before += t;
            chunk += t;
        }
        if (b < p.B) {
            const unsigned long long excl = before + inc - both;
            prefix[b] = running + (unsigned int)excl;
            zprefix[b] = zrunning + (unsigned int)(excl >> 32);
        }
        running += (unsigned int)chunk;
        zrunning += (unsigned int)(chunk >> 32);
    }
    if (threadIdx.x == 0) {
        prefix[p.B] = running;
        zprefix[p.B] = zrunning;
        sh->total = (long long)running * (p.Hkv * p.NCH);
    }
    __syncthreads();
    return sh->total;
}

// Walker at global tile `start` (one thread; `prefix` from sched_prefix, or null when every sequence
// has p.T rows). `end` is the range's end.
__device__ __forceinline__ Walker walker_locate(const DecodeParams& p, const unsigned int* prefix, long long start,
                                                long long end) {
    const int upb = p.Hkv * p.NCH;
    Walker w;
    w.g = start;
    w.end = end;
    const long long x = qdiv(start, upb);
    long long pb;
    if (!prefix) {
        const int nt = tiles_of(p.T);
        w.b = (int)qdiv(x, nt);
        pb = (long long)w.b * nt;
    } else {
        // last b with prefix[b] <= x (it has tiles, because prefix[b + 1] > x)
        int lo = 0, hi = p.B;            // invariant: prefix[lo] <= x < prefix[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((long long)prefix[mid] <= x) lo = mid;
            else hi = mid;
        }
        w.b = lo;
        pb = prefix[lo];
    }
    w.len = seq_len(p, w.b);
    w.nt = tiles_of(w.len);
    const long long rem = start - pb * upb;
    w.ub = (int)qdiv(rem, w.nt);
    w.ti = (int)(rem - (long long)w.ub * w.nt);
    return w;
}

// Walker at the first tile whose cost position is >= X under the cost-weighted split (one thread); X ==
// pl.ctot gives the end of the sequence (w.g == pl.total). `end` is stored as the range's end.
__device__ __forceinline__ Walker walker_locate_cost(const DecodeParams& p, const Plan& pl, long long X, long long end) {
    Walker w;
    w.end = end;
    w.b = 0; w.ub = 0; w.ti = 0; w.nt = 0; w.len = 0;
    if (X >= pl.ctot) {
        w.g = pl.total;
        return w;
    }
    const int upb = pl.upb;
    long long pb, zb;
    if (!pl.pre) {
        const long long per_seq = (long long)upb * (pl.ka * pl.nt_uniform + pl.kb);
        w.b = (int)qdiv(X, per_seq);
        pb = (long long)w.b * pl.nt_uniform;
        zb = w.b;
    } else {
        int lo = 0, hi = p.B;            // invariant: cost(lo) <= X < cost(hi)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (((long long)pl.ka * pl.pre[mid] + (long long)pl.kb * pl.zpre[mid]) * upb <= X) lo = mid;
            else hi = mid;
        }
        w.b = lo;
        pb = pl.pre[lo];
        zb = pl.zpre[lo];
    }
    w.len = seq_len(p, w.b);
    w.nt = tiles_of(w.len);
    const long long rem = X - (pl.ka * pb + pl.kb * zb) * upb;
    const int unit_cost = pl.ka * w.nt + pl.kb;
    w.ub = (int)qdiv(rem, unit_cost);
    const int o = (int)(rem - (long long)w.ub * unit_cost);
    w.ti = (o + pl.ka - 1) / pl.ka;      // first tile at or after the boundary
    if (w.ti >= w.nt) {                  // the boundary fell behind the unit's last tile: the next unit starts the range
        w.ti = 0;
        if (++w.ub >= upb) {
            w.ub = 0;
            pb += w.nt;
            do {
                ++w.b;
                w.len = w.b < p.B ? seq_len(p, w.b) : 0;
                w.nt = tiles_of(w.len);
            } while (w.nt == 0 && w.b < p.B);
            if (w.b >= p.B) {
                w.g = pl.total;
                return w;
            }
        }
    }
    w.g = pb * upb + (long long)w.ub * w.nt + w.ti;
    return w;
}

// Range r of the cost-weighted split, located by a whole (converged) warp: each boundary is a chain of
// dependent integer divisions that a single thread takes the better part of a microsecond over, and
// every CTA pays it before its first copy can go out - so odd and even lanes work out one boundary
// each, at the same time, and the warp shares the result.
__device__ __forceinline__ Walker walker_locate_cost_range(const DecodeParams& p, const Plan& pl, int r) {
    const int odd = threadIdx.x & 1;
    Walker w = walker_locate_cost(p, pl, cost_start(pl, r + odd), 0);
    const long long end = __shfl_sync(0xffffffffu, w.g, 1);
    w.g = __shfl_sync(0xffffffffu, w.g, 0);
    w.b = __shfl_sync(0xffffffffu, w.b, 0);
    w.ub = __shfl_sync(0xffffffffu, w.ub, 0);
    w.ti = __shfl_sync(0xffffffffu, w.ti, 0);
    w.nt = __shfl_sync(0xffffffffu, w.nt, 0);
    w.len = __shfl_sync(0xffffffffu, w.len, 0);
    w.end = end;
    return w;
}

// Step to the next tile (skipping empty sequences).
__device__ __forceinline__ void walker_advance(const DecodeParams& p, Walker& w) {
    ++w.g;
    if (++w.ti < w.nt) return;
    w.ti = 0;
    if (++w.ub < p.Hkv * p.NCH) return;
    w.ub = 0;
    if (w.g >= w.end) return;          // nothing follows in this range
    do {
        ++w.b;
        w.len = seq_len(p, w.b);
        w.nt = tiles_of(w.len);
    } while (w.nt == 0 && w.b + 1 < p.B);
}

// Where a finished segment goes.
struct SegDest {
    bool whole;          // the segment covers its whole unit: finish in place
    size_t slot;         // workspace slot otherwise
    long long unit;      // global unit index
    int b, h0;           // sequence and first query head of the unit
    int gvalid;          // query heads in this unit
    int r_first, r_last; // ranges holding the unit's first and last tile
    int nparts;          // ranges that deliver a partial for this unit
};

// `w` stands on the segment's last tile, inside range `r`.
__device__ __forceinline__ SegDest seg_dest(const DecodeParams& p, const Plan& pl, const Walker& w, int r,
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
    d.slot = (size_t)r + (size_t)d.unit;
    d.r_first = d.r_last = r;
    d.nparts = 1;
    if (!d.whole && pl.ctot) {
        const long long c0 = cost_of_unit(pl, w.b, w.ub, w.nt);
        d.r_first = cost_owner(pl, c0);
        d.r_last = cost_owner(pl, c0 + (long long)pl.ka * (w.nt - 1));
        d.nparts = d.r_last - d.r_first + 1;
    } else if (!d.whole) {
        d.r_first = range_of(pl, u_start);
        d.r_last = range_of(pl, u_end - 1);
        d.nparts = d.r_last - d.r_first + 1;
        if (!pl.per && pl.ncta > pl.total)           // more CTAs than tiles: some ranges are empty
            for (int c = d.r_first + 1; c < d.r_last; ++c)
                if (range_empty(pl, c)) --d.nparts;
    }
    return d;
}

// Final store of two adjacent elements (d, d+1) of head h of sequence b:
// normalised output in the storage type, or the raw triple for the
// multi-GPU layer.
// PEERS = false compiles the peer-exchange destination out (kernels that are short of registers have a
// variant of their own for the KV-length split).
template <typename T, bool PEERS = true>
__device__ __forceinline__ void emit_final2(const DecodeParams& p, unsigned int step, int b, int h, int d,
                                            float m_nat, float l, float a0, float a1, bool write_ml) {
    const size_t r = (size_t)b * p.Hq + h;
    if (PEERS && p.n_peers) {
        // one 16-byte word per element pair, the step number beside each value, into every rank's buffer
        const float e = __uint_as_float(step);
        for (int j = 0; j < p.n_peers; ++j) {
            float* blk = triple_block(p, j, step);
            *reinterpret_cast<float4*>(blk + p.triple_acc_off + (r * p.D + d) * 2) = make_float4(a0, e, a1, e);
            if (write_ml) *reinterpret_cast<float4*>(blk + r * 4) = make_float4(m_nat, e, l, e);
        }
    } else if (p.triple_ml) {
        float* blk = p.triple_ml;
        *reinterpret_cast<float2*>(blk + p.triple_acc_off + r * p.D + d) = make_float2(a0, a1);
        if (write_ml) *reinterpret_cast<float2*>(blk + r * 2) = make_float2(m_nat, l);
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
template <typename T, bool PEERS = true>
__device__ __forceinline__ void merge_unit(const DecodeParams& p, const Plan& pl, const SegDest& d, unsigned int step,
                                           int tid, int nthreads) {
    constexpr int BATCH = 8;                      // slots fetched together: one L2 round trip per batch
    const int D = p.D, halfd = D >> 1;
    const bool sparse = !pl.per && !pl.ctot && pl.ncta > pl.total;
    for (int e = tid; e < d.gvalid * halfd; e += nthreads) {
        const int g = e / halfd, dd = (e % halfd) * 2;
        float m = -INFINITY, l = 0.0f, a0 = 0.0f, a1 = 0.0f;
        for (int c0 = d.r_first; c0 <= d.r_last; c0 += BATCH) {
            float2 ml[BATCH], x[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                const int c = c0 + j;
                ml[j] = make_float2(0.0f, 0.0f);
                x[j] = make_float2(0.0f, 0.0f);
                if (c <= d.r_last && !(sparse && range_empty(pl, c))) {
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
                l = lse_fold(l, r_old, ml[j].y, r_new);
                a0 = lse_fold(a0, r_old, x[j].x, r_new);
                a1 = lse_fold(a1, r_old, x[j].y, r_new);
                m = m_new;
            }
        }
        emit_final2<T, PEERS>(p, step, d.b, d.h0 + g, dd, m, l, a0, a1, dd == 0);
    }
}

// ---- optional timeline (diagnostic builds only: -DFTK_TIMELINE; slots listed in decode_tc.cuh) ----
__device__ __forceinline__ unsigned long long timeline_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#ifdef FTK_TIMELINE
__device__ unsigned long long g_timeline[1024][24];
#define FTK_STAMP(cond, slot) do { if (cond) g_timeline[blockIdx.x][slot] = timeline_ns(); } while (0)
#define FTK_ADD(cond, slot, v) do { if (cond) g_timeline[blockIdx.x][slot] += (v); } while (0)
#define FTK_NOW() timeline_ns()
#else
#define FTK_STAMP(cond, slot) do { } while (0)
#define FTK_ADD(cond, slot, v) do { } while (0)
#define FTK_NOW() 0ull
#endif

// The same fold, same order, same arithmetic (bit for bit), organised for a unit that was split over
// many ranges - one long sequence spread over the whole grid:
//  - the partials are copied into shared memory with cp.async: no registers hold them while they are
//    in flight, so a whole round of them is requested at once (the version above costs one L2 round
//    trip per 8 partials and 32 registers);
//  - the two scale factors of every fold step, exp(m_before - m_after) and exp(m_j - m_after), depend
//    only on the (m, l) pairs, so one thread per (partial, head) works them out - all steps at the
//    same time, each from the running maximum before its partial - instead of every thread of a head
//    walking the same chain of dependent exponentials;
//  - what is left per element pair is one multiply-add per partial out of shared memory.
// `stage`: shared memory, 16-byte aligned, free for the calling threads, merge_stage_bytes(nthreads, S)
// bytes for rounds of S partials; `sync()` is a barrier over exactly the `nthreads` calling threads.
constexpr int MERGE_ENTRIES = 256;                                      // (partial, head) pairs per round
constexpr int MERGE_TABLE_BYTES = MERGE_ENTRIES * (8 + 16) + 2 * 16 * 4;   // (m, l), coefficients, running maxima
__host__ __device__ constexpr int merge_stage_bytes(int nthreads, int S) { return MERGE_TABLE_BYTES + S * nthreads * 8; }
template <typename T, bool PEERS = true, typename Sync>
__device__ __forceinline__ void merge_unit_staged(const DecodeParams& p, const Plan& pl, const SegDest& d,
                                                  unsigned int step, int tid, int nthreads, float* stage,
                                                  int stage_bytes, Sync sync) {
    const int P = d.r_last - d.r_first + 1;
    const int D = p.D, halfd = D >> 1;
    const int gv = d.gvalid;
    const int E = gv * halfd;                                      // element pairs of the unit
    // partials per round: what the stage holds, and no more than the tables have entries for
    const int S = min((stage_bytes - MERGE_TABLE_BYTES) / (nthreads * 8), MERGE_ENTRIES / gv);
    const bool sparse = !pl.per && !pl.ctot && pl.ncta > pl.total;
    float2* t_ml = reinterpret_cast<float2*>(stage);                                   // [S][gv] (m, l)
    float4* t_co = reinterpret_cast<float4*>(stage + MERGE_ENTRIES * 2);               // [S][gv] r_old, r_new, l * r_new, live
    float* t_run = stage + MERGE_ENTRIES * 6;                                          // [2][16] running maximum per head
    float2* t_acc = reinterpret_cast<float2*>(stage + MERGE_TABLE_BYTES / 4);          // [S][nthreads]
    for (int e0 = 0; e0 < E; e0 += nthreads) {                     // one pass unless the unit has more pairs than threads
        const int e = e0 + tid;
        const int g = e / halfd, dd = (e % halfd) * 2;
        const int pieces = min(nthreads, E - e0) >> 1;             // 16-byte pieces of a partial in this pass (E is even)
        float l = 0.0f, a0 = 0.0f, a1 = 0.0f;
        int round = 0;
        for (int j0 = 0; j0 < P; j0 += S, ++round) {
            const int n = min(S, P - j0);
            if (j0 | e0) sync();                                   // everybody is done reading the stage
            // (m, l) pairs first - into a register: their round trip overlaps the issue of the copies
            const int i_ml = tid;                                  // n * gv <= MERGE_ENTRIES <= nthreads is not assumed:
            float2 ml_mine = make_float2(0.0f, 0.0f);              // the first entry per thread here, the rest below
            if (i_ml < n * gv) {
                const int j = i_ml / gv, gg = i_ml - j * gv;
                const int c = d.r_first + j0 + j;
                if (!(sparse && range_empty(pl, c)))               // an empty range's entry stays "skip"
                    ml_mine = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + (((size_t)c + (size_t)d.unit) * p.GC + gg) * 2));
            }
            {
                // piece i = tid, tid + nthreads, ... of the round: (partial j, 16-byte piece k), stepped without a divide
                const int jstep = nthreads / pieces, kstep = nthreads - jstep * pieces;
                int j = tid / pieces, k = tid - j * pieces;
                const size_t slot_floats = (size_t)p.GC * D;
                const float* src0 = p.ws_acc + ((size_t)d.r_first + j0 + (size_t)d.unit) * slot_floats + (size_t)e0 * 2;
                for (; j < n; j += jstep) {
                    if (!(sparse && range_empty(pl, d.r_first + j0 + j))) {
                        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(t_acc + (size_t)j * nthreads + k * 2);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src0 + j * slot_floats + k * 4)
                                     : "memory");
                    }
                    k += kstep;
                    if (k >= pieces) { k -= pieces; ++j; }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (i_ml < n * gv) t_ml[i_ml] = ml_mine;
            for (int i = tid + nthreads; i < n * gv; i += nthreads) {
                const int j = i / gv, gg = i - j * gv;
                const int c = d.r_first + j0 + j;
                float2 v = make_float2(0.0f, 0.0f);
                if (!(sparse && range_empty(pl, c)))
                    v = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + (((size_t)c + (size_t)d.unit) * p.GC + gg) * 2));
                t_ml[i] = v;
            }
            if (j0 == 0 && tid < gv) t_run[tid] = -INFINITY;
            FTK_STAMP(tid == 0, 21);
            sync();
            // the fold steps' coefficients. A partial with l <= 0 is skipped; the first live one meets a running
            // maximum of -inf and gets the factors 0 and 1, which is the reference's "adopt it verbatim".
            for (int i = tid; i < n * gv; i += nthreads) {
                const int j = i / gv, gg = i - j * gv;
                float m_before = t_run[(round & 1) * 16 + gg];
                for (int k = 0; k < j; ++k) {
                    const float2 q = t_ml[k * gv + gg];
                    if (q.y > 0.0f) m_before = fmaxf(m_before, q.x);
                }
                const float2 ml = t_ml[i];
                float4 co = make_float4(1.0f, 0.0f, 0.0f, 0.0f);
                float m_after = m_before;
                if (ml.y > 0.0f) {
                    m_after = fmaxf(m_before, ml.x);
                    co.x = expf(m_before - m_after);
                    co.y = expf(ml.x - m_after);
                    co.z = __fmul_rn(ml.y, co.y);
                    co.w = 1.0f;
                }
                t_co[i] = co;
                if (j == n - 1) t_run[((round + 1) & 1) * 16 + gg] = m_after;
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
            sync();
            FTK_STAMP(tid == 0, 22);
            if (e < E) {
                // no branch in the loop, so that the shared-memory loads of several steps are in flight together: a
                // skipped partial has the factors (1, 0) and its values (never written, possibly NaN) are replaced by 0
#pragma unroll 4
                for (int j = 0; j < n; ++j) {
                    const float4 co = t_co[j * gv + g];
                    float2 v = t_acc[(size_t)j * nthreads + tid];
                    if (co.w == 0.0f) v = make_float2(0.0f, 0.0f);
                    l = fmaf(l, co.x, co.z);
                    a0 = lse_fold(a0, co.x, v.x, co.y);
                    a1 = lse_fold(a1, co.x, v.y, co.y);
                }
            }
        }
        FTK_STAMP(tid == 0, 23);
        if (e < E) emit_final2<T, PEERS>(p, step, d.b, d.h0 + g, dd, t_run[(round & 1) * 16 + g], l, a0, a1, dd == 0);
    }
}

// One thread per CTA calls this after every thread of the CTA has written and
// fenced its part of the partial. Returns true if this CTA delivered the last
// partial of the unit and must therefore merge it.
__device__ __forceinline__ bool deliver_partial(const DecodeParams& p, const SegDest& d) {
    const int old = atomicAdd(p.counters + d.unit, 1);
    const bool last = old == d.nparts - 1;
    if (last) {
        // acquire: the other partials were fenced before their arrivals were counted; ordering this thread's
        // view after the count, and the CTA's after this thread's through the barrier that follows, is enough
        // for the L2-only loads of the merge - no fence by every thread on the critical path
        __threadfence();
        p.counters[d.unit] = 0;                // ready for the next launch
    }
    return last;
}

// End of a KV-length-split step with direct peer exchange: the warps of the grid share the
// (sequence, query head) rows; for each of its rows a warp reads the n ranks' words of the row from
// its OWN rank's buffer, polling - bounded - until the step number in them is the current one, folds
// the n triples with the reference's merge rule (src/attention.cu:503-548) and stores the normalised
// row. `gwarp` of `nwarps` identifies the warp among all participating warps of the grid; every one
// of them must call this exactly once per launch (the last one advances the step number). Nothing
// here is waited for by any other rank: a rank stores its rows as it finishes them, before it starts
// waiting, so the waits cannot form a cycle.
// What peer_fold needs, by value: it is deliberately not inlined (it runs once, at the very end of a
// kernel, and must not cost the streaming loop any registers), and a reference to the kernel's parameter
// block would force a copy of the whole block onto the stack.
struct PeerFoldArgs {
    const float* parts;      // this rank's gather blocks of the current step parity: [n][nf]
    unsigned int* hdr;       // this rank's exchange-buffer header
    int* status;
    void* out;
    long long rows, nf;
    size_t acc_off;
    int D, n;
};
__device__ __forceinline__ PeerFoldArgs peer_fold_args(const DecodeParams& p, unsigned int step) {
    PeerFoldArgs a;
    a.parts = p.peer_blocks[p.peer_rank] + (size_t)(step & 1u) * p.n_peers * (size_t)p.peer_nf;
    a.hdr = p.peer_hdr[p.peer_rank];
    a.status = p.status;
    a.out = p.out;
    a.rows = (long long)p.B * p.Hq;
    a.nf = p.peer_nf;
    a.acc_off = p.triple_acc_off;
    a.D = p.D;
    a.n = p.n_peers;
    return a;
}

template <typename T>
__device__ __noinline__ void peer_fold(const PeerFoldArgs p, unsigned int step, int gwarp, int nwarps) {
    constexpr int RB = 4;                                     // ranks whose words are in flight together
    const int lane = threadIdx.x & 31;
    unsigned int* mine = p.hdr;
    const unsigned int e = step;
    const long long rows = p.rows;
    const int D = p.D, chunks = D >> 2, n = p.n;
    const float* parts = p.parts;
    T* out = reinterpret_cast<T*>(p.out);
    bool ok = true;
    unsigned long long t0 = 0;
    // true once both 8-byte halves of a word {x, step, y, step} carry this step
    auto ready = [&](const uint4& v) { return v.y == e && v.w == e; };
    // give up after XCHG_WAIT_NS of polling in this call (a peer never delivered): report, stay usable
    auto expired = [&]() {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t0 == 0) t0 = t1;
        if (t1 - t0 > XCHG_WAIT_NS) {
            atomicCAS(p.status, ST_OK, ST_PEER_TIMEOUT);
            ok = false;
        }
        return !ok;
    };
    for (long long r = gwarp; r < rows; r += nwarps) {
        float m = -INFINITY, l = 0.0f;
        float4 o[4];                                          // head dim <= 512: at most 4 chunks per lane
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < n && ok; s0 += RB) {
            // the (m, l) words of up to RB ranks, all requested before any is looked at
            uint4 wml[RB];
#pragma unroll
            for (int q = 0; q < RB; ++q)
                if (s0 + q < n) wml[q] = ld_peer16(parts + (size_t)(s0 + q) * (size_t)p.nf + (size_t)r * 4);
#pragma unroll
            for (int q = 0; q < RB; ++q)
                if (s0 + q < n)
                    for (unsigned int it = 1; !ready(wml[q]); ++it) {
                        if ((it & 63u) == 0 && expired()) break;
                        wml[q] = ld_peer16(parts + (size_t)(s0 + q) * (size_t)p.nf + (size_t)r * 4);
                    }
            // rescale factors of these ranks in order (the reference's rule: skip l <= 0, adopt the first)
            float r_old[RB], r_new[RB];
            bool adopt[RB], live[RB];
#pragma unroll
            for (int q = 0; q < RB; ++q) {
                r_old[q] = 1.0f; r_new[q] = 0.0f; adopt[q] = false; live[q] = false;
                if (s0 + q < n) {
                    const float mq = __uint_as_float(wml[q].x), lq = __uint_as_float(wml[q].z);
                    if (lq > 0.0f) {
                        live[q] = true;
                        if (l == 0.0f) {
                            adopt[q] = true;
                            m = mq;
                            l = lq;
                        } else {
                            const float m_new = fmaxf(m, mq);
                            r_old[q] = expf(m - m_new);
                            r_new[q] = expf(mq - m_new);
                            l = lse_fold(l, r_old[q], lq, r_new[q]);
                            m = m_new;
                        }
                    }
                }
            }
            // the acc words, one chunk (4 elements = two words) of all RB ranks at a time
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cc = lane + 32 * j;
                if (cc >= chunks) continue;
                uint4 lo[RB], hi[RB];
#pragma unroll
                for (int q = 0; q < RB; ++q)
                    if (s0 + q < n) {
                        const float* a = parts + (size_t)(s0 + q) * (size_t)p.nf + p.acc_off +
                                         ((size_t)r * D + (size_t)cc * 4) * 2;
                        lo[q] = ld_peer16(a);
                        hi[q] = ld_peer16(a + 4);
                    }
#pragma unroll
                for (int q = 0; q < RB; ++q)
                    if (s0 + q < n) {
                        const float* a = parts + (size_t)(s0 + q) * (size_t)p.nf + p.acc_off +
                                         ((size_t)r * D + (size_t)cc * 4) * 2;
                        for (unsigned int it = 1; !(ready(lo[q]) && ready(hi[q])); ++it) {
                            if ((it & 63u) == 0 && expired()) break;
                            lo[q] = ld_peer16(a);
                            hi[q] = ld_peer16(a + 4);
                        }
                        if (!live[q]) continue;
                        const float4 x = make_float4(__uint_as_float(lo[q].x), __uint_as_float(lo[q].z),
                                                     __uint_as_float(hi[q].x), __uint_as_float(hi[q].z));
                        if (adopt[q]) {
                            o[j] = x;
                        } else {
                            o[j].x = lse_fold(o[j].x, r_old[q], x.x, r_new[q]);
                            o[j].y = lse_fold(o[j].y, r_old[q], x.y, r_new[q]);
                            o[j].z = lse_fold(o[j].z, r_old[q], x.z, r_new[q]);
                            o[j].w = lse_fold(o[j].w, r_old[q], x.w, r_new[q]);
                        }
                    }
            }
        }
        if (!__all_sync(0xffffffffu, ok)) break;              // the row is incomplete: leave it unwritten
        T* orow = out + (size_t)r * D;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cc = lane + 32 * j;
            if (cc < chunks) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                if (l > 0.0f) y = make_float4(o[j].x / l, o[j].y / l, o[j].z / l, o[j].w / l);
                Store<T>::st4(orow + cc * 4, y);
            }
        }
    }
    // every warp has read the step number before it arrives here; the last one advances it
    __syncwarp();
    if (lane == 0) {
        const unsigned int arrived = atomicAdd(mine + 1, 1u);
        if (arrived == (unsigned int)nwarps - 1u) {
            mine[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(mine) = e;
        }
    }
}

}  // namespace ftk
