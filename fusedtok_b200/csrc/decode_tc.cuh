// Split-KV partial kernel for 16-bit caches (bf16 / fp16), head dims that are a
// multiple of 16 up to 256, up to 16 query heads per kv head and chunk: the sm_100a counterpart of the
// reference's attn_decode_kernel / attn_split_kernel / attn_split_paged_kernel
// (src/attention.cu:195-319, 336-466, 567-693), redesigned around the memory
// system instead of translated.
//
//  * One persistent CTA per SM: 1 producer warp + 8 consumer warps.
//  * The producer streams K/V tiles (64 cache rows) into a shared-memory ring
//    with TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, L2 evict-first),
//    completion signalled on mbarriers. It runs ahead across unit boundaries,
//    so the HBM stream never drains while consumers finish a unit.
//    The cache is described to TMA as a rank-3 tensor (64 elements, rows,
//    128-byte column blocks of a row), so ONE copy brings a [rows x D] box and
//    lays it out as [column block][row][128 B] in shared memory, the layout
//    the swizzled ldmatrix reads want. Contiguous cache: one 16 KB box for K
//    and one for V per tile. Paged cache: the block table is read one entry
//    per lane and every lane issues the two boxes of its own page, so the
//    indirection costs no per-row integer divide and no dependent load in
//    the consumers.
//  * The query heads of one GQA group are the M rows of an m16n8k16 tensor-core
//    tile (S = Q K^T, O += P V), so every K/V byte is read from HBM once and
//    from shared memory once, for all heads of the group. Tiles alternate
//    between two groups of 4 consumer warps; each warp owns 16 rows of a tile
//    and keeps an fp32 online-softmax state (m, l, O) in registers.
//  * At the end of a segment the 8 warp states are folded through shared
//    memory and either finished in place or written to the workspace; the
//    CTA that delivers the last partial of a unit merges them (no second
//    launch).
//  * The CTA works through RANGES of the tile sequence (common.cuh): its static
//    range first, then tail ranges that the producer takes from an atomic
//    counter (asked for while the previous range's last tile goes out, so the
//    round trip is hidden) and announces to the consumers through a small
//    ring of range descriptors in shared memory.
//  * KV-length split across GPUs: finished units are stored into every rank's
//    exchange buffer, the step number riding beside every value; at its end
//    the CTA folds its share of the rows over the n ranks (peer_fold) - one
//    launch per step and rank, no fence and no flag on the way.
//
// Every wait on an mbarrier is bounded (wall-clock limit); on expiry the
// kernel records a status code, stops waiting and still runs to completion,
// so a lost copy can never hang the GPU.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "common.cuh"

namespace ftk {

constexpr int NCW = 8;                        // consumer warps
constexpr int TC_THREADS = (NCW + 1) * 32;    // + 1 producer warp
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

// A range as the producer announces it to the consumers: the walker at its first tile and its index
// (r < 0: no more ranges for this CTA).
struct RangeDesc {
    long long g, end;
    int b, ub, ti, nt, len, r;
};
// Descriptors in flight. The producer writes descriptor j only after it has a free ring stage for the
// range's first tile, i.e. when the consumers are inside range j - NS or later (every range has at
// least one tile), so a ring of more than NS + 1 descriptors is never overwritten while still unread.
constexpr int QD = 16;

template <int D> struct TcCfg {
    static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head dim: a multiple of 16 up to 256");
    static constexpr int NH = (D + 63) / 64;           // 128-byte column blocks per row (the last one may be partial)
    static constexpr int DP = NH * 64;                 // row width in shared memory, elements
    static constexpr bool SPLIT = (D % 64) != 0;       // one copy per column block (rank-2 map) instead of one per box
    static constexpr int KV_BYTES = TILE * DP * 2;     // K (or V) bytes per stage
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    // Ring depth. MUST be even: tiles alternate between the two consumer
    // groups, and with an even depth a stage is always consumed by the same
    // group, which therefore observes every phase of that stage's barrier in
    // order. With an odd depth a group would wait on a stage it did not
    // consume the previous time round, and a parity wait cannot tell "not
    // filled yet" from "filled twice since".
    // Depth 4 x 32 KB (128 KB in flight per SM) measured faster than 6 x 32 KB:
    // more outstanding requests than that only lengthen the DRAM queues.
#ifdef FTK_NS
    static constexpr int NS = FTK_NS;
#else
    static constexpr int NS = (DP == 64) ? 8 : ((DP == 128) ? 4 : 2);   // 128 KB of K/V tiles (96 KB at 192)
#endif
    static_assert(NS % 2 == 0, "ring depth must be even (see above)");
    static constexpr int ACC_STRIDE = D + 4;           // floats; rows stay 16-byte aligned
    // Scratch of the segment-end fold ([8 warps x 8 heads] rows), also the stage of the cross-range merge:
    // rounds of 20 partials where that keeps the CTA inside the 196 KB shared-memory configuration.
    static constexpr int FOLD_BYTES = NCW * 8 * ACC_STRIDE * 4;
    static constexpr int MERGE_BYTES = merge_stage_bytes(NCW * 32, 20);
    static constexpr int SCRATCH_BYTES = (DP <= 128 && MERGE_BYTES > FOLD_BYTES) ? MERGE_BYTES : FOLD_BYTES;
    static constexpr int OFF_SCRATCH = NS * STAGE_BYTES;
    static constexpr int OFF_ML = OFF_SCRATCH + SCRATCH_BYTES;       // [NCW][8] float2
    static constexpr int OFF_BAR = OFF_ML + NCW * 8 * 8;             // full[NS], empty[NS]
    static constexpr int OFF_SCHED = OFF_BAR + 2 * NS * 8;
    static constexpr int OFF_ABORT = OFF_SCHED + (int)sizeof(SchedShared);
    static constexpr int OFF_DESC = (OFF_ABORT + 16 + 15) & ~15;               // RangeDesc[QD]
    static constexpr int OFF_DBAR = OFF_DESC + QD * (int)sizeof(RangeDesc);    // "descriptor written" barriers
    static constexpr int OFF_PREFIX = OFF_DBAR + QD * 8;                       // tile prefix sums per sequence
    static constexpr int OFF_ZPRE = OFF_PREFIX + (SCHED_MAX_B + 1) * 4;          // non-empty sequences before each one
    static constexpr int SMEM_BYTES = OFF_ZPRE + (SCHED_MAX_B + 1) * 4 + 8;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// ---- PTX wrappers ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait. Returns false when the limit expired or another warp already
// gave up; the caller then carries on without the data.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(status, ST_OK, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// Head dims that are not a multiple of 64: the cache is a rank-2 tensor (D elements, rows) and a box is copied
// one 64-element column block at a time; the part of the last block past D is zero-filled by the copy engine
// (never read: the MMAs stop at D), and nothing is read past the end of a row. Same shared-memory layout.
template <int NH>
__device__ __forceinline__ void tma_load_rows_split(uint32_t dst, const CUtensorMap* map, int row, uint32_t panel_bytes,
                                                    uint32_t bar, uint64_t pol) {
#pragma unroll
    for (int cb = 0; cb < NH; ++cb)
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%2, %3}], [%4], %5;"
            ::"r"(dst + cb * panel_bytes), "l"(map), "r"(cb * 64), "r"(row), "r"(bar), "l"(pol)
            : "memory");
}
// Box [64 elements, box_rows rows, D/64 column blocks] starting at row `row`.
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, int row, uint32_t bar,
                                              uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(0), "r"(bar), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr)
                 : "memory");
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Transpose an 8x8 matrix of 16-bit elements held one row pair per thread
// (row = lane / 4, columns 2 * (lane % 4) + {0, 1}) across the warp.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory"); }
// Barrier over the consumer warps that also ORs a predicate: every consumer thread gets the same answer.
__device__ __forceinline__ bool consumers_any(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "n"(NCW * 32)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- optional timeline (diagnostic builds only: -DFTK_TIMELINE) ----------------
// Per-CTA wall-clock stamps and accumulated durations of the last launch, written by one thread of
// consumer warp 0 (and one stamp by the producer); read back with ftk_debug_timeline(). Slots:
// 0 entry, 1 dependency wait done, 2 schedule done, 3 first tile landed, 4 producer issued its last
// copy, 5 last tile consumed, 6 exit, 7 ns spent at segment ends (sum), 8 segment ends, 9 ns spent
// waiting for tiles (sum), 10 ns in the final publish, 11 ranges processed, 12 ns waiting for range
// descriptors (sum), 13 the SM the CTA ran on, 14 units merged by this CTA, 15 producer issued its first copy,
// 16 producer warp starts, 17 its first range located, 18 first stage free and announced, 19 before the merge
// of a unit, 20 after it (last one of the CTA), 21-23 inside that merge: requests issued, data landed and
// coefficients ready, fold done. (Buffer and macros: common.cuh.)

// ---- the kernel ------------------------------------------------------------
// T: __nv_bfloat16 or __half. D: a multiple of 16 up to 256 (above 128, and where not a multiple of 64, with GP = 8 only). GP: 8 or 16 = query-head rows of
// the MMA tile that carry data (heads per unit <= GP). PAGED selects the
// block-table front end.
template <typename T, int D, int GP, bool PAGED>
__global__ void __launch_bounds__(TC_THREADS, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const DecodeParams p) {
    using Cfg = TcCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    SchedShared* sh = reinterpret_cast<SchedShared*>(smem + Cfg::OFF_SCHED);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_ABORT);
    RangeDesc* desc = reinterpret_cast<RangeDesc*>(smem + Cfg::OFF_DESC);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + Cfg::OFF_BAR;
    const uint32_t bar_empty = bar_full + Cfg::NS * 8;
    const uint32_t bar_desc = smem_base + Cfg::OFF_DBAR;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef FTK_TIMELINE
    if (threadIdx.x == 0) {
        for (int i = 0; i < 24; ++i) g_timeline[blockIdx.x][i] = 0;
        g_timeline[blockIdx.x][0] = global_ns();
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_timeline[blockIdx.x][13] = smid;
    }
#endif

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        if (smem_base & 1023u) {      // the swizzle pattern assumes 1024-byte aligned stages
            *abort_flag = 1;
            atomicCAS(p.status, ST_OK, ST_SMEM_MISALIGNED);
        }
        for (int s = 0; s < Cfg::NS; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 4);     // the 4 warps of the group that consumed the stage
        }
        for (int s = 0; s < QD; ++s) mbar_init(bar_desc + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
    }
    __syncthreads();
    // Programmatic dependent launch: everything above touched only this CTA's
    // shared memory and kernel parameters, so it may overlap the tail of the
    // previous kernel in the stream; from here on global memory is read and
    // written, which must wait for that kernel to have completed. Letting our
    // own dependents start early is always safe: they wait the same way.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int upb = p.Hkv * p.NCH;
    const int upb_nch = p.NCH;
    const unsigned int* prefix = nullptr;       // tile prefix sums, when the schedule needs them
    const unsigned int* zprefix = nullptr;      // ... and the count of non-empty sequences before each one
    Walker w0;                                  // equal-split range of this CTA (more sequences than the table holds)
    bool have0 = false, by_scan = false;
    long long total;
    unsigned int step = 0;                      // step number of a KV-length split with peer exchange
    Plan plan;
    bool located = false;                       // (producer warp) w0 already holds this CTA's range
    if (!p.lens) {
        // every sequence has p.T rows: the schedule - the plan and, in the producer warp, this CTA's range - is
        // arithmetic on kernel parameters and belongs to the part that may overlap the previous kernel
        total = (long long)p.B * tiles_of(p.T) * upb;
        plan = make_plan(total, p.ncta, p.dyn_chunk, p.dyn_tail_max);
        if (p.cost_split && total > 0)
            plan_enable_cost(plan, (long long)p.B * tiles_of(p.T), p.B, upb, nullptr, nullptr, tiles_of(p.T), p.cost_a,
                             p.cost_b);
        if (warp == NCW && plan.ctot) {
            w0 = walker_locate_cost_range(p, plan, static_range(plan, (int)blockIdx.x));
            located = true;
        }
        // The producer warp of a contiguous cache goes on without waiting - range descriptor, first tile's
        // coordinates, stage, expect-tx are all shared memory and arithmetic - and waits right before its first
        // copy; with a block table its very next step reads the table, so it waits here like everybody else.
        if (warp != NCW || PAGED) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            FTK_STAMP(threadIdx.x == 0, 1);
            step = peer_step(p);
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        FTK_STAMP(threadIdx.x == 0, 1);
        step = peer_step(p);
        if (p.sched_table) {
            unsigned int* table = reinterpret_cast<unsigned int*>(smem + Cfg::OFF_PREFIX);
            unsigned int* ztable = reinterpret_cast<unsigned int*>(smem + Cfg::OFF_ZPRE);
            total = sched_prefix<T>(p, sh, table, ztable, step);      // reads lens
            prefix = table;
            zprefix = ztable;
        } else {
            by_scan = true;                                     // the host disables the dynamic tail for these
            have0 = sched_init<T>(p, sh, w0, step);
            total = sh->total;
        }
    }
    if (*abort_flag) return;
    if (p.lens) {
        plan = make_plan(total, p.ncta, by_scan ? 0 : p.dyn_chunk, p.dyn_tail_max);
        if (p.cost_split && prefix && total > 0)
            plan_enable_cost(plan, prefix[p.B], zprefix[p.B], upb, prefix, zprefix, 0, p.cost_a, p.cost_b);
    }
    const Plan pl = plan;
    FTK_STAMP(threadIdx.x == 0, 2);

    if (warp == NCW) {
        // ===================== producer warp =====================
        // Everything a tile's copies need (row coordinates, block-table
        // entries, byte count) is worked out BEFORE the wait for its ring
        // stage, so that the copies go out the moment the stage is free.
        FTK_STAMP(lane == 0, 16);
        const uint64_t pol = policy_evict_first();
        int issued = 0;
        int kv = 0, unit_row0 = 0;          // of the current unit
        int row = 0, npg = 0;               // of the prepared tile (row: per lane for small pages)
        uint32_t bytes = 0;
        // paged cache: 32 consecutive block-table entries of the current sequence, one per lane,
        // fetched with one coalesced load and reused for the tiles they cover
        int tbl_b = -1, tbl_base = 0, tbl_val = 0;
        bool new_unit = true;
        Walker w = {};
        auto prepare = [&]() {
            if (new_unit) {
                kv = w.ub / upb_nch;
                unit_row0 = (w.b * p.Hkv + kv) * p.T;
            }
            if constexpr (!PAGED) {
                row = unit_row0 + w.ti * TILE;
                bytes = 2 * Cfg::KV_BYTES;
            } else {
                const int t0 = w.ti * TILE;
                if (p.page <= TILE) {
                    const int valid = min(TILE, w.len - t0);
                    npg = (valid + p.page - 1) >> p.box_shift;          // page == box rows, a power of two
                    const int pg0 = t0 >> p.box_shift;
                    if (tbl_b != w.b || pg0 < tbl_base || pg0 + npg > tbl_base + 32) {
                        tbl_b = w.b;
                        tbl_base = pg0;
                        const int idx = pg0 + lane;
                        tbl_val = idx < p.tbl_width ? __ldg(p.table + (size_t)w.b * p.tbl_width + idx) : 0;
                    }
                    const int blk = __shfl_sync(0xffffffffu, tbl_val, (pg0 - tbl_base + lane) & 31);
                    row = (blk * p.Hkv + kv) * p.page;
                    bytes = (uint32_t)(npg * p.page * Cfg::DP * 4);
                } else {
                    const int blk = __ldg(p.table + (size_t)w.b * p.tbl_width + t0 / p.page);
                    row = (blk * p.Hkv + kv) * p.page + (t0 % p.page);
                    bytes = 2 * Cfg::KV_BYTES;
                }
            }
            // (small pages: `row` is per lane, and only the lanes that will copy a page hold a page of this tile)
            if ((!PAGED || p.page > TILE || lane < npg) && !FTK_ROW_OK(p, row)) row = 0;
        };
        int s = 0;                 // ring stage of the next tile
        uint32_t ph = 0;           // phase parity of that stage's current use
        int nd = 0;                // ranges announced so far
        int r = static_range(pl, (int)blockIdx.x);               // the first range is this CTA's own
        const int tail_ranges = pl.ndyn;                         // 0 under the equal split
        int* next_tail = p.counters + (size_t)p.B * upb;         // hands out the tail ranges of this launch
        bool more = by_scan ? have0 : (total > 0 && !range_empty(pl, r));
        if (pl.ctot) {
            // cost-weighted split: this CTA's range is [first tile at cost >= X_r, first tile at cost >= X_{r+1})
            if (!located) w0 = walker_locate_cost_range(p, pl, r);
            more = w0.g < w0.end;
        }
        bool gave_up = false;
        bool dep_waited = PAGED || p.lens != nullptr;            // this warp has passed the dependency wait
        FTK_STAMP(lane == 0, 17);
        while (more) {
            w = (by_scan || pl.ctot) ? w0 : walker_locate(p, prefix, range_start(pl, r), range_start(pl, r + 1));
            bool announce = true;
            new_unit = true;
            prepare();
            // Ask for the range after this one right away: the answer is only needed once this whole range
            // has been issued, so the atomic's round trip (microseconds under full memory load) never holds
            // up a copy. A CTA thus always has one dynamic range in reserve.
            int taken = 0;
            if (pl.per && !dep_waited) {
                asm volatile("griddepcontrol.wait;" ::: "memory");          // the counter below is global memory
                dep_waited = true;
            }
            if (pl.per && lane == 0) taken = atomicAdd(next_tail, 1);
            while (w.g < w.end) {
                if (!mbar_wait(bar_empty + s * 8, ph ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY_TIMEOUT)) {
                    gave_up = true;
                    break;
                }
                if (announce) {
                    if (lane == 0) {
                        RangeDesc* dsc = desc + (nd % QD);
                        dsc->g = w.g; dsc->end = w.end;
                        dsc->b = w.b; dsc->ub = w.ub; dsc->ti = w.ti; dsc->nt = w.nt; dsc->len = w.len;
                        dsc->r = r;
                        mbar_arrive(bar_desc + (nd % QD) * 8);            // release: the descriptor is visible
                    }
                    ++nd;
                    announce = false;
                }
#ifdef FTK_TIMELINE
                if (lane == 0 && issued == 0) g_timeline[blockIdx.x][18] = global_ns();
#endif
                const uint32_t dst_k = smem_base + s * Cfg::STAGE_BYTES;
                const uint32_t dst_v = dst_k + Cfg::KV_BYTES;
                const uint32_t fb = bar_full + s * 8;
                if (lane == 0) mbar_expect_tx(fb, bytes);
                if (!dep_waited) {
                    asm volatile("griddepcontrol.wait;" ::: "memory");      // first global access of this warp
                    dep_waited = true;
                }
                const uint32_t panel_bytes = (uint32_t)p.box_rows * 128u;
                auto copy_box = [&](uint32_t dst, const CUtensorMap* map) {
                    if constexpr (Cfg::SPLIT) tma_load_rows_split<Cfg::NH>(dst, map, row, panel_bytes, fb, pol);
                    else tma_load_rows(dst, map, row, fb, pol);
                };
                if (!PAGED || p.page > TILE) {
                    if (lane == 0) {
                        copy_box(dst_k, &tm_k);
                        copy_box(dst_v, &tm_v);
                    }
                } else {
                    __syncwarp();                                            // expect_tx before any complete_tx
                    if (lane < npg) {
                        const uint32_t off = (uint32_t)(lane * p.page) * (uint32_t)(Cfg::DP * 2);   // page-major stage
                        copy_box(dst_k + off, &tm_k);
                        copy_box(dst_v + off, &tm_v);
                    }
                }
#ifdef FTK_TIMELINE
                if (lane == 0 && issued == 0) g_timeline[blockIdx.x][15] = global_ns();
#endif
                ++issued;
                const int ub_before = w.ub, b_before = w.b;
                walker_advance(p, w);
                if (++s == Cfg::NS) { s = 0; ph ^= 1u; }
                if (w.g < w.end) {
                    new_unit = (w.ub != ub_before) || (w.b != b_before);
                    prepare();
                }
            }
            if (gave_up) break;
            more = false;
            if (pl.per) {
                // every CTA takes from the counter until it is told "none left": tail_ranges + ncta
                // takes per launch in all, and whoever makes the last one leaves the counter at zero
                taken = __shfl_sync(0xffffffffu, taken, 0);
                if (lane == 0 && taken == tail_ranges + pl.ncta - 1) *next_tail = 0;
                if (taken < tail_ranges) {
                    r = dyn_range(pl, taken);
                    more = true;
                }
            }
        }
        FTK_STAMP(lane == 0, 4);
        if (!gave_up && lane == 0) {
            desc[nd % QD].r = -1;                                 // no more ranges for this CTA
            mbar_arrive(bar_desc + (nd % QD) * 8);
        }
        // If something went wrong, do not leave the CTA while our own copies
        // may still be landing in its shared memory: wait (bounded) for the
        // last phase of every stage that was issued.
        if (*abort_flag) {
            const int first = issued > Cfg::NS ? issued - Cfg::NS : 0;
            for (int i = first; i < issued; ++i) {
                const unsigned long long t0 = global_ns();
                while (!mbar_try_wait(bar_full + (i % Cfg::NS) * 8, (uint32_t)((i / Cfg::NS) & 1))) {
                    if (global_ns() - t0 > WAIT_LIMIT_NS) {
                        atomicCAS(p.status, ST_OK, ST_DRAIN_TIMEOUT);
                        break;
                    }
                }
            }
        }
        return;
    }

    // ======================= consumer warps =======================
    // Tokens are the M dimension of the MMA and query heads the N dimension
    // (8 per block): S^T[16 rows x 8 heads] = K[16 x D] . Q^T[D x 8] and
    // O^T[D x 8 heads] += V^T[D x 16 rows] . P^T[16 rows x 8 heads]. With up to
    // 8 heads per unit that is D/16 + D/16 MMAs per 16 cache rows - half of
    // what heads-on-M costs - which matters because the legacy mma.sync pipe is
    // the scarce compute resource of this kernel on sm_100.
    const int cg = warp >> 2;           // consumer group: takes every other tile
    const int wr = warp & 3;            // 16-row block of the tile
    const int quad = lane >> 2, qi = lane & 3;
    const float sl2 = p.scale * LOG2E;  // raw score differences -> ex2 arguments

    float* s_acc = reinterpret_cast<float*>(smem + Cfg::OFF_SCRATCH);
    float2* s_ml = reinterpret_cast<float2*>(smem + Cfg::OFF_ML);
    volatile int* s_last = abort_flag + 1;

    constexpr int KSTEPS = D / 16;      // k-steps of S^T = K Q^T
    constexpr int MT = D / 16;          // 16-row m-tiles of O^T = V^T P^T
    constexpr int NBK = GP / 8;         // 8-head blocks
    uint32_t qb[NBK][KSTEPS][2];        // Q^T as B fragments: head 8*nbk + quad, d = 16*kk + 2*qi + {0,1} (+8)
    float acc[NBK][MT][4];              // O^T: d = 16*mt + quad (+8 for [2],[3]); head 8*nbk + 2*qi + {0,1}
    float m_run[NBK][2], l_run[NBK][2]; // per head 8*nbk + 2*qi + e; l is this thread's share until the epilogue
    long long seg_first = 0;

    // Stage layout: boxes of `box_rows` rows back to back; inside a box the
    // D/64 column blocks one after the other, each [box_rows][128 B] with the
    // 16-byte chunks of a row XOR-swizzled by (row & 7).
    const int box_rows = p.box_rows, box_shift = p.box_shift;
    const uint32_t half_stride = (uint32_t)box_rows * 128u;
    auto row_off = [&](int r) -> uint32_t {
        return (uint32_t)(r >> box_shift) * (uint32_t)(box_rows * Cfg::DP * 2) + (uint32_t)(r & (box_rows - 1)) * 128u;
    };
    // per-lane ldmatrix geometry (constant over the kernel)
    const int lrow = lane & 7, lmat = lane >> 3;
    // K as the A operand: matrices (rows 0-7, chunk c), (rows 8-15, c), (rows 0-7, c+1), (rows 8-15, c+1)
    const uint32_t k_off = row_off(wr * 16 + (lmat & 1) * 8 + lrow);
    const int k_x = (lmat >> 1) ^ lrow;          // (chunk + csel) ^ lrow == chunk ^ (csel ^ lrow) for even chunk
    // V^T as the A operand (transposing load): (rows 0-7, chunk c), (rows 0-7, c+1), (rows 8-15, c), (rows 8-15, c+1)
    const uint32_t v_off = row_off(wr * 16 + (lmat >> 1) * 8 + lrow);
    const int v_x = (lmat & 1) ^ lrow;

    // One loop iteration per SEGMENT; inside, a tight loop over the tiles of
    // the segment that belong to this consumer group (every other tile). The
    // ring depth is even, so the stage of an own tile advances by 2 and keeps
    // its parity; `own` is the CTA-local index of this group's next tile.
    const float neg_inf = -INFINITY;
    int i0 = 0;                         // CTA-local index of the segment's first tile
    int own = cg;                       // next own tile (CTA-local index), always == cg (mod 2)
    int s = cg;                         // its ring stage ...
    uint32_t ph = 0;                    // ... and the phase parity of that stage's current use

    // QK^T, online softmax and PV for this warp's 16 rows of the tile in stage `s`.
    auto process = [&](auto ragged_tag, int rows_valid) {
        constexpr bool RAGGED = decltype(ragged_tag)::value;
        const uint32_t st_k = smem_base + s * Cfg::STAGE_BYTES;
        const uint32_t st_v = st_k + Cfg::KV_BYTES;
        // Rows at and past the sequence end may hold anything (stale or foreign
        // data, NaN included). Their scores are forced to -inf below; their V
        // values are cleared in the fragment registers (each register of a
        // transposed V fragment holds rows 2*qi and 2*qi + 1 of its 8-row half),
        // so that a zero weight times their contents stays zero.
        uint32_t vmask_lo = 0xffffffffu, vmask_hi = 0xffffffffu;
        if constexpr (RAGGED) {
            const int t = wr * 16 + qi * 2;
            vmask_lo = (t < rows_valid ? 0x0000ffffu : 0u) | (t + 1 < rows_valid ? 0xffff0000u : 0u);
            vmask_hi = (t + 8 < rows_valid ? 0x0000ffffu : 0u) | (t + 9 < rows_valid ? 0xffff0000u : 0u);
        }
        // Shared-memory fragment loads are issued a few steps ahead of the MMAs
        // that use them (the asm statements keep source order, so the order
        // below IS the schedule): PF fragments of K up front, the rest as the
        // MMAs free them; the first PF fragments of V before the softmax, whose
        // latency then hides theirs.
        constexpr int PF = 4;
        auto k_addr = [&](int kk) -> uint32_t {
            const int chunk = kk * 2;       // k_csel is folded into k_x
            return st_k + k_off + (chunk >> 3) * half_stride + ((uint32_t)((chunk & 7) ^ k_x) << 4);
        };
        auto v_addr = [&](int mt) -> uint32_t {
            const int chunk = mt * 2;
            return st_v + v_off + (chunk >> 3) * half_stride + ((uint32_t)((chunk & 7) ^ v_x) << 4);
        };
        uint32_t fk[PF][4], fv[PF][4];
#pragma unroll
        for (int j = 0; j < PF; ++j) ldsm_x4(k_addr(j), fk[j][0], fk[j][1], fk[j][2], fk[j][3]);
        // ---- S^T = K Q^T; even / odd k-steps in separate accumulators
        float sa[NBK][4], sb[NBK][4];
#pragma unroll
        for (int nbk = 0; nbk < NBK; ++nbk)
#pragma unroll
            for (int e = 0; e < 4; ++e) sa[nbk][e] = sb[nbk][e] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            uint32_t (&f)[4] = fk[kk % PF];
#pragma unroll
            for (int nbk = 0; nbk < NBK; ++nbk) {
                if (kk & 1) mma16816<T>(sb[nbk], f[0], f[1], f[2], f[3], qb[nbk][kk][0], qb[nbk][kk][1]);
                else mma16816<T>(sa[nbk], f[0], f[1], f[2], f[3], qb[nbk][kk][0], qb[nbk][kk][1]);
            }
            if (kk + PF < KSTEPS) ldsm_x4(k_addr(kk + PF), f[0], f[1], f[2], f[3]);
        }
#pragma unroll
        for (int j = 0; j < PF; ++j) ldsm_x4_t(v_addr(j), fv[j][0], fv[j][1], fv[j][2], fv[j][3]);
        // ---- online softmax. This thread holds, for heads 8*nbk + 2*qi + e, the raw
        // scores of rows `quad` ([e]) and `quad + 8` ([2 + e]) of the block. m_run is
        // kept in raw score units; sl2 = scale * log2(e) turns differences into ex2 arguments.
        const int r_lo = wr * 16 + quad;
        uint32_t pb[NBK][2];
#pragma unroll
        for (int nbk = 0; nbk < NBK; ++nbk) {
            float plo[2], phi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v0 = sa[nbk][e] + sb[nbk][e];
                float v1 = sa[nbk][2 + e] + sb[nbk][2 + e];
                if constexpr (RAGGED) {
                    if (r_lo >= rows_valid) v0 = neg_inf;
                    if (r_lo + 8 >= rows_valid) v1 = neg_inf;
                }
                float mx = fmaxf(v0, v1);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_old = m_run[nbk][e];
                const float m_new = fmaxf(m_old, mx);
                const float m_safe = (m_new == neg_inf) ? 0.0f : m_new;
                const float ms = -m_safe * sl2;
                const float alpha = ex2(fmaf(m_old, sl2, ms));
                plo[e] = ex2(fmaf(v0, sl2, ms));
                phi[e] = ex2(fmaf(v1, sl2, ms));
                l_run[nbk][e] = fmaf(l_run[nbk][e], alpha, plo[e] + phi[e]);
                m_run[nbk][e] = m_new;
                if (m_new != m_old) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        acc[nbk][mt][e] *= alpha;
                        acc[nbk][mt][2 + e] *= alpha;
                    }
                }
            }
            // P^T as the B operand: transpose the two 8x8 blocks (rows 0-7 / 8-15 of the block)
            pb[nbk][0] = movmatrix_trans(pack2<T>(plo[0], plo[1]));
            pb[nbk][1] = movmatrix_trans(pack2<T>(phi[0], phi[1]));
        }
        // ---- O^T += V^T P^T
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            uint32_t (&f)[4] = fv[mt % PF];
            if constexpr (RAGGED) {
                f[0] &= vmask_lo; f[1] &= vmask_lo;     // rows 0-7 of the block
                f[2] &= vmask_hi; f[3] &= vmask_hi;     // rows 8-15
            }
#pragma unroll
            for (int nbk = 0; nbk < NBK; ++nbk)
                mma16816<T>(acc[nbk][mt], f[0], f[1], f[2], f[3], pb[nbk][0], pb[nbk][1]);
            if (mt + PF < MT) ldsm_x4_t(v_addr(mt + PF), f[0], f[1], f[2], f[3]);
        }
    };

    // A partial is published one segment late: its stores are issued at the end of its own segment,
    // but the fence + arrival-counter update (and the merge, if this CTA turns out to be the unit's
    // last arriver) wait until the end of the NEXT segment, when the stores have long landed and
    // the round trip of the atomic hides under that segment's fold. The consumers therefore never
    // sit idle behind a memory fence in the middle of the stream.
    SegDest pend;
    bool have_pend = false;             // uniform over the consumer warps
    pend.whole = true; pend.slot = 0; pend.unit = 0; pend.b = pend.h0 = pend.gvalid = 0;
    pend.r_first = pend.r_last = pend.nparts = 0;
    const int tc = warp * 32 + lane;

    for (int nd = 0;; ++nd) {
        // ---- next range of this CTA, as announced by the producer
        [[maybe_unused]] const unsigned long long tl_d0 = FTK_NOW();
        const bool got = mbar_wait(bar_desc + (nd % QD) * 8, (uint32_t)((nd / QD) & 1), abort_flag, p.status,
                                   ST_WAIT_RANGE_TIMEOUT);
        if (consumers_any(!got)) break;               // the same decision in every consumer warp
        FTK_ADD(tc == 0, 12, FTK_NOW() - tl_d0);
        FTK_ADD(tc == 0, 11, 1);
        const RangeDesc rd = desc[nd % QD];
        if (rd.r < 0) break;
        const int r = rd.r;
        Walker w;
        w.g = rd.g; w.end = rd.end; w.b = rd.b; w.ub = rd.ub; w.ti = rd.ti; w.nt = rd.nt; w.len = rd.len;
    while (w.g < w.end) {
        // ---- segment begins: its tiles are local indices [i0, i0 + n)
        const long long left = w.end - w.g;
        const int n = (int)(left < (long long)(w.nt - w.ti) ? left : (long long)(w.nt - w.ti));
        seg_first = w.g;
        {
            // the unit's query rows as MMA B fragments
            const int kv = w.ub / upb_nch, ch = w.ub % upb_nch;
            const int gvalid = min(p.GC, p.G - ch * p.GC);
            const T* qbase = reinterpret_cast<const T*>(p.q) + ((size_t)w.b * p.Hq + kv * p.G + ch * p.GC) * D;
#pragma unroll
            for (int nbk = 0; nbk < NBK; ++nbk) {
                const int head = nbk * 8 + quad;
                const bool live = head < gvalid;
                const T* qrow = qbase + (size_t)head * D + qi * 2;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    qb[nbk][kk][0] = live ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16) : 0u;
                    qb[nbk][kk][1] = live ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8) : 0u;
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) acc[nbk][mt][0] = acc[nbk][mt][1] = acc[nbk][mt][2] = acc[nbk][mt][3] = 0.0f;
                m_run[nbk][0] = m_run[nbk][1] = neg_inf;
                l_run[nbk][0] = l_run[nbk][1] = 0.0f;
            }
        }
        // ---- this group's tiles of the segment
        for (; own < i0 + n; own += 2) {
            [[maybe_unused]] const unsigned long long tl_w0 = FTK_NOW();
            const bool ok = mbar_wait(bar_full + s * 8, ph, abort_flag, p.status, ST_WAIT_FULL_TIMEOUT);
            FTK_ADD(tc == 0, 9, FTK_NOW() - tl_w0);
#ifdef FTK_TIMELINE
            if (tc == 0 && g_timeline[blockIdx.x][3] == 0) g_timeline[blockIdx.x][3] = global_ns();
#endif
            const int rows_valid = w.len - (w.ti + (own - i0)) * TILE;      // >= 1
            if (ok) {
                if (rows_valid >= TILE) process(std::false_type{}, TILE);
                else if (wr * 16 < rows_valid) process(std::true_type{}, rows_valid);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);
            s += 2;
            if (s >= Cfg::NS) { s -= Cfg::NS; ph ^= 1u; }
        }
        i0 += n;
        // move the walker to the segment's last tile (same unit, no roll-over)
        w.g += n - 1;
        w.ti += n - 1;
        {
            // ---- fold the 8 warp states and emit
            [[maybe_unused]] const unsigned long long tl_s0 = FTK_NOW();
            FTK_STAMP(tc == 0, 5);
            const SegDest dst = seg_dest(p, pl, w, r, seg_first);
#pragma unroll
            for (int nbk = 0; nbk < NBK; ++nbk)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float l = l_run[nbk][e];
                    l += __shfl_xor_sync(0xffffffffu, l, 4);
                    l += __shfl_xor_sync(0xffffffffu, l, 8);
                    l += __shfl_xor_sync(0xffffffffu, l, 16);
                    l_run[nbk][e] = l;
                }
            if (have_pend) __threadfence();                        // the previous partial: stored a segment ago
            int arrivals = 0;
#pragma unroll
            for (int hh = 0; hh < NBK; ++hh) {
                bar_consumers();                                   // scratch is free again (and the fences above are done)
                // publish the previous partial; the answer is only looked at after this segment's fold
                if (hh == 0 && have_pend && tc == 0) arrivals = atomicAdd(p.counters + pend.unit, 1);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float* my = s_acc + ((size_t)warp * 8 + qi * 2 + e) * Cfg::ACC_STRIDE + quad;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        my[mt * 16] = acc[hh][mt][e];
                        my[mt * 16 + 8] = acc[hh][mt][2 + e];
                    }
                    if (quad == 0) s_ml[warp * 8 + qi * 2 + e] = make_float2(m_run[hh][e], l_run[hh][e]);
                }
                bar_consumers();
                for (int e = tc; e < 8 * (D / 2); e += NCW * 32) {
                    const int row = e / (D / 2), d = (e % (D / 2)) * 2;
                    const int g = hh * 8 + row;
                    if (g >= dst.gvalid) continue;
                    // every thread derives the merged maximum and the warps' scale factors of its row itself
                    // (8 values from shared memory, 8 ex2): cheaper than a third barrier per fold
                    float mw[NCW];
                    float mg = -INFINITY;
#pragma unroll
                    for (int ww = 0; ww < NCW; ++ww) {
                        mw[ww] = s_ml[ww * 8 + row].x;
                        mg = fmaxf(mg, mw[ww]);
                    }
                    const float mg_safe = (mg == -INFINITY) ? 0.0f : mg;
                    float a0 = 0.0f, a1 = 0.0f, lg = 0.0f;
#pragma unroll
                    for (int ww = 0; ww < NCW; ++ww) {
                        const float sc = ex2((mw[ww] - mg_safe) * sl2);
                        const float2 v = *reinterpret_cast<const float2*>(
                            s_acc + ((size_t)ww * 8 + row) * Cfg::ACC_STRIDE + d);
                        a0 += v.x * sc;
                        a1 += v.y * sc;
                        lg += s_ml[ww * 8 + row].y * sc;
                    }
                    const float2 ml = make_float2(mg * p.scale, lg);   // m from raw score units to natural-log units
                    if (dst.whole) {
                        emit_final2<T>(p, step, dst.b, dst.h0 + g, d, ml.x, ml.y, a0, a1, d == 0);
                    } else if (FTK_SLOT_OK(p, dst.slot, dst.unit)) {
                        const size_t pr = dst.slot * p.GC + g;
                        *reinterpret_cast<float2*>(p.ws_acc + pr * D + d) = make_float2(a0, a1);
                        if (d == 0) *reinterpret_cast<float2*>(p.ws_ml + pr * 2) = ml;
                    }
                }
            }
            if (have_pend) {
                // was that the unit's last partial? then this CTA merges the unit
                if (tc == 0) {
                    const bool last = arrivals == pend.nparts - 1;
                    if (last) {
                        __threadfence();                           // acquire (see deliver_partial)
                        p.counters[pend.unit] = 0;                 // ready for the next launch
                    }
                    *s_last = last ? 1 : 0;
                }
                bar_consumers();
                if (*s_last) {
                    merge_unit_staged<T>(p, pl, pend, step, tc, NCW * 32, s_acc, Cfg::SCRATCH_BYTES, [] { bar_consumers(); });
                    FTK_ADD(tc == 0, 14, 1);
                }
            }
            have_pend = !dst.whole && FTK_SLOT_OK(p, dst.slot, dst.unit);
            pend = dst;
            FTK_ADD(tc == 0, 7, FTK_NOW() - tl_s0);
            FTK_ADD(tc == 0, 8, 1);
        }
        walker_advance(p, w);
    }
    }
    [[maybe_unused]] const unsigned long long tl_f0 = FTK_NOW();
    if (have_pend) {
        // the last partial of this CTA: publish it now; the CTA that publishes a unit's last one merges it
        __threadfence();
        bar_consumers();
        if (tc == 0) *s_last = deliver_partial(p, pend) ? 1 : 0;
        bar_consumers();
        if (*s_last) {
            FTK_STAMP(tc == 0, 19);
            merge_unit_staged<T>(p, pl, pend, step, tc, NCW * 32, s_acc, Cfg::SCRATCH_BYTES, [] { bar_consumers(); });
            FTK_ADD(tc == 0, 14, 1);
            FTK_STAMP(tc == 0, 20);
        }
    }
    FTK_ADD(tc == 0, 10, FTK_NOW() - tl_f0);
    // KV-length split: fold this CTA's share of the rows over the n ranks (every consumer warp of the grid takes part)
    if (p.n_peers) peer_fold<T>(peer_fold_args(p, step), step, (int)blockIdx.x * NCW + warp, p.ncta * NCW);
    FTK_STAMP(tc == 0, 6);
}

}  // namespace ftk
