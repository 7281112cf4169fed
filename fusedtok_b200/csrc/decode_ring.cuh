// Split-KV partial kernel for float32 caches fed by a TMA ring: head dim 64 or 128, contiguous or paged
// (page a power of two >= 8), 16-byte aligned caches. Counterpart of the reference's attn_split_kernel /
// attn_split_paged_kernel in float32 (src/attention.cu:336-466, 567-693).
//
// float32 must stay within 1e-5 of the reference, so the arithmetic is the CUDA-core arithmetic of
// decode_simt.cuh (full fp32 products, one transposing warp reduction per step, one rescale per step).
// What changes is who moves the data: there, every lane copies its own 16-byte chunks with cp.async and
// generates its own addresses - exactly the issue slots that kernel is short of. Here one producer warp
// streams [32 rows x D] boxes of K and V into a shared-memory ring with cp.async.bulk.tensor (completion on
// mbarriers, L2 evict-first), 8 consumer warps read their 4 rows of a box with 128-bit shared-memory loads,
// and the persistent CTA (one per SM) walks the same equal-cost range plan as the tensor-core kernel. A
// 64-row tile of the schedule is two boxes of the ring; a box without valid rows is never copied.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a status code and still completes.
#pragma once

#include "common.cuh"
#include "decode_simt.cuh"
#include "decode_tc.cuh"

namespace ftk {

constexpr int RF_ROWS = 32;                 // cache rows per ring stage (half a tile)
constexpr int RF_THREADS = (NCW + 1) * 32;  // 8 consumer warps + 1 producer warp

template <int D, int GC> struct RfCfg {
    static_assert(D == 64 || D == 128, "head dim 64 or 128");
    static constexpr int KV_BYTES = RF_ROWS * D * 4;              // K (or V) bytes per stage
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int NS = (D == 128) ? 5 : 10;                // 160 KB of rows in flight or landed
    static constexpr int OFF_ACC = NS * STAGE_BYTES;              // fold scratch: [warp][GC][D] floats
    // (also the stage of the cross-range merge, in rounds of 20 partials)
    static constexpr int FOLD_BYTES = NCW * GC * D * 4;
    static constexpr int ACC_BYTES = FOLD_BYTES > merge_stage_bytes(NCW * 32, 20) ? FOLD_BYTES : merge_stage_bytes(NCW * 32, 20);
    static constexpr int OFF_ML = OFF_ACC + ACC_BYTES;            // [warp][GC] float2
    static constexpr int OFF_SCALE = OFF_ML + NCW * GC * 8;       // [warp][GC] float
    static constexpr int OFF_GLOB = OFF_SCALE + NCW * GC * 4;     // [GC] float2
    static constexpr int OFF_BAR = (OFF_GLOB + GC * 8 + 7) & ~7;  // full[NS], empty[NS]
    static constexpr int OFF_SCHED = OFF_BAR + 2 * NS * 8;
    static constexpr int OFF_FLAGS = OFF_SCHED + (int)sizeof(SchedShared);    // abort, last
    static constexpr int OFF_PREFIX = (OFF_FLAGS + 16 + 15) & ~15;
    static constexpr int OFF_ZPRE = OFF_PREFIX + (SCHED_MAX_B + 1) * 4;
    static constexpr int SMEM_BYTES = OFF_ZPRE + (SCHED_MAX_B + 1) * 4 + 8;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// Two float32 fused multiply-adds in one instruction (sm_100: fma.rn.f32x2). The consumers are bound by
// instruction issue, not by the FMA pipes, so halving the number of FMA instructions is what counts.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// Box [D floats, box_rows rows] of a rank-2 float32 tensor, no swizzle: lands row-major.
__device__ __forceinline__ void tma_load_rows_f32(uint32_t dst, const CUtensorMap* map, int row, uint32_t bar,
                                                  uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(bar), "l"(pol)
        : "memory");
}

template <int D, int GC, bool PAGED>
__global__ void __launch_bounds__(RF_THREADS, 1)
decode_ring_f32_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const DecodeParams p) {
    using Cfg = RfCfg<D, GC>;
    using T = float;
    constexpr int R = 4;                       // rows per warp and stage: 8 warps x 4 rows = one stage
    constexpr int NV = GC * R;                 // scores per step
    constexpr int SH = 5 - Log2<NV>::v;        // lane -> score number
    constexpr int CH = D / 4;                  // 4-element chunks per row: lanes 0 .. CH-1 carry data
    extern __shared__ __align__(1024) uint8_t smem[];
    SchedShared* sh = reinterpret_cast<SchedShared*>(smem + Cfg::OFF_SCHED);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_FLAGS);
    volatile int* s_last = abort_flag + 1;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + Cfg::OFF_BAR;
    const uint32_t bar_empty = bar_full + Cfg::NS * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < Cfg::NS; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, NCW);      // every consumer warp reads every stage
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
    }
    __syncthreads();
    // programmatic dependent launch: see decode_tc_kernel
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int upb = p.Hkv * p.NCH;
    const unsigned int* prefix = nullptr;
    const unsigned int* zprefix = nullptr;
    Walker w;                                   // this CTA's range (every warp walks it)
    bool by_scan = false, have = false;
    long long total;
    if (!p.lens) {
        // every sequence has p.T rows: plan and range are arithmetic on kernel parameters and may overlap the
        // previous kernel in the stream; the dependency wait follows them (below)
        total = (long long)p.B * tiles_of(p.T) * upb;
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (p.sched_table) {
            unsigned int* table = reinterpret_cast<unsigned int*>(smem + Cfg::OFF_PREFIX);
            unsigned int* ztable = reinterpret_cast<unsigned int*>(smem + Cfg::OFF_ZPRE);
            total = sched_prefix<T>(p, sh, table, ztable, 0u);
            prefix = table;
            zprefix = ztable;
        } else {
            by_scan = true;
            have = sched_init<T>(p, sh, w, 0u);
            total = sh->total;
        }
    }
    Plan plan = make_plan(total, p.ncta, 0, 0);
    if (p.cost_split && !by_scan && total > 0) {
        if (prefix) plan_enable_cost(plan, prefix[p.B], zprefix[p.B], upb, prefix, zprefix, 0, p.cost_a, p.cost_b);
        else plan_enable_cost(plan, (long long)p.B * tiles_of(p.T), p.B, upb, nullptr, nullptr, tiles_of(p.T), p.cost_a,
                              p.cost_b);
    }
    const Plan pl = plan;
    const int r = (int)blockIdx.x;
    if (!by_scan && total > 0) {
        if (pl.ctot) {
            w = walker_locate_cost_range(p, pl, r);
            have = w.g < w.end;
        } else if (!range_empty(pl, r)) {
            w = walker_locate(p, prefix, range_start(pl, r), range_start(pl, r + 1));
            have = true;
        }
    }
    if (!p.lens) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!have) return;

    // halves of a tile that hold valid rows: 1 or 2 (the walker never stands on an empty tile)
    auto halves_of = [&](const Walker& x) { return (x.len - x.ti * TILE) > RF_ROWS ? 2 : 1; };

    if (warp == NCW) {
        // ===================== producer warp =====================
        const uint64_t pol = policy_evict_first();
        int s = 0, issued = 0;
        uint32_t ph = 0;
        bool gave_up = false;
        while (w.g < w.end && !gave_up) {
            const int kv = w.ub / p.NCH;
            const int nh = halves_of(w);
            for (int h = 0; h < nh; ++h) {
                const int t0 = w.ti * TILE + h * RF_ROWS;
                int row = 0, npg = 1;
                uint32_t bytes = 2 * Cfg::KV_BYTES;
                if constexpr (!PAGED) {
                    row = (w.b * p.Hkv + kv) * p.T + t0;
                } else if (p.page <= RF_ROWS) {
                    // one box per page; lane j takes page j of this half tile (pages that hold valid rows only)
                    const int valid = min(RF_ROWS, w.len - t0);
                    npg = (valid + p.page - 1) >> p.box_shift;
                    const int idx = (t0 >> p.box_shift) + lane;
                    const int blk = (lane < npg && idx < p.tbl_width) ? __ldg(p.table + (size_t)w.b * p.tbl_width + idx) : 0;
                    row = (blk * p.Hkv + kv) * p.page;
                    bytes = (uint32_t)(npg * p.page * D * 4 * 2);
                } else {
                    const int blk = __ldg(p.table + (size_t)w.b * p.tbl_width + t0 / p.page);
                    row = (blk * p.Hkv + kv) * p.page + (t0 % p.page);
                }
                if (!FTK_ROW_OK(p, row)) row = 0;
                if (!mbar_wait(bar_empty + s * 8, ph ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY_TIMEOUT)) {
                    gave_up = true;
                    break;
                }
                const uint32_t dst_k = smem_base + s * Cfg::STAGE_BYTES;
                const uint32_t dst_v = dst_k + Cfg::KV_BYTES;
                const uint32_t fb = bar_full + s * 8;
                if (lane == 0) mbar_expect_tx(fb, bytes);
                if (!PAGED || p.page > RF_ROWS) {
                    if (lane == 0) {
                        tma_load_rows_f32(dst_k, &tm_k, row, fb, pol);
                        tma_load_rows_f32(dst_v, &tm_v, row, fb, pol);
                    }
                } else {
                    __syncwarp();                                            // expect_tx before any complete_tx
                    if (lane < npg) {
                        const uint32_t off = (uint32_t)(lane * p.page) * (uint32_t)(D * 4);
                        tma_load_rows_f32(dst_k + off, &tm_k, row, fb, pol);
                        tma_load_rows_f32(dst_v + off, &tm_v, row, fb, pol);
                    }
                }
                ++issued;
                if (++s == Cfg::NS) { s = 0; ph ^= 1u; }
            }
            walker_advance(p, w);
        }
        // do not leave while our own copies may still be landing in this CTA's shared memory
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
    // The arithmetic of decode_simt_kernel: a warp owns whole cache rows (lanes cover the head dim in 4-element
    // chunks), R = 4 rows per step, GC heads share each row; the R x GC scores of a step are reduced all at once,
    // after which lane L owns score number L >> SH = g * R + r and carries (m, l) of its own head only.
    float* s_acc = reinterpret_cast<float*>(smem + Cfg::OFF_ACC);          // [warp][GC][D]
    float2* s_ml = reinterpret_cast<float2*>(smem + Cfg::OFF_ML);          // [warp][GC]
    float* s_scale = reinterpret_cast<float*>(smem + Cfg::OFF_SCALE);      // [warp][GC]
    float2* s_glob = reinterpret_cast<float2*>(smem + Cfg::OFF_GLOB);      // [GC]
    const int my_idx = lane >> SH, my_g = my_idx / R, my_r = my_idx % R;
    const bool data_lane = lane < CH;
    float4 qv[GC], acc[GC];
    float m_own = -INFINITY, l_own = 0.0f;
    long long seg_first = w.g;
    int s = 0;
    uint32_t ph = 0;
    bool fresh = true;                          // the next tile starts a segment
    while (w.g < w.end) {
        const int kv = w.ub / p.NCH, ch = w.ub % p.NCH;
        const int gvalid = min(GC, p.G - ch * p.GC);
        if (fresh) {
            seg_first = w.g;
            const T* qb = reinterpret_cast<const T*>(p.q) + ((size_t)w.b * p.Hq + kv * p.G + ch * p.GC) * D;
            m_own = -INFINITY;
            l_own = 0.0f;
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
                qv[g] = (g < gvalid && data_lane) ? Store<T>::ld4(qb + (size_t)g * D + lane * 4)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            fresh = false;
        }
        const int nh = halves_of(w);
        for (int h = 0; h < nh; ++h) {
            const int t0 = w.ti * TILE + h * RF_ROWS + warp * R;      // this warp's first row of the stage
            const int t_end = w.len;
            const bool ok = mbar_wait(bar_full + s * 8, ph, abort_flag, p.status, ST_WAIT_FULL_TIMEOUT);
            if (ok && t0 < t_end) {
                // page-major stage for small pages, row-major otherwise: both are "row i at i * D floats"
                const float* st_k = reinterpret_cast<const float*>(smem + s * Cfg::STAGE_BYTES) + (warp * R) * D;
                const float* st_v = st_k + RF_ROWS * D;
                float4 kc[R], vc[R];
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const bool live = data_lane && (t0 + rr < t_end);
                    kc[rr] = live ? *reinterpret_cast<const float4*>(st_k + rr * D + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    vc[rr] = live ? *reinterpret_cast<const float4*>(st_v + rr * D + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float sc[NV];
#pragma unroll
                for (int g = 0; g < GC; ++g)
#pragma unroll
                    for (int rr = 0; rr < R; ++rr)
                    {
                        const float2 t = fma2(make_float2(qv[g].z, qv[g].w), make_float2(kc[rr].z, kc[rr].w),
                                              mul2(make_float2(qv[g].x, qv[g].y), make_float2(kc[rr].x, kc[rr].y)));
                        sc[g * R + rr] = t.x + t.y;
                    }
                // my score: head my_g, row t0 + my_r
                float s_own = lane_transpose_reduce<NV>(sc, lane) * p.scale;
                if (t0 + my_r >= t_end) s_own = -INFINITY;
                float mx = s_own;                                   // max over the R rows of my head
#pragma unroll
                for (int o = 1; o < R; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o << SH));
                const float m_new = fmaxf(m_own, mx);               // finite: row t0 is live
                const float r_own = expf(m_own - m_new);
                const float p_own = expf(s_own - m_new);
                l_own = l_own * r_own + p_own;
                m_own = m_new;
#pragma unroll
                for (int g = 0; g < GC; ++g) {
                    const float r_old = __shfl_sync(0xffffffffu, r_own, (g * R) << SH);
                    float pr[R];
#pragma unroll
                    for (int rr = 0; rr < R; ++rr) pr[rr] = __shfl_sync(0xffffffffu, p_own, (g * R + rr) << SH);
                    const float2 ro2 = make_float2(r_old, r_old);
                    float2 lo = mul2(make_float2(acc[g].x, acc[g].y), ro2);
                    float2 hi = mul2(make_float2(acc[g].z, acc[g].w), ro2);
#pragma unroll
                    for (int rr = 0; rr < R; ++rr) {
                        const float2 p2 = make_float2(pr[rr], pr[rr]);
                        lo = fma2(p2, make_float2(vc[rr].x, vc[rr].y), lo);
                        hi = fma2(p2, make_float2(vc[rr].z, vc[rr].w), hi);
                    }
                    acc[g] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);
            if (++s == Cfg::NS) { s = 0; ph ^= 1u; }
        }

        const bool seg_end = (w.ti == w.nt - 1) || (w.g + 1 == w.end);
        if (seg_end) {
            const SegDest dst = seg_dest(p, pl, w, r, seg_first);
            bar_consumers();                                  // scratch free
#pragma unroll
            for (int g = 0; g < GC; ++g)
                if (data_lane) *reinterpret_cast<float4*>(s_acc + ((size_t)warp * GC + g) * D + lane * 4) = acc[g];
            {
                float l_g = l_own;                               // total over the R row slots of my head
#pragma unroll
                for (int o = 1; o < R; o <<= 1) l_g += __shfl_xor_sync(0xffffffffu, l_g, o << SH);
                if ((lane & ((1 << SH) - 1)) == 0 && my_r == 0) s_ml[warp * GC + my_g] = make_float2(m_own, l_g);
            }
            bar_consumers();
            if (threadIdx.x < NCW * GC) {
                const int ww = threadIdx.x / GC, g = threadIdx.x % GC;
                float mg = -INFINITY;
                for (int x = 0; x < NCW; ++x)
                    if (s_ml[x * GC + g].y > 0.0f) mg = fmaxf(mg, s_ml[x * GC + g].x);
                s_scale[ww * GC + g] = (s_ml[ww * GC + g].y > 0.0f) ? expf(s_ml[ww * GC + g].x - mg) : 0.0f;
                if (ww == 0) {
                    float lg = 0.0f;
                    for (int x = 0; x < NCW; ++x)
                        if (s_ml[x * GC + g].y > 0.0f) lg += s_ml[x * GC + g].y * expf(s_ml[x * GC + g].x - mg);
                    s_glob[g] = make_float2(mg, lg);
                }
            }
            bar_consumers();
            constexpr int halfd = D >> 1;
            for (int e = threadIdx.x; e < gvalid * halfd; e += NCW * 32) {
                const int g = e / halfd, d = (e % halfd) * 2;
                float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
                for (int x = 0; x < NCW; ++x) {
                    const float scl = s_scale[x * GC + g];
                    a0 += s_acc[((size_t)x * GC + g) * D + d] * scl;
                    a1 += s_acc[((size_t)x * GC + g) * D + d + 1] * scl;
                }
                const float2 ml = s_glob[g];
                if (dst.whole) {
                    emit_final2<T, false>(p, 0u, dst.b, dst.h0 + g, d, ml.x, ml.y, a0, a1, d == 0);
                } else if (FTK_SLOT_OK(p, dst.slot, dst.unit)) {
                    const size_t pr = dst.slot * p.GC + g;
                    *reinterpret_cast<float2*>(p.ws_acc + pr * D + d) = make_float2(a0, a1);
                    if (d == 0) *reinterpret_cast<float2*>(p.ws_ml + pr * 2) = ml;
                }
            }
            if (!dst.whole && FTK_SLOT_OK(p, dst.slot, dst.unit)) {
                // publish the partial; the CTA that publishes a unit's last one merges it
                __threadfence();
                bar_consumers();
                if (threadIdx.x == 0) *s_last = deliver_partial(p, dst) ? 1 : 0;
                bar_consumers();
                if (*s_last) {
                    merge_unit_staged<T, false>(p, pl, dst, 0u, threadIdx.x, NCW * 32, reinterpret_cast<float*>(smem + Cfg::OFF_ACC),
                                                Cfg::ACC_BYTES, [] { bar_consumers(); });
                    bar_consumers();      // the stage is the next fold's scratch
                }
            }
            fresh = true;
        }
        walker_advance(p, w);
    }
}

}  // namespace ftk
