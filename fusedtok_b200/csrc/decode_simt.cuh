// Generic split-KV partial kernel on the CUDA cores: float32 caches (which
// must keep full fp32 products to stay within 1e-5 of the reference, so no
// tensor cores) and every 16-bit shape the tensor-core kernel does not take
// (head dims other than 64/128, pages that are not a power of two, ...).
// Same scheduler, workspace protocol and merge kernel as the tensor-core
// path; counterpart of the reference's attn_decode_kernel / attn_split_kernel /
// attn_split_paged_kernel (src/attention.cu:195-319, 336-466, 567-693).
//
// 8 warps per CTA. A warp owns whole cache rows (lanes cover the head dim in
// 4-element chunks, 128-bit accesses for fp32, 64-bit for 16-bit storage) and
// processes R rows per step so that R x GC shuffle reductions are in flight
// together; the softmax state is rescaled once per step instead of once per
// row. GC query heads of the GQA group share every loaded row.
//
// The rows of the NEXT step are always in flight while a step is computed:
// every lane copies its own chunks with cp.async into a private slot of a
// two-stage shared-memory area (no registers held across the wait, nothing
// shared between lanes, so no barrier), following its own copy of the tile
// walker one step ahead, across tile, unit and sequence boundaries.
#pragma once

#include "common.cuh"

namespace ftk {

constexpr int SIMT_WARPS = 8;
constexpr int SIMT_THREADS = SIMT_WARPS * 32;
// staging: [warp][2 stages][R rows][K, V][LC chunks][32 lanes] slots of 16 bytes; R * LC == 4 for every variant
constexpr int SIMT_STAGE_BYTES = SIMT_WARPS * 2 * 4 * 2 * 32 * 16;

// 16-byte (float32) or 8-byte (16-bit storage) asynchronous copy of 4 elements into this lane's slot;
// bytes == 0 fills the slot with zeros without reading.
template <typename T>
__device__ __forceinline__ void cp_async4(uint32_t dst, const T* src, bool live) {
    if constexpr (sizeof(T) == 4) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0)
                     : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(live ? 8 : 0)
                     : "memory");
    }
}
template <typename T> __device__ __forceinline__ float4 lds4(uint32_t addr) {
    if constexpr (sizeof(T) == 4) {
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
        return v;
    } else {
        uint2 u;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(u.x), "=r"(u.y) : "r"(addr));
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
            return make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            return make_float4(lo.x, lo.y, hi.x, hi.y);
        }
    }
}

// The sequence of row steps of one warp: tile by tile along the CTA's range, rows t0 = first row of
// the tile + warp * R, + 8 R, ... Tiles in which the warp has no row are skipped.
struct RowStep {
    Walker w;
    int t0, t_end;
    bool live;
};
__device__ __forceinline__ void rowstep_settle(const DecodeParams& p, RowStep& s, int first_off) {
    while (s.w.g < s.w.end) {
        const int t_base = s.w.ti * TILE;
        s.t_end = min(s.w.len, t_base + TILE);
        if (s.t0 < 0) s.t0 = t_base + first_off;
        if (s.t0 < s.t_end) {
            s.live = true;
            return;
        }
        walker_advance(p, s.w);
        s.t0 = -1;
    }
    s.live = false;
}

template <int N> struct Log2 { static constexpr int v = (N <= 1) ? 0 : 1 + Log2<N / 2>::v; };
template <> struct Log2<0> { static constexpr int v = 0; };

// Sum N per-lane values across the warp, all N at once: in every step a lane
// hands half of its values to its partner and keeps (and sums) the other half,
// so the N reductions cost N - 1 + (5 - log2 N) shuffles instead of 5 N. On
// return v[0] is the complete sum of value number `lane >> (5 - log2 N)`.
template <int N>
__device__ __forceinline__ float lane_transpose_reduce(float (&v)[N], int lane) {
    constexpr int K = Log2<N>::v;
#pragma unroll
    for (int s = 0; s < 5; ++s) {
        const int off = 16 >> s;
        if (s < K) {
            const int half = N >> (s + 1);
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int j = 0; j < (N > 1 ? N / 2 : 1); ++j) {
                if (j < half) {
                    const float send = up ? v[j] : v[j + half];
                    const float keep = up ? v[j + half] : v[j];
                    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
        }
    }
    return v[0];
}

// GC: query heads per unit (1, 2, 4, 8); LC: 4-element chunks per lane
// (head dim <= 128 * LC); PEERS: the KV-length split with direct peer exchange (its end-of-kernel fold is
// compiled into a variant of its own so that the ordinary kernel carries none of it).
template <typename T, int GC, int LC, bool PEERS>
__global__ void __launch_bounds__(SIMT_THREADS)
decode_simt_kernel(const DecodeParams p) {
    constexpr int R = (LC == 1) ? 4 : (LC == 2 ? 2 : 1);
    constexpr int DMAX = 128 * LC;
    __shared__ SchedShared sh;
    __shared__ __align__(16) float s_acc[SIMT_WARPS][GC][DMAX];
    __shared__ float2 s_ml[SIMT_WARPS][GC];
    __shared__ float s_scale[SIMT_WARPS][GC];
    __shared__ float2 s_glob[GC];
    __shared__ int s_last;

    // Launched with programmatic stream serialization: up to here (and, when every sequence has p.T
    // rows, through the arithmetic of the tile schedule) the kernel may overlap the tail of the
    // previous kernel in the stream; global memory is touched only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    Walker w;
    bool have_work;                             // block-uniform
    // (the step number of a KV-length split with peer exchange is re-read where it is needed - at segment
    // ends and at the very end - rather than carried in a register through the streaming loop)
    if (!p.lens) {
        have_work = sched_init<T>(p, &sh, w, 0u);
        asm volatile("griddepcontrol.wait;" ::: "memory");
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        have_work = sched_init<T>(p, &sh, w, PEERS ? peer_step(p) : 0u);   // reads lens
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (!have_work) {
        if constexpr (PEERS) {
            const unsigned int step = peer_step(p);
            peer_fold<T>(peer_fold_args(p, step), step, (int)blockIdx.x * SIMT_WARPS + warp, p.ncta * SIMT_WARPS);
        }
        return;
    }
    const int D = p.D;
    const int chunks = D >> 2;
    const T* kbase = reinterpret_cast<const T*>(p.k);
    const T* vbase = reinterpret_cast<const T*>(p.v);

    // this lane's staging slots: ((stage * R + r) * 2 + kv) * LC + j
    extern __shared__ __align__(16) unsigned char simt_stage[];
    const uint32_t slot0 = (uint32_t)__cvta_generic_to_shared(simt_stage) + (uint32_t)(warp * 2 * 4 * 2 * 32 + lane) * 16u;
    auto slot = [&](int stage, int r, int kvsel, int j) {
        return slot0 + (uint32_t)((((stage * R + r) * 2 + kvsel) * LC + j) * 32) * 16u;
    };
    // issue the copies of one step (or nothing when the steps are exhausted) and close the group
    auto prefetch = [&](const RowStep& s, int stage) {
        if (s.live) {
            const int kvh = s.w.ub / p.NCH;
            const int t_base = s.w.ti * TILE;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int t = s.t0 + r;
                const bool live = t < s.t_end;
                size_t row;
                if (p.table) {
                    const int tt = live ? t : t_base;
                    const int blk = __ldg(p.table + (size_t)s.w.b * p.tbl_width + tt / p.page);
                    row = ((size_t)blk * p.Hkv + kvh) * p.page + (tt % p.page);
                } else {
                    row = ((size_t)s.w.b * p.Hkv + kvh) * p.T + (live ? t : t_base);
                }
                const bool row_ok = FTK_ROW_OK(p, row);
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    const int c = lane + 32 * j;
                    const bool on = live && row_ok && c < chunks;
                    const size_t off = on ? row * D + c * 4 : 0;
                    cp_async4<T>(slot(stage, r, 0, j), kbase + off, on);
                    cp_async4<T>(slot(stage, r, 1, j), vbase + off, on);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    RowStep ahead;
    ahead.w = w;
    ahead.t0 = -1;
    rowstep_settle(p, ahead, warp * R);
    prefetch(ahead, 0);
    int stage = 0;

    // The R x GC scores of a step are reduced all at once (lane_transpose_reduce), after which lane
    // L owns score number L >> SH = g * R + r. The softmax state is kept the same way: a lane
    // carries (m, l) of its own head g only (l: the share of its own row slot r), computes ONE
    // weight and ONE rescale factor per step, and the warp shares them by shuffle.
    constexpr int NV = GC * R;                       // scores per step
    constexpr int SH = 5 - Log2<NV>::v;              // lane -> score number
    const int my_idx = lane >> SH, my_g = my_idx / R, my_r = my_idx % R;
    float4 qv[GC][LC], acc[GC][LC];
    float m_own = -INFINITY, l_own = 0.0f;
    long long seg_first = w.g;

    for (long long i = 0; w.g < w.end; ++i) {
        const int kv = w.ub / p.NCH, ch = w.ub % p.NCH;
        const int gvalid = min(GC, p.G - ch * p.GC);
        if (i == 0 || w.ti == 0) {
            seg_first = w.g;
            const T* qb = reinterpret_cast<const T*>(p.q) + ((size_t)w.b * p.Hq + kv * p.G + ch * p.GC) * D;
            m_own = -INFINITY;
            l_own = 0.0f;
#pragma unroll
            for (int g = 0; g < GC; ++g) {
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    const int c = lane + 32 * j;
                    acc[g][j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    qv[g][j] = (g < gvalid && c < chunks) ? Store<T>::ld4(qb + (size_t)g * D + c * 4)
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
        // rows of this tile: warp takes rows warp, warp + 8, ... in steps of R
        const int t_base = w.ti * TILE;
        const int t_end = min(w.len, t_base + TILE);
        for (int t0 = t_base + warp * R; t0 < t_end; t0 += SIMT_WARPS * R) {
            // next step's rows go in flight, then this step's (copied one step ago) are taken
            if (ahead.live) {
                ahead.t0 += SIMT_WARPS * R;
                if (ahead.t0 >= ahead.t_end) {
                    walker_advance(p, ahead.w);
                    ahead.t0 = -1;
                }
                rowstep_settle(p, ahead, warp * R);
            }
            prefetch(ahead, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            float4 kc[R][LC], vc[R][LC];
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    kc[r][j] = lds4<T>(slot(stage, r, 0, j));
                    vc[r][j] = lds4<T>(slot(stage, r, 1, j));
                }
            }
            stage ^= 1;
            float sc[NV];
#pragma unroll
            for (int g = 0; g < GC; ++g)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float d = 0.0f;
#pragma unroll
                    for (int j = 0; j < LC; ++j)
                        d += qv[g][j].x * kc[r][j].x + qv[g][j].y * kc[r][j].y +
                             qv[g][j].z * kc[r][j].z + qv[g][j].w * kc[r][j].w;
                    sc[g * R + r] = d;
                }
            // my score: head my_g, row t0 + my_r
            float s_own = lane_transpose_reduce<NV>(sc, lane) * p.scale;
            if (t0 + my_r >= t_end) s_own = -INFINITY;
            float mx = s_own;                                   // max over the R rows of my head
#pragma unroll
            for (int o = 1; o < R; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o << SH));
            const float m_new = fmaxf(m_own, mx);               // finite: row t0 is always live
            const float r_own = expf(m_own - m_new);
            const float p_own = expf(s_own - m_new);
            l_own = l_own * r_own + p_own;
            m_own = m_new;
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                const float r_old = __shfl_sync(0xffffffffu, r_own, (g * R) << SH);
                float pr[R];
#pragma unroll
                for (int r = 0; r < R; ++r) pr[r] = __shfl_sync(0xffffffffu, p_own, (g * R + r) << SH);
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    float4 a = acc[g][j];
                    a.x *= r_old; a.y *= r_old; a.z *= r_old; a.w *= r_old;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        a.x += pr[r] * vc[r][j].x;
                        a.y += pr[r] * vc[r][j].y;
                        a.z += pr[r] * vc[r][j].z;
                        a.w += pr[r] * vc[r][j].w;
                    }
                    acc[g][j] = a;
                }
            }
        }

        const bool seg_end = (w.ti == w.nt - 1) || (w.g + 1 == w.end);
        if (seg_end) {
            // this kernel always runs the equal split: one range per CTA
            const Plan pl = make_plan(sh.total, p.ncta, 0, 0);
            const unsigned int step = PEERS ? peer_step(p) : 0u;
            const SegDest dst = seg_dest(p, pl, w, (int)blockIdx.x, seg_first);
            __syncthreads();                                  // scratch free
#pragma unroll
            for (int g = 0; g < GC; ++g) {
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    const int c = lane + 32 * j;
                    if (c < chunks) *reinterpret_cast<float4*>(&s_acc[warp][g][c * 4]) = acc[g][j];
                }
            }
            {
                float l_g = l_own;                               // total over the R row slots of my head
#pragma unroll
                for (int o = 1; o < R; o <<= 1) l_g += __shfl_xor_sync(0xffffffffu, l_g, o << SH);
                if ((lane & ((1 << SH) - 1)) == 0 && my_r == 0) s_ml[warp][my_g] = make_float2(m_own, l_g);
            }
            __syncthreads();
            if (threadIdx.x < SIMT_WARPS * GC) {
                const int ww = threadIdx.x / GC, g = threadIdx.x % GC;
                float mg = -INFINITY;
                for (int x = 0; x < SIMT_WARPS; ++x)
                    if (s_ml[x][g].y > 0.0f) mg = fmaxf(mg, s_ml[x][g].x);
                s_scale[ww][g] = (s_ml[ww][g].y > 0.0f) ? expf(s_ml[ww][g].x - mg) : 0.0f;
                if (ww == 0) {
                    float lg = 0.0f;
                    for (int x = 0; x < SIMT_WARPS; ++x)
                        if (s_ml[x][g].y > 0.0f) lg += s_ml[x][g].y * expf(s_ml[x][g].x - mg);
                    s_glob[g] = make_float2(mg, lg);
                }
            }
            __syncthreads();
            const int halfd = D >> 1;
            for (int e = threadIdx.x; e < gvalid * halfd; e += SIMT_THREADS) {
                const int g = e / halfd, d = (e % halfd) * 2;
                float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
                for (int x = 0; x < SIMT_WARPS; ++x) {
                    const float sc = s_scale[x][g];
                    a0 += s_acc[x][g][d] * sc;
                    a1 += s_acc[x][g][d + 1] * sc;
                }
                const float2 ml = s_glob[g];
                if (dst.whole) {
                    emit_final2<T, PEERS>(p, step, dst.b, dst.h0 + g, d, ml.x, ml.y, a0, a1, d == 0);
                } else if (FTK_SLOT_OK(p, dst.slot, dst.unit)) {
                    const size_t pr = dst.slot * p.GC + g;
                    *reinterpret_cast<float2*>(p.ws_acc + pr * D + d) = make_float2(a0, a1);
                    if (d == 0) *reinterpret_cast<float2*>(p.ws_ml + pr * 2) = ml;
                }
            }
            if (!dst.whole && FTK_SLOT_OK(p, dst.slot, dst.unit)) {
                // publish the partial; the CTA that publishes a unit's last one merges it
                __threadfence();
                __syncthreads();
                if (threadIdx.x == 0) s_last = deliver_partial(p, dst) ? 1 : 0;
                __syncthreads();
                if (s_last) {
                    merge_unit<T, PEERS>(p, pl, dst, step, threadIdx.x, SIMT_THREADS);
                }
            }
        }
        walker_advance(p, w);
    }
    // KV-length split: fold this CTA's share of the rows over the n ranks (every warp of the grid takes part)
    if constexpr (PEERS) {
        const unsigned int step = peer_step(p);
        peer_fold<T>(peer_fold_args(p, step), step, (int)blockIdx.x * SIMT_WARPS + warp, p.ncta * SIMT_WARPS);
    }
}

}  // namespace ftk
