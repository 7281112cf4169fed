// Generic split-KV partial kernel on the CUDA cores: float32 caches (which
// must keep full fp32 products to stay within 1e-5 of the reference, so no
// tensor cores) and every 16-bit shape the tensor-core kernel does not take
// (head dims other than 64/128, pages that are not a power of two, ...).
// Same scheduler, workspace protocol and merge kernel as the tensor-core
// path; counterpart of the reference's attn_decode_kernel / attn_split_kernel /
// attn_split_paged_kernel (src/attention.cu:195-319, 336-466, 567-693).
//
// 8 warps per CTA. A warp owns whole cache rows (lanes cover the head dim in
// 4-element chunks, 128-bit loads for fp32, 64-bit for 16-bit storage) and
// processes R rows per step so that R independent K/V row loads and R x GC
// shuffle reductions are in flight together; the softmax state is rescaled
// once per step instead of once per row. GC query heads of the GQA group
// share every loaded row.
#pragma once

#include "common.cuh"

namespace ftk {

constexpr int SIMT_WARPS = 8;
constexpr int SIMT_THREADS = SIMT_WARPS * 32;

// GC: query heads per unit (1, 2, 4, 8); LC: 4-element chunks per lane
// (head dim <= 128 * LC).
template <typename T, int GC, int LC>
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

    Walker w;
    if (!sched_init<T>(p, &sh, w)) return;
    const long long total = sh.total;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D;
    const int chunks = D >> 2;
    const T* kbase = reinterpret_cast<const T*>(p.k);
    const T* vbase = reinterpret_cast<const T*>(p.v);

    float4 qv[GC][LC], acc[GC][LC];
    float m[GC], l[GC];
    long long seg_first = w.g;

    for (long long i = 0; w.g < w.end; ++i) {
        const int kv = w.ub / p.NCH, ch = w.ub % p.NCH;
        const int gvalid = min(GC, p.G - ch * p.GC);
        if (i == 0 || w.ti == 0) {
            seg_first = w.g;
            const T* qb = reinterpret_cast<const T*>(p.q) + ((size_t)w.b * p.Hq + kv * p.G + ch * p.GC) * D;
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                m[g] = -INFINITY;
                l[g] = 0.0f;
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
            float4 kc[R][LC], vc[R][LC];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int t = t0 + r;
                const bool live = t < t_end;
                size_t row;
                if (p.table) {
                    const int tt = live ? t : t_base;
                    const int blk = __ldg(p.table + (size_t)w.b * p.tbl_width + tt / p.page);
                    row = ((size_t)blk * p.Hkv + kv) * p.page + (tt % p.page);
                } else {
                    row = ((size_t)w.b * p.Hkv + kv) * p.T + (live ? t : t_base);
                }
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    const int c = lane + 32 * j;
                    if (live && c < chunks) {
                        kc[r][j] = Store<T>::ld4(kbase + row * D + c * 4);
                        vc[r][j] = Store<T>::ld4(vbase + row * D + c * 4);
                    } else {
                        kc[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        vc[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                float dot[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float s = 0.0f;
#pragma unroll
                    for (int j = 0; j < LC; ++j)
                        s += qv[g][j].x * kc[r][j].x + qv[g][j].y * kc[r][j].y +
                             qv[g][j].z * kc[r][j].z + qv[g][j].w * kc[r][j].w;
                    dot[r] = s;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                    for (int r = 0; r < R; ++r) dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], o);
                float mx = -INFINITY;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    dot[r] = (t0 + r < t_end) ? dot[r] * p.scale : -INFINITY;
                    mx = fmaxf(mx, dot[r]);
                }
                const float m_new = fmaxf(m[g], mx);          // finite: row t0 is always live
                const float r_old = expf(m[g] - m_new);
                float pr[R], psum = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    pr[r] = expf(dot[r] - m_new);
                    psum += pr[r];
                }
                l[g] = l[g] * r_old + psum;
                m[g] = m_new;
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
            const SegDest dst = seg_dest(p, w, total, seg_first);
            __syncthreads();                                  // scratch free
#pragma unroll
            for (int g = 0; g < GC; ++g) {
#pragma unroll
                for (int j = 0; j < LC; ++j) {
                    const int c = lane + 32 * j;
                    if (c < chunks) *reinterpret_cast<float4*>(&s_acc[warp][g][c * 4]) = acc[g][j];
                }
                if (lane == 0) s_ml[warp][g] = make_float2(m[g], l[g]);
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
                    emit_final2<T>(p, dst.b, dst.h0 + g, d, ml.x, ml.y, a0, a1, d == 0);
                } else {
                    const size_t pr = dst.slot * p.GC + g;
                    *reinterpret_cast<float2*>(p.ws_acc + pr * D + d) = make_float2(a0, a1);
                    if (d == 0) *reinterpret_cast<float2*>(p.ws_ml + pr * 2) = ml;
                }
            }
            if (!dst.whole) {
                // publish the partial; the CTA that publishes a unit's last one merges it
                __threadfence();
                __syncthreads();
                if (threadIdx.x == 0) s_last = deliver_partial(p, dst) ? 1 : 0;
                __syncthreads();
                if (s_last) {
                    __threadfence();
                    merge_unit<T>(p, dst, total, threadIdx.x, SIMT_THREADS);
                }
            }
        }
        walker_advance(p, w);
    }
}

}  // namespace ftk
