// Prefill (fresh-sequence self-attention) on CUDA cores: float32 storage and every shape the tensor-core
// prefill kernel does not take.
//
// Operator (reference: attention_prefill_cpu, src/attention.cu:1591-1638): q / out [B, Hq, S, D],
// k / v [B, Hkv, S, D]; out[b,h,i] = softmax_t(q[b,h,i] . k[b,kv(h),t] / sqrt(D)) . v[b,kv(h),t] over t <= i
// (causal) or all t. float32 must stay within 1e-5 of that CPU statement, so this path computes in plain
// fp32 FMAs (no TF32).
//
// One CTA of 256 threads (16 x 16) owns BM query rows of one (b, h) and walks the key/value rows in tiles
// of BN, flash-attention style: Q, K and V tiles live in shared memory as fp32 (row stride D+4 floats, so
// the 16 threads of a half warp reading 16 different key rows hit distinct banks), thread (ty, tx) computes
// the BM/16 x BN/16 scores of rows ty+16i and key rows tx+16j, the running max/sum are kept per row, the
// probabilities go through shared memory (over the consumed K tile) and each thread accumulates rows ty+16i x columns tx*4+64c of the
// output. Tile shape by head size (shared memory bound): D <= 128: 64x64, D <= 256: 32x32, D <= 512: 16x16.
#pragma once

#include "common.cuh"

namespace ftk {

struct PrefillParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    int B, Hq, Hkv, G, S, D;
    int causal;
    int q_tiles;         // ceil(S / BM)
    float scale;         // 1 / sqrt(D)
};

template <int BM, int BN> constexpr int prefill_simt_smem_floats(int dim) {
    const int kreg = BN * (dim + 4) > BM * (BN + 4) ? BN * (dim + 4) : BM * (BN + 4);   // K tile, later P
    return (BM + BN) * (dim + 4) + kreg;
}

template <typename T>
__device__ __forceinline__ void prefill_load_rows(float* dst, const T* src, int row0, int nrows, int seq, int dim,
                                                  int dp, int tid) {
    const int c4n = dim >> 2;
    for (int idx = tid; idx < nrows * c4n; idx += 256) {
        const int r = idx / c4n, c = (idx - r * c4n) << 2;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < seq) x = Store<T>::ld4(src + (size_t)(row0 + r) * dim + c);
        *reinterpret_cast<float4*>(dst + r * dp + c) = x;
    }
}

template <typename T, int BM, int BN>
__global__ void __launch_bounds__(256) prefill_simt_kernel(const PrefillParams p) {
    constexpr int TM = BM / 16, TN = BN / 16;
    constexpr int NC = BM == 64 ? 2 : (BM == 32 ? 4 : 8);      // 64-column output chunks per thread
    constexpr int PP = BN + 4;
    extern __shared__ __align__(16) float smem_f[];
    const int D = p.D, DP = D + 4;
    float* sQ = smem_f;
    float* sV = sQ + BM * DP;
    float* sK = sV + BN * DP;
    float* sP = sK;                                             // the probabilities replace the K tile

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int nbh = p.B * p.Hq;
    const int qt = p.q_tiles - 1 - (int)(blockIdx.x / nbh);     // long (late) row tiles first
    const int bh = blockIdx.x % nbh;
    const int b = bh / p.Hq, h = bh - b * p.Hq, kvh = h / p.G;
    const T* qb = static_cast<const T*>(p.q) + (size_t)bh * p.S * D;
    const T* kb = static_cast<const T*>(p.k) + ((size_t)b * p.Hkv + kvh) * p.S * D;
    const T* vb = static_cast<const T*>(p.v) + ((size_t)b * p.Hkv + kvh) * p.S * D;
    T* ob = static_cast<T*>(p.out) + (size_t)bh * p.S * D;
    const int q0 = qt * BM;
    const float sl2 = p.scale * 1.4426950408889634f;

    prefill_load_rows<T>(sQ, qb, q0, BM, p.S, D, DP, tid);

    float m_run[TM], l_run[TM], o[TM][NC][4];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[i][c][e] = 0.f;
    }

    const int kv_end = p.causal ? min(p.S, q0 + BM) : p.S;
    for (int k0 = 0; k0 < kv_end; k0 += BN) {
        __syncthreads();                                        // previous tile's K, V and P are consumed
        prefill_load_rows<T>(sK, kb, k0, BN, p.S, D, DP, tid);
        prefill_load_rows<T>(sV, vb, k0, BN, p.S, D, DP, tid);
        __syncthreads();

        float s[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) s[i][j] = 0.f;
        for (int d = 0; d < D; d += 4) {
            float4 qv[TM], kv4[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) qv[i] = *reinterpret_cast<const float4*>(sQ + (ty + 16 * i) * DP + d);
#pragma unroll
            for (int j = 0; j < TN; ++j) kv4[j] = *reinterpret_cast<const float4*>(sK + (tx + 16 * j) * DP + d);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    s[i][j] = fmaf(qv[i].x, kv4[j].x, s[i][j]);
                    s[i][j] = fmaf(qv[i].y, kv4[j].y, s[i][j]);
                    s[i][j] = fmaf(qv[i].z, kv4[j].z, s[i][j]);
                    s[i][j] = fmaf(qv[i].w, kv4[j].w, s[i][j]);
                }
        }

        __syncthreads();                                        // K tile consumed: its space takes P

        // online softmax in log2 units; rows are shared by the 16 threads of a half warp
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = q0 + ty + 16 * i;
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int c = k0 + tx + 16 * j;
                const bool dead = c >= p.S || (p.causal && c > r);
                s[i][j] = dead ? -INFINITY : s[i][j] * sl2;
                tmax = fmaxf(tmax, s[i][j]);
            }
#pragma unroll
            for (int off = 8; off; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
            const float m_new = fmaxf(m_run[i], tmax);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = exp2f(m_run[i] - m_use);
            m_run[i] = m_new;
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const float pr = exp2f(s[i][j] - m_use);
                psum += pr;
                sP[(ty + 16 * i) * PP + tx + 16 * j] = pr;
            }
            l_run[i] = l_run[i] * alpha + psum;
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[i][c][e] *= alpha;
        }
        __syncthreads();

        for (int c0 = 0; c0 < BN; c0 += 4) {
            float4 pv[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i) pv[i] = *reinterpret_cast<const float4*>(sP + (ty + 16 * i) * PP + c0);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int col = tx * 4 + 64 * c;
                if (col < D) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float4 vv = *reinterpret_cast<const float4*>(sV + (c0 + e) * DP + col);
#pragma unroll
                        for (int i = 0; i < TM; ++i) {
                            const float pe = e == 0 ? pv[i].x : (e == 1 ? pv[i].y : (e == 2 ? pv[i].z : pv[i].w));
                            o[i][c][0] = fmaf(pe, vv.x, o[i][c][0]);
                            o[i][c][1] = fmaf(pe, vv.y, o[i][c][1]);
                            o[i][c][2] = fmaf(pe, vv.z, o[i][c][2]);
                            o[i][c][3] = fmaf(pe, vv.w, o[i][c][3]);
                        }
                    }
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        float l = l_run[i];
#pragma unroll
        for (int off = 8; off; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        const int r = q0 + ty + 16 * i;
        if (r < p.S) {
            const float inv = 1.0f / l;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int col = tx * 4 + 64 * c;
                if (col < D)
                    Store<T>::st4(ob + (size_t)r * D + col,
                                  make_float4(o[i][c][0] * inv, o[i][c][1] * inv, o[i][c][2] * inv, o[i][c][3] * inv));
            }
        }
    }
}

}  // namespace ftk
