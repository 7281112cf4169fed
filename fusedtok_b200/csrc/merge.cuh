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
        l = l * r_old + ml.y * r_new;
#pragma unroll
        for (int j = 0; j < MAX_LANE_CHUNKS; ++j) {
            const int cc = lane + 32 * j;
            if (cc < chunks) {
                const float4 x = *reinterpret_cast<const float4*>(a + cc * 4);
                o[j].x = o[j].x * r_old + x.x * r_new;
                o[j].y = o[j].y * r_old + x.y * r_new;
                o[j].z = o[j].z * r_old + x.z * r_new;
                o[j].w = o[j].w * r_old + x.w * r_new;
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

// ---- direct peer exchange -------------------------------------------------------
// Exchange buffer of one rank (allocated by the library, mapped into every
// peer through CUDA IPC): a header of 32-bit words - [0] steps completed
// (epoch), [1] block arrival counter, [16 + parity*16 + j] "rank j's block for
// the step with this parity has landed" flags - and, from byte 1024 on, the
// triple blocks gather[2][n][nf] (double-buffered by step parity).
constexpr int XCHG_DATA_BYTES = 1024;
constexpr int XCHG_FLAG_WORD = 16;
constexpr unsigned long long XCHG_WAIT_NS = 2000000000ull;      // bounded wait: 2 s

struct ExchangeParams {
    unsigned int* base[MAX_PEERS];   // every rank's exchange buffer (own included)
    int n, rank;
    long long nf;                    // floats per triple block
    int* status;                     // device status word (0 = ok)
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Second (and last) kernel of a peer-exchange step. The partial kernel before
// it has stored this rank's triple block into every peer's buffer. Block 0
// raises this rank's flag on every peer; every block then waits (bounded) until
// all n flags of this step are up in its OWN buffer - the spin is on local
// memory - and folds the n blocks of its rows. The step number lives on the
// device (so a captured graph can be replayed): the last block to have read it
// advances it.
template <typename T>
__global__ void __launch_bounds__(MERGE_WARPS * 32)
merge_peers_kernel(const ExchangeParams x, T* __restrict__ out, long long rows, int D) {
    __shared__ unsigned int s_epoch;
    __shared__ int s_ok;
    unsigned int* mine = x.base[x.rank];
    // Warp 0 does the hand-shake, lane j talking to rank j: one system-scope fence, then the n
    // flag stores go out together (fence + relaxed store = release); the n polls run in parallel
    // too, followed by one fence (relaxed load + fence = acquire).
    if (threadIdx.x < 32) {
        const int j = threadIdx.x;
        const unsigned int e = *reinterpret_cast<volatile unsigned int*>(mine) + 1u;   // this step
        const unsigned int parity = e & 1u;
        if (blockIdx.x == 0) {
            __threadfence_system();                    // the partial kernel's peer stores come first
            if (j < x.n)
                *reinterpret_cast<volatile unsigned int*>(x.base[j] + XCHG_FLAG_WORD + parity * 16 + x.rank) = e;
        }
        int ok = 1;
        if (j < x.n) {
            const volatile unsigned int* f = mine + XCHG_FLAG_WORD + parity * 16 + j;
            unsigned long long t0;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            for (unsigned int it = 0; *f != e; ++it) {
                if ((it & 255u) == 255u) {
                    unsigned long long t1;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                    if (t1 - t0 > XCHG_WAIT_NS) {       // a peer never delivered: give up, report, stay usable
                        atomicCAS(x.status, 0, 5);
                        ok = 0;
                        break;
                    }
                }
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        __threadfence_system();                        // the blocks behind the flags are visible now
        if (j == 0) {
            s_epoch = e;
            s_ok = ok;
            // every block has read the step number before it arrives here; the last one advances it
            const unsigned int arrived = atomicAdd(mine + 1, 1u);
            if (arrived == gridDim.x - 1) {
                mine[1] = 0;
                __threadfence();
                *reinterpret_cast<volatile unsigned int*>(mine) = e;
            }
        }
    }
    __syncthreads();
    if (!s_ok) return;
    const unsigned int parity = s_epoch & 1u;
    const float* parts = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(mine) + XCHG_DATA_BYTES) +
                         (size_t)parity * x.n * (size_t)x.nf;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * MERGE_WARPS + warp;
    if (r >= rows) return;
    const int chunks = D >> 2;
    const size_t acc_off = triple_acc_offset(rows);
    float4 o[MAX_LANE_CHUNKS];
#pragma unroll
    for (int j = 0; j < MAX_LANE_CHUNKS; ++j) o[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    float m = -INFINITY, l = 0.0f;
    for (int s = 0; s < x.n; ++s) {
        const float* base = parts + (size_t)s * (size_t)x.nf;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + (size_t)r * 2));
        if (ml.y <= 0.0f) continue;
        const float* a = base + acc_off + (size_t)r * D;
        if (l == 0.0f) {
            m = ml.x;
            l = ml.y;
#pragma unroll
            for (int j = 0; j < MAX_LANE_CHUNKS; ++j) {
                const int cc = lane + 32 * j;
                if (cc < chunks) o[j] = __ldcg(reinterpret_cast<const float4*>(a + cc * 4));
            }
            continue;
        }
        const float m_new = fmaxf(m, ml.x);
        const float r_old = expf(m - m_new), r_new = expf(ml.x - m_new);
        l = l * r_old + ml.y * r_new;
#pragma unroll
        for (int j = 0; j < MAX_LANE_CHUNKS; ++j) {
            const int cc = lane + 32 * j;
            if (cc < chunks) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(a + cc * 4));
                o[j].x = o[j].x * r_old + v.x * r_new;
                o[j].y = o[j].y * r_old + v.y * r_new;
                o[j].z = o[j].z * r_old + v.z * r_new;
                o[j].w = o[j].w * r_old + v.w * r_new;
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

}  // namespace ftk
