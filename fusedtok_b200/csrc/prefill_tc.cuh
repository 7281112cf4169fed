// Prefill (fresh-sequence self-attention) on the 5th-generation tensor cores: bf16 / fp16 storage,
// head dim 64, 128 or 256.
//
// Operator: see prefill_simt.cuh (reference: attention_prefill_launch_bf16 / _fp16,
// include/fusedtok/cuda_launch.hpp:370-379; the reference's own tensor-core path is the mma.sync kernel at
// src/attention.cu:951-1217).
//
// One CTA owns 128 query rows of one (batch, query head) and walks the key/value rows in tiles of 64; two
// CTAs share an SM (96 KB of shared memory, 256 tensor-memory columns and half the register file each), so
// one CTA's softmax overlaps the other's MMAs:
//
//   warp 5  (producer)   TMA: the Q tile once, then K and V tiles into two 2-stage rings. Rank-4 tensor maps
//                        (64 elements, S rows, D/64 column blocks, B*H heads): rows past the end of a head are
//                        zero-filled by the copy engine, tiles land as [column block][row][128 B], 128-byte
//                        swizzled - exactly the K-major (Q, K) and MN-major (V) operand layouts of tcgen05.mma.
//   warp 4  (MMA issue)  one elected thread: S = Q.K^T (M=128, N=64, K=D) into one of two S buffers in tensor
//                        memory (the next tile's scores are computed while the softmax warps work on this
//                        one), and after the softmax warps have produced P: O += P.V (M=128, N=D, K=64, A = P from tensor memory);
//                        completion is signalled by tcgen05.commit on mbarriers.
//   warps 0-3 (softmax)  thread t owns query row t = tensor-memory lane t: reads its S row with tcgen05.ld
//                        (no shuffles), online softmax in fp32, writes P as bf16/fp16 back into tensor memory
//                        over the scores it came from (tcgen05.st; the P.V MMA takes its A operand from
//                        tensor memory, so P never touches shared memory, whose bandwidth the operand reads of
//                        the MMAs already use up). The output row accumulates in tensor memory
//                        (P.V with accumulate) against a lazily raised reference maximum; raising it
//                        rescales the row in tensor memory (tcgen05.ld / .st). At the end the row is read
//                        back, divided by the softmax sum and stored.
//                        These warps raise their register allowance (setmaxnreg), warps 4-7 lower theirs.
//
// Tensor memory: 256 columns (S/P: 2 x 64, O: D). Every wait is bounded (2 s): on expiry the kernel records
// a status code, all roles leave their loops, tensor memory is released and the kernel returns.
#pragma once

#include "decode_tc.cuh"
#include "prefill_simt.cuh"

namespace ftk {

constexpr int PF_THREADS = 256;
constexpr int ST_PREFILL_TIMEOUT = 6;

template <int D> struct PfCfg {
    static_assert(D == 64 || D == 128 || D == 256, "tensor-core prefill: head dim 64, 128 or 256");
    static constexpr int BM = 128, BN = 64, NST = 2;
    static constexpr int Q_PANEL = BM * 128;                   // bytes: 128 rows x 128 B
    static constexpr int KV_PANEL = BN * 128;                  // 64 rows x 128 B
    static constexpr int Q_BYTES = (D / 64) * Q_PANEL;
    static constexpr int KV_BYTES = (D / 64) * KV_PANEL;       // one K or V tile
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V = OFF_K + NST * KV_BYTES;
    static constexpr int OFF_BAR = OFF_V + NST * KV_BYTES;     // 16 mbarrier slots
    static constexpr int OFF_TMEM = OFF_BAR + 16 * 8;
    static constexpr int OFF_ABORT = OFF_TMEM + 8;
    static constexpr int SMEM_BYTES = OFF_ABORT + 8;
    // S0/P0 [0,64), S1/P1 [64,128), O [128,128+D). Head dim 256 needs 384 columns (allocations are powers of
    // two) and 192 KB of shared memory: one CTA per SM there, two otherwise.
    static constexpr uint32_t TMEM_COLS = D <= 128 ? 256 : 512;
    static_assert(D > 128 || 2 * (SMEM_BYTES + 1024) <= 233472, "two CTAs must fit the 228 KB of one SM");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// ---- tcgen05 wrappers -------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading/stride byte offsets (all >> 4),
// descriptor version 1 (bits 46-47), layout type 2 = SWIZZLE_128B (bits 61-63).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate (bits 4-5 = 1), A/B format (bits 7-9 / 10-12: 0 = f16,
// 1 = bf16), A/B major (bits 15 / 16: 0 = K-major, 1 = MN-major), N >> 3 (bits 17-22), M >> 4 (bits 24-28).
__host__ __device__ constexpr uint32_t umma_idesc(int fmt, int a_mn, int b_mn, int m, int n) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn << 15) |
           ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand (K-major, 16-bit elements packed two per column) read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// 32 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&x)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(r[i]);
}
// 64 consecutive fp32 columns of this thread's tensor-memory lane (two loads in flight, one wait).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&x)[64]) {
    uint32_t r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr), "r"(taddr + 32)
        : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) x[i] = __uint_as_float(r[i]);
}
// Write 32 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&x)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n\t"
        "tcgen05.wait::st.sync.aligned;"
        ::"r"(taddr), "r"(__float_as_uint(x[0])), "r"(__float_as_uint(x[1])), "r"(__float_as_uint(x[2])), "r"(__float_as_uint(x[3])), "r"(__float_as_uint(x[4])), "r"(__float_as_uint(x[5])), "r"(__float_as_uint(x[6])), "r"(__float_as_uint(x[7])), "r"(__float_as_uint(x[8])), "r"(__float_as_uint(x[9])), "r"(__float_as_uint(x[10])), "r"(__float_as_uint(x[11])), "r"(__float_as_uint(x[12])), "r"(__float_as_uint(x[13])), "r"(__float_as_uint(x[14])), "r"(__float_as_uint(x[15])), "r"(__float_as_uint(x[16])), "r"(__float_as_uint(x[17])), "r"(__float_as_uint(x[18])), "r"(__float_as_uint(x[19])), "r"(__float_as_uint(x[20])), "r"(__float_as_uint(x[21])), "r"(__float_as_uint(x[22])), "r"(__float_as_uint(x[23])), "r"(__float_as_uint(x[24])), "r"(__float_as_uint(x[25])), "r"(__float_as_uint(x[26])), "r"(__float_as_uint(x[27])), "r"(__float_as_uint(x[28])), "r"(__float_as_uint(x[29])), "r"(__float_as_uint(x[30])), "r"(__float_as_uint(x[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st32p(uint32_t taddr, const uint32_t (&x)[32]) {
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(x[i]);
    tmem_st32(taddr, f);
}
// Wait that ignores the abort flag: used on the way out, so that no copy or MMA of this CTA is still in
// flight when its shared and tensor memory are given back. Bounded all the same.
__device__ __forceinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return;
    const unsigned long long t0 = global_ns();
    while (!mbar_try_wait(bar, parity))
        if (global_ns() - t0 > WAIT_LIMIT_NS) return;
}
// Box [64 elements, box rows, D/64 column blocks, 1 head] at (row, head).
__device__ __forceinline__ void tma_load_tile4(uint32_t dst, const CUtensorMap* map, int row, int head, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(0), "r"(head), "r"(bar)
        : "memory");
}

template <typename T, int D>
__global__ void __launch_bounds__(PF_THREADS, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const PrefillParams p, int* status) {
    using C = PfCfg<D>;
    extern __shared__ __align__(1024) uint8_t pf_smem[];
    const uint32_t base = smem_u32(pf_smem);
    if (base & 1023u) {                                         // the swizzled operand layouts need it
        if (threadIdx.x == 0) atomicCAS(status, ST_OK, ST_SMEM_MISALIGNED);
        return;
    }
    volatile int* abort_flag = reinterpret_cast<volatile int*>(pf_smem + C::OFF_ABORT);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(pf_smem + C::OFF_TMEM);
    auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
    enum { B_QFULL = 0, B_KFULL = 1, B_VFULL = 3, B_KEMPTY = 5, B_VEMPTY = 7, B_SFULL = 9, B_PREADY = 11,
           B_OFULL = 12, B_DRAIN = 13 };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nbh = p.B * p.Hq;
    const int qt = p.q_tiles - 1 - (int)(blockIdx.x / nbh);     // long (late) row tiles first
    const int bh = blockIdx.x % nbh;
    const int b = bh / p.Hq, h = bh - b * p.Hq;
    const int kv_head = b * p.Hkv + h / p.G;
    const int q0 = qt * C::BM;
    const int kv_end = p.causal ? min(p.S, q0 + C::BM) : p.S;
    const int n_tiles = (kv_end + C::BN - 1) / C::BN;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(B_QFULL), 1);
        for (int s = 0; s < C::NST; ++s) {
            mbar_init(bar(B_KFULL + s), 1);
            mbar_init(bar(B_VFULL + s), 1);
            mbar_init(bar(B_KEMPTY + s), 1);
            mbar_init(bar(B_VEMPTY + s), 1);
            mbar_init(bar(B_SFULL + s), 1);
        }
        mbar_init(bar(B_PREADY), 128);
        mbar_init(bar(B_OFULL), 1);
        mbar_init(bar(B_DRAIN), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + C::OFF_TMEM), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + 128;

    if (warp >= 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 5 && lane == 0) {
            // -------------------------------------------------------- producer
            mbar_expect_tx(bar(B_QFULL), C::Q_BYTES);
            tma_load_tile4(base + C::OFF_Q, &tm_q, q0, bh, bar(B_QFULL));
            int issued = 0;
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                const uint32_t ph_prev = ((j / C::NST) - 1) & 1;
                if (j >= C::NST && !mbar_wait(bar(B_KEMPTY + s), ph_prev, abort_flag, status, ST_PREFILL_TIMEOUT)) break;
                mbar_expect_tx(bar(B_KFULL + s), C::KV_BYTES);
                tma_load_tile4(base + C::OFF_K + s * C::KV_BYTES, &tm_k, j * C::BN, kv_head, bar(B_KFULL + s));
                issued = 2 * j + 1;
                if (j >= C::NST && !mbar_wait(bar(B_VEMPTY + s), ph_prev, abort_flag, status, ST_PREFILL_TIMEOUT)) break;
                mbar_expect_tx(bar(B_VFULL + s), C::KV_BYTES);
                tma_load_tile4(base + C::OFF_V + s * C::KV_BYTES, &tm_v, j * C::BN, kv_head, bar(B_VFULL + s));
                issued = 2 * j + 2;
            }
            // every copy issued has landed before the CTA gives its shared memory back
            mbar_wait_drain(bar(B_QFULL), 0);
            const int k_issued = (issued + 1) / 2, v_issued = issued / 2;
            for (int j = max(0, k_issued - C::NST); j < k_issued; ++j)
                mbar_wait_drain(bar(B_KFULL + (j & 1)), (j / C::NST) & 1);
            for (int j = max(0, v_issued - C::NST); j < v_issued; ++j)
                mbar_wait_drain(bar(B_VFULL + (j & 1)), (j / C::NST) & 1);
        } else if (warp == 4 && lane == 0) {
            // -------------------------------------------------------- MMA issue
            constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
            constexpr uint32_t IDESC_S = umma_idesc(FMT, 0, 0, C::BM, C::BN);   // Q (K-major) x K^T (K-major)
            constexpr uint32_t IDESC_O = umma_idesc(FMT, 0, 1, C::BM, D);       // P (K-major) x V (MN-major)
            const uint32_t qa = base + C::OFF_Q;
            auto issue_scores = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(bar(B_KFULL + s), (j / C::NST) & 1, abort_flag, status, ST_PREFILL_TIMEOUT)) return false;
                tc_fence_after();
                const uint32_t ka = base + C::OFF_K + s * C::KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_f16(tmem + s * C::BN,
                             umma_desc_sw128(qa + (ks >> 2) * C::Q_PANEL + (ks & 3) * 32, 16, 1024),
                             umma_desc_sw128(ka + (ks >> 2) * C::KV_PANEL + (ks & 3) * 32, 16, 1024), IDESC_S, ks > 0);
                umma_commit(bar(B_KEMPTY + s));
                umma_commit(bar(B_SFULL + s));
                return true;
            };
            bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, status, ST_PREFILL_TIMEOUT);
            ok = ok && issue_scores(0);
            for (int j = 0; ok && j < n_tiles; ++j) {
                const int s = j & 1;
                // the next tile's scores go to the other S buffer while the softmax warps work on this one
                // (that buffer's last reader, tile j-1, signalled P ready before its P.V was issued)
                if (j + 1 < n_tiles && !(ok = issue_scores(j + 1))) break;
                if (!(ok = mbar_wait(bar(B_PREADY), j & 1, abort_flag, status, ST_PREFILL_TIMEOUT))) break;
                if (!(ok = mbar_wait(bar(B_VFULL + s), (j / C::NST) & 1, abort_flag, status, ST_PREFILL_TIMEOUT))) break;
                tc_fence_after();
                const uint32_t va = base + C::OFF_V + s * C::KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < C::BN / 16; ++ks)
                    umma_f16_ts(tmem_o, tmem + s * C::BN + ks * 8,
                                umma_desc_sw128(va + ks * 2048, C::KV_PANEL, 1024), IDESC_O, (j | ks) > 0);
                umma_commit(bar(B_VEMPTY + s));
                umma_commit(bar(B_OFULL));
            }
            // every MMA issued has completed before tensor memory is released
            umma_commit(bar(B_DRAIN));
            mbar_wait_drain(bar(B_DRAIN), 0);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ------------------------------------------------------------ softmax, rescale, store
        const int row = threadIdx.x;                        // 0..127 = tensor-memory lane
        const int r_glob = q0 + row;
        const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
        const float sl2 = p.scale * 1.4426950408889634f;
        const int lim = p.causal ? min(p.S - 1, r_glob) : p.S - 1;      // last live column of this row
        // The output row accumulates in tensor memory across tiles (P.V with accumulate), relative to a
        // reference maximum m_ref that is only raised when a tile's maximum exceeds it by more than 2^8:
        // probabilities then stay below 256 (exact in bf16/fp16 terms), the sum l uses the same reference,
        // and out = O / l does not depend on the reference. Raising it rescales O in tensor memory.
        float m_ref = 0.f, l_run = 0.f;
        // warp-uniform result: the tensor-memory loads and stores below are warp-wide instructions
        auto wait_all = [&](uint32_t b, uint32_t parity) {
            return __all_sync(0xffffffffu, mbar_wait(b, parity, abort_flag, status, ST_PREFILL_TIMEOUT)) != 0;
        };
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int k0 = j * C::BN;
            if (!(ok = wait_all(bar(B_SFULL + (j & 1)), (j / 2) & 1))) break;
            tc_fence_after();
            float x[64];
            tmem_ld64(tmem + lane_base + (j & 1) * C::BN, x);
            if ((k0 + C::BN > p.S) || (p.causal && k0 + C::BN - 1 > q0)) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (k0 + i > lim) x[i] = -INFINITY;
            }
            float mx8[8];                                   // eight independent chains, then a tree
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = x[i];
#pragma unroll
            for (int i = 8; i < 64; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], x[i]);
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                                   fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            bool o_free = j == 0;                           // P.V of the previous tile has completed
            if (j == 0) {
                m_ref = mx == -INFINITY ? 0.f : mx;
            } else if (__any_sync(0xffffffffu, (mx - m_ref) * sl2 > 8.0f)) {
                const float m_new = fmaxf(m_ref, mx);
                const float alpha = ex2((m_ref - m_new) * sl2);
                m_ref = m_new;
                l_run *= alpha;
                if (!(ok = wait_all(bar(B_OFULL), (j - 1) & 1))) break;
                tc_fence_after();
                o_free = true;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_base + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= alpha;
                    tmem_st32(tmem_o + lane_base + c * 32, o);
                }
            }
            const float neg_ms = -m_ref * sl2;
            uint32_t pk[32];
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const float a = ex2(fmaf(x[i], sl2, neg_ms)), bq = ex2(fmaf(x[i + 1], sl2, neg_ms));
                ps4[(i >> 1) & 3] += a + bq;
                pk[i >> 1] = pack2<T>(a, bq);
            }
            l_run += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
            // Keeps this thread in step with the P.V completions (a parity wait must never fall two
            // completions behind); tile j-1's P.V was issued a whole softmax ago, so this rarely waits.
            if (!o_free) {
                if (!(ok = wait_all(bar(B_OFULL), (j - 1) & 1))) break;
            }
            // P replaces the scores it came from: 64 probabilities = 32 packed columns of this lane, the
            // K-major A operand of the P.V MMA read straight from tensor memory.
            tmem_st32p(tmem + lane_base + (j & 1) * C::BN, pk);
            tc_fence_before();
            mbar_arrive(bar(B_PREADY));
        }
        if (ok) ok = wait_all(bar(B_OFULL), (n_tiles - 1) & 1);
        if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l_run;
            T* orow = static_cast<T*>(p.out) + ((size_t)bh * p.S + r_glob) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                float o[32];
                tmem_ld32(tmem_o + lane_base + c * 32, o);          // warp-wide: every lane takes part
                if (r_glob < p.S) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u;
                        u.x = pack2<T>(o[i] * inv, o[i + 1] * inv);
                        u.y = pack2<T>(o[i + 2] * inv, o[i + 3] * inv);
                        u.z = pack2<T>(o[i + 4] * inv, o[i + 5] * inv);
                        u.w = pack2<T>(o[i + 6] * inv, o[i + 7] * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + i) = u;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

}  // namespace ftk
