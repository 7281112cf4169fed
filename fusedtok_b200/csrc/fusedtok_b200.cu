// Host side of the C ABI declared in include/fusedtok_b200.h: argument
// validation with the reference's error contract, per-device workspace,
// TMA descriptor encoding, kernel selection and launch. Counterpart of the
// reference's launchers (src/attention.cu:1468-1585, 1791-1915), its staged
// bindings (src/bindings.cpp:2402-2436, 2507-2565) and cuda_available
// (src/fusedtok.cu:34-37).

#include "../../include/fusedtok_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "decode_simt.cuh"
#include "decode_tc.cuh"
#include "decode_ring.cuh"
#include "kv_append.cuh"
#include "prefill_simt.cuh"
#include "prefill_tc.cuh"
#include "rope.cuh"
#include "rope_append.cuh"
#include "merge.cuh"

namespace {

using namespace ftk;

thread_local std::string g_err;
thread_local long long g_launches = 0;

int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}
int cuda_fail(const char* what, cudaError_t e) {
    return fail(FUSEDTOK_RUNTIME_ERROR, std::string(what) + ": " + cudaGetErrorString(e));
}
// launch failures surface as runtime errors (reference: check_launch, src/cuda_util.cuh:21-25)
int check_launch(const char* what) {
    ++g_launches;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(what, e);
    return FUSEDTOK_OK;
}
// reference: stream_is_capturing, src/cuda_util.cuh:259-264
bool stream_is_capturing(cudaStream_t s) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) cudaGetLastError();
    return st == cudaStreamCaptureStatusActive;
}

enum DType { F32 = 0, BF16 = 1, F16 = 2 };
inline size_t dtype_size(int dt) { return dt == F32 ? 4 : 2; }

// ---- per-device state --------------------------------------------------------
constexpr int kMaxDevices = 64;
constexpr size_t kArenaMin = 32u << 20;      // first allocation: covers common shapes

struct DeviceState {
    bool init = false;
    int sm_count = 0;
    char* arena = nullptr;                   // current arena (older ones stay alive: graphs may hold them)
    size_t arena_bytes = 0;
    int* status = nullptr;                   // separate small allocation, never moves
    int* counters = nullptr;                 // per-unit arrival counters, zero between launches
    size_t counters_cap = 0;                 // in units
    bool smem_attr_set = false;
    bool prefill_attr_set = false;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode_fn() {
    if (g_encode) return FUSEDTOK_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess)
        return fail(FUSEDTOK_RUNTIME_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return FUSEDTOK_OK;
}

template <typename K> int set_smem(K kernel, int bytes) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
    return FUSEDTOK_OK;
}

int set_all_smem_attrs() {
    int rc = 0;
#define FTK_SET(T, D, GP, PG) \
    if ((rc = set_smem(decode_tc_kernel<T, D, GP, PG>, TcCfg<D>::SMEM_BYTES))) return rc;
#define FTK_SET_ALL(T)                                                                          \
    FTK_SET(T, 64, 8, false) FTK_SET(T, 64, 16, false) FTK_SET(T, 64, 8, true) FTK_SET(T, 64, 16, true) \
    FTK_SET(T, 128, 8, false) FTK_SET(T, 128, 16, false) FTK_SET(T, 128, 8, true) FTK_SET(T, 128, 16, true) \
    FTK_SET(T, 192, 8, false) FTK_SET(T, 192, 8, true) FTK_SET(T, 256, 8, false) FTK_SET(T, 256, 8, true) \
    FTK_SET(T, 32, 8, false) FTK_SET(T, 32, 8, true) FTK_SET(T, 80, 8, false) FTK_SET(T, 80, 8, true)       \
    FTK_SET(T, 96, 8, false) FTK_SET(T, 96, 8, true) FTK_SET(T, 112, 8, false) FTK_SET(T, 112, 8, true)     \
    FTK_SET(T, 160, 8, false) FTK_SET(T, 160, 8, true)
    FTK_SET_ALL(__nv_bfloat16)
    FTK_SET_ALL(__half)
#undef FTK_SET_ALL
#undef FTK_SET
#define FTK_SET_SIMT1(T, GC, LC)                                                                      \
    if ((rc = set_smem(decode_simt_kernel<T, GC, LC, false>, SIMT_STAGE_BYTES))) return rc;           \
    if ((rc = set_smem(decode_simt_kernel<T, GC, LC, true>, SIMT_STAGE_BYTES))) return rc;
#define FTK_SET_SIMT(T)                                                                               \
    FTK_SET_SIMT1(T, 1, 1) FTK_SET_SIMT1(T, 4, 1) FTK_SET_SIMT1(T, 8, 1) FTK_SET_SIMT1(T, 1, 2)       \
    FTK_SET_SIMT1(T, 4, 2) FTK_SET_SIMT1(T, 1, 4) FTK_SET_SIMT1(T, 2, 4)
    FTK_SET_SIMT(float)
    FTK_SET_SIMT(__nv_bfloat16)
    FTK_SET_SIMT(__half)
#undef FTK_SET_SIMT1
#define FTK_SET_RING(D, GC)                                                                                  \
    if ((rc = set_smem(decode_ring_f32_kernel<D, GC, false>, RfCfg<D, GC>::SMEM_BYTES))) return rc;          \
    if ((rc = set_smem(decode_ring_f32_kernel<D, GC, true>, RfCfg<D, GC>::SMEM_BYTES))) return rc;
    FTK_SET_RING(64, 1) FTK_SET_RING(64, 4) FTK_SET_RING(64, 8)
    FTK_SET_RING(128, 1) FTK_SET_RING(128, 4) FTK_SET_RING(128, 8)
#undef FTK_SET_RING
#undef FTK_SET_SIMT
    return rc;
}

int set_prefill_smem_attrs() {
    int rc = 0;
#define FTK_SET_PF(T)                                                                                       \
    if ((rc = set_smem(prefill_simt_kernel<T, 64, 64>, prefill_simt_smem_floats<64, 64>(128) * 4))) return rc; \
    if ((rc = set_smem(prefill_simt_kernel<T, 32, 32>, prefill_simt_smem_floats<32, 32>(256) * 4))) return rc; \
    if ((rc = set_smem(prefill_simt_kernel<T, 16, 16>, prefill_simt_smem_floats<16, 16>(512) * 4))) return rc;
    FTK_SET_PF(float)
    FTK_SET_PF(__nv_bfloat16)
    FTK_SET_PF(__half)
#undef FTK_SET_PF
    if ((rc = set_smem(prefill_tc_kernel<__nv_bfloat16, 64>, PfCfg<64>::SMEM_BYTES))) return rc;
    if ((rc = set_smem(prefill_tc_kernel<__nv_bfloat16, 128>, PfCfg<128>::SMEM_BYTES))) return rc;
    if ((rc = set_smem(prefill_tc_kernel<__half, 64>, PfCfg<64>::SMEM_BYTES))) return rc;
    if ((rc = set_smem(prefill_tc_kernel<__half, 128>, PfCfg<128>::SMEM_BYTES))) return rc;
    if ((rc = set_smem(prefill_tc_kernel<__nv_bfloat16, 256>, PfCfg<256>::SMEM_BYTES))) return rc;
    if ((rc = set_smem(prefill_tc_kernel<__half, 256>, PfCfg<256>::SMEM_BYTES))) return rc;
    return rc;
}

int device_state(DeviceState** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
    if (dev < 0 || dev >= kMaxDevices) return fail(FUSEDTOK_RUNTIME_ERROR, "device index out of range");
    DeviceState& d = g_dev[dev];
    if (!d.init) {
        e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail("cudaDeviceGetAttribute", e);
        d.init = true;
    }
    *out = &d;
    return FUSEDTOK_OK;
}

struct Arena {
    int* status;
    int* counters;
    float* ws_ml;
    float* ws_acc;
};
constexpr size_t kCountersMin = 1u << 16;    // units covered by the first counters allocation

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Workspace of `ml_b + acc_b` bytes of partial slots and `words` counter words. Grow-only;
// allocation is refused while the stream is being captured.
int get_arena(DeviceState& d, cudaStream_t cs, size_t words, size_t ml_b, size_t acc_b, bool need_smem_attr,
              Arena* a) {
    const size_t need = ml_b + acc_b;
    const size_t units = words;
    std::lock_guard<std::mutex> lock(g_mutex);
    const bool first = d.status == nullptr || (need_smem_attr && !d.smem_attr_set);
    if (first || need > d.arena_bytes || units > d.counters_cap) {
        if (stream_is_capturing(cs))
            return fail(FUSEDTOK_RUNTIME_ERROR,
                        "decode attention workspace must be allocated outside a CUDA graph capture - "
                        "warm the shape up once before capturing");
        if (!d.status) {
            cudaError_t e = cudaMalloc(&d.status, 256);
            if (e != cudaSuccess) return cuda_fail("status word allocation failed", e);
            e = cudaMemset(d.status, 0, 256);
            if (e != cudaSuccess) return cuda_fail("status word clear failed", e);
        }
        if (need_smem_attr && !d.smem_attr_set) {
            const int rc = set_all_smem_attrs();
            if (rc) return rc;
            d.smem_attr_set = true;
        }
        if (units > d.counters_cap) {
            // counters live apart from the slots: slot regions of different shapes overlap, counters
            // must stay zero between launches whatever shape ran last
            const size_t cap = std::max(units, kCountersMin);
            int* mem = nullptr;
            cudaError_t e = cudaMalloc(&mem, cap * sizeof(int));
            if (e != cudaSuccess) {
                cudaGetLastError();
                return fail(FUSEDTOK_RUNTIME_ERROR, "decode attention workspace allocation failed");
            }
            if ((e = cudaMemset(mem, 0, cap * sizeof(int))) != cudaSuccess) return cuda_fail("counter clear failed", e);
            d.counters = mem;       // the previous block is kept alive for graphs captured earlier
            d.counters_cap = cap;
        }
        if (need > d.arena_bytes) {
            const size_t bytes = std::max(need, kArenaMin);
            char* mem = nullptr;
            const cudaError_t e = cudaMalloc(&mem, bytes);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return fail(FUSEDTOK_RUNTIME_ERROR, "decode attention workspace allocation failed");
            }
            d.arena = mem;          // the previous arena is deliberately kept: captured graphs may point into it
            d.arena_bytes = bytes;
        }
    }
    a->status = d.status;
    a->counters = d.counters;
    a->ws_ml = reinterpret_cast<float*>(d.arena);
    a->ws_acc = reinterpret_cast<float*>(d.arena + ml_b);
    return FUSEDTOK_OK;
}

// True if get_arena would hand these sizes out without allocating anything.
bool arena_covers(DeviceState& d, size_t words, size_t ml_b, size_t acc_b) {
    std::lock_guard<std::mutex> lock(g_mutex);
    return d.status != nullptr && d.smem_attr_set && ml_b + acc_b <= d.arena_bytes && words <= d.counters_cap;
}

// reference: attention_check, src/attention.cu:184-193
int attention_check(int batch, int hq, int hkv, long long t_seq, int dim) {
    if (batch < 0 || hq < 1 || hkv < 1 || t_seq < 0 || dim < 1)
        return fail(FUSEDTOK_INVALID_ARGUMENT,
                    "attention shapes must satisfy batch>=0, heads>=1, rows>=0, dim>=1");
    if (hq % hkv != 0)
        return fail(FUSEDTOK_INVALID_ARGUMENT,
                    "q heads must be a multiple of kv heads (contiguous GQA groups)");
    if (dim % 4 != 0 || dim > 512)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be a multiple of 4 and at most 512");
    return FUSEDTOK_OK;
}

// The cache as a rank-3 tensor: (64 elements, rows with a stride of one cache row, D/64 column blocks of
// 128 bytes). A box [64, box_rows, D/64] is one copy and lands as [column block][row][128 B].
int encode_map(CUtensorMap* map, int dt, const void* base, unsigned long long rows, int dim, int box_rows) {
    // A descriptor is a pure function of these five values, and a decode loop asks for the same two every
    // step: keep the last few per thread and skip the driver call.
    struct Entry {
        const void* base = nullptr;
        unsigned long long rows = 0;
        int dt = -1, dim = 0, box_rows = 0;
        CUtensorMap map;
    };
    constexpr int kSlots = 8;
    thread_local Entry cache[kSlots];
    Entry& e = cache[(reinterpret_cast<uintptr_t>(base) >> 8) % kSlots];
    if (e.base == base && e.rows == rows && e.dt == dt && e.dim == dim && e.box_rows == box_rows) {
        *map = e.map;
        return FUSEDTOK_OK;
    }
    const CUtensorMapDataType dtype = dt == BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r;
    if (dim % 64 == 0) {
        const cuuint64_t gdim[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(dim / 64)};
        const cuuint64_t gstride[2] = {(cuuint64_t)dim * 2, 128u};
        const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)(dim / 64)};
        r = g_encode(map, dtype, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        // rank 2: (D elements, rows); a box is one 64-element column block of box_rows rows, the part of the
        // last block past D comes back as zeros
        const cuuint64_t gdim[2] = {(cuuint64_t)dim, (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)dim * 2};
        const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
        r = g_encode(map, dtype, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS)
        return fail(FUSEDTOK_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (code " + std::to_string((int)r) + ")");
    e.base = base; e.rows = rows; e.dt = dt; e.dim = dim; e.box_rows = box_rows;
    e.map = *map;
    return FUSEDTOK_OK;
}

// The float32 cache as a rank-2 tensor (D floats, rows), no swizzle: a box [D, box_rows] lands row-major.
int encode_map_f32(CUtensorMap* map, const void* base, unsigned long long rows, int dim, int box_rows) {
    const cuuint64_t gdim[2] = {(cuuint64_t)dim, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)dim * 4};
    const cuuint32_t box[2] = {(cuuint32_t)dim, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(FUSEDTOK_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (code " + std::to_string((int)r) + ")");
    return FUSEDTOK_OK;
}

template <int D, int GC, bool PG>
void launch_ring(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, cudaStream_t cs) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.ncta);
    cfg.blockDim = dim3(RF_THREADS);
    cfg.dynamicSmemBytes = RfCfg<D, GC>::SMEM_BYTES;
    cfg.stream = cs;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, decode_ring_f32_kernel<D, GC, PG>, mk, mv, p);
}
void launch_ring_any(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, bool paged, cudaStream_t cs) {
#define FTK_GO(D, GC)                                          \
    do {                                                       \
        if (paged) launch_ring<D, GC, true>(mk, mv, p, cs);    \
        else launch_ring<D, GC, false>(mk, mv, p, cs);         \
    } while (0)
    if (p.D == 64) { if (p.GC == 1) FTK_GO(64, 1); else if (p.GC == 4) FTK_GO(64, 4); else FTK_GO(64, 8); }
    else { if (p.GC == 1) FTK_GO(128, 1); else if (p.GC == 4) FTK_GO(128, 4); else FTK_GO(128, 8); }
#undef FTK_GO
}

template <typename T, int D, int GP, bool PG>
void launch_tc(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, cudaStream_t cs) {
    // launched with programmatic stream serialization: the kernel's prologue may overlap the tail
    // of the previous kernel in the stream (it waits with griddepcontrol.wait before touching memory)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.ncta);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = TcCfg<D>::SMEM_BYTES;
    cfg.stream = cs;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, decode_tc_kernel<T, D, GP, PG>, mk, mv, p);
}
template <typename T>
void launch_tc_t(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, int gp, bool paged,
                 cudaStream_t cs) {
#define FTK_GO(D, GP)                                              \
    do {                                                           \
        if (paged) launch_tc<T, D, GP, true>(mk, mv, p, cs);       \
        else launch_tc<T, D, GP, false>(mk, mv, p, cs);            \
    } while (0)
    if (p.D == 64) { if (gp == 8) FTK_GO(64, 8); else FTK_GO(64, 16); }
    else if (p.D == 128) { if (gp == 8) FTK_GO(128, 8); else FTK_GO(128, 16); }
    else if (p.D == 192) FTK_GO(192, 8);
    else if (p.D == 256) FTK_GO(256, 8);
    else if (p.D == 32) FTK_GO(32, 8);
    else if (p.D == 80) FTK_GO(80, 8);
    else if (p.D == 96) FTK_GO(96, 8);
    else if (p.D == 112) FTK_GO(112, 8);
    else FTK_GO(160, 8);
#undef FTK_GO
}

template <typename T> void launch_simt_t(const DecodeParams& p, int lc, cudaStream_t cs) {
    // programmatic stream serialization, as for the tensor-core kernel
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.ncta);
    cfg.blockDim = dim3(SIMT_THREADS);
    cfg.dynamicSmemBytes = SIMT_STAGE_BYTES;
    cfg.stream = cs;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define FTK_GO(GC, LC)                                                                 \
    do {                                                                               \
        if (p.n_peers) cudaLaunchKernelEx(&cfg, decode_simt_kernel<T, GC, LC, true>, p); \
        else cudaLaunchKernelEx(&cfg, decode_simt_kernel<T, GC, LC, false>, p);        \
    } while (0)
    if (lc == 1) { if (p.GC == 1) FTK_GO(1, 1); else if (p.GC == 4) FTK_GO(4, 1); else FTK_GO(8, 1); }
    else if (lc == 2) { if (p.GC == 1) FTK_GO(1, 2); else FTK_GO(4, 2); }
    else { if (p.GC == 1) FTK_GO(1, 4); else FTK_GO(2, 4); }
#undef FTK_GO
}

// ---- launch plan ---------------------------------------------------------------
// Everything about a decode launch that follows from the shapes, the operand alignment and the SM
// count: which kernel, how the GQA group is chunked, the grid, how the tile sequence is cut into
// ranges, and the layout of the split-KV scratch. Both the allocating launchers and the
// allocation-free one launch from the same plan, so they run the same kernel on the same split.
// Blocks in the paged pool of the launches that follow, when a test has said so (fusedtok_debug_set_pool_blocks);
// 0 = unknown. Only the self-checking build looks at what is derived from it.
std::atomic<long long> g_debug_pool_blocks{0};

struct DecodePlan {
    bool use_tc = false, use_ring = false, paged = false;
    bool unit_split = false;   // generic kernel, one CTA per unit, no workspace (first call inside a capture)
    int GC = 1, NCH = 1, lc = 1, gp = 8;
    int ncta = 1;
    int box_rows = TILE, box_shift = 6;
    int dyn_chunk = 0, dyn_tail_max = 0;          // static + dynamic-tail ranges (0: equal split)
    int sched_table = 0;                           // per-sequence tile prefix sums fit the kernel's table
    unsigned long long units = 0, map_rows = 0;
    size_t words = 0;                              // counter words: one per unit + the tail-range counter
    size_t slots = 0, ml_b = 0, acc_b = 0;         // partial slots and their two regions
};

// The fixed scratch of the allocation-free launcher: [256 B header | counters | (m, l) slots | acc slots].
constexpr size_t kNoAllocBytes = 4u << 20;          // the stated maximum: 4 MiB of scratch
constexpr size_t kNoAllocUnits = 16384;             // counter words it holds (64 KiB)
// Finer tail ranges mean more partial slots. The plan only refines while the slots stay inside what
// the fixed scratch can hold, so that every launcher runs a shape on the same split.
constexpr size_t kSlotBudgetBytes = kNoAllocBytes - 256 - kNoAllocUnits * sizeof(int) - 512;
constexpr int kDynTailMax = 32;                     // most tiles per CTA handed out dynamically

// The static + dynamic plan is off unless FUSEDTOK_DYN_CHUNK (tiles per dynamic range) is set in the
// environment: measured on B200 it evens out the finish times of the CTAs but every additional range end
// stalls a CTA's consumers for about 2 us, during which its ring of copies drains, and that costs more
// than the balance gains (configuration 2: 79 us equal split, 88-98 us with 1-4 dynamic ranges per CTA).
// FUSEDTOK_DYN_TAIL overrides the number of tiles per CTA that are handed out dynamically.
const int g_env_dyn_chunk = [] {
    const char* e = std::getenv("FUSEDTOK_DYN_CHUNK");
    return e ? std::atoi(e) : -1;
}();
// FUSEDTOK_COST_SPLIT=0 cuts the ranges at equal tile counts instead of equal cost (for A/B measurements).
const bool g_env_cost_split = [] {
    const char* e = std::getenv("FUSEDTOK_COST_SPLIT");
    return !(e && e[0] == '0');
}();
// FUSEDTOK_COST_A / FUSEDTOK_COST_B: cost of a tile and of a unit end under the cost-weighted split (1 and 1).
const int g_env_cost_a = [] {
    const char* e = std::getenv("FUSEDTOK_COST_A");
    return e ? std::max(1, std::atoi(e)) : 1;
}();
const int g_env_cost_b = [] {
    const char* e = std::getenv("FUSEDTOK_COST_B");
    return e ? std::max(0, std::atoi(e)) : 1;
}();
// FUSEDTOK_F32_RING=0 keeps float32 caches on the generic CUDA-core kernel (for A/B measurements).
const bool g_env_f32_ring = [] {
    const char* e = std::getenv("FUSEDTOK_F32_RING");
    return !(e && e[0] == '0');
}();
const int g_env_dyn_tail = [] {
    const char* e = std::getenv("FUSEDTOK_DYN_TAIL");
    return e ? std::atoi(e) : -1;
}();

inline bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
// head dims the tensor-core decode kernel is instantiated for
inline bool tc_head_dim(int d) {
    return d == 32 || d == 64 || d == 80 || d == 96 || d == 112 || d == 128 || d == 160 || d == 192 || d == 256;
}

DecodePlan plan_decode(int dt, const void* q, const void* k, const void* v, bool paged, bool has_lens, int batch,
                       int hq, int hkv, int rows, int page, int dim, int sm_count, bool peers = false,
                       bool unit_split = false) {
    DecodePlan pl;
    const int G = hq / hkv;
    pl.paged = paged;
    pl.unit_split = unit_split;
    pl.map_rows = paged ? 0ull : (unsigned long long)batch * hkv * (unsigned long long)rows;
    pl.use_tc = !unit_split && dt != F32 && tc_head_dim(dim) &&
                ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0 &&
                ((reinterpret_cast<uintptr_t>(q)) & 3u) == 0;
    if (pl.use_tc && !paged && pl.map_rows >= (1ull << 31)) pl.use_tc = false;
    if (pl.use_tc && paged && !(is_pow2(page) && page >= 8)) pl.use_tc = false;
    // float32: the TMA-fed CUDA-core kernel for the common head dims (the KV-length split with peer exchange and
    // every other shape stay on the generic kernel)
    // (launches of at most two tiles per SM are all latency: the generic kernel's two small CTAs per SM start faster)
    const unsigned long long rough_tiles = (unsigned long long)batch * hkv * (unsigned long long)((rows + TILE - 1) / TILE);
    pl.use_ring = !unit_split && dt == F32 && g_env_f32_ring && !peers && (dim == 64 || dim == 128) &&
                  rough_tiles > 2ull * (unsigned long long)sm_count &&
                  ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(q)) & 15u) == 0 &&
                  (paged ? (is_pow2(page) && page >= 8) : pl.map_rows < (1ull << 31));
    if (pl.use_ring) {
        pl.GC = G == 1 ? 1 : (G <= 4 ? 4 : 8);
        pl.box_rows = paged ? std::min(page, RF_ROWS) : RF_ROWS;
        pl.box_shift = 0;
        while ((1 << pl.box_shift) < pl.box_rows) ++pl.box_shift;
    } else if (pl.use_tc) {
        pl.GC = std::min(G, (dim == 64 || dim == 128) ? 16 : 8);   // only these two have the 16-head MMA tile
        pl.gp = pl.GC <= 8 ? 8 : 16;
        pl.box_rows = paged ? std::min(page, TILE) : TILE;
        pl.box_shift = 0;
        while ((1 << pl.box_shift) < pl.box_rows) ++pl.box_shift;
    } else {
        pl.lc = dim <= 128 ? 1 : (dim <= 256 ? 2 : 4);
        if (G == 1) pl.GC = 1;
        else if (pl.lc == 1) pl.GC = G <= 4 ? 4 : 8;
        else if (pl.lc == 2) pl.GC = 4;
        else pl.GC = 2;
    }
    pl.NCH = (G + pl.GC - 1) / pl.GC;
    pl.units = (unsigned long long)batch * hkv * pl.NCH;
    const unsigned long long tiles_per_seq = (unsigned long long)((rows + TILE - 1) / TILE);
    const unsigned long long max_tiles = pl.units * tiles_per_seq;
    pl.ncta = (int)std::min<unsigned long long>((unsigned long long)sm_count * ((pl.use_tc || pl.use_ring) ? 1 : 2),
                                                max_tiles);
    if (pl.ncta < 1) pl.ncta = 1;
    if (unit_split) pl.ncta = (int)std::min<unsigned long long>(pl.units, 0x7fffffffull);   // (the caller checks the bound)
    pl.words = (size_t)pl.units + 1;

    const size_t slot_bytes = (size_t)pl.GC * (dim + 2) * sizeof(float);
    size_t ranges = (size_t)pl.ncta;
    if (pl.use_ring)
        pl.sched_table = has_lens && batch <= SCHED_MAX_B && (unsigned long long)batch * tiles_per_seq < (1ull << 31);
    if (pl.use_tc) {
        pl.sched_table = has_lens && batch <= SCHED_MAX_B && (unsigned long long)batch * tiles_per_seq < (1ull << 31);
        const unsigned long long per_max = max_tiles / (unsigned long long)pl.ncta;
        if (g_env_dyn_chunk > 0 && (!has_lens || pl.sched_table) && per_max >= (unsigned long long)DYN_MIN_PER &&
            per_max < (1ull << 30)) {
            int tail = (int)std::min<unsigned long long>(per_max / 6, (unsigned long long)kDynTailMax);
            if (g_env_dyn_tail > 0) tail = g_env_dyn_tail;
            const size_t base = (size_t)pl.units + (size_t)pl.ncta;
            for (int chunk = 2; chunk <= 16 && !pl.dyn_chunk; chunk *= 2) {
                if (g_env_dyn_chunk >= 0) chunk = g_env_dyn_chunk;
                if (chunk <= 0 || tail < chunk) break;
                const size_t tail_ranges = (size_t)pl.ncta * (tail / chunk) + (size_t)pl.ncta / chunk + 2;
                if (g_env_dyn_chunk > 0 || (base + tail_ranges) * slot_bytes <= kSlotBudgetBytes) {
                    pl.dyn_chunk = chunk;
                    pl.dyn_tail_max = tail;
                    ranges = (size_t)pl.ncta + tail_ranges;
                }
                if (g_env_dyn_chunk >= 0) break;
            }
        }
    }
    pl.slots = (size_t)pl.units + ranges;
    pl.ml_b = align_up(pl.slots * pl.GC * 2 * sizeof(float), 256);
    pl.acc_b = align_up(pl.slots * pl.GC * (size_t)dim * sizeof(float), 256);
    return pl;
}

// Split-KV scratch of one launch, wherever it lives.
struct Scratch {
    int* status;
    int* counters;
    float* ws_ml;
    float* ws_acc;
};

struct PeerDest {                    // direct peer exchange of the raw triples (KV-length split)
    void* const* bases;              // host array: every rank's exchange buffer, own included
    int n, rank;
};

// Operands must be aligned to 4 elements (the kernels read and write 4 elements, or 16 bytes, at a time);
// views that start at an odd element offset are refused here rather than faulting on the device.
int check_aligned4(int dt, std::initializer_list<const void*> ptrs) {
    uintptr_t all = 0;
    for (const void* ptr : ptrs) all |= reinterpret_cast<uintptr_t>(ptr);
    if (all & (4 * dtype_size(dt) - 1))
        return fail(FUSEDTOK_INVALID_ARGUMENT, "attention operands must be aligned to 4 elements");
    return FUSEDTOK_OK;
}

// Fill the kernel parameters from the plan and launch. table == nullptr: contiguous cache with `rows`
// cache rows per (b, kv); otherwise paged pools with `page` rows per block and `tbl_width` entries per
// sequence. partial != nullptr (or peers): emit raw triples instead of the normalised output.
int decode_launch(const DecodePlan& pl, const Scratch& sc, int dt, const void* q, const void* k, const void* v,
                  const int* table, const int* lens, void* out, float* partial, int batch, int hq, int hkv, int rows,
                  int page, int tbl_width, int dim, cudaStream_t cs, const PeerDest* peers) {
    const long long out_rows = (long long)batch * hq;
    DecodeParams p;
    memset(&p, 0, sizeof(p));
    p.q = q; p.k = k; p.v = v; p.out = out; p.lens = lens; p.table = table;
    p.triple_ml = partial;
    p.triple_acc_off = triple_acc_offset(out_rows);
    if (peers) {
        p.n_peers = peers->n;
        p.peer_rank = peers->rank;
        p.triple_acc_off = xchg_acc_off(out_rows);
        p.peer_nf = (long long)xchg_block_floats(out_rows, dim);
        for (int j = 0; j < peers->n; ++j) {
            p.peer_hdr[j] = static_cast<unsigned int*>(peers->bases[j]);
            p.peer_blocks[j] = reinterpret_cast<float*>(static_cast<unsigned char*>(peers->bases[j]) + XCHG_DATA_BYTES);
        }
        p.peer_epoch = p.peer_hdr[peers->rank];
        p.triple_ml = p.peer_blocks[peers->rank];     // non-null: "emit raw triples"
    }
    p.B = batch; p.Hq = hq; p.Hkv = hkv; p.G = hq / hkv; p.T = rows; p.D = dim;
    p.page = page; p.tbl_width = tbl_width;
    p.scale = 1.0f / sqrtf((float)dim);
    p.GC = pl.GC; p.NCH = pl.NCH; p.ncta = pl.ncta;
    p.box_rows = pl.box_rows; p.box_shift = pl.box_shift;
    p.dyn_chunk = pl.dyn_chunk; p.dyn_tail_max = pl.dyn_tail_max; p.sched_table = pl.sched_table;
    p.cost_split = (g_env_cost_split && (pl.use_tc || pl.use_ring) && !pl.dyn_chunk) ? 1 : 0;
    p.cost_a = g_env_cost_a;
    p.cost_b = g_env_cost_b;
    p.unit_split = pl.unit_split ? 1 : 0;
    // what this launch owns (read by the self-checking build only)
    p.bound_rows = pl.paged ? (unsigned long long)g_debug_pool_blocks * (unsigned long long)hkv * (unsigned long long)page
                            : pl.map_rows;
    p.bound_slots = sc.ws_ml ? (unsigned int)std::min<size_t>(pl.slots, 0xffffffffu) : 0u;
    p.bound_words = sc.counters ? (unsigned int)std::min<size_t>(pl.words, 0xffffffffu) : 0u;
    p.ws_ml = sc.ws_ml; p.ws_acc = sc.ws_acc; p.counters = sc.counters; p.status = sc.status;

    if (pl.use_ring) {
        int rc = get_encode_fn();
        if (rc) return rc;
        CUtensorMap mk, mv;
        const unsigned long long trows = pl.paged ? (1ull << 31) - 1 : pl.map_rows;
        if ((rc = encode_map_f32(&mk, k, trows, dim, pl.box_rows))) return rc;
        if ((rc = encode_map_f32(&mv, v, trows, dim, pl.box_rows))) return rc;
        launch_ring_any(mk, mv, p, pl.paged, cs);
        return check_launch("attention split-KV float32 ring kernel launch");
    }
    if (pl.use_tc) {
        int rc = get_encode_fn();
        if (rc) return rc;
        CUtensorMap mk, mv;
        // paged: pool rows are not known here (table values are trusted): describe the largest range
        // the int32 TMA coordinate can address; the hardware zero-fills nothing it is not asked for
        const unsigned long long trows = pl.paged ? (1ull << 31) - 1 : pl.map_rows;
        if ((rc = encode_map(&mk, dt, k, trows, dim, pl.box_rows))) return rc;
        if ((rc = encode_map(&mv, dt, v, trows, dim, pl.box_rows))) return rc;
        if (dt == BF16) launch_tc_t<__nv_bfloat16>(mk, mv, p, pl.gp, pl.paged, cs);
        else launch_tc_t<__half>(mk, mv, p, pl.gp, pl.paged, cs);
        return check_launch("attention split-KV tensor-core kernel launch");
    }
    if (dt == F32) launch_simt_t<float>(p, pl.lc, cs);
    else if (dt == BF16) launch_simt_t<__nv_bfloat16>(p, pl.lc, cs);
    else launch_simt_t<__half>(p, pl.lc, cs);
    return check_launch("attention split-KV kernel launch");
}

// The launcher behind every allocating zero-copy entry point.
int decode_common(int dt, const void* q, const void* k, const void* v, const int* table, const int* lens,
                  void* out, float* partial, int batch, int hq, int hkv, int rows, int page, int tbl_width,
                  int dim, uintptr_t stream, const PeerDest* peers = nullptr) {
    cudaStream_t cs = (cudaStream_t)stream;
    if (batch == 0) return FUSEDTOK_OK;                       // nothing to compute (src/attention.cu:1474)
    const long long out_rows = (long long)batch * hq;

    if (rows == 0 && peers)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "the peer exchange needs at least one cache row per rank");
    if (rows == 0) {
        // empty cache: zero rows (src/attention.cu:211-216) or empty triples
        if (partial) {
            const long long n = out_rows * dim;
            fill_empty_triple_kernel<<<(unsigned)((n + 255) / 256), 256, 0, cs>>>(
                partial, partial + triple_acc_offset(out_rows), out_rows, dim);
            return check_launch("attention empty-triple kernel launch");
        }
        const cudaError_t e = cudaMemsetAsync(out, 0, (size_t)out_rows * dim * dtype_size(dt), cs);
        if (e != cudaSuccess) return cuda_fail("attention zero fill failed", e);
        return FUSEDTOK_OK;
    }
    int rc = check_aligned4(dt, {q, k, v, out});
    if (rc) return rc;

    DeviceState* dev = nullptr;
    if ((rc = device_state(&dev))) return rc;
    const DecodePlan pl = plan_decode(dt, q, k, v, table != nullptr, lens != nullptr, batch, hq, hkv, rows, page, dim,
                                      dev->sm_count, peers != nullptr);
    if (!peers && !partial && !arena_covers(*dev, pl.words, pl.ml_b, pl.acc_b) && stream_is_capturing(cs)) {
        // The workspace this launch wants does not exist yet and a capture is no place to allocate it. Like
        // the reference, which then uses its workspace-free single kernel for this launch and for the whole
        // captured graph (src/attention.cu:1498-1509), degrade to a launch that needs none: the generic kernel,
        // one CTA per unit, every unit whole. Later calls outside a capture set the workspace up as usual.
        const DecodePlan up = plan_decode(dt, q, k, v, table != nullptr, lens != nullptr, batch, hq, hkv, rows, page,
                                          dim, dev->sm_count, false, true);
        if (up.units > 0x7fffffffull)
            return fail(FUSEDTOK_RUNTIME_ERROR,
                        "decode attention workspace must be allocated outside a CUDA graph capture - "
                        "warm the shape up once before capturing");
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            if (!dev->smem_attr_set) {
                if ((rc = set_all_smem_attrs())) return rc;      // not a stream operation: legal while capturing
                dev->smem_attr_set = true;
            }
        }
        const Scratch none{nullptr, nullptr, nullptr, nullptr};
        return decode_launch(up, none, dt, q, k, v, table, lens, out, partial, batch, hq, hkv, rows, page, tbl_width,
                             dim, cs, nullptr);
    }
    Arena a;
    if ((rc = get_arena(*dev, cs, pl.words, pl.ml_b, pl.acc_b, true, &a))) return rc;
    const Scratch sc{a.status, a.counters, a.ws_ml, a.ws_acc};
    return decode_launch(pl, sc, dt, q, k, v, table, lens, out, partial, batch, hq, hkv, rows, page, tbl_width, dim,
                         cs, peers);
}

int decode_contig(int dt, const void* q, const void* k, const void* v, const int* lens, void* out,
                  float* partial, int batch, int hq, int hkv, int t_seq, int dim, uintptr_t stream) {
    const int rc = attention_check(batch, hq, hkv, t_seq, dim);
    if (rc) return rc;
    return decode_common(dt, q, k, v, nullptr, lens, out, partial, batch, hq, hkv, t_seq, 0, 0, dim, stream);
}

// reference: attention_decode_paged_launch_t, src/attention.cu:1791-1815
int decode_paged(int dt, const void* q, const void* kp, const void* vp, const int* table, const int* lens,
                 void* out, int batch, int hq, int hkv, int page, int tbl_width, int dim, uintptr_t stream) {
    const long long span = (long long)tbl_width * page;
    if (span > (1LL << 30)) return fail(FUSEDTOK_INVALID_ARGUMENT, "table capacity too large");
    const int rc = attention_check(batch, hq, hkv, span, dim);
    if (rc) return rc;
    if (page < 1) return fail(FUSEDTOK_INVALID_ARGUMENT, "page size must be >= 1");
    if (tbl_width < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "table width must be >= 0");
    return decode_common(dt, q, kp, vp, table, lens, out, nullptr, batch, hq, hkv, (int)span, page, tbl_width,
                         dim, stream);
}

// Launch configuration with programmatic stream serialization allowed (the kernel starts with
// griddepcontrol.wait, so it touches memory only after the kernel before it has completed).
struct PdlLaunch {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    PdlLaunch(dim3 grid, dim3 block, size_t smem, cudaStream_t cs) : cfg{} {
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = cs;
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
};

// reference: kv_append_launch_t / kv_append_paged_launch_t, src/attention.cu:1924-1941, 1989-2005
int kv_append_common(int dt, const void* k_new, const void* v_new, const int* table, const int* lens,
                     void* k_dst, void* v_dst, int batch, int hkv, int dim, int rows, int tbl_width,
                     uintptr_t stream) {
    if (batch <= 0) return FUSEDTOK_OK;                       // nothing to append
    if (dim % 4 != 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be a multiple of 4");
    if (table && rows < 1) return fail(FUSEDTOK_INVALID_ARGUMENT, "page size must be >= 1");
    if (hkv < 1 || dim < 1 || rows < 0 || tbl_width < 0)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "kv append shapes must satisfy heads>=1, dim>=1, rows>=0");
    if (!lens) return fail(FUSEDTOK_INVALID_ARGUMENT, "lens is required (it is the write position)");
    AppendParams p;
    p.k_new = static_cast<const uint8_t*>(k_new);
    p.v_new = static_cast<const uint8_t*>(v_new);
    p.k_dst = static_cast<uint8_t*>(k_dst);
    p.v_dst = static_cast<uint8_t*>(v_dst);
    p.lens = lens; p.table = table;
    p.B = batch; p.Hkv = hkv;
    p.row_bytes = dim * (int)dtype_size(dt);
    p.rows = rows; p.tbl_width = tbl_width;
    const uintptr_t all = reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) |
                          reinterpret_cast<uintptr_t>(k_dst) | reinterpret_cast<uintptr_t>(v_dst);
    if (all & 7u)       // rows are copied 16 or 8 bytes at a time
        return fail(FUSEDTOK_INVALID_ARGUMENT, "kv append operands must be aligned to 8 bytes");
    const bool wide = (p.row_bytes % 16 == 0) && (all & 15u) == 0;
    const int vec = wide ? 16 : 8;
    const int chunks = hkv * (p.row_bytes / vec);
    dim3 grid((unsigned)batch, (unsigned)((chunks + 255) / 256));
    cudaStream_t cs = (cudaStream_t)stream;
    PdlLaunch l(grid, dim3(256), 0, cs);
    if (wide) cudaLaunchKernelEx(&l.cfg, kv_append_kernel<uint4>, p);
    else cudaLaunchKernelEx(&l.cfg, kv_append_kernel<uint2>, p);
    return check_launch("kv append kernel launch");
}

// FUSEDTOK_PREFILL_SIMT=1 in the environment keeps half-precision prefill on the CUDA-core kernel
// (diagnostics: the two kernels can then be compared on the same inputs).
const bool g_prefill_force_simt = [] {
    const char* e = std::getenv("FUSEDTOK_PREFILL_SIMT");
    return e && e[0] == '1';
}();

// One head's rows as a rank-4 tensor: (64 elements, S rows, D/64 column blocks of 128 bytes, heads). A box
// [64, box rows, D/64, 1] is one tile of one head; rows past S are zero-filled by the copy.
int encode_head_map(CUtensorMap* map, int dt, const void* base, int seq, int dim, long long heads, int box_rows) {
    const cuuint64_t gdim[4] = {64u, (cuuint64_t)seq, (cuuint64_t)(dim / 64), (cuuint64_t)heads};
    const cuuint64_t gstride[3] = {(cuuint64_t)dim * 2, 128u, (cuuint64_t)seq * dim * 2};
    const cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, (cuuint32_t)(dim / 64), 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUresult r = g_encode(map, dt == BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                4, const_cast<void*>(base), gdim, gstride, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(FUSEDTOK_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (code " + std::to_string((int)r) + ")");
    return FUSEDTOK_OK;
}

template <typename T>
void launch_prefill_tc_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p,
                         int* status, cudaStream_t cs) {
    const unsigned grid = (unsigned)((long long)p.B * p.Hq * p.q_tiles);
    if (p.D == 64)
        prefill_tc_kernel<T, 64><<<grid, PF_THREADS, PfCfg<64>::SMEM_BYTES, cs>>>(mq, mk, mv, p, status);
    else if (p.D == 128)
        prefill_tc_kernel<T, 128><<<grid, PF_THREADS, PfCfg<128>::SMEM_BYTES, cs>>>(mq, mk, mv, p, status);
    else
        prefill_tc_kernel<T, 256><<<grid, PF_THREADS, PfCfg<256>::SMEM_BYTES, cs>>>(mq, mk, mv, p, status);
}

// Prefill launcher. reference: attention_prefill_launch_t, src/attention.cu:1649-1712.
template <typename T> void launch_prefill_simt_t(const PrefillParams& p0, cudaStream_t cs) {
    PrefillParams p = p0;
    const long long nbh = (long long)p.B * p.Hq;
    if (p.D <= 128) {
        p.q_tiles = (p.S + 63) / 64;
        prefill_simt_kernel<T, 64, 64><<<(unsigned)(nbh * p.q_tiles), 256, prefill_simt_smem_floats<64, 64>(p.D) * 4, cs>>>(p);
    } else if (p.D <= 256) {
        p.q_tiles = (p.S + 31) / 32;
        prefill_simt_kernel<T, 32, 32><<<(unsigned)(nbh * p.q_tiles), 256, prefill_simt_smem_floats<32, 32>(p.D) * 4, cs>>>(p);
    } else {
        p.q_tiles = (p.S + 15) / 16;
        prefill_simt_kernel<T, 16, 16><<<(unsigned)(nbh * p.q_tiles), 256, prefill_simt_smem_floats<16, 16>(p.D) * 4, cs>>>(p);
    }
}

int prefill_common(int dt, const void* q, const void* k, const void* v, void* out, int batch, int hq, int hkv,
                   int seq, int dim, int causal, uintptr_t stream) {
    int rc = attention_check(batch, hq, hkv, seq, dim);
    if (rc) return rc;
    if (batch == 0 || seq == 0) return FUSEDTOK_OK;           // nothing to compute (src/attention.cu:1654)
    if (!q || !k || !v || !out) return fail(FUSEDTOK_INVALID_ARGUMENT, "null attention operand");
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out);
    if (all & (4 * dtype_size(dt) - 1))
        return fail(FUSEDTOK_INVALID_ARGUMENT, "prefill operands must be aligned to 4 elements");
    const long long q_tiles_min = ((long long)seq + 63) / 64;
    if ((long long)batch * hq * q_tiles_min * 4 > 0x7fffffffLL || (long long)seq * dim > 0x7fffffffLL)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "prefill shape too large for one launch");
    DeviceState* dev = nullptr;
    if ((rc = device_state(&dev))) return rc;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!dev->prefill_attr_set) {
            if ((rc = set_prefill_smem_attrs())) return rc;
            dev->prefill_attr_set = true;
        }
    }
    cudaStream_t cs = (cudaStream_t)stream;
    PrefillParams p{};
    p.q = q; p.k = k; p.v = v; p.out = out;
    p.B = batch; p.Hq = hq; p.Hkv = hkv; p.G = hq / hkv; p.S = seq; p.D = dim;
    p.causal = causal ? 1 : 0;
    p.scale = 1.0f / sqrtf((float)dim);
    // tensor-core path: half storage, head dim 64 / 128, 16-byte aligned operands
    const bool use_tc = dt != F32 && (dim == 64 || dim == 128 || dim == 256) && (all & 15u) == 0 &&
                        !g_prefill_force_simt;
    if (use_tc) {
        if ((rc = get_encode_fn())) return rc;
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            if (!dev->status) {
                if (stream_is_capturing(cs))
                    return fail(FUSEDTOK_RUNTIME_ERROR,
                                "the status word must be allocated outside a CUDA graph capture - warm the "
                                "shape up once before capturing");
                cudaError_t e = cudaMalloc(&dev->status, 256);
                if (e != cudaSuccess) return cuda_fail("status word allocation failed", e);
                e = cudaMemset(dev->status, 0, 256);
                if (e != cudaSuccess) return cuda_fail("status word clear failed", e);
            }
        }
        CUtensorMap mq, mk, mv;
        if ((rc = encode_head_map(&mq, dt, q, seq, dim, (long long)batch * hq, 128))) return rc;
        if ((rc = encode_head_map(&mk, dt, k, seq, dim, (long long)batch * hkv, 64))) return rc;
        if ((rc = encode_head_map(&mv, dt, v, seq, dim, (long long)batch * hkv, 64))) return rc;
        p.q_tiles = (seq + 127) / 128;
        if (dt == BF16) launch_prefill_tc_t<__nv_bfloat16>(mq, mk, mv, p, dev->status, cs);
        else launch_prefill_tc_t<__half>(mq, mk, mv, p, dev->status, cs);
        return check_launch("attention prefill kernel launch");
    }
    if (dt == F32) launch_prefill_simt_t<float>(p, cs);
    else if (dt == BF16) launch_prefill_simt_t<__nv_bfloat16>(p, cs);
    else launch_prefill_simt_t<__half>(p, cs);
    return check_launch("attention prefill kernel launch");
}

// reference: rope_launch / rope_neox_launch (+ _bf16), src/rope.cu:148-190 and its checks at :20-32
int rope_common(int dt, int neox, const void* x, void* y, int seq, int dim, float theta, int pos_offset,
                uintptr_t stream) {
    if (seq < 0 || dim <= 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "seq must be >= 0 and dim must be > 0");
    if (dim % 2 != 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be even (RoPE pairs elements)");
    if (pos_offset < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "pos_offset must be >= 0");
    if (!(theta > 0.0f)) return fail(FUSEDTOK_INVALID_ARGUMENT, "theta must be positive");
    if (seq == 0) return FUSEDTOK_OK;
    if (!x || !y) return fail(FUSEDTOK_INVALID_ARGUMENT, "null rope operand");
    DeviceState* dev = nullptr;
    int rc = device_state(&dev);
    if (rc) return rc;
    RopeParams p{};
    p.x = x; p.y = y; p.seq = seq; p.dim = dim; p.pos_offset = pos_offset; p.neox = neox ? 1 : 0;
    p.log2_theta = std::log2((double)theta);
    p.ratio = std::exp2(-2.0 / dim * p.log2_theta);
    const size_t es = dtype_size(dt);
    const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y);
    // two pairs per thread need every access (2 elements, rows and halves included) aligned to 2 elements
    const bool vec = dim % 4 == 0 && (all & (2 * es - 1)) == 0;
    const long long work = (long long)seq * (vec ? dim / 4 : dim / 2);
    const long long want = (work + 255) / 256;
    const unsigned grid = (unsigned)std::min<long long>(want, (long long)dev->sm_count * 16);
    cudaStream_t cs = (cudaStream_t)stream;
    if (dt == F32) {
        if (vec) rope_kernel<float, true><<<grid, 256, 0, cs>>>(p);
        else rope_kernel<float, false><<<grid, 256, 0, cs>>>(p);
    } else {
        if (vec) rope_kernel<__nv_bfloat16, true><<<grid, 256, 0, cs>>>(p);
        else rope_kernel<__nv_bfloat16, false><<<grid, 256, 0, cs>>>(p);
    }
    return check_launch("rope kernel launch");
}

// The decode step's three elementwise launches in one (no reference counterpart as a single call; it composes
// rope_launch* on one-row matrices, src/rope.cu:148-190, with kv_append[_paged]_launch*, src/attention.cu:1924-2005).
int rope_append_common(int dt, int neox, const void* q, void* q_out, const void* k_new, const void* v_new,
                       const int* table, const int* lens, void* k_dst, void* v_dst, int batch, int hq, int hkv,
                       int dim, int rows, int tbl_width, float theta, int pos_offset, uintptr_t stream) {
    if (dt < 0 || dt > 2) return fail(FUSEDTOK_INVALID_ARGUMENT, "dtype must be 0 (f32), 1 (bf16) or 2 (fp16)");
    if (batch <= 0) return FUSEDTOK_OK;
    if (dim < 4 || dim % 4 != 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be a multiple of 4");
    if (hq < 1 || hkv < 1 || hq % hkv != 0)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "q_heads must be a positive multiple of kv_heads");
    if (table && rows < 1) return fail(FUSEDTOK_INVALID_ARGUMENT, "page size must be >= 1");
    if (rows < 0 || tbl_width < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "cache rows and table width must be >= 0");
    if (pos_offset < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "pos_offset must be >= 0");
    if (!(theta > 0.0f)) return fail(FUSEDTOK_INVALID_ARGUMENT, "theta must be positive");
    if (!lens) return fail(FUSEDTOK_INVALID_ARGUMENT, "lens is required (it is the write position)");
    if (!q || !q_out || !k_new || !v_new || !k_dst || !v_dst)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "null rope/append operand");
    const size_t es = dtype_size(dt);
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(q_out) |
                          reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) |
                          reinterpret_cast<uintptr_t>(k_dst) | reinterpret_cast<uintptr_t>(v_dst);
    if (all & (2 * es - 1)) return fail(FUSEDTOK_INVALID_ARGUMENT, "operands must be aligned to two elements");
    RopeAppendParams p{};
    p.q = q; p.q_out = q_out; p.k_new = k_new; p.v_new = v_new; p.k_dst = k_dst; p.v_dst = v_dst;
    p.lens = lens; p.table = table;
    p.B = batch; p.Hq = hq; p.Hkv = hkv; p.D = dim; p.rows = rows; p.tbl_width = tbl_width;
    p.pos_offset = pos_offset; p.neox = neox ? 1 : 0;
    p.log2_theta = std::log2((double)theta);
    p.ratio = std::exp2(-2.0 / dim * p.log2_theta);
    const long long work = (long long)(hq + 2 * hkv) * (dim / 4);
    dim3 grid((unsigned)batch, (unsigned)((work + 255) / 256));
    cudaStream_t cs = (cudaStream_t)stream;
    PdlLaunch l(grid, dim3(256), 0, cs);
    if (dt == F32) cudaLaunchKernelEx(&l.cfg, rope_append_kernel<float>, p);
    else if (dt == BF16) cudaLaunchKernelEx(&l.cfg, rope_append_kernel<__nv_bfloat16>, p);
    else cudaLaunchKernelEx(&l.cfg, rope_append_kernel<__half>, p);
    return check_launch("rope + kv append kernel launch");
}

// RAII device buffer for the staged paths (reference: DevBuf, src/bindings.cpp:47-66)
struct DevBuf {
    void* p = nullptr;
    cudaError_t err = cudaSuccess;
    explicit DevBuf(size_t bytes) {
        if (bytes) err = cudaMalloc(&p, bytes);
    }
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
};

}  // namespace

extern "C" {

const char* fusedtok_last_error(void) { return g_err.c_str(); }

int fusedtok_cuda_available(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return count > 0;
}

int fusedtok_attention_decode_launch(const float* q, const float* k, const float* v, const int* lens,
                                     float* out, int batch, int q_heads, int kv_heads, int cache_rows,
                                     int dim, uintptr_t stream) {
    return decode_contig(F32, q, k, v, lens, out, nullptr, batch, q_heads, kv_heads, cache_rows, dim, stream);
}
int fusedtok_attention_decode_launch_bf16(const void* q, const void* k, const void* v, const int* lens,
                                          void* out, int batch, int q_heads, int kv_heads, int cache_rows,
                                          int dim, uintptr_t stream) {
    return decode_contig(BF16, q, k, v, lens, out, nullptr, batch, q_heads, kv_heads, cache_rows, dim, stream);
}
int fusedtok_attention_decode_launch_fp16(const void* q, const void* k, const void* v, const int* lens,
                                          void* out, int batch, int q_heads, int kv_heads, int cache_rows,
                                          int dim, uintptr_t stream) {
    return decode_contig(F16, q, k, v, lens, out, nullptr, batch, q_heads, kv_heads, cache_rows, dim, stream);
}

int fusedtok_attention_decode_paged_launch(const float* q, const float* k_pool, const float* v_pool,
                                           const int* table, const int* lens, float* out, int batch,
                                           int q_heads, int kv_heads, int page, int tbl_width, int dim,
                                           uintptr_t stream) {
    return decode_paged(F32, q, k_pool, v_pool, table, lens, out, batch, q_heads, kv_heads, page, tbl_width, dim,
                        stream);
}
int fusedtok_attention_decode_paged_launch_bf16(const void* q, const void* k_pool, const void* v_pool,
                                                const int* table, const int* lens, void* out, int batch,
                                                int q_heads, int kv_heads, int page, int tbl_width, int dim,
                                                uintptr_t stream) {
    return decode_paged(BF16, q, k_pool, v_pool, table, lens, out, batch, q_heads, kv_heads, page, tbl_width,
                        dim, stream);
}
int fusedtok_attention_decode_paged_launch_fp16(const void* q, const void* k_pool, const void* v_pool,
                                                const int* table, const int* lens, void* out, int batch,
                                                int q_heads, int kv_heads, int page, int tbl_width, int dim,
                                                uintptr_t stream) {
    return decode_paged(F16, q, k_pool, v_pool, table, lens, out, batch, q_heads, kv_heads, page, tbl_width,
                        dim, stream);
}

int fusedtok_attention_decode(const float* q, const float* k, const float* v, const int* lens, float* out,
                              int batch, int q_heads, int kv_heads, int cache_rows, int dim) {
    int rc = attention_check(batch, q_heads, kv_heads, cache_rows, dim);
    if (rc) return rc;
    if (lens)
        for (int i = 0; i < batch; ++i)
            if (lens[i] < 0 || lens[i] > cache_rows)
                return fail(FUSEDTOK_INVALID_ARGUMENT, "lens entries must be within [0, cache rows]");
    const size_t q_b = (size_t)batch * q_heads * dim * 4;
    const size_t kv_b = (size_t)batch * kv_heads * cache_rows * dim * 4;
    if (q_b == 0) return FUSEDTOK_OK;
    DevBuf dq(q_b), dk(kv_b), dv(kv_b), dl(lens ? (size_t)batch * 4 : 0), dy(q_b);
    for (const DevBuf* b : {&dq, &dk, &dv, &dl, &dy})
        if (b->err != cudaSuccess) return cuda_fail("cudaMalloc failed", b->err);
    cudaError_t e;
    if ((e = cudaMemcpy(dq.p, q, q_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if (kv_b) {
        if ((e = cudaMemcpy(dk.p, k, kv_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
        if ((e = cudaMemcpy(dv.p, v, kv_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    }
    if (lens && (e = cudaMemcpy(dl.p, lens, (size_t)batch * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
        return cuda_fail("H2D copy failed", e);
    rc = fusedtok_attention_decode_launch((const float*)dq.p, (const float*)dk.p, (const float*)dv.p,
                                          lens ? (const int*)dl.p : nullptr, (float*)dy.p, batch, q_heads,
                                          kv_heads, cache_rows, dim, 0);
    if (rc) return rc;
    if ((e = cudaMemcpy(out, dy.p, q_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("attention decode kernel failed", e);
    return FUSEDTOK_OK;
}

int fusedtok_attention_decode_paged(const float* q, const float* k_pool, const float* v_pool, const int* table,
                                    const int* lens, float* out, int batch, int q_heads, int kv_heads,
                                    int page, int tbl_width, int num_blocks, int dim) {
    const long long span = (long long)tbl_width * page;
    if (span > (1LL << 30)) return fail(FUSEDTOK_INVALID_ARGUMENT, "table capacity too large");
    int rc = attention_check(batch, q_heads, kv_heads, span, dim);
    if (rc) return rc;
    if (page < 1) return fail(FUSEDTOK_INVALID_ARGUMENT, "page size must be >= 1");
    if (num_blocks < 0 || tbl_width < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "attention operand size mismatch");
    // host-side validation of table and lens values (src/bindings.cpp:2524-2539)
    const size_t tbl_n = (size_t)batch * tbl_width;
    for (size_t i = 0; i < tbl_n; ++i)
        if (table[i] < 0 || table[i] >= num_blocks)
            return fail(FUSEDTOK_INVALID_ARGUMENT, "block table entries must be valid pool block ids");
    if (lens)
        for (int i = 0; i < batch; ++i)
            if (lens[i] < 0 || lens[i] > span)
                return fail(FUSEDTOK_INVALID_ARGUMENT, "lens entries must be within [0, table width * page]");
    const size_t q_b = (size_t)batch * q_heads * dim * 4;
    const size_t kv_b = (size_t)num_blocks * kv_heads * page * dim * 4;
    if (q_b == 0) return FUSEDTOK_OK;
    DevBuf dq(q_b), dk(kv_b), dv(kv_b), dt(tbl_n * 4), dl(lens ? (size_t)batch * 4 : 0), dy(q_b);
    for (const DevBuf* b : {&dq, &dk, &dv, &dt, &dl, &dy})
        if (b->err != cudaSuccess) return cuda_fail("cudaMalloc failed", b->err);
    cudaError_t e;
    if ((e = cudaMemcpy(dq.p, q, q_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if (kv_b) {
        if ((e = cudaMemcpy(dk.p, k_pool, kv_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
        if ((e = cudaMemcpy(dv.p, v_pool, kv_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    }
    if (tbl_n && (e = cudaMemcpy(dt.p, table, tbl_n * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
        return cuda_fail("H2D copy failed", e);
    if (lens && (e = cudaMemcpy(dl.p, lens, (size_t)batch * 4, cudaMemcpyHostToDevice)) != cudaSuccess)
        return cuda_fail("H2D copy failed", e);
    rc = fusedtok_attention_decode_paged_launch((const float*)dq.p, (const float*)dk.p, (const float*)dv.p,
                                                (const int*)dt.p, lens ? (const int*)dl.p : nullptr,
                                                (float*)dy.p, batch, q_heads, kv_heads, page, tbl_width, dim, 0);
    if (rc) return rc;
    if ((e = cudaMemcpy(out, dy.p, q_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("attention decode paged kernel failed", e);
    return FUSEDTOK_OK;
}

int fusedtok_attention_prefill_launch(const float* q, const float* k, const float* v, float* out, int batch,
                                      int q_heads, int kv_heads, int seq, int dim, int causal, uintptr_t stream) {
    return prefill_common(F32, q, k, v, out, batch, q_heads, kv_heads, seq, dim, causal, stream);
}
int fusedtok_attention_prefill_launch_bf16(const void* q, const void* k, const void* v, void* out, int batch,
                                           int q_heads, int kv_heads, int seq, int dim, int causal,
                                           uintptr_t stream) {
    return prefill_common(BF16, q, k, v, out, batch, q_heads, kv_heads, seq, dim, causal, stream);
}
int fusedtok_attention_prefill_launch_fp16(const void* q, const void* k, const void* v, void* out, int batch,
                                           int q_heads, int kv_heads, int seq, int dim, int causal,
                                           uintptr_t stream) {
    return prefill_common(F16, q, k, v, out, batch, q_heads, kv_heads, seq, dim, causal, stream);
}

int fusedtok_attention_prefill(const float* q, const float* k, const float* v, float* out, int batch, int q_heads,
                               int kv_heads, int seq, int dim, int causal) {
    int rc = attention_check(batch, q_heads, kv_heads, seq, dim);
    if (rc) return rc;
    const size_t q_b = (size_t)batch * q_heads * seq * dim * 4;
    const size_t kv_b = (size_t)batch * kv_heads * seq * dim * 4;
    if (q_b == 0) return FUSEDTOK_OK;
    DevBuf dq(q_b), dk(kv_b), dv(kv_b), dy(q_b);
    for (const DevBuf* b : {&dq, &dk, &dv, &dy})
        if (b->err != cudaSuccess) return cuda_fail("cudaMalloc failed", b->err);
    cudaError_t e;
    if ((e = cudaMemcpy(dq.p, q, q_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dk.p, k, kv_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dv.p, v, kv_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    rc = fusedtok_attention_prefill_launch((const float*)dq.p, (const float*)dk.p, (const float*)dv.p, (float*)dy.p,
                                           batch, q_heads, kv_heads, seq, dim, causal, 0);
    if (rc) return rc;
    if ((e = cudaMemcpy(out, dy.p, q_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("attention prefill kernel failed", e);
    return FUSEDTOK_OK;
}

int fusedtok_rope_launch(int neox, const float* x, float* y, int seq, int dim, float theta, int pos_offset,
                         uintptr_t stream) {
    return rope_common(F32, neox, x, y, seq, dim, theta, pos_offset, stream);
}
int fusedtok_rope_launch_bf16(const void* x, void* y, int seq, int dim, float theta, int pos_offset,
                              uintptr_t stream) {
    return rope_common(BF16, 0, x, y, seq, dim, theta, pos_offset, stream);
}
int fusedtok_rope_neox_launch_bf16(const void* x, void* y, int seq, int dim, float theta, int pos_offset,
                                   uintptr_t stream) {
    return rope_common(BF16, 1, x, y, seq, dim, theta, pos_offset, stream);
}

int fusedtok_rope(int neox, const float* q, const float* k, float* q_out, float* k_out, int seq, int dim,
                  float theta, int pos_offset) {
    if (seq < 0 || dim <= 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "seq must be >= 0 and dim must be > 0");
    if (dim % 2 != 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be even (RoPE pairs elements)");
    if (pos_offset < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "pos_offset must be >= 0");
    const size_t bytes = (size_t)seq * dim * 4;
    if (bytes == 0) return FUSEDTOK_OK;
    const int n = k ? 2 : 1;
    DevBuf dx(bytes * n), dy(bytes * n);
    for (const DevBuf* b : {&dx, &dy})
        if (b->err != cudaSuccess) return cuda_fail("cudaMalloc failed", b->err);
    cudaError_t e;
    if ((e = cudaMemcpy(dx.p, q, bytes, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if (k && (e = cudaMemcpy((char*)dx.p + bytes, k, bytes, cudaMemcpyHostToDevice)) != cudaSuccess)
        return cuda_fail("H2D copy failed", e);
    for (int i = 0; i < n; ++i) {
        const int rc = fusedtok_rope_launch(neox, (const float*)((char*)dx.p + i * bytes),
                                            (float*)((char*)dy.p + i * bytes), seq, dim, theta, pos_offset, 0);
        if (rc) return rc;
    }
    if ((e = cudaMemcpy(q_out, dy.p, bytes, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if (k && (e = cudaMemcpy(k_out, (char*)dy.p + bytes, bytes, cudaMemcpyDeviceToHost)) != cudaSuccess)
        return cuda_fail("D2H copy failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("rope kernel failed", e);
    return FUSEDTOK_OK;
}

int fusedtok_rope_kv_append_launch(int dtype, int neox, const void* q, void* q_out, const void* k_new,
                                   const void* v_new, const int* lens, void* k_cache, void* v_cache, int batch,
                                   int q_heads, int kv_heads, int dim, int cache_rows, float theta, int pos_offset,
                                   uintptr_t stream) {
    return rope_append_common(dtype, neox, q, q_out, k_new, v_new, nullptr, lens, k_cache, v_cache, batch, q_heads,
                              kv_heads, dim, cache_rows, 0, theta, pos_offset, stream);
}
int fusedtok_rope_kv_append_paged_launch(int dtype, int neox, const void* q, void* q_out, const void* k_new,
                                         const void* v_new, const int* table, const int* lens, void* k_pool,
                                         void* v_pool, int batch, int q_heads, int kv_heads, int dim, int page,
                                         int tbl_width, float theta, int pos_offset, uintptr_t stream) {
    if (!table) return fail(FUSEDTOK_INVALID_ARGUMENT, "block table is required");
    return rope_append_common(dtype, neox, q, q_out, k_new, v_new, table, lens, k_pool, v_pool, batch, q_heads,
                              kv_heads, dim, page, tbl_width, theta, pos_offset, stream);
}

int fusedtok_kv_append_launch(const float* k_new, const float* v_new, const int* lens, float* k_cache,
                              float* v_cache, int batch, int kv_heads, int dim, int cache_rows, uintptr_t stream) {
    return kv_append_common(F32, k_new, v_new, nullptr, lens, k_cache, v_cache, batch, kv_heads, dim, cache_rows, 0, stream);
}
int fusedtok_kv_append_launch_bf16(const void* k_new, const void* v_new, const int* lens, void* k_cache,
                                   void* v_cache, int batch, int kv_heads, int dim, int cache_rows, uintptr_t stream) {
    return kv_append_common(BF16, k_new, v_new, nullptr, lens, k_cache, v_cache, batch, kv_heads, dim, cache_rows, 0, stream);
}
int fusedtok_kv_append_launch_fp16(const void* k_new, const void* v_new, const int* lens, void* k_cache,
                                   void* v_cache, int batch, int kv_heads, int dim, int cache_rows, uintptr_t stream) {
    return kv_append_common(F16, k_new, v_new, nullptr, lens, k_cache, v_cache, batch, kv_heads, dim, cache_rows, 0, stream);
}
int fusedtok_kv_append_paged_launch(const float* k_new, const float* v_new, const int* table, const int* lens,
                                    float* k_pool, float* v_pool, int batch, int kv_heads, int dim, int page,
                                    int tbl_width, uintptr_t stream) {
    if (!table) return fail(FUSEDTOK_INVALID_ARGUMENT, "block table must not be null");
    return kv_append_common(F32, k_new, v_new, table, lens, k_pool, v_pool, batch, kv_heads, dim, page, tbl_width, stream);
}
int fusedtok_kv_append_paged_launch_bf16(const void* k_new, const void* v_new, const int* table, const int* lens,
                                         void* k_pool, void* v_pool, int batch, int kv_heads, int dim, int page,
                                         int tbl_width, uintptr_t stream) {
    if (!table) return fail(FUSEDTOK_INVALID_ARGUMENT, "block table must not be null");
    return kv_append_common(BF16, k_new, v_new, table, lens, k_pool, v_pool, batch, kv_heads, dim, page, tbl_width, stream);
}
int fusedtok_kv_append_paged_launch_fp16(const void* k_new, const void* v_new, const int* table, const int* lens,
                                         void* k_pool, void* v_pool, int batch, int kv_heads, int dim, int page,
                                         int tbl_width, uintptr_t stream) {
    if (!table) return fail(FUSEDTOK_INVALID_ARGUMENT, "block table must not be null");
    return kv_append_common(F16, k_new, v_new, table, lens, k_pool, v_pool, batch, kv_heads, dim, page, tbl_width, stream);
}

// Staged appends: HOST buffers; the caches are updated in place on the host
// (reference: pybind `kv_append` / `kv_append_paged`, src/bindings.cpp:2766-2800, 2636-2696):
// host values are validated, everything is copied to the device, the float32
// launcher runs on the default stream and the caches are copied back.
int fusedtok_kv_append(const float* k_new, const float* v_new, const int* lens, float* k_cache, float* v_cache,
                       int batch, int kv_heads, int dim, int cache_rows) {
    if (batch <= 0) return FUSEDTOK_OK;
    if (dim % 4 != 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be a multiple of 4");
    if (kv_heads < 1 || dim < 1 || cache_rows < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "kv append operand size mismatch");
    if (!lens) return fail(FUSEDTOK_INVALID_ARGUMENT, "lens is required (it is the write position)");
    for (int i = 0; i < batch; ++i)
        if (lens[i] < 0 || lens[i] >= cache_rows)
            return fail(FUSEDTOK_INVALID_ARGUMENT, "lens entries must be within [0, cache rows)");
    const size_t new_b = (size_t)batch * kv_heads * dim * 4;
    const size_t cache_b = (size_t)batch * kv_heads * cache_rows * dim * 4;
    DevBuf dkn(new_b), dvn(new_b), dl((size_t)batch * 4), dk(cache_b), dv(cache_b);
    for (const DevBuf* b : {&dkn, &dvn, &dl, &dk, &dv})
        if (b->err != cudaSuccess) return cuda_fail("cudaMalloc failed", b->err);
    cudaError_t e;
    if ((e = cudaMemcpy(dkn.p, k_new, new_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dvn.p, v_new, new_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dl.p, lens, (size_t)batch * 4, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dk.p, k_cache, cache_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dv.p, v_cache, cache_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    const int rc = fusedtok_kv_append_launch((const float*)dkn.p, (const float*)dvn.p, (const int*)dl.p, (float*)dk.p,
                                             (float*)dv.p, batch, kv_heads, dim, cache_rows, 0);
    if (rc) return rc;
    if ((e = cudaMemcpy(k_cache, dk.p, cache_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaMemcpy(v_cache, dv.p, cache_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("kv append kernel failed", e);
    return FUSEDTOK_OK;
}

int fusedtok_kv_append_paged(const float* k_new, const float* v_new, const int* table, const int* lens,
                             float* k_pool, float* v_pool, int batch, int kv_heads, int dim, int page,
                             int tbl_width, int num_blocks) {
    if (batch <= 0) return FUSEDTOK_OK;
    if (dim % 4 != 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "dim must be a multiple of 4");
    if (page < 1) return fail(FUSEDTOK_INVALID_ARGUMENT, "page size must be >= 1");
    if (kv_heads < 1 || dim < 1 || tbl_width < 0 || num_blocks < 0 || !table)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "kv append operand size mismatch");
    if ((long long)tbl_width * page > (1LL << 30)) return fail(FUSEDTOK_INVALID_ARGUMENT, "table capacity too large");
    if (!lens) return fail(FUSEDTOK_INVALID_ARGUMENT, "lens is required (it is the write position)");
    for (int i = 0; i < batch; ++i) {
        if (lens[i] < 0 || lens[i] >= tbl_width * page)
            return fail(FUSEDTOK_INVALID_ARGUMENT, "lens entries must be within [0, table width * page)");
        const int blk = table[(size_t)i * tbl_width + lens[i] / page];
        if (blk < 0 || blk >= num_blocks)
            return fail(FUSEDTOK_INVALID_ARGUMENT, "block table entries must be valid pool block ids");
    }
    const size_t new_b = (size_t)batch * kv_heads * dim * 4;
    const size_t pool_b = (size_t)num_blocks * kv_heads * page * dim * 4;
    const size_t tbl_b = (size_t)batch * tbl_width * 4;
    DevBuf dkn(new_b), dvn(new_b), dl((size_t)batch * 4), dt(tbl_b), dk(pool_b), dv(pool_b);
    for (const DevBuf* b : {&dkn, &dvn, &dl, &dt, &dk, &dv})
        if (b->err != cudaSuccess) return cuda_fail("cudaMalloc failed", b->err);
    cudaError_t e;
    if ((e = cudaMemcpy(dkn.p, k_new, new_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dvn.p, v_new, new_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dl.p, lens, (size_t)batch * 4, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dt.p, table, tbl_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dk.p, k_pool, pool_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    if ((e = cudaMemcpy(dv.p, v_pool, pool_b, cudaMemcpyHostToDevice)) != cudaSuccess) return cuda_fail("H2D copy failed", e);
    const int rc = fusedtok_kv_append_paged_launch((const float*)dkn.p, (const float*)dvn.p, (const int*)dt.p,
                                                   (const int*)dl.p, (float*)dk.p, (float*)dv.p, batch, kv_heads, dim,
                                                   page, tbl_width, 0);
    if (rc) return rc;
    if ((e = cudaMemcpy(k_pool, dk.p, pool_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaMemcpy(v_pool, dv.p, pool_b, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("D2H copy failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("kv append paged kernel failed", e);
    return FUSEDTOK_OK;
}

int fusedtok_attention_decode_partial_launch(int dtype, const void* q, const void* k, const void* v,
                                             const int* lens, float* partial, int batch, int q_heads,
                                             int kv_heads, int cache_rows, int dim, uintptr_t stream) {
    if (dtype < 0 || dtype > 2) return fail(FUSEDTOK_INVALID_ARGUMENT, "dtype must be 0 (f32), 1 (bf16) or 2 (fp16)");
    if (!partial) return fail(FUSEDTOK_INVALID_ARGUMENT, "partial buffer must not be null");
    return decode_contig(dtype, q, k, v, lens, nullptr, partial, batch, q_heads, kv_heads, cache_rows, dim, stream);
}

long long fusedtok_attention_partial_floats(int batch, int q_heads, int dim) {
    const long long rows = (long long)batch * q_heads;
    return (long long)ftk::triple_acc_offset(rows) + rows * dim;
}

int fusedtok_attention_merge_partials_launch(int dtype, const float* partials, int n_parts, void* out, int batch,
                                             int q_heads, int dim, uintptr_t stream) {
    if (dtype < 0 || dtype > 2) return fail(FUSEDTOK_INVALID_ARGUMENT, "dtype must be 0 (f32), 1 (bf16) or 2 (fp16)");
    if (batch < 0 || q_heads < 1 || n_parts < 1 || dim < 1 || dim % 4 != 0 || dim > 512)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "merge shapes must satisfy batch>=0, heads>=1, parts>=1, dim%4==0, dim<=512");
    const long long rows = (long long)batch * q_heads;
    if (rows == 0) return FUSEDTOK_OK;
    cudaStream_t cs = (cudaStream_t)stream;
    const unsigned grid = (unsigned)((rows + ftk::MERGE_WARPS - 1) / ftk::MERGE_WARPS);
    if (dtype == F32)
        ftk::merge_parts_kernel<float><<<grid, ftk::MERGE_WARPS * 32, 0, cs>>>(partials, n_parts, (float*)out, rows, dim);
    else if (dtype == BF16)
        ftk::merge_parts_kernel<__nv_bfloat16><<<grid, ftk::MERGE_WARPS * 32, 0, cs>>>(partials, n_parts, (__nv_bfloat16*)out, rows, dim);
    else
        ftk::merge_parts_kernel<__half><<<grid, ftk::MERGE_WARPS * 32, 0, cs>>>(partials, n_parts, (__half*)out, rows, dim);
    return check_launch("attention partial-merge kernel launch");
}

// ---- direct peer exchange for the KV-length split ---------------------------------
int fusedtok_exchange_alloc(int n_ranks, int batch, int q_heads, int dim, void** buffer, long long* bytes) {
    if (!buffer || n_ranks < 1 || n_ranks > ftk::MAX_PEERS || batch < 0 || q_heads < 1 || dim < 1)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "exchange buffer: 1..16 ranks, batch>=0, heads>=1, dim>=1");
    const size_t nf = ftk::xchg_block_floats((long long)batch * q_heads, dim);
    const size_t total = ftk::XCHG_DATA_BYTES + (size_t)2 * n_ranks * nf * sizeof(float);
    void* mem = nullptr;
    cudaError_t e = cudaMalloc(&mem, total);
    if (e != cudaSuccess) return cuda_fail("exchange buffer allocation failed", e);
    if ((e = cudaMemset(mem, 0, total)) != cudaSuccess) return cuda_fail("exchange buffer clear failed", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("exchange buffer clear failed", e);
    *buffer = mem;
    if (bytes) *bytes = (long long)total;
    return FUSEDTOK_OK;
}
int fusedtok_exchange_free(void* buffer) {
    if (buffer && cudaFree(buffer) != cudaSuccess) return cuda_fail("exchange buffer free failed", cudaGetLastError());
    return FUSEDTOK_OK;
}
int fusedtok_exchange_export(const void* buffer, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(buffer));
    if (e != cudaSuccess) return cuda_fail("cudaIpcGetMemHandle failed", e);
    memcpy(handle, &h, 64);
    return FUSEDTOK_OK;
}
int fusedtok_exchange_open(const unsigned char handle[64], void** buffer) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    const cudaError_t e = cudaIpcOpenMemHandle(buffer, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail("cudaIpcOpenMemHandle failed", e);
    return FUSEDTOK_OK;
}
int fusedtok_exchange_close(void* buffer) {
    if (buffer && cudaIpcCloseMemHandle(buffer) != cudaSuccess) return cuda_fail("cudaIpcCloseMemHandle failed", cudaGetLastError());
    return FUSEDTOK_OK;
}

int fusedtok_attention_decode_exchange_launch(int dtype, const void* q, const void* k, const void* v, const int* lens,
                                              void* out, void* const* buffers, int n_ranks, int rank, int batch,
                                              int q_heads, int kv_heads, int cache_rows, int dim, uintptr_t stream) {
    if (dtype < 0 || dtype > 2) return fail(FUSEDTOK_INVALID_ARGUMENT, "dtype must be 0 (f32), 1 (bf16) or 2 (fp16)");
    if (!buffers || n_ranks < 1 || n_ranks > ftk::MAX_PEERS || rank < 0 || rank >= n_ranks)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "exchange needs 1..16 ranks and 0 <= rank < ranks");
    for (int j = 0; j < n_ranks; ++j) {
        if (!buffers[j]) return fail(FUSEDTOK_INVALID_ARGUMENT, "exchange buffer pointers must not be null");
        for (int i = 0; i < j; ++i)
            if (buffers[i] == buffers[j])
                return fail(FUSEDTOK_INVALID_ARGUMENT, "exchange buffers of different ranks must be distinct");
    }
    int rc = attention_check(batch, q_heads, kv_heads, cache_rows, dim);
    if (rc) return rc;
    if (batch == 0) return FUSEDTOK_OK;
    if (!out) return fail(FUSEDTOK_INVALID_ARGUMENT, "null attention operand");
    {
        // this rank's own buffer has to be memory of the device the kernel runs on: its flags are polled
        // there. Checked once per buffer and thread (the answer cannot change while the buffer lives).
        thread_local const void* checked = nullptr;
        if (checked != buffers[rank]) {
            int cur = -1;
            cudaPointerAttributes at;
            if (cudaGetDevice(&cur) != cudaSuccess || cudaPointerGetAttributes(&at, buffers[rank]) != cudaSuccess) {
                cudaGetLastError();
                return fail(FUSEDTOK_INVALID_ARGUMENT, "this rank's exchange buffer is not a CUDA allocation");
            }
            if (at.type != cudaMemoryTypeDevice || at.device != cur)
                return fail(FUSEDTOK_INVALID_ARGUMENT,
                            "this rank's exchange buffer must be device memory of the current device (device " +
                                std::to_string(cur) + "), allocated with fusedtok_exchange_alloc");
            checked = buffers[rank];
        }
    }
    PeerDest pd{buffers, n_ranks, rank};
    return decode_common(dtype, q, k, v, nullptr, lens, out, nullptr, batch, q_heads, kv_heads, cache_rows, 0, 0, dim,
                         stream, &pd);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the contiguous-cache launcher.
//
// Some hosts may never call cudaMalloc once they are up: an inference server
// that hands its whole memory budget to its own pool at start-up and treats any
// later driver allocation as a bug, a process running under a memory-accounting
// shim that forbids allocations outside a registered allocator, or code inside
// a real-time loop where cudaMalloc's implicit device synchronisation is not
// acceptable. For them the split-KV workspace below lives in the library image
// itself: a fixed 4 MiB __device__ array that every GPU loading the library
// carries until the process exits. Nothing is allocated, by this function or by
// anything it calls.
//
// The array's name is only a host-side handle; its device address is looked up
// with cudaGetSymbolAddress once per device (with that device current), on the
// first call made on that device, together with the kernels' shared-memory
// attribute. That first call must come before any stream capture; one that
// arrives while the stream is capturing is refused.
//
// All calls on a device share the one array and it keeps whatever the previous
// call left there. Its first 256 bytes hold the status word of this path
// (reported and cleared by fusedtok_attention_device_status together with the
// allocating path's word); the arrival counters that follow are left at zero by
// the kernels themselves (and cleared by fusedtok_attention_device_status after
// a launch that gave up); everything else is written before it is read within a
// call. Two calls that overlap on the GPU (different streams) race on it.
// ---------------------------------------------------------------------------
}  // extern "C"

namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

struct NoAllocDevice {
    bool ready = false;
    unsigned char* base = nullptr;                  // device address of g_noalloc_scratch on this device
};
NoAllocDevice g_noalloc_dev[kMaxDevices];
std::mutex g_noalloc_mutex;

int noalloc_setup(cudaStream_t cs, unsigned char** base_out, int* sm_count) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
    if (dev < 0 || dev >= kMaxDevices) return fail(FUSEDTOK_RUNTIME_ERROR, "device index out of range");
    e = cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail("cudaDeviceGetAttribute", e);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocDevice& d = g_noalloc_dev[dev];
    if (!d.ready) {
        if (stream_is_capturing(cs))
            return fail(FUSEDTOK_RUNTIME_ERROR,
                        "the first allocation-free decode call on a device sets the library up and cannot be "
                        "captured - warm the shape up once before capturing");
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return cuda_fail("cudaGetSymbolAddress(static scratch)", e);
        const int rc = set_all_smem_attrs();
        if (rc) return rc;
        d.base = static_cast<unsigned char*>(ptr);
        d.ready = true;
    }
    *base_out = d.base;
    return FUSEDTOK_OK;
}

}  // namespace

extern "C" {

int fusedtok_attention_decode_launch_noalloc(int dtype, const void* q, const void* k, const void* v,
                                             const int* lens, void* out, int batch, int q_heads, int kv_heads,
                                             int cache_rows, int dim, uintptr_t stream) {
    if (dtype < 0 || dtype > 2) return fail(FUSEDTOK_INVALID_ARGUMENT, "dtype must be 0 (f32), 1 (bf16) or 2 (fp16)");
    int rc = attention_check(batch, q_heads, kv_heads, cache_rows, dim);
    if (rc) return rc;
    if (batch == 0) return FUSEDTOK_OK;
    cudaStream_t cs = (cudaStream_t)stream;
    const long long out_rows = (long long)batch * q_heads;
    if (cache_rows == 0) {
        const cudaError_t e = cudaMemsetAsync(out, 0, (size_t)out_rows * dim * dtype_size(dtype), cs);
        if (e != cudaSuccess) return cuda_fail("attention zero fill failed", e);
        return FUSEDTOK_OK;
    }
    if ((rc = check_aligned4(dtype, {q, k, v, out}))) return rc;
    unsigned char* base = nullptr;
    int sm_count = 0;
    if ((rc = noalloc_setup(cs, &base, &sm_count))) return rc;

    // the same plan as the allocating launcher: same kernel, same split, same slot layout
    const DecodePlan pl = plan_decode(dtype, q, k, v, false, lens != nullptr, batch, q_heads, kv_heads, cache_rows, 0,
                                      dim, sm_count);
    // carve the static array: [256 B header | counters (fixed size) | (m, l) slots | acc slots].
    // The counter region has a fixed place and size so that it is never reused as slot storage:
    // counters must read zero at the start of every call whatever shape ran before.
    const size_t cnt_b = kNoAllocUnits * sizeof(int);
    const size_t need = 256 + cnt_b + pl.ml_b + pl.acc_b;
    if (pl.words > kNoAllocUnits)
        return fail(FUSEDTOK_INVALID_ARGUMENT,
                    "shape has " + std::to_string(pl.units) + " (sequence, kv head) units but the allocation-free "
                    "entry point is limited to " + std::to_string(kNoAllocUnits - 1));
    if (need > kNoAllocBytes)
        return fail(FUSEDTOK_INVALID_ARGUMENT,
                    "shape needs " + std::to_string(need) + " bytes of split-KV scratch but the allocation-free "
                    "entry point has a fixed " + std::to_string(kNoAllocBytes) + " bytes; use "
                    "fusedtok_attention_decode_launch* for this shape");
    const Scratch sc{reinterpret_cast<int*>(base), reinterpret_cast<int*>(base + 256),
                     reinterpret_cast<float*>(base + 256 + cnt_b),
                     reinterpret_cast<float*>(base + 256 + cnt_b + pl.ml_b)};
    return decode_launch(pl, sc, dtype, q, k, v, nullptr, lens, out, nullptr, batch, q_heads, kv_heads, cache_rows, 0,
                         0, dim, cs, nullptr);
}

int fusedtok_attention_device_status(int* status) {
    if (!status) return fail(FUSEDTOK_INVALID_ARGUMENT, "status pointer must not be null");
    *status = 0;
    DeviceState* dev = nullptr;
    const int rc = device_state(&dev);
    if (rc) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail("device synchronize failed", e);
    int word = 0;
    if (dev->status) {
        if ((e = cudaMemcpy(&word, dev->status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
            return cuda_fail("status read failed", e);
        if (word != 0) {
            // a launch that gave up may have left arrival counters half-way: start clean
            if ((e = cudaMemset(dev->status, 0, sizeof(int))) != cudaSuccess) return cuda_fail("status clear failed", e);
            if (dev->counters && (e = cudaMemset(dev->counters, 0, dev->counters_cap * sizeof(int))) != cudaSuccess)
                return cuda_fail("counter clear failed", e);
            *status = word;
        }
    }
    // the allocation-free path keeps its own word in the header of its static scratch (no allocation here
    // either: the address was cached by that path's first call)
    int cur = 0;
    unsigned char* fixed = nullptr;
    if (cudaGetDevice(&cur) == cudaSuccess && cur >= 0 && cur < kMaxDevices) {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_dev[cur].ready) fixed = g_noalloc_dev[cur].base;
    }
    if (fixed) {
        if ((e = cudaMemcpy(&word, fixed, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
            return cuda_fail("status read failed", e);
        if (word != 0) {
            if ((e = cudaMemset(fixed, 0, 256 + kNoAllocUnits * sizeof(int))) != cudaSuccess)
                return cuda_fail("static scratch clear failed", e);
            if (*status == 0) *status = word;
        }
    }
    return FUSEDTOK_OK;
}

int fusedtok_debug_read_stream(const void* src, unsigned long long bytes, uintptr_t stream) {
    if (!src || (reinterpret_cast<uintptr_t>(src) & 15u) || bytes < 16)
        return fail(FUSEDTOK_INVALID_ARGUMENT, "read stream: a 16-byte aligned device buffer of at least 16 bytes");
    DeviceState* dev = nullptr;
    const int rc = device_state(&dev);
    if (rc) return rc;
    read_stream_kernel<<<dev->sm_count * 8, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4*>(src),
                                                                          (size_t)(bytes / 16), nullptr);
    return check_launch("read stream kernel launch");
}

int fusedtok_debug_set_pool_blocks(long long blocks) {
    if (blocks < 0) return fail(FUSEDTOK_INVALID_ARGUMENT, "pool blocks must be >= 0");
    g_debug_pool_blocks.store(blocks);
    return FUSEDTOK_OK;
}

int fusedtok_debug_poke_status(int which, int code, int counter_index) {
    DeviceState* dev = nullptr;
    int rc = device_state(&dev);
    if (rc) return rc;
    int* word = nullptr;
    int* counters = nullptr;
    if (which == 0) {
        word = dev->status;
        counters = dev->counters;
    } else {
        int cur = 0;
        if (cudaGetDevice(&cur) != cudaSuccess) return cuda_fail("cudaGetDevice", cudaGetLastError());
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_dev[cur].ready) {
            word = reinterpret_cast<int*>(g_noalloc_dev[cur].base);
            counters = reinterpret_cast<int*>(g_noalloc_dev[cur].base + 256);
        }
    }
    if (!word) return fail(FUSEDTOK_RUNTIME_ERROR, "that path has not run on this device yet");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail("device synchronize failed", e);
    if (code >= 0 && (e = cudaMemcpy(word, &code, sizeof(int), cudaMemcpyHostToDevice)) != cudaSuccess)
        return cuda_fail("status write failed", e);
    if (counter_index >= 0) {
        if (code >= 0) {
            const int one = 1;
            if ((e = cudaMemcpy(counters + counter_index, &one, sizeof(int), cudaMemcpyHostToDevice)) != cudaSuccess)
                return cuda_fail("counter write failed", e);
        } else {
            int v = 0;
            if ((e = cudaMemcpy(&v, counters + counter_index, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
                return cuda_fail("counter read failed", e);
            return 100 + v;
        }
    }
    return FUSEDTOK_OK;
}

#ifdef FTK_TIMELINE
// Diagnostic builds only: copies the per-CTA timeline of the last tensor-core decode launch (1024 x 24
// 64-bit words, see decode_tc.cuh) to `host` after synchronising the device.
int ftk_debug_timeline(void* host) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail("device synchronize failed", e);
    e = cudaMemcpyFromSymbol(host, ftk::g_timeline, sizeof(unsigned long long) * 1024 * 24);
    if (e != cudaSuccess) return cuda_fail("timeline read failed", e);
    return FUSEDTOK_OK;
}
#endif

long long fusedtok_attention_launch_count(int reset) {
    const long long n = g_launches;
    if (reset) g_launches = 0;
    return n;
}

}  // extern "C"
