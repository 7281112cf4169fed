/*
 * fusedtok_b200 - C ABI of the B200 (sm_100a) decode-attention library.
 *
 * Drop-in boundary for fusedtok's decode-attention launchers: every entry
 * point below replaces the C++ launcher (or pybind staged binding) of the
 * same name in the reference, with the same parameter order and meaning.
 * Differences from the reference's C++ interface are only those a C ABI
 * forces: functions return an int status instead of throwing
 * (FUSEDTOK_INVALID_ARGUMENT <-> std::invalid_argument -> Python ValueError,
 * FUSEDTOK_RUNTIME_ERROR <-> std::runtime_error -> Python RuntimeError) and
 * the message is fetched with fusedtok_last_error().
 *
 * Contract of the *_launch functions (reference:
 * include/fusedtok/cuda_launch.hpp:3-17): all pointers are caller-owned DEVICE
 * memory on the current device; the work is asynchronous on `stream` (0 = the
 * default stream); nothing is synchronised, read back or retained except the
 * library-owned fp32 workspace, which is allocated (per device, grow-only,
 * never freed) on first use. A decode call that would have to allocate while
 * `stream` is being captured into a CUDA graph allocates nothing: like the
 * reference (src/attention.cu:1498-1509) it runs that launch on a slower
 * kernel that needs no workspace (one CTA per (sequence, kv head) unit), and
 * the captured graph keeps it; warm a shape up once outside the capture to
 * capture the fast one. Other calls that would allocate during a capture
 * (exchange buffers, prefill) fail with FUSEDTOK_RUNTIME_ERROR. Launches on different streams of one
 * device share the workspace and must not overlap (same rule as the
 * reference, include/fusedtok/cuda_launch.hpp:187-190).
 *
 * Shapes: q [B, Hq, D]; contiguous cache k, v [B, Hkv, T, D]; paged pools
 * [Nb, Hkv, P, D] with block table [B, S] (token t of sequence b lives at
 * pool[table[b][t / P]][kv][t % P]); lens [B] int32 or NULL (all rows valid);
 * out [B, Hq, D] in the storage type. Query head h reads kv head
 * h / (Hq / Hkv). Rows at and past lens[b] are never used; lens[b] == 0 or
 * T == 0 gives an exact zero row. D % 4 == 0, D <= 512, Hq % Hkv == 0.
 * Softmax scale 1/sqrt(D); accumulation in float32. q, k, v and out must be
 * aligned to 4 elements (16 bytes for float32, 8 for the 16-bit types): a view
 * that starts at an odd element offset is refused with
 * FUSEDTOK_INVALID_ARGUMENT instead of faulting on the device.
 */
#ifndef FUSEDTOK_B200_H
#define FUSEDTOK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FUSEDTOK_OK 0
#define FUSEDTOK_INVALID_ARGUMENT 1
#define FUSEDTOK_RUNTIME_ERROR 2

/* Message of the last failing call on this thread ("" if none). */
const char* fusedtok_last_error(void);

/* 1 if a usable CUDA device is present. Replaces fusedtok::cuda_available,
 * src/fusedtok.cu:34-37. */
int fusedtok_cuda_available(void);

/* ---- contiguous cache, zero-copy ------------------------------------------
 * Replace fusedtok::attention_decode_launch / _bf16 / _fp16,
 * include/fusedtok/cuda_launch.hpp:334-355 (src/attention.cu:1557-1585). */
int fusedtok_attention_decode_launch(const float* q, const float* k, const float* v,
                                     const int* lens, float* out, int batch, int q_heads,
                                     int kv_heads, int cache_rows, int dim, uintptr_t stream);
int fusedtok_attention_decode_launch_bf16(const void* q, const void* k, const void* v,
                                          const int* lens, void* out, int batch, int q_heads,
                                          int kv_heads, int cache_rows, int dim, uintptr_t stream);
int fusedtok_attention_decode_launch_fp16(const void* q, const void* k, const void* v,
                                          const int* lens, void* out, int batch, int q_heads,
                                          int kv_heads, int cache_rows, int dim, uintptr_t stream);

/* ---- paged cache, zero-copy -----------------------------------------------
 * Replace fusedtok::attention_decode_paged_launch / _bf16 / _fp16,
 * include/fusedtok/cuda_launch.hpp:381-407 (src/attention.cu:1879-1915).
 * Table VALUES are trusted (device memory is not read back). Superset of the
 * reference: any GQA group size is accepted (the reference launcher rejects
 * groups other than 1/2/4/8/16, src/attention.cu:1807-1812; the Python
 * wrapper of this package keeps that rejection). */
int fusedtok_attention_decode_paged_launch(const float* q, const float* k_pool,
                                           const float* v_pool, const int* table, const int* lens,
                                           float* out, int batch, int q_heads, int kv_heads,
                                           int page, int tbl_width, int dim, uintptr_t stream);
int fusedtok_attention_decode_paged_launch_bf16(const void* q, const void* k_pool,
                                                const void* v_pool, const int* table,
                                                const int* lens, void* out, int batch, int q_heads,
                                                int kv_heads, int page, int tbl_width, int dim,
                                                uintptr_t stream);
int fusedtok_attention_decode_paged_launch_fp16(const void* q, const void* k_pool,
                                                const void* v_pool, const int* table,
                                                const int* lens, void* out, int batch, int q_heads,
                                                int kv_heads, int page, int tbl_width, int dim,
                                                uintptr_t stream);

/* ---- staged entry points: HOST buffers in, HOST buffer out ----------------
 * Replace the pybind bindings `attention_decode` / `attention_decode_paged`,
 * src/bindings.cpp:2402-2436 and :2507-2565: float32 only; device buffers are
 * allocated, filled, the float32 launcher runs on the default stream, the
 * result is copied back and the device is synchronised. Host lens / table
 * values are validated (lens in [0, rows], every table entry in [0,
 * num_blocks)). */
int fusedtok_attention_decode(const float* q, const float* k, const float* v, const int* lens,
                              float* out, int batch, int q_heads, int kv_heads, int cache_rows,
                              int dim);
int fusedtok_attention_decode_paged(const float* q, const float* k_pool, const float* v_pool,
                                    const int* table, const int* lens, float* out, int batch,
                                    int q_heads, int kv_heads, int page, int tbl_width,
                                    int num_blocks, int dim);

/* ---- prefill: fresh-sequence self-attention over S query rows ---------------
 * q / out [B, Hq, S, D]; k / v [B, Hkv, S, D]; query row i attends key rows
 * [0, i] when causal != 0, all S rows otherwise; same GQA mapping and shape
 * rules as decode. Device pointers (aligned to 4 elements), asynchronous on
 * `stream`, capturable, no workspace. Replace fusedtok::attention_prefill_launch
 * / _bf16 / _fp16, include/fusedtok/cuda_launch.hpp:362-379
 * (src/attention.cu:1649-1739). The staged form takes HOST float32 buffers
 * and returns after the result is back (src/bindings.cpp:2863-2886). */
int fusedtok_attention_prefill_launch(const float* q, const float* k, const float* v, float* out,
                                      int batch, int q_heads, int kv_heads, int seq, int dim,
                                      int causal, uintptr_t stream);
int fusedtok_attention_prefill_launch_bf16(const void* q, const void* k, const void* v, void* out,
                                           int batch, int q_heads, int kv_heads, int seq, int dim,
                                           int causal, uintptr_t stream);
int fusedtok_attention_prefill_launch_fp16(const void* q, const void* k, const void* v, void* out,
                                           int batch, int q_heads, int kv_heads, int seq, int dim,
                                           int causal, uintptr_t stream);
int fusedtok_attention_prefill(const float* q, const float* k, const float* v, float* out,
                               int batch, int q_heads, int kv_heads, int seq, int dim, int causal);

/* ---- rotary position embedding (the step that produces q and k_new) ---------
 * One [seq, dim] matrix per call, dim even: row r has absolute position
 * r + pos_offset, pair j is rotated by (r + pos_offset) * theta^(-2j/dim);
 * neox == 0 pairs elements (2j, 2j+1), neox != 0 pairs (j, j + dim/2). x and y
 * may be the same buffer. Device pointers, asynchronous on `stream`, capturable.
 * Replace fusedtok::rope_launch / rope_neox_launch (selected by the pybind's
 * bool, src/bindings.cpp:722-735) and rope_launch_bf16 / rope_neox_launch_bf16,
 * include/fusedtok/cuda_launch.hpp (src/rope.cu:148-190). The staged form takes
 * HOST float32 q and optional k (k, k_out may be NULL) and rotates both
 * (src/bindings.cpp:683-716). */
int fusedtok_rope_launch(int neox, const float* x, float* y, int seq, int dim, float theta,
                         int pos_offset, uintptr_t stream);
int fusedtok_rope_launch_bf16(const void* x, void* y, int seq, int dim, float theta,
                              int pos_offset, uintptr_t stream);
int fusedtok_rope_neox_launch_bf16(const void* x, void* y, int seq, int dim, float theta,
                                   int pos_offset, uintptr_t stream);
int fusedtok_rope(int neox, const float* q, const float* k, float* q_out, float* k_out, int seq,
                  int dim, float theta, int pos_offset);

/* ---- kv-cache append: the write side of the decode loop --------------------
 * Scatter ONE fresh token's K and V rows per sequence (k_new, v_new
 * [B, Hkv, D]) into the cache at position lens[b] (lens is required):
 * contiguous caches [B, Hkv, T, D] at row lens[b]; paged pools at block
 * table[b][lens[b] / P], offset lens[b] % P. In place, asynchronous on `stream`,
 * capturable, no workspace. Replace fusedtok::kv_append_launch / _bf16 / _fp16
 * and kv_append_paged_launch / _bf16 / _fp16, include/fusedtok/cuda_launch.hpp:
 * 416-430 and 443-454 (src/attention.cu:1924-2035). Device lens / table values
 * are trusted; a position outside the cache is skipped instead of written. */
int fusedtok_kv_append_launch(const float* k_new, const float* v_new, const int* lens,
                              float* k_cache, float* v_cache, int batch, int kv_heads, int dim,
                              int cache_rows, uintptr_t stream);
int fusedtok_kv_append_launch_bf16(const void* k_new, const void* v_new, const int* lens,
                                   void* k_cache, void* v_cache, int batch, int kv_heads, int dim,
                                   int cache_rows, uintptr_t stream);
int fusedtok_kv_append_launch_fp16(const void* k_new, const void* v_new, const int* lens,
                                   void* k_cache, void* v_cache, int batch, int kv_heads, int dim,
                                   int cache_rows, uintptr_t stream);
int fusedtok_kv_append_paged_launch(const float* k_new, const float* v_new, const int* table,
                                    const int* lens, float* k_pool, float* v_pool, int batch,
                                    int kv_heads, int dim, int page, int tbl_width,
                                    uintptr_t stream);
int fusedtok_kv_append_paged_launch_bf16(const void* k_new, const void* v_new, const int* table,
                                         const int* lens, void* k_pool, void* v_pool, int batch,
                                         int kv_heads, int dim, int page, int tbl_width,
                                         uintptr_t stream);
int fusedtok_kv_append_paged_launch_fp16(const void* k_new, const void* v_new, const int* table,
                                         const int* lens, void* k_pool, void* v_pool, int batch,
                                         int kv_heads, int dim, int page, int tbl_width,
                                         uintptr_t stream);
/* Staged appends: HOST float32 buffers, caches updated in place on the host,
 * lens / table values validated (lens in [0, rows), used table entries in
 * [0, num_blocks)). Replace the pybind bindings `kv_append` / `kv_append_paged`,
 * src/bindings.cpp:2766-2800 and :2636-2696. */
int fusedtok_kv_append(const float* k_new, const float* v_new, const int* lens, float* k_cache,
                       float* v_cache, int batch, int kv_heads, int dim, int cache_rows);
int fusedtok_kv_append_paged(const float* k_new, const float* v_new, const int* table,
                             const int* lens, float* k_pool, float* v_pool, int batch,
                             int kv_heads, int dim, int page, int tbl_width, int num_blocks);

/* ---- rotary embedding + kv-cache append in ONE launch (decode step) ---------
 * The elementwise work that precedes a decode-attention call, fused: q
 * [B, Hq, D] is rotated to position lens[b] + pos_offset into q_out (which may
 * be q), k_new [B, Hkv, D] is rotated to the same position and written
 * straight into the cache at position lens[b], v_new is copied beside it.
 * dtype: 0 float32, 1 bfloat16, 2 float16 (all operands); dim a multiple of 4.
 * No single counterpart in the reference: it composes fusedtok::rope_launch* /
 * rope_neox_launch* on one-row matrices (src/rope.cu:148-190) with
 * kv_append_launch* / kv_append_paged_launch* (src/attention.cu:1924-2035),
 * and its results are bit-identical to fusedtok_rope_launch* followed by
 * fusedtok_kv_append*_launch*. Asynchronous on `stream`, capturable, no
 * workspace; a position outside the cache skips the K/V write. */
int fusedtok_rope_kv_append_launch(int dtype, int neox, const void* q, void* q_out,
                                   const void* k_new, const void* v_new, const int* lens,
                                   void* k_cache, void* v_cache, int batch, int q_heads,
                                   int kv_heads, int dim, int cache_rows, float theta,
                                   int pos_offset, uintptr_t stream);
int fusedtok_rope_kv_append_paged_launch(int dtype, int neox, const void* q, void* q_out,
                                         const void* k_new, const void* v_new, const int* table,
                                         const int* lens, void* k_pool, void* v_pool, int batch,
                                         int q_heads, int kv_heads, int dim, int page,
                                         int tbl_width, float theta, int pos_offset,
                                         uintptr_t stream);

/* ---- KV-length split across GPUs (no counterpart in the reference, which is
 * single-GPU; the exchanged triple and the merge rule are the reference's
 * intra-GPU ones, src/attention.cu:434-463 and :503-548) --------------------
 * *_partial_launch*: same inputs as the contiguous launchers over THIS GPU's
 * slice of the cache rows, but instead of the normalised output it writes the
 * raw triple of every (b, h): `partial` is float32
 * [B*Hq*2 (m, l), padded to a multiple of 4 floats | B*Hq*D unnormalised acc],
 * i.e. fusedtok_attention_partial_floats(batch, q_heads, dim) floats; empty
 * rows give (-inf, 0, 0).
 * dtype: 0 float32, 1 bfloat16, 2 float16.
 * merge_partials_launch: folds n such blocks laid out back to back (the
 * layout an all-gather produces) into the normalised output [B, Hq, D]. */
int fusedtok_attention_decode_partial_launch(int dtype, const void* q, const void* k, const void* v,
                                             const int* lens, float* partial, int batch,
                                             int q_heads, int kv_heads, int cache_rows, int dim,
                                             uintptr_t stream);
long long fusedtok_attention_partial_floats(int batch, int q_heads, int dim);
int fusedtok_attention_merge_partials_launch(int dtype, const float* partials, int n_parts,
                                             void* out, int batch, int q_heads, int dim,
                                             uintptr_t stream);

/* ---- KV-length split with direct peer exchange (no counterpart in the
 * reference) ------------------------------------------------------------------
 * The same split as above, but the ranks exchange their raw triples themselves
 * instead of through a collective library, inside the ONE kernel a step
 * launches per rank: every rank owns an exchange buffer
 * (fusedtok_exchange_alloc), exports it (fusedtok_exchange_export: a 64-byte
 * CUDA IPC handle to hand to the other processes by any means) and maps its
 * peers' buffers (fusedtok_exchange_open). The split-KV kernel stores the rows
 * of every (sequence, kv head) unit it finishes into EVERY rank's buffer with
 * plain stores over NVLink, the step number riding beside every value (each
 * 8-byte half validates itself: no fence, no separate flag); at its end each
 * CTA reads the n ranks' words of its share of the rows from its own rank's
 * memory - polling, bounded, until they carry the current step - and folds the
 * n blocks into `out` (every rank gets the
 * whole output). `buffers` is a HOST array of n distinct device pointers, entry
 * `rank` being the rank's own buffer, which must be memory of the current
 * device. All ranks must make the same sequence of calls with the same shapes.
 * The step number lives in the buffer, so a captured CUDA graph can be
 * replayed. A peer that never delivers makes the wait expire after 2 s: the
 * call's output is then invalid, fusedtok_attention_device_status reports 5,
 * the context stays usable. */
int fusedtok_exchange_alloc(int n_ranks, int batch, int q_heads, int dim, void** buffer,
                            long long* bytes);
int fusedtok_exchange_free(void* buffer);
int fusedtok_exchange_export(const void* buffer, unsigned char handle[64]);
int fusedtok_exchange_open(const unsigned char handle[64], void** buffer);
int fusedtok_exchange_close(void* buffer);
int fusedtok_attention_decode_exchange_launch(int dtype, const void* q, const void* k, const void* v,
                                              const int* lens, void* out, void* const* buffers,
                                              int n_ranks, int rank, int batch, int q_heads,
                                              int kv_heads, int cache_rows, int dim,
                                              uintptr_t stream);

/* ---- allocation-free launcher (no counterpart in the reference, whose split
 * path always allocates its workspace with cudaMalloc) -------------------------
 * For callers that may not allocate device memory once they are running (a
 * server that pre-budgets all of HBM into its own pool, a host under an
 * allocator-policing shim, a latency-critical loop that cannot take
 * cudaMalloc's implicit sync).
 * Same inputs, outputs and results as fusedtok_attention_decode_launch{,_bf16,
 * _fp16} (dtype 0 float32, 1 bfloat16, 2 float16) - same kernel, same split -
 * but the split-KV scratch is a fixed 4 MiB array inside the library image,
 * held by every GPU that loads the library until the process exits. Calls no
 * cudaMalloc / cudaFree and no allocating library routine. Shapes whose scratch
 * would exceed 4 MiB (256 B header + 64 KiB of counters + slots *
 * heads_per_chunk * (dim + 2) floats, slots = units + ranges of the launch), or
 * with more than 16383 (sequence, kv head, chunk) units, are rejected with
 * FUSEDTOK_INVALID_ARGUMENT. The first call on a device looks up the array's
 * device address and sets kernel attributes: make it before any stream capture
 * (a first call that arrives during a capture fails with
 * FUSEDTOK_RUNTIME_ERROR). All calls on a device share the array; calls that
 * overlap on the GPU race on it. Its header holds this path's status word,
 * which fusedtok_attention_device_status reports and clears. */
int fusedtok_attention_decode_launch_noalloc(int dtype, const void* q, const void* k, const void* v,
                                             const int* lens, void* out, int batch, int q_heads,
                                             int kv_heads, int cache_rows, int dim, uintptr_t stream);

/* ---- diagnostics -----------------------------------------------------------
 * Every device-side wait in the kernels is bounded; a wait that expires stores
 * a non-zero code in a per-device status word and the kernel still completes.
 * This call synchronises the current device, returns the word through
 * `status` (0 = ok) and clears it. It covers both the workspace the allocating
 * launchers own and the static scratch of the allocation-free launcher (the
 * first non-zero of the two is returned); after a non-zero word the arrival
 * counters of that path are cleared too, so the next launch starts clean. */
int fusedtok_attention_device_status(int* status);

/* Number of kernels this library has launched on this thread since the last
 * call with reset != 0 (benchmark bookkeeping). */
long long fusedtok_attention_launch_count(int reset);

/* Test hook for the status path (no GPU fault involved): with the device idle,
 * writes `code` (>= 0) into the status word of the allocating path (which == 0)
 * or of the allocation-free path (which == 1) and, when counter_index >= 0,
 * sets that arrival counter to 1 - the state a launch that gave up would leave.
 * With code < 0 it instead returns 100 + the current value of that counter.
 * Fails if the chosen path has not run on the current device yet. */
int fusedtok_debug_poke_status(int which, int code, int counter_index);

/* Test hook of the self-checking build (the library compiled with -DFTK_BOUNDS:
 * every cache row, partial slot and arrival counter a decode kernel computes is
 * compared with what the launch owns; a value out of range sets status 8 and the
 * access is redirected or left out instead of made). The contiguous entry points
 * know the size of their cache; the paged ones are not told the size of the pool,
 * so a test states it here (0 = unknown, page ids unchecked). No effect on the
 * product build; no counterpart in the reference. */
int fusedtok_debug_set_pool_blocks(long long blocks);

/* Measurement aid (bench.py's roofline): launches a kernel that reads `bytes`
 * of device memory at `src` (16-byte aligned) once with plain streaming loads
 * and discards them - a read-only bandwidth figure to set beside the copy
 * bandwidth the roofline is quoted against. No counterpart in the reference. */
int fusedtok_debug_read_stream(const void* src, unsigned long long bytes, uintptr_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FUSEDTOK_B200_H */
