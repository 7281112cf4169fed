// TEST INFRASTRUCTURE ONLY - C-ABI shim over the UNMODIFIED reference sources.
//
// oracle/build_oracle.py compiles this file together with the reference's own
// src/attention.cu (read in place from the reference checkout, never copied)
// into oracle/_ref/libfusedtok_ref.so. The shim only converts plain pointers
// into the std::vector arguments the reference's CPU functions take
// (reference: include/fusedtok/attention.hpp:28-61) and forwards to the
// reference's GPU launchers (reference: include/fusedtok/cuda_launch.hpp:334-407)
// so that the reference kernels can be timed beside ours on the same GPU.
// Exceptions become return codes: 0 ok, 1 std::invalid_argument, 2 other.

#include "fusedtok/attention.hpp"
#include "fusedtok/fusedtok.hpp"
#include "fusedtok/cuda_launch.hpp"

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace {
thread_local std::string g_err;

template <typename F> int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::invalid_argument& e) {
        g_err = e.what();
        return 1;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 2;
    }
}
} // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// reference: fusedtok::attention_decode_cpu, src/attention.cu:1318-1373
int ref_attention_decode_cpu(const float* q, const float* k, const float* v,
                             const int* lens, float* out, int batch, int hq,
                             int hkv, int t_seq, int dim) {
    return guarded([&] {
        if (batch < 0 || hq < 0 || hkv < 0 || t_seq < 0 || dim < 0)
            throw std::invalid_argument("negative shape");
        const size_t nq = (size_t)batch * hq * dim;
        const size_t nkv = (size_t)batch * hkv * t_seq * dim;
        std::vector<float> qv(q, q + nq), kv(k, k + nkv), vv(v, v + nkv);
        std::vector<int> lv;
        if (lens) lv.assign(lens, lens + batch);
        std::vector<float> y = fusedtok::attention_decode_cpu(
            qv, kv, vv, lens ? &lv : nullptr, batch, hq, hkv, t_seq, dim);
        if (!y.empty()) std::memcpy(out, y.data(), y.size() * sizeof(float));
    });
}

// reference: fusedtok::attention_decode_paged_cpu, src/attention.cu:1382-1456
int ref_attention_decode_paged_cpu(const float* q, const float* k_pool,
                                   const float* v_pool, const int* table,
                                   const int* lens, float* out, int batch,
                                   int hq, int hkv, int page, int tbl_width,
                                   int num_blocks, int dim) {
    return guarded([&] {
        if (batch < 0 || hq < 0 || hkv < 0 || page < 0 || tbl_width < 0 ||
            num_blocks < 0 || dim < 0)
            throw std::invalid_argument("negative shape");
        const size_t nq = (size_t)batch * hq * dim;
        const size_t np = (size_t)num_blocks * hkv * page * dim;
        std::vector<float> qv(q, q + nq), kv(k_pool, k_pool + np),
            vv(v_pool, v_pool + np);
        std::vector<int> tv(table, table + (size_t)batch * tbl_width);
        std::vector<int> lv;
        if (lens) lv.assign(lens, lens + batch);
        std::vector<float> y = fusedtok::attention_decode_paged_cpu(
            qv, kv, vv, tv, lens ? &lv : nullptr, batch, hq, hkv, page,
            tbl_width, num_blocks, dim);
        if (!y.empty()) std::memcpy(out, y.data(), y.size() * sizeof(float));
    });
}

// reference: fusedtok::kv_append_cpu / kv_append_paged_cpu, src/attention.cu:2037-2099.
// The caches are updated in place.
int ref_kv_append_cpu(const float* k_new, const float* v_new, const int* lens, float* k_cache,
                      float* v_cache, int batch, int hkv, int dim, int t_rows) {
    return guarded([&] {
        const size_t nn = (size_t)batch * hkv * dim, nc = (size_t)batch * hkv * t_rows * dim;
        std::vector<float> kn(k_new, k_new + nn), vn(v_new, v_new + nn), kc(k_cache, k_cache + nc),
            vc(v_cache, v_cache + nc);
        std::vector<int> lv(lens, lens + batch);
        fusedtok::kv_append_cpu(kn, vn, lv, kc, vc, batch, hkv, dim, t_rows);
        std::memcpy(k_cache, kc.data(), nc * sizeof(float));
        std::memcpy(v_cache, vc.data(), nc * sizeof(float));
    });
}
int ref_kv_append_paged_cpu(const float* k_new, const float* v_new, const int* table, const int* lens,
                            float* k_pool, float* v_pool, int batch, int hkv, int dim, int page,
                            int tbl_width, int num_blocks) {
    return guarded([&] {
        const size_t nn = (size_t)batch * hkv * dim, np = (size_t)num_blocks * hkv * page * dim;
        std::vector<float> kn(k_new, k_new + nn), vn(v_new, v_new + nn), kp(k_pool, k_pool + np),
            vp(v_pool, v_pool + np);
        std::vector<int> lv(lens, lens + batch), tv(table, table + (size_t)batch * tbl_width);
        fusedtok::kv_append_paged_cpu(kn, vn, tv, lv, kp, vp, batch, hkv, dim, page, tbl_width, num_blocks);
        std::memcpy(k_pool, kp.data(), np * sizeof(float));
        std::memcpy(v_pool, vp.data(), np * sizeof(float));
    });
}

// reference: fusedtok::attention_prefill_cpu, src/attention.cu:1591-1638
int ref_attention_prefill_cpu(const float* q, const float* k, const float* v, float* out, int batch,
                              int hq, int hkv, int seq, int dim, int causal) {
    return guarded([&] {
        if (batch < 0 || hq < 0 || hkv < 0 || seq < 0 || dim < 0)
            throw std::invalid_argument("negative shape");
        const size_t nq = (size_t)batch * hq * seq * dim, nkv = (size_t)batch * hkv * seq * dim;
        std::vector<float> qv(q, q + nq), kv(k, k + nkv), vv(v, v + nkv);
        std::vector<float> y = fusedtok::attention_prefill_cpu(qv, kv, vv, batch, hq, hkv, seq, dim, causal != 0);
        if (!y.empty()) std::memcpy(out, y.data(), y.size() * sizeof(float));
    });
}

// reference: fusedtok::rope_cpu / rope_neox_cpu, src/rope.cu:95-146 (one matrix per call)
int ref_rope_cpu(const float* x, float* y, int seq, int dim, float theta, int pos_offset, int neox) {
    return guarded([&] {
        if (seq < 0 || dim < 0) throw std::invalid_argument("negative shape");
        std::vector<float> xv(x, x + (size_t)seq * dim);
        auto res = neox ? fusedtok::rope_neox_cpu(xv, nullptr, seq, dim, theta, pos_offset)
                        : fusedtok::rope_cpu(xv, nullptr, seq, dim, theta, pos_offset);
        if (!res.first.empty()) std::memcpy(y, res.first.data(), res.first.size() * sizeof(float));
    });
}

// The reference GPU launchers, device pointers in, asynchronous on `stream`.
// dtype: 0 = float32, 1 = bfloat16, 2 = float16.
int ref_attention_decode_launch(int dtype, const void* q, const void* k,
                                const void* v, const int* lens, void* out,
                                int batch, int hq, int hkv, int t_seq, int dim,
                                std::uintptr_t stream) {
    return guarded([&] {
        if (dtype == 0)
            fusedtok::attention_decode_launch(
                (const float*)q, (const float*)k, (const float*)v, lens,
                (float*)out, batch, hq, hkv, t_seq, dim, stream);
        else if (dtype == 1)
            fusedtok::attention_decode_launch_bf16(q, k, v, lens, out, batch,
                                                   hq, hkv, t_seq, dim, stream);
        else
            fusedtok::attention_decode_launch_fp16(q, k, v, lens, out, batch,
                                                   hq, hkv, t_seq, dim, stream);
    });
}

int ref_attention_decode_paged_launch(int dtype, const void* q,
                                      const void* k_pool, const void* v_pool,
                                      const int* table, const int* lens,
                                      void* out, int batch, int hq, int hkv,
                                      int page, int tbl_width, int dim,
                                      std::uintptr_t stream) {
    return guarded([&] {
        if (dtype == 0)
            fusedtok::attention_decode_paged_launch(
                (const float*)q, (const float*)k_pool, (const float*)v_pool,
                table, lens, (float*)out, batch, hq, hkv, page, tbl_width, dim,
                stream);
        else if (dtype == 1)
            fusedtok::attention_decode_paged_launch_bf16(
                q, k_pool, v_pool, table, lens, out, batch, hq, hkv, page,
                tbl_width, dim, stream);
        else
            fusedtok::attention_decode_paged_launch_fp16(
                q, k_pool, v_pool, table, lens, out, batch, hq, hkv, page,
                tbl_width, dim, stream);
    });
}

// reference: attention_prefill_launch{,_bf16,_fp16}, include/fusedtok/cuda_launch.hpp:362-379
int ref_attention_prefill_launch(int dtype, const void* q, const void* k, const void* v, void* out,
                                 int batch, int hq, int hkv, int seq, int dim, int causal,
                                 std::uintptr_t stream) {
    return guarded([&] {
        if (dtype == 0)
            fusedtok::attention_prefill_launch((const float*)q, (const float*)k, (const float*)v, (float*)out,
                                               batch, hq, hkv, seq, dim, causal != 0, stream);
        else if (dtype == 1)
            fusedtok::attention_prefill_launch_bf16(q, k, v, out, batch, hq, hkv, seq, dim, causal != 0, stream);
        else
            fusedtok::attention_prefill_launch_fp16(q, k, v, out, batch, hq, hkv, seq, dim, causal != 0, stream);
    });
}

} // extern "C"
