/*
 * TEST INFRASTRUCTURE ONLY - CPU oracle for fusedtok's decode attention.
 *
 * A plain-C restatement of the reference's CPU implementation of the
 * decode-attention path. It exists to check the CUDA kernels; nothing in the
 * shipped package links, loads or calls it. Only the tests, the smoke check
 * and the benchmark's CPU-baseline leg may use it.
 *
 * Parity status: PINNED. The restatement is checked bit-for-bit against the
 * reference's own attention_decode_cpu / attention_decode_paged_cpu compiled
 * from the reference sources (oracle/_ref, see oracle/build_oracle.py) and
 * against golden outputs generated from that build (tests/golden/).
 *
 * Algorithm (reference: src/attention.cu:1318-1373 contiguous,
 * src/attention.cu:1382-1456 paged): for every (sequence b, query head h)
 * with kv = h / (Hq / Hkv):
 *   pass 1  s[t] = (sum_d q[d] * K[t][d]) * (1/sqrtf(D));  m = max_t s[t]
 *   pass 2  l = sum_t expf(s[t] - m)
 *   pass 3  out[d] += (expf(s[t] - m) / l) * V[t][d]      (t ascending)
 * All arithmetic in float32, sums strictly sequential in t and d, libm expf,
 * len == 0 leaves a zero row. Compile WITHOUT -ffast-math / FMA contraction
 * so the operation order matches the reference build.
 *
 * Return codes: 0 ok, 1 invalid argument (the reference throws
 * std::invalid_argument for the same conditions).
 */

#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_MAX_DIM 512 /* reference: kAttMaxDim, src/attention.cu:67 */

/* reference: attention_check, src/attention.cu:184-193 */
static int oracle_check(int batch, int hq, int hkv, long long t_seq, int dim)
{
    if (batch < 0 || hq < 1 || hkv < 1 || t_seq < 0 || dim < 1)
        return 1;
    if (hq % hkv != 0)
        return 1;
    if (dim % 4 != 0 || dim > ORACLE_MAX_DIM)
        return 1;
    return 0;
}

/*
 * Contiguous cache. q [B,Hq,D], k/v [B,Hkv,T,D], lens [B] or NULL,
 * out [B,Hq,D] (fully written). reference: src/attention.cu:1318-1373.
 */
int oracle_attention_decode(const float *q, const float *k, const float *v,
                            const int *lens, float *out, int batch, int hq,
                            int hkv, int t_seq, int dim)
{
    if (oracle_check(batch, hq, hkv, t_seq, dim))
        return 1;
    if (lens)
        for (int i = 0; i < batch; ++i)
            if (lens[i] < 0 || lens[i] > t_seq)
                return 1; /* src/attention.cu:1331-1336 */

    const int group = hq / hkv;
    const float scale = 1.0f / sqrtf((float)dim);
    memset(out, 0, (size_t)batch * hq * dim * sizeof(float));
    float *scores = (float *)malloc(sizeof(float) * (size_t)(t_seq > 0 ? t_seq : 1));
    if (!scores)
        return 1;
    for (int bi = 0; bi < batch; ++bi) {
        const int len = lens ? lens[bi] : t_seq;
        if (len == 0)
            continue; /* zero-row convention, src/attention.cu:1345-1346 */
        for (int h = 0; h < hq; ++h) {
            const int kv = h / group;
            const float *qp = q + ((size_t)bi * hq + h) * dim;
            const float *kp = k + (((size_t)bi * hkv + kv) * t_seq) * dim;
            const float *vp = v + (((size_t)bi * hkv + kv) * t_seq) * dim;
            float m = -INFINITY;
            for (int t = 0; t < len; ++t) {
                float dot = 0.0f;
                for (int d = 0; d < dim; ++d)
                    dot += qp[d] * kp[(size_t)t * dim + d];
                scores[t] = dot * scale;
                m = fmaxf(m, scores[t]);
            }
            float l = 0.0f;
            for (int t = 0; t < len; ++t)
                l += expf(scores[t] - m);
            float *op = out + ((size_t)bi * hq + h) * dim;
            for (int t = 0; t < len; ++t) {
                const float p = expf(scores[t] - m) / l;
                for (int d = 0; d < dim; ++d)
                    op[d] += p * vp[(size_t)t * dim + d];
            }
        }
    }
    free(scores);
    return 0;
}

/*
 * Paged cache. pools [Nb,Hkv,P,D], table [B,S] block ids, lens [B] or NULL
 * (NULL = S*P rows). Token t of sequence b lives at
 * pool[table[b][t / P]][kv][t % P][:]. Every table entry that a sequence
 * actually uses is validated against [0, Nb). reference:
 * src/attention.cu:1382-1456.
 */
int oracle_attention_decode_paged(const float *q, const float *k_pool,
                                  const float *v_pool, const int *table,
                                  const int *lens, float *out, int batch,
                                  int hq, int hkv, int page, int tbl_width,
                                  int num_blocks, int dim)
{
    if (oracle_check(batch, hq, hkv, (long long)tbl_width * page, dim))
        return 1;
    if (page < 1)
        return 1;
    const int span = tbl_width * page;
    if (lens)
        for (int i = 0; i < batch; ++i)
            if (lens[i] < 0 || lens[i] > span)
                return 1;
    for (int bi = 0; bi < batch; ++bi) {
        const int used = lens ? lens[bi] : span;
        const int pages = (used + page - 1) / page;
        for (int s = 0; s < pages; ++s) {
            const int blk = table[(size_t)bi * tbl_width + s];
            if (blk < 0 || blk >= num_blocks)
                return 1; /* src/attention.cu:1405-1414 */
        }
    }

    const int group = hq / hkv;
    const float scale = 1.0f / sqrtf((float)dim);
    memset(out, 0, (size_t)batch * hq * dim * sizeof(float));
    float *scores = (float *)malloc(sizeof(float) * (size_t)(span > 0 ? span : 1));
    if (!scores)
        return 1;
    for (int bi = 0; bi < batch; ++bi) {
        const int len = lens ? lens[bi] : span;
        if (len == 0)
            continue;
        const int *row_t = table + (size_t)bi * tbl_width;
        for (int h = 0; h < hq; ++h) {
            const int kv = h / group;
            const float *qp = q + ((size_t)bi * hq + h) * dim;
            float m = -INFINITY;
            for (int t = 0; t < len; ++t) {
                const size_t base =
                    ((size_t)row_t[t / page] * hkv + kv) * page + (t % page);
                const float *kp = k_pool + base * dim;
                float dot = 0.0f;
                for (int d = 0; d < dim; ++d)
                    dot += qp[d] * kp[d];
                scores[t] = dot * scale;
                m = fmaxf(m, scores[t]);
            }
            float l = 0.0f;
            for (int t = 0; t < len; ++t)
                l += expf(scores[t] - m);
            float *op = out + ((size_t)bi * hq + h) * dim;
            for (int t = 0; t < len; ++t) {
                const size_t base =
                    ((size_t)row_t[t / page] * hkv + kv) * page + (t % page);
                const float *vp = v_pool + base * dim;
                const float p = expf(scores[t] - m) / l;
                for (int d = 0; d < dim; ++d)
                    op[d] += p * vp[d];
            }
        }
    }
    free(scores);
    return 0;
}

/*
 * Split-KV algebra used by the multi-GPU layer, restated on the CPU so the
 * merge rule can be checked without a GPU. A partial over rows [t0, t1) of
 * one (b, h) is the triple (m, l, acc[D]) with m = max score, l = sum
 * exp(s - m), acc = sum exp(s - m) * V (unnormalised). reference: the
 * workspace triple written at src/attention.cu:434-463.
 */
int oracle_attention_partial(const float *q, const float *k, const float *v,
                             float *m_out, float *l_out, float *acc, int t0,
                             int t1, int dim)
{
    const float scale = 1.0f / sqrtf((float)dim);
    float m = -INFINITY, l = 0.0f;
    for (int d = 0; d < dim; ++d)
        acc[d] = 0.0f;
    for (int t = t0; t < t1; ++t) {
        float dot = 0.0f;
        for (int d = 0; d < dim; ++d)
            dot += q[d] * k[(size_t)t * dim + d];
        const float s = dot * scale;
        const float m_new = fmaxf(m, s);
        const float r = expf(m - m_new), p = expf(s - m_new);
        l = l * r + p;
        for (int d = 0; d < dim; ++d)
            acc[d] = acc[d] * r + p * v[(size_t)t * dim + d];
        m = m_new;
    }
    *m_out = m;
    *l_out = l;
    return 0;
}

/*
 * Merge n partial triples of one (b, h) into the normalised output row.
 * Rule (reference: attn_reduce_kernel, src/attention.cu:503-548): skip
 * partials with l <= 0, adopt the first live one verbatim, fold later ones
 * with the max-rescale rule, divide by l; all-empty gives a zero row.
 * ml is [n][2] = (m, l); acc is [n][dim].
 */
int oracle_attention_merge(const float *ml, const float *acc, int n, int dim,
                           float *out)
{
    float m = -INFINITY, l = 0.0f;
    for (int d = 0; d < dim; ++d)
        out[d] = 0.0f;
    for (int s = 0; s < n; ++s) {
        const float ms = ml[2 * s], ls = ml[2 * s + 1];
        if (ls <= 0.0f)
            continue;
        const float *a = acc + (size_t)s * dim;
        if (l == 0.0f) {
            m = ms;
            l = ls;
            for (int d = 0; d < dim; ++d)
                out[d] = a[d];
            continue;
        }
        const float m_new = fmaxf(m, ms);
        const float r_old = expf(m - m_new), r_new = expf(ms - m_new);
        l = l * r_old + ls * r_new;
        for (int d = 0; d < dim; ++d)
            out[d] = out[d] * r_old + a[d] * r_new;
        m = m_new;
    }
    if (l <= 0.0f) {
        for (int d = 0; d < dim; ++d)
            out[d] = 0.0f;
        return 0;
    }
    for (int d = 0; d < dim; ++d)
        out[d] = out[d] / l;
    return 0;
}

/*
 * kv-cache append, contiguous: one fresh token's K and V rows per sequence are
 * copied to cache row lens[b]. reference: kv_append_cpu,
 * src/attention.cu:2064-2099. Caches [B,Hkv,T,D] are updated in place.
 */
int oracle_kv_append(const float *k_new, const float *v_new, const int *lens,
                     float *k_cache, float *v_cache, int batch, int hkv,
                     int dim, int t_rows)
{
    if (dim % 4 != 0)
        return 1;
    for (int bi = 0; bi < batch; ++bi)
        if (lens[bi] < 0 || lens[bi] >= t_rows)
            return 1;
    for (int bi = 0; bi < batch; ++bi) {
        const int pos = lens[bi];
        for (int h = 0; h < hkv; ++h) {
            const size_t dst = (((size_t)bi * hkv + h) * t_rows + pos) * dim;
            const size_t src = ((size_t)bi * hkv + h) * dim;
            memcpy(k_cache + dst, k_new + src, sizeof(float) * dim);
            memcpy(v_cache + dst, v_new + src, sizeof(float) * dim);
        }
    }
    return 0;
}

/*
 * kv-cache append, paged: rows land in pool block table[b][lens[b] / P] at
 * offset lens[b] % P. reference: kv_append_paged_cpu,
 * src/attention.cu:2037-2062 (lens in [0, S*P), used block ids in [0, Nb)).
 */
int oracle_kv_append_paged(const float *k_new, const float *v_new,
                           const int *table, const int *lens, float *k_pool,
                           float *v_pool, int batch, int hkv, int dim,
                           int page, int tbl_width, int num_blocks)
{
    if (dim % 4 != 0 || page < 1)
        return 1;
    for (int bi = 0; bi < batch; ++bi) {
        const int pos = lens[bi];
        if (pos < 0 || pos >= tbl_width * page)
            return 1;
        const int blk = table[(size_t)bi * tbl_width + pos / page];
        if (blk < 0 || blk >= num_blocks)
            return 1;
    }
    for (int bi = 0; bi < batch; ++bi) {
        const int pos = lens[bi];
        const int blk = table[(size_t)bi * tbl_width + pos / page];
        const int off = pos % page;
        for (int h = 0; h < hkv; ++h) {
            const size_t dst = (((size_t)blk * hkv + h) * page + off) * dim;
            const size_t src = ((size_t)bi * hkv + h) * dim;
            memcpy(k_pool + dst, k_new + src, sizeof(float) * dim);
            memcpy(v_pool + dst, v_new + src, sizeof(float) * dim);
        }
    }
    return 0;
}

/*
 * Prefill (fresh-sequence self-attention over S query rows), restating
 * attention_prefill_cpu (reference: src/attention.cu:1591-1638).
 * q / out [B, Hq, S, D]; k / v [B, Hkv, S, D]. Query row i attends key rows
 * [0, i] when causal, all S rows otherwise. Per row the same three passes as
 * decode: scores and max, sum of expf, then out += (expf(s - m) / l) * V[t].
 */
int oracle_attention_prefill(const float *q, const float *k, const float *v,
                             float *out, int batch, int hq, int hkv, int seq,
                             int dim, int causal)
{
    if (oracle_check(batch, hq, hkv, seq, dim))
        return 1;
    const int group = hq / hkv;
    const float scale = 1.0f / sqrtf((float)dim);
    const size_t qn = (size_t)batch * hq * seq * dim;
    memset(out, 0, qn * sizeof(float));
    float *scores = (float *)malloc(sizeof(float) * (seq > 0 ? seq : 1));
    if (!scores)
        return 2;
    for (int bi = 0; bi < batch; ++bi)
        for (int h = 0; h < hq; ++h) {
            const int kv = h / group;
            const float *qp = q + (((size_t)bi * hq + h) * seq) * dim;
            const float *kp = k + (((size_t)bi * hkv + kv) * seq) * dim;
            const float *vp = v + (((size_t)bi * hkv + kv) * seq) * dim;
            for (int i = 0; i < seq; ++i) {
                const int lim = causal ? i + 1 : seq;
                const float *qr = qp + (size_t)i * dim;
                float m = -INFINITY;
                for (int t = 0; t < lim; ++t) {
                    float dot = 0.0f;
                    for (int d = 0; d < dim; ++d)
                        dot += qr[d] * kp[(size_t)t * dim + d];
                    scores[t] = dot * scale;
                    m = fmaxf(m, scores[t]);
                }
                float l = 0.0f;
                for (int t = 0; t < lim; ++t)
                    l += expf(scores[t] - m);
                float *op = out + (((size_t)bi * hq + h) * seq + i) * dim;
                for (int t = 0; t < lim; ++t) {
                    const float p = expf(scores[t] - m) / l;
                    for (int d = 0; d < dim; ++d)
                        op[d] += p * vp[(size_t)t * dim + d];
                }
            }
        }
    free(scores);
    return 0;
}

/*
 * Rotary position embedding on one [seq, dim] matrix, restating rope_cpu /
 * rope_neox_cpu (reference: src/rope.cu:95-146). Row r has absolute position
 * m = r + pos_offset; pair j is rotated by angle m * theta^(-2j/dim), computed
 * in double like the reference. neox == 0: pairs (2j, 2j+1); neox != 0: pairs
 * (j, j + dim/2).
 */
int oracle_rope(const float *x, float *y, int seq, int dim, float theta,
                int pos_offset, int neox)
{
    if (seq < 0 || dim <= 0 || dim % 2 != 0 || pos_offset < 0)
        return 1;
    for (int r = 0; r < seq; ++r) {
        const int m = r + pos_offset;
        for (int j = 0; j < dim / 2; ++j) {
            const double angle = m * pow((double)theta, -2.0 * j / dim);
            const double c = cos(angle), s = sin(angle);
            const size_t a = neox ? (size_t)r * dim + j : (size_t)r * dim + 2 * j;
            const size_t b = neox ? a + dim / 2 : a + 1;
            const float xa = x[a], xb = x[b];
            y[a] = (float)(xa * c - xb * s);
            y[b] = (float)(xa * s + xb * c);
        }
    }
    return 0;
}
