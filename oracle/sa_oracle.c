/*
 * CPU oracle for the decode-attention path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C with double-precision accumulation, the
 * arithmetic that the StreamAttn reference performs on its decode path.  It is
 * the checker that the CUDA kernels are compared against; nothing in the
 * shipped package may call it.  Parity status: PINNED - every function here
 * is compared against outputs of the reference itself (imported as a Python
 * package) and against the reference's own test vectors; the fixtures live in
 * tests/golden/ together with the script that generated them.
 *
 * Reference anchors (paths inside the StreamAttn project):
 *   exact decode      stream_attention/gate1.py:157-183  (dense_attention_forward:
 *                     softmax(q K^T / sqrt(D)) V, GQA map kv_head = head / group)
 *   paged decode      stream_attention/paged.py:201-256  (paged_exact_reference:
 *                     per-page online softmax, page_table indirection, tail clip)
 *   seed block rule   stream_attention/seed_selectors.py:77-104 (policy_seed_blocks)
 *                     == kernel rule kernels/gate0_seed_only_triton.py:64-79
 *   seed token set    stream_attention/seed_selectors.py:107-133 (seed_indices),
 *                     :152-173 (seed_token_indices_from_blocks)
 *   seed-only decode  benchmarks/profile_seed_only_route_bundle_decode.py:450-507
 *                     (softmax restricted to the seed token set)
 *   split-state merge kernels/paged_exact_triton.py:144-186 (exact (m,l,o) merge)
 *
 * All tensors are float32 (callers upcast bf16/fp16 exactly) and addressed by
 * element strides so that BNHD, head-major, NHD and HND layouts share code.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* One query row against a gathered token sequence; returns o[D] and (m,l). */
typedef struct {
    const float *k;      /* base of K for this (batch row, kv head)        */
    const float *v;
    int64_t stride_n;    /* elements between consecutive tokens             */
} kv_row_t;

static void attend_tokens(const float *q, int dim, double scale,
                          const float *k_base, const float *v_base,
                          const int64_t *token_offsets, int64_t num_tokens,
                          double *o_unnorm, double *m_out, double *l_out)
{
    /* Two-pass softmax in double: max, then exp-sum and weighted values. */
    double m = -INFINITY;
    double *scores = (double *)malloc(sizeof(double) * (size_t)(num_tokens > 0 ? num_tokens : 1));
    for (int64_t t = 0; t < num_tokens; ++t) {
        const float *kr = k_base + token_offsets[t];
        double s = 0.0;
        for (int d = 0; d < dim; ++d) s += (double)q[d] * (double)kr[d];
        s *= scale;
        scores[t] = s;
        if (s > m) m = s;
    }
    double l = 0.0;
    for (int d = 0; d < dim; ++d) o_unnorm[d] = 0.0;
    for (int64_t t = 0; t < num_tokens; ++t) {
        double p = exp(scores[t] - m);
        l += p;
        const float *vr = v_base + token_offsets[t];
        for (int d = 0; d < dim; ++d) o_unnorm[d] += p * (double)vr[d];
    }
    free(scores);
    *m_out = m;
    *l_out = l;
}

/*
 * Exact contiguous GQA decode (gate1.py:157-183).  q[B,Hq,D] with strides,
 * k/v addressed as base + b*sb + n*sn + h*sh (D contiguous).  lengths may be
 * NULL (all rows use kv_len); otherwise row b attends tokens [0, lengths[b]).
 * out is [B,Hq,D] contiguous float.  If state != NULL it receives the
 * unnormalised split state [B,Hq,D+2] = (o, m, l) with m in natural-log units
 * of the scaled score.
 */
ORACLE_API int oracle_exact_decode(const float *q, const float *k, const float *v,
                                   float *out, float *state, const int64_t *lengths,
                                   int batch, int q_heads, int kv_heads, int dim, int64_t kv_len,
                                   int64_t q_sb, int64_t q_sh,
                                   int64_t kv_sb, int64_t kv_sn, int64_t kv_sh,
                                   int64_t token_begin, int64_t token_end)
{
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return 1;
    const int group = q_heads / kv_heads;
    const double scale = 1.0 / sqrt((double)dim);
    int err = 0;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < q_heads; ++h) {
            int64_t n = lengths ? lengths[b] : kv_len;
            if (n > kv_len) n = kv_len;
            int64_t lo = token_begin < 0 ? 0 : token_begin;
            int64_t hi = (token_end < 0 || token_end > n) ? n : token_end;
            int64_t cnt = hi > lo ? hi - lo : 0;
            int64_t *offs = (int64_t *)malloc(sizeof(int64_t) * (size_t)(cnt > 0 ? cnt : 1));
            double *o = (double *)malloc(sizeof(double) * (size_t)dim);
            for (int64_t t = 0; t < cnt; ++t) offs[t] = (lo + t) * kv_sn;
            const int kvh = h / group;
            double m, l;
            attend_tokens(q + b * q_sb + h * q_sh, dim, scale,
                          k + b * kv_sb + kvh * kv_sh, v + b * kv_sb + kvh * kv_sh,
                          offs, cnt, o, &m, &l);
            float *orow = out ? out + ((int64_t)b * q_heads + h) * dim : NULL;
            if (orow) {
                for (int d = 0; d < dim; ++d) orow[d] = cnt > 0 ? (float)(o[d] / l) : 0.0f;
            }
            if (state) {
                float *srow = state + ((int64_t)b * q_heads + h) * (dim + 2);
                for (int d = 0; d < dim; ++d) srow[d] = (float)o[d];
                srow[dim] = (float)m;
                srow[dim + 1] = (float)l;
            }
            free(offs);
            free(o);
        }
    }
    return err;
}

/*
 * Paged exact decode (paged.py:201-256).  Pages addressed as
 *   base + page*sp + token_in_page*st + kv_head*sh   (D contiguous)
 * so NHD is (sp, st, sh) = (page*Hkv*D, Hkv*D, D) and HND is (Hkv*page*D, D, page*D).
 * page_table[B,max_pages] (int64 here), lengths[B].  The online softmax is
 * advanced page by page exactly like the reference loop.  If traversal != NULL
 * it receives, for each row, the physical page visited at each logical page
 * ([B,max_pages], untouched slots left as-is): the page-table walk that the
 * CUDA kernel must reproduce bit-exactly.  Returns non-zero on an invalid
 * active page entry (the reference raises ValueError, paged.py:168-182).
 */
ORACLE_API int oracle_paged_decode(const float *q, const float *k_pages, const float *v_pages,
                                   const int64_t *page_table, const int64_t *lengths,
                                   float *out, int64_t *traversal,
                                   int batch, int q_heads, int kv_heads, int dim,
                                   int page_size, int max_pages, int64_t num_pages,
                                   int64_t sp, int64_t st, int64_t sh)
{
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return 1;
    const int group = q_heads / kv_heads;
    const double scale = 1.0 / sqrt((double)dim);
    for (int b = 0; b < batch; ++b) {
        int64_t n = lengths[b];
        if (n <= 0) return 2;
        if (n > (int64_t)max_pages * page_size) return 3;
        int64_t active = (n + page_size - 1) / page_size;
        for (int64_t lp = 0; lp < active; ++lp) {
            int64_t pp = page_table[(int64_t)b * max_pages + lp];
            if (pp < 0 || pp >= num_pages) return 4;
            if (traversal) traversal[(int64_t)b * max_pages + lp] = pp;
        }
    }
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < q_heads; ++h) {
            const int kvh = h / group;
            const float *qr = q + ((int64_t)b * q_heads + h) * dim;
            int64_t n = lengths[b];
            int64_t active = (n + page_size - 1) / page_size;
            double run_max = -INFINITY, den = 0.0;
            double *num = (double *)calloc((size_t)dim, sizeof(double));
            double *scores = (double *)malloc(sizeof(double) * (size_t)page_size);
            for (int64_t lp = 0; lp < active; ++lp) {
                int64_t pp = page_table[(int64_t)b * max_pages + lp];
                int64_t valid = n - lp * page_size;
                if (valid > page_size) valid = page_size;
                const float *kp = k_pages + pp * sp + kvh * sh;
                const float *vp = v_pages + pp * sp + kvh * sh;
                double page_max = -INFINITY;
                for (int64_t t = 0; t < valid; ++t) {
                    double s = 0.0;
                    for (int d = 0; d < dim; ++d) s += (double)kp[t * st + d] * (double)qr[d];
                    s *= scale;
                    scores[t] = s;
                    if (s > page_max) page_max = s;
                }
                double new_max = run_max > page_max ? run_max : page_max;
                double corr = exp(run_max - new_max);
                for (int d = 0; d < dim; ++d) num[d] *= corr;
                den *= corr;
                for (int64_t t = 0; t < valid; ++t) {
                    double p = exp(scores[t] - new_max);
                    den += p;
                    for (int d = 0; d < dim; ++d) num[d] += p * (double)vp[t * st + d];
                }
                run_max = new_max;
            }
            float *orow = out + ((int64_t)b * q_heads + h) * dim;
            for (int d = 0; d < dim; ++d) orow[d] = (float)(num[d] / den);
            free(num);
            free(scores);
        }
    }
    return 0;
}

/*
 * Seed block rule (seed_selectors.py:77-104): sink blocks [0,sink), recent
 * blocks [nb-recent, nb), then middle blocks (sequential: sink+i; otherwise
 * nb-recent-1-i); out-of-range and duplicate blocks dropped, order preserved.
 * block_order: 0 sequential, 1 recent_first, 2 sink_recent_first
 * (decode.py:676-683).  Returns the number of blocks written (<= cap) or -1.
 */
ORACLE_API int oracle_seed_blocks(int64_t seq_len, int block_size, int sink_blocks,
                                  int recent_blocks, int middle_blocks, int block_order,
                                  int64_t *blocks_out, int cap)
{
    if (seq_len <= 0 || block_size <= 0) return -1;
    int64_t nb = (seq_len + block_size - 1) / block_size;
    int64_t recent_start = nb - recent_blocks;
    int total = sink_blocks + recent_blocks + middle_blocks;
    int64_t *cand = (int64_t *)malloc(sizeof(int64_t) * (size_t)(total > 0 ? total : 1));
    int c = 0;
    for (int i = 0; i < sink_blocks; ++i) cand[c++] = i;
    for (int64_t blk = recent_start; blk < nb; ++blk) cand[c++] = blk;
    for (int i = 0; i < middle_blocks; ++i)
        cand[c++] = block_order == 0 ? (int64_t)sink_blocks + i : recent_start - 1 - i;
    int n = 0;
    for (int i = 0; i < c; ++i) {
        int64_t blk = cand[i];
        if (blk < 0 || blk >= nb) continue;
        int dup = 0;
        for (int j = 0; j < n; ++j) if (blocks_out[j] == blk) { dup = 1; break; }
        if (dup) continue;
        if (n >= cap) { free(cand); return -1; }
        blocks_out[n++] = blk;
    }
    free(cand);
    return n;
}

static int cmp_i64(const void *a, const void *b)
{
    int64_t x = *(const int64_t *)a, y = *(const int64_t *)b;
    return (x > y) - (x < y);
}

/*
 * Token set of a block list (seed_selectors.py:152-173): tokens
 * block*bs + [0,bs) clipped to seq_len, blocks starting past seq_len skipped,
 * duplicates removed, ascending.  Returns the count (<= cap) or -1.
 */
ORACLE_API int64_t oracle_seed_tokens_from_blocks(int64_t seq_len, int block_size,
                                                  const int64_t *blocks, int num_blocks,
                                                  int64_t *tokens_out, int64_t cap)
{
    int64_t n = 0;
    for (int i = 0; i < num_blocks; ++i) {
        int64_t start = blocks[i] * block_size;
        if (blocks[i] < 0 || start >= seq_len) continue;
        int64_t end = start + block_size;
        if (end > seq_len) end = seq_len;
        for (int64_t t = start; t < end; ++t) {
            if (n >= cap) return -1;
            tokens_out[n++] = t;
        }
    }
    qsort(tokens_out, (size_t)n, sizeof(int64_t), cmp_i64);
    int64_t w = 0;
    for (int64_t i = 0; i < n; ++i)
        if (w == 0 || tokens_out[w - 1] != tokens_out[i]) tokens_out[w++] = tokens_out[i];
    return w;
}

/*
 * Seed-only decode over an explicit token index set
 * (profile_seed_only_route_bundle_decode.py:450-507): exact softmax attention
 * restricted to `tokens` (shared by every row and head).
 */
ORACLE_API int oracle_seed_decode(const float *q, const float *k, const float *v, float *out,
                                  const int64_t *tokens, int64_t num_tokens,
                                  int batch, int q_heads, int kv_heads, int dim,
                                  int64_t q_sb, int64_t q_sh,
                                  int64_t kv_sb, int64_t kv_sn, int64_t kv_sh)
{
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return 1;
    const int group = q_heads / kv_heads;
    const double scale = 1.0 / sqrt((double)dim);
    int64_t *offs = (int64_t *)malloc(sizeof(int64_t) * (size_t)(num_tokens > 0 ? num_tokens : 1));
    for (int64_t t = 0; t < num_tokens; ++t) offs[t] = tokens[t] * kv_sn;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < q_heads; ++h) {
            double *o = (double *)malloc(sizeof(double) * (size_t)dim);
            const int kvh = h / group;
            double m, l;
            attend_tokens(q + b * q_sb + h * q_sh, dim, scale,
                          k + b * kv_sb + kvh * kv_sh, v + b * kv_sb + kvh * kv_sh,
                          offs, num_tokens, o, &m, &l);
            float *orow = out + ((int64_t)b * q_heads + h) * dim;
            for (int d = 0; d < dim; ++d) orow[d] = num_tokens > 0 ? (float)(o[d] / l) : 0.0f;
            free(o);
        }
    }
    free(offs);
    return 0;
}

/*
 * Exact merge of split states (paged_exact_triton.py:144-186):
 *   m = max_i m_i ; l = sum_i l_i e^{m_i-m} ; o = sum_i o_i e^{m_i-m} / l.
 * states is [parts, rows, D+2] = (o unnormalised, m, l) with m in the units
 * given by log2_domain (0: natural log, 1: base-2).  Parts with l == 0 are empty.
 */
ORACLE_API int oracle_merge_states(const float *states, int parts, int64_t rows, int dim,
                                   int log2_domain, float *out)
{
    for (int64_t r = 0; r < rows; ++r) {
        double m = -INFINITY;
        for (int p = 0; p < parts; ++p) {
            const float *s = states + ((int64_t)p * rows + r) * (dim + 2);
            if (s[dim + 1] > 0.0f && (double)s[dim] > m) m = (double)s[dim];
        }
        double l = 0.0;
        double *acc = (double *)calloc((size_t)dim, sizeof(double));
        for (int p = 0; p < parts; ++p) {
            const float *s = states + ((int64_t)p * rows + r) * (dim + 2);
            if (!(s[dim + 1] > 0.0f)) continue;
            double w = log2_domain ? exp2((double)s[dim] - m) : exp((double)s[dim] - m);
            l += w * (double)s[dim + 1];
            for (int d = 0; d < dim; ++d) acc[d] += w * (double)s[d];
        }
        for (int d = 0; d < dim; ++d) out[r * dim + d] = l > 0.0 ? (float)(acc[d] / l) : 0.0f;
        free(acc);
    }
    return 0;
}

ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
