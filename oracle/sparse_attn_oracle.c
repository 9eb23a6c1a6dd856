/*
 * CPU oracle for the sparse-attention forward.  TEST INFRASTRUCTURE ONLY: the
 * shipped library never links, imports or calls anything in this directory;
 * only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark do.
 *
 * The arithmetic restates ma-transformer's CPU engine,
 * src/csrc/ma_core.cpp:160-246 (compute_sparse_attention), step for step:
 *   scale = 1/sqrt(head_dim)                               (ma_core.cpp:188)
 *   score_j = (sum_d q[d]*k_j[d], sequential in d) * scale (ma_core.cpp:202-209)
 *   m = max_j score_j, left to right                       (ma_core.cpp:216-219)
 *   e_j = exp(score_j - m); s = sum_j e_j, sequential      (ma_core.cpp:222-226)
 *   p_j = e_j / s                                          (ma_core.cpp:229-231)
 *   out[d] = sum_j p_j * v_j[d], sequential in j           (ma_core.cpp:233-240)
 * over the tensor layout [B,S,H,D] with D contiguous
 * (src/csrc/tensor.cpp:104-110).  The reference fixes the key set of row i to
 * [i-w, i+w] (ma_core.cpp:197-198); here the key set comes from a pattern
 * description so that the same arithmetic also covers the causal, dilated,
 * block-sparse and Longformer sets:
 *   window      src/csrc/sparse_attention.cpp:190-197, dilation per
 *               doc/sparse_attention_whitepaper.md:102-105
 *   block       src/csrc/sparse_attention.cpp:209-227 generalised to an
 *               explicit block-CSR layout (the reference's |bi-bj|<=1 layout is
 *               one instance)
 *   longformer  src/csrc/sparse_attention.cpp:241-256, sorted and de-duplicated,
 *               with an arbitrary list of global positions
 *
 * Build with -ffp-contract=off and without -ffast-math so that float sums keep
 * the reference's order and rounding (the reference is built with plain -O3,
 * setup.py:55).  Parity status: pinned.  On the reference's own +-w key set the
 * output is compared bit for bit with the compiled reference engine and with
 * the committed golden vectors (tests/golden).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORACLE_WINDOW = 0, ORACLE_BLOCK = 1, ORACLE_LONGFORMER = 2 };

typedef struct {
    int32_t kind;          /* ORACLE_* */
    int32_t causal;        /* block kind: drop keys behind the query (j > p) */
    int64_t left;          /* taps before the query, in dilation steps */
    int64_t right;         /* taps after the query, in dilation steps */
    int64_t dilation;      /* >= 1 */
    int64_t block;         /* block edge for the block kind */
    int64_t n_qblocks;     /* rows of the block-CSR layout */
    const int32_t *blk_rowptr; /* [n_qblocks+1] */
    const int32_t *blk_colidx; /* key-block ids, any order */
    int64_t n_global;
    const int64_t *global_idx; /* key-coordinate positions, any order */
    int64_t q_offset;      /* key-coordinate position of query row 0 */
} oracle_spec;

static int cmp_i64(const void *a, const void *b) {
    int64_t x = *(const int64_t *)a, y = *(const int64_t *)b;
    return (x > y) - (x < y);
}

static int64_t sort_unique(int64_t *v, int64_t n) {
    if (n <= 1) return n;
    qsort(v, (size_t)n, sizeof(int64_t), cmp_i64);
    int64_t m = 1;
    for (int64_t t = 1; t < n; ++t)
        if (v[t] != v[m - 1]) v[m++] = v[t];
    return m;
}

static int is_global(const oracle_spec *sp, int64_t p) {
    for (int64_t g = 0; g < sp->n_global; ++g)
        if (sp->global_idx[g] == p) return 1;
    return 0;
}

/*
 * Sorted, duplicate-free key positions of query row i (key coordinates
 * p = i + q_offset).  Returns the count, or -(needed) when cap is too small,
 * or INT64_MIN for a malformed description.  out may be NULL to size a buffer.
 */
int64_t oracle_rowset(const oracle_spec *sp, int64_t s_kv, int64_t i,
                      int64_t *out, int64_t cap) {
    const int64_t p = i + sp->q_offset;
    int64_t n = 0;
#define PUSH(j) do { if (out && n < cap) out[n] = (j); ++n; } while (0)
    if (sp->kind == ORACLE_WINDOW ||
        (sp->kind == ORACLE_LONGFORMER && !is_global(sp, p))) {
        const int64_t dil = sp->kind == ORACLE_WINDOW ? sp->dilation : 1;
        if (dil < 1 || sp->left < 0 || sp->right < 0) return INT64_MIN;
        /* clamp the tap range first so that huge windows cost O(S) */
        int64_t k_lo = -sp->left, k_hi = sp->right;
        if (p + k_lo * dil < 0) k_lo = -(p / dil);
        if (p + k_hi * dil >= s_kv) k_hi = (s_kv - 1 - p) / dil;
        for (int64_t t = k_lo; t <= k_hi; ++t) {
            int64_t j = p + t * dil;
            if (j >= 0 && j < s_kv) PUSH(j);
        }
        if (sp->kind == ORACLE_LONGFORMER)
            for (int64_t g = 0; g < sp->n_global; ++g) {
                int64_t j = sp->global_idx[g];
                if (j >= 0 && j < s_kv) PUSH(j);
            }
    } else if (sp->kind == ORACLE_LONGFORMER) {
        for (int64_t j = 0; j < s_kv; ++j) PUSH(j);
    } else if (sp->kind == ORACLE_BLOCK) {
        if (sp->block < 1) return INT64_MIN;
        const int64_t r = p / sp->block;
        if (r < sp->n_qblocks)
            for (int32_t e = sp->blk_rowptr[r]; e < sp->blk_rowptr[r + 1]; ++e) {
                int64_t c = sp->blk_colidx[e];
                int64_t j0 = c * sp->block;
                int64_t j1 = j0 + sp->block < s_kv ? j0 + sp->block : s_kv;
                for (int64_t j = j0; j < j1; ++j)
                    if (!sp->causal || j <= p) PUSH(j);
            }
    } else {
        return INT64_MIN;
    }
#undef PUSH
    if (out == NULL) return n;
    if (n > cap) return -n;
    return sort_unique(out, n);
}

/* Total number of (row, key) pairs over rows [0, s_q): the pattern's nnz. */
int64_t oracle_pattern_nnz(const oracle_spec *sp, int64_t s_q, int64_t s_kv) {
    int64_t *buf = (int64_t *)malloc(sizeof(int64_t) * (size_t)(2 * s_kv + sp->n_global + 8));
    if (!buf) return -1;
    int64_t total = 0;
    for (int64_t i = 0; i < s_q; ++i) {
        int64_t n = oracle_rowset(sp, s_kv, i, buf, 2 * s_kv + sp->n_global + 8);
        if (n < 0) { free(buf); return -1; }
        total += n;
    }
    free(buf);
    return total;
}

/*
 * Forward pass in fp32.  q, o: [B,S_q,H,D] / [B,S_q,H,Dv]; k: [B,S_kv,H,D];
 * v: [B,S_kv,H,Dv].  scale <= 0 selects 1/sqrt(D) as the reference does.
 * A row with an empty key set yields zeros.  nthreads <= 0 uses every core.
 * Returns 0, or -1 on a malformed description / allocation failure.
 */
int oracle_sparse_attn_fwd_f32(const float *q, const float *k, const float *v, float *o,
                               int64_t B, int64_t S_q, int64_t S_kv, int64_t H,
                               int64_t D, int64_t Dv, const oracle_spec *sp,
                               float scale, int nthreads) {
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)D);
    const int64_t cap = 2 * S_kv + sp->n_global + 8;
    int failed = 0;
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
    nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
    {
        int64_t *keys = (int64_t *)malloc(sizeof(int64_t) * (size_t)cap);
        float *sc = (float *)malloc(sizeof(float) * (size_t)cap);
        if (!keys || !sc) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for collapse(2) schedule(dynamic, 16)
        for (int64_t b = 0; b < B; ++b)
            for (int64_t i = 0; i < S_q; ++i) {
                if (!keys || !sc) continue;
                int64_t n = oracle_rowset(sp, S_kv, i, keys, cap);
                if (n < 0) {
#pragma omp atomic write
                    failed = 1;
                    continue;
                }
                for (int64_t h = 0; h < H; ++h) {
                    const float *qr = q + ((b * S_q + i) * H + h) * D;
                    float *orow = o + ((b * S_q + i) * H + h) * Dv;
                    if (n == 0) { memset(orow, 0, sizeof(float) * (size_t)Dv); continue; }
                    for (int64_t t = 0; t < n; ++t) {
                        const float *kr = k + ((b * S_kv + keys[t]) * H + h) * D;
                        float s = 0.0f;
                        for (int64_t d = 0; d < D; ++d) s += qr[d] * kr[d];
                        sc[t] = s * scale;
                    }
                    float m = sc[0];
                    for (int64_t t = 1; t < n; ++t) m = sc[t] > m ? sc[t] : m;
                    float sum = 0.0f;
                    for (int64_t t = 0; t < n; ++t) { sc[t] = expf(sc[t] - m); sum += sc[t]; }
                    for (int64_t t = 0; t < n; ++t) sc[t] /= sum;
                    for (int64_t d = 0; d < Dv; ++d) {
                        float acc = 0.0f;
                        for (int64_t t = 0; t < n; ++t)
                            acc += sc[t] * v[((b * S_kv + keys[t]) * H + h) * Dv + d];
                        orow[d] = acc;
                    }
                }
            }
        free(keys);
        free(sc);
    }
    return failed ? -1 : 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
