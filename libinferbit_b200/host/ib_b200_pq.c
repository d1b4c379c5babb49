/*
 * ib_pq_matmul_fp32-shaped and ib_kmeans_assign-shaped entry points over the CUDA backend.
 * Host pointers in, host pointers out; the heavy arrays (PQ codes, k-means points) are copied to
 * HBM once and reused, the small ones (activations, centroids, results) move per call.
 */
#include "ib_b200_internal.h"
#include <stdlib.h>
#include <string.h>

/* ── PQ tensors cached on the device, keyed by the address of the caller's struct ── */
#define PQ_CACHE 64
typedef struct {
    const ib_b200_pq_tensor* key;
    ibcu_pq_t dev;
    void* bufs[13];
} pq_entry;
static pq_entry g_pq[PQ_CACHE];
static int g_npq;

static void pq_drop(pq_entry* e) {
    for (int i = 0; i < 13; i++) if (e->bufs[i]) ibcu_free(g_ib.ctx, e->bufs[i]);
    memset(e, 0, sizeof *e);
}
void ib_b200_pq_release(const ib_b200_pq_tensor* t) {
    ib_b200_lock();
    for (int i = 0; i < g_npq; i++)
        if (g_pq[i].key == t) { pq_drop(&g_pq[i]); g_pq[i] = g_pq[--g_npq]; memset(&g_pq[g_npq], 0, sizeof g_pq[0]); break; }
    ib_b200_unlock();
}
void ib_b200_pq_release_all(void) {
    for (int i = 0; i < g_npq; i++) pq_drop(&g_pq[i]);
    g_npq = 0;
}

static int up(void** dst, const void* src, size_t bytes) {
    int rc = ibcu_malloc(g_ib.ctx, bytes, dst);
    if (!rc) rc = ibcu_memcpy_h2d(g_ib.ctx, *dst, src, bytes);
    return rc;
}

static pq_entry* pq_get(const ib_b200_pq_tensor* t) {
    for (int i = 0; i < g_npq; i++) if (g_pq[i].key == t) return &g_pq[i];
    if (g_npq == PQ_CACHE) { ib_b200_set_error(IBCU_ERR_NOMEM, "PQ tensor cache full (%d); release some with ib_b200_pq_release", PQ_CACHE); return NULL; }
    /* what the backend takes: one or two levels (second level: at most 256 entries, one-byte or 4-bit packed indices), an
     * optional int8 outlier sidecar; anything else (uint16 second-level indices, other formats) stays with the caller */
    const int two = t->n_levels == 2;
    const int K2 = two ? (t->K_l2 > 0 ? t->K_l2 : t->K) : 0;                 /* src/pq_decode.c:1099-1101 */
    const int l2_bytes = t->l2_idx_bytes > 0 ? t->l2_idx_bytes : 1;
    if ((t->n_levels != 1 && t->n_levels != 2) || t->n_outlier < 0 || t->n_outlier >= t->N || t->G <= 0 || (t->G & 1) ||
        (t->N - t->n_outlier) % t->G || t->K < 1 || t->K > 256 || t->format < 0 || t->format > 3 ||      /* 4: the pyramid format, other arithmetic */
        !t->codebook_l1_l || !t->codebook_l1_r || !t->indices_l1_l || !t->indices_l1_r || !t->row_scale ||
        (two && (K2 > 256 || (K2 != 16 && l2_bytes != 1) || !t->codebook_l2_l || !t->codebook_l2_r || !t->indices_l2_l || !t->indices_l2_r)) ||
        (t->n_outlier > 0 && (!t->outlier_cols || !t->outlier_sidecar || !t->outlier_scale))) {
        ib_b200_set_error(IBCU_ERR_PARAM, "PQ tensor outside the supported subset (levels=%d K_l2=%d l2 index bytes=%d outliers=%d G=%d K=%d format=%d)",
                          t->n_levels, t->K_l2, t->l2_idx_bytes, t->n_outlier, t->G, t->K, t->format);
        return NULL;
    }
    pq_entry* e = &g_pq[g_npq];
    memset(e, 0, sizeof *e);
    const int C = (t->N - t->n_outlier) / t->G, half = t->G / 2;
    int rc = up(&e->bufs[0], t->codebook_l1_l, (size_t)t->K * half * 2);
    if (!rc) rc = up(&e->bufs[1], t->codebook_l1_r, (size_t)t->K * half * 2);
    if (!rc) rc = up(&e->bufs[2], t->indices_l1_l, (size_t)t->M * C);
    if (!rc) rc = up(&e->bufs[3], t->indices_l1_r, (size_t)t->M * C);
    if (!rc) rc = up(&e->bufs[4], t->row_scale, (size_t)t->M * 2);
    if (!rc && two) {
        const size_t stride = K2 == 16 ? (size_t)(C + 1) / 2 : (size_t)C;
        rc = up(&e->bufs[6], t->codebook_l2_l, (size_t)K2 * half * 2);
        if (!rc) rc = up(&e->bufs[7], t->codebook_l2_r, (size_t)K2 * half * 2);
        if (!rc) rc = up(&e->bufs[8], t->indices_l2_l, (size_t)t->M * stride);
        if (!rc) rc = up(&e->bufs[9], t->indices_l2_r, (size_t)t->M * stride);
    }
    if (!rc && t->n_outlier > 0) {
        rc = up(&e->bufs[10], t->outlier_cols, (size_t)t->n_outlier * sizeof(int32_t));
        if (!rc) rc = up(&e->bufs[11], t->outlier_sidecar, (size_t)t->M * t->n_outlier);
        if (!rc) rc = up(&e->bufs[12], t->outlier_scale, (size_t)t->n_outlier * 2);
    }
    if (!rc) {
        e->dev.M = t->M; e->dev.N = t->N; e->dev.G = t->G; e->dev.K = t->K;
        e->dev.codebook_l = e->bufs[0]; e->dev.codebook_r = e->bufs[1]; e->dev.cb_chunk_stride = 0;
        e->dev.idx_l = e->bufs[2]; e->dev.idx_r = e->bufs[3]; e->dev.row_scale = e->bufs[4];
        e->dev.K_l2 = K2; e->dev.codebook2_l = e->bufs[6]; e->dev.codebook2_r = e->bufs[7]; e->dev.idx2_l = e->bufs[8]; e->dev.idx2_r = e->bufs[9];
        e->dev.n_outlier = t->n_outlier; e->dev.outlier_cols = e->bufs[10]; e->dev.outlier_sidecar = e->bufs[11]; e->dev.outlier_scale = e->bufs[12];
        rc = ibcu_malloc(g_ib.ctx, ibcu_pq_prepared_bytes(&e->dev), &e->bufs[5]);
    }
    if (!rc) rc = ibcu_pq_prepare(g_ib.ctx, &e->dev, (uint8_t*)e->bufs[5]);
    if (!rc) rc = ibcu_sync(g_ib.ctx);
    if (ib_b200_check(rc, "PQ tensor upload")) { pq_drop(e); return NULL; }
    e->key = t;
    g_npq++;
    return e;
}

static int pq_matmul_batch_unlocked(const ib_b200_pq_tensor* t, const float* x, float* out, int B) {
    if (!t || !x || !out || B < 1) return -1;                /* src/pq_decode.c:1506 */
    if (!g_ib.ctx) { ib_b200_set_error(IBCU_ERR_STATE, "ib_b200_pq_matmul_fp32 before ib_b200_init"); return -1; }
    pq_entry* e = pq_get(t);
    if (!e) return -1;
    void *hx, *dx, *ho, *dout;
    const size_t xb = (size_t)B * t->N * sizeof(float), ob = (size_t)B * t->M * sizeof(float);
    if (ib_b200_stage(0, xb, &hx, &dx) || ib_b200_stage(2, ob, &ho, &dout)) return -1;
    memcpy(hx, x, xb);
    int rc = ibcu_memcpy_h2d(g_ib.ctx, dx, hx, xb);
    if (!rc) rc = ibcu_pq_matmul_fp32(g_ib.ctx, &e->dev, (const float*)dx, (float*)dout, B);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, ho, dout, ob);
    if (!rc) rc = ibcu_sync(g_ib.ctx);
    if (ib_b200_check(rc, "ib_b200_pq_matmul_fp32")) return -1;
    memcpy(out, ho, ob);
    return 0;
}
int ib_b200_pq_matmul_fp32_batch(const ib_b200_pq_tensor* t, const float* x, float* out, int B) {
    ib_b200_lock();
    int r = pq_matmul_batch_unlocked(t, x, out, B);
    ib_b200_unlock();
    return r;
}
int ib_b200_pq_matmul_fp32(const ib_b200_pq_tensor* t, const float* x, float* out) { return ib_b200_pq_matmul_fp32_batch(t, x, out, 1); }
int ib_b200_pq_matmul_fp32_threaded(const ib_b200_pq_tensor* t, const float* x, float* out, void* pool) {
    (void)pool;                                              /* the grid is the pool */
    return ib_b200_pq_matmul_fp32_batch(t, x, out, 1);
}
int ib_b200_pq_matmul_fp32_streaming(const ib_b200_pq_tensor* t, const float* x, float* out) { return ib_b200_pq_matmul_fp32_batch(t, x, out, 1); }

static int pq_topk_unlocked(const ib_b200_pq_tensor* t, const float* x, int K_top, float* out_logits, int32_t* out_token_ids) {
    if (!t || !x || !out_logits || !out_token_ids) return -1;            /* src/pq_decode.c:2261-2262 */
    if (K_top <= 0 || K_top > t->M) return -1;
    if (!g_ib.ctx) { ib_b200_set_error(IBCU_ERR_STATE, "ib_b200_pq_lm_head_topk before ib_b200_init"); return -1; }
    pq_entry* e = pq_get(t);
    if (!e) return -1;
    void *hx, *dx, *ho, *dout;
    const size_t xb = (size_t)t->N * sizeof(float), ob = (size_t)K_top * (sizeof(float) + sizeof(int32_t));
    if (ib_b200_stage(0, xb, &hx, &dx) || ib_b200_stage(2, ob, &ho, &dout)) return -1;
    memcpy(hx, x, xb);
    int rc = ibcu_memcpy_h2d(g_ib.ctx, dx, hx, xb);
    if (!rc) rc = ibcu_pq_lm_head_topk(g_ib.ctx, &e->dev, (const float*)dx, K_top, (float*)dout, (int32_t*)((float*)dout + K_top));
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, ho, dout, ob);
    if (!rc) rc = ibcu_sync(g_ib.ctx);
    if (ib_b200_check(rc, "ib_b200_pq_lm_head_topk")) return -1;
    memcpy(out_logits, ho, (size_t)K_top * sizeof(float));
    memcpy(out_token_ids, (const float*)ho + K_top, (size_t)K_top * sizeof(int32_t));
    return 0;
}
int ib_b200_pq_lm_head_topk(const ib_b200_pq_tensor* t, const float* x, int K_top, float* out_logits, int32_t* out_token_ids) {
    ib_b200_lock();
    int r = pq_topk_unlocked(t, x, K_top, out_logits, out_token_ids);
    ib_b200_unlock();
    return r;
}

/* ── k-means ── */
typedef struct { void *X, *C, *idx, *dist, *sums, *counts, *inertia; int owns_X; } km_bufs;

static void km_free(km_bufs* b) {
    if (b->owns_X && b->X) ibcu_free(g_ib.ctx, b->X);
    void* v[] = { b->C, b->idx, b->dist, b->sums, b->counts, b->inertia };
    for (int i = 0; i < 6; i++) if (v[i]) ibcu_free(g_ib.ctx, v[i]);
}

static int km_alloc(km_bufs* b, const float* X, int N, int D, int K) {
    memset(b, 0, sizeof *b);
    const size_t xb = (size_t)N * D * sizeof(float);
    b->X = ib_b200_translate(X, xb);
    int rc = 0;
    if (!b->X) { b->owns_X = 1; rc = ibcu_malloc(g_ib.ctx, xb, &b->X); if (!rc) rc = ibcu_memcpy_h2d(g_ib.ctx, b->X, X, xb); }
    if (!rc) rc = ibcu_malloc(g_ib.ctx, (size_t)K * D * sizeof(float), &b->C);
    if (!rc) rc = ibcu_malloc(g_ib.ctx, (size_t)N * sizeof(int32_t), &b->idx);
    if (!rc) rc = ibcu_malloc(g_ib.ctx, (size_t)N * sizeof(float), &b->dist);
    if (!rc) rc = ibcu_malloc(g_ib.ctx, (size_t)K * D * sizeof(float), &b->sums);
    if (!rc) rc = ibcu_malloc(g_ib.ctx, (size_t)K * sizeof(int32_t), &b->counts);
    if (!rc) rc = ibcu_malloc(g_ib.ctx, 16, &b->inertia);
    return rc;
}

static int ib_b200_kmeans_assign_unlocked(const float* X, int N, int D, const float* centers, int K, int32_t* indices_out, void* pool) {
    (void)pool;
    if (!X || !centers || !indices_out || N <= 0 || K <= 0 || D <= 0) return -1;      /* src/pq_kmeans.c:403 */
    if (!g_ib.ctx) { ib_b200_set_error(IBCU_ERR_STATE, "ib_b200_kmeans_assign before ib_b200_init"); return -1; }
    km_bufs b;
    int rc = km_alloc(&b, X, N, D, K);
    if (!rc) rc = ibcu_memcpy_h2d(g_ib.ctx, b.C, centers, (size_t)K * D * sizeof(float));
    if (!rc) rc = ibcu_kmeans_assign(g_ib.ctx, (const float*)b.X, N, D, (const float*)b.C, K, (int32_t*)b.idx, NULL);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, indices_out, b.idx, (size_t)N * sizeof(int32_t));
    if (!rc) rc = ibcu_sync(g_ib.ctx);
    ib_b200_check(rc, "ib_b200_kmeans_assign");
    km_free(&b);
    return rc ? -1 : 0;
}

static int ib_b200_kmeans_lloyd_unlocked(const float* X, int N, int D, int K, int iters, float tol,
                         float* centers, int32_t* indices_out, double* inertia_out) {
    if (!X || !centers || N <= 0 || K <= 0 || D <= 0 || iters <= 0) return -1;
    if (!g_ib.ctx) { ib_b200_set_error(IBCU_ERR_STATE, "ib_b200_kmeans_lloyd before ib_b200_init"); return -1; }
    km_bufs b;
    int rc = km_alloc(&b, X, N, D, K), done = 0;
    void* shift_d = NULL;
    if (!rc) rc = ibcu_malloc(g_ib.ctx, 16, &shift_d);
    if (!rc) rc = ibcu_memcpy_h2d(g_ib.ctx, b.C, centers, (size_t)K * D * sizeof(float));
    double prev = 0.0, inertia = 0.0;
    for (int it = 0; !rc && it < iters; it++) {
        rc = ibcu_kmeans_assign(g_ib.ctx, (const float*)b.X, N, D, (const float*)b.C, K, (int32_t*)b.idx, (float*)b.dist);
        if (!rc) rc = ibcu_kmeans_accumulate(g_ib.ctx, (const float*)b.X, N, D, K, (const int32_t*)b.idx, (const float*)b.dist,
                                             (float*)b.sums, (int32_t*)b.counts, (double*)b.inertia);
        if (!rc) rc = ibcu_kmeans_update(g_ib.ctx, (float*)b.C, K, D, (const float*)b.sums, (const int32_t*)b.counts, (float*)shift_d);
        done = it + 1;
        if (rc || tol < 0.0f) continue;
        /* the reference's two stopping rules (src/pq_kmeans.c:285-288) need the scalars on the host */
        float shift = 0.0f;
        rc = ibcu_memcpy_d2h(g_ib.ctx, &shift, shift_d, sizeof shift);
        if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, &inertia, b.inertia, sizeof inertia);
        if (!rc) rc = ibcu_sync(g_ib.ctx);
        if (rc) break;
        if (shift < tol) break;
        double diff = prev - inertia; if (diff < 0) diff = -diff;
        if (it > 0 && diff < (double)tol * (prev + 1e-12)) break;
        prev = inertia;
    }
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, centers, b.C, (size_t)K * D * sizeof(float));
    if (!rc && indices_out) rc = ibcu_memcpy_d2h(g_ib.ctx, indices_out, b.idx, (size_t)N * sizeof(int32_t));
    if (!rc && inertia_out) rc = ibcu_memcpy_d2h(g_ib.ctx, inertia_out, b.inertia, sizeof(double));
    if (!rc) rc = ibcu_sync(g_ib.ctx);
    ib_b200_check(rc, "ib_b200_kmeans_lloyd");
    if (shift_d) ibcu_free(g_ib.ctx, shift_d);
    km_free(&b);
    return rc ? -1 : done;
}

int ib_b200_kmeans_assign(const float* X, int N, int D, const float* centers, int K, int32_t* indices_out, void* pool) {
    ib_b200_lock();
    int r = ib_b200_kmeans_assign_unlocked(X, N, D, centers, K, indices_out, pool);
    ib_b200_unlock();
    return r;
}

int ib_b200_kmeans_lloyd(const float* X, int N, int D, int K, int iters, float tol,
                         float* centers, int32_t* indices_out, double* inertia_out) {
    ib_b200_lock();
    int r = ib_b200_kmeans_lloyd_unlocked(X, N, D, K, iters, tol, centers, indices_out, inertia_out);
    ib_b200_unlock();
    return r;
}
