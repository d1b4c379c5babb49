/*
 * Decode step over a model resident in HBM: the launch sequence of forward_single_ex /
 * forward_batch (src/forward.c:518-664, :682-846) with FP32 activations (IB_W4A8=0) and an FP32
 * KV cache, issued through the CUDA backend and replayed as a CUDA graph. The position of the step
 * lives in device memory (the attention kernels read it there), so one captured graph per batch size
 * serves every position: autoregressive decoding replays, it does not re-capture.
 *
 * With a communicator on the context every linear layer holds only this rank's contiguous slice of
 * output rows (the reference's own unit of parallelism, src/threading.c:220-241); each rank computes
 * its slice into the full-size activation buffer and the slices are all-gathered, so all ranks hold
 * identical activations and run the small element-wise work redundantly.
 */
#include "ib_b200_internal.h"
#include <stdlib.h>
#include <string.h>

#define ROW_ALIGN 32          /* shard boundaries in units of the kernel's row block */
#define MAX_GRAPHS 8

typedef struct {
    void* w; void* scale;     /* this rank's rows */
    int M, N, bits;           /* full shape */
    int row0, rows;           /* this rank's slice */
} lin;

typedef struct { lin t[7]; void *in_norm, *post_norm, *k_cache, *v_cache; } layer;

struct ib_b200_model {
    ibcu_ctx* ctx;
    ib_b200_model_cfg c;
    int rank, world;
    layer* L;
    lin head;
    void *embed, *embed_scale, *final_norm;
    int embed_bits;           /* 8 (INT8 rows, fp16 row scales), 4 (nibbles, fp16 row scales) or 16 (fp16 rows) */
    /* activations, all [IB max batch][...] */
    float *x, *xb, *q, *k, *v, *att, *hg, *hu, *logits;
    float* amax;              /* [BMAX][AMAX_PARTS] pieces of max|silu(gate)*up| per position */
    int32_t* tokens;
    int32_t* pos_dev;         /* position of the first token of the step, read by the attention kernels */
    void* pin;                /* pinned staging for tokens / logits */
    size_t pin_bytes;
    struct { int B, last_only, id; } graphs[MAX_GRAPHS];
    int n_graphs;
    int use_graph;            /* 1: replay a captured graph per batch size (default); 0: issue the launches one by one */
    int dyn_pos;              /* 1: the attention shape allows the position-independent launch */
    size_t weight_bytes;
};

#define BMAX 32
#define AMAX_PARTS 28

static int dmalloc(ib_b200_model* m, void** p, size_t bytes) { return ibcu_malloc(m->ctx, bytes ? bytes : 16, p); }
/* activations that are all-gathered live in the peer window when the context has one (same order, hence same
 * offsets, on every rank), so that the gather is a push over NVLink; elsewhere ordinary device memory */
static int amalloc(ib_b200_model* m, void** p, size_t bytes) {
    if (m->world > 1 && ibcu_window_alloc(m->ctx, bytes ? bytes : 16, p) == 0) return 0;
    return dmalloc(m, p, bytes);
}

static int lin_alloc(ib_b200_model* m, lin* t, int M, int N, int bits) {
    t->M = M; t->N = N; t->bits = bits;
    ibcu_shard_rows(M, m->world, m->rank, ROW_ALIGN, &t->row0, &t->rows);
    const size_t rb = bits == 8 ? (size_t)N : (size_t)N / 2;
    int rc = dmalloc(m, &t->w, (size_t)t->rows * rb);
    if (!rc) rc = dmalloc(m, &t->scale, (size_t)t->rows * 2);
    m->weight_bytes += (size_t)t->rows * rb + (size_t)t->rows * 2;
    return rc;
}

static int bits_ok(int b) { return b == 4 || b == 8; }

ib_b200_model* ib_b200_model_create_bits(ibcu_ctx* ctx, const ib_b200_model_cfg* cfg, const int* linear_bits, int embed_bits) {
    if (!ctx || !cfg) return NULL;
    const ib_b200_model_cfg c = *cfg;
    if (c.hidden <= 0 || c.inter <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 ||
        c.vocab <= 0 || c.max_ctx <= 0 || c.n_heads % c.n_kv_heads || c.hidden != c.n_heads * c.head_dim ||
        !bits_ok(c.attn_bits) || !bits_ok(c.mlp_bits) || !bits_ok(c.head_bits))
        return NULL;
    if (embed_bits != 8 && embed_bits != 4 && embed_bits != 16) return NULL;
    if (linear_bits) for (int i = 0; i < c.n_layers * 7 + 1; i++) if (!bits_ok(linear_bits[i])) return NULL;
    ib_b200_model* m = (ib_b200_model*)calloc(1, sizeof *m);
    if (!m) return NULL;
    m->ctx = ctx; m->c = c; m->embed_bits = embed_bits;
    ibcu_comm_rank(ctx, &m->rank, &m->world);
    m->L = (layer*)calloc((size_t)c.n_layers, sizeof(layer));
    if (!m->L) { free(m); return NULL; }
    const int H = c.hidden, I = c.inter, kv = c.n_kv_heads * c.head_dim;
    int rc = 0;
    for (int l = 0; l < c.n_layers && !rc; l++) {
        layer* y = &m->L[l];
        const int Ms[7] = { H, kv, kv, H, I, I, H }, Ns[7] = { H, H, H, H, H, H, I };
        for (int i = 0; i < 7 && !rc; i++)
            rc = lin_alloc(m, &y->t[i], Ms[i], Ns[i], linear_bits ? linear_bits[l * 7 + i] : (i <= IB_B200_O ? c.attn_bits : c.mlp_bits));
        if (!rc) rc = dmalloc(m, &y->in_norm, (size_t)H * 2);
        if (!rc) rc = dmalloc(m, &y->post_norm, (size_t)H * 2);
        if (!rc) rc = dmalloc(m, &y->k_cache, (size_t)c.max_ctx * kv * sizeof(float));
        if (!rc) rc = dmalloc(m, &y->v_cache, (size_t)c.max_ctx * kv * sizeof(float));
    }
    if (!rc) rc = lin_alloc(m, &m->head, c.vocab, H, linear_bits ? linear_bits[c.n_layers * 7] : c.head_bits);
    if (!rc) rc = dmalloc(m, &m->embed, embed_bits == 16 ? (size_t)c.vocab * H * 2 : (embed_bits == 8 ? (size_t)c.vocab * H : (size_t)c.vocab * H / 2));
    if (!rc) rc = dmalloc(m, &m->embed_scale, (size_t)c.vocab * 2);
    if (!rc) rc = dmalloc(m, &m->final_norm, (size_t)H * 2);
    void** act[] = { (void**)&m->x, (void**)&m->xb, (void**)&m->q, (void**)&m->k, (void**)&m->v, (void**)&m->att, (void**)&m->hg, (void**)&m->hu, (void**)&m->logits };
    const size_t asz[] = { (size_t)H, (size_t)H, (size_t)H, (size_t)kv, (size_t)kv, (size_t)H, (size_t)I, (size_t)I, (size_t)c.vocab };
    for (int i = 0; i < 9 && !rc; i++) rc = amalloc(m, act[i], asz[i] * BMAX * sizeof(float));
    if (!rc) rc = dmalloc(m, (void**)&m->tokens, BMAX * sizeof(int32_t));
    if (!rc) rc = dmalloc(m, (void**)&m->pos_dev, 16);
    m->use_graph = 1;
    m->dyn_pos = c.n_heads / c.n_kv_heads <= 8 && c.head_dim % 4 == 0 && c.head_dim <= 256;
    if (!rc) rc = dmalloc(m, (void**)&m->amax, (size_t)BMAX * AMAX_PARTS * sizeof(float));
    m->pin_bytes = (size_t)BMAX * c.vocab * sizeof(float) + 256;
    if (!rc) rc = ibcu_host_alloc(ctx, m->pin_bytes, &m->pin);
    if (rc) { ib_b200_model_free(m); return NULL; }
    return m;
}

ib_b200_model* ib_b200_model_create(ibcu_ctx* ctx, const ib_b200_model_cfg* cfg) {
    return ib_b200_model_create_bits(ctx, cfg, NULL, 8);
}

void ib_b200_model_free(ib_b200_model* m) {
    if (!m) return;
    ibcu_sync(m->ctx);
    for (int g = 0; g < m->n_graphs; g++) ibcu_graph_destroy(m->ctx, m->graphs[g].id);
    for (int l = 0; m->L && l < m->c.n_layers; l++) {
        layer* y = &m->L[l];
        for (int i = 0; i < 7; i++) { ibcu_free(m->ctx, y->t[i].w); ibcu_free(m->ctx, y->t[i].scale); }
        ibcu_free(m->ctx, y->in_norm); ibcu_free(m->ctx, y->post_norm); ibcu_free(m->ctx, y->k_cache); ibcu_free(m->ctx, y->v_cache);
    }
    ibcu_free(m->ctx, m->head.w); ibcu_free(m->ctx, m->head.scale);
    void* v[] = { m->embed, m->embed_scale, m->final_norm, m->x, m->xb, m->q, m->k, m->v, m->att, m->hg, m->hu, m->logits, m->tokens, m->amax, m->pos_dev };
    for (unsigned i = 0; i < sizeof v / sizeof *v; i++) ibcu_free(m->ctx, v[i]);
    if (m->pin) ibcu_host_free(m->ctx, m->pin);
    free(m->L);
    free(m);
}

size_t ib_b200_model_weight_bytes(const ib_b200_model* m) { return m ? m->weight_bytes : 0; }
void*  ib_b200_model_tokens(ib_b200_model* m) { return m ? m->tokens : NULL; }
float* ib_b200_model_logits(ib_b200_model* m) { return m ? m->logits : NULL; }
void   ib_b200_model_use_graph(ib_b200_model* m, int on) { if (m) m->use_graph = on ? 1 : 0; }

static lin* pick(ib_b200_model* m, int layer_i, int which) {
    if (which == IB_B200_HEAD) return &m->head;
    if (which < 0 || which > IB_B200_DOWN || layer_i < 0 || layer_i >= m->c.n_layers) return NULL;
    return &m->L[layer_i].t[which];
}

/* Every tensor is a function of (seed, its place in the model) alone and a rank fills its rows with the bytes
 * the whole tensor has at those rows: the model is the same model however many ranks hold it. */
int ib_b200_model_fill_random(ib_b200_model* m, uint64_t seed, int kv_fill) {
    if (!m || kv_fill < 0 || kv_fill > m->c.max_ctx) return IBCU_ERR_PARAM;
    const ib_b200_model_cfg* c = &m->c;
    const int H = c->hidden, kv = c->n_kv_heads * c->head_dim;
    int rc = 0;
    uint64_t s = seed * 1000003ull;
    for (int l = 0; l <= c->n_layers && !rc; l++) {
        const int nt = l < c->n_layers ? 7 : 1;
        for (int i = 0; i < nt && !rc; i++) {
            lin* t = l < c->n_layers ? &m->L[l].t[i] : &m->head;
            const size_t rb = t->bits == 8 ? (size_t)t->N : (size_t)t->N / 2;
            rc = ibcu_fill_hash_bytes_at(m->ctx, t->w, (size_t)t->rows * rb, ++s, (size_t)t->row0 * rb);
            /* per-row scales drawn uniformly from a range twenty times below the benchmark's U[0.001, 0.01]
             * (INT8) / U[0.002, 0.02] (INT4), so that 32 random layers keep the residual stream of order
             * one; the bytes streamed and the arithmetic are the same */
            const float lo = t->bits == 8 ? 0.001f : 0.002f;
            if (!rc) rc = ibcu_fill_hash_fp16_uniform_at(m->ctx, t->scale, (size_t)t->rows, ++s, lo * 0.05f, lo * 0.5f, (size_t)t->row0);
        }
        if (l < c->n_layers && !rc) {
            layer* y = &m->L[l];
            uint64_t ls = seed * 7919ull + (uint64_t)l * 131;
            rc = ibcu_fill_hash_fp16_uniform(m->ctx, y->in_norm, (size_t)H, ls + 1, 0.9f, 1.1f);
            if (!rc) rc = ibcu_fill_hash_fp16_uniform(m->ctx, y->post_norm, (size_t)H, ls + 2, 0.9f, 1.1f);
            /* earlier positions of the KV cache: bell-shaped values of unit variance */
            if (!rc && kv_fill) rc = ibcu_fill_hash_f32_normal_at(m->ctx, (float*)y->k_cache, (size_t)kv_fill * kv, ls + 3, 0.0f, 1.0f, 0);
            if (!rc && kv_fill) rc = ibcu_fill_hash_f32_normal_at(m->ctx, (float*)y->v_cache, (size_t)kv_fill * kv, ls + 4, 0.0f, 1.0f, 0);
        }
    }
    uint64_t es = seed * 104729ull;
    const size_t eb = m->embed_bits == 16 ? (size_t)c->vocab * H * 2 : (m->embed_bits == 8 ? (size_t)c->vocab * H : (size_t)c->vocab * H / 2);
    if (!rc) rc = ibcu_fill_hash_bytes(m->ctx, m->embed, eb, es + 1);
    if (!rc) rc = ibcu_fill_hash_fp16_uniform(m->ctx, m->embed_scale, (size_t)c->vocab, es + 2, 0.001f, 0.01f);
    if (!rc) rc = ibcu_fill_hash_fp16_uniform(m->ctx, m->final_norm, (size_t)H, es + 3, 0.9f, 1.1f);
    if (!rc) rc = ibcu_sync(m->ctx);
    return rc;
}

int ib_b200_model_set_linear(ib_b200_model* m, int layer_i, int which, const void* w, const uint16_t* scales) {
    if (!m || !w) return IBCU_ERR_PARAM;
    lin* t = pick(m, layer_i, which);
    if (!t) return IBCU_ERR_PARAM;
    const size_t rb = t->bits == 8 ? (size_t)t->N : (size_t)t->N / 2;
    int rc = ibcu_memcpy_h2d(m->ctx, t->w, (const char*)w + (size_t)t->row0 * rb, (size_t)t->rows * rb);
    if (!rc && scales) rc = ibcu_memcpy_h2d(m->ctx, t->scale, scales + t->row0, (size_t)t->rows * 2);
    if (!rc) rc = ibcu_sync(m->ctx);
    if (!rc && !scales) {                                     /* a tensor stored without scales has scale 1 (src/forward.c:152-156) */
        uint16_t* one = (uint16_t*)malloc((size_t)(t->rows ? t->rows : 1) * 2);
        if (!one) return IBCU_ERR_NOMEM;
        for (int i = 0; i < t->rows; i++) one[i] = 0x3C00;
        rc = ibcu_memcpy_h2d(m->ctx, t->scale, one, (size_t)t->rows * 2);
        if (!rc) rc = ibcu_sync(m->ctx);
        free(one);
    }
    return rc;
}
int ib_b200_model_set_norms(ib_b200_model* m, int l, const uint16_t* a, const uint16_t* b) {
    if (!m || !a || !b || l < 0 || l >= m->c.n_layers) return IBCU_ERR_PARAM;
    int rc = ibcu_memcpy_h2d(m->ctx, m->L[l].in_norm, a, (size_t)m->c.hidden * 2);
    if (!rc) rc = ibcu_memcpy_h2d(m->ctx, m->L[l].post_norm, b, (size_t)m->c.hidden * 2);
    if (!rc) rc = ibcu_sync(m->ctx);
    return rc;
}
int ib_b200_model_set_embedding(ib_b200_model* m, const void* e, const uint16_t* es, const uint16_t* fn) {
    if (!m || !e || !fn) return IBCU_ERR_PARAM;
    const size_t V = (size_t)m->c.vocab, H = (size_t)m->c.hidden;
    const size_t eb = m->embed_bits == 16 ? V * H * 2 : (m->embed_bits == 8 ? V * H : V * H / 2);
    int rc = ibcu_memcpy_h2d(m->ctx, m->embed, e, eb);
    if (!rc && es) rc = ibcu_memcpy_h2d(m->ctx, m->embed_scale, es, V * 2);
    if (!rc) rc = ibcu_memcpy_h2d(m->ctx, m->final_norm, fn, H * 2);
    if (!rc) rc = ibcu_sync(m->ctx);
    if (!rc && !es) {                                         /* rows stored without scales are used as they are (src/forward.c:107-111) */
        uint16_t* one = (uint16_t*)malloc(V * 2);
        if (!one) return IBCU_ERR_NOMEM;
        for (size_t i = 0; i < V; i++) one[i] = 0x3C00;
        rc = ibcu_memcpy_h2d(m->ctx, m->embed_scale, one, V * 2);
        if (!rc) rc = ibcu_sync(m->ctx);
        free(one);
    }
    return rc;
}
int ib_b200_model_set_kv(ib_b200_model* m, int l, const float* k, const float* v, int n) {
    if (!m || !k || !v || l < 0 || l >= m->c.n_layers || n < 0 || n > m->c.max_ctx) return IBCU_ERR_PARAM;
    const size_t b = (size_t)n * m->c.n_kv_heads * m->c.head_dim * sizeof(float);
    int rc = ibcu_memcpy_h2d(m->ctx, m->L[l].k_cache, k, b);
    if (!rc) rc = ibcu_memcpy_h2d(m->ctx, m->L[l].v_cache, v, b);
    if (!rc) rc = ibcu_sync(m->ctx);
    return rc;
}
int ib_b200_model_get_kv(ib_b200_model* m, int l, float* k, float* v, int n) {
    if (!m || !k || !v || l < 0 || l >= m->c.n_layers || n < 0 || n > m->c.max_ctx) return IBCU_ERR_PARAM;
    const size_t b = (size_t)n * m->c.n_kv_heads * m->c.head_dim * sizeof(float);
    int rc = ibcu_memcpy_d2h(m->ctx, k, m->L[l].k_cache, b);
    if (!rc) rc = ibcu_memcpy_d2h(m->ctx, v, m->L[l].v_cache, b);
    if (!rc) rc = ibcu_sync(m->ctx);
    return rc;
}

/* descriptor of this rank's slice of tensor t writing into the full-width buffer `out` */
static ibcu_linear_t desc(const lin* t, float* out, int epilogue) {
    ibcu_linear_t d = { t->w, t->scale, out + t->row0, t->rows, t->M, 0, epilogue };
    return d;
}

/* Up to three tensors that read the same activation: tensors of equal bit width share a launch (a file may
 * give every tensor its own width: the converter stores o_proj at the default width and q, k, v at the
 * sensitive one, src/convert.c:572-578), then one gather for all of them. */
static int linear_group(ib_b200_model* m, lin* const* ts, float* const* outs, int n, const float* x, int N, int B,
                        const ibcu_prologue_t* pro, int epilogue) {
    int done[3] = { 0, 0, 0 }, rc = 0;
    float* bufs[3]; int M[3];
    for (int i = 0; i < n; i++) { bufs[i] = outs[i]; M[i] = ts[i]->M; }
    /* announce the gather: launches that can store their rows into the peers' copies from their epilogue then do */
    if (m->world > 1) rc = ibcu_allgather_rows_prepare(m->ctx, bufs, M, n);
    for (int i = 0; i < n && !rc; i++) {
        if (done[i]) continue;
        ibcu_linear_t d[3];
        int nd = 0;
        for (int j = i; j < n; j++)
            if (!done[j] && ts[j]->bits == ts[i]->bits) { d[nd++] = desc(ts[j], outs[j], epilogue); done[j] = 1; }
        rc = ibcu_linear_ex(m->ctx, d, nd, x, N, B, ts[i]->bits, pro);
    }
    if (rc || m->world == 1) return rc;
    return ibcu_allgather_rows_n(m->ctx, bufs, M, M, n, B, ROW_ALIGN);
}

/* the launch sequence of one step; everything stays on the device. head_last: logits of the last position
 * only, left in row 0 of the logits buffer (what ib_forward keeps of a multi-token call, src/forward.c:872-901) */
static int issue(ib_b200_model* m, int pos0, int B, int head_last) {
    const ib_b200_model_cfg* c = &m->c;
    ibcu_ctx* ctx = m->ctx;
    const int H = c->hidden;
    int rc = ibcu_embed_rows(ctx, m->embed, (const uint16_t*)m->embed_scale, m->tokens, m->x, H, B, m->embed_bits);
    for (int l = 0; l < c->n_layers && !rc; l++) {
        layer* y = &m->L[l];
        /* RMSNorm is folded into the activation preparation of the projections that consume it */
        ibcu_prologue_t n1 = { IBCU_PRO_RMSNORM, NULL, (const uint16_t*)y->in_norm, c->eps, NULL, 0 };
        lin* qkv[3] = { &y->t[IB_B200_Q], &y->t[IB_B200_K], &y->t[IB_B200_V] };
        float* qkv_out[3] = { m->q, m->k, m->v };
        rc = linear_group(m, qkv, qkv_out, 3, m->x, H, B, &n1, IBCU_EPI_STORE);
        /* RoPE, the KV-cache write and the attention itself are one step on the device */
        if (!rc) rc = m->dyn_pos
            ? ibcu_attention_decode_at(ctx, m->q, m->k, m->v, (float*)y->k_cache, (float*)y->v_cache, m->att,
                                       c->n_heads, c->n_kv_heads, c->head_dim, m->pos_dev, c->max_ctx, B, c->theta)
            : ibcu_attention_decode(ctx, m->q, m->k, m->v, (float*)y->k_cache, (float*)y->v_cache, m->att,
                                    c->n_heads, c->n_kv_heads, c->head_dim, pos0, B, c->theta);
        /* o_proj and down_proj add straight into the residual stream (src/forward.c:620-622, 644-646) */
        lin* o[1] = { &y->t[IB_B200_O] }; float* xo[1] = { m->x };
        if (!rc) rc = linear_group(m, o, xo, 1, m->att, H, B, NULL, IBCU_EPI_ADD);
        ibcu_prologue_t n2 = { IBCU_PRO_RMSNORM, NULL, (const uint16_t*)y->post_norm, c->eps, NULL, 0 };
        lin* gu[2] = { &y->t[IB_B200_GATE], &y->t[IB_B200_UP] };
        float* gu_out[2] = { m->hg, m->hu };
        if (!rc) rc = linear_group(m, gu, gu_out, 2, m->x, H, B, &n2, IBCU_EPI_STORE);
        /* silu(gate) * up (src/forward.c:637-640) in one small launch that also leaves max|h| for down_proj,
         * whose blocks then turn h into their integer operand without a reduction of their own */
        if (!rc) rc = ibcu_silu_mul_amax(ctx, m->hg, m->hg, m->hu, c->inter, B, m->amax, AMAX_PARTS);
        ibcu_prologue_t km = { IBCU_PRO_KNOWN_MAX, NULL, NULL, 0.0f, m->amax, AMAX_PARTS };
        lin* dn[1] = { &y->t[IB_B200_DOWN] };
        if (!rc) rc = linear_group(m, dn, xo, 1, m->hg, c->inter, B, &km, IBCU_EPI_ADD);
    }
    ibcu_prologue_t nf = { IBCU_PRO_RMSNORM, NULL, (const uint16_t*)m->final_norm, c->eps, NULL, 0 };
    lin* hd[1] = { &m->head }; float* lg[1] = { m->logits };
    if (!rc) rc = head_last ? linear_group(m, hd, lg, 1, m->x + (size_t)(B - 1) * H, H, 1, &nf, IBCU_EPI_STORE)
                            : linear_group(m, hd, lg, 1, m->x, H, B, &nf, IBCU_EPI_STORE);
    return rc;
}

static int step_device(ib_b200_model* m, int pos0, int B, int head_last) {
    if (!m || B < 1 || B > BMAX || pos0 < 0 || pos0 + B > m->c.max_ctx) return IBCU_ERR_PARAM;   /* src/forward.c:696-699, 857-862 */
    int rc = ibcu_store_i32(m->ctx, m->pos_dev, pos0);
    if (rc) return rc;
    if (!m->use_graph || !m->dyn_pos) return issue(m, pos0, B, head_last);
    for (int g = 0; g < m->n_graphs; g++)
        if (m->graphs[g].B == B && m->graphs[g].last_only == head_last) return ibcu_graph_launch(m->ctx, m->graphs[g].id);
    /* first use of this batch size: run once eagerly (sizes scratch), then capture for replay */
    rc = issue(m, pos0, B, head_last);
    if (!rc) rc = ibcu_sync(m->ctx);
    if (rc) return rc;
    if (m->n_graphs == MAX_GRAPHS) { ibcu_graph_destroy(m->ctx, m->graphs[0].id); m->graphs[0] = m->graphs[--m->n_graphs]; }
    int id = -1;
    rc = ibcu_graph_begin(m->ctx);
    if (!rc) { int r2 = issue(m, pos0, B, head_last); rc = ibcu_graph_end(m->ctx, &id); if (r2) rc = r2; }
    if (rc) return rc;                                     /* the eager result of this step stands; the failure is reported */
    m->graphs[m->n_graphs].B = B; m->graphs[m->n_graphs].last_only = head_last; m->graphs[m->n_graphs].id = id; m->n_graphs++;
    return 0;
}

int ib_b200_forward_step_device(ib_b200_model* m, int pos0, int B) { return step_device(m, pos0, B, 0); }

static int step_host(ib_b200_model* m, const int32_t* tokens, int pos0, int B, float* logits, int head_last) {
    if (!m || !tokens || B < 1 || B > BMAX) return IBCU_ERR_PARAM;
    for (int b = 0; b < B; b++) if (tokens[b] < 0 || tokens[b] >= m->c.vocab) return IBCU_ERR_PARAM;
    int rc = ibcu_sync(m->ctx);                            /* the pinned staging area is reused from call to call */
    if (rc) return rc;
    memcpy(m->pin, tokens, (size_t)B * sizeof(int32_t));
    rc = ibcu_memcpy_h2d(m->ctx, m->tokens, m->pin, (size_t)B * sizeof(int32_t));
    if (!rc) rc = step_device(m, pos0, B, head_last);
    float* stage = (float*)((char*)m->pin + 256);
    const size_t lb = (size_t)(head_last ? 1 : B) * m->c.vocab * sizeof(float);
    if (!rc && logits) rc = ibcu_memcpy_d2h(m->ctx, stage, m->logits, lb);
    if (!rc) rc = ibcu_sync(m->ctx);
    if (!rc && logits) memcpy(logits, stage, lb);
    return rc;
}

int ib_b200_forward_step(ib_b200_model* m, const int32_t* tokens, int pos0, int B, float* logits) {
    return step_host(m, tokens, pos0, B, logits, 0);
}
int ib_b200_forward_step_last(ib_b200_model* m, const int32_t* tokens, int pos0, int B, float* logits_last) {
    return step_host(m, tokens, pos0, B, logits_last, 1);
}
