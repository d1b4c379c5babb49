/*
 * Process-wide backend state, weight registration and the ib_kernels-shaped table entries.
 * Every entry takes host pointers like the reference's kernels do, moves the small operands
 * (activations, scales, outputs) through pinned staging buffers and runs the CUDA backend on the
 * device copy of the weights. No compute happens on the host.
 */
#include "ib_b200_internal.h"
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

ib_b200_state g_ib;

/* The reference's pool workers call the table concurrently with row slices of one tensor
 * (src/threading.c:220-241). The staging buffers, the scale cache, the stream and the sticky error are
 * process-wide, so every entry runs under this lock: concurrent calls are accepted and serialised. */
static pthread_mutex_t g_lock = PTHREAD_MUTEX_INITIALIZER;
void ib_b200_lock(void) { pthread_mutex_lock(&g_lock); }
void ib_b200_unlock(void) { pthread_mutex_unlock(&g_lock); }

void ib_b200_set_error(int code, const char* fmt, ...) {
    if (g_ib.status != 0) return;                 /* first failure wins */
    g_ib.status = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_ib.msg, sizeof g_ib.msg, fmt, ap);
    va_end(ap);
}

/* copy a failure of the CUDA backend into the host layer's sticky error */
int ib_b200_check(int rc, const char* what) {
    if (rc != 0) {
        ib_b200_set_error(rc, "%s: %s", what, g_ib.ctx ? ibcu_last_error(g_ib.ctx) : "backend not initialised");
        if (g_ib.ctx) ibcu_clear_error(g_ib.ctx);
    }
    return rc;
}

int ib_b200_init(int device) {
    if (g_ib.ctx) return 0;
    memset(&g_ib, 0, sizeof g_ib);
    int rc = ibcu_ctx_create(device, &g_ib.ctx);
    if (rc) { g_ib.ctx = NULL; ib_b200_set_error(rc, "ibcu_ctx_create(device %d) failed: no usable sm_100 GPU", device); return rc; }
    return 0;
}

static void scale_entry_drop(ib_b200_scale_entry* e) {
    if (e->dev) ibcu_free(g_ib.ctx, e->dev);
    free(e->host);
    memset(e, 0, sizeof *e);
}

void ib_b200_shutdown(void) {
    if (!g_ib.ctx) return;
    ib_b200_pq_release_all();
    for (int i = 0; i < IB_B200_SCALE_SLOTS; i++) if (g_ib.scales[i].weights) scale_entry_drop(&g_ib.scales[i]);
    for (int i = 0; i < g_ib.n_ranges; i++) ibcu_free(g_ib.ctx, g_ib.ranges[i].dev);
    for (int i = 0; i < IB_B200_NSTAGE; i++) {
        if (g_ib.stage_dev[i]) ibcu_free(g_ib.ctx, g_ib.stage_dev[i]);
        if (g_ib.stage_host[i]) ibcu_host_free(g_ib.ctx, g_ib.stage_host[i]);
    }
    ibcu_ctx_destroy(g_ib.ctx);
    memset(&g_ib, 0, sizeof g_ib);
}

ibcu_ctx* ib_b200_ctx(void) { return g_ib.ctx; }
int ib_b200_status(void) { return g_ib.status; }
const char* ib_b200_last_error(void) {
    static char out[sizeof g_ib.msg];
    memcpy(out, g_ib.msg, sizeof out);
    g_ib.msg[0] = 0;
    g_ib.status = 0;
    return out;
}

int ib_b200_register(const void* host_base, size_t bytes) {
    if (!g_ib.ctx) { ib_b200_set_error(IBCU_ERR_STATE, "ib_b200_register before ib_b200_init"); return IBCU_ERR_STATE; }
    if (!host_base || !bytes) { ib_b200_set_error(IBCU_ERR_PARAM, "ib_b200_register: empty range"); return IBCU_ERR_PARAM; }
    if (g_ib.n_ranges == IB_B200_MAX_RANGES) { ib_b200_set_error(IBCU_ERR_NOMEM, "ib_b200_register: range table full"); return IBCU_ERR_NOMEM; }
    void* dev = NULL;
    int rc = ib_b200_check(ibcu_malloc(g_ib.ctx, bytes, &dev), "ib_b200_register");
    if (rc) return rc;
    rc = ibcu_memcpy_h2d(g_ib.ctx, dev, host_base, bytes);
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, "ib_b200_register copy")) { ibcu_free(g_ib.ctx, dev); return rc; }
    ib_b200_range* r = &g_ib.ranges[g_ib.n_ranges++];
    r->host = (const char*)host_base; r->bytes = bytes; r->dev = (char*)dev;
    return 0;
}

int ib_b200_unregister(const void* host_base) {
    for (int i = 0; i < g_ib.n_ranges; i++)
        if (g_ib.ranges[i].host == (const char*)host_base) {
            /* scale vectors cached for tensors of this range go with it (the table is rebuilt: open addressing) */
            ib_b200_scale_entry keep[IB_B200_SCALE_SLOTS];
            int nkeep = 0;
            for (int k = 0; k < IB_B200_SCALE_SLOTS; k++) {
                ib_b200_scale_entry* e = &g_ib.scales[k];
                if (!e->weights) continue;
                if ((const char*)e->weights >= g_ib.ranges[i].host && (const char*)e->weights < g_ib.ranges[i].host + g_ib.ranges[i].bytes) scale_entry_drop(e);
                else { keep[nkeep++] = *e; memset(e, 0, sizeof *e); }
            }
            for (int k = 0; k < nkeep; k++) {
                unsigned h = (unsigned)(((uintptr_t)keep[k].weights >> 6) * 2654435761u) % IB_B200_SCALE_SLOTS;
                while (g_ib.scales[h].weights) h = (h + 1) % IB_B200_SCALE_SLOTS;
                g_ib.scales[h] = keep[k];
            }
            ibcu_free(g_ib.ctx, g_ib.ranges[i].dev);
            g_ib.ranges[i] = g_ib.ranges[--g_ib.n_ranges];
            return 0;
        }
    return IBCU_ERR_PARAM;
}

/* host address -> device address when [p, p+bytes) lies inside a registered range, else NULL */
void* ib_b200_translate(const void* p, size_t bytes) {
    const char* c = (const char*)p;
    for (int i = 0; i < g_ib.n_ranges; i++) {
        const ib_b200_range* r = &g_ib.ranges[i];
        if (c >= r->host && c + bytes <= r->host + r->bytes) return r->dev + (c - r->host);
    }
    return NULL;
}

/* pinned host + device staging pair number `slot`, at least `bytes` long */
int ib_b200_stage(int slot, size_t bytes, void** host, void** dev) {
    if (g_ib.stage_bytes[slot] < bytes) {
        size_t want = bytes < 65536 ? 65536 : bytes + bytes / 4;
        if (g_ib.stage_dev[slot]) ibcu_free(g_ib.ctx, g_ib.stage_dev[slot]);
        if (g_ib.stage_host[slot]) ibcu_host_free(g_ib.ctx, g_ib.stage_host[slot]);
        g_ib.stage_dev[slot] = g_ib.stage_host[slot] = NULL; g_ib.stage_bytes[slot] = 0;
        int rc = ibcu_malloc(g_ib.ctx, want, &g_ib.stage_dev[slot]);
        if (!rc) rc = ibcu_host_alloc(g_ib.ctx, want, &g_ib.stage_host[slot]);
        if (ib_b200_check(rc, "staging buffer")) return rc;
        g_ib.stage_bytes[slot] = want;
    }
    *host = g_ib.stage_host[slot]; *dev = g_ib.stage_dev[slot];
    return 0;
}

enum { ST_X = 0, ST_SCALE, ST_OUT, ST_AUX };

/* host array -> staging slot -> device; returns the device pointer or NULL */
static void* push(int slot, const void* src, size_t bytes) {
    void *h, *d;
    if (ib_b200_stage(slot, bytes, &h, &d)) return NULL;
    memcpy(h, src, bytes);
    if (ib_b200_check(ibcu_memcpy_h2d(g_ib.ctx, d, h, bytes), "h2d")) return NULL;
    g_ib.h2d_bytes += bytes;
    return d;
}

/* device copy of the FP32 row scales of the tensor at `weights`: uploaded when first seen or changed */
static void* scales_on_device(const void* weights, const float* scales, int M) {
    const size_t bytes = (size_t)M * sizeof(float);
    unsigned h = (unsigned)(((uintptr_t)weights >> 6) * 2654435761u) % IB_B200_SCALE_SLOTS;
    ib_b200_scale_entry* e = NULL;
    for (int probe = 0; probe < 64; probe++, h = (h + 1) % IB_B200_SCALE_SLOTS) {
        if (!g_ib.scales[h].weights || (g_ib.scales[h].weights == weights && g_ib.scales[h].M == M)) { e = &g_ib.scales[h]; break; }
    }
    if (!e) return push(1 /* ST_SCALE */, scales, bytes);               /* neighbourhood full: no caching for this tensor */
    if (e->weights && memcmp(e->host, scales, bytes) == 0) return e->dev;
    if (!e->weights) {
        e->host = (float*)malloc(bytes);
        if (!e->host || ib_b200_check(ibcu_malloc(g_ib.ctx, bytes, &e->dev), "scale cache")) { free(e->host); memset(e, 0, sizeof *e); return push(1, scales, bytes); }
        e->weights = weights; e->M = M;
    }
    memcpy(e->host, scales, bytes);
    void* staged = push(1, scales, bytes);
    if (!staged || ib_b200_check(ibcu_memcpy_d2d(g_ib.ctx, e->dev, staged, bytes), "scale cache copy")) return staged;
    return e->dev;
}

void ib_b200_copy_stats(unsigned long long* h2d_bytes, unsigned long long* d2h_bytes) {
    if (h2d_bytes) *h2d_bytes = g_ib.h2d_bytes;
    if (d2h_bytes) *d2h_bytes = g_ib.d2h_bytes;
}


static int ready(const char* who) {
    if (g_ib.ctx) return 1;
    ib_b200_set_error(IBCU_ERR_STATE, "%s called before ib_b200_init", who);
    return 0;
}

/* shared body of the FP32-activation entries */
static void linear_fp32(const char* who, float* out, const void* weights, const float* scales, const float* input,
                        int M, int N, int B, int M_stride, int bits) {
    if (!ready(who)) return;
    if (!out || !weights || !scales || !input || M <= 0 || N <= 0 || B <= 0 || M_stride < M) {
        ib_b200_set_error(IBCU_ERR_PARAM, "%s: bad arguments", who); return;
    }
    const size_t wbytes = (size_t)M * (bits == 8 ? (size_t)N : (size_t)(N / 2));
    void* dw = ib_b200_translate(weights, wbytes);
    if (!dw) { ib_b200_set_error(IBCU_ERR_STATE, "%s: weights %p (+%zu) are not inside a registered range; there is no CPU path", who, weights, wbytes); return; }
    void* dx = push(ST_X, input, (size_t)B * N * sizeof(float));
    void* ds = scales_on_device(weights, scales, M);
    void *ho, *dout;
    const size_t obytes = ((size_t)(B - 1) * M_stride + M) * sizeof(float);
    if (!dx || !ds || ib_b200_stage(ST_OUT, obytes, &ho, &dout)) return;
    /* small results are written by the kernel straight into the pinned host buffer (it is mapped into the
     * device's address space): no copy launch between the kernel and the host's wait */
    const int direct = obytes <= (1u << 20);
    ibcu_linear_t t = { dw, ds, (float*)(direct ? ho : dout), M, M_stride, 1, IBCU_EPI_STORE };
    int rc = ibcu_linear(g_ib.ctx, &t, 1, (const float*)dx, N, B, bits);
    if (!rc && !direct) rc = ibcu_memcpy_d2h(g_ib.ctx, ho, dout, obytes);
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, who)) return;
    g_ib.d2h_bytes += (size_t)B * M * sizeof(float);
    for (int b = 0; b < B; b++) memcpy(out + (size_t)b * M_stride, (const float*)ho + (size_t)b * M_stride, (size_t)M * sizeof(float));
}

void ib_b200_matmul_int4(float* out, const void* w, const float* s, const float* x, int M, int N) {
    ib_b200_lock(); linear_fp32("matmul_int4", out, w, s, x, M, N, 1, M, 4); ib_b200_unlock();
}
void ib_b200_matmul_int8(float* out, const void* w, const float* s, const float* x, int M, int N) {
    ib_b200_lock(); linear_fp32("matmul_int8", out, w, s, x, M, N, 1, M, 8); ib_b200_unlock();
}
void ib_b200_matmul_int8_batch(float* out, const void* w, const float* s, const float* x, int M, int N, int B, int M_stride) {
    ib_b200_lock(); linear_fp32("matmul_int8_batch", out, w, s, x, M, N, B, M_stride, 8); ib_b200_unlock();
}

static void ib_b200_matmul_w4a8_batch_unlocked(float* out, const void* weights, const float* scales_w, const int8_t* input,
                               const float* scales_a, int M, int N, int B, int M_stride) {
    const char* who = "matmul_w4a8_batch";
    if (!ready(who)) return;
    if (!out || !weights || !scales_w || !input || !scales_a || M <= 0 || N <= 0 || (N & 1) || B <= 0 || M_stride < M) {
        ib_b200_set_error(IBCU_ERR_PARAM, "%s: bad arguments", who); return;
    }
    const int groups = (N + 127) / 128;
    void* dw = ib_b200_translate(weights, (size_t)M * (N / 2));
    if (!dw) { ib_b200_set_error(IBCU_ERR_STATE, "%s: weights are not inside a registered range; there is no CPU path", who); return; }
    void* dx = push(ST_X, input, (size_t)B * N);
    void* ds = push(ST_SCALE, scales_w, (size_t)M * sizeof(float));
    void* da = push(ST_AUX, scales_a, (size_t)B * groups * sizeof(float));
    void *ho, *dout;
    const size_t obytes = ((size_t)(B - 1) * M_stride + M) * sizeof(float);
    if (!dx || !ds || !da || ib_b200_stage(ST_OUT, obytes, &ho, &dout)) return;
    ibcu_linear_t t = { dw, ds, (float*)dout, M, M_stride, 1, IBCU_EPI_STORE };
    int rc = ibcu_linear_w4a8(g_ib.ctx, &t, (const int8_t*)dx, (const float*)da, N, B);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, ho, dout, obytes);
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, who)) return;
    for (int b = 0; b < B; b++) memcpy(out + (size_t)b * M_stride, (const float*)ho + (size_t)b * M_stride, (size_t)M * sizeof(float));
}
void ib_b200_matmul_w4a8(float* out, const void* w, const float* sw, const int8_t* xq, const float* sa, int M, int N) {
    ib_b200_matmul_w4a8_batch(out, w, sw, xq, sa, M, N, 1, M);                    /* takes the lock */
}

static int ib_b200_quantize_input_int8_g128_unlocked(const float* input, int8_t* out_q, float* out_scales, int N) {
    if (!ready("quantize_input_int8_g128") || !input || !out_q || !out_scales || N <= 0) return 0;
    const int groups = (N + 127) / 128;
    void* dx = push(ST_X, input, (size_t)N * sizeof(float));
    void *hq, *dq, *hs, *ds;
    if (!dx || ib_b200_stage(ST_OUT, (size_t)N, &hq, &dq) || ib_b200_stage(ST_AUX, (size_t)groups * sizeof(float), &hs, &ds)) return 0;
    int rc = ibcu_quantize_input_int8_g128(g_ib.ctx, (const float*)dx, (int8_t*)dq, (float*)ds, N, 1);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, hq, dq, (size_t)N);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, hs, ds, (size_t)groups * sizeof(float));
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, "quantize_input_int8_g128")) return 0;
    memcpy(out_q, hq, (size_t)N);
    memcpy(out_scales, hs, (size_t)groups * sizeof(float));
    return groups;
}

/* ── element-wise entries: operands are O(hidden), moved per call ── */
static void ib_b200_rmsnorm_unlocked(float* out, const float* input, const float* weight, float eps, int N) {
    if (!ready("rmsnorm") || !out || !input || !weight || N <= 0) return;
    /* the table hands over weights already widened to FP32 (src/forward.c:322-327) */
    void* dx = push(ST_X, input, (size_t)N * sizeof(float));
    void* dw = push(ST_SCALE, weight, (size_t)N * sizeof(float));
    void *ho, *dout;
    if (!dx || !dw || ib_b200_stage(ST_OUT, (size_t)N * sizeof(float), &ho, &dout)) return;
    int rc = ibcu_rmsnorm_f32w(g_ib.ctx, (float*)dout, (const float*)dx, (const float*)dw, eps, N, 1);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, ho, dout, (size_t)N * sizeof(float));
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, "rmsnorm")) return;
    memcpy(out, ho, (size_t)N * sizeof(float));
}

static void ib_b200_rope_unlocked(float* q, float* k, int head_dim, int pos, float theta) {
    if (!ready("rope") || !q || !k || head_dim <= 0 || (head_dim & 1)) return;
    const size_t hb = (size_t)head_dim * sizeof(float);
    void *hq, *dq, *hk, *dk;
    if (ib_b200_stage(ST_X, hb, &hq, &dq) || ib_b200_stage(ST_SCALE, hb, &hk, &dk)) return;
    memcpy(hq, q, hb); memcpy(hk, k, hb);
    int rc = ibcu_memcpy_h2d(g_ib.ctx, dq, hq, hb);
    if (!rc) rc = ibcu_memcpy_h2d(g_ib.ctx, dk, hk, hb);
    /* one Q head, one K head, position `pos`, no cache write */
    if (!rc) rc = ibcu_rope_kv_write(g_ib.ctx, (float*)dq, (float*)dk, NULL, NULL, NULL, 1, 1, head_dim, pos, 1, theta);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, hq, dq, hb);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, hk, dk, hb);
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, "rope")) return;
    memcpy(q, hq, hb); memcpy(k, hk, hb);
}

static void ib_b200_softmax_unlocked(float* data, int N) {
    if (!ready("softmax") || !data || N <= 0) return;
    void *h, *d;
    const size_t nb = (size_t)N * sizeof(float);
    if (ib_b200_stage(ST_X, nb, &h, &d)) return;
    memcpy(h, data, nb);
    int rc = ibcu_memcpy_h2d(g_ib.ctx, d, h, nb);
    if (!rc) rc = ibcu_softmax(g_ib.ctx, (float*)d, N, 1);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, h, d, nb);
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, "softmax")) return;
    memcpy(data, h, nb);
}

static void ib_b200_silu_mul_unlocked(float* out, const float* gate, const float* up, int N) {
    if (!ready("silu_mul") || !out || !gate || !up || N <= 0) return;
    const size_t nb = (size_t)N * sizeof(float);
    void* dg = push(ST_X, gate, nb);
    void* du = push(ST_SCALE, up, nb);
    void *ho, *dout;
    if (!dg || !du || ib_b200_stage(ST_OUT, nb, &ho, &dout)) return;
    int rc = ibcu_silu_mul(g_ib.ctx, (float*)dout, (const float*)dg, (const float*)du, (size_t)N);
    if (!rc) rc = ibcu_memcpy_d2h(g_ib.ctx, ho, dout, nb);
    if (!rc) rc = ibcu_sync_spin(g_ib.ctx);
    if (ib_b200_check(rc, "silu_mul")) return;
    memcpy(out, ho, nb);
}


void ib_b200_matmul_w4a8_batch(float* out, const void* weights, const float* scales_w, const int8_t* input,
                               const float* scales_a, int M, int N, int B, int M_stride) {
    ib_b200_lock();
    ib_b200_matmul_w4a8_batch_unlocked(out, weights, scales_w, input, scales_a, M, N, B, M_stride);
    ib_b200_unlock();
}

int ib_b200_quantize_input_int8_g128(const float* input, int8_t* out_q, float* out_scales, int N) {
    ib_b200_lock();
    int r = ib_b200_quantize_input_int8_g128_unlocked(input, out_q, out_scales, N);
    ib_b200_unlock();
    return r;
}

void ib_b200_rmsnorm(float* out, const float* input, const float* weight, float eps, int N) {
    ib_b200_lock();
    ib_b200_rmsnorm_unlocked(out, input, weight, eps, N);
    ib_b200_unlock();
}

void ib_b200_rope(float* q, float* k, int head_dim, int pos, float theta) {
    ib_b200_lock();
    ib_b200_rope_unlocked(q, k, head_dim, pos, theta);
    ib_b200_unlock();
}

void ib_b200_softmax(float* data, int N) {
    ib_b200_lock();
    ib_b200_softmax_unlocked(data, N);
    ib_b200_unlock();
}

void ib_b200_silu_mul(float* out, const float* gate, const float* up, int N) {
    ib_b200_lock();
    ib_b200_silu_mul_unlocked(out, gate, up, N);
    ib_b200_unlock();
}

void ib_b200_install_kernels(void* table) {
    ib_b200_kernels* t = (ib_b200_kernels*)table;
    if (!t) return;
    t->matmul_int4 = ib_b200_matmul_int4;
    t->matmul_int8 = ib_b200_matmul_int8;
    t->rmsnorm = ib_b200_rmsnorm;
    t->rope = ib_b200_rope;
    t->softmax = ib_b200_softmax;
    t->silu_mul = ib_b200_silu_mul;
    t->matmul_w4a8 = ib_b200_matmul_w4a8;
    t->matmul_w4a8_batch = ib_b200_matmul_w4a8_batch;
    t->matmul_int8_batch = ib_b200_matmul_int8_batch;
}
