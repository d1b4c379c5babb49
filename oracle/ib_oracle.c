/*
 * ib_oracle.c — plain-C CPU restatement of libinferbit's quantized-weight product hot path.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels. Nothing in the product
 * libraries links, loads or calls this file. Build with -ffp-contract=off so that every
 * fused multiply-add below is an explicit fmaf() and every unfused one stays unfused.
 *
 * Parity status: PINNED against the unmodified reference compiled by oracle/Makefile
 * (tests/test_oracle_vs_ref.py) and against its recorded outputs in tests/golden/.
 */
#include "ib_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ── binary16 <-> binary32 ───────────────────────────────────────────────────────────── */

/* src/pq_decode.c:263-288 (same mapping as src/forward.c:38-70). */
float ibo_fp16_to_fp32(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    int e = (h >> 10) & 31;
    uint32_t m = h & 1023u;
    uint32_t bits;
    if (e == 31) {
        bits = s | 0x7F800000u | (m << 13);
    } else if (e != 0) {
        bits = s | ((uint32_t)(e + 112) << 23) | (m << 13);
    } else if (m == 0) {
        bits = s;
    } else {
        int sh = 0;
        while (!(m & 1024u)) { m <<= 1; sh++; }      /* normalise the subnormal */
        bits = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

void ibo_fp16_array_to_fp32(const uint16_t* in, float* out, int n) {
    for (int i = 0; i < n; i++) out[i] = ibo_fp16_to_fp32(in[i]);
}

/* src/pq_decode.c:295-337. Round to nearest, ties to even; NaN keeps a quiet bit. */
uint16_t ibo_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    int e = (int)((x >> 23) & 255u) - 112;           /* re-biased exponent */
    uint32_t m = x & 0x7FFFFFu;
    /* exponent overflow: the reference sets the quiet bit whenever the fp32 mantissa is non-zero,
     * for finite values too (src/pq_decode.c:322-323); kept as is. */
    if (e >= 31) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0u));
    if (e <= 0) {
        if (e < -10) return sign;
        m = (m | 0x800000u) >> (1 - e);
    }
    uint32_t keep = m >> 13, rest = m & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (keep & 1u))) keep++;
    if (e <= 0) return (uint16_t)(sign | keep);       /* a carry lands in exponent 1, as it should */
    if (keep & 0x400u) { keep = 0; e++; if (e >= 31) return (uint16_t)(sign | 0x7C00u); }
    return (uint16_t)(sign | ((uint32_t)e << 10) | keep);
}

/* ── INT4 / INT8 matvec ──────────────────────────────────────────────────────────────── */

/* src/kernels/scalar.c:9-27. Byte b of a row carries column 2b in its low nibble and column
 * 2b+1 in its high nibble, both biased by 8. FP32 running sum in column order; the row scale
 * multiplies the finished sum. */
void ibo_matmul_int4(float* out, const uint8_t* w, const float* scales, const float* x, int M, int N) {
    int row_bytes = N / 2;
    for (int r = 0; r < M; r++) {
        const uint8_t* row = w + (size_t)r * row_bytes;
        float acc = 0.0f;
        for (int j = 0; j < N; j += 2) {
            uint8_t b = row[j >> 1];
            acc += (float)((int)(b & 15u) - 8) * x[j];
            if (j + 1 < N) acc += (float)((int)(b >> 4) - 8) * x[j + 1];
        }
        out[r] = acc * scales[r];
    }
}

/* src/kernels/scalar.c:29-41 */
void ibo_matmul_int8(float* out, const int8_t* w, const float* scales, const float* x, int M, int N) {
    for (int r = 0; r < M; r++) {
        const int8_t* row = w + (size_t)r * N;
        float acc = 0.0f;
        for (int j = 0; j < N; j++) acc += (float)row[j] * x[j];
        out[r] = acc * scales[r];
    }
}

/* src/kernels/scalar.c:70-84 — out[b*M_stride + r], x[b*N + j]. */
void ibo_matmul_int8_batch(float* out, const int8_t* w, const float* scales, const float* x,
                           int M, int N, int B, int M_stride) {
    for (int b = 0; b < B; b++)
        for (int r = 0; r < M; r++) {
            const int8_t* row = w + (size_t)r * N;
            const float* xb = x + (size_t)b * N;
            float acc = 0.0f;
            for (int j = 0; j < N; j++) acc += (float)row[j] * xb[j];
            out[(size_t)b * M_stride + r] = acc * scales[r];
        }
}

/* src/forward.c:226-233 — the per-position loop the reference falls back to for INT4 + FP32 x. */
void ibo_matmul_int4_batch(float* out, const uint8_t* w, const float* scales, const float* x,
                           int M, int N, int B, int M_stride) {
    for (int b = 0; b < B; b++)
        ibo_matmul_int4(out + (size_t)b * M_stride, w, scales, x + (size_t)b * N, M, N);
}

/* src/threading.c:401-432. 128-wide groups; scale = maxabs/127; q = trunc(v*(1/scale) ± 0.5)
 * clamped to ±127; an all-(near-)zero group gets scale 1e-10 and zeros. */
int ibo_quantize_input_int8_g128(const float* x, int8_t* q, float* sa, int N) {
    int g = 0;
    for (int lo = 0; lo < N; lo += 128, g++) {
        int hi = lo + 128 < N ? lo + 128 : N;
        float amax = 0.0f;
        for (int i = lo; i < hi; i++) {
            float a = x[i] < 0 ? -x[i] : x[i];
            if (a > amax) amax = a;
        }
        if (amax < 1e-10f) {
            sa[g] = 1e-10f;
            memset(q + lo, 0, (size_t)(hi - lo));
            continue;
        }
        float s = amax / 127.0f, inv = 1.0f / s;
        for (int i = lo; i < hi; i++) {
            int v = (int)(x[i] * inv + (x[i] >= 0 ? 0.5f : -0.5f));
            q[i] = (int8_t)(v > 127 ? 127 : (v < -127 ? -127 : v));
        }
        sa[g] = s;
    }
    return g;
}

/* src/kernels/scalar.c:43-68 */
void ibo_matmul_w4a8(float* out, const uint8_t* w, const float* sw, const int8_t* xq,
                     const float* sa, int M, int N) {
    ibo_matmul_w4a8_batch(out, w, sw, xq, sa, M, N, 1, M);
}

/* src/kernels/scalar.c:86-124 — exact int32 dot per 128-group, scaled by the group's activation
 * scale into an FP32 row accumulator, then by the row's weight scale. */
void ibo_matmul_w4a8_batch(float* out, const uint8_t* w, const float* sw, const int8_t* xq,
                           const float* sa, int M, int N, int B, int M_stride) {
    int groups = (N + 127) / 128, row_bytes = N / 2;
    for (int b = 0; b < B; b++) {
        const int8_t* xb = xq + (size_t)b * N;
        const float* sab = sa + (size_t)b * groups;
        for (int r = 0; r < M; r++) {
            const uint8_t* row = w + (size_t)r * row_bytes;
            float acc = 0.0f;
            for (int g = 0; g < groups; g++) {
                int lo = g * 128, hi = lo + 128 < N ? lo + 128 : N;
                int32_t dot = 0;
                for (int j = lo; j < hi; j += 2) {
                    uint8_t byte = row[j >> 1];
                    dot += ((int)(byte & 15u) - 8) * (int)xb[j];
                    if (j + 1 < hi) dot += ((int)(byte >> 4) - 8) * (int)xb[j + 1];
                }
                acc += (float)dot * sab[g];
            }
            out[(size_t)b * M_stride + r] = acc * sw[r];
        }
    }
}

/* ── PQ matvec ───────────────────────────────────────────────────────────────────────── */

static float dot_seq(const float* a, const float* b, int n, int fused) {
    float s = 0.0f;
    if (fused) for (int i = 0; i < n; i++) s = fmaf(a[i], b[i], s);
    else       for (int i = 0; i < n; i++) s = s + a[i] * b[i];
    return s;
}

/* src/pq_decode.c:1504-1682 with n_levels == 1 and no outlier columns (inner_cols = identity). */
int ibo_pq_matmul_fp32(int M, int N, int G, int K,
                       const uint16_t* cb_l, const uint16_t* cb_r, long cb_chunk_stride,
                       const uint8_t* idx_l, const uint8_t* idx_r, const uint16_t* row_scale,
                       const float* x, float* out, int fused, int* n_skipped) {
    if (!cb_l || !cb_r || !idx_l || !idx_r || !row_scale || !x || !out) return -1;
    if (M <= 0 || N <= 0 || G <= 0 || (G & 1) || G > 32 || K <= 0 || K > 256 || N % G) return -1;
    int half = G / 2, C = N / G;
    float* lut_l = (float*)malloc((size_t)C * K * sizeof(float));
    float* lut_r = (float*)malloc((size_t)C * K * sizeof(float));
    float* ent = (float*)malloc((size_t)half * sizeof(float));
    unsigned char* live = (unsigned char*)malloc((size_t)C);
    if (!lut_l || !lut_r || !ent || !live) { free(lut_l); free(lut_r); free(ent); free(live); return -1; }

    /* :1582-1616 — a chunk all of whose |x| fall under 1 % of the vector's max is dropped. */
    float amax = 0.0f;
    for (int j = 0; j < N; j++) { float a = x[j] < 0 ? -x[j] : x[j]; if (a > amax) amax = a; }
    int dropped = 0;
    for (int c = 0; c < C; c++) {
        live[c] = 1;
        if (amax > 0.0f) {
            float cmax = 0.0f, thr = amax * 0.01f;
            for (int i = 0; i < G; i++) {
                float a = x[c * G + i]; if (a < 0) a = -a;
                if (a > cmax) cmax = a;
            }
            if (!(cmax >= thr)) { live[c] = 0; dropped++; }
        }
    }
    /* :1621-1658 — per live chunk, K partial dots on each side. */
    for (int c = 0; c < C; c++) {
        if (!live[c]) continue;
        const uint16_t* tl = cb_l + (size_t)c * cb_chunk_stride;
        const uint16_t* tr = cb_r + (size_t)c * cb_chunk_stride;
        for (int k = 0; k < K; k++) {
            for (int i = 0; i < half; i++) ent[i] = ibo_fp16_to_fp32(tl[k * half + i]);
            lut_l[(size_t)c * K + k] = dot_seq(ent, x + c * G, half, fused);
            for (int i = 0; i < half; i++) ent[i] = ibo_fp16_to_fp32(tr[k * half + i]);
            lut_r[(size_t)c * K + k] = dot_seq(ent, x + c * G + half, half, fused);
        }
    }
    /* :1441-1496 — per row, chunk order, (left + right) then accumulate; scale last. */
    for (int r = 0; r < M; r++) {
        const uint8_t* il = idx_l + (size_t)r * C;
        const uint8_t* ir = idx_r + (size_t)r * C;
        float acc = 0.0f;
        for (int c = 0; c < C; c++) {
            if (!live[c]) continue;
            acc += lut_l[(size_t)c * K + il[c]] + lut_r[(size_t)c * K + ir[c]];
        }
        out[r] = acc * ibo_fp16_to_fp32(row_scale[r]);
    }
    if (n_skipped) *n_skipped = dropped;
    free(lut_l); free(lut_r); free(ent); free(live);
    return 0;
}

/* The same path with the production extras: a second residual level (src/pq_decode.c:1441-1496 TL2/TR2
 * terms; index forms of :1058-1075: one byte, or two 4-bit indices per byte, low nibble = even chunk, when
 * K_l2 == 16) and the outlier sidecar (:1394-1409 scalar form): outlier columns are taken out of the
 * activation before the tables are built (inner_cols, :1538-1546), so N - n_outlier = C * G, and come
 * back as out[r] += (sidecar[r][j] * scale[j]) * x[col[j]] after the row scale. NULL / 0 switch a part off. */
int ibo_pq_matmul_fp32_ex(int M, int N, int G, int K, int K_l2,
                          const uint16_t* cb1_l, const uint16_t* cb1_r, const uint16_t* cb2_l, const uint16_t* cb2_r,
                          const uint8_t* idx1_l, const uint8_t* idx1_r, const uint8_t* idx2_l, const uint8_t* idx2_r,
                          const uint16_t* row_scale, int n_outlier, const int32_t* outlier_cols,
                          const int8_t* outlier_sidecar, const uint16_t* outlier_scale,
                          const float* x, float* out, int fused) {
    if (!cb1_l || !cb1_r || !idx1_l || !idx1_r || !row_scale || !x || !out) return -1;
    if (M <= 0 || N <= 0 || G <= 0 || (G & 1) || G > 32 || K <= 0 || K > 256 || n_outlier < 0 || (N - n_outlier) % G) return -1;
    const int two = cb2_l && cb2_r && idx2_l && idx2_r;
    if (two && (K_l2 <= 0 || K_l2 > 256)) return -1;
    int half = G / 2, n_inner = N - n_outlier, C = n_inner / G;
    const int packed = two && K_l2 == 16;
    const size_t l2_stride = packed ? (size_t)((C + 1) / 2) : (size_t)C;
    int* inner = (int*)malloc((size_t)n_inner * sizeof(int));
    unsigned char* mask = (unsigned char*)calloc((size_t)N, 1);
    float* xi = (float*)malloc((size_t)n_inner * sizeof(float));
    float* t1l = (float*)malloc((size_t)C * K * sizeof(float));
    float* t1r = (float*)malloc((size_t)C * K * sizeof(float));
    float* t2l = two ? (float*)malloc((size_t)C * K_l2 * sizeof(float)) : NULL;
    float* t2r = two ? (float*)malloc((size_t)C * K_l2 * sizeof(float)) : NULL;
    float* ent = (float*)malloc((size_t)half * sizeof(float));
    unsigned char* live = (unsigned char*)malloc((size_t)C);
    int rc = -1;
    if (!inner || !mask || !xi || !t1l || !t1r || (two && (!t2l || !t2r)) || !ent || !live) goto done;
    for (int j = 0; j < n_outlier; j++) mask[outlier_cols[j]] = 1;
    { int kk = 0; for (int j = 0; j < N; j++) if (!mask[j] && kk < n_inner) inner[kk++] = j; }
    for (int j = 0; j < n_inner; j++) xi[j] = x[inner[j]];
    {
        float amax = 0.0f;
        for (int j = 0; j < n_inner; j++) { float a = xi[j] < 0 ? -xi[j] : xi[j]; if (a > amax) amax = a; }
        for (int c = 0; c < C; c++) {
            live[c] = 1;
            if (amax > 0.0f) {
                float cmax = 0.0f, thr = amax * 0.01f;
                for (int i = 0; i < G; i++) { float a = xi[c * G + i]; if (a < 0) a = -a; if (a > cmax) cmax = a; }
                if (!(cmax >= thr)) live[c] = 0;
            }
        }
    }
    for (int c = 0; c < C; c++) {
        if (!live[c]) continue;
        for (int k = 0; k < K; k++) {
            for (int i = 0; i < half; i++) ent[i] = ibo_fp16_to_fp32(cb1_l[k * half + i]);
            t1l[(size_t)c * K + k] = dot_seq(ent, xi + c * G, half, fused);
            for (int i = 0; i < half; i++) ent[i] = ibo_fp16_to_fp32(cb1_r[k * half + i]);
            t1r[(size_t)c * K + k] = dot_seq(ent, xi + c * G + half, half, fused);
        }
        for (int k = 0; two && k < K_l2; k++) {
            for (int i = 0; i < half; i++) ent[i] = ibo_fp16_to_fp32(cb2_l[k * half + i]);
            t2l[(size_t)c * K_l2 + k] = dot_seq(ent, xi + c * G, half, fused);
            for (int i = 0; i < half; i++) ent[i] = ibo_fp16_to_fp32(cb2_r[k * half + i]);
            t2r[(size_t)c * K_l2 + k] = dot_seq(ent, xi + c * G + half, half, fused);
        }
    }
    for (int r = 0; r < M; r++) {
        const uint8_t* il = idx1_l + (size_t)r * C;
        const uint8_t* ir = idx1_r + (size_t)r * C;
        const uint8_t* jl = two ? idx2_l + (size_t)r * l2_stride : NULL;
        const uint8_t* jr = two ? idx2_r + (size_t)r * l2_stride : NULL;
        float acc = 0.0f;
        for (int c = 0; c < C; c++) {
            if (!live[c]) continue;
            acc += t1l[(size_t)c * K + il[c]] + t1r[(size_t)c * K + ir[c]];
            if (two) {
                int a = packed ? ((c & 1) ? (jl[c >> 1] >> 4) & 15 : jl[c >> 1] & 15) : jl[c];
                int b = packed ? ((c & 1) ? (jr[c >> 1] >> 4) & 15 : jr[c >> 1] & 15) : jr[c];
                acc += t2l[(size_t)c * K_l2 + a] + t2r[(size_t)c * K_l2 + b];
            }
        }
        out[r] = acc * ibo_fp16_to_fp32(row_scale[r]);
    }
    for (int j = 0; j < n_outlier; j++) {
        float os = ibo_fp16_to_fp32(outlier_scale[j]), xj = x[outlier_cols[j]];
        for (int r = 0; r < M; r++) {
            float w = (float)outlier_sidecar[(size_t)r * n_outlier + j] * os;
            out[r] += w * xj;
        }
    }
    rc = 0;
done:
    free(inner); free(mask); free(xi); free(t1l); free(t1r); free(t2l); free(t2r); free(ent); free(live);
    return rc;
}

/* ── top-K LM head (src/pq_decode.c:2085-2341) ──────────────────────────────────────── */

typedef struct {
    int M, N, G, K, K_l2, C, half, n_outlier, two, packed;
    const uint16_t *cb1_l, *cb1_r, *cb2_l, *cb2_r, *row_scale, *outlier_scale;
    const uint8_t *idx1_l, *idx1_r, *idx2_l, *idx2_r;
    const int32_t* outlier_cols;
    const int8_t* outlier_sidecar;
    int* inner;                                  /* [N - n_outlier] the columns that are not outlier columns, ascending */
} pq_view;

/* src/pq_decode.c:2085-2143 (ib_pq_matmul_fp32_l1_only): first level only, NO 1 % rule, row scale, then the
 * outlier sidecar; per chunk one table per side, out[r] += TL[i] + TR[j] in chunk order. */
static void pq_l1_only(const pq_view* v, const float* x, float* out, float* tl, float* tr, float* ent, int fused) {
    float xs[32];
    memset(out, 0, (size_t)v->M * sizeof(float));
    for (int c = 0; c < v->C; c++) {
        for (int i = 0; i < v->G; i++) xs[i] = x[v->inner[c * v->G + i]];
        for (int k = 0; k < v->K; k++) {
            for (int i = 0; i < v->half; i++) ent[i] = ibo_fp16_to_fp32(v->cb1_l[k * v->half + i]);
            tl[k] = dot_seq(ent, xs, v->half, fused);
            for (int i = 0; i < v->half; i++) ent[i] = ibo_fp16_to_fp32(v->cb1_r[k * v->half + i]);
            tr[k] = dot_seq(ent, xs + v->half, v->half, fused);
        }
        for (int r = 0; r < v->M; r++)
            out[r] += tl[v->idx1_l[(size_t)r * v->C + c]] + tr[v->idx1_r[(size_t)r * v->C + c]];
    }
    for (int r = 0; r < v->M; r++) out[r] *= ibo_fp16_to_fp32(v->row_scale[r]);
    for (int j = 0; j < v->n_outlier; j++) {                  /* apply_outliers, src/pq_decode.c:1394-1409 */
        float os = ibo_fp16_to_fp32(v->outlier_scale[j]), xj = x[v->outlier_cols[j]];
        for (int r = 0; r < v->M; r++) out[r] += ((float)v->outlier_sidecar[(size_t)r * v->n_outlier + j] * os) * xj;
    }
}

/* src/pq_decode.c:2145-2248 (ib_pq_matmul_fp32_subset): every level of one row, entry times activation added
 * one product at a time in the order left[j], right[j] per j, level 1 then level 2 per chunk. */
static float pq_row_full(const pq_view* v, const float* x, int r, int fused) {
    const size_t l2_stride = v->packed ? (size_t)((v->C + 1) / 2) : (size_t)v->C;
    float acc = 0.0f;
    for (int c = 0; c < v->C; c++) {
        const int base = c * v->G;
        for (int lvl = 0; lvl < (v->two ? 2 : 1); lvl++) {
            int a, b;
            const uint16_t *cl, *cr;
            if (lvl == 0) { a = v->idx1_l[(size_t)r * v->C + c]; b = v->idx1_r[(size_t)r * v->C + c]; cl = v->cb1_l; cr = v->cb1_r; }
            else {
                const uint8_t* jl = v->idx2_l + (size_t)r * l2_stride;
                const uint8_t* jr = v->idx2_r + (size_t)r * l2_stride;
                a = v->packed ? ((c & 1) ? (jl[c >> 1] >> 4) & 15 : jl[c >> 1] & 15) : jl[c];
                b = v->packed ? ((c & 1) ? (jr[c >> 1] >> 4) & 15 : jr[c >> 1] & 15) : jr[c];
                cl = v->cb2_l; cr = v->cb2_r;
            }
            for (int j = 0; j < v->half; j++) {
                float el = ibo_fp16_to_fp32(cl[a * v->half + j]), er = ibo_fp16_to_fp32(cr[b * v->half + j]);
                float xl = x[v->inner[base + j]], xr = x[v->inner[base + v->half + j]];
                if (fused) { acc = fmaf(el, xl, acc); acc = fmaf(er, xr, acc); }
                else { acc += el * xl; acc += er * xr; }
            }
        }
    }
    acc *= ibo_fp16_to_fp32(v->row_scale[r]);
    for (int j = 0; j < v->n_outlier; j++) {
        float w = (float)v->outlier_sidecar[(size_t)r * v->n_outlier + j] * ibo_fp16_to_fp32(v->outlier_scale[j]);
        if (fused) acc = fmaf(w, x[v->outlier_cols[j]], acc); else acc += w * x[v->outlier_cols[j]];
    }
    return acc;
}

static void heap_sift_down(float* val, int32_t* id, int n, int i) {
    for (;;) {
        int l = 2 * i + 1, r = l + 1, m = i;
        if (l < n && val[l] < val[m]) m = l;
        if (r < n && val[r] < val[m]) m = r;
        if (m == i) return;
        float tv = val[i]; val[i] = val[m]; val[m] = tv;
        int32_t ti = id[i]; id[i] = id[m]; id[m] = ti;
        i = m;
    }
}

/* src/pq_decode.c:2259-2341 (ib_pq_lm_head_topk): coarse logits from the first level over all rows; the K_top
 * largest kept in a min-heap seeded with rows 0..K_top-1 (a later row replaces the root only when strictly
 * larger); those rows refined with every level; insertion sort by refined logit, descending, which keeps the
 * heap's order among equal logits. coarse_out (may be NULL) receives the M coarse logits. */
int ibo_pq_lm_head_topk(int M, int N, int G, int K, int K_l2,
                        const uint16_t* cb1_l, const uint16_t* cb1_r, const uint16_t* cb2_l, const uint16_t* cb2_r,
                        const uint8_t* idx1_l, const uint8_t* idx1_r, const uint8_t* idx2_l, const uint8_t* idx2_r,
                        const uint16_t* row_scale, int n_outlier, const int32_t* outlier_cols,
                        const int8_t* outlier_sidecar, const uint16_t* outlier_scale,
                        const float* x, int K_top, float* out_logits, int32_t* out_ids, float* coarse_out, int fused) {
    if (!cb1_l || !cb1_r || !idx1_l || !idx1_r || !row_scale || !x || !out_logits || !out_ids) return -1;
    if (M <= 0 || N <= 0 || G <= 0 || (G & 1) || G > 32 || K <= 0 || K > 256 || n_outlier < 0 || (N - n_outlier) % G) return -1;
    if (K_top <= 0 || K_top > M) return -1;
    pq_view v;
    memset(&v, 0, sizeof v);
    v.M = M; v.N = N; v.G = G; v.K = K; v.K_l2 = K_l2; v.half = G / 2; v.n_outlier = n_outlier; v.C = (N - n_outlier) / G;
    v.two = cb2_l && cb2_r && idx2_l && idx2_r;
    if (v.two && (K_l2 <= 0 || K_l2 > 256)) return -1;
    v.packed = v.two && K_l2 == 16;
    v.cb1_l = cb1_l; v.cb1_r = cb1_r; v.cb2_l = cb2_l; v.cb2_r = cb2_r; v.row_scale = row_scale; v.outlier_scale = outlier_scale;
    v.idx1_l = idx1_l; v.idx1_r = idx1_r; v.idx2_l = idx2_l; v.idx2_r = idx2_r; v.outlier_cols = outlier_cols; v.outlier_sidecar = outlier_sidecar;
    int rc = -1;
    unsigned char* mask = (unsigned char*)calloc((size_t)N, 1);
    v.inner = (int*)malloc((size_t)(N - n_outlier) * sizeof(int));
    float* coarse = (float*)malloc((size_t)M * sizeof(float));
    float* tab = (float*)malloc((size_t)(2 * K + 32) * sizeof(float));
    float* val = (float*)malloc((size_t)K_top * sizeof(float));
    int32_t* id = (int32_t*)malloc((size_t)K_top * sizeof(int32_t));
    if (!mask || !v.inner || !coarse || !tab || !val || !id) goto done;
    for (int j = 0; j < n_outlier; j++) mask[outlier_cols[j]] = 1;
    { int kk = 0; for (int j = 0; j < N; j++) if (!mask[j] && kk < N - n_outlier) v.inner[kk++] = j; }
    pq_l1_only(&v, x, coarse, tab, tab + K, tab + 2 * K, fused);
    if (coarse_out) memcpy(coarse_out, coarse, (size_t)M * sizeof(float));
    for (int i = 0; i < K_top; i++) { id[i] = i; val[i] = coarse[i]; }
    for (int s = K_top / 2 - 1; s >= 0; s--) heap_sift_down(val, id, K_top, s);
    for (int j = K_top; j < M; j++)
        if (coarse[j] > val[0]) { val[0] = coarse[j]; id[0] = j; heap_sift_down(val, id, K_top, 0); }
    for (int i = 0; i < K_top; i++) val[i] = pq_row_full(&v, x, id[i], fused);
    for (int i = 1; i < K_top; i++) {
        float tv = val[i]; int32_t ti = id[i]; int j = i - 1;
        while (j >= 0 && val[j] < tv) { val[j + 1] = val[j]; id[j + 1] = id[j]; j--; }
        val[j + 1] = tv; id[j + 1] = ti;
    }
    memcpy(out_logits, val, (size_t)K_top * sizeof(float));
    memcpy(out_ids, id, (size_t)K_top * sizeof(int32_t));
    rc = 0;
done:
    free(mask); free(v.inner); free(coarse); free(tab); free(val); free(id);
    return rc;
}

/* src/pq_decode.c:3565-3651 (int4_matmul_rows_skip, scalar form) with the skip mask of :3854-3882 (build_skip_mask;
 * eps_act_rel <= 0 is the reference's default: no group is left out): group-scaled INT4 rows of the session engine.
 * gacc += lo * x[j] + hi * x[j + 1] per byte, acc += scale * gacc per group, then the row's outlier columns.
 * PARITY UNPINNED: static functions of the reference's session engine, reachable only through a model file of its
 * own format; `fused` picks whether products and sums contract as an -mfma build may. */
int ibo_int4g_matmul_fp32(int M, int N, int G, const uint8_t* q, const uint16_t* s, int K_out,
                          const uint16_t* outl_idx, const uint16_t* outl_val, const float* x, float* out,
                          float eps_act_rel, int fused) {
    if (!q || !s || !x || !out || M <= 0 || N <= 0 || G <= 0 || (G & 1) || N % G || K_out < 0) return -1;
    if (K_out > 0 && (!outl_idx || !outl_val)) return -1;
    const int ng = N / G;
    unsigned char* skip = NULL;
    if (eps_act_rel > 0.0f) {
        float xmax = 0.0f;
        for (int j = 0; j < N; j++) { float a = fabsf(x[j]); if (a > xmax) xmax = a; }
        const float thr = eps_act_rel * xmax;
        skip = (unsigned char*)malloc((size_t)ng);
        if (!skip) return -1;
        for (int g = 0; g < ng; g++) {
            float gm = 0.0f;
            for (int j = 0; j < G; j++) { float a = fabsf(x[g * G + j]); if (a > gm) gm = a; }
            skip[g] = gm <= thr;
        }
    }
    for (int m = 0; m < M; m++) {
        const uint8_t* qrow = q + (size_t)m * (N / 2);
        float acc = 0.0f;
        for (int g = 0; g < ng; g++) {
            if (skip && skip[g]) continue;
            const float scale = ibo_fp16_to_fp32(s[(size_t)m * ng + g]);
            const float* xg = x + g * G;
            float gacc = 0.0f;
            for (int j = 0; j < G; j += 2) {
                const uint8_t b = qrow[(g * G + j) / 2];
                const float lo = (float)((int)(b & 0x0F) - 8), hi = (float)((int)(b >> 4) - 8);
                if (fused) gacc += fmaf(lo, xg[j], hi * xg[j + 1]);
                else gacc += lo * xg[j] + hi * xg[j + 1];
            }
            if (fused) acc = fmaf(scale, gacc, acc); else acc += scale * gacc;
        }
        for (int k = 0; k < K_out; k++) {
            const float v = ibo_fp16_to_fp32(outl_val[(size_t)m * K_out + k]), xv = x[outl_idx[(size_t)m * K_out + k]];
            if (fused) acc = fmaf(v, xv, acc); else acc += v * xv;
        }
        out[m] = acc;
    }
    free(skip);
    return 0;
}

/* src/pq_decode.c:5008-5066 — encode of one K or V row into the PQ KV cache: per-vector scale max|v| / 7 (floor
 * 1e-12), normalise, nearest codeword per half chunk (distance accumulated in dimension order, strict '<').
 * PARITY UNPINNED: the reference has this only inline in its session step (no entry point to call), and its build
 * may or may not contract ed*ed + d; `fused` picks. */
void ibo_pqkv_encode(const float* vec, int dim, int G, int K1, const uint16_t* cb_l, const uint16_t* cb_r,
                     uint8_t* idx, float* scale, int fused) {
    int half = G / 2, C = dim / G;
    float m = 1e-12f;
    for (int d = 0; d < dim; d++) { float a = fabsf(vec[d]); if (a > m) m = a; }
    float s = m / 7.0f;
    if (s < 1e-12f) s = 1e-12f;
    float inv = 1.0f / s;
    *scale = s;
    for (int c = 0; c < C; c++) {
        for (int side = 0; side < 2; side++) {
            const uint16_t* cb = side ? cb_r : cb_l;
            int best = 0; float best_d = 1e30f;
            for (int k = 0; k < K1; k++) {
                float d = 0.0f;
                for (int j = 0; j < half; j++) {
                    float ed = vec[c * G + side * half + j] * inv - ibo_fp16_to_fp32(cb[(size_t)k * half + j]);
                    d = fused ? fmaf(ed, ed, d) : d + ed * ed;
                }
                if (d < best_d) { best_d = d; best = k; }
            }
            idx[side * C + c] = (uint8_t)best;
        }
    }
}

/* src/pq_decode.c:1103-1196 with n_levels == 1, no outliers. */
int ibo_pq_reconstruct_fp32(int M, int N, int G, int K,
                            const uint16_t* cb_l, const uint16_t* cb_r,
                            const uint8_t* idx_l, const uint8_t* idx_r, const uint16_t* row_scale,
                            float* W) {
    if (!cb_l || !cb_r || !idx_l || !idx_r || !row_scale || !W || G <= 0 || (G & 1) || N % G) return -1;
    (void)K;
    int half = G / 2, C = N / G;
    for (int r = 0; r < M; r++) {
        float s = ibo_fp16_to_fp32(row_scale[r]);
        for (int c = 0; c < C; c++) {
            const uint16_t* el = cb_l + (size_t)idx_l[(size_t)r * C + c] * half;
            const uint16_t* er = cb_r + (size_t)idx_r[(size_t)r * C + c] * half;
            float* dst = W + (size_t)r * N + (size_t)c * G;
            for (int i = 0; i < half; i++) {
                dst[i]        = ibo_fp16_to_fp32(ibo_fp32_to_fp16(ibo_fp16_to_fp32(el[i]) * s));
                dst[half + i] = ibo_fp16_to_fp32(ibo_fp32_to_fp16(ibo_fp16_to_fp32(er[i]) * s));
            }
        }
    }
    return 0;
}

/* ── k-means ─────────────────────────────────────────────────────────────────────────── */

/* src/pq_kmeans.c:99-106. `fused` selects how s += v*v rounds:
 *   0  multiply then add (two roundings) for every d;
 *   1  fmaf for every d;
 *   2  what the reference's x86-64 Release build (gcc 13, -O3 -mavx2 -mfma, contraction on)
 *      actually executes: gcc vectorises the loop four dimensions at a time with an in-order
 *      reduction (vector multiply, then scalar adds: unfused) and contracts only the scalar
 *      remainder loop, so dimensions below 4*floor(D/4) are unfused and the last D%4 are fused.
 *      Established by running the compiled reference on near-tie inputs for D = 1..32
 *      (tests/test_oracle_vs_ref.py::test_kmeans_rounding_mode). */
static float sqdist(const float* x, const float* c, int D, int fused) {
    float s = 0.0f;
    int body = fused == 0 ? D : (fused == 1 ? 0 : (D & ~3));
    for (int d = 0; d < body; d++) { float v = x[d] - c[d]; s = s + v * v; }
    for (int d = body; d < D; d++) { float v = x[d] - c[d]; s = fmaf(v, v, s); }
    return s;
}

/* src/pq_kmeans.c:111-122 — centroid 0 seeds the best; a later one wins only when strictly
 * closer, so the lowest index wins ties and a NaN distance never wins. */
static int nearest(const float* x, const float* C, int K, int D, int fused, float* dist) {
    int arg = 0;
    float best = sqdist(x, C, D, fused);
    for (int k = 1; k < K; k++) {
        float d = sqdist(x, C + (size_t)k * D, D, fused);
        if (d < best) { best = d; arg = k; }
    }
    *dist = best;
    return arg;
}

void ibo_kmeans_assign(const float* X, long N, int D, const float* C, int K,
                       int32_t* idx, float* dist_out, int fused) {
    for (long i = 0; i < N; i++) {
        float d;
        idx[i] = nearest(X + (size_t)i * D, C, K, D, fused, &d);
        if (dist_out) dist_out[i] = d;
    }
}

/* src/pq_kmeans.c:252-283 */
float ibo_kmeans_update(float* C, int K, int D, const float* sums, const int32_t* counts) {
    float shift = 0.0f;
    for (int k = 0; k < K; k++) {
        if (counts[k] <= 0) continue;                 /* empty cluster: centroid stays */
        float inv = 1.0f / (float)counts[k];
        for (int d = 0; d < D; d++) {
            float nv = sums[(size_t)k * D + d] * inv;
            float mv = nv - C[(size_t)k * D + d];
            shift += mv * mv;
            C[(size_t)k * D + d] = nv;
        }
    }
    return shift;
}

/* src/pq_kmeans.c:183-201 on one lane, followed by the update above. */
float ibo_kmeans_lloyd_iter(const float* X, long N, int D, float* C, int K, int32_t* idx,
                            float* sums, int32_t* counts, double* inertia, int fused) {
    memset(sums, 0, (size_t)K * D * sizeof(float));
    memset(counts, 0, (size_t)K * sizeof(int32_t));
    double tot = 0.0;
    for (long i = 0; i < N; i++) {
        const float* xi = X + (size_t)i * D;
        float d;
        int k = nearest(xi, C, K, D, fused, &d);
        if (idx) idx[i] = k;
        counts[k]++;
        for (int j = 0; j < D; j++) sums[(size_t)k * D + j] += xi[j];
        tot += (double)d;
    }
    if (inertia) *inertia = tot;
    return ibo_kmeans_update(C, K, D, sums, counts);
}

/* ── element-wise glue (src/kernels/scalar.c:126-181) ────────────────────────────────── */

void ibo_rmsnorm(float* out, const float* x, const float* w, float eps, int N) {
    float ss = 0.0f;
    for (int i = 0; i < N; i++) ss += x[i] * x[i];
    float r = 1.0f / sqrtf(ss / (float)N + eps);
    for (int i = 0; i < N; i++) out[i] = x[i] * r * w[i];
}

/* Adjacent pairs (2m, 2m+1); freq = 1/powf(theta, 2m/head_dim). */
void ibo_rope(float* q, float* k, int head_dim, int pos, float theta) {
    for (int i = 0; i + 1 < head_dim; i += 2) {
        float ang = (float)pos * (1.0f / powf(theta, (float)i / (float)head_dim));
        float c = cosf(ang), s = sinf(ang);
        float a = q[i], b = q[i + 1];
        q[i] = a * c - b * s;  q[i + 1] = a * s + b * c;
        if (k) { a = k[i]; b = k[i + 1]; k[i] = a * c - b * s;  k[i + 1] = a * s + b * c; }
    }
}

void ibo_softmax(float* v, int N) {
    float mx = v[0];
    for (int i = 1; i < N; i++) if (v[i] > mx) mx = v[i];
    float tot = 0.0f;
    for (int i = 0; i < N; i++) { v[i] = expf(v[i] - mx); tot += v[i]; }
    float inv = 1.0f / tot;
    for (int i = 0; i < N; i++) v[i] *= inv;
}

void ibo_silu_mul(float* out, const float* gate, const float* up, int N) {
    for (int i = 0; i < N; i++) out[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}

/* ── decode step ─────────────────────────────────────────────────────────────────────── */

/* src/forward.c:144-185 / :200-246 with IB_W4A8=0: fp16 scales widened per call, then the table
 * kernel for the tensor's bit width; B positions -> int8 batch kernel or one INT4 call each. */
static void linear(const ibo_linear* t, const float* x, float* out, int B, float* scale_buf) {
    ibo_fp16_array_to_fp32(t->scale, scale_buf, t->M);
    if (t->bits == 8) ibo_matmul_int8_batch(out, (const int8_t*)t->w, scale_buf, x, t->M, t->N, B, t->M);
    else              ibo_matmul_int4_batch(out, (const uint8_t*)t->w, scale_buf, x, t->M, t->N, B, t->M);
}

static void norm_fp16(float* out, const float* x, const uint16_t* w16, float eps, int N, float* wbuf) {
    ibo_fp16_array_to_fp32(w16, wbuf, N);
    ibo_rmsnorm(out, x, wbuf, eps, N);
}

/* src/forward.c:463-504 — one query head against its KV head's cache rows 0..pos. */
static void attend(const ibo_model* m, const ibo_layer* L, const float* q, int h, int pos,
                   float* att, float* out) {
    int hd = m->head_dim, kv_dim = m->n_kv_heads * hd;
    int kvh = h / (m->n_heads / m->n_kv_heads);
    float sc = 1.0f / sqrtf((float)hd);
    for (int t = 0; t <= pos; t++) {
        const float* kt = L->k_cache + (size_t)t * kv_dim + (size_t)kvh * hd;
        float s = 0.0f;
        for (int d = 0; d < hd; d++) s += q[d] * kt[d];
        att[t] = s * sc;
    }
    ibo_softmax(att, pos + 1);
    for (int d = 0; d < hd; d++) out[d] = 0.0f;
    for (int t = 0; t <= pos; t++) {
        const float* vt = L->v_cache + (size_t)t * kv_dim + (size_t)kvh * hd;
        for (int d = 0; d < hd; d++) out[d] += att[t] * vt[d];
    }
}

/* src/forward.c:518-664 (B == 1) and :682-846 (B > 1, consecutive positions of one sequence). */
int ibo_decode_step(ibo_model* m, const int32_t* tokens, int pos0, int B,
                    float* logits, float* hidden_out) {
    if (!m || !tokens || B < 1 || B > 32 || pos0 < 0 || pos0 + B > m->max_ctx) return -1;
    int H = m->hidden, I = m->inter, hd = m->head_dim;
    int kv_dim = m->n_kv_heads * hd, group = m->n_heads / m->n_kv_heads;
    int big = H > I ? H : I; if (m->vocab > big) big = m->vocab;
    size_t nf = (size_t)B * (4 * (size_t)H + 2 * (size_t)kv_dim + 2 * (size_t)I) + (size_t)big + (size_t)m->max_ctx + 8;
    float* buf = (float*)malloc(nf * sizeof(float));
    if (!buf) return -1;
    float* x = buf;               float* xb = x + (size_t)B * H;    float* xa = xb + (size_t)B * H;
    float* q = xa + (size_t)B * H; float* k = q + (size_t)B * H;     float* v = k + (size_t)B * kv_dim;
    float* hg = v + (size_t)B * kv_dim; float* hu = hg + (size_t)B * I;
    float* tmp = hu + (size_t)B * I;    float* att = tmp + big;

    for (int b = 0; b < B; b++) {                       /* src/forward.c:94-106 */
        const int8_t* row = m->embed + (size_t)tokens[b] * H;
        float s = ibo_fp16_to_fp32(m->embed_scale[tokens[b]]);
        for (int i = 0; i < H; i++) x[(size_t)b * H + i] = (float)row[i] * s;
    }
    for (int l = 0; l < m->n_layers; l++) {
        ibo_layer* L = &m->layers[l];
        for (int b = 0; b < B; b++) norm_fp16(xb + (size_t)b * H, x + (size_t)b * H, L->input_norm, m->eps, H, tmp);
        linear(&L->q, xb, q, B, tmp);
        linear(&L->k, xb, k, B, tmp);
        linear(&L->v, xb, v, B, tmp);
        for (int b = 0; b < B; b++) {
            int pos = pos0 + b;
            float* qb = q + (size_t)b * H; float* kb = k + (size_t)b * kv_dim; float* vb = v + (size_t)b * kv_dim;
            for (int h = 0; h < m->n_heads; h++)        /* K head rotated once, by its first Q head */
                ibo_rope(qb + (size_t)h * hd, (h % group == 0) ? kb + (size_t)(h / group) * hd : NULL, hd, pos, m->theta);
            memcpy(L->k_cache + (size_t)pos * kv_dim, kb, (size_t)kv_dim * sizeof(float));
            memcpy(L->v_cache + (size_t)pos * kv_dim, vb, (size_t)kv_dim * sizeof(float));
            for (int h = 0; h < m->n_heads; h++)
                attend(m, L, qb + (size_t)h * hd, h, pos, att, xa + (size_t)b * H + (size_t)h * hd);
        }
        linear(&L->o, xa, xb, B, tmp);
        for (size_t i = 0; i < (size_t)B * H; i++) x[i] += xb[i];
        for (int b = 0; b < B; b++) norm_fp16(xb + (size_t)b * H, x + (size_t)b * H, L->post_attn_norm, m->eps, H, tmp);
        linear(&L->gate, xb, hg, B, tmp);
        linear(&L->up, xb, hu, B, tmp);
        for (int b = 0; b < B; b++) ibo_silu_mul(hg + (size_t)b * I, hg + (size_t)b * I, hu + (size_t)b * I, I);
        linear(&L->down, hg, xb, B, tmp);
        for (size_t i = 0; i < (size_t)B * H; i++) x[i] += xb[i];
    }
    if (logits || hidden_out) {
        for (int b = 0; b < B; b++) norm_fp16(x + (size_t)b * H, x + (size_t)b * H, m->final_norm, m->eps, H, tmp);
        if (hidden_out) memcpy(hidden_out, x, (size_t)B * H * sizeof(float));
        if (logits) linear(&m->head, x, logits, B, tmp);
    }
    free(buf);
    return 0;
}
