/* Reader for the product-quantised model files ("IBF v5") behind the reference's ib_pq_load_single / ib_pq_load_multi
 * (src/pq_decode.h:89-135; format and checks as read by src/pq_decode.c:391-546 and :726-852), with the reference's
 * own names, plus forwarders that run a loaded tensor on the GPU.
 *
 * File: 32-byte preamble ("INFERBIT", version 5 at byte 8, header length at byte 12, both little-endian uint32), a JSON
 * header of that length, then the blocks. Header: "weight_data_start" (file offset that block offsets count from),
 * "tensors" {name: {"format", "shape": [M, N], "G", "K", "n_levels", "rotate", "K_l2", "l2_packed_bits",
 * "outlier": {"n_cols"}, and one {"offset", "size"} member per block}}, optionally "raw_tensors" {name: {"dtype", "shape",
 * "offset", "size"}} and a free-form "config" object. */
#include "inferbit_gpu.h"
#include "ib_b200.h"
#include "ibf_json.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

enum { V5_PREAMBLE = 32, V5_VERSION = 5 };
enum { FMT_NONE = 0, FMT_L1, FMT_L2, FMT_L1_L2, FMT_PYRAMID };      /* ib_pq_format, src/pq_decode.h:26-37 */

static int parse_format(const char* s) {
    if (!s) return FMT_NONE;
    if (!strcmp(s, "pq2d_v1_l1")) return FMT_L1;
    if (!strcmp(s, "pq2d_v1_l2")) return FMT_L2;
    if (!strcmp(s, "pq2d_v1_l1_l2")) return FMT_L1_L2;
    if (!strcmp(s, "pq2d_v1_pyramid")) return FMT_PYRAMID;
    return FMT_NONE;
}

/* n_bits-wide little-endian fields, one after the other, to uint16 (src/pq_decode.c:1078-1095) */
static void unpack_bits_u16(const uint8_t* src, size_t src_len, uint16_t* dst, size_t n, int n_bits) {
    const uint32_t mask = n_bits == 16 ? 0xFFFFu : ((1u << n_bits) - 1u);
    size_t bit = 0;
    for (size_t i = 0; i < n; i++, bit += (size_t)n_bits) {
        const size_t b = bit >> 3;
        uint32_t w = 0;
        for (int k = 0; k < 3; k++) if (b + (size_t)k < src_len) w |= (uint32_t)src[b + (size_t)k] << (8 * k);
        dst[i] = (uint16_t)((w >> (bit & 7)) & mask);
    }
}

typedef struct { FILE* f; ibj_node* root; size_t data_start, file_size; } v5_file;

static void v5_close(v5_file* v) {
    if (v->root) ibj_free(v->root);
    if (v->f) fclose(v->f);
    memset(v, 0, sizeof *v);
}

static int v5_open(const char* path, v5_file* v) {
    memset(v, 0, sizeof *v);
    v->f = fopen(path, "rb");
    if (!v->f) return -1;
    if (fseek(v->f, 0, SEEK_END) != 0) { v5_close(v); return -1; }
    const long sz = ftell(v->f);
    if (sz < V5_PREAMBLE) { v5_close(v); return -1; }
    v->file_size = (size_t)sz;
    rewind(v->f);
    uint8_t pre[V5_PREAMBLE];
    if (fread(pre, 1, V5_PREAMBLE, v->f) != V5_PREAMBLE || memcmp(pre, "INFERBIT", 8) != 0) { v5_close(v); return -1; }
    uint32_t version, hlen;
    memcpy(&version, pre + 8, 4);
    memcpy(&hlen, pre + 12, 4);
    if (version != V5_VERSION || (size_t)hlen > v->file_size - V5_PREAMBLE) { v5_close(v); return -1; }
    char* text = (char*)malloc((size_t)hlen + 1);
    if (!text) { v5_close(v); return -1; }
    if (fread(text, 1, hlen, v->f) != hlen) { free(text); v5_close(v); return -1; }
    size_t n = hlen;
    while (n > 0 && (text[n - 1] == '\0' || text[n - 1] == ' ' || text[n - 1] == '\n')) n--;       /* the header is padded to its reserved length */
    size_t err_at = 0;
    v->root = ibj_parse(text, n, &err_at);
    free(text);
    if (!v->root) { v5_close(v); return -1; }
    v->data_start = (size_t)ibj_num(v->root, "weight_data_start", 0);
    return 0;
}

/* block `key` of tensor header tm, which must be `want` bytes long and lie inside the file, into dst */
static int read_block(v5_file* v, const ibj_node* tm, const char* key, void* dst, size_t want) {
    const ibj_node* b = ibj_get(tm, key);
    if (!b || b->type != IBJ_OBJ) return -1;
    const double off = ibj_num(b, "offset", -1), sz = ibj_num(b, "size", 0);
    if (off < 0 || (size_t)sz != want) return -1;
    const size_t at = v->data_start + (size_t)off;
    if (at + want > v->file_size) return -1;
    if (fseek(v->f, (long)at, SEEK_SET) != 0) return -1;
    return fread(dst, 1, want, v->f) == want ? 0 : -1;
}

static int load_tensor(v5_file* v, const ibj_node* tm, ib_b200_pq_tensor* out) {
    memset(out, 0, sizeof *out);
    out->format = parse_format(ibj_str(tm, "format", ""));
    if (out->format == FMT_NONE) return -1;
    const ibj_node* shape = ibj_get(tm, "shape");
    if (!shape || shape->type != IBJ_ARR || ibj_len(shape) != 2) return -1;
    out->M = (int)ibj_at(shape, 0)->num;
    out->N = (int)ibj_at(shape, 1)->num;
    out->G = (int)ibj_num(tm, "G", 0);
    out->K = (int)ibj_num(tm, "K", 0);
    out->n_levels = (int)ibj_num(tm, "n_levels", 0);
    out->rotate = ibj_bool(tm, "rotate", 0);
    const ibj_node* outl = ibj_get(tm, "outlier");
    out->n_outlier = (outl && outl->type == IBJ_OBJ) ? (int)ibj_num(outl, "n_cols", 0) : 0;
    out->K_l2 = (int)ibj_num(tm, "K_l2", 0);
    const int M = out->M, G = out->G, K = out->K, n_inner = out->N - out->n_outlier;
    if (M <= 0 || G <= 0 || K <= 0 || (G & 1) || out->n_outlier < 0 || n_inner <= 0 || n_inner % G) return -1;
    const int C = out->C = n_inner / G;
    const int K2 = out->K_l2 > 0 ? out->K_l2 : K;
    if (out->n_levels == 2 && out->format != FMT_PYRAMID && K2 != 16 && K2 != 64 && K2 != K) return -1;      /* src/pq_decode.c:425-427 */
    const int packed4 = K2 == 16;
    out->l2_idx_bytes = (out->format == FMT_PYRAMID && K2 > 256) ? 2 : 1;
    out->l2_packed_bits = (int)ibj_num(tm, "l2_packed_bits", 0);
    if (out->l2_packed_bits < 0 || out->l2_packed_bits > 16) return -1;
    const int bitpacked = out->n_levels == 2 && out->l2_packed_bits > 0 && !packed4;      /* on disk n-bit fields, in memory uint16 */
    const size_t l2_row = packed4 ? (size_t)((C + 1) / 2) : (size_t)C * (size_t)(bitpacked ? 2 : out->l2_idx_bytes);
    const size_t l2_row_disk = bitpacked ? ((size_t)C * (size_t)out->l2_packed_bits + 7) >> 3 : l2_row;
    const size_t cb = (size_t)K * (G / 2) * 2, cb2 = (size_t)K2 * (G / 2) * 2, idx = (size_t)M * C, idx2 = (size_t)M * l2_row,
                 rs = (size_t)M * 2, oc = (size_t)out->n_outlier * 4, os = (size_t)M * out->n_outlier, osc = (size_t)out->n_outlier * 2;
    size_t total = 2 * cb + 2 * idx + rs + 16;
    if (out->n_levels == 2) total += 2 * cb2 + 2 * idx2 + 16;
    if (out->n_outlier > 0) total += oc + os + osc + 16;
    uint8_t* arena = (uint8_t*)malloc(total);
    if (!arena) return -1;
    out->_arena = arena; out->_arena_size = total;
    size_t cur = 0;
#define TAKE(field, type, bytes) do { (field) = (type*)(arena + cur); cur += ((bytes) + 3) & ~(size_t)3; } while (0)
    TAKE(out->codebook_l1_l, uint16_t, cb); TAKE(out->codebook_l1_r, uint16_t, cb);
    TAKE(out->indices_l1_l, uint8_t, idx);  TAKE(out->indices_l1_r, uint8_t, idx);
    TAKE(out->row_scale, uint16_t, rs);
    int rc = read_block(v, tm, "codebook_l1_l", out->codebook_l1_l, cb) | read_block(v, tm, "codebook_l1_r", out->codebook_l1_r, cb) |
             read_block(v, tm, "indices_l1_l", out->indices_l1_l, idx) | read_block(v, tm, "indices_l1_r", out->indices_l1_r, idx) |
             read_block(v, tm, "row_scale", out->row_scale, rs);
    if (!rc && out->n_levels == 2) {
        TAKE(out->codebook_l2_l, uint16_t, cb2); TAKE(out->codebook_l2_r, uint16_t, cb2);
        TAKE(out->indices_l2_l, uint8_t, idx2);  TAKE(out->indices_l2_r, uint8_t, idx2);
        rc = read_block(v, tm, "codebook_l2_l", out->codebook_l2_l, cb2) | read_block(v, tm, "codebook_l2_r", out->codebook_l2_r, cb2);
        if (!rc && bitpacked) {
            const size_t disk = (size_t)M * l2_row_disk;
            uint8_t* tmp = (uint8_t*)malloc(disk ? disk : 1);
            if (!tmp) rc = -1;
            for (int side = 0; !rc && side < 2; side++) {
                rc = read_block(v, tm, side ? "indices_l2_r" : "indices_l2_l", tmp, disk);
                uint16_t* dst = (uint16_t*)(side ? out->indices_l2_r : out->indices_l2_l);
                for (int r = 0; !rc && r < M; r++)
                    unpack_bits_u16(tmp + (size_t)r * l2_row_disk, l2_row_disk, dst + (size_t)r * C, (size_t)C, out->l2_packed_bits);
            }
            free(tmp);
        } else if (!rc) {
            rc = read_block(v, tm, "indices_l2_l", out->indices_l2_l, idx2) | read_block(v, tm, "indices_l2_r", out->indices_l2_r, idx2);
        }
    }
    if (!rc && out->n_outlier > 0) {
        TAKE(out->outlier_cols, int32_t, oc); TAKE(out->outlier_sidecar, int8_t, os); TAKE(out->outlier_scale, uint16_t, osc);
        rc = read_block(v, tm, "outlier_cols", out->outlier_cols, oc) | read_block(v, tm, "outlier_sidecar", out->outlier_sidecar, os) |
             read_block(v, tm, "outlier_scale", out->outlier_scale, osc);
    }
#undef TAKE
    if (rc) { free(arena); memset(out, 0, sizeof *out); return -1; }
    return 0;
}

IBG_API void ib_pq_free(ib_b200_pq_tensor* t) {
    if (!t) return;
    ib_b200_pq_release(t);                                    /* the copy in HBM, if the tensor was ever used */
    free(t->_arena);
    memset(t, 0, sizeof *t);
}

IBG_API int ib_pq_load_single(const char* path, ib_b200_pq_tensor* out) {
    if (!out || !path) return -1;
    memset(out, 0, sizeof *out);
    v5_file v;
    if (v5_open(path, &v)) return -1;
    const ibj_node* tensors = ibj_get(v.root, "tensors");
    int rc = -1;
    if (tensors && tensors->type == IBJ_OBJ && tensors->child) rc = load_tensor(&v, tensors->child, out);
    v5_close(&v);
    return rc;
}

/* JSON text of a subtree, without spaces: what config_json holds */
typedef struct { char* s; size_t n, cap; int bad; } sbuf;
static void put(sbuf* b, const char* p, size_t n) {
    if (b->bad) return;
    if (b->n + n + 1 > b->cap) {
        size_t cap = b->cap ? b->cap * 2 : 256;
        while (cap < b->n + n + 1) cap *= 2;
        char* s = (char*)realloc(b->s, cap);
        if (!s) { b->bad = 1; return; }
        b->s = s; b->cap = cap;
    }
    memcpy(b->s + b->n, p, n); b->n += n; b->s[b->n] = '\0';
}
static void put_str(sbuf* b, const char* s) {
    put(b, "\"", 1);
    for (; s && *s; s++) {
        const unsigned char c = (unsigned char)*s;
        if (c == '"' || c == '\\') { char e[2] = { '\\', (char)c }; put(b, e, 2); }
        else if (c == '\n') put(b, "\\n", 2);
        else if (c == '\t') put(b, "\\t", 2);
        else if (c == '\r') put(b, "\\r", 2);
        else if (c < 0x20) { char e[8]; snprintf(e, sizeof e, "\\u%04x", c); put(b, e, 6); }
        else put(b, (const char*)&c, 1);
    }
    put(b, "\"", 1);
}
static void put_node(sbuf* b, const ibj_node* n) {
    char num[40];
    switch (n->type) {
    case IBJ_NULL: put(b, "null", 4); break;
    case IBJ_BOOL: if (n->num != 0) put(b, "true", 4); else put(b, "false", 5); break;
    case IBJ_NUM:
        if (n->num == (double)(long long)n->num && n->num > -1e15 && n->num < 1e15) snprintf(num, sizeof num, "%lld", (long long)n->num);
        else snprintf(num, sizeof num, "%.17g", n->num);
        put(b, num, strlen(num)); break;
    case IBJ_STR: put_str(b, n->str); break;
    default:
        put(b, n->type == IBJ_OBJ ? "{" : "[", 1);
        for (const ibj_node* m = n->child; m; m = m->next) {
            if (n->type == IBJ_OBJ) { put_str(b, m->key); put(b, ":", 1); }
            put_node(b, m);
            if (m->next) put(b, ",", 1);
        }
        put(b, n->type == IBJ_OBJ ? "}" : "]", 1);
    }
}

IBG_API void ib_pq_multi_free(ib_b200_pq_multi* m) {
    if (!m) return;
    for (int i = 0; m->names && i < m->n; i++) free(m->names[i]);
    free(m->names);
    for (int i = 0; m->tensors && i < m->n; i++) ib_pq_free(&m->tensors[i]);
    free(m->tensors);
    for (int i = 0; m->raw_tensors && i < m->n_raw; i++) {
        free(m->raw_tensors[i].name);
        if (m->raw_tensors[i]._owns_data) free(m->raw_tensors[i].data);
    }
    free(m->raw_tensors);
    free(m->config_json);
    memset(m, 0, sizeof *m);
}

IBG_API int ib_pq_load_multi(const char* path, ib_b200_pq_multi* out) {
    if (!out || !path) return -1;
    memset(out, 0, sizeof *out);
    v5_file v;
    if (v5_open(path, &v)) return -1;
    const ibj_node* tensors = ibj_get(v.root, "tensors");
    if (!tensors || tensors->type != IBJ_OBJ) { v5_close(&v); return -1; }
    const int n = ibj_len(tensors);
    if (n > 0) {
        out->names = (char**)calloc((size_t)n, sizeof(char*));
        out->tensors = (ib_b200_pq_tensor*)calloc((size_t)n, sizeof(ib_b200_pq_tensor));
        if (!out->names || !out->tensors) { v5_close(&v); ib_pq_multi_free(out); return -1; }
    }
    int i = 0;
    for (const ibj_node* it = tensors->child; it; it = it->next, i++) {
        out->n = i + 1;                                       /* what a failure below has to free */
        out->names[i] = strdup(it->key ? it->key : "");
        if (!out->names[i] || load_tensor(&v, it, &out->tensors[i])) { v5_close(&v); ib_pq_multi_free(out); return -1; }
    }
    const ibj_node* raws = ibj_get(v.root, "raw_tensors");
    const int rn = (raws && raws->type == IBJ_OBJ) ? ibj_len(raws) : 0;
    if (rn > 0) {
        out->raw_tensors = (ib_b200_pq_raw_tensor*)calloc((size_t)rn, sizeof(ib_b200_pq_raw_tensor));
        if (!out->raw_tensors) { v5_close(&v); ib_pq_multi_free(out); return -1; }
        static const char* const dtypes[] = { "float32", "float16", "int32", "int16", "int8", "uint8", "uint16" };   /* ib_raw_dtype, src/pq_decode.h:98-106 */
        int ri = 0;
        for (const ibj_node* it = raws->child; it; it = it->next, ri++) {
            ib_b200_pq_raw_tensor* rt = &out->raw_tensors[ri];
            out->n_raw = ri + 1;
            rt->name = strdup(it->key ? it->key : "");
            const char* dt = ibj_str(it, "dtype", "float32");
            rt->dtype = -1;
            for (int d = 0; d < 7; d++) if (!strcmp(dt, dtypes[d])) rt->dtype = d;
            const ibj_node* shape = ibj_get(it, "shape");
            rt->ndim = (shape && shape->type == IBJ_ARR) ? ibj_len(shape) : 0;
            if (rt->ndim > 4) rt->ndim = 4;
            for (int d = 0; d < rt->ndim; d++) rt->shape[d] = (int)ibj_at(shape, d)->num;
            const ibj_node* oit = ibj_get(it, "offset");
            const ibj_node* sit = ibj_get(it, "size");
            int bad = !rt->name || rt->dtype < 0 || !oit || oit->type != IBJ_NUM || !sit || sit->type != IBJ_NUM;
            if (!bad) {
                rt->size_bytes = (size_t)sit->num;
                const size_t at = v.data_start + (size_t)oit->num;
                rt->data = malloc(rt->size_bytes ? rt->size_bytes : 1);
                rt->_owns_data = 1;
                bad = !rt->data || at + rt->size_bytes > v.file_size || fseek(v.f, (long)at, SEEK_SET) != 0 ||
                      fread(rt->data, 1, rt->size_bytes, v.f) != rt->size_bytes;
            }
            if (bad) { v5_close(&v); ib_pq_multi_free(out); return -1; }
        }
    }
    const ibj_node* cfg = ibj_get(v.root, "config");
    if (cfg && cfg->type == IBJ_OBJ) {
        sbuf b = { 0 };
        put_node(&b, cfg);
        if (b.bad) free(b.s); else out->config_json = b.s;
    }
    v5_close(&v);
    return 0;
}

IBG_API const ib_b200_pq_tensor* ib_pq_multi_find(const ib_b200_pq_multi* m, const char* name) {
    if (!m || !name) return NULL;
    for (int i = 0; i < m->n; i++) if (m->names[i] && !strcmp(m->names[i], name)) return &m->tensors[i];
    return NULL;
}

/* The reference's matvec names over the GPU host layer (src/pq_decode.h:189-222, :2259) */
IBG_API int ib_pq_matmul_fp32(const ib_b200_pq_tensor* t, const float* x, float* out) { return ib_b200_pq_matmul_fp32(t, x, out); }
IBG_API int ib_pq_lm_head_topk(const ib_b200_pq_tensor* t, const float* x, int K_top, float* out_logits, int32_t* out_token_ids) {
    return ib_b200_pq_lm_head_topk(t, x, K_top, out_logits, out_token_ids);
}
