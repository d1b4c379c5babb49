/*
 * The reference's public entry points for this path (include/inferbit.h:43-135 in the reference checkout)
 * over the B200 backend: configuration, the IBF-v1 reader with upload to HBM, forward, KV-cache control,
 * model info and the thread-local error string. Built as libinferbit.so beside the other two libraries.
 */
#include "inferbit_gpu.h"
#include "ib_b200.h"
#include "ibf_json.h"

#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#define IBF_PREAMBLE 32
#define IBF_VERSION 1
#define BATCH_MAX 32                    /* IB_BATCH_MAX, src/inferbit_internal.h:287 */

/* ── error string (src/error.c:5-22) ── */
static _Thread_local char err_buf[512];
static _Thread_local int err_set;

static void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf, sizeof err_buf, fmt, ap);
    va_end(ap);
    err_set = 1;
}
const char* inferbit_last_error(void) {
    if (!err_set) return NULL;
    err_set = 0;
    return err_buf;
}

/* ── configuration (src/config.c) ── */
struct inferbit_config { int threads, context_length, kv_dynamic, native_parse, native_bits; };

inferbit_config* inferbit_config_create(void) {
    inferbit_config* c = (inferbit_config*)calloc(1, sizeof *c);
    if (!c) { set_error("failed to allocate config"); return NULL; }
    c->native_bits = 4;
    return c;
}
void inferbit_config_free(inferbit_config* c) { free(c); }
void inferbit_config_set_threads(inferbit_config* c, int v) { if (c) c->threads = v; }
void inferbit_config_set_context_length(inferbit_config* c, int v) { if (c) c->context_length = v; }
void inferbit_config_set_kv_cache_dynamic(inferbit_config* c, int v) { if (c) c->kv_dynamic = v != 0; }
void inferbit_config_set_native_parse(inferbit_config* c, int v) { if (c) c->native_parse = v != 0; }
void inferbit_config_set_native_bits(inferbit_config* c, int v) { if (c) c->native_bits = v; }

/* ── model ── */
typedef struct { size_t offset, size, scale_offset, scale_size; int bits; } tmeta;

struct inferbit_model {
    ib_b200_model* m;
    char architecture[64];
    int num_layers, hidden, vocab, max_context, default_bits, kv_bits, num_kv_heads, head_dim;
    int capacity;                       /* KV rows allocated = the context limit enforced */
    int kv_len;
    size_t weight_bytes;
};

static tmeta read_tensor(const ibj_node* obj) {      /* src/ibf_loader.c:66-90 */
    tmeta t;
    memset(&t, 0, sizeof t);
    if (!obj || obj->type != IBJ_OBJ) return t;
    t.offset = (size_t)ibj_num(obj, "offset", 0);
    t.size = (size_t)ibj_num(obj, "size", 0);
    t.bits = (int)ibj_num(obj, "bits", 16);
    t.scale_offset = (size_t)ibj_num(obj, "scale_offset", 0);
    t.scale_size = (size_t)ibj_num(obj, "scale_size", 0);
    return t;
}

static int ends_with(const char* s, const char* suf) {
    const size_t a = strlen(s), b = strlen(suf);
    return b <= a && !strcmp(s + a - b, suf);
}

/* a tensor's bytes inside the mapped data section, or NULL with the error set */
static const void* span(const unsigned char* data, size_t data_size, size_t off, size_t need, const char* what) {
    if (off > data_size || need > data_size - off) {
        set_error("IBF tensor %s lies outside the weight data (offset %zu + %zu > %zu)", what, off, need, data_size);
        return NULL;
    }
    return data + off;
}

static int upload_linear(ib_b200_model* m, int layer, int which, const tmeta* t, int M, int N,
                         const unsigned char* data, size_t data_size, const char* name) {
    const size_t rb = t->bits == 8 ? (size_t)N : (size_t)N / 2;
    const void* w = span(data, data_size, t->offset, (size_t)M * rb, name);
    if (!w) return -1;
    const void* s = NULL;
    if (t->scale_offset || t->scale_size) {            /* src/forward.c:31-34 */
        s = span(data, data_size, t->scale_offset, (size_t)M * 2, name);
        if (!s) return -1;
    }
    const int rc = ib_b200_model_set_linear(m, layer, which, w, (const uint16_t*)s);
    if (rc) { set_error("uploading %s to the GPU failed (%d): %s", name, rc, ibcu_last_error(ib_b200_ctx())); return -1; }
    return 0;
}

inferbit_model* inferbit_load(const char* path, const inferbit_config* config) {
    if (!path) { set_error("path is NULL"); return NULL; }
    if (config && config->native_parse) { set_error("native parse mode not yet implemented"); return NULL; }
    if (!ends_with(path, ".ibf")) { set_error("expected .ibf file (use native_parse mode for safetensors/GGUF)"); return NULL; }

    const int fd = open(path, O_RDONLY);
    if (fd < 0) { set_error("failed to open %s: %s", path, strerror(errno)); return NULL; }
    struct stat st;
    if (fstat(fd, &st) < 0) { set_error("failed to stat %s: %s", path, strerror(errno)); close(fd); return NULL; }
    const size_t file_size = (size_t)st.st_size;
    if (file_size < IBF_PREAMBLE) { set_error("file too small to be IBF: %zu bytes", file_size); close(fd); return NULL; }
    unsigned char pre[IBF_PREAMBLE];
    if (read(fd, pre, IBF_PREAMBLE) != IBF_PREAMBLE) { set_error("failed to read IBF preamble"); close(fd); return NULL; }
    if (memcmp(pre, "INFERBIT", 8) != 0) { set_error("invalid IBF magic number"); close(fd); return NULL; }
    uint32_t version, header_size;
    memcpy(&version, pre + 8, 4);
    memcpy(&header_size, pre + 12, 4);
    if (version > IBF_VERSION) { set_error("unsupported IBF version: %u (max supported: %u)", version, IBF_VERSION); close(fd); return NULL; }
    if ((size_t)IBF_PREAMBLE + header_size > file_size) { set_error("IBF header size exceeds file size"); close(fd); return NULL; }

    unsigned char* map = (unsigned char*)mmap(NULL, file_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) { set_error("failed to mmap %s: %s", path, strerror(errno)); close(fd); return NULL; }
    inferbit_model* model = NULL;
    ibj_node* root = NULL;
    int* bits = NULL;
    size_t err_at = 0;
    root = ibj_parse((const char*)map + IBF_PREAMBLE, header_size, &err_at);
    if (!root) { set_error("failed to parse IBF JSON header: near byte %zu", err_at); goto fail; }

    model = (inferbit_model*)calloc(1, sizeof *model);
    if (!model) { set_error("failed to allocate model"); goto fail; }
    {
        /* header fields and their defaults as in src/ibf_loader.c:138-191 */
        const ibj_node* jm = ibj_get(root, "model");
        strncpy(model->architecture, ibj_str(jm, "architecture", "unknown"), sizeof model->architecture - 1);
        const ibj_node* ja = ibj_get(root, "architecture");
        ib_b200_model_cfg c;
        memset(&c, 0, sizeof c);
        c.n_layers = (int)ibj_num(ja, "num_layers", 0);
        c.hidden = (int)ibj_num(ja, "hidden_size", 0);
        c.n_heads = (int)ibj_num(ja, "num_heads", 0);
        c.n_kv_heads = (int)ibj_num(ja, "num_kv_heads", c.n_heads);
        c.head_dim = (int)ibj_num(ja, "head_dim", c.n_heads > 0 ? c.hidden / c.n_heads : 0);
        c.inter = (int)ibj_num(ja, "intermediate_size", 0);
        c.vocab = (int)ibj_num(ja, "vocab_size", 0);
        c.max_ctx = (int)ibj_num(ja, "max_context_length", 2048);
        c.theta = (float)ibj_num(ja, "rope_theta", 10000.0);
        c.eps = (float)ibj_num(ja, "norm_epsilon", 1e-5);
        const ibj_node* jq = ibj_get(root, "quantization");
        model->default_bits = jq ? (int)ibj_num(jq, "default_bits", 4) : 0;
        const ibj_node* jkv = ibj_get(root, "kv_cache");
        model->kv_bits = jkv ? (int)ibj_num(jkv, "bits", 8) : 0;
        const ibj_node* jd = ibj_get(root, "data");
        const size_t hdr_data_off = jd ? (size_t)ibj_num(jd, "weight_data_offset", 0) : 0;
        const size_t hdr_data_size = jd ? (size_t)ibj_num(jd, "weight_data_size", 0) : 0;

        if (c.n_layers <= 0 || c.hidden <= 0 || c.vocab <= 0) { set_error("IBF header missing required architecture fields"); goto fail; }
        if (c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.inter <= 0 || c.max_ctx <= 0 || c.n_heads % c.n_kv_heads ||
            c.hidden != c.n_heads * c.head_dim) {
            set_error("IBF header describes a shape this backend does not run (heads %d, kv heads %d, head_dim %d, hidden %d, intermediate %d)",
                      c.n_heads, c.n_kv_heads, c.head_dim, c.hidden, c.inter);
            goto fail;
        }
        if (strcmp(ibj_str(ja, "norm_type", "rmsnorm"), "rmsnorm") || strcmp(ibj_str(ja, "activation", "silu"), "silu")) {
            set_error("IBF header asks for norm_type %s / activation %s; this backend runs rmsnorm / silu", ibj_str(ja, "norm_type", "rmsnorm"), ibj_str(ja, "activation", "silu"));
            goto fail;
        }
        if (model->kv_bits < 16) {
            set_error("unsupported kv_bits=%d: this backend keeps an FP32 KV cache (kv_cache.bits 16)", model->kv_bits);
            goto fail;
        }
        model->num_layers = c.n_layers; model->hidden = c.hidden; model->vocab = c.vocab; model->max_context = c.max_ctx;
        model->num_kv_heads = c.n_kv_heads; model->head_dim = c.head_dim;
        model->capacity = (config && config->context_length > 0 && config->context_length < c.max_ctx) ? config->context_length : c.max_ctx;

        /* data section (src/ibf_loader.c:455-466) */
        size_t data_off = ((size_t)IBF_PREAMBLE + header_size + 63) & ~(size_t)63;
        if (hdr_data_off > 0) data_off = hdr_data_off;
        if (data_off > file_size) { set_error("IBF weight data offset %zu exceeds file size %zu", data_off, file_size); goto fail; }
        size_t data_size = file_size - data_off;
        if (hdr_data_size > 0 && hdr_data_size < data_size) data_size = hdr_data_size;
        const unsigned char* data = map + data_off;
        model->weight_bytes = data_size;

        /* per-tensor metadata */
        static const char* names[7] = { "q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj" };
        const ibj_node* jl = ibj_get(root, "layers");
        if (!jl || jl->type != IBJ_ARR || ibj_len(jl) < c.n_layers) { set_error("IBF header lists %d layers, architecture says %d", ibj_len(jl), c.n_layers); goto fail; }
        bits = (int*)calloc((size_t)c.n_layers * 7 + 1, sizeof(int));
        if (!bits) { set_error("failed to allocate layer metadata"); goto fail; }
        for (int l = 0; l < c.n_layers; l++) {
            const ibj_node* w = ibj_get(ibj_at(jl, l), "weights");
            for (int i = 0; i < 7; i++) {
                const tmeta t = read_tensor(ibj_get(w, names[i]));
                if (t.bits != 4 && t.bits != 8) {
                    set_error("layer %d %s is stored at %d bits; this backend runs 4- and 8-bit linear layers", l, names[i], t.bits);
                    goto fail;
                }
                bits[l * 7 + i] = t.bits;
            }
        }
        const ibj_node* jo = ibj_get(root, "output");
        const tmeta t_head = read_tensor(ibj_get(jo, "head")), t_onorm = read_tensor(ibj_get(jo, "norm"));
        const tmeta t_emb = read_tensor(ibj_get(ibj_get(root, "embeddings"), "token_embedding"));
        if (t_head.bits != 4 && t_head.bits != 8) { set_error("output head is stored at %d bits; this backend runs 4- and 8-bit linear layers", t_head.bits); goto fail; }
        if (t_emb.bits != 8 && t_emb.bits != 4 && t_emb.bits != 16) { set_error("token embedding is stored at %d bits (8, 4 or 16 supported)", t_emb.bits); goto fail; }
        bits[c.n_layers * 7] = t_head.bits;
        c.attn_bits = bits[0]; c.mlp_bits = bits[4]; c.head_bits = t_head.bits;
        c.max_ctx = model->capacity;

        /* the GPU */
        const char* dev_env = getenv("INFERBIT_B200_DEVICE");
        const int rc0 = ib_b200_init(dev_env ? atoi(dev_env) : 0);
        if (rc0) { set_error("no usable B200 (%s); this library has no CPU path", ib_b200_last_error()); goto fail; }
        model->m = ib_b200_model_create_bits(ib_b200_ctx(), &c, bits, t_emb.bits);
        if (!model->m) { set_error("failed to allocate the model on the GPU: %s", ibcu_last_error(ib_b200_ctx())); goto fail; }

        /* upload */
        const int H = c.hidden, I = c.inter, kv = c.n_kv_heads * c.head_dim;
        const int Ms[7] = { H, kv, kv, H, I, I, H }, Ns[7] = { H, H, H, H, H, H, I };
        for (int l = 0; l < c.n_layers; l++) {
            const ibj_node* w = ibj_get(ibj_at(jl, l), "weights");
            char name[64];
            for (int i = 0; i < 7; i++) {
                const tmeta t = read_tensor(ibj_get(w, names[i]));
                snprintf(name, sizeof name, "layers[%d].%s", l, names[i]);
                if (upload_linear(model->m, l, i, &t, Ms[i], Ns[i], data, data_size, name)) goto fail;
            }
            const tmeta n1 = read_tensor(ibj_get(w, "input_norm")), n2 = read_tensor(ibj_get(w, "post_attn_norm"));
            snprintf(name, sizeof name, "layers[%d] norms", l);
            const void* p1 = span(data, data_size, n1.offset, (size_t)H * 2, name);
            const void* p2 = span(data, data_size, n2.offset, (size_t)H * 2, name);
            if (!p1 || !p2) goto fail;
            if (ib_b200_model_set_norms(model->m, l, (const uint16_t*)p1, (const uint16_t*)p2)) { set_error("uploading %s failed: %s", name, ibcu_last_error(ib_b200_ctx())); goto fail; }
        }
        if (upload_linear(model->m, 0, IB_B200_HEAD, &t_head, c.vocab, H, data, data_size, "output.head")) goto fail;
        const size_t emb_bytes = t_emb.bits == 16 ? (size_t)c.vocab * H * 2 : (t_emb.bits == 8 ? (size_t)c.vocab * H : (size_t)c.vocab * H / 2);
        const void* pe = span(data, data_size, t_emb.offset, emb_bytes, "embeddings.token_embedding");
        const void* pn = span(data, data_size, t_onorm.offset, (size_t)H * 2, "output.norm");
        const void* ps = NULL;
        if (t_emb.bits != 16 && (t_emb.scale_offset || t_emb.scale_size)) {
            ps = span(data, data_size, t_emb.scale_offset, (size_t)c.vocab * 2, "embeddings.token_embedding scales");
            if (!ps) goto fail;
        }
        if (!pe || !pn) goto fail;
        if (ib_b200_model_set_embedding(model->m, pe, (const uint16_t*)ps, (const uint16_t*)pn)) { set_error("uploading the embedding failed: %s", ibcu_last_error(ib_b200_ctx())); goto fail; }
    }
    free(bits);
    ibj_free(root);
    munmap(map, file_size);             /* the tensors live in HBM now */
    close(fd);
    return model;

fail:
    free(bits);
    ibj_free(root);
    munmap(map, file_size);
    close(fd);
    if (model) { if (model->m) ib_b200_model_free(model->m); free(model); }
    return NULL;
}

void inferbit_free(inferbit_model* model) {
    if (!model) return;
    ib_b200_model_free(model->m);
    free(model);
}

/* ── forward (src/generate.c:225-241, src/forward.c:850-902) ── */
int inferbit_forward(inferbit_model* model, const int32_t* tokens, int num_tokens, float* out_logits, int vocab_size) {
    if (!model || !tokens || !out_logits) { set_error("NULL argument to inferbit_forward"); return INFERBIT_ERROR_PARAM; }
    if (vocab_size != model->vocab) { set_error("vocab_size mismatch: %d vs %d", vocab_size, model->vocab); return INFERBIT_ERROR_PARAM; }
    if (num_tokens <= 0) { set_error("invalid arguments to ib_forward"); return INFERBIT_ERROR_PARAM; }
    if (model->kv_len + num_tokens > model->capacity) {
        set_error("context length exceeded: %d + %d > %d", model->kv_len, num_tokens, model->capacity);
        return INFERBIT_ERROR_CONTEXT;
    }
    for (int i = 0; i < num_tokens; i++)
        if (tokens[i] < 0 || tokens[i] >= model->vocab) {
            set_error("token ID out of range: %d (vocab_size=%d)", tokens[i], model->vocab);
            return INFERBIT_ERROR_PARAM;
        }
    /* positions go through in groups of up to 32 (causal inside a group, so the result is that of one
     * position at a time); only the last position's logits are wanted */
    for (int done = 0; done < num_tokens;) {
        const int B = num_tokens - done < BATCH_MAX ? num_tokens - done : BATCH_MAX;
        const int last = done + B == num_tokens;
        const int rc = ib_b200_forward_step_last(model->m, tokens + done, model->kv_len, B, last ? out_logits : NULL);
        if (rc) {
            set_error("GPU forward failed (%d): %s", rc, ibcu_last_error(ib_b200_ctx()));
            ibcu_clear_error(ib_b200_ctx());
            return INFERBIT_ERROR_INTERNAL;
        }
        done += B;
        model->kv_len += B;
    }
    return INFERBIT_OK;
}

/* ── KV-cache control (src/kv_cache.c:5-26): rows beyond the length are simply written again later ── */
void inferbit_kv_clear(inferbit_model* model) { if (model) model->kv_len = 0; }
void inferbit_kv_truncate(inferbit_model* model, int length) {
    if (!model) return;
    if (length < 0) length = 0;
    if (model->kv_len > length) model->kv_len = length;
}
int inferbit_kv_length(const inferbit_model* model) { return model ? model->kv_len : 0; }

/* ── model info (src/model.c:98-158) ── */
const char* inferbit_model_architecture(const inferbit_model* m) { return m ? m->architecture : "unknown"; }
int inferbit_model_num_layers(const inferbit_model* m) { return m ? m->num_layers : 0; }
int inferbit_model_hidden_size(const inferbit_model* m) { return m ? m->hidden : 0; }
int inferbit_model_vocab_size(const inferbit_model* m) { return m ? m->vocab : 0; }
int inferbit_model_max_context(const inferbit_model* m) { return m ? m->max_context : 0; }
int inferbit_model_default_bits(const inferbit_model* m) { return m ? m->default_bits : 0; }
size_t inferbit_model_weight_memory(const inferbit_model* m) { return m ? m->weight_bytes : 0; }
size_t inferbit_model_kv_memory(const inferbit_model* m) {
    if (!m) return 0;
    /* the reference's own accounting: capacity x kv_heads x head_dim x bits / 8, keys + values, per layer */
    const size_t per_token = (size_t)m->num_kv_heads * m->head_dim * m->kv_bits / 8;
    return (size_t)m->num_layers * m->capacity * per_token * 2;
}
size_t inferbit_model_total_memory(const inferbit_model* m) { return inferbit_model_weight_memory(m) + inferbit_model_kv_memory(m); }
