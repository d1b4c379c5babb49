#include "ibf_json.h"
#include <stdlib.h>
#include <string.h>

typedef struct { const char* s; size_t n, i; int depth; } cur;

static void skip_ws(cur* c) {
    while (c->i < c->n && (c->s[c->i] == ' ' || c->s[c->i] == '\t' || c->s[c->i] == '\n' || c->s[c->i] == '\r')) c->i++;
}

static ibj_node* node_new(int type) {
    ibj_node* n = (ibj_node*)calloc(1, sizeof *n);
    if (n) n->type = type;
    return n;
}

void ibj_free(ibj_node* n) {
    while (n) {
        ibj_node* next = n->next;
        ibj_free(n->child);
        free(n->str);
        free(n->key);
        free(n);
        n = next;
    }
}

static int hex4(cur* c, unsigned* out) {
    if (c->i + 4 > c->n) return -1;
    unsigned v = 0;
    for (int k = 0; k < 4; k++) {
        const char ch = c->s[c->i + k];
        v <<= 4;
        if (ch >= '0' && ch <= '9') v |= (unsigned)(ch - '0');
        else if (ch >= 'a' && ch <= 'f') v |= (unsigned)(ch - 'a' + 10);
        else if (ch >= 'A' && ch <= 'F') v |= (unsigned)(ch - 'A' + 10);
        else return -1;
    }
    c->i += 4;
    *out = v;
    return 0;
}

/* a string starting at the opening quote; returns a malloc'd, NUL-terminated copy with escapes resolved */
static char* parse_string(cur* c) {
    if (c->i >= c->n || c->s[c->i] != '"') return NULL;
    c->i++;
    size_t cap = 32, len = 0;
    char* out = (char*)malloc(cap);
    if (!out) return NULL;
    while (c->i < c->n) {
        unsigned char ch = (unsigned char)c->s[c->i++];
        if (ch == '"') { out[len] = 0; return out; }
        if (len + 5 > cap) { cap *= 2; char* t = (char*)realloc(out, cap); if (!t) { free(out); return NULL; } out = t; }
        if (ch != '\\') { out[len++] = (char)ch; continue; }
        if (c->i >= c->n) break;
        ch = (unsigned char)c->s[c->i++];
        switch (ch) {
            case '"': case '\\': case '/': out[len++] = (char)ch; break;
            case 'b': out[len++] = '\b'; break;
            case 'f': out[len++] = '\f'; break;
            case 'n': out[len++] = '\n'; break;
            case 'r': out[len++] = '\r'; break;
            case 't': out[len++] = '\t'; break;
            case 'u': {
                unsigned u;
                if (hex4(c, &u)) { free(out); return NULL; }
                if (u >= 0xD800 && u <= 0xDBFF && c->i + 6 <= c->n && c->s[c->i] == '\\' && c->s[c->i + 1] == 'u') {
                    c->i += 2;
                    unsigned lo;
                    if (hex4(c, &lo) || lo < 0xDC00 || lo > 0xDFFF) { free(out); return NULL; }
                    u = 0x10000 + ((u - 0xD800) << 10) + (lo - 0xDC00);
                }
                if (u < 0x80) out[len++] = (char)u;
                else if (u < 0x800) { out[len++] = (char)(0xC0 | (u >> 6)); out[len++] = (char)(0x80 | (u & 63)); }
                else if (u < 0x10000) { out[len++] = (char)(0xE0 | (u >> 12)); out[len++] = (char)(0x80 | ((u >> 6) & 63)); out[len++] = (char)(0x80 | (u & 63)); }
                else { out[len++] = (char)(0xF0 | (u >> 18)); out[len++] = (char)(0x80 | ((u >> 12) & 63)); out[len++] = (char)(0x80 | ((u >> 6) & 63)); out[len++] = (char)(0x80 | (u & 63)); }
                break;
            }
            default: free(out); return NULL;
        }
    }
    free(out);
    return NULL;
}

static ibj_node* parse_value(cur* c);

static ibj_node* parse_container(cur* c, int is_obj) {
    ibj_node* box = node_new(is_obj ? IBJ_OBJ : IBJ_ARR);
    if (!box) return NULL;
    const char close = is_obj ? '}' : ']';
    c->i++;                                   /* the opening bracket */
    if (++c->depth > 64) { ibj_free(box); return NULL; }
    ibj_node** tail = &box->child;
    skip_ws(c);
    if (c->i < c->n && c->s[c->i] == close) { c->i++; c->depth--; return box; }
    for (;;) {
        skip_ws(c);
        char* key = NULL;
        if (is_obj) {
            key = parse_string(c);
            if (!key) break;
            skip_ws(c);
            if (c->i >= c->n || c->s[c->i] != ':') { free(key); break; }
            c->i++;
        }
        ibj_node* v = parse_value(c);
        if (!v) { free(key); break; }
        v->key = key;
        *tail = v; tail = &v->next;
        skip_ws(c);
        if (c->i >= c->n) break;
        if (c->s[c->i] == ',') { c->i++; continue; }
        if (c->s[c->i] == close) { c->i++; c->depth--; return box; }
        break;
    }
    ibj_free(box);
    return NULL;
}

static ibj_node* parse_value(cur* c) {
    skip_ws(c);
    if (c->i >= c->n) return NULL;
    const char ch = c->s[c->i];
    if (ch == '{') return parse_container(c, 1);
    if (ch == '[') return parse_container(c, 0);
    if (ch == '"') {
        char* s = parse_string(c);
        if (!s) return NULL;
        ibj_node* n = node_new(IBJ_STR);
        if (!n) { free(s); return NULL; }
        n->str = s;
        return n;
    }
    if (c->n - c->i >= 4 && !memcmp(c->s + c->i, "true", 4)) { c->i += 4; ibj_node* n = node_new(IBJ_BOOL); if (n) n->num = 1; return n; }
    if (c->n - c->i >= 5 && !memcmp(c->s + c->i, "false", 5)) { c->i += 5; return node_new(IBJ_BOOL); }
    if (c->n - c->i >= 4 && !memcmp(c->s + c->i, "null", 4)) { c->i += 4; return node_new(IBJ_NULL); }
    if (ch == '-' || (ch >= '0' && ch <= '9')) {
        char tmp[64];
        size_t k = 0;
        while (c->i + k < c->n && k < sizeof tmp - 1) {
            const char d = c->s[c->i + k];
            if ((d >= '0' && d <= '9') || d == '-' || d == '+' || d == '.' || d == 'e' || d == 'E') tmp[k++] = d; else break;
        }
        tmp[k] = 0;
        char* end = NULL;
        const double v = strtod(tmp, &end);
        if (end == tmp) return NULL;
        c->i += (size_t)(end - tmp);
        ibj_node* n = node_new(IBJ_NUM);
        if (n) n->num = v;
        return n;
    }
    return NULL;
}

ibj_node* ibj_parse(const char* text, size_t len, size_t* err_at) {
    cur c = { text, len, 0, 0 };
    ibj_node* root = parse_value(&c);
    if (root) { skip_ws(&c); if (c.i != c.n) { ibj_free(root); root = NULL; } }
    if (!root && err_at) *err_at = c.i;
    return root;
}

const ibj_node* ibj_get(const ibj_node* obj, const char* key) {
    if (!obj || obj->type != IBJ_OBJ) return NULL;
    for (const ibj_node* m = obj->child; m; m = m->next) if (m->key && !strcmp(m->key, key)) return m;
    return NULL;
}
const ibj_node* ibj_at(const ibj_node* arr, int i) {
    if (!arr || (arr->type != IBJ_ARR && arr->type != IBJ_OBJ) || i < 0) return NULL;
    const ibj_node* m = arr->child;
    while (m && i-- > 0) m = m->next;
    return m;
}
int ibj_len(const ibj_node* n) {
    int k = 0;
    if (n && (n->type == IBJ_ARR || n->type == IBJ_OBJ)) for (const ibj_node* m = n->child; m; m = m->next) k++;
    return k;
}
const char* ibj_str(const ibj_node* obj, const char* key, const char* dflt) {
    const ibj_node* m = ibj_get(obj, key);
    return (m && m->type == IBJ_STR && m->str) ? m->str : dflt;
}
double ibj_num(const ibj_node* obj, const char* key, double dflt) {
    const ibj_node* m = ibj_get(obj, key);
    return (m && m->type == IBJ_NUM) ? m->num : dflt;
}
int ibj_bool(const ibj_node* obj, const char* key, int dflt) {
    const ibj_node* m = ibj_get(obj, key);
    return (m && m->type == IBJ_BOOL) ? (m->num != 0) : dflt;
}
