/* A small JSON reader for the IBF-v1 header (objects, arrays, strings, numbers, true/false/null).
 * The reference reads the same header through a third-party JSON library (src/ibf_loader.c:127-236);
 * this one is written for this loader and keeps only what the header needs. */
#ifndef IBF_JSON_H
#define IBF_JSON_H
#include <stddef.h>

enum { IBJ_NULL = 0, IBJ_BOOL, IBJ_NUM, IBJ_STR, IBJ_ARR, IBJ_OBJ };

typedef struct ibj_node {
    int type;
    double num;                 /* IBJ_NUM; IBJ_BOOL: 0 or 1 */
    char* str;                  /* IBJ_STR */
    char* key;                  /* name, when the node is a member of an object */
    struct ibj_node* child;     /* first member / element */
    struct ibj_node* next;      /* next sibling */
} ibj_node;

/* Parses text[0..len). Returns the root or NULL; on failure *err_at is the offset of the offending byte. */
ibj_node* ibj_parse(const char* text, size_t len, size_t* err_at);
void      ibj_free(ibj_node* n);
/* Member `key` of an object (case-sensitive), or NULL. */
const ibj_node* ibj_get(const ibj_node* obj, const char* key);
/* Element i of an array, or NULL; ibj_len counts members / elements. */
const ibj_node* ibj_at(const ibj_node* arr, int i);
int       ibj_len(const ibj_node* n);
/* Typed reads with a default for a missing member or a member of another type. */
const char* ibj_str(const ibj_node* obj, const char* key, const char* dflt);
double    ibj_num(const ibj_node* obj, const char* key, double dflt);
int       ibj_bool(const ibj_node* obj, const char* key, int dflt);
#endif
