/* Shared state of the C host layer (not part of the ABI). */
#ifndef IB_B200_INTERNAL_H
#define IB_B200_INTERNAL_H
#include "ib_b200.h"

#define IB_B200_MAX_RANGES 256
#define IB_B200_NSTAGE 4
#define IB_B200_SCALE_SLOTS 2048   /* open-addressed cache of row-scale vectors, keyed by the weight pointer */

typedef struct { const char* host; size_t bytes; char* dev; } ib_b200_range;

/* FP32 row scales of one registered tensor as last seen at a call: the table hands them over on every
 * call (src/forward.c:152-156 widens them into a scratch vector), but they belong to the model, so the
 * device copy is reused for as long as the host vector compares equal */
typedef struct { const void* weights; int M; float* host; void* dev; } ib_b200_scale_entry;

typedef struct {
    ibcu_ctx* ctx;
    int status;
    char msg[512];
    ib_b200_range ranges[IB_B200_MAX_RANGES];
    int n_ranges;
    void* stage_host[IB_B200_NSTAGE];
    void* stage_dev[IB_B200_NSTAGE];
    size_t stage_bytes[IB_B200_NSTAGE];
    ib_b200_scale_entry scales[IB_B200_SCALE_SLOTS];
    unsigned long long h2d_bytes, d2h_bytes;       /* moved by table calls since init */
} ib_b200_state;

extern ib_b200_state g_ib;

void  ib_b200_set_error(int code, const char* fmt, ...);
int   ib_b200_check(int rc, const char* what);
void* ib_b200_translate(const void* p, size_t bytes);
int   ib_b200_stage(int slot, size_t bytes, void** host, void** dev);
void  ib_b200_pq_release_all(void);
void  ib_b200_lock(void);
void  ib_b200_unlock(void);
#endif
