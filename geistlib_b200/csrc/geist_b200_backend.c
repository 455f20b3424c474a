/*
 * geist_b200_backend.c — the B200 sampler behind geistlib's backend operator slot.
 *
 * geistlib's arch layer reaches a device-side greedy argmax through the fused table of a backend
 * descriptor (include/geist_backend.h:414-421), after asking the backend's `supported` probe once at
 * plan-build time (include/geist_backend.h:276-326, src/archs/transformer/exec_plan.c:185-187, use at
 * src/archs/transformer/forward/head.c:131-143). This file defines those two functions with the
 * reference's exact signatures over libgeist_b200.so, plus the minimum of a backend around them (buffers
 * that live in device memory) so that the slot's contract test of the reference
 * (tests/test_fused_probe_agreement_unit.c:139-160) can be run against it.
 *
 * It is compiled against the geistlib headers where they lie (`make -C geistlib_b200/csrc backend
 * GEIST_INCLUDE=<geistlib>/include`); nothing of geistlib is copied here. A geistlib build that wants the
 * slot adds this file to a backend of its own, points `fused->supported` / `fused->argmax_f32` of its
 * descriptor at geist_b200_fused_supported / geist_b200_fused_argmax_f32, keeps a geist_b200_ctx in
 * `be->state` (geist_b200_backend_state) and registers the descriptor in
 * src/engine/backend_registry.c:40-57 behind a GEIST_BACKEND_B200 define.
 *
 * Contract kept (include/geist_backend.h:315-321, :416-418): when the probe said yes for (ARGMAX_F32,
 * m = 1, d_model = n) the op never returns GEIST_E_UNSUPPORTED for such a row; ties go to the lowest
 * index; a row this backend cannot read (foreign buffer, not F32 DENSE [1, n]) returns
 * GEIST_E_UNSUPPORTED and the arch scans on the host, as it does for the reference's GPU backends
 * (src/backends/vulkan/ops.c:1004-1033).
 */
#include <pthread.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "geist.h"
#include "geist_backend.h"
#include "geist_types.h"

#include <cuda_runtime_api.h>

/* from include/geist_b200.h; that header repeats the enums of geist.h only when geist.h is absent */
struct geist_b200_ctx;
enum geist_status geist_b200_ctx_create(int device, struct geist_b200_ctx **out);
void              geist_b200_ctx_destroy(struct geist_b200_ctx *ctx);
enum geist_status geist_b200_argmax_f32(struct geist_b200_ctx *ctx, const float *logits_dev, size_t n, int32_t *out_index);
int               geist_b200_argmax_f32_supported(size_t m, size_t n_vocab);
const char       *geist_b200_errmsg(void);

/* What this backend keeps behind `be->state`. */
struct geist_b200_backend_state {
    struct geist_b200_ctx *ctx;
    int                    device;
};

/* struct geist_buffer is backend-private (include/geist_types.h:123-124); here: a run of device memory. */
#define GEIST_B200_BUFFER_MAGIC 0xB2005A3Du
struct geist_buffer {
    unsigned magic;
    void    *dev;   /* device pointer */
    void    *host;  /* pinned staging while mapped, else NULL */
    size_t   bytes;
};

/* The engine provides this one (src/engine/backend.c:147-166); the weak twin below only serves a build of
 * this file outside of the engine, e.g. the contract check at the end. */
__attribute__((weak)) void geist_backend_set_error(struct geist_backend *be, enum geist_status code, const char *fmt, ...) {
    if (be == NULL) {
        return;
    }
    pthread_mutex_lock(&be->err_mu);
    be->err_code = code;
    va_list ap;
    va_start(ap, fmt);
    if (vsnprintf(be->err_msg, sizeof(be->err_msg), fmt, ap) < 0) {
        be->err_msg[0] = '\0';
    }
    va_end(ap);
    pthread_mutex_unlock(&be->err_mu);
}

/* Likewise the engine's shared all-null table (include/geist_backend.h:613-617). */
__attribute__((weak)) const struct geist_backend_fused geist_backend_no_fused = {0};

/* ---- the two slot functions ---- */

/* include/geist_backend.h:326: the load-time probe. Only ARGMAX_F32 is answered with yes, for the decode
 * regime (m == 1) and a vocabulary the kernels have a launch shape for. */
bool geist_b200_fused_supported(struct geist_backend *be, const struct geist_fusion_query *q) {
    if (be == NULL || q == NULL || be->state == NULL) {
        return false;
    }
    if (q->op != GEIST_FUSED_ARGMAX_F32) {
        return false;
    }
    const struct geist_b200_backend_state *st = be->state;
    if (cudaSetDevice(st->device) != cudaSuccess) {
        return false;
    }
    return geist_b200_argmax_f32_supported(q->m, q->d_model) != 0;
}

/* include/geist_backend.h:419-421. */
enum geist_status geist_b200_fused_argmax_f32(struct geist_backend *be, const struct geist_tensor *logits, int32_t *out_index) {
    if (be == NULL || be->state == NULL || logits == NULL || out_index == NULL) {
        return GEIST_E_UNSUPPORTED; /* the arch scans on the host */
    }
    const struct geist_b200_backend_state *st = be->state;
    const struct geist_buffer             *b  = logits->buffer;
    if (b == NULL || b->magic != GEIST_B200_BUFFER_MAGIC || b->dev == NULL) {
        return GEIST_E_UNSUPPORTED; /* not one of this backend's buffers */
    }
    if (logits->dtype != GEIST_DTYPE_F32 || logits->layout != GEIST_LAYOUT_DENSE) {
        return GEIST_E_UNSUPPORTED;
    }
    /* a [1, n] row (or a plain [n] vector), unit stride along the vocabulary */
    int64_t n = 0, step = 1;
    if (logits->ndim == 2 && logits->shape[0] == 1) {
        n    = logits->shape[1];
        step = logits->stride[1];
    } else if (logits->ndim == 1) {
        n    = logits->shape[0];
        step = logits->stride[0];
    } else {
        return GEIST_E_UNSUPPORTED;
    }
    if (n <= 0 || (step != 1 && step != 0 && n > 1) || (logits->offset % sizeof(float)) != 0 ||
        logits->offset + (size_t) n * sizeof(float) > b->bytes) {
        return GEIST_E_UNSUPPORTED;
    }
    if (step == 0 && n > 1) {
        return GEIST_E_UNSUPPORTED; /* stride left unset by a caller that means "dense" is written as 1 by the engine */
    }
    if (!geist_b200_argmax_f32_supported(1, (size_t) n)) {
        return GEIST_E_UNSUPPORTED; /* the probe would have said no */
    }
    const float      *row = (const float *) ((const unsigned char *) b->dev + logits->offset);
    int32_t           idx = -1;
    enum geist_status s   = geist_b200_argmax_f32(st->ctx, row, (size_t) n, &idx);
    if (s != GEIST_OK) {
        /* the probe said yes: a failure here is a real error, never "unsupported" */
        geist_backend_set_error(be, s == GEIST_E_UNSUPPORTED ? GEIST_E_BACKEND : s, "b200 argmax_f32: %s", geist_b200_errmsg());
        return s == GEIST_E_UNSUPPORTED ? GEIST_E_BACKEND : s;
    }
    *out_index = idx;
    return GEIST_OK;
}

/* The fused table a descriptor points at (all other slots: decomposed). */
const struct geist_backend_fused geist_b200_fused = {
        .supported  = geist_b200_fused_supported,
        .argmax_f32 = geist_b200_fused_argmax_f32,
};

/* ---- the minimum of a backend around the slot: state and device buffers ---- */

enum geist_status geist_b200_backend_state_create(int device, struct geist_b200_backend_state **out) {
    static struct geist_b200_backend_state pool[16];
    static int                             used = 0;
    if (out == NULL || used >= 16) {
        return GEIST_E_INVALID_ARG;
    }
    struct geist_b200_backend_state *st = &pool[used];
    st->device                          = device;
    const enum geist_status s           = geist_b200_ctx_create(device, &st->ctx);
    if (s != GEIST_OK) {
        return s;
    }
    used++;
    *out = st;
    return GEIST_OK;
}

void geist_b200_backend_state_destroy(struct geist_b200_backend_state *st) {
    if (st != NULL && st->ctx != NULL) {
        geist_b200_ctx_destroy(st->ctx);
        st->ctx = NULL;
    }
}

/* buffer_create / buffer_map / buffer_unmap / buffer_destroy of the core table, for device memory: map hands
 * out pinned staging, unmap uploads it. */
enum geist_status geist_b200_buffer_create(struct geist_backend *be, size_t bytes, struct geist_buffer **out) {
    static struct geist_buffer pool[64];
    static int                 used = 0;
    (void) be;
    if (out == NULL || bytes == 0 || used >= 64) {
        return GEIST_E_INVALID_ARG;
    }
    struct geist_buffer *b = &pool[used];
    memset(b, 0, sizeof *b);
    if (cudaMalloc(&b->dev, bytes) != cudaSuccess) {
        return GEIST_E_OOM;
    }
    b->magic = GEIST_B200_BUFFER_MAGIC;
    b->bytes = bytes;
    used++;
    *out = b;
    return GEIST_OK;
}

void *geist_b200_buffer_map(struct geist_buffer *b) {
    if (b == NULL || b->magic != GEIST_B200_BUFFER_MAGIC) {
        return NULL;
    }
    if (b->host == NULL && cudaMallocHost(&b->host, b->bytes) != cudaSuccess) {
        b->host = NULL;
        return NULL;
    }
    if (cudaMemcpy(b->host, b->dev, b->bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
        return NULL;
    }
    return b->host;
}

void geist_b200_buffer_unmap(struct geist_buffer *b) {
    if (b != NULL && b->host != NULL) {
        cudaMemcpy(b->dev, b->host, b->bytes, cudaMemcpyHostToDevice);
    }
}

void geist_b200_buffer_destroy(struct geist_buffer *b) {
    if (b == NULL || b->magic != GEIST_B200_BUFFER_MAGIC) {
        return;
    }
    cudaFree(b->dev);
    if (b->host != NULL) {
        cudaFreeHost(b->host);
    }
    memset(b, 0, sizeof *b);
}

/* ---- the slot's contract, as tests/test_fused_probe_agreement_unit.c:139-160 states it ---- */

/*
 * Runs the reference's check through the function pointers of the fused table: probe (ARGMAX_F32, m = 1,
 * d_model = 256); a [1, 256] F32 DENSE row with 100 at index 77 and i % 7 elsewhere; the op must return
 * GEIST_OK and 77. Further cases on the same table: an offset view, ties (lowest index wins), a foreign
 * buffer and a wrong dtype (GEIST_E_UNSUPPORTED: host scan). Returns the number of failed expectations;
 * `detail` receives a line per failure.
 */
int geist_b200_slot_contract_check(int device, char *detail, size_t detail_cap) {
    int    fails = 0;
    size_t used  = 0;
#define EXPECT(cond, text)                                                              \
    do {                                                                                \
        if (!(cond)) {                                                                  \
            fails++;                                                                    \
            if (detail != NULL && used < detail_cap) {                                  \
                used += (size_t) snprintf(detail + used, detail_cap - used, "%s\n", text); \
            }                                                                           \
        }                                                                               \
    } while (0)
    if (detail != NULL && detail_cap > 0) {
        detail[0] = '\0';
    }
    struct geist_b200_backend_state *st = NULL;
    if (geist_b200_backend_state_create(device, &st) != GEIST_OK) {
        EXPECT(0, "backend state could not be created");
        return fails;
    }
    static const struct geist_backend_descriptor desc = {.name = "b200", .fused = &geist_b200_fused};
    struct geist_backend                         be;
    memset(&be, 0, sizeof be);
    be.desc  = &desc;
    be.state = st;
    pthread_mutex_init(&be.err_mu, NULL);
    const struct geist_backend_fused *fused = geist_backend_fused_tbl(&be);

    struct geist_fusion_query aq = {.op = GEIST_FUSED_ARGMAX_F32, .m = 1, .d_model = 256};
    EXPECT(fused->supported != NULL && fused->argmax_f32 != NULL, "the table carries both slots");
    EXPECT(fused->supported(&be, &aq), "probe: ARGMAX_F32, m = 1, d_model = 256 is supported");
    struct geist_fusion_query pq = {.op = GEIST_FUSED_ARGMAX_F32, .m = 4, .d_model = 256};
    EXPECT(!fused->supported(&be, &pq), "probe: m > 1 is not");
    struct geist_fusion_query oq = {.op = GEIST_FUSED_RMSNORM_ADD, .m = 1, .d_model = 256};
    EXPECT(!fused->supported(&be, &oq), "probe: other ops are not");

    struct geist_buffer *bl = NULL;
    if (geist_b200_buffer_create(&be, 512 * sizeof(float), &bl) == GEIST_OK) {
        float *pm = geist_b200_buffer_map(bl);
        if (pm != NULL) {
            for (int i = 0; i < 256; i++) {
                pm[i] = (float) (i == 77 ? 100 : i % 7);
            }
            for (int i = 256; i < 512; i++) {
                pm[i] = (float) ((i - 256) % 5 == 4 ? 9 : 1); /* ties: the first 9 is at 4 */
            }
            geist_b200_buffer_unmap(bl);
            struct geist_tensor tl  = {.buffer = bl, .dtype = GEIST_DTYPE_F32, .layout = GEIST_LAYOUT_DENSE, .ndim = 2, .shape = {1, 256}, .stride = {256, 1}};
            int32_t             idx = -1;
            EXPECT(fused->argmax_f32(&be, &tl, &idx) == GEIST_OK && idx == 77, "probe said yes: argmax_f32 must return OK and index 77");
            struct geist_tensor tv = tl;
            tv.offset              = 256 * sizeof(float);
            idx                    = -1;
            EXPECT(fused->argmax_f32(&be, &tv, &idx) == GEIST_OK && idx == 4, "an offset view: ties go to the lowest index (4)");
            struct geist_tensor t1 = {.buffer = bl, .dtype = GEIST_DTYPE_F32, .layout = GEIST_LAYOUT_DENSE, .ndim = 1, .shape = {256}, .stride = {1}};
            idx                    = -1;
            EXPECT(fused->argmax_f32(&be, &t1, &idx) == GEIST_OK && idx == 77, "a [256] vector reads like a [1, 256] row");
            struct geist_tensor th = tl;
            th.dtype               = GEIST_DTYPE_F16;
            EXPECT(fused->argmax_f32(&be, &th, &idx) == GEIST_E_UNSUPPORTED, "F16 logits: unsupported, host scan");
            struct geist_tensor tb = tl;
            tb.shape[1]            = 1024;
            EXPECT(fused->argmax_f32(&be, &tb, &idx) == GEIST_E_UNSUPPORTED, "a view beyond its buffer: unsupported");
            struct geist_buffer foreign;
            memset(&foreign, 0, sizeof foreign);
            struct geist_tensor tf = tl;
            tf.buffer              = &foreign;
            EXPECT(fused->argmax_f32(&be, &tf, &idx) == GEIST_E_UNSUPPORTED, "a buffer of another backend: unsupported, host scan");
        } else {
            EXPECT(0, "buffer_map failed");
        }
        geist_b200_buffer_destroy(bl);
    } else {
        EXPECT(0, "buffer_create failed");
    }
    pthread_mutex_destroy(&be.err_mu);
    geist_b200_backend_state_destroy(st);
#undef EXPECT
    return fails;
}
