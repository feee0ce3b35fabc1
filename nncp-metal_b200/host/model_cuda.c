/*
 * model_cuda.c -- fills the plugin table (nch_model_ops) from libnncu.so.  The library is
 * opened with dlopen so that this host code carries no link-time CUDA dependency; when it
 * cannot be loaded, or no B200 is present, binding fails: there is no CPU model to fall
 * back to.  Mirrors what nncp_init does with np->model_class (nncp.c:2762-2800).
 */
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "nncp_host.h"

typedef struct {
    void *dl;
    nncu_model *model;
    int (*destroy)(nncu_model *);
    int (*reset)(nncu_model *);
    int (*set_lr)(nncu_model *, float);
    int (*eval)(nncu_model *, int, const int32_t *);
    int (*read_probs)(nncu_model *, int, int, float *);
    int (*coder_paths)(nncu_model *, int, int, const int32_t *, uint16_t *, int *);
    int (*coder_trees)(nncu_model *, int, int, uint16_t *);
    int (*eval_end)(nncu_model *);
    int (*eval_gradient)(nncu_model *, const int32_t *, float *);
    int (*update)(nncu_model *);
    int (*paths_begin)(nncu_model *, int, int, const int32_t *);
    int (*paths_end)(nncu_model *, uint16_t *, int *);
    int (*read_loss)(nncu_model *, float *);
    int (*decoder_begin)(nncu_model *, const uint8_t *, size_t);
    int (*decode_steps)(nncu_model *, int, int, const int32_t *, int, int, int32_t *);
    int (*decoder_end)(nncu_model *, size_t *);
} cuda_ctx;

static int c_reset(void *c) { cuda_ctx *x = c; return x->reset(x->model); }
static int c_set_lr(void *c, float lr) { cuda_ctx *x = c; return x->set_lr(x->model, lr); }
static int c_eval(void *c, int oi, const int32_t *in) { cuda_ctx *x = c; return x->eval(x->model, oi, in); }
static int c_read_probs(void *c, int t0, int nt, float *p) { cuda_ctx *x = c; return x->read_probs(x->model, t0, nt, p); }
static int c_paths(void *c, int t0, int nt, const int32_t *s, uint16_t *o, int *nb)
{
    cuda_ctx *x = c;
    return x->coder_paths(x->model, t0, nt, s, o, nb);
}
static int c_trees(void *c, int t0, int nt, uint16_t *o) { cuda_ctx *x = c; return x->coder_trees(x->model, t0, nt, o); }
static int c_eval_end(void *c) { cuda_ctx *x = c; return x->eval_end(x->model); }
static int c_grad(void *c, const int32_t *e, float *l) { cuda_ctx *x = c; return x->eval_gradient(x->model, e, l); }
static int c_update(void *c) { cuda_ctx *x = c; return x->update(x->model); }
static int c_paths_begin(void *c, int t0, int nt, const int32_t *s) { cuda_ctx *x = c; return x->paths_begin(x->model, t0, nt, s); }
static int c_paths_end(void *c, uint16_t *o, int *nb) { cuda_ctx *x = c; return x->paths_end(x->model, o, nb); }
static int c_grad_queue(void *c, const int32_t *e) { cuda_ctx *x = c; return x->eval_gradient(x->model, e, NULL); }
static int c_read_loss(void *c, float *l) { cuda_ctx *x = c; return x->read_loss(x->model, l); }
static int c_dec_begin(void *c, const uint8_t *p, size_t n) { cuda_ctx *x = c; return x->decoder_begin(x->model, p, n); }
static int c_dec_steps(void *c, int t0, int nt, const int32_t *ids, int lt, int lb, int32_t *out)
{
    cuda_ctx *x = c;
    return x->decode_steps(x->model, t0, nt, ids, lt, lb, out);
}
static int c_dec_end(void *c, size_t *n) { cuda_ctx *x = c; return x->decoder_end(x->model, n); }

int nch_bind_cuda(const char *libnncu_path, const nncu_params *p, nch_model_ops *ops)
{
    if (!libnncu_path || !p || !ops)
        return NCH_ERR_INVALID;
    memset(ops, 0, sizeof(*ops));
    cuda_ctx *x = calloc(1, sizeof(*x));
    if (!x)
        return NCH_ERR_NOMEM;
    x->dl = dlopen(libnncu_path, RTLD_NOW | RTLD_GLOBAL);
    if (!x->dl) {
        free(x);
        return NCH_ERR_MODEL;
    }
    int (*create)(const nncu_params *, nncu_model **) = dlsym(x->dl, "nncu_create");
    x->destroy = dlsym(x->dl, "nncu_destroy");
    x->reset = dlsym(x->dl, "nncu_reset");
    x->set_lr = dlsym(x->dl, "nncu_set_lr");
    x->eval = dlsym(x->dl, "nncu_eval");
    x->read_probs = dlsym(x->dl, "nncu_read_probs");
    x->coder_paths = dlsym(x->dl, "nncu_coder_paths");
    x->coder_trees = dlsym(x->dl, "nncu_coder_trees");
    x->eval_end = dlsym(x->dl, "nncu_eval_end");
    x->eval_gradient = dlsym(x->dl, "nncu_eval_gradient");
    x->update = dlsym(x->dl, "nncu_update");
    x->paths_begin = dlsym(x->dl, "nncu_coder_paths_begin");
    x->paths_end = dlsym(x->dl, "nncu_coder_paths_end");
    x->read_loss = dlsym(x->dl, "nncu_read_loss");
    x->decoder_begin = dlsym(x->dl, "nncu_decoder_begin");
    x->decode_steps = dlsym(x->dl, "nncu_decode_steps");
    x->decoder_end = dlsym(x->dl, "nncu_decoder_end");
    if (!create || !x->destroy || !x->reset || !x->set_lr || !x->eval || !x->read_probs || !x->coder_paths ||
        !x->coder_trees || !x->eval_end || !x->eval_gradient || !x->update || create(p, &x->model) != NNCU_OK) {
        dlclose(x->dl);
        free(x);
        return NCH_ERR_MODEL;
    }
    ops->ctx = x;
    ops->n_streams = p->n_streams;
    ops->seg_len = p->seg_len;
    ops->n_symbols = p->n_symbols;
    ops->reset = c_reset;
    ops->set_lr = c_set_lr;
    ops->eval = c_eval;
    ops->read_probs = c_read_probs;
    ops->coder_paths = c_paths;
    ops->coder_trees = c_trees;
    ops->eval_end = c_eval_end;
    ops->eval_gradient = c_grad;
    ops->update = c_update;
    if (x->paths_begin && x->paths_end && x->read_loss) {
        ops->coder_paths_begin = c_paths_begin;
        ops->coder_paths_end = c_paths_end;
        ops->eval_gradient_queue = c_grad_queue;
        ops->read_loss = c_read_loss;
    }
    if (x->decoder_begin && x->decode_steps && x->decoder_end) {
        ops->decoder_begin = c_dec_begin;
        ops->decode_steps = c_dec_steps;
        ops->decoder_end = c_dec_end;
    }
    return NCH_OK;
}

void nch_unbind_cuda(nch_model_ops *ops)
{
    if (!ops || !ops->ctx)
        return;
    cuda_ctx *x = ops->ctx;
    x->destroy(x->model);
    dlclose(x->dl);
    free(x);
    memset(ops, 0, sizeof(*ops));
}
