/*
 * nncu_on_oracle.c -- TEST INFRASTRUCTURE ONLY.  The dozen entry points of include/nncu.h that the
 * reference's model plugin adapter (host/dropin/trf_cuda_model.inc) calls, implemented on the CPU
 * oracle (trf_oracle.c) instead of the CUDA library.  Linked with the reference's unmodified
 * nncp.c and that adapter it gives _ref/nncp_oracle: the reference's own command line -- its
 * encode_file, decode_file, process_block, retrain_block, header and preprocessor code -- runnable
 * on a CPU, with the very model the host-code tests use.  The tests compare the files it writes
 * with what this repository's host code (nch_compress, nch_words_encode) writes for the same
 * parameters.  Never part of the product: libnncu.so has no CPU path.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nncu.h"

typedef struct orc_model orc_model;
int orc_create(const nncu_params *p, orc_model **out);
void orc_destroy(orc_model *m);
int orc_param_count(const orc_model *m);
float *orc_probs(orc_model *m);
void orc_reset(orc_model *m);
void orc_set_lr(orc_model *m, float lr);
int orc_eval(orc_model *m, int output_index, const int32_t *input, float *probs_out);
int orc_eval_gradient(orc_model *m, const int32_t *targets, float *loss_out);
int orc_update(orc_model *m);

struct nncu_model {
    orc_model *o;
    int T, B, V;
    float *scratch; /* orc_eval wants somewhere to put the rows it evaluated */
};

static char g_err[128] = "";
const char *nncu_last_error(void) { return g_err; }

void nncu_default_params(nncu_params *p)
{
    memset(p, 0, sizeof(*p));
    p->n_layer = 4; p->d_model = 256; p->n_head = 8; p->d_key = 32; p->d_value = 32;
    p->d_inner = 512; p->d_pos = 32; p->mem_len = 32; p->seg_len = 32; p->n_streams = 16;
    p->n_symbols = 256; p->use_bias = 1; p->use_w_r = 1; p->tied_w_r = 1; p->tied_b_r = 1;
    p->ln_flags = NNCU_LN_POST; p->ff_act = NNCU_FF_GELU; p->embed_mult = 1.0f;
    p->init_range = 1.0f; p->init_kind = NNCU_INIT_UNIFORM; p->seed = 123;
    p->lr = 3e-4f; p->beta2 = 0.99f; p->eps = 1e-8f; p->device = -1;
}

int nncu_create(const nncu_params *p, nncu_model **out)
{
    nncu_params q = *p;
    q.use_bf16 = 0; /* the oracle computes in fp32 */
    nncu_model *m = calloc(1, sizeof(*m));
    if (!m)
        return NNCU_ERR_NOMEM;
    int rc = orc_create(&q, &m->o);
    if (rc) {
        snprintf(g_err, sizeof(g_err), "orc_create: %d", rc);
        free(m);
        return NNCU_ERR_INVALID;
    }
    m->T = q.seg_len; m->B = q.n_streams; m->V = q.n_symbols;
    m->scratch = malloc(sizeof(float) * (size_t)m->T * m->B * m->V);
    *out = m;
    return NNCU_OK;
}

int nncu_destroy(nncu_model *m)
{
    if (m) {
        orc_destroy(m->o);
        free(m->scratch);
        free(m);
    }
    return NNCU_OK;
}

int nncu_param_count(const nncu_model *m) { return orc_param_count(m->o); }
int nncu_reset(nncu_model *m) { orc_reset(m->o); return NNCU_OK; }
int nncu_set_lr(nncu_model *m, float lr) { orc_set_lr(m->o, lr); return NNCU_OK; }
int nncu_eval(nncu_model *m, int output_index, const int32_t *ids) { return orc_eval(m->o, output_index, ids, m->scratch) ? NNCU_ERR_INVALID : NNCU_OK; }
int nncu_eval_end(nncu_model *m) { (void)m; return NNCU_OK; }
int nncu_eval_gradient(nncu_model *m, const int32_t *targets, float *loss) { return orc_eval_gradient(m->o, targets, loss) ? NNCU_ERR_INVALID : NNCU_OK; }
int nncu_update(nncu_model *m) { return orc_update(m->o) ? NNCU_ERR_INVALID : NNCU_OK; }

int nncu_read_probs(nncu_model *m, int t0, int nt, float *out)
{
    const size_t row = (size_t)m->B * m->V;
    memcpy(out, orc_probs(m->o) + (size_t)t0 * row, sizeof(float) * (size_t)nt * row);
    return NNCU_OK;
}
