/*
 * trf_oracle.c -- CPU restatement of NNCP's Transformer-XL train step.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it is the checker the CUDA path is compared against and
 * the "port" CPU baseline the benchmark times.
 *
 * PARITY UNPINNED against the reference binary: the reference implements this
 * path on LibNC, whose implementation is not part of the reference tree, and
 * the reference's tests hold no numerical vectors for it.  The restatement is
 * pinned instead against committed golden vectors produced by an independent
 * PyTorch/autograd restatement of the same graph (tests/golden).
 *
 * What follows what (reference paths):
 *   orc_create            trf_init                    nncp.c:304-520
 *   orc_eval              trf_eval                    nncp.c:581-1029
 *   orc_eval_gradient     trf_eval_gradient           nncp.c:1099-1193
 *                         (the backward pass is the hand-derived adjoint of
 *                          the forward graph; LibNC's autograd is not in-tree)
 *   orc_update            trf_update / mem_update     nncp.c:1205-1235
 *   orc_reset             trf_reset                   nncp.c:1195-1203
 *   op semantics          nc_masked_fill libnc.h:242-244, nc_pad :333-335,
 *                         nc_rel_shift :396-397, nc_soft_max :382,
 *                         nc_indexed_log :385-388, nc_layer_norm/nc_rms_norm
 *                         :389-390, nc_get_col :374-375
 *
 * Build-defined semantics (LibNC internals unknown): GELU is the tanh form;
 * LayerNorm uses the biased variance with eps 1e-5 inside the square root;
 * the optimizer is v = b2*v + (1-b2)*g^2, w -= lr*g/(sqrt(v)+eps), with an
 * optional elementwise gradient clamp and optional 1/(1-b2^t) correction.
 *
 * Layout: rows are (time, stream) positions, row index = time*B + stream;
 * per layer "hcat" holds [mem ; segment] rows, memory first.  Weights are
 * row-major [out][in].
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../include/nncu.h"

#define MAXP 1024

typedef struct {
    char name[32];
    size_t numel, off;
} orc_pinfo;

typedef struct {
    /* offsets into the flat buffers; (size_t)-1 when absent */
    size_t w_q, w_kv, b_q, w_o, ff1, ff_bias1, ff2, ff_bias2, w_r, b_r;
    size_t ln_g1, ln_b1, ln_g2, ln_b2;
    size_t alpha; /* LN_COEF: the scalar both sub-layer outputs are multiplied by before the residual (nncp.c:435-437, 892-894, 975-977) */
    /* activations */
    float *xin, *hcat, *q, *kv, *P, *o, *s1, *y, *u, *hpre, *hact, *s2;
    float *a1, *a2; /* LN_COEF: the sub-layer outputs before the multiplication */
    float *st_pre1, *st_1, *st_pre2, *st_2; /* [rows][2] mean, rstd */
} orc_layer;

typedef struct orc_model {
    nncu_params p;
    int L, HD, F1, TB, LB, Bt;
    int n_params;
    orc_pinfo pinfo[MAXP];
    size_t n_floats;
    float *w, *g, *v;
    size_t ln_g, ln_b, embed, embed_out, out_bias;
    orc_layer *layers;
    float *xlast, *xf, *st_f, *probs;
    int32_t *ids;
    float lr;
    int64_t step;
    int steps_done; /* incremental mode: number of time steps evaluated */
} orc_model;

#define NONE ((size_t)-1)

/* x * sigmoid(x): the gate function of FF_ACT_GATED_SILU (nc_gated_swish with beta 1, nncp.c:957-962) */
static float silu_f(float x) { return x / (1.0f + expf(-x)); }
static float silu_grad(float x)
{
    float s = 1.0f / (1.0f + expf(-x));
    return s * (1.0f + x * (1.0f - s));
}

/* ------------------------------------------------------------------ */
/* deterministic parameter initialisation (counter-based, integer hash) */

static uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

static uint64_t name_hash(const char *s)
{
    uint64_t h = 0xcbf29ce484222325ull;
    while (*s) {
        h ^= (uint8_t)*s++;
        h *= 0x100000001b3ull;
    }
    return h;
}

/* uniform in [0,1) with 24 random bits: exact in fp32 */
static float u01(uint64_t key, uint64_t idx, uint32_t k)
{
    uint64_t r = splitmix64(key ^ splitmix64(idx * 16 + k));
    return (float)(r >> 40) * (1.0f / 16777216.0f);
}

void orc_init_values(float *dst, size_t n, const char *name, uint32_t seed, int kind,
                     float scale)
{
    uint64_t key = splitmix64(name_hash(name) ^ ((uint64_t)seed << 32));
    for (size_t i = 0; i < n; i++) {
        if (kind == NNCU_INIT_NORMAL) {
            /* Irwin-Hall: sum of 12 uniforms minus 6 has unit variance */
            float s = 0.0f;
            for (uint32_t k = 0; k < 12; k++)
                s += u01(key, i, k);
            dst[i] = (s - 6.0f) * scale;
        } else {
            dst[i] = (2.0f * u01(key, i, 0) - 1.0f) * scale;
        }
    }
}

/* ------------------------------------------------------------------ */
/* dense helpers */

/* C[m][n] (+)= sum_k A[m][k] * B[n][k]  (+ bias[n]) */
static void gemm_nt(int M, int N, int K, const float *A, int lda, const float *B, int ldb,
                    float *C, int ldc, const float *bias, int acc)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        const float *a = A + (size_t)m * lda;
        for (int n = 0; n < N; n++) {
            const float *b = B + (size_t)n * ldb;
            float s = 0.0f;
#pragma omp simd reduction(+ : s)
            for (int k = 0; k < K; k++)
                s += a[k] * b[k];
            if (bias)
                s += bias[n];
            if (acc)
                C[(size_t)m * ldc + n] += s;
            else
                C[(size_t)m * ldc + n] = s;
        }
    }
}

/* C[m][n] (+)= sum_k A[m][k] * B[k][n] */
static void gemm_nn(int M, int N, int K, const float *A, int lda, const float *B, int ldb,
                    float *C, int ldc, int acc)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        float *c = C + (size_t)m * ldc;
        if (!acc)
            memset(c, 0, sizeof(float) * N);
        for (int k = 0; k < K; k++) {
            float a = A[(size_t)m * lda + k];
            const float *b = B + (size_t)k * ldb;
#pragma omp simd
            for (int n = 0; n < N; n++)
                c[n] += a * b[n];
        }
    }
}

/* C[m][n] (+)= sum_r A[r][m] * B[r][n]   (contraction over R rows) */
static void gemm_tn(int M, int N, int R, const float *A, int lda, const float *B, int ldb,
                    float *C, int ldc, int acc)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        float *c = C + (size_t)m * ldc;
        if (!acc)
            memset(c, 0, sizeof(float) * N);
        for (int r = 0; r < R; r++) {
            float a = A[(size_t)r * lda + m];
            const float *b = B + (size_t)r * ldb;
#pragma omp simd
            for (int n = 0; n < N; n++)
                c[n] += a * b[n];
        }
    }
}

static void colsum(int R, int N, const float *A, int lda, float *out, int acc)
{
    for (int n = 0; n < N; n++) {
        double s = 0;
        for (int r = 0; r < R; r++)
            s += A[(size_t)r * lda + n];
        out[n] = (acc ? out[n] : 0.0f) + (float)s;
    }
}

/* layer_norm(), nncp.c:279-288 */
static void norm_fwd(int rows, int D, const float *x, float *y, const float *g,
                     const float *b, int rms, float *st)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * D;
        float *yr = y + (size_t)r * D;
        double mu = 0, var = 0;
        if (!rms) {
            for (int i = 0; i < D; i++)
                mu += xr[i];
            mu /= D;
        }
        for (int i = 0; i < D; i++)
            var += (xr[i] - mu) * (xr[i] - mu);
        var /= D;
        float rstd = (float)(1.0 / sqrt(var + 1e-5));
        st[2 * r] = (float)mu;
        st[2 * r + 1] = rstd;
        for (int i = 0; i < D; i++)
            yr[i] = (xr[i] - (float)mu) * rstd * g[i] + b[i];
    }
}

/* dx (=/+=) adjoint of norm_fwd; dg, db accumulate */
static void norm_bwd(int rows, int D, const float *dy, const float *x, const float *g,
                     int rms, const float *st, float *dx, int acc, float *dg, float *db)
{
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * D, *dyr = dy + (size_t)r * D;
        float *dxr = dx + (size_t)r * D;
        float mu = st[2 * r], rstd = st[2 * r + 1];
        double s1 = 0, s2 = 0;
        for (int i = 0; i < D; i++) {
            float xh = (xr[i] - mu) * rstd;
            float dxh = dyr[i] * g[i];
            s1 += dxh;
            s2 += dxh * xh;
            dg[i] += dyr[i] * xh;
            db[i] += dyr[i];
        }
        s1 /= D;
        s2 /= D;
        for (int i = 0; i < D; i++) {
            float xh = (xr[i] - mu) * rstd;
            float dxh = dyr[i] * g[i];
            float v = rms ? rstd * (dxh - xh * (float)s2)
                          : rstd * (dxh - (float)s1 - xh * (float)s2);
            dxr[i] = (acc ? dxr[i] : 0.0f) + v;
        }
    }
}

static float gelu_f(float x)
{
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

static float gelu_grad(float x)
{
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    float t = tanhf(u);
    float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}

/* ------------------------------------------------------------------ */
/* relative-position attention, nncp.c:722-800 (and Appendix-style adjoint) */

typedef struct {
    int B, H, dk, T, M, P, attn_len;
    float br_scale;
} attn_dims;

/* q [T*B][H*dk], kv [L*B][2*H*dk], out [T*B][H*dk]; Pm [B][H][T][L] probabilities
   (may be NULL); lse [B*H][T] (may be NULL).  Queries t0..t1-1 only. */
static void attn_fwd(const attn_dims *d, int t0, int t1, const float *q, const float *kv,
                     const float *w_r, const float *b_r, float *out, float *Pm, float *lse)
{
    const int B = d->B, H = d->H, dk = d->dk, T = d->T, M = d->M, P = d->P;
    const int L = M + T, HD = H * dk;
    const float inv = 1.0f / sqrtf((float)dk);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++) {
        for (int h = 0; h < H; h++) {
            float *a = (float *)malloc(sizeof(float) * L);
            for (int i = t0; i < t1; i++) {
                const float *qi = q + ((size_t)i * B + b) * HD + h * dk;
                float mx = -INFINITY;
                for (int j = 0; j < L; j++) {
                    int pos = (i + M) - j;
                    if (!(pos >= 0 && pos < d->attn_len)) {
                        a[j] = -INFINITY;
                        continue;
                    }
                    const float *kj = kv + ((size_t)j * B + b) * 2 * HD + h * dk;
                    float s = 0;
                    for (int e = 0; e < dk; e++)
                        s += qi[e] * kj[e];
                    int r = j + (T - 1) - i; /* nc_rel_shift(-(T-1)), nncp.c:784 */
                    float z = 0;
                    if (r < L) {
                        z = d->br_scale * b_r[(size_t)h * L + r];
                        if (w_r) {
                            int pi = r - (L - P); /* nc_pad left, duplicate edge, nncp.c:777 */
                            if (pi < 0)
                                pi = 0;
                            const float *wr = w_r + ((size_t)h * P + pi) * dk;
                            float e1 = 0;
                            for (int e = 0; e < dk; e++)
                                e1 += qi[e] * wr[e];
                            z += e1;
                        }
                    }
                    a[j] = (s + z) * inv;
                    if (a[j] > mx)
                        mx = a[j];
                }
                double sum = 0;
                for (int j = 0; j < L; j++) {
                    a[j] = (a[j] == -INFINITY) ? 0.0f : expf(a[j] - mx);
                    sum += a[j];
                }
                float rs = (float)(1.0 / sum);
                float *oi = out + ((size_t)i * B + b) * HD + h * dk;
                for (int e = 0; e < dk; e++)
                    oi[e] = 0;
                for (int j = 0; j < L; j++) {
                    float p = a[j] * rs;
                    if (Pm)
                        Pm[(((size_t)b * H + h) * T + i) * L + j] = p;
                    if (p == 0.0f)
                        continue;
                    const float *vj = kv + ((size_t)j * B + b) * 2 * HD + HD + h * dk;
                    for (int e = 0; e < dk; e++)
                        oi[e] += p * vj[e];
                }
                if (lse)
                    lse[((size_t)b * H + h) * T + i] = mx + logf((float)sum);
            }
            free(a);
        }
    }
}

/* dq [T*B][HD], dkv [L*B][2HD] are overwritten; dw_r [H][P][dk], db_r [H][L] accumulate. */
static void attn_bwd(const attn_dims *d, const float *q, const float *kv, const float *w_r,
                     const float *b_r, const float *Pm, const float *dout, float *dq,
                     float *dkv, float *dw_r, float *db_r)
{
    const int B = d->B, H = d->H, dk = d->dk, T = d->T, M = d->M, P = d->P;
    const int L = M + T, HD = H * dk;
    const float inv = 1.0f / sqrtf((float)dk);
    (void)b_r;
    memset(dq, 0, sizeof(float) * (size_t)T * B * HD);
    memset(dkv, 0, sizeof(float) * (size_t)L * B * 2 * HD);
    /* streams in order so that the table gradients have a fixed summation order */
    for (int b = 0; b < B; b++) {
#pragma omp parallel for schedule(static)
        for (int h = 0; h < H; h++) {
            float *dp = (float *)malloc(sizeof(float) * L);
            for (int i = 0; i < T; i++) {
                const float *p = Pm + (((size_t)b * H + h) * T + i) * L;
                const float *doi = dout + ((size_t)i * B + b) * HD + h * dk;
                const float *qi = q + ((size_t)i * B + b) * HD + h * dk;
                float *dqi = dq + ((size_t)i * B + b) * HD + h * dk;
                double dot = 0;
                for (int j = 0; j < L; j++) {
                    dp[j] = 0;
                    if (p[j] == 0.0f)
                        continue;
                    const float *vj = kv + ((size_t)j * B + b) * 2 * HD + HD + h * dk;
                    float *dvj = dkv + ((size_t)j * B + b) * 2 * HD + HD + h * dk;
                    float s = 0;
                    for (int e = 0; e < dk; e++) {
                        s += doi[e] * vj[e];
                        dvj[e] += p[j] * doi[e];
                    }
                    dp[j] = s;
                    dot += (double)s * p[j];
                }
                for (int j = 0; j < L; j++) {
                    if (p[j] == 0.0f)
                        continue;
                    float ds = p[j] * (dp[j] - (float)dot) * inv;
                    const float *kj = kv + ((size_t)j * B + b) * 2 * HD + h * dk;
                    float *dkj = dkv + ((size_t)j * B + b) * 2 * HD + h * dk;
                    for (int e = 0; e < dk; e++) {
                        dqi[e] += ds * kj[e];
                        dkj[e] += ds * qi[e];
                    }
                    int r = j + (T - 1) - i;
                    if (r < L) {
                        db_r[(size_t)h * L + r] += d->br_scale * ds;
                        if (w_r) {
                            int pi = r - (L - P);
                            if (pi < 0)
                                pi = 0;
                            const float *wr = w_r + ((size_t)h * P + pi) * dk;
                            float *dwr = dw_r + ((size_t)h * P + pi) * dk;
                            for (int e = 0; e < dk; e++) {
                                dqi[e] += ds * wr[e];
                                dwr[e] += ds * qi[e];
                            }
                        }
                    }
                }
            }
            free(dp);
        }
    }
}

/* ------------------------------------------------------------------ */
/* model */

static size_t add_param(orc_model *m, const char *base, int idx, size_t numel)
{
    orc_pinfo *pi = &m->pinfo[m->n_params++];
    if (idx >= 0)
        snprintf(pi->name, sizeof(pi->name), "%s_%d", base, idx);
    else
        snprintf(pi->name, sizeof(pi->name), "%s", base);
    pi->numel = numel;
    pi->off = m->n_floats;
    m->n_floats += (numel + 127) & ~(size_t)127; /* 512-byte aligned slots */
    return pi->off;
}

static float *falloc(size_t n)
{
    return (float *)calloc(n ? n : 1, sizeof(float));
}

int orc_validate(const nncu_params *p)
{
    if (p->n_layer < 1 || p->n_layer > NNCU_N_LAYER_MAX || p->d_model < 1 || p->n_head < 1 ||
        p->d_key < 1 || p->d_value != p->d_key || p->d_inner < 1 || p->seg_len < 1 ||
        p->mem_len < 0 || p->n_streams < 1 || p->n_symbols < 2)
        return NNCU_ERR_INVALID;
    if (p->d_pos < 1 || p->d_pos > p->mem_len + p->seg_len)
        return NNCU_ERR_INVALID;
    if ((p->ln_flags & NNCU_LN_PRE) && (p->ln_flags & NNCU_LN_POST))
        return NNCU_ERR_INVALID;
    if (p->ff_act > NNCU_FF_GATED_SILU)
        return NNCU_ERR_INVALID;
    return NNCU_OK;
}

int orc_create(const nncu_params *p, orc_model **out)
{
    int rc = orc_validate(p);
    if (rc)
        return rc;
    orc_model *m = (orc_model *)calloc(1, sizeof(*m));
    m->p = *p;
    const int D = p->d_model, H = p->n_head, dk = p->d_key, F = p->d_inner, T = p->seg_len;
    const int B = p->n_streams, V = p->n_symbols;
    m->L = p->mem_len + T;
    m->HD = H * dk;
    m->F1 = (p->ff_act == NNCU_FF_GEGLU || p->ff_act == NNCU_FF_GATED_SILU) ? 2 * F : F;
    m->TB = T * B;
    m->LB = m->L * B;
    m->Bt = p->n_streams_total > 0 ? p->n_streams_total : B;
    m->lr = p->lr;
    m->layers = (orc_layer *)calloc(p->n_layer, sizeof(orc_layer));
    const int has_ln = (p->ln_flags & (NNCU_LN_POST | NNCU_LN_PRE)) != 0;
    for (int l = 0; l < p->n_layer; l++) {
        orc_layer *y = &m->layers[l];
        y->w_q = add_param(m, "w_q", l, (size_t)m->HD * D);
        y->w_kv = add_param(m, "w_kv", l, (size_t)2 * m->HD * D);
        y->b_q = p->query_bias ? add_param(m, "b_q", l, m->HD) : NONE;
        y->w_o = add_param(m, "w_o", l, (size_t)D * m->HD);
        y->ff1 = add_param(m, "ff1", l, (size_t)m->F1 * D);
        y->ff_bias1 = p->use_bias ? add_param(m, "ff_bias1", l, m->F1) : NONE;
        y->ff2 = add_param(m, "ff2", l, (size_t)D * F);
        y->ff_bias2 = p->use_bias ? add_param(m, "ff_bias2", l, D) : NONE;
        if (p->use_w_r)
            y->w_r = (l == 0 || !p->tied_w_r) ? add_param(m, "w_r", l, (size_t)H * p->d_pos * dk)
                                              : m->layers[0].w_r;
        else
            y->w_r = NONE;
        y->b_r = (l == 0 || !p->tied_b_r) ? add_param(m, "b_r", l, (size_t)H * m->L)
                                          : m->layers[0].b_r;
        if (has_ln) {
            y->ln_g1 = add_param(m, "ln_g", 2 * l, D);
            y->ln_b1 = add_param(m, "ln_b", 2 * l, D);
            y->ln_g2 = add_param(m, "ln_g", 2 * l + 1, D);
            y->ln_b2 = add_param(m, "ln_b", 2 * l + 1, D);
        } else {
            y->ln_g1 = y->ln_b1 = y->ln_g2 = y->ln_b2 = NONE;
        }
        y->alpha = (p->ln_flags & NNCU_LN_COEF) ? add_param(m, "alpha", l, 1) : NONE; /* starts at 0, nncp.c:437 */
    }
    if (p->ln_flags & NNCU_LN_FINAL) {
        m->ln_g = add_param(m, "ln_g", 2 * p->n_layer, D);
        m->ln_b = add_param(m, "ln_b", 2 * p->n_layer, D);
    } else {
        m->ln_g = m->ln_b = NONE;
    }
    m->embed = add_param(m, "embed", -1, (size_t)V * D);
    m->embed_out = add_param(m, "embed_out", -1, (size_t)V * D);
    m->out_bias = p->use_bias ? add_param(m, "out_bias", -1, V) : NONE;

    m->w = falloc(m->n_floats);
    m->g = falloc(m->n_floats);
    m->v = falloc(m->n_floats);

    /* initial values: trf_init, nncp.c:341-497 */
    float a = p->init_kind == NNCU_INIT_NORMAL ? p->init_range
                                               : p->init_range / sqrtf((float)D);
    for (int i = 0; i < m->n_params; i++) {
        orc_pinfo *pi = &m->pinfo[i];
        float *dst = m->w + pi->off;
        if (!strncmp(pi->name, "ln_g", 4)) {
            for (size_t k = 0; k < pi->numel; k++)
                dst[k] = 1.0f;
        } else if (!strncmp(pi->name, "w_", 2) || !strncmp(pi->name, "ff1", 3) ||
                   !strncmp(pi->name, "embed", 5)) {
            orc_init_values(dst, pi->numel, pi->name, p->seed, p->init_kind, a);
        } else if (!strncmp(pi->name, "ff2", 3)) {
            orc_init_values(dst, pi->numel, pi->name, p->seed, p->init_kind,
                            a * sqrtf((float)D / (float)F)); /* nncp.c:421-423 */
        } /* biases, b_r, ln_b: zero */
    }

    for (int l = 0; l < p->n_layer; l++) {
        orc_layer *y = &m->layers[l];
        y->xin = falloc((size_t)m->TB * D);
        y->hcat = falloc((size_t)m->LB * D);
        y->q = falloc((size_t)m->TB * m->HD);
        y->kv = falloc((size_t)m->LB * 2 * m->HD);
        y->P = falloc((size_t)B * H * T * m->L);
        y->o = falloc((size_t)m->TB * m->HD);
        y->s1 = falloc((size_t)m->TB * D);
        y->y = falloc((size_t)m->TB * D);
        y->u = falloc((size_t)m->TB * D);
        y->hpre = falloc((size_t)m->TB * m->F1);
        y->hact = falloc((size_t)m->TB * F);
        y->s2 = falloc((size_t)m->TB * D);
        y->a1 = falloc((size_t)m->TB * D);
        y->a2 = falloc((size_t)m->TB * D);
        y->st_pre1 = falloc((size_t)m->TB * 2);
        y->st_1 = falloc((size_t)m->TB * 2);
        y->st_pre2 = falloc((size_t)m->TB * 2);
        y->st_2 = falloc((size_t)m->TB * 2);
    }
    m->xlast = falloc((size_t)m->TB * D);
    m->xf = falloc((size_t)m->TB * D);
    m->st_f = falloc((size_t)m->TB * 2);
    m->probs = falloc((size_t)m->TB * V);
    m->ids = (int32_t *)calloc(m->TB, sizeof(int32_t));
    *out = m;
    return NNCU_OK;
}

void orc_destroy(orc_model *m)
{
    if (!m)
        return;
    for (int l = 0; l < m->p.n_layer; l++) {
        orc_layer *y = &m->layers[l];
        float *bufs[] = {y->xin, y->hcat, y->q, y->kv, y->P, y->o, y->s1, y->y, y->u,
                         y->hpre, y->hact, y->s2, y->st_pre1, y->st_1, y->st_pre2, y->st_2, y->a1, y->a2};
        for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); i++)
            free(bufs[i]);
    }
    free(m->layers);
    free(m->w);
    free(m->g);
    free(m->v);
    free(m->xlast);
    free(m->xf);
    free(m->st_f);
    free(m->probs);
    free(m->ids);
    free(m);
}

int orc_param_count(const orc_model *m) { return m->n_params; }

int orc_param_info(const orc_model *m, int i, char *name, size_t cap, size_t *numel,
                   size_t *off)
{
    if (i < 0 || i >= m->n_params)
        return NNCU_ERR_INVALID;
    if (name)
        snprintf(name, cap, "%s", m->pinfo[i].name);
    if (numel)
        *numel = m->pinfo[i].numel;
    if (off)
        *off = m->pinfo[i].off;
    return NNCU_OK;
}

float *orc_weights(orc_model *m) { return m->w; }
float *orc_grads(orc_model *m) { return m->g; }
float *orc_moments(orc_model *m) { return m->v; }
size_t orc_n_floats(const orc_model *m) { return m->n_floats; }
float *orc_probs(orc_model *m) { return m->probs; }
/* memory of layer l: [M*B][D] */
float *orc_mem(orc_model *m, int l) { return m->layers[l].hcat; }

/* OpenMP team size of the oracle's loops.  orc_set_threads(n > 0) fixes it for later calls
 * whatever OMP_NUM_THREADS said when the library was loaded (a launcher such as
 * torch.distributed.run exports OMP_NUM_THREADS=1 to its children); both return the size in
 * force. */
#ifdef _OPENMP
#include <omp.h>
int orc_set_threads(int n)
{
    if (n > 0)
        omp_set_num_threads(n);
    return omp_get_max_threads();
}
int orc_get_threads(void) { return omp_get_max_threads(); }
#else
int orc_set_threads(int n) { (void)n; return 1; }
int orc_get_threads(void) { return 1; }
#endif

void orc_reset(orc_model *m)
{
    for (int l = 0; l < m->p.n_layer; l++)
        memset(m->layers[l].hcat, 0, sizeof(float) * (size_t)m->p.mem_len * m->p.n_streams *
                                         m->p.d_model);
}

void orc_set_lr(orc_model *m, float lr) { m->lr = lr; }

#define W(off) (m->w + (off))
#define G(off) (m->g + (off))
#define WN(off) ((off) == NONE ? NULL : m->w + (off))

/* forward over times [t0, t1): trf_eval, nncp.c:581-1029.  input is [T][B]. */
static void forward_range(orc_model *m, const int32_t *input, int t0, int t1)
{
    const nncu_params *p = &m->p;
    const int D = p->d_model, H = p->n_head, dk = p->d_key, F = p->d_inner, T = p->seg_len;
    const int B = p->n_streams, V = p->n_symbols, M = p->mem_len, L = m->L, HD = m->HD;
    const int r0 = t0 * B, nr = (t1 - t0) * B; /* segment-row range */
    const int rms = (p->ln_flags & NNCU_LN_RMSNORM) != 0;
    const float emul = sqrtf((float)D) * p->embed_mult;

    for (int r = r0; r < r0 + nr; r++) {
        int id = input[r];
        m->ids[r] = id;
        const float *e = W(m->embed) + (size_t)id * D;
        float *x = m->layers[0].xin + (size_t)r * D;
        for (int i = 0; i < D; i++)
            x[i] = e[i] * emul; /* nncp.c:625-630 */
    }
    for (int l = 0; l < p->n_layer; l++) {
        orc_layer *y = &m->layers[l];
        float *xin = y->xin + (size_t)r0 * D;
        float *x1 = y->hcat + ((size_t)M * B + r0) * D; /* this is train_h, nncp.c:646-657 */
        if (p->ln_flags & NNCU_LN_PRE)
            norm_fwd(nr, D, xin, x1, W(y->ln_g1), W(y->ln_b1), rms, y->st_pre1 + 2 * r0);
        else
            memcpy(x1, xin, sizeof(float) * (size_t)nr * D);
        /* projections, nncp.c:659-695: memory K/V once per segment */
        gemm_nt(nr, HD, D, x1, D, W(y->w_q), D, y->q + (size_t)r0 * HD, HD, WN(y->b_q), 0);
        if (t0 == 0 && M > 0)
            gemm_nt(M * B, 2 * HD, D, y->hcat, D, W(y->w_kv), D, y->kv, 2 * HD, NULL, 0);
        gemm_nt(nr, 2 * HD, D, x1, D, W(y->w_kv), D, y->kv + ((size_t)M * B + r0) * 2 * HD,
                2 * HD, NULL, 0);
        attn_dims ad = {B, H, dk, T, M, p->d_pos, p->attn_len[l] ? p->attn_len[l] : L,
                        sqrtf((float)dk * (float)D)};
        attn_fwd(&ad, t0, t1, y->q, y->kv, WN(y->w_r), W(y->b_r), y->o, y->P, NULL);
        /* w_o + residual (+ post-LN), nncp.c:865-920 */
        float *s1 = y->s1 + (size_t)r0 * D, *yy = y->y + (size_t)r0 * D;
        gemm_nt(nr, D, HD, y->o + (size_t)r0 * HD, HD, W(y->w_o), HD, s1, D, NULL, 0);
        if (y->alpha != NONE) { /* LN_COEF, nncp.c:892-894 */
            float *a1 = y->a1 + (size_t)r0 * D;
            const float al = W(y->alpha)[0];
            for (size_t i = 0; i < (size_t)nr * D; i++) {
                a1[i] = s1[i];
                s1[i] = al * a1[i];
            }
        }
        for (size_t i = 0; i < (size_t)nr * D; i++)
            s1[i] += xin[i];
        if (p->ln_flags & NNCU_LN_POST)
            norm_fwd(nr, D, s1, yy, W(y->ln_g1), W(y->ln_b1), rms, y->st_1 + 2 * r0);
        else
            memcpy(yy, s1, sizeof(float) * (size_t)nr * D);
        /* feed-forward, nncp.c:925-986 */
        float *u = y->u + (size_t)r0 * D;
        if (p->ln_flags & NNCU_LN_PRE)
            norm_fwd(nr, D, yy, u, W(y->ln_g2), W(y->ln_b2), rms, y->st_pre2 + 2 * r0);
        else
            memcpy(u, yy, sizeof(float) * (size_t)nr * D);
        float *hpre = y->hpre + (size_t)r0 * m->F1, *hact = y->hact + (size_t)r0 * F;
        gemm_nt(nr, m->F1, D, u, D, W(y->ff1), D, hpre, m->F1, WN(y->ff_bias1), 0);
        for (int r = 0; r < nr; r++) {
            for (int i = 0; i < F; i++) {
                float a = hpre[(size_t)r * m->F1 + i], o;
                if (p->ff_act == NNCU_FF_RELU)
                    o = a > 0 ? a : 0;
                else if (p->ff_act == NNCU_FF_GELU)
                    o = gelu_f(a);
                else if (p->ff_act == NNCU_FF_GEGLU)
                    o = gelu_f(a) * hpre[(size_t)r * m->F1 + F + i]; /* nncp.c:945-951 */
                else
                    o = silu_f(a) * hpre[(size_t)r * m->F1 + F + i]; /* nncp.c:957-962 */
                hact[(size_t)r * F + i] = o;
            }
        }
        float *s2 = y->s2 + (size_t)r0 * D;
        gemm_nt(nr, D, F, hact, F, W(y->ff2), F, s2, D, WN(y->ff_bias2), 0);
        if (y->alpha != NONE) { /* LN_COEF, nncp.c:975-977 */
            float *a2 = y->a2 + (size_t)r0 * D;
            const float al = W(y->alpha)[0];
            for (size_t i = 0; i < (size_t)nr * D; i++) {
                a2[i] = s2[i];
                s2[i] = al * a2[i];
            }
        }
        for (size_t i = 0; i < (size_t)nr * D; i++)
            s2[i] += yy[i];
        float *xout = (l + 1 < p->n_layer) ? m->layers[l + 1].xin + (size_t)r0 * D
                                           : m->xlast + (size_t)r0 * D;
        if (p->ln_flags & NNCU_LN_POST)
            norm_fwd(nr, D, s2, xout, W(y->ln_g2), W(y->ln_b2), rms, y->st_2 + 2 * r0);
        else
            memcpy(xout, s2, sizeof(float) * (size_t)nr * D);
    }
    float *xl = m->xlast + (size_t)r0 * D, *xf = m->xf + (size_t)r0 * D;
    if (p->ln_flags & NNCU_LN_FINAL)
        norm_fwd(nr, D, xl, xf, W(m->ln_g), W(m->ln_b), rms, m->st_f + 2 * r0);
    else
        memcpy(xf, xl, sizeof(float) * (size_t)nr * D);
    float *pr = m->probs + (size_t)r0 * V;
    gemm_nt(nr, V, D, xf, D, W(m->embed_out), D, pr, V, WN(m->out_bias), 0);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < nr; r++) { /* nc_soft_max over the symbols, nncp.c:1008 */
        float *z = pr + (size_t)r * V;
        float mx = z[0];
        for (int i = 1; i < V; i++)
            if (z[i] > mx)
                mx = z[i];
        double s = 0;
        for (int i = 0; i < V; i++) {
            z[i] = expf(z[i] - mx);
            s += z[i];
        }
        float rs = (float)(1.0 / s);
        for (int i = 0; i < V; i++)
            z[i] *= rs;
    }
}

/* model_eval.  probs_out (may be NULL) receives [T][B][V] (batched) or [B][V] (step). */
int orc_eval(orc_model *m, int output_index, const int32_t *input, float *probs_out)
{
    const int T = m->p.seg_len, B = m->p.n_streams, V = m->p.n_symbols;
    if (output_index >= T)
        return NNCU_ERR_INVALID;
    if (output_index < 0) {
        forward_range(m, input, 0, T);
        m->steps_done = T;
        if (probs_out)
            memcpy(probs_out, m->probs, sizeof(float) * (size_t)T * B * V);
    } else {
        if (output_index != 0 && output_index != m->steps_done)
            return NNCU_ERR_STATE;
        forward_range(m, input, output_index, output_index + 1);
        m->steps_done = output_index + 1;
        if (probs_out)
            memcpy(probs_out, m->probs + (size_t)output_index * B * V,
                   sizeof(float) * (size_t)B * V);
    }
    return NNCU_OK;
}

/* model_eval_gradient, nncp.c:1099-1193.  targets [T][B]; returns sum ln p[target]. */
int orc_eval_gradient(orc_model *m, const int32_t *targets, float *loss_out)
{
    const nncu_params *p = &m->p;
    const int D = p->d_model, H = p->n_head, dk = p->d_key, F = p->d_inner, T = p->seg_len;
    const int B = p->n_streams, V = p->n_symbols, M = p->mem_len, L = m->L, HD = m->HD;
    const int TB = m->TB, LB = m->LB, F1 = m->F1;
    const int rms = (p->ln_flags & NNCU_LN_RMSNORM) != 0;
    if (m->steps_done != T)
        return NNCU_ERR_STATE;
    memset(m->g, 0, sizeof(float) * m->n_floats);

    float *dz = falloc((size_t)TB * V);
    float *dx = falloc((size_t)TB * D), *dt = falloc((size_t)TB * D), *dy = falloc((size_t)TB * D);
    float *dal = falloc((size_t)TB * D); /* LN_COEF: alpha * d(sum) */
    float *dh = falloc((size_t)TB * F), *dhp = falloc((size_t)TB * F1);
    float *dof = falloc((size_t)TB * HD), *dq = falloc((size_t)TB * HD);
    float *dkv = falloc((size_t)LB * 2 * HD);
    const float sc = 1.0f / ((float)T * (float)m->Bt);
    double loss = 0;
    for (int r = 0; r < TB; r++) {
        const float *pr = m->probs + (size_t)r * V;
        loss += log((double)pr[targets[r]]); /* nc_indexed_log + nc_sum, nncp.c:1170-1173 */
        for (int i = 0; i < V; i++)
            dz[(size_t)r * V + i] = (pr[i] - (i == targets[r] ? 1.0f : 0.0f)) * sc;
    }
    if (loss_out)
        *loss_out = (float)loss;
    if (m->out_bias != NONE)
        colsum(TB, V, dz, V, G(m->out_bias), 0);
    gemm_tn(V, D, TB, dz, V, m->xf, D, G(m->embed_out), D, 0);
    gemm_nn(TB, D, V, dz, V, W(m->embed_out), D, dt, D, 0);
    if (p->ln_flags & NNCU_LN_FINAL)
        norm_bwd(TB, D, dt, m->xlast, W(m->ln_g), rms, m->st_f, dx, 0, G(m->ln_g), G(m->ln_b));
    else
        memcpy(dx, dt, sizeof(float) * (size_t)TB * D);

    for (int l = p->n_layer - 1; l >= 0; l--) {
        orc_layer *y = &m->layers[l];
        /* dx = d(layer output).  ds2 -> dt */
        if (p->ln_flags & NNCU_LN_POST)
            norm_bwd(TB, D, dx, y->s2, W(y->ln_g2), rms, y->st_2, dt, 0, G(y->ln_g2), G(y->ln_b2));
        else
            memcpy(dt, dx, sizeof(float) * (size_t)TB * D);
        /* LN_COEF: the branch sees alpha * ds2, alpha collects sum(ds2 . branch output); the residual keeps ds2 */
        const float *da = dt;
        if (y->alpha != NONE) {
            const float al = W(y->alpha)[0];
            double acc = 0.0;
            for (size_t i = 0; i < (size_t)TB * D; i++) {
                acc += (double)dt[i] * (double)y->a2[i];
                dal[i] = al * dt[i];
            }
            G(y->alpha)[0] += (float)acc;
            da = dal;
        }
        if (y->ff_bias2 != NONE)
            colsum(TB, D, da, D, G(y->ff_bias2), 0);
        gemm_tn(D, F, TB, da, D, y->hact, F, G(y->ff2), F, 0);
        gemm_nn(TB, F, D, da, D, W(y->ff2), F, dh, F, 0);
        for (int r = 0; r < TB; r++) {
            for (int i = 0; i < F; i++) {
                float a = y->hpre[(size_t)r * F1 + i], d = dh[(size_t)r * F + i];
                if (p->ff_act == NNCU_FF_RELU) {
                    dhp[(size_t)r * F1 + i] = a > 0 ? d : 0;
                } else if (p->ff_act == NNCU_FF_GELU) {
                    dhp[(size_t)r * F1 + i] = d * gelu_grad(a);
                } else {
                    const int silu = p->ff_act == NNCU_FF_GATED_SILU;
                    float gate = y->hpre[(size_t)r * F1 + F + i];
                    dhp[(size_t)r * F1 + i] = d * gate * (silu ? silu_grad(a) : gelu_grad(a));
                    dhp[(size_t)r * F1 + F + i] = d * (silu ? silu_f(a) : gelu_f(a));
                }
            }
        }
        if (y->ff_bias1 != NONE)
            colsum(TB, F1, dhp, F1, G(y->ff_bias1), 0);
        gemm_tn(F1, D, TB, dhp, F1, y->u, D, G(y->ff1), D, 0);
        /* du -> dy, then dy += ds2 */
        if (p->ln_flags & NNCU_LN_PRE) {
            gemm_nn(TB, D, F1, dhp, F1, W(y->ff1), D, dx, D, 0);
            memcpy(dy, dt, sizeof(float) * (size_t)TB * D);
            norm_bwd(TB, D, dx, y->y, W(y->ln_g2), rms, y->st_pre2, dy, 1, G(y->ln_g2), G(y->ln_b2));
        } else {
            memcpy(dy, dt, sizeof(float) * (size_t)TB * D);
            gemm_nn(TB, D, F1, dhp, F1, W(y->ff1), D, dy, D, 1);
        }
        /* ds1 -> dt */
        if (p->ln_flags & NNCU_LN_POST)
            norm_bwd(TB, D, dy, y->s1, W(y->ln_g1), rms, y->st_1, dt, 0, G(y->ln_g1), G(y->ln_b1));
        else
            memcpy(dt, dy, sizeof(float) * (size_t)TB * D);
        da = dt;
        if (y->alpha != NONE) {
            const float al = W(y->alpha)[0];
            double acc = 0.0;
            for (size_t i = 0; i < (size_t)TB * D; i++) {
                acc += (double)dt[i] * (double)y->a1[i];
                dal[i] = al * dt[i];
            }
            G(y->alpha)[0] += (float)acc;
            da = dal;
        }
        gemm_tn(D, HD, TB, da, D, y->o, HD, G(y->w_o), HD, 0);
        gemm_nn(TB, HD, D, da, D, W(y->w_o), HD, dof, HD, 0);
        attn_dims ad = {B, H, dk, T, M, p->d_pos, p->attn_len[l] ? p->attn_len[l] : L,
                        sqrtf((float)dk * (float)D)};
        /* tied tables accumulate into layer 0's gradient, nncp.c:742-744, 758-760 */
        attn_bwd(&ad, y->q, y->kv, WN(y->w_r), W(y->b_r), y->P, dof, dq, dkv,
                 y->w_r == NONE ? NULL : G(y->w_r), G(y->b_r));
        gemm_tn(HD, D, TB, dq, HD, y->hcat + (size_t)M * B * D, D, G(y->w_q), D, 0);
        if (y->b_q != NONE)
            colsum(TB, HD, dq, HD, G(y->b_q), 0);
        gemm_tn(2 * HD, D, LB, dkv, 2 * HD, y->hcat, D, G(y->w_kv), D, 0);
        /* dx1 = dq.w_q + dkv[segment rows].w_kv ; no gradient into the memory rows */
        gemm_nn(TB, D, HD, dq, HD, W(y->w_q), D, dy, D, 0);
        gemm_nn(TB, D, 2 * HD, dkv + (size_t)M * B * 2 * HD, 2 * HD, W(y->w_kv), D, dy, D, 1);
        /* dxin = ds1 + (pre-LN adjoint of dx1 | dx1) */
        memcpy(dx, dt, sizeof(float) * (size_t)TB * D);
        if (p->ln_flags & NNCU_LN_PRE)
            norm_bwd(TB, D, dy, y->xin, W(y->ln_g1), rms, y->st_pre1, dx, 1, G(y->ln_g1), G(y->ln_b1));
        else
            for (size_t i = 0; i < (size_t)TB * D; i++)
                dx[i] += dy[i];
    }
    /* embedding: dense scatter-add in row order (nc_get_col adjoint) */
    const float emul = sqrtf((float)D) * p->embed_mult;
    for (int r = 0; r < TB; r++) {
        float *ge = G(m->embed) + (size_t)m->ids[r] * D;
        for (int i = 0; i < D; i++)
            ge[i] += dx[(size_t)r * D + i] * emul;
    }
    free(dz); free(dx); free(dt); free(dy); free(dh); free(dhp); free(dof); free(dq); free(dkv); free(dal);
    return NNCU_OK;
}

/* model_update: optimizer, then mem_update (nncp.c:1205-1235) */
int orc_update(orc_model *m)
{
    const nncu_params *p = &m->p;
    m->step++;
    float corr = 1.0f;
    if (p->bias_correction)
        corr = 1.0f / (1.0f - powf(p->beta2, (float)m->step));
    for (int i = 0; i < m->n_params; i++) {
        orc_pinfo *pi = &m->pinfo[i];
        float *w = m->w + pi->off, *g = m->g + pi->off, *v = m->v + pi->off;
        for (size_t k = 0; k < pi->numel; k++) {
            float gg = g[k];
            if (p->gradient_clip != 0.0f) {
                if (gg > p->gradient_clip) gg = p->gradient_clip;
                if (gg < -p->gradient_clip) gg = -p->gradient_clip;
            }
            v[k] = p->beta2 * v[k] + (1.0f - p->beta2) * gg * gg;
            w[k] -= m->lr * gg / (sqrtf(v[k] * corr) + p->eps);
        }
    }
    /* memory <- last M rows (in time) of [mem ; segment] */
    const size_t rowsz = (size_t)p->n_streams * p->d_model;
    for (int l = 0; l < p->n_layer; l++) {
        float *h = m->layers[l].hcat;
        memmove(h, h + (size_t)p->seg_len * rowsz, sizeof(float) * (size_t)p->mem_len * rowsz);
    }
    m->steps_done = 0;
    return NNCU_OK;
}

/* ---- isolated attention op, same math as the model's (for the op-level tests) ---- */
int orc_attention_forward(const nncu_attn_shape *s, const float *q, const float *kv,
                          const float *w_r, const float *b_r, float *out, float *Pm, float *lse)
{
    attn_dims ad = {s->n_streams, s->n_head, s->d_key, s->seg_len, s->mem_len, s->d_pos,
                    s->attn_len ? s->attn_len : s->mem_len + s->seg_len, s->br_scale};
    attn_fwd(&ad, s->t0, s->t1, q, kv, w_r, b_r, out, Pm, lse);
    return NNCU_OK;
}

int orc_attention_backward(const nncu_attn_shape *s, const float *q, const float *kv,
                           const float *w_r, const float *b_r, const float *Pm,
                           const float *dout, float *dq, float *dkv, float *dw_r, float *db_r)
{
    attn_dims ad = {s->n_streams, s->n_head, s->d_key, s->seg_len, s->mem_len, s->d_pos,
                    s->attn_len ? s->attn_len : s->mem_len + s->seg_len, s->br_scale};
    attn_bwd(&ad, q, kv, w_r, b_r, Pm, dout, dq, dkv, dw_r, db_r);
    return NNCU_OK;
}
