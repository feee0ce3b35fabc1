/*
 * stream.c -- stream layout, learning-rate schedule, container header and the block loop.
 *
 *   nch_get_symb / nch_put_symb   nncp.c:2945-2965
 *   nch_interp                    cp_utils.c:380-410
 *   nch_process_block             nncp.c:2968-3147
 *   header                        nncp.c:2662-2690 (file), 1297-1365 (schedules, model)
 *   nch_compress / nch_decompress nncp.c:3414-3475, 3508-3677 (block sizing and loop)
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <zlib.h>

#include "nncp_host.h"

int nch_get_symb(const uint16_t *buf, int stride, int rem, int stream_idx, int pos)
{
    int len = stride + (stream_idx < rem);
    if (pos < 0 || pos >= len)
        return 0;
    return buf[(size_t)stride * stream_idx + (stream_idx < rem ? stream_idx : rem) + pos];
}

int nch_put_symb(uint16_t *buf, int stride, int rem, int stream_idx, int pos, int c)
{
    int len = stride + (stream_idx < rem);
    if (pos < 0 || pos >= len)
        return NCH_ERR_INVALID;
    buf[(size_t)stride * stream_idx + (stream_idx < rem ? stream_idx : rem) + pos] = (uint16_t)c;
    return NCH_OK;
}

float nch_interp(const nch_interp_params *p, int64_t pos)
{
    for (int i = 0; i < p->n_steps; i++) {
        if (pos < p->pos[i]) {
            int64_t from = i ? p->pos[i - 1] : 0;
            float t = (float)(pos - from) / (float)(p->pos[i] - from);
            return p->val[i] + t * (p->val[i + 1] - p->val[i]);
        }
    }
    float last = p->val[p->n_steps];
    if (p->decay_power == 0.0f || p->n_steps == 0)
        return last;
    float x = (float)pos / (float)p->pos[p->n_steps - 1];
    if (p->decay_power == 0.5f)
        return last / sqrtf(x); /* independent of pow() rounding, as the reference */
    return (float)(last * pow(x, -p->decay_power));
}

/* ------------------------------------------------------------------ block loop */

typedef struct {
    const nch_model_ops *m;
    nch_enc *enc;
    nch_dec *dec;
    int out_mode, n_bits;
    float *probs;      /* [rows][V]   (float mode) */
    uint16_t *coded;   /* paths [rows][n_bits] or trees [rows][1 << depth] */
    int32_t *syms;     /* [rows] */
} coder_io;

/* codes (or decodes) rows [t0, t0+nt) x streams; `limit_t`/`limit_b`: positions at
   t == limit_t with stream >= limit_b, and all t > limit_t, are skipped (block tail). */
static int code_rows(coder_io *io, uint16_t *buf, int stride, int rem, int base_pos, int t0, int nt,
                     int limit_t, int limit_b, int32_t *expected)
{
    const nch_model_ops *m = io->m;
    const int B = m->n_streams, V = m->n_symbols;
    if (io->enc) {
        for (int t = 0; t < nt; t++)
            for (int b = 0; b < B; b++)
                io->syms[t * B + b] = nch_get_symb(buf, stride, rem, b, base_pos + t0 + t);
        if (io->out_mode == NCH_OUT_CODER_READY) {
            int nb = 0;
            if (m->coder_paths(m->ctx, t0, nt, io->syms, io->coded, &nb))
                return NCH_ERR_MODEL;
            io->n_bits = nb;
        } else if (m->read_probs(m->ctx, t0, nt, io->probs)) {
            return NCH_ERR_MODEL;
        }
        for (int t = 0; t < nt; t++)
            for (int b = 0; b < B; b++) {
                int tt = t0 + t, c = io->syms[t * B + b];
                if (tt < limit_t || (tt == limit_t && b < limit_b)) {
                    if (io->out_mode == NCH_OUT_CODER_READY)
                        nch_write_sym_path_any(io->enc, io->coded + (size_t)(t * B + b) * io->n_bits, V, c);
                    else
                        nch_write_sym(io->enc, io->probs + (size_t)(t * B + b) * V, V, c);
                }
                if (expected)
                    expected[tt * B + b] = c;
            }
    } else {
        if (io->out_mode == NCH_OUT_CODER_READY) {
            if (m->coder_trees(m->ctx, t0, nt, io->coded))
                return NCH_ERR_MODEL;
        } else if (m->read_probs(m->ctx, t0, nt, io->probs)) {
            return NCH_ERR_MODEL;
        }
        for (int t = 0; t < nt; t++)
            for (int b = 0; b < B; b++) {
                int tt = t0 + t, c = 0;
                if (tt < limit_t || (tt == limit_t && b < limit_b)) {
                    if (io->out_mode == NCH_OUT_CODER_READY)
                        c = nch_read_sym_tree(io->dec, io->coded + ((size_t)(t * B + b) << nch_tree_depth(V)), V);
                    else
                        c = nch_read_sym(io->dec, io->probs + (size_t)(t * B + b) * V, V);
                    nch_put_symb(buf, stride, rem, b, base_pos + tt, c);
                }
                if (expected)
                    expected[tt * B + b] = c;
            }
    }
    return NCH_OK;
}

int nch_process_block(const nch_model_ops *m, nch_enc *enc, nch_dec *dec, uint16_t *block_buf,
                      int block_len, const nch_interp_params *lr, int64_t *train_step, int eval_mode,
                      int out_mode, nch_block_stats *stats)
{
    if (!m || (!enc) == (!dec) || !block_buf || block_len < 0 || !lr || !train_step)
        return NCH_ERR_INVALID;
    const int B = m->n_streams, T = m->seg_len, V = m->n_symbols;
    if (dec)
        eval_mode = NCH_EVAL_STEP; /* the next input is the symbol just decoded */
    if (out_mode == NCH_OUT_DEVICE)
        out_mode = NCH_OUT_CODER_READY; /* the device decoder is nch_decompress's; here the walk is the host's */
    if (out_mode == NCH_OUT_CODER_READY && (V < 2 || !m->coder_paths || !m->coder_trees))
        out_mode = NCH_OUT_FLOAT;
    const int stride = block_len / B, rem = block_len % B;
    coder_io io;
    memset(&io, 0, sizeof(io));
    io.m = m; io.enc = enc; io.dec = dec; io.out_mode = out_mode;
    const int rows = (eval_mode == NCH_EVAL_SEGMENT ? T : 1) * B;
    int32_t *input = (int32_t *)calloc((size_t)T * B, sizeof(int32_t));
    int32_t *expected = (int32_t *)calloc((size_t)T * B, sizeof(int32_t));
    io.syms = (int32_t *)calloc((size_t)rows, sizeof(int32_t));
    if (out_mode == NCH_OUT_CODER_READY)
        io.coded = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)rows * (enc ? 32 : (size_t)1 << nch_tree_depth(V)));
    else
        io.probs = (float *)malloc(sizeof(float) * (size_t)rows * V);
    int rc = NCH_OK;
    if (!input || !expected || !io.syms || (!io.coded && !io.probs)) {
        rc = NCH_ERR_NOMEM;
        goto done;
    }
    if (m->reset(m->ctx)) {
        rc = NCH_ERR_MODEL;
        goto done;
    }
    int pos = 0;
    /* Encoder order.  An encoder knows a segment's symbols before it codes them, and the next
       segment's too, so per full segment it queues: the coder values of this segment, its backward
       pass and update, and the next segment's forward pass -- and only then waits for the coder values
       and range-codes them, while the GPU trains.  Same kernels in the same order on the device, so
       the coded bytes are those of the loop below (process_block, nncp.c:3003-3053, runs eval, coder
       and gradient strictly in turn). */
    if (enc && eval_mode == NCH_EVAL_SEGMENT && out_mode == NCH_OUT_CODER_READY && m->coder_paths_begin &&
        m->coder_paths_end && m->eval_gradient_queue && m->read_loss) {
        int32_t *next_input = (int32_t *)calloc((size_t)T * B, sizeof(int32_t));
        if (!next_input) { rc = NCH_ERR_NOMEM; goto done; }
        int queued = 0;
        while (pos + T <= stride) {
            if (!queued) {
                for (int t = 0; t < T; t++)
                    for (int b = 0; b < B; b++)
                        input[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + t - 1);
                if (m->eval(m->ctx, -1, input)) { rc = NCH_ERR_MODEL; break; }
            }
            queued = 0;
            for (int t = 0; t < T; t++)
                for (int b = 0; b < B; b++)
                    expected[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + t);
            if (m->coder_paths_begin(m->ctx, 0, T, expected) || m->set_lr(m->ctx, nch_interp(lr, *train_step)) ||
                m->eval_gradient_queue(m->ctx, expected) || m->update(m->ctx)) { rc = NCH_ERR_MODEL; break; }
            if (pos + 2 * T <= stride) { /* the next full segment of this block */
                for (int t = 0; t < T; t++)
                    for (int b = 0; b < B; b++)
                        next_input[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + T + t - 1);
                if (m->eval(m->ctx, -1, next_input)) { rc = NCH_ERR_MODEL; break; }
                queued = 1;
            }
            int nbits = 0;
            if (m->coder_paths_end(m->ctx, io.coded, &nbits)) { rc = NCH_ERR_MODEL; break; }
            if (nbits != nch_tree_depth(V)) { rc = NCH_ERR_MODEL; break; }
            nch_write_sym_paths_any(enc, io.coded, V, expected, (size_t)T * B);
            float loss = 0.0f;
            if (m->read_loss(m->ctx, &loss)) { rc = NCH_ERR_MODEL; break; }
            (*train_step)++;
            pos += T;
            if (stats) {
                stats->train_steps++;
                stats->n_symbols += (int64_t)T * B;
                stats->sum_log2 -= (double)loss / 0.6931471805599453;
            }
        }
        free(next_input);
        if (rc) goto done;
    }
    /* full segments: code, then train on what was coded */
    while (pos + T <= stride) {
        if (eval_mode == NCH_EVAL_SEGMENT) {
            for (int t = 0; t < T; t++)
                for (int b = 0; b < B; b++)
                    input[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + t - 1);
            if (m->eval(m->ctx, -1, input)) { rc = NCH_ERR_MODEL; goto done; }
            rc = code_rows(&io, block_buf, stride, rem, pos, 0, T, T, 0, expected);
            if (rc) goto done;
        } else {
            for (int t = 0; t < T; t++) {
                for (int b = 0; b < B; b++)
                    input[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + t - 1);
                if (m->eval(m->ctx, t, input)) { rc = NCH_ERR_MODEL; goto done; }
                rc = code_rows(&io, block_buf, stride, rem, pos, t, 1, T, 0, expected);
                if (rc) goto done;
            }
        }
        if (m->set_lr(m->ctx, nch_interp(lr, *train_step))) { rc = NCH_ERR_MODEL; goto done; }
        float loss = 0.0f;
        if (m->eval_gradient(m->ctx, expected, &loss) || m->update(m->ctx)) { rc = NCH_ERR_MODEL; goto done; }
        (*train_step)++;
        pos += T;
        if (stats) {
            stats->train_steps++;
            stats->n_symbols += (int64_t)T * B;
            stats->sum_log2 -= (double)loss / 0.6931471805599453;
        }
    }
    /* tail: coded without training (nncp.c:3076-3143) */
    {
        const int tail2 = stride - pos, tail1 = tail2 + (rem != 0);
        if (tail1 > 0) {
            memset(input, 0, sizeof(int32_t) * (size_t)T * B);
            if (eval_mode == NCH_EVAL_SEGMENT) {
                for (int t = 0; t < tail1; t++)
                    for (int b = 0; b < B; b++)
                        input[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + t - 1);
                if (m->eval(m->ctx, -1, input)) { rc = NCH_ERR_MODEL; goto done; }
                rc = code_rows(&io, block_buf, stride, rem, pos, 0, tail1, tail2, rem, NULL);
                if (rc) goto done;
            } else {
                for (int t = 0; t < tail1; t++) {
                    for (int b = 0; b < B; b++)
                        input[t * B + b] = nch_get_symb(block_buf, stride, rem, b, pos + t - 1);
                    if (m->eval(m->ctx, t, input)) { rc = NCH_ERR_MODEL; goto done; }
                    rc = code_rows(&io, block_buf, stride, rem, pos, t, 1, tail2, rem, NULL);
                    if (rc) goto done;
                }
            }
            if (m->eval_end(m->ctx)) { rc = NCH_ERR_MODEL; goto done; }
            if (stats)
                stats->n_symbols += (int64_t)tail2 * B + rem;
        }
    }
done:
    free(input);
    free(expected);
    free(io.syms);
    free(io.coded);
    free(io.probs);
    return rc;
}

/* The decode side of process_block with the range decoder on the device: the same walk over the
   block (full segments decoded and trained on, then the untrained tail), one decode_steps call per
   segment instead of one eval + tree download + host walk per symbol. */
static int decode_block_device(const nch_model_ops *m, uint16_t *block_buf, int block_len,
                               const nch_interp_params *lr, int64_t *train_step)
{
    const int B = m->n_streams, T = m->seg_len;
    const int stride = block_len / B, rem = block_len % B;
    int32_t *ids0 = (int32_t *)calloc((size_t)B, sizeof(int32_t));
    int32_t *syms = (int32_t *)calloc((size_t)T * B, sizeof(int32_t));
    int rc = NCH_OK;
    if (!ids0 || !syms) {
        rc = NCH_ERR_NOMEM;
        goto done;
    }
    if (m->reset(m->ctx)) { rc = NCH_ERR_MODEL; goto done; }
    int pos = 0;
    while (pos + T <= stride) {
        for (int b = 0; b < B; b++)
            ids0[b] = nch_get_symb(block_buf, stride, rem, b, pos - 1);
        if (m->decode_steps(m->ctx, 0, T, ids0, T, 0, syms)) { rc = NCH_ERR_MODEL; goto done; }
        for (int t = 0; t < T; t++)
            for (int b = 0; b < B; b++)
                nch_put_symb(block_buf, stride, rem, b, pos + t, syms[t * B + b]);
        float loss = 0.0f;
        if (m->set_lr(m->ctx, nch_interp(lr, *train_step)) || m->eval_gradient(m->ctx, syms, &loss) ||
            m->update(m->ctx)) {
            rc = NCH_ERR_MODEL;
            goto done;
        }
        (*train_step)++;
        pos += T;
    }
    {
        const int tail2 = stride - pos, tail1 = tail2 + (rem != 0);
        if (tail1 > 0) {
            for (int b = 0; b < B; b++)
                ids0[b] = nch_get_symb(block_buf, stride, rem, b, pos - 1);
            if (m->decode_steps(m->ctx, 0, tail1, ids0, tail2, rem, syms)) { rc = NCH_ERR_MODEL; goto done; }
            for (int t = 0; t < tail1; t++)
                for (int b = 0; b < B; b++)
                    if (t < tail2 || b < rem)
                        nch_put_symb(block_buf, stride, rem, b, pos + t, syms[t * B + b]);
            if (m->eval_end(m->ctx)) { rc = NCH_ERR_MODEL; goto done; }
        }
    }
done:
    free(ids0);
    free(syms);
    return rc;
}

/* ------------------------------------------------------------------ header */

#define FILE_MAGIC 0xb727ac58u

typedef struct {
    uint8_t *p;
    size_t len, cap;
    int overflow;
} wbuf;
static void w8(wbuf *w, unsigned v)
{
    if (w->len < w->cap)
        w->p[w->len] = (uint8_t)v;
    else
        w->overflow = 1;
    w->len++;
}
static void w16(wbuf *w, unsigned v) { w8(w, v >> 8); w8(w, v); }
static void w32(wbuf *w, uint32_t v) { w16(w, v >> 16); w16(w, v & 0xffff); }
static void wf32(wbuf *w, float f) { uint32_t u; memcpy(&u, &f, 4); w32(w, u); }
static void winterp(wbuf *w, const nch_interp_params *p)
{
    w8(w, p->n_steps);
    for (int i = 0; i <= p->n_steps; i++)
        wf32(w, p->val[i]);
    for (int i = 0; i < p->n_steps; i++)
        w32(w, (uint32_t)p->pos[i]);
    wf32(w, p->decay_power);
}

typedef struct {
    const uint8_t *p;
    size_t len, pos;
    int bad;
} rbuf;
static unsigned r8(rbuf *r)
{
    if (r->pos >= r->len) {
        r->bad = 1;
        return 0;
    }
    return r->p[r->pos++];
}
static unsigned r16(rbuf *r) { unsigned a = r8(r); return (a << 8) | r8(r); }
static uint32_t r32(rbuf *r) { uint32_t a = r16(r); return (a << 16) | r16(r); }
static float rf32(rbuf *r) { uint32_t u = r32(r); float f; memcpy(&f, &u, 4); return f; }
static int rinterp(rbuf *r, nch_interp_params *p)
{
    memset(p, 0, sizeof(*p));
    unsigned n = r8(r);
    if (n > NCH_INTERP_MAX_STEPS)
        return -1;
    p->n_steps = (int)n;
    for (unsigned i = 0; i <= n; i++)
        p->val[i] = rf32(r);
    for (unsigned i = 0; i < n; i++)
        p->pos[i] = r32(r);
    p->decay_power = rf32(r);
    return 0;
}

/* Version 1 is the reference layout byte for byte.  Version 2 appends two bytes
   (init_kind, bias_correction) for the build-defined options the reference has no field for.
   Version 3 appends a third: the number of ranks the streams were sharded over.  The gradient sum
   over ranks has an order that depends on that number, so a file decodes only with the same one
   (the reference records use_cuda for the same reason and refuses a mismatch, nncp.c:2669,
   3543-3550). */
int nch_write_header(const nch_file_params *fp, uint32_t n_symbols_in_file, uint8_t *out, size_t cap,
                     size_t *len)
{
    if (!fp || !len)
        return NCH_ERR_INVALID;
    const nncu_params *m = &fp->model;
    const int v3 = fp->n_ranks > 1;
    const int v2 = v3 || m->init_kind != NNCU_INIT_UNIFORM || m->bias_correction != 0;
    if (fp->n_ranks > 255)
        return NCH_ERR_INVALID;
    wbuf w = {out, 0, out ? cap : 0, 0};
    w32(&w, FILE_MAGIC);
    w16(&w, v3 ? 3 : (v2 ? 2 : 1));
    w8(&w, 1);                 /* use_cuda */
    w8(&w, m->use_bf16);
    w16(&w, m->n_streams);     /* batch_size */
    w16(&w, m->seg_len);
    w16(&w, m->n_symbols);
    w32(&w, m->seed);
    winterp(&w, &fp->lr);
    winterp(&w, &fp->block_len);
    w32(&w, fp->retrain_period);
    if (fp->retrain_period != 0) { /* nncp.c:2679-2686 */
        w32(&w, fp->retrain_len);
        w8(&w, fp->has_retrain_lr != 0);
        if (fp->has_retrain_lr)
            winterp(&w, &fp->retrain_lr);
    }
    w8(&w, 0);                 /* model_id of the Transformer class */
    w8(&w, m->n_layer);
    w8(&w, m->n_head);
    w16(&w, m->d_key);
    w16(&w, m->d_value);
    w16(&w, m->d_inner);
    w16(&w, m->d_pos);
    w16(&w, m->mem_len);
    for (int i = 0; i < m->n_layer; i++)
        w16(&w, m->attn_len[i] ? m->attn_len[i] : m->mem_len + m->seg_len);
    w8(&w, 0);                 /* tied_embed */
    w8(&w, m->use_bias);
    w8(&w, m->use_w_r);
    w8(&w, m->tied_w_r);
    w8(&w, m->tied_b_r);
    w8(&w, m->query_bias);
    w8(&w, 0);                 /* rotary_pos_embed */
    w8(&w, m->ln_flags);
    wf32(&w, m->init_range);
    wf32(&w, m->embed_mult);
    w8(&w, m->ff_act);
    w8(&w, 1);                 /* SGD_OPT_ADAM, beta1 = 0: RMSProp */
    wf32(&w, 0.0f);
    wf32(&w, m->beta2);
    wf32(&w, m->eps);
    wf32(&w, m->gradient_clip);
    if (fp->retrain_period != 0) { /* dropout_prob, dropout_att_prob of the retrain pass (nncp.c:1360-1363) */
        wf32(&w, 0.0f);
        wf32(&w, 0.0f);
    }
    w8(&w, 0);                 /* use_sparse_grad */
    if (v2) {
        w8(&w, m->init_kind);
        w8(&w, m->bias_correction != 0);
    }
    if (v3)
        w8(&w, fp->n_ranks);
    if (fp->dict && fp->dict_len) {
        /* the dictionary text, deflated at level 9 behind its two sizes (nncp.c:3222-3261) */
        uLongf zlen = compressBound(fp->dict_len);
        uint8_t *z = (uint8_t *)malloc(zlen);
        if (!z)
            return NCH_ERR_NOMEM;
        if (compress2(z, &zlen, fp->dict, fp->dict_len, Z_BEST_COMPRESSION) != Z_OK) {
            free(z);
            return NCH_ERR_INVALID;
        }
        w8(&w, 1);
        w32(&w, fp->dict_len);
        w32(&w, (uint32_t)zlen);
        for (uLongf i = 0; i < zlen; i++)
            w8(&w, z[i]);
        free(z);
    } else {
        w8(&w, 0);             /* no preprocessing dictionary */
    }
    w32(&w, n_symbols_in_file);
    *len = w.len;
    return (out && w.overflow) ? NCH_ERR_INVALID : NCH_OK;
}

static int read_header(const uint8_t *in, size_t n, nch_file_params *fp, uint32_t *n_symbols_in_file,
                       size_t *consumed, size_t *z_at, size_t *z_len)
{
    if (!in || !fp)
        return NCH_ERR_INVALID;
    rbuf r = {in, n, 0, 0};
    memset(fp, 0, sizeof(*fp));
    nncu_params *m = &fp->model;
    if (r32(&r) != FILE_MAGIC)
        return NCH_ERR_FORMAT;
    unsigned ver = r16(&r);
    if (ver < 1 || ver > 3)
        return NCH_ERR_FORMAT;
    r8(&r); /* use_cuda */
    m->use_bf16 = (uint8_t)r8(&r);
    m->n_streams = (int)r16(&r);
    m->seg_len = (int)r16(&r);
    m->n_symbols = (int)r16(&r);
    m->seed = r32(&r);
    if (rinterp(&r, &fp->lr) || rinterp(&r, &fp->block_len))
        return NCH_ERR_FORMAT;
    fp->retrain_period = r32(&r);
    if (fp->retrain_period != 0) {
        fp->retrain_len = r32(&r);
        fp->has_retrain_lr = (int32_t)r8(&r);
        if (fp->has_retrain_lr && rinterp(&r, &fp->retrain_lr))
            return NCH_ERR_FORMAT;
        if (fp->retrain_len == 0)
            return NCH_ERR_FORMAT;
    }
    if (r8(&r) != 0)
        return NCH_ERR_FORMAT; /* not the Transformer class */
    m->n_layer = (int)r8(&r);
    m->n_head = (int)r8(&r);
    m->d_key = (int)r16(&r);
    m->d_value = (int)r16(&r);
    m->d_inner = (int)r16(&r);
    m->d_pos = (int)r16(&r);
    m->mem_len = (int)r16(&r);
    if (m->n_layer < 1 || m->n_layer > NNCU_N_LAYER_MAX)
        return NCH_ERR_FORMAT;
    for (int i = 0; i < m->n_layer; i++)
        m->attn_len[i] = (int)r16(&r);
    if (r8(&r) != 0)
        return NCH_ERR_FORMAT; /* tied_embed */
    m->use_bias = (uint8_t)r8(&r);
    m->use_w_r = (uint8_t)r8(&r);
    m->tied_w_r = (uint8_t)r8(&r);
    m->tied_b_r = (uint8_t)r8(&r);
    m->query_bias = (uint8_t)r8(&r);
    if (r8(&r) != 0)
        return NCH_ERR_FORMAT; /* rotary */
    m->ln_flags = (uint8_t)r8(&r);
    m->init_range = rf32(&r);
    m->embed_mult = rf32(&r);
    m->ff_act = (uint8_t)r8(&r);
    if (r8(&r) != 1)
        return NCH_ERR_FORMAT;
    rf32(&r); /* beta1 */
    m->beta2 = rf32(&r);
    m->eps = rf32(&r);
    m->gradient_clip = rf32(&r);
    if (fp->retrain_period != 0) {
        const float drop = rf32(&r), drop_att = rf32(&r);
        if (drop != 0.0f || drop_att != 0.0f)
            return NCH_ERR_FORMAT; /* retrain with dropout: not built */
    }
    r8(&r); /* use_sparse_grad */
    if (ver >= 2) {
        m->init_kind = (int)r8(&r);
        m->bias_correction = (int)r8(&r);
    }
    fp->n_ranks = ver >= 3 ? (int)r8(&r) : 1;
    if (fp->n_ranks < 1)
        return NCH_ERR_FORMAT;
    const unsigned has_dict = r8(&r) & 1;
    if (has_dict) { /* raw size, deflated size, zlib stream: skipped here, nch_read_dict inflates it */
        fp->dict_len = r32(&r);
        const uint32_t zlen = r32(&r);
        if (r.bad || zlen > r.len - r.pos || fp->dict_len == 0 || fp->dict_len > (1u << 28))
            return NCH_ERR_FORMAT; /* 65535 entries of 4096 bytes is the most the reference's decoder takes */
        if (z_at)
            *z_at = r.pos;
        if (z_len)
            *z_len = zlen;
        r.pos += zlen;
    }
    uint32_t nsym = r32(&r);
    if (r.bad)
        return NCH_ERR_FORMAT;
    m->d_model = m->d_key * m->n_head; /* not stored (nncp.c:1383) */
    m->n_streams_total = 0;
    m->device = -1;
    m->lr = fp->lr.val[0];
    if (n_symbols_in_file)
        *n_symbols_in_file = nsym;
    if (consumed)
        *consumed = r.pos;
    return NCH_OK;
}

int nch_read_header(const uint8_t *in, size_t n, nch_file_params *fp, uint32_t *n_symbols_in_file,
                    size_t *consumed)
{
    return read_header(in, n, fp, n_symbols_in_file, consumed, NULL, NULL);
}

int nch_read_dict(const uint8_t *in, size_t n, uint8_t **dict, size_t *dict_len)
{
    if (!in || !dict || !dict_len)
        return NCH_ERR_INVALID;
    nch_file_params fp;
    size_t z_at = 0, z_len = 0;
    *dict = NULL;
    *dict_len = 0;
    const int rc = read_header(in, n, &fp, NULL, NULL, &z_at, &z_len);
    if (rc || fp.dict_len == 0)
        return rc;
    uint8_t *text = (uint8_t *)malloc(fp.dict_len);
    if (!text)
        return NCH_ERR_NOMEM;
    uLongf got = fp.dict_len;
    if (uncompress(text, &got, in + z_at, (uLong)z_len) != Z_OK || got != fp.dict_len) {
        free(text);
        return NCH_ERR_FORMAT;
    }
    *dict = text;
    *dict_len = got;
    return NCH_OK;
}

/* ------------------------------------------------------------------ file loops */

int nch_next_block_len(const nch_file_params *fp, size_t file_pos, size_t remaining)
{
    const int unit = fp->model.seg_len * fp->model.n_streams;
    long bl = lrintf(nch_interp(&fp->block_len, (int64_t)file_pos));
    long k = bl / unit;
    if (k < 1)
        k = 1;
    bl = k * unit;
    if ((size_t)bl > remaining)
        bl = (long)remaining;
    return (int)bl;
}

void nch_free(void *p) { free(p); }

/* ---- the retrain pass between blocks (retrain_block, nncp.c:2821-2941) ---- */
typedef struct {
    uint16_t *ring;    /* the last retrain_len symbols coded */
    int size, next, len;
    int64_t since;     /* symbols coded since the last pass */
    int64_t step;      /* the pass's own step counter, for its own schedule */
} retrain_state;

static int retrain_init(retrain_state *rs, const nch_file_params *fp)
{
    memset(rs, 0, sizeof(*rs));
    if (fp->retrain_period == 0)
        return NCH_OK;
    rs->size = (int)fp->retrain_len;
    rs->ring = (uint16_t *)calloc((size_t)rs->size, sizeof(uint16_t));
    return rs->ring ? NCH_OK : NCH_ERR_NOMEM;
}

/* symbol idx of the ring counted from its oldest one; 0 in front of it (get_symb_fifo, nncp.c:2811-2819) */
static int ring_at(const retrain_state *rs, int idx)
{
    return idx < 0 ? 0 : rs->ring[(rs->next + idx) % rs->len];
}

/* The block just coded goes into the ring; once retrain_period symbols have gone by, the model is
   reset and trained over the ring: n_streams contiguous runs of it side by side, whole segments
   only, with the pass's own schedule and step counter when it has one and the coder's otherwise. */
static int retrain_pass(const nch_model_ops *m, retrain_state *rs, const nch_file_params *fp, const uint16_t *block,
                        int block_len, int64_t *train_step)
{
    if (fp->retrain_period == 0)
        return NCH_OK;
    for (int done = 0; done < block_len;) {
        int l = rs->size - rs->next < block_len - done ? rs->size - rs->next : block_len - done;
        memcpy(rs->ring + rs->next, block + done, sizeof(uint16_t) * (size_t)l);
        rs->next = rs->next + l == rs->size ? 0 : rs->next + l;
        done += l;
    }
    rs->len = rs->len + block_len < rs->size ? rs->len + block_len : rs->size;
    rs->since += block_len;
    if (rs->since < (int64_t)fp->retrain_period)
        return NCH_OK;
    rs->since = 0;
    const int B = m->n_streams, T = m->seg_len, run = rs->len / B;
    if (run == 0)
        return NCH_OK;
    int32_t *input = (int32_t *)malloc(sizeof(int32_t) * (size_t)T * B);
    int32_t *expected = (int32_t *)malloc(sizeof(int32_t) * (size_t)T * B);
    int rc = (input && expected) ? NCH_OK : NCH_ERR_NOMEM;
    if (!rc && m->reset(m->ctx))
        rc = NCH_ERR_MODEL;
    for (int at = 0; !rc && (int64_t)rs->len >= (int64_t)(T + at) * B; at += T) {
        for (int t = 0; t < T; t++)
            for (int b = 0; b < B; b++) {
                input[t * B + b] = ring_at(rs, run * b + at + t - 1);
                expected[t * B + b] = ring_at(rs, run * b + at + t);
            }
        const float lr = fp->has_retrain_lr ? nch_interp(&fp->retrain_lr, rs->step) : nch_interp(&fp->lr, *train_step);
        float loss = 0.0f;
        if (m->eval(m->ctx, -1, input) || m->set_lr(m->ctx, lr) || m->eval_gradient(m->ctx, expected, &loss) ||
            m->update(m->ctx))
            rc = NCH_ERR_MODEL;
        if (fp->has_retrain_lr)
            rs->step++;
        else
            (*train_step)++;
    }
    free(input);
    free(expected);
    return rc;
}

int nch_compress(const nch_model_ops *m, const nch_file_params *fp, const uint16_t *symbols, size_t n,
                 int eval_mode, int out_mode, uint8_t **out, size_t *out_len, nch_block_stats *stats)
{
    if (!m || !fp || (!symbols && n) || !out || !out_len)
        return NCH_ERR_INVALID;
    if (fp->n_ranks > 1)
        return NCH_ERR_RANKS; /* one process cannot produce the sums of n_ranks */
    size_t hlen = 0;
    nch_write_header(fp, (uint32_t)n, NULL, 0, &hlen);
    nch_enc *enc = nch_enc_new();
    if (!enc)
        return NCH_ERR_NOMEM;
    int rc = NCH_OK;
    int64_t train_step = 0;
    uint16_t *block = NULL;
    size_t pos = 0;
    retrain_state rs;
    if (retrain_init(&rs, fp)) {
        nch_enc_free(enc);
        return NCH_ERR_NOMEM;
    }
    while (pos < n) {
        int bl = nch_next_block_len(fp, pos, n - pos);
        uint16_t *nb = (uint16_t *)realloc(block, sizeof(uint16_t) * (size_t)bl);
        if (!nb) { rc = NCH_ERR_NOMEM; break; }
        block = nb;
        memcpy(block, symbols + pos, sizeof(uint16_t) * (size_t)bl);
        rc = nch_process_block(m, enc, NULL, block, bl, &fp->lr, &train_step, eval_mode, out_mode, stats);
        if (rc)
            break;
        pos += (size_t)bl;
        if (pos < n) { /* no pass after the last block (nncp.c:3470-3474) */
            rc = retrain_pass(m, &rs, fp, symbols + pos - (size_t)bl, bl, &train_step);
            if (rc)
                break;
        }
    }
    free(block);
    free(rs.ring);
    if (rc == NCH_OK) {
        const uint8_t *payload = NULL;
        size_t plen = nch_enc_finish(enc, &payload);
        uint8_t *buf = (uint8_t *)malloc(hlen + plen + 1);
        if (!buf) {
            rc = NCH_ERR_NOMEM;
        } else {
            nch_write_header(fp, (uint32_t)n, buf, hlen, &hlen);
            if (plen)
                memcpy(buf + hlen, payload, plen);
            *out = buf;
            *out_len = hlen + plen;
        }
    }
    nch_enc_free(enc);
    return rc;
}

int nch_decompress(const nch_model_ops *m, const nch_file_params *fp, const uint8_t *payload, size_t n,
                   uint32_t n_symbols_in_file, int out_mode, uint16_t *symbols_out)
{
    if (!m || !fp || (!payload && n) || (!symbols_out && n_symbols_in_file))
        return NCH_ERR_INVALID;
    if (fp->n_ranks > 1)
        return NCH_ERR_RANKS; /* coded by a job of n_ranks processes: this single-process loop cannot repeat its sums */
    int rc = NCH_OK;
    int64_t train_step = 0;
    size_t pos = 0, total = n_symbols_in_file;
    if (out_mode == NCH_OUT_DEVICE) {
        /* a model without a device decoder, or one that refuses this geometry, decodes on the host;
           so does a file with a retrain pass, whose train steps run between the blocks */
        if (fp->retrain_period == 0 && m->decoder_begin && m->decode_steps && m->decoder_end && m->n_symbols >= 2 &&
            m->decoder_begin(m->ctx, payload, n) == 0) {
            while (pos < total) {
                int bl = nch_next_block_len(fp, pos, total - pos);
                rc = decode_block_device(m, symbols_out + pos, bl, &fp->lr, &train_step);
                if (rc)
                    break;
                pos += (size_t)bl;
            }
            size_t used = 0;
            if (m->decoder_end(m->ctx, &used) && !rc)
                rc = NCH_ERR_MODEL;
            return rc;
        }
        out_mode = NCH_OUT_CODER_READY;
    }
    nch_dec *dec = nch_dec_new(payload, n);
    if (!dec)
        return NCH_ERR_NOMEM;
    retrain_state rs;
    if (retrain_init(&rs, fp)) {
        nch_dec_free(dec);
        return NCH_ERR_NOMEM;
    }
    while (pos < total) {
        int bl = nch_next_block_len(fp, pos, total - pos);
        rc = nch_process_block(m, NULL, dec, symbols_out + pos, bl, &fp->lr, &train_step, NCH_EVAL_STEP,
                               out_mode, NULL);
        if (rc)
            break;
        pos += (size_t)bl;
        if (pos < total) {
            rc = retrain_pass(m, &rs, fp, symbols_out + pos - (size_t)bl, bl, &train_step);
            if (rc)
                break;
        }
    }
    free(rs.ring);
    nch_dec_free(dec);
    return rc;
}
