/*
 * ref_glue.c -- handle-based wrappers around the REFERENCE's own coder
 * (arith.c, cp_utils.c, cutils.c compiled unchanged from the reference tree)
 * so that tests can drive it through ctypes.  TEST INFRASTRUCTURE ONLY.
 *
 * The only definition added is vec_sum_f32 (declared libnc.h:600, implemented
 * in LibNC, which the reference tree does not contain): the halving recursion
 * that makes each node's left-half sum a node of one fp32 reduction tree.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/types.h>

#include "cutils.h"
#include "arith.h"
#include "libnc.h"
#include "cp_utils.h"

float vec_sum_f32(const float *tab, size_t n)
{
    if (n == 0)
        return 0.0f;
    if (n == 1)
        return tab[0];
    size_t h = n >> 1;
    return vec_sum_f32(tab, h) + vec_sum_f32(tab + h, n - h);
}

typedef struct {
    PutBitState pb;
    uint8_t chunk[4096];
    uint8_t *out;
    size_t len, cap;
} ref_enc;

static void ref_write(void *opaque, const uint8_t *buf, size_t n)
{
    ref_enc *e = opaque;
    if (e->len + n > e->cap) {
        e->cap = (e->len + n) * 2;
        e->out = realloc(e->out, e->cap);
    }
    memcpy(e->out + e->len, buf, n);
    e->len += n;
}

ref_enc *ref_enc_new(void)
{
    ref_enc *e = calloc(1, sizeof(*e));
    put_bit_init(&e->pb, e->chunk, sizeof(e->chunk), ref_write, e);
    return e;
}

void ref_enc_put_sym(ref_enc *e, const float *prob, int n_symb, int sym)
{
    write_sym(&e->pb, prob, n_symb, sym);
}

void ref_enc_put_bit(ref_enc *e, int prob0, int bit) { put_bit(&e->pb, prob0, bit); }

size_t ref_enc_finish(ref_enc *e, const uint8_t **out)
{
    put_bit_flush(&e->pb);
    *out = e->out;
    return e->len;
}

void ref_enc_free(ref_enc *e)
{
    if (e) {
        free(e->out);
        free(e);
    }
}

typedef struct {
    GetBitState gb;
    uint8_t *copy;
} ref_dec;

ref_dec *ref_dec_new(const uint8_t *buf, size_t len)
{
    ref_dec *d = calloc(1, sizeof(*d));
    d->copy = malloc(len ? len : 1);
    memcpy(d->copy, buf, len);
    get_bit_init(&d->gb, d->copy, len, NULL, NULL);
    return d;
}

int ref_dec_read_sym(ref_dec *d, const float *prob, int n_symb)
{
    return read_sym(&d->gb, prob, n_symb);
}

int ref_dec_get_bit(ref_dec *d, int prob0) { return get_bit(&d->gb, prob0); }

void ref_dec_free(ref_dec *d)
{
    if (d) {
        free(d->copy);
        free(d);
    }
}

/* learning-rate / block-length schedule, cp_utils.c:380-410 */
float ref_interp(int n_steps, const float *val, const int64_t *pos, float decay_power,
                 int64_t at)
{
    InterpParams p;
    memset(&p, 0, sizeof(p));
    p.n_steps = n_steps;
    for (int i = 0; i <= n_steps; i++)
        p.val[i] = val[i];
    for (int i = 0; i < n_steps; i++)
        p.pos[i] = pos[i];
    p.decay_power = decay_power;
    return get_interp_param(&p, at);
}
