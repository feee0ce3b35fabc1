/*
 * coder.c -- binary range coder with 15-bit probabilities and the n-ary symbol coder on
 * top of it.  Produces / consumes the byte stream of the reference coder bit for bit
 * (put_bit, get_bit, put_bit_flush: arith.c:43-310; write_sym, read_sym:
 * cp_utils.c:299-349): range in [0xFF01, 0xFF0000], one byte shifted out per
 * renormalisation, carries resolved through a counter of pending 0xFF bytes, the decoder
 * padding with zero bytes past the end of its input.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "nncp_host.h"

#define P_BITS 15
#define P_ONE (1 << P_BITS)
#define R_SHIFT 16
#define R_LOW ((0xffu << (R_SHIFT - 8)) + 1u) /* renormalise below this */
#define R_TOP (0xffu << R_SHIFT)

struct nch_enc {
    uint32_t low, range;
    uint32_t run;  /* bytes held back: `head` followed by run-1 times 0xff */
    uint8_t head;
    uint8_t *buf;
    size_t len, cap;
};

static void enc_byte(nch_enc *e, unsigned v)
{
    if (e->len == e->cap) {
        size_t ncap = e->cap ? e->cap * 2 : 1 << 16;
        uint8_t *nb = (uint8_t *)realloc(e->buf, ncap);
        if (!nb)
            abort();
        e->buf = nb;
        e->cap = ncap;
    }
    e->buf[e->len++] = (uint8_t)v;
}

/* v in [0, 0x1fe]: bit 8 is a carry into the bytes held back */
static void enc_shift_out(nch_enc *e, unsigned v)
{
    if (v == 0xff) { /* cannot know yet whether a carry will ripple through it */
        e->run++;
        return;
    }
    if (e->run) {
        unsigned carry = v >> 8;
        enc_byte(e, e->head + carry);
        for (uint32_t i = 1; i < e->run; i++)
            enc_byte(e, (0xff + carry) & 0xff);
    }
    e->run = 1;
    e->head = (uint8_t)v;
}

static void enc_normalise(nch_enc *e)
{
    while (e->range < R_LOW) {
        enc_shift_out(e, e->low >> R_SHIFT);
        e->low = (e->low & ((1u << R_SHIFT) - 1u)) << 8;
        e->range <<= 8;
    }
}

nch_enc *nch_enc_new(void)
{
    nch_enc *e = (nch_enc *)calloc(1, sizeof(*e));
    if (e) {
        e->range = R_TOP;
        e->head = 0xff;
    }
    return e;
}

void nch_enc_put_bit(nch_enc *e, int prob0, int bit)
{
    uint32_t split = (uint32_t)(((uint64_t)e->range * (uint32_t)prob0) >> P_BITS);
    if (bit) {
        e->low += split;
        e->range -= split;
    } else {
        e->range = split;
    }
    enc_normalise(e);
}

size_t nch_enc_bytes(const nch_enc *e) { return e->len + e->run; }

size_t nch_enc_finish(nch_enc *e, const uint8_t **out)
{
    if (e->range < (1u << R_SHIFT)) {
        enc_shift_out(e, e->low >> R_SHIFT);
        e->low = (e->low & ((1u << R_SHIFT) - 1u)) << 8;
        e->range <<= 8;
    }
    int n = 0; /* largest n with 2^n <= range: the value is rounded up to n trailing zero bits */
    while ((1u << (n + 1)) <= e->range)
        n++;
    uint32_t v = e->low, mask = (1u << n) - 1u;
    if (v & mask)
        v = (v + (1u << n)) & ~mask;
    enc_shift_out(e, v >> R_SHIFT);
    if (e->run)
        enc_shift_out(e, 0); /* pushes the held bytes out; the 0 itself stays held */
    if (out)
        *out = e->buf;
    return e->len;
}

void nch_enc_free(nch_enc *e)
{
    if (e) {
        free(e->buf);
        free(e);
    }
}

struct nch_dec {
    const uint8_t *buf;
    size_t len, pos;
    uint32_t low, range;
};

static void dec_pull(nch_dec *d)
{
    d->range <<= 8;
    d->low <<= 8;
    if (d->pos < d->len)
        d->low += d->buf[d->pos++];
}

nch_dec *nch_dec_new(const uint8_t *buf, size_t len)
{
    nch_dec *d = (nch_dec *)calloc(1, sizeof(*d));
    if (!d)
        return NULL;
    d->buf = buf;
    d->len = len;
    for (int i = 0; i <= R_SHIFT; i += 8)
        dec_pull(d);
    d->range = R_TOP;
    return d;
}

int nch_dec_get_bit(nch_dec *d, int prob0)
{
    uint32_t split = (uint32_t)(((uint64_t)d->range * (uint32_t)prob0) >> P_BITS);
    int bit = d->low >= split;
    if (bit) {
        d->low -= split;
        d->range -= split;
    } else {
        d->range = split;
    }
    while (d->range < R_LOW)
        dec_pull(d);
    return bit;
}

void nch_dec_free(nch_dec *d) { free(d); }

/* ---- symbols ---- */

float nch_vec_sum_f32(const float *tab, size_t n)
{
    if (n <= 1)
        return n ? tab[0] : 0.0f;
    size_t h = n >> 1;
    return nch_vec_sum_f32(tab, h) + nch_vec_sum_f32(tab + h, n - h);
}

static int quantise(float p0, float p)
{
    int q = (int)lrintf(p0 * P_ONE / p);
    return q < 1 ? 1 : (q > P_ONE - 1 ? P_ONE - 1 : q);
}

void nch_write_sym(nch_enc *e, const float *prob, int n_symb, int sym)
{
    int lo = 0, n = n_symb;
    float mass = 1.0f;
    while (n > 1) {
        int h = n >> 1;
        float left = nch_vec_sum_f32(prob + lo, h);
        int right = sym >= lo + h;
        nch_enc_put_bit(e, quantise(left, mass), right);
        if (right) {
            lo += h;
            n -= h;
            mass -= left;
        } else {
            n = h;
            mass = left;
        }
    }
}

int nch_read_sym(nch_dec *d, const float *prob, int n_symb)
{
    int lo = 0, n = n_symb;
    float mass = 1.0f;
    while (n > 1) {
        int h = n >> 1;
        float left = nch_vec_sum_f32(prob + lo, h);
        if (nch_dec_get_bit(d, quantise(left, mass))) {
            lo += h;
            n -= h;
            mass -= left;
        } else {
            n = h;
            mass = left;
        }
    }
    return lo;
}

void nch_write_sym_path(nch_enc *e, const uint16_t *prob0, int n_bits, int sym)
{
    for (int k = 0; k < n_bits; k++)
        nch_enc_put_bit(e, prob0[k], (sym >> (n_bits - 1 - k)) & 1);
}

/* write_sym's walk over any alphabet: the node covering [lo, lo + n) sends n >> 1 symbols left */
void nch_write_sym_path_any(nch_enc *e, const uint16_t *prob0, int n_symb, int sym)
{
    int lo = 0, n = n_symb, k = 0;
    while (n > 1) {
        const int h = n >> 1, right = sym >= lo + h;
        nch_enc_put_bit(e, prob0[k++], right);
        if (right) {
            lo += h;
            n -= h;
        } else {
            n = h;
        }
    }
}

int nch_read_sym_tree(nch_dec *d, const uint16_t *tree, int n_symb)
{
    int lo = 0, n = n_symb, k = 1;
    while (n > 1) {
        const int h = n >> 1, right = nch_dec_get_bit(d, tree[k]);
        k = 2 * k + right;
        if (right) {
            lo += h;
            n -= h;
        } else {
            n = h;
        }
    }
    return lo;
}

int nch_tree_depth(int n_symb)
{
    int d = 0;
    while ((1 << d) < n_symb)
        d++;
    return d;
}

void nch_write_sym_paths(nch_enc *e, const uint16_t *prob0, int n_bits, const int32_t *sym, size_t n)
{
    for (size_t i = 0; i < n; i++)
        nch_write_sym_path(e, prob0 + i * (size_t)n_bits, n_bits, sym[i]);
}

void nch_write_sym_paths_any(nch_enc *e, const uint16_t *prob0, int n_symb, const int32_t *sym, size_t n)
{
    const size_t stride = (size_t)nch_tree_depth(n_symb);
    for (size_t i = 0; i < n; i++)
        nch_write_sym_path_any(e, prob0 + i * stride, n_symb, sym[i]);
}

void nch_read_sym_trees(nch_dec *d, const uint16_t *trees, int n_symb, size_t n, int32_t *sym_out)
{
    const size_t stride = (size_t)1 << nch_tree_depth(n_symb);
    for (size_t i = 0; i < n; i++)
        sym_out[i] = nch_read_sym_tree(d, trees + i * stride, n_symb);
}
