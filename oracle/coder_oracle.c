/*
 * coder_oracle.c -- CPU restatement of NNCP's symbol coder and range coder.
 *
 * TEST INFRASTRUCTURE ONLY (see trf_oracle.c).  Pinned bit for bit against the
 * reference's own arith.c + cp_utils.c, which compile here unchanged into
 * oracle/_ref/libref_coder.so (tests/test_coder_oracle.py).
 *
 *   orc_vec_sum_f32     vec_sum_f32, a LibNC symbol (libnc.h:600) whose
 *                       order the backend defines; here it is the coder's own
 *                       halving recursion so that every node's left-half sum is
 *                       one node of a single bottom-up fp32 reduction tree
 *   orc_enc_put_sym     write_sym            cp_utils.c:299-323
 *   orc_dec_read_sym    read_sym             cp_utils.c:325-349
 *   put_bit / renorm    put_bit, put_val     arith.c:43-145
 *   flush               put_bit_flush        arith.c:162-194
 *   get_bit / refill    get_bit, refill      arith.c:208-283
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PROB_BITS 15
#define PROB_ONE (1 << PROB_BITS)
#define RMIN_BITS 16
#define RMIN ((0xff << (RMIN_BITS - 8)) + 1)
#define RMAX (0xff << RMIN_BITS)

float orc_vec_sum_f32(const float *tab, size_t n)
{
    if (n == 0)
        return 0.0f;
    if (n == 1)
        return tab[0];
    size_t h = n >> 1;
    return orc_vec_sum_f32(tab, h) + orc_vec_sum_f32(tab + h, n - h);
}

typedef struct {
    uint32_t range, low;
    uint8_t pending;     /* first byte of the pending run (never 0xff) */
    uint32_t n_pending;  /* run length: pending, then n_pending-1 times 0xff */
    uint8_t *buf;
    size_t cap, len;
} orc_enc;

static void emit(orc_enc *e, int v)
{
    if (e->len == e->cap) {
        e->cap = e->cap ? e->cap * 2 : 4096;
        e->buf = (uint8_t *)realloc(e->buf, e->cap);
    }
    e->buf[e->len++] = (uint8_t)v;
}

/* carry-propagating byte output, arith.c:72-94 */
static void out_val(orc_enc *e, int v)
{
    if (v == 0xff) {
        e->n_pending++;
        return;
    }
    if (e->n_pending > 0) {
        int carry = v >> 8;
        emit(e, e->pending + carry);
        int fill = (0xff + carry) & 0xff;
        for (; e->n_pending > 1; e->n_pending--)
            emit(e, fill);
    }
    e->n_pending = 1;
    e->pending = (uint8_t)v;
}

static void renorm(orc_enc *e)
{
    while (e->range < RMIN) {
        out_val(e, e->low >> RMIN_BITS);
        e->low = (e->low & ((1u << RMIN_BITS) - 1)) << 8;
        e->range <<= 8;
    }
}

orc_enc *orc_enc_new(void)
{
    orc_enc *e = (orc_enc *)calloc(1, sizeof(*e));
    e->range = RMAX;
    e->pending = 0xff;
    return e;
}

void orc_enc_put_bit(orc_enc *e, int prob0, int bit)
{
    uint32_t r0 = (uint32_t)(((uint64_t)e->range * (uint32_t)prob0) >> PROB_BITS);
    if (!bit) {
        e->range = r0;
    } else {
        e->low += r0;
        e->range -= r0;
    }
    renorm(e);
}

void orc_enc_put_sym(orc_enc *e, const float *prob, int n_symb, int sym)
{
    int start = 0, range = n_symb;
    float p = 1.0f;
    while (range > 1) {
        int half = range >> 1;
        float p0 = orc_vec_sum_f32(prob + start, half);
        int prob0 = (int)lrintf(p0 * PROB_ONE / p);
        if (prob0 < 1) prob0 = 1;
        if (prob0 > PROB_ONE - 1) prob0 = PROB_ONE - 1;
        int bit = sym >= start + half;
        orc_enc_put_bit(e, prob0, bit);
        if (bit) {
            start += half;
            range -= half;
            p = p - p0;
        } else {
            p = p0;
            range = half;
        }
    }
}

/* arith.c:162-194; returns the byte count, *out points at the bytes */
size_t orc_enc_finish(orc_enc *e, const uint8_t **out)
{
    if (e->range < (1u << RMIN_BITS)) {
        out_val(e, e->low >> RMIN_BITS);
        e->low = (e->low & ((1u << RMIN_BITS) - 1)) << 8;
        e->range <<= 8;
    }
    int n = 0;
    while ((1u << (n + 1)) <= e->range)
        n++;
    uint32_t val = e->low, mask = (1u << n) - 1;
    if (val & mask)
        val = (val + (1u << n)) & ~mask;
    out_val(e, val >> RMIN_BITS);
    if (e->n_pending > 0)
        out_val(e, 0);
    *out = e->buf;
    return e->len;
}

void orc_enc_free(orc_enc *e)
{
    if (e) {
        free(e->buf);
        free(e);
    }
}

typedef struct {
    const uint8_t *buf;
    size_t len, idx;
    uint32_t range, low;
} orc_dec;

static void refill(orc_dec *d)
{
    d->range <<= 8;
    d->low <<= 8;
    if (d->idx < d->len)
        d->low += d->buf[d->idx++]; /* past the end: zero padding, arith.c:209-223 */
}

orc_dec *orc_dec_new(const uint8_t *buf, size_t len)
{
    orc_dec *d = (orc_dec *)calloc(1, sizeof(*d));
    d->buf = buf;
    d->len = len;
    for (int i = 0; i <= RMIN_BITS; i += 8)
        refill(d);
    d->range = RMAX;
    return d;
}

int orc_dec_get_bit(orc_dec *d, int prob0)
{
    uint32_t r0 = (uint32_t)(((uint64_t)d->range * (uint32_t)prob0) >> PROB_BITS);
    int b = d->low >= r0;
    if (b) {
        d->low -= r0;
        d->range -= r0;
    } else {
        d->range = r0;
    }
    while (d->range < RMIN)
        refill(d);
    return b;
}

int orc_dec_read_sym(orc_dec *d, const float *prob, int n_symb)
{
    int start = 0, range = n_symb;
    float p = 1.0f;
    while (range > 1) {
        int half = range >> 1;
        float p0 = orc_vec_sum_f32(prob + start, half);
        int prob0 = (int)lrintf(p0 * PROB_ONE / p);
        if (prob0 < 1) prob0 = 1;
        if (prob0 > PROB_ONE - 1) prob0 = PROB_ONE - 1;
        int bit = orc_dec_get_bit(d, prob0);
        if (bit) {
            start += half;
            range -= half;
            p = p - p0;
        } else {
            p = p0;
            range = half;
        }
    }
    return start;
}

void orc_dec_free(orc_dec *d) { free(d); }

/* The prob0 values write_sym would emit for sym, root first; returns their count. */
int orc_sym_path(const float *prob, int n_symb, int sym, uint16_t *prob0_out)
{
    int start = 0, range = n_symb, k = 0;
    float p = 1.0f;
    while (range > 1) {
        int half = range >> 1;
        float p0 = orc_vec_sum_f32(prob + start, half);
        int prob0 = (int)lrintf(p0 * PROB_ONE / p);
        if (prob0 < 1) prob0 = 1;
        if (prob0 > PROB_ONE - 1) prob0 = PROB_ONE - 1;
        prob0_out[k++] = (uint16_t)prob0;
        if (sym >= start + half) {
            start += half;
            range -= half;
            p = p - p0;
        } else {
            p = p0;
            range = half;
        }
    }
    return k;
}

/* Every node's prob0 in heap order (root 1, children 2k and 2k+1; the node covering n symbols
   sends n >> 1 of them left, as write_sym does): what read_sym would hand get_bit at that node.
   tree_out has 1 << ceil(log2 n_symb) entries; entry 0 and the slots of one-symbol nodes stay 0. */
static void sym_tree_node(const float *prob, int start, int range, float p, unsigned k, uint16_t *tree_out)
{
    if (range <= 1)
        return;
    int half = range >> 1;
    float p0 = orc_vec_sum_f32(prob + start, half);
    int prob0 = (int)lrintf(p0 * PROB_ONE / p);
    if (prob0 < 1) prob0 = 1;
    if (prob0 > PROB_ONE - 1) prob0 = PROB_ONE - 1;
    tree_out[k] = (uint16_t)prob0;
    sym_tree_node(prob, start, half, p0, 2 * k, tree_out);
    sym_tree_node(prob, start + half, range - half, p - p0, 2 * k + 1, tree_out);
}

int orc_sym_tree(const float *prob, int n_symb, uint16_t *tree_out)
{
    int depth = 0;
    while ((1 << depth) < n_symb)
        depth++;
    memset(tree_out, 0, sizeof(uint16_t) << depth);
    sym_tree_node(prob, 0, n_symb, 1.0f, 1, tree_out);
    return 1 << depth;
}
