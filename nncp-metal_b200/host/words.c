/*
 * words.c -- the word tokenizer that sits in front of the model when text preprocessing is on
 * (nch_words_encode / nch_words_decode / nch_words_count of include/nncp_host.h).
 *
 * It restates the reference preprocessor (preprocess.c) so that a dictionary and a symbol
 * stream made here are byte for byte the ones `nncp --preprocess n_words,min_freq` makes, and
 * either side decodes the other's files:
 *   - case/space folding (preprocess.c:967-1041): a run of letters becomes
 *     [NO_SPACE]? [ALL_UPPER | FIRST_UPPER]? ' ' lower-case letters, the space in front of
 *     a word is absorbed into the marker, and input bytes 1..4 are escaped;
 *   - the dictionary (preprocess.c:1093-1226): rounds of pair merging.  Every round counts the
 *     adjacent pairs of the buffer, scores each by the bits it would save (fixed point log2
 *     with 10 fractional bits, :675-760), takes at most 100 of the best that do not chain with
 *     one another (:762-822), substitutes them greedily left to right, and expands again the
 *     words that then occur fewer than min_freq times (:887-927);
 *   - the output (preprocess.c:397-528): entries 0..255 are the bytes, the words that survived
 *     follow in byte order; the dictionary is one entry per line with '\n' written "\\n" and
 *     '\\' written "\\\\";
 *   - decoding (preprocess.c:1051-1091, 1227-1323).
 * Where the reference leaves the order of equal keys to the C library's qsort, this file keeps
 * the order of first occurrence (a stable sort), which is what a merge-sort qsort gives it.
 *
 * The results are the reference's; the way to them is not.  The reference counts every pair of
 * the buffer anew in each round.  Here the pair counts are made once and then follow each rewrite
 * of the buffer (a substitution or an expansion changes the pairs inside it and the two across its
 * borders), the symbol counts likewise; only candidates with a positive score are sorted, and the
 * place of first occurrence, which only breaks ties between equal scores, is looked up for the
 * tied candidates the selection actually reaches.  A round then costs two streaming passes over
 * the buffer and table work in proportion to what changed.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "nncp_host.h"

enum {
    N_BYTES = 256,       /* symbols below this are plain bytes */
    M_NO_SPACE = 1,      /* markers of the folded text */
    M_ALL_UPPER = 2,
    M_FIRST_UPPER = 3,
    M_ESCAPE = 4,
    LOG_FRAC = 10,
    LOG_ONE = 1 << LOG_FRAC,
    ROUND_WORDS = 100,   /* new words per round at most */
    KEY_BYTES = 512,     /* bytes of a word that take part in the final ordering */
    SYMBOL_LIMIT = 0xffff
};
#define COST_PER_WORD ((int64_t)(7.0 * LOG_ONE + 0.5))  /* bits (x 1024) a new dictionary entry costs */
#define COST_PER_USE ((int64_t)(1.3 * LOG_ONE + 0.5))   /* bits (x 1024) charged per use of the new word */

/* ------------------------------------------------------------------ small containers */

typedef struct {
    uint16_t *v;
    size_t n, cap;
} symvec;

static int sv_push(symvec *s, uint16_t c)
{
    if (s->n == s->cap) {
        size_t cap = s->cap ? s->cap + s->cap / 2 : 1024;
        uint16_t *v = realloc(s->v, cap * sizeof(*v));
        if (!v)
            return -1;
        s->v = v;
        s->cap = cap;
    }
    s->v[s->n++] = c;
    return 0;
}

typedef struct {
    uint8_t *v;
    size_t n, cap;
} bytevec;

static int bv_push(bytevec *s, uint8_t c)
{
    if (s->n == s->cap) {
        size_t cap = s->cap ? s->cap + s->cap / 2 : 1024;
        uint8_t *v = realloc(s->v, cap);
        if (!v)
            return -1;
        s->v = v;
        s->cap = cap;
    }
    s->v[s->n++] = c;
    return 0;
}

/* pairs of symbols in order of first insertion, found again through an open-addressing index */
typedef struct {
    uint16_t *a, *b;
    uint32_t *freq;
    size_t n, cap;
    uint64_t *slot; /* the pair in the high half, index + 1 in the low half; 0 = free */
    size_t n_slots; /* power of two */
} pairtab;

static inline uint64_t slot_entry(uint16_t a, uint16_t b, size_t index)
{
    return (uint64_t)((uint32_t)a << 16 | b) << 32 | (uint32_t)(index + 1);
}

static size_t pair_hash(uint16_t a, uint16_t b, size_t n_slots)
{
    uint32_t k = ((uint32_t)a << 16 | b) * 0x9E3779B1u;
    k ^= k >> 15;
    return (size_t)k & (n_slots - 1);
}

static void pt_free(pairtab *t)
{
    free(t->a);
    free(t->b);
    free(t->freq);
    free(t->slot);
    memset(t, 0, sizeof(*t));
}

static int pt_rehash(pairtab *t, size_t n_slots)
{
    uint64_t *slot = calloc(n_slots, sizeof(*slot));
    if (!slot)
        return -1;
    free(t->slot);
    t->slot = slot;
    t->n_slots = n_slots;
    for (size_t i = 0; i < t->n; i++) {
        size_t h = pair_hash(t->a[i], t->b[i], n_slots);
        while (slot[h])
            h = (h + 1) & (n_slots - 1);
        slot[h] = slot_entry(t->a[i], t->b[i], i);
    }
    return 0;
}

static long pt_find(const pairtab *t, uint16_t a, uint16_t b)
{
    if (!t->n_slots)
        return -1;
    size_t h = pair_hash(a, b, t->n_slots);
    const uint32_t key = (uint32_t)a << 16 | b;
    uint64_t e;
    while ((e = t->slot[h]) != 0) {
        if ((uint32_t)(e >> 32) == key)
            return (long)((uint32_t)e - 1);
        h = (h + 1) & (t->n_slots - 1);
    }
    return -1;
}

/* index of the pair, appended with frequency 0 when new; -1: out of memory */
static long pt_get(pairtab *t, uint16_t a, uint16_t b)
{
    long i = pt_find(t, a, b);
    if (i >= 0)
        return i;
    if (t->n == t->cap) {
        size_t cap = t->cap ? t->cap * 2 : 1024;
        uint16_t *na = realloc(t->a, cap * sizeof(*na));
        if (na)
            t->a = na;
        uint16_t *nb = realloc(t->b, cap * sizeof(*nb));
        if (nb)
            t->b = nb;
        uint32_t *nf = realloc(t->freq, cap * sizeof(*nf));
        if (nf)
            t->freq = nf;
        if (!na || !nb || !nf)
            return -1;
        t->cap = cap;
    }
    if ((t->n + 1) * 2 > t->n_slots && pt_rehash(t, t->n_slots ? t->n_slots * 2 : 4096))
        return -1;
    i = (long)t->n++;
    t->a[i] = a;
    t->b[i] = b;
    t->freq[i] = 0;
    size_t h = pair_hash(a, b, t->n_slots);
    while (t->slot[h])
        h = (h + 1) & (t->n_slots - 1);
    t->slot[h] = slot_entry(a, b, (size_t)i);
    return i;
}

/* stable merge sort of 32-bit items; before(x, y, ctx) != 0 when x must come strictly first */
typedef int (*before_fn)(uint32_t x, uint32_t y, const void *ctx);

static int stable_sort(uint32_t *v, size_t n, before_fn before, const void *ctx)
{
    if (n < 2)
        return 0;
    uint32_t *tmp = malloc(n * sizeof(*tmp)), *src = v, *dst = tmp;
    if (!tmp)
        return -1;
    for (size_t w = 1; w < n; w *= 2) {
        for (size_t lo = 0; lo < n; lo += 2 * w) {
            const size_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            size_t i = lo, j = mid, k = lo;
            while (i < mid && j < hi)
                dst[k++] = before(src[j], src[i], ctx) ? src[j++] : src[i++]; /* ties: the left run first */
            while (i < mid)
                dst[k++] = src[i++];
            while (j < hi)
                dst[k++] = src[j++];
        }
        uint32_t *t = src;
        src = dst;
        dst = t;
    }
    if (src != v)
        memcpy(v, src, n * sizeof(*v));
    free(tmp);
    return 0;
}

/* ------------------------------------------------------------------ case / space folding */

enum { K_OTHER, K_LOWER, K_UPPER };

static int letter_kind(unsigned c)
{
    if ((c >= 'a' && c <= 'z') || c >= 128)
        return K_LOWER; /* bytes of multi-byte characters count as lower-case letters */
    if (c >= 'A' && c <= 'Z')
        return K_UPPER;
    return K_OTHER;
}

static int fold_case_space(const uint8_t *in, size_t n, symvec *out)
{
    size_t i = 0;
    int bad = 0;
    while (i < n && !bad) {
        const int kind = letter_kind(in[i]);
        if (kind == K_OTHER) {
            if (in[i] >= M_NO_SPACE && in[i] <= M_ESCAPE)
                bad |= sv_push(out, M_ESCAPE);
            bad |= sv_push(out, in[i++]);
            continue;
        }
        size_t end = i + 1;
        int marker = 0;
        if (kind == K_LOWER) {
            while (end < n && letter_kind(in[end]) == K_LOWER)
                end++;
        } else if (end < n && letter_kind(in[end]) == K_UPPER) {
            marker = M_ALL_UPPER;
            while (end < n && letter_kind(in[end]) == K_UPPER)
                end++;
        } else {
            marker = M_FIRST_UPPER;
            while (end < n && letter_kind(in[end]) == K_LOWER)
                end++;
        }
        if (out->n && out->v[out->n - 1] == ' ')
            out->n--; /* the space in front of the word lives in the marker below */
        else
            bad |= sv_push(out, M_NO_SPACE);
        if (marker)
            bad |= sv_push(out, (uint16_t)marker);
        bad |= sv_push(out, ' ');
        for (; i < end; i++)
            bad |= sv_push(out, (uint16_t)(letter_kind(in[i]) == K_UPPER ? in[i] - 'A' + 'a' : in[i]));
    }
    return bad ? NCH_ERR_NOMEM : NCH_OK;
}

typedef struct {
    int pending_space; /* the next ' ' marker stands for a real space */
    int next_case, word_case, escaped;
} unfold_state;

/* the byte to write for folded symbol c, or -1 */
static int unfold_case_space(unfold_state *s, int c)
{
    if (s->escaped) {
        s->escaped = 0;
        return c;
    }
    switch (c) {
    case M_ALL_UPPER:
    case M_FIRST_UPPER:
        s->next_case = c;
        return -1;
    case M_NO_SPACE:
        s->pending_space = 0;
        return -1;
    case M_ESCAPE:
        s->escaped = 1;
        return -1;
    case ' ': {
        const int emit = s->pending_space;
        s->word_case = s->next_case;
        s->next_case = 0;
        s->pending_space = 1;
        return emit ? ' ' : -1;
    }
    default:
        if (s->word_case) {
            if (c >= 'a' && c <= 'z')
                c = c - 'a' + 'A';
            if (s->word_case == M_FIRST_UPPER)
                s->word_case = 0;
        }
        s->pending_space = 1;
        return c;
    }
}

/* ------------------------------------------------------------------ fixed-point log2 */

static uint16_t g_log_tab[LOG_ONE];
static int g_log_ready;

static void log_tab_init(void)
{
    if (g_log_ready)
        return;
    for (int i = 0; i < LOG_ONE; i++)
        g_log_tab[i] = (uint16_t)lrint(log2(1.0 + (double)i / LOG_ONE) * LOG_ONE);
    g_log_ready = 1;
}

/* log2(n) * 1024 from the top 11 bits of n; 0 for n = 0 */
static int fixed_log2(uint32_t n)
{
    if (n == 0)
        return 0;
    const int lz = __builtin_clz(n);
    const uint32_t top = (n << lz) >> (31 - LOG_FRAC);
    return g_log_tab[top - LOG_ONE] + ((31 - lz) << LOG_FRAC);
}

/* ------------------------------------------------------------------ dictionary building */

typedef struct {
    pairtab words;             /* word k is symbol N_BYTES + k; freq 0: not in use */
    pairtab pairs;             /* every pair of neighbours the buffer has held, with its count in the buffer now
                                  (kept up to date by each rewrite of the buffer; entries that fell to 0 stay) */
    uint32_t byte_freq[N_BYTES];
    symvec buf;
} builder;

/* bits (x 1024) one occurrence of symbol c costs now; a word not in use costs its two halves */
static int64_t symbol_bits(const builder *b, uint32_t c, uint32_t total)
{
    if (c < N_BYTES)
        return -(int64_t)(fixed_log2(b->byte_freq[c]) - fixed_log2(total));
    const size_t k = c - N_BYTES;
    if (b->words.freq[k] == 0)
        return symbol_bits(b, b->words.a[k], total) + symbol_bits(b, b->words.b[k], total);
    return -(int64_t)(fixed_log2(b->words.freq[k]) - fixed_log2(total));
}

static void count_symbols(builder *b)
{
    memset(b->byte_freq, 0, sizeof(b->byte_freq));
    for (size_t k = 0; k < b->words.n; k++)
        b->words.freq[k] = 0;
    for (size_t i = 0; i < b->buf.n; i++) {
        const uint32_t c = b->buf.v[i];
        if (c < N_BYTES)
            b->byte_freq[c]++;
        else
            b->words.freq[c - N_BYTES]++;
    }
}

/* Counts the adjacent pairs of v[0..n) into t (once, for the folded text; from then on the counts
   follow the rewrites). */
static int count_pairs(const uint16_t *v, size_t n, pairtab *t)
{
    for (size_t i = 0; i + 1 < n; i++) {
        const long k = pt_get(t, v[i], v[i + 1]);
        if (k < 0)
            return -1;
        t->freq[k]++;
    }
    return 0;
}

/* A rewrite of the buffer goes through it once, left to right, in steps: some old symbols become
   some new symbols.  The pair counts change only around the steps that change something: the pair
   across the boundary to the previous step, and the pairs inside the step. */
typedef struct {
    builder *b;
    int have_prev, prev_changed, bad;
    uint16_t prev_old, prev_new; /* last symbol of the previous step, before and after */
} rewrite;

static void pair_gone(builder *b, uint16_t x, uint16_t y)
{
    const long k = pt_find(&b->pairs, x, y);
    if (k >= 0 && b->pairs.freq[k])
        b->pairs.freq[k]--;
}

static int pair_new(builder *b, uint16_t x, uint16_t y)
{
    const long k = pt_get(&b->pairs, x, y);
    if (k < 0)
        return -1;
    b->pairs.freq[k]++;
    return 0;
}

static void rewrite_step(rewrite *r, const uint16_t *old, int n_old, const uint16_t *now, int n_now, int changed)
{
    builder *b = r->b;
    if (r->have_prev && (changed || r->prev_changed)) {
        pair_gone(b, r->prev_old, old[0]);
        r->bad |= pair_new(b, r->prev_new, now[0]);
    }
    if (changed) {
        for (int t = 0; t + 1 < n_old; t++)
            pair_gone(b, old[t], old[t + 1]);
        for (int t = 0; t + 1 < n_now; t++)
            r->bad |= pair_new(b, now[t], now[t + 1]);
    }
    r->prev_old = old[n_old - 1];
    r->prev_new = now[n_now - 1];
    r->prev_changed = changed;
    r->have_prev = 1;
}

/* a symbol that stays as it is: nothing to do unless the step before changed something */
static inline void rewrite_keep(rewrite *r, uint16_t c)
{
    if (r->prev_changed) {
        rewrite_step(r, &c, 1, &c, 1, 0);
    } else {
        r->prev_old = r->prev_new = c;
        r->have_prev = 1;
    }
}

/* writes symbol c of an expansion, words out of use as their halves, counting what it writes */
static int emit_counted(builder *b, uint32_t c, symvec *out)
{
    if (c >= N_BYTES) {
        const size_t k = c - N_BYTES;
        if (b->words.freq[k] == 0)
            return emit_counted(b, b->words.a[k], out) | emit_counted(b, b->words.b[k], out);
        b->words.freq[k]++;
    } else {
        b->byte_freq[c]++;
    }
    return sv_push(out, (uint16_t)c);
}

/* With the symbol counts of the buffer at hand (every rewrite keeps them): words seen fewer
   than min_freq times go out of use and the buffer is rewritten without them, the symbol and pair
   counts following.  Returns the number of words that passed the threshold, or -1. */
static long prune_rare_words(builder *b, uint32_t min_freq)
{
    size_t kept = 0, to_expand = 0;
    for (size_t k = 0; k < b->words.n; k++) {
        if (b->words.freq[k] >= min_freq) {
            kept++;
        } else {
            to_expand += b->words.freq[k] != 0;
            b->words.freq[k] = 0;
        }
    }
    if (to_expand == 0)
        return (long)kept; /* no word of the buffer fell out of use: rewriting it would change nothing */
    symvec out = {0};
    out.cap = b->buf.n + b->buf.n / 8 + 16;
    out.v = malloc(out.cap * sizeof(*out.v));
    if (!out.v)
        return -1;
    rewrite rw = {b, 0, 0, 0, 0, 0};
    int bad = 0;
    const uint16_t *v = b->buf.v;
    const size_t n = b->buf.n;
    for (size_t i = 0; i < n && !bad;) {
        size_t e = i; /* the stretch of symbols that stay moves as it is */
        while (e < n && !(v[e] >= N_BYTES && b->words.freq[v[e] - N_BYTES] == 0))
            e++;
        if (e > i) {
            rewrite_keep(&rw, v[i]);
            rw.prev_old = rw.prev_new = v[e - 1];
            if (out.n + (e - i) > out.cap) {
                const size_t cap = out.n + (e - i) + (n - e) + (n - e) / 8 + 16;
                uint16_t *grown = realloc(out.v, cap * sizeof(*grown));
                if (!grown) {
                    bad = 1;
                    break;
                }
                out.v = grown;
                out.cap = cap;
            }
            memcpy(out.v + out.n, v + i, (e - i) * sizeof(*v));
            out.n += e - i;
            i = e;
        }
        if (i < n) {
            const uint16_t c = v[i++];
            const size_t at = out.n;
            bad = emit_counted(b, b->words.a[c - N_BYTES], &out) | emit_counted(b, b->words.b[c - N_BYTES], &out);
            if (!bad)
                rewrite_step(&rw, &c, 1, out.v + at, (int)(out.n - at), 1);
        }
    }
    if (bad || rw.bad) {
        free(out.v);
        return -1;
    }
    free(b->buf.v);
    b->buf = out;
    return (long)kept;
}

static int score_before(uint32_t x, uint32_t y, const void *ctx)
{
    const int64_t *score = ctx;
    return score[x] > score[y];
}

static int place_before(uint32_t x, uint32_t y, const void *ctx)
{
    const uint32_t *first_at = ctx;
    return first_at[x] < first_at[y];
}

enum { NOT_TIED = 0xffffffffu, NOT_SEEN = 0xfffffffeu };

/* order[lo..hi) is sorted by falling score and holds whole groups of equal scores.  Candidates with
   equal scores have to come in the order in which their pairs first occur in the buffer (the
   reference lists its candidates in that order and sorts them stably): one pass over the buffer
   finds those places, for the tied candidates only, and stops when it has them all. */
static int order_ties(const builder *b, uint32_t *order, size_t lo, size_t hi, const int64_t *score)
{
    const pairtab *p = &b->pairs;
    size_t tied = 0;
    for (size_t r = lo; r + 1 < hi; r++)
        tied += score[order[r]] == score[order[r + 1]];
    if (!tied)
        return 0;
    const size_t n_sym = N_BYTES + b->words.n;
    uint32_t *first_at = malloc((p->n + 1) * sizeof(*first_at));
    uint8_t *side = calloc(n_sym, 1);
    if (!first_at || !side) {
        free(first_at);
        free(side);
        return -1;
    }
    memset(first_at, 0xff, (p->n + 1) * sizeof(*first_at)); /* NOT_TIED */
    size_t waiting = 0;
    for (size_t r = lo; r < hi; r++) {
        const int with_prev = r > lo && score[order[r]] == score[order[r - 1]];
        const int with_next = r + 1 < hi && score[order[r]] == score[order[r + 1]];
        if (with_prev || with_next) {
            const uint32_t k = order[r];
            first_at[k] = NOT_SEEN;
            side[p->a[k]] |= 1;
            side[p->b[k]] |= 2;
            waiting++;
        }
    }
    const uint16_t *v = b->buf.v;
    for (size_t i = 0; i + 1 < b->buf.n && waiting; i++) {
        if (!(side[v[i]] & 1) || !(side[v[i + 1]] & 2))
            continue;
        const long k = pt_find(p, v[i], v[i + 1]);
        if (k >= 0 && first_at[k] == NOT_SEEN) {
            first_at[k] = (uint32_t)i;
            waiting--;
        }
    }
    int bad = 0;
    for (size_t r = lo; r < hi && !bad;) {
        size_t e = r + 1;
        while (e < hi && score[order[e]] == score[order[r]])
            e++;
        if (e - r > 1)
            bad = stable_sort(order + r, e - r, place_before, first_at);
        r = e;
    }
    free(first_at);
    free(side);
    return bad;
}

/* one round: adds up to `limit` new words to b->words.  Returns how many, or -1. */
static long pick_words(builder *b, long limit, uint32_t min_freq)
{
    const pairtab *cand = &b->pairs;
    int64_t *score = NULL;
    uint32_t *order = NULL;
    uint8_t *opens = NULL, *closes = NULL;
    long added = -1;
    const uint32_t total = (uint32_t)b->buf.n;

    score = malloc((cand->n + 1) * sizeof(*score));
    order = malloc((cand->n + 1) * sizeof(*order));
    const size_t n_sym = N_BYTES + b->words.n;
    opens = calloc(n_sym, 1);
    closes = calloc(n_sym, 1);
    if (!score || !order || !opens || !closes)
        goto done;
    /* the selection below stops at the first score that is not positive, so only the candidates
       with a positive score need sorting */
    size_t n_pos = 0;
    for (size_t k = 0; k < cand->n; k++) {
        const int64_t f = cand->freq[k];
        if (f <= 1)
            continue; /* a pair seen once (or no longer) saves nothing */
        const int64_t as_two = (symbol_bits(b, cand->a[k], total) + symbol_bits(b, cand->b[k], total)) * f;
        const int64_t as_one = (-(int64_t)(fixed_log2((uint32_t)f) - fixed_log2(total)) + COST_PER_USE) * f + COST_PER_WORD;
        score[k] = as_two - as_one;
        if (score[k] > 0)
            order[n_pos++] = (uint32_t)k;
    }
    if (stable_sort(order, n_pos, score_before, score))
        goto done;
    added = 0;
    size_t settled = 0; /* order[0..settled) has its ties in place; the selection rarely goes far */
    for (size_t r = 0; r < n_pos; r++) {
        if (r >= settled) {
            size_t hi = settled ? 2 * settled : 256;
            hi = hi < n_pos ? hi : n_pos;
            while (hi < n_pos && score[order[hi]] == score[order[hi - 1]])
                hi++; /* whole groups only */
            if (order_ties(b, order, settled, hi, score)) {
                added = -1;
                goto done;
            }
            settled = hi;
        }
        const size_t k = order[r];
        if (cand->freq[k] < min_freq)
            break;
        const uint16_t a = cand->a[k], c = cand->b[k];
        if (closes[a] || opens[c])
            continue; /* would chain with a word already taken this round */
        opens[a] = 1;
        closes[c] = 1;
        if (pt_find(&b->words, a, c) < 0 && N_BYTES + b->words.n + 1 >= SYMBOL_LIMIT) {
            added = -2; /* more words than 16-bit symbols */
            goto done;
        }
        if (pt_get(&b->words, a, c) < 0) {
            added = -1;
            goto done;
        }
        if (++added >= limit)
            break;
    }
done:
    free(score);
    free(order);
    free(opens);
    free(closes);
    return added;
}

/* every pair of the buffer that is a word (in use or not) becomes that word, greedily from the
   left; the symbol and pair counts follow */
static int substitute_words(builder *b)
{
    uint16_t *v = b->buf.v;
    size_t n = b->buf.n, i = 0, j = 0;
    /* only a word whose pair occurs in the buffer can match, and most positions start none: the
       table is asked only where the two symbols can be the halves of such a word */
    const size_t n_sym = N_BYTES + b->words.n;
    uint8_t *half = calloc(n_sym, 1);
    if (!half)
        return -1;
    size_t active = 0;
    for (size_t k = 0; k < b->words.n; k++) {
        const long at = pt_find(&b->pairs, b->words.a[k], b->words.b[k]);
        if (at >= 0 && b->pairs.freq[at]) {
            half[b->words.a[k]] |= 1;
            half[b->words.b[k]] |= 2;
            active++;
        }
    }
    if (!active) {
        free(half);
        return 0;
    }
    rewrite rw = {b, 0, 0, 0, 0, 0};
    while (i < n) {
        /* the stretch up to the next place where a word can start moves as it is */
        size_t e = i;
        while (e + 1 < n && !((half[v[e]] & 1) && (half[v[e + 1]] & 2)))
            e++;
        long k = e + 1 < n ? pt_find(&b->words, v[e], v[e + 1]) : -1;
        if (k < 0)
            e++; /* v[e] starts no word either (or is the last symbol) */
        if (e > i) {
            rewrite_keep(&rw, v[i]);
            rw.prev_old = rw.prev_new = v[e - 1];
            if (j != i)
                memmove(v + j, v + i, (e - i) * sizeof(*v));
            j += e - i;
            i = e;
        }
        if (k >= 0) {
            const uint16_t w = (uint16_t)(N_BYTES + k);
            rewrite_step(&rw, v + i, 2, &w, 1, 1); /* v[i], v[i + 1] are still the old symbols: j <= i */
            for (int t = 0; t < 2; t++) {
                if (v[i + t] < N_BYTES)
                    b->byte_freq[v[i + t]]--;
                else
                    b->words.freq[v[i + t] - N_BYTES]--;
            }
            b->words.freq[k]++;
            v[j++] = w;
            i += 2;
        }
    }
    b->buf.n = j;
    free(half);
    return rw.bad ? -1 : 0;
}

/* the first `room` bytes of symbol c; returns how many were written */
static int word_prefix(const pairtab *w, uint32_t c, uint8_t *out, int room)
{
    if (c < N_BYTES) {
        if (room < 1)
            return 0;
        out[0] = (uint8_t)c;
        return 1;
    }
    int n = word_prefix(w, w->a[c - N_BYTES], out, room);
    return n + word_prefix(w, w->b[c - N_BYTES], out + n, room - n);
}

typedef struct {
    const uint8_t *keys; /* [n_words][KEY_BYTES] */
    const uint16_t *len;
} key_ctx;

static int key_before(uint32_t x, uint32_t y, const void *ctx)
{
    const key_ctx *k = ctx;
    const size_t i = x - N_BYTES, j = y - N_BYTES;
    const int m = k->len[i] < k->len[j] ? k->len[i] : k->len[j];
    const int r = memcmp(k->keys + i * KEY_BYTES, k->keys + j * KEY_BYTES, (size_t)m);
    return r ? r < 0 : k->len[i] < k->len[j];
}

static int write_entry(const pairtab *w, uint32_t c, bytevec *out)
{
    if (c >= N_BYTES)
        return write_entry(w, w->a[c - N_BYTES], out) | write_entry(w, w->b[c - N_BYTES], out);
    if (c == '\n')
        return bv_push(out, '\\') | bv_push(out, 'n');
    if (c == '\\')
        return bv_push(out, '\\') | bv_push(out, '\\');
    return bv_push(out, (uint8_t)c);
}

static int emit_final(const builder *b, const uint32_t *new_id, uint32_t c, symvec *out)
{
    if (c >= N_BYTES && b->words.freq[c - N_BYTES] == 0)
        return emit_final(b, new_id, b->words.a[c - N_BYTES], out) | emit_final(b, new_id, b->words.b[c - N_BYTES], out);
    return sv_push(out, (uint16_t)new_id[c]);
}

enum { SEEN_MAX = 64, STALL_MAX = 4096 };

static uint64_t buffer_hash(const symvec *s)
{
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < s->n; i++)
        h = (h ^ s->v[i]) * 0x100000001b3ull;
    return h;
}

int nch_words_encode(const uint8_t *text, size_t n, int n_words, int min_word_freq, uint8_t **dict,
                     size_t *dict_len, uint16_t **symbols, size_t *n_symbols, int *n_entries)
{
    if ((!text && n) || !dict || !dict_len || !symbols || !n_symbols || n_words > SYMBOL_LIMIT || n > ((size_t)1 << 30))
        return NCH_ERR_INVALID; /* positions and counts are 32-bit, as in the reference */
    log_tab_init();
    builder b;
    memset(&b, 0, sizeof(b));
    uint32_t *order = NULL, *new_id = NULL;
    uint8_t *keys = NULL;
    uint16_t *key_len = NULL;
    bytevec text_out = {0};
    symvec sym_out = {0};
    const uint32_t min_freq = (uint32_t)min_word_freq; /* compared unsigned, as preprocess.c:900 does */
    int rc = fold_case_space(text, n, &b.buf);
    if (rc)
        goto done;
    count_symbols(&b);
    if (count_pairs(b.buf.v, b.buf.n, &b.pairs)) {
        rc = NCH_ERR_NOMEM;
        goto done;
    }

    /* Rounds that add no new entry to the word table can fall into a cycle (a word goes out of use,
       the next round takes it again, the one after drops it ...): the reference never returns from
       such an input.  The state of a round is the buffer and the count in use; the same state twice
       while the table stood still proves the cycle, and the loop ends there (as it does after
       STALL_MAX rounds without a new entry, should a cycle be longer than the states kept). */
    uint64_t seen[SEEN_MAX][3];
    long stalled = 0; /* rounds since the table last grew */
    size_t table_size = 0;
    const long target = (long)n_words - N_BYTES;
    for (long in_use = 0; in_use < target && b.buf.n >= 2;) {
        if (b.words.n != table_size) {
            table_size = b.words.n;
            stalled = 0;
        }
        const uint64_t state[3] = {buffer_hash(&b.buf), b.buf.n, (uint64_t)in_use};
        int cycle = 0;
        for (long i = 0; i < stalled && i < SEEN_MAX; i++)
            cycle |= seen[i][0] == state[0] && seen[i][1] == state[1] && seen[i][2] == state[2];
        if (cycle || stalled >= STALL_MAX)
            break;
        memcpy(seen[stalled++ % SEEN_MAX], state, sizeof(state));
        const long room = target - in_use;
        const long added = pick_words(&b, room < ROUND_WORDS ? room : ROUND_WORDS, min_freq);
        if (added < 0) {
            rc = added == -2 ? NCH_ERR_INVALID : NCH_ERR_NOMEM;
            goto done;
        }
        if (added == 0)
            break;
        if (substitute_words(&b)) {
            rc = NCH_ERR_NOMEM;
            goto done;
        }
        const long before = in_use;
        in_use = prune_rare_words(&b, min_freq);
        if (in_use < 0) {
            rc = NCH_ERR_NOMEM;
            goto done;
        }
        if (in_use == before)
            break;
    }

    /* final numbering: the bytes, then the words in use ordered by their first KEY_BYTES bytes */
    const size_t n_all = N_BYTES + b.words.n;
    order = malloc(n_all * sizeof(*order));
    new_id = malloc(n_all * sizeof(*new_id));
    keys = malloc((b.words.n + 1) * (size_t)KEY_BYTES);
    key_len = malloc((b.words.n + 1) * sizeof(*key_len));
    if (!order || !new_id || !keys || !key_len) {
        rc = NCH_ERR_NOMEM;
        goto done;
    }
    size_t n_out = 0;
    for (size_t c = 0; c < n_all; c++) {
        if (c >= N_BYTES) {
            if (b.words.freq[c - N_BYTES] == 0)
                continue;
            key_len[c - N_BYTES] = (uint16_t)word_prefix(&b.words, (uint32_t)c, keys + (c - N_BYTES) * KEY_BYTES, KEY_BYTES);
        }
        order[n_out++] = (uint32_t)c;
    }
    const key_ctx kc = {keys, key_len};
    if (stable_sort(order + N_BYTES, n_out - N_BYTES, key_before, &kc)) {
        rc = NCH_ERR_NOMEM;
        goto done;
    }
    int bad = 0;
    for (size_t i = 0; i < n_all; i++)
        new_id[i] = 0;
    for (size_t i = 0; i < n_out && !bad; i++) {
        new_id[order[i]] = (uint32_t)i;
        bad = write_entry(&b.words, order[i], &text_out) | bv_push(&text_out, '\n');
    }
    for (size_t i = 0; i < b.buf.n && !bad; i++)
        bad = emit_final(&b, new_id, b.buf.v[i], &sym_out);
    if (bad) {
        rc = NCH_ERR_NOMEM;
        goto done;
    }
    *dict = text_out.v;
    *dict_len = text_out.n;
    *symbols = sym_out.v;
    *n_symbols = sym_out.n;
    if (n_entries)
        *n_entries = (int)n_out;
    text_out.v = NULL;
    sym_out.v = NULL;
done:
    free(order);
    free(new_id);
    free(keys);
    free(key_len);
    free(text_out.v);
    free(sym_out.v);
    free(b.buf.v);
    pt_free(&b.words);
    pt_free(&b.pairs);
    return rc;
}

/* ------------------------------------------------------------------ decoding */

typedef struct {
    uint8_t *bytes;
    size_t *start; /* [n + 1] */
    size_t n;
} wordlist;

static void wl_free(wordlist *w)
{
    free(w->bytes);
    free(w->start);
    memset(w, 0, sizeof(*w));
}

/* one entry per '\n'-terminated line; "\\n" and "\\\\" are the only escapes; empty lines and an
   unterminated last line are dropped (preprocess.c:1227-1268).  The reference refuses an entry above
   4096 bytes although its encoder can make one (a long passage repeated); here any length decodes. */
static int wl_parse(const uint8_t *dict, size_t dict_len, wordlist *w)
{
    memset(w, 0, sizeof(*w));
    size_t lines = 0;
    for (size_t i = 0; i < dict_len; i++)
        lines += dict[i] == '\n';
    w->bytes = malloc(dict_len + 1);
    w->start = malloc((lines + 1) * sizeof(*w->start));
    if (!w->bytes || !w->start) {
        wl_free(w);
        return NCH_ERR_NOMEM;
    }
    size_t pos = 0, line_start = 0;
    w->start[0] = 0;
    for (size_t i = 0; i < dict_len; i++) {
        unsigned c = dict[i];
        if (c == '\n') {
            if (pos > line_start)
                w->start[++w->n] = pos;
            line_start = pos;
            continue;
        }
        if (c == '\\') {
            if (++i >= dict_len)
                break;
            c = dict[i];
            if (c == 'n')
                c = '\n';
            else if (c != '\\')
                goto bad;
        }
        w->bytes[pos++] = (uint8_t)c;
    }
    return NCH_OK;
bad:
    wl_free(w);
    return NCH_ERR_FORMAT;
}

int nch_words_count(const uint8_t *dict, size_t dict_len)
{
    wordlist w;
    if (!dict && dict_len)
        return -NCH_ERR_INVALID;
    const int rc = wl_parse(dict, dict_len, &w);
    if (rc)
        return -rc;
    const int n = (int)w.n;
    wl_free(&w);
    return n;
}

int nch_words_decode(const uint8_t *dict, size_t dict_len, const uint16_t *symbols, size_t n_symbols,
                     uint8_t **text, size_t *text_len)
{
    if ((!dict && dict_len) || (!symbols && n_symbols) || !text || !text_len)
        return NCH_ERR_INVALID;
    wordlist w;
    int rc = wl_parse(dict, dict_len, &w);
    if (rc)
        return rc;
    bytevec out = {0};
    unfold_state st = {1, 0, 0, 0};
    int bad = 0;
    for (size_t i = 0; i < n_symbols && !bad; i++) {
        const size_t c = symbols[i];
        if (c >= w.n) {
            rc = NCH_ERR_FORMAT;
            break;
        }
        for (size_t k = w.start[c]; k < w.start[c + 1] && !bad; k++) {
            const int ch = unfold_case_space(&st, w.bytes[k]);
            if (ch >= 0)
                bad = bv_push(&out, (uint8_t)ch);
        }
    }
    wl_free(&w);
    if (bad)
        rc = NCH_ERR_NOMEM;
    if (rc) {
        free(out.v);
        return rc;
    }
    if (!out.v && !(out.v = malloc(1)))
        return NCH_ERR_NOMEM;
    *text = out.v;
    *text_len = out.n;
    return NCH_OK;
}
