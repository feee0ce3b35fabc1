/*
 * libnc_shim.c -- the handful of LibNC entry points NNCP's host flow uses outside the model
 * functions (context, devices, host tensors of ids and probabilities, allocation), on plain
 * host memory.  Prototypes come from the reference's libnc.h (libnc.h:117-227, 600); LibNC's own
 * implementation is not part of the reference tree.  The tensor-graph entry points that only the
 * replaced model functions call are in libnc_stubs.c.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "cutils.h"
#include "libnc.h"

struct NCContext { int nb_threads; };
struct NCDevice { int is_cuda; };
struct NCRNDState { uint32_t seed; };
struct NCTensor {
    NCTypeEnum type;
    int n_dims;
    size_t dims[4];
    size_t elt;
    void *data;
    int refs;
};

void *nc_malloc(size_t size) { void *p = malloc(size ? size : 1); if (!p) abort(); return p; }
void *nc_mallocz(size_t size) { void *p = calloc(1, size ? size : 1); if (!p) abort(); return p; }
void nc_free(void *ptr) { free(ptr); }

NCContext *nc_context_init(int nb_threads)
{
    NCContext *m = nc_mallocz(sizeof(*m));
    m->nb_threads = nb_threads;
    return m;
}
void nc_context_end(NCContext *m) { free(m); }
NCDevice *nc_new_cpu_device(NCContext *m) { (void)m; return nc_mallocz(sizeof(NCDevice)); }
NCDevice *nc_new_cuda_device(NCContext *m, int device_index)
{
    NCDevice *d = nc_mallocz(sizeof(NCDevice));
    (void)m; (void)device_index;
    d->is_cuda = 1;
    return d;
}
NCRNDState *nc_rnd_init(NCDevice *d, uint32_t seed)
{
    NCRNDState *s = nc_mallocz(sizeof(*s));
    (void)d;
    s->seed = seed;
    return s;
}
void nc_rnd_end(NCRNDState *s) { free(s); }
void nc_prof_dump(void) {}

static NCTensor *new_tensor(NCTypeEnum type, int n_dims, size_t n0, size_t n1, size_t n2)
{
    NCTensor *x = nc_mallocz(sizeof(*x));
    x->type = type;
    x->n_dims = n_dims;
    x->dims[0] = n0; x->dims[1] = n1; x->dims[2] = n2; x->dims[3] = 1;
    x->elt = (type == NC_TYPE_I8 || type == NC_TYPE_U8) ? 1 : (type == NC_TYPE_I16 || type == NC_TYPE_U16 ||
             type == NC_TYPE_BF16 || type == NC_TYPE_F16) ? 2 : 4;
    x->data = nc_mallocz(x->elt * n0 * n1 * n2);
    x->refs = 1;
    return x;
}
NCTensor *nc_new_tensor_2d(NCDevice *d, NCTypeEnum type, size_t n0, size_t n1)
{
    (void)d;
    return new_tensor(type, 2, n0, n1, 1);
}
NCTensor *nc_new_tensor_3d(NCDevice *d, NCTypeEnum type, size_t n0, size_t n1, size_t n2)
{
    (void)d;
    return new_tensor(type, 3, n0, n1, n2);
}
NCTensor *nc_dup_tensor(const NCTensor *x)
{
    ((NCTensor *)x)->refs++;
    return (NCTensor *)x;
}
void nc_free_tensor(NCTensor *x)
{
    if (x && --x->refs == 0) {
        free(x->data);
        free(x);
    }
}
/* dimension 0 is the contiguous one (libnc.h:183-185) */
void nc_set1_i32_2d(NCTensor *y, size_t i0, size_t i1, int32_t val)
{
    ((int32_t *)y->data)[i0 + i1 * y->dims[0]] = val;
}
NCTensor *nc_tensor_to_cpu_device(NCTensor *x) { return x; }
void *nc_tensor_get_ptr(const NCTensor *x, size_t *pstride)
{
    if (pstride)
        *pstride = x->dims[0];
    return x->data;
}

/* the coder's own halving recursion: every node's left-half sum is one node of a single
   bottom-up reduction tree, which is what the device computes for coder-ready output */
float vec_sum_f32(const float *tab, size_t n)
{
    if (n <= 1)
        return n ? tab[0] : 0.0f;
    size_t h = n >> 1;
    return vec_sum_f32(tab, h) + vec_sum_f32(tab + h, n - h);
}
