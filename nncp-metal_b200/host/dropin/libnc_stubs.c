/*
 * libnc_stubs.c -- LibNC tensor-graph entry points that only the reference's own LibNC model
 * functions (trf_init ... trf_update, the LSTM class) reference.  With the Transformer class
 * re-pointed at the B200 library they are never reached; they exist so that the unmodified
 * nncp.c links, and abort loudly if a code path that needs LibNC itself is taken (for
 * example the LSTM profiles).  Declared without prototypes on purpose: only the names matter.
 */
#include <stdio.h>
#include <stdlib.h>

#define LIBNC_STUB(name)                                                              \
    void name(void)                                                                   \
    {                                                                                 \
        fprintf(stderr, "%s: LibNC is not part of this build (B200 backend)\n", #name); \
        abort();                                                                      \
    }

LIBNC_STUB(nc_add)
LIBNC_STUB(nc_backward)
LIBNC_STUB(nc_cmul)
LIBNC_STUB(nc_combine_nodes)
LIBNC_STUB(nc_concat)
LIBNC_STUB(nc_concat_node)
LIBNC_STUB(nc_concat_optimization)
LIBNC_STUB(nc_convert)
LIBNC_STUB(nc_dup_node)
LIBNC_STUB(nc_free_node)
LIBNC_STUB(nc_gated_swish)
LIBNC_STUB(nc_gelu)
LIBNC_STUB(nc_get_col)
LIBNC_STUB(nc_get_node)
LIBNC_STUB(nc_get_param_count)
LIBNC_STUB(nc_get_scalar_f32)
LIBNC_STUB(nc_get_tensor_device)
LIBNC_STUB(nc_hconcat)
LIBNC_STUB(nc_indexed_log)
LIBNC_STUB(nc_layer_norm)
LIBNC_STUB(nc_lerp)
LIBNC_STUB(nc_lstm_clamped)
LIBNC_STUB(nc_masked_fill)
LIBNC_STUB(nc_matmul)
LIBNC_STUB(nc_matmul_add)
LIBNC_STUB(nc_mul)
LIBNC_STUB(nc_new_f32)
LIBNC_STUB(nc_new_param)
LIBNC_STUB(nc_new_scalar)
LIBNC_STUB(nc_new_tensor_1d)
LIBNC_STUB(nc_new_tensor_4d)
LIBNC_STUB(nc_new_tensor_from_tensor_nz)
LIBNC_STUB(nc_node_set_arg)
LIBNC_STUB(nc_node_set_parent)
LIBNC_STUB(nc_pad)
LIBNC_STUB(nc_param_list_end)
LIBNC_STUB(nc_param_list_init)
LIBNC_STUB(nc_permute)
LIBNC_STUB(nc_permute_4d)
LIBNC_STUB(nc_reduce_sum)
LIBNC_STUB(nc_rel_shift)
LIBNC_STUB(nc_relu)
LIBNC_STUB(nc_repeat_1d)
LIBNC_STUB(nc_repeat_2d)
LIBNC_STUB(nc_reshape_1d)
LIBNC_STUB(nc_reshape_2d)
LIBNC_STUB(nc_reshape_3d)
LIBNC_STUB(nc_reshape_4d)
LIBNC_STUB(nc_rms_norm)
LIBNC_STUB(nc_sgd_opt_end)
LIBNC_STUB(nc_sgd_opt_init)
LIBNC_STUB(nc_sgd_opt_set_all)
LIBNC_STUB(nc_sgd_opt_set_lr)
LIBNC_STUB(nc_sgd_opt_update)
LIBNC_STUB(nc_sigmoid)
LIBNC_STUB(nc_slice)
LIBNC_STUB(nc_slice_alias)
LIBNC_STUB(nc_soft_max)
LIBNC_STUB(nc_split)
LIBNC_STUB(nc_sum)
LIBNC_STUB(nc_tanh)
LIBNC_STUB(nc_tensor_copy)
LIBNC_STUB(nc_tensor_copy_slice)
LIBNC_STUB(nc_tensor_get_dims)
LIBNC_STUB(nc_tensor_set_dropout)
LIBNC_STUB(nc_tensor_set_f32)
LIBNC_STUB(nc_tensor_set_name)
LIBNC_STUB(nc_tensor_set_rnd_unif)
LIBNC_STUB(nc_tensor_set_zero)
LIBNC_STUB(nc_tensor_to_device)
LIBNC_STUB(nc_vconcat)
LIBNC_STUB(sgd_opt_update_var)
