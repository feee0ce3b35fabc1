"""ctypes view of include/nncu.h: the parameter block and the entry-point prototypes."""
import ctypes as C

N_LAYER_MAX = 32
LN_POST, LN_PRE, LN_FINAL, LN_COEF, LN_RMSNORM = 1, 2, 4, 8, 16
FF_RELU, FF_GELU, FF_GEGLU, FF_GATED_SILU = 0, 1, 2, 3
INIT_UNIFORM, INIT_NORMAL = 0, 1
GEMM_AUTO, GEMM_SIMT, GEMM_TCGEN05 = 0, 1, 2
NOALLOC_SCRATCH_FLOATS = 4 << 20
OK, ERR_INVALID, ERR_CUDA, ERR_NOMEM, ERR_STATE, ERR_TIMEOUT, ERR_RANGE = range(7)


class Params(C.Structure):
    """struct nncu_params (include/nncu.h), field for field."""
    _fields_ = [
        ("n_layer", C.c_int32), ("d_model", C.c_int32), ("n_head", C.c_int32),
        ("d_key", C.c_int32), ("d_value", C.c_int32), ("d_inner", C.c_int32),
        ("d_pos", C.c_int32), ("mem_len", C.c_int32), ("seg_len", C.c_int32),
        ("n_streams", C.c_int32), ("n_streams_total", C.c_int32), ("n_symbols", C.c_int32),
        ("attn_len", C.c_int32 * N_LAYER_MAX),
        ("use_bias", C.c_uint8), ("use_w_r", C.c_uint8), ("tied_w_r", C.c_uint8),
        ("tied_b_r", C.c_uint8), ("query_bias", C.c_uint8), ("ln_flags", C.c_uint8),
        ("ff_act", C.c_uint8), ("use_bf16", C.c_uint8),
        ("embed_mult", C.c_float), ("init_range", C.c_float), ("init_kind", C.c_int32),
        ("seed", C.c_uint32),
        ("lr", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
        ("gradient_clip", C.c_float), ("bias_correction", C.c_int32),
        ("gemm_backend", C.c_int32), ("device", C.c_int32),
    ]

    def copy(self, **over):
        p = Params.from_buffer_copy(bytes(self))
        for k, v in over.items():
            setattr(p, k, v)
        return p


def make_params(**kw):
    """Params with the defaults of the reference's "default" profile sizes replaced by kw."""
    base = dict(n_layer=2, d_model=128, n_head=4, d_key=32, d_inner=512, d_pos=64, mem_len=32,
                seg_len=32, n_streams=4, n_streams_total=0, n_symbols=256, use_bias=1, use_w_r=1,
                tied_w_r=0, tied_b_r=0, query_bias=1, ln_flags=LN_POST, ff_act=FF_GELU,
                use_bf16=0, embed_mult=1.0, init_range=0.02, init_kind=INIT_NORMAL, seed=123,
                lr=3e-4, beta2=0.99, eps=1e-8, gradient_clip=0.0, bias_correction=0,
                gemm_backend=GEMM_AUTO, device=-1)
    attn_len = kw.pop("attn_len", None)
    base.update(kw)
    base.setdefault("d_value", base["d_key"])
    p = Params()
    for k, v in base.items():
        setattr(p, k, v)
    if attn_len is not None:
        for i, v in enumerate(attn_len[:N_LAYER_MAX]):
            p.attn_len[i] = int(v)
    return p


class AttnShape(C.Structure):
    """struct nncu_attn_shape (include/nncu.h)."""
    _fields_ = [
        ("n_streams", C.c_int32), ("n_head", C.c_int32), ("d_key", C.c_int32),
        ("seg_len", C.c_int32), ("mem_len", C.c_int32), ("d_pos", C.c_int32),
        ("attn_len", C.c_int32), ("t0", C.c_int32), ("t1", C.c_int32),
        ("br_scale", C.c_float), ("dtype_bf16", C.c_int32),
    ]


class Profile(C.Structure):
    """struct nncu_profile (include/nncu.h)."""
    _fields_ = [("launches", C.c_uint64), ("gemm_launches", C.c_uint64),
                ("gemm_ms", C.c_double), ("gemm_flops", C.c_double)]


_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_pi32, _pf = C.POINTER(C.c_int32), C.POINTER(C.c_float)

# name -> (restype, argtypes); every symbol include/nncu.h declares
PROTOTYPES = {
    "nncu_default_params": (None, [C.POINTER(Params)]),
    "nncu_abi_version": (_i, []),
    "nncu_last_error": (C.c_char_p, []),
    "nncu_create": (_i, [C.POINTER(Params), C.POINTER(_vp)]),
    "nncu_destroy": (_i, [_vp]),
    "nncu_set_stream": (_i, [_vp, _vp]),
    "nncu_reset": (_i, [_vp]),
    "nncu_set_lr": (_i, [_vp, C.c_float]),
    "nncu_eval": (_i, [_vp, _i, _vp]),
    "nncu_eval_dev": (_i, [_vp, _i, _vp]),
    "nncu_eval_end": (_i, [_vp]),
    "nncu_read_probs": (_i, [_vp, _i, _i, _vp]),
    "nncu_probs_dev": (_i, [_vp, C.POINTER(_vp)]),
    "nncu_eval_gradient": (_i, [_vp, _vp, _pf]),
    "nncu_eval_gradient_dev": (_i, [_vp, _vp]),
    "nncu_eval_gradient_update": (_i, [_vp, _vp, C.POINTER(C.c_float)]),
    "nncu_eval_gradient_update_dev": (_i, [_vp, _vp]),
    "nncu_read_loss": (_i, [_vp, _pf]),
    "nncu_update": (_i, [_vp]),
    "nncu_optimizer_step": (_i, [_vp]),
    "nncu_memory_shift": (_i, [_vp]),
    "nncu_synchronize": (_i, [_vp]),
    "nncu_selftest_expired_wait": (_i, [_vp]),
    "nncu_param_count": (_i, [_vp]),
    "nncu_param_info": (_i, [_vp, _i, C.c_char_p, _sz, C.POINTER(_sz), C.POINTER(_sz)]),
    "nncu_param_get": (_i, [_vp, _i, _vp, _sz]),
    "nncu_param_set": (_i, [_vp, _i, _vp, _sz]),
    "nncu_grad_get": (_i, [_vp, _i, _vp, _sz]),
    "nncu_flat_buffers": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                               C.POINTER(_sz)]),
    "nncu_comm_unique_id": (_i, [_vp]),
    "nncu_comm_init": (_i, [_vp, _i, _i, _vp]),
    "nncu_comm_gather_master": (_i, [_vp]),
    "nncu_weights_hash": (_i, [_vp, C.POINTER(C.c_uint64)]),
    "nncu_coder_paths": (_i, [_vp, _i, _i, _vp, _vp, C.POINTER(_i)]),
    "nncu_coder_paths_begin": (_i, [_vp, _i, _i, _vp]),
    "nncu_coder_paths_end": (_i, [_vp, _vp, C.POINTER(_i)]),
    "nncu_coder_trees": (_i, [_vp, _i, _i, _vp]),
    "nncu_decoder_begin": (_i, [_vp, _vp, C.c_size_t]),
    "nncu_decode_steps": (_i, [_vp, _i, _i, _vp, _i, _i, _vp]),
    "nncu_decoder_end": (_i, [_vp, C.POINTER(C.c_size_t)]),
    "nncu_attention_forward": (_i, [C.POINTER(AttnShape), _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "nncu_attention_backward": (_i, [C.POINTER(AttnShape)] + [_vp] * 12),
    "nncu_attention_backward_noalloc": (_i, [C.POINTER(AttnShape)] + [_vp] * 12),
    "nncu_attention_reduce_tables": (_i, [C.POINTER(AttnShape), _vp, _vp, _vp, _vp, _i, _vp]),
    "nncu_profile_begin": (_i, [_i]),
    "nncu_profile_end": (_i, [C.POINTER(Profile)]),
    "nncu_gemm_bf16": (_i, [_i, _i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp]),
    "nncu_gemm_bf16_nt": (_i, [_i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp]),
}


def bind(lib):
    """Attach restype/argtypes to a loaded libnncu; raises AttributeError on a missing symbol."""
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib
