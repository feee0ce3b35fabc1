"""ctypes view of include/nncp_host.h (libnncp_host.so): coder, stream layout, schedule,
container header and the block loop, with the CUDA model bound through nch_bind_cuda."""
import ctypes as C
import os

import numpy as np

from . import abi
from .loader import HOSTLIB, LIB, LibraryMissing

INTERP_MAX_STEPS = 8
EVAL_STEP, EVAL_SEGMENT = 0, 1
OUT_FLOAT, OUT_CODER_READY, OUT_DEVICE = 0, 1, 2
_vp = C.c_void_p


class InterpParams(C.Structure):
    _fields_ = [("n_steps", C.c_int32), ("val", C.c_float * (INTERP_MAX_STEPS + 1)),
                ("pos", C.c_int64 * INTERP_MAX_STEPS), ("decay_power", C.c_float)]

    @staticmethod
    def make(vals, pos=(), decay_power=0.0):
        p = InterpParams()
        p.n_steps = len(pos)
        for i, v in enumerate(vals):
            p.val[i] = v
        for i, v in enumerate(pos):
            p.pos[i] = v
        p.decay_power = decay_power
        return p


class FileParams(C.Structure):
    _fields_ = [("model", abi.Params), ("lr", InterpParams), ("block_len", InterpParams), ("n_ranks", C.c_int32),
                ("dict", C.c_void_p), ("dict_len", C.c_uint32), ("retrain_period", C.c_uint32),
                ("retrain_len", C.c_uint32), ("has_retrain_lr", C.c_int32), ("retrain_lr", InterpParams)]


class BlockStats(C.Structure):
    _fields_ = [("n_symbols", C.c_int64), ("train_steps", C.c_int64), ("sum_log2", C.c_double)]


_I = C.c_int
FN_CTX = C.CFUNCTYPE(_I, _vp)
FN_SET_LR = C.CFUNCTYPE(_I, _vp, C.c_float)
FN_EVAL = C.CFUNCTYPE(_I, _vp, _I, C.POINTER(C.c_int32))
FN_PROBS = C.CFUNCTYPE(_I, _vp, _I, _I, C.POINTER(C.c_float))
FN_PATHS = C.CFUNCTYPE(_I, _vp, _I, _I, C.POINTER(C.c_int32), C.POINTER(C.c_uint16), C.POINTER(_I))
FN_TREES = C.CFUNCTYPE(_I, _vp, _I, _I, C.POINTER(C.c_uint16))
FN_GRAD = C.CFUNCTYPE(_I, _vp, C.POINTER(C.c_int32), C.POINTER(C.c_float))
FN_PATHS_BEGIN = C.CFUNCTYPE(_I, _vp, _I, _I, C.POINTER(C.c_int32))
FN_PATHS_END = C.CFUNCTYPE(_I, _vp, C.POINTER(C.c_uint16), C.POINTER(_I))
FN_GRAD_QUEUE = C.CFUNCTYPE(_I, _vp, C.POINTER(C.c_int32))
FN_READ_LOSS = C.CFUNCTYPE(_I, _vp, C.POINTER(C.c_float))
FN_DEC_BEGIN = C.CFUNCTYPE(_I, _vp, C.POINTER(C.c_uint8), C.c_size_t)
FN_DEC_STEPS = C.CFUNCTYPE(_I, _vp, _I, _I, C.POINTER(C.c_int32), _I, _I, C.POINTER(C.c_int32))
FN_DEC_END = C.CFUNCTYPE(_I, _vp, C.POINTER(C.c_size_t))


class ModelOps(C.Structure):
    _fields_ = [("ctx", _vp), ("n_streams", _I), ("seg_len", _I), ("n_symbols", _I),
                ("reset", FN_CTX), ("set_lr", FN_SET_LR), ("eval", FN_EVAL), ("read_probs", FN_PROBS),
                ("coder_paths", FN_PATHS), ("coder_trees", FN_TREES), ("eval_end", FN_CTX),
                ("eval_gradient", FN_GRAD), ("update", FN_CTX), ("coder_paths_begin", FN_PATHS_BEGIN),
                ("coder_paths_end", FN_PATHS_END), ("eval_gradient_queue", FN_GRAD_QUEUE), ("read_loss", FN_READ_LOSS),
                ("decoder_begin", FN_DEC_BEGIN),
                ("decode_steps", FN_DEC_STEPS), ("decoder_end", FN_DEC_END)]


_lib = None


def library():
    global _lib
    if _lib is None:
        if not os.path.exists(HOSTLIB):
            raise LibraryMissing(f"{HOSTLIB} is not built; run __graft_entry__.build()")
        L = C.CDLL(HOSTLIB)
        L.nch_enc_new.restype = _vp
        L.nch_enc_put_bit.argtypes = [_vp, _I, _I]
        L.nch_enc_put_bit.restype = None
        L.nch_enc_finish.argtypes = [_vp, C.POINTER(_vp)]
        L.nch_enc_finish.restype = C.c_size_t
        L.nch_enc_bytes.argtypes = [_vp]
        L.nch_enc_bytes.restype = C.c_size_t
        L.nch_enc_free.argtypes = [_vp]
        L.nch_enc_free.restype = None
        L.nch_dec_new.argtypes = [_vp, C.c_size_t]
        L.nch_dec_new.restype = _vp
        L.nch_dec_get_bit.argtypes = [_vp, _I]
        L.nch_dec_free.argtypes = [_vp]
        L.nch_dec_free.restype = None
        L.nch_vec_sum_f32.argtypes = [_vp, C.c_size_t]
        L.nch_vec_sum_f32.restype = C.c_float
        L.nch_write_sym.argtypes = [_vp, _vp, _I, _I]
        L.nch_write_sym.restype = None
        L.nch_read_sym.argtypes = [_vp, _vp, _I]
        L.nch_write_sym_path.argtypes = [_vp, _vp, _I, _I]
        L.nch_write_sym_path.restype = None
        L.nch_read_sym_tree.argtypes = [_vp, _vp, _I]
        L.nch_write_sym_paths.argtypes = [_vp, _vp, _I, _vp, C.c_size_t]
        L.nch_write_sym_paths.restype = None
        L.nch_write_sym_path_any.argtypes = [_vp, _vp, _I, _I]
        L.nch_write_sym_path_any.restype = None
        L.nch_write_sym_paths_any.argtypes = [_vp, _vp, _I, _vp, C.c_size_t]
        L.nch_write_sym_paths_any.restype = None
        L.nch_tree_depth.argtypes = [_I]
        L.nch_read_sym_trees.argtypes = [_vp, _vp, _I, C.c_size_t, _vp]
        L.nch_read_sym_trees.restype = None
        L.nch_next_block_len.argtypes = [C.POINTER(FileParams), C.c_size_t, C.c_size_t]
        L.nch_interp.argtypes = [C.POINTER(InterpParams), C.c_int64]
        L.nch_interp.restype = C.c_float
        L.nch_get_symb.argtypes = [_vp, _I, _I, _I, _I]
        L.nch_put_symb.argtypes = [_vp, _I, _I, _I, _I, _I]
        L.nch_bind_cuda.argtypes = [C.c_char_p, C.POINTER(abi.Params), C.POINTER(ModelOps)]
        L.nch_unbind_cuda.argtypes = [C.POINTER(ModelOps)]
        L.nch_unbind_cuda.restype = None
        L.nch_process_block.argtypes = [C.POINTER(ModelOps), _vp, _vp, _vp, _I, C.POINTER(InterpParams),
                                        C.POINTER(C.c_int64), _I, _I, C.POINTER(BlockStats)]
        L.nch_write_header.argtypes = [C.POINTER(FileParams), C.c_uint32, _vp, C.c_size_t,
                                       C.POINTER(C.c_size_t)]
        L.nch_read_header.argtypes = [_vp, C.c_size_t, C.POINTER(FileParams), C.POINTER(C.c_uint32),
                                      C.POINTER(C.c_size_t)]
        L.nch_compress.argtypes = [C.POINTER(ModelOps), C.POINTER(FileParams), _vp, C.c_size_t, _I, _I,
                                   C.POINTER(_vp), C.POINTER(C.c_size_t), C.POINTER(BlockStats)]
        L.nch_decompress.argtypes = [C.POINTER(ModelOps), C.POINTER(FileParams), _vp, C.c_size_t,
                                     C.c_uint32, _I, _vp]
        L.nch_free.argtypes = [_vp]
        L.nch_free.restype = None
        L.nch_read_dict.argtypes = [_vp, C.c_size_t, C.POINTER(_vp), C.POINTER(C.c_size_t)]
        L.nch_words_encode.argtypes = [_vp, C.c_size_t, _I, _I, C.POINTER(_vp), C.POINTER(C.c_size_t),
                                       C.POINTER(_vp), C.POINTER(C.c_size_t), C.POINTER(_I)]
        L.nch_words_decode.argtypes = [_vp, C.c_size_t, _vp, C.c_size_t, C.POINTER(_vp), C.POINTER(C.c_size_t)]
        L.nch_words_count.argtypes = [_vp, C.c_size_t]
        _lib = L
    return _lib


def file_params(model_params, lr=None, block_len=500000, dictionary=None, retrain_period=0, retrain_len=0,
                retrain_lr=None):
    """`dictionary`: the text nch_words_encode made; the file then carries it (deflated) in its header.
    `retrain_period`, `retrain_len`, `retrain_lr`: the retrain pass between blocks (without dropout)."""
    fp = FileParams()
    fp.model = model_params
    fp.lr = lr if lr is not None else InterpParams.make([model_params.lr])
    fp.block_len = InterpParams.make([float(block_len)])
    if dictionary:
        fp._dict_keep = C.create_string_buffer(bytes(dictionary), len(dictionary))   # owned by fp
        fp.dict = C.cast(fp._dict_keep, C.c_void_p)
        fp.dict_len = len(dictionary)
    if retrain_period:
        fp.retrain_period, fp.retrain_len = retrain_period, retrain_len
        if retrain_lr is not None:
            fp.has_retrain_lr, fp.retrain_lr = 1, retrain_lr
    return fp


def words_encode(text, n_words, min_word_freq):
    """word_encode of the reference preprocessor on memory: returns (dictionary text, uint16 symbols,
    number of dictionary entries).  The model's alphabet is `alphabet_size(entries)`."""
    L = library()
    text = bytes(text)
    d, dn, s, sn, ne = _vp(), C.c_size_t(), _vp(), C.c_size_t(), _I()
    rc = L.nch_words_encode(text, len(text), n_words, min_word_freq, C.byref(d), C.byref(dn), C.byref(s),
                            C.byref(sn), C.byref(ne))
    if rc != 0:
        raise ValueError(f"nch_words_encode: {rc}")
    dictionary = C.string_at(d.value, dn.value)
    syms = np.frombuffer(C.string_at(s.value, 2 * sn.value), np.uint16).copy() if sn.value else np.zeros(0, np.uint16)
    L.nch_free(d)
    L.nch_free(s)
    return dictionary, syms, ne.value


def words_decode(dictionary, symbols):
    """word_decode on memory: the text the symbols stand for."""
    L = library()
    s = np.ascontiguousarray(symbols, np.uint16)
    t, tn = _vp(), C.c_size_t()
    rc = L.nch_words_decode(bytes(dictionary), len(dictionary), s.ctypes.data_as(_vp), s.size, C.byref(t),
                            C.byref(tn))
    if rc != 0:
        raise ValueError(f"nch_words_decode: {rc}")
    text = C.string_at(t.value, tn.value)
    L.nch_free(t)
    return text


def words_count(dictionary):
    n = library().nch_words_count(bytes(dictionary), len(dictionary))
    if n < 0:
        raise ValueError(f"bad dictionary: {-n}")
    return n


def alphabet_size(n_entries):
    """Symbols of the model for a dictionary of n_entries: the next multiple of 8 (nncp.c:3382)."""
    return (n_entries + 7) & ~7


def read_dict(data):
    """The dictionary text a compressed file carries, or None."""
    L = library()
    d, dn = _vp(), C.c_size_t()
    rc = L.nch_read_dict(bytes(data), len(data), C.byref(d), C.byref(dn))
    if rc != 0:
        raise ValueError(f"nch_read_dict: {rc}")
    if not d.value:
        return None
    text = C.string_at(d.value, dn.value)
    L.nch_free(d)
    return text


def header_bytes(fp, n_symbols):
    L = library()
    n = C.c_size_t()
    L.nch_write_header(C.byref(fp), n_symbols, None, 0, C.byref(n))
    buf = C.create_string_buffer(n.value)
    assert L.nch_write_header(C.byref(fp), n_symbols, buf, n.value, C.byref(n)) == 0
    return buf.raw[: n.value]


def read_header(data):
    L = library()
    fp, nsym, used = FileParams(), C.c_uint32(), C.c_size_t()
    buf = C.create_string_buffer(data, len(data))
    rc = L.nch_read_header(buf, len(data), C.byref(fp), C.byref(nsym), C.byref(used))
    if rc != 0:
        raise ValueError(f"bad header: {rc}")
    return fp, nsym.value, used.value


def _model_error():
    """What the CUDA library last complained about (status 8 of the host code means a model call failed)."""
    try:
        L = C.CDLL(LIB)
        L.nncu_last_error.restype = C.c_char_p
        return L.nncu_last_error().decode()
    except OSError:
        return "libnncu.so not loaded"


def compress(ops, fp, symbols, eval_mode=EVAL_SEGMENT, out_mode=OUT_CODER_READY):
    """encode_file on memory: returns (bytes, BlockStats)."""
    L = library()
    s = np.ascontiguousarray(symbols, np.uint16)
    out, n, st = _vp(), C.c_size_t(), BlockStats()
    rc = L.nch_compress(C.byref(ops), C.byref(fp), s.ctypes.data_as(_vp), s.size, eval_mode, out_mode,
                        C.byref(out), C.byref(n), C.byref(st))
    if rc != 0:
        raise RuntimeError(f"nch_compress: {rc} ({_model_error()})")
    data = C.string_at(out.value, n.value)
    L.nch_free(out)
    return data, st


def decompress(ops, data, out_mode=OUT_CODER_READY):
    """decode_file on memory: returns the uint16 symbols."""
    L = library()
    fp, nsym, used = read_header(data)
    payload = data[used:]
    buf = C.create_string_buffer(payload, len(payload))
    out = np.zeros(nsym, np.uint16)
    rc = L.nch_decompress(C.byref(ops), C.byref(fp), buf, len(payload), nsym, out_mode,
                          out.ctypes.data_as(_vp))
    if rc != 0:
        raise RuntimeError(f"nch_decompress: {rc} ({_model_error()})")
    return out


def bind_cuda(model_params):
    L = library()
    ops = ModelOps()
    rc = L.nch_bind_cuda(LIB.encode(), C.byref(model_params), C.byref(ops))
    if rc != 0:
        raise LibraryMissing(f"nch_bind_cuda failed ({rc}): no CUDA model, and no other implementation")
    return ops


def unbind_cuda(ops):
    library().nch_unbind_cuda(C.byref(ops))


def compress_text(text, n_words, min_word_freq, model_params, bind=bind_cuda, unbind=unbind_cuda, lr=None,
                  block_len=500000, eval_mode=EVAL_SEGMENT, out_mode=OUT_CODER_READY, pad_alphabet=False):
    """`nncp --preprocess n_words,min_word_freq c` on memory: tokenises the text (nch_words_encode),
    sizes the model's alphabet to the dictionary ((entries + 7) & ~7, nncp.c:3382), and codes the
    symbols into a file that carries the dictionary.  `model_params` gives everything but n_symbols;
    `bind(params)` makes the model ops (the CUDA model by default).  Returns (file bytes, BlockStats).
    `pad_alphabet` rounds the alphabet up to a power of two instead (symbols past the dictionary never
    occur; any decoder reads the size from the header): the coder's tree is then even, which is the
    shape the register-level path kernel for 1024..16384 symbols is written for."""
    dictionary, syms, entries = words_encode(text, n_words, min_word_freq)
    n_symbols = alphabet_size(entries)
    if pad_alphabet:
        n_symbols = 1 << (n_symbols - 1).bit_length()
    p = model_params.copy(n_symbols=n_symbols)
    fp = file_params(p, lr=lr, block_len=block_len, dictionary=dictionary)
    ops = bind(p)
    try:
        return compress(ops, fp, syms, eval_mode, out_mode)
    finally:
        unbind(ops)


def decompress_text(data, bind=bind_cuda, unbind=unbind_cuda, out_mode=OUT_DEVICE):
    """The inverse: rebuilds the model from the file's header, decodes the symbols and turns them back
    into text with the file's dictionary (a file without one holds bytes, returned as they are)."""
    fp, _, _ = read_header(data)
    dictionary = read_dict(data)
    ops = bind(fp.model)
    try:
        syms = decompress(ops, data, out_mode)
    finally:
        unbind(ops)
    if dictionary is None:
        return syms.astype(np.uint8).tobytes()
    return words_decode(dictionary, syms)
