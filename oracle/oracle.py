"""ctypes loader for the test-only CPU oracle (liboracle.so) and for what oracle/Makefile builds from
the reference's own sources into _ref/: its coder (libref_coder.so), its word preprocessor as a tool
(preprocess_ref), its shipped --cpu codec (libref_cpu_codec.so) and its nncp command line on the CPU
oracle (nncp_oracle).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs, never by the shipped package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t


def reference_dir():
    """Directory of the reference project's sources, or None: $NNCP_REFERENCE_DIR, else the
    `reference_path` the repository's BASELINE.json records, when that directory exists."""
    import json
    cand = os.environ.get("NNCP_REFERENCE_DIR")
    if not cand:
        try:
            cand = json.load(open(os.path.join(os.path.dirname(HERE), "BASELINE.json"))).get("reference_path")
        except (OSError, ValueError):
            cand = None
    return cand if cand and os.path.isfile(os.path.join(cand, "arith.c")) else None


def build(force=False):
    """Compiles liboracle.so (and _ref/ when the reference tree is present)."""
    so = os.path.join(HERE, "liboracle.so")
    srcs = [os.path.join(HERE, f) for f in ("trf_oracle.c", "coder_oracle.c")]
    stale = (not os.path.exists(so)) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs)
    ref = reference_dir()
    have_ref = all(os.path.exists(os.path.join(HERE, "_ref", f))
                   for f in ("libref_coder.so", "preprocess_ref", "libref_cpu_codec.so", "nncp_oracle"))
    if force or stale or (ref and not have_ref):
        subprocess.run(["make", "-C", HERE, "all", f"REF={ref or ''}"], check=True, capture_output=True)
    return so


def cpu_codec_ref():
    """The reference's shipped `--cpu` codec (nncp_original_compress / _decompress of its
    src/metal/nncp_original_port.c, compiled unchanged by the Makefile here), or None."""
    so = os.path.join(HERE, "_ref", "libref_cpu_codec.so")
    if not os.path.exists(so):
        return None
    L = C.CDLL(so)
    for f in (L.nncp_original_compress, L.nncp_original_decompress):
        f.argtypes = [_vp, _sz, _vp, _sz, C.POINTER(_sz), C.c_bool]
        f.restype = C.c_bool
    return L


def nncp_oracle():
    """Path of the reference's own `nncp` command line built on the CPU oracle (its unmodified nncp.c +
    the model plugin adapter of the drop-in + nncu_on_oracle.c), or None when it was never built.
    Options and verbs are the reference's (`nncp_oracle --cuda [options] c in out`, `... d in out`)."""
    exe = os.path.join(HERE, "_ref", "nncp_oracle")
    return exe if os.access(exe, os.X_OK) else None


def preprocess_ref():
    """Path of the reference's stand-alone word preprocessor (built from its preprocess.c by the
    Makefile here), or None when it was never built: `preprocess_ref c dict in out n_words min_freq`
    encodes, `preprocess_ref d dict in out` decodes."""
    exe = os.path.join(HERE, "_ref", "preprocess_ref")
    return exe if os.access(exe, os.X_OK) else None


_lib = None


def lib():
    global _lib
    if _lib is None:
        so = build()
        L = C.CDLL(so)
        L.orc_create.argtypes = [_vp, C.POINTER(_vp)]
        L.orc_destroy.argtypes = [_vp]
        L.orc_destroy.restype = None
        L.orc_param_count.argtypes = [_vp]
        L.orc_param_info.argtypes = [_vp, _i, C.c_char_p, _sz, C.POINTER(_sz), C.POINTER(_sz)]
        for f in ("orc_weights", "orc_grads", "orc_moments", "orc_probs"):
            getattr(L, f).argtypes = [_vp]
            getattr(L, f).restype = C.POINTER(C.c_float)
        L.orc_mem.argtypes = [_vp, _i]
        L.orc_mem.restype = C.POINTER(C.c_float)
        L.orc_n_floats.argtypes = [_vp]
        L.orc_n_floats.restype = _sz
        L.orc_reset.argtypes = [_vp]
        L.orc_reset.restype = None
        L.orc_set_lr.argtypes = [_vp, C.c_float]
        L.orc_set_lr.restype = None
        L.orc_eval.argtypes = [_vp, _i, _vp, _vp]
        L.orc_eval_gradient.argtypes = [_vp, _vp, C.POINTER(C.c_float)]
        L.orc_update.argtypes = [_vp]
        L.orc_init_values.argtypes = [_vp, _sz, C.c_char_p, C.c_uint32, _i, C.c_float]
        L.orc_init_values.restype = None
        L.orc_attention_forward.argtypes = [_vp] * 8
        L.orc_attention_backward.argtypes = [_vp] * 11
        L.orc_vec_sum_f32.argtypes = [_vp, _sz]
        L.orc_vec_sum_f32.restype = C.c_float
        L.orc_enc_new.restype = _vp
        L.orc_enc_put_sym.argtypes = [_vp, _vp, _i, _i]
        L.orc_enc_put_sym.restype = None
        L.orc_enc_put_bit.argtypes = [_vp, _i, _i]
        L.orc_enc_put_bit.restype = None
        L.orc_enc_finish.argtypes = [_vp, C.POINTER(_vp)]
        L.orc_enc_finish.restype = _sz
        L.orc_enc_free.argtypes = [_vp]
        L.orc_enc_free.restype = None
        L.orc_dec_new.argtypes = [_vp, _sz]
        L.orc_dec_new.restype = _vp
        L.orc_dec_read_sym.argtypes = [_vp, _vp, _i]
        L.orc_dec_get_bit.argtypes = [_vp, _i]
        L.orc_dec_free.argtypes = [_vp]
        L.orc_dec_free.restype = None
        L.orc_sym_path.argtypes = [_vp, _i, _i, _vp]
        L.orc_sym_tree.argtypes = [_vp, _i, _vp]
        L.orc_set_threads.argtypes = [_i]
        L.orc_set_threads.restype = _i
        L.orc_get_threads.restype = _i
        _lib = L
    return _lib


_ref = None


def ref_lib():
    """The reference's own coder, compiled unchanged (None if it was never built)."""
    global _ref
    if _ref is None:
        so = os.path.join(HERE, "_ref", "libref_coder.so")
        if not os.path.exists(so):
            build()
        if not os.path.exists(so):
            return None
        L = C.CDLL(so)
        L.ref_enc_new.restype = _vp
        L.ref_enc_put_sym.argtypes = [_vp, _vp, _i, _i]
        L.ref_enc_put_sym.restype = None
        L.ref_enc_put_bit.argtypes = [_vp, _i, _i]
        L.ref_enc_put_bit.restype = None
        L.ref_enc_finish.argtypes = [_vp, C.POINTER(_vp)]
        L.ref_enc_finish.restype = _sz
        L.ref_enc_free.argtypes = [_vp]
        L.ref_enc_free.restype = None
        L.ref_dec_new.argtypes = [_vp, _sz]
        L.ref_dec_new.restype = _vp
        L.ref_dec_read_sym.argtypes = [_vp, _vp, _i]
        L.ref_dec_get_bit.argtypes = [_vp, _i]
        L.ref_dec_free.argtypes = [_vp]
        L.ref_dec_free.restype = None
        L.ref_interp.argtypes = [_i, _vp, _vp, C.c_float, C.c_int64]
        L.ref_interp.restype = C.c_float
        _ref = L
    return _ref


def _ptr(a):
    return a.ctypes.data_as(_vp)


class OracleModel:
    """The oracle behind the same verbs as the model plugin (eval / eval_gradient / update)."""

    def __init__(self, params):
        self.L = lib()
        self.p = params
        h = _vp()
        rc = self.L.orc_create(C.byref(params), C.byref(h))
        if rc != 0:
            raise ValueError(f"orc_create failed: {rc}")
        self.h = h
        self.T, self.B, self.V = params.seg_len, params.n_streams, params.n_symbols
        self.info = {}
        name = C.create_string_buffer(32)
        n, off = _sz(), _sz()
        for i in range(self.L.orc_param_count(h)):
            self.L.orc_param_info(h, i, name, 32, C.byref(n), C.byref(off))
            self.info[name.value.decode()] = (off.value, n.value)
        self.n_floats = self.L.orc_n_floats(h)

    def close(self):
        if getattr(self, "h", None):
            self.L.orc_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def _flat(self, fn):
        return np.ctypeslib.as_array(fn(self.h), shape=(self.n_floats,))

    def get_param(self, name):
        off, n = self.info[name]
        return self._flat(self.L.orc_weights)[off:off + n].copy()

    def set_param(self, name, value):
        off, n = self.info[name]
        self._flat(self.L.orc_weights)[off:off + n] = np.asarray(value, np.float32).reshape(-1)

    def get_grad(self, name):
        off, n = self.info[name]
        return self._flat(self.L.orc_grads)[off:off + n].copy()

    def mem(self, layer):
        n = self.p.mem_len * self.B * self.p.d_model
        return np.ctypeslib.as_array(self.L.orc_mem(self.h, layer), shape=(max(n, 1),))[:n].copy()

    def reset(self):
        self.L.orc_reset(self.h)

    def set_lr(self, lr):
        self.L.orc_set_lr(self.h, lr)

    def eval(self, output_index, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        n = self.T if output_index < 0 else 1
        out = np.empty((n, self.B, self.V), np.float32)
        rc = self.L.orc_eval(self.h, output_index, _ptr(ids), _ptr(out))
        if rc != 0:
            raise RuntimeError(f"orc_eval: {rc}")
        return out

    def eval_gradient(self, targets):
        t = np.ascontiguousarray(targets, np.int32)
        loss = C.c_float()
        rc = self.L.orc_eval_gradient(self.h, _ptr(t), C.byref(loss))
        if rc != 0:
            raise RuntimeError(f"orc_eval_gradient: {rc}")
        return loss.value

    def update(self):
        self.L.orc_update(self.h)


def vec_sum(a):
    a = np.ascontiguousarray(a, np.float32)
    return lib().orc_vec_sum_f32(_ptr(a), a.size)


class Encoder:
    def __init__(self, use_ref=False):
        self.L = ref_lib() if use_ref else lib()
        self.pre = "ref" if use_ref else "orc"
        self.h = getattr(self.L, self.pre + "_enc_new")()

    def put_sym(self, prob, sym):
        prob = np.ascontiguousarray(prob, np.float32)
        getattr(self.L, self.pre + "_enc_put_sym")(self.h, _ptr(prob), prob.size, int(sym))

    def put_bit(self, prob0, bit):
        getattr(self.L, self.pre + "_enc_put_bit")(self.h, int(prob0), int(bit))

    def finish(self):
        out = _vp()
        n = getattr(self.L, self.pre + "_enc_finish")(self.h, C.byref(out))
        data = C.string_at(out.value, n) if n else b""
        getattr(self.L, self.pre + "_enc_free")(self.h)
        self.h = None
        return data


class Decoder:
    def __init__(self, data, use_ref=False):
        self.L = ref_lib() if use_ref else lib()
        self.pre = "ref" if use_ref else "orc"
        self.buf = C.create_string_buffer(data, len(data))
        self.h = getattr(self.L, self.pre + "_dec_new")(C.cast(self.buf, _vp), len(data))

    def read_sym(self, prob):
        prob = np.ascontiguousarray(prob, np.float32)
        return getattr(self.L, self.pre + "_dec_read_sym")(self.h, _ptr(prob), prob.size)

    def get_bit(self, prob0):
        return getattr(self.L, self.pre + "_dec_get_bit")(self.h, int(prob0))

    def close(self):
        if self.h:
            getattr(self.L, self.pre + "_dec_free")(self.h)
            self.h = None


def sym_tree(prob):
    """prob0 of every node of the coder's tree over this row, heap order, 2^ceil(log2 V) entries."""
    prob = np.ascontiguousarray(prob, np.float32)
    depth = int(np.ceil(np.log2(prob.size)))
    out = np.zeros(1 << depth, np.uint16)
    lib().orc_sym_tree(_ptr(prob), prob.size, _ptr(out))
    return out


def sym_path(prob, sym):
    prob = np.ascontiguousarray(prob, np.float32)
    out = np.zeros(32, np.uint16)
    k = lib().orc_sym_path(_ptr(prob), prob.size, int(sym), _ptr(out))
    return out[:k].copy()
