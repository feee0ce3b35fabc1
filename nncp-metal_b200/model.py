"""TrfModel: the model-plugin verbs of the reference (NNCPModelClass, nncp.c:49-69) over
the C ABI.  Every method is one ABI call; arrays are numpy on the host."""
import ctypes as C

import numpy as np

from . import abi
from .loader import library

_vp = C.c_void_p


def _ptr(a):
    return a.ctypes.data_as(_vp)


class NncuError(RuntimeError):
    pass


class TrfModel:
    def __init__(self, params):
        self.lib = library()
        self.p = params
        self.h = _vp()
        self._ck(self.lib.nncu_create(C.byref(params), C.byref(self.h)))
        self.T, self.B, self.V = params.seg_len, params.n_streams, params.n_symbols
        self.has_comm = False
        self.info = {}
        self.index = {}
        name = C.create_string_buffer(32)
        n, off = C.c_size_t(), C.c_size_t()
        for i in range(self.lib.nncu_param_count(self.h)):
            self._ck(self.lib.nncu_param_info(self.h, i, name, 32, C.byref(n), C.byref(off)))
            self.info[name.value.decode()] = (off.value, n.value)
            self.index[name.value.decode()] = i

    def _ck(self, rc):
        if rc != 0:
            raise NncuError(f"nncu error {rc}: {self.lib.nncu_last_error().decode()}")

    def close(self):
        if getattr(self, "h", None):
            self.lib.nncu_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- plugin verbs -------------------------------------------------
    def set_stream(self, cuda_stream):
        self._ck(self.lib.nncu_set_stream(self.h, _vp(cuda_stream)))

    def reset(self):
        self._ck(self.lib.nncu_reset(self.h))

    def set_lr(self, lr):
        self._ck(self.lib.nncu_set_lr(self.h, float(lr)))

    def eval(self, output_index, ids, read=True):
        """model_eval: ids int32 [T, B].  Returns probs [T or 1, B, V] when read."""
        ids = np.ascontiguousarray(ids, np.int32)
        assert ids.size == self.T * self.B
        self._ck(self.lib.nncu_eval(self.h, int(output_index), _ptr(ids)))
        if not read:
            return None
        return self.read_probs(0, self.T) if output_index < 0 else self.read_probs(output_index, 1)

    def eval_dev(self, output_index, ids_dev_ptr):
        self._ck(self.lib.nncu_eval_dev(self.h, int(output_index), _vp(ids_dev_ptr)))

    def eval_end(self):
        self._ck(self.lib.nncu_eval_end(self.h))

    def read_probs(self, t0, nt):
        out = np.empty((nt, self.B, self.V), np.float32)
        self._ck(self.lib.nncu_read_probs(self.h, t0, nt, _ptr(out)))
        return out

    def probs_dev(self):
        p = _vp()
        self._ck(self.lib.nncu_probs_dev(self.h, C.byref(p)))
        return p.value

    def eval_gradient(self, targets):
        t = np.ascontiguousarray(targets, np.int32)
        loss = C.c_float()
        self._ck(self.lib.nncu_eval_gradient(self.h, _ptr(t), C.byref(loss)))
        return loss.value

    def eval_gradient_dev(self, targets_dev_ptr):
        self._ck(self.lib.nncu_eval_gradient_dev(self.h, _vp(targets_dev_ptr)))

    def eval_gradient_update(self, targets, wait_loss=True):
        """Backward pass with the optimizer step queued per layer; follow with memory_shift()."""
        t = np.ascontiguousarray(targets, np.int32)
        loss = C.c_float()
        self._ck(self.lib.nncu_eval_gradient_update(self.h, _ptr(t), C.byref(loss) if wait_loss else None))
        return loss.value if wait_loss else None

    def eval_gradient_update_dev(self, targets_dev_ptr):
        self._ck(self.lib.nncu_eval_gradient_update_dev(self.h, _vp(targets_dev_ptr)))

    def read_loss(self):
        loss = C.c_float()
        self._ck(self.lib.nncu_read_loss(self.h, C.byref(loss)))
        return loss.value

    def update(self):
        self._ck(self.lib.nncu_update(self.h))

    def optimizer_step(self):
        self._ck(self.lib.nncu_optimizer_step(self.h))

    def memory_shift(self):
        self._ck(self.lib.nncu_memory_shift(self.h))

    def synchronize(self):
        self._ck(self.lib.nncu_synchronize(self.h))

    # --- parameters ---------------------------------------------------
    def get_param(self, name):
        off, n = self.info[name]
        out = np.empty(n, np.float32)
        self._ck(self.lib.nncu_param_get(self.h, self.index[name], _ptr(out), n))
        return out

    def set_param(self, name, value):
        off, n = self.info[name]
        v = np.ascontiguousarray(np.asarray(value, np.float32).reshape(-1))
        assert v.size == n, (name, v.size, n)
        self._ck(self.lib.nncu_param_set(self.h, self.index[name], _ptr(v), n))

    def get_grad(self, name):
        off, n = self.info[name]
        out = np.empty(n, np.float32)
        self._ck(self.lib.nncu_grad_get(self.h, self.index[name], _ptr(out), n))
        return out

    def flat_buffers(self):
        w, g, v, n = _vp(), _vp(), _vp(), C.c_size_t()
        self._ck(self.lib.nncu_flat_buffers(self.h, C.byref(w), C.byref(g), C.byref(v),
                                            C.byref(n)))
        return w.value, g.value, v.value, n.value

    def comm_init(self, n_ranks, rank, unique_id):
        """Attach an NCCL communicator: eval_gradient then leaves globally summed gradients."""
        buf = C.create_string_buffer(bytes(unique_id), 128)
        self._ck(self.lib.nncu_comm_init(self.h, n_ranks, rank, buf))
        self.has_comm = True

    def gather_master(self):
        """Collective (every rank calls it): completes the sharded optimizer state on every rank."""
        self._ck(self.lib.nncu_comm_gather_master(self.h))

    def weights_hash(self):
        """Under a communicator this is a collective: the sharded master weights are gathered first."""
        if self.has_comm:
            self.gather_master()
        h = C.c_uint64()
        self._ck(self.lib.nncu_weights_hash(self.h, C.byref(h)))
        return h.value

    # --- coder-ready output -------------------------------------------
    def coder_paths(self, t0, nt, syms):
        s = np.ascontiguousarray(syms, np.int32)
        nb = C.c_int()
        out = np.zeros((nt * self.B, 32), np.uint16)
        tmp = np.zeros(nt * self.B * 32, np.uint16)
        self._ck(self.lib.nncu_coder_paths(self.h, t0, nt, _ptr(s), _ptr(tmp), C.byref(nb)))
        return tmp[: nt * self.B * nb.value].reshape(nt * self.B, nb.value).copy()

    def coder_trees(self, t0, nt):
        """prob0 of every tree node, heap order: [nt * B][2^ceil(log2 V)]"""
        out = np.zeros((nt * self.B, 1 << (self.V - 1).bit_length()), np.uint16)
        self._ck(self.lib.nncu_coder_trees(self.h, t0, nt, _ptr(out)))
        return out

    # --- range decoder on the device ------------------------------------
    def decoder_begin(self, payload):
        buf = np.frombuffer(bytes(payload), np.uint8)
        self._ck(self.lib.nncu_decoder_begin(self.h, _ptr(buf) if buf.size else None, buf.size))

    def decode_steps(self, t0, nt, ids_t0=None, limit_t=None, limit_b=0):
        """Steps t0 .. t0+nt-1: returns the decoded symbols [nt][B]."""
        ids = None if ids_t0 is None else np.ascontiguousarray(ids_t0, np.int32)
        out = np.zeros((nt, self.B), np.int32)
        self._ck(self.lib.nncu_decode_steps(self.h, t0, nt, None if ids is None else _ptr(ids),
                                            self.T if limit_t is None else limit_t, limit_b, _ptr(out)))
        return out

    def decoder_end(self):
        n = C.c_size_t()
        self._ck(self.lib.nncu_decoder_end(self.h, C.byref(n)))
        return n.value
