"""Seeded parameter values for the digest goldens (dig_*.npz), too large to store.

The values come from the oracle's counter-based generator (orc_init_values in
oracle/trf_oracle.c: integer hashing of (seed, parameter name, index), sum of 12 uniforms), so the
script that makes a golden and the test that checks it rebuild exactly the same fp32 weights
without a 60 MB fixture.  Test infrastructure only.
"""
import numpy as np


def seeded_params(orc, shapes, seed, wscale):
    """{name: float32 array} for (name, shape) pairs; `orc` is the oracle.oracle module."""
    L = orc.lib()
    out = {}
    for name, shape in shapes:
        n = int(np.prod(shape))
        buf = np.empty(n, np.float32)
        L.orc_init_values(buf.ctypes.data, n, name.encode(), int(seed), 1, 1.0)
        if name.startswith("ln_g"):
            v = 1.0 + 0.1 * buf
        elif name.startswith(("ln_b", "ff_bias", "out_bias", "b_q")):
            v = 0.05 * buf
        elif name.startswith("b_r"):
            v = 0.02 * buf
        else:
            v = wscale * buf
        out[name] = np.ascontiguousarray(v.astype(np.float32)).reshape(shape)
    return out


def subsample(a, cap=4096):
    """(stride, a.flat[::stride]) with at most `cap` (+1) elements."""
    flat = np.asarray(a).reshape(-1)
    stride = max(1, flat.size // cap)
    return stride, flat[::stride]
