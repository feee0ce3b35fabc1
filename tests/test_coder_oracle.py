"""The coder restatement against the reference's own arith.c + cp_utils.c (compiled unchanged
into oracle/_ref/libref_coder.so): identical bytes out, identical symbols back."""
import numpy as np
import pytest

from oracle import oracle as orc

needs_ref = pytest.mark.skipif(orc.ref_lib() is None, reason="oracle/_ref was never built")


def _tables(rng, n, V, sharp):
    z = rng.standard_normal((n, V)).astype(np.float32) * sharp
    e = np.exp(z - z.max(1, keepdims=True))
    return (e / e.sum(1, keepdims=True)).astype(np.float32)


@needs_ref
@pytest.mark.parametrize("V,sharp", [(2, 1.0), (16, 1.0), (256, 3.0), (24, 2.0), (1000, 4.0),
                                     (16384, 6.0)])
def test_bytes_match_reference(V, sharp):
    rng = np.random.default_rng(V)
    n = 300 if V <= 1000 else 40
    probs = _tables(rng, n, V, sharp)
    syms = np.array([rng.choice(V, p=p.astype(np.float64) / p.astype(np.float64).sum())
                     for p in probs])
    a, b = orc.Encoder(False), orc.Encoder(True)
    for p, s in zip(probs, syms):
        a.put_sym(p, s)
        b.put_sym(p, s)
    da, db = a.finish(), b.finish()
    assert da == db and len(da) > 0
    for use_ref in (False, True):
        d = orc.Decoder(da, use_ref)
        back = [d.read_sym(p) for p in probs]
        d.close()
        assert back == list(syms)


@needs_ref
def test_raw_bits_and_carry_runs_match_reference():
    rng = np.random.default_rng(7)
    # extreme probabilities force long 0xff runs and carries (arith.c:72-94)
    pr = rng.choice([1, 2, 16384, 32766, 32767], size=20000)
    bits = (rng.random(20000) < 0.5).astype(int)
    a, b = orc.Encoder(False), orc.Encoder(True)
    for q, bit in zip(pr, bits):
        a.put_bit(q, bit)
        b.put_bit(q, bit)
    da, db = a.finish(), b.finish()
    assert da == db
    d0, d1 = orc.Decoder(da, False), orc.Decoder(da, True)
    for q, bit in zip(pr, bits):
        assert d0.get_bit(q) == bit
        assert d1.get_bit(q) == bit


def test_empty_stream_and_truncated_input():
    e = orc.Encoder(False)
    data = e.finish()
    assert isinstance(data, bytes)
    # the decoder zero-pads past the end instead of failing (arith.c:209-223)
    d = orc.Decoder(b"", False)
    p = np.full(16, 1 / 16, np.float32)
    assert 0 <= d.read_sym(p) < 16


def test_vec_sum_is_the_halving_tree():
    rng = np.random.default_rng(3)
    for n in (1, 2, 3, 7, 8, 24, 255, 256, 1000):
        a = rng.random(n).astype(np.float32)

        def rec(x):
            if len(x) == 1:
                return np.float32(x[0])
            h = len(x) >> 1
            return np.float32(rec(x[:h]) + rec(x[h:]))
        assert orc.vec_sum(a) == rec(a)


def test_sym_path_matches_put_sym():
    rng = np.random.default_rng(11)
    probs = _tables(rng, 50, 256, 3.0)
    syms = rng.integers(0, 256, 50)
    a, b = orc.Encoder(False), orc.Encoder(False)
    for p, s in zip(probs, syms):
        a.put_sym(p, s)
        path = orc.sym_path(p, s)
        assert len(path) == 8
        for k, q in enumerate(path):
            b.put_bit(q, (int(s) >> (7 - k)) & 1)
    assert a.finish() == b.finish()


@needs_ref
def test_interp_param_reference_values():
    """get_interp_param (cp_utils.c:380-410) through the reference build: the values the
    host-side schedule restatement is pinned to."""
    L = orc.ref_lib()
    val = np.array([3e-4, 1e-4], np.float32)
    pos = np.array([156250], np.int64)
    f = lambda at, dp=0.0: L.ref_interp(1, val.ctypes.data, pos.ctypes.data, dp, at)
    assert f(0) == np.float32(3e-4)
    assert abs(f(78125) - 2e-4) < 1e-9
    assert f(156250) == np.float32(1e-4)
    assert f(10 ** 7) == np.float32(1e-4)
    assert abs(f(625000, 0.5) - 0.5e-4) < 1e-10
