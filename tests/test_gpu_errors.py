"""The error path of a bounded device-side wait: it runs out, the kernel returns, the host reads
NNCU_ERR_TIMEOUT once, and the model computes the same step afterwards as one that never saw it."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

KW = dict(n_layer=2, d_model=256, n_head=4, d_key=64, d_inner=512, d_pos=48, mem_len=16, seg_len=32,
          n_streams=4, n_symbols=512, use_bf16=1, lr=1e-3, init_range=0.03)


def test_expired_wait_is_reported_once_and_the_model_survives(pkg):
    p = pkg.abi.make_params(**KW)
    a, b = pkg.TrfModel(p), pkg.TrfModel(p)
    rng = np.random.default_rng(2)
    ids = rng.integers(0, 512, (32, 4)).astype(np.int32)
    tg = rng.integers(0, 512, (32, 4)).astype(np.int32)
    assert a.lib.nncu_selftest_expired_wait(a.h) == 0
    assert a.lib.nncu_synchronize(a.h) == pkg.abi.ERR_TIMEOUT
    assert b"bounded device-side wait" in a.lib.nncu_last_error()
    assert a.lib.nncu_synchronize(a.h) == 0          # the flag was cleared by the report
    for m in (a, b):
        m.reset()
        m.eval(-1, ids, read=False)
        m.eval_gradient(tg)
        m.update()
    assert a.weights_hash() == b.weights_hash()
    a.close()
    b.close()
