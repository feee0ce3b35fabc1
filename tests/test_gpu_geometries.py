"""Whole-model parity of the CUDA path at the geometries BASELINE.json names.

  config[0]   exactly (2 layers, d_model 128, 4 x 32 heads, d_ff 512, seg 32, mem 32, 4 streams,
              vocab 256, fp32): against the float64 digest golden and the oracle.
  config[2]   its widths (d_model 512, 8 x 64 heads, d_ff 2048, vocab 16384, seg 64, mem 64) with
              fewer layers and streams: fp32 against the digest golden, bf16 (tcgen05 GEMMs,
              tensor-core attention) against the oracle.
  config[3]   its widths (d_model 1024, 16 x 64 heads, d_ff 4096, mem 256, d_pos 320), one layer,
              two streams, bf16 against the oracle.
  config[4]   one-symbol steps against the whole segment, bit for bit, with a 512-row memory and
              128 streams.

Tolerances as everywhere in this suite: fp32 1e-3, bf16 2e-2 (max-abs-diff over max-abs-ref).
"""
import numpy as np
import pytest

from conftest import (check_digest_step, check_updated_weights, load_digest, params_from_cfg, rel_err)

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FP32_TOL, BF16_TOL = 1e-3, 2e-2


def _bf16_round(a):
    return torch.as_tensor(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("name", ["c0", "c2_geometry"])
def test_fp32_model_vs_digest_golden_and_oracle(pkg, oracle, name):
    cfg, z, params = load_digest(name)
    p = params_from_cfg(pkg, cfg)
    m, o = pkg.TrfModel(p), oracle.OracleModel(p)
    for pname in m.info:
        m.set_param(pname, params[pname])
        o.set_param(pname, params[pname])
    m.reset(); o.reset()
    m.set_lr(cfg["lr"]); o.set_lr(cfg["lr"])
    for s in range(z["ids"].shape[0]):
        probs, probs_o = m.eval(-1, z["ids"][s]), o.eval(-1, z["ids"][s])
        assert rel_err(probs, probs_o) < FP32_TOL
        loss, loss_o = m.eval_gradient(z["targets"][s]), o.eval_gradient(z["targets"][s])
        assert abs(loss - loss_o) < FP32_TOL * abs(loss_o)
        check_digest_step(m, z, s, FP32_TOL, FP32_TOL, probs, loss)
        grads, before = {}, {}
        for pname in m.info:
            g_ref = o.get_grad(pname)
            grads[pname], before[pname] = g_ref, o.get_param(pname)
            scale = max(np.abs(g_ref).max(), 1e-9)
            assert np.abs(m.get_grad(pname) - g_ref).max() / scale < FP32_TOL, (pname, s)
        m.update(); o.update()
        for pname in m.info:
            check_updated_weights(m.get_param(pname), o.get_param(pname), before[pname], grads[pname],
                                  FP32_TOL, cfg["lr"], cfg["beta2"], (pname, s))
            stride = int(z[f"stride/{pname}"])
            bound = 2 * FP32_TOL * max(np.abs(z[f"p{s+1}/{pname}"]).max(), 1e-3) + \
                2.1 * cfg["lr"] / np.sqrt(1 - cfg["beta2"])
            assert np.abs(m.get_param(pname)[::stride] - z[f"p{s+1}/{pname}"]).max() < bound, (pname, s)
        for pname in m.info:      # keep the two trajectories together: step 2 then tests step 2
            o.set_param(pname, m.get_param(pname))
    m.close()


def _bf16_vs_oracle(pkg, oracle, kw, steps, seed, wscale):
    import sys
    from conftest import GOLDEN_DIR
    sys.path.insert(0, GOLDEN_DIR)
    import seeded_params as sp
    import trf_torch as tt
    m = pkg.TrfModel(pkg.abi.make_params(use_bf16=1, gemm_backend=2, **kw))
    o = oracle.OracleModel(pkg.abi.make_params(use_bf16=0, **kw))
    cfg = dict(kw, ff_act=1, query_bias=1, use_bias=1, use_w_r=1, tied_w_r=0, tied_b_r=0, ln_flags=1)
    params = sp.seeded_params(oracle, tt.param_shapes(cfg), seed, wscale)
    assert set(params) == set(m.info)
    for pname in m.info:
        w = _bf16_round(params[pname])
        m.set_param(pname, w)
        o.set_param(pname, w)
    rng = np.random.default_rng(seed)
    T, B, V = kw["seg_len"], kw["n_streams"], kw["n_symbols"]
    m.reset(); o.reset()
    for s in range(steps):
        ids = rng.integers(0, V, (T, B)).astype(np.int32)
        tg = rng.integers(0, V, (T, B)).astype(np.int32)
        probs, probs_o = m.eval(-1, ids), o.eval(-1, ids)
        assert rel_err(probs, probs_o) < BF16_TOL, s
        loss, loss_o = m.eval_gradient(tg), o.eval_gradient(tg)
        assert abs(loss - loss_o) < BF16_TOL * abs(loss_o)
        grads, before = {}, {}
        for pname in m.info:
            g_ref = o.get_grad(pname)
            grads[pname], before[pname] = g_ref, o.get_param(pname)
            scale = max(np.abs(g_ref).max(), 1e-9)
            assert np.abs(m.get_grad(pname) - g_ref).max() / scale < 5 * BF16_TOL, (pname, s)
        m.update(); o.update()
        for pname in m.info:
            check_updated_weights(m.get_param(pname), o.get_param(pname), before[pname], grads[pname],
                                  BF16_TOL, kw["lr"], 0.99, (pname, s))
        for pname in m.info:
            o.set_param(pname, m.get_param(pname))
    m.synchronize()
    m.close()


def test_bf16_model_at_config2_widths_vs_oracle(pkg, oracle):
    """d_model 512, 8 x 64 heads, d_ff 2048, vocab 16384, seg 64, mem 64, two layers, four streams:
    the register-resident norm kernels at D = 512, the row-in-registers softmax at V = 16384, the
    vector activation kernels at F = 2048, the split-K head and the wide GEMM tiles, assembled."""
    kw = dict(n_layer=2, d_model=512, n_head=8, d_key=64, d_inner=2048, d_pos=128, mem_len=64, seg_len=64,
              n_streams=4, n_symbols=16384, lr=3e-4)
    _bf16_vs_oracle(pkg, oracle, kw, 2, 2002, 0.044)


def test_bf16_model_at_config3_widths_vs_oracle(pkg, oracle):
    kw = dict(n_layer=1, d_model=1024, n_head=16, d_key=64, d_inner=4096, d_pos=320, mem_len=256, seg_len=64,
              n_streams=2, n_symbols=16384, lr=3e-4)
    _bf16_vs_oracle(pkg, oracle, kw, 2, 2003, 0.031)


@pytest.mark.parametrize("n_layer", [2])
def test_config4_one_symbol_steps_equal_whole_segment_bitwise(pkg, n_layer):
    """BASELINE config[4] geometry (the decoder's one-symbol step): memory 512, 128 streams, d_model
    512, 8 x 64 heads, vocab 16384, bf16.  After one train step (so that the memory is not zero) every
    one-symbol step reproduces the whole-segment rows bit for bit, and so does the train step after."""
    kw = dict(n_layer=n_layer, d_model=512, n_head=8, d_key=64, d_inner=2048, d_pos=576, mem_len=512,
              seg_len=64, n_streams=128, n_symbols=16384, use_bf16=1, init_range=0.03)
    a, b = pkg.TrfModel(pkg.abi.make_params(**kw)), pkg.TrfModel(pkg.abi.make_params(**kw))
    rng = np.random.default_rng(4)
    T, B, V = 64, 128, 16384
    for m in (a, b):
        m.reset()
    for s in range(2):
        ids = rng.integers(0, V, (T, B)).astype(np.int32)
        tg = rng.integers(0, V, (T, B)).astype(np.int32)
        full = a.eval(-1, ids)
        for t in range(T):
            step = b.eval(t, ids)
            assert np.array_equal(step[0], full[t]), (s, t)
        assert a.eval_gradient(tg) == b.eval_gradient(tg)
        a.update(); b.update()
        assert a.weights_hash() == b.weights_hash()
    a.close(); b.close()
