"""The C oracle against the committed golden vectors (PyTorch float64 autograd restatement).

Tolerances: the oracle computes in fp32; the golden values are float64 results rounded to
fp32, so 2e-4 relative (max-abs-diff over max-abs-ref) covers fp32 accumulation noise.
"""
import numpy as np
import pytest

from conftest import (DIGEST_NAMES, GOLDEN_NAMES, check_digest_step, check_updated_weights, load_digest,
                      load_golden, params_from_cfg, rel_err)

TOL = 2e-4


def _load_params(model, z, step):
    for name in model.info:
        model.set_param(name, z[f"p{step}/{name}"])


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_two_steps(pkg, oracle, name):
    cfg, z = load_golden(name)
    p = params_from_cfg(pkg, cfg)
    m = oracle.OracleModel(p)
    assert set(m.info) == {k[3:] for k in z.files if k.startswith("p0/")}
    _load_params(m, z, 0)
    m.reset()
    m.set_lr(cfg["lr"])
    for s in range(z["ids"].shape[0]):
        probs = m.eval(-1, z["ids"][s])
        assert rel_err(probs, z["probs"][s]) < TOL
        loss = m.eval_gradient(z["targets"][s])
        assert abs(loss - z["loss"][s]) < TOL * abs(z["loss"][s])
        for pname in m.info:
            g_ref = z[f"g{s}/{pname}"]
            scale = max(np.abs(g_ref).max(), 1e-6)
            err = np.abs(m.get_grad(pname) - g_ref.reshape(-1)).max() / scale
            assert err < 5e-4, (pname, s, err)
        before = {pname: m.get_param(pname) for pname in m.info}
        m.update()
        for l in range(cfg["n_layer"]):
            assert rel_err(m.mem(l), z[f"mem{s+1}"][l]) < TOL, ("mem", l)
        for pname in m.info:
            check_updated_weights(m.get_param(pname), z[f"p{s+1}/{pname}"].reshape(-1), before[pname],
                                  z[f"g{s}/{pname}"].reshape(-1), TOL, cfg["lr"], cfg["beta2"], (pname, s))
        # continue from the golden weights so that step 2 is checked in isolation
        # from step-1 rounding differences
        for pname in m.info:
            m.set_param(pname, z[f"p{s+1}/{pname}"])
    m.close()


@pytest.mark.parametrize("name", DIGEST_NAMES)
def test_oracle_at_baseline_geometries(pkg, oracle, name):
    """BASELINE config[0] exactly and config[2]'s widths (d_model 512, 8 x 64 heads, d_ff 2048,
    vocab 16384, seg 64, mem 64): the oracle against float64 digests of the PyTorch restatement.
    The second step continues from the oracle's own updated weights, so it also checks the update."""
    cfg, z, params = load_digest(name)
    m = oracle.OracleModel(params_from_cfg(pkg, cfg))
    for pname in m.info:
        m.set_param(pname, params[pname])
    m.reset()
    m.set_lr(cfg["lr"])
    for s in range(z["ids"].shape[0]):
        probs = m.eval(-1, z["ids"][s])
        loss = m.eval_gradient(z["targets"][s])
        # step 2 starts from fp32 weights whose least-determined elements moved by one RMSProp
        # step of either sign: twice the tolerance there
        k = 1 if s == 0 else 2
        check_digest_step(m, z, s, k * TOL, k * 5e-4, probs, loss)
        m.update()
        for pname in m.info:
            stride = int(z[f"stride/{pname}"])
            w, w_ref = m.get_param(pname)[::stride], z[f"p{s+1}/{pname}"]
            bound = k * TOL * max(np.abs(w_ref).max(), 1e-3) + 2.1 * cfg["lr"] / np.sqrt(1 - cfg["beta2"])
            assert np.abs(w - w_ref).max() < bound, (pname, s)
    m.close()


@pytest.mark.parametrize("name", ["post_gelu", "pre_final_geglu_rms", "short_mem_window"])
def test_oracle_incremental_equals_batched(pkg, oracle, name):
    cfg, z = load_golden(name)
    p = params_from_cfg(pkg, cfg)
    a, b = oracle.OracleModel(p), oracle.OracleModel(p)
    for m in (a, b):
        _load_params(m, z, 0)
        m.reset()
    ids = z["ids"][0]
    full = a.eval(-1, ids)
    for t in range(cfg["seg_len"]):
        step = b.eval(t, ids)
        np.testing.assert_array_equal(step[0], full[t])
    la, lb = a.eval_gradient(z["targets"][0]), b.eval_gradient(z["targets"][0])
    assert la == lb
    for pname in a.info:
        np.testing.assert_array_equal(a.get_grad(pname), b.get_grad(pname))


def test_oracle_rejects_bad_options(pkg, oracle):
    cfg, _ = load_golden("post_gelu")
    for over in (dict(d_pos=100), dict(ln_flags=3), dict(ff_act=4),
                 dict(d_value=4), dict(n_layer=0)):
        with pytest.raises(ValueError):
            oracle.OracleModel(params_from_cfg(pkg, cfg, **over))
