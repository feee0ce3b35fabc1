import importlib.util
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """Imports the package directory `nncp-metal_b200/` under the name nncp_metal_b200."""
    name = "nncp_metal_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = os.path.join(ROOT, "nncp-metal_b200")
    spec = importlib.util.spec_from_file_location(
        name, os.path.join(pkg_dir, "__init__.py"), submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
GOLDEN_NAMES = sorted(f[4:-4] for f in os.listdir(GOLDEN_DIR)
                      if f.startswith("trf_") and f.endswith(".npz"))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, f"trf_{name}.npz"))
    cfg = json.loads(str(z["cfg_json"]))
    return cfg, z


DIGEST_NAMES = sorted(f[4:-4] for f in os.listdir(GOLDEN_DIR) if f.startswith("dig_") and f.endswith(".npz"))


def load_digest(name):
    """A digest golden (BASELINE geometries): configuration, the npz, and the seeded fp32
    parameters it was made from (rebuilt with the oracle's counter-based generator)."""
    sys.path.insert(0, GOLDEN_DIR)
    import seeded_params as sp
    import trf_torch as tt
    from oracle import oracle as orc
    z = np.load(os.path.join(GOLDEN_DIR, f"dig_{name}.npz"))
    cfg = json.loads(str(z["cfg_json"]))
    params = sp.seeded_params(orc, tt.param_shapes(cfg), cfg["param_seed"], cfg["wscale"])
    return cfg, z, params


def check_digest_step(model, z, s, tol, gtol, probs=None, loss=None):
    """Probabilities (sampled columns, target column, row maxima), loss and the strided subsample of
    every gradient of step `s` against a digest golden."""
    cols = z["prob_cols"]
    if probs is not None:
        T, B, _ = probs.shape
        scale = float(z["probs_rowmax"][s].max())
        assert np.abs(probs[..., cols] - z["probs_sample"][s]).max() / scale < tol
        tg = z["targets"][s]
        pt = np.take_along_axis(probs, tg[..., None].astype(np.int64), 2)[..., 0]
        assert np.abs(pt - z["probs_target"][s]).max() / scale < tol
        assert np.abs(probs.max(-1) - z["probs_rowmax"][s]).max() / scale < tol
    if loss is not None:
        assert abs(loss - z["loss"][s]) < tol * abs(z["loss"][s]), (loss, z["loss"][s])
    for pname in model.info:
        stride = int(z[f"stride/{pname}"])
        g = model.get_grad(pname)[::stride]
        scale = max(float(z[f"gmax{s}/{pname}"]), 1e-9)
        err = np.abs(g - z[f"g{s}/{pname}"]).max() / scale
        assert err < gtol, (pname, s, err)


def params_from_cfg(pkg, cfg, **over):
    keys = ["n_layer", "d_model", "n_head", "d_key", "d_value", "d_inner", "d_pos", "mem_len",
            "seg_len", "n_streams", "n_symbols", "use_bias", "use_w_r", "tied_w_r", "tied_b_r",
            "query_bias", "ln_flags", "ff_act", "embed_mult", "beta2", "eps", "lr",
            "gradient_clip"]
    kw = {k: cfg[k] for k in keys}
    kw["attn_len"] = cfg["attn_len"]
    kw.update(over)
    return pkg.abi.make_params(**kw)


def rel_err(a, b):
    """max |a-b| / max(|b|): the relative error every parity test in this suite uses."""
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    d = float(np.max(np.abs(a - b))) if a.size else 0.0
    s = float(np.max(np.abs(b))) if b.size else 0.0
    return d / max(s, 1e-30)


def check_updated_weights(w, w_ref, w_before, g_ref, tol, lr, beta2, what):
    """RMSProp moves a weight by lr*g/sqrt(v): at the first step that is +-lr/sqrt(1-beta2)
    whatever |g| is, so where the reference gradient is below the arithmetic noise its SIGN,
    and with it the whole update, is not determined.  The noise of a gradient element is about
    tol * max|g| (the bound the gradient comparison itself uses), so every element whose gradient
    is ten times above that must match within tol of the weights plus 10*tol of the update
    (lr*g/sqrt(v) amplifies gradient noise wherever v is small); only the elements below may
    differ by a full update each way.  The second moment has no sign to lose: it is checked
    indirectly through the size of the update (|w - w_before| against the reference's)."""
    scale = max(np.abs(w_ref).max(), 1e-3)
    upd = np.abs(w_ref - w_before).max(initial=0.0)
    sure = np.abs(g_ref) > 10 * tol * max(np.abs(g_ref).max(), 1e-12)
    d = np.abs(w - w_ref)
    assert d[sure].max(initial=0.0) < tol * scale + 10 * tol * upd, what
    assert d.max(initial=0.0) < tol * scale + 2.1 * lr / np.sqrt(1.0 - beta2), what


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    orc.lib()
    return orc
