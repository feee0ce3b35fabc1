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
    and with it the whole update, is not determined.  Elements with a clearly non-zero
    gradient must match within tol of the weights plus 10*tol of the update itself (the
    update lr*g/sqrt(v) amplifies gradient noise wherever v is small); the rest may differ by at most one full update each way."""
    scale = max(np.abs(w_ref).max(), 1e-3)
    upd = np.abs(w_ref - w_before).max(initial=0.0)
    sure = np.abs(g_ref) > 0.1 * max(np.abs(g_ref).max(), 1e-12)
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
