"""The retrain pass between blocks (no dropout) through this repository's host code on the CUDA model:
the same file as the reference's own command line on the same library writes, and the host code decodes
it.  The pass itself is pinned on the CPU against the reference's code (tests/test_ref_cli_cpu.py)."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT

BIN = os.path.join(ROOT, "nncp-metal_b200", "host", "dropin", "_build", "nncp_b200")
OPTS = ["--cuda", "-q", "--n_layer", "2", "--d_model", "64", "--n_head", "2", "--d_inner", "128",
        "--batch_size", "4", "--train_len", "16", "--mem_len", "16", "--d_pos", "16"]


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BIN), reason="host/dropin/_build/nncp_b200 was never built")
def test_host_code_retrain_pass_writes_the_reference_cli_file(pkg, tmp_path):
    H = pkg.host
    rng = np.random.default_rng(13)
    words = [bytes(rng.integers(97, 123, rng.integers(2, 8)).astype(np.uint8)) for _ in range(40)]
    data = b" ".join(words[i] for i in rng.integers(0, 40, 400))[:1400]
    src, out = tmp_path / "in", tmp_path / "out"
    src.write_bytes(data)
    r = subprocess.run([BIN] + OPTS + ["--block_len", "400", "--retrain_period", "700", "--retrain_len", "1000",
                                       "--retrain_dropout", "0", "--retrain_dropout_att", "0", "c", str(src), str(out)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    blob = out.read_bytes()
    p = pkg.abi.make_params(n_layer=2, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=16,
                            seg_len=16, n_streams=4, n_symbols=256, use_bias=1, use_w_r=1, tied_w_r=1,
                            tied_b_r=1, query_bias=0, ln_flags=1, ff_act=1, init_range=1.0, init_kind=0,
                            seed=123, beta2=0.9999, eps=1e-8, gradient_clip=0.1, lr=3e-4)
    fp = H.file_params(p, lr=H.InterpParams.make([3e-4, 1e-4], [156250]), block_len=400, retrain_period=700,
                       retrain_len=1000)
    ops = H.bind_cuda(p)
    mine, _ = H.compress(ops, fp, np.frombuffer(data, np.uint8).astype(np.uint16), H.EVAL_SEGMENT, H.OUT_CODER_READY)
    H.unbind_cuda(ops)
    assert mine == blob
    fp2, _, _ = H.read_header(blob)
    ops = H.bind_cuda(fp2.model)
    back = H.decompress(ops, blob, H.OUT_DEVICE)     # a file with a retrain pass decodes through the host walk
    H.unbind_cuda(ops)
    assert back.astype(np.uint8).tobytes() == data
