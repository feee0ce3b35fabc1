"""The reference's own command-line compressor (nncp.c, unmodified, built by
nncp-metal_b200/host/dropin/Makefile with its Transformer class re-pointed at libnncu.so) on the GPU: compress and
decompress round-trip through the reference's encode_file / decode_file / process_block, and
the file it writes is byte-identical to what this repository's host code (nch_compress, the
restatement of those functions) writes for the same parameters."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT

BIN = os.path.join(ROOT, "nncp-metal_b200", "host", "dropin", "_build", "nncp_b200")
OPTS = ["--cuda", "-q", "--n_layer", "2", "--d_model", "64", "--n_head", "2", "--d_inner", "128",
        "--batch_size", "4", "--train_len", "16", "--mem_len", "16", "--d_pos", "16"]


def _text(n, seed):
    rng = np.random.default_rng(seed)
    words = [bytes(rng.integers(97, 123, rng.integers(2, 8)).astype(np.uint8)) for _ in range(60)]
    out = b" ".join(words[i] for i in rng.integers(0, 60, n // 4))
    return out[:n]


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BIN), reason="host/dropin/_build/nncp_b200 was never built")
@pytest.mark.parametrize("bf16", [0, 1])
def test_reference_cli_round_trip_and_same_file_as_host_code(pkg, tmp_path, bf16):
    data = _text(6000, 3)
    src, cmp_, back = tmp_path / "in.bin", tmp_path / "out.nncp", tmp_path / "back.bin"
    src.write_bytes(data)
    opts = OPTS + (["--bf16", "1"] if bf16 else [])
    r = subprocess.run([BIN] + opts + ["c", str(src), str(cmp_)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([BIN, "-q", "--cuda", "d", str(cmp_), str(back)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert back.read_bytes() == data
    blob = cmp_.read_bytes()
    assert len(blob) < 0.8 * len(data)
    # the same parameters through this repository's host code
    p = pkg.abi.make_params(n_layer=2, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=16,
                            seg_len=16, n_streams=4, n_symbols=256, use_bias=1, use_w_r=1, tied_w_r=1,
                            tied_b_r=1, query_bias=0, ln_flags=1, ff_act=1, init_range=1.0, init_kind=0,
                            seed=123, beta2=0.9999, eps=1e-8, gradient_clip=0.1, lr=3e-4, use_bf16=bf16)
    fp = pkg.host.file_params(p, lr=pkg.host.InterpParams.make([3e-4, 1e-4], [156250]), block_len=500000)
    ops = pkg.host.bind_cuda(p)
    mine, _ = pkg.host.compress(ops, fp, np.frombuffer(data, np.uint8).astype(np.uint16), pkg.host.EVAL_SEGMENT,
                                pkg.host.OUT_CODER_READY)
    pkg.host.unbind_cuda(ops)
    assert mine == blob


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BIN), reason="host/dropin/_build/nncp_b200 was never built")
def test_reference_cli_with_its_tokenizer_round_trips(tmp_path):
    """--preprocess: the reference's own word tokenizer (preprocess.c, compiled unmodified into the
    drop-in) turns the text into 16-bit symbols of a dictionary it builds, the container carries the
    dictionary (nncp.c:3357-3413), and the B200 model codes an alphabet that is neither 256 nor a
    power of two ((n_words + 7) & ~7 symbols, nncp.c:3382)."""
    data = _text(30000, 5)
    src, cmp_, back = tmp_path / "in.txt", tmp_path / "out.nncp", tmp_path / "back.txt"
    src.write_bytes(data)
    opts = OPTS + ["--preprocess", "300,2"]
    r = subprocess.run([BIN] + opts + ["c", str(src), str(cmp_)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([BIN, "-q", "--cuda", "d", str(cmp_), str(back)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert back.read_bytes() == data
    assert cmp_.stat().st_size < 0.5 * len(data)


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BIN), reason="host/dropin/_build/nncp_b200 was never built")
def test_host_code_tokenizer_writes_and_reads_the_reference_cli_file(pkg, tmp_path):
    """The repository's own tokenizer and container (nch_words_encode, the dictionary in the header)
    against the reference CLI with --preprocess: the same file byte for byte, and each side decodes
    the other's file back to the text."""
    H = pkg.host
    data = _text(12000, 7)
    src, cmp_, back = tmp_path / "in.txt", tmp_path / "out.nncp", tmp_path / "back.txt"
    src.write_bytes(data)
    r = subprocess.run([BIN] + OPTS + ["--preprocess", "300,2", "c", str(src), str(cmp_)], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    blob = cmp_.read_bytes()

    d, syms, n_entries = H.words_encode(data, 300, 2)
    assert H.read_dict(blob) == d
    p = pkg.abi.make_params(n_layer=2, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=16,
                            seg_len=16, n_streams=4, n_symbols=H.alphabet_size(n_entries), use_bias=1, use_w_r=1,
                            tied_w_r=1, tied_b_r=1, query_bias=0, ln_flags=1, ff_act=1, init_range=1.0,
                            init_kind=0, seed=123, beta2=0.9999, eps=1e-8, gradient_clip=0.1, lr=3e-4)
    fp = H.file_params(p, lr=H.InterpParams.make([3e-4, 1e-4], [156250]), block_len=500000, dictionary=d)
    ops = H.bind_cuda(p)
    mine, _ = H.compress(ops, fp, syms, H.EVAL_SEGMENT, H.OUT_CODER_READY)
    H.unbind_cuda(ops)
    assert mine == blob
    # the reference CLI decodes the file of the host code (the same bytes, written by this side) ...
    (tmp_path / "mine.nncp").write_bytes(mine)
    r = subprocess.run([BIN, "-q", "--cuda", "d", str(tmp_path / "mine.nncp"), str(back)], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert back.read_bytes() == data
    # ... and the host code decodes the CLI's
    fp2, _, _ = H.read_header(blob)
    ops = H.bind_cuda(fp2.model)
    out = H.decompress(ops, blob, H.OUT_CODER_READY)
    H.unbind_cuda(ops)
    assert H.words_decode(H.read_dict(blob), out) == data


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BIN), reason="host/dropin/_build/nncp_b200 was never built")
def test_reference_cli_retrain_without_dropout_round_trips(tmp_path):
    """--retrain_period / --retrain_len: the reference's retrain_block (nncp.c:2821-2941, host code
    compiled unmodified into the drop-in) re-trains the model on the symbols already coded, on both
    sides; the file must still round-trip, must differ from the file coded without retraining, and
    retraining with dropout is refused."""
    data = _text(40000, 9)
    src, plain, cmp_, back = tmp_path / "in.bin", tmp_path / "plain.nncp", tmp_path / "out.nncp", tmp_path / "back.bin"
    src.write_bytes(data)
    small = OPTS + ["--block_len", "8192"]
    r = subprocess.run([BIN] + small + ["c", str(src), str(plain)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    opts = small + ["--retrain_period", "8192", "--retrain_len", "16384", "--retrain_dropout", "0", "--retrain_dropout_att", "0"]
    r = subprocess.run([BIN] + opts + ["c", str(src), str(cmp_)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([BIN, "-q", "--cuda", "d", str(cmp_), str(back)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert back.read_bytes() == data
    assert cmp_.read_bytes()[64:] != plain.read_bytes()[64:]
    bad = small + ["--retrain_period", "8192", "--retrain_len", "16384", "--retrain_dropout", "0.1"]
    r = subprocess.run([BIN] + bad + ["c", str(src), str(tmp_path / "x")], capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "dropout" in (r.stdout + r.stderr)


@pytest.mark.skipif(not os.path.exists(BIN), reason="host/dropin/_build/nncp_b200 was never built")
def test_reference_cli_fails_loudly_without_a_gpu(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    src = tmp_path / "in.bin"
    src.write_bytes(b"hello world " * 50)
    r = subprocess.run([BIN] + OPTS + ["c", str(src), str(tmp_path / "o")], capture_output=True, text=True, timeout=60)
    assert r.returncode != 0 and "no CUDA device" in (r.stdout + r.stderr)
