"""The reference's own command-line compressor on the CPU: its unmodified nncp.c (encode_file,
decode_file, process_block, header, preprocessor) built by oracle/Makefile with the model plugin
adapter of the drop-in and the CPU oracle behind it (oracle/_ref/nncp_oracle).  This repository's
host code, driving the same oracle through the plugin table, must write the same files byte for
byte, and each side must decode the other's.  Skipped where oracle/_ref was never built (no
reference tree)."""
import subprocess

import numpy as np
import pytest

from conftest import ROOT  # noqa: F401
from oracle import oracle as orc
from test_host_code import _oracle_ops

EXE = orc.nncp_oracle()
pytestmark = pytest.mark.skipif(EXE is None, reason="oracle/_ref/nncp_oracle is not built (no reference tree)")

OPTS = ["--cuda", "-q", "--n_layer", "1", "--d_model", "32", "--n_head", "2", "--d_inner", "64",
        "--batch_size", "4", "--train_len", "16", "--mem_len", "16", "--d_pos", "16"]


def _params(pkg, **over):
    kw = dict(n_layer=1, d_model=32, n_head=2, d_key=16, d_inner=64, d_pos=16, mem_len=16, seg_len=16,
              n_streams=4, n_symbols=256, use_bias=1, use_w_r=1, tied_w_r=1, tied_b_r=1, query_bias=0,
              ln_flags=1, ff_act=1, init_range=1.0, init_kind=0, seed=123, beta2=0.9999, eps=1e-8,
              gradient_clip=0.1, lr=3e-4)
    kw.update(over)
    return pkg.abi.make_params(**kw)


def _text(n, seed):
    rng = np.random.default_rng(seed)
    words = [bytes(rng.integers(97, 123, rng.integers(2, 8)).astype(np.uint8)) for _ in range(40)]
    caps = [w.capitalize() if rng.random() < 0.2 else w for w in words]
    return b" ".join(caps[i] for i in rng.integers(0, 40, n // 4 + 2))[:n]


def _cli(args, timeout=300):
    r = subprocess.run([EXE] + args, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-1000:]


def _schedule(pkg):
    return pkg.host.InterpParams.make([3e-4, 1e-4], [156250])      # the default profile's (nncp.c:2505-2509)


@pytest.mark.parametrize("n,block_len", [(1500, 500000), (1111, 300), (3, 500000), (0, 500000)])
def test_same_file_as_the_reference_cli(pkg, tmp_path, n, block_len):
    """Bytes in, several blocks with ragged tails, an input shorter than one segment, an empty one."""
    H = pkg.host
    data = _text(n, 3)
    src, out, back = tmp_path / "in", tmp_path / "out", tmp_path / "back"
    src.write_bytes(data)
    _cli(OPTS + ["--block_len", str(block_len), "c", str(src), str(out)])
    blob = out.read_bytes()
    p = _params(pkg)
    fp = H.file_params(p, lr=_schedule(pkg), block_len=block_len)
    mine, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, np.frombuffer(data, np.uint8).astype(np.uint16),
                         H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert mine == blob
    # each side decodes the other's file (the same bytes, written by the other side)
    (tmp_path / "mine").write_bytes(mine)
    _cli(["-q", "--cuda", "d", str(tmp_path / "mine"), str(back)])
    assert back.read_bytes() == data
    fp2, n_sym, _ = H.read_header(blob)
    got = H.decompress(_oracle_ops(pkg, orc.OracleModel(fp2.model)), blob, H.OUT_FLOAT)
    assert n_sym == n == len(data) and got.astype(np.uint8).tobytes() == data


def test_same_file_with_the_word_preprocessor(pkg, tmp_path):
    """--preprocess: the reference tokenises with its preprocess.c and carries the dictionary; this
    side does both with host/words.c and the container code of host/stream.c."""
    H = pkg.host
    data = _text(4000, 5)
    src, out, back = tmp_path / "in.txt", tmp_path / "out", tmp_path / "back"
    src.write_bytes(data)
    _cli(OPTS + ["--preprocess", "300,2", "c", str(src), str(out)])
    blob = out.read_bytes()
    d, syms, entries = H.words_encode(data, 300, 2)
    assert H.read_dict(blob) == d
    p = _params(pkg, n_symbols=H.alphabet_size(entries))
    fp = H.file_params(p, lr=_schedule(pkg), block_len=500000, dictionary=d)
    mine, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert mine == blob
    (tmp_path / "mine").write_bytes(mine)
    _cli(["-q", "--cuda", "d", str(tmp_path / "mine"), str(back)])
    assert back.read_bytes() == data
    assert H.decompress_text(blob, bind=lambda q: _oracle_ops(pkg, orc.OracleModel(q)), unbind=lambda o: None) == data


@pytest.mark.parametrize("opts,over", [
    (["--ln_flags", "6", "--ff_act", "2"], dict(ln_flags=6, ff_act=2)),
    (["--tied_w_r", "0", "--tied_b_r", "0", "--query_bias", "1", "--use_bias", "0"],
     dict(tied_w_r=0, tied_b_r=0, query_bias=1, use_bias=0)),
    (["--use_w_r", "0", "--ff_act", "3", "--ln_flags", "9", "--embed_mult", "0.5", "--init_range", "0.7"],
     dict(use_w_r=0, ff_act=3, ln_flags=9, embed_mult=0.5, init_range=0.7)),
    (["--n_layer", "2", "--attn_len", "20,32", "--gradient_clip", "0.05", "--ff_act", "0", "--seed", "7"],
     dict(n_layer=2, attn_len=[20, 32], gradient_clip=0.05, ff_act=0, seed=7)),
])
def test_same_file_for_model_variants(pkg, tmp_path, opts, over):
    """Options of the reference's command line reach the header and the model the same way on both sides."""
    H = pkg.host
    data = _text(900, 9)
    src, out = tmp_path / "in", tmp_path / "out"
    src.write_bytes(data)
    _cli(OPTS + opts + ["c", str(src), str(out)])
    p = _params(pkg, **over)
    fp = H.file_params(p, lr=_schedule(pkg), block_len=500000)
    mine, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, np.frombuffer(data, np.uint8).astype(np.uint16),
                         H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert mine == out.read_bytes()


@pytest.mark.parametrize("own_schedule", [False, True])
def test_same_file_with_the_retrain_pass(pkg, tmp_path, own_schedule):
    """--retrain_period / --retrain_len (dropout 0): between blocks the reference resets the model and
    trains it again over a ring of the last symbols (retrain_block, nncp.c:2821-2941), with the coder's
    schedule and step counter or with the pass's own; host/stream.c restates that pass."""
    H = pkg.host
    data = _text(2600, 11)
    src, out, back = tmp_path / "in", tmp_path / "out", tmp_path / "back"
    src.write_bytes(data)
    opts = OPTS + ["--block_len", "400", "--retrain_period", "700", "--retrain_len", "1000", "--retrain_dropout", "0",
                   "--retrain_dropout_att", "0"] + (["--retrain_lr", "1e-3,5,2e-4"] if own_schedule else [])
    _cli(opts + ["c", str(src), str(out)])
    blob = out.read_bytes()
    p = _params(pkg)
    fp = H.file_params(p, lr=_schedule(pkg), block_len=400, retrain_period=700, retrain_len=1000,
                       retrain_lr=H.InterpParams.make([1e-3, 2e-4], [5]) if own_schedule else None)
    syms = np.frombuffer(data, np.uint8).astype(np.uint16)
    mine, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert mine == blob
    plain, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p)), H.file_params(p, lr=_schedule(pkg), block_len=400), syms,
                          H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert plain[len(H.header_bytes(H.file_params(p, lr=_schedule(pkg), block_len=400), syms.size)):] != \
        mine[len(H.header_bytes(fp, syms.size)):]                  # the pass did change the model
    (tmp_path / "mine").write_bytes(mine)
    _cli(["-q", "--cuda", "d", str(tmp_path / "mine"), str(back)])
    assert back.read_bytes() == data
    fp2, _, _ = H.read_header(blob)
    assert fp2.retrain_period == 700 and fp2.retrain_len == 1000 and bool(fp2.has_retrain_lr) == own_schedule
    got = H.decompress(_oracle_ops(pkg, orc.OracleModel(fp2.model)), blob, H.OUT_DEVICE)
    assert got.astype(np.uint8).tobytes() == data


def test_front_end_level_table_is_the_reference_default_profile(pkg, tmp_path):
    """nncpm_level_params (levels 4..6) claims the "default" profile of nncp.c:2471-2513: the reference CLI
    run with no model options at all must then write the header, and the file, that those parameters give."""
    import ctypes as C
    H = pkg.host
    data = _text(1500, 4)
    src, out = tmp_path / "in", tmp_path / "out"
    src.write_bytes(data)
    _cli(["--cuda", "-q", "c", str(src), str(out)])
    blob = out.read_bytes()
    L = H.library()
    L.nncpm_level_params.argtypes = [C.c_int, C.POINTER(H.FileParams)]
    fp = H.FileParams()
    assert L.nncpm_level_params(5, C.byref(fp)) == 0
    hdr = H.header_bytes(fp, len(data))
    assert blob[:len(hdr)] == hdr
    mine, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(fp.model)), fp, np.frombuffer(data, np.uint8).astype(np.uint16),
                         H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert mine == blob
