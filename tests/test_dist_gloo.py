"""Stream sharding over 2 ranks on the CPU (gloo): each rank trains its half of the streams with
the CPU oracle as the model, gradients are all-reduced, and both ranks must end with the same
weights as a single process that trains all streams."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_golden, load_package, params_from_cfg, rel_err

STEPS = 3


def _data(cfg, B):
    rng = np.random.default_rng(0)
    T, V = cfg["seg_len"], cfg["n_symbols"]
    return (rng.integers(0, V, (STEPS, T, B)).astype(np.int32),
            rng.integers(0, V, (STEPS, T, B)).astype(np.int32))


def _run(pkg, orc, cfg, z, ids, tg, rank, world, B_total):
    sl = pkg.dist.stream_slice(rank, world, B_total)
    p = params_from_cfg(pkg, cfg, n_streams=B_total // world, n_streams_total=B_total)
    m = orc.OracleModel(p)
    for name in m.info:
        m.set_param(name, z[f"p0/{name}"])
    m.reset()
    grads = torch.from_numpy(np.ctypeslib.as_array(m.L.orc_grads(m.h), shape=(m.n_floats,)))
    step = pkg.dist.ShardedStep(m, grads, world=world)
    losses = [step.step_host(np.ascontiguousarray(ids[s][:, sl]), np.ascontiguousarray(tg[s][:, sl]))
              for s in range(STEPS)]
    return m, losses


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_package()
    from oracle import oracle as orc
    cfg, z = load_golden("c0_like")
    ids, tg = _data(cfg, 4)
    m, losses = _run(pkg, orc, cfg, z, ids, tg, rank, world, 4)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), loss=np.array(losses),
             **{k: m.get_param(k) for k in m.info})
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_process(tmp_path, pkg, oracle):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    cfg, z = load_golden("c0_like")
    ids, tg = _data(cfg, 4)
    single, losses = _run(pkg, oracle, cfg, z, ids, tg, 0, 1, 4)
    for k in single.info:
        assert np.array_equal(r0[k], r1[k]), k            # ranks hold identical weights
        assert rel_err(r0[k], single.get_param(k)) < 2e-3, k   # and follow the 1-process run
    assert abs((r0["loss"] + r1["loss"]).sum() - np.sum(losses)) < 1e-3 * abs(np.sum(losses))


def test_stream_slice_partitions_the_streams(pkg):
    for world in (1, 2, 4, 8):
        cols = []
        for r in range(world):
            s = pkg.dist.stream_slice(r, world, 32)
            cols += list(range(32))[s]
        assert cols == list(range(32))
    with pytest.raises(ValueError):
        pkg.dist.stream_slice(0, 3, 32)


# ---- the coder side of a sharded job: paths / tables to rank 0 when encoding, symbols back when decoding

def _codec_source(n):
    rng = np.random.default_rng(3)
    return np.array([(5 * i) % 7 if rng.random() < 0.8 else rng.integers(0, 16) for i in range(n)], np.uint16)


def _codec(pkg, orc, cfg, z, rank, world, B_total):
    p = params_from_cfg(pkg, cfg, n_streams=B_total // world, n_streams_total=B_total, lr=1e-2)
    m = orc.OracleModel(p)
    for name in m.info:
        m.set_param(name, z[f"p0/{name}"])
    grads = torch.from_numpy(np.ctypeslib.as_array(m.L.orc_grads(m.h), shape=(m.n_floats,)))
    step = pkg.dist.ShardedStep(m, grads, world=world)
    return pkg.dist.ShardedCodec(pkg.host, m, p, step), p


def _codec_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_package()
    from oracle import oracle as orc
    cfg, z = load_golden("post_gelu")
    syms = _codec_source(301)
    enc, p = _codec(pkg, orc, cfg, z, rank, world, 4)
    data = enc.compress(pkg.host.file_params(p, block_len=96), syms)
    box = [data]
    dist.broadcast_object_list(box, src=0)        # every rank decodes the same file
    dec, _ = _codec(pkg, orc, cfg, z, rank, world, 4)
    back = dec.decompress(box[0])
    if rank == 0:
        np.savez(os.path.join(out_dir, "codec.npz"), data=np.frombuffer(data, np.uint8), back=back)
    else:
        assert data is None and np.array_equal(back, syms)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_codec_round_trip_and_rank_count_in_header(tmp_path, pkg, oracle):
    """Two ranks code one file between them (ragged blocks, several blocks, training in between) and
    decode it again; the header says 2 ranks, and neither the single-process decoder nor a
    one-rank codec accepts the file."""
    port = 31500 + os.getpid() % 2000
    mp.spawn(_codec_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    zf = np.load(tmp_path / "codec.npz")
    data, syms = zf["data"].tobytes(), _codec_source(301)
    assert np.array_equal(zf["back"], syms)
    fp, n, used = pkg.host.read_header(data)
    assert data[4:6] == b"\x00\x03" and fp.n_ranks == 2 and fp.model.n_streams == 4 and n == 301
    cfg, z = load_golden("post_gelu")
    one, p1 = _codec(pkg, oracle, cfg, z, 0, 1, 4)
    with pytest.raises(ValueError):
        one.decompress(data)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_host_code import _oracle_ops
    with pytest.raises(RuntimeError):
        pkg.host.decompress(_oracle_ops(pkg, oracle.OracleModel(p1)), data, pkg.host.OUT_FLOAT)


def test_one_rank_codec_writes_the_single_process_file(pkg, oracle):
    """With one rank the sharded block walk must produce the bytes of nch_compress."""
    from test_host_code import _oracle_ops
    cfg, z = load_golden("post_gelu")
    syms = _codec_source(230)
    codec, p = _codec(pkg, oracle, cfg, z, 0, 1, 4)
    a = codec.compress(pkg.host.file_params(p, block_len=96), syms)
    m = oracle.OracleModel(p)
    for name in m.info:
        m.set_param(name, z[f"p0/{name}"])
    b, _ = pkg.host.compress(_oracle_ops(pkg, m), pkg.host.file_params(p, block_len=96), syms,
                             pkg.host.EVAL_SEGMENT, pkg.host.OUT_FLOAT)
    assert a == b and a[4:6] != b"\x00\x03"      # no rank count in a one-process file
    codec2, _ = _codec(pkg, oracle, cfg, z, 0, 1, 4)
    assert np.array_equal(codec2.decompress(a), syms)


# ---- tokenised text through a sharded job: the dictionary rides in the header beside the rank count

_TEXT = (b"the cat sat on the mat. The dog sat on the log; the cat and the dog sat. " * 12)[:700]


class _ReadyModel:
    """The CPU oracle with the two coder-ready calls a CUDA model offers (prob0 paths and trees made
    from its tables by the coder oracle), so that the codec's integer exchange runs on the CPU."""

    def __init__(self, orc, p):
        self._o, self._orc = orc.OracleModel(p), orc
        self._depth = int(np.ceil(np.log2(p.n_symbols)))

    def __getattr__(self, name):
        return getattr(self._o, name)

    def eval(self, output_index, ids, read=True):
        self._pr = self._o.eval(output_index, ids)      # [T or 1][B][V]
        return self._pr if read else None

    def coder_paths(self, t0, nt, syms):
        out = np.zeros((nt * self._o.B, self._depth), np.uint16)
        for t in range(nt):
            for b in range(self._o.B):
                q = self._orc.sym_path(self._pr[t0 + t, b], int(syms[t, b]))
                out[t * self._o.B + b, :len(q)] = q
        return out

    def coder_trees(self, t, nt):
        assert nt == 1 and self._pr.shape[0] == 1
        return np.stack([self._orc.sym_tree(self._pr[0, b]) for b in range(self._o.B)])


def _text_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_package()
    from oracle import oracle as orc
    H = pkg.host
    d, syms, entries = H.words_encode(_TEXT, 280, 2)
    cfg, z = load_golden("post_gelu")

    def codec(ready):
        p = params_from_cfg(pkg, cfg, n_streams=2, n_streams_total=4, lr=1e-2, n_symbols=H.alphabet_size(entries))
        m = _ReadyModel(orc, p) if ready else orc.OracleModel(p)
        grads = torch.from_numpy(np.ctypeslib.as_array(m.L.orc_grads(m.h), shape=(m.n_floats,)))
        c = pkg.dist.ShardedCodec(H, m, p, pkg.dist.ShardedStep(m, grads, world=world))
        assert c.ready == ready
        return c, p

    enc, p = codec(False)
    data = enc.compress(H.file_params(p, block_len=96, dictionary=d), syms)
    # the same job exchanging integer paths instead of float tables (an alphabet that is not a power of two)
    enc2, _ = codec(True)
    data2 = enc2.compress(H.file_params(p, block_len=96, dictionary=d), syms)
    assert data2 == data
    box = [data]
    dist.broadcast_object_list(box, src=0)
    dec, _ = codec(True)                              # decodes from integer trees
    back = dec.decompress(box[0])
    fp, n, _ = H.read_header(box[0])
    assert fp.n_ranks == 2 and fp.dict_len == len(d) and n == syms.size
    assert H.words_decode(H.read_dict(box[0]), back) == _TEXT
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_codec_carries_the_dictionary(tmp_path, pkg, oracle):
    port = 33500 + os.getpid() % 2000
    mp.spawn(_text_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
