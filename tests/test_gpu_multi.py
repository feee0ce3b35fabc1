"""Two ranks on two GPUs (skipped where fewer are visible): the in-library NCCL communicator leaves
identical weights on both, and the sharded codec round-trips a file whose header names the rank count.

NVLS is off (NCCL_NVLS_ENABLE=0): a rank that dies in a test must not leave its memory bound to an
NVLS group of the switch."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_package

pytestmark = pytest.mark.gpu

KW = dict(n_layer=2, d_model=256, n_head=4, d_key=64, d_inner=512, d_pos=64, mem_len=32, seg_len=32,
          n_symbols=1024, use_bf16=1, lr=1e-3, init_range=0.03, use_bias=1, use_w_r=1, query_bias=1, ln_flags=1,
          ff_act=1)
B_TOTAL = 8


def _source(n, V):
    rng = np.random.default_rng(17)
    nxt = rng.integers(0, V, size=(V, 2))
    out, s = np.empty(n, np.uint16), 0
    for i in range(n):
        s = nxt[s, rng.integers(0, 2)] if rng.random() < 0.9 else rng.integers(0, V)
        out[i] = s
    return out


def _worker(rank, world, port, out_dir, shard):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NNCU_SHARDED_UPDATE=shard)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pkg = load_package()
    lib = pkg.library()
    p = pkg.abi.make_params(n_streams=B_TOTAL // world, n_streams_total=B_TOTAL, device=rank, **KW)

    def model():
        m = pkg.TrfModel(p)
        pkg.dist.attach_library_comm(m, lib, rank, world, torch.device("cuda", rank))
        return m, pkg.dist.ShardedStep(m, None, world=world)

    # (1) three train steps on different data per rank: the same weights everywhere afterwards
    m, step = model()
    rng = np.random.default_rng(100 + rank)
    m.reset()
    for s in range(3):
        ids = rng.integers(0, KW["n_symbols"], (KW["seg_len"], p.n_streams)).astype(np.int32)
        tg = rng.integers(0, KW["n_symbols"], (KW["seg_len"], p.n_streams)).astype(np.int32)
        step.step_host(ids, tg)
    h = m.weights_hash()
    hs = [None] * world
    dist.all_gather_object(hs, h)
    m.close()
    # (1b) the fused step (reduce-scatter, update of the own shard, all-gather; embedding gradient from
    # gathered ids and rows) against all-reduce + whole update on the same data.  With two ranks every sum
    # of the matrices' gradients is one addition either way, so after one step they agree bit for bit.
    out = {}
    for fused in (False, True):
        m, step = model()
        rng = np.random.default_rng(100 + rank)
        ids = rng.integers(0, KW["n_symbols"], (KW["seg_len"], p.n_streams)).astype(np.int32)
        tg = rng.integers(0, KW["n_symbols"], (KW["seg_len"], p.n_streams)).astype(np.int32)
        m.reset()
        m.set_lr(1e-3)
        if fused:
            for s in range(3):
                m.eval(-1, ids, read=False)
                m.eval_gradient_update(tg)
                m.memory_shift()
                if s == 0:
                    if shard == "1":
                        with pytest.raises(RuntimeError):  # sharded state: single-rank reads are refused
                            m.get_param("ff1_0")
                    m.gather_master()
                    out[fused] = {k: m.get_param(k) for k in ("ff1_0", "w_q_1", "embed_out", "embed", "ln_g_0", "b_q_1")}
        else:
            step.step_host(ids, tg)
            out[fused] = {k: m.get_param(k) for k in ("ff1_0", "w_q_1", "embed_out", "embed", "ln_g_0", "b_q_1")}
        hf = m.weights_hash()
        m.close()
    hs_f = [None] * world
    dist.all_gather_object(hs_f, hf)
    same_matrices = all(np.array_equal(out[True][k], out[False][k]) for k in ("ff1_0", "w_q_1", "embed_out", "ln_g_0", "b_q_1"))
    d = np.abs(out[True]["embed"] - out[False]["embed"])
    embed_close = bool((d > 1e-6).mean() < 1e-3)   # rows a symbol hits on both ranks are summed in another order
    # (2) one file coded and decoded by the two ranks together
    syms = _source(1500, KW["n_symbols"])
    m, step = model()
    codec = pkg.dist.ShardedCodec(pkg.host, m, p, step, device=f"cuda:{rank}")
    data = codec.compress(pkg.host.file_params(p, block_len=768), syms)
    box = [data]
    dist.broadcast_object_list(box, src=0)
    m.close()
    m, step = model()
    codec = pkg.dist.ShardedCodec(pkg.host, m, p, step, device=f"cuda:{rank}")
    back = codec.decompress(box[0])
    m.close()
    if rank == 0:
        np.savez(os.path.join(out_dir, "multi.npz"), hashes=np.array(hs, np.uint64), hashes_fused=np.array(hs_f, np.uint64),
                 same_matrices=same_matrices, embed_close=embed_close,
                 data=np.frombuffer(box[0], np.uint8), back=back)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("shard", ["0", "1"])
def test_two_gpus_identical_weights_and_sharded_round_trip(tmp_path, pkg, shard):
    """shard "1": the fused step with NNCU_SHARDED_UPDATE=1 (reduce-scatter, update of the own shard,
    all-gather, embedding gradient from gathered rows); "0": the default all-reduce per layer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 32500 + os.getpid() % 2000 + int(shard)
    mp.spawn(_worker, args=(2, port, str(tmp_path), shard), nprocs=2, join=True)
    z = np.load(tmp_path / "multi.npz")
    assert z["hashes"][0] == z["hashes"][1]
    assert z["hashes_fused"][0] == z["hashes_fused"][1]
    assert bool(z["same_matrices"]) and bool(z["embed_close"])
    data = z["data"].tobytes()
    fp, n, _ = pkg.host.read_header(data)
    assert fp.n_ranks == 2 and fp.model.n_streams == B_TOTAL and n == 1500
    assert np.array_equal(z["back"], _source(1500, KW["n_symbols"]))
    assert len(data) < 1500 * 10 // 8          # 10 bits per symbol raw
    # one process refuses the two-rank file
    p1 = pkg.abi.make_params(n_streams=B_TOTAL, n_streams_total=B_TOTAL, **KW)
    ops = pkg.host.bind_cuda(p1)
    with pytest.raises(RuntimeError):
        pkg.host.decompress(ops, data, pkg.host.OUT_CODER_READY)
    pkg.host.unbind_cuda(ops)
