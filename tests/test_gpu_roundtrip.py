"""compress -> decompress through the host C code and the CUDA model: bit-exact round trips.

The encoder runs whole segments (one model_eval per segment, coder-ready prob0 paths from the
device); the decoder can only run one symbol per stream at a time (prob0 trees from the
device).  They agree because every forward row is bit-identical between the two modes."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _markov_source(n, V, seed):
    rng = np.random.default_rng(seed)
    nxt = rng.integers(0, V, size=(V, 3))
    out, s = np.empty(n, np.uint16), 0
    for i in range(n):
        s = nxt[s, rng.integers(0, 3)] if rng.random() < 0.9 else rng.integers(0, V)
        out[i] = s
    return out


CASES = {
    "fp32_bytes": (dict(n_layer=2, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=24, mem_len=16, seg_len=16,
                        n_streams=4, n_symbols=256, use_bf16=0, lr=2e-3, init_range=0.05), 1500, 640),
    "bf16_tcgen05_tokens": (dict(n_layer=2, d_model=256, n_head=4, d_key=64, d_inner=512, d_pos=64, mem_len=32,
                                 seg_len=32, n_streams=8, n_symbols=4096, use_bf16=1, lr=1e-3,
                                 init_range=0.03), 1800, 1024),
    "bf16_ragged_streams": (dict(n_layer=1, d_model=64, n_head=4, d_key=16, d_inner=128, d_pos=20, mem_len=24,
                                 seg_len=8, n_streams=3, n_symbols=64, use_bf16=1, lr=2e-3,
                                 init_range=0.05), 333, 100),
}


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("out_mode", [0, 1, 2])
def test_round_trip_is_bit_exact(pkg, name, out_mode):
    """out_mode 2: the range decoder runs on the device as well (nncu_decode_steps)."""
    kw, n, block_len = CASES[name]
    if out_mode == 0 and kw["n_symbols"] > 256:
        pytest.skip("float tables of 4096 symbols per position: covered by the coder-ready mode")
    p = pkg.abi.make_params(**kw)
    syms = _markov_source(n, kw["n_symbols"], 5)
    fp = pkg.host.file_params(p, block_len=block_len)
    enc = pkg.host.bind_cuda(p)
    data, st = pkg.host.compress(enc, fp, syms, pkg.host.EVAL_SEGMENT, out_mode)
    pkg.host.unbind_cuda(enc)
    assert st.n_symbols == n and st.train_steps > 0
    dec = pkg.host.bind_cuda(p)
    back = pkg.host.decompress(dec, data, out_mode)
    pkg.host.unbind_cuda(dec)
    assert np.array_equal(back, syms)


@pytest.mark.parametrize("V", [512, 296, 1000])
def test_device_decoder_steps_match_the_host_walk(pkg, V):
    """296, 1000: alphabets that are not a power of two (the uneven tree of write_sym).
    nncu_decode_steps against nch_read_sym_tree over nncu_coder_trees, step by step on two models
    with identical weights: the same symbols, and the same number of payload bytes consumed.  The
    payload is random bytes (any byte string decodes to something), the second call starts in the
    middle of a segment, and the last one has a ragged limit."""
    import ctypes as C
    kw = dict(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=24, mem_len=16, seg_len=8,
              n_streams=5, n_symbols=V, use_bf16=0, lr=2e-3, init_range=0.05)
    p = pkg.abi.make_params(**kw)
    T, B = 8, 5
    rng = np.random.default_rng(11)
    payload = rng.integers(0, 256, 4000, dtype=np.uint8).tobytes()
    L = pkg.host.library()
    dev, ref = pkg.TrfModel(p), pkg.TrfModel(p)
    for m in (dev, ref):
        m.reset()
    dev.decoder_begin(payload)
    buf = C.create_string_buffer(payload, len(payload))
    hd = L.nch_dec_new(buf, len(payload))
    ids0 = rng.integers(0, V, B).astype(np.int32)

    def host_steps(t0, nt, ids_first, limit_t, limit_b):
        out = np.zeros((nt, B), np.int32)
        ids = np.zeros((T, B), np.int32)
        for t in range(t0, t0 + nt):
            ids[t] = ids_first if t == t0 else out[t - t0 - 1]
            ref.eval(t, ids, read=False)
            trees = np.ascontiguousarray(ref.coder_trees(t, 1))
            for b in range(B):
                if t < limit_t or (t == limit_t and b < limit_b):
                    out[t - t0, b] = L.nch_read_sym_tree(hd, trees[b].ctypes.data_as(C.c_void_p), V)
        return out

    a = dev.decode_steps(0, 3, ids0)
    b = host_steps(0, 3, ids0, T, 0)
    assert np.array_equal(a, b)
    a2 = dev.decode_steps(3, 5)                      # continues from the symbols decoded at step 2
    b2 = host_steps(3, 5, b[-1], T, 0)
    assert np.array_equal(a2, b2)
    tg = np.concatenate([a, a2]).astype(np.int32)
    for m in (dev, ref):
        m.set_lr(2e-3)
        m.eval_gradient(tg)
        m.update()
    assert dev.weights_hash() == ref.weights_hash()
    a3 = dev.decode_steps(0, 4, a2[-1], limit_t=3, limit_b=2)   # a block tail: 3 full steps + 2 streams
    b3 = host_steps(0, 4, b2[-1], 3, 2)
    assert np.array_equal(a3, b3) and not a3[3, 2:].any()
    assert dev.decoder_end() > 0
    L.nch_dec_free(hd)
    dev.close()
    ref.close()


def test_device_decoder_graphs_survive_a_larger_second_payload(pkg):
    """On a non-default stream every decode step replays a CUDA graph that holds the payload buffer's
    address; a second, larger payload moves the buffer, so the graphs must be captured again.  Two
    files of different sizes decoded by one model, each compared with a model that decodes it eagerly."""
    import torch
    kw = dict(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=24, mem_len=16, seg_len=8,
              n_streams=4, n_symbols=256, use_bf16=0, lr=2e-3, init_range=0.05)
    p = pkg.abi.make_params(**kw)
    T, B = 8, 4
    rng = np.random.default_rng(21)
    m, ref = pkg.TrfModel(p), pkg.TrfModel(p)      # both see both payloads, so their weights stay equal
    st = torch.cuda.Stream()
    m.set_stream(st.cuda_stream)
    for n_bytes in (300, 5000):
        payload = rng.integers(0, 256, n_bytes, dtype=np.uint8).tobytes()
        outs = []
        for mod in (m, ref):
            mod.reset()
            mod.decoder_begin(payload)
            ids0, segs = np.zeros(B, np.int32), []
            for _seg in range(4):                      # graphs are captured on the second use of a memory twin
                sy = mod.decode_steps(0, T, ids0)
                mod.set_lr(2e-3)
                mod.eval_gradient(sy)
                mod.update()
                ids0 = sy[-1]
                segs.append(sy)
            outs.append((np.stack(segs), mod.decoder_end()))
        assert np.array_equal(outs[0][0], outs[1][0]) and outs[0][1] == outs[1][1]
    assert m.weights_hash() == ref.weights_hash()
    m.close()
    ref.close()


@pytest.mark.parametrize("V", [256, 296])
def test_coder_ready_and_float_output_give_the_same_file(pkg, V):
    """296: an alphabet that is not a power of two (a word dictionary's), coded from the integer
    paths and trees of the uneven tree; out_mode 2 walks that tree in the device decoder."""
    kw, n, block_len = CASES["fp32_bytes"]
    p = pkg.abi.make_params(**dict(kw, n_symbols=V))
    syms = _markov_source(700, V, 6)
    fp = pkg.host.file_params(p, block_len=block_len)
    outs = []
    for eval_mode, out_mode in ((1, 1), (1, 0), (0, 1)):
        ops = pkg.host.bind_cuda(p)
        outs.append(pkg.host.compress(ops, fp, syms, eval_mode, out_mode)[0])
        pkg.host.unbind_cuda(ops)
    assert outs[0] == outs[1] == outs[2]
    for out_mode in (1, 2):
        ops = pkg.host.bind_cuda(p)
        back = pkg.host.decompress(ops, outs[0], out_mode)
        pkg.host.unbind_cuda(ops)
        assert np.array_equal(back, syms)


def test_model_learns_the_source(pkg):
    kw, _, _ = CASES["fp32_bytes"]
    p = pkg.abi.make_params(**kw)
    syms = _markov_source(6000, 256, 8)
    fp = pkg.host.file_params(p)
    ops = pkg.host.bind_cuda(p)
    data, st = pkg.host.compress(ops, fp, syms, 1, 1)
    pkg.host.unbind_cuda(ops)
    assert len(data) < 0.8 * len(syms)     # raw: 1 byte per symbol
