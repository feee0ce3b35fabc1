"""Host-side C code (libnncp_host.so) on the CPU: range coder and symbol coder against the
reference's own sources (oracle/_ref) and the oracle, schedule, stream layout, container
header, and the block loop driven by the CPU oracle as the model (test-only plumbing: the
shipped binding, nch_bind_cuda, only ever binds the CUDA library)."""
import ctypes as C
import struct

import numpy as np
import pytest

from conftest import load_golden, params_from_cfg
from oracle import oracle as orc

_vp = C.c_void_p
needs_ref = pytest.mark.skipif(orc.ref_lib() is None, reason="oracle/_ref was never built")


def _tables(rng, n, V, sharp):
    z = rng.standard_normal((n, V)).astype(np.float32) * sharp
    e = np.exp(z - z.max(1, keepdims=True))
    return (e / e.sum(1, keepdims=True)).astype(np.float32)


class HostEnc:
    def __init__(self, L):
        self.L, self.h = L, L.nch_enc_new()

    def put_sym(self, p, s):
        p = np.ascontiguousarray(p, np.float32)
        self.L.nch_write_sym(self.h, p.ctypes.data_as(_vp), p.size, int(s))

    def finish(self):
        out = _vp()
        n = self.L.nch_enc_finish(self.h, C.byref(out))
        data = C.string_at(out.value, n) if n else b""
        self.L.nch_enc_free(self.h)
        return data


@needs_ref
@pytest.mark.parametrize("V,sharp", [(2, 1.0), (256, 3.0), (24, 2.0), (1000, 5.0), (16384, 6.0)])
def test_host_coder_bytes_equal_reference(pkg, V, sharp):
    L = pkg.host.library()
    rng = np.random.default_rng(V + 1)
    n = 400 if V <= 1000 else 30
    probs = _tables(rng, n, V, sharp)
    syms = rng.integers(0, V, n)
    a, b = HostEnc(L), orc.Encoder(True)
    for p, s in zip(probs, syms):
        a.put_sym(p, s)
        b.put_sym(p, s)
    da = a.finish()
    assert da == b.finish() and len(da) > 0
    buf = C.create_string_buffer(da, len(da))
    d = L.nch_dec_new(buf, len(da))
    back = [L.nch_read_sym(d, np.ascontiguousarray(p).ctypes.data_as(_vp), V) for p in probs]
    L.nch_dec_free(d)
    assert back == list(syms)


@needs_ref
def test_host_coder_carry_runs_equal_reference(pkg):
    L = pkg.host.library()
    rng = np.random.default_rng(9)
    pr = rng.choice([1, 3, 16384, 32765, 32767], size=30000)
    bits = (rng.random(30000) < 0.5).astype(int)
    e, r = L.nch_enc_new(), orc.Encoder(True)
    for q, bit in zip(pr, bits):
        L.nch_enc_put_bit(e, int(q), int(bit))
        r.put_bit(q, bit)
    out = _vp()
    n = L.nch_enc_finish(e, C.byref(out))
    data = C.string_at(out.value, n)
    L.nch_enc_free(e)
    assert data == r.finish()
    buf = C.create_string_buffer(data, len(data))
    d = L.nch_dec_new(buf, len(data))
    assert [L.nch_dec_get_bit(d, int(q)) for q in pr] == list(bits)
    L.nch_dec_free(d)


def test_path_and_tree_coding_equal_table_coding(pkg):
    L = pkg.host.library()
    rng = np.random.default_rng(4)
    V, nb = 64, 6
    probs = _tables(rng, 100, V, 3.0)
    syms = rng.integers(0, V, 100)
    a, e = HostEnc(L), L.nch_enc_new()
    trees = []
    for p, s in zip(probs, syms):
        a.put_sym(p, s)
        path = orc.sym_path(p, s)
        L.nch_write_sym_path(e, path.ctypes.data_as(_vp), nb, int(s))
        tree = np.zeros(V, np.uint16)   # heap-ordered prob0 of every node, from the oracle's paths
        for leaf in range(V):
            pth, k = orc.sym_path(p, leaf), 1
            for lvl in range(nb):
                tree[k] = pth[lvl]
                k = 2 * k + ((leaf >> (nb - 1 - lvl)) & 1)
        trees.append(tree)
    out = _vp()
    n = L.nch_enc_finish(e, C.byref(out))
    data = C.string_at(out.value, n)
    L.nch_enc_free(e)
    assert data == a.finish()
    buf = C.create_string_buffer(data, len(data))
    d = L.nch_dec_new(buf, len(data))
    assert [L.nch_read_sym_tree(d, t.ctypes.data_as(_vp), V) for t in trees] == list(syms)
    L.nch_dec_free(d)


@needs_ref
def test_schedule_equals_reference(pkg):
    L, R = pkg.host.library(), orc.ref_lib()
    cases = [([3e-4, 1e-4], [156250], 0.0), ([1.6e-4, 1e-4], [10000], 0.5), ([1e-3], [], 0.0),
             ([1e-3, 5e-4, 2e-4], [100, 1000], 0.3)]
    for vals, pos, dp in cases:
        ip = pkg.host.InterpParams.make(vals, pos, dp)
        v = np.array(vals, np.float32)
        ps = np.array(pos + [0], np.int64)
        for at in (0, 1, 50, 99, 100, 101, 999, 1000, 5000, 10000, 40000, 156249, 156250, 10 ** 7):
            want = R.ref_interp(len(pos), v.ctypes.data, ps.ctypes.data, dp, at)
            assert L.nch_interp(C.byref(ip), at) == want, (vals, at)


def test_stream_layout(pkg):
    L = pkg.host.library()
    block_len, B = 23, 4                       # stride 5, 3 streams get one extra symbol
    buf = np.arange(100, 100 + block_len, dtype=np.uint16)
    stride, rem = block_len // B, block_len % B
    seen = []
    for s in range(B):
        n = stride + (s < rem)
        assert L.nch_get_symb(buf.ctypes.data_as(_vp), stride, rem, s, -1) == 0
        assert L.nch_get_symb(buf.ctypes.data_as(_vp), stride, rem, s, n) == 0
        seen += [L.nch_get_symb(buf.ctypes.data_as(_vp), stride, rem, s, i) for i in range(n)]
    assert seen == list(buf)                   # streams tile the block contiguously, in order
    out = np.zeros(block_len, np.uint16)
    for s in range(B):
        for i in range(stride + (s < rem)):
            assert L.nch_put_symb(out.ctypes.data_as(_vp), stride, rem, s, i, 7 * s + i) == 0
    assert L.nch_put_symb(out.ctypes.data_as(_vp), stride, rem, 3, stride, 1) != 0


def test_header_layout_and_round_trip(pkg):
    p = pkg.abi.make_params(n_layer=2, d_model=128, n_head=4, d_key=32, d_inner=512, d_pos=48, mem_len=32,
                            seg_len=32, n_streams=4, n_symbols=256, init_kind=0, init_range=1.0,
                            beta2=0.9999, gradient_clip=0.1, seed=123)
    fp = pkg.host.file_params(p, lr=pkg.host.InterpParams.make([3e-4, 1e-4], [156250]))
    h = pkg.host.header_bytes(fp, 1000)
    # the reference layout (nncp.c:2665-2690, 1297-1365), field by field, big-endian
    want = struct.pack(">IHBBHHHI", 0xb727ac58, 1, 1, 0, 4, 32, 256, 123)
    want += struct.pack(">Bffif", 1, 3e-4, 1e-4, 156250, 0.0) + struct.pack(">Bff", 0, 500000.0, 0.0)
    want += struct.pack(">IB", 0, 0) + struct.pack(">BBHHHHH", 2, 4, 32, 32, 512, 48, 32)
    want += struct.pack(">HH", 64, 64) + bytes([0, 1, 1, 0, 0, 1, 0, 1]) + struct.pack(">ffB", 1.0, 1.0, 1)
    want += struct.pack(">Bffff", 1, 0.0, 0.9999, 1e-8, 0.1) + bytes([0]) + bytes([0]) + struct.pack(">I", 1000)
    assert h == want
    fp2, nsym, used = pkg.host.read_header(h + b"payload")
    assert nsym == 1000 and used == len(h)
    for f in ("n_layer", "d_model", "n_head", "d_key", "d_inner", "d_pos", "mem_len", "seg_len", "n_streams",
              "n_symbols", "use_bias", "use_w_r", "query_bias", "ln_flags", "ff_act", "init_kind", "seed"):
        assert getattr(fp2.model, f) == getattr(p, f), f
    assert abs(fp2.model.beta2 - 0.9999) < 1e-7 and fp2.lr.n_steps == 1 and fp2.lr.pos[0] == 156250
    # build-defined options travel in version 2
    h2 = pkg.host.header_bytes(pkg.host.file_params(p.copy(init_kind=1, init_range=0.02)), 5)
    assert h2[4:6] == b"\x00\x02" and pkg.host.read_header(h2)[0].model.init_kind == 1
    for bad in (b"", h[:10], b"\x00" + h[1:], h[:4] + b"\x00\x09" + h[6:]):
        with pytest.raises(ValueError):
            pkg.host.read_header(bad)


def _oracle_ops(pkg, model, with_decoder=False, with_encoder_order=False):
    """nch_model_ops backed by the CPU oracle (tests only)."""
    H = pkg.host
    T, B, V = model.T, model.B, model.V
    keep = {}

    def ev(ctx, oi, inp):
        ids = np.ctypeslib.as_array(inp, shape=(T * B,)).reshape(T, B)
        model.eval(oi, ids)
        return 0

    def probs(ctx, t0, nt, out):
        src = np.ctypeslib.as_array(model.L.orc_probs(model.h), shape=(T * B * V,))
        C.memmove(out, src[t0 * B * V:].ctypes.data, 4 * nt * B * V)
        return 0

    def grad(ctx, exp, loss):
        tg = np.ctypeslib.as_array(exp, shape=(T * B,)).reshape(T, B)
        loss[0] = model.eval_gradient(tg)
        return 0

    def setlr(ctx, lr):
        model.set_lr(lr)
        return 0

    keep["fns"] = [H.FN_CTX(lambda c: (model.reset(), 0)[1]), H.FN_SET_LR(setlr), H.FN_EVAL(ev),
                   H.FN_PROBS(probs), H.FN_CTX(lambda c: 0), H.FN_GRAD(grad),
                   H.FN_CTX(lambda c: (model.update(), 0)[1])]
    f = keep["fns"]
    ops = H.ModelOps(None, B, T, V, f[0], f[1], f[2], f[3], H.FN_PATHS(), H.FN_TREES(), f[4], f[5], f[6])
    if with_decoder:
        # the three decoder ops as a model with its own decoder would provide them: here the oracle's
        # tables and the host's read_sym, holding the decoder state on the model's side of the boundary
        L = H.library()
        st = {}

        def dbegin(ctx, payload, n):
            st["buf"] = C.create_string_buffer(C.string_at(payload, n), n) if n else C.create_string_buffer(1)
            st["dec"] = L.nch_dec_new(st["buf"], n)
            st["ids"] = np.zeros((T, B), np.int32)
            return 0

        def dsteps(ctx, t0, nt, ids0, limit_t, limit_b, out):
            o = np.ctypeslib.as_array(out, shape=(nt * B,)).reshape(nt, B)
            o[:] = 0
            if ids0:
                st["ids"][t0] = np.ctypeslib.as_array(ids0, shape=(B,))
            for t in range(t0, t0 + nt):
                model.eval(t, st["ids"])
                pr = np.ctypeslib.as_array(model.L.orc_probs(model.h), shape=(T * B * V,)).reshape(T, B, V)
                for b in range(B):
                    if t < limit_t or (t == limit_t and b < limit_b):
                        row = np.ascontiguousarray(pr[t, b])
                        o[t - t0, b] = L.nch_read_sym(st["dec"], row.ctypes.data_as(C.c_void_p), V)
                if t + 1 < T:
                    st["ids"][t + 1] = o[t - t0]
            return 0

        def dend(ctx, used):
            L.nch_dec_free(st.pop("dec"))
            return 0

        keep["dec"] = [H.FN_DEC_BEGIN(dbegin), H.FN_DEC_STEPS(dsteps), H.FN_DEC_END(dend)]
        ops.decoder_begin, ops.decode_steps, ops.decoder_end = keep["dec"]
    if with_encoder_order:
        # coder-ready paths from the oracle's tables (sym_path = write_sym's prob0 values) and the four
        # ops of the encoder order; the log records the order in which the block loop calls the model
        st2 = {}
        log = keep.setdefault("log", [])
        depth = int(np.ceil(np.log2(V)))

        def padded_path(row, sym):
            """depth entries per row, as the device writes them: a leaf one level up leaves the last 0"""
            out = np.zeros(depth, np.uint16)
            q = orc.sym_path(row, sym)
            out[:len(q)] = q
            return out

        def paths(ctx, t0, nt, sym, out, nbp):
            pr = np.ctypeslib.as_array(model.L.orc_probs(model.h), shape=(T * B * V,)).reshape(T * B, V)
            sy = np.ctypeslib.as_array(sym, shape=(nt * B,))
            flat = np.concatenate([padded_path(pr[t0 * B + i], int(sy[i])) for i in range(nt * B)])
            C.memmove(out, flat.ctypes.data, flat.nbytes)
            nbp[0] = depth
            return 0

        def pbegin(ctx, t0, nt, sym):
            log.append("paths_begin")
            sy = np.ctypeslib.as_array(sym, shape=(nt * B,)).copy()
            pr = np.ctypeslib.as_array(model.L.orc_probs(model.h), shape=(T * B * V,)).reshape(T * B, V)
            st2["rows"] = [padded_path(pr[t0 * B + i], int(sy[i])) for i in range(nt * B)]   # computed now: the
            return 0                                                       # next forward pass overwrites the tables

        def pend(ctx, out, nbp):
            log.append("paths_end")
            flat = np.concatenate(st2["rows"]).astype(np.uint16)
            C.memmove(out, flat.ctypes.data, flat.nbytes)
            nbp[0] = depth
            return 0

        def gqueue(ctx, exp):
            log.append("gradient")
            tg = np.ctypeslib.as_array(exp, shape=(T * B,)).reshape(T, B)
            st2["loss"] = model.eval_gradient(tg)
            return 0

        def rloss(ctx, loss):
            log.append("read_loss")
            loss[0] = st2["loss"]
            return 0

        def ev_logged(ctx, oi, inp):
            log.append("eval")
            return ev(ctx, oi, inp)

        def trees(ctx, t0, nt, out):
            pr = np.ctypeslib.as_array(model.L.orc_probs(model.h), shape=(T * B * V,)).reshape(T * B, V)
            flat = np.concatenate([orc.sym_tree(pr[t0 * B + i]) for i in range(nt * B)])
            C.memmove(out, flat.ctypes.data, flat.nbytes)
            return 0

        keep["enc"] = [H.FN_PATHS(paths), H.FN_TREES(trees), H.FN_PATHS_BEGIN(pbegin), H.FN_PATHS_END(pend),
                       H.FN_GRAD_QUEUE(gqueue), H.FN_READ_LOSS(rloss), H.FN_EVAL(ev_logged)]
        (ops.coder_paths, ops.coder_trees, ops.coder_paths_begin, ops.coder_paths_end, ops.eval_gradient_queue,
         ops.read_loss, ops.eval) = keep["enc"]
    ops._keep = keep
    return ops


@pytest.mark.parametrize("n_sym,block_len", [(0, 500), (1, 500), (37, 500), (4 * 2 * 6, 500), (301, 96),
                                             (250, 1000)])
def test_block_loop_round_trip_with_oracle_model(pkg, n_sym, block_len):
    """encode with one model_eval per segment, decode one symbol at a time: identical symbols back.
    Covers empty input, inputs shorter than one segment, ragged tails (block_len % streams != 0),
    several blocks, and training between segments."""
    cfg, z = load_golden("post_gelu")
    p = params_from_cfg(pkg, cfg, n_streams=2, seg_len=4, lr=1e-2)
    rng = np.random.default_rng(n_sym)
    # a learnable source: mostly a short cycle, sometimes noise
    syms = np.array([(3 * i) % 5 if rng.random() < 0.85 else rng.integers(0, 16) for i in range(n_sym)],
                    np.uint16)
    fp = pkg.host.file_params(p, block_len=block_len)
    enc_model, dec_model = orc.OracleModel(p), orc.OracleModel(p)
    data, st = pkg.host.compress(_oracle_ops(pkg, enc_model), fp, syms, pkg.host.EVAL_SEGMENT,
                                 pkg.host.OUT_FLOAT)
    assert st.n_symbols == n_sym
    back = pkg.host.decompress(_oracle_ops(pkg, dec_model), data, pkg.host.OUT_FLOAT)
    assert np.array_equal(back, syms)
    # the block walk that hands whole segments to a decoder on the model's side
    # (NCH_OUT_DEVICE), and its fallback when the model has no such decoder
    back = pkg.host.decompress(_oracle_ops(pkg, orc.OracleModel(p), with_decoder=True), data, pkg.host.OUT_DEVICE)
    assert np.array_equal(back, syms)
    back = pkg.host.decompress(_oracle_ops(pkg, orc.OracleModel(p)), data, pkg.host.OUT_DEVICE)
    assert np.array_equal(back, syms)
    if n_sym >= 250:
        assert st.train_steps > 0
        # the model learns the cycle: fewer bits than the 4 bits/symbol of a uniform coder
        hdr = len(pkg.host.header_bytes(fp, n_sym))
        assert (len(data) - hdr) * 8 < 0.8 * 4 * n_sym


@pytest.mark.parametrize("V", [16, 24, 21, 3])
def test_coder_ready_walks_serve_any_alphabet(pkg, V):
    """Integer prob0 paths (encode) and trees (decode) in place of the float tables, for alphabets
    that are and are not a power of two (a word dictionary gives (entries + 7) & ~7 symbols): the
    same bytes as write_sym on the float tables, and read_sym_tree brings the symbols back."""
    cfg, z = load_golden("post_gelu")
    p = params_from_cfg(pkg, cfg, n_streams=2, seg_len=4, lr=1e-2, n_symbols=V)
    rng = np.random.default_rng(V)
    syms = np.array([(3 * i) % min(V, 5) if rng.random() < 0.8 else rng.integers(0, V) for i in range(91)], np.uint16)
    syms[:3] = [0, V - 1, V // 2]
    fp = pkg.host.file_params(p, block_len=40)
    H = pkg.host
    plain, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, H.EVAL_SEGMENT, H.OUT_FLOAT)
    for mode in (H.EVAL_SEGMENT, H.EVAL_STEP):
        ready, _ = H.compress(_oracle_ops(pkg, orc.OracleModel(p), with_encoder_order=True), fp, syms, mode,
                              H.OUT_CODER_READY)
        assert ready == plain
    back = H.decompress(_oracle_ops(pkg, orc.OracleModel(p), with_encoder_order=True), plain, H.OUT_CODER_READY)
    assert np.array_equal(back, syms)


def test_encoder_order_block_loop_gives_the_same_bytes(pkg):
    """A model that offers the encoder order (coder values begun / collected separately, gradient queued,
    loss read later): the block loop queues the next segment's forward pass before it collects and codes
    the current one, never across a block boundary or into the tail, and writes the same bytes."""
    cfg, z = load_golden("post_gelu")
    p = params_from_cfg(pkg, cfg, n_streams=2, seg_len=4, lr=1e-2)
    syms = np.array([(3 * i) % 5 for i in range(77)], np.uint16)     # blocks of 32: 4 segments each, then a ragged tail
    fp = pkg.host.file_params(p, block_len=32)
    plain, _ = pkg.host.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, pkg.host.EVAL_SEGMENT, pkg.host.OUT_FLOAT)
    ops = _oracle_ops(pkg, orc.OracleModel(p), with_encoder_order=True)
    fast, st = pkg.host.compress(ops, fp, syms, pkg.host.EVAL_SEGMENT, pkg.host.OUT_CODER_READY)
    assert fast == plain and st.n_symbols == 77 and st.train_steps == 9
    log = ops._keep["log"]
    per_block = ["eval", "paths_begin", "gradient", "eval", "paths_end", "read_loss"] + \
                ["paths_begin", "gradient", "eval", "paths_end", "read_loss"] * 2 + \
                ["paths_begin", "gradient", "paths_end", "read_loss"]
    assert log[:len(per_block)] == per_block           # block 1: the last segment queues nothing
    assert log[len(per_block):2 * len(per_block)] == per_block
    back = pkg.host.decompress(_oracle_ops(pkg, orc.OracleModel(p)), fast, pkg.host.OUT_FLOAT)
    assert np.array_equal(back, syms)


def test_step_mode_encoder_gives_the_same_bytes(pkg):
    cfg, z = load_golden("post_gelu")
    p = params_from_cfg(pkg, cfg, n_streams=2, seg_len=4)
    syms = (np.arange(90) * 7 % 16).astype(np.uint16)
    fp = pkg.host.file_params(p, block_len=64)
    a, _ = pkg.host.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, pkg.host.EVAL_SEGMENT, 0)
    b, _ = pkg.host.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, pkg.host.EVAL_STEP, 0)
    assert a == b


def test_truncated_payload_decodes_without_failing(pkg):
    """The decoder zero-pads past the end of its input (arith.c:209-223): a truncated stream
    yields wrong symbols, never an error or a crash."""
    cfg, z = load_golden("post_gelu")
    p = params_from_cfg(pkg, cfg, n_streams=2, seg_len=4)
    syms = (np.arange(60) % 16).astype(np.uint16)
    fp = pkg.host.file_params(p)
    data, _ = pkg.host.compress(_oracle_ops(pkg, orc.OracleModel(p)), fp, syms, 1, 0)
    back = pkg.host.decompress(_oracle_ops(pkg, orc.OracleModel(p)), data[:-3], 0)
    assert back.shape == syms.shape and back.max() < 16


def test_cuda_binding_fails_loudly_without_a_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.LibraryMissing):
        pkg.host.bind_cuda(pkg.abi.make_params())


def test_integer_walks_equal_the_float_coder_for_every_small_alphabet(pkg):
    """For V = 2 .. 40 and a few larger odd sizes: coding every symbol of a random row from the
    oracle's prob0 path (nch_write_sym_path_any) gives the bytes of nch_write_sym on the floats, and
    nch_read_sym_tree on the oracle's tree reads them back; the tree has 2^ceil(log2 V) slots."""
    L = pkg.host.library()
    vp = C.c_void_p
    rng = np.random.default_rng(2)
    for V in list(range(2, 41)) + [100, 257, 1000]:
        x = rng.standard_normal(V) * 3
        prob = np.exp(x - x.max())
        prob = (prob / prob.sum()).astype(np.float32)
        syms = list(range(V)) if V <= 40 else [0, V - 1, V // 2] + list(rng.integers(0, V, 20))
        depth = L.nch_tree_depth(V)
        assert (1 << depth) >= V > (1 << depth) // 2
        tree = orc.sym_tree(prob)
        assert tree.size == 1 << depth
        ea, eb = L.nch_enc_new(), L.nch_enc_new()
        for s in syms:
            L.nch_write_sym(ea, prob.ctypes.data_as(vp), V, int(s))
            path = np.zeros(depth, np.uint16)
            q = orc.sym_path(prob, int(s))
            path[:len(q)] = q
            L.nch_write_sym_path_any(eb, path.ctypes.data_as(vp), V, int(s))
        pa, pb = vp(), vp()
        na, nb = L.nch_enc_finish(ea, C.byref(pa)), L.nch_enc_finish(eb, C.byref(pb))
        a, b = C.string_at(pa.value, na), C.string_at(pb.value, nb)
        assert a == b, V
        buf = C.create_string_buffer(a, max(len(a), 1))
        d = L.nch_dec_new(buf, len(a))
        assert [L.nch_read_sym_tree(d, tree.ctypes.data_as(vp), V) for _ in syms] == [int(s) for s in syms], V
        L.nch_dec_free(d)
        L.nch_enc_free(ea)
        L.nch_enc_free(eb)
