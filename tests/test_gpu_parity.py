"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the golden vectors.

Tolerances (relative error = max|a-b| / max|b|):
  fp32 model  1e-3   (north-star figure for logits and updated weights)
  bf16 model  2e-2
Bit-exact where the domain is integer or where two CUDA paths must agree with each other
(one-symbol steps vs whole segment, run-to-run, coder-ready output vs the coder oracle).
"""
import ctypes as C

import numpy as np
import pytest

from conftest import GOLDEN_NAMES, check_updated_weights, load_golden, params_from_cfg, rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FP32_TOL, BF16_TOL = 1e-3, 2e-2


def _dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def _bf16_round(a):
    return torch.as_tensor(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def _load(model, z, step=0, rounder=None):
    for name in model.info:
        v = z[f"p{step}/{name}"]
        model.set_param(name, rounder(v) if rounder else v)


# ---------------------------------------------------------------- dense contraction

@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 512), (2048, 512, 512), (100, 72, 40),
                                   (32, 16384, 512), (2048, 2048, 512), (4096, 1024, 512), (8, 16, 16),
                                   (300, 200, 1000),
                                   # long contractions into narrow outputs (many k-blocks per tile)
                                   (2048, 512, 2048), (32, 512, 2048), (100, 72, 2048), (4096, 1024, 4096),
                                   (130, 200, 1544)])
@pytest.mark.parametrize("c_f32", [0, 1])
def test_gemm_tcgen05_and_simt_vs_fp32(pkg, M, N, K, c_f32):
    lib = pkg.library()
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).cuda()
    ref = a.float() @ b.float().T + bias
    outs = {}
    for backend in (pkg.abi.GEMM_SIMT, pkg.abi.GEMM_TCGEN05):
        c = torch.full((M, N), float("nan"), device="cuda",
                       dtype=torch.float32 if c_f32 else torch.bfloat16)
        rc = lib.nncu_gemm_bf16_nt(backend, M, N, K, a.data_ptr(), K, b.data_ptr(), K, c.data_ptr(), N,
                                   c_f32, bias.data_ptr(), None)
        assert rc == 0, lib.nncu_last_error()
        torch.cuda.synchronize()
        outs[backend] = c.float()
        tol = 2e-5 if c_f32 else 1e-2
        err = (c.float() - ref).abs().max().item() / ref.abs().max().item()
        assert err < tol, (backend, err)
    # the two engines accumulate in fp32 over the same bf16 products
    d = (outs[pkg.abi.GEMM_SIMT] - outs[pkg.abi.GEMM_TCGEN05]).abs().max().item()
    assert d <= (1e-4 if c_f32 else 0.07) * ref.abs().max().item()


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (2048, 512, 512), (512, 2048, 2048), (1024, 512, 4096),
                                   (104, 72, 40), (16384, 512, 2048), (2048, 512, 16384), (200, 136, 1000)])
def test_gemm_mn_major_operands(pkg, mode, M, N, K):
    """dx = dy W (mode 1, B read as [K][N]) and dW = dy^T x (mode 2, both operands [K][.]) on the
    tensor-core engine against fp32 torch and the CUDA-core engine."""
    lib = pkg.library()
    g = torch.Generator(device="cpu").manual_seed(M + N + K + mode)
    a = torch.randn((M, K) if mode == 1 else (K, M), generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(K, N, generator=g).to(torch.bfloat16).cuda()
    ref = (a.float() if mode == 1 else a.float().T) @ b.float()
    for backend in (pkg.abi.GEMM_SIMT, pkg.abi.GEMM_TCGEN05):
        c = torch.full((M, N), float("nan"), device="cuda")
        rc = lib.nncu_gemm_bf16(backend, mode, M, N, K, a.data_ptr(), a.shape[1], b.data_ptr(), N, c.data_ptr(),
                                N, 1, None)
        assert rc == 0, lib.nncu_last_error()
        torch.cuda.synchronize()
        err = (c - ref).abs().max().item() / ref.abs().max().item()
        assert err < 5e-5, (backend, err)


def test_gemm_rows_do_not_depend_on_the_launch(pkg):
    """A row computed in a 32-row launch equals the same row of a 2048-row launch, bit for bit,
    on both engines (what lets the encoder run whole segments and the decoder single symbols)."""
    lib = pkg.library()
    g = torch.Generator(device="cpu").manual_seed(5)
    a = torch.randn(2048, 512, generator=g).to(torch.bfloat16).cuda()
    # N = 512 / 1536 / 16384: the 2048-row and the 32-row launch pick different tile widths
    for N, c_f32 in ((512, 0), (1536, 0), (16384, 1)):
        b = torch.randn(N, 512, generator=g).to(torch.bfloat16).cuda()
        dt = torch.float32 if c_f32 else torch.bfloat16
        for backend in (pkg.abi.GEMM_SIMT, pkg.abi.GEMM_TCGEN05):
            full = torch.zeros(2048, N, device="cuda", dtype=dt)
            part = torch.zeros(32, N, device="cuda", dtype=dt)
            assert lib.nncu_gemm_bf16_nt(backend, 2048, N, 512, a.data_ptr(), 512, b.data_ptr(), 512,
                                         full.data_ptr(), N, c_f32, None, None) == 0, lib.nncu_last_error()
            off = 1000
            assert lib.nncu_gemm_bf16_nt(backend, 32, N, 512, a[off:].data_ptr(), 512, b.data_ptr(), 512,
                                         part.data_ptr(), N, c_f32, None, None) == 0, lib.nncu_last_error()
            torch.cuda.synchronize()
            assert torch.equal(full[off:off + 32], part), (backend, N)
    # the second feed-forward projection (K = 2048 into N = 512, with its bias): 32 k-blocks dealt to
    # the two issuing threads, for 2048 rows and for 32 rows alike
    a2 = torch.randn(2048, 2048, generator=g).to(torch.bfloat16).cuda()
    b2 = torch.randn(512, 2048, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(512, generator=g).cuda()
    full = torch.zeros(2048, 512, device="cuda", dtype=torch.bfloat16)
    part = torch.zeros(32, 512, device="cuda", dtype=torch.bfloat16)
    tcg = pkg.abi.GEMM_TCGEN05
    assert lib.nncu_gemm_bf16_nt(tcg, 2048, 512, 2048, a2.data_ptr(), 2048, b2.data_ptr(), 2048, full.data_ptr(), 512, 0,
                                 bias.data_ptr(), None) == 0, lib.nncu_last_error()
    assert lib.nncu_gemm_bf16_nt(tcg, 32, 512, 2048, a2[1000:].data_ptr(), 2048, b2.data_ptr(), 2048, part.data_ptr(), 512,
                                 0, bias.data_ptr(), None) == 0, lib.nncu_last_error()
    torch.cuda.synchronize()
    assert torch.equal(full[1000:1032], part)


# ---------------------------------------------------------------- attention op

def _attn_case(pkg, oracle, B, H, dk, T, M, P, attn_len, bf16, seed):
    L = M + T
    rng = np.random.default_rng(seed)
    rnd = (lambda *s: _bf16_round(rng.standard_normal(s))) if bf16 else \
          (lambda *s: rng.standard_normal(s).astype(np.float32))
    q, kv, dout = rnd(T * B, H * dk), rnd(L * B, 2 * H * dk), rnd(T * B, H * dk)
    w_r = (0.02 * rng.standard_normal((H, P, dk))).astype(np.float32)
    b_r = (0.02 * rng.standard_normal((H, L))).astype(np.float32)
    if bf16:
        w_r = _bf16_round(w_r)   # the kernel stages the table in the activation type
    shp = pkg.abi.AttnShape(B, H, dk, T, M, P, attn_len, 0, T, float(np.sqrt(dk * 512.0)), int(bf16))
    # oracle
    O = oracle.lib()
    out_ref = np.zeros((T * B, H * dk), np.float32)
    Pm = np.zeros((B, H, T, L), np.float32)
    lse_ref = np.zeros((B * H, T), np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    O.orc_attention_forward(C.byref(shp), p(q), p(kv), p(w_r), p(b_r), p(out_ref), p(Pm), p(lse_ref))
    dq_ref, dkv_ref = np.zeros_like(q), np.zeros_like(kv)
    dwr_ref, dbr_ref = np.zeros_like(w_r), np.zeros_like(b_r)
    O.orc_attention_backward(C.byref(shp), p(q), p(kv), p(w_r), p(b_r), p(Pm), p(dout), p(dq_ref),
                             p(dkv_ref), p(dwr_ref), p(dbr_ref))
    # device
    lib = pkg.library()
    dt = torch.bfloat16 if bf16 else torch.float32
    dq_, dkv_, ddout = _dev(q, dt), _dev(kv, dt), _dev(dout, dt)
    dwr, dbr = _dev(w_r), _dev(b_r)
    out = torch.zeros(T * B, H * dk, device="cuda", dtype=dt)
    lse = torch.zeros(B * H, T, device="cuda")
    assert lib.nncu_attention_forward(C.byref(shp), dq_.data_ptr(), dkv_.data_ptr(), dwr.data_ptr(),
                                      dbr.data_ptr(), out.data_ptr(), lse.data_ptr(), None) == 0, \
        lib.nncu_last_error()
    gq, gkv = torch.zeros_like(dq_), torch.zeros_like(dkv_)
    pw = torch.zeros(B, H, P, dk, device="cuda")
    pb = torch.zeros(B, H, L, device="cuda")
    assert lib.nncu_attention_backward(C.byref(shp), dq_.data_ptr(), dkv_.data_ptr(), dwr.data_ptr(),
                                       dbr.data_ptr(), out.data_ptr(), lse.data_ptr(), ddout.data_ptr(),
                                       gq.data_ptr(), gkv.data_ptr(), pw.data_ptr(), pb.data_ptr(),
                                       None) == 0, lib.nncu_last_error()
    gw, gb = torch.zeros(H, P, dk, device="cuda"), torch.zeros(H, L, device="cuda")
    assert lib.nncu_attention_reduce_tables(C.byref(shp), pw.data_ptr(), pb.data_ptr(), gw.data_ptr(),
                                            gb.data_ptr(), 0, None) == 0
    torch.cuda.synchronize()
    tol = BF16_TOL if bf16 else FP32_TOL
    res = dict(out=(out, out_ref), lse=(lse, lse_ref), dq=(gq, dq_ref), dkv=(gkv, dkv_ref),
               dw_r=(gw, dwr_ref), db_r=(gb, dbr_ref))
    for k, (got, want) in res.items():
        e = rel_err(got.float().cpu().numpy(), want)
        assert e < tol, (k, e)


def test_attention_op_config1_bf16(pkg, oracle):
    # BASELINE config[1]: 16 streams, 8 heads, d_head 64, query 64, keys 64+64, R of length 128
    _attn_case(pkg, oracle, 16, 8, 64, 64, 64, 128, 0, True, 1)


@pytest.mark.parametrize("B,H,dk,T,M,P,alen", [(2, 2, 16, 6, 6, 9, 0), (2, 3, 32, 20, 70, 50, 60),
                                               (1, 2, 64, 64, 128, 192, 0), (2, 2, 128, 33, 31, 64, 40),
                                               (3, 1, 32, 64, 0, 64, 0),
                                               # memories longer than one staged key tile: BASELINE config[3]
                                               # (mem 256) and config[4] (mem 512) head geometry, a windowed
                                               # layer whose first key tiles are never attended, a table
                                               # shorter than the keys, and wide heads over several key tiles
                                               (2, 2, 64, 64, 256, 320, 0), (1, 2, 64, 64, 512, 576, 0),
                                               (2, 1, 32, 40, 300, 200, 150), (1, 2, 64, 64, 448, 64, 0),
                                               (1, 2, 128, 48, 150, 198, 0), (1, 1, 16, 64, 200, 40, 100),
                                               # d_head 64 (the tcgen05 kernels): an attention window over
                                               # three key blocks, fewer than 64 queries with an odd stream
                                               # count, and a table far shorter than the memory
                                               (2, 2, 64, 64, 256, 320, 150), (3, 2, 64, 40, 100, 90, 0),
                                               (4, 1, 64, 64, 300, 20, 0)])
def test_attention_op_tensor_core_shapes_bf16(pkg, oracle, B, H, dk, T, M, P, alen):
    _attn_case(pkg, oracle, B, H, dk, T, M, P, alen, True, 3)


@pytest.mark.parametrize("B,H,dk,T,M,P,alen", [(3, 2, 8, 6, 2, 5, 3), (2, 4, 32, 32, 32, 64, 0),
                                               (1, 1, 16, 4, 10, 14, 0), (2, 2, 8, 5, 0, 3, 0)])
def test_attention_op_ragged_fp32(pkg, oracle, B, H, dk, T, M, P, alen):
    _attn_case(pkg, oracle, B, H, dk, T, M, P, alen, False, 2)


# ---------------------------------------------------------------- whole train step

@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_train_step_fp32_vs_golden_and_oracle(pkg, oracle, name):
    cfg, z = load_golden(name)
    p = params_from_cfg(pkg, cfg)
    m, o = pkg.TrfModel(p), oracle.OracleModel(p)
    _load(m, z)
    _load(o, z)
    m.reset(); o.reset()
    m.set_lr(cfg["lr"]); o.set_lr(cfg["lr"])
    for s in range(z["ids"].shape[0]):
        probs = m.eval(-1, z["ids"][s])
        assert rel_err(probs, z["probs"][s]) < FP32_TOL
        assert rel_err(probs, o.eval(-1, z["ids"][s])) < FP32_TOL
        loss = m.eval_gradient(z["targets"][s])
        assert abs(loss - z["loss"][s]) < FP32_TOL * abs(z["loss"][s])
        o.eval_gradient(z["targets"][s])
        for pname in m.info:
            g_ref = z[f"g{s}/{pname}"].reshape(-1)
            scale = max(np.abs(g_ref).max(), 1e-6)
            assert np.abs(m.get_grad(pname) - g_ref).max() / scale < FP32_TOL, (pname, s)
            assert np.abs(m.get_grad(pname) - o.get_grad(pname)).max() / scale < FP32_TOL, (pname, s)
        before = {pname: m.get_param(pname) for pname in m.info}
        m.update(); o.update()
        for pname in m.info:
            check_updated_weights(m.get_param(pname), z[f"p{s+1}/{pname}"].reshape(-1), before[pname],
                                  z[f"g{s}/{pname}"].reshape(-1), FP32_TOL, cfg["lr"], cfg["beta2"], (pname, s))
        # continue from the golden weights: step 2 is then checked on its own
        for pname in m.info:
            m.set_param(pname, z[f"p{s+1}/{pname}"])
            o.set_param(pname, z[f"p{s+1}/{pname}"])
    m.close()


@pytest.mark.parametrize("name,bf16,backend", [("c0_like", 0, 1), ("post_gelu", 0, 1),
                                               ("pre_final_geglu_rms", 0, 1), ("short_mem_window", 0, 1),
                                               ("c0_like", 1, 1), ("c0_like", 1, 2),
                                               ("pre_final_geglu_rms", 1, 2), ("tied_tables_longmem", 1, 2),
                                               ("mma_dk16", 1, 2), ("mma_two_key_blocks", 1, 2),
                                               ("mma_two_key_blocks", 1, 1), ("mma_long_memory", 1, 2),
                                               ("ln_coef_post", 1, 2), ("ln_coef_pre_rms", 0, 1)])
def test_one_symbol_steps_equal_whole_segment_bitwise(pkg, name, bf16, backend):
    cfg, z = load_golden(name)
    p = params_from_cfg(pkg, cfg, use_bf16=bf16, gemm_backend=backend)
    a, b = pkg.TrfModel(p), pkg.TrfModel(p)
    for m in (a, b):
        _load(m, z)
        m.reset()
    for s in range(2):
        ids, tg = z["ids"][s], z["targets"][s]
        full = a.eval(-1, ids)
        for t in range(cfg["seg_len"]):
            step = b.eval(t, ids)
            assert np.array_equal(step[0], full[t]), (s, t)
        la, lb = a.eval_gradient(tg), b.eval_gradient(tg)
        assert la == lb
        a.update(); b.update()
        assert a.weights_hash() == b.weights_hash()
    a.close(); b.close()


@pytest.mark.parametrize("name", ["c0_like", "pre_final_geglu_rms", "tied_tables_longmem", "mma_dk16",
                                  "mma_two_key_blocks", "mma_long_memory", "post_gelu", "gated_silu_wide",
                                  "ln_coef_post", "ln_coef_pre_rms"])
@pytest.mark.parametrize("backend", [1, 2])
def test_train_step_bf16_vs_oracle(pkg, oracle, name, backend):
    cfg, z = load_golden(name)
    p = params_from_cfg(pkg, cfg, use_bf16=1, gemm_backend=backend)
    m, o = pkg.TrfModel(p), oracle.OracleModel(params_from_cfg(pkg, cfg))
    _load(m, z, rounder=_bf16_round)
    _load(o, z, rounder=_bf16_round)
    m.reset(); o.reset()
    m.set_lr(cfg["lr"]); o.set_lr(cfg["lr"])
    for s in range(2):
        probs, probs_ref = m.eval(-1, z["ids"][s]), o.eval(-1, z["ids"][s])
        assert rel_err(probs, probs_ref) < BF16_TOL
        loss, loss_ref = m.eval_gradient(z["targets"][s]), o.eval_gradient(z["targets"][s])
        assert abs(loss - loss_ref) < BF16_TOL * abs(loss_ref)
        gmax = max(np.abs(o.get_grad(pname)).max() for pname in m.info)
        for pname in m.info:
            g_ref = o.get_grad(pname)
            scale = max(np.abs(g_ref).max(), 1e-6)
            # LN_COEF's alpha is ONE number: the sum of T*B*D signed products of bf16-rounded factors, most of
            # which cancel.  Its rounding noise is set by the products, not by the (small) sum, so it is
            # measured against the largest gradient entry of the model instead of against itself.
            if pname.startswith("alpha"):
                scale = max(scale, gmax)
            assert np.abs(m.get_grad(pname) - g_ref).max() / scale < 5 * BF16_TOL, (pname, s)
        grads = {pname: o.get_grad(pname) for pname in m.info}
        before = {pname: o.get_param(pname) for pname in m.info}
        m.update(); o.update()
        for pname in m.info:
            check_updated_weights(m.get_param(pname), o.get_param(pname), before[pname], grads[pname],
                                   BF16_TOL, cfg["lr"], cfg["beta2"], (pname, s))
        # keep the two trajectories together so that step 2 tests step 2
        for pname in m.info:
            o.set_param(pname, m.get_param(pname))
    m.close()


def test_output_head_split_k_vs_oracle(pkg, oracle):
    """n_symbols >= 8192 with 128 rows: the output head's dX contraction (K = n_symbols) runs as four
    partial products per tile plus an ordered sum; every gradient below the head depends on it."""
    kw = dict(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=8, seg_len=8,
              n_streams=16, n_symbols=8192, init_range=0.05, lr=1e-3)
    m = pkg.TrfModel(pkg.abi.make_params(use_bf16=1, gemm_backend=2, **kw))
    o = oracle.OracleModel(pkg.abi.make_params(use_bf16=0, **kw))
    for name in m.info:
        w = _bf16_round(m.get_param(name))
        m.set_param(name, w)
        o.set_param(name, w)
    rng = np.random.default_rng(11)
    ids = rng.integers(0, 8192, (8, 16)).astype(np.int32)
    tg = rng.integers(0, 8192, (8, 16)).astype(np.int32)
    m.reset(); o.reset()
    assert rel_err(m.eval(-1, ids), o.eval(-1, ids)) < BF16_TOL
    loss, loss_ref = m.eval_gradient(tg), o.eval_gradient(tg)
    assert abs(loss - loss_ref) < BF16_TOL * abs(loss_ref)
    for name in m.info:
        g_ref = o.get_grad(name)
        scale = max(np.abs(g_ref).max(), 1e-6)
        assert np.abs(m.get_grad(name) - g_ref).max() / scale < 5 * BF16_TOL, name
    m.close()


@pytest.mark.parametrize("name,bf16,graphs", [("c0_like", 1, 0), ("c0_like", 1, 1), ("tied_tables_longmem", 1, 1),
                                              ("post_gelu", 0, 1), ("ln_coef_post", 1, 1)])
def test_fused_gradient_and_update_gives_the_same_bits(pkg, name, bf16, graphs):
    """nncu_eval_gradient_update + nncu_memory_shift against nncu_eval_gradient + nncu_update over six
    steps with a changing learning rate and bias correction on: same losses, same weights; eager
    (default stream) and with the captured graphs (own stream)."""
    cfg, z = load_golden(name)
    res = []
    for fused in (False, True):
        m = pkg.TrfModel(params_from_cfg(pkg, cfg, use_bf16=bf16, bias_correction=1))
        stream = torch.cuda.Stream() if graphs else None
        if stream is not None:
            m.set_stream(stream.cuda_stream)
        _load(m, z)
        m.reset()
        losses = []
        for s in range(6):
            m.set_lr(cfg["lr"] * (1.0 + 0.25 * s))
            m.eval(-1, z["ids"][s % 2], read=False)
            if fused:
                losses.append(m.eval_gradient_update(z["targets"][s % 2]))
                m.memory_shift()
            else:
                losses.append(m.eval_gradient(z["targets"][s % 2]))
                m.update()
        m.synchronize()
        res.append((losses, m.weights_hash()))
        m.close()
    assert res[0][0] == res[1][0]
    assert res[0][1] == res[1][1]


def test_two_runs_are_bit_identical(pkg):
    cfg, z = load_golden("c0_like")
    hashes = []
    for _ in range(2):
        m = pkg.TrfModel(params_from_cfg(pkg, cfg, use_bf16=1))
        _load(m, z)
        m.reset()
        for s in range(2):
            m.eval(-1, z["ids"][s], read=False)
            m.eval_gradient(z["targets"][s])
            m.update()
        hashes.append(m.weights_hash())
        m.close()
    assert hashes[0] == hashes[1]


@pytest.mark.parametrize("name,bf16", [("c0_like", 0), ("mma_two_key_blocks", 1), ("tied_tables_longmem", 1),
                                       ("mma_long_memory", 1), ("ln_coef_pre_rms", 1)])
def test_graph_replay_equals_eager(pkg, name, bf16):
    """On a non-default stream forward and backward are captured into CUDA graphs on their second
    use; six steps there must give the same bits as six eager steps on the default stream."""
    cfg, z = load_golden(name)
    rng = np.random.default_rng(1)
    T, B, V = cfg["seg_len"], cfg["n_streams"], cfg["n_symbols"]
    ids = rng.integers(0, V, (6, T, B)).astype(np.int32)
    tg = rng.integers(0, V, (6, T, B)).astype(np.int32)
    hashes, losses = [], []
    for use_stream in (False, True):
        m = pkg.TrfModel(params_from_cfg(pkg, cfg, use_bf16=bf16))
        _load(m, z)
        s = torch.cuda.Stream()
        if use_stream:
            m.set_stream(s.cuda_stream)
        m.reset()
        ls = []
        for k in range(6):
            m.eval(-1, ids[k], read=False)
            ls.append(m.eval_gradient(tg[k]))
            m.update()
        m.synchronize()
        hashes.append(m.weights_hash())
        losses.append(ls)
        m.close()
    assert losses[0] == losses[1]
    assert hashes[0] == hashes[1]


def test_initial_values_match_the_oracle(pkg, oracle):
    p = pkg.abi.make_params(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=8,
                            seg_len=8, n_streams=2, n_symbols=64)
    for kind in (0, 1):
        q = p.copy(init_kind=kind, seed=77)
        m, o = pkg.TrfModel(q), oracle.OracleModel(q)
        for name in m.info:
            assert np.array_equal(m.get_param(name), o.get_param(name)), name
        m.close()


# ---------------------------------------------------------------- coder-ready output

def test_encoder_order_queues_everything_and_gives_the_same_bits(pkg):
    """eval, coder_paths_begin, eval_gradient (loss not awaited), update, coder_paths_end, read_loss
    must give the coder values, losses and weights of the strictly sequential order of
    process_block (eval, coder_paths, eval_gradient, update)."""
    import ctypes as C
    cfg, z = load_golden("c0_like")
    lib = pkg.library()
    res = []
    for pipelined in (False, True):
        m = pkg.TrfModel(params_from_cfg(pkg, cfg, use_bf16=1))
        _load(m, z)
        m.reset()
        T, B = cfg["seg_len"], cfg["n_streams"]
        out = []
        for s in range(4):
            ids, tg = z["ids"][s % 2], z["targets"][s % 2]
            tgc = np.ascontiguousarray(tg, np.int32)
            m.eval(-1, ids, read=False)
            if not pipelined:
                paths = m.coder_paths(0, T, tgc)
                loss = m.eval_gradient(tgc)
                m.update()
            else:
                buf = np.zeros(T * B * 32, np.uint16)
                nb = C.c_int()
                assert lib.nncu_coder_paths_begin(m.h, 0, T, tgc.ctypes.data_as(C.c_void_p)) == 0
                # a second begin before the end is refused, and so is the one-call form
                assert lib.nncu_coder_paths_begin(m.h, 0, T, tgc.ctypes.data_as(C.c_void_p)) == pkg.abi.ERR_STATE
                assert lib.nncu_eval_gradient(m.h, tgc.ctypes.data_as(C.c_void_p), None) == 0
                m.update()
                assert lib.nncu_coder_paths_end(m.h, buf.ctypes.data_as(C.c_void_p), C.byref(nb)) == 0
                paths = buf[: T * B * nb.value].reshape(T * B, nb.value).copy()
                loss = m.read_loss()
            out.append((paths, loss))
        res.append((out, m.weights_hash()))
        m.close()
    assert res[0][1] == res[1][1]
    for (pa, la), (pb, lb) in zip(res[0][0], res[1][0]):
        assert np.array_equal(pa, pb)
        assert la == lb


def test_coder_paths_and_trees_match_the_coder_oracle(pkg, oracle):
    p = pkg.abi.make_params(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=8,
                            seg_len=8, n_streams=4, n_symbols=256, init_range=0.3)
    m = pkg.TrfModel(p)
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 256, (8, 4)).astype(np.int32)
    syms = rng.integers(0, 256, (8, 4)).astype(np.int32)
    probs = m.eval(-1, ids)
    paths = m.coder_paths(0, 8, syms)
    trees = m.coder_trees(0, 8)
    enc_a, enc_b = oracle.Encoder(False), oracle.Encoder(False)
    for t in range(8):
        for b in range(4):
            row = t * 4 + b
            want = oracle.sym_path(probs[t, b], syms[t, b])
            assert np.array_equal(paths[row], want), (t, b)
            k = 1
            for lvl in range(8):          # the tree holds the same values on the symbol's path
                assert trees[row, k] == want[lvl]
                k = 2 * k + ((int(syms[t, b]) >> (7 - lvl)) & 1)
            enc_a.put_sym(probs[t, b], syms[t, b])
            for lvl, q in enumerate(want):
                enc_b.put_bit(q, (int(syms[t, b]) >> (7 - lvl)) & 1)
    data = enc_a.finish()
    assert data == enc_b.finish()
    # decode with nothing but the integer trees
    dec = oracle.Decoder(data, False)
    for t in range(8):
        for b in range(4):
            k = 1
            while k < 256:
                k = 2 * k + dec.get_bit(int(trees[t * 4 + b, k]))
            assert k - 256 == syms[t, b]
    m.close()


@pytest.mark.parametrize("V", [1024, 4096, 16384])
def test_coder_paths_large_alphabets_match_the_coder_oracle(pkg, oracle, V):
    """The register / shuffle form of the pairwise sum tree (1024 <= V <= 16384) against write_sym's
    arithmetic, including symbols at the edges of the alphabet; a peaked row makes the running mass
    collapse on the unlikely side."""
    p = pkg.abi.make_params(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=8,
                            seg_len=8, n_streams=4, n_symbols=V, init_range=0.5)
    m = pkg.TrfModel(p)
    rng = np.random.default_rng(V)
    ids = rng.integers(0, V, (8, 4)).astype(np.int32)
    syms = rng.integers(0, V, (8, 4)).astype(np.int32)
    syms[0, :] = [0, V - 1, V // 2, V // 2 - 1]
    probs = m.eval(-1, ids)
    paths = m.coder_paths(0, 8, syms)
    nb = int(np.log2(V))
    assert paths.shape == (32, nb)
    for t in range(8):
        for b in range(4):
            want = oracle.sym_path(probs[t, b], syms[t, b])
            assert np.array_equal(paths[t * 4 + b], want), (t, b)
    m.close()


@pytest.mark.parametrize("V", [24, 288, 1000, 5000])
def test_coder_paths_and_trees_of_any_alphabet_match_the_coder_oracle(pkg, oracle, V):
    """Alphabets that are not a power of two (what a word dictionary gives): write_sym's tree is then
    uneven, leaves at depth L-1 and L.  Paths (L entries a row, the last 0 for a leaf one level up) and
    trees (2^L entries a row, heap order) against the oracle's restatement of write_sym / read_sym."""
    p = pkg.abi.make_params(n_layer=1, d_model=64, n_head=2, d_key=32, d_inner=128, d_pos=16, mem_len=8,
                            seg_len=8, n_streams=4, n_symbols=V, init_range=0.5)
    m = pkg.TrfModel(p)
    rng = np.random.default_rng(V)
    ids = rng.integers(0, V, (8, 4)).astype(np.int32)
    syms = rng.integers(0, V, (8, 4)).astype(np.int32)
    syms[0, :] = [0, V - 1, V // 2, V // 2 - 1]
    probs = m.eval(-1, ids)
    paths = m.coder_paths(0, 8, syms)
    trees = m.coder_trees(0, 8)
    L = (V - 1).bit_length()
    assert paths.shape == (32, L) and trees.shape == (32, 1 << L)
    for t in range(8):
        for b in range(4):
            row = t * 4 + b
            want = oracle.sym_path(probs[t, b], syms[t, b])
            assert np.array_equal(paths[row, :len(want)], want) and not paths[row, len(want):].any(), (t, b)
            assert np.array_equal(trees[row], oracle.sym_tree(probs[t, b])), (t, b)
    m.close()


# ---------------------------------------------------------------- full-size properties

@pytest.mark.parametrize("streams", [32, 8, 4])
def test_config2_scale_step_properties(pkg, streams):
    """BASELINE config[2] sizes (fewer layers to bound the test time), whole job and the 8- and
    4-stream shards a rank holds at 4 and 8 GPUs: probabilities are normalised and finite, the
    loss is finite, and a second identical run gives the same bits."""
    hashes = []
    for _ in range(2):
        p = pkg.abi.make_params(n_layer=3, d_model=512, n_head=8, d_key=64, d_inner=2048, d_pos=128,
                                mem_len=64, seg_len=64, n_streams=streams, n_streams_total=32,
                                n_symbols=16384, use_bf16=1)
        m = pkg.TrfModel(p)
        rng = np.random.default_rng(3)
        ids = rng.integers(0, 16384, (64, streams)).astype(np.int32)
        tg = rng.integers(0, 16384, (64, streams)).astype(np.int32)
        for _s in range(2):
            probs = m.eval(-1, ids)
            assert np.isfinite(probs).all()
            assert np.abs(probs.sum(-1) - 1.0).max() < 1e-4
            loss = m.eval_gradient(tg)
            assert np.isfinite(loss) and loss < 0
            m.update()
        m.synchronize()
        hashes.append(m.weights_hash())
        m.close()
    assert hashes[0] == hashes[1]
