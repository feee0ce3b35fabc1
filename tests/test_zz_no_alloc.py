"""nncu_attention_backward_noalloc: the attention backward pass for callers that cannot
allocate device memory (a host that gave the whole GPU to its own pool, or a loop that cannot
afford the device-wide synchronisation of cudaMalloc/cudaFree).  Its partial table gradients
live in a fixed array inside the library instead of caller-provided buffers.

Checked against the existing pair nncu_attention_backward + nncu_attention_reduce_tables on
the same inputs, on two calls in a row that share the built-in array (the second with another
shape, so stale contents of the first would show).  Both paths run the same kernels in the
same order, so the comparison is exact; the suite's bf16 tolerance is the stated bound.
This file sorts last on purpose: a failure here cannot hide the other tests from `-x`.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2


def _run_both(pkg, B, H, dk, T, M, P, bf16, seed):
    lib = pkg.library()
    L = M + T
    dt = torch.bfloat16 if bf16 else torch.float32
    g = torch.Generator(device="cpu").manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dt).cuda()
    q, kv, dout = rnd(T * B, H * dk), rnd(L * B, 2 * H * dk), rnd(T * B, H * dk)
    w_r = (0.02 * torch.randn(H, P, dk, generator=g)).cuda()
    b_r = (0.02 * torch.randn(H, L, generator=g)).cuda()
    shp = pkg.abi.AttnShape(B, H, dk, T, M, P, 0, 0, T, float(np.sqrt(dk * 512.0)), int(bf16))
    out = torch.zeros(T * B, H * dk, device="cuda", dtype=dt)
    lse = torch.zeros(B * H, T, device="cuda")
    assert lib.nncu_attention_forward(C.byref(shp), q.data_ptr(), kv.data_ptr(), w_r.data_ptr(), b_r.data_ptr(),
                                      out.data_ptr(), lse.data_ptr(), None) == 0, lib.nncu_last_error()
    # existing entry points: caller-provided partial buffers, then the reduction over streams
    dq0, dkv0 = torch.zeros_like(q), torch.zeros_like(kv)
    pw, pb = torch.zeros(B, H, P, dk, device="cuda"), torch.zeros(B, H, L, device="cuda")
    gw0, gb0 = torch.zeros(H, P, dk, device="cuda"), torch.zeros(H, L, device="cuda")
    assert lib.nncu_attention_backward(C.byref(shp), q.data_ptr(), kv.data_ptr(), w_r.data_ptr(), b_r.data_ptr(),
                                       out.data_ptr(), lse.data_ptr(), dout.data_ptr(), dq0.data_ptr(),
                                       dkv0.data_ptr(), pw.data_ptr(), pb.data_ptr(), None) == 0
    assert lib.nncu_attention_reduce_tables(C.byref(shp), pw.data_ptr(), pb.data_ptr(), gw0.data_ptr(),
                                            gb0.data_ptr(), 0, None) == 0
    # the entry point that allocates nothing
    dq1, dkv1 = torch.full_like(q, float("nan")), torch.full_like(kv, float("nan"))
    gw1 = torch.full((H, P, dk), float("nan"), device="cuda")
    gb1 = torch.full((H, L), float("nan"), device="cuda")
    # Device memory as the driver sees it (cudaMemGetInfo): an allocation inside the library would
    # not show in torch's own allocator statistics.  A first call loads the kernels and looks the
    # array's address up (both may take device memory once per process); the measured call is the
    # second one.
    assert lib.nncu_attention_backward_noalloc(C.byref(shp), q.data_ptr(), kv.data_ptr(), w_r.data_ptr(),
                                               b_r.data_ptr(), out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
                                               dq1.data_ptr(), dkv1.data_ptr(), gw1.data_ptr(), gb1.data_ptr(),
                                               None) == 0, lib.nncu_last_error()
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    assert lib.nncu_attention_backward_noalloc(C.byref(shp), q.data_ptr(), kv.data_ptr(), w_r.data_ptr(),
                                               b_r.data_ptr(), out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
                                               dq1.data_ptr(), dkv1.data_ptr(), gw1.data_ptr(), gb1.data_ptr(),
                                               None) == 0, lib.nncu_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == before, "the call changed the device's free memory"
    for name, a, b in (("dq", dq1, dq0), ("dkv", dkv1, dkv0), ("dw_r", gw1, gw0), ("db_r", gb1, gb0)):
        a, b = a.float(), b.float()
        assert torch.isfinite(a).all(), name
        err = (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)
        assert err <= BF16_TOL, (name, err)
        assert torch.equal(a, b), name      # same kernels, same order: in fact identical


def test_no_alloc_entry_point_matches_existing_one_twice_in_a_row(pkg):
    _run_both(pkg, 16, 8, 64, 64, 64, 128, True, 1)    # BASELINE config[1], tensor-core kernels
    _run_both(pkg, 3, 2, 8, 6, 2, 5, False, 2)         # smaller, fp32, CUDA-core kernels: reuses the array


def test_no_alloc_entry_point_refuses_shapes_beyond_its_array(pkg):
    lib = pkg.library()
    B, H, dk, T, M, P = 64, 16, 64, 64, 256, 320      # 64*16*(320*64 + 320) floats > 4 Mi floats
    assert B * H * (P * dk + M + T) > pkg.abi.NOALLOC_SCRATCH_FLOATS
    shp = pkg.abi.AttnShape(B, H, dk, T, M, P, 0, 0, T, 1.0, 1)
    one = torch.zeros(16, device="cuda")
    ptr = one.data_ptr()   # never dereferenced: the size check comes before any launch
    rc = lib.nncu_attention_backward_noalloc(C.byref(shp), ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr,
                                             None)
    assert rc == pkg.abi.ERR_RANGE
    assert b"scratch floats" in lib.nncu_last_error()
