"""Generates tests/golden/trf_*.npz from the PyTorch restatement (trf_torch.py).

Run from the repository root:  python tests/golden/make_golden.py
The restatement is evaluated in float64 so that the stored float32 values are
correctly rounded references for the fp32 oracle and the CUDA path.

Each file holds, for a two-step run of one small configuration:
  cfg_json           the configuration (JSON string)
  p0/<name>          initial parameters
  ids, targets       int32 [steps, T, B]
  probs              [steps, T, B, V]
  loss               [steps]                (sum ln p[target], un-averaged)
  g<s>/<name>        gradients of -loss/(T*B) at step s
  p<s+1>/<name>      parameters after the update of step s
  mem<s+1>           [n_layer, M, B, D] memory after step s

Digest goldens (dig_*.npz) cover the BASELINE geometries, whose tensors are too large to store:
the parameters are rebuilt from a seed (seeded_params.py) and the file keeps the loss, the
probabilities of sampled columns plus the target column, and a strided subsample of every
gradient and updated parameter (with each gradient's max-abs as the error scale).
  python tests/golden/make_golden.py digest
"""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import trf_torch as tt  # noqa: E402

BASE = dict(n_layer=2, d_model=16, n_head=2, d_key=8, d_inner=32, d_pos=8, mem_len=4,
            seg_len=4, n_streams=2, n_symbols=16, attn_len=[0] * 32, use_bias=1, use_w_r=1,
            tied_w_r=0, tied_b_r=0, query_bias=1, ln_flags=tt.LN_POST, ff_act=tt.FF_GELU,
            embed_mult=1.0, beta2=0.99, eps=1e-8, lr=3e-3, gradient_clip=0.0)

CONFIGS = {
    # name: overrides
    "post_gelu": dict(),
    "pre_final_geglu_rms": dict(ln_flags=tt.LN_PRE | tt.LN_FINAL | tt.LN_RMSNORM,
                                ff_act=tt.FF_GEGLU, d_pos=6, mem_len=6),
    "pre_final_ln_relu": dict(ln_flags=tt.LN_PRE | tt.LN_FINAL, ff_act=tt.FF_RELU,
                              use_bias=0, query_bias=0),
    "tied_tables_longmem": dict(tied_w_r=1, tied_b_r=1, mem_len=10, d_pos=14, n_layer=3),
    "ln_coef_post": dict(ln_flags=tt.LN_POST | tt.LN_COEF),
    "ln_coef_pre_rms": dict(ln_flags=tt.LN_PRE | tt.LN_FINAL | tt.LN_RMSNORM | tt.LN_COEF, ff_act=tt.FF_GEGLU, n_streams=3),
    "gated_silu_wide": dict(ff_act=tt.FF_GATED_SILU, n_layer=2, d_model=32, n_head=2, d_key=16, d_inner=64,
                            d_pos=10, mem_len=6, seg_len=6, n_streams=3, n_symbols=32, wscale=0.1),
    "short_mem_window": dict(mem_len=2, d_pos=5, seg_len=6,
                             attn_len=[3, 5] + [0] * 30, n_streams=3),
    "no_w_r_noln_clip": dict(use_w_r=0, ln_flags=0, gradient_clip=0.05, n_symbols=24),
    # head sizes that are multiples of 16: the bf16 model takes the tensor-core attention path
    "mma_dk16": dict(n_layer=2, d_model=32, n_head=2, d_key=16, d_inner=64, d_pos=9, mem_len=6,
                     seg_len=6, n_streams=3, n_symbols=32),
    "mma_two_key_blocks": dict(n_layer=2, d_model=64, n_head=2, d_key=32, d_inner=64, d_pos=50,
                               mem_len=70, seg_len=20, n_streams=2, n_symbols=32,
                               attn_len=[60, 0] + [0] * 30, ln_flags=tt.LN_PRE | tt.LN_FINAL,
                               wscale=0.1),
    # memory longer than the 128 keys the tensor-core attention stages at a time, a windowed layer
    # whose oldest key tile is never attended, and a position table shorter than the keys
    "mma_long_memory": dict(n_layer=2, d_model=64, n_head=2, d_key=32, d_inner=64, d_pos=160,
                            mem_len=200, seg_len=24, n_streams=2, n_symbols=32,
                            attn_len=[90, 0] + [0] * 30, ln_flags=tt.LN_PRE | tt.LN_FINAL,
                            wscale=0.1),
    "c0_like": dict(n_layer=2, d_model=32, n_head=4, d_key=8, d_inner=64, d_pos=16,
                    mem_len=8, seg_len=8, n_streams=4, n_symbols=32),
}
STEPS = 2


def make(name, over, out_dir):
    c = dict(BASE)
    c.update(over)
    wscale = c.pop("wscale", 0.25)
    c["d_value"] = c["d_key"]
    if c["d_pos"] > c["mem_len"] + c["seg_len"]:
        raise ValueError("d_pos > L")
    gen = torch.Generator().manual_seed(sum(map(ord, name)))
    params, moments = {}, {}
    for pname, shape in tt.param_shapes(c):
        if pname.startswith("ln_g"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float64)
        elif pname.startswith(("ln_b", "ff_bias", "out_bias", "b_q")):
            t = 0.05 * torch.randn(shape, generator=gen, dtype=torch.float64)
        elif pname.startswith("b_r"):
            t = 0.02 * torch.randn(shape, generator=gen, dtype=torch.float64)
        else:
            t = wscale * torch.randn(shape, generator=gen, dtype=torch.float64)
        # keep exactly-representable fp32 starting values
        params[pname] = t.float().double()
        moments[pname] = torch.zeros(shape, dtype=torch.float64)
    T, B, V = c["seg_len"], c["n_streams"], c["n_symbols"]
    ids = torch.randint(0, V, (STEPS, T, B), generator=gen)
    targets = torch.randint(0, V, (STEPS, T, B), generator=gen)
    mem = [torch.zeros(c["mem_len"], B, c["d_model"], dtype=torch.float64)
           for _ in range(c["n_layer"])]
    out = {"cfg_json": np.array(json.dumps(c)),
           "ids": ids.numpy().astype(np.int32), "targets": targets.numpy().astype(np.int32)}
    for k, p in params.items():
        out[f"p0/{k}"] = p.numpy().astype(np.float32)
    probs, losses = [], []
    for s in range(STEPS):
        r = tt.train_step(params, moments, c, ids[s], targets[s], mem, c["lr"])
        mem = r["mem"]
        probs.append(r["probs"].numpy().astype(np.float32))
        losses.append(r["loss"])
        for k in params:
            out[f"g{s}/{k}"] = r["grads"][k].numpy().astype(np.float32)
            out[f"p{s+1}/{k}"] = params[k].detach().numpy().astype(np.float32)
        out[f"mem{s+1}"] = torch.stack(mem).numpy().astype(np.float32)
    out["probs"] = np.stack(probs)
    out["loss"] = np.array(losses, dtype=np.float64)
    path = os.path.join(out_dir, f"trf_{name}.npz")
    np.savez_compressed(path, **out)
    print(f"{path}: {os.path.getsize(path)} bytes, loss {losses}")


# BASELINE.json geometries (config[0] exactly; config[2]'s widths with one layer and four streams)
DIGESTS = {
    "c0": dict(n_layer=2, d_model=128, n_head=4, d_key=32, d_inner=512, d_pos=64, mem_len=32, seg_len=32,
               n_streams=4, n_symbols=256, lr=3e-4, wscale=0.09, param_seed=1001, steps=2),
    "c2_geometry": dict(n_layer=1, d_model=512, n_head=8, d_key=64, d_inner=2048, d_pos=128, mem_len=64,
                        seg_len=64, n_streams=4, n_symbols=16384, lr=3e-4, wscale=0.044, param_seed=1002,
                        steps=2),
}
N_COLS = 48


def make_digest(name, over, out_dir):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from oracle import oracle as orc
    import seeded_params as sp
    c = dict(BASE)
    c.update(over)
    steps = c.pop("steps")
    c["d_value"] = c["d_key"]
    shapes = tt.param_shapes(c)
    p32 = sp.seeded_params(orc, shapes, c["param_seed"], c["wscale"])
    params = {k: torch.from_numpy(v).double() for k, v in p32.items()}
    moments = {k: torch.zeros_like(v) for k, v in params.items()}
    T, B, V = c["seg_len"], c["n_streams"], c["n_symbols"]
    gen = torch.Generator().manual_seed(c["param_seed"])
    ids = torch.randint(0, V, (steps, T, B), generator=gen)
    targets = torch.randint(0, V, (steps, T, B), generator=gen)
    cols = torch.randperm(V, generator=gen)[:N_COLS].sort().values
    mem = [torch.zeros(c["mem_len"], B, c["d_model"], dtype=torch.float64) for _ in range(c["n_layer"])]
    out = {"cfg_json": np.array(json.dumps(c)), "ids": ids.numpy().astype(np.int32),
           "targets": targets.numpy().astype(np.int32), "prob_cols": cols.numpy().astype(np.int32)}
    losses, ps, pt, pmax = [], [], [], []
    for s in range(steps):
        r = tt.train_step(params, moments, c, ids[s], targets[s], mem, c["lr"])
        mem = r["mem"]
        losses.append(r["loss"])
        ps.append(r["probs"][..., cols].numpy().astype(np.float32))
        pt.append(torch.gather(r["probs"], 2, targets[s].unsqueeze(-1)).squeeze(-1).numpy().astype(np.float32))
        pmax.append(r["probs"].max(-1).values.numpy().astype(np.float32))
        for k in params:
            g = r["grads"][k].numpy()
            stride, sub = sp.subsample(g)
            out[f"stride/{k}"] = np.array(stride, np.int64)
            out[f"g{s}/{k}"] = sub.astype(np.float32)
            out[f"gmax{s}/{k}"] = np.array(np.abs(g).max(), np.float32)
            out[f"p{s+1}/{k}"] = sp.subsample(params[k].detach().numpy())[1].astype(np.float32)
        # later steps start from the stored-precision state the tests can rebuild: keep going in
        # float64 here; the tests re-synchronise their weights only through these subsamples
    out["probs_sample"] = np.stack(ps)
    out["probs_target"] = np.stack(pt)
    out["probs_rowmax"] = np.stack(pmax)
    out["loss"] = np.array(losses, dtype=np.float64)
    path = os.path.join(out_dir, f"dig_{name}.npz")
    np.savez_compressed(path, **out)
    print(f"{path}: {os.path.getsize(path)} bytes, loss {losses}")


if __name__ == "__main__":
    torch.manual_seed(0)
    d = os.path.dirname(os.path.abspath(__file__))
    if len(sys.argv) > 1 and sys.argv[1] == "digest":
        for n, o in DIGESTS.items():
            make_digest(n, o, d)
    elif len(sys.argv) > 2 and sys.argv[1] == "only":   # python make_golden.py only <name> ...
        for n in sys.argv[2:]:
            make(n, CONFIGS[n], d)
    else:
        for n, o in CONFIGS.items():
            make(n, o, d)
