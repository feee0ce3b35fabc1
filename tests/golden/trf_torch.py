"""PyTorch (CPU, autograd) restatement of NNCP's Transformer-XL train step.

Test infrastructure only: it exists to produce the committed golden vectors
(make_golden.py) that pin the C oracle's hand-written backward pass.  It
follows the reference graph op by op:

  forward            nncp.c:581-1029   (trf_eval, batched mode)
  loss / objective   nncp.c:1170-1175  (sum ln p[target]; objective -loss/(T*B))
  memory shift       nncp.c:1205-1221  (mem_update)
  optimizer          RMSProp as this build defines it (LibNC's Adam internals
                     are not in the reference tree): v = b2*v + (1-b2)*g^2,
                     w -= lr*g/(sqrt(v)+eps)

Tensors are time-major: activations [T, B, D], memory [M, B, D], ids [T, B].
Weights are [out, in]; w_r is [H, P, dk]; b_r is [H, L].
"""
import math

import torch

LN_POST, LN_PRE, LN_FINAL, LN_COEF, LN_RMSNORM = 1, 2, 4, 8, 16
FF_RELU, FF_GELU, FF_GEGLU, FF_GATED_SILU = 0, 1, 2, 3


def param_shapes(c):
    """Parameter names (nncp.c:371-497 naming) and shapes, in flat-buffer order."""
    D, H, dk, F, P = c["d_model"], c["n_head"], c["d_key"], c["d_inner"], c["d_pos"]
    L = c["mem_len"] + c["seg_len"]
    V = c["n_symbols"]
    F1 = 2 * F if c["ff_act"] in (FF_GEGLU, FF_GATED_SILU) else F
    out = []
    for l in range(c["n_layer"]):
        out.append((f"w_q_{l}", (H * dk, D)))
        out.append((f"w_kv_{l}", (2 * H * dk, D)))
        if c["query_bias"]:
            out.append((f"b_q_{l}", (H * dk,)))
        out.append((f"w_o_{l}", (D, H * dk)))
        out.append((f"ff1_{l}", (F1, D)))
        if c["use_bias"]:
            out.append((f"ff_bias1_{l}", (F1,)))
        out.append((f"ff2_{l}", (D, F)))
        if c["use_bias"]:
            out.append((f"ff_bias2_{l}", (D,)))
        if c["use_w_r"] and (l == 0 or not c["tied_w_r"]):
            out.append((f"w_r_{l}", (H, P, dk)))
        if l == 0 or not c["tied_b_r"]:
            out.append((f"b_r_{l}", (H, L)))
        if c["ln_flags"] & (LN_POST | LN_PRE):
            out.append((f"ln_g_{2 * l}", (D,)))
            out.append((f"ln_b_{2 * l}", (D,)))
            out.append((f"ln_g_{2 * l + 1}", (D,)))
            out.append((f"ln_b_{2 * l + 1}", (D,)))
        if c["ln_flags"] & LN_COEF:
            out.append((f"alpha_{l}", (1,)))
    if c["ln_flags"] & LN_FINAL:
        out.append((f"ln_g_{2 * c['n_layer']}", (D,)))
        out.append((f"ln_b_{2 * c['n_layer']}", (D,)))
    out.append(("embed", (V, D)))
    out.append(("embed_out", (V, D)))
    if c["use_bias"]:
        out.append(("out_bias", (V,)))
    return out


def norm(x, g, b, flags):
    """layer_norm(), nncp.c:279-288; eps 1e-5 inside the square root."""
    if flags & LN_RMSNORM:
        xn = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5)
    else:
        mu = x.mean(-1, keepdim=True)
        xc = x - mu
        xn = xc * torch.rsqrt((xc * xc).mean(-1, keepdim=True) + 1e-5)
    return xn * g + b


def gelu(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def attention(q, k, v, w_r, b_r, c, attn_len, t0=0):
    """nncp.c:722-800 for queries t0..t0+Tq-1.  q [Tq,B,H,dk]; k, v [L,B,H,dk]."""
    Tq, B, H, dk = q.shape
    L = k.shape[0]
    T, M, P, D = c["seg_len"], c["mem_len"], c["d_pos"], c["d_model"]
    sc = torch.einsum("ibhd,jbhd->bhij", q, k)
    i = torch.arange(t0, t0 + Tq).view(Tq, 1)
    j = torch.arange(L).view(1, L)
    r = j + (T - 1) - i                       # nc_rel_shift(-(T-1), 1), nncp.c:784
    valid = r < L
    rc = r.clamp(max=L - 1)
    z = (math.sqrt(dk * D) * b_r).view(1, H, 1, L).expand(B, H, Tq, L)   # nncp.c:751-757
    if w_r is not None:
        e = torch.einsum("ibhd,hpd->bhip", q, w_r)       # nncp.c:775-776
        pad_idx = (torch.arange(L) - (L - P)).clamp(min=0)  # nc_pad NC_PAD_DUP, nncp.c:777
        z = z + e[..., pad_idx]
    sp = torch.gather(z, 3, rc.view(1, 1, Tq, L).expand(B, H, Tq, L))
    sp = torch.where(valid.view(1, 1, Tq, L), sp, torch.zeros_like(sp))
    a = (sc + sp) * (1.0 / math.sqrt(dk))               # nncp.c:789
    pos = (i + M) - j
    masked = ~((pos >= 0) & (pos < attn_len))            # nncp.c:357-361
    a = a.masked_fill(masked.view(1, 1, Tq, L), float("-inf"))
    p = torch.softmax(a, dim=-1)
    return torch.einsum("bhij,jbhd->ibhd", p, v)


def forward(params, c, ids, mem):
    """ids [T,B] long; mem list of [M,B,D].  Returns (probs [T,B,V], new layer inputs)."""
    T, B = ids.shape
    D, H, dk = c["d_model"], c["n_head"], c["d_key"]
    fl = c["ln_flags"]
    L = c["mem_len"] + T
    x = params["embed"][ids] * (math.sqrt(D) * c["embed_mult"])       # nncp.c:625-630
    train_h = []
    for l in range(c["n_layer"]):
        g = lambda n: params[f"{n}_{l}"]
        x1 = norm(x, params[f"ln_g_{2*l}"], params[f"ln_b_{2*l}"], fl) if fl & LN_PRE else x
        train_h.append(x1.detach())
        q = x1 @ g("w_q").T
        if c["query_bias"]:
            q = q + g("b_q")
        hcat = torch.cat([mem[l], x1], 0)          # no gradient into mem (nncp.c:676-695)
        kv = hcat @ g("w_kv").T
        k, v = kv[..., : H * dk], kv[..., H * dk:]
        wr_l = 0 if c["tied_w_r"] else l
        br_l = 0 if c["tied_b_r"] else l
        w_r = params[f"w_r_{wr_l}"] if c["use_w_r"] else None
        alen = c["attn_len"][l] if c["attn_len"][l] else L
        o = attention(q.view(T, B, H, dk), k.reshape(L, B, H, dk), v.reshape(L, B, H, dk),
                      w_r, params[f"b_r_{br_l}"], c, alen)
        y = o.reshape(T, B, H * dk) @ g("w_o").T
        if fl & LN_COEF:
            y = y * g("alpha")                                        # nncp.c:892-894
        y = y + x                                                     # nncp.c:872, 896
        if fl & LN_POST:
            y = norm(y, params[f"ln_g_{2*l}"], params[f"ln_b_{2*l}"], fl)
        u = norm(y, params[f"ln_g_{2*l+1}"], params[f"ln_b_{2*l+1}"], fl) if fl & LN_PRE else y
        h = u @ g("ff1").T
        if c["use_bias"]:
            h = h + g("ff_bias1")
        if c["ff_act"] == FF_RELU:
            h = torch.relu(h)
        elif c["ff_act"] == FF_GELU:
            h = gelu(h)
        elif c["ff_act"] == FF_GEGLU:
            F = c["d_inner"]
            h = gelu(h[..., :F]) * h[..., F:]                         # nncp.c:945-951
        else:
            F = c["d_inner"]
            h = h[..., :F] * torch.sigmoid(h[..., :F]) * h[..., F:]   # nncp.c:957-962
        z = h @ g("ff2").T
        if c["use_bias"]:
            z = z + g("ff_bias2")
        if fl & LN_COEF:
            z = z * g("alpha")                                        # nncp.c:975-977
        x = z + y                                                     # nncp.c:979
        if fl & LN_POST:
            x = norm(x, params[f"ln_g_{2*l+1}"], params[f"ln_b_{2*l+1}"], fl)
    if fl & LN_FINAL:
        n = 2 * c["n_layer"]
        x = norm(x, params[f"ln_g_{n}"], params[f"ln_b_{n}"], fl)
    logits = x @ params["embed_out"].T
    if c["use_bias"]:
        logits = logits + params["out_bias"]
    return torch.softmax(logits, -1), train_h


def mem_update(mem, train_h, c):
    M, T = c["mem_len"], c["seg_len"]
    out = []
    for m, h in zip(mem, train_h):
        if M > T:
            out.append(torch.cat([m[T:], h], 0))
        else:
            out.append(h[T - M:].clone())
    return out


def train_step(params, moments, c, ids, targets, mem, lr, n_streams_total=None):
    """One eval + gradient + RMSProp update + memory shift.  Returns dict of results."""
    T, B = ids.shape
    Bt = n_streams_total or B
    for p in params.values():
        p.requires_grad_(True)
        p.grad = None
    probs, train_h = forward(params, c, ids, mem)
    logp = torch.log(torch.gather(probs, 2, targets.unsqueeze(-1)))
    loss = logp.sum()
    (loss * (-1.0 / (T * Bt))).backward()
    grads = {k: (p.grad.detach().clone() if p.grad is not None else torch.zeros_like(p))
             for k, p in params.items()}
    b2, eps = c["beta2"], c["eps"]
    with torch.no_grad():
        for k, p in params.items():
            g = grads[k]
            if c.get("gradient_clip", 0.0):
                g = g.clamp(-c["gradient_clip"], c["gradient_clip"])
            moments[k].mul_(b2).add_((1 - b2) * g * g)
            p.sub_(lr * g / (moments[k].sqrt() + eps))
    for p in params.values():
        p.requires_grad_(False)
    return {"probs": probs.detach(), "loss": float(loss.detach()), "grads": grads,
            "mem": mem_update(mem, train_h, c)}
