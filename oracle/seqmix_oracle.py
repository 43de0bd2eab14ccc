"""Plain, slow restatement of the layer-list model families (dnet_b200/core/models/seqmix.py) in float64 on the CPU.

One function per mechanism, whole sequences only: there is no cache, no page and no carried state here, so whatever
the product computes through portions, batches, pages and slots has to equal what these functions give for the whole
token list.  Notation: T tokens, W width, H heads, G key heads, dk / dv key / value size per head, S streams.
Nothing here is imported by the product, and nothing of the product is imported here.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def short_conv(u: torch.Tensor, w: Optional[torch.Tensor]) -> torch.Tensor:
    """depthwise causal FIR over time: y[t, c] = sum_j w[c, j] u[t - (J-1) + j, c], zeros before t = 0.  u [T, C], w [C, J]"""
    if w is None:
        return u
    T, C = u.shape
    J = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(J):
            src = t - (J - 1) + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def rotate_pairs(z: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """z [T, heads, d]: dims (2i, 2i+1), i < dims/2, turn by positions * base^(-2i/dims); the rest pass"""
    if dims <= 0:
        return z
    out = z.clone()
    for i in range(dims // 2):
        ang = positions.to(F) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = z[..., 2 * i], z[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def visible(T: int, block: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff j <= i and (no block or both lie in the same block of `block` positions)"""
    i = torch.arange(T)
    ok = i[None, :] <= i[:, None]
    if block > 0:
        ok &= (i[None, :] // block) == (i[:, None] // block)
    return ok


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, block: int) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; head h reads key head h // (H/G)"""
    T, H, _ = q.shape
    G = k.shape[1]
    ok = visible(T, block)
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """q, k [T, dk]; v [T, dv]; beta, decay [T].  M <- decay M;  M <- M + k (beta (v - M^T k))^T;  o = M^T q"""
    T, dk = q.shape
    M = torch.zeros(dk, v.shape[1], dtype=F)
    o = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        M = decay[t] * M
        M = M + torch.outer(k[t], beta[t] * (v[t] - M.T @ k[t]))
        o[t] = M.T @ q[t]
    return o


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gated_ff(h: torch.Tensor, Wg: torch.Tensor, Wu: torch.Tensor, Wd: torch.Tensor) -> torch.Tensor:
    return (gelu_tanh(h @ Wg.T) * (h @ Wu.T)) @ Wd.T


def streams_read(xs: List[torch.Tensor], w_in: Optional[torch.Tensor]) -> torch.Tensor:
    return xs[0] if w_in is None else sum(w_in[s] * xs[s] for s in range(len(xs)))


def streams_write(xs: List[torch.Tensor], y: torch.Tensor, mix: Optional[torch.Tensor], w_out: Optional[torch.Tensor]) -> List[torch.Tensor]:
    """x_t <- sum_s mix[s, t] x_s + out[t] y; without streams x <- x + y"""
    if mix is None:
        return [xs[0] + y]
    S = len(xs)
    return [sum(mix[s, t] * xs[s] for s in range(S)) + w_out[t] * y for t in range(S)]


def attention_mixer(h, W, p, mx, eps, positions, kv_store, li):
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
    rot = mx.get("rot") or {}
    rd, rb = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    q = short_conv(h @ W[p + "mix.q"].T, W.get(p + "mix.q.conv"))
    q = rotate_pairs((rms_unit(q, eps) * W[p + "mix.q.norm"]).reshape(T, H, dk), positions, rd, rb)
    if mx.get("kv_from") is not None:
        k, v = kv_store[int(mx["kv_from"])]
    else:
        k = short_conv(h @ W[p + "mix.k"].T, W.get(p + "mix.k.conv"))
        k = rotate_pairs((rms_unit(k, eps) * W[p + "mix.k.norm"]).reshape(T, G, dk), positions, rd, rb)
        v = short_conv(h @ W[p + "mix.v"].T, W.get(p + "mix.v.conv")).reshape(T, G, dv)
        kv_store[li] = (k, v)
    o = softmax_attention(q, k, v, float(mx.get("scale", dk ** -0.5)), int((mx.get("mask") or {}).get("size", 0)))
    return o.reshape(T, H * dv) @ W[p + "mix.o"].T


def delta_mixer(h, W, p, mx, eps):
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
    q = silu(short_conv(h @ W[p + "mix.q"].T, W.get(p + "mix.q.conv"))).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "mix.k"].T, W.get(p + "mix.k.conv"))).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "mix.v"].T, W.get(p + "mix.v.conv"))).reshape(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "mix.b"].T)
    decay = torch.exp(-torch.exp(W[p + "mix.A_log"]) * torch.nn.functional.softplus(h @ W[p + "mix.a"].T + W[p + "mix.dt_bias"]))
    o = torch.stack([delta_rule(q[:, hh // (H // G)], k[:, hh // (H // G)], v[:, hh], beta[:, hh], decay[:, hh]) for hh in range(H)], 1)
    o = rms_unit(o, eps) * W[p + "mix.norm"] * silu(h @ W[p + "mix.g"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + "mix.o"].T


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] (float64) of one whole sequence; layers_out collects the residual after every layer"""
    W = {k: v.to(F) for k, v in weights.items()}
    eps = float((cfg.get("norm") or {}).get("eps", 1e-6))
    S = int(cfg.get("streams", 0) or 0)
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(tok))
    x0 = W["embed"][tok] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    xs = [x0.clone() for _ in range(max(S, 1))]
    kv_store: dict = {}
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = rms_unit(streams_read(xs, W[p + "hc1.in"] if S else None), eps) * (1.0 + W[p + "norm1"])
        if L["type"] == "attention":
            y = attention_mixer(h, W, p, L["mixer"], eps, positions, kv_store, li)
        else:
            y = delta_mixer(h, W, p, L["mixer"], eps)
        xs = streams_write(xs, y, W[p + "hc1.mix"] if S else None, W[p + "hc1.out"] if S else None)
        if L.get("mlp"):
            h = rms_unit(streams_read(xs, W[p + "hc2.in"] if S else None), eps) * (1.0 + W[p + "norm2"])
            y = gated_ff(h, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
            xs = streams_write(xs, y, W[p + "hc2.mix"] if S else None, W[p + "hc2.out"] if S else None)
        if layers_out is not None:
            layers_out.append(sum(xs))
    return (rms_unit(sum(xs), eps) * (1.0 + W["final.norm"])) @ W["head"].T


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """checkpoint name -> shape for a config"""
    Wd, V, S = cfg["width"], cfg["vocab"], int(cfg.get("streams", 0) or 0)
    out = {"embed": (V, Wd), "final.norm": (Wd,), "head": (V, Wd)}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        H, G, dk, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
        att = L["type"] == "attention"
        cq, ck, cv = (H if att else G) * dk, G * dk, (G if att else H) * dv
        own = not (att and mx.get("kv_from") is not None)
        J = int(mx.get("conv", 0) or 0)
        out[p + "norm1"] = (Wd,)
        out[p + "mix.q"], out[p + "mix.o"] = (cq, Wd), (Wd, H * dv)
        if own:
            out[p + "mix.k"], out[p + "mix.v"] = (ck, Wd), (cv, Wd)
        if J:
            out[p + "mix.q.conv"] = (cq, J)
            if own:
                out[p + "mix.k.conv"], out[p + "mix.v.conv"] = (ck, J), (cv, J)
        if att:
            out[p + "mix.q.norm"] = (cq,)
            if own:
                out[p + "mix.k.norm"] = (ck,)
        else:
            out[p + "mix.a"] = out[p + "mix.b"] = (H, Wd)
            out[p + "mix.g"] = (H * dv, Wd)
            out[p + "mix.A_log"] = out[p + "mix.dt_bias"] = (H,)
            out[p + "mix.norm"] = (dv,)
        if L.get("mlp"):
            F_ = L["mlp"]["ff"]
            out[p + "norm2"] = (Wd,)
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (F_, Wd)
            out[p + "mlp.down"] = (Wd, F_)
        for qn in (("hc1", "hc2") if L.get("mlp") else ("hc1",)) if S else ():
            out[p + qn + ".in"] = out[p + qn + ".out"] = (S,)
            out[p + qn + ".mix"] = (S, S)
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bf16 weights whose activations stay O(1) through the layers: projections ~ N(0, 1/fan_in), norm weights and
    stream mixes near their neutral values, conv taps and gates of order one"""
    g = torch.Generator().manual_seed(seed)
    S = int(cfg.get("streams", 0) or 0)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        r = torch.randn(shape, generator=g, dtype=torch.float32)
        if leaf in ("norm1", "norm2", "final.norm"):
            t = 0.1 * r
        elif leaf in ("mix.q.norm", "mix.k.norm", "mix.norm"):
            t = 1.0 + 0.1 * r
        elif leaf.endswith(".conv"):
            t = 0.5 * r
        elif leaf == "mix.A_log":
            t = -1.0 + 0.5 * r
        elif leaf == "mix.dt_bias":
            t = 0.5 * r
        elif leaf.endswith(".in"):
            t = 1.0 / S + 0.1 * r
        elif leaf.endswith(".out"):
            t = 1.0 + 0.1 * r
        elif leaf.endswith(".mix"):
            t = torch.eye(S) + 0.1 * r
        elif leaf == "embed":
            t = r
        else:
            t = r / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
