"""Plain, slow restatement of the Filinex layer-list family (dnet_b200/core/models/seqmix.py) in float64 on the CPU.

One function per mechanism, whole sequences only: no cache, no page, no carried state.  Whatever the product
computes through portions, batches, pages and slots has to equal what these functions give for the whole token
list.  Notation: T tokens, W width, H heads, G key heads, dk / dv key / value size per head, E experts.
Nothing here is imported by the product, and nothing of the product is imported here.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def dyt(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """dynamic tanh: tanh(alpha x) * weight + bias, elementwise (no statistics of x enter)"""
    return torch.tanh(w[name + ".alpha"].to(F) * x) * w[name].to(F) + w[name + ".b"].to(F)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x @ w.to(F).T


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: float,
                   sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv].  Causal, no positions; scores are scaled, then capped
    by cap * tanh(s / cap); the softmax denominator holds one more term exp(sink_h) that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)
    ok = i[None, :] <= i[:, None]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap and softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~ok, float("-inf"))
        if sink is not None:
            s = torch.cat([s, sink[h].to(F).expand(T, 1)], dim=1)
            p = torch.softmax(s, -1)[:, :T]
        else:
            p = torch.softmax(s, -1)
        out[:, h] = p @ v[:, g]
    return out


def decayed_outer_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                             bonus: Optional[torch.Tensor]) -> torch.Tensor:
    """One head.  q, k, decay [T, dk]; v [T, dv]; bonus [dk] or None.
    Without bonus:  M <- diag(decay_t) M + k_t v_t^T;  o_t = M^T q_t                      (read after the write)
    With bonus:     o_t = (M + diag(bonus) k_t v_t^T)^T q_t;  M <- diag(decay_t) M + k_t v_t^T   (read before it)"""
    T, dk = q.shape
    M = torch.zeros(dk, v.shape[1], dtype=F)
    o = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        kv = k[t][:, None] * v[t][None, :]
        if bonus is None:
            M = decay[t][:, None] * M + kv
            o[t] = M.T @ q[t]
        else:
            o[t] = (M + bonus[:, None] * kv).T @ q[t]
            M = decay[t][:, None] * M + kv
    return o


def mixer_parallel(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    L, R = mx["left"], mx["right"]
    # left: softmax attention with a sink, capped scores and a per-head output gate
    H, G, dk, dv = L["heads"], L.get("kv_heads", L["heads"]), L["dim"], L.get("vdim", L["dim"])
    q = lin(h, w[p + "left.q"]).view(T, H, dk)
    k = lin(h, w[p + "left.k"]).view(T, G, dk)
    v = lin(h, w[p + "left.v"]).view(T, G, dv)
    o = sink_attention(q, k, v, L["scale"], L.get("softcap", 0.0), w.get(p + "left.sink"))
    o = o * torch.sigmoid(lin(h, w[p + "left.g"]))[:, :, None]
    left = lin(o.reshape(T, H * dv), w[p + "left.o"])
    # right: gated linear attention, one decay per key channel
    H, dk, dv = R["heads"], R["dim"], R.get("vdim", R["dim"])
    q = (lin(h, w[p + "right.q"]) * dk ** -0.5).view(T, H, dk)
    k = lin(h, w[p + "right.k"]).view(T, H, dk)
    v = lin(h, w[p + "right.v"]).view(T, H, dv)
    z = lin(lin(h, w[p + "right.a1"]), w[p + "right.a2"]) + w[p + "right.a2.b"].to(F)
    decay = torch.sigmoid(z).pow(1.0 / R["tau"]).view(T, H, dk)
    o = torch.stack([decayed_outer_recurrence(q[:, i], k[:, i], v[:, i], decay[:, i], None) for i in range(H)], 1)
    o = rms_unit(o, eps) * w[p + "right.norm"].to(F)
    g = lin(h, w[p + "right.g"])
    right = lin(o.reshape(T, H * dv) * (g * torch.sigmoid(g)), w[p + "right.o"])
    return mx.get("left_scale", 1.0) * left + mx.get("right_scale", 1.0) * right


def mixer_wkv(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dk = mx["heads"], mx["dim"]
    dv = w[p + "v"].shape[0] // H
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]], 0)
    mix = {s: h + (prev - h) * w[p + "mu." + s].to(F) for s in "rkvgw"}
    r = lin(mix["r"], w[p + "r"]).view(T, H, dk)
    k = lin(mix["k"], w[p + "k"]).view(T, H, dk)
    v = lin(mix["v"], w[p + "v"]).view(T, H, dv)
    g = lin(mix["g"], w[p + "g"])
    gate = g * torch.sigmoid(g)
    decay = torch.exp(-torch.exp(lin(torch.tanh(lin(mix["w"], w[p + "w1"])), w[p + "w2"]) + w[p + "w0"].to(F))).view(T, H, dk)
    u = w[p + "u"].to(F).view(H, dk)
    o = torch.stack([decayed_outer_recurrence(r[:, i], k[:, i], v[:, i], decay[:, i], u[i]) for i in range(H)], 1)
    o = rms_unit(o, eps).reshape(T, H * dv) * w[p + "norm"].to(F) * gate
    return lin(o, w[p + "o"])


def clamped_glu_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(lin(h, w[p + "gate"]), max=limit)
    u = torch.clamp(lin(h, w[p + "up"]), -limit, limit)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = lin(h, w[p + "router"]) + w[p + "router.b"].to(F)
    val, idx = torch.topk(z, top, dim=-1)
    pw = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += pw[t, j] * clamped_glu_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_glu_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def layer_runs(cfg: dict) -> List[dict]:
    """the order in which layers run: (layer index, whether a new pass of the loop starts before it)"""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [{"layer": i, "inject": False} for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    runs = [{"layer": i, "inject": False} for i in range(a)]
    for _ in range(times):
        runs += [{"layer": i, "inject": i == a} for i in range(a, b)]
    runs += [{"layer": i, "inject": False} for i in range(b, n)]
    return runs


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of one whole sequence; layers_out collects the residual after every layer run"""
    eps = cfg["norm"]["eps"]
    x = w["embed"].to(F)[torch.tensor(tokens)]
    x = dyt(x, w, "embed.norm")
    x0 = x
    for run in layer_runs(cfg):
        i = run["layer"]
        L = cfg["layers"][i]
        p = f"l{i}."
        if run["inject"]:
            x = lin(torch.cat([x, x0], -1), w["loop.in"])
        h = dyt(x, w, p + "norm1")
        if L["type"] == "parallel":
            y = mixer_parallel(h, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "wkv":
            y = mixer_wkv(h, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + dyt(y, w, p + "norm1b")
        if L.get("mlp"):
            x = x + dyt(moe(dyt(x, w, p + "norm2"), w, p + "mlp.", L["mlp"]), w, p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    z = lin(dyt(x, w, "final.norm"), w["head"])
    cap = cfg.get("logit_softcap", 0.0)
    return cap * torch.tanh(z / cap) if cap and cap > 0 else z


def tensor_shapes(cfg: dict, rank: int = 8) -> Dict[str, tuple]:
    """every tensor of a checkpoint of this family; `rank` is the inner size of the two-step decay projections"""
    W, V = cfg["width"], cfg["vocab"]
    s: Dict[str, tuple] = {"embed": (V, W), "head": (V, W)}

    def norm(n):
        s[n], s[n + ".b"], s[n + ".alpha"] = (W,), (W,), ()

    norm("embed.norm")
    norm("final.norm")
    if cfg.get("loop"):
        s["loop.in"] = (W, 2 * W)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        norm(p + "norm1")
        norm(p + "norm1b")
        mx = L["mixer"]
        if L["type"] == "parallel":
            a, b = mx["left"], mx["right"]
            H, G, dk, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            s[p + "mix.left.q"], s[p + "mix.left.k"], s[p + "mix.left.v"] = (H * dk, W), (G * dk, W), (G * dv, W)
            s[p + "mix.left.sink"], s[p + "mix.left.g"], s[p + "mix.left.o"] = (H,), (H, W), (W, H * dv)
            H, dk, dv = b["heads"], b["dim"], b.get("vdim", b["dim"])
            s[p + "mix.right.q"] = s[p + "mix.right.k"] = (H * dk, W)
            s[p + "mix.right.v"] = s[p + "mix.right.g"] = (H * dv, W)
            s[p + "mix.right.o"], s[p + "mix.right.norm"] = (W, H * dv), (dv,)
            s[p + "mix.right.a1"], s[p + "mix.right.a2"], s[p + "mix.right.a2.b"] = (rank, W), (H * dk, rank), (H * dk,)
        else:
            H, dk = mx["heads"], mx["dim"]
            dv = mx.get("vdim", dk)
            for m in "rkvgw":
                s[p + "mix.mu." + m] = (W,)
            s[p + "mix.r"] = s[p + "mix.k"] = (H * dk, W)
            s[p + "mix.v"] = s[p + "mix.g"] = (H * dv, W)
            s[p + "mix.w1"], s[p + "mix.w2"], s[p + "mix.w0"] = (rank, W), (H * dk, rank), (H * dk,)
            s[p + "mix.u"], s[p + "mix.norm"], s[p + "mix.o"] = (H, dk), (H * dv,), (W, H * dv)
        mlp = L.get("mlp")
        if mlp:
            norm(p + "norm2")
            norm(p + "norm2b")
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            s[p + "mlp.router"], s[p + "mlp.router.b"] = (E, W), (E,)
            for e in range(E):
                s[f"{p}mlp.e{e}.gate"] = s[f"{p}mlp.e{e}.up"] = (ff, W)
                s[f"{p}mlp.e{e}.down"] = (W, ff)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                s[p + "mlp.shared.gate"] = s[p + "mlp.shared.up"] = (sf, W)
                s[p + "mlp.shared.down"] = (W, sf)
    return s


def random_weights(cfg: dict, seed: int = 0, rank: int = 8) -> Dict[str, torch.Tensor]:
    """random bf16-representable weights whose activations stay of order one through every layer"""
    g = torch.Generator().manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        leaf = name.split(".")[-1]
        if name.endswith(".alpha"):
            t = torch.tensor(0.5 + 0.5 * float(torch.rand((), generator=g)))
        elif name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2") or name.endswith("norm1b") or name.endswith("norm2b"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "b" or leaf in ("sink", "w0", "u") or ".mu." in name:
            t = 0.5 * torch.randn(shape, generator=g) if ".mu." not in name else torch.rand(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w
