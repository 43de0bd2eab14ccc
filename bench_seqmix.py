"""bench_seqmix.py -- `bench.py --config seqmix`: prefill and decode throughput of a layer-list model (Moputar:
chunk-masked attention, attention that reads an earlier layer's pages, gated delta rule, S residual streams) beside
the llama family at equal width, heads, feed-forward width and depth.  Random weights, synthetic tokens, one GPU.

Per size it reports
  * prefill: one P-token prompt in one step (tokens / second), device time by CUDA events, L2 flushed between steps;
  * decode: one token per step at the end of a P-token context (four sequences: P / 4 tokens each);
  * the device time of every phase of the step (the library's phase timers) next to the llama family's per-kernel
    times (dn_layer_forward_timed), each with its algorithmic FLOPs or bytes and the fraction of the measured peak.
"""
from __future__ import annotations

import ctypes as C

SIZES = {
    "1k": dict(width=1024, heads=8, kv_heads=2, ff=4096),
    "2k": dict(width=2048, heads=16, kv_heads=4, ff=8192),
    "4k": dict(width=4096, heads=32, kv_heads=8, ff=14336),
}
HD = 128
VOCAB = 32768
PATTERN = ("attention", "attention_shared", "delta")


def moputar_config(sz: dict, repeats: int, chunk: int, streams: int) -> dict:
    layers = []
    for r in range(repeats):
        base = len(layers)
        for kind in PATTERN:
            if kind == "delta":
                mixer = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": HD, "vdim": HD, "conv": 4}
                layers.append({"type": "delta", "mixer": mixer, "mlp": {"kind": "dense", "ff": sz["ff"]}})
                continue
            mixer = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": HD, "vdim": HD, "conv": 4, "scale": HD ** -0.5,
                     "rot": {"base": 500000.0, "dims": 64}, "mask": {"size": chunk}}
            if kind == "attention_shared":
                mixer["kv_from"] = base
            layers.append({"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": sz["ff"]}})
    return {"architecture": "Moputar", "vocab": VOCAB, "width": sz["width"], "streams": streams, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.0}, "layers": layers}


def llama_config(sz: dict, n_layers: int) -> dict:
    return dict(hidden_size=sz["width"], num_attention_heads=sz["heads"], num_key_value_heads=sz["kv_heads"], head_dim=HD,
                intermediate_size=sz["ff"], vocab_size=VOCAB, num_hidden_layers=n_layers, rms_norm_eps=1e-5, rope_theta=500000.0,
                model_type="llama", tie_word_embeddings=False, torch_dtype="bfloat16")


def _rand(shape, g, std, dev):
    import torch

    return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(torch.bfloat16).contiguous()


def moputar_weights(model, g, dev):
    import torch

    items = []
    S = int(model._cfg_struct.streams)
    for name, shape in model.expected_tensors().items():
        leaf = name.split(".", 1)[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        elif leaf in ("mix.q.norm", "mix.k.norm", "mix.norm"):
            t = torch.ones(shape, dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".in"):
            t = torch.full(shape, 1.0 / max(1, S), dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".out"):
            t = torch.full(shape, 0.5, dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".mix"):
            t = (torch.eye(shape[0], device=dev) * 0.9 + 0.1 / shape[0]).to(torch.bfloat16).contiguous()
        elif leaf in ("mix.A_log", "mix.dt_bias"):
            t = _rand(shape, g, 0.5, dev)
        elif leaf.endswith(".conv"):
            t = _rand(shape, g, 0.5, dev)
        elif name == "embed":
            t = _rand(shape, g, 1.0, dev)
        else:
            t = _rand(shape, g, shape[-1] ** -0.5, dev)
        items.append((name, t))
    return items


def llama_weights(cfg: dict, g, dev):
    import torch

    W, H, G, F, V = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    w = {"model.embed_tokens.weight": _rand((V, W), g, 1.0, dev), "model.norm.weight": torch.ones(W, dtype=torch.bfloat16, device=dev),
         "lm_head.weight": _rand((V, W), g, W ** -0.5, dev)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = _rand((H * HD, W), g, W ** -0.5, dev)
        w[p + "self_attn.k_proj.weight"] = _rand((G * HD, W), g, W ** -0.5, dev)
        w[p + "self_attn.v_proj.weight"] = _rand((G * HD, W), g, W ** -0.5, dev)
        w[p + "self_attn.o_proj.weight"] = _rand((W, H * HD), g, (H * HD) ** -0.5, dev)
        w[p + "mlp.gate_proj.weight"] = _rand((F, W), g, W ** -0.5, dev)
        w[p + "mlp.up_proj.weight"] = _rand((F, W), g, W ** -0.5, dev)
        w[p + "mlp.down_proj.weight"] = _rand((W, F), g, F ** -0.5, dev)
        w[p + "input_layernorm.weight"] = torch.ones(W, dtype=torch.bfloat16, device=dev)
        w[p + "post_attention_layernorm.weight"] = torch.ones(W, dtype=torch.bfloat16, device=dev)
    return w


class _Flusher:
    """Writes a buffer twice the size of L2 between timed steps."""

    def __init__(self, dev):
        import torch

        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.v = 0

    def __call__(self):
        self.v = (self.v + 1) & 0xFF
        self.buf.fill_(self.v)


def _timed(fn, prep, steps: int, warmup: int, flush) -> float:
    """Median-free mean of `steps` device times (ms) of fn(); prep() runs untimed before each call."""
    import torch

    times = []
    for i in range(warmup + steps):
        prep()
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
    return sum(times) / len(times)


def moputar_algorithmic(cfg: dict, N: int, ctx0: int, n_seqs: int) -> dict:
    """FLOPs and the bytes that must move per phase, for a step of n_seqs entries x (N / n_seqs) tokens whose
    sequences already hold ctx0 tokens each; summed over the layers."""
    W = cfg["width"]
    f = {k: 0.0 for k in ("proj", "attn", "delta_rule", "out_proj", "ff_up", "ff_down", "head")}
    by = dict(f)
    per = N // n_seqs
    for L in cfg["layers"]:
        mx = L["mixer"]
        H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        co = H * dv
        if L["type"] == "attention":
            cols = H * dk + (0 if "kv_from" in mx else G * (dk + dv))
            chunk = mx["mask"]["size"]
            vis = sum((p % chunk) + 1 for p in range(ctx0, ctx0 + per)) * n_seqs
            f["attn"] += 2.0 * (dk + dv) * H * vis
            # keys and values of the visible span are read once per kv head group and step
            span = per + (ctx0 % chunk)
            by["attn"] += 2.0 * n_seqs * span * G * (dk + dv) + 2.0 * N * (H * dk + co)
        else:
            cols = 2 * G * dk + H * dv + 2 * H + co
            f["delta_rule"] += 6.0 * dk * dv * H * N
            by["delta_rule"] += 8.0 * n_seqs * H * dk * dv + 4.0 * N * (2 * G * dk + 2 * H * dv)
        f["proj"] += 2.0 * N * W * cols
        by["proj"] += 2.0 * W * cols
        f["out_proj"] += 2.0 * N * co * W
        by["out_proj"] += 2.0 * co * W
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            f["ff_up"] += 4.0 * N * W * ff
            by["ff_up"] += 4.0 * W * ff
            f["ff_down"] += 2.0 * N * W * ff
            by["ff_down"] += 2.0 * W * ff
    return {"flops": f, "bytes": by}


def llama_algorithmic(cfg: dict, N: int, ctx0: int) -> dict:
    W, H, G, F, L = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    vis = sum(p + 1 for p in range(ctx0, ctx0 + N))
    f = {"proj": 2.0 * N * W * (H + 2 * G) * HD * L, "attn": 4.0 * HD * H * vis * L, "out_proj": 2.0 * N * H * HD * W * L,
         "ff_up": 4.0 * N * W * F * L, "ff_down": 2.0 * N * W * F * L}
    by = {"proj": 2.0 * W * (H + 2 * G) * HD * L, "attn": (4.0 * (ctx0 + N) * G * HD + 4.0 * N * H * HD) * L, "out_proj": 2.0 * H * HD * W * L,
          "ff_up": 4.0 * W * F * L, "ff_down": 2.0 * W * F * L}
    return {"flops": f, "bytes": by}


FP32_PHASES = ("delta_rule",)      # the recurrence is fp32 FMA on the CUDA cores: its compute bound is the fp32 rate


def _roofline(ms: dict, alg: dict, tf_peak: float, gbs_peak: float, f32_tf: float = 0.0) -> dict:
    """Per phase: time, the larger of its compute-bound and its HBM-bound target time, and target / achieved."""
    out = {}
    for k, t in ms.items():
        if k not in alg["flops"] or t <= 0:
            continue
        f32 = k in FP32_PHASES and f32_tf > 0
        t_f = alg["flops"][k] / ((f32_tf if f32 else tf_peak) * 1e12) * 1e3
        t_b = alg["bytes"][k] / (gbs_peak * 1e9) * 1e3
        tgt = max(t_f, t_b)
        out[k] = {"ms": round(t, 4), "target_ms": round(tgt, 4), "bound": ("fp32" if f32 else "tensor") if t_f >= t_b else "hbm",
                  "frac": round(tgt / t, 4)}
    return out


def _run_moputar(sz: dict, args, P: int, flush, dev) -> dict:
    import torch

    from dnet_b200.core.models import get_ring_model

    cfg = moputar_config(sz, args.seqmix_repeats, args.seqmix_chunk, args.seqmix_streams)
    pages = 4 * ((P + 64 + 63) // 64)
    model = get_ring_model("moputar", cfg, assigned_layers=list(range(len(cfg["layers"]))), dtype="bfloat16", kv_pool_pages=pages,
                           max_seqs=4, max_batch_tokens=max(P, 64))
    g = torch.Generator(device=dev).manual_seed(7)
    model.load_weights(moputar_weights(model, g, dev), strict=True)
    assert not model.missing_tensors()
    prompt = torch.randint(0, VOCAB, (P,), generator=torch.Generator().manual_seed(11)).tolist()
    K, Wm = args.steps, args.warmup
    live = []
    st = torch.cuda.current_stream()      # run_seqmix made a side stream current: decode steps replay graphs there

    def fresh(n):
        for h in live:
            h.free()
        live.clear()
        live.extend(model.make_cache(stream=st) for _ in range(n))

    res = {"config": {"layers": [l["type"] + ("<-%d" % l["mixer"]["kv_from"] if "kv_from" in l["mixer"] else "") for l in cfg["layers"]],
                      "streams": cfg["streams"], "chunk": args.seqmix_chunk, "conv": 4, "rot_dims": 64}}
    # prefill: one P-token entry, logits of the last token
    t = _timed(lambda: model.step([(live[0], prompt)], [P - 1], stream=st), lambda: fresh(1), K, Wm, flush)
    res["prefill"] = {"ms": t, "tok_s": P / t * 1e3}
    fresh(1)
    model.profile(True)
    model.step([(live[0], prompt)], [P - 1], stream=st)
    res["prefill"]["phases_ms"] = model.profile_read(reset=True)
    model.profile(False)
    # decode at the end of a P-token context: 1 sequence, then 4 with P / 4 tokens each.  The decoded token sits at
    # the last position of its attention block, so it sees a whole block (or all of the shorter context).
    for n_seq in (1, 4):
        ctx = (P if n_seq == 1 else P // 4) - 1
        fresh(n_seq)
        model.step([(h, prompt[:ctx]) for h in live], [], stream=st)
        toks = [[int(prompt[(i * 7 + 3) % P])] for i in range(n_seq)]
        want = list(range(n_seq))
        t = _timed(lambda: model.step([(h, toks[i]) for i, h in enumerate(live)], want, stream=st), lambda: None, K, Wm, flush)
        key = "decode_bs%d" % n_seq
        res[key] = {"ms": t, "tok_s": n_seq / t * 1e3, "context": ctx}
        model.profile(True)
        for _ in range(4):
            flush()
            model.step([(h, toks[i]) for i, h in enumerate(live)], want, stream=st)
        ph = model.profile_read(reset=True)
        model.profile(False)
        res[key]["phases_ms"] = {k: v / 4 for k, v in ph.items()}
    model.check(st)
    fresh(0)
    launches = int(model._lib.dn_seq_launch_count())
    model.destroy()
    res["cfg"] = cfg
    res["launches"] = launches
    return res


def _run_llama(sz: dict, args, P: int, n_layers: int, flush, dev) -> dict:
    import torch

    from dnet_b200 import _cabi
    from dnet_b200.core.models import get_ring_model

    cfg = llama_config(sz, n_layers)
    layers = list(range(n_layers))
    model = get_ring_model("llama", cfg, assigned_layers=layers, kv_pool_pages=2 * ((P + 128 + 63) // 64) + 8)
    g = torch.Generator(device=dev).manual_seed(7)
    w = llama_weights(cfg, g, dev)
    model.load_weights(w)
    cache = model.make_cache(P + 128)
    ids = torch.randint(0, VOCAB, (P,), generator=torch.Generator().manual_seed(11)).to(dev, torch.int32)
    K, Wm = args.steps, args.warmup
    res = {}

    def prefill():
        x = model.embed(ids)
        model.window_forward(layers, x, cache)
        model.head_logits(x[-1:], want_f32=True, want_bf16=False)

    t = _timed(prefill, lambda: cache.reset(), K, Wm, flush)
    res["prefill"] = {"ms": t, "tok_s": P / t * 1e3}
    # per-kernel times of the same prompt, chunk by chunk as window_forward cuts it
    from dnet_b200.core.models.base import _decompose

    ms5 = (C.c_float * 5)()
    sums = [0.0] * 5
    cache.reset()
    x = model.embed(ids)
    t0 = 0
    for c in _decompose(P, model.max_chunk, model.max_prefill_chunk):
        for li in layers:
            _cabi.check(model._lib.dn_layer_forward_timed(model._h, li, x[t0:t0 + c].data_ptr(), c, cache._h, None, ms5))
            sums = [a + float(b) for a, b in zip(sums, ms5)]
        cache.advance(c)
        t0 += c
    names = ["proj", "attn", "out_proj", "ff_up", "ff_down"]
    res["prefill"]["phases_ms"] = dict(zip(names, sums))
    # decode: one token at a P-token context through the per-layer kernels (the cache holds P tokens now)
    one = ids[:1].clone()

    def decode():
        x1 = model.embed(one)
        model.window_forward(layers, x1, cache)
        model.head_logits(x1, want_f32=True, want_bf16=False)

    t = _timed(decode, lambda: None, K, Wm, flush)
    res["decode_bs1"] = {"ms": t, "tok_s": 1e3 / t, "context": P, "path": "per-layer kernels (dn_window_forward, T = 1)"}
    sums = [0.0] * 5
    x1 = model.embed(one)
    for rep in range(4):
        flush()
        for li in layers:
            _cabi.check(model._lib.dn_layer_forward_timed(model._h, li, x1.data_ptr(), 1, cache._h, None, ms5))
            sums = [a + float(b) for a, b in zip(sums, ms5)]
    res["decode_bs1"]["phases_ms"] = {n: s / 4 for n, s in zip(names, sums)}
    torch.cuda.synchronize()
    cache.free()
    model.destroy()
    res["cfg"] = cfg
    return res


def run_seqmix(args, rank: int, local_rank: int, world: int) -> None:
    import torch

    import bench as B
    from bench import ClockSampler, log

    if world != 1:
        raise SystemExit("--config seqmix runs on one GPU")
    dev = torch.device("cuda", local_rank)
    P = int(args.seqmix_prompt)
    gbs, peak_src = B.peaks()
    tf = B.tensor_peak_tf()
    props = torch.cuda.get_device_properties(dev)
    f32_tf = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12      # fp32 FMA lanes x 2 x the maximum SM clock
    flush = _Flusher(dev)
    side = torch.cuda.Stream(device=dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    import time

    tw0 = time.perf_counter()
    sizes = {}
    launches = 0
    for name in args.seqmix_sizes.split(","):
        sz = SIZES[name]
        with torch.cuda.stream(side):
            mo = _run_moputar(sz, args, P, flush, dev)
        side.synchronize()
        log(f"{name}: moputar prefill {mo['prefill']['ms']:.2f} ms, phases " + ", ".join(f"{k} {v:.2f}" for k, v in mo["prefill"]["phases_ms"].items() if v > 0))
        log(f"{name}: moputar decode bs1 {mo['decode_bs1']['ms']:.3f} ms, phases " + ", ".join(f"{k} {v:.3f}" for k, v in mo["decode_bs1"]["phases_ms"].items() if v > 0))
        ll = _run_llama(sz, args, P, len(mo["cfg"]["layers"]), flush, dev)
        launches += mo.pop("launches")
        mcfg, lcfg = mo.pop("cfg"), ll.pop("cfg")
        for key in ("prefill", "decode_bs1", "decode_bs4"):
            n_seq = 4 if key.endswith("4") else 1
            if key == "prefill":
                N, ctx0 = P, 0
            else:
                N, ctx0 = n_seq, mo[key]["context"]
            mo[key]["roofline"] = _roofline(mo[key]["phases_ms"], moputar_algorithmic(mcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            if key in ll:
                ll[key]["roofline"] = _roofline(ll[key]["phases_ms"], llama_algorithmic(lcfg, N, ctx0), tf, gbs)
                mo[key]["vs_llama"] = round(mo[key]["tok_s"] / ll[key]["tok_s"], 4)
        sizes[name] = {"dims": sz, "moputar": mo, "llama": ll}
        log(f"{name}: moputar prefill {mo['prefill']['tok_s']:,.0f} tok/s, decode {mo['decode_bs1']['tok_s']:,.1f} / "
            f"{mo['decode_bs4']['tok_s']:,.1f} tok/s (bs 1 / 4); llama prefill {ll['prefill']['tok_s']:,.0f}, decode {ll['decode_bs1']['tok_s']:,.1f}")
    tw1 = time.perf_counter()
    head = sizes[args.seqmix_sizes.split(",")[-1]]
    out = {"metric": "prefill tok/s Moputar (layer-list family) at llama-equal size, one prompt in one step", "value": head["moputar"]["prefill"]["tok_s"],
           "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["moputar"]["prefill"]["ms"],
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"model": "Moputar, random weights", "prompt_len": P, "sizes": args.seqmix_sizes,
                      "timing": "CUDA events around each step, a 256 MB buffer written between steps (L2 flush)",
                      "peaks": {"bf16_tflops": tf, "hbm_gbs": gbs, "source": peak_src, "fp32_tflops_nominal": round(f32_tf, 1)}},
           "gpu_launches": launches, "sizes": sizes, "clocks": sampler.summary(tw0, tw1)}
    sampler.stop()
    B.emit(out)
