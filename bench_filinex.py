"""bench_filinex.py -- `bench.py --config filinex`: prefill and decode throughput of the Filinex family (parallel
mixer = sink attention beside gated linear attention, wkv mixer, routed clamped-GLU experts with a shared one, a
looped span of layers) beside Moputar, the closest family of this framework (same library, same ragged-batch step,
attention + an fp32 recurrence + a gated feed-forward), at equal width, heads, layer runs and active feed-forward
width.  Random weights, synthetic tokens, one GPU.

Per size: prefill (one P-token prompt in one step), decode of one and of four sequences at the end of a P-token
context, and the device time of every phase of the step (the library's phase timers) with its algorithmic FLOPs or
bytes and the fraction of the measured peak, for both families.
"""
from __future__ import annotations

from bench_seqmix import HD, SIZES, VOCAB, _Flusher, _rand, _roofline, _run_moputar, _timed, moputar_algorithmic

EXPERTS, TOP, RANK = 16, 2, 64


def filinex_config(sz: dict) -> dict:
    """4 layers (wkv, parallel, wkv, parallel), the middle two run twice: 6 layer runs.  Active feed-forward width =
    top x expert width + shared width = the dense width of the size."""
    W, H, G, ff = sz["width"], sz["heads"], sz["kv_heads"], sz["ff"]
    moe = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP}, "expert": {"ff": ff // 4, "limit": 7.0},
           "shared": {"ff": ff // 2, "limit": 7.0}}
    wkv = {"type": "wkv", "mixer": {"heads": W // 64, "dim": 64, "rank": RANK}, "mlp": moe}
    par = {"type": "parallel", "mlp": moe,
           "mixer": {"left": {"heads": H, "kv_heads": G, "dim": HD, "vdim": HD, "scale": HD ** -0.5, "softcap": 30.0},
                     "right": {"heads": H // 2, "dim": 64, "vdim": HD, "tau": 8.0, "rank": RANK}, "left_scale": 1.0, "right_scale": 0.5}}
    return {"architecture": "Filinex", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
            "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [wkv, par, wkv, par]}


def filinex_weights(model, g, dev):
    import torch

    items = []
    for name, shape in model.expected_tensors().items():
        leaf = name.split(".", 1)[-1]
        if name.endswith(".alpha"):
            t = torch.full(shape, 0.7, dtype=torch.bfloat16, device=dev)
        elif leaf in ("norm1", "norm2", "post1", "post2", "mix.norm", "r.norm", "norm") or name in ("final.norm", "embed.norm"):
            t = torch.ones(shape, dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".b") or leaf in ("sink", "bonus") or name.endswith("norm.b"):
            t = _rand(shape, g, 0.1, dev) if shape else torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        elif leaf.startswith("mu."):
            t = torch.full(shape, 0.5, dtype=torch.bfloat16, device=dev)
        elif name == "embed":
            t = _rand(shape, g, 1.0, dev)
        else:
            t = _rand(shape, g, shape[-1] ** -0.5, dev)
        items.append((name, t))
    return items


def runs_of(cfg: dict):
    lp, n = cfg.get("loop"), len(cfg["layers"])
    if not lp:
        return list(range(n)), 0
    order = list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))
    return order, lp["times"]


def filinex_algorithmic(cfg: dict, N: int, ctx0: int, n_seqs: int) -> dict:
    """FLOPs and the bytes that must move per phase, for a step of n_seqs entries x (N / n_seqs) tokens whose
    sequences already hold ctx0 tokens each; summed over the layer runs."""
    W = cfg["width"]
    keys = ("proj", "attn", "recur", "out_proj", "moe_up", "moe_down", "ff_up", "ff_down")
    f = {k: 0.0 for k in keys}
    by = dict(f)
    per = N // n_seqs
    order, passes = runs_of(cfg)
    for i in order:
        L = cfg["layers"][i]
        mx = L["mixer"]
        if L["type"] == "parallel":
            a, r = mx["left"], mx["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            rh, rk, rv, rank = r["heads"], r["dim"], r["vdim"], r["rank"]
            cols = H * dk + G * (dk + dv) + H + 2 * rh * rk + 2 * rh * rv + rank
            f["proj"] += 2.0 * N * (W * cols + rank * rh * rk)
            by["proj"] += 2.0 * (W * cols + rank * rh * rk)
            vis = sum(p + 1 for p in range(ctx0, ctx0 + per)) * n_seqs
            f["attn"] += 2.0 * (dk + dv) * H * vis
            by["attn"] += 2.0 * n_seqs * (ctx0 + per) * G * (dk + dv) + 2.0 * N * H * (dk + dv)
            f["recur"] += 4.0 * rk * rv * rh * N
            by["recur"] += 8.0 * n_seqs * rh * rk * rv + 4.0 * N * (3 * rh * rk + 2 * rh * rv)
            f["out_proj"] += 2.0 * N * W * (H * dv + rh * rv)
            by["out_proj"] += 2.0 * W * (H * dv + rh * rv)
        else:
            H, dk, rank = mx["heads"], mx["dim"], mx["rank"]
            dv = mx.get("vdim", dk)
            cols = 2 * H * dk + 2 * H * dv + rank
            f["proj"] += 2.0 * N * (W * cols + rank * H * dk)
            by["proj"] += 2.0 * (W * cols + rank * H * dk)
            f["recur"] += 6.0 * dk * dv * H * N
            by["recur"] += 8.0 * n_seqs * H * dk * dv + 4.0 * N * (3 * H * dk + 2 * H * dv)
            f["out_proj"] += 2.0 * N * W * H * dv
            by["out_proj"] += 2.0 * W * H * dv
        mlp = L.get("mlp")
        if mlp:
            E, top, ef = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            hit = min(E, N * top)          # experts whose weights a step can touch at all
            f["moe_up"] += 4.0 * N * top * W * ef
            by["moe_up"] += 4.0 * hit * W * ef
            f["moe_down"] += 2.0 * N * top * W * ef
            by["moe_down"] += 2.0 * hit * W * ef
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                # steps of up to 8 tokens run the shared expert's rows inside the routed experts' two launches
                up, down = ("moe_up", "moe_down") if N <= 8 else ("ff_up", "ff_down")
                f[up] += 4.0 * N * W * sf
                by[up] += 4.0 * W * sf
                f[down] += 2.0 * N * W * sf
                by[down] += 2.0 * W * sf
    return {"flops": f, "bytes": by}


def _run_filinex(sz: dict, args, P: int, flush, dev) -> dict:
    import torch

    from dnet_b200.core.models import get_ring_model

    cfg = filinex_config(sz)
    pages = 4 * ((P + 64 + 63) // 64)
    model = get_ring_model("filinex", cfg, assigned_layers=list(range(len(cfg["layers"]))), dtype="bfloat16", kv_pool_pages=pages,
                           max_seqs=4, max_batch_tokens=max(P, 64))
    g = torch.Generator(device=dev).manual_seed(7)
    model.load_weights(filinex_weights(model, g, dev), strict=True)
    assert not model.missing_tensors()
    prompt = torch.randint(0, VOCAB, (P,), generator=torch.Generator().manual_seed(11)).tolist()
    K, Wm = args.steps, args.warmup
    live = []
    st = torch.cuda.current_stream()

    def fresh(n):
        for h in live:
            h.free()
        live.clear()
        live.extend(model.make_cache(stream=st) for _ in range(n))

    res = {"config": {"layers": [l["type"] for l in cfg["layers"]], "loop": cfg["loop"], "layer_runs": model.layer_runs,
                      "experts": EXPERTS, "top": TOP}}
    t = _timed(lambda: model.step([(live[0], prompt)], [P - 1], stream=st), lambda: fresh(1), K, Wm, flush)
    res["prefill"] = {"ms": t, "tok_s": P / t * 1e3}
    fresh(1)
    model.profile(True)
    model.step([(live[0], prompt)], [P - 1], stream=st)
    res["prefill"]["phases_ms"] = model.profile_read(reset=True)
    model.profile(False)
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


FP32 = ("recur", "delta_rule")


def run_filinex(args, rank: int, local_rank: int, world: int) -> None:
    import time

    import torch

    import bench as B
    import bench_seqmix as BS
    from bench import ClockSampler, log

    if world != 1:
        raise SystemExit("--config filinex runs on one GPU")
    dev = torch.device("cuda", local_rank)
    P = int(args.seqmix_prompt)
    gbs, peak_src = B.peaks()
    tf = B.tensor_peak_tf()
    props = torch.cuda.get_device_properties(dev)
    f32_tf = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    flush = _Flusher(dev)
    side = torch.cuda.Stream(device=dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    tw0 = time.perf_counter()
    BS.FP32_PHASES = FP32
    sizes, launches = {}, 0
    args.seqmix_repeats = 2          # Moputar: (attention, attention on shared pages, delta) x 2 = 6 layers
    for name in args.seqmix_sizes.split(","):
        sz = SIZES[name]
        with torch.cuda.stream(side):
            fx = _run_filinex(sz, args, P, flush, dev)
            mo = _run_moputar(sz, args, P, flush, dev)
        side.synchronize()
        launches += fx.pop("launches") + mo.pop("launches")
        fcfg, mcfg = fx.pop("cfg"), mo.pop("cfg")
        for key in ("prefill", "decode_bs1", "decode_bs4"):
            n_seq = 4 if key.endswith("4") else 1
            N, ctx0 = (P, 0) if key == "prefill" else (n_seq, fx[key]["context"])
            fx[key]["roofline"] = _roofline(fx[key]["phases_ms"], filinex_algorithmic(fcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            mo[key]["roofline"] = _roofline(mo[key]["phases_ms"], moputar_algorithmic(mcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            fx[key]["vs_moputar"] = round(fx[key]["tok_s"] / mo[key]["tok_s"], 4)
            log(f"{name} {key}: filinex {fx[key]['ms']:.3f} ms ({fx[key]['tok_s']:,.0f} tok/s), moputar {mo[key]['ms']:.3f} ms ({mo[key]['tok_s']:,.0f} tok/s)")
            log("   filinex " + ", ".join(f"{k} {v['ms']:.3f}ms/{v['frac']:.3f}" for k, v in fx[key]["roofline"].items()))
            log("   moputar " + ", ".join(f"{k} {v['ms']:.3f}ms/{v['frac']:.3f}" for k, v in mo[key]["roofline"].items()))
            log("   filinex phases " + ", ".join(f"{k} {v:.3f}" for k, v in fx[key]["phases_ms"].items() if v > 0))
        sizes[name] = {"dims": sz, "filinex": fx, "moputar": mo}
    tw1 = time.perf_counter()
    head = sizes[args.seqmix_sizes.split(",")[-1]]
    out = {"metric": "prefill tok/s Filinex (layer-list family) beside Moputar at equal size, one prompt in one step",
           "value": head["filinex"]["prefill"]["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": head["filinex"]["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic",
           "config": {"model": "Filinex, random weights", "prompt_len": P, "sizes": args.seqmix_sizes,
                      "timing": "CUDA events around each step, a 256 MB buffer written between steps (L2 flush)",
                      "peaks": {"bf16_tflops": tf, "hbm_gbs": gbs, "source": peak_src, "fp32_tflops_nominal": round(f32_tf, 1)}},
           "gpu_launches": launches, "sizes": sizes, "clocks": sampler.summary(tw0, tw1)}
    sampler.stop()
    B.emit(out)
