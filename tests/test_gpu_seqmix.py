"""The layer-list model families (core/models/seqmix.py, shard/batching.py, libdnet_b200_seq) against the float64
oracle (oracle/seqmix_oracle.py): every mechanism alone, then portions, batches, page and slot reuse, block edges,
long decoding and greedy generation through the batcher's token loop.  fp32 runs are held to 2e-4 of the logits'
spread, bf16 runs to the spread of the oracle fed bf16-rounded activations would give (a fixed 4e-2)."""
from __future__ import annotations

import copy

import pytest
import torch

from oracle import seqmix_oracle as so

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}


def attn(**kw):
    mx = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.4}
    mx.update(kw.pop("mixer", {}))
    return {"type": "attention", "mixer": mx, "mlp": kw.get("mlp")}


def delta(**kw):
    mx = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 4}
    mx.update(kw.pop("mixer", {}))
    return {"type": "delta", "mixer": mx, "mlp": kw.get("mlp")}


def config(layers, streams=0, width=48, vocab=96, eps=1e-5, scale=3.0):
    c = {"architecture": "Moputar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers}
    if streams:
        c["streams"] = streams
    return c


FF = {"kind": "dense", "ff": 80}
FULL = config([
    attn(mixer={"conv": 3, "rot": {"base": 500.0, "dims": 8}, "mask": {"size": 40}}, mlp=FF),
    attn(mixer={"conv": 3, "rot": {"base": 500.0, "dims": 8}, "mask": {"size": 40}, "kv_from": 0}, mlp=FF),
    delta(),
    attn(mixer={"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "conv": 2, "rot": {"base": 100.0, "dims": 8}, "mask": {"size": 70}}, mlp=FF),
    delta(mixer={"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 40, "conv": 2}, mlp=FF),
], streams=3)


class Rig:
    """a model + batcher on the GPU and the oracle's view of the same weights"""

    def __init__(self, cfg, dtype="float32", seed=1, max_tokens=1024, max_seqs=4, max_batch_tokens=512, weights=None):
        from dnet_b200.shard.batching import SequenceBatcher, load_model
        from dnet_b200.utils.model import HostDictSource

        self.cfg, self.dtype = cfg, dtype
        self.w = weights if weights is not None else so.random_weights(cfg, seed)
        self.model = load_model(HostDictSource(self.w, cfg), dtype, max_tokens=max_tokens, max_seqs=max_seqs,
                                max_batch_tokens=max_batch_tokens)
        self.eng = SequenceBatcher(self.model)

    def oracle(self, tokens, layers_out=None):
        return so.forward(self.cfg, self.w, tokens, layers_out)

    def close(self):
        self.eng.close()
        self.model.destroy()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """worst row of: rms of the difference (mean removed) over the rms spread of the reference row"""
    d = got.double().cpu() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    r = ref.double() - ref.double().mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def toks(n, vocab=96, seed=0):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_schedule(rig: Rig, tokens, cuts, rid="r"):
    """feed tokens in portions of the given sizes (the rest one by one); logits of every position"""
    out, at = [], 0
    for c in list(cuts) + [1] * len(tokens):
        if at >= len(tokens):
            break
        part = tokens[at:at + c]
        out.append(rig.eng.step([(rid, part, list(range(len(part))))]))
        at += len(part)
    rig.eng.finish(rid)
    return torch.cat(out)


# -- each mechanism alone ---------------------------------------------------------------------------------------
MECHANISMS = {
    "attention_plain": config([attn()]),
    "attention_mha_equal_sizes": config([attn(mixer={"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8})]),
    "attention_one_head": config([attn(mixer={"heads": 1, "kv_heads": 1, "dim": 32, "vdim": 40})]),
    "conv_2": config([attn(mixer={"conv": 2})]),
    "conv_4": config([attn(mixer={"conv": 4})]),
    "conv_1": config([attn(mixer={"conv": 1})]),
    "rot_partial": config([attn(mixer={"rot": {"base": 50.0, "dims": 6}})]),
    "rot_full": config([attn(mixer={"rot": {"base": 10000.0, "dims": 16}})]),
    "block_mask": config([attn(mixer={"mask": {"size": 7}, "scale": 2.0})]),
    "block_mask_page_multiple": config([attn(mixer={"mask": {"size": 64}, "scale": 2.0})]),
    "borrowed_keys": config([attn(mixer={"conv": 3, "rot": {"base": 50.0, "dims": 4}}),
                             attn(mixer={"conv": 2, "kv_from": 0, "rot": {"base": 50.0, "dims": 4}, "mask": {"size": 9}})]),
    "delta": config([delta()]),
    "delta_no_conv_one_group": config([delta(mixer={"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 8, "conv": 0})]),
    "delta_wide": config([delta(mixer={"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 72, "conv": 3})]),
    "delta_dim_128": config([delta(mixer={"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 40, "conv": 2})]),
    "delta_dim_192": config([delta(mixer={"heads": 2, "kv_heads": 2, "dim": 192, "vdim": 8, "conv": 2})]),
    "delta_dim_320": config([delta(mixer={"heads": 1, "kv_heads": 1, "dim": 320, "vdim": 33, "conv": 0})]),
    "delta_dim_600": config([delta(mixer={"heads": 1, "kv_heads": 1, "dim": 600, "vdim": 8, "conv": 2})]),
    "attention_odd_sizes": config([attn(mixer={"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 7, "rot": {"base": 20.0, "dims": 4}})]),
    "attention_wide_values": config([attn(mixer={"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 256})]),
    "feed_forward": config([attn(mlp=FF)]),
    "streams_1": config([attn(mlp=FF), delta()], streams=1),
    "streams_4": config([attn(mlp=FF), delta(mlp=FF)], streams=4),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_alone_fp32(name):
    cfg = MECHANISMS[name]
    t = toks(150, seed=3)
    with Rig(cfg, "float32", seed=sum(map(ord, name))) as rig:
        lo = []
        ref = rig.oracle(t, lo)
        got, trace = rig.eng.step([("a", t, list(range(len(t))))], layer_trace=True)
        for i, l in enumerate(lo):
            assert err(trace[i], l) < TOL["float32"], f"{name}: residual after layer {i}"
        assert err(got, ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_model_whole_prompt(dtype):
    t = toks(200, seed=5)
    with Rig(FULL, dtype) as rig:
        got = rig.eng.step([("a", t, list(range(len(t))))])
        assert err(got, rig.oracle(t)) < TOL[dtype]


# -- schedules ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token(dtype):
    t = toks(90, seed=7)
    with Rig(FULL, dtype) as rig:
        ref = rig.oracle(t)
        assert err(run_schedule(rig, t, []), ref) < TOL[dtype]              # every token alone, from the first
        assert err(run_schedule(rig, t, [50]), ref) < TOL[dtype]            # a prompt, then decoding


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 5, 64, 1, 2, 40], [39, 2, 41, 2, 63, 1, 64], [128, 2], [1, 1, 1, 2, 200]])
def test_portions_of_any_size(cuts):
    t = toks(230, seed=11)
    with Rig(FULL, "float32") as rig:
        assert err(run_schedule(rig, t, cuts), rig.oracle(t)) < TOL["float32"]


def test_results_do_not_depend_on_the_cut_beyond_rounding():
    t = toks(130, seed=13)
    with Rig(FULL, "bfloat16") as rig:
        a = run_schedule(rig, t, [130])
        b = run_schedule(rig, t, [3, 61, 2, 30])
        assert err(b, a.cpu()) < 2e-2


def test_unequal_requests_in_one_batch_equal_each_alone():
    lens = [5, 77, 140, 33]
    seqs = [toks(n, seed=20 + i) for i, n in enumerate(lens)]
    with Rig(FULL, "float32") as rig:
        refs = [rig.oracle(s) for s in seqs]
        at = [0] * 4
        portions = [[2, 3], [40, 2, 35], [64, 64, 12], [1] * 33]
        got = [[] for _ in seqs]
        step = 0
        while any(at[i] < lens[i] for i in range(4)):
            entries = []
            for i in range(4):
                if at[i] < lens[i] and (step + i) % 3 != 2:              # requests sit out some steps
                    n = portions[i][0] if portions[i] else 1
                    portions[i] = portions[i][1:]
                    part = seqs[i][at[i]:at[i] + n]
                    entries.append((f"q{i}", part, list(range(len(part)))))
                    at[i] += len(part)
            step += 1
            if not entries:
                continue
            lg = rig.eng.step(entries)
            row = 0
            for rid, part, _ in entries:
                got[int(rid[1:])].append(lg[row:row + len(part)])
                row += len(part)
        for i in range(4):
            assert err(torch.cat(got[i]), refs[i]) < TOL["float32"], f"request {i}"


def test_pages_and_slots_are_reused():
    """a pool of 4 pages and 2 slots serves 6 requests one after the other and two at a time; a request that does
    not fit is refused without disturbing the live ones"""
    from dnet_b200._cabi import DnError

    with Rig(FULL, "float32", max_tokens=256, max_seqs=2, max_batch_tokens=256) as rig:
        for rnd in range(3):
            a, b = toks(100 + rnd, seed=30 + rnd), toks(120 - rnd, seed=40 + rnd)
            la = rig.eng.step([("a", a[:70], []), ("b", b[:3], [])])
            assert la is None
            la = rig.eng.step([("a", a[70:], list(range(len(a) - 70))), ("b", b[3:], list(range(len(b) - 3)))])
            assert err(la[:len(a) - 70], rig.oracle(a)[70:]) < TOL["float32"]
            assert err(la[len(a) - 70:], rig.oracle(b)[3:]) < TOL["float32"]
            assert rig.model.free_pages == 0 and rig.model.free_slots == 0
            with pytest.raises(DnError):
                rig.eng.step([("a", toks(60), [])])                        # a fifth page does not exist
            with pytest.raises(DnError):
                rig.eng.step([("c", [1], [])])                            # nor a third slot
            rig.eng.live.pop("c", None)
            rig.eng.finish("a")
            rig.eng.finish("b")
            assert rig.model.free_pages == 4 and rig.model.free_slots == 2


def test_a_freed_slot_starts_from_zero_state():
    cfg = config([delta(), delta(mlp=FF)], streams=2)
    with Rig(cfg, "float32", max_seqs=1) as rig:
        first = toks(80, seed=50)
        rig.eng.step([("x", first, [])])
        rig.eng.finish("x")
        t = toks(40, seed=51)
        assert err(run_schedule(rig, t, [10, 2]), rig.oracle(t)) < TOL["float32"]


# -- edges, with scores made to stand out ----------------------------------------------------------------------------
def peaky(cfg):
    """the same config with attention scales that make one key dominate a row: a key wrongly seen or missed shows"""
    c = copy.deepcopy(cfg)
    for L in c["layers"]:
        if L["type"] == "attention":
            L["mixer"]["scale"] = 4.0
    return c


@pytest.mark.parametrize("block", [5, 64, 90, 100])
def test_block_edges_in_prompts_and_in_decoding(block):
    cfg = peaky(config([attn(mixer={"mask": {"size": block}, "conv": 3, "rot": {"base": 30.0, "dims": 8}}, mlp=FF),
                        attn(mixer={"mask": {"size": block}, "kv_from": 0, "rot": {"base": 30.0, "dims": 8}})], streams=2))
    n = 2 * block + 7
    t = toks(n, seed=60 + block)
    with Rig(cfg, "float32") as rig:
        ref = rig.oracle(t)
        # the test can tell a mask that is one position off: the oracle with a neighbouring block size differs
        off = copy.deepcopy(cfg)
        for L in off["layers"]:
            L["mixer"]["mask"]["size"] = block + 1
        assert err(so.forward(off, rig.w, t)[block:], ref[block:]) > 100 * TOL["float32"]
        assert err(run_schedule(rig, t, [n]), ref) < TOL["float32"]                       # edges inside a prompt
        assert err(run_schedule(rig, t, [block - 1]), ref) < TOL["float32"]               # decoding across both edges
        assert err(run_schedule(rig, t, [block - 1, 2, block - 2, 2]), ref) < TOL["float32"]   # portions straddling them


def test_far_key_among_hundreds():
    """plain causal attention, one early key made to match the last queries from pages away"""
    cfg = config([attn(mixer={"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 16, "scale": 0.5})], vocab=64)
    w = so.random_weights(cfg, 70)
    # keys are projected with minus the first query head's weights: a query scores -|q|^2 against its own token and
    # +0.9 |q|^2 against a token whose embedding points the other way.  Token 63 is such a token for token 62; it
    # appears once, at position 3, and token 62 ends the prompt.
    g = torch.Generator().manual_seed(71)
    e = w["embed"].float()
    e[63] = -e[62] + 0.4 * torch.randn(e.shape[1], generator=g)
    w["embed"] = e.to(torch.bfloat16)
    w["l0.mix.k"] = (-w["l0.mix.q"][:64].float()).to(torch.bfloat16)
    w["l0.mix.q.norm"] = torch.ones_like(w["l0.mix.q.norm"])
    w["l0.mix.k.norm"] = torch.ones_like(w["l0.mix.k.norm"])
    t = torch.randint(0, 62, (700,), generator=g).tolist()
    t[3] = 63
    t += [62] * 6
    with Rig(cfg, "float32", weights=w) as rig:
        ref = rig.oracle(t)
        t_without = list(t)
        t_without[3] = 5
        assert err(rig.oracle(t_without)[-6:], ref[-6:]) > 100 * TOL["float32"]       # the far key matters
        assert err(run_schedule(rig, t, [len(t)]), ref) < TOL["float32"]
        assert err(run_schedule(rig, t, [300, 2, 250, 148]), ref) < TOL["float32"]    # the last six decoded one by one


def test_first_tokens_of_a_sequence():
    with Rig(FULL, "float32") as rig:
        for n in (1, 2, 3, 4):
            t = toks(n, seed=80 + n)
            assert err(run_schedule(rig, t, [n]), rig.oracle(t)) < TOL["float32"]
            assert err(run_schedule(rig, t, []), rig.oracle(t)) < TOL["float32"]


def test_long_decoding():
    t = toks(420, seed=90)
    with Rig(FULL, "float32") as rig:
        assert err(run_schedule(rig, t, [20]), rig.oracle(t)) < TOL["float32"]


def test_a_step_larger_than_the_batch_buffer_is_cut_inside():
    t = toks(300, seed=95)
    with Rig(FULL, "float32", max_batch_tokens=64) as rig:
        got = rig.eng.step([("a", t[:290], [0, 63, 64, 289]), ("b", t[:70], [69])])
        ref = rig.oracle(t)
        assert err(got[:4], ref[[0, 63, 64, 289]]) < TOL["float32"]
        assert err(got[4:], ref[[69]]) < TOL["float32"]


# -- the token loop ---------------------------------------------------------------------------------------------------
def test_greedy_generation_through_the_batcher():
    from dnet_b200.shard.batching import GenRequest

    with Rig(FULL, "float32", max_tokens=320, max_seqs=2) as rig:
        rig.eng.step_tokens = 48
        reqs = [GenRequest(f"g{i}", toks(n, seed=100 + i), max_new_tokens=m) for i, (n, m) in enumerate([(30, 6), (100, 4), (3, 9), (65, 5)])]
        out = rig.eng.generate(reqs)
        assert rig.model.free_slots == 2 and rig.model.free_pages == 5
        for r in reqs:
            seq = list(r.prompt)
            for tok in out[r.id]:
                lg = rig.oracle(seq)[-1]
                top = torch.topk(lg, 2).values
                if float(top[0] - top[1]) > 1e-3 * float(lg.std()):            # ties aside, the greedy token is the oracle's
                    assert tok == int(lg.argmax()), r.id
                seq.append(tok)
            assert len(out[r.id]) == r.max_new_tokens


# -- widths whose products run on the tcgen05 GEMM (bf16, 16 tokens and more), the row kernel (a few tokens) and the tiles ----
WIDE = config([
    attn(mixer={"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "conv": 3, "rot": {"base": 300.0, "dims": 16}, "mask": {"size": 48}},
         mlp={"kind": "dense", "ff": 192}),
    attn(mixer={"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "conv": 3, "rot": {"base": 300.0, "dims": 16}, "mask": {"size": 48},
                "kv_from": 0}, mlp={"kind": "dense", "ff": 192}),
    delta(mixer={"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "conv": 4}),
], streams=2, width=128, vocab=160)


def test_tensor_core_products_whole_prompt_and_portions():
    t = toks(333, seed=120)
    with Rig(WIDE, "bfloat16") as rig:
        ref = rig.oracle(t)
        assert err(run_schedule(rig, t, [333]), ref) < TOL["bfloat16"]
        # 200 tokens on the GEMM, 12 on the tiles, 5 on the row kernel, 100 on the GEMM, the rest one by one
        assert err(run_schedule(rig, t, [200, 12, 5, 100]), ref) < TOL["bfloat16"]
        assert rig.model.check() is None


def test_tensor_core_products_in_a_mixed_batch():
    a, b, c = toks(150, seed=121), toks(40, seed=122), toks(9, seed=123)
    with Rig(WIDE, "bfloat16") as rig:
        rig.eng.step([("c", c[:8], [])])
        lg = rig.eng.step([("a", a, list(range(150))), ("b", b, list(range(40))), ("c", c[8:], [0])])
        assert err(lg[:150], rig.oracle(a)) < TOL["bfloat16"]
        assert err(lg[150:190], rig.oracle(b)) < TOL["bfloat16"]
        assert err(lg[190:], rig.oracle(c)[8:]) < TOL["bfloat16"]


@pytest.mark.parametrize("block", [5, 64, 90, 100])
def test_block_edges_on_the_attention_tiles(block):
    """bf16 portions of 16 tokens and more take the MMA-tile attention: the rows at a block's start, whole and cut"""
    cfg = peaky(config([attn(mixer={"mask": {"size": block}, "conv": 3, "rot": {"base": 30.0, "dims": 8}}, mlp=FF),
                        attn(mixer={"mask": {"size": block}, "kv_from": 0, "rot": {"base": 30.0, "dims": 8}})], streams=2))
    n = max(2 * block + 7, 40)
    t = toks(n, seed=60 + block)
    edges = [r for r in range(block - 1, n, block)] + [r for r in range(block, n, block)]
    with Rig(cfg, "bfloat16") as rig:
        ref = rig.oracle(t)
        for d in (1, -1):           # a block that is one token longer or shorter moves these rows far beyond the tolerance
            off = copy.deepcopy(cfg)
            for L in off["layers"]:
                L["mixer"]["mask"]["size"] = block + d
            assert err(so.forward(off, rig.w, t)[[block]], ref[[block]]) > 4 * TOL["bfloat16"]
        for cuts in ([n], [block + 3, 17, n], [16, 16, 16, n]):
            got = run_schedule(rig, t, cuts)
            assert err(got, ref) < TOL["bfloat16"], cuts
            assert err(got[edges], ref[edges]) < TOL["bfloat16"], cuts


def test_far_key_on_the_attention_tiles():
    """700 keys back, through eleven pages, on the tiles (bf16, whole prompt and 16-token tail portions)"""
    cfg = config([attn(mixer={"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 16, "scale": 0.5})], vocab=64)
    w = so.random_weights(cfg, 70)
    g = torch.Generator().manual_seed(71)
    e = w["embed"].float()
    e[63] = -e[62] + 0.4 * torch.randn(e.shape[1], generator=g)
    w["embed"] = e.to(torch.bfloat16)
    w["l0.mix.k"] = (-w["l0.mix.q"][:64].float()).to(torch.bfloat16)
    w["l0.mix.q.norm"] = torch.ones_like(w["l0.mix.q.norm"])
    w["l0.mix.k.norm"] = torch.ones_like(w["l0.mix.k.norm"])
    t = torch.randint(0, 62, (700,), generator=g).tolist()
    t[3] = 63
    t += [62] * 6
    with Rig(cfg, "bfloat16", weights=w) as rig:
        ref = rig.oracle(t)
        t_without = list(t)
        t_without[3] = 5
        assert err(rig.oracle(t_without)[-6:], ref[-6:]) > 4 * TOL["bfloat16"]
        assert err(run_schedule(rig, t, [len(t)])[-6:], ref[-6:]) < TOL["bfloat16"]
        assert err(run_schedule(rig, t, [300, 2, 388, 16])[-6:], ref[-6:]) < TOL["bfloat16"]


def test_wide_model_fp32_is_exact_on_the_cuda_core_path():
    t = toks(140, seed=124)
    with Rig(WIDE, "float32") as rig:
        assert err(run_schedule(rig, t, [100, 3]), rig.oracle(t)) < TOL["float32"]


# -- from a checkpoint folder, through the command lines --------------------------------------------------------------
def write_checkpoint(folder, cfg, weights):
    """config.json + model.safetensors (bf16 tensors), written by hand: header length, JSON header, data"""
    import json
    import struct

    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (folder / "config.json").write_text(json.dumps(cfg))


def test_command_lines_on_a_checkpoint_folder(tmp_path):
    import json
    import pathlib
    import subprocess
    import sys

    import numpy as np

    root = pathlib.Path(__file__).resolve().parent.parent
    w = so.random_weights(FULL, 9)
    write_checkpoint(tmp_path, FULL, w)
    a, b = toks(70, seed=130), toks(21, seed=131)
    # replay: a's prompt in two portions beside b, then a decoded token of each; the cache holds 3 pages
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": []}, {"id": "b", "tokens": b[:20], "want": [19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:69], "want": [0, 28]}, {"id": "b", "tokens": b[20:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 2"]
    ra, rb = so.forward(FULL, w, a), so.forward(FULL, w, b)
    V = FULL["vocab"]
    got = {i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)) for i in range(3)}
    assert err(got[0], rb[[19]]) < TOL["float32"]
    assert err(got[1], torch.stack([ra[40], ra[68], rb[20]])) < TOL["float32"]
    assert err(got[2], ra[[69]]) < TOL["float32"]
    # generation: greedy tokens of two requests equal the oracle's (ties aside)
    reqs = [{"id": "x", "prompt": a[:30], "max_new_tokens": 4}, {"id": "y", "prompt": b[:5]}]
    r = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--model", str(tmp_path), "--dtype", "float32", "--max-new-tokens", "3",
                        "--max-tokens", "128", "--max-seqs", "2"], input="".join(json.dumps(q) + "\n" for q in reqs), capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    res = {o["id"]: o["tokens"] for o in map(json.loads, r.stdout.strip().splitlines())}
    assert len(res["x"]) == 4 and len(res["y"]) == 3
    for q in reqs:
        seq = list(q["prompt"])
        for tok in res[q["id"]]:
            lg = so.forward(FULL, w, seq)[-1]
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(lg.std()):
                assert tok == int(lg.argmax())
            seq.append(tok)


def test_decode_graphs_replay_the_same_kernels():
    """decode steps replay a captured graph; the launch-by-launch path gives the same bits, also after a slot and its
    pages went to another request and with a different number of live requests"""
    a, b = toks(90, seed=140), toks(50, seed=141)
    outs = []
    for graphs in (True, False):
        with Rig(FULL, "bfloat16") as rig:
            rig.model.set_graphs(graphs)
            got = []
            rig.eng.step([("a", a[:60], []), ("b", b[:30], [])])
            for i in range(20):                                           # two live requests, one token each
                got.append(rig.eng.step([("a", [a[60 + i]], [0]), ("b", [b[30 + i]], [0])]))
            rig.eng.finish("b")
            for i in range(10):                                           # one live request
                got.append(rig.eng.step([("a", [a[80 + i]], [0])]))
            rig.eng.finish("a")
            rig.eng.step([("c", b[:7], [])])                             # the freed slots and pages, another request
            for i in range(12):
                got.append(rig.eng.step([("c", [b[7 + i]], [0])]))
            rig.model.check()
            outs.append(torch.cat(got).cpu())
            if graphs:
                ref_a, ref_b = rig.oracle(a), rig.oracle(b[:19])
                assert err(outs[0][0:40:2], ref_a[60:80]) < TOL["bfloat16"]
                assert err(outs[0][40:50], ref_a[80:90]) < TOL["bfloat16"]
                assert err(outs[0][50:], ref_b[7:19]) < TOL["bfloat16"]
    assert torch.equal(outs[0], outs[1])


# -- head sizes of real models: 16-byte key and value loads in decoding, MMA tiles and the wider delta-rule layouts --------
BIG = config([
    attn(mixer={"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "conv": 2, "rot": {"base": 1000.0, "dims": 32}, "mask": {"size": 50}}),
    attn(mixer={"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 256}),
    delta(mixer={"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 64, "conv": 3}),
], streams=2, width=64, vocab=96)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_head_sizes_prompt_portions_and_decoding(dtype):
    t = toks(330, seed=150)
    with Rig(BIG, dtype) as rig:
        ref = rig.oracle(t)
        assert err(run_schedule(rig, t, [290, 17]), ref) < TOL[dtype]        # the last 23 decoded, each warp with tiles of its own
        assert err(run_schedule(rig, t, [3, 100, 2, 200]), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_allow_no_wide_loads(dtype):
    """width, feed-forward and vocabulary that are multiples of neither 4 nor 8: the scalar forms of every kernel"""
    cfg = config([attn(mixer={"conv": 3, "rot": {"base": 40.0, "dims": 6}, "mask": {"size": 33}}, mlp={"kind": "dense", "ff": 90}),
                  delta(mlp={"kind": "dense", "ff": 45}),
                  attn(mixer={"kv_from": 0, "mask": {"size": 20}})], streams=3, width=50, vocab=77)
    t = toks(120, vocab=77, seed=160)
    with Rig(cfg, dtype) as rig:
        ref = rig.oracle(t)
        assert err(run_schedule(rig, t, [120]), ref) < TOL[dtype]
        assert err(run_schedule(rig, t, [70, 2, 20]), ref) < TOL[dtype]


# -- a wider model: products with many k-blocks and several tiles each way on the tcgen05 GEMM ---------------------------
WIDER = config([
    attn(mixer={"heads": 6, "kv_heads": 3, "dim": 64, "vdim": 32, "conv": 4, "rot": {"base": 10000.0, "dims": 32}, "mask": {"size": 128}},
         mlp={"kind": "dense", "ff": 640}),
    delta(mixer={"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 96, "conv": 4}, mlp={"kind": "dense", "ff": 1100}),
    attn(mixer={"heads": 6, "kv_heads": 3, "dim": 64, "vdim": 32, "conv": 2, "rot": {"base": 10000.0, "dims": 32}, "kv_from": 0}),
], streams=4, width=512, vocab=600, scale=1.0)


def test_wider_model_on_the_tensor_core_products():
    t = toks(420, vocab=600, seed=170)
    with Rig(WIDER, "bfloat16", max_tokens=1024, max_batch_tokens=512) as rig:
        ref = rig.oracle(t)
        assert err(run_schedule(rig, t, [400, 3]), ref) < TOL["bfloat16"]            # 400 rows: four token tiles, a ragged last one
        assert err(run_schedule(rig, t, [130, 33, 16, 200, 24]), ref) < TOL["bfloat16"]
        b = toks(90, vocab=600, seed=171)
        rig.eng.step([("b", b[:50], [])])
        lg = rig.eng.step([("a", t[:300], [299]), ("b", b[50:], list(range(40)))])   # a mixed step of 340 rows
        assert err(lg[:1], ref[[299]]) < TOL["bfloat16"]
        assert err(lg[1:], rig.oracle(b)[50:]) < TOL["bfloat16"]
        assert rig.model.check() is None


# -- through the shard runtime: load_model_core picks the batched policy, frames of tokens come back as final tokens ----
def test_served_by_the_shard_runtime():
    import queue

    from dnet_b200.shard.models import ShardLoadModelRequest
    from dnet_b200.shard.policies.batched import BatchedStepPolicy
    from dnet_b200.shard.runtime import ShardRuntime
    from dnet_b200.utils.model import HostDictSource
    from tests.helpers import ring_generate, token_message

    w = so.random_weights(FULL, 21)
    n = len(FULL["layers"])
    rt = ShardRuntime(shard_id="s0", queue_size=64)
    rt.kv_cache_config.max_tokens = 256
    rt.load_model_core(ShardLoadModelRequest(model_path=HostDictSource(w, FULL), total_layers=n, layers=list(range(n)), window_size=n,
                                             residency_size=n, kv_bits="fp16"))
    try:
        assert isinstance(rt.policy, BatchedStepPolicy)

        def oracle_greedy(prompt, got):
            seq = list(prompt)
            for tok in got:
                lg = so.forward(FULL, w, seq)[-1]
                top = torch.topk(lg, 2).values
                if float(top[0] - top[1]) > 2e-2 * float(lg.std()):        # bf16 serving: only clear winners are compared
                    assert tok == int(lg.argmax())
                seq.append(tok)

        a, b = toks(45, seed=180), toks(70, seed=181)
        out_a = [t for t, _, _ in ring_generate([rt], "na", a, 5)]
        oracle_greedy(a, out_a)
        # a second request, its prompt in three chunks (the first two emit nothing), while "na" is still live
        for part in (b[:30], b[30:64]):
            rt.policy.process(token_message(rt, "nb", part, more=True))
            with pytest.raises(queue.Empty):
                rt.activation_send_queue.get_nowait()
        out_b = [t for t, _, _ in ring_generate([rt], "nb", b[64:], 4)]
        oracle_greedy(b, out_b)
        assert rt.model.free_slots == 6
        rt.release_nonce("na")
        rt.release_nonce_deferred("nb")
        assert rt.model.free_slots == 8 and rt.model.free_pages == rt.model.pool_pages
        # a partial assignment is refused
        rt2 = ShardRuntime(shard_id="s1", queue_size=8)
        with pytest.raises(ValueError):
            rt2.load_model_core(ShardLoadModelRequest(model_path=HostDictSource(w, FULL), total_layers=n, layers=[0, 1], window_size=2,
                                                      residency_size=2, kv_bits="fp16"))
    finally:
        assert rt.unload_model_core().success
