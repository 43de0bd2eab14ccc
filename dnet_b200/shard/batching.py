"""Continuous batching for models that run ragged-batch steps (core/models/seqmix.py).

The ring policies of this package run one request per step; here one *step* carries the next tokens of every live
request -- a portion of a prompt for some, the one decoded token for others -- through all layers at once.

``SequenceBatcher`` is the step function and the scheduler:
  * ``admit`` / ``finish`` lease and return a state slot and the request's cache pages;
  * ``step(entries)`` runs exactly the tokens it is given (cut into sub-steps only when they exceed the model's
    ``max_batch_tokens``; the result does not depend on the cut);
  * ``generate(requests)`` is the token loop: it admits waiting requests while slots and pages last, gives every
    step a token budget -- decode tokens first, prompt portions with what is left -- samples with ``Sampler`` and
    retires finished requests, whose slots and pages the next waiting request takes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from dnet_b200.core.decoding.config import DecodingConfig
from dnet_b200.core.decoding.sampler import Sampler
from dnet_b200.core.models import get_ring_model
from dnet_b200.core.models.seqmix import SeqHandle, SeqMixRingModel
from dnet_b200.utils.model import get_model_metadata, load_weight

PAGE = 64


@dataclass
class GenRequest:
    id: str
    prompt: Sequence[int]
    max_new_tokens: int = 16
    decoding: DecodingConfig = field(default_factory=lambda: DecodingConfig(temperature=0.0))
    stop_ids: Tuple[int, ...] = ()


def load_model(model_path, dtype: str = "bfloat16", *, max_tokens: int = 4096, max_seqs: int = 4,
               max_batch_tokens: int = 2048) -> SeqMixRingModel:
    """Checkpoint folder (or an in-memory source) -> a resident model: the registry picks the class from the config,
    the cache pool holds ``max_tokens`` tokens in 64-token pages."""
    if not torch.cuda.is_available():
        raise RuntimeError("dnet_b200 needs a CUDA device: there is no CPU fallback")
    md = get_model_metadata(model_path)
    n = md.num_layers
    pages = max(1, (int(max_tokens) + PAGE - 1) // PAGE)
    groups = (md.embed_tokens, md.norm, md.lm_head)
    shapes = {f"l{li}.{suffix}": tuple(info.shape) for li, tensors in md.weight_info.items() for suffix, info in tensors.items()}
    shapes.update({k[4:]: tuple(info.shape) for g in groups for k, info in g.items() if k.startswith("seq:")})
    model = get_ring_model(md.model_type, md.model_config, assigned_layers=list(range(n)), dtype=dtype, kv_pool_pages=pages,
                           max_seqs=max_seqs, max_batch_tokens=max_batch_tokens, tensor_shapes=shapes)
    if not getattr(model, "batched_step", False):
        model.destroy()
        raise ValueError(f"model type {md.model_type!r} does not run batched steps; serve it through ShardRuntime")
    mapped: dict = {}
    items = []

    def dev(info):
        t = load_weight(info, mapped, md.source)
        if not t.dtype.is_floating_point:
            return t.to("cuda").contiguous()
        return t.to(device="cuda", dtype=model.dtype).contiguous()

    for li, tensors in md.weight_info.items():
        for suffix, info in tensors.items():
            items.append((f"l{li}.{suffix}", dev(info)))
    for name, group in (("embed", md.embed_tokens), ("final.norm", md.norm), ("head", md.lm_head)):
        if "weight" in group:
            items.append((name, dev(group["weight"])))
        items += [(k[4:], dev(info)) for k, info in group.items() if k.startswith("seq:")]
    model.load_weights(items, strict=True)
    for f in mapped.values():
        f.close()
    miss = model.missing_tensors()
    if miss:
        model.destroy()
        raise ValueError(f"checkpoint lacks {miss[:4]}{' ...' if len(miss) > 4 else ''}")
    torch.cuda.synchronize()
    return model


class SequenceBatcher:
    def __init__(self, model: SeqMixRingModel, stream: Optional[torch.cuda.Stream] = None, step_tokens: int = 512):
        self.model = model
        self.stream = stream or torch.cuda.Stream()
        self.step_tokens = max(1, min(int(step_tokens), model.max_batch_tokens))
        self.live: Dict[str, SeqHandle] = {}
        self.steps_run = 0

    # -- leases ------------------------------------------------------------------------------------
    def admit(self, rid: str) -> SeqHandle:
        if rid in self.live:
            raise KeyError(f"request {rid!r} is live already")
        h = self.live[rid] = self.model.make_cache(stream=self.stream)
        return h

    def finish(self, rid: str) -> None:
        h = self.live.pop(rid, None)
        if h is not None:
            # kernels that read the slot are queued on the one stream the next user's zeroing is queued on too
            h.free()

    def close(self) -> None:
        self.stream.synchronize()
        for rid in list(self.live):
            self.finish(rid)

    # -- one step ----------------------------------------------------------------------------------
    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], layer_trace: bool = False):
        """entries: (request id, its next tokens, places among them whose logits are wanted).  A request is admitted
        at its first entry.  Returns fp32 [wanted, vocab] in the order of entries and places (None if nothing is)."""
        cap = self.model.max_batch_tokens
        if layer_trace and sum(len(t) for _, t, _ in entries) > cap:
            raise ValueError("layer_trace needs the step to fit max_batch_tokens")
        out: List[torch.Tensor] = []
        trace = None
        # cursors into each entry; a sub-step takes whole entries while they fit and cuts the one that does not
        cur = [0] * len(entries)
        while any(cur[i] < len(e[1]) for i, e in enumerate(entries)):
            room, sub, want, row0 = cap, [], [], 0
            order: List[Tuple[int, int, int]] = []          # (entry, place) -> row, to restore the caller's order
            for i, (rid, toks, places) in enumerate(entries):
                if cur[i] >= len(toks) or room == 0:
                    continue
                n = min(room, len(toks) - cur[i])
                h = self.live.get(rid) or self.admit(rid)
                sub.append((h, toks[cur[i]:cur[i] + n]))
                for p in places:
                    if cur[i] <= p < cur[i] + n:
                        order.append((i, p, row0 + p - cur[i]))
                cur[i] += n
                row0 += n
                room -= n
            want = [r for _, _, r in order]
            with torch.cuda.stream(self.stream):
                res = self.model.step(sub, want, stream=self.stream, layer_trace=layer_trace)
            self.steps_run += 1
            torch.cuda.current_stream().wait_stream(self.stream)     # the caller's stream may read what the step wrote
            if layer_trace:
                res, trace = res
            if want:
                out.append((order, res))
        if not out:
            return (None, trace) if layer_trace else None
        if len(out) == 1:
            logits = out[0][1]
        else:
            keyed = sorted(((i, p, k, j) for k, (order, _) in enumerate(out) for j, (i, p, _) in enumerate(order)))
            logits = torch.stack([out[k][1][j] for _, _, k, j in keyed])
        return (logits, trace) if layer_trace else logits

    # -- the token loop -------------------------------------------------------------------------------
    def generate(self, requests: Iterable[GenRequest], generator=None) -> Dict[str, List[int]]:
        waiting = list(requests)
        done: Dict[str, List[int]] = {}
        state: Dict[str, dict] = {}
        while waiting or state:
            # admission: a request needs a slot and pages for its prompt and what it may generate
            while waiting and self.model.free_slots > 0:
                r = waiting[0]
                need = (len(r.prompt) + r.max_new_tokens + PAGE - 1) // PAGE
                held = sum((len(s["req"].prompt) + s["req"].max_new_tokens + PAGE - 1) // PAGE - s["pages"]() for s in state.values())
                if need > self.model.free_pages - held:
                    if not state:
                        raise RuntimeError(f"request {r.id!r} needs {need} pages, the pool has {self.model.pool_pages}")
                    break
                waiting.pop(0)
                if len(r.prompt) == 0:
                    raise ValueError(f"request {r.id!r} has an empty prompt")
                h = self.admit(r.id)
                state[r.id] = {"req": r, "fed": 0, "out": [], "next": None,
                               "pages": (lambda hh=h: (hh.offset + PAGE - 1) // PAGE)}
            budget = self.step_tokens
            entries = []
            for rid, s in state.items():                      # decode tokens first ...
                if s["next"] is not None and budget > 0:
                    entries.append((rid, [s["next"]], [0]))
                    budget -= 1
            for rid, s in state.items():                      # ... prompt portions with what is left
                r = s["req"]
                if s["next"] is None and s["fed"] < len(r.prompt) and budget > 0:
                    n = min(budget, len(r.prompt) - s["fed"])
                    toks = list(r.prompt[s["fed"]:s["fed"] + n])
                    last = s["fed"] + n == len(r.prompt)
                    entries.append((rid, toks, [n - 1] if last else []))
                    s["fed"] += n
                    budget -= n
            logits = self.step(entries)
            row = 0
            for rid, toks, places in entries:
                if not places:
                    continue
                s = state[rid]
                r = s["req"]
                tok = Sampler.sample(logits[row], r.decoding, generator=generator).token_id
                row += 1
                s["out"].append(tok)
                s["next"] = tok
                if len(s["out"]) >= r.max_new_tokens or tok in r.stop_ids:
                    done[rid] = s["out"]
                    self.finish(rid)
                    del state[rid]
        return done
