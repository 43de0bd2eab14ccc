"""Models given as a list of layers, each a sequence mixer plus an optional gated feed-forward, on
libdnet_b200_seq (include/dnet_b200_seq.h).

The llama-family classes of this package run one request per step and hand a [T, hidden] activation from layer to
layer; the families here run a *ragged batch* per step (portions of prompts beside single decoded tokens of up to
``max_seqs`` live sequences) through all layers, because what a layer carries between tokens is not only a KV page:
a recurrent mixer keeps an fp32 state and the last inputs of its short convolution per sequence, and the residual
is S fp32 streams.  The model owns the page pool and the state slots; ``SeqHandle`` is a sequence's lease on them,
the counterpart of ``KVHandle``.

``SeqMixRingModel`` reads the layer list from the config:

    {"architecture": NAME, "vocab": V, "width": W, "streams": S, "norm": {"eps": e}, "embedding": {"scale": c},
     "layers": [{"type": "attention" | "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv",             # both mixers
                           "scale", "rot": {"base", "dims"}, "mask": {"size"},     # attention
                           "kv_from": j},                                          # attention, optional
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Absent keys switch a mechanism off (no ``streams``: plain residual; no ``mask``: plain causal; no ``rot``: no
rotation; no ``conv``: no convolution; no ``kv_from``: own keys and values).
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from dnet_b200 import _seqabi
from .base import BaseRingModel, _stream_ptr


class SeqHandle:
    """One live sequence: a state slot of the model and the pages it has taken so far."""

    def __init__(self, model: "SeqMixRingModel", stream=None):
        self.model = model
        slot = C.c_int(-1)
        _seqabi.check(model._lib.dn_seq_open(model._h, _stream_ptr(stream), C.byref(slot)))
        self.slot = int(slot.value)

    @property
    def offset(self) -> int:
        return int(self.model._lib.dn_seq_length(self.model._h, self.slot)) if self.slot >= 0 else 0

    def free(self) -> None:
        if self.slot >= 0 and self.model._h:
            _seqabi.check(self.model._lib.dn_seq_close(self.model._h, self.slot))
        self.slot = -1


def parse_layer_list(cfg: dict) -> Tuple[_seqabi.SeqCfg, List[_seqabi.LayerCfg]]:
    """config.json of a layer-list family -> the C structs (every size and constant comes from the config)."""
    layers = []
    for i, L in enumerate(cfg["layers"]):
        mx = L["mixer"]
        kind = L["type"]
        lc = _seqabi.LayerCfg()
        if kind == "attention":
            lc.mixer = _seqabi.DN_MIX_ATTENTION
            lc.scale = float(mx.get("scale", float(mx["dim"]) ** -0.5))
            lc.chunk = int((mx.get("mask") or {}).get("size", 0))
            rot = mx.get("rot") or {}
            lc.rot_dims = int(rot.get("dims", 0))
            lc.rot_base = float(rot.get("base", 10000.0))
            lc.kv_from = int(mx["kv_from"]) if mx.get("kv_from") is not None else -1
        elif kind == "delta":
            lc.mixer = _seqabi.DN_MIX_DELTA
            lc.kv_from = -1
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        lc.heads, lc.kv_heads = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"]))
        lc.dim, lc.vdim = int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
        lc.conv = int(mx.get("conv", 0) or 0)
        mlp = L.get("mlp")
        if mlp:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} unsupported")
            lc.ff = int(mlp["ff"])
        layers.append(lc)
    sc = _seqabi.SeqCfg(width=int(cfg["width"]), vocab=int(cfg["vocab"]), n_layers=len(layers), streams=int(cfg.get("streams", 0) or 0),
                        eps=float((cfg.get("norm") or {}).get("eps", 1e-6)),
                        embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)))
    return sc, layers


class SeqMixRingModel(BaseRingModel):
    """A whole layer-list model on one GPU: owns cache pool + state slots, runs ragged-batch steps."""

    model_type: Optional[str] = None
    step_kernel_ok = False
    batched_step = True        # ShardRuntime loads it whole and serves it with the `batched` policy over shard.batching.SequenceBatcher

    def __init__(self, model_config: Any, assigned_layers: Optional[List[int]] = None, is_api_layer: bool = False, *,
                 dtype: str = "bfloat16", kv_pool_pages: int = 0, max_seqs: int = 4, max_batch_tokens: int = 2048, **_ignored):
        if is_api_layer and assigned_layers:
            raise RuntimeError("API layer doesn't handle layers")
        self.config = dict(model_config)
        self.model_config = model_config
        sc, layers = parse_layer_list(self.config)
        n = len(layers)
        if assigned_layers is not None and sorted(assigned_layers) != list(range(n)):
            raise ValueError("a layer-list model is served whole by one shard: its layers share pages (kv_from) and fp32 "
                             f"residual streams; assign all {n} layers")
        if dtype in ("bfloat16", "bf16"):
            self.dtype, sc.dtype = torch.bfloat16, _seqabi.DN_SEQ_BF16
        elif dtype in ("float32", "fp32"):
            self.dtype, sc.dtype = torch.float32, _seqabi.DN_SEQ_F32
        else:
            raise ValueError(f"dtype {dtype!r} unsupported (bfloat16 or float32)")
        sc.pool_pages = int(kv_pool_pages) or 64
        sc.max_seqs, sc.max_batch_tokens = int(max_seqs), int(max_batch_tokens)
        self._lib = _seqabi.load()
        self.device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        _seqabi.init(self.device)
        arr = (_seqabi.LayerCfg * n)(*layers)
        h = C.c_void_p()
        _seqabi.check(self._lib.dn_seq_model_create(C.byref(sc), arr, C.byref(h)))
        self._h = h.value
        self._cfg_struct, self._layer_structs = sc, layers
        self.layers = list(range(n))
        self.abs_to_local = {i: i for i in self.layers}
        self.hidden_size, self.vocab_size = int(sc.width), int(sc.vocab)
        self.max_seqs, self.max_batch_tokens, self.pool_pages = int(sc.max_seqs), int(sc.max_batch_tokens), int(sc.pool_pages)
        self._bound: Dict[str, torch.Tensor] = {}

    # -- weights -----------------------------------------------------------------------------
    def expected_tensors(self) -> Dict[str, Tuple[int, ...]]:
        """Checkpoint name -> shape, from the config alone."""
        W, V, S = self.hidden_size, self.vocab_size, int(self._cfg_struct.streams)
        out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
        for i, lc in enumerate(self._layer_structs):
            p = f"l{i}."
            att = lc.mixer == _seqabi.DN_MIX_ATTENTION
            cq = (lc.heads if att else lc.kv_heads) * lc.dim
            ck, cv = lc.kv_heads * lc.dim, (lc.kv_heads if att else lc.heads) * lc.vdim
            co = lc.heads * lc.vdim
            own = not (att and lc.kv_from >= 0)
            out[p + "norm1"] = (W,)
            out[p + "mix.q"] = (cq, W)
            out[p + "mix.o"] = (W, co)
            if own:
                out[p + "mix.k"], out[p + "mix.v"] = (ck, W), (cv, W)
            if lc.conv > 0:
                out[p + "mix.q.conv"] = (cq, lc.conv)
                if own:
                    out[p + "mix.k.conv"], out[p + "mix.v.conv"] = (ck, lc.conv), (cv, lc.conv)
            if att:
                out[p + "mix.q.norm"] = (cq,)
                if own:
                    out[p + "mix.k.norm"] = (ck,)
            else:
                out[p + "mix.a"] = out[p + "mix.b"] = (lc.heads, W)
                out[p + "mix.g"] = (co, W)
                out[p + "mix.A_log"] = out[p + "mix.dt_bias"] = (lc.heads,)
                out[p + "mix.norm"] = (lc.vdim,)
            if lc.ff > 0:
                out[p + "norm2"] = (W,)
                out[p + "mlp.gate"] = out[p + "mlp.up"] = (lc.ff, W)
                out[p + "mlp.down"] = (W, lc.ff)
            if S > 0:
                for q in ("hc1", "hc2") if lc.ff > 0 else ("hc1",):
                    out[p + q + ".in"] = out[p + q + ".out"] = (S,)
                    out[p + q + ".mix"] = (S, S)
        return out

    def load_weights(self, file_or_weights, strict: bool = True):
        """Bind tensors by pointer.  Names: the checkpoint's (``l3.mix.q``, ``embed``, ``final.norm``, ``head``) or the
        loader's (``layers.3.mix.q``, ``embed_tokens.weight``, ``norm.weight``, ``lm_head.weight``)."""
        items = file_or_weights.items() if isinstance(file_or_weights, dict) else file_or_weights
        want = self.expected_tensors()
        alias = {"embed_tokens.weight": "embed", "norm.weight": "final.norm", "lm_head.weight": "head"}
        for key, t in items:
            key = key.decode() if isinstance(key, (bytes, bytearray)) else str(key)
            key = key[6:] if key.startswith("model.") else key
            key = alias.get(key, key)
            if key.startswith("layers."):
                _, idx, rest = key.split(".", 2)
                key = f"l{idx}.{rest}"
            shape = want.get(key)
            if shape is None:
                if strict:
                    raise ValueError(f"unexpected tensor {key}")
                continue
            if tuple(t.shape) != shape:
                raise ValueError(f"{key}: shape {tuple(t.shape)}, the config asks for {shape}")
            if not t.is_cuda or t.dtype != self.dtype or not t.is_contiguous():
                raise ValueError(f"{key}: expected a contiguous {self.dtype} CUDA tensor")
            if key in _seqabi.MODEL_SLOT:
                _seqabi.check(self._lib.dn_seq_bind(self._h, -1, _seqabi.MODEL_SLOT[key], t.data_ptr()))
            else:
                lname, suffix = key.split(".", 1)
                _seqabi.check(self._lib.dn_seq_bind(self._h, int(lname[1:]), _seqabi.LAYER_SLOT[suffix], t.data_ptr()))
            self._bound[key] = t     # keep the borrowed memory alive
        return self

    def missing_tensors(self) -> List[str]:
        return sorted(set(self.expected_tensors()) - set(self._bound))

    # -- sequences and the step ----------------------------------------------------------------
    def make_cache(self, max_tokens: int = 0, stream=None) -> SeqHandle:
        return SeqHandle(self, stream)

    @property
    def free_pages(self) -> int:
        return int(self._lib.dn_seq_free_pages(self._h))

    @property
    def free_slots(self) -> int:
        return int(self._lib.dn_seq_free_slots(self._h))

    def step(self, entries: Sequence[Tuple[SeqHandle, Sequence[int]]], want: Sequence[int], stream=None,
             layer_trace: bool = False):
        """One batched step.  entries: (sequence, its next tokens); want: rows of the concatenated tokens whose
        logits are returned as fp32 [len(want), vocab] (None if empty).  With layer_trace also the residual after
        every layer, fp32 [layers, N, width]."""
        E = len(entries)
        slots = (C.c_int32 * E)(*[h.slot for h, _ in entries])
        counts = (C.c_int32 * E)(*[len(t) for _, t in entries])
        flat = [int(x) for _, t in entries for x in t]
        N = len(flat)
        toks = (C.c_int32 * N)(*flat)
        nw = len(want)
        wr = (C.c_int32 * max(1, nw))(*[int(x) for x in want])
        dev = torch.device("cuda", self.device)
        logits = torch.empty(nw, self.vocab_size, dtype=torch.float32, device=dev) if nw else None
        trace = torch.empty(len(self.layers), N, self.hidden_size, dtype=torch.float32, device=dev) if layer_trace else None
        _seqabi.check(self._lib.dn_seq_step(self._h, E, slots, counts, toks, nw, wr, logits.data_ptr() if nw else None,
                                            trace.data_ptr() if layer_trace else None, _stream_ptr(stream)))
        return (logits, trace) if layer_trace else logits

    def check(self, stream=None) -> None:
        """Synchronise and raise if a bounded wait inside a kernel ever ran out (results would be invalid)."""
        _seqabi.check(self._lib.dn_seq_check(self._h, _stream_ptr(stream)))

    def profile(self, on: bool) -> None:
        """Switch the per-phase device timers of the step on or off."""
        _seqabi.check(self._lib.dn_seq_profile(self._h, int(bool(on))))

    def set_graphs(self, on: bool) -> None:
        """Decode steps replay a captured CUDA graph (default) or launch their kernels one by one."""
        _seqabi.check(self._lib.dn_seq_set_graphs(self._h, int(bool(on))))

    def profile_read(self, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per phase over the steps run since the last read (synchronises)."""
        ms = (C.c_double * len(_seqabi.PHASES))()
        _seqabi.check(self._lib.dn_seq_profile_read(self._h, ms, int(bool(reset))))
        return {n: float(ms[i]) for i, n in enumerate(_seqabi.PHASES)}

    # -- BaseRingModel surface ---------------------------------------------------------------------
    def _whole(self, *_a, **_k):
        raise NotImplementedError("layer-list models run whole batched steps (SeqMixRingModel.step); the residual between "
                                  "their layers is S fp32 streams, not a [T, hidden] activation of the wire dtype")

    embed = normalize = lm_project = apply_single_layer = _whole

    @property
    def decoding_layers(self):
        return self.layers

    @property
    def head_dim(self) -> Tuple[int, int]:
        lc = self._layer_structs[0]
        return (int(lc.dim), int(lc.vdim))

    @property
    def n_kv_heads(self) -> int:
        return int(self._layer_structs[0].kv_heads)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def unload_layers(self, abs_layers: List[int]) -> None:
        raise NotImplementedError("layer-list models stay resident")

    def is_bound(self, abs_layer: int) -> bool:
        return not any(k.startswith(f"l{abs_layer}.") for k in self.missing_tensors())

    def apply_quantization_from_config(self, model_config: Any, model_metadata: Any) -> bool:
        return False

    def destroy(self) -> None:
        if getattr(self, "_h", None):
            self._lib.dn_seq_model_destroy(self._h)
            self._h = None
            self._bound.clear()


class MoputarRingModel(SeqMixRingModel):
    """Moputar: chunk-masked attention layers (some reading an earlier layer's keys and values) interleaved with
    gated delta-rule layers, short convolutions on q / k / v, hyper-connected residual streams."""

    model_type = "moputar"
