"""``batched`` policy: a layer-list model (core/models/seqmix.py) served whole by this shard.

The fit / offload policies run one request's activation through a run of layers and hand it on; a layer-list model
is resident on one GPU and steps ragged batches, so this policy's ``process`` is short: a ``tokens`` frame of a nonce
becomes one entry of a ``SequenceBatcher.step`` (the nonce is the request id, admitted at its first frame), the last
position's logits are sampled with the framework's ``Sampler`` from the frame's decoding fields, and the final token
leaves through ``runtime.emit_result`` like the end shard's of the ring.  A prompt sent in chunks (every frame but
the last with ``batch_size == 0``) fills the cache and state and emits nothing until the last chunk.  A nonce gives
its state slot and pages back on ``runtime.release_nonce`` or after the runtime's KV time-to-live without a frame.
"""
from __future__ import annotations

import time

import numpy as np
import torch

from dnet_b200.core.decoding.config import DecodingConfig
from dnet_b200.core.decoding.sampler import Sampler
from dnet_b200.core.types.messages import ActivationMessage
from dnet_b200.utils.logger import logger
from dnet_b200.utils.time import utc_epoch_now
from . import _cuda_common as cc
from .base import ComputePolicy, register_policy


@register_policy("batched")
class BatchedStepPolicy(ComputePolicy):
    """One request per frame through the batched step of a resident layer-list model."""

    def configure_policy_for_model(self, req) -> None:
        self._mode = "batched"
        self.window_size = max(1, len(self.runtime.assigned_layers))
        self._last_seen: dict[str, float] = {}

    def release(self, nonce: str) -> None:
        """The request's slot and pages go back (kernels that still read them are ahead on the same stream)."""
        self._last_seen.pop(nonce, None)
        b = getattr(self.runtime, "batcher", None)
        if b is not None:
            b.finish(nonce)

    def _sweep(self, keep: str) -> None:
        ttl, now = float(self.runtime._kv_ttl_s), time.perf_counter()
        for n, ts in list(self._last_seen.items()):
            if n != keep and now - ts > ttl:
                self.release(n)

    def process(self, msg: ActivationMessage) -> None:
        rt = self.runtime
        try:
            with rt._model_lock:
                b = getattr(rt, "batcher", None)
                if not (rt.model and b is not None and rt.input_pool):
                    logger.error("Runtime %s: cannot process activation - model not loaded", rt.shard_id)
                    return
                if msg.dtype != "tokens":
                    logger.error("Runtime %s: a layer-list model takes token frames only (got %s)", rt.shard_id, msg.dtype)
                    rt.input_pool.release(msg.pool_id)
                    return
                T = int(np.prod(msg.shape))
                buf = rt.input_pool.get_buffer(msg.pool_id)
                if buf is None or T <= 0:
                    logger.error("Failed to get input buffer %s", msg.pool_id)
                    return
                ids = [int(t) for t in buf[:T].tolist()]
                rt.input_pool.release(msg.pool_id)
                self._sweep(msg.nonce)
                self._last_seen[msg.nonce] = time.perf_counter()
                more = cc.more_chunks_follow(msg)
                rt._compute_busy.set()
                logits = b.step([(msg.nonce, ids, [] if more else [T - 1])])
                if more:
                    return
                cfg = DecodingConfig(temperature=msg.temperature, top_p=msg.top_p, top_k=msg.top_k,
                                     repetition_penalty=msg.repetition_penalty, min_p=msg.min_p,
                                     min_tokens_to_keep=msg.min_tokens_to_keep)
                with torch.cuda.stream(rt.compute_stream):
                    res = Sampler.sample(logits[0], cfg, req_logprobs=msg.req_logprobs, req_top_logprobs=msg.req_top_logprobs)
                rt.emit_result(ActivationMessage(
                    nonce=msg.nonce, layer_id=rt._assigned_sorted[-1], pool_id=-1, shape=(1, 1, int(rt.model.hidden_size)),
                    batch_size=msg.batch_size, timestamp=utc_epoch_now(), node_origin=f"shard_{rt.shard_id}",
                    dtype=rt._wire_dtype_str, callback_url=msg.callback_url, lane=msg.lane, seq0=msg.seq0, is_final=True,
                    token_id=res.token_id, logprob=res.logprob, top_logprobs=res.top_logprobs))
        except Exception as e:
            logger.exception("Error in batched policy process: %s", e)
        finally:
            try:
                rt._compute_busy.clear()
            except Exception:
                pass

    def clear(self):
        b = getattr(self.runtime, "batcher", None)
        if b is not None:
            try:
                b.close()
            except Exception:
                pass
        self._last_seen = {}
