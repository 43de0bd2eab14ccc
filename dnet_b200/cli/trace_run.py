"""Replay a trace of steps through a model's batched step and write the logits that are asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input: one JSON object a line, {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.  All entries
of a step run as one batch through ``SequenceBatcher.step``; for a step with wanted places the logits go to
OUT/<step>.f32 (little-endian fp32 [wanted, vocab], in the order of entries and places); every step is answered with
a line ``done <step>``.  Nothing is sampled.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the logits are written to")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the cache pool holds (64-token pages)")
    ap.add_argument("--max-seqs", type=int, default=4, help="state slots (live requests)")
    a = ap.parse_args(argv)

    import torch

    from dnet_b200.shard.batching import SequenceBatcher, load_model

    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens, max_seqs=a.max_seqs,
                       max_batch_tokens=max(64, min(a.max_tokens, 8192)))
    eng = SequenceBatcher(model)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        entries = [(str(e["id"]), e["tokens"], e.get("want") or []) for e in st.get("entries", []) if e.get("tokens")]
        logits = eng.step(entries) if entries else None
        if logits is not None:
            model.check(eng.stream)
            data = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False).tobytes()
            tmp = os.path.join(a.out, ".%s.part" % st["step"])
            with open(tmp, "wb") as f:
                f.write(data)
            os.replace(tmp, os.path.join(a.out, "%s.f32" % st["step"]))
        for rid in st.get("end", []):
            eng.finish(str(rid))
        sys.stdout.write("done %s\n" % st["step"])
        sys.stdout.flush()
    eng.close()
    model.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
