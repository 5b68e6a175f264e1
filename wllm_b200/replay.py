"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing and owns no forward pass, cache or loader: it builds the model
and the runner as generation does and calls the same `ModelRunner.step`.  Steps are
read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` are one batch (a request's next tokens and the places among them whose
logits are wanted); `end` lists the requests that are finished after the step, whose
pages go back to the pool.  For a step that wants something, `<out>/<step>.f32`
receives the logits [wanted, vocab] as little-endian 32-bit floats in the order of
the entries and of `want`.  After every step a line `done <step>` is printed and
flushed.  The pool holds ceil(N / page size) pages, so pages are used again.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .config import EngineConfig
    from .engine import StepEntry, build_model, build_runner

    os.makedirs(args.out, exist_ok=True)
    engine = EngineConfig(dtype=args.dtype, block_size=args.block_size, max_num_seqs=16, device=args.device)
    model = build_model(args.model, engine.dtype, engine.device)
    pages = max(1, -(-args.max_tokens // engine.block_size))
    runner = build_runner(model, engine, num_pages=pages)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in live:
                live[rid] = runner.cache.open(rid)
            entries.append(StepEntry(live[rid], e["tokens"], e.get("want", [])))
        logits = runner.step(entries)
        if logits.shape[0] > 0:
            logits.detach().to("cpu").numpy().astype("<f4").tofile(os.path.join(args.out, f"{rec['step']}.f32"))
        for rid in rec.get("end", []):
            if rid in live:
                runner.cache.close(live.pop(rid))
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
