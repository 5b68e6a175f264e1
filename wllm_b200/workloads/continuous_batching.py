"""Continuous batching at a Gemma shape with random weights: many requests of mixed prompt lengths,
chunked prefill beside decoding requests, greedy decoding.

    python -m wllm_b200.workloads.continuous_batching --shape gemma-7b --requests 64 --min-prompt 128 \\
        --max-prompt 4096 --new-tokens 256 --chunk 2048

Prints one JSON line: wall time, prompt and generated tokens per second, steps, preemptions, pages at the
high-water mark, and the steps by kind (steps that carry prompt tokens, steps that only decode) with their
time on the device and, for the decode steps, the bytes they have to read (every weight once and the live
requests' keys and values) over that time.  Prompts are seeded uniform random token ids; nothing is read from
disk.  The policy it exercises is the reference's (src/wllm/engine/scheduler.py:207-274): requests mid-prompt
first, then new ones, under a budget of prompt tokens a step, decoding requests riding along.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

SHAPES = {
    "gemma-2b": dict(num_hidden_layers=18, hidden_size=2048, num_attention_heads=8, num_key_value_heads=1,
                     head_dim=256, intermediate_size=16384),
    "gemma-7b": dict(num_hidden_layers=28, hidden_size=3072, num_attention_heads=16, num_key_value_heads=16,
                     head_dim=256, intermediate_size=24576),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m wllm_b200.workloads.continuous_batching")
    ap.add_argument("--shape", default="gemma-7b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=4096)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--chunk", type=int, default=2048, help="prompt tokens per step (chunked prefill)")
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--async-scheduling", action="store_true", help="launch each step before the previous step's tokens are read")
    ap.add_argument("--page-fraction", type=float, default=1.0,
                    help="of the pages that all requests would need at their ends (below 1: requests wait, or are preempted)")
    ap.add_argument("--admission", default="worst_case", choices=["worst_case", "optimistic"])
    args = ap.parse_args(argv)

    from .. import LLM, SamplingParams
    from ..config import GemmaConfig
    raw = dict(SHAPES[args.shape], architectures=["GemmaForCausalLM"], vocab_size=256000, max_position_embeddings=8192,
               rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = GemmaConfig.from_dict(raw)
    g = torch.Generator().manual_seed(args.seed)
    lengths = torch.randint(args.min_prompt, args.max_prompt + 1, (args.requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lengths]
    blocks = sum(-(-(n + args.new_tokens) // args.block_size) for n in lengths) + 1
    blocks = max(int(blocks * args.page_fraction), -(-(max(lengths) + args.new_tokens) // args.block_size) + 1)
    llm = LLM(None, config=cfg, random_seed=1, dtype=args.dtype, block_size=args.block_size, num_blocks=blocks,
              chunked_prefill_tokens=args.chunk, max_num_seqs=args.requests, cuda_graphs=not args.no_graphs,
              async_scheduling=args.async_scheduling, admission=args.admission)
    sp = SamplingParams(temperature=0.0, max_tokens=args.new_tokens, ignore_eos=True)
    llm.generate(prompts[:2], SamplingParams(max_tokens=4, ignore_eos=True))        # warm-up: kernels, graphs
    torch.cuda.synchronize()
    for k in llm.scheduler.stats:
        llm.scheduler.stats[k] = 0
    cache, sched = llm.runner.cache, llm.scheduler
    page_bytes = cache.bytes_per_token() * cache.page_size
    weight_bytes = llm.model.weight_bytes()
    marks, loads = [], []          # an event in front of every step; (prompt tokens, decoded tokens, pages held) of the step
    start = time.perf_counter()
    reqs = [llm.add_request(p, sp) for p in prompts]
    while llm.has_unfinished():
        before = (sched.stats["prefill_tokens"], sched.stats["decode_tokens"])
        mark = torch.cuda.Event(enable_timing=True)
        mark.record()
        llm.step()
        held = cache.groups[0].pool.num_pages - cache.groups[0].pool.num_free
        marks.append(mark)
        loads.append((sched.stats["prefill_tokens"] - before[0], sched.stats["decode_tokens"] - before[1], held))
    last = torch.cuda.Event(enable_timing=True)
    last.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - start
    marks.append(last)
    outs = reqs
    kinds = {"prompt_steps": [], "decode_steps": []}
    decode_gbs = []
    for i, (prompt_tokens, decoded, held) in enumerate(loads):
        ms = marks[i].elapsed_time(marks[i + 1])
        if prompt_tokens > 0:
            kinds["prompt_steps"].append(ms)
        elif decoded > 0:
            kinds["decode_steps"].append(ms)
            decode_gbs.append((weight_bytes + held * page_bytes) / ms / 1e6)
    by_kind = {k: {"steps": len(v), "ms_total": round(sum(v), 1), "ms_mean": round(sum(v) / len(v), 3) if v else None}
               for k, v in kinds.items()}
    if decode_gbs:
        by_kind["decode_steps"]["gbs_mean"] = round(sum(decode_gbs) / len(decode_gbs), 0)
        by_kind["decode_steps"]["weight_gb"] = round(weight_bytes / 1e9, 2)
    from ..kernels import ops
    st = llm.stats
    generated = sum(len(o.output_token_ids) for o in outs)
    print(json.dumps({
        "workload": "continuous batching", "shape": args.shape, "layers": cfg.num_hidden_layers, "dtype": args.dtype,
        "requests": args.requests, "prompt_tokens": sum(lengths), "generated_tokens": generated,
        "wall_s": round(wall, 3), "prompt_tokens_per_s": round(sum(lengths) / wall, 1),
        "generated_tokens_per_s": round(generated / wall, 1), "total_tokens_per_s": round((sum(lengths) + generated) / wall, 1),
        "steps": st["steps"], "preemptions": st["preemptions"], "pages_high_water": st["pages_high_water"],
        "pages": blocks, "chunk": args.chunk, "kernel_status": ops.tc_gemm_status(llm.engine_config.device),
        "by_kind": by_kind,
        "all_finished_by_length": all(o.finish_reason == "length" and len(o.output_token_ids) == args.new_tokens for o in outs)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
