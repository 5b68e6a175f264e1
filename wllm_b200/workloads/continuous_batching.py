"""Continuous batching at a Gemma shape with random weights: many requests of mixed prompt lengths,
chunked prefill beside decoding requests, greedy decoding.

    python -m wllm_b200.workloads.continuous_batching --shape gemma-7b --requests 64 --min-prompt 128 \\
        --max-prompt 4096 --new-tokens 256 --chunk 2048

Prints one JSON line: wall time, prompt and generated tokens per second, steps, preemptions, pages at the
high-water mark.  Prompts are seeded uniform random token ids; nothing is read from disk.
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
    llm = LLM(None, config=cfg, random_seed=1, dtype=args.dtype, block_size=args.block_size, num_blocks=blocks,
              chunked_prefill_tokens=args.chunk, max_num_seqs=args.requests, cuda_graphs=not args.no_graphs,
              async_scheduling=args.async_scheduling)
    sp = SamplingParams(temperature=0.0, max_tokens=args.new_tokens, ignore_eos=True)
    llm.generate(prompts[:2], SamplingParams(max_tokens=4, ignore_eos=True))        # warm-up: kernels, graphs
    torch.cuda.synchronize()
    for k in llm.scheduler.stats:
        llm.scheduler.stats[k] = 0
    start = time.perf_counter()
    outs = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    wall = time.perf_counter() - start
    from ..kernels import ops
    st = llm.stats
    generated = sum(len(o.token_ids) for o in outs)
    print(json.dumps({
        "workload": "continuous batching", "shape": args.shape, "layers": cfg.num_hidden_layers, "dtype": args.dtype,
        "requests": args.requests, "prompt_tokens": sum(lengths), "generated_tokens": generated,
        "wall_s": round(wall, 3), "prompt_tokens_per_s": round(sum(lengths) / wall, 1),
        "generated_tokens_per_s": round(generated / wall, 1), "total_tokens_per_s": round((sum(lengths) + generated) / wall, 1),
        "steps": st["steps"], "preemptions": st["preemptions"], "pages_high_water": st["pages_high_water"],
        "pages": blocks, "chunk": args.chunk, "kernel_status": ops.tc_gemm_status(llm.engine_config.device),
        "all_finished_by_length": all(o.finish_reason == "length" and len(o.token_ids) == args.new_tokens for o in outs)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
