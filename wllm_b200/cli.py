"""Command line: offline generation from token ids.

    python -m wllm_b200 --model DIR --prompt-ids 2,651,6037 --max-tokens 32
    python -m wllm_b200 --write-random-model DIR --config-json cfg.json --random-seed 1

Engine options carry the reference's names and meanings (src/wllm/cli.py:21-56):
--model, --device, --num-blocks, --block-size, --dtype, --cuda-graphs,
--chunked-prefill-tokens, --log-level.  The reference's command only starts its HTTP
server; servers are outside this engine, so the command generates instead, and the
sampling options of the reference's requests (temperature, top_k, top_p, min_p,
repetition_penalty, seed, max_tokens; src/wllm/api/schemas.py:30-47) become flags.
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
import time


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="wllm_b200", description="Gemma 1 inference on one B200")
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--device", default="cuda", choices=["cuda"], help="the engine has no CPU path")
    ap.add_argument("--num-blocks", type=int, default=256, help="KV cache blocks (block_size tokens each)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--cuda-graphs", action="store_true", help="replay captured CUDA graphs for decode steps")
    ap.add_argument("--async-scheduling", action="store_true",
                    help="launch each step before the host has read the tokens of the step before")
    ap.add_argument("--chunked-prefill-tokens", type=int, default=None,
                    help="max prompt tokens processed per scheduler step (enables chunked prefill)")
    ap.add_argument("--max-num-seqs", type=int, default=256, help="requests that may be live at once")
    ap.add_argument("--admission", default="worst_case", choices=["worst_case", "optimistic"])
    ap.add_argument("--log-level", default="INFO", choices=["DEBUG", "INFO", "WARNING", "ERROR"])
    g = ap.add_argument_group("prompts (token ids)")
    g.add_argument("--prompt-ids", action="append", default=[], metavar="I,J,K", help="one prompt; may be repeated")
    g.add_argument("--prompt-lens", default=None, metavar="N,M", help="random prompts of these lengths")
    g.add_argument("--prompt-seed", type=int, default=0)
    s = ap.add_argument_group("sampling")
    s.add_argument("--max-tokens", type=int, default=16)
    s.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    s.add_argument("--top-k", type=int, default=0)
    s.add_argument("--top-p", type=float, default=1.0)
    s.add_argument("--min-p", type=float, default=0.0)
    s.add_argument("--repetition-penalty", type=float, default=1.0)
    s.add_argument("--seed", type=int, default=None)
    s.add_argument("--ignore-eos", action="store_true")
    r = ap.add_argument_group("random weights")
    r.add_argument("--write-random-model", metavar="DIR", help="write config.json and model.safetensors, then exit")
    r.add_argument("--config-json", metavar="FILE", help="configuration for --write-random-model")
    r.add_argument("--random-seed", type=int, default=0)
    return ap


def main(argv=None) -> int:
    args = parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, args.log_level), format="%(asctime)s %(levelname)s %(message)s")
    log = logging.getLogger("wllm_b200")
    if args.write_random_model:
        if not args.config_json:
            parser().error("--write-random-model needs --config-json")
        from .weights import write_random_model
        with open(args.config_json, "r", encoding="utf-8") as f:
            raw = json.load(f)
        import torch
        write_random_model(args.write_random_model, raw, args.random_seed,
                           dtype=torch.float32 if args.dtype == "float32" else torch.bfloat16)
        log.info("wrote %s", args.write_random_model)
        return 0
    if not args.model:
        parser().error("--model is required")
    from . import LLM, SamplingParams
    llm = LLM(args.model, dtype=args.dtype, block_size=args.block_size, num_blocks=args.num_blocks,
              chunked_prefill_tokens=args.chunked_prefill_tokens, max_num_seqs=args.max_num_seqs,
              cuda_graphs=args.cuda_graphs, device="cuda:0", admission=args.admission,
              async_scheduling=args.async_scheduling)
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    if args.prompt_lens:
        import torch
        g = torch.Generator().manual_seed(args.prompt_seed)
        vocab = llm.model.plan.vocab_size
        prompts += [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in args.prompt_lens.split(",")]
    if not prompts:
        parser().error("give --prompt-ids or --prompt-lens")
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                        repetition_penalty=args.repetition_penalty, seed=args.seed, max_tokens=args.max_tokens,
                        ignore_eos=args.ignore_eos)
    start = time.time()
    outs = llm.generate(prompts, sp)
    elapsed = time.time() - start
    for o in outs:
        print(json.dumps({"request": o.request_id, "prompt_tokens": len(o.prompt_token_ids), "token_ids": o.token_ids,
                          "finish_reason": o.finish_reason}))
    st = llm.stats
    log.info("%d requests, %d prompt + %d generated tokens in %.2f s; %d steps, %d preemptions, pages high-water %s",
             len(outs), sum(len(o.prompt_token_ids) for o in outs), sum(len(o.token_ids) for o in outs), elapsed,
             st["steps"], st["preemptions"],
             st["pages_high_water"])
    return 0


if __name__ == "__main__":
    sys.exit(main())
