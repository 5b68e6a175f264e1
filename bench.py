"""Gemma-2B decode and prefill throughput on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]

A step is one decode step of `batch` requests whose caches hold `context` tokens.
Prints ONE JSON line: `value` = decoded tokens per second timed on the device with CUDA
events over exactly K steps; `e2e` = the same through the Python entry point
(`LLM.step`: pinned host index arrays in, sampled token ids out, every step);
`prefill` = one prompt of 2,048 tokens; `roofline` = bytes a decode step has to read
(every weight once and the live requests' cache) over its time, against the measured copy
bandwidth; `points` = decode at batch 1 and 64 at the same context, at batch 1, 8 and 64 with
1,024 cached tokens, and the headline case without captured graphs.  The headline is the median
of `--regions` timed regions of exactly K steps each (`ms_per_step_regions` lists them all).  Weights are random N(0, 0.02), token ids
are seeded uniform random, the caches of the device-timed runs are filled with random
keys and values (synthetic context); the end-to-end run prefills its prompts for real.
Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from
the fallback figures of an earlier measurement on this pool.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GEMMA_2B = dict(vocab_size=256000, hidden_size=2048, intermediate_size=16384, num_hidden_layers=18,
                num_attention_heads=8, num_key_value_heads=1, head_dim=256, rms_norm_eps=1e-6, rope_theta=10000.0,
                max_position_embeddings=8192, tie_word_embeddings=True)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()
        self.file.close()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.file.name) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 6 or not parts[0].isdigit():
                        continue
                    sm.append(int(parts[0]))
                    mx.append(int(parts[1]))
                    reasons.update(n for n, v in zip(names, parts[2:6]) if v.lower().startswith("active"))
            os.unlink(self.file.name)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def fill_synthetic_context(runner, caches, context: int, seed: int) -> None:
    """Give every request `context` cached tokens of random keys and values without running the model."""
    import torch
    for rc in caches:
        runner.cache.reserve([(rc, context)])
        runner.cache.commit(rc, context)
    g = torch.Generator(device=runner.device).manual_seed(seed)
    for group in runner.cache.groups:
        pages = group.pages
        flat = pages.view(-1)
        step = 1 << 26
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randn(n, generator=g, device=runner.device, dtype=torch.float32).to(pages.dtype)


def decode_run(model, engine_cfg, batch: int, context: int, steps: int, warmup: int, page_size: int, regions: int = 1):
    """Device-timed decode of `batch` single tokens a step, from `context` cached tokens on: `regions` timed
    regions of exactly `steps` steps each, one after the other (CUDA events around each, a synchronize on both
    sides).  Returns the median region's milliseconds per step, the kernel launches of one region, the bytes of
    keys and values a step reads at the middle of the run, the clock samples, and every region's ms per step."""
    import torch
    from wllm_b200.engine import StepEntry, build_runner
    from wllm_b200.kernels import ops
    from wllm_b200.sampling import SamplingParams
    from wllm_b200.sampling.sampler import Sampler
    total = context + warmup + regions * steps + 1
    pages = batch * (-(-total // page_size)) + 1
    runner = build_runner(model, engine_cfg, num_pages=pages)
    if engine_cfg.cuda_graphs:
        runner.enable_graphs()
    sampler = Sampler(runner.device)
    caches = [runner.cache.open(i) for i in range(batch)]
    fill_synthetic_context(runner, caches, context, seed=3)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, model.plan.vocab_size, (warmup + regions * steps, batch), generator=g).tolist()
    greedy = [SamplingParams()] * batch
    zeros, empty = [0] * batch, [set()] * batch

    def one(i):
        logits = runner.step([StepEntry(rc, [tokens[i][b]], [0]) for b, rc in enumerate(caches)])
        sampler.launch(logits, greedy, zeros, zeros, empty)
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()

    def table_width(tokens):       # captured decode steps are keyed by the block table's width, a power of two
        width = 8
        while width * page_size < tokens:
            width *= 2
        return width
    if engine_cfg.cuda_graphs and table_width(context + warmup + 1) != table_width(context + warmup + regions * steps):
        print(f"note: the timed steps cross from {table_width(context + warmup + 1)} to "
              f"{table_width(context + warmup + regions * steps)} pages a request: one of them captures a new graph, and "
              "the time per step of that region includes the capture", file=sys.stderr)
    per_region, launches = [], 0
    with ClockSampler() as clocks:
        for r in range(regions):
            launches0, graph0 = ops.launches, runner.graph_launches
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for i in range(warmup + r * steps, warmup + (r + 1) * steps):
                one(i)
            end.record()
            torch.cuda.synchronize()
            per_region.append(start.elapsed_time(end) / steps)
            launches = (ops.launches - launches0) + (runner.graph_launches - graph0)
    ms = statistics.median(per_region)
    kv_bytes = batch * (context + warmup + regions * steps / 2.0) * runner.cache.bytes_per_token()
    for rc in caches:
        runner.cache.close(rc)
    del runner
    torch.cuda.empty_cache()
    return ms, launches, kv_bytes, clocks.summary(), per_region


def prefill_run(model, engine_cfg, tokens: int, page_size: int, repeats: int = 3):
    import torch
    from wllm_b200.engine import StepEntry, build_runner
    runner = build_runner(model, engine_cfg, num_pages=-(-tokens // page_size) + 1)
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, model.plan.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(repeats + 1):
        rc = runner.cache.open(i)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(rc, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i > 0:
            times.append(start.elapsed_time(end))
        runner.cache.close(rc)
    del runner
    torch.cuda.empty_cache()
    return min(times)


def prefill_flops(cfg, layers: int, tokens: int) -> float:
    H, I, nq, nkv, hd, V = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                            cfg.head_dim, cfg.vocab_size)
    per_layer = 2.0 * tokens * ((nq + 2 * nkv) * hd * H + nq * hd * H + 3 * I * H) + 2.0 * nq * hd * tokens * tokens
    return layers * per_layer + 2.0 * V * H


def e2e_run(cfg, args, page_size: int):
    """The same decode through LLM.add_request / LLM.step: real prefill of the prompts, then `--regions` timed
    regions of exactly K steps each by the host's clock (a synchronize on both sides of each); the median region
    is reported, as for the device-timed number."""
    import torch
    from wllm_b200 import LLM, SamplingParams
    # requests that finish their prompt early decode while the others still prefill: leave room for that
    prefill_steps = args.batch * (-(-args.context // 2048)) + 1
    timed = args.regions * args.steps
    context = min(args.context, cfg.max_position_embeddings - (args.warmup + timed) - prefill_steps - 4)
    total = context + args.warmup + timed + prefill_steps + 4
    llm = LLM(None, config=cfg, random_seed=1, dtype="bfloat16", block_size=page_size,
              num_blocks=args.batch * (-(-total // page_size)) + 1, chunked_prefill_tokens=2048,
              max_num_seqs=max(args.batch, 8), cuda_graphs=not args.no_graphs, async_scheduling=True)
    g = torch.Generator().manual_seed(11)
    sp = SamplingParams(temperature=0.0, max_tokens=args.warmup + timed + prefill_steps + 2, ignore_eos=True)
    for _ in range(args.batch):
        llm.add_request(torch.randint(0, cfg.vocab_size, (context,), generator=g).tolist(), sp)
    while any(r.status.value != "running" for r in llm.scheduler.live) or llm.scheduler.waiting:
        llm.step()
    for _ in range(args.warmup):
        llm.step()
    per_region = []
    for _ in range(args.regions):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            got = llm.step()       # launches this step, then reads the tokens of the step before (pipelined)
            assert len(got) == args.batch
        torch.cuda.synchronize()
        per_region.append((time.perf_counter() - t0) / args.steps)
    sec = sorted(per_region)[len(per_region) // 2]
    h2d = llm.runner.h2d_bytes + llm.sampler.h2d_bytes
    d2h = llm.sampler.d2h_bytes
    del llm
    torch.cuda.empty_cache()
    return args.batch / sec, h2d, d2h


def reference_arm(args) -> int:
    """The unmodified reference from baseline/_ref through its own classes: GemmaForCausalLM with random
    weights, KVCacheManager, Scheduler (src/wllm/engine/scheduler.py).

    Prefill: one request of 2,048 random tokens with max_new_tokens=1 goes Scheduler.step -> _prefill ->
    prefill_with_cache... (the vendor's matrix library and torch's fused attention) and finishes there
    (scheduler.py:276-288, 460-463): the second half of the headline metric, on the stock path.
    Decode: needs the reference's own CUDA kernel, which it builds at first use.  Where that build fails (it
    passes an MSVC-only flag), the decode half is `unavailable`; beside it, labelled as what it is, stands the
    reference's model with its own plain-PyTorch attention (`_paged_attention_decode_cpu`, device-agnostic) put
    in the kernel's place on the GPU: not the stock path, but the floor that a plain PyTorch engine reaches."""
    def unavailable(why: str, **more) -> int:
        print(json.dumps(dict({"impl": "reference", "unavailable": " ".join(why.split())[:400]}, **more)))
        return 0
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "wllm")):
        return unavailable("the reference is not installed under baseline/_ref (pip install --no-index --no-deps "
                           "--target baseline/_ref <reference checkout>)")
    sys.path.insert(0, ref)
    try:
        import torch
        import wllm.kernels.paged_attention as ref_attention
        from wllm.engine.kv_cache import KVCacheManager
        from wllm.engine.scheduler import Scheduler
        from wllm.engine.sequence import Sequence
        from wllm.models.config import ModelConfig
        from wllm.models.gemma import GemmaForCausalLM
    except Exception as e:   # noqa: BLE001
        return unavailable(f"the reference does not import here: {type(e).__name__}: {e}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    c = GEMMA_2B
    cfg = ModelConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"],
                      num_hidden_layers=args.layers or c["num_hidden_layers"], num_attention_heads=c["num_attention_heads"],
                      num_key_value_heads=c["num_key_value_heads"], rms_norm_eps=c["rms_norm_eps"],
                      rope_theta=c["rope_theta"], max_position_embeddings=c["max_position_embeddings"],
                      tie_word_embeddings=True, attention_bias=False, explicit_head_dim=c["head_dim"])
    torch.manual_seed(1)
    model = GemmaForCausalLM(cfg)
    with torch.no_grad():
        for p in model.parameters():
            p.normal_(0, 0.02)
    model = model.to(device="cuda", dtype=torch.bfloat16).eval()
    g = torch.Generator().manual_seed(11)

    def new_cache(tokens_each: int, requests: int):
        blocks = requests * (-(-tokens_each // 16)) + 1
        return KVCacheManager(cfg.num_hidden_layers, blocks, 16, cfg.num_key_value_heads, cfg.head_dim, device="cuda")

    # -- prefill of 2,048 tokens, stock path -----------------------------------------------------
    T = 2048
    sched = Scheduler(model, new_cache(T + 2, 1))
    times = []
    for i in range(4):
        sched.add_request(Sequence(seq_id=i, prompt_token_ids=torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist(),
                                   max_new_tokens=1))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done = sched.step()
        torch.cuda.synchronize()
        if i > 0:
            times.append(time.perf_counter() - t0)
        assert len(done) == 1 and done[0].is_finished()
    prefill = {"value": round(T / min(times), 1), "tokens": T, "ms": round(min(times) * 1e3, 3),
               "path": "Scheduler.step -> _prefill, stock"}
    del sched
    torch.cuda.empty_cache()

    context = args.context or c["max_position_embeddings"] - (args.warmup + args.steps) - 2

    def decode(steps: int, warmup: int):
        sched = Scheduler(model, new_cache(context + warmup + steps + 66, args.batch), max_prefill_tokens_per_step=2048)
        for i in range(args.batch):
            sched.add_request(Sequence(seq_id=100 + i, prompt_token_ids=torch.randint(0, cfg.vocab_size, (context,), generator=g).tolist(),
                                       max_new_tokens=warmup + steps + 64))
        while sched.waiting or any(s.status.value != "running" for s in sched.running):
            sched.step()
        for _ in range(warmup):
            sched.step()
        torch.cuda.synchronize()
        with ClockSampler() as clocks:
            t0 = time.perf_counter()
            for _ in range(steps):
                sched.step()
            torch.cuda.synchronize()
            sec = (time.perf_counter() - t0) / steps
        return sec, clocks.summary()

    config = {"model": "gemma-2b", "layers": cfg.num_hidden_layers, "global_batch": args.batch, "seq_len": context,
              "page_size": 16}
    try:
        ref_attention._get_ext()           # the reference's own JIT build of csrc/paged_attention.cu
    except Exception as e:   # noqa: BLE001
        first = str(e).strip().splitlines()[0] if str(e).strip() else type(e).__name__
        fallback = None
        try:
            # not the stock path: the reference's device-agnostic attention where its kernel would stand
            ref_attention.paged_attention_decode = ref_attention._paged_attention_decode_cpu
            sec, clocks = decode(min(args.steps, 8), 2)
            fallback = {"value": round(args.batch / sec, 1), "unit": "tokens/s", "ms_per_step": round(sec * 1e3, 3),
                        "steps": min(args.steps, 8), "clocks": clocks,
                        "path": "reference model and scheduler, its plain-PyTorch attention in place of its CUDA kernel (not stock)"}
        except Exception as e2:   # noqa: BLE001
            fallback = {"unavailable": f"{type(e2).__name__}: {str(e2)[:200]}"}
        return unavailable("decode: the reference's CUDA decode kernel does not build on this box (it passes the MSVC-only "
                           f"flag /Zc:preprocessor, src/wllm/kernels/paged_attention.py:16-20): {first}",
                           metric="Gemma-2B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tokens", config=config,
                           prefill=prefill, decode_torch_fallback=fallback)
    sec, clocks = decode(args.steps, args.warmup)
    print(json.dumps({"metric": "Gemma-2B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tokens", "impl": "reference",
                      "value": round(args.batch / sec, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 4), "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                      "config": config, "prefill": prefill, "clocks": clocks}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None, help="cached tokens per request when the timed steps begin")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    from wllm_b200.config import EngineConfig, GemmaConfig
    from wllm_b200.engine import build_model

    raw = dict(GEMMA_2B, architectures=["GemmaForCausalLM"])
    layers_full = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = GemmaConfig.from_dict(raw)
    args.regions = max(1, args.regions)
    if args.context is None:
        args.context = cfg.max_position_embeddings - (args.warmup + args.regions * args.steps) - 2
    ps = args.page_size
    engine_cfg = EngineConfig(dtype="bfloat16", block_size=ps, max_num_seqs=max(64, args.batch), cuda_graphs=not args.no_graphs)
    pk = peaks()
    model = build_model(None, engine_cfg.dtype, engine_cfg.device, config=cfg, random_seed=1)
    weight_bytes = model.weight_bytes()

    ms, launches, kv_bytes, clocks, per_region = decode_run(model, engine_cfg, args.batch, args.context, args.steps,
                                                            args.warmup, ps, args.regions)
    value = args.batch / (ms / 1e3)
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9

    # decode at batch 1 and 64 at the same context, at batch 1 / 8 / 64 with 1,024 cached tokens (the prompt length
    # that the benchmark's configuration names), and the headline case without captured graphs; each with the
    # fraction of the measured copy bandwidth that its bytes (weights once, the live cache) over its time come to
    points = {}
    if not args.no_points:
        def point(name, cfg_run, b, context, regions):
            pms, _, kvb, _, _ = decode_run(model, cfg_run, b, context, min(args.steps, 32), args.warmup, ps, regions)
            points[name] = round(b / (pms / 1e3), 1)
            points[name + "_hbm_frac"] = round((weight_bytes + kvb) / (pms / 1e3) / 1e9 / pk["hbm_gbs"], 3)
        for b in (1, 64):
            point(f"decode_b{b}", engine_cfg, b, args.context, 3)
        for b in (1, 8, 64):
            point(f"decode_b{b}_ctx1024", engine_cfg, b, 1024, 3)
        eager = EngineConfig(dtype="bfloat16", block_size=ps, max_num_seqs=max(64, args.batch), cuda_graphs=False)
        point(f"decode_b{args.batch}_no_graphs", eager, args.batch, args.context, 3)

    T = 2048
    pre_ms = prefill_run(model, engine_cfg, T, ps)
    flops = prefill_flops(cfg, cfg.num_hidden_layers, T)
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    del model
    torch.cuda.empty_cache()

    e2e = None
    if not args.no_e2e:
        ev, h2d, d2h = e2e_run(cfg, args, ps)
        e2e = {"value": round(ev, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}

    line = {
        "metric": "Gemma-2B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tokens",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids, random cached keys/values)",
        "impl": "ours",
        "config": {"model": "gemma-2b", "layers": cfg.num_hidden_layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": args.context, "page_size": ps, "prefill_tokens": T,
                   "cuda_graphs": not args.no_graphs, "e2e_async_scheduling": True, "parallelism": "single-gpu",
                   "timed_regions": args.regions,
                   "l2": "inputs larger than L2 (weights %.2f GB read every step)" % (weight_bytes / 1e9),
                   "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "ms_per_step_regions": [round(x, 4) for x in per_region],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
