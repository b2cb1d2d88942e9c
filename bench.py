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

    python bench.py --design pesanex [--steps K] [--warmup W] [--batch 8] [--context 2048]

is another workload (the default one and its line are unchanged): Pesanex models at layer sizes of real models
(random weights) beside a Gemma of the same width, feed-forward, attention heads and number of layers: prefill of one
2,048-token prompt and decode at `batch` requests, device-timed; and the new design's kernels one by one at those
shapes (L2 flushed before each timed launch), each with the bytes it must move over the measured copy bandwidth,
beside the like kernel of the Gemma layer.  One JSON line.

    python bench.py --design gudarax [--steps K] [--warmup W] [--batch 8] [--context 2048] [--sizes 2k,4k]

Gudarax beside a Zafilix of equal layer sizes (the closest of the other designs), and its kernels one by one beside their like kernels.

    python bench.py --design taritar [--steps K] [--warmup W] [--batch 8] [--context 2048] [--sizes 2k,4k]

the same for Taritar (several residual streams, attention with a score cap behind a window that keeps first keys, layers
that share keys and values, dense and routed feed-forwards): models of four layers at two real layer sizes beside a Gemma
of equal width, dense feed-forward, heads and layers, and the design's kernels one by one beside their like kernels.
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
        for pages in (group.pages, group.key_pages, group.value_pages):
            if pages is None:
                continue
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


PESANEX_SIZES = {
    # name: width, feed-forward, attention (heads, kv heads, head size), linear attention (heads, key size, value size, rank)
    "2b": dict(width=2048, ff=16384, attn=(8, 1, 256), lin=(8, 128, 256, 64), vocab=32000, layers=4),
    "7b": dict(width=4096, ff=14336, attn=(32, 8, 128), lin=(16, 128, 256, 64), vocab=32000, layers=4),
}


def pesanex_config(size: dict, layout: str) -> dict:
    """'parallel': every layer runs attention with sinks beside gated linear attention, and a feed-forward (a Gemma layer
    plus the second mixer); 'mixed': gated linear attention, the parallel layer, retention, the parallel layer."""
    nq, nkv, hd = size["attn"]
    lh, ld, lv, rank = size["lin"]
    par = {"type": "parallel", "mlp": {"kind": "dense", "ff": size["ff"]},
           "mixer": {"left": {"heads": nq, "kv_heads": nkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                              "rot": {"dims": hd // 2, "base": 1e6}},
                     "right": {"heads": lh, "dim": ld, "vdim": lv, "tau": 16.0, "rank": rank}}}
    gla = {"type": "gla", "mlp": None, "mixer": {"heads": lh, "dim": ld, "vdim": lv, "tau": 16.0, "rank": rank}}
    ret = {"type": "retention", "mlp": None,
           "mixer": {"heads": lh, "dim": ld, "vdim": lv, "rot": {"dims": ld, "base": 1e6},
                     "decay": [1.0 - 2.0 ** (-5 - 6.0 * i / max(1, lh - 1)) for i in range(lh)]}}
    layers = [par] * size["layers"] if layout == "parallel" else ([gla, par, ret, par] * size["layers"])[:size["layers"]]
    return {"architecture": "Pesanex", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-6}, "layers": layers}


def timed_us(fn, flush, repeats: int = 10) -> float:
    """Median device time of fn() in microseconds: three warm-up launches, then `repeats` timed ones, each behind a
    write of a buffer larger than the L2."""
    import torch
    for _ in range(3):
        fn()
    times = []
    for _ in range(repeats):
        flush.add_(1.0)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    return statistics.median(times)


def pesanex_kernel_table(size: dict, pk: dict, T: int, batch: int, context: int) -> dict:
    """The new design's kernels alone at one size's shapes, and the like kernels of the Gemma layer: microseconds, the bytes
    each must move at the measured copy bandwidth (`floor_us`), and how many times the floor it takes (`x_floor`)."""
    import torch
    from wllm_b200.kernels import ops
    dev, bf, f32 = "cuda:0", torch.bfloat16, torch.float32
    flush = torch.zeros(160 << 20, dtype=f32, device=dev)
    W = size["width"]
    nq, nkv, hd = size["attn"]
    H, D, V, rank = size["lin"]
    ps = 64
    out = {}

    def row(name, fn, bytes_moved, flops=0.0):
        us = timed_us(fn, flush)
        floor = max(bytes_moved / (pk["hbm_gbs"] * 1e3), flops / (pk["bf16_tflops"] * 1e6))
        out[name] = {"us": round(us, 1), "floor_us": round(floor, 2), "x_floor": round(us / max(floor, 1e-9), 1)}

    g = torch.Generator(device=dev).manual_seed(1)

    def rnd(*shape, dtype=f32):
        return torch.randn(*shape, generator=g, device=dev, dtype=f32).to(dtype)
    # ---- norms: Gemma's residual norm; the centred norm; the norm of a branch; the mean of two normed branches
    for n, tag in ((T, "prefill"), (batch, "decode")):
        resid, delta, w = rnd(n, W), rnd(n, W, dtype=bf), rnd(W, dtype=bf)
        o = torch.empty(n, W, dtype=bf, device=dev)
        o32 = torch.empty(n, W, device=dev)
        row(f"{tag}/gemma rmsnorm+add", lambda: ops.rmsnorm(resid, delta, w, 1e-6, 1.0, o), n * W * (4 + 4 + 2 + 2))
        row(f"{tag}/layernorm+add", lambda: ops.rmsnorm(resid, o32, w, 1e-6, 0.0, o, center=True), n * W * (4 + 4 + 4 + 2))
        row(f"{tag}/branch layernorm", lambda: ops.branch_norm((delta, 0), w, o32, 1e-6, center=True), n * W * (2 + 4))
        row(f"{tag}/mean of two normed branches", lambda: ops.branch_norm((delta, 0), w, o32, 1e-6, factor=0.5, b=(delta, 0), weight_b=w),
            n * W * (2 + 2 + 4))
    # ---- rotary + cache write, with and without unit-norm heads
    pages = batch * (-(-(context + 1) // ps)) + -(-T // ps) + 1
    kp, vp = rnd(pages, nkv, ps, hd, dtype=bf), rnd(pages, nkv, ps, hd, dtype=bf)
    inv_freq = torch.arange(hd // 4, device=dev, dtype=f32).neg().div(hd // 4).exp()
    for n, tag in ((T, "prefill"), (batch, "decode")):
        qkv = rnd(n, (nq + 2 * nkv) * hd, dtype=bf)
        qo = torch.empty(n, nq * hd, dtype=bf, device=dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        slots = torch.arange(n, dtype=torch.int32, device=dev)
        moved = n * (nq + 2 * nkv) * hd * 2 * 2
        row(f"{tag}/gemma rotary+cache write", lambda: ops.rope_kv_write(qkv, qo, pos, slots, inv_freq, kp, vp, nq, nkv, hd, hd // 2, ps), moved)
        row(f"{tag}/rotary+unit norm+cache write",
            lambda: ops.rope_kv_write(qkv, qo, pos, slots, inv_freq, kp, vp, nq, nkv, hd, hd // 2, ps, unit_norm_eps=1e-6), moved)
    # ---- attention: prefill of T tokens, decode of `batch` requests over `context` keys; with and without sinks
    sinks = rnd(nq)
    one = torch.ones(1, dtype=torch.int32, device=dev)
    table = torch.arange(-(-T // ps), dtype=torch.int32, device=dev).view(1, -1)
    q = rnd(T, nq * hd, dtype=bf)
    ao = torch.empty(T, nq * hd, dtype=bf, device=dev)
    flops = 4.0 * nq * hd * T * T / 2
    for name, extra in (("gemma attention", {}), ("attention with sinks", {"sinks": sinks})):
        row(f"prefill/{name}", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, 0,
                                                                  hd ** -0.5, skip_single=False, **extra), T * nq * hd * 4, flops)
    per = -(-(context + 1) // ps)
    dtable = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
    qd, od = rnd(batch, nq * hd, dtype=bf), torch.empty(batch, nq * hd, dtype=bf, device=dev)
    starts, lens = torch.arange(batch, dtype=torch.int32, device=dev), torch.ones(batch, dtype=torch.int32, device=dev)
    ctxs = lens * context
    split_keys, max_splits = ops.decode_split_plan(batch * nkv, -(-context // 512) * 512, 32 if hd % 64 == 0 else 64)
    scratch = torch.empty(ops.attention_mma_scratch_floats(batch, nq, hd, max_splits), device=dev)
    for name, extra in (("gemma attention", {}), ("attention with sinks", {"sinks": sinks})):
        row(f"decode/{name}", lambda: ops.attention_mma_decode(qd, od, kp, vp, starts, lens, ctxs, dtable, nq, nkv, hd, ps, 0, hd ** -0.5,
                                                                 split_keys, max_splits, scratch, **extra), batch * context * nkv * hd * 2 * 2)
    # ---- the recurrence: its inputs from the fused product, the walk, the heads' norm and gate
    w2, b2, nw = rnd(H * D, rank, dtype=bf), rnd(H * D, dtype=bf), rnd(V, dtype=bf)
    state = torch.zeros(batch + 1, H, D, V, device=dev)
    for n, tag, R in ((T, "prefill", 1), (batch, "decode", batch)):
        fused = rnd(n, 2 * H * D + 2 * H * V + rank, dtype=bf)
        bufs = [torch.empty(n, H * D, device=dev), torch.empty(n, H * D, device=dev), torch.empty(n, H * V, device=dev)]
        decay = torch.empty(n, H * D, device=dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        row(f"{tag}/recurrence inputs (decay from the low-rank map)",
            lambda: ops.linattn_prepare(fused, 0, 0, H * D, 2 * H * D, H, D, V, pos, *bufs, q_scale=D ** -0.5,
                                        low_off=2 * H * D + 2 * H * V, w2=w2, b2=b2, tau=16.0, decay=decay),
            n * ((2 * H * D + H * V + rank) * 2 + (3 * H * D + H * V) * 4))
        o = torch.empty(n, H * V, device=dev)
        if R == 1:
            rs, rl, rslot = one * 0, one * n, one * 0
            seg_len, max_seg = ops.linattn_segment_plan(n, 1, H, V)
        else:
            rs, rl, rslot = starts, lens, starts
            seg_len, max_seg = 0, 1
        seg_state = torch.empty(R * max_seg * H * D * V, device=dev)
        seg_decay = torch.empty(R * max_seg * H * D, device=dev)
        walk_bytes = n * (3 * H * D + 2 * H * V) * 4 + R * 2 * H * D * V * 4
        row(f"{tag}/recurrence" + (f" ({max_seg} segments of {seg_len})" if max_seg > 1 else ""),
            lambda: ops.linattn_scan(bufs[0], bufs[1], bufs[2], decay, None, state, o, rs, rl, rslot, H, D, V, seg_len, max_seg,
                                     seg_state, seg_decay), walk_bytes, 4.0 * n * H * D * V)
        gated = torch.empty(n, H * V, dtype=bf, device=dev)
        row(f"{tag}/head norm and gate", lambda: ops.head_gate_norm(o, fused, 0, 2 * H * D + H * V, nw, 1e-6, gated, H, V),
            n * H * V * (4 + 2 + 2))
    return out


def pesanex_bench(args) -> int:
    import torch
    from wllm_b200.config import EngineConfig, GemmaConfig, PesanexConfig
    from wllm_b200.engine import build_model
    pk = peaks()
    ps, T = args.page_size, 2048
    context = args.context or 2048
    engine_cfg = EngineConfig(dtype="bfloat16", block_size=ps, max_num_seqs=max(64, args.batch), cuda_graphs=not args.no_graphs)
    sizes = {}
    for name in args.sizes.split(","):
        size = PESANEX_SIZES[name]
        nq, nkv, hd = size["attn"]
        models = {
            "gemma": GemmaConfig.from_dict(dict(architectures=["GemmaForCausalLM"], vocab_size=size["vocab"], hidden_size=size["width"],
                                                intermediate_size=size["ff"], num_hidden_layers=size["layers"],
                                                num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
                                                max_position_embeddings=8192)),
            "pesanex_parallel": PesanexConfig.from_dict(pesanex_config(size, "parallel")),
            "pesanex_mixed": PesanexConfig.from_dict(pesanex_config(size, "mixed")),
        }
        res = {}
        for label, cfg in models.items():
            model = build_model(None, engine_cfg.dtype, engine_cfg.device, config=cfg, random_seed=1)
            pre_ms = prefill_run(model, engine_cfg, T, ps)
            ms, launches, _, clocks, _ = decode_run(model, engine_cfg, args.batch, context, min(args.steps, 32), args.warmup, ps, 3)
            res[label] = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "prefill_tok_s": round(T / (pre_ms / 1e3), 1),
                          "prefill_ms": round(pre_ms, 3), "decode_tok_s": round(args.batch / (ms / 1e3), 1),
                          "decode_ms_per_step": round(ms, 4), "decode_launches": launches,
                          "decode_weights_hbm_frac": round(model.weight_bytes() / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3),
                          "clocks": clocks}
            del model
            torch.cuda.empty_cache()
        sizes[name] = {"shape": size, "models": res}
        if not args.no_points:
            sizes[name]["kernels"] = pesanex_kernel_table(size, pk, T, args.batch, context)
    print(json.dumps({"metric": "Pesanex beside Gemma at equal layer sizes: prefill tok/s @ 2048 tokens, decode tok/s",
                      "design": "pesanex", "unit": "tokens/s", "n_gpus": 1, "steps": min(args.steps, 32), "warmup": args.warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids, random cached keys/values, zero states)",
                      "config": {"global_batch": args.batch, "seq_len": context, "prefill_tokens": T, "page_size": ps,
                                 "cuda_graphs": not args.no_graphs, "peaks": pk["source"],
                                 "l2": "kernel table: a 640 MB buffer is written before every timed launch"},
                      "peaks": pk, "sizes": sizes}))
    return 0


TARITAR_SIZES = {
    # width, dense feed-forward, attention (heads, kv heads, head size), window, kept first keys, experts (count, top, ff, groups, kept groups), shared ff
    "2k": dict(width=2048, ff=8192, attn=(16, 4, 128), window=1024, keep=4, experts=(32, 4, 1024, 4, 2), shared=2048, vocab=32000, layers=4),
    "4k": dict(width=4096, ff=14336, attn=(32, 8, 128), window=2048, keep=4, experts=(64, 6, 1408, 8, 4), shared=2816, vocab=32000, layers=4),
}


def taritar_config(size: dict, streams: int = 2) -> dict:
    """Four layers: dense, routed experts, dense on the keys and values of layer 0, routed experts on those of layer 1."""
    nq, nkv, hd = size["attn"]
    E, top, eff, groups, kept = size["experts"]

    def mixer(src=None):
        m = {"heads": nq, "kv_heads": nkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 30.0,
             "rot": {"dims": hd // 2, "base": 1e6}, "mask": {"size": size["window"], "keep_first": size["keep"]}}
        if src is not None:
            m["kv_from"] = src
        return m
    dense = {"kind": "dense", "ff": size["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": E, "top": top, "groups": {"count": groups, "keep": kept}},
           "shared": {"ff": size["shared"], "limit": 7.0}}
    layers = [{"type": "attention", "mixer": mixer(), "mlp": dense}, {"type": "attention", "mixer": mixer(), "mlp": moe},
              {"type": "attention", "mixer": mixer(0), "mlp": dense}, {"type": "attention", "mixer": mixer(1), "mlp": moe}]
    return {"architecture": "Taritar", "vocab": size["vocab"], "width": size["width"], "max_positions": 16384, "streams": streams,
            "logit_softcap": 30.0, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "layers": layers[:size["layers"]]}


def taritar_kernel_table(size: dict, pk: dict, T: int, batch: int, context: int) -> dict:
    """Taritar's kernels alone at one size's shapes beside the like kernels of the Gemma layer: microseconds, the time the
    bytes each must move (or its arithmetic) take at the measured peaks (`floor_us`), and how many times that it takes."""
    import torch
    from wllm_b200.kernels import ops
    dev, bf, f32, i32 = "cuda:0", torch.bfloat16, torch.float32, torch.int32
    flush = torch.zeros(160 << 20, dtype=f32, device=dev)
    W = size["width"]
    nq, nkv, hd = size["attn"]
    E, top, eff, groups, kept = size["experts"]
    window, keep = size["window"], size["keep"]
    ps, S = 64, 2
    out = {}

    def row(name, fn, bytes_moved, flops=0.0):
        us = timed_us(fn, flush)
        floor = max(bytes_moved / (pk["hbm_gbs"] * 1e3), flops / (pk["bf16_tflops"] * 1e6))
        out[name] = {"us": round(us, 1), "floor_us": round(floor, 2), "x_floor": round(us / max(floor, 1e-9), 1)}
    g = torch.Generator(device=dev).manual_seed(1)

    def rnd(*shape, dtype=f32, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev, dtype=f32) * scale).to(dtype)
    # ---- the norm in front of a sublayer: Gemma's (residual += branch, norm) and the two-stream one (update, read, norm)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        resid, delta, w = rnd(n, W), rnd(n, W, dtype=bf), rnd(W, dtype=bf)
        o = torch.empty(n, W, dtype=bf, device=dev)
        streams, gain = rnd(S, n, W), rnd(W)
        mix, w_out, w_in = rnd(S, S), rnd(S), rnd(S)
        row(f"{tag}/gemma rmsnorm+add", lambda: ops.rmsnorm(resid, delta, w, 1e-6, 1.0, o), n * W * (4 + 4 + 2 + 2))
        row(f"{tag}/norm over {S} streams with their update", lambda: ops.hyper_norm(streams, streams, S, (delta, 0), mix, w_out, w_in, gain, 1e-6, o),
            n * W * (8 * S + 2 + 2))
    # ---- rotary + cache write: halves (Gemma) and interleaved pairs
    pages = batch * (-(-(context + 1) // ps)) + -(-T // ps) + 1
    kp, vp = rnd(pages, nkv, ps, hd, dtype=bf), rnd(pages, nkv, ps, hd, dtype=bf)
    inv_freq = torch.arange(hd // 4, device=dev, dtype=f32).neg().div(hd // 4).exp()
    for n, tag in ((T, "prefill"), (batch, "decode")):
        qkv = rnd(n, (nq + 2 * nkv) * hd, dtype=bf)
        qo = torch.empty(n, nq * hd, dtype=bf, device=dev)
        pos = torch.arange(n, dtype=i32, device=dev)
        moved = n * (nq + 2 * nkv) * hd * 2 * 2
        row(f"{tag}/gemma rotary+cache write", lambda: ops.rope_kv_write(qkv, qo, pos, pos, inv_freq, kp, vp, nq, nkv, hd, hd // 2, ps), moved)
        row(f"{tag}/rotary of interleaved pairs+cache write",
            lambda: ops.rope_kv_write(qkv, qo, pos, pos, inv_freq, kp, vp, nq, nkv, hd, hd // 2, ps, pairing="interleaved"), moved)
    # ---- attention: Gemma's over all keys; Taritar's with cap, window and kept keys (what a row sees is what is counted)
    one = torch.ones(1, dtype=i32, device=dev)
    table = torch.arange(-(-T // ps), dtype=i32, device=dev).view(1, -1)
    q = rnd(T, nq * hd, dtype=bf)
    ao = torch.empty(T, nq * hd, dtype=bf, device=dev)
    seen = sum(min(p + 1, window + keep) for p in range(T))
    row("prefill/gemma attention (all keys)", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, 0,
                                                                                 hd ** -0.5, skip_single=False), T * nq * hd * 4, 4.0 * nq * hd * T * T / 2)
    row("prefill/gemma attention (window)", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, window,
                                                                               hd ** -0.5, skip_single=False), T * nq * hd * 4, 4.0 * nq * hd * seen)
    row("prefill/attention with cap, window and kept keys",
        lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, window, hd ** -0.5,
                                          skip_single=False, cap=30.0, keep=keep), T * nq * hd * 4, 4.0 * nq * hd * seen)
    per = -(-(context + 1) // ps)
    dtable = torch.arange(batch * per, dtype=i32, device=dev).view(batch, per)
    qd, od = rnd(batch, nq * hd, dtype=bf), torch.empty(batch, nq * hd, dtype=bf, device=dev)
    starts, lens = torch.arange(batch, dtype=i32, device=dev), torch.ones(batch, dtype=i32, device=dev)
    ctxs = lens * context
    split_keys, max_splits = ops.decode_split_plan(batch * nkv, -(-context // 512) * 512, 32 if hd % 64 == 0 else 64)
    scratch = torch.empty(ops.attention_mma_scratch_floats(batch, nq, hd, max_splits), device=dev)
    read = min(context, window + keep)
    row("decode/gemma attention (all keys)", lambda: ops.attention_mma_decode(qd, od, kp, vp, starts, lens, ctxs, dtable, nq, nkv, hd, ps, 0, hd ** -0.5,
                                                                               split_keys, max_splits, scratch), batch * context * nkv * hd * 2 * 2)
    row("decode/gemma attention (window)", lambda: ops.attention_mma_decode(qd, od, kp, vp, starts, lens, ctxs, dtable, nq, nkv, hd, ps, window, hd ** -0.5,
                                                                             split_keys, max_splits, scratch), batch * read * nkv * hd * 2 * 2)
    row("decode/attention with cap, window and kept keys",
        lambda: ops.attention_mma_decode(qd, od, kp, vp, starts, lens, ctxs, dtable, nq, nkv, hd, ps, window, hd ** -0.5, split_keys,
                                         max_splits, scratch, cap=30.0, keep=keep), batch * read * nkv * hd * 2 * 2)
    # ---- feed-forward: Gemma's dense unit; the clamped unit; the router, the plan and the grouped products of the experts
    for n, tag in ((T, "prefill"), (batch, "decode")):
        x = rnd(n, W, dtype=bf)
        for ff, what in ((size["ff"], "dense"), (top * eff, "dense of the experts' total width")):
            wgu, wd = rnd(2 * ff, W, dtype=bf, scale=0.02), rnd(W, ff, dtype=bf, scale=0.02)
            act = torch.empty(n, ff, dtype=bf, device=dev)
            gu = torch.empty(n, 2 * ff, dtype=bf, device=dev)
            bytes_gu, bytes_d = 2 * ff * W * 2 + n * (W + ff) * 2, ff * W * 2 + n * (W + ff) * 2
            if what == "dense":
                row(f"{tag}/gemma gate|up with tanh-GELU", lambda: ops.gated_linear(x, wgu, "gelu_tanh", act, lambda sh, dt: gu), bytes_gu, 4.0 * n * ff * W)
            row(f"{tag}/{what}: gate|up with the clamped unit", lambda: ops.gated_linear(x, wgu, "capped_swish", act, lambda sh, dt: gu, 7.0, 1.702),
                bytes_gu, 4.0 * n * ff * W)
            parts = {}
            row(f"{tag}/{what}: down", lambda: ops.project(act, wd, lambda name, sh, dt: parts.setdefault((name, sh), torch.empty(sh, dtype=dt, device=dev))),
                bytes_d, 2.0 * n * ff * W)
        wr, wg = rnd(E, W, scale=0.05), rnd(W, scale=0.05)
        chosen, weights, gate = torch.empty(n, top, dtype=i32, device=dev), torch.empty(n, top, device=dev), torch.empty(n, device=dev)
        row(f"{tag}/router (scores, groups, choice, shared gate)", lambda: ops.moe_route(x, wr, wg, chosen, weights, gate, groups, kept),
            n * W * 2 + (E + 1) * W * 4)
        pairs = n * top
        count, offset = torch.empty(E, dtype=i32, device=dev), torch.empty(E + 1, dtype=i32, device=dev)
        order, place = torch.empty(pairs, dtype=i32, device=dev), torch.empty(pairs, dtype=i32, device=dev)
        row(f"{tag}/pairs sorted by expert", lambda: ops.moe_plan(chosen, count, offset, order, place), pairs * 4 * 3)
        w_gu, w_d = rnd(E, 2 * eff, W, dtype=bf, scale=0.02), rnd(E, W, eff, dtype=bf, scale=0.02)
        act, y = torch.empty(pairs, eff, dtype=bf, device=dev), torch.empty(pairs, W, device=dev)
        used = min(E, pairs)           # experts whose weights a step reads at most
        row(f"{tag}/experts: gate|up with the clamped unit (grouped, mma.sync)", lambda: ops.moe_grouped(x, w_gu, act, offset, order, top, True, 7.0, 1.702),
            used * 2 * eff * W * 2 + pairs * (W + eff) * 2, 4.0 * pairs * eff * W)
        row(f"{tag}/experts: down (grouped, mma.sync)", lambda: ops.moe_grouped(act, w_d, y, offset, order, top, False),
            used * eff * W * 2 + pairs * (eff * 2 + W * 4), 2.0 * pairs * eff * W)
        if pairs >= 1024:      # portions of prompts: the experts' products on the tensor-memory kernel, over rows copied into sorted order
            tiles = torch.empty(1 + 3 * ops.moe_row_tiles(pairs, E), dtype=i32, device=dev)
            scratch = torch.empty(ops.MOE_PLAN_SEGMENTS * E, dtype=i32, device=dev)
            row(f"{tag}/pairs sorted by expert, with the table of row tiles", lambda: ops.moe_plan(chosen, count, offset, order, place, tiles, scratch), pairs * 4 * 3)
            xs = torch.empty(pairs, W, dtype=bf, device=dev)
            row(f"{tag}/experts: the tokens' rows into sorted order", lambda: ops.moe_gather(x, order, top, xs), pairs * W * 4)
            row(f"{tag}/experts: gate|up with the clamped unit (grouped, tensor memory)", lambda: ops.gemm_bf16_tc_grouped(xs, w_gu, act, tiles, True, 7.0, 1.702),
                used * 2 * eff * W * 2 + pairs * (W + eff) * 2, 4.0 * pairs * eff * W)
            row(f"{tag}/experts: down (grouped, tensor memory)", lambda: ops.gemm_bf16_tc_grouped(act, w_d, y, tiles, False),
                used * eff * W * 2 + pairs * (eff * 2 + W * 4), 2.0 * pairs * eff * W)
        shared, o32 = rnd(n, W, dtype=bf), torch.empty(n, W, device=dev)
        row(f"{tag}/experts' outputs weighted and summed, shared unit gated and added", lambda: ops.moe_combine(y, place, weights, (shared, 0), gate, o32),
            pairs * W * 4 + n * W * (2 + 4))
    # ---- embedding with a position row; capped logits
    emb, pos_table = rnd(size["vocab"], W, dtype=bf), rnd(4096, W, dtype=bf)
    ids = torch.randint(0, size["vocab"], (T,), generator=g, device=dev, dtype=i32)
    at = torch.arange(T, dtype=i32, device=dev)
    r32 = torch.empty(T, W, device=dev)
    row("prefill/gemma embedding", lambda: ops.embed_gather(ids, emb, 1.0, r32), T * W * (2 + 4))
    row("prefill/embedding with position rows", lambda: ops.embed_gather(ids, emb, 1.0, r32, pos_table, at), T * W * (2 + 2 + 4))
    logits = rnd(batch, size["vocab"])
    row("decode/tanh cap of the logits", lambda: ops.tanh_cap(logits, 30.0), batch * size["vocab"] * 8)
    return out


def taritar_bench(args) -> int:
    import torch
    from wllm_b200.config import EngineConfig, GemmaConfig, TaritarConfig
    from wllm_b200.engine import build_model
    pk = peaks()
    ps, T = args.page_size, 2048
    context = args.context or 2048
    engine_cfg = EngineConfig(dtype="bfloat16", block_size=ps, max_num_seqs=max(64, args.batch), cuda_graphs=not args.no_graphs)
    sizes = {}
    for name in (args.sizes if args.sizes != "2b,7b" else "2k,4k").split(","):
        size = TARITAR_SIZES[name]
        nq, nkv, hd = size["attn"]
        models = {
            "gemma": GemmaConfig.from_dict(dict(architectures=["GemmaForCausalLM"], vocab_size=size["vocab"], hidden_size=size["width"],
                                                intermediate_size=size["ff"], num_hidden_layers=size["layers"],
                                                num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
                                                max_position_embeddings=16384)),
            "taritar": TaritarConfig.from_dict(taritar_config(size)),
        }
        res = {}
        for label, cfg in models.items():
            model = build_model(None, engine_cfg.dtype, engine_cfg.device, config=cfg, random_seed=1)
            pre_ms = prefill_run(model, engine_cfg, T, ps)
            ms, launches, _, clocks, _ = decode_run(model, engine_cfg, args.batch, context, min(args.steps, 32), args.warmup, ps, 3)
            res[label] = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "prefill_tok_s": round(T / (pre_ms / 1e3), 1),
                          "prefill_ms": round(pre_ms, 3), "decode_tok_s": round(args.batch / (ms / 1e3), 1),
                          "decode_ms_per_step": round(ms, 4), "decode_launches": launches,
                          "decode_weights_hbm_frac": round(model.weight_bytes() / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3), "clocks": clocks}
            del model
            torch.cuda.empty_cache()
        sizes[name] = {"shape": size, "models": res}
        if not args.no_points:
            sizes[name]["kernels"] = taritar_kernel_table(size, pk, T, args.batch, context)
    print(json.dumps({"metric": "Taritar beside Gemma at equal layer sizes: prefill tok/s @ 2048 tokens, decode tok/s",
                      "design": "taritar", "unit": "tokens/s", "n_gpus": 1, "steps": min(args.steps, 32), "warmup": args.warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids, random cached keys/values)",
                      "config": {"global_batch": args.batch, "seq_len": context, "prefill_tokens": T, "page_size": ps,
                                 "cuda_graphs": not args.no_graphs, "peaks": pk["source"],
                                 "l2": "kernel table: a 640 MB buffer is written before every timed launch"},
                      "peaks": pk, "sizes": sizes}))
    return 0


ZAFILIX_SIZES = {
    # width, feed-forward, attention (heads, kv heads, head size) in blocks, latent attention (heads, plain, turning, value, latent row) in a window
    "2k": dict(width=2048, ff=8192, attn=(16, 4, 128), block=1024, latent=(16, 128, 64, 128, 512), window=1024, vocab=32000),
    "4k": dict(width=4096, ff=14336, attn=(32, 8, 128), block=1024, latent=(32, 128, 64, 128, 512), window=1024, vocab=32000),
}


def zafilix_config(size: dict) -> dict:
    """Four layer runs: attention in blocks, latent attention in a window, and each once more on the same tensors."""
    nq, nkv, hd = size["attn"]
    H, dim, rot, vd, rank = size["latent"]
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": size["ff"]},
           "mixer": {"heads": nq, "kv_heads": nkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": size["block"]},
                     "rot": {"dims": hd, "base": 1000000.0, "scaling": {"factor": 4.0}}}}
    lat = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": size["ff"]},
           "mixer": {"heads": H, "dim": dim, "rot_dim": rot, "vdim": vd, "kv_rank": rank, "scale": (dim + rot) ** -0.5,
                     "mask": {"size": size["window"]}, "rot": {"dims": rot, "base": 10000.0}}}
    return {"architecture": "Zafilix", "vocab": size["vocab"], "width": size["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "logit_scale": 0.5, "logit_softcap": 30.0, "layers": [att, lat, dict(att, weights_of=0), dict(lat, weights_of=1)]}


def zafilix_kernel_table(size: dict, pk: dict, T: int, batch: int, context: int) -> dict:
    """Zafilix's kernels alone at one size's shapes beside the like kernels of the Gemma layer: microseconds, the time the
    bytes each must move (or its arithmetic) take at the measured peaks (`floor_us`), and how many times that it takes."""
    import torch
    from wllm_b200.kernels import ops
    dev, bf, f32, i32 = "cuda:0", torch.bfloat16, torch.float32, torch.int32
    flush = torch.zeros(160 << 20, dtype=f32, device=dev)
    W, ff = size["width"], size["ff"]
    nq, nkv, hd = size["attn"]
    H, dim, rot, vd, rank = size["latent"]
    block, window = size["block"], size["window"]
    row_len = rank + rot
    ps = 64
    out = {}

    def row(name, fn, bytes_moved, flops=0.0):
        us = timed_us(fn, flush)
        floor = max(bytes_moved / (pk["hbm_gbs"] * 1e3), flops / (pk["bf16_tflops"] * 1e6))
        out[name] = {"us": round(us, 1), "floor_us": round(floor, 2), "x_floor": round(us / max(floor, 1e-9), 1)}
    g = torch.Generator(device=dev).manual_seed(1)

    def rnd(*shape, dtype=f32, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev, dtype=f32) * scale).to(dtype)

    def held(store):
        return lambda name, sh, dt: store.setdefault((name, sh), torch.empty(sh, dtype=dt, device=dev))
    # ---- the norm: Gemma's in front of a sublayer; Zafilix's behind one, with the add and the rounded copy the next sublayer reads
    for n, tag in ((T, "prefill"), (batch, "decode")):
        resid, delta, w = rnd(n, W), rnd(n, W, dtype=bf), rnd(W, dtype=bf)
        o = torch.empty(n, W, dtype=bf, device=dev)
        row(f"{tag}/gemma rmsnorm+add", lambda: ops.rmsnorm(resid, delta, w, 1e-6, 1.0, o), n * W * (4 + 4 + 2 + 2))
        row(f"{tag}/norm behind the sublayer+add+rounded copy", lambda: ops.sandwich_norm(resid, (delta, 0), o, w, False, 1e-6, None, 0.0, False, 0.0,
                                                                                         post_offset=1.0), n * W * (4 + 4 + 2 + 2))
    # ---- rotary + cache write: Gemma's; rows normed as wholes first; the latent row and the queries' parts
    pages = batch * (-(-(context + 1) // ps)) + -(-T // ps) + 1
    kp, vp = rnd(pages, nkv, ps, hd, dtype=bf), rnd(pages, nkv, ps, hd, dtype=bf)
    lp = rnd(pages, 1, ps, row_len, dtype=bf)
    inv_freq = torch.arange(hd // 2, device=dev, dtype=f32).neg().div(hd // 2).exp()
    inv_rot = torch.arange(rot // 2, device=dev, dtype=f32).neg().div(rot // 2).exp()
    q_gain, k_gain, l_gain = rnd(nq * hd, dtype=bf), rnd(nkv * hd, dtype=bf), rnd(rank, dtype=bf)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        qkv = rnd(n, (nq + 2 * nkv) * hd, dtype=bf)
        qo = torch.empty(n, nq * hd, dtype=bf, device=dev)
        pos = torch.arange(n, dtype=i32, device=dev)
        moved = n * (nq + 2 * nkv) * hd * 2 * 2
        row(f"{tag}/gemma rotary+cache write", lambda: ops.rope_kv_write(qkv, qo, pos, pos, inv_freq, kp, vp, nq, nkv, hd, hd, ps), moved)
        row(f"{tag}/row norms+rotary of neighbours+cache write",
            lambda: ops.rope_row_norm_kv_write(qkv, qo, pos, pos, inv_freq, kp, vp, nq, nkv, hd, hd, ps, q_gain, k_gain, 1e-6, nq * hd, nkv * hd,
                                               pairing="interleaved"), moved)
        fused = rnd(n, H * (dim + rot) + row_len, dtype=bf)
        q_plain, q_mapped = torch.empty(n, H * dim, dtype=bf, device=dev), torch.empty(n, H * row_len, dtype=bf, device=dev)
        row(f"{tag}/latent row (norm, turn, cache write) and the queries' parts",
            # a prompt's product leaves one bfloat16 tensor: the queries' plain parts are read where they are, not copied
            lambda: ops.latent_prepare(fused, 0, pos, pos, inv_rot, l_gain, 1e-6, lp, ps, None if tag == "prefill" else q_plain, q_mapped, H, dim,
                                       rot, rot, rank, row_len),
            n * (H * (dim + rot) + row_len) * 2 * 2)
        w_uk, w_uv = rnd(H, rank, dim, dtype=bf, scale=0.05), rnd(H, vd, rank, dtype=bf, scale=0.05)
        mixed, heads_out = rnd(n, H, rank, dtype=bf), torch.empty(n, H, vd, dtype=bf, device=dev)
        row(f"{tag}/latent: the keys' map on the queries", lambda: ops.head_linear(q_plain.view(n, H, dim), w_uk, q_mapped.view(n, H, row_len)[:, :, :rank]),
            H * rank * dim * 2 + n * H * (dim + rank) * 2, 2.0 * n * H * dim * rank)
        row(f"{tag}/latent: the values' map on the outputs", lambda: ops.head_linear(mixed, w_uv, heads_out),
            H * rank * vd * 2 + n * H * (vd + rank) * 2, 2.0 * n * H * vd * rank)
        gate_in = rnd(n, nq * hd * 2, dtype=bf)
        attn = rnd(n, nq * hd, dtype=bf)
        row(f"{tag}/sigmoid gate on the heads' outputs", lambda: ops.sigmoid_gate(attn, gate_in, 0, nq * hd), n * nq * hd * 2 * 3)
    # ---- attention over a prompt of T tokens: Gemma's over all keys and in a window; in blocks; over latent rows in a window
    one = torch.ones(1, dtype=i32, device=dev)
    table = torch.arange(-(-T // ps), dtype=i32, device=dev).view(1, -1)
    q, ao = rnd(T, nq * hd, dtype=bf), torch.empty(T, nq * hd, dtype=bf, device=dev)
    in_window = sum(min(p + 1, window) for p in range(T))
    in_block = sum(p % block + 1 for p in range(T))
    row("prefill/gemma attention (all keys)", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, 0,
                                                                                 hd ** -0.5, skip_single=False), T * nq * hd * 4, 4.0 * nq * hd * T * T / 2)
    row("prefill/gemma attention (window)", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, window,
                                                                               hd ** -0.5, skip_single=False), T * nq * hd * 4, 4.0 * nq * hd * in_window)
    row("prefill/attention in blocks", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, -block,
                                                                          hd ** -0.5, skip_single=False), T * nq * hd * 4, 4.0 * nq * hd * in_block)
    ql, mixed_l = rnd(T, H * row_len, dtype=bf, scale=0.2), torch.empty(T, H * rank, dtype=bf, device=dev)
    pos_t, req_t = torch.arange(T, dtype=i32, device=dev), torch.zeros(T, dtype=i32, device=dev)
    latent_flops = 2.0 * H * (row_len + rank) * in_window
    if ops.latent_mma_ok(H, rank, row_len, ps):
        row("prefill/attention over latent rows (window, tensor cores)",
            lambda: ops.latent_attention_mma(ql, mixed_l, lp, one * 0, one * T, one * T, table, T, H, rank, row_len, ps, window, (dim + rot) ** -0.5),
            T * H * (row_len + rank) * 2, latent_flops)
    if T * H <= 8192:       # the general kernel, a warp a row: minutes of its time would say nothing new
        row("prefill/attention over latent rows (window, general kernel)",
            lambda: ops.paged_attention_simt(ql, mixed_l, lp, lp, req_t, pos_t, table, H, 1, row_len, ps, window, (dim + rot) ** -0.5, vd=rank,
                                             values_in_keys=True), T * H * (row_len + rank) * 2, latent_flops)
    # ---- one decoded token of `batch` requests over `context` cached tokens
    per = -(-(context + 1) // ps)
    dtable = torch.arange(batch * per, dtype=i32, device=dev).view(batch, per)
    qd, od = rnd(batch, nq * hd, dtype=bf), torch.empty(batch, nq * hd, dtype=bf, device=dev)
    starts, lens = torch.arange(batch, dtype=i32, device=dev), torch.ones(batch, dtype=i32, device=dev)
    ctxs = lens * context
    split_keys, max_splits = ops.decode_split_plan(batch * nkv, -(-context // 512) * 512, 32 if hd % 64 == 0 else 64)
    scratch = torch.empty(ops.attention_mma_scratch_floats(batch, nq, hd, max_splits), device=dev)
    read_w, read_b = min(context, window), (context - 1) % block + 1
    for what, win, read in (("gemma attention (all keys)", 0, context), ("gemma attention (window)", window, read_w), ("attention in blocks", -block, read_b)):
        row(f"decode/{what}", lambda: ops.attention_mma_decode(qd, od, kp, vp, starts, lens, ctxs, dtable, nq, nkv, hd, ps, win, hd ** -0.5,
                                                               split_keys, max_splits, scratch), batch * read * nkv * hd * 2 * 2)
    qdl, odl = rnd(batch, H * row_len, dtype=bf, scale=0.2), torch.empty(batch, H * rank, dtype=bf, device=dev)
    dpos = (ctxs - 1).to(i32)
    chunks = ops.simt_chunks(context, window)
    lscratch = torch.empty(batch * H * chunks * (rank + 2), device=dev)
    latent_bytes = batch * read_w * row_len * 2 + batch * H * (row_len + rank) * 2
    row("decode/attention over latent rows (window, general kernel, keys in chunks)",
        lambda: ops.paged_attention_simt(qdl, odl, lp, lp, starts, dpos, dtable, H, 1, row_len, ps, window, (dim + rot) ** -0.5, lscratch, chunks,
                                         vd=rank, values_in_keys=True), latent_bytes, 2.0 * batch * H * (row_len + rank) * read_w)
    if ops.latent_mma_ok(H, rank, row_len, ps):
        split_tiles, lat_splits = ops.latent_split_plan(batch, H, -(-context // ps) * ps, window)
        mscratch = torch.empty(ops.latent_mma_scratch_floats(batch, H, rank, lat_splits), device=dev)
        row("decode/attention over latent rows (window, tensor cores, keys in splits)",
            lambda: ops.latent_attention_mma(qdl, odl, lp, starts, lens, ctxs, dtable, 1, H, rank, row_len, ps, window, (dim + rot) ** -0.5,
                                             split_tiles=split_tiles, max_splits=lat_splits, scratch=mscratch),
            latent_bytes, 2.0 * batch * H * (row_len + rank) * read_w)
    # ---- feed-forward: Gemma's gated unit; up with the squared ReLU; down
    for n, tag in ((T, "prefill"), (batch, "decode")):
        x = rnd(n, W, dtype=bf)
        wgu, wu, wd = rnd(2 * ff, W, dtype=bf, scale=0.02), rnd(ff, W, dtype=bf, scale=0.02), rnd(W, ff, dtype=bf, scale=0.02)
        act, gu = torch.empty(n, ff, dtype=bf, device=dev), torch.empty(n, 2 * ff, dtype=bf, device=dev)
        row(f"{tag}/gemma gate|up with tanh-GELU", lambda: ops.gated_linear(x, wgu, "gelu_tanh", act, lambda sh, dt: gu),
            2 * ff * W * 2 + n * (W + ff) * 2, 4.0 * n * ff * W)
        row(f"{tag}/up with the squared ReLU", lambda: ops.unit_linear(x, wu, "relu_squared", act, lambda sh, dt: gu[:, :ff]),
            ff * W * 2 + n * (W + ff) * 2, 2.0 * n * ff * W)
        parts = {}
        row(f"{tag}/down", lambda: ops.project(act, wd, held(parts)), ff * W * 2 + n * (W + ff) * 2, 2.0 * n * ff * W)
    return out


def zafilix_bench(args) -> int:
    import torch
    from wllm_b200.config import EngineConfig, GemmaConfig, ZafilixConfig
    from wllm_b200.engine import build_model
    pk = peaks()
    ps, T = args.page_size, 2048
    context = args.context or 2048
    engine_cfg = EngineConfig(dtype="bfloat16", block_size=ps, max_num_seqs=max(64, args.batch), cuda_graphs=not args.no_graphs)
    sizes = {}
    for name in (args.sizes if args.sizes != "2b,7b" else "2k,4k").split(","):
        size = ZAFILIX_SIZES[name]
        nq, nkv, hd = size["attn"]
        raw = zafilix_config(size)
        models = {
            "gemma": GemmaConfig.from_dict(dict(architectures=["GemmaForCausalLM"], vocab_size=size["vocab"], hidden_size=size["width"],
                                                intermediate_size=size["ff"], num_hidden_layers=len(raw["layers"]),
                                                num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
                                                max_position_embeddings=16384)),
            "zafilix": ZafilixConfig.from_dict(raw),
        }
        res = {}
        for label, cfg in models.items():
            model = build_model(None, engine_cfg.dtype, engine_cfg.device, config=cfg, random_seed=1)
            pre_ms = prefill_run(model, engine_cfg, T, ps)
            ms, launches, _, clocks, _ = decode_run(model, engine_cfg, args.batch, context, min(args.steps, 32), args.warmup, ps, 3)
            res[label] = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "prefill_tok_s": round(T / (pre_ms / 1e3), 1),
                          "prefill_ms": round(pre_ms, 3), "decode_tok_s": round(args.batch / (ms / 1e3), 1),
                          "decode_ms_per_step": round(ms, 4), "decode_launches": launches,
                          "decode_weights_hbm_frac": round(model.weight_bytes() / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3), "clocks": clocks}
            del model
            torch.cuda.empty_cache()
        sizes[name] = {"shape": size, "models": res}
        if not args.no_points:
            sizes[name]["kernels"] = zafilix_kernel_table(size, pk, T, args.batch, context)
    print(json.dumps({"metric": "Zafilix beside Gemma at equal layer sizes: prefill tok/s @ 2048 tokens, decode tok/s",
                      "design": "zafilix", "unit": "tokens/s", "n_gpus": 1, "steps": min(args.steps, 32), "warmup": args.warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids, random cached keys/values)",
                      "config": {"global_batch": args.batch, "seq_len": context, "prefill_tokens": T, "page_size": ps,
                                 "cuda_graphs": not args.no_graphs, "peaks": pk["source"],
                                 "l2": "kernel table: a 640 MB buffer is written before every timed launch"},
                      "peaks": pk, "sizes": sizes}))
    return 0


GUDARAX_SIZES = {
    # width, dense feed-forward, attention (heads, kv heads, head size) in a window, latent attention (heads, head size, value size, latent
    # row, the queries' latent row), delta (value heads, query/key heads, key size, value size, taps), experts (number, chosen, width)
    "2k": dict(width=2048, ff=8192, attn=(16, 4, 128), window=1024, latent=(16, 128, 128, 512, 768), delta=(16, 4, 128, 128, 4),
               experts=(16, 2, 2048), side=256, vocab=32000),
    "4k": dict(width=4096, ff=14336, attn=(32, 8, 128), window=1024, latent=(32, 128, 128, 512, 1536), delta=(32, 8, 128, 128, 4),
               experts=(16, 2, 4096), side=256, vocab=32000),
}


def gudarax_config(size: dict) -> dict:
    """Four layers: attention in a window (the first of the two that blend values), latent attention, the delta rule, attention again;
    dense feed-forwards behind the first two, routed experts behind the others; a token input in every layer."""
    nq, nkv, hd = size["attn"]
    H, dim, vd, rank, q_rank = size["latent"]
    dh, dg, dd, dv, taps = size["delta"]
    E, top, eff = size["experts"]
    dense = {"kind": "dense", "ff": size["ff"]}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}}
    att = {"type": "attention", "mixer": {"heads": nq, "kv_heads": nkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                                          "mask": {"size": size["window"]}, "v_mix": True}}
    lat = {"type": "latent_attention", "mixer": {"heads": H, "dim": dim, "vdim": vd, "kv_rank": rank, "q_rank": q_rank, "scale": dim ** -0.5}}
    dlt = {"type": "delta", "mixer": {"heads": dh, "kv_heads": dg, "dim": dd, "vdim": dv, "conv": taps}}
    return {"architecture": "Gudarax", "vocab": size["vocab"], "width": size["width"], "max_positions": 16384, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "token_side": {"dim": size["side"]},
            "layers": [dict(att, mlp=dense), dict(lat, mlp=dense), dict(dlt, mlp=moe), dict(att, mlp=moe)]}


def gudarax_kernel_table(size: dict, pk: dict, T: int, batch: int, context: int) -> dict:
    """Gudarax's kernels alone at one size's shapes beside their like kernels of the framework's other designs: microseconds, the
    time the bytes each must move (or its arithmetic) take at the measured peaks (`floor_us`), and how many times that it takes."""
    import torch
    from wllm_b200.kernels import ops
    dev, bf, f32, i32 = "cuda:0", torch.bfloat16, torch.float32, torch.int32
    flush = torch.zeros(160 << 20, dtype=f32, device=dev)
    W = size["width"]
    nq, nkv, hd = size["attn"]
    H, dim, vd, rank, q_rank = size["latent"]
    dh, dg, dd, dv, taps = size["delta"]
    E, top, eff = size["experts"]
    window, side = size["window"], size["side"]
    ps = 64
    out = {}

    def row(name, fn, bytes_moved, flops=0.0):
        us = timed_us(fn, flush)
        floor = max(bytes_moved / (pk["hbm_gbs"] * 1e3), flops / (pk["bf16_tflops"] * 1e6))
        out[name] = {"us": round(us, 1), "floor_us": round(floor, 2), "x_floor": round(us / max(floor, 1e-9), 1)}
    g = torch.Generator(device=dev).manual_seed(1)

    def rnd(*shape, dtype=f32, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev, dtype=f32) * scale).to(dtype)
    one = torch.ones(1, dtype=i32, device=dev)
    starts, lens = torch.arange(batch, dtype=i32, device=dev), torch.ones(batch, dtype=i32, device=dev)
    # ---- q | k | v into the pages: rows normed as wholes (Zafilix's), and with biases and blended values in front (this design's)
    pages = batch * (-(-(context + 1) // ps)) + -(-T // ps) + 1
    kp, vp = rnd(pages, nkv, ps, hd, dtype=bf), rnd(pages, nkv, ps, hd, dtype=bf)
    none = torch.empty(0, dtype=f32, device=dev)
    q_gain, k_gain = rnd(nq * hd, dtype=bf), rnd(nkv * hd, dtype=bf)
    bias, blend = rnd((nq + 2 * nkv) * hd), torch.full((1,), 0.4, device=dev)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        qkv = rnd(n, (nq + 2 * nkv) * hd, dtype=bf)
        qo = torch.empty(n, nq * hd, dtype=bf, device=dev)
        first = torch.empty(n, nkv * hd, device=dev)
        pos = torch.arange(n, dtype=i32, device=dev)
        moved = n * (nq + 2 * nkv) * hd * 2 * 2
        row(f"{tag}/row norms+cache write (no turn)",
            lambda: ops.rope_row_norm_kv_write(qkv, qo, pos, pos, none, kp, vp, nq, nkv, hd, 0, ps, q_gain, k_gain, 1e-6, nq * hd, nkv * hd), moved)
        row(f"{tag}/biases+row norms+cache write, values left for later layers",
            lambda: ops.rope_row_norm_kv_write(qkv, qo, pos, pos, none, kp, vp, nq, nkv, hd, 0, ps, q_gain, k_gain, 1e-6, nq * hd, nkv * hd,
                                               bias=bias, v_first=first, mix="first"), moved + n * nkv * hd * 4)
        row(f"{tag}/biases+row norms+cache write, values blended",
            lambda: ops.rope_row_norm_kv_write(qkv, qo, pos, pos, none, kp, vp, nq, nkv, hd, 0, ps, q_gain, k_gain, 1e-6, nq * hd, nkv * hd,
                                               bias=bias, v_first=first, blend=blend, mix="later"), moved + n * nkv * hd * 4)
    # ---- attention in a window over a prompt of T tokens and for one decoded token: plain, and with the bias by distance
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq)], dtype=f32, device=dev)
    table = torch.arange(-(-T // ps), dtype=i32, device=dev).view(1, -1)
    q, ao = rnd(T, nq * hd, dtype=bf), torch.empty(T, nq * hd, dtype=bf, device=dev)
    in_window = sum(min(p + 1, window) for p in range(T))
    for what, extra in (("attention in a window", {}), ("attention in a window with a bias by distance", {"slopes": slopes})):
        row(f"prefill/{what}", lambda: ops.attention_mma_prefill(q, ao, kp, vp, one * 0, one * T, one * T, table, T, nq, nkv, hd, ps, window,
                                                                 hd ** -0.5, skip_single=False, **extra), T * nq * hd * 4, 4.0 * nq * hd * in_window)
    per = -(-(context + 1) // ps)
    dtable = torch.arange(batch * per, dtype=i32, device=dev).view(batch, per)
    qd, od = rnd(batch, nq * hd, dtype=bf), torch.empty(batch, nq * hd, dtype=bf, device=dev)
    ctxs = lens * context
    split_keys, max_splits = ops.decode_split_plan(batch * nkv, -(-context // 512) * 512, 32 if hd % 64 == 0 else 64)
    scratch = torch.empty(ops.attention_mma_scratch_floats(batch, nq, hd, max_splits), device=dev)
    read_w = min(context, window)
    for what, extra in (("attention in a window", {}), ("attention in a window with a bias by distance", {"slopes": slopes})):
        row(f"decode/{what}", lambda: ops.attention_mma_decode(qd, od, kp, vp, starts, lens, ctxs, dtable, nq, nkv, hd, ps, window, hd ** -0.5,
                                                               split_keys, max_splits, scratch, **extra), batch * read_w * nkv * hd * 2 * 2)
    # ---- latent attention: the cache row and the queries' latent row; the queries' products; attention over every earlier row
    lp = rnd(pages, 1, ps, rank, dtype=bf)
    l_gain, cq_gain = rnd(rank, dtype=bf), rnd(q_rank, dtype=bf)
    w_uq = rnd(H * dim, q_rank, dtype=bf, scale=0.03)
    w_uk, w_uv = rnd(H, rank, dim, dtype=bf, scale=0.05), rnd(H, vd, rank, dtype=bf, scale=0.05)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        pos = torch.arange(n, dtype=i32, device=dev)
        plain = rnd(n, H * dim + rank, dtype=bf)
        q_plain, q_mapped = torch.empty(n, H * dim, dtype=bf, device=dev), torch.empty(n, H * rank, dtype=bf, device=dev)
        row(f"{tag}/latent row (norm, cache write), queries projected directly (Zafilix's form without a turn)",
            lambda: ops.latent_prepare(plain, 0, pos, pos, none, l_gain, 1e-6, lp, ps, None if tag == "prefill" else q_plain, q_mapped, H, dim, 0, 0,
                                       rank, rank), n * (H * dim + rank) * 2 * 2)
        fused = rnd(n, q_rank + rank + H * vd, dtype=bf)
        cq = torch.empty(n, q_rank, dtype=bf, device=dev)
        row(f"{tag}/latent row and the queries' latent row (two norms, cache write)",
            lambda: ops.latent_prepare(fused, 0, pos, pos, none, l_gain, 1e-6, lp, ps, None, q_mapped, H, dim, 0, 0, rank, rank, q_rank=q_rank,
                                       q_gain=cq_gain, cq_out=cq), n * (q_rank + rank) * 2 * 2)
        qu = torch.empty(n, H * dim, dtype=bf, device=dev)
        row(f"{tag}/latent: queries from their latent row", lambda: ops.linear(cq, w_uq, qu), H * dim * q_rank * 2 + n * (q_rank + H * dim) * 2,
            2.0 * n * H * dim * q_rank)
        row(f"{tag}/latent: the keys' map on the queries", lambda: ops.head_linear(qu.view(n, H, dim), w_uk, q_mapped.view(n, H, rank)),
            H * rank * dim * 2 + n * H * (dim + rank) * 2, 2.0 * n * H * dim * rank)
        heads_out = rnd(n, H * vd, dtype=bf)
        row(f"{tag}/sigmoid gate on the heads' outputs", lambda: ops.sigmoid_gate(heads_out, fused, 0, q_rank + rank), n * H * vd * 2 * 3)
    ql, mixed_l = rnd(T, H * rank, dtype=bf, scale=0.2), torch.empty(T, H * rank, dtype=bf, device=dev)
    seen = T * (T + 1) // 2
    if ops.latent_mma_ok(H, rank, rank, ps):
        row("prefill/attention over latent rows (every earlier row, tensor cores)",
            lambda: ops.latent_attention_mma(ql, mixed_l, lp, one * 0, one * T, one * T, table, T, H, rank, rank, ps, 0, dim ** -0.5),
            T * H * 2 * rank * 2, 4.0 * H * rank * seen)
        qdl, odl = rnd(batch, H * rank, dtype=bf, scale=0.2), torch.empty(batch, H * rank, dtype=bf, device=dev)
        split_tiles, lat_splits = ops.latent_split_plan(batch, H, -(-context // ps) * ps, 0)
        mscratch = torch.empty(ops.latent_mma_scratch_floats(batch, H, rank, lat_splits), device=dev)
        row("decode/attention over latent rows (every earlier row, tensor cores, keys in splits)",
            lambda: ops.latent_attention_mma(qdl, odl, lp, starts, lens, ctxs, dtable, 1, H, rank, rank, ps, 0, dim ** -0.5, split_tiles=split_tiles,
                                             max_splits=lat_splits, scratch=mscratch),
            batch * context * rank * 2 + batch * H * 2 * rank * 2, 4.0 * batch * H * rank * context)
    # ---- recurrences: Pesanex's decayed state with a fixed decay per head, and the gated delta rule, at the same head sizes
    GD, HV = dg * dd, dh * dv
    Wd = 2 * GD + 2 * HV + 2 * dh
    off = {"q": 0, "k": GD, "v": 2 * GD, "g": 2 * GD + HV, "b": 2 * GD + 2 * HV, "a": 2 * GD + 2 * HV + dh}
    conv = [rnd(c, taps, dtype=bf) for c in (GD, GD, HV)]
    a_log, dt_bias, nw = rnd(dh, dtype=bf), rnd(dh, dtype=bf), rnd(dv, dtype=bf)
    head_decay = torch.full((dh,), 0.97, device=dev)
    for n, tag, R in ((T, "prefill", 1), (batch, "decode", batch)):
        rs, rl, rslot = (one * 0, one * n, one * 0) if R == 1 else (starts, lens, starts)
        token_req = torch.zeros(n, dtype=i32, device=dev) if R == 1 else starts
        pos = torch.arange(n, dtype=i32, device=dev)
        # Pesanex's recurrence with as many query/key heads as value heads (it has no grouped form)
        wide = rnd(n, 2 * dh * dd + 2 * HV, dtype=bf)
        bufs = [torch.empty(n, dh * dd, device=dev), torch.empty(n, dh * dd, device=dev), torch.empty(n, HV, device=dev)]
        row(f"{tag}/decayed state: inputs (scales, no turn)",
            lambda: ops.linattn_prepare(wide, 0, 0, dh * dd, 2 * dh * dd, dh, dd, dv, pos, *bufs, q_scale=dd ** -0.5),
            n * ((2 * dh * dd + HV) * 2 + (2 * dh * dd + HV) * 4))
        state = torch.zeros(batch + 1, dh, dd, dv, device=dev)
        o = torch.empty(n, HV, device=dev)
        seg_len, max_seg = ops.linattn_segment_plan(n, 1, dh, dv) if R == 1 else (0, 1)
        seg_state, seg_decay = torch.empty(R * max_seg * dh * dd * dv, device=dev), torch.empty(R * max_seg * dh * dd, device=dev)
        row(f"{tag}/decayed state: recurrence" + (f" ({max_seg} segments of {seg_len})" if max_seg > 1 else ""),
            lambda: ops.linattn_scan(bufs[0], bufs[1], bufs[2], None, head_decay, state, o, rs, rl, rslot, dh, dd, dv, seg_len, max_seg, seg_state,
                                     seg_decay), n * (2 * dh * dd + 2 * HV) * 4 + R * 2 * dh * dd * dv * 4, 4.0 * n * dh * dd * dv)
        fused = rnd(n, Wd, dtype=bf)
        dq, dk, dvv = torch.empty(n, GD, device=dev), torch.empty(n, GD, device=dev), torch.empty(n, HV, device=dev)
        beta, decay = torch.empty(n, dh, device=dev), torch.empty(n, dh, device=dev)
        conv_state = torch.zeros(batch + 1, taps - 1, 2 * GD + HV, device=dev)
        row(f"{tag}/delta rule: inputs (convolutions, SiLU, unit norms, step sizes, decays)",
            lambda: ops.delta_prepare(fused, 0, off, dh, dg, dd, dv, taps, *conv, a_log, dt_bias, token_req, rs, rslot, conv_state, 1e-6, dd ** -0.5,
                                      dq, dk, dvv, beta, decay), n * ((2 * GD + HV + 2 * dh) * 2 * min(taps, 2) + (2 * GD + HV + 2 * dh) * 4))
        row(f"{tag}/delta rule: the convolutions' kept inputs",
            lambda: ops.delta_conv_update(fused, 0, off, dh, dg, dd, dv, taps, rs, rl, rslot, conv_state), R * (taps - 1) * (2 * GD + HV) * (2 + 4))
        dstate = torch.zeros(batch + 1, dh, dd, dv, device=dev)
        do = torch.empty(n, HV, device=dev)
        row(f"{tag}/delta rule: recurrence", lambda: ops.delta_scan(dq, dk, dvv, beta, decay, dstate, do, rs, rl, rslot, dh, dg, dd, dv),
            n * (2 * GD + 2 * HV + 2 * dh) * 4 + R * 2 * dh * dd * dv * 4, 6.0 * n * dh * dd * dv)
        gated = torch.empty(n, HV, dtype=bf, device=dev)
        row(f"{tag}/head norm and gate", lambda: ops.head_gate_norm(do, fused, 0, off["g"], nw, 1e-6, gated, dh, dv), n * HV * (4 + 2 + 2))
    # ---- experts: Taritar's gated clamped unit with softmax scores, and this design's (sigmoid scores on the inputs, no gate, squared ReLU)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        x = rnd(n, W, dtype=bf)
        wr = rnd(E, W, scale=0.05)
        chosen, weights = torch.empty(n, top, dtype=i32, device=dev), torch.empty(n, top, device=dev)
        for scores in ("softmax", "sigmoid"):
            row(f"{tag}/router ({scores} scores, choice)", lambda: ops.moe_route(x, wr, None, chosen, weights, None, 1, 1, scores=scores),
                n * W * 2 + E * W * 4)
        pairs = n * top
        count, offset = torch.empty(E, dtype=i32, device=dev), torch.empty(E + 1, dtype=i32, device=dev)
        order, place = torch.empty(pairs, dtype=i32, device=dev), torch.empty(pairs, dtype=i32, device=dev)
        tiles = torch.empty(1 + 3 * ops.moe_row_tiles(pairs, E), dtype=i32, device=dev)
        plan_scratch = torch.empty(ops.MOE_PLAN_SEGMENTS * E, dtype=i32, device=dev)
        ops.moe_plan(chosen, count, offset, order, place, tiles, plan_scratch)
        w_gu, w_u, w_d = rnd(E, 2 * eff, W, dtype=bf, scale=0.02), rnd(E, eff, W, dtype=bf, scale=0.02), rnd(E, W, eff, dtype=bf, scale=0.02)
        act, y = torch.empty(pairs, eff, dtype=bf, device=dev), torch.empty(pairs, W, device=dev)
        used = min(E, pairs)
        flat = weights.view(-1)
        if pairs >= 1024:
            xs = torch.empty(pairs, W, dtype=bf, device=dev)
            row(f"{tag}/experts: the tokens' rows into sorted order", lambda: ops.moe_gather(x, order, top, xs), pairs * W * 4)
            row(f"{tag}/experts: the tokens' rows into sorted order, times their scores", lambda: ops.moe_gather(x, order, top, xs, row_weights=flat),
                pairs * W * 4)
            row(f"{tag}/experts: gate|up with the clamped unit (grouped, tensor memory)",
                lambda: ops.gemm_bf16_tc_grouped(xs, w_gu, act, tiles, True, 7.0, 1.702), used * 2 * eff * W * 2 + pairs * (W + eff) * 2, 4.0 * pairs * eff * W)
            row(f"{tag}/experts: up with the squared ReLU (grouped, tensor memory)",
                lambda: ops.gemm_bf16_tc_grouped(xs, w_u, act, tiles, False, unit="relu_squared"), used * eff * W * 2 + pairs * (W + eff) * 2,
                2.0 * pairs * eff * W)
            row(f"{tag}/experts: down (grouped, tensor memory)", lambda: ops.gemm_bf16_tc_grouped(act, w_d, y, tiles, False),
                used * eff * W * 2 + pairs * (eff * 2 + W * 4), 2.0 * pairs * eff * W)
        else:
            row(f"{tag}/experts: gate|up with the clamped unit (grouped, mma.sync)", lambda: ops.moe_grouped(x, w_gu, act, offset, order, top, True, 7.0, 1.702),
                used * 2 * eff * W * 2 + pairs * (W + eff) * 2, 4.0 * pairs * eff * W)
            row(f"{tag}/experts: up with the squared ReLU on scored inputs (grouped, mma.sync)",
                lambda: ops.moe_grouped(x, w_u, act, offset, order, top, False, unit="relu_squared", row_weights=flat),
                used * eff * W * 2 + pairs * (W + eff) * 2, 2.0 * pairs * eff * W)
            row(f"{tag}/experts: down (grouped, mma.sync)", lambda: ops.moe_grouped(act, w_d, y, offset, order, top, False),
                used * eff * W * 2 + pairs * (eff * 2 + W * 4), 2.0 * pairs * eff * W)
        o32 = torch.empty(n, W, device=dev)
        row(f"{tag}/experts' outputs weighted and summed", lambda: ops.moe_combine(y, place, weights, None, None, o32), pairs * W * 4 + n * W * 4)
        row(f"{tag}/experts' outputs summed as they are", lambda: ops.moe_combine(y, place, None, None, None, o32), pairs * W * 4 + n * W * 4)
    # ---- the token's own input: the gate on the table row (beside the gated activation of a feed-forward of that width)
    tbl = rnd(size["vocab"], side, dtype=bf)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        ids = torch.randint(0, size["vocab"], (n,), generator=g, device=dev, dtype=i32)
        z, gu = rnd(n, side, dtype=bf), rnd(n, 2 * side, dtype=bf)
        tg = torch.empty(n, side, dtype=bf, device=dev)
        row(f"{tag}/gated activation of a feed-forward of the token input's width", lambda: ops.gated_act(gu, tg, "gelu_tanh"), n * side * 2 * 3)
        row(f"{tag}/token input: gelu_tanh of the projection times the table row", lambda: ops.token_gate(z, 0, ids, tbl, "gelu_tanh", tg), n * side * 2 * 3)
    return out


def gudarax_bench(args) -> int:
    import torch
    from wllm_b200.config import EngineConfig, GudaraxConfig, ZafilixConfig
    from wllm_b200.engine import build_model
    pk = peaks()
    ps, T = args.page_size, 2048
    context = args.context or 2048
    engine_cfg = EngineConfig(dtype="bfloat16", block_size=ps, max_num_seqs=max(64, args.batch), cuda_graphs=not args.no_graphs)
    sizes = {}
    for name in (args.sizes if args.sizes != "2b,7b" else "2k,4k").split(","):
        size = GUDARAX_SIZES[name]
        nq, nkv, hd = size["attn"]
        H, dim, vd, rank, _ = size["latent"]
        # the closest existing design at equal sizes: Zafilix (attention with whole-row norms, in blocks of the window's size; latent
        # attention in a window of that size with a turning part of 64), dense feed-forwards of the dense width
        zaf = dict(ZAFILIX_SIZES[name], width=size["width"], ff=size["ff"], attn=(nq, nkv, hd), block=size["window"],
                   latent=(H, dim, 64, vd, rank), window=size["window"], vocab=size["vocab"])
        models = {"zafilix": ZafilixConfig.from_dict(zafilix_config(zaf)), "gudarax": GudaraxConfig.from_dict(gudarax_config(size))}
        res = {}
        for label, cfg in models.items():
            model = build_model(None, engine_cfg.dtype, engine_cfg.device, config=cfg, random_seed=1)
            pre_ms = prefill_run(model, engine_cfg, T, ps)
            ms, launches, _, clocks, _ = decode_run(model, engine_cfg, args.batch, context, min(args.steps, 32), args.warmup, ps, 3)
            res[label] = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "prefill_tok_s": round(T / (pre_ms / 1e3), 1),
                          "prefill_ms": round(pre_ms, 3), "decode_tok_s": round(args.batch / (ms / 1e3), 1),
                          "decode_ms_per_step": round(ms, 4), "decode_launches": launches,
                          "decode_weights_hbm_frac": round(model.weight_bytes() / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3), "clocks": clocks}
            del model
            torch.cuda.empty_cache()
        sizes[name] = {"shape": size, "models": res}
        if not args.no_points:
            sizes[name]["kernels"] = gudarax_kernel_table(size, pk, T, args.batch, context)
    print(json.dumps({"metric": "Gudarax beside Zafilix at equal layer sizes: prefill tok/s @ 2048 tokens, decode tok/s",
                      "design": "gudarax", "unit": "tokens/s", "n_gpus": 1, "steps": min(args.steps, 32), "warmup": args.warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids, random cached keys/values)",
                      "config": {"global_batch": args.batch, "seq_len": context, "prefill_tokens": T, "page_size": ps,
                                 "cuda_graphs": not args.no_graphs, "peaks": pk["source"],
                                 "l2": "kernel table: a 640 MB buffer is written before every timed launch"},
                      "peaks": pk, "sizes": sizes}))
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
    ap.add_argument("--design", default="gemma", choices=["gemma", "pesanex", "taritar", "zafilix", "gudarax"],
                    help="gemma: the default workload; pesanex, taritar, zafilix, gudarax: models of that design beside a Gemma of equal layer sizes (another line)")
    ap.add_argument("--sizes", default="2b,7b", help="which of the layer sizes to run (--design pesanex: 2b, 7b; taritar, zafilix, gudarax: 2k, 4k)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)
    if args.design == "pesanex":
        return pesanex_bench(args)
    if args.design == "taritar":
        return taritar_bench(args)
    if args.design == "zafilix":
        return zafilix_bench(args)
    if args.design == "gudarax":
        return gudarax_bench(args)
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
