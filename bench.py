#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Llama shapes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model llama31-8b|llama32-3b|llama2-7b] [--dtype bf16|fp16|fp32]
                    [--workload decode|serve] [--layers L] [--batch B] [--context S] [--trials N]

Prints ONE JSON line.

`--workload decode` (the default): `value` is decoded tokens per second at batch 8 with S cached
tokens per request (8192 for the 8B shape): the median of N trials (five by default), each of K
decode steps (forward pass of 8 single tokens over the paged cache, sampling included) timed with
CUDA events after W warm-up steps.  Trials of the different points alternate (batch 8, 1, 64,
then again), and every point reports median, minimum and maximum, the rule the reference sets for
its own numbers (docs/ARCHITECTURE.md:228).  `points` holds decode at batch 1 and 64 at the same
context, and the model's own decode workload (1024-token prompts and 256 new tokens for the 8B
shape, 4096-token prompts for the 3B shape): all 256 new tokens are timed.  `prefill` is a
2048-token prompt in one step; `roofline` is the decode step's bytes over its time against the
measured copy bandwidth; `e2e` is the headline point through `ferrum_b200.Engine.step()`: token
ids in from pinned host memory, sampled ids back to the host, every step.

`--workload serve`: continuous batching of 64 requests with prompts of 128 to 2048 tokens and
128 to 512 new tokens each, prompts cut into portions (`--chunk-size`), through `Engine`.
`value` is generated tokens per second over the whole run; the line also gives the time to the
first token (median and 95th percentile), preemptions, and what a step that cannot be replayed
from a CUDA graph costs the host.

Weights are random N(0, 0.02); token ids are uniform random from a seed.  No L2 flush is needed
between steps: a step reads gigabytes of weights, far more than the 126 MB L2 holds.
"""
import argparse
import gc
import json
import os
import random
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
# Two more shapes that the reference's workloads name, for `--model`.
LLAMA2_7B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 128, "intermediate_size": 11008, "vocab_size": 32000,
    "rope_theta": 10000.0, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
LLAMA32_3B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 3072, "num_hidden_layers": 28, "num_attention_heads": 24,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
# name -> (printed name, config, default context of the headline point, prompt length of the model's
# own decode workload or None)
MODELS = {"llama31-8b": ("Llama-3.1-8B", LLAMA31_8B, 8192, 1024), "llama2-7b": ("Llama-2-7B", LLAMA2_7B, 2048, None),
          "llama32-3b": ("Llama-3.2-3B", LLAMA32_3B, 4096, 4096)}
NEW_TOKENS = 256          # new tokens of the decode workloads
DTYPES = {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32"}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = {k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops") if k in d}
        if "bf16_tflops_sustained" in d:
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        if "hbm_gbs" in out and "bf16_tflops" in out:
            out["source"] = "measured"
            return out
    except (OSError, ValueError, KeyError, TypeError):
        pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with NVML (read-only) while a region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, period=0.1):
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            idx = int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
            self._nv, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
                mask = self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def reference_arm():
    """The reference is a Rust workspace with no Python packaging and there is no Rust
    toolchain in this image, so it cannot be installed or run here."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "JustinA988/ferrum is a CPU-only Rust workspace: pip reports 'neither setup.py nor "
                      "pyproject.toml found' and no cargo/rustc is installed, so it cannot be built offline"}))
    return 0


def layer_params(c):
    e, f = c["hidden_size"], c["intermediate_size"]
    q, kv = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    return e * q + 2 * e * kv + q * e + 3 * e * f


def spread(values, digits=1):
    """median, range and count of a point's trials."""
    return {"median": round(statistics.median(values), digits), "min": round(min(values), digits),
            "max": round(max(values), digits), "n": len(values)}


def shape_config(model_name, cfgd, L, full_layers, extra):
    out = {"model": f"{model_name} shape, random weights N(0,0.02)", "layers": L, "layers_full_model": full_layers,
           "hidden": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"], "kv_heads": cfgd["num_key_value_heads"],
           "head_dim": cfgd["head_dim"], "intermediate": cfgd["intermediate_size"], "vocab": cfgd["vocab_size"]}
    out.update(extra)
    assert len(out) <= 20
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--model", default="llama31-8b", choices=sorted(MODELS), help="layer sizes (random weights)")
    ap.add_argument("--dtype", default="bf16", choices=sorted(DTYPES), help="compute dtype; fp32 is the true 32-bit path")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None,
                    help="cached tokens per request of the headline point (default 8192 for llama31-8b, 4096 for "
                         "llama32-3b, 2048 for llama2-7b and for fp32: what lets the batch-64 point fit the memory)")
    ap.add_argument("--trials", type=int, default=5, help="timed regions per point; median and range are reported")
    ap.add_argument("--chunk-size", type=int, default=512, help="serve: the longest prompt portion of a step")
    ap.add_argument("--requests", type=int, default=64, help="serve: number of requests")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.workload == "serve":
        return serve(args)
    return decode(args)


def build_model(args, max_positions):
    import torch
    from ferrum_b200.config import registry
    from ferrum_b200.engine.api import parse_dtype
    from ferrum_b200.weights import init_random
    model_name, shape, _, _ = MODELS[args.model]
    cfgd = dict(shape)
    full_layers = cfgd["num_hidden_layers"]
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    arch = registry.lookup(cfgd["architectures"][0])
    cfg = arch.read_config(cfgd)
    td = parse_dtype(DTYPES[args.dtype])
    torch.manual_seed(0)
    model = arch.build(cfg, td, "cuda", max_positions=max_positions)
    init_random(model, 0, "cuda")
    return model, cfg, cfgd, td, model_name, full_layers


# ---------------------------------------------------------------------------------- decode workload
def decode(args):
    import torch
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.engine import ModelRunner, StepEntry
    from ferrum_b200.engine.api import Engine
    from ferrum_b200.ops import lib as ops

    W, K, N_TRIALS = max(3, args.warmup), max(1, args.steps), max(1, args.trials)
    pk = peaks()
    _, _, default_ctx, prompt_len = MODELS[args.model]
    if args.context is None:
        args.context = min(default_ctx, 2048) if args.dtype == "fp32" else default_ctx
    ctx_len, B = args.context, args.batch
    esize = 4 if args.dtype == "fp32" else 2
    page = 16
    max_len = max(ctx_len, (prompt_len or 0) + NEW_TOKENS) + W + K + 128 + 4 * B
    model, cfg, cfgd, td, model_name, full_layers = build_model(args, max_len)
    L = cfgd["num_hidden_layers"]
    gen = torch.Generator().manual_seed(0)

    def tokens(n):
        return torch.randint(0, cfg.n_vocab, (n,), generator=gen).tolist()

    tied = bool(cfgd.get("tie_word_embeddings"))
    weight_bytes = esize * (L * layer_params(cfgd) + cfgd["vocab_size"] * cfgd["hidden_size"]) + 4 * (2 * L + 1) * cfgd["hidden_size"]
    kv_per_token = 2 * cfgd["num_key_value_heads"] * cfgd["head_dim"] * esize * L

    # One cache and one runner serve every point: requests are opened at the point's context and
    # closed after its trial, so trials of different points can alternate.
    max_b = B if args.skip_points else max(B, 64)
    cache = CacheStorage(model, td, "cuda", page_size=page, max_tokens=max_b * (max_len + page), max_requests=max_b,
                         max_model_len=max_len)
    for p in cache.pools:
        p.normal_(0.0, 0.02)                       # contents of a cache that earlier steps left
    runner = ModelRunner(model, cache, max_batch_tokens=2048, max_batch_requests=max_b)
    mgr = cache.manager
    ids = torch.empty(max_b, dtype=torch.int32, device="cuda")

    def decode_trial(batch, start, steps, warm):
        """`steps` timed decode steps of `batch` requests that hold `start` tokens each when timing
        begins (the warm-up steps come before, at shorter contexts).  (tok/s, ms per step, launches)"""
        slots = [cache.open() for _ in range(batch)]
        first = start - warm
        for s in slots:
            mgr.grow(s, first - 1)
            mgr.commit(s, first - 1)

        def one(i):
            entries = [StepEntry(s, first - 1 + i, [t], [0]) for s, t in zip(slots, tokens(batch))]
            logits = runner.step(entries, check=False)
            ops.sample(logits, batch, ids, runner.ctx.err)

        for i in range(warm):
            one(i)
        torch.cuda.synchronize()
        l0 = ops.launches
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            one(warm + i)
        ev1.record()
        torch.cuda.synchronize()
        runner.check_device_errors()
        ms = ev0.elapsed_time(ev1) / steps
        launches = ops.launches - l0
        for s in slots:
            cache.close(s)
        return batch / ms * 1e3, ms, launches

    # (name, batch, context at the first timed step, timed steps)
    plan = [(f"decode_b{B}", B, ctx_len, K)]
    if not args.skip_points:
        plan += [(f"decode_b{b}", b, ctx_len, max(4, K // 2)) for b in (1, 64) if b != B]
        if prompt_len:
            plan += [(f"decode_b{b}_prompt{prompt_len}_new{NEW_TOKENS}", b, prompt_len, NEW_TOKENS) for b in (1, 8, 64)]
    results = {name: [] for name, *_ in plan}
    ms_main, launches = [], 0
    with ClockSampler() as clk:
        for trial in range(N_TRIALS):
            for name, b, start, steps in plan:
                r, ms, n = decode_trial(b, start, steps, W)
                results[name].append(r)
                if name == plan[0][0]:
                    ms_main.append(ms)
                    launches = n
    clocks = clk.summary()
    value = statistics.median(results[plan[0][0]])
    ms_step = statistics.median(ms_main)
    step_bytes = weight_bytes + B * cfgd["hidden_size"] * esize + B * ctx_len * kv_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]}
    points, trials = {}, {}
    for name, b, start, steps in plan:
        trials[name] = spread(results[name])
        if name != plan[0][0]:
            points[name] = trials[name]["median"]
            # every point against the copy peak: weights once, the cache of its requests (mean context)
            mean_ctx = start + (steps - 1) / 2
            bytes_ = weight_bytes + b * mean_ctx * kv_per_token
            trials[name]["hbm_frac"] = round(bytes_ * trials[name]["median"] / b / 1e9 / pk["hbm_gbs"], 4)

    # ------------------------------------------------------------ prefill of 2048 tokens
    prefill = None
    if not args.skip_prefill:
        T = 2048
        times = []
        for it in range(W + N_TRIALS):
            slot = cache.open()
            toks = tokens(T)
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            runner.step([StepEntry(slot, 0, toks, [T - 1])], check=False)
            ev1.record()
            torch.cuda.synchronize()
            if it >= W:
                times.append(ev0.elapsed_time(ev1))
            cache.close(slot)
        runner.check_device_errors()
        ms = statistics.median(times)
        hq, d = cfgd["num_attention_heads"], cfgd["head_dim"]
        flops = 2.0 * L * layer_params(cfgd) * T + 2.0 * cfgd["vocab_size"] * cfgd["hidden_size"] + L * 4.0 * hq * d * T * T / 2
        if args.dtype == "fp32":     # the CUDA cores' own peak: SMs x 128 lanes x 2 flops x the maximum clock
            peak, of = ops.sm_count() * 128 * 2 * (clocks["sm_max_mhz"] or 1965) * 1e6, "nominal ffma"
        else:
            peak, of = pk["bf16_tflops"] * 1e12, pk["source"]
        prefill = {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3), "ms_min": round(min(times), 3),
                   "ms_max": round(max(times), 3), "frac": round(flops / (ms * 1e-3) / peak, 4), "of": of}
    del runner, cache
    torch.cuda.empty_cache()

    # ------------------------------------------------------------ end to end through the Engine
    e2e = None
    if not args.skip_e2e:
        eng = Engine(model=model, page_size=page, num_pages=(B * (max_len + page)) // page, max_batch_tokens=8192,
                     max_batch_seqs=B, max_model_len=max_len)
        for _ in range(B):
            eng.submit(tokens(ctx_len - 1), W + K + 80 + 4 * B)
        started = set()
        while len(started) < B:                        # prompts, untimed; ends with every request decoding
            started.update(ev.id for ev in eng.step() if ev.kind == "token")
        # The prompts have just run at the power cap; the first dozen decode steps after them are
        # up to 10 % slow while the clocks come back.  They are part of the warm-up.
        e2e_warm = W + 16
        for _ in range(e2e_warm):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        got = 0
        for _ in range(K):
            got += sum(1 for ev in eng.step() if ev.kind == "token")
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert got == B * K, (got, B * K)
        e2e = {"value": round(got / dt, 1), "unit": "tok/s", "h2d_bytes_per_step": int(eng.runner.ctx.h2d_bytes),
               "d2h_bytes_per_step": int(eng.sampler.d2h_bytes), "ms_per_step": round(dt / K * 1e3, 3),
               "warmup": e2e_warm}

    line = {
        "metric": f"decode tok/s ({model_name} {args.dtype}, batch {B}, context {ctx_len})", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "impl": "ours",
        "config": shape_config(model_name, cfgd, L, full_layers, {
            "global_batch": B, "seq_len": ctx_len, "page_size": page, "prefill_tokens": 2048, "parallelism": "single GPU",
            "trials": f"{N_TRIALS} alternating trials per point, median reported",
            "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step)",
            "sampling": "greedy on device, inside the step", "tied_output": tied}),
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill, "roofline": roofline,
        "points": points, "trials": trials,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------- serving workload
def serve(args):
    """Continuous batching through the Python entry point, the reference's fourth configuration:
    64 requests, prompt lengths uniform in [128, 2048], 128 to 512 new tokens, chunked prefill."""
    import torch
    from ferrum_b200.engine.api import Engine
    from ferrum_b200.ops import lib as ops

    pk = peaks()
    n_req, chunk = args.requests, args.chunk_size
    max_len = 2048 + 512 + 16
    model, cfg, cfgd, td, model_name, full_layers = build_model(args, max_len)
    L = cfgd["num_hidden_layers"]
    rng = random.Random(0)
    reqs = [(rng.randint(128, 2048), rng.randint(128, 512)) for _ in range(n_req)]
    page = 16
    runs = []
    clk = ClockSampler()
    with clk:
        for rep in range(2):                              # the first run compiles nothing but captures the graphs
            eng = Engine(model=model, page_size=page, num_pages=(n_req * max_len) // page, max_batch_tokens=2048,
                         max_batch_seqs=n_req, chunk_size=chunk, max_model_len=max_len)
            gen = torch.Generator().manual_seed(1)
            launch_ms = []
            inner = eng._launch

            def timed_launch(plan, ahead_of_commit=False, inner=inner, launch_ms=launch_ms):
                replays = eng.runner.graph_replays
                t = time.perf_counter()
                out = inner(plan, ahead_of_commit=ahead_of_commit)
                if eng.runner.graph_replays == replays:      # launched kernel by kernel: what the host spends on it
                    launch_ms.append((time.perf_counter() - t) * 1e3)
                return out

            eng._launch = timed_launch
            ids = [eng.submit(torch.randint(0, cfg.n_vocab, (n,), generator=gen).tolist(), new) for n, new in reqs]
            torch.cuda.synchronize()
            l0 = ops.launches
            t0 = time.perf_counter()
            first, done, generated, steps = {}, 0, 0, 0
            while done < n_req:
                events = eng.step()
                now = time.perf_counter()
                steps += 1
                for ev in events:
                    if ev.kind == "token":
                        generated += 1
                        first.setdefault(ev.id, now - t0)
                    else:
                        done += 1
            while eng.step():
                pass
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            st = eng.stats()
            ttft = sorted(first[i] for i in ids)
            runs.append({"seconds": round(dt, 3), "generated_tok_s": round(generated / dt, 1),
                         "total_tok_s": round((generated + st["prompt_tokens"]) / dt, 1), "steps": steps,
                         "generated": generated, "prompt_tokens": int(st["prompt_tokens"]),
                         "ttft_ms_median": round(statistics.median(ttft) * 1e3, 1),
                         "ttft_ms_p95": round(ttft[min(len(ttft) - 1, int(0.95 * len(ttft)))] * 1e3, 1),
                         "preemptions": int(st["preemptions"]), "graph_replays": int(eng.runner.graph_replays),
                         "non_graph_steps": len(launch_ms),
                         "host_ms_per_non_graph_step": round(statistics.median(launch_ms), 3) if launch_ms else None,
                         "gpu_launches": int(ops.launches - l0)})
            eng._launch = None            # (the timing wrapper holds the engine: break the cycle so that its cache is freed)
            del eng, inner, timed_launch
            gc.collect()
            torch.cuda.empty_cache()
    best = runs[-1]
    line = {
        "metric": f"generated tok/s ({model_name} {args.dtype}, {n_req} requests, prompts U[128,2048], 128-512 new tokens, "
                  f"continuous batching, portions of {chunk})",
        "value": best["generated_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": best["steps"], "warmup": runs[0]["steps"],
        "ms_per_step": round(best["seconds"] / best["steps"] * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "impl": "ours",
        "config": shape_config(model_name, cfgd, L, full_layers, {
            "global_batch": n_req, "seq_len": 2560, "page_size": page, "chunk_size": chunk, "max_batch_tokens": 2048,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (the weights are read every step)",
            "sampling": "greedy on device, inside the step",
            "timing": "host clock around the whole run, after one identical warm-up run"}),
        "clocks": clk.summary(), "serve": best, "warmup_run": runs[0], "gpu_launches": best["gpu_launches"],
        "e2e": {"value": best["generated_tok_s"], "unit": "tok/s", "note": "the workload itself runs through Engine.step()"},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
