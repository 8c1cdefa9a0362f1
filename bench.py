#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Llama-3.1-8B shapes, bf16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with 8192 tokens of
context per request: K decode steps (forward pass of 8 single tokens over the paged cache,
sampling included) timed with CUDA events after W warm-up steps.  `e2e` is the same through
`ferrum_b200.Engine.step()`: token ids in from pinned host memory, sampled ids back to the
host, every step.  `prefill` is a 2048-token prompt in one step; `points` are decode at
batch 1 and 64; `roofline` is the decode step's bytes over its time against the measured
copy bandwidth.  Weights are random N(0, 0.02); token ids are uniform random from a seed.
No L2 flush is needed between steps: a step reads 15 GB of weights, far more than the
126 MB L2 holds.
"""
import argparse
import json
import os
import subprocess
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
# Two more shapes that the reference's workloads name (its configs 3 and 4), for `--model`.
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
MODELS = {"llama31-8b": ("Llama-3.1-8B", LLAMA31_8B), "llama2-7b": ("Llama-2-7B", LLAMA2_7B),
          "llama32-3b": ("Llama-3.2-3B", LLAMA32_3B)}
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--model", default="llama31-8b", choices=sorted(MODELS), help="layer sizes (random weights)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None,
                    help="cached tokens per request (default 8192; 4096 for llama32-3b and 2048 for llama2-7b, whose batch-64 point fits the memory then)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    W, K = max(3, args.warmup), max(1, args.steps)

    import torch
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.config import registry
    from ferrum_b200.engine import ModelRunner, StepEntry
    from ferrum_b200.engine.api import Engine
    from ferrum_b200.ops import lib as ops
    from ferrum_b200.weights import init_random

    pk = peaks()
    model_name, shape = MODELS[args.model]
    cfgd = dict(shape)
    full_layers = cfgd["num_hidden_layers"]
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    L = cfgd["num_hidden_layers"]
    arch = registry.lookup(cfgd["architectures"][0])
    cfg = arch.read_config(cfgd)
    if args.context is None:
        args.context = {"llama32-3b": 4096, "llama2-7b": 2048}.get(args.model, 8192)
    ctx_len, B = args.context, args.batch
    max_len = ctx_len + W + K + 128 + 4 * args.batch
    page = 16
    torch.manual_seed(0)
    model = arch.build(cfg, torch.bfloat16, "cuda", max_positions=max_len)
    init_random(model, 0, "cuda")
    gen = torch.Generator().manual_seed(0)

    def tokens(n):
        return torch.randint(0, cfg.n_vocab, (n,), generator=gen).tolist()

    weight_bytes = 2 * (L * layer_params(cfgd) + cfgd["vocab_size"] * cfgd["hidden_size"]) + 4 * (2 * L + 1) * cfgd["hidden_size"]
    kv_per_token = 2 * cfgd["num_key_value_heads"] * cfgd["head_dim"] * 2 * L

    # ------------------------------------------------------------ decode, device-timed
    def decode_rate(batch, steps, warm):
        cache = CacheStorage(model, torch.bfloat16, "cuda", page_size=page, max_tokens=batch * (max_len + page),
                             max_requests=batch, max_model_len=max_len)
        for p in cache.pools:
            p.normal_(0.0, 0.02)                       # contents of a cache that earlier steps left
        runner = ModelRunner(model, cache, max_batch_tokens=max(batch, 16), max_batch_requests=batch)
        mgr = cache.manager
        slots = [cache.open() for _ in range(batch)]
        for s in slots:
            mgr.grow(s, ctx_len - 1)
            mgr.commit(s, ctx_len - 1)
        ids = torch.empty(batch, dtype=torch.int32, device="cuda")

        def one(i):
            entries = [StepEntry(s, ctx_len - 1 + i, [t], [0]) for s, t in zip(slots, tokens(batch))]
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
        del runner, cache
        torch.cuda.empty_cache()
        return batch / ms * 1e3, ms, launches

    with ClockSampler() as clk:
        value, ms_step, launches = decode_rate(B, K, W)
    clocks = clk.summary()
    step_bytes = weight_bytes + B * cfgd["hidden_size"] * 2 + B * ctx_len * kv_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r, _, _ = decode_rate(b, max(4, K // 2), W)
            points[f"decode_b{b}"] = round(r, 1)

    # ------------------------------------------------------------ prefill of 2048 tokens
    prefill = None
    if not args.skip_prefill:
        T = 2048
        cache = CacheStorage(model, torch.bfloat16, "cuda", page_size=page, max_tokens=T + page, max_requests=2,
                             max_model_len=T + page)
        runner = ModelRunner(model, cache, max_batch_tokens=T, max_batch_requests=2)
        times = []
        for it in range(W + 3):
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
        ms = sorted(times)[len(times) // 2]
        hq, d = cfgd["num_attention_heads"], cfgd["head_dim"]
        flops = 2.0 * L * layer_params(cfgd) * T + 2.0 * cfgd["vocab_size"] * cfgd["hidden_size"] + L * 4.0 * hq * d * T * T / 2
        prefill = {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                   "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"]}
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
        "metric": f"decode tok/s ({model_name} bf16, batch {B}, context {ctx_len})", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"{model_name} shape, random weights N(0,0.02)", "layers": L, "layers_full_model": full_layers,
                   "hidden": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"],
                   "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                   "intermediate": cfgd["intermediate_size"], "vocab": cfgd["vocab_size"], "global_batch": B,
                   "seq_len": ctx_len, "context_len": ctx_len, "page_size": page, "prefill_tokens": 2048,
                   "parallelism": "single GPU", "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step)",
                   "sampling": "greedy on device, inside the step"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill, "roofline": roofline,
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
