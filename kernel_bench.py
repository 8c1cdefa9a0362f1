#!/usr/bin/env python3
"""Times one kernel of the engine in isolation (CUDA events, warm-up, inputs larger than L2)
and prints one JSON line with its achieved bandwidth or throughput against the measured
peaks.  This is the small case that `ncu` captures are taken on.

    python kernel_bench.py attn_decode [--batch 8] [--context 8192] [--layers 4]
    python kernel_bench.py attn_prefill [--tokens 2048]
    python kernel_bench.py gemm --tokens 8 --n 6144 --k 4096 [--epilogue store|residual|swiglu] [--copies 8]
    python kernel_bench.py gemm|attn_decode|attn_prefill ... --dtype fp32    (the CUDA-core kernels of the 32-bit path)
    python kernel_bench.py rmsnorm|rope --tokens 8
    python kernel_bench.py step --tokens 2048 [--layers 2] [--dtype bf16|fp16|fp32]   (one prompt portion through the model)
    FERRUM_KERNEL_TRACE=1 python kernel_bench.py timeline [--batch 8] [--context 8192] [--layers 4]
`step` runs whole steps of one request's prompt portion of `--tokens` tokens through a model of
`--layers` layers (the step function, cache and kernels that generation uses) and prints the
step's time; under `ncu --metrics gpu__time_duration.sum` it is the list of the step's launches.
`timeline` runs decode steps of a model with `--layers` layers on the library built with the
kernel trace (block 0 of every instrumented kernel records the GPU's global timer at entry,
after its dependency wait and at exit) and prints one line per launch of the last step: what
each kernel costs once its inputs are there, and what the hand-over between kernels costs.
Shapes default to Llama-3.1-8B (32 query heads, 8 KV heads, head size 128, width 4096).
"""
import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["attn_decode", "attn_prefill", "gemm", "rmsnorm", "rope", "step", "timeline"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--epilogue", default="store", choices=["store", "residual", "swiglu"])
    ap.add_argument("--ctas", type=int, default=0, help="gemm: CTAs of the grid (0 = one per SM)")
    ap.add_argument("--copies", type=int, default=8, help="distinct weight/cache copies cycled through, to defeat L2")
    ap.add_argument("--layers", type=int, default=4, help="cache planes cycled through (attention)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--deferred", action="store_true", help="gemm: leave the partials to the consumer (as decoding does)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"],
                    help="fp32 times the CUDA-core kernels of the true 32-bit path (its fraction is of the FFMA peak)")
    ap.add_argument("--attention-pair", choices=["on", "off"], default=None,
                    help="attn_prefill at head size 128: the kernel of two CTAs on one tile (on) or of one CTA (off)")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--no-dependent-launch", action="store_true", help="plain stream order between the launches")
    args = ap.parse_args()

    if args.kernel == "timeline":
        return timeline(args)
    if args.kernel == "step":
        return prompt_step(args)
    import torch
    from bench import peaks
    from ferrum_b200.engine.batch import StepContext, StepEntry
    from ferrum_b200.ops import lib as ops
    ops.require_cuda()
    ops.set_dependent_launch(not args.no_dependent_launch)
    if args.attention_pair is not None:
        ops.set_attention_pair_kernel(args.attention_pair == "on")
    pk = peaks()
    dev = "cuda"
    td = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    esize = 4 if args.dtype == "fp32" else 2
    Hq, Hkv, D, ps = args.hq, args.hkv, args.head_dim, args.page_size
    gen = torch.Generator(device=dev).manual_seed(0)
    runs = []

    if args.kernel in ("attn_decode", "attn_prefill"):
        from ferrum_b200.parts import PagedAttention, attention as attention_part
        # In a step a product follows the attention kernel; here attention launches follow each
        # other, and released early they would only take each other's places on the SMs.
        attention_part.EARLY_TRIGGER_MAX_TOKENS = 0
        decode = args.kernel == "attn_decode"
        R = args.batch if decode else 1
        qlen = 1 if decode else args.tokens
        ctx_len = args.context if decode else args.tokens
        n_pages = R * ((ctx_len + ps - 1) // ps)
        width = (ctx_len + ps - 1) // ps
        planes = [torch.randn(n_pages, 2, Hkv, ps, D, device=dev, generator=gen).mul_(0.5).to(td) for _ in range(args.layers)]
        perm = torch.randperm(n_pages).view(R, width).tolist()
        ctx = StepContext(dev, max(16, R * qlen), R, [width])
        ctx.fixed_shapes = False
        ctx.fill([StepEntry(r, ctx_len - qlen, [1] * qlen) for r in range(R)], [perm])
        T = R * qlen
        q = torch.randn(T, Hq * D, device=dev, generator=gen).to(td)
        out = torch.empty(T, Hq * D, device=dev, dtype=td)
        att = PagedAttention(Hq * D, Hq, Hkv, D, None, td)

        class Cache:
            pass
        caches = []
        for pl in planes:
            c = Cache()
            c.plane, c.page_stride, c.page_size, c.group, c.writes = pl, pl.stride(0), ps, 0, True
            caches.append(c)
        table = ctx.block_tables[0]
        run_attention = att._flash if ops.attention_flash_supported(td, D) else att._generic
        runs = [lambda c=c: run_attention(q, out, ctx, c, table) for c in caches]
        kv_bytes = R * ctx_len * 2 * Hkv * D * esize
        flops = 4.0 * Hq * D * (ctx_len * qlen if decode else qlen * qlen / 2) * R
        work = {"bytes": kv_bytes + 2 * T * Hq * D * esize, "flops": flops, "bound": "hbm" if decode else "tensor"}
    elif args.kernel == "gemm":
        M, N, K = args.tokens, args.n, args.k
        dual = args.epilogue == "swiglu"
        ws_f, tiles = ops.gemm_tc_workspace(M, N, K, dual)
        ws = torch.empty(ws_f, device=dev)
        cnt = torch.zeros(max(tiles, 1), dtype=torch.int32, device=dev)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        x = torch.randn(M, K, device=dev, generator=gen).to(td)
        weights = [torch.randn(N * (2 if dual else 1), K, device=dev, generator=gen).mul_(0.02).to(td) for _ in range(args.copies)]
        if args.epilogue == "residual":
            o = torch.zeros(M, N, device=dev)
            epi = ops.TC_RESIDUAL
        else:
            o = torch.empty(M, N * (2 if dual and args.dtype == "fp32" else 1), device=dev, dtype=td)
            epi = ops.TC_SWIGLU if dual else ops.TC_STORE_BF16
        if args.dtype == "fp32":     # the CUDA-core product (gate and up as one product of 2N rows; the activation is a kernel of its own)
            gepi = ops.EPI_RESIDUAL if args.epilogue == "residual" else ops.EPI_STORE
            runs = [lambda w=w: ops.gemm_generic(x, w, o, gepi) for w in weights]
        else:
            runs = [lambda w=w: ops.gemm_tc(x, w, o, epi, err, ws, cnt, N=N, dual_offset=N if dual else 0, n_ctas=args.ctas) for w in weights]
        if args.deferred and args.dtype != "fp32":
            if not ops.gemm_tc_can_defer(M, N, K, dual):
                sys.exit("this shape cannot defer its reduction")
            runs = [lambda w=w: ops.gemm_tc_deferred(x, w, err, ws, N=N, dual_offset=N if dual else 0) for w in weights]
        wb = N * K * esize * (2 if dual else 1)
        work = {"bytes": wb + M * K * esize + M * N * (4 if args.epilogue == "residual" else esize),
                "flops": 2.0 * M * N * K * (2 if dual else 1), "bound": "hbm" if M <= 128 else "tensor"}
    elif args.kernel == "rmsnorm":
        T, E = args.tokens, args.k
        x = torch.randn(T, E, device=dev, generator=gen)
        w = torch.ones(E, device=dev)
        o = torch.empty(T, E, device=dev, dtype=torch.bfloat16)
        runs = [lambda: ops.rmsnorm(x, w, o, 1e-5)]
        work = {"bytes": T * E * 6, "flops": 3.0 * T * E, "bound": "hbm"}
    else:
        from ferrum_b200.parts.rope import RotaryEmbedding
        T = args.tokens
        rot = RotaryEmbedding(D, D, 500000.0, None, "half", args.context + 8, dev)
        width = (args.context + ps) // ps
        plane = torch.zeros(T * width, 2, Hkv, ps, D, device=dev, dtype=torch.bfloat16)
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev, generator=gen).bfloat16()
        pos = torch.full((T,), args.context - 1, dtype=torch.int32, device=dev)
        req = torch.arange(T, dtype=torch.int32, device=dev)
        table = torch.arange(T * width, dtype=torch.int32, device=dev).view(T, width)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        runs = [lambda: ops.rope_cache_write(qkv, T, pos, req, table, rot.cos_sin, plane, plane.stride(0), ps, Hq, Hkv, D, D,
                                             rot.pairing, True, err)]
        work = {"bytes": T * (Hq + 2 * Hkv) * D * 2 * 2, "flops": 0.0, "bound": "hbm"}

    for i in range(args.warmup):
        runs[i % len(runs)]()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.no_graph:
        ev0.record()
        for i in range(args.iters):
            runs[i % len(runs)]()
        ev1.record()
    else:
        # the launches go into one CUDA graph so that the host's launch rate does not bound
        # the measurement of kernels that take a few microseconds
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.iters):
                runs[i % len(runs)]()
        graph.replay()
        torch.cuda.synchronize()
        ev0.record()
        graph.replay()
        ev1.record()
    torch.cuda.synchronize()
    us = ev0.elapsed_time(ev1) / args.iters * 1e3
    gbs = work["bytes"] / (us * 1e-6) / 1e9
    tf = work["flops"] / (us * 1e-6) / 1e12
    if work["bound"] == "hbm":
        frac = gbs / pk["hbm_gbs"]
    elif args.dtype == "fp32":       # the CUDA cores' own peak: SMs x 128 lanes x 2 flops x the maximum clock
        frac = tf / (ops.sm_count() * 128 * 2 * 1.965e9 / 1e12)
        work["bound"] = "ffma"
    else:
        frac = tf / pk["bf16_tflops"]
    print(json.dumps({"kernel": args.kernel, "us": round(us, 2), "GBps": round(gbs, 1), "TFLOPs": round(tf, 2),
                      "bound": work["bound"], "frac_of_peak": round(frac, 4), "peaks": pk["source"],
                      "args": {k: v for k, v in vars(args).items() if k != "kernel"}}))
    return 0


def prompt_step(args):
    import torch
    from bench import LLAMA31_8B
    from ferrum_b200.cache.storage import CacheStorage
    from ferrum_b200.config import registry
    from ferrum_b200.engine.batch import StepEntry
    from ferrum_b200.engine.runner import ModelRunner
    from ferrum_b200.ops import lib as ops
    from ferrum_b200.weights import init_random
    ops.require_cuda()
    td = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    T = args.tokens
    cfgd = dict(LLAMA31_8B)
    cfgd["num_hidden_layers"] = args.layers
    arch = registry.lookup("LlamaForCausalLM")
    cfg = arch.read_config(cfgd)
    model = arch.build(cfg, td, "cuda", max_positions=T + 64)
    init_random(model, 0)
    cache = CacheStorage(model, td, "cuda", page_size=args.page_size, max_tokens=2 * (T + 64), max_requests=4, max_model_len=T + 64)
    runner = ModelRunner(model, cache, max_batch_tokens=T, max_batch_requests=2)
    gen = torch.Generator().manual_seed(1)
    times = []
    for rep in range(args.warmup + args.iters):
        slot = cache.open()
        toks = torch.randint(0, cfg.n_vocab, (T,), generator=gen).tolist()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        l0 = ops.launches
        ev0.record()
        runner.step([StepEntry(slot, 0, toks, [T - 1])], check=True)
        ev1.record()
        torch.cuda.synchronize()
        if rep >= args.warmup:
            times.append(ev0.elapsed_time(ev1))
        launches = ops.launches - l0
        cache.close(slot)
    times.sort()
    print(json.dumps({"kernel": "step", "tokens": T, "layers": args.layers, "dtype": args.dtype, "launches": int(launches),
                      "ms_median": round(times[len(times) // 2], 3), "ms_min": round(times[0], 3), "ms_max": round(times[-1], 3)}))
    return 0


def timeline(args):
    import ctypes
    import torch
    from bench import LLAMA31_8B
    from ferrum_b200.cache.storage import CacheStorage
    from ferrum_b200.config import registry
    from ferrum_b200.engine.batch import StepEntry
    from ferrum_b200.engine.runner import ModelRunner
    from ferrum_b200.ops import build, lib as ops
    from ferrum_b200.weights import init_random
    if not build.trace_build():
        sys.exit("timeline needs the trace build: set FERRUM_KERNEL_TRACE=1")
    B, C = args.batch, args.context
    cfgd = dict(LLAMA31_8B)
    cfgd["num_hidden_layers"] = args.layers
    arch = registry.lookup("LlamaForCausalLM")
    model = arch.build(arch.read_config(cfgd), torch.bfloat16, "cuda", max_positions=C + 64)
    init_random(model, 0)
    cache = CacheStorage(model, torch.bfloat16, "cuda", page_size=args.page_size, max_tokens=B * (C + 64), max_requests=B,
                         max_model_len=C + 64)
    runner = ModelRunner(model, cache, max_batch_tokens=max(B, 16), max_batch_requests=B)
    slots = [cache.open() for _ in range(B)]
    for s in slots:
        cache.manager.grow(s, C - 1)
        cache.manager.commit(s, C - 1)
    ids = torch.empty(B, dtype=torch.int32, device="cuda")

    def step(i):
        logits = runner.step([StepEntry(s, C - 1 + i, [7], [0]) for s in slots], check=False)
        ops.sample(logits, B, ids, runner.ctx.err)

    readers = [getattr(ops.lib(), n) for n in ("ferrum_trace_gemm", "ferrum_trace_elementwise", "ferrum_trace_flash")]

    def read():
        out = []
        for fn in readers:
            buf = (ctypes.c_ulonglong * (8192 * 4))()
            n = ctypes.c_uint(0)
            if fn(buf, ctypes.byref(n)):
                sys.exit("reading the trace failed")
            out += [tuple(buf[i * 4 + k] for k in range(4)) for i in range(min(n.value, 8192))]
        return sorted(out, key=lambda e: e[1])

    for i in range(6):          # warm-up; the decode graph is captured on the second step
        step(i)
    read()
    step(6)
    ev = read()
    names = {2: "norm", 3: "rotary+cache", 4: "swiglu_reduce", 5: "attention", 6: "combine"}
    t0, prev_exit = ev[0][1], None
    print(f"decode step, batch {B}, context {C}, {args.layers} layers; microseconds; block 0 of each launch")
    print(f"{'kernel':22s} {'entry':>9s} {'waited':>9s} {'exit':>9s} | {'work':>7s} {'hand-over':>9s}")
    for kind, entry, waited, exit_ in ev:
        if kind % 8 == 1:
            name = f"product N={kind // 16 * 64}" + (" x2" if kind & 8 else "")
        else:
            name = names.get(kind, str(kind))
        hand = (waited - prev_exit) / 1e3 if prev_exit else 0.0
        print(f"{name:22s} {(entry - t0) / 1e3:9.2f} {(waited - t0) / 1e3:9.2f} {(exit_ - t0) / 1e3:9.2f} | "
              f"{(exit_ - waited) / 1e3:7.2f} {hand:9.2f}")
        prev_exit = exit_
    return 0


if __name__ == "__main__":
    sys.exit(main())
