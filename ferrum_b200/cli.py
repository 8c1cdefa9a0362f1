"""`ferrum` command line.

In the manner of the reference's CLI (crates/ferrum-cli/src/main.rs): a hand-written
argument parser, `--flag VALUE` and `--flag=VALUE`, unknown commands and arguments are
errors, exit code 2 for usage errors and 1 for runtime errors, messages prefixed
`ferrum: `.  The reference's only command, `serve`, is answered as it answers it without
`--mock`: this engine has no server.  Request options carry the names of the reference's
`SubmitRequest` and `SamplingParams` (crates/core-types/src/schedule.rs:16-49).

    ferrum generate --model DIR|FILE.gguf --prompt-tokens 1,2,3 [--prompt-tokens ...]
                    [--dtype bfloat16|float16|float32] [--max-new-tokens N] [--temperature T] [--top-p 1]
                    [--seed S] [--stop-tokens a,b] [--max-batch-tokens N] [--max-batch-seqs N]
                    [--chunk-size N] [--page-size N] [--num-pages N] [--max-model-len N]
                    [--random-weights] [--weights-seed S] [--stats] [--profile]
    ferrum random-weights --config CONFIG.json --out DIR [--seed S] [--dtype float32|bfloat16|float16] [--gguf]
    ferrum bench --model DIR|CONFIG.json [--random-weights] [--dtype D] [--batch B] [--prompt-len P] [--new-tokens N]
                 [--layers L] [--page-size N] [--chunk-size N] [--seed S]
    ferrum replay --model DIR --dtype D --out DIR --max-tokens N        (steps on standard input)
    ferrum dump FILE.gguf|FILE.safetensors|DIR
    ferrum serve                                                          (not part of this engine)
"""
from __future__ import annotations

import json
import os
import sys

USAGE = "usage: ferrum generate|random-weights|bench|replay|dump|serve [options]  (ferrum --help lists them)"

# option -> (kind, repeatable)
OPTIONS = {
    "generate": {"--model": "str", "--prompt-tokens": "tokens+", "--prompt-file": "str", "--dtype": "str",
                 "--max-new-tokens": "int", "--temperature": "float", "--top-p": "float", "--seed": "int",
                 "--stop-tokens": "tokens", "--max-batch-tokens": "int", "--max-batch-seqs": "int",
                 "--chunk-size": "int", "--page-size": "int", "--num-pages": "int", "--max-model-len": "int",
                 "--random-weights": "flag", "--weights-seed": "int", "--stats": "flag", "--profile": "flag"},
    "random-weights": {"--config": "str", "--out": "str", "--seed": "int", "--dtype": "str", "--gguf": "flag"},
    "bench": {"--model": "str", "--random-weights": "flag", "--dtype": "str", "--batch": "int", "--prompt-len": "int",
              "--new-tokens": "int", "--layers": "int", "--page-size": "int", "--chunk-size": "int", "--seed": "int"},
    "replay": {"--model": "str", "--dtype": "str", "--out": "str", "--max-tokens": "int", "--page-size": "int",
               "--max-requests": "int"},
    "dump": {},
    "serve": {"--mock": "flag", "--bind": "str"},
}


class CliError(Exception):
    pass


def _convert(kind, flag, text):
    try:
        if kind == "int":
            return int(text)
        if kind == "float":
            return float(text)
        if kind.startswith("tokens"):
            return [int(t) for t in text.replace(" ", "").split(",") if t != ""]
    except ValueError:
        raise CliError(f"{flag}: cannot read {text!r}") from None
    return text


def parse_args(argv):
    """(command, options dict, positional list).  Errors follow the reference's wording."""
    args = list(argv)
    if not args:
        raise CliError(USAGE)
    command = args.pop(0)
    if command in ("-h", "--help", "help"):
        return "help", {}, []
    if command not in OPTIONS:
        raise CliError(f"unknown command: {command}")
    spec, opts, positional = OPTIONS[command], {}, []
    while args:
        arg = args.pop(0)
        flag, eq, inline = arg.partition("=")
        if not arg.startswith("--"):
            if command == "dump":
                positional.append(arg)
                continue
            raise CliError(f"unknown argument: {arg}")
        if flag not in spec:
            raise CliError(f"unknown argument: {arg}")
        kind = spec[flag]
        if kind == "flag":
            if eq:
                raise CliError(f"{flag} takes no value")
            opts[flag] = True
            continue
        if eq:
            value = inline
        else:
            if not args or (args[0].startswith("--") and not kind.startswith("tokens")):
                raise CliError(f"{flag} requires a value")
            value = args.pop(0)
        if value == "":
            raise CliError(f"{flag} requires a value")
        value = _convert(kind, flag, value)
        if kind.endswith("+"):
            opts.setdefault(flag, []).append(value)
        elif flag in opts:
            raise CliError(f"{flag} specified more than once")
        else:
            opts[flag] = value
    return command, opts, positional


def _need(opts, flag):
    if flag not in opts:
        raise CliError(f"{flag} is required")
    return opts[flag]


def cmd_generate(opts):
    from .engine.api import Engine, SamplingParams
    model = _need(opts, "--model")
    prompts = list(opts.get("--prompt-tokens", []))
    if "--prompt-file" in opts:
        with open(opts["--prompt-file"]) as f:
            for line in f:
                if line.strip():
                    prompts.append(_convert("tokens", "--prompt-file", line.strip()))
    if not prompts:
        raise CliError("--prompt-tokens is required")
    kw = {}
    for flag, name in (("--page-size", "page_size"), ("--num-pages", "num_pages"), ("--max-batch-tokens", "max_batch_tokens"),
                       ("--max-batch-seqs", "max_batch_seqs"), ("--chunk-size", "chunk_size"),
                       ("--max-model-len", "max_model_len")):
        if flag in opts:
            kw[name] = opts[flag]
    eng = Engine(model, dtype=opts.get("--dtype", "bfloat16"), random_weights=bool(opts.get("--random-weights")),
                 seed=opts.get("--weights-seed", 0), profile=bool(opts.get("--profile")), **kw)
    sp = SamplingParams(opts.get("--temperature", 0.0), opts.get("--top-p", 1.0), opts.get("--seed", 0))
    ids = [eng.submit(p, opts.get("--max-new-tokens", 16), sp, opts.get("--stop-tokens", [])) for p in prompts]
    out, reasons = {i: [] for i in ids}, {}
    while len(reasons) < len(ids):
        for ev in eng.step():
            if ev.kind == "token":
                out[ev.id].append(ev.token)
            else:
                reasons[ev.id] = ev.reason
    for i in ids:
        print(json.dumps({"id": i, "tokens": out[i], "finish_reason": reasons[i]}))
    if opts.get("--stats"):
        print(json.dumps(eng.stats()), file=sys.stderr)
    if opts.get("--profile"):
        # per kernel: launches, milliseconds, share of the GPU time; products also GB/s, TFLOP/s, fraction of the roofline
        rows = eng.profile_report()
        print(f"{'kernel':24s} {'launches':>8s} {'ms':>10s} {'share':>7s} {'us/launch':>10s} {'GB/s':>9s} {'TFLOP/s':>9s} {'roofline':>9s}",
              file=sys.stderr)
        for r in rows:
            print(f"{r['kernel']:24s} {r['launches']:8d} {r['ms']:10.3f} {r['share'] * 100:6.1f}% {r['us_per_launch']:10.2f} "
                  f"{r.get('GBps', ''):>9} {r.get('TFLOPs', ''):>9} {r.get('frac_of_roofline', ''):>9}", file=sys.stderr)
    return 0


def cmd_random_weights(opts):
    from .weights import write_random_gguf, write_random_model
    with open(_need(opts, "--config")) as f:
        cfg = json.load(f)
    out = _need(opts, "--out")
    if opts.get("--gguf"):
        write_random_gguf(cfg, out, opts.get("--seed", 0), opts.get("--dtype", "float16"))
    else:
        write_random_model(cfg, out, opts.get("--seed", 0), opts.get("--dtype", "float32"))
    print(out)
    return 0


def cmd_bench(opts):
    """B random prompts of P tokens, N new tokens each, greedy, through the engine's own entry
    point: one JSON line with the time of the prompts (until every request has its first token)
    and the decoded tokens a second after that.  `--model` names a model folder, or with
    `--random-weights` a config.json whose sizes are built with random weights (`--layers`
    overrides its layer count, for shapes that would not fit otherwise)."""
    import random
    import time
    import torch
    from .config import registry
    from .engine.api import Engine, load_model, parse_dtype
    from .weights import init_random
    model_arg = _need(opts, "--model")
    dtype = opts.get("--dtype", "bfloat16")
    B, P, N = opts.get("--batch", 8), opts.get("--prompt-len", 128), opts.get("--new-tokens", 64)
    if min(B, P, N) < 1:
        raise CliError("--batch, --prompt-len and --new-tokens must be positive")
    page = opts.get("--page-size", 16)
    max_len = P + N + page
    if opts.get("--random-weights"):
        path = os.path.join(model_arg, "config.json") if os.path.isdir(model_arg) else model_arg
        with open(path) as f:
            cfgd = json.load(f)
        if "--layers" in opts:
            cfgd["num_hidden_layers"] = opts["--layers"]
        arch = registry.lookup(cfgd["architectures"][0])
        model = arch.build(arch.read_config(cfgd), parse_dtype(dtype), "cuda", max_positions=max_len)
        init_random(model, opts.get("--seed", 0))
    else:
        model, _ = load_model(model_arg, dtype, max_positions=max_len)
    eng = Engine(model=model, page_size=page, num_pages=B * (-(-max_len // page)), max_batch_tokens=max(2048, B),
                 max_batch_seqs=B, chunk_size=opts.get("--chunk-size", 0), max_model_len=max_len)
    rng = random.Random(opts.get("--seed", 0))
    vocab = model.n_vocab
    for rep in range(2):                       # the first run captures the decode graphs
        ids = [eng.submit([rng.randrange(vocab) for _ in range(P)], N) for _ in range(B)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first, done, t_first, tokens = set(), 0, None, 0
        while done < B:
            for ev in eng.step():
                if ev.kind == "token":
                    tokens += 1
                    first.add(ev.id)
                else:
                    done += 1
            if t_first is None and len(first) == B:
                t_first = time.perf_counter()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    decoded = tokens - B
    print(json.dumps({"batch": B, "prompt_len": P, "new_tokens": N, "dtype": dtype, "layers": len(model.blocks),
                      "prompt_ms": round((t_first - t0) * 1e3, 3), "prompt_tok_s": round(B * P / (t_first - t0), 1),
                      "decode_tok_s": round(decoded / (t1 - t_first), 1) if decoded and t1 > t_first else None,
                      "total_s": round(t1 - t0, 4)}))
    return 0


def cmd_replay(opts):
    from .engine.trace import TraceSession
    s = TraceSession(_need(opts, "--model"), _need(opts, "--dtype"), _need(opts, "--max-tokens"),
                     opts.get("--page-size", 16), opts.get("--max-requests", 8))
    s.run_stream(sys.stdin, _need(opts, "--out"), sys.stdout)
    return 0


def cmd_dump(positional):
    if len(positional) != 1:
        raise CliError("usage: ferrum dump FILE.gguf|FILE.safetensors|DIR")
    path = positional[0]
    if path.endswith(".gguf"):
        from .weights.gguf_io import GGUFFile
        sys.stdout.write(GGUFFile(path).dump())
        return 0
    from .weights.loader import open_source
    src = open_source(path)
    print(f"ferrum-safetensors tensors={len(src.entries)}")
    for name, (shape, dtype, _) in src.entries.items():
        print(f"{name} [{', '.join(str(d) for d in shape)}] {str(dtype).replace('torch.', '')}")
    return 0


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    try:
        command, opts, positional = parse_args(argv)
    except CliError as e:
        print(f"ferrum: {e}", file=sys.stderr)
        return 2
    try:
        if command == "help":
            print(__doc__)
            return 0
        if command == "serve":
            # crates/ferrum-cli/src/main.rs:17-20 answers `serve` without --mock the same way
            print("ferrum: the HTTP server is not part of this engine; use `ferrum generate` or the Python API",
                  file=sys.stderr)
            return 1
        if command == "generate":
            return cmd_generate(opts)
        if command == "random-weights":
            return cmd_random_weights(opts)
        if command == "bench":
            return cmd_bench(opts)
        if command == "replay":
            return cmd_replay(opts)
        return cmd_dump(positional)
    except CliError as e:
        print(f"ferrum: {e}", file=sys.stderr)
        return 2
    except Exception as e:                      # runtime errors: exit 1, one line
        print(f"ferrum: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
