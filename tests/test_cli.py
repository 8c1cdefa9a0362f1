"""The command line: argument errors and exit codes in the reference's manner
(crates/ferrum-cli/tests/cli.rs), and the commands that need no GPU."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT, TINY_A, TINY_B

FERRUM = [sys.executable, os.path.join(ROOT, "bin", "ferrum")]


def ferrum(*args, stdin=None):
    return subprocess.run(FERRUM + list(args), capture_output=True, text=True, input=stdin, timeout=600)


def test_missing_command_is_usage():
    p = ferrum()
    assert p.returncode == 2 and "usage: ferrum" in p.stderr


def test_unknown_command_and_argument():
    p = ferrum("bake")
    assert p.returncode == 2 and "unknown command: bake" in p.stderr
    p = ferrum("generate", "--model", "x", "--wat")
    assert p.returncode == 2 and "unknown argument: --wat" in p.stderr


def test_value_errors():
    from ferrum_b200.cli import CliError, parse_args
    with pytest.raises(CliError, match="--model requires a value"):
        parse_args(["generate", "--model"])
    with pytest.raises(CliError, match="--model requires a value"):
        parse_args(["generate", "--model", "--dtype", "float32"])
    with pytest.raises(CliError, match="--model specified more than once"):
        parse_args(["generate", "--model", "a", "--model=b"])
    with pytest.raises(CliError, match="cannot read"):
        parse_args(["generate", "--max-new-tokens", "many"])
    cmd, opts, _ = parse_args(["generate", "--model=m", "--prompt-tokens", "1,2,3", "--prompt-tokens=4", "--temperature",
                               "0.8", "--stats"])
    assert cmd == "generate" and opts == {"--model": "m", "--prompt-tokens": [[1, 2, 3], [4]], "--temperature": 0.8,
                                          "--stats": True}


def test_bench_options_parse():
    from ferrum_b200.cli import CliError, parse_args
    cmd, opts, _ = parse_args(["bench", "--model", "cfg.json", "--random-weights", "--batch=4", "--prompt-len", "32",
                               "--new-tokens", "8", "--layers", "2"])
    assert cmd == "bench" and opts == {"--model": "cfg.json", "--random-weights": True, "--batch": 4, "--prompt-len": 32,
                                       "--new-tokens": 8, "--layers": 2}
    with pytest.raises(CliError, match="unknown argument: --prompt-tokens"):
        parse_args(["bench", "--model", "m", "--prompt-tokens", "1,2"])
    p = ferrum("bench")
    assert p.returncode == 2 and "--model is required" in p.stderr


def test_serve_names_the_missing_server():
    p = ferrum("serve")
    assert p.returncode == 1 and "not part of this engine" in p.stderr


def test_random_weights_and_dump(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    p = ferrum("random-weights", "--config", str(cfg), "--out", str(out), "--seed", "1", "--dtype", "bfloat16")
    assert p.returncode == 0, p.stderr
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    p = ferrum("dump", str(out))
    assert p.returncode == 0 and "model.layers.2.mlp.down_proj.weight [96, 256] bfloat16" in p.stdout
    g = tmp_path / "b.gguf"
    p = ferrum("random-weights", "--config", str(cfg), "--out", str(g), "--seed", "1", "--gguf")
    assert p.returncode == 0, p.stderr
    p = ferrum("dump", str(g))
    lines = p.stdout.splitlines()
    assert lines[0].startswith("ferrum-gguf version=3 alignment=32 metadata=") and lines[0].endswith("tensors=29")
    assert "blk.0.attn_q.weight [96, 96] F16" in lines and "token_embd.weight [96, 512] F16" in lines
    p = ferrum("dump", str(tmp_path / "nope.gguf"))
    assert p.returncode == 1 and p.stderr.startswith("ferrum: ")


@pytest.mark.gpu
def test_generate_command(cuda, model_dirs):
    p = ferrum("generate", "--model", model_dirs["A"], "--dtype", "float32", "--prompt-tokens", "5,17,3",
               "--prompt-tokens", "9,9", "--max-new-tokens", "4", "--num-pages", "16", "--max-model-len", "64",
               "--stats")
    assert p.returncode == 0, p.stderr
    recs = [json.loads(l) for l in p.stdout.splitlines()]
    assert [len(r["tokens"]) for r in recs] == [4, 4] and recs[0]["finish_reason"] == "length"
    import plain_llama as P
    cfg, w = P.read_model(model_dirs["A"])
    assert recs[0]["tokens"] == P.generate(cfg, w, [5, 17, 3], 4)
    assert json.loads(p.stderr.strip().splitlines()[-1])["finished"] == 2
    p = ferrum("generate", "--model", model_dirs["A"], "--prompt-tokens", "999")
    assert p.returncode == 1 and "vocabulary" in p.stderr


def test_interface_revision_names_this_surface():
    """The public surface that INTERFACE_REVISION stands for: a change here is a change of the number."""
    import inspect
    import ferrum_b200
    from ferrum_b200 import cli
    from ferrum_b200.engine import api
    from ferrum_b200.parts import base
    assert ferrum_b200.INTERFACE_REVISION == 2
    methods = sorted(n for n, _ in inspect.getmembers(api.Engine, inspect.isfunction) if not n.startswith("_"))
    assert methods == ["cancel", "generate", "profile_report", "stats", "step", "step_raw", "submit"]
    assert list(inspect.signature(api.Engine.submit).parameters)[1:6] == ["prompt_tokens", "max_new_tokens", "sampling",
                                                                           "stop_tokens", "request_id"]
    assert sorted(cli.OPTIONS) == ["bench", "dump", "generate", "random-weights", "replay", "serve"]
    assert {"--model", "--prompt-tokens", "--dtype", "--max-new-tokens", "--temperature", "--seed", "--stop-tokens",
            "--max-batch-tokens", "--chunk-size", "--page-size", "--num-pages", "--max-model-len"} <= set(cli.OPTIONS["generate"])
    for cls, names in ((base.Mixer, ["param_specs", "cache_need", "forward", "plan"]), (base.FeedForward, ["param_specs", "forward"]),
                       (base.Norm, ["param_specs", "forward"]), (base.PositionEncoding, ["param_specs", "rotary", "on_embedding"])):
        for n in names:
            assert hasattr(cls, n), (cls.__name__, n)
