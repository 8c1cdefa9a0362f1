"""Generation through the Python entry point against the plain implementation."""
import numpy as np
import pytest

import plain_llama as P
from conftest import TINY
from helpers import random_tokens

pytestmark = pytest.mark.gpu


def engine(model_dirs, name, dtype, **kw):
    from ferrum_b200 import Engine
    args = dict(dtype=dtype, num_pages=64, max_batch_tokens=64, max_batch_seqs=4, max_model_len=256)
    args.update(kw)
    return Engine(model_dirs[name], **args)


def check_against_plain(folder, dtype, prompt, got, temperature=0.0, seed=0):
    """Token by token, teacher-forced on the engine's own tokens.  In float32 every token equals
    the plain implementation's.  In a 16-bit dtype a greedy token may differ only where the plain
    logits have a near-tie: the margin between the plain top-1 and the engine's choice is within
    twice the logit bound of helpers.C_16BIT (either logit may move by the bound).  The comparison
    goes on after such a flip, with the engine's token in the context.  Returns the number of
    tokens that were equal."""
    from helpers import C_16BIT, round_to
    cfg, w = P.read_model(folder, weights_as=round_to(dtype))
    toks = list(prompt)
    same = 0
    for n, t in enumerate(got):
        logits = P.forward(cfg, w, toks)[-1]
        want = P.sample(logits, temperature, seed, n)
        if t == want:
            same += 1
        else:
            assert dtype != "float32" and temperature == 0.0, (n, t, want)
            margin = logits.max() - logits[t]
            assert margin <= 2 * C_16BIT[dtype] * logits.std(), (n, t, want, margin, logits.std())
        toks.append(t)
    return same


@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_greedy_generation(cuda, model_dirs, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    prompt = random_tokens(16, vocab, 40)
    eng = engine(model_dirs, name, dtype)
    got = eng.generate([prompt], max_new_tokens=16)[0]
    assert len(got) == 16
    same = check_against_plain(model_dirs[name], dtype, prompt, got)
    assert same == 16 or dtype != "float32"
    assert same >= 14, same           # near-ties are rare: most tokens are simply equal


def test_temperature_generation_float32(cuda, model_dirs):
    vocab = TINY["B"][0]["vocab_size"]
    prompt = random_tokens(7, vocab, 41)
    eng = engine(model_dirs, "B", "float32")
    got = eng.generate([prompt], max_new_tokens=12, temperature=0.8, seed=1)[0]
    assert check_against_plain(model_dirs["B"], "float32", prompt, got, 0.8, 1) == 12
    again = engine(model_dirs, "B", "float32").generate([prompt], max_new_tokens=12, temperature=0.8, seed=1)[0]
    other = engine(model_dirs, "B", "float32").generate([prompt], max_new_tokens=12, temperature=0.8, seed=2)[0]
    assert again == got and other != got


def test_continuous_batching_gives_each_request_what_it_gets_alone(cuda, model_dirs):
    """The mixed workload of the second tiny configuration: prompts of 7, 33 and 1 tokens,
    portions of 8, greedy and temperature 0.8 with seed 1 side by side."""
    vocab = TINY["B"][0]["vocab_size"]
    prompts = [random_tokens(n, vocab, 50 + n) for n in (7, 33, 1)]
    alone = []
    for i, p in enumerate(prompts):
        t = 0.8 if i == 1 else 0.0
        alone.append(engine(model_dirs, "B", "float32").generate([p], max_new_tokens=10, temperature=t, seed=1)[0])
    from ferrum_b200 import SamplingParams
    eng = engine(model_dirs, "B", "float32", chunk_size=8, max_batch_tokens=12)
    ids = [eng.submit(p, 10, SamplingParams(0.8 if i == 1 else 0.0, 1.0, 1)) for i, p in enumerate(prompts)]
    out = {i: [] for i in ids}
    reasons = {}
    while len(reasons) < 3:
        for ev in eng.step():
            if ev.kind == "token":
                out[ev.id].append(ev.token)
            else:
                reasons[ev.id] = ev.reason
    assert [out[i] for i in ids] == alone
    assert set(reasons.values()) == {"length"}
    st = eng.stats()
    assert st["pages_used"] == [0] and st["finished"] == 3 and st["prompt_tokens"] == 41


def test_preemption_in_the_engine_keeps_outputs(cuda, model_dirs):
    """So few pages that two decoding requests cannot both stay: one is preempted and
    recomputed, and both still produce what they produce alone."""
    vocab = TINY["A"][0]["vocab_size"]
    prompts = [random_tokens(20, vocab, 60), random_tokens(20, vocab, 61)]
    alone = [engine(model_dirs, "A", "float32").generate([p], max_new_tokens=40)[0] for p in prompts]
    eng = engine(model_dirs, "A", "float32", num_pages=6, max_model_len=64)      # 96 tokens of cache, 120 needed
    assert eng.generate(prompts, max_new_tokens=40) == alone
    assert eng.stats()["preemptions"] >= 1 and eng.stats()["pages_used"] == [0]


def test_stop_tokens_cancel_and_errors(cuda, model_dirs):
    from ferrum_b200 import InvalidRequest, NotFound
    vocab = TINY["A"][0]["vocab_size"]
    prompt = random_tokens(9, vocab, 62)
    eng = engine(model_dirs, "A", "float32")
    free = eng.generate([prompt], max_new_tokens=8)[0]
    stopped = eng.generate([prompt], max_new_tokens=8, stop_tokens=[free[3]])[0]
    assert stopped == free[:free.index(free[3]) + 1]                 # the stopping token is emitted
    with pytest.raises(InvalidRequest):
        eng.submit([], 4)
    with pytest.raises(InvalidRequest):
        eng.submit([vocab], 4)
    rid = eng.submit(prompt, 50)
    eng.step()
    eng.cancel(rid)
    with pytest.raises(NotFound):
        eng.cancel(rid)
    assert eng.step() == [] and eng.stats()["pages_used"] == [0]


def test_missing_extension_or_device_fails_loudly(cuda, monkeypatch):
    import torch
    from ferrum_b200 import KernelError
    from ferrum_b200.ops import lib
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(KernelError, match="CUDA device only"):
        lib.require_cuda()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_steps_queued_ahead_change_nothing(cuda, model_dirs, dtype):
    """The engine queues the next decode step before it has read the current one's tokens (the
    ids go from the sampling kernel to the next step on the device).  Same tokens, same finish
    reasons as with one step at a time: greedy and temperature rows, a request that stops on a
    token (its row of the step already queued is computed for nothing), one cancelled in flight."""
    from ferrum_b200 import SamplingParams
    vocab = TINY["D"][0]["vocab_size"]
    prompts = [random_tokens(n, vocab, 70 + n) for n in (5, 19, 2, 11)]
    probe = engine(model_dirs, "D", dtype, plan_ahead=False).generate([prompts[2]], max_new_tokens=12)[0]

    def run(ahead):
        eng = engine(model_dirs, "D", dtype, plan_ahead=ahead)
        ids = [eng.submit(p, 12, SamplingParams(0.7 if i == 1 else 0.0, 1.0, 3), stop_tokens=[probe[5]] if i == 2 else [])
               for i, p in enumerate(prompts)]
        out, reasons, steps = {i: [] for i in ids}, {}, 0
        while len(reasons) < 3:
            for ev in eng.step():
                if ev.kind == "token":
                    out[ev.id].append(ev.token)
                else:
                    reasons[ev.id] = ev.reason
            steps += 1
            if steps == 4:
                eng.cancel(ids[3])
            assert steps < 100
        while eng.step():
            pass
        assert eng.stats()["pages_used"] == [0] and eng.stats()["active"] == 0
        return [out[i] for i in ids[:3]], reasons

    one_by_one, r0 = run(False)
    queued, r1 = run(True)
    assert queued == one_by_one and r0 == r1
    assert one_by_one[2] == probe[:probe.index(probe[5]) + 1] and r0[2] == "stop"


def test_profile_mode_times_every_kernel(cuda, model_dirs):
    """Engine(profile=True): every launch is timed on its own (no CUDA graphs, one step at a time);
    the report has one row per kernel, the shares add up, the products report their rates, and the
    tokens are those of an ordinary engine."""
    vocab = TINY["D"][0]["vocab_size"]
    prompt = random_tokens(40, vocab, 95)
    want = engine(model_dirs, "D", "bfloat16").generate([prompt], max_new_tokens=6)[0]
    eng = engine(model_dirs, "D", "bfloat16", profile=True)
    assert eng.generate([prompt], max_new_tokens=6) == [want]
    rows = eng.profile_report()
    names = {r["kernel"] for r in rows}
    assert {"rmsnorm", "rope_cache_write", "sample"} <= names and any(n.startswith("gemm_tc") for n in names), names
    assert abs(sum(r["share"] for r in rows) - 1.0) < 0.01 and all(r["ms"] >= 0 and r["launches"] > 0 for r in rows)
    gemm = next(r for r in rows if r["kernel"].startswith("gemm_tc"))
    assert gemm["GBps"] > 0 and gemm["TFLOPs"] > 0
    assert eng.runner.graph_replays == 0 and eng.profile_report() == []


def test_step_raw_is_the_step_function_below_the_scheduler(cuda, model_dirs):
    """Engine.step_raw runs given entries on slots of the engine's own cache and returns logits;
    it refuses while requests are in flight."""
    import torch
    from ferrum_b200.engine import StepEntry
    vocab = TINY["A"][0]["vocab_size"]
    toks = random_tokens(20, vocab, 90)
    eng = engine(model_dirs, "A", "float32")
    slot = eng.cache.open()
    a = eng.step_raw([StepEntry(slot, 0, toks[:13], [12])])
    b = eng.step_raw([StepEntry(slot, 13, toks[13:], list(range(7)))])
    eng.cache.close(slot)
    got = torch.cat([a[:1], b[:7]]).cpu().numpy()
    cfg, w = P.read_model(model_dirs["A"])
    ref = P.forward(cfg, w, toks)[12:]
    from helpers import assert_close
    assert_close(got, ref, "float32", "step_raw")
    eng.submit(toks, 2)
    with pytest.raises(RuntimeError, match="in flight"):
        eng.step_raw([])
    assert eng.generate([toks], max_new_tokens=2)


def test_bench_command(cuda, tmp_path):
    import json, os, subprocess, sys
    from conftest import ROOT, TINY_D
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_D))
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ferrum"), "bench", "--model", str(cfg), "--random-weights",
                        "--batch", "3", "--prompt-len", "40", "--new-tokens", "6", "--dtype", "bfloat16"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["batch"] == 3 and line["decode_tok_s"] > 0 and line["prompt_tok_s"] > 0
