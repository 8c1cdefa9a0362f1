"""The engine against the plain implementation, under every way of cutting the work."""
import numpy as np
import pytest

from helpers import Replay, assert_close, plain_logits, random_tokens
from conftest import TINY

pytestmark = pytest.mark.gpu

CASES = [(m, d) for m in ("A", "B", "C", "D") for d in ("float32", "bfloat16")]


def session(model_dirs, name, dtype, max_tokens, **kw):
    from ferrum_b200.engine.trace import TraceSession
    return TraceSession(model_dirs[name], dtype, max_tokens, **kw)


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt(cuda, model_dirs, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    toks = random_tokens(97, vocab, 10)
    r = Replay(session(model_dirs, name, dtype, 128))
    r.step([("a", toks, "all")], end=["a"])
    assert_close(r.logits("a", len(toks)), plain_logits(model_dirs[name], dtype, toks), dtype, f"{name} whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens(cuda, model_dirs, name, dtype):
    """A sequence's first tokens: one token alone, then two, each as a step of its own."""
    vocab = TINY[name][0]["vocab_size"]
    toks = random_tokens(3, vocab, 11)
    r = Replay(session(model_dirs, name, dtype, 64))
    r.step([("a", toks[:1], "all")])
    r.step([("a", toks[1:3], "all")], end=["a"])
    assert_close(r.logits("a", 3), plain_logits(model_dirs[name], dtype, toks), dtype, f"{name} first tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_decode_one_by_one(cuda, model_dirs, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    toks = random_tokens(120, vocab, 12)
    ref = plain_logits(model_dirs[name], dtype, toks)
    r = Replay(session(model_dirs, name, dtype, 128))
    r.step([("a", toks[:-32], "all")])
    for t in toks[-32:]:
        r.step([("a", [t], "all")])
    assert_close(r.logits("a", len(toks)), ref, dtype, f"{name} prefill+decode")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(cuda, model_dirs, name, dtype):
    vocab = TINY[name][0]["vocab_size"]
    toks = random_tokens(150, vocab, 13)
    ref = plain_logits(model_dirs[name], dtype, toks)
    r = Replay(session(model_dirs, name, dtype, 192))
    sizes, i, k = [5, 2, 7, 3, 2, 16, 17, 2, 31, 1, 33, 2], 0, 0
    while i < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - i)
        r.step([("a", toks[i:i + n], "all")])
        i += n
        k += 1
    assert_close(r.logits("a", len(toks)), ref, dtype, f"{name} portions")


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_page_reuse(cuda, model_dirs, name, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool
    so small that pages freed by finished requests are used again by later ones."""
    vocab = TINY[name][0]["vocab_size"]
    lens = {"a": 70, "b": 45, "c": 33, "d": 90, "e": 50, "f": 21}
    toks = {k: random_tokens(n, vocab, 20 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: plain_logits(model_dirs[name], dtype, v) for k, v in toks.items()}
    # a+b+c+d rounded up to 64 each = 128+64+64+128 = 384 tokens live at most
    s = session(model_dirs, name, dtype, 384)
    r = Replay(s)
    cur = {k: 0 for k in toks}

    def take(k, n):
        out = toks[k][cur[k]:cur[k] + n]
        cur[k] += len(out)
        return out

    def done(k):
        return cur[k] >= len(toks[k])

    live, waiting, step = ["a", "b", "c", "d"], ["e", "f"], 0
    pattern = {0: [7, 1, 2, 13], 1: [1, 5, 1, 2], 2: [16, 1, 3, 1], 3: [2, 2, 1, 30]}
    seen_pages = set()
    while live:
        sizes = pattern[step % 4]
        entries, ended = [], []
        for j, k in enumerate(list(live)):
            if step % 5 == 4 and j == 1:
                continue                      # a request may sit out a step and go on later
            part = take(k, sizes[j % 4])
            if part:
                entries.append((k, part, "all"))
            if done(k):
                ended.append(k)
        r.step(entries, end=ended)
        for k in live:
            if k in s.slots:
                seen_pages.update(p for p in s.cache.manager.table(0, s.slots[k]) if p >= 0)
        for k in ended:
            live.remove(k)
            if waiting:
                live.append(waiting.pop(0))
        step += 1
        assert s.cache.manager.check() == ""
    for k in toks:
        assert_close(r.logits(k, len(toks[k])), ref[k], dtype, f"{name} mixed {k}")
    assert s.cache.manager.used_pages(0) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_model_with_many_tokens_per_step(cuda, model_dirs, dtype):
    """A model wide enough (1024 features, head size 128) and steps long enough for the kernels
    that the tiny configurations never reach: products of 300 to 400 tokens on CTA pairs, cut
    across several CTAs; products of 200 tokens whose reduction is left to the next kernel;
    tcgen05 attention over several work items, with and without history; decoded tokens of one
    request beside a prompt portion of another."""
    from conftest import MID_E
    vocab = MID_E["vocab_size"]
    a, b = random_tokens(730, vocab, 31), random_tokens(215, vocab, 32)
    r = Replay(session(model_dirs, "E", dtype, 1152))
    r.step([("a", a[:400], "all")])
    r.step([("a", a[400:700], "all")])
    r.step([("a", a[700:701], "all"), ("b", b[:200], "all")])
    for i in range(15):
        r.step([("a", a[701 + i:702 + i], "all"), ("b", b[200 + i:201 + i], "all")])
    r.step([("a", a[716:730], "all")], end=["a", "b"])
    assert_close(r.logits("a", len(a)), plain_logits(model_dirs["E"], dtype, a), dtype, "wide a")
    assert_close(r.logits("b", len(b)), plain_logits(model_dirs["E"], dtype, b), dtype, "wide b")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(cuda, model_dirs, dtype):
    """Several hundred tokens one by one: many pages, many page edges."""
    vocab = TINY["C"][0]["vocab_size"]
    toks = random_tokens(300, vocab, 14)
    ref = plain_logits(model_dirs["C"], dtype, toks)
    r = Replay(session(model_dirs, "C", dtype, 320))
    r.step([("a", toks[:4], "all")])
    for t in toks[4:]:
        r.step([("a", [t], "all")])
    assert_close(r.logits("a", len(toks)), ref, dtype, "long decode")


def test_split_invariance_float32(cuda, model_dirs):
    """In float32 the ways of cutting agree with each other far more tightly than with the
    plain implementation: the kernels reduce in an order that does not depend on the batch."""
    vocab = TINY["A"][0]["vocab_size"]
    toks = random_tokens(80, vocab, 15)
    r1 = Replay(session(model_dirs, "A", "float32", 128))
    r1.step([("a", toks, "all")])
    r2 = Replay(session(model_dirs, "A", "float32", 128))
    for i in range(0, 80, 3):
        r2.step([("a", toks[i:i + 3], "all")])
    d = np.abs(r1.logits("a", 80) - r2.logits("a", 80)).max()
    assert d <= 2e-6, d


def test_trace_run_program(cuda, model_dirs, tmp_path):
    """bin/trace_run as a user runs it: a subprocess, JSON lines in, .f32 files out."""
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = random_tokens(40, TINY["A"][0]["vocab_size"], 16)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:], "want": []}], "end": []},
             {"step": 2, "entries": [], "end": ["x"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dirs["A"], "--dtype",
                        "float32", "--out", str(out), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    got = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    ref = plain_logits(model_dirs["A"], "float32", toks[:30])
    assert_close(got, ref[[0, 29]], "float32", "trace_run")
    assert not (out / "1.f32").exists()


@pytest.mark.parametrize("name", ["B", "D"])
def test_decode_graph_replay_matches_kernel_launches(cuda, model_dirs, name):
    """Decode steps replayed from a captured CUDA graph give the logits that the same steps
    give when launched kernel by kernel, while requests grow across page and split edges."""
    vocab = TINY[name][0]["vocab_size"]
    toks = {k: random_tokens(170, vocab, 30 + i) for i, k in enumerate("abc")}
    outs = []
    for graphs in (False, True):
        s = session(model_dirs, name, "bfloat16", 3 * 192)
        s.runner.use_graphs = graphs
        r = Replay(s)
        r.step([(k, toks[k][:40 + 7 * i], []) for i, k in enumerate("abc")])
        cur = {k: 40 + 7 * i for i, k in enumerate("abc")}
        for _ in range(100):
            r.step([(k, [toks[k][cur[k]]], "all") for k in "abc"])
            for k in "abc":
                cur[k] += 1
        assert (s.runner.graph_replays > 90) == graphs
        outs.append(np.stack([r.rows[(k, p)] for k in "abc" for p in range(40 + 7 * "abc".index(k), 140)]))
    assert np.abs(outs[0] - outs[1]).max() <= 1e-6
    ref = plain_logits(model_dirs[name], "bfloat16", toks["a"][:140])
    got = np.stack([r.rows[("a", p)] for p in range(40, 140)])
    assert_close(got, ref[40:140], "bfloat16", "graph decode")
