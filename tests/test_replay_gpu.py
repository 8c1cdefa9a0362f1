"""The engine against the plain implementation, under every way of cutting the work."""
import numpy as np
import pytest

from helpers import Replay, assert_close, mixed_case, pages_were_reused, plain_logits, random_tokens, run_mixed
from conftest import TINY

pytestmark = pytest.mark.gpu

CASES = [(m, d) for m in ("A", "B", "C", "D") for d in ("float32", "bfloat16", "float16")]


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
    smaller than the requests need together: a page freed by a finished request is held by a later one."""
    s, toks, schedule = mixed_case(model_dirs, name, dtype)
    r, owners = run_mixed(s, toks, schedule)
    assert pages_were_reused(owners), "no page was ever held by two requests"
    # the held pages were the whole pool at the peak (the sequence of tokens after a wait sees a reused page)
    assert len(owners) == s.cache.manager.free_pages(0)
    for k in toks:
        assert_close(r.logits(k, len(toks[k])), plain_logits(model_dirs[name], dtype, toks[k]), dtype, f"{name} mixed {k}")
    assert s.cache.manager.used_pages(0) == 0


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("A", "bfloat16"), ("G", "float32")])
def test_tokens_of_a_request_share_key_tiles(cuda, model_dirs, name, dtype, monkeypatch):
    """The CUDA-core attention's kernel for steps of many tokens (up to eight tokens of a request
    per CTA, found on the device from the requests' token offsets), forced on every step of the
    mixed workload and of portions of changing size: chunks that end inside a request, requests of
    one decoded token beside portions, windows."""
    from ferrum_b200.parts import attention
    monkeypatch.setattr(attention, "GENERIC_SPLIT_BELOW", 0)
    s, toks, schedule = mixed_case(model_dirs, name, dtype)
    r, owners = run_mixed(s, toks, schedule)
    for k in toks:
        assert_close(r.logits(k, len(toks[k])), plain_logits(model_dirs[name], dtype, toks[k]), dtype, f"{name} token tiles {k}")
    import conftest
    vocab = getattr(conftest, "TINY_" + name)["vocab_size"]
    long = random_tokens(150, vocab, 21)
    r = Replay(session(model_dirs, name, dtype, 192))
    sizes, i, k = [9, 8, 17, 1, 2, 31, 16, 7, 40, 3], 0, 0
    while i < len(long):
        n = min(sizes[k % len(sizes)], len(long) - i)
        r.step([("a", long[i:i + n], "all")])
        i += n
        k += 1
    assert_close(r.logits("a", len(long)), plain_logits(model_dirs[name], dtype, long), dtype, f"{name} token tiles, portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("page_size", [8, 32])
def test_other_page_sizes_through_a_whole_model(cuda, model_dirs, dtype, page_size):
    """Pages of 8 and of 32 positions (the tensor-core kernels' gather, the rotary kernel's
    page arithmetic) under the mixed workload and under portions, on the configuration that runs
    the tensor-core kernels."""
    s, toks, schedule = mixed_case(model_dirs, "D", dtype, page_size=page_size)
    r, owners = run_mixed(s, toks, schedule)
    assert pages_were_reused(owners)
    for k in toks:
        assert_close(r.logits(k, len(toks[k])), plain_logits(model_dirs["D"], dtype, toks[k]), dtype, f"page {page_size} {k}")
    long = random_tokens(330, TINY["D"][0]["vocab_size"], 77)
    r = Replay(session(model_dirs, "D", dtype, 352, page_size=page_size))
    r.step([("a", long[:290], "all")])
    for i in range(290, 330, 3):
        r.step([("a", long[i:i + 3], "all")])
    assert_close(r.logits("a", 330), plain_logits(model_dirs["D"], dtype, long), dtype, f"page {page_size} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wrong_page_index_is_caught(cuda, model_dirs, dtype, monkeypatch):
    """The comparisons above can fail: with one entry of one block table off by one on the host
    (still a page of the pool, so nothing faults) for the second half of the run, a request
    reads another page's keys and its logits leave the tolerance."""
    import ctypes
    from ferrum_b200 import host
    s, toks, schedule = mixed_case(model_dirs, "D", dtype)
    n_pages = s.cache.manager.free_pages(0)
    real = host.module().copy_tables
    calls = {"n": 0}

    def off_by_one(cache, group, slots, dst, row_stride):
        real(cache, group, slots, dst, row_stride)
        calls["n"] += 1
        row = (ctypes.c_int32 * row_stride).from_address(dst)          # the first request's table row
        if calls["n"] > len(schedule) // 2 and row[0] >= 0 and cache.seq_len(slots[0]) >= 16:
            row[0] = (row[0] + 1) % n_pages

    monkeypatch.setattr(host.module(), "copy_tables", off_by_one)
    r, _ = run_mixed(s, toks, schedule)
    with pytest.raises(AssertionError):
        for k in toks:
            assert_close(r.logits(k, len(toks[k])), plain_logits(model_dirs["D"], dtype, toks[k]), dtype, f"mutated {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_many_query_heads_on_one_kv_head(cuda, model_dirs, dtype):
    """32 query heads share one KV head: a decoded token brings 32 rows, twice what the 16-row
    tile of the tensor-core kernel takes, so decoding runs on the 64-row class and without a
    CUDA graph.  Decodes well past the step at which a graph would have been captured."""
    from conftest import TINY_G
    toks = random_tokens(100, TINY_G["vocab_size"], 78)
    s = session(model_dirs, "G", dtype, 128)
    assert not s.runner.use_graphs or dtype == "float32"
    r = Replay(s)
    r.step([("a", toks[:70], "all")])
    for t in toks[70:]:
        r.step([("a", [t], "all")])
    assert_close(r.logits("a", 100), plain_logits(model_dirs["G"], dtype, toks), dtype, "32 heads per kv head")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
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


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_decode_graph_replay_matches_kernel_launches(cuda, model_dirs, name, dtype):
    """Decode steps replayed from a captured CUDA graph give the logits that the same steps
    give when launched kernel by kernel, while requests grow across page and split edges."""
    vocab = TINY[name][0]["vocab_size"]
    toks = {k: random_tokens(170, vocab, 30 + i) for i, k in enumerate("abc")}
    outs = []
    for graphs in (False, True):
        s = session(model_dirs, name, dtype, 3 * 192)
        s.runner.use_graphs = graphs
        r = Replay(s)
        r.step([(k, toks[k][:40 + 7 * i], []) for i, k in enumerate("abc")])
        cur = {k: 40 + 7 * i for i, k in enumerate("abc")}
        for _ in range(100):
            r.step([(k, [toks[k][cur[k]]], "all") for k in "abc"])
            for k in "abc":
                cur[k] += 1
        assert (s.runner.graph_replays > 90) == (graphs and s.runner.use_graphs)
        outs.append(np.stack([r.rows[(k, p)] for k in "abc" for p in range(40 + 7 * "abc".index(k), 140)]))
    assert np.abs(outs[0] - outs[1]).max() <= 1e-6
    ref = plain_logits(model_dirs[name], dtype, toks["a"][:140])
    got = np.stack([r.rows[("a", p)] for p in range(40, 140)])
    assert_close(got, ref[40:140], dtype, "graph decode")


@pytest.fixture(scope="module")
def wide_layer(tmp_path_factory):
    """One layer at the widths of Llama-3.1-8B (4096 features, 32 query heads on 8 KV heads of 128,
    14336 hidden features), a small vocabulary; stored in bfloat16."""
    from ferrum_b200.weights import write_random_model
    cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 1, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 257, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}
    d = tmp_path_factory.mktemp("wide_layer")
    write_random_model(cfg, str(d), 9, dtype="bfloat16")
    toks = random_tokens(64, cfg["vocab_size"], 80)
    import plain_llama as P
    cfg_p, w = P.read_model(str(d))                    # bfloat16 values, exact in every compute dtype but float16
    return str(d), toks, P.forward(cfg_p, w, toks)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_at_the_widths_of_the_8b_model(cuda, wide_layer, dtype):
    """The products at their real sizes (reductions over 4096 and 14336 elements) against the plain
    implementation: 64 tokens, the first 40 in one step, then portions and single tokens.  In
    float32 the bound is the reference's for reductions longer than 4096 (relative 1e-3,
    docs/ARCHITECTURE.md:142-153); the engine is in fact far inside it."""
    from ferrum_b200.engine.trace import TraceSession
    folder, toks, ref = wide_layer
    r = Replay(TraceSession(folder, dtype, 64))
    r.step([("a", toks[:40], "all")])
    r.step([("a", toks[40:57], "all")])
    for t in toks[57:]:
        r.step([("a", [t], "all")])
    got = r.logits("a", 64)
    if dtype == "float32":
        lim = np.maximum(1e-6, 1e-3 * np.maximum(1.0, np.abs(ref)))
        assert np.isfinite(got).all() and (np.abs(got - ref) <= lim).all(), np.abs(got - ref).max()
        assert np.abs(got - ref).max() <= 2e-5, np.abs(got - ref).max()        # what float32 sums of this length give
        assert (got.argmax(-1) == ref.argmax(-1)).mean() >= 0.99
    else:
        assert_close(got, ref, dtype, "8b widths")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("D", "bfloat16"), ("D", "float16"), ("D", "float32")])
def test_no_kernel_writes_past_its_scratch_buffers(cuda, model_dirs, name, dtype, monkeypatch):
    """The debugging mode with guarded scratch buffers: every buffer of a step is allocated to its
    exact size with guard words behind it, and after every step of the mixed workload (portions,
    single tokens, tails of every tile shape) the guard words are intact.  That the check can fail
    is shown by overwriting one guard word by hand."""
    from ferrum_b200 import KernelError
    monkeypatch.setenv("FERRUM_CANARY", "1")
    s, toks, schedule = mixed_case(model_dirs, name, dtype)
    assert s.runner.ctx.scratch.guard == 64 and not s.runner.use_graphs
    r, _ = run_mixed(s, toks, schedule)              # (every step ends with the check: runner.check_device_errors)
    assert s.runner.ctx.scratch.check() == [] and len(s.runner.ctx.scratch._guards) >= 5
    for k in toks:
        assert_close(r.logits(k, len(toks[k])), plain_logits(model_dirs[name], dtype, toks[k]), dtype, f"guarded {k}")
    first = next(iter(s.runner.ctx.scratch._guards))
    s.runner.ctx.scratch._guards[first][3] = 0
    with pytest.raises(KernelError, match="wrote past the end of: " + first):
        s.runner.check_device_errors()
