"""Helpers of the GPU tests: traces, comparison with the plain implementation."""
import numpy as np

import plain_llama as P

# The reference's tolerance form (docs/ARCHITECTURE.md "Kernel tolerance";
# tests/accept/tests/kernels_contract.rs:21-24): |x - ref| <= max(1e-6, rel * max(1, |ref|)).
REL_F32 = 1e-4
# bfloat16: 8 bits of mantissa in every activation between kernels; the reference's own
# half-precision acceptance bound is an absolute logit difference (docs/ARCHITECTURE.md:215-222).
ABS_BF16 = 0.06


def assert_close_f32(x, ref, what=""):
    x, ref = np.asarray(x, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    lim = np.maximum(1e-6, REL_F32 * np.maximum(1.0, np.abs(ref)))
    bad = np.abs(x - ref) > lim
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} differ, worst {np.abs(x - ref).max():.3e} at {np.argwhere(bad)[0]}"


def assert_close_bf16(x, ref, what="", abs_tol=ABS_BF16):
    x, ref = np.asarray(x, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    err = np.abs(x - ref)
    assert err.max() <= abs_tol * max(1.0, np.abs(ref).max()), \
        f"{what}: worst abs error {err.max():.4f} at {np.unravel_index(err.argmax(), err.shape)}"


def assert_close(x, ref, dtype, what=""):
    (assert_close_f32 if dtype == "float32" else assert_close_bf16)(x, ref, what)


def plain_logits(folder, dtype, tokens):
    cfg, w = P.read_model(folder, weights_as="bfloat16" if dtype == "bfloat16" else "stored")
    return P.forward(cfg, w, tokens)


def random_tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


class Replay:
    """Feeds steps to a TraceSession and collects logits per (request, position)."""

    def __init__(self, session):
        self.session = session
        self.rows = {}          # (request id, position) -> logits row
        self.fed = {}           # request id -> tokens fed so far
        self.step_no = 0

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want) with want = indices into tokens or "all"."""
        rec = {"step": self.step_no, "entries": [], "end": list(end)}
        for rid, toks, want in entries:
            want = list(range(len(toks))) if want == "all" else list(want)
            rec["entries"].append({"id": rid, "tokens": list(toks), "want": want})
        out = self.session.run_step(rec)
        self.step_no += 1
        k = 0
        host = out.detach().float().cpu().numpy() if out is not None else None
        for e in rec["entries"]:
            base = self.fed.get(e["id"], 0)
            for i in e["want"]:
                self.rows[(e["id"], base + i)] = host[k]
                k += 1
            self.fed[e["id"]] = base + len(e["tokens"])
        for rid in end:
            self.fed.pop(rid, None)

    def logits(self, rid, n):
        return np.stack([self.rows[(rid, p)] for p in range(n)])
