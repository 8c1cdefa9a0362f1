"""GGUF files: round trip, the reference's parse errors, and a model loaded from one."""
import struct

import numpy as np
import pytest
import torch

import plain_llama as P
from conftest import TINY_B
from ferrum_b200.errors import FileFormatError
from ferrum_b200.weights import GGUFFile, write_gguf, write_random_gguf


def test_round_trip_and_independent_reader(tmp_path):
    t = {"token_embd.weight": torch.randn(5, 4).half(), "b": torch.randn(7), "c": torch.randn(2, 3).bfloat16()}
    path = str(tmp_path / "x.gguf")
    write_gguf(path, {"general.architecture": "llama", "n": 3, "big": 2 ** 40, "f": 0.5, "names": ["a", "b"],
                      "flag": True}, t)
    g = GGUFFile(path)
    assert g.version == 3 and g.alignment == 32 and g.metadata["names"] == ["a", "b"] and g.metadata["big"] == 2 ** 40
    for k, v in t.items():
        assert torch.equal(g.tensor(k), v) and g.shape(k) == tuple(v.shape)
    import gguf                                     # the format library in the image, as an outside reading
    seen = {x.name: ([int(d) for d in x.shape], x.tensor_type.name) for x in gguf.GGUFReader(path).tensors}
    assert seen == {"token_embd.weight": ([4, 5], "F16"), "b": ([7], "F32"), "c": ([3, 2], "BF16")}


def header(version=3, n_tensors=0, n_kv=0, magic=b"GGUF"):
    return magic + struct.pack("<IQQ", version, n_tensors, n_kv)


def s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


@pytest.mark.parametrize("blob,msg", [
    (b"GGU", "end of file"), (header(magic=b"GGML"), "bad gguf magic"), (header(version=1), "unsupported gguf version 1"),
    (header(n_tensors=2 ** 60), "count exceeds"), (header(n_kv=1) + s("k") + struct.pack("<I", 99), "unknown metadata type"),
    (header(n_kv=1) + s("k") + struct.pack("<IB", 7, 2), "bool is not 0 or 1"),
    (header(n_kv=1) + struct.pack("<Q", 2) + b"\xff\xfe" + struct.pack("<II", 4, 1), "UTF-8"),
    (header(n_kv=1) + s("general.alignment") + struct.pack("<II", 4, 12), "multiple of 8"),
    (header(n_kv=2) + (s("k") + struct.pack("<II", 4, 1)) * 2, "duplicate metadata key"),
    (header(n_tensors=1) + s("t") + struct.pack("<IQIQ", 1, 4, 0, 0), "padding exceeds file"),
    (header(n_tensors=1) + s("t") + struct.pack("<IQIQ", 1, 400, 0, 0) + b"\0" * 64, "extends past end"),
    (header(n_tensors=1) + s("t") + struct.pack("<IQIQ", 1, 4, 0, 8) + b"\0" * 64, "not aligned"),
    (header(n_tensors=1) + s("t") + struct.pack("<IQIQ", 1, 4, 77, 0) + b"\0" * 64, "unknown ggml type"),
    (header(n_tensors=2) + (s("t") + struct.pack("<IQIQ", 1, 4, 0, 0)) * 2 + b"\0" * 64, "duplicate tensor"),
    (header() + b"\1" * 8, "padding is not zero"),
])
def test_malformed_files_are_errors(tmp_path, blob, msg):
    p = tmp_path / "bad.gguf"
    p.write_bytes(blob)
    with pytest.raises(FileFormatError, match=msg):
        GGUFFile(str(p))


def test_nested_arrays_have_a_depth_cap(tmp_path):
    blob = header(n_kv=1) + s("k") + struct.pack("<I", 9) + struct.pack("<IQ", 9, 1) * 70 + struct.pack("<IQ", 4, 0)
    p = tmp_path / "deep.gguf"
    p.write_bytes(blob)
    with pytest.raises(FileFormatError, match="nested too deeply"):
        GGUFFile(str(p))


def test_quantized_tensors_are_named_and_refused(tmp_path):
    blob = header(n_tensors=1) + s("blk.0.attn_q.weight") + struct.pack("<IQIQ", 1, 32, 8, 0)
    blob += b"\0" * ((-len(blob)) % 32) + b"\0" * 64
    p = tmp_path / "q.gguf"
    p.write_bytes(blob)
    g = GGUFFile(str(p))
    assert "blk.0.attn_q.weight [32] Q8_0" in g.dump()
    with pytest.raises(FileFormatError, match="Q8_0"):
        g.tensor("blk.0.attn_q.weight")


def test_random_bytes_never_crash(tmp_path):
    rng = np.random.default_rng(1)
    p = tmp_path / "r.gguf"
    for n in (0, 3, 24, 25, 60, 200, 2000):
        for _ in range(30):
            body = rng.integers(0, 256, size=n, dtype=np.uint8).tobytes()
            blob = (b"GGUF" + struct.pack("<I", 3) + body) if rng.random() < 0.7 else body
            p.write_bytes(blob)
            try:
                GGUFFile(str(p))
            except FileFormatError:
                pass


def test_config_from_a_gguf_file(tmp_path):
    from ferrum_b200.config import registry
    path = write_random_gguf(TINY_B, str(tmp_path / "b.gguf"), 1)
    arch, cfg = registry.read_config(path)
    assert arch.name == "LlamaForCausalLM" and cfg.rope_pairing == "adjacent" and cfg.n_vocab == 512
    assert cfg.rope_scaling.original_max_position_embeddings == 64 and cfg.n_head_kv == 1 and cfg.rms_norm_eps == pytest.approx(1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_model_from_gguf_rotates_adjacent_pairs(cuda, tmp_path, dtype):
    """The second tiny configuration as an F16 GGUF file: the engine's logits equal the plain
    implementation's with the reference's adjacent-pair rotation on the same (unpermuted) rows.
    The plain side reads the file with its own reader and takes every size from the file's own
    metadata.  Whole and in two portions, in portions of changing size, and mixed with page reuse."""
    from ferrum_b200.engine.trace import TraceSession
    from helpers import Replay, assert_close, mixed_case, pages_were_reused, random_tokens, round_to, run_mixed
    path = write_random_gguf(TINY_B, str(tmp_path / "b.gguf"), 1)
    cfg, w = P.read_gguf_model(path, weights_as=round_to(dtype))
    toks = random_tokens(60, 512, 70)
    ref = P.forward(cfg, w, toks, pairing="adjacent")
    r = Replay(TraceSession(path, dtype, 64))
    r.step([("a", toks[:41], "all")])
    r.step([("a", toks[41:], "all")])
    assert_close(r.logits("a", 60), ref, dtype, "gguf")
    assert np.abs(ref - P.forward(cfg, w, toks, pairing="half")).max() > 1e-3     # the pairing matters
    # portions of changing size, down to two tokens
    r = Replay(TraceSession(path, dtype, 64))
    sizes, i, k = [5, 2, 7, 3, 2, 16, 17, 2], 0, 0
    while i < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - i)
        r.step([("a", toks[i:i + n], "all")])
        i, k = i + n, k + 1
    assert_close(r.logits("a", 60), ref, dtype, "gguf portions")
    # mixed, with pages used again
    s, mtoks, schedule = mixed_case(None, "B", dtype, model_path=path)
    r, owners = run_mixed(s, mtoks, schedule)
    assert pages_were_reused(owners)
    for name, t in mtoks.items():
        assert_close(r.logits(name, len(t)), P.forward(cfg, w, t, pairing="adjacent"), dtype, f"gguf mixed {name}")
