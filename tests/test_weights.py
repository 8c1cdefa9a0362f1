"""Weight files and the loader's single error (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_llama as P
from conftest import TINY, TINY_A, TINY_B
from ferrum_b200.config import registry
from ferrum_b200.errors import FileFormatError, WeightsError
from ferrum_b200.weights import SafetensorsFile, load_weights, write_random_model, write_safetensors


def build(folder, dtype=torch.float32):
    arch, cfg = registry.read_config(folder)
    return arch, cfg, arch.build(cfg, dtype, "cpu", max_positions=8)


def test_random_model_folder_loads_and_matches_the_plain_reader(model_dirs):
    for name in ("A", "B"):
        arch, cfg, model = build(model_dirs[name])
        load_weights(model, model_dirs[name], arch.hf_names(cfg), device="cpu")
        _, w = P.read_model(model_dirs[name])
        blk = model.blocks[0]
        q = w["model.layers.0.self_attn.q_proj.weight"]
        assert np.array_equal(blk.mixer.w_qkv[:q.shape[0]].double().numpy(), q)
        assert np.array_equal(blk.norm1.w_weight.double().numpy(), w["model.layers.0.input_layernorm.weight"])
        assert blk.norm1.w_weight.dtype == torch.float32           # vectors stay 32-bit
        tied = TINY[name][0]["tie_word_embeddings"]
        assert ("lm_head.weight" not in w) == tied
        assert (model.head.w_weight is model.embedding.w_weight) == tied


def test_same_seed_same_file_other_seed_other_file(tmp_path):
    a, b, c = (str(tmp_path / x) for x in "abc")
    write_random_model(TINY_A, a, 5); write_random_model(TINY_A, b, 5); write_random_model(TINY_A, c, 6)
    ra, rb, rc = (open(os.path.join(d, "model.safetensors"), "rb").read() for d in (a, b, c))
    assert ra == rb and ra != rc
    _, w = P.read_model(a)
    m = w["model.layers.1.mlp.down_proj.weight"]
    assert abs(m.std() - 0.02) < 0.002 and abs(w["model.norm.weight"].mean() - 1.0) < 0.02


def test_bfloat16_compute_dtype_rounds_matrices_only(model_dirs):
    arch, cfg, model = build(model_dirs["A"], torch.bfloat16)
    load_weights(model, model_dirs["A"], arch.hf_names(cfg), device="cpu")
    _, w = P.read_model(model_dirs["A"], weights_as="bfloat16")
    assert model.blocks[1].ffn.w_down_weight.dtype == torch.bfloat16
    assert np.array_equal(model.blocks[1].ffn.w_down_weight.double().numpy(), w["model.layers.1.mlp.down_proj.weight"])
    assert model.final_norm.w_weight.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path, model_dirs):
    src = SafetensorsFile(os.path.join(model_dirs["A"], "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["rope_freqs.weight"] = torch.zeros(8)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 171)
    d = tmp_path / "broken"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(str(d / "model.safetensors"), tensors)
    arch, cfg, model = build(str(d))
    with pytest.raises(WeightsError) as e:
        load_weights(model, str(d), arch.hf_names(cfg), device="cpu")
    msg = str(e.value)
    for needle in ("missing:", "model.layers.1.mlp.up_proj.weight", "model.norm.weight", "unexpected:",
                   "model.layers.0.self_attn.q_proj.bias", "rope_freqs.weight", "wrong shape:",
                   "model.layers.0.mlp.down_proj.weight: shape [64, 171], expected [64, 172]"):
        assert needle in msg, (needle, msg)


def test_untied_config_needs_no_lm_head_when_the_file_has_none(tmp_path):
    """The reference's rule: no output.weight means the embedding is shared
    (crates/model/src/llama.rs:103-111); tie_word_embeddings=True forbids an lm_head."""
    d = str(tmp_path / "m")
    write_random_model(TINY_A, d, 1, tie=True)             # config says untied, file has no lm_head
    arch, cfg, model = build(d)
    load_weights(model, d, arch.hf_names(cfg), device="cpu")
    assert model.head.w_weight is model.embedding.w_weight
    d2 = str(tmp_path / "m2")
    write_random_model(TINY_B, d2, 1)                      # config says tied, file gets an lm_head
    src = SafetensorsFile(os.path.join(d2, "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    src.close()
    write_safetensors(os.path.join(d2, "model.safetensors"), tensors)
    arch, cfg, model = build(d2)
    with pytest.raises(WeightsError, match="unexpected: lm_head.weight"):
        load_weights(model, d2, arch.hf_names(cfg), device="cpu")


@pytest.mark.parametrize("blob,msg", [
    (b"", "shorter"), (struct.pack("<Q", 10 ** 12), "header length"), (struct.pack("<Q", 4) + b"{no}", "not JSON"),
    (struct.pack("<Q", 2) + b"[]", "not a JSON object"),
])
def test_malformed_safetensors_is_an_error_not_a_crash(tmp_path, blob, msg):
    p = tmp_path / "x.safetensors"
    p.write_bytes(blob)
    with pytest.raises(FileFormatError, match=msg):
        SafetensorsFile(str(p))


def test_safetensors_offsets_are_checked(tmp_path):
    def mk(entry):
        h = json.dumps({"t": entry}).encode()
        p = tmp_path / "y.safetensors"
        p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 16)
        return str(p)
    with pytest.raises(FileFormatError, match="outside the file"):
        SafetensorsFile(mk({"dtype": "F32", "shape": [8], "data_offsets": [0, 32]}))
    with pytest.raises(FileFormatError, match="bytes for shape"):
        SafetensorsFile(mk({"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}))
    with pytest.raises(FileFormatError, match="unsupported dtype"):
        SafetensorsFile(mk({"dtype": "Q8_0", "shape": [4], "data_offsets": [0, 16]}))
    ok = SafetensorsFile(mk({"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}))
    assert ok.tensor("t").shape == (2, 2)


def test_random_bytes_never_crash_the_reader(tmp_path):
    """The property the reference fuzzes for its own container (fuzz/fuzz_targets/gguf_parse.rs)."""
    rng = np.random.default_rng(0)
    p = tmp_path / "z.safetensors"
    for n in list(range(0, 24)) + [64, 300, 5000]:
        for _ in range(20):
            blob = rng.integers(0, 256, size=n, dtype=np.uint8).tobytes()
            if n >= 8 and rng.random() < 0.5:         # a plausible header length followed by noise
                blob = struct.pack("<Q", int(rng.integers(0, max(1, n)))) + blob[8:]
            p.write_bytes(blob)
            try:
                SafetensorsFile(str(p))
            except FileFormatError:
                pass


def test_a_part_brings_its_own_initialisation(tmp_path):
    """The random-weights mode draws a parameter as its ParamSpec says: a registered name or a
    function of the part's own; an unknown name is an error that lists the known ones."""
    import torch
    from ferrum_b200.parts.base import ParamSpec
    from ferrum_b200.weights import random_init
    spec = ParamSpec((3, 5), init=lambda shape, g, device, std: torch.full(shape, 7.0, device=device))
    assert torch.equal(random_init._tensor("x", spec, 0, "cpu", 0.02), torch.full((3, 5), 7.0))
    random_init.register_init("halves", lambda shape, g, device, std: torch.full(shape, 0.5, device=device))
    try:
        assert random_init._tensor("x", ParamSpec((2,), kind="vector", init="halves"), 0, "cpu", 0.02).tolist() == [0.5, 0.5]
    finally:
        random_init.INITS.pop("halves")
    with pytest.raises(ValueError, match="unknown initialisation 'nope'.*normal"):
        random_init._tensor("x", ParamSpec((2,), init="nope"), 0, "cpu", 0.02)
