"""Weights: the container, loading by name, types, the one error that lists everything, and
the random-weights mode."""
import json
import os

import numpy as np
import pytest
import torch

import wpc_engine_b200 as wpc
from conftest import TINY_A, TINY_B
from plain import qwen2_plain as P
from wpc_engine_b200.config import Qwen2Config
from wpc_engine_b200.registry import resolve
from wpc_engine_b200.weights import (ModelFiles, SafetensorsFile, WeightError, WeightFileError, load_weights,
                                     write_random_model, write_safetensors)


def read_all(folder):
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    out = {n: f.read(n) for n in f.names()}
    f.close()
    return out


def rewrite(folder, tensors):
    write_safetensors(os.path.join(folder, "model.safetensors"), list(tensors.items()))


def fresh_model(raw):
    return resolve(raw).build(Qwen2Config.from_dict(raw))


def test_container_round_trip_and_plain_reader_agree(tmp_path):
    ts = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, list(ts.items()))
    f = SafetensorsFile(path)
    assert sorted(f.names()) == ["a", "b", "c"] and f.shape("a") == (3, 5) and f.dtype_name("b") == "BF16"
    for n, t in ts.items():
        got = f.read(n)
        assert got.dtype == t.dtype and torch.equal(got, t)
    f.close()
    (tmp_path / "config.json").write_text("{}")
    _, plain = P.read_model_folder(str(tmp_path))
    for n, t in ts.items():
        assert np.array_equal(plain[n], t.float().numpy())


def test_truncated_or_garbled_files_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightFileError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightFileError, match="header length"):
        SafetensorsFile(str(p))
    with pytest.raises(WeightFileError, match="neither"):
        ModelFiles(str(tmp_path / "empty"))


def test_sharded_folder(tmp_path, folders):
    whole = read_all(folders[("A", "float32")])
    names = sorted(whole)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), [(n, whole[n]) for n in names[:half]])
    write_safetensors(str(tmp_path / "s2.safetensors"), [(n, whole[n]) for n in names[half:]])
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    files = ModelFiles(str(tmp_path))
    assert sorted(files.names()) == names and torch.equal(files.read(names[-1]), whole[names[-1]])
    files.close()


def test_types_are_kept(folders):
    for stored, dtype, want_matrix in [("bfloat16", torch.bfloat16, torch.bfloat16),
                                       ("float32", torch.bfloat16, torch.float32),     # stored in 32 bits: stays so
                                       ("bfloat16", torch.float32, torch.float32)]:
        model = fresh_model(TINY_B)
        load_weights(model, folders[("B", stored)], dtype, "cpu")
        attn = model.blocks[0].mixer
        assert attn.qkv.weight.dtype == want_matrix and model.embedding.table.dtype == want_matrix
        assert attn.qkv.bias.dtype == torch.float32 and model.final_norm.gain.dtype == torch.float32
        assert model.head.table.dtype == want_matrix


def test_fusion_is_a_pure_relayout(folders):
    folder = folders[("B", "bfloat16")]
    stored = read_all(folder)
    model = fresh_model(TINY_B)
    load_weights(model, folder, torch.bfloat16, "cpu")
    attn, mlp = model.blocks[1].mixer, model.blocks[1].ffn
    p = "model.layers.1."
    assert torch.equal(attn.qkv.weight, torch.cat([stored[p + f"self_attn.{x}_proj.weight"] for x in "qkv"]))
    assert torch.equal(attn.qkv.bias, torch.cat([stored[p + f"self_attn.{x}_proj.bias"].float() for x in "qkv"]))
    assert mlp.group == 200                       # 64 does not divide 200: all gates, then all ups
    assert torch.equal(mlp.gate_up.weight, torch.cat([stored[p + "mlp.gate_proj.weight"], stored[p + "mlp.up_proj.weight"]]))
    assert torch.equal(attn.q_proj.weight, stored[p + "self_attn.q_proj.weight"])


def test_gate_up_interleave_is_a_pure_relayout(tmp_path):
    raw = dict(TINY_B, intermediate_size=256, num_hidden_layers=1)
    folder = write_random_model(str(tmp_path), Qwen2Config.from_dict(raw), 3, torch.bfloat16)
    stored = read_all(folder)
    model = fresh_model(raw)
    load_weights(model, folder, torch.bfloat16, "cpu")
    mlp = model.blocks[0].ffn
    g, u = stored["model.layers.0.mlp.gate_proj.weight"], stored["model.layers.0.mlp.up_proj.weight"]
    assert mlp.group == 64
    assert torch.equal(mlp.gate_up.weight, torch.cat([t[i:i + 64] for i in range(0, 256, 64) for t in (g, u)]))
    assert torch.equal(mlp.gate_proj.weight.reshape(256, 96), g) and torch.equal(mlp.up_proj.weight.reshape(256, 96), u)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, folders):
    ts = read_all(folders[("B", "float32")])
    del ts["model.layers.1.self_attn.k_proj.bias"]
    del ts["model.norm.weight"]
    ts["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    ts["model.layers.0.mlp.down_proj.weight"] = ts["model.layers.0.mlp.down_proj.weight"].t().contiguous()
    ts["model.embed_tokens.weight"] = ts["model.embed_tokens.weight"].to(torch.int32)
    rewrite(str(tmp_path), ts)
    with pytest.raises(WeightError) as e:
        load_weights(fresh_model(TINY_B), str(tmp_path), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.mlp.up_proj.weight"]
    assert len(err.wrong_shape) == 1 and "down_proj" in err.wrong_shape[0] and "[200, 96]" in err.wrong_shape[0]
    assert len(err.wrong_dtype) == 1 and "I32" in err.wrong_dtype[0]
    text = str(err)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "unusable dtypes (1)"):
        assert word in text


def test_untied_needs_lm_head_and_tied_ignores_it(tmp_path, folders):
    ts = read_all(folders[("B", "float32")])
    del ts["lm_head.weight"]
    rewrite(str(tmp_path), ts)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(fresh_model(TINY_B), str(tmp_path), torch.float32, "cpu")
    ts = read_all(folders[("A", "float32")])
    ts["lm_head.weight"] = torch.zeros(256, 64)
    rewrite(str(tmp_path), ts)
    load_weights(fresh_model(TINY_A), str(tmp_path), torch.float32, "cpu")       # present but unused: fine


def test_random_weights_mode_is_reproducible_and_distributed_as_stated(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_B)
    a = write_random_model(str(tmp_path / "a"), cfg, 5, torch.float32)
    b = write_random_model(str(tmp_path / "b"), cfg, 5, torch.float32)
    c = write_random_model(str(tmp_path / "c"), cfg, 6, torch.float32)
    ta, tb, tc = read_all(a), read_all(b), read_all(c)
    assert all(torch.equal(ta[n], tb[n]) for n in ta) and any(not torch.equal(ta[n], tc[n]) for n in ta)
    w = ta["model.layers.0.mlp.gate_proj.weight"]
    assert abs(w.mean().item()) < 2e-3 and abs(w.std().item() - 0.02) < 2e-3
    g = ta["model.layers.2.input_layernorm.weight"]
    assert abs(g.mean().item() - 1.0) < 0.02 and g.min().item() > 0.8
    with open(os.path.join(a, "config.json")) as f:
        raw = json.load(f)
    assert raw["architectures"] == ["Qwen2ForCausalLM"] and Qwen2Config.from_dict(raw) == cfg
    assert os.path.getsize(os.path.join(write_random_model(str(tmp_path / "h"), cfg, 5, torch.bfloat16),
                                        "model.safetensors")) < os.path.getsize(os.path.join(a, "model.safetensors"))


def test_a_32_bit_checkpoint_under_bfloat16_stays_32_bit_and_says_so(folders, capsys):
    """Nothing is converted silently: matrices stored in 32 bits stay float32 (their products
    then run on the CUDA cores), and one line on standard error names that path."""
    model = fresh_model(TINY_A)
    load_weights(model, folders[("A", "float32")], torch.bfloat16, "cpu")
    err = capsys.readouterr().err
    assert "stay float32" in err and "model.embed_tokens.weight" in err and err.count("\n") == 1
    assert model.embedding.table.dtype == torch.float32
    load_weights(fresh_model(TINY_A), folders[("A", "bfloat16")], torch.bfloat16, "cpu")
    load_weights(fresh_model(TINY_A), folders[("A", "float32")], torch.float32, "cpu")
    assert capsys.readouterr().err == ""


def test_integer_tables_are_kept_as_int32_and_filled_by_the_random_mode(tmp_path):
    """A part may want a table of integers (kind "index"): stored as I32 or I64, kept as int32,
    and the random-weights mode draws it evenly from 0 .. high - 1."""
    import dataclasses
    from wpc_engine_b200.models.decoder import DecoderModel
    from wpc_engine_b200.parts import Embedding, OutputHead, ParamSpec, Part, RMSNorm

    class Lookup(Part):
        def param_specs(self):
            return {"map": ParamSpec((40,), kind="index", high=7), "zeros": ParamSpec((3, 2), kind="index")}

        def bind(self, tensors):
            self.map, self.zeros = tensors["map"], tensors["zeros"]

    @dataclasses.dataclass(frozen=True)
    class Cfg:
        vocab_size: int = 40
        width: int = 8

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["width"])

        def to_dict(self):
            return dict(dataclasses.asdict(self), architectures=["ToyLookupLM"])

    class WithLookup(DecoderModel):
        def roots(self):
            return super().roots() + [("lookup", self.lookup)]

    def build(c):
        emb = Embedding(c.vocab_size, c.width)
        m = WithLookup(c, emb, [], RMSNorm(c.width, 1e-5), OutputHead(c.vocab_size, c.width, tied_to=emb))
        m.lookup = Lookup()
        return m

    wpc.register_architecture("ToyLookupLM", Cfg, build)
    try:
        folder = write_random_model(str(tmp_path / "lookup"), Cfg(), 4, torch.bfloat16)
        stored = read_all(folder)
        assert stored["lookup.map"].dtype == torch.int32 and 0 <= int(stored["lookup.map"].min()) \
            and int(stored["lookup.map"].max()) == 6 and len(set(stored["lookup.map"].tolist())) == 7
        assert not stored["lookup.zeros"].any()
        model = build(Cfg())
        load_weights(model, folder, torch.bfloat16, "cpu")
        assert model.lookup.map.dtype == torch.int32 and torch.equal(model.lookup.map, stored["lookup.map"])
    finally:
        wpc.unregister_architecture("ToyLookupLM")
