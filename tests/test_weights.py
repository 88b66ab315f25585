"""Weights by tensor name, the one error that lists every problem, the random-weights writer (no GPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B, TINY_A_INIT
from sharpinference_b200.registry import resolve
from sharpinference_b200.weights import WeightError, declared_tensors, write_random_model
from sharpinference_b200.weights import safetensors_io
from sharpinference_b200.weights.source import FileWeights


def test_writer_makes_a_folder_another_reader_opens(model_dirs):
    d = model_dirs["A"]
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    t = load_file(os.path.join(d, "model.safetensors"))           # the safetensors library, not our reader
    assert t["model.embed_tokens.weight"].shape == (256, 64) and t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.feed_forward.experts.gate_up_proj"].shape == (4, 64, 256)
    assert t["model.layers.0.feed_forward.experts.down_proj"].shape == (4, 128, 64)
    assert t["model.layers.3.feed_forward.router.weight"].shape == (4, 64)
    assert abs(float(t["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
    norm = t["model.norm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.06 and 0.04 < float(norm.std()) < 0.2
    with open(os.path.join(d, "config.json")) as fh:
        cfg = json.load(fh)
    assert cfg["architectures"] == ["Llama4ForCausalLM"] and cfg["hidden_size"] == 64


def test_same_seed_same_bytes_other_seed_other_bytes(tmp_path):
    a = write_random_model(dict(TINY_A), str(tmp_path / "a"), 5)
    b = write_random_model(dict(TINY_A), str(tmp_path / "b"), 5)
    c = write_random_model(dict(TINY_A), str(tmp_path / "c"), 6)
    ra, rb, rc = (open(os.path.join(x, "model.safetensors"), "rb").read() for x in (a, b, c))
    assert ra == rb and ra != rc


def test_dense_and_moe_layers_have_their_own_tensors(model_dirs):
    names = set(load_file(os.path.join(model_dirs["B"], "model.safetensors")))
    assert "model.layers.0.feed_forward.gate_proj.weight" in names
    assert "model.layers.0.feed_forward.router.weight" not in names
    assert "model.layers.1.feed_forward.router.weight" in names
    assert "model.layers.1.feed_forward.gate_proj.weight" not in names
    assert "lm_head.weight" in names


def test_own_reader_matches_library(model_dirs):
    path = os.path.join(model_dirs["B"], "model.safetensors")
    theirs = load_file(path)
    ours = safetensors_io.open_model(model_dirs["B"])
    assert set(ours) == set(theirs)
    for name, entry in ours.items():
        assert torch.equal(entry.load(), theirs[name]), name


def _check(folder, cfg):
    arch, typed = resolve(cfg)
    fw = FileWeights(folder, torch.bfloat16, "cpu")
    decls = declared_tensors(arch, typed)
    fw.choose_prefix(decls)
    fw.check(decls)
    return fw


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    t = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    del t["model.layers.1.self_attn.k_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    t["model.layers.0.feed_forward.router.weight"] = torch.zeros(5, 64, dtype=torch.bfloat16)
    t["model.layers.9.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    t["lm_head.weight"] = t["lm_head.weight"].to(torch.int32)
    save_file(t, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as exc:
        _check(str(tmp_path), TINY_A)
    text = str(exc.value)
    assert "missing (2)" in text and "model.layers.1.self_attn.k_proj.weight" in text and "model.norm.weight" in text
    assert "wrong shape (2)" in text and "[64, 63], expected [64, 64]" in text and "[5, 64], expected [4, 64]" in text
    assert "unexpected (1)" in text and "model.layers.9.extra.weight" in text
    assert "unsupported dtype (1)" in text and "lm_head.weight" in text


def test_language_model_prefix_is_found(model_dirs, tmp_path):
    t = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    t = {"language_model." + k: v for k, v in t.items()}
    t["vision_model.patch.weight"] = torch.zeros(3)
    save_file(t, str(tmp_path / "model.safetensors"))
    fw = _check(str(tmp_path), TINY_A)
    assert fw.prefix == "language_model."


def test_experts_kept_apart_load_like_the_fused_tensors(model_dirs, tmp_path):
    """A folder may hold one [out, in] matrix per expert and projection instead of the fused input-major
    tensors: the builder asks for what is there, the check accepts it, and the model gets the same weights;
    a folder that lacks one of the per-expert matrices is told so."""
    import json
    import shutil
    from sharpinference_b200.weights.loading import load_model
    fused = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    E, I = TINY_A["num_local_experts"], TINY_A["intermediate_size"]
    apart = {}
    for name, t in fused.items():
        if name.endswith("feed_forward.experts.gate_up_proj"):
            base = name[: -len("gate_up_proj")]
            for e in range(E):
                apart[f"{base}{e}.gate_proj.weight"] = t[e, :, :I].t().contiguous()
                apart[f"{base}{e}.up_proj.weight"] = t[e, :, I:].t().contiguous()
        elif name.endswith("feed_forward.experts.down_proj"):
            base = name[: -len("down_proj")]
            for e in range(E):
                apart[f"{base}{e}.down_proj.weight"] = t[e].t().contiguous()
        else:
            apart[name] = t
    folder = tmp_path / "apart"
    folder.mkdir()
    shutil.copy(os.path.join(model_dirs["A"], "config.json"), folder / "config.json")
    save_file(apart, str(folder / "model.safetensors"))
    a = load_model(model_dirs["A"], dtype="bfloat16", device="cpu")
    b = load_model(str(folder), dtype="bfloat16", device="cpu")
    for blk_a, blk_b in zip(a.blocks, b.blocks):
        assert torch.equal(blk_a.ffn.experts_gate_up.weight, blk_b.ffn.experts_gate_up.weight)
        assert torch.equal(blk_a.ffn.experts_down.weight, blk_b.ffn.experts_down.weight)
    del apart["model.layers.2.feed_forward.experts.3.up_proj.weight"]
    save_file(apart, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match=r"missing \(1\)[\s\S]*experts\.3\.up_proj"):
        load_model(str(folder), dtype="bfloat16", device="cpu")


def test_dtype_rules(model_dirs, tmp_path):
    t = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    t["model.layers.0.self_attn.o_proj.weight"] = t["model.layers.0.self_attn.o_proj.weight"].float()
    save_file(t, str(tmp_path / "model.safetensors"))
    fw = _check(str(tmp_path), TINY_A)
    assert fw.matrix("model.layers.0.self_attn.o_proj.weight", (64, 64)).dtype == torch.float32   # stored 32-bit stays
    assert fw.matrix("model.layers.1.self_attn.o_proj.weight", (64, 64)).dtype == torch.bfloat16
    assert fw.vector("model.norm.weight", (64,)).dtype == torch.float32
    fw32 = FileWeights(str(tmp_path), torch.float32, "cpu")
    assert fw32.matrix("model.layers.1.self_attn.o_proj.weight", (64, 64)).dtype == torch.float32


def test_sharded_folder_and_bad_files(model_dirs, tmp_path):
    t = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    save_file({n: t[n] for n in names[:half]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({n: t[n] for n in names[half:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    with open(tmp_path / "model.safetensors.index.json", "w") as fh:
        json.dump(index, fh)
    _check(str(tmp_path), TINY_A)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(safetensors_io.SafetensorsError):
        safetensors_io.open_model(str(empty))
    (empty / "model.safetensors").write_bytes(b"\x05\x00")
    with pytest.raises(safetensors_io.SafetensorsError):
        safetensors_io.open_model(str(empty))
