import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from rosellm_b200.config import GPT2Config, load_config
from rosellm_b200.config.base import resolve_architecture
from rosellm_b200.models import Model, named_params_of_spec
from rosellm_b200.weights import WeightError, random_tensors, read_safetensors, write_model_folder
from tiny import TINY

CFG = TINY["B"]["config"]


def spec_of(cfg):
    return resolve_architecture(cfg.to_dict()).build_spec(cfg)


def test_folder_round_trip_and_device_dtypes(tmp_path):
    d = write_model_folder(CFG, 5, str(tmp_path / "m"))
    assert load_config(d) == CFG
    t = read_safetensors(d)
    assert t["h.0.attn.c_attn.weight"].shape == (96, 288)  # Conv1D layout [in, out]
    assert t["h.0.attn.c_attn.weight"].dtype == torch.bfloat16 and t["h.0.ln_1.weight"].dtype == torch.float32
    for dtype in (torch.bfloat16, torch.float32):
        m = Model(spec_of(CFG), dtype, "cpu")
        m.load_tensors(t, d)
        mixer = m.layers[0].mixer
        assert mixer.qkv_weight.shape == (288, 96) and mixer.qkv_weight.dtype == dtype  # [out, in] for the kernels
        assert torch.equal(mixer.qkv_weight.float(), t["h.0.attn.c_attn.weight"].float().t())
        assert mixer.qkv_bias.dtype == torch.float32 and m.layers[0].norm_mixer.weight.dtype == torch.float32
        assert m.head.weight.data_ptr() == m.embedding.weight.data_ptr()  # tied, one copy


def test_one_error_lists_everything_wrong(tmp_path):
    d = write_model_folder(CFG, 5, str(tmp_path / "m"))
    t = read_safetensors(d)
    del t["wpe.weight"], t["h.2.mlp.c_fc.bias"]
    t["h.1.ln_2.weight"] = torch.zeros(7)
    t["h.0.attn.c_proj.weight"] = torch.zeros(96, 95)
    t["stray.tensor"] = torch.zeros(1)
    t["ln_f.bias"] = torch.zeros(96, dtype=torch.int32)
    with pytest.raises(WeightError) as e:
        Model(spec_of(CFG), torch.float32, "cpu").load_tensors(t, d)
    err = e.value
    assert err.missing == ["h.2.mlp.c_fc.bias", "wpe.weight"]
    assert err.unexpected == ["stray.tensor"]
    assert {n for n, _, _ in err.wrong_shape} == {"h.1.ln_2.weight", "h.0.attn.c_proj.weight"}
    assert [n for n, _ in err.wrong_dtype] == ["ln_f.bias"]
    msg = str(err)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [96], file has [7]", "stray.tensor"):
        assert piece in msg


def test_prefix_and_checkpoint_buffers_are_accepted(tmp_path):
    d = write_model_folder(CFG, 5, str(tmp_path / "m"))
    t = {"transformer." + k: v for k, v in read_safetensors(d).items()}
    t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 4, 4)
    t["transformer.h.1.attn.masked_bias"] = torch.tensor(-1e4)
    t["lm_head.weight"] = t["transformer.wte.weight"]
    Model(spec_of(CFG), torch.float32, "cpu").load_tensors(t, "prefixed")


def test_random_weights_depend_on_seed_and_name_only():
    params = named_params_of_spec(spec_of(CFG))
    a = random_tensors(params, 3)
    b = random_tensors(list(reversed(params)), 3)
    c = random_tensors(params, 4)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["wte.weight"], c["wte.weight"])
    small = GPT2Config(**dict(CFG.flat(), n_layer=1))
    s = random_tensors(named_params_of_spec(spec_of(small)), 3)
    assert torch.equal(s["h.0.mlp.c_fc.weight"], a["h.0.mlp.c_fc.weight"])
    ident = random_tensors(params, 3, norm_affine="identity")
    assert torch.equal(ident["ln_f.weight"], torch.ones(96)) and torch.equal(ident["ln_f.bias"], torch.zeros(96))
    assert not torch.equal(a["ln_f.weight"], torch.ones(96))
    assert abs(float(a["wte.weight"].float().std()) - 0.02) < 2e-3


def test_missing_weight_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG.to_dict()))
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        read_safetensors(str(tmp_path))


def test_sharded_weights(tmp_path):
    d = write_model_folder(CFG, 5, str(tmp_path / "m"))
    t = load_file(os.path.join(d, "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    save_file({k: t[k] for k in names[:half]}, os.path.join(d, "a.safetensors"))
    save_file({k: t[k] for k in names[half:]}, os.path.join(d, "b.safetensors"))
    os.remove(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {k: ("a.safetensors" if i < half else "b.safetensors") for i, k in enumerate(names)}}, f)
    got = read_safetensors(d)
    assert sorted(got) == names and torch.equal(got[names[-1]], t[names[-1]])


def test_a_tensor_of_a_part_made_of_several_tensors_of_the_file():
    """A checkpoint that stores queries, keys and values apart feeds the mixer that wants them
    packed: the pieces are checked one by one (each by its own name in the error) and joined."""
    import dataclasses

    from rosellm_b200.parts import Concat

    small = GPT2Config(n_layer=1, n_embd=32, n_head=2, n_inner=64, vocab_size=50, n_positions=16,
                       layer_norm_epsilon=1e-5, activation_function="gelu_new")
    spec = spec_of(small)
    layer = spec.layers[0]
    mixer = layer.part("mixer")
    split = dataclasses.replace(mixer, tensors={
        **mixer.tensors,
        # Conv1D layout [in, out]: the pieces lie side by side along dimension 1
        "qkv_weight": Concat(("h.0.attn.q.weight", "h.0.attn.k.weight", "h.0.attn.v.weight"), dim=1),
        "qkv_bias": Concat(("h.0.attn.q.bias", "h.0.attn.k.bias", "h.0.attn.v.bias"), dim=0, sizes=(32, 32, 32)),
    })
    parts = tuple((n, c, split if n == "mixer" else s) for n, c, s in layer.parts)
    spec2 = dataclasses.replace(spec, layers=(dataclasses.replace(layer, parts=parts),))
    packed = random_tensors(named_params_of_spec(spec), 3)
    pieces = dict(packed)
    w, b = pieces.pop("h.0.attn.c_attn.weight"), pieces.pop("h.0.attn.c_attn.bias")
    for i, n in enumerate("qkv"):
        pieces[f"h.0.attn.{n}.weight"] = w[:, 32 * i:32 * (i + 1)].contiguous()
        pieces[f"h.0.attn.{n}.bias"] = b[32 * i:32 * (i + 1)].contiguous()
    one, two = Model(spec, torch.float32, "cpu"), Model(spec2, torch.float32, "cpu")
    one.load_tensors(packed)
    two.load_tensors(pieces)
    assert torch.equal(one.layers[0].mixer.qkv_weight, two.layers[0].mixer.qkv_weight)
    assert torch.equal(one.layers[0].mixer.qkv_bias, two.layers[0].mixer.qkv_bias)
    # the random-weights mode writes the pieces under their own names
    assert {"h.0.attn.q.weight", "h.0.attn.k.bias"} <= set(random_tensors(named_params_of_spec(spec2), 3))
    del pieces["h.0.attn.k.weight"]
    pieces["h.0.attn.v.bias"] = torch.zeros(31)
    with pytest.raises(WeightError) as e:
        two.load_tensors(pieces)
    assert e.value.missing == ["h.0.attn.k.weight"] and e.value.wrong_shape == [("h.0.attn.v.bias", (32,), (31,))]
    with pytest.raises(ValueError, match="do not make up"):
        Concat(("a", "b"), 0, (3, 4)).piece_shapes((8, 2))
