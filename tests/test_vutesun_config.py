"""The Vutesun configuration, its tensor names and its cache needs; no GPU."""
import copy
import json

import pytest
import torch

from tensorline_b200.cache import PagedKV, SlotState
from tensorline_b200.config.base import ConfigError
from tensorline_b200.config.vutesun import VutesunConfig
from tensorline_b200.models import build_model, expected_tensors, load_config
from tensorline_b200.parts import Runtime
from tests.tiny_vutesun import CONFIGS, V1, V2


@pytest.mark.parametrize("name", ["V1", "V2"])
def test_the_configuration_reads_every_key_and_writes_them_back(name, tmp_path):
    cfg = VutesunConfig.from_dict(CONFIGS[name])
    assert cfg.to_json_dict() == CONFIGS[name]
    (tmp_path / "config.json").write_text(json.dumps(CONFIGS[name]))
    arch, again = load_config(tmp_path)                      # chosen by the single name under `architecture`
    assert arch.name == "Vutesun" and again == cfg
    assert cfg.vocab_size == CONFIGS[name]["vocab"] and cfg.hidden_size == CONFIGS[name]["width"]


def test_tensor_names_and_shapes_follow_the_layers():
    names = expected_tensors(VutesunConfig.from_dict(V1))
    shape = lambda n: tuple(names[n].shape)
    assert shape("embed") == (131, 48) and shape("head") == (131, 48) and shape("final.norm") == (48,)
    assert shape("l0.mix.q") == (24, 48) and shape("l0.mix.v") == (72, 48) and shape("l0.mix.o") == (48, 72)
    assert shape("l0.mix.i") == (3, 48) and shape("l0.mix.f.b") == (3,) and shape("l0.mix.norm") == (72,)
    assert shape("l0.mlp.router") == (5, 48) and shape("l0.mlp.router.b") == (5,) and shape("l0.mlp.e4.up") == (40, 48)
    assert shape("l1.mix.left.q") == (96, 48) and shape("l1.mix.left.k.b") == (32,) and shape("l1.mix.left.v") == (48, 48)
    assert shape("l1.mix.left.o") == (48, 144) and shape("l1.mix.left.sink") == (6,)
    assert shape("l1.mix.right.v") == (16, 48) and shape("l1.mix.right.o") == (48, 16) and shape("l1.mix.left.out") == (48,)
    assert names["l1.norm2"].optional and not any(n.startswith("l1.mlp") for n in names)    # a layer without a feed-forward
    assert "l2.norm2" in names and "l2.mlp.e2.down" in names and "l2.mlp.e3.down" not in names


def test_cache_needs_pages_for_attention_and_a_state_slot_for_every_recurrence():
    model = build_model(VutesunConfig.from_dict(V2), Runtime(torch.device("cpu"), torch.float32))
    needs = model.cache_needs()
    assert set(needs) == {(0, "left"), (0, "right"), 1, 2}
    assert needs[(0, "left")] == PagedKV(1, 64, None)
    assert all(isinstance(needs[k], SlotState) for k in ((0, "right"), 1, 2))
    wide = build_model(VutesunConfig.from_dict(V1), Runtime(torch.device("cpu"), torch.bfloat16)).cache_needs()
    assert wide[(1, "left")] == PagedKV(2, 32, None)         # values of 24 beside keys of 16: one padded head size of 32
    assert wide[(2, "left")].head_dim == 32


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_a_wrong_configuration_names_its_key(edit, word):
    raw = copy.deepcopy(V1)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        VutesunConfig.from_dict(raw)


def test_the_command_writes_random_weights_for_the_design(tmp_path):
    from tensorline_b200 import cli
    from tensorline_b200.weights import load_weights
    (tmp_path / "c.json").write_text(json.dumps(V2))
    out = tmp_path / "model"
    assert cli.main(["random-weights", "--config", str(tmp_path / "c.json"), "--out", str(out), "--seed", "1"]) == 0
    assert json.loads((out / "config.json").read_text()) == V2
    cfg = VutesunConfig.from_dict(V2)
    w = load_weights(out, expected_tensors(cfg))             # every tensor the model expects, nothing else
    assert w["l0.mix.left.sink"].shape == (4,) and "l1.norm2" not in w and w["l2.mlp.e1.up"].shape == (16, 72)
