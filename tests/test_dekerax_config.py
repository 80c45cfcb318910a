"""The Dekerax configuration and model description, without a GPU."""
import copy

import pytest

from tensorline_b200.config import ConfigError
from tensorline_b200.config.dekerax import DekeraxConfig
from tensorline_b200.models import expected_tensors
from tensorline_b200.models.dekerax import describe_dekerax
from tensorline_b200.models.registry import architecture, registered_architectures
from tests.plain.dekerax_plain import run_order
from tests.tiny_dekerax import CONFIGS


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_registry(name):
    cfg = DekeraxConfig.from_dict(CONFIGS[name])
    assert cfg.to_json_dict() == CONFIGS[name]
    assert "Dekerax" in registered_architectures() and architecture("Dekerax").config_class is DekeraxConfig
    assert cfg.vocab_size == CONFIGS[name]["vocab"] and cfg.hidden_size == CONFIGS[name]["width"]
    assert cfg.num_parameters() > 0


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_run_order_is_the_plain_model_s(name):
    """Layers before the loop once, the loop's layers `times` times with the pass number in front of the first, the rest
    once; every entry owns its cache."""
    cfg = DekeraxConfig.from_dict(CONFIGS[name])
    spec = describe_dekerax(cfg)
    assert [(e.layer, e.add_row) for e in spec.run] == run_order(CONFIGS[name]) == cfg.run_order()
    assert all(e.reads_cache_of is None for e in spec.run)
    loop = CONFIGS[name].get("loop")
    assert spec.stream_rows == (loop["times"] if loop else 0)
    empty = copy.deepcopy(CONFIGS[name])
    empty["loop"] = {"start": 1, "stop": 1, "times": 4}          # a loop over nothing: every layer once, the table still expected
    cfg = DekeraxConfig.from_dict(empty)
    assert cfg.run_order() == run_order(empty) == [(i, None) for i in range(len(cfg.layers))]
    assert tuple(expected_tensors(cfg)["loop.step"].shape) == (4, cfg.width)
    assert len(spec.run) == len(cfg.layers) + ((loop["times"] - 1) * (loop["stop"] - loop["start"]) if loop else 0)


def test_tensor_names_and_shapes():
    names = expected_tensors(DekeraxConfig.from_dict(CONFIGS["D1"]))
    want = {"embed": (131, 48), "embed.norm": (48,), "loop.step": (3, 48), "final.norm": (48,), "head": (131, 48),
            "l0.norm1": (48,), "l0.norm1b": (48,), "l0.norm2": (48,), "l0.norm2b": (48,),
            "l0.mix.q": (96, 48), "l0.mix.k": (32, 48), "l0.mix.v": (48, 48), "l0.mix.o": (48, 144),
            "l0.mlp.gate": (56, 48), "l0.mlp.up": (56, 48), "l0.mlp.down": (48, 56),
            "l1.mix.q": (16, 48), "l1.mix.q.conv": (16, 4), "l1.mix.k": (16, 48), "l1.mix.k.conv": (16, 4), "l1.mix.v": (96, 48),
            "l1.mix.v.conv": (96, 4), "l1.mix.b": (4, 48), "l1.mix.a": (4, 48), "l1.mix.A_log": (4,), "l1.mix.dt_bias": (4,),
            "l1.mix.g": (96, 48), "l1.mix.norm": (24,), "l1.mix.o": (48, 96),
            "l1.mlp.router": (5, 48), "l1.mlp.e4.gate": (40, 48), "l1.mlp.e0.up": (40, 48), "l1.mlp.e2.down": (48, 40),
            "l1.mlp.shared.gate": (24, 48), "l1.mlp.shared.up": (24, 48), "l1.mlp.shared.down": (48, 24), "l1.mlp.shared.sg": (1, 48),
            "l2.mix.dq": (20, 48), "l2.mix.dq.norm": (20,), "l2.mix.uq": (72, 20), "l2.mix.dkv": (32, 48), "l2.mix.dkv.norm": (24,),
            "l2.mix.uk": (48, 24), "l2.mix.uv": (72, 24), "l2.mix.o": (48, 72), "l3.mlp.router": (3, 48)}
    for k, shape in want.items():
        assert tuple(names[k].shape) == shape, k
    assert names["l2.norm2"].optional and names["l2.norm2b"].optional          # a layer without a feed-forward
    assert "l3.mlp.shared.sg" not in names and "l1.mlp.router.b" not in names and "l1.mlp.e5.up" not in names
    assert "loop.step" not in expected_tensors(DekeraxConfig.from_dict(CONFIGS["D3"]))


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "layer type"),
    (("layers", 0, "mixer", "heads"), 5, "kv_heads"),
    (("layers", 1, "mixer", "conv"), 0, "conv"),
    (("layers", 2, "mixer", "rot", "dims"), 10, "dims"),
    (("layers", 2, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 1, "mlp", "router", "top"), 6, "top"),
    (("layers", 0, "mlp", "kind"), "glu", "kind"),
    (("loop", "stop"), 5, "loop"),
    (("loop", "times"), 0, "times"),
    (("norm", "eps"), 0.0, "eps"),
    (("width",), None, "width"),
])
def test_errors_name_the_key(path, value, word):
    raw = copy.deepcopy(CONFIGS["D1"])
    at = raw
    for p in path[:-1]:
        at = at[p]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        DekeraxConfig.from_dict(raw)
    assert word in str(e.value)
