"""Tiny Vutesun configurations of the tests and a helper that writes their model folders.

V1 and V2 differ in every size and option, and from sizes that happen to coincide elsewhere: value heads of another
size than query/key heads (both ways), partial and absent rotation, one KV head / as many as query heads, one head,
one expert a token / several, layers without a feed-forward, a residual multiplier of one and another, widths and
head sizes that are no multiples of 16, a head wider than 128.  The weights are drawn wide enough for attention
scores and gates to spread over several units; sinks, biases and gate biases are scaled up after the draw so that
leaving one out shows in the logits.
"""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tensorline_b200.config.vutesun import VutesunConfig
from tensorline_b200.models import expected_tensors
from tensorline_b200.weights import write_random_model
from tensorline_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def _moe(ff, experts, top):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


V1 = {"architecture": "Vutesun", "vocab": 131, "width": 48, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "layers": [
    {"type": "mlstm", "mixer": {"heads": 3, "dim": 8, "vdim": 24, "gate_cap": 8.0}, "mlp": _moe(40, 5, 2)},
    {"type": "parallel", "mixer": {
        "left": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "rot": {"base": 10000.0, "dims": 8}},
        "right": {"heads": 2, "dim": 24, "vdim": 8, "decay": [0.9, 0.995], "rot": {"base": 100.0, "dims": 24}}}, "mlp": None},
    {"type": "parallel", "mixer": {
        "left": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "rot": {"base": 50.0, "dims": 32}},
        "right": {"heads": 1, "dim": 16, "vdim": 40, "decay": [0.97], "rot": {"base": 3000.0, "dims": 4}}}, "mlp": _moe(24, 3, 1)},
]}
V2 = {"architecture": "Vutesun", "vocab": 90, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 1.0, "layers": [
    {"type": "parallel", "mixer": {
        "left": {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.11, "rot": {"base": 1e6, "dims": 64}},
        "right": {"heads": 3, "dim": 40, "vdim": 20, "decay": [0.8, 0.96, 0.999], "rot": {"base": 7.0, "dims": 0}}}, "mlp": _moe(56, 9, 4)},
    {"type": "mlstm", "mixer": {"heads": 1, "dim": 40, "vdim": 72, "gate_cap": 15.0}, "mlp": None},
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 136, "vdim": 8, "gate_cap": 3.0}, "mlp": _moe(16, 2, 2)},
]}
# recurrences only: no keys or values anywhere, so no page group at all
V3 = {"architecture": "Vutesun", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 1.3, "layers": [
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 20, "vdim": 12, "gate_cap": 10.0}, "mlp": None},
    {"type": "mlstm", "mixer": {"heads": 5, "dim": 8, "vdim": 8, "gate_cap": 15.0}, "mlp": _moe(32, 4, 4)},
]}
# attention without rotation and with as many KV heads as query heads beside a retention of full rotation; every expert chosen
V4 = {"architecture": "Vutesun", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "residual_mult": 0.9, "layers": [
    {"type": "parallel", "mixer": {
        "left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 8, "scale": 0.25, "rot": {"base": 10.0, "dims": 0}},
        "right": {"heads": 2, "dim": 8, "vdim": 16, "decay": [0.5, 1.0], "rot": {"base": 10.0, "dims": 8}}}, "mlp": _moe(8, 3, 3)},
    {"type": "parallel", "mixer": {
        "left": {"heads": 1, "kv_heads": 1, "dim": 48, "vdim": 48, "scale": 0.2, "rot": {"base": 1e4, "dims": 2}},
        "right": {"heads": 1, "dim": 4, "vdim": 4, "decay": [0.9], "rot": {"base": 2.0, "dims": 2}}}, "mlp": None},
]}
CONFIGS = {"V1": V1, "V2": V2, "V3": V3, "V4": V4}
PAGE_SIZE = {"V1": 8, "V2": 16, "V3": 4, "V4": 16}


def write_tiny_vutesun(name: str, folder=None, seed: int = 0) -> Path:
    cfg = VutesunConfig.from_dict(CONFIGS[name])
    folder = Path(folder) if folder is not None else Path(tempfile.mkdtemp(prefix=f"tiny_{name}_"))
    write_random_model(folder, cfg, expected_tensors(cfg), seed=seed, std=0.12, norm_std=0.1)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    for n, t in tensors.items():
        if n.endswith(".sink"):
            tensors[n] = (t.float() * 15.0 + 0.5).to(t.dtype)        # of the order of the scores: some heads lose half their weight
        elif n.endswith((".i.b", ".f.b")):
            tensors[n] = (t.float() * 4.0 + (2.0 if n.endswith(".f.b") else -1.0)).to(t.dtype)
        elif n.endswith(".b"):
            tensors[n] = (t.float() * 4.0).to(t.dtype)
        elif n.endswith((".i", ".f")):
            tensors[n] = (t.float() * 1.5).to(t.dtype)              # gates that move from token to token
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt"})
    return folder
