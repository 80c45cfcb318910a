"""Tiny Dekerax configurations of the tests and a helper that writes their model folders.

D1 to D4 differ in every size and option: query/key heads wider and narrower than value heads, grouped and ungrouped
heads in attention and in the delta rule, windows that are no multiples of the page, no window, a window of one, a
rotation over part of the rotated key, latents narrower and wider than the heads, convolutions of one to five taps, one
to every expert a token, with and without a shared expert, layers without a feed-forward, loops that start at the first
layer or later, run once or three times, or are absent, head sizes that are no multiples of 16 and one above 128.  The
attention scales are large, so that a softmax is decided by few keys and a key that is wrongly seen (or not seen) shows.
"""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tensorline_b200.config.dekerax import DekeraxConfig
from tensorline_b200.models import expected_tensors
from tensorline_b200.weights import write_random_model
from tensorline_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def _moe(ff, experts, top, shared=None):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _dense(ff):
    return {"ff": ff, "kind": "dense"}


D1 = {"architecture": "Dekerax", "vocab": 131, "width": 48, "norm": {"eps": 1e-6}, "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.9, "mask": {"size": 11}}, "mlp": _dense(56)},
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 24, "conv": 4}, "mlp": _moe(40, 5, 2, 24)},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "rot": {"base": 100.0, "dims": 8}, "vdim": 24, "q_rank": 20,
                                           "kv_rank": 24, "scale": 0.7, "mask": {"size": 19}}, "mlp": None},
    {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.5}, "mlp": _moe(24, 3, 1)},
]}
D2 = {"architecture": "Dekerax", "vocab": 90, "width": 72, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 1, "times": 2}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 24, "rot_dim": 16, "rot": {"base": 10000.0, "dims": 8}, "vdim": 40, "q_rank": 36,
                                           "kv_rank": 40, "scale": 0.4, "mask": {"size": 33}}, "mlp": _moe(16, 9, 4, 56)},
    {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 72, "conv": 2}, "mlp": _dense(100)},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.3, "mask": {"size": 64}}, "mlp": None},
    {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 136, "vdim": 8, "conv": 1}, "mlp": _moe(8, 2, 2, 8)},
]}
# the delta rule only: no keys or values anywhere, so no page group at all; no loop
D3 = {"architecture": "Dekerax", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "layers": [
    {"type": "delta", "mixer": {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 12, "conv": 3}, "mlp": None},
    {"type": "delta", "mixer": {"heads": 5, "kv_heads": 5, "dim": 8, "vdim": 8, "conv": 5}, "mlp": _moe(32, 4, 4, 16)},
]}
# a window of one token, a latent without a window, a loop of one pass in the middle
D4 = {"architecture": "Dekerax", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "loop": {"start": 1, "stop": 2, "times": 1}, "layers": [
    {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 8, "scale": 0.6, "mask": {"size": 1}}, "mlp": _dense(24)},
    {"type": "latent_attention", "mixer": {"heads": 1, "dim": 8, "rot_dim": 4, "rot": {"base": 50.0, "dims": 4}, "vdim": 48, "q_rank": 8,
                                           "kv_rank": 12, "scale": 0.8}, "mlp": _moe(8, 3, 3)},
    {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 48, "vdim": 48, "scale": 0.2, "mask": {"size": 7}}, "mlp": None},
]}
# sizes that are multiples of nothing much: a width of 52, a vocabulary of 101, odd inner sizes, a latent without a rotated part
D5 = {"architecture": "Dekerax", "vocab": 101, "width": 52, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 3, "times": 2}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 5, "dim": 12, "rot_dim": 6, "rot": {"base": 30.0, "dims": 6}, "vdim": 20, "q_rank": 14,
                                           "kv_rank": 10, "scale": 0.5, "mask": {"size": 23}}, "mlp": _dense(30)},
    {"type": "delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 12, "vdim": 20, "conv": 3}, "mlp": _moe(18, 7, 3, 10)},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 10, "rot_dim": 0, "vdim": 6, "q_rank": 6, "kv_rank": 18, "scale": 0.4,
                                           "mask": {"size": 40}}, "mlp": None},
]}
CONFIGS = {"D1": D1, "D2": D2, "D3": D3, "D4": D4, "D5": D5}
PAGE_SIZE = {"D1": 8, "D2": 16, "D3": 4, "D4": 16, "D5": 16}


def write_tiny_dekerax(name: str, folder=None, seed: int = 0, config: dict | None = None, std: float = 0.12) -> Path:
    cfg = DekeraxConfig.from_dict(config or CONFIGS[name])
    folder = Path(folder) if folder is not None else Path(tempfile.mkdtemp(prefix=f"tiny_{name}_"))
    write_random_model(folder, cfg, expected_tensors(cfg), seed=seed, std=std, norm_std=0.1)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    g = torch.Generator().manual_seed(seed + 17)
    for n, t in tensors.items():
        if n.endswith(".A_log"):                               # decays from about 0.7 to 0.999 a token
            tensors[n] = (torch.rand(t.shape, generator=g) * 5.0 - 6.0).to(t.dtype)
        elif n.endswith(".dt_bias"):
            tensors[n] = (torch.rand(t.shape, generator=g) * 2.0 - 1.0).to(t.dtype)
        elif n.endswith((".mix.b", ".mix.a")):                  # gates that move from token to token
            tensors[n] = (t.float() * 3.0).to(t.dtype)
        elif n.endswith(".conv"):
            tensors[n] = (t.float() * 4.0).to(t.dtype)
        elif n == "loop.step":
            tensors[n] = (t.float() * 8.0).to(t.dtype)         # of the order of the stream: leaving a pass's vector out shows
        elif n.endswith((".router", ".sg")):
            tensors[n] = (t.float() * 3.0).to(t.dtype)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt"})
    return folder
