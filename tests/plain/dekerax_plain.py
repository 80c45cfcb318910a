"""A plain, slow implementation of the Dekerax decoder, used only as the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 on the CPU, written from the
design's equations in the notation below; it shares no code with the package under test.

Notation.  x_t: residual stream at token t (positions from 0); W: matrices stored [out, in], applied as W h;
unit(v) = v / sqrt(mean(v^2) + eps) with the model's eps; n(v; w) = unit(v) * w.

  start      x = n(embed[token]; embed.norm)
  order      layers [0, start), then `times` passes over layers [start, stop) (pass p first adds loop.step[p] to x,
             and owns its keys, values and states), then layers [stop, L)
  layer      x <- x + n(mixer(n(x; norm1)); norm1b);  x <- x + n(ff(n(x; norm2)); norm2b)  (if it has a feed-forward)
  attention  q, k, v without biases or rotation; query head a reads KV head a // (heads / kv_heads);
             p_tj = softmax_j(scale q_t . k_j) over t - size < j <= t; o_t = sum_j p_tj v_j; y = Wo o
  latent     cq = n(Wdq h; dq.norm), q = Wuq cq, head by head [dim plain | rot_dim turned];
             Wdkv h = [kv_rank | rot_dim]: c = n(first; dkv.norm), r = the rest turned by position (one for all heads);
             k_head = Wuk c, v_head = Wuv c; score = scale (q_plain . k_head + q_turned . r); window and softmax as above
  turning    pair (i, i + dims/2) of the first `dims` dimensions, angle t * base^(-2i / dims):
             (u, v) -> (u cos - v sin, v cos + u sin)
  delta      q, k (kv_heads x dim), v, gate (heads x vdim) projections; q, k, v through a causal convolution over time
             per channel (taps, the last weight on the current token, zeros before the start) and silu;
             q, k -> v / sqrt(sum v^2 + 1e-6) per head, q also times dim^-1/2;
             beta = sigmoid(Wb h); g = exp(-exp(A_log) softplus(Wa h + dt_bias));
             S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
             y = Wo (unit(o) per head * norm * silu(gate))
  dense      Wdown (gelu_tanh(Wgate h) * Wup h)
  experts    s = sigmoid(Wrouter h); the `top` largest; y = sum_e Wdown_e (silu(Wgate_e (s_e h)) * Wup_e (s_e h))
             + sigmoid(Wsg h) * shared(h), shared of the same form with silu
  output     logits = Whead n(x; final.norm)
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from tests.plain.qwen2_plain import read_safetensors

F64 = torch.float64


def unit(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def turn(x, pos, dims, base):
    """x [T, heads, d]: the first `dims` dimensions of every head turned by position, pairs (i, i + dims/2)."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = torch.as_tensor(pos, dtype=F64)[:, None] * float(base) ** (-2.0 * i / dims)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half], out[..., half:dims] = a * c - b * s, b * c + a * s
    return out


def windowed_softmax_sum(scores_of, values_of, T, size):
    """o_t = sum_j softmax_j(scores_of(t, lo, hi)) values_of(lo, hi) over lo = max(0, t - size + 1) .. t."""
    out = []
    for t in range(T):
        lo = 0 if size is None else max(0, t - size + 1)
        s = scores_of(t, lo, t + 1)
        p = torch.softmax(s, 0)
        out.append(p @ values_of(lo, t + 1))
    return torch.stack(out)


def attention(h, w, c):
    """w: q, k, v, o."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    size = (c.get("mask") or {}).get("size")
    q, k, v = (h @ w["q"].T).view(T, H, d), (h @ w["k"].T).view(T, G, d), (h @ w["v"].T).view(T, G, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        o[:, a] = windowed_softmax_sum(lambda t, lo, hi: (k[lo:hi, g] @ q[t, a]) * c["scale"],
                                       lambda lo, hi: v[lo:hi, g], T, size)
    return o.reshape(T, H * dv) @ w["o"].T


def latent_attention(h, w, c, eps, pos=None):
    """w: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o."""
    T = h.shape[0]
    H, d, dr, dv, R = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    size = (c.get("mask") or {}).get("size")
    pos = list(range(T)) if pos is None else pos
    rot = c.get("rot") or {"dims": 0, "base": 1.0}              # nothing to rotate: the constants may be left out
    cq = unit(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(T, H, d + dr)
    q_plain, q_turned = q[..., :d], turn(q[..., d:], pos, rot["dims"], rot["base"])
    down = h @ w["dkv"].T
    lat = unit(down[:, :R], eps) * w["dkv.norm"]
    shared = turn(down[:, None, R:], pos, rot["dims"], rot["base"])[:, 0]
    k = (lat @ w["uk"].T).view(T, H, d)
    v = (lat @ w["uv"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        o[:, a] = windowed_softmax_sum(
            lambda t, lo, hi: (k[lo:hi, a] @ q_plain[t, a] + shared[lo:hi] @ q_turned[t, a]) * c["scale"],
            lambda lo, hi: v[lo:hi, a], T, size)
    return o.reshape(T, H * dv) @ w["o"].T


def short_convolution(x, taps_w):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] x_(t - taps + 1 + j), zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x])
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j]
    return y


def delta(h, w, c, eps):
    """w: q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, g, norm, o."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    silu = torch.nn.functional.silu
    q = silu(short_convolution(h @ w["q"].T, w["q.conv"])).view(T, G, d)
    k = silu(short_convolution(h @ w["k"].T, w["k.conv"])).view(T, G, d)
    v = silu(short_convolution(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)
    g = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        j = a // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = g[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            o[t, a] = S.T @ q[t, j]
    y = unit(o, eps) * w["norm"] * silu(h @ w["g"].T).view(T, H, dv)
    return y.reshape(T, H * dv) @ w["o"].T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_unit(h, w, act):
    """w: gate, up, down."""
    return (act(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def experts(h, w, c):
    """w: router, e<k>.{gate,up,down}, shared.{gate,up,down,sg}."""
    silu = torch.nn.functional.silu
    top = c["router"]["top"]
    s = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros(h.shape[0], h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        val, idx = torch.topk(s[t], top)
        for j in range(top):
            e = int(idx[j])
            out[t] += gated_unit(val[j] * h[t], {n: w[f"e{e}.{n}"] for n in ("gate", "up", "down")}, silu)
    if c.get("shared"):
        sh = {n: w[f"shared.{n}"] for n in ("gate", "up", "down")}
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * gated_unit(h, sh, silu)
    return out


def feed_forward(h, w, c):
    return gated_unit(h, w, gelu_tanh) if c["kind"] == "dense" else experts(h, w, c)


class PlainDekerax:
    def __init__(self, folder):
        folder = Path(folder)
        self.cfg = json.loads((folder / "config.json").read_text())
        self.w = {k: v.to(F64) for k, v in read_safetensors(folder / "model.safetensors").items()}
        self.eps = self.cfg["norm"]["eps"]

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}


def run_order(cfg):
    """[(layer, pass number or None for 'no vector in front')]: the vector of a pass goes in front of its first layer."""
    L, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(L)]
    order = [(i, None) for i in range(loop["start"])]
    for p in range(loop["times"]):
        order += [(i, p if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], L)]


def forward(model: PlainDekerax, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence."""
    w, eps = model.w, model.eps
    x = unit(w["embed"][torch.tensor(tokens)], eps) * w["embed.norm"]
    for i, p in run_order(model.cfg):
        layer = model.cfg["layers"][i]
        if p is not None:
            x = x + w["loop.step"][p]
        h = unit(x, eps) * w[f"l{i}.norm1"]
        mix, c = model.sub(f"l{i}.mix."), layer["mixer"]
        if layer["type"] == "attention":
            y = attention(h, mix, c)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, mix, c, eps)
        else:
            y = delta(h, mix, c, eps)
        x = x + unit(y, eps) * w[f"l{i}.norm1b"]
        if layer.get("mlp") is not None:
            y = feed_forward(unit(x, eps) * w[f"l{i}.norm2"], model.sub(f"l{i}.mlp."), layer["mlp"])
            x = x + unit(y, eps) * w[f"l{i}.norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (unit(x, eps) * w["final.norm"]) @ w["head"].T


def greedy_generate(model: PlainDekerax, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(model, seq)[-1].argmax()))
    return seq[len(prompt):]
