"""A plain, slow implementation of the Vutesun decoder, used only as the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 on the CPU, written from the
design's equations in the notation below; it shares no code with the package under test (own container
reader, own config reading, own arithmetic).

Notation.  x_t: residual stream at token t (positions count from 0); h_t: a normalised input; W: matrices
stored [out, in] and applied as W h; rms(v) = sqrt(mean(v^2) + eps) with the model's eps.

  layer      x <- x + r * mixer(norm(x; w1)),  x <- x + r * experts(norm(x; w2))   (the second only if the layer has
             a feed-forward), r = residual_mult, norm(x; w) = x / rms(x) * (1 + w)
  sink attention (left)   q, k, v with biases; the first `dims` dimensions of every q and k head rotated in pairs
             (2i, 2i + 1) by the angle t * base^(-2i / dims); a_tj = exp(scale q_t . k_j) for j <= t,
             o_t = sum_j a_tj v_j / (sum_j a_tj + exp(sink_head)); query head n reads KV head n // (heads / kv_heads)
  retention (right)       q, k rotated in pairs (i, i + dims / 2), then k scaled by dim^-1/2;
             S_t = decay_head S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; o / rms(o) per head, times silu(Wg h)
  pair       0.5 * (L / rms(L) * w_left + R / rms(R) * w_right), L and R the two branches after their output matrices
  mlstm      q scaled by dim^-1/2; i_t = cap tanh((Wi h + bi) / cap), f_t = logsigmoid(cap tanh((Wf h + bf) / cap));
             m_t = max(f_t + m_(t-1), i_t) with m before the first token 0; S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) +
             exp(i_t - m_t) k_t v_t^T, n_t the same with k_t alone; o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6);
             o / rms(o) per head, times the weight over all heads, times sigmoid(Wg h)
  experts    z = Wr h + br; the `top` largest z, their weights the softmax over those alone;
             y = sum_e weight_e Wdown_e relu(Wup_e h)^2
  output     logits = Whead norm(x; w_final)
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from tests.plain.qwen2_plain import read_safetensors

F64 = torch.float64


def rms_div(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_div(x, eps) * (1.0 + w)


def rotate(x, pos, dims, base, layout):
    """x [T, heads, d]; the first `dims` dimensions of every head rotated by position; layout "pairs": (2i, 2i + 1),
    "halves": (i, i + dims / 2)."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.as_tensor(pos, dtype=F64)[:, None] * float(base) ** (-2.0 * i / dims)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if layout == "pairs":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = a * c - b * s, b * c + a * s
    return out


def sink_attention(h, w, c, pos=None):
    """w: q, q.b, k, k.b, v, v.b, sink, o."""
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    pos = list(range(T)) if pos is None else pos
    q = rotate((h @ w["q"].T + w["q.b"]).view(T, H, d), pos, c["rot"]["dims"], c["rot"]["base"], "pairs")
    k = rotate((h @ w["k"].T + w["k.b"]).view(T, G, d), pos, c["rot"]["dims"], c["rot"]["base"], "pairs")
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for n in range(H):
        g = n // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, n]) * c["scale"]
            top = max(float(s.max()), float(w["sink"][n]))
            a = torch.exp(s - top)
            o[t, n] = (a @ v[:t + 1, g]) / (a.sum() + math.exp(float(w["sink"][n]) - top))
    return o.reshape(T, H * dv) @ w["o"].T


def retention(h, w, c, eps, pos=None):
    """w: q, k, v, g, o."""
    T = h.shape[0]
    H, d, dv = c["heads"], c["dim"], c["vdim"]
    pos = list(range(T)) if pos is None else pos
    q = rotate((h @ w["q"].T).view(T, H, d), pos, c["rot"]["dims"], c["rot"]["base"], "halves")
    k = rotate((h @ w["k"].T).view(T, H, d), pos, c["rot"]["dims"], c["rot"]["base"], "halves") * d ** -0.5
    v = (h @ w["v"].T).view(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    decay = torch.tensor(c["decay"], dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms_div(o, eps).reshape(T, H * dv) * torch.nn.functional.silu(h @ w["g"].T)
    return y @ w["o"].T


def mixer_pair(h, w, c, eps):
    """w: names under left.* and right.*, left.out, right.out."""
    left = sink_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, c["left"])
    right = retention(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, c["right"], eps)
    return 0.5 * (rms_div(left, eps) * w["left.out"] + rms_div(right, eps) * w["right.out"])


def mlstm(h, w, c, eps):
    """w: q, k, v, g, o, norm, i, i.b, f, f.b."""
    T = h.shape[0]
    H, d, dv, cap = c["heads"], c["dim"], c["vdim"], c["gate_cap"]
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    S, n, m = torch.zeros(H, d, dv, dtype=F64), torch.zeros(H, d, dtype=F64), torch.zeros(H, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        keep, take = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    y = rms_div(o, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return y @ w["o"].T


def experts(h, w, c):
    """w: router, router.b, e<k>.up, e<k>.down."""
    top = c["router"]["top"]
    z = h @ w["router"].T + w["router.b"]
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        val, idx = torch.topk(z[t], top)
        share = torch.softmax(val, 0)
        for j in range(top):
            e = int(idx[j])
            out[t] += share[j] * (w[f"e{e}.down"] @ torch.relu(w[f"e{e}.up"] @ h[t]) ** 2)
    return out


class PlainVutesun:
    def __init__(self, folder):
        folder = Path(folder)
        self.cfg = json.loads((folder / "config.json").read_text())
        self.w = {k: v.to(F64) for k, v in read_safetensors(folder / "model.safetensors").items()}
        self.eps = self.cfg["norm"]["eps"]

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}


def forward(model: PlainVutesun, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence."""
    w, eps, r = model.w, model.eps, model.cfg["residual_mult"]
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(model.cfg["layers"]):
        h = norm_one_plus(x, w[f"l{i}.norm1"], eps)
        mix = model.sub(f"l{i}.mix.")
        y = mlstm(h, mix, layer["mixer"], eps) if layer["type"] == "mlstm" else mixer_pair(h, mix, layer["mixer"], eps)
        x = x + r * y
        if layer["mlp"] is not None:
            x = x + r * experts(norm_one_plus(x, w[f"l{i}.norm2"], eps), model.sub(f"l{i}.mlp."), layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(model: PlainVutesun, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(model, seq)[-1].argmax()))
    return seq[len(prompt):]
