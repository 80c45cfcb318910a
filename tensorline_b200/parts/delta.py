"""The gated delta rule: a mixer that keeps a matrix per head and corrects it towards every new value.

    q, k (nqk heads of d), v (H heads of dv), gate (H dv): projections of h; q, k, v then pass a causal convolution over
    time per channel (`taps` weights, the last on the current token, zeros before the start) and silu;
    q, k scaled to unit length per head, x / sqrt(sum x^2 + 1e-6), q also by d^-1/2
    beta = sigmoid(Wb h),   g = exp(-exp(A_log) softplus(Wa h + dt_bias))          one of each per head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                  (head h reads q/k head h // (H / nqk))
    y = Wo [o / rms(o) per head * norm * silu(gate)]

Between steps a request keeps, in its state slots, S (float32, in the scan kernel's own layout) and the convolution's
last `taps - 1` inputs (float32); both start at zero.  Everything that enters the recurrence beside the projections is
float32 in both engines; the stacked projection's float32 accumulators are kept as they are.  The mixer reads the step from
device tensors only (single-token steps sit in CUDA graphs).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import SlotState
from .base import Part, Runtime, TensorSpec, register_mixer
from .linear import matmul, resolve

_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a": "a",
          "A_log": "A_log", "dt_bias": "dt_bias", "g": "g", "norm": "norm", "o": "o"}


@register_mixer("gated_delta")
class GatedDelta(Part):
    graph_capturable = True
    unit_eps = 1e-6

    def __init__(self, rt: Runtime, hidden: int, num_heads: int, num_qk_heads: int, head_dim: int, v_head_dim: int, taps: int,
                 norm_eps: float, names: dict | None = None):
        super().__init__(rt)
        if num_heads % num_qk_heads:
            raise ValueError(f"{num_heads} value heads are not a multiple of {num_qk_heads} q/k heads")
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the scan kernel keeps at most 256 rows of state a head")
        self.hidden, self.H, self.nqk, self.d, self.dv, self.taps, self.eps = hidden, num_heads, num_qk_heads, head_dim, v_head_dim, taps, norm_eps
        self.C = 2 * num_qk_heads * head_dim + num_heads * v_head_dim          # channels that pass the convolution
        # the 32-bit engine keeps every state element as a pair of floats (see csrc/delta.cu): a float alone gathers one
        # rounding a token, which a read-out that is a small difference of large sums shows after a thousand tokens
        self.compensated = rt.exact
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.w_o = self.taps_w = self.A_log = self.dt_bias = self.head_weight = None

    def _state_floats(self) -> int:
        """As `ops.delta_state_floats` says on the device: R rows in each of IS x 16 threads."""
        d = self.d
        rows, per_column = (4, 8) if d <= 32 else (8, 8) if d <= 64 else (8, 16) if d <= 128 else (8, 32)
        return rows * per_column * 16 * (2 if self.compensated else 1)

    def cache_need(self):
        need = {"memory": SlotState((self.H * -(-self.dv // 16) * self._state_floats(),), "float32")}
        if self.taps > 1:
            need["inputs"] = SlotState(((self.taps - 1) * self.C,), "float32")
        return need

    def expected_tensors(self, prefix):
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        W, H, nqk, d, dv = self.hidden, self.H, self.nqk, self.d, self.dv
        return {n["q"]: TensorSpec((nqk * d, W)), n["k"]: TensorSpec((nqk * d, W)), n["v"]: TensorSpec((H * dv, W)),
                n["q_conv"]: TensorSpec((nqk * d, self.taps)), n["k_conv"]: TensorSpec((nqk * d, self.taps)),
                n["v_conv"]: TensorSpec((H * dv, self.taps)), n["b"]: TensorSpec((H, W)), n["a"]: TensorSpec((H, W)),
                n["A_log"]: TensorSpec((H,), init="zeros"), n["dt_bias"]: TensorSpec((H,), init="zeros"),
                n["g"]: TensorSpec((H * dv, W)), n["norm"]: TensorSpec((dv,), init="ones"), n["o"]: TensorSpec((W, H * dv))}

    def bind(self, weights, prefix):
        n = {k: f"{prefix}.{v}" for k, v in self.names.items()}
        # one stacked projection: q | k | v | gate | b | a; its float32 accumulators are what the recurrence reads
        self.w_in = self._compute_copy(torch.cat([weights[n[k]] for k in ("q", "k", "v", "g", "b", "a")], dim=0))
        self.taps_w = torch.cat([weights[n[k]] for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.A_log = weights[n["A_log"]].float().contiguous()
        self.dt_bias = weights[n["dt_bias"]].float().contiguous()
        self.head_weight = weights[n["norm"]].repeat(self.H).contiguous()      # one weight for all heads
        self.w_o = self._compute_copy(weights[n["o"]])
        if self.rt.device.type == "cuda":
            if ops.delta_columns() != 16 or ops.delta_state_floats(self.d, self.compensated) != self._state_floats():
                raise ops.KernelError("the delta kernel's state layout is not the one this mixer sizes its slots for")

    def forward(self, h, ctx, cache):
        H, nqk, d, dv, C = self.H, self.nqk, self.d, self.dv, self.C
        h = resolve(h)
        T = h.shape[0]
        proj = resolve(matmul(h, self.w_in, out_dtype=torch.float32))           # q | k | v | gate | b | a, float32 accumulators
        gates = proj[:, C + H * dv:]                                            # the write strengths' and decays' pre-activations
        qkv = torch.empty((T, C), dtype=torch.float32, device=h.device)
        inputs = cache["inputs"].state if self.taps > 1 else None
        ops.conv_prep(proj, self.taps_w, inputs, ctx.q_start, ctx.slots, qkv, B=ctx.B, max_q_len=ctx.max_q_len, nqk=nqk, d=d,
                      nv=H, dv=dv, unit_eps=self.unit_eps, q_scale=d ** -0.5)
        o = torch.empty((T, H * dv), dtype=torch.float32, device=h.device)
        ops.delta_scan(qkv, gates, self.A_log, self.dt_bias, cache["memory"].state, ctx.q_start, ctx.slots, o, B=ctx.B, H=H,
                       nqk=nqk, d=d, dv=dv, max_q_len=ctx.max_q_len, compensated=self.compensated)
        y = torch.empty((T, H * dv), dtype=h.dtype, device=h.device)
        ops.head_norm_gate(o, y, H, dv, self.eps, weight=self.head_weight, gate=proj, gate_off=C, act="silu")
        return matmul(y, self.w_o)
