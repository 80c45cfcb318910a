"""Routed feed-forward (mixture of experts).

    z = h Wr^T + br                      router logits, float32 in both engines
    chosen: the `top` largest z;         weights = softmax over the chosen logits only
    y = sum_j weight_j * Wdown[e_j] act(Wup[e_j] h)          experts without biases, act = relu(.)^2

The experts' matrices are stacked ([E, F, K] and [E, K, F]) at load time.  Steps of few tokens stream, for every
(token, chosen expert) pair, that expert's rows (`ops.moe_up`, `ops.moe_down`): nothing is sorted and nothing comes
back to the host, so the step sits in a CUDA graph.  Steps of many tokens sort the pairs by expert on the device,
gather the tokens' rows in that order, every expert's run into `cap` rows of its own (the longest run, rounded up), and
run two batched dense products over all experts (the library's, as the engine's other long products are), which needs
the runs' bounds on the host.  The 32-bit engine streams always: a token's result is then the
same chain of additions in every step, whatever else the step holds.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_feed_forward
from .linear import resolve

# up to this many tokens a step the experts are streamed pair by pair
STREAM_MAX_TOKENS = int(os.environ.get("TENSORLINE_B200_MOE_STREAM_MAX_TOKENS", 32))


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    graph_capturable = True              # a captured step streams the experts whatever its size (see forward)

    def __init__(self, rt: Runtime, hidden: int, inner: int, experts: int, top: int, activation: str = "relu_squared",
                 router_bias: bool = True, names: dict | None = None):
        super().__init__(rt)
        if activation != "relu_squared":
            raise ValueError(f"routed_experts runs 'relu_squared', not {activation!r}")
        if not 1 <= top <= min(experts, 32) or experts > 1024:
            raise ValueError(f"routed_experts: top {top} of {experts} experts is outside what the choice kernel takes")
        self.hidden, self.inner, self.E, self.top, self.router_bias = hidden, inner, experts, top, router_bias
        self.names = {"router": "router", "router_bias": "router.b", "expert": "e{}", "up": "up", "down": "down", **(names or {})}
        self.w_router = self.b_router = self.w_up = self.w_down = None

    def _expert(self, prefix, e, which):
        return f"{prefix}.{self.names['expert'].format(e)}.{self.names[which]}"

    def expected_tensors(self, prefix):
        out = {f"{prefix}.{self.names['router']}": TensorSpec((self.E, self.hidden))}
        if self.router_bias:
            out[f"{prefix}.{self.names['router_bias']}"] = TensorSpec((self.E,))
        for e in range(self.E):
            out[self._expert(prefix, e, "up")] = TensorSpec((self.inner, self.hidden))
            out[self._expert(prefix, e, "down")] = TensorSpec((self.hidden, self.inner))
        return out

    def bind(self, weights, prefix):
        self.w_router = weights[f"{prefix}.{self.names['router']}"].contiguous()
        if self.router_bias:
            self.b_router = weights[f"{prefix}.{self.names['router_bias']}"].to(self.w_router.dtype).contiguous()
        self.w_up = self._compute_copy(torch.stack([weights[self._expert(prefix, e, "up")] for e in range(self.E)]))
        self.w_down = self._compute_copy(torch.stack([weights[self._expert(prefix, e, "down")] for e in range(self.E)]))

    def forward(self, h, ctx):
        h = resolve(h)
        T, top = h.shape[0], self.top
        z = torch.empty((T, self.E), dtype=torch.float32, device=h.device)
        ops.small_proj(h, self.w_router, self.b_router, z)
        idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
        wts = torch.empty((T, top), dtype=torch.float32, device=h.device)
        ops.topk_softmax(z, top, idx, wts)
        y = torch.empty((T, self.hidden), dtype=h.dtype, device=h.device)
        if T <= STREAM_MAX_TOKENS or ctx.graph_max_ctx or self.rt.exact:
            a = torch.empty((T * top, self.inner), dtype=h.dtype, device=h.device)
            ops.moe_up(h, self.w_up, idx, a)
            ops.moe_down(a, self.w_down, idx, wts, y)
            return y
        offsets, place_of, pair_at = ops.moe_sort(idx, self.E)
        bounds = offsets.tolist()                        # the one read-back of the step: where every expert's run ends
        longest = max(bounds[e + 1] - bounds[e] for e in range(self.E))
        cap = -(-longest // 64) * 64                     # rows every expert gets in the batched products
        rows = torch.empty((self.E * cap, self.hidden), dtype=h.dtype, device=h.device)
        ops.moe_gather(h, pair_at, idx, offsets, top, rows, cap=cap)
        inner = torch.bmm(rows.view(self.E, cap, self.hidden), self.w_up.transpose(1, 2))      # [E, cap, F]
        ops.mark("library product")
        ops.relu_square(inner)
        outs = torch.bmm(inner, self.w_down.transpose(1, 2))                                    # [E, cap, K]
        ops.mark("library product")
        ops.moe_combine(outs.view(self.E * cap, self.hidden), place_of, idx, offsets, wts, y, cap=cap)
        return y
