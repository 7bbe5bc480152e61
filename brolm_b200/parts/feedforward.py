"""Feed-forward parts."""
from __future__ import annotations

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part
from .linear import linear


class GatedFeedForward(Part):
    """down(act(gate(x)) * up(x)), dense, no bias
    (wlejon/brolm src/gemma2.cpp:378-382 with act = gelu, tanh form).
    Gate and up run as one product over the rows [Wg; Wu].

    ``activation`` "clamped_gate" is a pair function of its own instead of act(gate) * up:
    g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1), with ``limit`` > 0."""

    kind = "feedforward"
    graph_safe = True

    def __init__(self, hidden: int, inter: int, activation: str = "gelu_tanh", limit: float = 0.0):
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"feed-forward: unknown activation '{activation}'")
        if activation == "clamped_gate" and not limit > 0:
            raise ValueError("feed-forward: the clamped gate needs a positive limit")
        self.hidden, self.inter, self.activation, self.limit = hidden, inter, activation, float(limit)

    def param_specs(self):
        return {"gate": ParamSpec((self.inter, self.hidden)), "up": ParamSpec((self.inter, self.hidden)),
                "down": ParamSpec((self.hidden, self.inter))}

    def bind(self, params):
        kinds = {params[n].dtype for n in ("gate", "up")}
        dt = torch.float32 if (len(kinds) > 1 or torch.float32 in kinds) else next(iter(kinds))
        self.w_gate_up = torch.cat([params["gate"].to(dt), params["up"].to(dt)], dim=0).contiguous()
        self.w_down = params["down"]
        self.params = {}

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x (tokens, hidden) -> (tokens, hidden) float32."""
        act = torch.empty((x.shape[0], self.inter), dtype=ctx.dtype, device=x.device)
        if kernels.skinny_ok(x, self.w_gate_up):
            # few tokens: both products and the activation in one pass over the weights
            kernels.skinny_gemm(x, self.w_gate_up, act, "gated", self.activation, limit=self.limit)
        elif self.inter % 64 == 0 and kernels.stream_rows(x, self.w_gate_up):
            # 17 to 128 tokens: the same on the tcgen05 weight stream
            kernels.gemm_stream(x, self.w_gate_up, act, "gated", self.activation, limit=self.limit)
        elif self.inter % 128 == 0 and kernels.gemm_tc_ok(x, self.w_gate_up, gated=True):
            # many tokens: the activation is the epilogue of the product; [gate | up] never reaches memory
            kernels.gemm_tc(x, self.w_gate_up, act, "gated", self.activation, limit=self.limit)
        else:
            gate_up = linear(x, self.w_gate_up, out_dtype=ctx.dtype)
            kernels.gated_act(gate_up, act, self.activation, self.limit)
        return linear(act, self.w_down, out_dtype=torch.float32, parts_ok=True)


register_part("feedforward", "gated", GatedFeedForward)


class DenseFeedForward(Part):
    """down(act(up(x) + b_up)) + b_down: one hidden layer, no gate, biases optional.  ``activation``: "relu2"
    (the square of relu), "gelu_tanh", "silu" or "none".  The products' float32 sums take bias and activation
    in one row-wise pass."""

    kind = "feedforward"
    graph_safe = True

    def __init__(self, hidden: int, inter: int, activation: str = "relu2", bias: bool = True):
        if activation not in kernels.ROW_ACTS:
            raise ValueError(f"feed-forward: unknown activation '{activation}'")
        self.hidden, self.inter, self.activation, self.bias = hidden, inter, activation, bool(bias)

    def param_specs(self):
        specs = {"up": ParamSpec((self.inter, self.hidden)), "down": ParamSpec((self.hidden, self.inter))}
        if self.bias:
            specs["up_bias"] = ParamSpec((self.inter,), "vector")
            specs["down_bias"] = ParamSpec((self.hidden,), "vector")
        return specs

    def bind(self, params):
        self.w_up, self.w_down = params["up"], params["down"]
        self.b_up = params["up_bias"].float().contiguous() if self.bias else None
        self.b_down = params["down_bias"].float().contiguous() if self.bias else None
        self.params = {}

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x (tokens, hidden) -> (tokens, hidden) float32 (or partial sums when there is no bias to add)."""
        up = linear(x, self.w_up, out_dtype=torch.float32, parts_ok=True)
        act = torch.empty((x.shape[0], self.inter), dtype=ctx.dtype, device=x.device)
        kernels.bias_act(up, self.b_up, self.activation, act)
        y = linear(act, self.w_down, out_dtype=torch.float32, parts_ok=True)
        if self.b_down is None:
            return y
        out = torch.empty((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        kernels.bias_act(y, self.b_down, "none", out)
        return out


register_part("feedforward", "dense", DenseFeedForward)
