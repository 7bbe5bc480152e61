"""Routed experts: a feed-forward made of many small ones, of which a token uses a few."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part
from .linear import linear


class RoutedExperts(Part):
    """y = sum over the token's ``top`` experts e of  W_down[e] act(W_up[e] (g_e x)),  no biases.

    Router: z = W_r x summed in float (by the router kernel in one fixed order; for a prompt in bfloat16 by a
    matrix product with float accumulation); the ``top`` largest z are chosen; g_e = logistic(z_e), not
    renormalised.  With ``scale_input`` the gate multiplies the expert's input (one rounding to the step's
    element type), not its output.  ``activation``: "relu2" (the square of relu) or "none".

    On the device: route -> sort the (token, choice) pairs by expert -> one grouped product per matrix over
    tiles of each expert's pairs -> float results [top, tokens, hidden], which the residual kernel
    adds in the order of the choices.  Nothing is read back to the host.  With many pairs per expert (a
    prompt) the products run on tcgen05 over 128-row tiles, the tokens' rows first copied into expert order;
    with few (decoding) on mma.sync over 64-row tiles, as a stream of the chosen experts' matrices.

    Options beside those (any of them selects the second form of the pass, ``_forward_weighted``):

    * ``router="softmax"``: s = softmax(z) over all experts; with ``correction`` a learned number per expert is
      added to s for the choice alone; the weights are the chosen s over their sum (+ 1e-20);
    * ``scale_input=False``: the weight multiplies the expert's result, in float, when the results are added;
    * ``gated=True``: an expert is W_down (act(W_gate x) * (W_up x)) with ``activation`` "silu" or "gelu_tanh";
      gate and up run as one grouped product over the rows [W_gate; W_up];
    * ``identity`` = n: the router has n more outputs, after the experts'; a token that chooses one of them
      gets its own input back (times the weight).  They have no tensors and take no part in the products;
    * ``shared``: a feed-forward part that every token runs; its result is added; with ``shared_gate`` it is first
      multiplied by sigmoid(w_sg . x), one number per token (tensor ``shared_gate``, one row);
    * ``groups`` = (count, keep) with the softmax router: the experts form ``count`` equal groups of neighbours, a
      group's score is its largest s (+ correction), and only experts of the ``keep`` best groups can be chosen;
    * ``renorm=False`` with the softmax router: the weights are the chosen s themselves, not divided by their sum;
    * ``weight_scale``: a constant that multiplies the weights.

    The result of that form is one float32 (tokens, hidden) array: weights, identity experts and the shared
    expert are folded in by one row-wise kernel.
    """

    kind = "feedforward"
    ROUTER_PRODUCT_ROWS = 256      # from this many tokens on the router's scores are a matrix product

    def __init__(self, hidden: int, inter: int, experts: int, top: int, activation: str = "relu2",
                 scale_input: bool = True, router: str = "logistic", correction: bool = False, gated: bool = False,
                 identity: int = 0, shared: Optional[Part] = None, shared_gate: bool = False, groups=None,
                 renorm: bool = True, weight_scale: float = 1.0):
        count, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        if (count, keep) != (1, 1) or not renorm or float(weight_scale) != 1.0:
            if router != "softmax":
                raise ValueError("routed experts: groups, unnormalised weights and a weight scale go with the softmax router")
            if identity:
                raise ValueError("routed experts: groups or unnormalised weights together with identity experts are not built")
            if count < 1 or not 1 <= keep <= count or experts % count or top > keep * (experts // count):
                raise ValueError(f"routed experts: {experts} experts in {count} groups of which {keep} stay open cannot "
                                 f"give {top} choices")
        if shared_gate and shared is None:
            raise ValueError("routed experts: a gate of the shared expert needs a shared expert")
        self.groups, self.keep, self.renorm, self.weight_scale = count, keep, bool(renorm), float(weight_scale)
        self.has_shared_gate = bool(shared_gate)
        if experts < 0 or identity < 0 or not 1 <= top <= experts + identity:
            raise ValueError("routed experts: 1 <= top <= experts + identity")
        if router not in kernels.ROUTE_MODES:
            raise ValueError(f"routed experts: unknown router '{router}'")
        if correction and router != "softmax":
            raise ValueError("routed experts: a correction of the choice goes with the softmax router")
        self.weighted = bool(router != "logistic" or not scale_input or gated or identity or shared is not None)
        self.route_opts = dict(groups=count, keep=keep, renorm=bool(renorm), scale=float(weight_scale)) \
            if router == "softmax" else {}
        if self.weighted:
            if scale_input:
                raise ValueError("routed experts: with these options the weight goes on the expert's result "
                                 "(scale_input=False)")
            if gated and activation not in kernels.ACTIVATIONS:
                raise ValueError(f"routed experts: unknown gated activation '{activation}'")
            if not gated and activation not in kernels.EXPERT_ACTS:
                raise ValueError(f"routed experts: unknown activation '{activation}'")
        elif activation not in kernels.EXPERT_ACTS:
            raise ValueError(f"routed experts: unknown activation '{activation}'")
        self.hidden, self.inter, self.experts, self.top, self.activation = hidden, inter, experts, top, activation
        self.route_mode, self.has_correction, self.gated, self.identity, self.shared = router, correction, gated, identity, shared

    @property
    def graph_safe(self) -> bool:
        return self.shared is None or self.shared.graph_safe

    def param_specs(self):
        specs = {"router": ParamSpec((self.experts + self.identity, self.hidden))}
        if self.has_correction:
            specs["correction"] = ParamSpec((self.experts + self.identity,), "vector")
        if self.has_shared_gate:
            specs["shared_gate"] = ParamSpec((1, self.hidden))
        for e in range(self.experts):
            if self.gated:
                specs[f"e{e}.gate"] = ParamSpec((self.inter, self.hidden))
            specs[f"e{e}.up"] = ParamSpec((self.inter, self.hidden))
            specs[f"e{e}.down"] = ParamSpec((self.hidden, self.inter))
        return specs

    def bind(self, params):
        self.router = params["router"]
        mats = ("gate", "up", "down") if self.gated else ("up", "down")
        kinds = {params[f"e{e}.{n}"].dtype for e in range(self.experts) for n in mats} | {self.router.dtype}
        if len(kinds) > 1:
            raise TypeError("routed experts: the experts' matrices and the router must have one element type")
        self.correction = params["correction"].float().contiguous() if self.has_correction else None
        self.w_shared_gate = params["shared_gate"].to(self.router.dtype).reshape(-1).contiguous() \
            if self.has_shared_gate else None
        if self.experts:
            if self.gated:      # per expert the rows [W_gate; W_up]
                self.w_up = torch.stack([torch.cat([params[f"e{e}.gate"], params[f"e{e}.up"]], dim=0)
                                         for e in range(self.experts)]).contiguous()
            else:
                self.w_up = torch.stack([params[f"e{e}.up"] for e in range(self.experts)]).contiguous()
            self.w_down = torch.stack([params[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        self.params = {}

    def _route(self, x: torch.Tensor, ids: torch.Tensor, gates: torch.Tensor) -> None:
        n = self.router.shape[0]
        if x.dtype == torch.bfloat16 and x.shape[0] >= self.ROUTER_PRODUCT_ROWS and n <= 1024 and self.hidden % 8 == 0:
            # a prompt: the scores as one matrix product (bfloat16 products are exact in float, the sums are
            # float), then the choice; the router kernel's float multiply-adds are what bounds it from here on
            kernels.route_pick(linear(x, self.router, out_dtype=torch.float32), self.top, ids, gates, self.route_mode,
                               self.correction, **self.route_opts)
        else:
            kernels.route_topk(x, self.router, self.top, ids, gates, self.route_mode, self.correction, **self.route_opts)

    def _forward_weighted(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x (tokens, hidden) -> (tokens, hidden) float32: the weighted sum of the chosen experts' results,
        identity experts and the shared expert included."""
        T, dev, E = x.shape[0], x.device, self.experts
        pairs = T * self.top
        ids = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        gates = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        self._route(x, ids, gates)
        y = None
        if E:
            # pairs that chose an identity expert are in no group; their places in perm stay zero
            perm = torch.zeros(pairs, dtype=torch.int32, device=dev)
            offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
            n_up = self.w_up.shape[1]
            u = torch.empty((pairs, n_up), dtype=x.dtype, device=dev)
            act = "none" if self.gated else self.activation
            tc = kernels.experts_tc_ok(x, self.w_up, self.w_down, pairs)
            rows = kernels.GROUP_ROWS_TC if tc else kernels.GROUP_ROWS
            tiles = torch.empty((2, kernels.group_tiles(pairs, E, rows)), dtype=torch.int32, device=dev)
            kernels.group_pairs(ids, E, perm, offsets, tiles, rows)
            if tc:
                xs = torch.empty((pairs, self.hidden), dtype=x.dtype, device=dev)
                kernels.gather_rows(x, perm, self.top, xs)
                kernels.experts_linear_tc(xs, self.w_up, u, perm, offsets, tiles, self.top, T, activation=act)
            else:
                kernels.experts_linear(x, self.w_up, u, perm, offsets, tiles, self.top, T, activation=act)
            if self.gated:
                a = torch.empty((pairs, self.inter), dtype=x.dtype, device=dev)
                kernels.gated_act(u, a, self.activation)
                u = a
            y = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
            if tc:
                kernels.experts_linear_tc(u, self.w_down, y, perm, offsets, tiles, self.top, T, down=True)
            else:
                kernels.experts_linear(u, self.w_down, y, perm, offsets, tiles, self.top, T, down=True)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
        kernels.experts_combine(y, ids, gates, E, x, shared, out, self.w_shared_gate)
        return out

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x (tokens, hidden) -> [top, tokens, hidden] float32 partial results."""
        T, dev = x.shape[0], x.device
        if x.dtype != self.router.dtype:
            x = x.to(self.router.dtype)
        if self.weighted:
            return self._forward_weighted(x, ctx)
        pairs = T * self.top
        ids = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        gates = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        if x.dtype == torch.bfloat16 and T >= self.ROUTER_PRODUCT_ROWS and self.experts <= 1024 and self.hidden % 8 == 0:
            # a prompt: the scores as one matrix product (bfloat16 products are exact in float, the sums are
            # float), then the choice; the router kernel's float multiply-adds are what bounds it from here on
            kernels.route_pick(linear(x, self.router, out_dtype=torch.float32), self.top, ids, gates)
        else:
            kernels.route_topk(x, self.router, self.top, ids, gates)
        perm = torch.empty(pairs, dtype=torch.int32, device=dev)
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        u = torch.empty((pairs, self.inter), dtype=x.dtype, device=dev)
        if kernels.experts_tc_ok(x, self.w_up, self.w_down, pairs):
            rows = kernels.GROUP_ROWS_TC
            tiles = torch.empty((2, kernels.group_tiles(pairs, self.experts, rows)), dtype=torch.int32, device=dev)
            kernels.group_pairs(ids, self.experts, perm, offsets, tiles, rows)
            xs = torch.empty((pairs, self.hidden), dtype=x.dtype, device=dev)
            kernels.gather_rows(x, perm, self.top, xs)
            kernels.experts_linear_tc(xs, self.w_up, u, perm, offsets, tiles, self.top, T, scale=gates,
                                      activation=self.activation)
            y = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
            kernels.experts_linear_tc(u, self.w_down, y, perm, offsets, tiles, self.top, T, down=True)
            return y
        tiles = torch.empty((2, kernels.group_tiles(pairs, self.experts)), dtype=torch.int32, device=dev)
        kernels.group_pairs(ids, self.experts, perm, offsets, tiles)
        kernels.experts_linear(x, self.w_up, u, perm, offsets, tiles, self.top, T, scale=gates,
                               activation=self.activation)
        y = torch.empty((self.top, T, self.hidden), dtype=torch.float32, device=dev)
        kernels.experts_linear(u, self.w_down, y, perm, offsets, tiles, self.top, T, down=True)
        return y


register_part("feedforward", "routed_experts", RoutedExperts)
