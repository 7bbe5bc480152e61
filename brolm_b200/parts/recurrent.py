"""Mixers that carry a state of fixed size from token to token: a gated diagonal recurrence
and a selective state space, each behind a short causal convolution.

Both keep, per sequence, one float32 row of a state group: the recurrence's state first, then the
convolution's last ``taps - 1`` inputs (zeros before the sequence's start).  The row is zero when a slot is
taken, read at the start of a sequence's tokens in a step and written at their end; the same kernels serve
a prompt and a decode step, and nothing is read back to the host.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateSpec
from .base import ParamSpec, Part, register_part
from .linear import linear


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.float().contiguous()


class GatedRecurrence(Part):
    """The recurrent block of Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with Local
    Attention for Efficient Language Models") with its real-gated linear recurrent unit.

    Two branches of ``width`` channels: g = gelu_tanh(W_y x + b_y) and u = conv(W_x x + b_x), a causal
    convolution per channel with ``taps`` taps, a bias and no activation.  u is cut into ``blocks`` equal
    parts; in each, r = sigmoid(Ra u + ra) and i = sigmoid(Ri u + ri) with square matrices of the part's
    size.  Per channel: a = exp(-decay_scale * r * softplus(lam)), S <- a S + sqrt(1 - a^2) (i u), and the
    result is W_o (S g).  S, the gates, the decay and the convolution are float32 in every mode; the block
    products run over float32 rows of u (for a prompt of a bfloat16 step: over u in two bfloat16 halves, which
    keep 16 bits of it, with float sums).
    """

    kind = "mixer"
    graph_safe = True
    SPLIT_ROWS = 64          # from this many tokens on a bfloat16 step's gate products run on the tensor cores

    def __init__(self, hidden: int, width: int, blocks: int, taps: int, decay_scale: float = 8.0):
        if width % blocks:
            raise ValueError("gated recurrence: width must be a multiple of blocks")
        if taps < 1:
            raise ValueError("gated recurrence: the convolution needs at least one tap")
        self.hidden, self.width, self.blocks, self.taps = hidden, width, blocks, taps
        self.bs = width // blocks
        self.decay_scale = float(decay_scale)
        self.tail_off = width

    def param_specs(self):
        W, nb, bs = self.width, self.blocks, self.bs
        return {"y": ParamSpec((W, self.hidden)), "y_bias": ParamSpec((W,), "vector"),
                "x": ParamSpec((W, self.hidden)), "x_bias": ParamSpec((W,), "vector"),
                "conv": ParamSpec((W, self.taps), "vector"), "conv_bias": ParamSpec((W,), "vector"),
                "ra": ParamSpec((nb, bs, bs)), "ra_bias": ParamSpec((nb, bs), "vector"),
                "ri": ParamSpec((nb, bs, bs)), "ri_bias": ParamSpec((nb, bs), "vector"),
                "lam": ParamSpec((W,), "vector"), "o": ParamSpec((self.hidden, W))}

    def bind(self, params):
        kinds = {params[n].dtype for n in ("y", "x")}
        dt = torch.float32 if (len(kinds) > 1 or torch.float32 in kinds) else next(iter(kinds))
        # one product for both branches: rows [Wy; Wx]
        self.w_in = torch.cat([params["y"].to(dt), params["x"].to(dt)], dim=0).contiguous()
        self.w_o = params["o"]
        # per block the rows [Ra; Ri], as float32: the gates' products take float32 rows of u
        self.w_gates = torch.cat([params["ra"].float(), params["ri"].float()], dim=1).contiguous()
        # the same rows as stored, when stored in bfloat16: a prompt's gate products run on the tensor cores over u in
        # two bfloat16 halves (16 bits of u; the products with bfloat16 matrices are exact in float)
        self.w_gates_bf16 = None
        if params["ra"].dtype == torch.bfloat16 and params["ri"].dtype == torch.bfloat16 and self.bs % 8 == 0:
            self.w_gates_bf16 = torch.cat([params["ra"], params["ri"]], dim=1).contiguous()
        self.y_bias, self.x_bias = _f32(params["y_bias"]), _f32(params["x_bias"])
        self.conv, self.conv_bias = _f32(params["conv"]), _f32(params["conv_bias"])
        self.r_bias, self.i_bias = _f32(params["ra_bias"]).view(-1), _f32(params["ri_bias"]).view(-1)
        self.lam = _f32(params["lam"])
        self.params = {}

    def cache_spec(self):
        return StateSpec((self.width * self.taps,), torch.float32)          # S, then taps - 1 rows of inputs

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        """x (tokens, hidden) -> (tokens, hidden) float32, or partial sums [parts, tokens, hidden]."""
        if not writes_cache:
            raise NotImplementedError("a mixer with a state cannot run on another layer's state")
        T, W = x.shape[0], self.width
        state = ctx.state(entry)
        seq = (ctx.cu_q, ctx.kv_len, ctx.slots_dev, state)
        proj = linear(x, self.w_in, out_dtype=torch.float32)              # [ y_raw | x_raw ]
        x_raw = proj[:, W:]
        u = torch.empty((T, W), dtype=torch.float32, device=x.device)
        kernels.causal_conv(x_raw, self.x_bias, self.conv, self.conv_bias, "none", ctx.tok_seq, ctx.positions, *seq,
                            self.tail_off, u)
        pre_lo = None
        if kernels.block_matvec_ok(T, self.bs):
            pre = torch.empty((T, 2 * W), dtype=torch.float32, device=x.device)
            kernels.block_matvec_f32(u, self.bs, self.w_gates, pre, 2 * self.bs)       # a handful of tokens: a stream of the matrices
        elif ctx.dtype == torch.bfloat16 and self.w_gates_bf16 is not None and T >= self.SPLIT_ROWS:
            halves = torch.empty((2 * T, W), dtype=torch.bfloat16, device=x.device)
            kernels.split_halves(u, halves)
            both = torch.empty((2 * T, 2 * W), dtype=torch.float32, device=x.device)
            kernels.heads_linear(halves, self.bs, self.w_gates_bf16, both, 2 * self.bs)
            pre, pre_lo = both[:T], both[T:]
        else:
            pre = torch.empty((T, 2 * W), dtype=torch.float32, device=x.device)
            kernels.heads_linear(u, self.bs, self.w_gates, pre, 2 * self.bs)
        out = torch.empty((T, W), dtype=ctx.dtype, device=x.device)
        kernels.gated_scan(pre, u, proj[:, :W], self.y_bias, self.r_bias, self.i_bias, self.lam, self.decay_scale,
                           self.bs, ctx.positions, *seq, out, ctx.batch, ctx.max_q_len, pre_lo=pre_lo)
        kernels.conv_tail(x_raw, self.x_bias, self.taps, *seq, self.tail_off, ctx.batch)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)


register_part("mixer", "gated_recurrence", GatedRecurrence)


class StateSpace(Part):
    """The Mamba-2 mixer (Dao and Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms
    Through Structured State Space Duality").

    W_in x is laid out as [z: inner | x: inner | B: groups*N | C: groups*N | dt: heads], inner = heads * P.
    x, B and C pass a causal convolution per channel (``taps`` taps, bias) and silu.  Per head h of group
    h // (heads / groups): dt = softplus(dt + dt_bias), S <- exp(-exp(A_log) dt) S + dt B x^T (S is N x P),
    y = S^T C + D x.  Then y * silu(z), an RMS norm over each of ``norm_groups`` equal parts with a gain, and
    W_o.  S, dt, the decay and the norm are float32 in every mode.
    """

    kind = "mixer"
    graph_safe = True

    def __init__(self, hidden: int, heads: int, head_size: int, state: int, groups: int, norm_groups: int, taps: int,
                 eps: float):
        if heads % groups:
            raise ValueError("state space: heads must be a multiple of groups")
        if (heads * head_size) % norm_groups:
            raise ValueError("state space: heads * head_size must be a multiple of norm_groups")
        if state > 256:
            raise ValueError("state space: a state of more than 256 numbers per channel is beyond the kernel")
        self.hidden, self.heads, self.P, self.N, self.groups = hidden, heads, head_size, state, groups
        self.norm_groups, self.taps, self.eps = norm_groups, taps, float(eps)
        self.inner = heads * head_size
        self.conv_cols = self.inner + 2 * groups * state
        self.in_cols = 2 * self.inner + 2 * groups * state + heads
        self.tail_off = heads * head_size * state

    def param_specs(self):
        return {"in": ParamSpec((self.in_cols, self.hidden)), "conv": ParamSpec((self.conv_cols, self.taps), "vector"),
                "conv_bias": ParamSpec((self.conv_cols,), "vector"), "dt_bias": ParamSpec((self.heads,), "vector"),
                "A_log": ParamSpec((self.heads,), "vector"), "D": ParamSpec((self.heads,), "vector"),
                "norm": ParamSpec((self.inner,), "vector"), "o": ParamSpec((self.hidden, self.inner))}

    def bind(self, params):
        self.w_in, self.w_o = params["in"], params["o"]
        self.conv, self.conv_bias = _f32(params["conv"]), _f32(params["conv_bias"])
        self.dt_bias, self.a_log, self.d = _f32(params["dt_bias"]), _f32(params["A_log"]), _f32(params["D"])
        self.gain = params["norm"].contiguous()
        self.params = {}

    def cache_spec(self):
        return StateSpec((self.tail_off + (self.taps - 1) * self.conv_cols,), torch.float32)

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        if not writes_cache:
            raise NotImplementedError("a mixer with a state cannot run on another layer's state")
        T, inner = x.shape[0], self.inner
        state = ctx.state(entry)
        seq = (ctx.cu_q, ctx.kv_len, ctx.slots_dev, state)
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        raw = proj[:, inner:inner + self.conv_cols]
        xbc = torch.empty((T, self.conv_cols), dtype=torch.float32, device=x.device)
        kernels.causal_conv(raw, None, self.conv, self.conv_bias, "silu", ctx.tok_seq, ctx.positions, *seq,
                            self.tail_off, xbc)
        y = torch.empty((T, inner), dtype=torch.float32, device=x.device)
        kernels.ssm_scan(xbc, proj[:, inner + self.conv_cols:], self.dt_bias, self.a_log, self.d, self.heads, self.groups,
                         self.P, self.N, *seq, y, ctx.batch, ctx.max_q_len)
        kernels.conv_tail(raw, None, self.taps, *seq, self.tail_off, ctx.batch)
        out = torch.empty((T, inner), dtype=ctx.dtype, device=x.device)
        kernels.gate_group_norm(y, proj[:, :inner], self.gain, self.eps, self.norm_groups, out)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)


register_part("mixer", "state_space", StateSpace)


class DecayLinearAttention(Part):
    """Linear attention with one fixed decay per head ("lightning" attention).

    q = act(W_q x), k = act(W_k x) (``heads`` x ``dim``) and v = act(W_v x) (``heads`` x ``v_dim``), laid out head by
    head; per head S <- decay_h S + k v^T and o = S^T q, with no other scale.  The heads' results together pass an
    RMS norm over the whole row with a gain (``norm``), are multiplied by sigmoid(W_g x) (``gate``) and go through
    W_o.  ``decay``: one number per head.  The projection's sums, the activation, S and the norm are float32 in
    every mode; S is a state row per sequence, zero at the sequence's start."""

    kind = "mixer"
    graph_safe = True

    def __init__(self, hidden: int, heads: int, dim: int, v_dim: int, decay, eps: float, activation: str = "silu",
                 norm: bool = True, gate: bool = True):
        decay = [float(d) for d in decay]
        if len(decay) != heads:
            raise ValueError(f"decay attention: {len(decay)} decays for {heads} heads")
        if any(not 0.0 <= d <= 1.0 for d in decay):
            raise ValueError("decay attention: every decay lies between 0 and 1")
        if activation not in kernels.SCAN_ACTS:
            raise ValueError(f"decay attention: unknown activation '{activation}'")
        if dim > 512:
            raise ValueError("decay attention: more than 512 query/key entries per head are beyond the kernel")
        self.hidden, self.heads, self.dim, self.v_dim, self.decay = hidden, heads, dim, v_dim, decay
        self.eps, self.activation, self.has_norm, self.has_gate = float(eps), activation, bool(norm), bool(gate)
        self.qk_cols, self.v_cols = heads * dim, heads * v_dim

    def param_specs(self):
        specs = {"q": ParamSpec((self.qk_cols, self.hidden)), "k": ParamSpec((self.qk_cols, self.hidden)),
                 "v": ParamSpec((self.v_cols, self.hidden)), "o": ParamSpec((self.hidden, self.v_cols))}
        if self.has_gate:
            specs["g"] = ParamSpec((self.v_cols, self.hidden))
        if self.has_norm:
            specs["norm"] = ParamSpec((self.v_cols,), "vector")
        return specs

    def bind(self, params):
        names = ("q", "k", "v") + (("g",) if self.has_gate else ())
        kinds = {params[n].dtype for n in names}
        dt = torch.float32 if (len(kinds) > 1 or torch.float32 in kinds) else next(iter(kinds))
        # one product for q, k, v and the gate's logits: rows [Wq; Wk; Wv; Wg]
        self.w_in = torch.cat([params[n].to(dt) for n in names], dim=0).contiguous()
        self.w_o = params["o"]
        self.gain = params["norm"].contiguous() if self.has_norm else None
        # decay - 1, taken in double: what a float keeps of it is far finer than what it keeps of the decay itself
        self.decay_m1 = torch.tensor([d - 1.0 for d in self.decay], dtype=torch.float64).to(torch.float32) \
            .to(self.w_in.device)
        self.params = {}

    def cache_spec(self):
        return StateSpec((kernels.decay_state_size(self.heads, self.dim, self.v_dim),), torch.float32)

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        """x (tokens, hidden) -> (tokens, hidden) float32, or partial sums [parts, tokens, hidden]."""
        if not writes_cache:
            raise NotImplementedError("a mixer with a state cannot run on another layer's state")
        T = x.shape[0]
        proj = linear(x, self.w_in, out_dtype=torch.float32)              # [ q | k | v | gate logits ]
        y = torch.empty((T, self.v_cols), dtype=torch.float32, device=x.device)
        act = self.activation
        if act != "none" and ctx.max_q_len > 1:
            # a prompt: every block of a head's scan would apply the activation to the head's q and k anew, so it
            # is applied once, in place, by a pass of its own; a step of single tokens leaves it to the scan
            qkv = proj[:, :2 * self.qk_cols + self.v_cols]
            kernels.bias_act(qkv, None, act, qkv)
            act = "none"
        kernels.decay_scan(proj, 0, self.qk_cols, 2 * self.qk_cols, self.heads, self.dim, self.v_dim, act,
                           self.decay_m1, ctx.cu_q, ctx.kv_len, ctx.slots_dev, ctx.state(entry), y, ctx.batch, ctx.max_q_len)
        if self.has_norm or self.has_gate:
            out = torch.empty((T, self.v_cols), dtype=ctx.dtype, device=x.device)
            if self.has_gate:
                kernels.norm_sigmoid_gate(y, proj[:, 2 * self.qk_cols + self.v_cols:], self.gain, self.eps, out)
            else:
                kernels.rmsnorm(y, self.gain, self.eps, 0.0, out)
        else:
            out = y if ctx.dtype == torch.float32 else y.to(ctx.dtype)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)


register_part("mixer", "decay_attention", DecayLinearAttention)


class SideBySide(Part):
    """Two mixers that read the same input; the result is left_scale * left + right_scale * right.
    Each keeps what it keeps: the pair's cache spec is the tuple of both."""

    kind = "mixer"

    def __init__(self, left: Part, right: Part, left_scale: float = 1.0, right_scale: float = 1.0):
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def cache_spec(self):
        return (self.left.cache_spec(), self.right.cache_spec())

    def prepare(self, max_positions, device):
        self.left.prepare(max_positions, device)
        self.right.prepare(max_positions, device)

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        a = self.left.forward(x, ctx, entry.parts[0], writes_cache)
        b = self.right.forward(x, ctx, entry.parts[1], writes_cache)
        out = torch.empty(a.shape[-2:], dtype=torch.float32, device=x.device)
        kernels.scaled_sum(a, self.left_scale, b, self.right_scale, out)
        return out


register_part("mixer", "side_by_side", SideBySide)
