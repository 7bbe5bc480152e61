"""Position encodings."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Part, register_part


class RotaryEmbedding(Part):
    """Rotation of the pairs (i, i + rot/2) of a head by pos * theta^(-2i/rot); with ``pairing``
    "interleaved" the pair of that angle is (2i, 2i + 1) instead (the table is the same, the kernel that
    rotates is told which elements belong together).

    Frequencies as wlejon/brolm states them (src/qwen35_text.cpp:220-256);
    the pairing is the checkpoint's, see csrc/core.cu.  The table of
    (cos, sin) is computed in float64 on the host and kept as float32, so the
    angles carry no rounding of their own.

    ``stretch`` = {factor, original, fast, slow} blends stretched and plain frequencies as YaRN does (Peng et al.,
    "YaRN: Efficient Context Window Extension of Large Language Models"): with n(t) = rot ln(original / (2 pi t)) /
    (2 ln theta) the number of the dimension that makes t turns over ``original`` positions, lo = max(floor(n(fast)),
    0), hi = min(ceil(n(slow)), rot - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes
    f_i / factor * r_i + f_i (1 - r_i), and cos and sin are both multiplied by 0.1 ln(factor) + 1 (the table holds
    the products, so whoever rotates with it needs to know nothing of this).
    """

    kind = "position"

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, pairing: str = "half",
                 stretch: Optional[dict] = None):
        if stretch is not None:
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in stretch]
            if missing or not float(stretch["factor"]) > 0:
                raise ValueError(f"rotary: stretch needs a positive factor, original, fast and slow (missing: {missing})")
        self.stretch = dict(stretch) if stretch is not None else None
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary: unknown pairing '{pairing}' (half, interleaved)")
        self.pairing = pairing
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = rotary_dim or head_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.table: Optional[torch.Tensor] = None
        self._outgrown: list = []      # earlier, shorter tables: a captured step may still read them

    def prepare(self, max_positions: int, device: torch.device) -> None:
        if self.table is not None and self.table.shape[0] >= max_positions and self.table.device == device:
            return
        if self.table is not None:
            # The part is shared by every layer and by every engine of its model; a CUDA graph that an
            # earlier engine captured holds the old table's address, so the old table is never freed.
            self._outgrown.append(self.table)
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv_freq = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * i / self.rotary_dim)
        magnitude = 1.0
        if self.stretch is not None:
            st, rot = self.stretch, self.rotary_dim
            factor = float(st["factor"])

            def number(turns: float) -> float:
                return rot * math.log(float(st["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(number(float(st["fast"]))), 0)
            hi = min(math.ceil(number(float(st["slow"]))), rot - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv_freq = inv_freq / factor * ramp + inv_freq * (1.0 - ramp)
            magnitude = 0.1 * math.log(factor) + 1.0
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.table = (torch.stack([ang.cos(), ang.sin()], dim=-1) * magnitude).to(torch.float32).contiguous().to(device)


register_part("position", "rope", RotaryEmbedding)
