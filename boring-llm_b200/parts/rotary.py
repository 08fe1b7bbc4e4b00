"""Position encodings applied between projection and cache write."""
from __future__ import annotations

import math

import numpy as np
import torch


class RotaryTable:
    """Per-pair rotation table, as the reference builds it (src/math.br:107-113, 161-171):
    `inv_freq[j] = 1 / base^(2j / n_rot)` in 32-bit for the n_rot/2 rotated pairs, zero past them, a
    magnitude scale for cos/sin, the number of rotated pairs, and which dimensions form a pair:
    "halves" (j, j + n_rot/2) inside each head, the NEOX style of this architecture, or "interleaved"
    (2j, 2j + 1) (src/math.br:128-157, the `neox` argument). Every variant of rotary scaling is just
    another table, so the kernel never branches on the variant.
    """

    PAIR_LAYOUTS = {"halves": 0, "interleaved": 1}

    def __init__(self, head_dim: int, base: float, n_rot: int | None = None, mscale: float = 1.0,
                 pairs: str = "halves", inv_freq=None):
        """`inv_freq`: the angles per position of the rotated pairs when they are not base^(-2j / n_rot) (a scaled
        variant: `RotaryTable.yarn`)."""
        n_rot = head_dim if n_rot is None else n_rot
        if pairs not in self.PAIR_LAYOUTS:
            raise ValueError(f"rotary: pairs must be one of {sorted(self.PAIR_LAYOUTS)}, got {pairs!r}")
        self.pairs, self.pair_layout = pairs, self.PAIR_LAYOUTS[pairs]
        if n_rot % 2 != 0 or n_rot > head_dim or n_rot < 0:
            raise ValueError(f"rotary: {n_rot} rotated dimensions do not fit a head of {head_dim}")
        self.head_dim, self.base, self.n_rot, self.mscale = head_dim, float(base), n_rot, float(mscale)
        self.rot_half = n_rot // 2
        f = np.zeros(head_dim // 2, dtype=np.float32)
        j = np.arange(self.rot_half, dtype=np.float32)
        if self.rot_half:
            expo = (np.float32(2.0) * j) / np.float32(n_rot)
            f[: self.rot_half] = np.float32(1.0) / np.power(np.float32(base), expo, dtype=np.float32)
        if inv_freq is not None:
            given = np.asarray(inv_freq, dtype=np.float64)
            if given.shape != (self.rot_half,):
                raise ValueError(f"rotary: {given.shape} angles given for {self.rot_half} rotated pairs")
            f[: self.rot_half] = given.astype(np.float32)
        self.variant = None if inv_freq is None else tuple(float(v) for v in f[: self.rot_half])
        self.inv_freq_host = f
        self.inv_freq: torch.Tensor | None = None

    @classmethod
    def yarn(cls, head_dim: int, base: float, n_rot: int, factor: float, original: float, fast: float, slow: float,
             pairs: str = "halves") -> "RotaryTable":
        """Angles stretched for contexts longer than the `original` one: with f_j = base^(-2j / n_rot), pairs that make
        more than `fast` turns over `original` positions keep f_j, pairs that make fewer than `slow` turns get
        f_j / factor, and between the two pair indices lo = max(floor(p(fast)), 0) and hi = min(ceil(p(slow)), n_rot - 1),
        p(t) = n_rot ln(original / (2 pi t)) / (2 ln base), a linear ramp r_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1)
        blends them: f_j / factor * r_j + f_j (1 - r_j). cos and sin are both multiplied by 0.1 ln(factor) + 1."""
        half = n_rot // 2
        j = np.arange(half, dtype=np.float64)
        f = np.power(float(base), -2.0 * j / n_rot) if half else j

        def pair_of(turns):
            return n_rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), n_rot - 1)
        ramp = np.clip((j - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return cls(head_dim, base, n_rot=n_rot, mscale=0.1 * math.log(factor) + 1.0, pairs=pairs,
                   inv_freq=f / factor * ramp + f * (1.0 - ramp))

    def to(self, device):
        self.inv_freq = torch.from_numpy(self.inv_freq_host).to(device)
        return self

    def step_table(self, ctx):
        """(cos, sin), float32 [T, rot_half] each, of the step's tokens: worked out by the first layer that asks and
        kept in the step's memo for the others (the positions are the same for every layer)."""
        key = ("rotary table", self.head_dim, self.base, self.n_rot, self.mscale, self.variant)     # the layers' tables are equal, not the same object
        if key not in ctx.memo:
            from ..kernels import ops
            ctx.memo[key] = ops.rope_table(ctx.positions, self.inv_freq, self.rot_half, self.mscale)
        return ctx.memo[key]
