"""Rotary position encoding (pyre/model.py:41-63): half-split pairs, theta from the
configuration, angles in fp32."""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import HeadGeometry, PositionEncoding, register_part


class Rotary(PositionEncoding):
    """inv_freq[j] = theta^(-2j / rotary_dim) for j < rotary_dim / 2, computed with the
    reference's fp32 expression (pyre/model.py:45-47), or in 64-bit rounded once (``exact_frequencies``); per step, cos and sin of
    float(position) * inv_freq for the step's tokens, shared by all layers that have
    the same settings.  ``rotary_dim`` < head_dim rotates only the first dims of a head.  Bias, rotation of
    q and k and the paged write of k and v are one kernel (``ops.qkv_rope_write``).

    ``scaling``: ``{"factor", "low", "high", "original"}`` stretches the slow frequencies for contexts beyond the
    ``original`` length: with the wavelength l = 2 pi / f, a frequency stays where l < original / high, becomes
    f / factor where l > original / low, and between the two is the blend (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low).  Computed once, in 64-bit.

    ``scaling`` with the keys ``{"factor", "original", "fast", "slow"}`` is another rule: with d(t) = rotary_dim
    ln(original / (2 pi t)) / (2 ln theta), the pair index whose wave turns t times within ``original`` positions,
    lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and the ramp r_j = clamp((j - lo) /
    max(hi - lo, 0.001), 0, 1), pair j gets the frequency f_j / factor * r_j + f_j (1 - r_j), and cos and sin are
    multiplied by the amplitude 0.1 ln(factor) + 1."""

    graph_safe = True

    def __init__(self, dtype, device, head_dim: int, theta: float, rotary_dim: "int | None" = None,
                 pairing: str = "half", exact_frequencies: bool = False, scaling: "dict | None" = None):
        super().__init__(dtype, device)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        self.theta = float(theta)
        if pairing not in ("half", "interleaved"):
            raise ops.UnsupportedSize(f"rotary pairing {pairing!r}: known are 'half' and 'interleaved'")
        # "half" pairs dims (j, j + rotary_dim / 2), "interleaved" pairs neighbours (2j, 2j + 1); the angles are the
        # same.  The fused q/k/v kernels of ``apply`` rotate half-split pairs only; a mixer with a kernel of its own
        # takes the tables (``rotation``) and ``pairing``.
        self.pairing = pairing
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ops.UnsupportedSize(f"rotary_dim {self.rotary_dim} must be even and <= head_dim")
        if exact_frequencies:
            # theta^(-2j / rotary_dim) in 64-bit, rounded once to fp32
            inv = (self.theta ** (-torch.arange(0, self.rotary_dim, 2, dtype=torch.float64) / self.rotary_dim)).float()
        else:
            inv = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
        self.scaling = None
        self.amplitude = 1.0
        if scaling and ("fast" in scaling or "slow" in scaling):
            try:
                fac, orig, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
            except KeyError as e:
                raise ValueError(f"rotary scaling needs factor, original, fast and slow; {e.args[0]!r} is missing") from None
            if not (fac > 0 and orig > 0 and fast > 0 and slow > 0 and self.theta > 1):
                raise ValueError(f"rotary scaling {scaling!r}: factor, original, fast and slow are positive")
            self.scaling = ("turns", fac, orig, fast, slow)
            f = self.theta ** (-torch.arange(0, self.rotary_dim, 2, dtype=torch.float64) / self.rotary_dim)

            def turn_index(t):
                return self.rotary_dim * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(turn_index(fast)), 0)
            hi = min(math.ceil(turn_index(slow)), self.rotary_dim - 1)
            ramp = ((torch.arange(self.rotary_dim // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            inv = (f / fac * ramp + f * (1.0 - ramp)).float()
            self.amplitude = 0.1 * math.log(fac) + 1.0
        elif scaling:
            try:
                fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            except KeyError as e:
                raise ValueError(f"rotary scaling needs factor, low, high and original; {e.args[0]!r} is missing") from None
            if not (fac > 0 and hi > lo and orig > 0):
                raise ValueError(f"rotary scaling {scaling!r}: factor and original are positive, high is above low")
            self.scaling = (fac, lo, hi, orig)
            f = inv.double() if not exact_frequencies else self.theta ** (-torch.arange(0, self.rotary_dim, 2, dtype=torch.float64) / self.rotary_dim)
            wave = 2.0 * math.pi / f
            s = (orig / wave - lo) / (hi - lo)
            blend = (1.0 - s) * f / fac + s * f
            inv = torch.where(wave > orig / lo, f / fac, torch.where(wave < orig / hi, f, blend)).float()
        self.inv_freq = inv.to(self.device)
        self._key = ("rotary", self.rotary_dim, self.theta, bool(exact_frequencies), self.scaling)

    def kernel_libraries(self):
        return ["elementwise"] + (["seqmix"] if self.amplitude != 1.0 else [])

    def tables(self, ctx):
        tab = ctx.scratch.get(self._key)
        if tab is None:
            tab = ops.rope_table(ctx.positions, self.inv_freq)
            if self.amplitude != 1.0:
                for t in tab:
                    ops.scale_cap(t, self.amplitude)
            ctx.scratch[self._key] = tab
        return tab


    def rotation(self, ctx, qk_dim: int):
        if qk_dim != self.head_dim:
            raise ValueError(f"rotary part built for head_dim {self.head_dim}, used with {qk_dim}")
        cos, sin = self.tables(ctx)
        return cos, sin, self.rotary_dim

    def apply_layout(self, ctx, proj, layout, q_norm, k_norm, norm_eps, kv, cache_layer, **kw):
        if self.pairing != "half":
            raise ops.UnsupportedSize("the q/k/v kernels rotate half-split pairs only")
        return super().apply_layout(ctx, proj, layout, q_norm, k_norm, norm_eps, kv, cache_layer, **kw)

    def apply(self, ctx, qkv, bias, heads: HeadGeometry, kv, cache_layer):
        if self.pairing != "half":
            raise ops.UnsupportedSize("the q/k/v kernels rotate half-split pairs only")
        if heads.head_dim != self.head_dim:
            raise ValueError(f"rotary part built for head_dim {self.head_dim}, used with {heads.head_dim}")
        cos, sin = self.tables(ctx)
        return ops.qkv_rope_write(qkv, bias, cos, sin, cache_layer, kv.slot_mapping, heads.n_heads, heads.n_kv_heads,
                                  heads.head_dim, self.rotary_dim, kv.page_size)


class NoPosition(PositionEncoding):
    """No position encoding: queries and keys are used as projected."""

    graph_safe = True

    def __init__(self, dtype, device):
        super().__init__(dtype, device)

    def kernel_libraries(self):
        return ["elementwise"]


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
