"""Rotary position encoding, rotate-half form (reference: engine/engine.py:113-122).

The part owns the angle tables; the rotation itself is fused into the kernel that also
normalises q/k heads and writes the cache, which takes the tables as arguments. Another position
encoding is another part: with ``fused_tables = True`` and ``tables(n)`` (cos, sin [n, dim/2]
float32) if the fused kernel can use it, or with ``apply(qkv, ctx, n_heads, n_kv_heads, head_dim)``
for one that rewrites the q and k heads of the projection rows [tokens, (nh + 2 nkv) * hd] in place
itself; the attention part then runs the fused kernel without rotation. ``apply`` runs before the
cache write and cannot be combined with a per-head q/k norm (which would have to come first): the
attention part refuses that pair."""
import torch

from ..config.specs import RotaryHalfSpec, RotaryPairsSpec, RotaryPartSpec, SinusoidSpec
from .base import Part, register_part


class RotaryHalf(Part):
    fused_tables = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self._n = 0
        self._cos = self._sin = None

    def tables(self, n):
        """cos, sin [>= n, dim/2] float32: angle(p, j) = p * theta^(-2j/dim), computed in float32."""
        if n > self._n:
            n = max(n, 2 * self._n, 256)
            dim, theta = self.spec.dim, self.spec.theta
            inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=self.rt.device, dtype=torch.float32) / dim))
            ang = torch.outer(torch.arange(n, device=self.rt.device, dtype=torch.float32), inv)
            self._cos, self._sin, self._n = ang.cos().contiguous(), ang.sin().contiguous(), n
        return self._cos, self._sin


register_part(RotaryHalfSpec, RotaryHalf)


class Sinusoid(Part):
    """Absolute sinusoidal position vector, added to the embedding by the embedding kernel. The part
    owns the frequencies base^(-2i/dim), worked out in float64 on the host; the kernel forms
    position * frequency in float64 too, so the angle is right to float32 rounding at any position."""
    added_to_embedding = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        i = torch.arange(spec.dim // 2, dtype=torch.float64)
        self.inv_freq = (float(spec.base) ** (-2.0 * i / spec.dim)).to(rt.device)


register_part(SinusoidSpec, Sinusoid)


class RotaryPart(Part):
    """Angle tables of a rotation over the first ``dim`` coordinates of a head: frequencies base^(-2i/dim) made
    in float64 and rounded to float32 once, angle = float32(position) * frequency in float32, its cosine and
    sine taken in float64 and rounded. The mixer that owns the part hands the tables and ``dim`` to the kernel
    that rotates (``csrc.api.conv_norm_rope``)."""
    fused_tables = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.dim % 2 or spec.dim < 0:
            raise ValueError(f"a rotation over {spec.dim} coordinates: the number must be even")
        self._n = 0
        self._cos = self._sin = None

    def tables(self, n):
        """cos, sin [>= n, dim/2] float32."""
        if n > self._n:
            n = max(n, 2 * self._n, 256)
            dim = self.spec.dim
            i = torch.arange(dim // 2, dtype=torch.float64)
            freq = (float(self.spec.base) ** (-2.0 * i / dim)).to(torch.float32)
            ang = (torch.arange(n, dtype=torch.float32)[:, None] * freq[None, :]).to(torch.float64)
            self._cos = ang.cos().to(torch.float32).to(self.rt.device).contiguous()
            self._sin = ang.sin().to(torch.float32).to(self.rt.device).contiguous()
            self._n = n
        return self._cos, self._sin


register_part(RotaryPartSpec, RotaryPart)


class RotaryPairs(RotaryPart):
    """The same angle tables for a rotation of neighbouring pairs (coordinate 2i with 2i + 1) over the first ``dim``
    coordinates; the kernel of the mixer that owns the part turns the pairs."""
    pairs = True


register_part(RotaryPairsSpec, RotaryPairs)
