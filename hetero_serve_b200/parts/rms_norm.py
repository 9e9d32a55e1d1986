"""Root-mean-square norm: ``y = x / sqrt(mean(x^2) + eps) * weight`` (``one_plus``: times
``1 + weight``), statistics in float32.

Besides the usual ``forward`` (normalise rows of the stream for a part that reads them) it can
be applied to a sublayer's OUTPUT and added into the stream in one pass (``add_normed``), which
is what an arrangement with norms behind its sublayers calls.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import Norm, TensorRequest, register_norm


@dataclass
class NormedPair:
    """A sublayer output that is not formed yet: ``mix * (rms(a) * wa + rms(b) * wb)`` of two
    float32 blocks [T, width].  A mixer may hand this to the arrangement instead of writing
    its output, so that the norm behind the sublayer forms it on the way."""

    a: torch.Tensor
    wa: torch.Tensor
    b: torch.Tensor
    wb: torch.Tensor
    mix: float
    eps: float


class RMSNorm(Norm):
    def __init__(self, *, width: int, eps: float, weight: str, one_plus: bool = False):
        self.width, self.eps, self.wn = width, float(eps), weight
        self.one_plus = bool(one_plus)
        self.weight = None

    def tensor_requests(self):
        return {self.wn: TensorRequest((self.width,), "vector")}

    def bind(self, tensors):
        self.weight = tensors[self.wn]
        # the fused add takes plain weights: one-plus weights are formed once
        self.add_weight = (1.0 + self.weight) if self.one_plus else self.weight

    def forward(self, ctx, out, x, rows=None):
        ctx.ops.rms_norm(out, x, self.weight, self.eps, rows, one_plus=self.one_plus)

    def add_normed(self, ctx, x, y, h=None):
        """x += norm(y), where ``y`` is a float32 block or a :class:`NormedPair`; ``h``, if
        given, receives the new rows of x in the compute type."""
        if isinstance(y, NormedPair):
            ctx.ops.rms_norm_add(x, y.a, self.add_weight, self.eps, h=h, b=y.b, wa=y.wa,
                                 wb=y.wb, mix=y.mix, eps_in=y.eps)
        else:
            ctx.ops.rms_norm_add(x, y, self.add_weight, self.eps, h=h)


register_norm("rms_norm", RMSNorm)
