"""Dynamic Tanh: a norm that takes no statistic of the row,

    y = tanh(alpha * x) * weight + bias,

with one learned scalar ``alpha`` beside the weight and bias vectors.
"""

from __future__ import annotations

from .base import Norm, TensorRequest, register_norm


class DynamicTanh(Norm):
    def __init__(self, *, width: int, weight: str, bias: str, alpha: str):
        self.width = width
        self.wn, self.bn, self.an = weight, bias, alpha
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensor_requests(self):
        return {self.wn: TensorRequest((self.width,), "vector"),
                self.bn: TensorRequest((self.width,), "vector"),
                self.an: TensorRequest((), "vector")}

    def bind(self, tensors):
        self.weight, self.bias = tensors[self.wn], tensors[self.bn]
        self.alpha = float(tensors[self.an])          # one number: handed to the kernel by value

    def forward(self, ctx, out, x, rows=None):
        ctx.ops.dyt_norm(out, x, self.weight, self.bias, self.alpha, rows)


register_norm("dynamic_tanh", DynamicTanh)
