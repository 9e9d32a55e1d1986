"""The gated delta rule with a decay per head and key channel: a recurrent mixer whose
per-request state is a float32 matrix S [dim, vdim] per head, plus the last ``taps - 1`` inputs
of the short convolutions.

Per token (head h uses the q/k head h // (heads / kv_heads)):

    q, k, v  = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))     (causal, per channel)
    q, k     = unit vectors per head (sum of squares + 1e-6 under the root); q also * dim^-1/2
    beta     = sigmoid(W_b x)                                    one per head
    decay    = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 x) + dt_bias))     [heads, dim]
    S <- decay * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out      = W_o [ o / rms(o) * norm * sigmoid(W_g2 (W_g1 x)) ]

The six projections of x are one matrix product; everything behind it that enters the
recurrence is float32 in both precisions.  The inner sizes of the two low-rank pairs
(a1/a2, g1/g2) are read off the checkpoint's tensors.
"""

from __future__ import annotations

import torch

from .base import Mixer, TensorRequest, register_mixer


class ChannelDeltaRule(Mixer):
    def __init__(self, *, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int,
                 taps: int, eps: float, prefix: str):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        if taps < 1:
            raise ValueError("a short convolution has at least one tap")
        self.width, self.H, self.HK, self.D, self.V = width, n_heads, n_kv_heads, dim, vdim
        self.taps, self.eps, self.p = int(taps), float(eps), prefix
        self.channels = 2 * self.HK * self.D + self.H * self.V
        self.shape = None

    def tensor_requests(self):
        p, W = self.p, self.width
        qk, hv, hd = self.HK * self.D, self.H * self.V, self.H * self.D
        return {
            p + "q": TensorRequest((qk, W), "matrix"), p + "k": TensorRequest((qk, W), "matrix"),
            p + "v": TensorRequest((hv, W), "matrix"),
            p + "q.conv": TensorRequest((qk, self.taps), "float32"),
            p + "k.conv": TensorRequest((qk, self.taps), "float32"),
            p + "v.conv": TensorRequest((hv, self.taps), "float32"),
            p + "b": TensorRequest((self.H, W), "matrix"),
            p + "A_log": TensorRequest((self.H,), "vector"),
            p + "norm": TensorRequest((self.V,), "vector"),
            p + "a1": TensorRequest((None, W), "matrix"),
            p + "a2": TensorRequest((hd, None), "float32"),
            p + "dt_bias": TensorRequest((hd,), "vector"),
            p + "g1": TensorRequest((None, W), "matrix"),
            p + "g2": TensorRequest((hv, None), "float32"),
            p + "o": TensorRequest((W, hv), "matrix"),
        }

    def bind(self, tensors):
        p = self.p
        t = tensors
        ra, rg = t[p + "a1"].shape[0], t[p + "g1"].shape[0]
        if t[p + "a2"].shape[1] != ra or t[p + "g2"].shape[1] != rg:
            raise ValueError(f"{p}: the low-rank pairs a1/a2 or g1/g2 do not fit each other")
        self.w_in = torch.cat([t[p + "q"], t[p + "k"], t[p + "v"], t[p + "b"], t[p + "a1"],
                               t[p + "g1"]]).contiguous()
        self.conv_w = torch.cat([t[p + "q.conv"], t[p + "k.conv"], t[p + "v.conv"]]).contiguous()
        # the kernels read these two with the summed index slowest
        self.a2, self.g2 = t[p + "a2"].t().contiguous(), t[p + "g2"].t().contiguous()
        # prompt portions in bfloat16 form W_a2 a and W_g2 g as matrix products on the tensor
        # cores (the checkpoint's bfloat16 values, as stored: [out, in])
        self.a2_nk = self.g2_nk = None
        if t[p + "q"].dtype == torch.bfloat16 and ra % 32 == 0 and rg % 32 == 0:
            self.a2_nk = t[p + "a2"].to(torch.bfloat16).unsqueeze(0).contiguous()
            self.g2_nk = t[p + "g2"].to(torch.bfloat16).unsqueeze(0).contiguous()
        self.dt_bias, self.a_log, self.norm_w = t[p + "dt_bias"], t[p + "A_log"], t[p + "norm"]
        self.w_out = t[p + "o"]
        self.shape = dict(heads=self.H, kv_heads=self.HK, dim=self.D, vdim=self.V,
                          taps=self.taps, a_rank=ra, g_rank=rg)
        self.in_width = self.channels + self.H + ra + rg

    def state_shape(self):
        return (self.H * self.D * self.V + (self.taps - 1) * self.channels,)

    def forward(self, ctx, h, x, cache):
        ops, T = ctx.ops, h.shape[0]
        f32 = torch.float32
        proj = ctx.buffer("delta_proj", (T, self.in_width), f32)
        ops.linear(proj, h, self.w_in)
        qn = ctx.buffer("delta_q", (T, self.HK * self.D), f32)
        kn = ctx.buffer("delta_k", (T, self.HK * self.D), f32)
        vv = ctx.buffer("delta_v", (T, self.H * self.V), f32)
        beta = ctx.buffer("delta_beta", (T, self.H), f32)
        decay = ctx.buffer("delta_decay", (T, self.H * self.D), f32)
        state = ctx.state()
        z_a = z_g = None
        if self.a2_nk is not None and T >= 64:
            ra, rg = self.shape["a_rank"], self.shape["g_rank"]
            z_a = ctx.buffer("delta_za", (T, self.H * self.D), f32)
            ops.grouped_linear(z_a, proj, self.a2.unsqueeze(0), a_offset=self.channels + self.H,
                               a_group_stride=ra, w_nk=self.a2_nk)
            z_g = ctx.buffer("delta_zg", (T, self.H * self.V), f32)
            ops.grouped_linear(z_g, proj, self.g2.unsqueeze(0),
                               a_offset=self.channels + self.H + ra, a_group_stride=rg,
                               w_nk=self.g2_nk)
        ops.delta_prepare(qn, kn, vv, beta, decay, proj, self.conv_w, self.a2, self.dt_bias,
                          self.a_log, state, ctx.tok_req, ctx.req_start, ctx.req_len,
                          ctx.req_slot, self.shape, z_a=z_a)
        o = ctx.buffer("delta_o", (T, self.H * self.V), f32)
        ops.delta_recurrence(o, state, qn, kn, vv, beta, decay, ctx.req_start, ctx.req_len,
                             ctx.req_slot, self.shape)
        gated = ctx.buffer("delta_gated", (T, self.H * self.V), ctx.dtype)
        ops.delta_finish(gated, o, proj, self.g2, self.norm_w, ctx.tok_req, self.eps, self.shape,
                         z_g=z_g)
        ops.linear(x, gated, self.w_out, None, residual=x)


register_mixer("channel_delta_rule", ChannelDeltaRule)
