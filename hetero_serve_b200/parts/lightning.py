"""Lightning attention: linear attention with a constant decay per head, a recurrent mixer
whose per-request state is one float32 matrix S [dim, vdim] per head.

Per token:

    q, k = silu(W_q x), silu(W_k x)   [heads, dim];   v = silu(W_v x)   [heads, vdim]
    S_h <- decay_h * S_h + k_h v_h^T ;   o_h = S_h^T q_h
    out = W_o [ rms(o_0 .. o_H-1) * w_norm * sigmoid(W_g x) ]      (one norm over all heads)

The four projections of x are one product; the activations, the state, the norm and the gate
are float32 in both precisions.  The state starts at zero (the runner clears a slot when a
request is opened) and is carried from step to step.  Like the attention beside it, the mixer
can run on a slice of a wider projection (``input_projection`` / ``forward_projected``).
"""

from __future__ import annotations

import torch

from .base import Mixer, TensorRequest, register_mixer


class LightningAttention(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, n_heads: int, dim: int, vdim: int, decay, eps: float,
                 prefix: str):
        decay = [float(d) for d in decay]
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        self.width, self.H, self.D, self.V = width, n_heads, dim, vdim
        self.decay_values, self.eps, self.p = decay, float(eps), prefix
        self.n_in = 2 * self.H * self.D + 2 * self.H * self.V             # q | k | v | gate

    def tensor_requests(self):
        p, W, hd, hv = self.p, self.width, self.H * self.D, self.H * self.V
        return {p + "q": TensorRequest((hd, W), "matrix"), p + "k": TensorRequest((hd, W), "matrix"),
                p + "v": TensorRequest((hv, W), "matrix"), p + "g": TensorRequest((hv, W), "matrix"),
                p + "o": TensorRequest((W, hv), "matrix"), p + "norm": TensorRequest((hv,), "vector")}

    def bind(self, tensors):
        p, t = self.p, tensors
        pad = -self.n_in % 8
        w = [t[p + "q"], t[p + "k"], t[p + "v"], t[p + "g"]]
        if pad:
            w.append(w[0].new_zeros(pad, self.width))
        self.w_in = torch.cat(w).contiguous()
        self.norm_w, self.w_out = t[p + "norm"], t[p + "o"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_out.device)

    def state_shape(self):
        return (self.H * self.D * self.V,)

    def input_projection(self):
        return self.w_in, None

    def forward_projected(self, ctx, h, proj, offset, out, cache, accumulate=False):
        ops, T = ctx.ops, h.shape[0]
        hd, hv = self.H * self.D, self.H * self.V
        o = ctx.buffer("lightning_o", (T, hv), torch.float32)
        ops.lightning_recurrence(o, ctx.state(), proj, self.decay, ctx.req_start, ctx.req_len,
                                 ctx.req_slot, q_off=offset, k_off=offset + hd,
                                 v_off=offset + 2 * hd, heads=self.H, dim=self.D, vdim=self.V,
                                 act="silu")
        gated = ctx.buffer("lightning_gated", (T, hv), ctx.dtype)
        ops.rms_norm(gated, o, self.norm_w, self.eps, gate=proj, gate_offset=offset + 2 * hd + hv)
        ops.linear(out, gated, self.w_out, None, residual=out if accumulate else None)

    def forward(self, ctx, h, x, cache, fresh=False):
        proj = ctx.buffer("lightning_proj", (h.shape[0], self.w_in.shape[0]), torch.float32)
        ctx.ops.linear(proj, h, self.w_in)
        self.forward_projected(ctx, h, proj, 0, x, cache, accumulate=not fresh)


register_mixer("lightning_attention", LightningAttention)
