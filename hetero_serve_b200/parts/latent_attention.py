"""Causal attention whose keys and values are expanded from one shared latent per token.

Per token the cache keeps a single row for all heads: the RMS-normed latent ``c`` (``kv_rank``
numbers) and one rotated key part ``kr`` (``rot_dim`` numbers).  Head ``h`` has the key
``[W_uk[h] c | kr]`` and the value ``W_uv[h] c``; its query is ``[q_plain | q_rot]``.  Since
``q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c``, the kernels work on the latent directly:

    qa[h]  = W_uk[h]^T q_plain[h]                       (absorbed query, kv_rank numbers)
    score  = (qa[h] . c_j + q_rot[h] . kr_j) * scale    over j <= i
    weight = softmax over the scores and one sink logit per head (no key, no value)
    out[h] = W_uv[h] (sum_j weight_j c_j)

Rotary positions act on interleaved pairs of the rotated parts.  A layer built with
``shares_cache`` has no latent projection: it reads the rows another layer call wrote (the
schedule names the entry) with its own queries, expansions and sink.
"""

from __future__ import annotations

import torch

from .base import CacheRequest, Mixer, TensorRequest, register_mixer


class LatentAttention(Mixer):
    def __init__(self, *, width: int, n_heads: int, dim: int, rot_dim: int, vdim: int,
                 kv_rank: int, scale: float, rot_base: float, rot_dims: int, eps: float,
                 q_weight: str, latent_weight: str | None, latent_norm: str | None,
                 key_up: str, value_up: str, sink: str, out_weight: str,
                 shares_cache: bool = False):
        if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError(f"rot_dims must be even and at most rot_dim, got {rot_dims}")
        if shares_cache == (latent_weight is not None):
            raise ValueError("a layer either projects its own latent or shares another's")
        self.width, self.H, self.D, self.P, self.V, self.R = (width, n_heads, dim, rot_dim, vdim,
                                                              kv_rank)
        self.scale = float(torch.tensor(float(scale), dtype=torch.float64).to(torch.float32))
        self.rot_base, self.rot_dims, self.eps = float(rot_base), int(rot_dims), float(eps)
        self.names = dict(q=q_weight, dkv=latent_weight, dkv_norm=latent_norm, uk=key_up,
                          uv=value_up, sink=sink, o=out_weight)
        self.shares_cache = bool(shares_cache)
        self.q_width = self.H * (self.D + self.P)
        self.in_width = self.q_width + (0 if shares_cache else self.R + self.P)

    def tensor_requests(self):
        n = self.names
        req = {n["q"]: TensorRequest((self.q_width, self.width), "matrix"),
               n["uk"]: TensorRequest((self.H * self.D, self.R), "matrix"),
               n["uv"]: TensorRequest((self.H * self.V, self.R), "matrix"),
               n["sink"]: TensorRequest((self.H,), "vector"),
               n["o"]: TensorRequest((self.width, self.H * self.V), "matrix")}
        if not self.shares_cache:
            req[n["dkv"]] = TensorRequest((self.R + self.P, self.width), "matrix")
            req[n["dkv_norm"]] = TensorRequest((self.R,), "vector")
        return req

    def bind(self, tensors):
        n = self.names
        wq = tensors[n["q"]]
        # one input projection: the queries, then (for a layer with a latent of its own) the
        # latent and the shared key part
        self.w_in = wq if self.shares_cache else torch.cat([wq, tensors[n["dkv"]]]).contiguous()
        self.norm_w = None if self.shares_cache else tensors[n["dkv_norm"]]
        # k-major per head: [H, D, R] maps q_plain to the latent, [H, R, V] maps it to a value
        self.w_absorb = tensors[n["uk"]].view(self.H, self.D, self.R).contiguous()
        self.w_expand = tensors[n["uv"]].view(self.H, self.V, self.R).transpose(1, 2).contiguous()
        # the same two, [H, out, in], for the tensor-core form that prompt portions take
        self.w_absorb_nk = self.w_expand_nk = None
        if wq.dtype == torch.bfloat16:
            self.w_absorb_nk = self.w_absorb.transpose(1, 2).contiguous()
            self.w_expand_nk = tensors[n["uv"]].view(self.H, self.V, self.R).contiguous()
        self.sink = tensors[n["sink"]]
        self.w_out = tensors[n["o"]]
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64),
                         -2.0 * i / max(1, self.rot_dims))
        self.freq = freq.to(torch.float32).to(wq.device)

    def cache_request(self):
        return CacheRequest(kv_heads=1, head_dim=self.R + self.P, window=0, planes=1)

    def forward(self, ctx, h, x, cache):
        ops, T = ctx.ops, h.shape[0]
        H, D, P, V, R = self.H, self.D, self.P, self.V, self.R
        proj = ctx.buffer("latent_proj", (T, self.in_width), torch.float32)
        ops.linear(proj, h, self.w_in)
        # both rotations are fused: the key part turns as it is written to the page, the query
        # parts as the attention kernel reads them
        rot = dict(freq=self.freq, rot_dims=self.rot_dims) if self.rot_dims else {}
        if cache.writes:
            if self.shares_cache:
                raise RuntimeError("a layer that shares a latent cache cannot write it")
            ops.latent_append(cache.pool, proj, self.norm_w, cache.table, ctx.tok_pos,
                              ctx.tok_req, c_offset=self.q_width, rank=R, rot_dim=P,
                              eps=self.eps, page_size=cache.page_size, status=ctx.status, **rot)
        qa = ctx.buffer("latent_qa", (T, H * R), torch.float32)
        ops.grouped_linear(qa, proj, self.w_absorb, a_offset=0, a_group_stride=D + P,
                           w_nk=self.w_absorb_nk)
        lat = ctx.buffer("latent_mix", (T, H * R), torch.float32)
        ops.latent_attention(lat, qa, proj, cache.pool, cache.table, ctx.tok_pos, ctx.tok_req,
                             self.sink, n_heads=H, rank=R, rot_dim=P, qr_head_stride=D + P,
                             qr_offset=D, scale=self.scale, page_size=cache.page_size,
                             status=ctx.status, plan=ctx.plan, **rot)
        att = ctx.buffer("latent_heads", (T, H * V), ctx.dtype)
        ops.grouped_linear(att, lat, self.w_expand, w_nk=self.w_expand_nk)
        ops.linear(x, att, self.w_out, None, residual=x)


register_mixer("latent_attention", LatentAttention)
