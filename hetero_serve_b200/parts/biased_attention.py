"""Softmax attention with a learned bias of the distance, a tanh cap on the scores and a chunked
causal mask, over the paged cache.

Per token (query head h uses key/value head h // (heads / kv_heads)):

    q = W_q x + b_q,  k = W_k x + b_k            the values are the keys as projected: v = k
    qn = q / rms(q) * w_qn,  kn = k / rms(k) * w_kn      each over its WHOLE projection, all
                                                         heads at once (``qk_norm``)
    score(i, j) = cap * tanh((qn_i . kn_j) * scale / cap) + rel[bucket(i - j), h]
    visible: j <= i and floor(i / chunk) == floor(j / chunk)   (chunks counted from position 0)
    o_h = softmax(score) v * sigmoid(W_g x)_h ;   out = W_o [o_0 .. o_H-1] + b_o

``rel`` has B rows: the first B / 2 are the exact distances 0 .. B/2 - 1, the others grow
logarithmically up to ``bias_max``:  bucket(n) = min(B - 1, B/2 + floor(ln(n / (B/2)) /
ln(bias_max / (B/2)) * (B - B/2))).  The rows are expanded once at binding into a table
[heads, distances] (float64 on the host), as far as a query can see: a chunk, or the model's
positions.

The cache keeps two planes per token and key/value head: the normed keys and the values (the
un-normed keys), so the attention kernel reads what any attention kernel reads; the cache
manager gives the pages of chunks that have passed back at once.  q, k and the
gate's logits are ONE product; norms, scores, softmax and the gate are float32 in both
precisions.  The mixer can also run on a slice of a wider projection that a mixer around it
formed (``input_projection`` / ``forward_projected``).
"""

from __future__ import annotations

import math

import torch

from .base import CacheRequest, Mixer, TensorRequest, register_mixer


def distance_buckets(n_dist: int, rows: int, far: float) -> list[int]:
    """Row of the bias table for every distance 0 .. n_dist - 1."""
    half = rows // 2
    out = []
    for n in range(n_dist):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
            continue
        step = math.floor(math.log(n / half) / math.log(far / half) * (rows - half))
        out.append(min(rows - 1, half + step))
    return out


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class BiasedChunkAttention(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, softcap: float, chunk: int, bias_max: float, eps: float,
                 max_distance: int, prefix: str, window: int = 0, qk_norm: bool = True):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        if chunk < 0 or window < 0 or softcap < 0:
            raise ValueError("chunk, window and softcap are not negative (0: none)")
        self.width, self.H, self.G, self.D = width, n_heads, n_kv_heads, head_dim
        self.scale, self.cap = float(scale), float(softcap)
        self.chunk, self.window = int(chunk), int(window)
        self.bias_max, self.eps, self.p = float(bias_max), float(eps), prefix
        self.qk_norm = bool(qk_norm)
        reach = [n for n in (self.chunk, self.window, int(max_distance)) if n > 0]
        self.n_dist = max(1, min(reach)) if reach else 1      # distances a query can see
        self.n_in = self.H * self.D + self.G * self.D + self.H          # q | k | gate logits

    def tensor_requests(self):
        p, W, qw, kw = self.p, self.width, self.H * self.D, self.G * self.D
        req = {p + "q": TensorRequest((qw, W), "matrix"), p + "q.b": TensorRequest((qw,), "vector"),
               p + "k": TensorRequest((kw, W), "matrix"), p + "k.b": TensorRequest((kw,), "vector"),
               p + "rel": TensorRequest((None, self.H), "float32"),
               p + "g": TensorRequest((self.H, W), "matrix"),
               p + "o": TensorRequest((W, qw), "matrix"), p + "o.b": TensorRequest((W,), "vector")}
        if self.qk_norm:
            req[p + "q.norm"] = TensorRequest((qw,), "vector")
            req[p + "k.norm"] = TensorRequest((kw,), "vector")
        return req

    def bind(self, tensors):
        p, t = self.p, tensors
        pad = _pad8(self.n_in) - self.n_in
        w = [t[p + "q"], t[p + "k"], t[p + "g"]]
        b = [t[p + "q.b"], t[p + "k.b"], t[p + "q.b"].new_zeros(self.H + pad)]
        if pad:
            w.append(w[0].new_zeros(pad, self.width))
        self.w_in, self.b_in = torch.cat(w).contiguous(), torch.cat(b).contiguous()
        self.w_qn = t[p + "q.norm"] if self.qk_norm else None
        self.w_kn = t[p + "k.norm"] if self.qk_norm else None
        rel = t[p + "rel"]
        rows = distance_buckets(self.n_dist, rel.shape[0], self.bias_max)
        self.bias = rel[torch.tensor(rows, device=rel.device)].t().contiguous()   # [H, n_dist]
        self.w_out, self.b_out = t[p + "o"], t[p + "o.b"]

    def cache_request(self):
        return CacheRequest(self.G, self.D, self.window, 2, self.chunk)

    def input_projection(self):
        """(weight [n, width], bias [n]) of this mixer's columns in a projection of the input;
        n is a multiple of 8."""
        return self.w_in, self.b_in

    def forward_projected(self, ctx, h, proj, offset, out, cache, accumulate=False):
        ops, T = ctx.ops, h.shape[0]
        qw, kw = self.H * self.D, self.G * self.D
        q = ctx.buffer("biased_q", (T, qw), ctx.dtype)
        ops.qk_prepare(q, cache.pool, proj, self.w_qn, self.w_kn, cache.table, ctx.tok_pos,
                       ctx.tok_req, q_off=offset, k_off=offset + qw, v_off=None, eps=self.eps,
                       writes=cache.writes, n_heads=self.H, n_kv_heads=self.G, head_dim=self.D,
                       page_size=cache.page_size, status=ctx.status)
        att = ctx.buffer("biased_att", (T, qw), ctx.dtype)
        ops.biased_attention(att, q, cache.pool, cache.table, ctx.tok_pos, ctx.tok_req,
                             bias=self.bias, gate=proj, gate_offset=offset + qw + kw,
                             n_heads=self.H, n_kv_heads=self.G, head_dim=self.D,
                             page_size=cache.page_size, scale=self.scale, cap=self.cap,
                             chunk=self.chunk, window=self.window, status=ctx.status,
                             plan=getattr(ctx, "plan", None))
        ops.linear(out, att, self.w_out, self.b_out, residual=out if accumulate else None)

    def forward(self, ctx, h, x, cache, fresh=False):
        proj = ctx.buffer("biased_proj", (h.shape[0], self.w_in.shape[0]), torch.float32)
        ctx.ops.linear(proj, h, self.w_in, self.b_in)
        self.forward_projected(ctx, h, proj, 0, x, cache, accumulate=not fresh)


register_mixer("biased_chunk_attention", BiasedChunkAttention)
