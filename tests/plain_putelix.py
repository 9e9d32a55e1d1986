"""A plain, slow implementation of the Putelix decoder, one function per mechanism, written
from the design's equations in float64.  It is the oracle of the tests: it shares no code
with the package, processes a whole sequence at once (the recurrent half of the mixer token
by token) and keeps no cache.

Notation: ``h`` is a [T, width] block of rows of the residual stream, matrices are stored
[out, in] and applied as ``h @ W.T``; ``w`` maps tensor names to float64 tensors and ``pre``
is the prefix of a layer's tensors.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def prepare(raw, round_to=None):
    """float64 copies of the stored tensors; ``round_to`` rounds matrices to that type first,
    as a model bound for it holds them."""
    out = {}
    for name, t in raw.items():
        if not t.dtype.is_floating_point:
            out[name] = t.clone()
            continue
        if round_to is not None and t.dim() >= 2:
            t = t.to(round_to)
        out[name] = t.to(F64)
    return out


# ---------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------

def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance table for a key ``n`` positions back: the first half of the rows
    are exact distances, the other half grow logarithmically up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    step = math.floor(math.log(n / half) / math.log(far / half) * (rows - half))
    return min(rows - 1, half + step)


# ---------------------------------------------------------------------------------------
# the two halves of the mixer
# ---------------------------------------------------------------------------------------

def chunk_attention(h, w, pre, m, eps):
    """Softmax attention inside chunks of ``mask.size`` positions.  Keys double as values
    (the values are the projected keys before their norm); queries and keys are RMS-normed
    over their whole projection; the score is scaled, soft-capped by a tanh and shifted by a
    learned bias of the distance; every head's output is gated by a sigmoid of the input."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = h @ w[pre + "q"].T + w[pre + "q.b"]
    k = h @ w[pre + "k"].T + w[pre + "k.b"]
    v = k.view(T, G, D)
    qn = rms_norm(q, w[pre + "q.norm"], eps).view(T, H, D)
    kn = rms_norm(k, w[pre + "k.norm"], eps).view(T, G, D)
    rel = w[pre + "rel"]
    B = rel.shape[0]
    gate = torch.sigmoid(h @ w[pre + "g"].T)                        # [T, H]
    cap, chunk = float(m["softcap"]), int(m["mask"]["size"])
    out = torch.zeros(T, H, D, dtype=F64)
    for i in range(T):
        first = i // chunk * chunk
        for head in range(H):
            g = head // (H // G)
            s = (kn[first:i + 1, g] @ qn[i, head]) * m["scale"]
            s = cap * torch.tanh(s / cap)
            s = s + torch.stack([rel[distance_bucket(i - j, B, m["bias_max"]), head]
                                 for j in range(first, i + 1)])
            p = torch.softmax(s, 0)
            out[i, head] = (p[:, None] * v[first:i + 1, g]).sum(0) * gate[i, head]
    return out.reshape(T, H * D) @ w[pre + "o"].T + w[pre + "o.b"]


def lightning_attention(h, w, pre, m, eps, state=None):
    """Linear attention with a constant decay per head: S <- decay S + k v^T, o = S^T q,
    token after token; the heads' outputs are RMS-normed together, gated and projected."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].T).view(T, H, D)
    k = silu(h @ w[pre + "k"].T).view(T, H, D)
    v = silu(h @ w[pre + "v"].T).view(T, H, V)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        for head in range(H):
            S[head] = m["decay"][head] * S[head] + torch.outer(k[t, head], v[t, head])
            o[t, head] = S[head].T @ q[t, head]
    y = rms_norm(o.reshape(T, H * V), w[pre + "norm"], eps)
    y = y * torch.sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


def paired_mixer(h, w, pre, m, eps):
    """Both halves read the same rows; each result is RMS-normed over the width with a weight
    of its own, and the mixer's output is half their sum."""
    a = chunk_attention(h, w, pre + "left.", m["left"], eps)
    b = lightning_attention(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms_norm(a, w[pre + "left.out"], eps) + rms_norm(b, w[pre + "right.out"], eps))


# ---------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------

def dense_feed_forward(h, w, pre):
    u = torch.relu(h @ w[pre + "up"].T)
    return (u * u) @ w[pre + "down"].T


def gated_expert(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(z, top):
    """The ``top`` largest logits of each row (the lower index wins a tie) and the softmax
    over the chosen logits alone."""
    idx = torch.zeros(z.shape[0], top, dtype=torch.long)
    for t in range(z.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))
        idx[t] = torch.tensor(order[:top])
    chosen = torch.gather(z, 1, idx)
    return idx, torch.softmax(chosen, 1)


def routed_feed_forward(h, w, pre, f):
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    idx, weights = route(z, f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += weights[t, j] * gated_expert(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if f.get("shared") is not None:
        s = torch.sigmoid(h @ w[pre + "shared.sg"].T)               # [T, 1]
        out = out + s * gated_expert(h, w, pre + "shared.")
    return out


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0; with ``return_layers`` also the
    residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    x = w["embed"][ids] + w["pos"][:T]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        assert layer["type"] == "parallel"
        x = x + rms_norm(paired_mixer(x, w, pre + "mix.", layer["mixer"], eps), w[pre + "norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                y = dense_feed_forward(x, w, pre + "mlp.")
            else:
                y = routed_feed_forward(x, w, pre + "mlp.", f)
            x = x + rms_norm(y, w[pre + "norm2"], eps)
        layers.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, layers) if return_layers else logits
