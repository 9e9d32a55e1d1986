"""Small Pedorax configurations for the tests, model folders with random weights for them, and
the plain implementation's logits.  The configurations differ from each other in every size and
constant; the second one sets to 1 (or makes equal) what the first one keeps apart."""

import json
import math
from pathlib import Path

import torch

import plain_pedorax


def _moe(ff, experts, top, count, keep, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, base, dims, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale, "rot": {"base": base, "dims": dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _delta(heads, kv_heads, dim, vdim, conv, a_rank, g_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "a_rank": a_rank, "g_rank": g_rank}


# delta rule with grouped q/k heads, two latents of which one is read by two layers, a layer
# without feed-forward, several groups of experts
CASE_A = {
    "architecture": "Pedorax", "vocab": 120, "width": 48, "embedding": {"scale": 1.5},
    "logit_scale": 0.75, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 8, 12, 20, 28, 3000.0, 12, 0.2),
         "mlp": _moe(20, 8, 3, 4, 2, 1.5)},
        {"type": "channel_delta", "mixer": _delta(4, 2, 12, 20, 3, 5, 7),
         "mlp": None},
        {"type": "latent_attention", "mixer": _latent(2, 16, 12, 8, 28, 3000.0, 12, 0.3, kv_from=0),
         "mlp": _moe(20, 8, 3, 4, 2, 1.5)},
        {"type": "latent_attention", "mixer": _latent(2, 8, 4, 8, 40, 777.0, 4, 0.35),
         "mlp": None},
        {"type": "channel_delta", "mixer": _delta(2, 2, 40, 36, 5, 3, 4),
         "mlp": _moe(12, 6, 2, 3, 3, 4.0)},
        {"type": "latent_attention", "mixer": _latent(5, 8, 12, 4, 28, 3000.0, 12, 0.25, kv_from=0),
         "mlp": _moe(20, 8, 3, 4, 2, 1.5)},
    ],
}

# one q/k head for all heads, one tap (no history), one group, one expert chosen, groups of one
# expert, a rotation on part of the rotated vector, scales of 1
CASE_B = {
    "architecture": "Pedorax", "vocab": 77, "width": 40, "embedding": {"scale": 1.0},
    "logit_scale": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "channel_delta", "mixer": _delta(3, 1, 8, 8, 1, 4, 4), "mlp": _moe(16, 4, 1, 1, 1, 2.5)},
        {"type": "latent_attention", "mixer": _latent(1, 16, 8, 16, 16, 50.0, 4, 1.0), "mlp": _moe(8, 5, 2, 5, 3, 9.0)},
        {"type": "channel_delta", "mixer": _delta(1, 1, 72, 8, 2, 9, 2), "mlp": _moe(16, 4, 1, 1, 1, 2.5)},
    ],
}

# only recurrent layers (no page group at all), and only attention layers (no state slot in use)
CASE_C = {
    "architecture": "Pedorax", "vocab": 50, "width": 24, "embedding": {"scale": 0.5},
    "logit_scale": -2.0, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "channel_delta", "mixer": _delta(2, 1, 8, 12, 4, 3, 3), "mlp": None},
        {"type": "channel_delta", "mixer": _delta(3, 3, 4, 4, 2, 2, 5), "mlp": _moe(8, 2, 2, 2, 2, 1.0)},
    ],
}
CASE_D = {
    "architecture": "Pedorax", "vocab": 61, "width": 28, "embedding": {"scale": 1.25},
    "logit_scale": 0.5, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(2, 4, 6, 10, 9, 100.0, 0, 0.5), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(3, 6, 6, 4, 9, 100.0, 0, 0.4, kv_from=0),
         "mlp": _moe(10, 3, 1, 3, 2, 2.0)},
        {"type": "latent_attention", "mixer": _latent(1, 6, 2, 4, 7, 9.0, 2, 0.4), "mlp": None},
    ],
}

# sizes that are multiples of 32, as the tensor-core kernels of prompt portions want them: the
# sorted experts, the tile attention, the per-head products and the low-rank second projections
CASE_E = {
    "architecture": "Pedorax", "vocab": 90, "width": 64, "embedding": {"scale": 1.0},
    "logit_scale": 0.5, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "channel_delta", "mixer": _delta(2, 1, 16, 16, 4, 32, 32), "mlp": _moe(32, 4, 3, 2, 2, 3.0)},
        {"type": "latent_attention", "mixer": _latent(4, 32, 16, 16, 32, 1000.0, 16, 0.15), "mlp": _moe(32, 4, 3, 2, 2, 3.0)},
        {"type": "latent_attention", "mixer": _latent(2, 32, 16, 32, 32, 1000.0, 16, 0.15, kv_from=1), "mlp": None},
    ],
}

CASES = {"case_a": (CASE_A, 11), "case_b": (CASE_B, 12), "case_c": (CASE_C, 13),
         "case_d": (CASE_D, 14), "case_e": (CASE_E, 15)}


class Case:
    def __init__(self, name, folder, config, seed):
        from hetero_serve_b200.weights import read_safetensors
        self.name, self.dir, self.config, self.seed = name, str(folder), config, seed
        self.raw = read_safetensors(Path(folder) / "model.safetensors")
        self.plain = plain_pedorax.prepare(self.raw)
        self.plain_bf16 = plain_pedorax.prepare(self.raw, round_to=torch.bfloat16)
        self.vocab = config["vocab"]
        self._memo = {}

    def logits(self, tokens, dtype="float32"):
        key = (tuple(tokens), dtype)
        if key not in self._memo:
            w = self.plain_bf16 if dtype == "bfloat16" else self.plain
            self._memo[key] = plain_pedorax.forward(self.config, w, tokens)
        return self._memo[key]

    def tokens(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, self.vocab, (n,), generator=g).tolist()


def make_cases(tmp_path_factory):
    from hetero_serve_b200.weights import write_model_dir
    out = {}
    for name, (cfg, seed) in CASES.items():
        folder = tmp_path_factory.mktemp(name)
        # one case is stored in bfloat16, as released checkpoints are: parts that look at the
        # stored values (a router whose numbers are bfloat16 numbers) see what they would there
        write_model_dir(folder, cfg, seed, "bfloat16" if name == "case_e" else "float32")
        stored = json.loads((folder / "config.json").read_text())
        out[name] = Case(name, folder, stored, seed)
    return out


def rms_error(got, want):
    """Root mean square of the difference with its mean taken off, over the root mean square
    of the wanted row: what a change of the logits means for the distribution behind them."""
    d = got.double() - want.double()
    d = d - d.mean()
    return math.sqrt(float((d * d).mean())) / max(1e-12, math.sqrt(float((want.double() ** 2).mean())))
