"""Small Putelix configurations for the tests, with random weights written to temporary folders,
and the plain implementation's view of the same weights."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

import plain_putelix


def _left(heads, kv_heads, dim, chunk, scale, softcap, bias_max, bias_rows):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
            "softcap": softcap, "bias_max": bias_max, "bias_rows": bias_rows,
            "mask": {"size": chunk}}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def _moe(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layer(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _model(vocab, width, max_positions, eps, layers):
    return {"architecture": "Putelix", "vocab": vocab, "width": width,
            "max_positions": max_positions, "norm": {"eps": eps}, "layers": layers}


# chunks that are no multiple of a page (16), grouped query heads, a table whose logarithmic
# half saturates inside a chunk, three kinds of feed-forward, layers that differ from each other
CASE_A = _model(320, 48, 300, 1e-5, [
    _layer(_left(4, 2, 16, 24, 0.3, 8.0, 20, 10), _right(3, 8, 12, [0.5, 0.9, 0.99]),
           {"kind": "dense", "ff": 80}),
    _layer(_left(6, 3, 8, 37, 0.5, 3.0, 30, 14), _right(2, 16, 8, [0.97, 0.7]),
           _moe(24, 5, 2, shared=40)),
    _layer(_left(4, 2, 16, 24, 0.3, 8.0, 20, 10), _right(3, 8, 12, [0.5, 0.9, 0.99]), None),
])
# what the first case keeps apart is equal or 1 here: one head, one key/value head, one lightning
# head with decay 1 (a plain running sum) and sizes that are no multiple of 16, a chunk shorter
# than a page, one chosen expert without a shared one, then all experts chosen
CASE_B = _model(257, 40, 200, 1e-6, [
    _layer(_left(1, 1, 32, 7, 1.0, 1.5, 5, 6), _right(1, 20, 5, [1.0]), _moe(16, 2, 1)),
    _layer(_left(2, 2, 16, 50, 0.25, 50.0, 64, 32), _right(1, 20, 5, [0.9]),
           _moe(8, 3, 3, shared=8)),
])
# sizes the tile kernels take (multiples of 32, heads of 64), stored in bfloat16
CASE_C = _model(512, 128, 640, 1e-6, [
    _layer(_left(4, 1, 32, 64, 0.18, 25.0, 48, 16), _right(2, 64, 32, [0.8, 0.995]),
           {"kind": "dense", "ff": 256}),
    _layer(_left(4, 1, 32, 64, 0.18, 25.0, 48, 16), _right(2, 64, 32, [0.8, 0.995]),
           _moe(64, 8, 2, shared=96)),
])

# sizes no fast path takes: a head size that is no multiple of 16, five ungrouped heads, widths
# and inner sizes that are no multiple of 32, seven experts of which three are chosen
CASE_D = _model(301, 72, 400, 1e-6, [
    _layer(_left(5, 5, 24, 100, 0.2, 12.0, 150, 20), _right(2, 40, 36, [0.93, 0.998]),
           _moe(40, 7, 3, shared=24)),
    _layer(_left(5, 1, 24, 100, 0.2, 12.0, 150, 20), _right(2, 40, 36, [0.93, 0.998]),
           {"kind": "dense", "ff": 100}),
])

CASES = {"case_a": (CASE_A, 21), "case_b": (CASE_B, 22), "case_c": (CASE_C, 23),
         "case_d": (CASE_D, 24)}


class Case:
    def __init__(self, name, folder, config, seed):
        from hetero_serve_b200.weights import read_safetensors
        self.name, self.dir, self.config, self.seed = name, str(folder), config, seed
        self.raw = read_safetensors(Path(folder) / "model.safetensors")
        self.plain = plain_putelix.prepare(self.raw)
        self.plain_bf16 = plain_putelix.prepare(self.raw, round_to=torch.bfloat16)
        self.vocab = config["vocab"]
        self._memo = {}

    def logits(self, tokens, dtype="float32"):
        key = (tuple(tokens), dtype)
        if key not in self._memo:
            w = self.plain_bf16 if dtype == "bfloat16" else self.plain
            self._memo[key] = plain_putelix.forward(self.config, w, tokens)
        return self._memo[key]

    def tokens(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, self.vocab, (n,), generator=g).tolist()


def make_cases(tmp_path_factory):
    from hetero_serve_b200.weights import write_model_dir
    out = {}
    for name, (cfg, seed) in CASES.items():
        folder = tmp_path_factory.mktemp("putelix_" + name)
        write_model_dir(folder, cfg, seed, "bfloat16" if name == "case_c" else "float32")
        stored = json.loads((folder / "config.json").read_text())
        out[name] = Case(name, folder, stored, seed)
    return out


def rms_error(got, want):
    """Root mean square of the difference with its mean taken off, over the root mean square
    of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean()
    return math.sqrt(float((d * d).mean())) / max(1e-12, math.sqrt(float((want.double() ** 2).mean())))
