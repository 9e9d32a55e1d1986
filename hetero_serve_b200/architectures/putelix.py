"""Putelix: a decoder whose layers are listed one by one in config.json.  A learned position
table is added to the token embedding.  Every layer normalises its sublayers' OUTPUTS,

    x += norm1(mixer(x));   x += norm2(feed_forward(x))          (RMS norms; the sublayers read x)

and its mixer is a pair side by side (``type: "parallel"``): softmax attention inside chunks of
positions with a learned bias of the distance, capped scores, keys that double as values and a
gate per head (``left``), beside lightning attention, a linear attention with a constant decay
per head and a float32 state per request (``right``); each half is RMS-normed over the width
and the mixer's output is half their sum.  The feed-forward is dense (squared ReLU), a mixture
of experts (softmax over the chosen logits, silu-gated experts, an optional shared expert with
a sigmoid gate per token) or absent.  The model's norm and the token table as the head follow.

config.json::

    {"architecture": "Putelix", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                    "bias_max", "mask": {"size"}},
                           "right": {"heads", "dim", "vdim", "decay": [one per head]}},
                 "mlp": {"kind": "dense", "ff"}
                      | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"},
                         "shared": {"ff"} (optional)}
                      | null}, ...]}

Tensors: ``embed``, ``pos``; per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.left.{q, q.b,
k, k.b, q.norm, k.norm, rel, g, o, o.b, out}``, ``l<i>.mix.right.{q, k, v, g, o, norm, out}``,
``l<i>.mlp.{up, down}`` or ``l<i>.mlp.{router, router.b, e<k>.{gate, up, down},
shared.{gate, up, down, sg}}``; ``final.norm``.  The number of rows of ``rel`` is read off the
tensor (``bias_rows`` in a ``left`` section only tells the random initialisation what to draw).
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Mapping

import torch

from ..config.model_config import (Architecture, ConfigError, need, positive_int,
                                   register_architecture)
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

LAYER_TYPES = ("parallel",)


def _number(name: str, v: Any, positive: bool = False) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{name} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _section(raw: Mapping, key: str, where: str) -> Mapping:
    v = raw.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where} needs an object {key!r}")
    return v


def _check_mlp(i: int, mlp) -> None:
    if mlp is None:
        return
    where = f"layers[{i}].mlp"
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where} must be null or an object of kind 'dense' or 'moe'")
    if mlp["kind"] == "dense":
        positive_int(f"{where}.ff", need(mlp, "ff"))
        return
    positive_int(f"{where}.expert.ff", need(_section(mlp, "expert", where), "ff"))
    ro = _section(mlp, "router", where)
    E = positive_int(f"{where}.router.experts", need(ro, "experts"))
    top = positive_int(f"{where}.router.top", need(ro, "top"))
    if top > E:
        raise ConfigError(f"{where}.router: {top} chosen experts do not fit into {E}")
    if mlp.get("shared") is not None:
        positive_int(f"{where}.shared.ff", need(_section(mlp, "shared", where), "ff"))


def _decays(right: Mapping, where: str) -> list:
    """One decay per lightning head; a single number stands for all heads."""
    decay = need(right, "decay")
    if isinstance(decay, (int, float)) and not isinstance(decay, bool):
        return [decay] * right["heads"]
    if not isinstance(decay, (list, tuple)) or len(decay) != right["heads"]:
        raise ConfigError(f"{where}.decay must list one decay per head")
    return list(decay)


def _check_layer(i: int, layer) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, Mapping) or layer.get("type") not in LAYER_TYPES:
        raise ConfigError(f"{where}.type must be one of {LAYER_TYPES}")
    m = _section(layer, "mixer", where)
    left, right = _section(m, "left", where + ".mixer"), _section(m, "right", where + ".mixer")
    wl, wr = where + ".mixer.left", where + ".mixer.right"
    for key in ("heads", "kv_heads", "dim", "vdim"):
        positive_int(f"{wl}.{key}", need(left, key))
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"{wl}.heads is not a multiple of kv_heads")
    if left["vdim"] != left["dim"]:
        raise ConfigError(f"{wl}.vdim must equal dim: the values are the keys")
    _number(f"{wl}.scale", need(left, "scale"))
    _number(f"{wl}.softcap", need(left, "softcap"), positive=True)
    _number(f"{wl}.bias_max", need(left, "bias_max"), positive=True)
    positive_int(f"{wl}.mask.size", need(_section(left, "mask", wl), "size"))
    for key in ("heads", "dim", "vdim"):
        positive_int(f"{wr}.{key}", need(right, key))
    for d in _decays(right, wr):
        _number(f"{wr}.decay[]", d)
    _check_mlp(i, layer.get("mlp"))


@dataclass(frozen=True)
class PutelixConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple                       # the layer entries of config.json, as they stand
    architectures: tuple[str, ...] = ("Putelix",)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PutelixConfig":
        vocab = positive_int("vocab", need(raw, "vocab"))
        width = positive_int("width", need(raw, "width"))
        max_positions = positive_int("max_positions", need(raw, "max_positions"))
        eps = _number("norm.eps", need(_section(raw, "norm", "config.json"), "eps"), positive=True)
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        for i, layer in enumerate(layers):
            _check_layer(i, layer)
        return cls(vocab, width, max_positions, eps, tuple(copy.deepcopy(list(layers))))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": "Putelix", "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(list(self.layers))}

    def num_parameters(self) -> int:
        return sum(math.prod(t.shape) for t in init_weights(self, 0, shapes_only=True).values())


def _norm_spec(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec("rms_norm", dict(width=width, eps=eps, weight=name))


def build_spec(cfg: PutelixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        attention = PartSpec("biased_chunk_attention", dict(
            width=W, n_heads=left["heads"], n_kv_heads=left["kv_heads"], head_dim=left["dim"],
            scale=left["scale"], softcap=left["softcap"], chunk=left["mask"]["size"],
            bias_max=left["bias_max"], eps=eps, max_distance=cfg.max_positions,
            prefix=p + "mix.left."))
        lightning = PartSpec("lightning_attention", dict(
            width=W, n_heads=right["heads"], dim=right["dim"], vdim=right["vdim"],
            decay=tuple(_decays(right, p + "mixer.right")), eps=eps, prefix=p + "mix.right."))
        mixer = PartSpec("normed_pair", dict(
            width=W, eps=eps, left=attention, right=lightning, left_weight=p + "mix.left.out",
            right_weight=p + "mix.right.out", mix=0.5))
        mlp = layer.get("mlp")
        if mlp is None:
            ff = None
        elif mlp["kind"] == "dense":
            ff = PartSpec("dense", dict(width=W, inner=mlp["ff"], activation="relu2",
                                        in_weight=p + "mlp.up", in_bias=None,
                                        out_weight=p + "mlp.down", out_bias=None,
                                        stored_in_out=False))
        else:
            shared = None
            if mlp.get("shared") is not None:
                s = p + "mlp.shared."
                shared = PartSpec("gated", dict(width=W, inner=mlp["shared"]["ff"],
                                                activation="silu", gate_weight=s + "gate",
                                                up_weight=s + "up", down_weight=s + "down",
                                                token_gate=s + "sg"))
            ff = PartSpec("routed_experts", dict(
                width=W, ff=mlp["expert"]["ff"], experts=mlp["router"]["experts"],
                top=mlp["router"]["top"], scoring="softmax_top", activation="silu",
                router=p + "mlp.router", router_bias=p + "mlp.router.b",
                expert_prefix=p + "mlp.e", shared=shared))
        parts = dict(norm1=_norm_spec(p + "norm1", W, eps), mixer=mixer)
        if ff is not None:
            parts.update(norm2=_norm_spec(p + "norm2", W, eps), feed_forward=ff)
        layers.append(LayerSpec("output_norm", parts))
        schedule.append(LayerCall(i))
    return ModelSpec(
        name="Putelix", vocab_size=cfg.vocab, width=W, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=W, table="embed")),
        position=PartSpec("learned", dict(max_positions=cfg.max_positions, width=W, table="pos")),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=_norm_spec("final.norm", W, eps),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=W, weight="embed")),
        eos_token_id=None)


def init_weights(cfg: PutelixConfig, seed: int, shapes_only: bool = False):
    """Seeded random float32 weights under the checkpoint's names, drawn from one CPU generator
    in the order the names are listed here.  Matrices ~ N(0, 1/sqrt(in)); norm weights near 1;
    biases, distance biases and router biases spread enough that leaving one out changes the
    logits."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    w: dict[str, torch.Tensor] = {}

    def put(name, shape, std=None, mean=0.0):
        if shapes_only:
            w[name] = torch.empty(shape, device="meta")
            return
        if std is None:
            std = 1.0 / math.sqrt(shape[-1])
        w[name] = torch.randn(shape, generator=gen, dtype=torch.float32) * std + mean

    W = cfg.width
    put("embed", (cfg.vocab, W), 0.5)
    put("pos", (cfg.max_positions, W), 0.2)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        put(p + "norm1", (W,), 0.1, 1.0)
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        H, G, D = left["heads"], left["kv_heads"], left["dim"]
        a = p + "mix.left."
        put(a + "q", (H * D, W)); put(a + "q.b", (H * D,), 0.3)
        put(a + "k", (G * D, W)); put(a + "k.b", (G * D,), 0.3)
        put(a + "q.norm", (H * D,), 0.2, 1.5); put(a + "k.norm", (G * D,), 0.2, 1.5)
        put(a + "rel", (int(left.get("bias_rows", 32)), H), 1.0)
        put(a + "g", (H, W), 2.0 / math.sqrt(W))
        put(a + "o", (W, H * D)); put(a + "o.b", (W,), 0.1)
        HR, DR, VR = right["heads"], right["dim"], right["vdim"]
        b = p + "mix.right."
        put(b + "q", (HR * DR, W)); put(b + "k", (HR * DR, W)); put(b + "v", (HR * VR, W))
        put(b + "g", (HR * VR, W), 2.0 / math.sqrt(W))
        put(b + "o", (W, HR * VR)); put(b + "norm", (HR * VR,), 0.1, 1.0)
        put(a + "out", (W,), 0.1, 1.0); put(b + "out", (W,), 0.1, 1.0)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        put(p + "norm2", (W,), 0.1, 1.0)
        if mlp["kind"] == "dense":
            put(p + "mlp.up", (mlp["ff"], W), 1.5 / math.sqrt(W))
            put(p + "mlp.down", (W, mlp["ff"]))
            continue
        ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
        for e in range(E):
            put(f"{p}mlp.e{e}.gate", (ff, W), 2.0 / math.sqrt(W))
            put(f"{p}mlp.e{e}.up", (ff, W), 2.0 / math.sqrt(W))
            put(f"{p}mlp.e{e}.down", (W, ff))
        put(p + "mlp.router", (E, W), 2.0 / math.sqrt(W))
        put(p + "mlp.router.b", (E,), 0.5)
        if mlp.get("shared") is not None:
            sf = mlp["shared"]["ff"]
            put(p + "mlp.shared.gate", (sf, W), 2.0 / math.sqrt(W))
            put(p + "mlp.shared.up", (sf, W), 2.0 / math.sqrt(W))
            put(p + "mlp.shared.down", (W, sf))
            put(p + "mlp.shared.sg", (1, W), 2.0 / math.sqrt(W))
    put("final.norm", (W,), 0.1, 1.0)
    return w


def _pair(heads, kv_heads, dim, chunk, lin_heads, lin_dim, lin_vdim, decay=None, scale=None,
          softcap=30.0, bias_max=128, bias_rows=32):
    decay = decay or [1.0 - 2.0 ** (-3 - 5 * h / max(1, lin_heads - 1)) for h in range(lin_heads)]
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                     "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
                     "softcap": softcap, "bias_max": bias_max, "bias_rows": bias_rows,
                     "mask": {"size": chunk}},
            "right": {"heads": lin_heads, "dim": lin_dim, "vdim": lin_vdim, "decay": decay}}


def _moe(ff, experts, top, shared_ff=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def _preset(vocab, width, max_positions, layers, eps=1e-6):
    return {"architecture": "Putelix", "vocab": vocab, "width": width,
            "max_positions": max_positions, "norm": {"eps": eps}, "layers": layers}


def _stack(n, pair, dense_ff, moe):
    """n layers, dense and routed feed-forwards in turn."""
    return [{"type": "parallel", "mixer": copy.deepcopy(pair),
             "mlp": {"kind": "dense", "ff": dense_ff} if i % 2 == 0 else copy.deepcopy(moe)}
            for i in range(n)]


PRESETS: dict[str, dict] = {
    # a few hundred thousand parameters: for demonstrations and smoke runs
    "putelix-tiny": _preset(384, 96, 512, [
        {"type": "parallel", "mixer": _pair(4, 2, 16, 40, 2, 16, 24, bias_max=64, bias_rows=12),
         "mlp": {"kind": "dense", "ff": 160}},
        {"type": "parallel", "mixer": _pair(4, 2, 16, 40, 2, 16, 24, bias_max=64, bias_rows=12),
         "mlp": _moe(48, 6, 2, shared_ff=64)},
        {"type": "parallel", "mixer": _pair(4, 2, 16, 40, 2, 16, 24, bias_max=64, bias_rows=12),
         "mlp": None},
    ]),
    # layer sizes of a small and a mid-sized production model, few layers: for measurements
    "putelix-1k": _preset(32768, 1024, 4096, _stack(
        4, _pair(16, 4, 64, 512, 8, 128, 128, bias_max=512), 4096, _moe(512, 32, 4, 1024))),
    "putelix-2k": _preset(32768, 2048, 4096, _stack(
        4, _pair(32, 8, 64, 512, 16, 128, 128, bias_max=512), 8192, _moe(1024, 64, 6, 2048))),
}

PUTELIX = Architecture(name="Putelix", config_cls=PutelixConfig, build_spec=build_spec,
                       init_weights=init_weights, model_types=("putelix",), presets=PRESETS,
                       preset_aliases={})
register_architecture(PUTELIX, replace=True)
