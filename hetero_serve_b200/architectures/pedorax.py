"""Pedorax: a decoder whose layers are listed one by one in config.json.  Every layer is a
parallel block (one Dynamic Tanh norm; mixer and feed-forward both read it) whose mixer is
either attention over a shared latent (``latent_attention``) or the gated delta rule with a
decay per key channel (``channel_delta``), and whose feed-forward is a routed mixture of
experts or absent.  The token table is scaled at the input and reused, unscaled, as the head,
whose logits are scaled by ``logit_scale``.

config.json::

    {"architecture": "Pedorax", "vocab": V, "width": W, "embedding": {"scale": s},
     "logit_scale": l, "norm": {"eps": e},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                           "rot": {"base", "dims"}, "kv_from": j (optional)},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"},
                         "router": {"experts", "top", "groups": {"count", "keep"}}} | null},
                {"type": "channel_delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...}, ...]}

Tensors: ``embed``; per layer ``l<i>.norm1`` (+ ``.b``, ``.alpha``), ``l<i>.mix.*``,
``l<i>.mlp.router``, ``l<i>.mlp.e<k>.{gate,up,down}``; ``final.norm`` (+ ``.b``, ``.alpha``).
The inner sizes of the delta rule's low-rank pairs are read off the tensors; the optional
mixer keys ``a_rank`` / ``g_rank`` only tell the random initialisation what to draw.
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

LAYER_TYPES = ("latent_attention", "channel_delta")


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
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"{where} must be null or an object of kind 'moe'")
    ex, ro = _section(mlp, "expert", where), _section(mlp, "router", where)
    positive_int(f"{where}.expert.ff", need(ex, "ff"))
    _number(f"{where}.expert.limit", need(ex, "limit"), positive=True)
    E = positive_int(f"{where}.router.experts", need(ro, "experts"))
    top = positive_int(f"{where}.router.top", need(ro, "top"))
    gr = _section(ro, "groups", where + ".router")
    count = positive_int(f"{where}.router.groups.count", need(gr, "count"))
    keep = positive_int(f"{where}.router.groups.keep", need(gr, "keep"))
    if E % count or keep > count or top > keep * (E // count):
        raise ConfigError(f"{where}.router: {E} experts, {count} groups of which {keep} are "
                          f"kept and {top} chosen experts do not fit together")


def _check_layer(i: int, layer, layers) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, Mapping) or layer.get("type") not in LAYER_TYPES:
        raise ConfigError(f"{where}.type must be one of {LAYER_TYPES}")
    m = _section(layer, "mixer", where)
    for key in ("heads", "dim", "vdim"):
        positive_int(f"{where}.mixer.{key}", need(m, key))
    if layer["type"] == "latent_attention":
        for key in ("rot_dim", "kv_rank"):
            positive_int(f"{where}.mixer.{key}", need(m, key))
        _number(f"{where}.mixer.scale", need(m, "scale"))
        rot = _section(m, "rot", where + ".mixer")
        _number(f"{where}.mixer.rot.base", need(rot, "base"), positive=True)
        dims = need(rot, "dims")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims % 2 or \
                not 0 <= dims <= m["rot_dim"]:
            raise ConfigError(f"{where}.mixer.rot.dims must be even and at most rot_dim")
        src = m.get("kv_from")
        if src is not None:
            ok = isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i \
                and layers[src].get("type") == "latent_attention" \
                and layers[src]["mixer"].get("kv_from") is None
            if not ok:
                raise ConfigError(f"{where}.mixer.kv_from must name an earlier latent_attention "
                                  f"layer that has a latent of its own, got {src!r}")
            theirs = layers[src]["mixer"]
            if any(theirs[k] != m[k] for k in ("kv_rank", "rot_dim", "rot")):
                raise ConfigError(f"{where}.mixer: kv_rank, rot_dim and rot must equal those of "
                                  f"layer {src}, whose cache it reads")
    else:
        kvh = positive_int(f"{where}.mixer.kv_heads", need(m, "kv_heads"))
        if m["heads"] % kvh:
            raise ConfigError(f"{where}.mixer.heads is not a multiple of kv_heads")
        positive_int(f"{where}.mixer.conv", need(m, "conv"))
    _check_mlp(i, layer.get("mlp"))


@dataclass(frozen=True)
class PedoraxConfig:
    vocab: int
    width: int
    embedding_scale: float
    logit_scale: float
    norm_eps: float
    layers: tuple                       # the layer entries of config.json, as they stand
    architectures: tuple[str, ...] = ("Pedorax",)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PedoraxConfig":
        vocab = positive_int("vocab", need(raw, "vocab"))
        width = positive_int("width", need(raw, "width"))
        scale = _number("embedding.scale", need(_section(raw, "embedding", "config.json"), "scale"))
        logit_scale = _number("logit_scale", need(raw, "logit_scale"))
        eps = _number("norm.eps", need(_section(raw, "norm", "config.json"), "eps"), positive=True)
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        for i, layer in enumerate(layers):
            _check_layer(i, layer, layers)
        return cls(vocab, width, scale, logit_scale, eps, tuple(copy.deepcopy(list(layers))))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": "Pedorax", "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}

    def num_parameters(self) -> int:
        return sum(math.prod(t.shape) for t in init_weights(self, 0, shapes_only=True).values())


def _norm_spec(prefix: str, width: int) -> PartSpec:
    return PartSpec("dynamic_tanh", dict(width=width, weight=prefix, bias=prefix + ".b",
                                         alpha=prefix + ".alpha"))


def build_spec(cfg: PedoraxConfig) -> ModelSpec:
    W = cfg.width
    layers, schedule = [], []
    entry_of: dict[int, int] = {}          # layer -> the cache entry it owns
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        call = None
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            own = src is None
            mixer = PartSpec("latent_attention", dict(
                width=W, n_heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                kv_rank=m["kv_rank"], scale=m["scale"], rot_base=m["rot"]["base"],
                rot_dims=m["rot"]["dims"], eps=cfg.norm_eps, q_weight=p + "mix.q",
                latent_weight=p + "mix.dkv" if own else None,
                latent_norm=p + "mix.dkv.norm" if own else None,
                key_up=p + "mix.uk", value_up=p + "mix.uv", sink=p + "mix.sink",
                out_weight=p + "mix.o", shares_cache=not own))
            if own:
                entry_of[i] = len(entry_of)
                call = LayerCall(i, entry_of[i], True)
            else:
                call = LayerCall(i, entry_of[src], False)      # reads what layer src wrote
        else:
            mixer = PartSpec("channel_delta_rule", dict(
                width=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], dim=m["dim"],
                vdim=m["vdim"], taps=m["conv"], eps=cfg.norm_eps, prefix=p + "mix."))
            entry_of[i] = len(entry_of)
            call = LayerCall(i, entry_of[i], True)               # an entry number, never a pool
        mlp = layer.get("mlp")
        if mlp is None:
            ff = PartSpec("none", {})
        else:
            r = mlp["router"]
            ff = PartSpec("routed_experts", dict(
                width=W, ff=mlp["expert"]["ff"], experts=r["experts"], top=r["top"],
                groups=r["groups"]["count"], keep=r["groups"]["keep"],
                limit=mlp["expert"]["limit"], router=p + "mlp.router",
                expert_prefix=p + "mlp.e"))
        layers.append(LayerSpec("parallel", norm1=_norm_spec(p + "norm1", W), mixer=mixer,
                                feed_forward=ff))
        schedule.append(call)
    return ModelSpec(
        name="Pedorax", vocab_size=cfg.vocab, width=W, max_positions=None,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=W, table="embed",
                                               scale=cfg.embedding_scale)),
        position=PartSpec("none", {}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=_norm_spec("final.norm", W),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=W, weight="embed",
                                     scale=cfg.logit_scale)),
        eos_token_id=None)


def init_weights(cfg: PedoraxConfig, seed: int, shapes_only: bool = False):
    """Seeded random float32 weights under the checkpoint's names, drawn from one CPU
    generator in the order the names are listed here.  Matrices ~ N(0, 1/sqrt(in)); norm
    weights near 1, alphas near 0.7, sinks, decays and biases spread enough that leaving one
    out changes the logits."""
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

    def norm(prefix, width):
        put(prefix, (width,), 0.1, 1.0)
        put(prefix + ".b", (width,), 0.05)
        put(prefix + ".alpha", (), 0.05, 0.7)

    W = cfg.width
    put("embed", (cfg.vocab, W), 0.5)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1", W)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            P, R = m["rot_dim"], m["kv_rank"]
            put(p + "mix.q", (H * (D + P), W))
            if m.get("kv_from") is None:
                put(p + "mix.dkv", (R + P, W))
                put(p + "mix.dkv.norm", (R,), 0.1, 1.0)
            put(p + "mix.uk", (H * D, R))
            put(p + "mix.uv", (H * V, R))
            put(p + "mix.sink", (H,), 1.0)
            put(p + "mix.o", (W, H * V), 0.5 / math.sqrt(H * V))
        else:
            HK, taps = m["kv_heads"], m["conv"]
            ra = int(m.get("a_rank", max(4, D // 2)))
            rg = int(m.get("g_rank", max(4, V // 2)))
            for name, rows in (("q", HK * D), ("k", HK * D), ("v", H * V)):
                put(p + "mix." + name, (rows, W))
                put(p + "mix." + name + ".conv", (rows, taps), 0.5)
            put(p + "mix.b", (H, W))
            put(p + "mix.A_log", (H,), 0.5, -1.0)
            put(p + "mix.norm", (V,), 0.1, 1.0)
            put(p + "mix.a1", (ra, W))
            put(p + "mix.a2", (H * D, ra))
            put(p + "mix.dt_bias", (H * D,), 0.5)
            put(p + "mix.g1", (rg, W))
            put(p + "mix.g2", (H * V, rg))
            put(p + "mix.o", (W, H * V), 0.5 / math.sqrt(H * V))
        mlp = layer.get("mlp")
        if mlp is not None:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            for e in range(E):
                put(f"{p}mlp.e{e}.gate", (ff, W), 2.0 / math.sqrt(W))
                put(f"{p}mlp.e{e}.up", (ff, W), 2.0 / math.sqrt(W))
                put(f"{p}mlp.e{e}.down", (W, ff), 0.5 / math.sqrt(ff))
            put(p + "mlp.router", (E, W), 2.0 / math.sqrt(W))
    norm("final.norm", W)
    return w


def _moe(ff, experts, top, count, keep, limit=7.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, dims=None, scale=None,
            kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim),
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _delta(heads, kv_heads, dim, vdim, conv=4, **more):
    return dict({"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
                **more)


def _preset(vocab, width, layers, embedding_scale=1.0, logit_scale=1.0, eps=1e-6):
    return {"architecture": "Pedorax", "vocab": vocab, "width": width,
            "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale,
            "norm": {"eps": eps}, "layers": layers}


def _stack(n, width_heads, dim, vdim, rot_dim, kv_rank, ff, experts, top, count, keep):
    """n layers alternating delta rule and latent attention; every second attention layer
    reads the cache of the one before it."""
    layers, last_own = [], None
    for i in range(n):
        if i % 2 == 0:
            layers.append({"type": "channel_delta",
                           "mixer": _delta(width_heads, width_heads, dim, vdim),
                           "mlp": _moe(ff, experts, top, count, keep)})
        else:
            share = last_own is not None and (i // 2) % 2 == 1
            layers.append({"type": "latent_attention",
                           "mixer": _latent(width_heads, dim, rot_dim, vdim, kv_rank,
                                            kv_from=last_own if share else None),
                           "mlp": _moe(ff, experts, top, count, keep)})
            if not share:
                last_own = i
    return layers


PRESETS: dict[str, dict] = {
    # a few hundred thousand parameters: for demonstrations and smoke runs
    "pedorax-tiny": _preset(384, 96, [
        {"type": "channel_delta", "mixer": _delta(4, 2, 16, 24, conv=3, a_rank=6, g_rank=10),
         "mlp": _moe(48, 8, 2, 4, 2, limit=3.0)},
        {"type": "latent_attention", "mixer": _latent(3, 16, 8, 24, 40, base=5000.0), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(3, 16, 8, 24, 40, base=5000.0, kv_from=1),
         "mlp": _moe(48, 8, 2, 4, 2, limit=3.0)},
    ], embedding_scale=2.0, logit_scale=0.25),
    # layer sizes of a small and a mid-sized production model, few layers: for measurements
    "pedorax-1k": _preset(32768, 1024, _stack(4, 8, 128, 128, 64, 256, 512, 32, 4, 4, 2),
                          embedding_scale=1.0, logit_scale=1.0),
    "pedorax-2k": _preset(32768, 2048, _stack(4, 16, 128, 128, 64, 512, 1024, 64, 6, 8, 4),
                          embedding_scale=1.0, logit_scale=1.0),
}

PEDORAX = Architecture(name="Pedorax", config_cls=PedoraxConfig, build_spec=build_spec,
                       init_weights=init_weights, model_types=("pedorax",), presets=PRESETS,
                       preset_aliases={})
register_architecture(PEDORAX, replace=True)
