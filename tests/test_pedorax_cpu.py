"""Pedorax without a GPU: configuration, spec and weights, and the engine's step function,
cache and state slots with the kernels replaced by their plain twins (tests/plain_ops.py) —
against the plain implementation of the whole model (tests/plain_pedorax.py)."""

import copy
import io

import pytest
import torch

import pedorax_cases as pc
import plain_ops
import plain_pedorax
import traces
from hetero_serve_b200.config import ConfigError
from hetero_serve_b200.config.model_config import architecture_of
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.replay import replay
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import Model
from hetero_serve_b200.weights import WeightError, load_checkpoint, write_model_dir

TOL = 2e-5


def _replay(case, steps, tmp_path, max_tokens, **kw):
    out = tmp_path / "out"
    out.mkdir(exist_ok=True)
    rep = io.StringIO()
    assert replay(model_dir=case.dir, dtype="float32", out_dir=out, max_tokens=max_tokens,
                  lines=traces.lines_of(steps), report=rep, device="cpu",
                  ops=plain_ops.PlainOps(), **kw) == 0
    return out


def _worst(case, out, index, reqs):
    got = traces.collect(out, index, case.vocab)
    return traces.worst_error(got, {r: case.logits(t) for r, t in reqs.items()})


# -- configuration and spec -----------------------------------------------------------------
def test_config_is_read_and_written_back(pedorax_case):
    arch = architecture_of(pedorax_case.config)
    cfg = arch.config_cls.from_dict(pedorax_case.config)
    assert arch.name == "Pedorax"
    again = arch.config_cls.from_dict(cfg.to_dict())
    assert again == cfg and cfg.width == pedorax_case.config["width"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),        # not an attention layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),        # itself
    (lambda c: c["layers"][5]["mixer"].update(kv_from=2), "kv_from"),        # a sharer has no latent
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=30), "equal"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "fit"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "fit"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "even"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
])
def test_config_errors(change, message):
    cfg = copy.deepcopy(pc.CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).config_cls.from_dict(cfg)


def test_spec_shares_cache_entries_and_sizes_state(pedorax_cases):
    case = pedorax_cases["case_a"]
    arch = architecture_of(case.config)
    model = Model(arch.build_spec(arch.config_cls.from_dict(case.config)))
    calls = model.schedule
    assert calls[2].cache == calls[0].cache == calls[5].cache and not calls[2].writes_cache
    assert not calls[5].writes_cache and calls[3].writes_cache and calls[3].cache != calls[0].cache
    groups = {(g.head_dim, g.planes, g.kv_heads): len(g.entries) for g in model.cache_groups}
    assert groups == {(40, 1, 1): 1, (44, 1, 1): 1}         # kv_rank + rot_dim, one row a token
    assert model.state_shapes == {1: (4 * 12 * 20 + 2 * (2 * 2 * 12 + 4 * 20),),
                                  4: (2 * 40 * 36 + 4 * (2 * 2 * 40 + 2 * 36),)}
    assert model.spec.max_positions is None


def test_inner_sizes_of_low_rank_pairs_come_from_the_tensors(pedorax_cases, tmp_path):
    """Another a_rank / g_rank than the default is loaded without being in the config."""
    case = pedorax_cases["case_a"]
    cfg = copy.deepcopy(case.config)
    for layer in cfg["layers"]:
        layer["mixer"].pop("a_rank", None)
        layer["mixer"].pop("g_rank", None)
    (tmp_path / "m").mkdir()
    import json
    import shutil
    shutil.copy(case.dir + "/model.safetensors", tmp_path / "m" / "model.safetensors")
    (tmp_path / "m" / "config.json").write_text(json.dumps(cfg))
    model, _ = load_model(tmp_path / "m", "float32", "cpu")
    assert model.blocks[1].mixer.shape["a_rank"] == 5 and model.blocks[4].mixer.shape["g_rank"] == 4


def test_checkpoint_problems_are_listed(pedorax_cases, tmp_path):
    from hetero_serve_b200.weights import read_safetensors, write_safetensors
    case = pedorax_cases["case_b"]
    raw = dict(read_safetensors(case.dir + "/model.safetensors"))
    del raw["l1.mix.sink"]
    raw["l0.mix.a2"] = raw["l0.mix.a2"][:, :3].contiguous()       # no longer fits a1
    raw["l0.mlp.e1.up"] = raw["l0.mlp.e1.up"][:5].contiguous()
    (tmp_path / "m").mkdir()
    import shutil
    shutil.copy(case.dir + "/config.json", tmp_path / "m" / "config.json")
    write_safetensors(tmp_path / "m" / "model.safetensors", raw)
    arch = architecture_of(case.config)
    model = Model(arch.build_spec(arch.config_cls.from_dict(case.config)))
    with pytest.raises(WeightError) as err:
        load_checkpoint(tmp_path / "m", model)
    assert err.value.missing == ["l1.mix.sink"] and "l0.mlp.e1.up" in err.value.wrong_shape
    with pytest.raises(ValueError, match="low-rank"):
        raw["l1.mix.sink"] = torch.zeros(1)
        raw["l0.mlp.e1.up"] = torch.zeros(16, 40)
        write_safetensors(tmp_path / "m" / "model.safetensors", raw)
        load_model(tmp_path / "m", "float32", "cpu")


# -- the plain implementation's own sanity ----------------------------------------------------
def test_plain_routing_respects_groups():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([3.0, -9.0, 2.0, 2.5, 0.1, 0.2], dtype=torch.float64)
    idx, wt = plain_pedorax.route(z, r)            # group sums: 0 -> s(3)+s(-9), 1 -> s(2)+s(2.5)
    assert sorted(idx.tolist()) == [2, 3] and abs(float(wt.sum()) - 1) < 1e-12


def test_plain_prefix_property(pedorax_case):
    """Causality of the whole plain model: logits of a prefix equal those inside a longer run."""
    toks = pedorax_case.tokens(21, 5)
    full, part = pedorax_case.logits(toks), pedorax_case.logits(toks[:9])
    assert (full[:9] - part).abs().max() < 1e-9


# -- the engine with plain kernels -------------------------------------------------------------
@pytest.mark.parametrize("driver", ["whole", "tail", "portions"])
def test_cuts_agree_with_the_plain_model(pedorax_case, tmp_path, driver):
    reqs = {f"r{i}": pedorax_case.tokens(n, 50 + i) for i, n in enumerate((1, 19, 37))}
    if driver == "whole":
        steps, index = traces.whole(reqs)
    elif driver == "tail":
        steps, index = traces.tail_one_by_one(reqs, tail=9)
    else:
        steps, index = traces.portions(reqs, sizes=(7, 2, 16, 3, 2, 5))
    out = _replay(pedorax_case, steps, tmp_path, max_tokens=64)
    err, where = _worst(pedorax_case, out, index, reqs)
    assert err < TOL, (err, where)


def test_mixed_batches_reuse_pages_and_slots(pedorax_case, tmp_path):
    reqs = {f"r{i}": pedorax_case.tokens(n, 70 + i) for i, n in
            enumerate((33, 5, 18, 40, 3, 26))}
    steps, index, peak = traces.mixed(reqs, seed=3, max_live=3, sizes=(1, 2, 5, 1, 17, 3, 1, 9))
    out = _replay(pedorax_case, steps, tmp_path, max_tokens=peak, max_requests=3)
    err, where = _worst(pedorax_case, out, index, reqs)
    assert sum(len(v) for v in index.values()) > 20 and err < TOL, (err, where)


def test_a_slot_is_cleared_for_its_next_owner(pedorax_cases):
    case = pedorax_cases["case_a"]
    model, _ = load_model(case.dir, "float32", "cpu")
    rn = Runner(model, num_pages=6, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    a, b = case.tokens(30, 1), case.tokens(17, 2)
    rn.step([StepEntry("a", a)])
    rn.close("a")
    res = rn.step([StepEntry("b", b[:10]), ])
    res = rn.step([StepEntry("b", b[10:], want=[6])])
    assert (res.logits[0].double() - case.logits(b)[16]).abs().max() < TOL
    rn.manager.check()


def test_models_with_layers_of_one_kind(pedorax_one_kind, tmp_path):
    """Only recurrent layers (the cache has no page group), or only attention layers (no state;
    no rotation at all in two of them, a negative logit scale in the other model)."""
    case = pedorax_one_kind
    reqs = {f"r{i}": case.tokens(n, 90 + i) for i, n in enumerate((21, 40, 3))}
    steps, index, peak = traces.mixed(reqs, seed=5, max_live=2, sizes=(1, 2, 7, 1, 17, 3))
    out = _replay(case, steps, tmp_path, max_tokens=peak, max_requests=2)
    err, where = _worst(case, out, index, reqs)
    assert err < TOL, (err, where)
