"""Putelix without a GPU: configuration, spec and weights, and the engine's step function,
cache and state slots with the kernels replaced by their plain twins (tests/plain_ops.py) —
against the plain implementation of the whole model (tests/plain_putelix.py)."""

import copy
import io
import math

import pytest
import torch

import plain_ops
import plain_putelix
import putelix_cases as uc
import traces
from hetero_serve_b200.config import ConfigError
from hetero_serve_b200.config.model_config import architecture_of
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.replay import replay
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import Model
from hetero_serve_b200.parts.biased_attention import distance_buckets
from hetero_serve_b200.weights import WeightError, load_checkpoint, read_safetensors, \
    write_safetensors

TOL = 2e-5


def _replay(case, steps, tmp_path, max_tokens, **kw):
    out = tmp_path / "out"
    out.mkdir(exist_ok=True)
    assert replay(model_dir=case.dir, dtype="float32", out_dir=out, max_tokens=max_tokens,
                  lines=traces.lines_of(steps), report=io.StringIO(), device="cpu",
                  ops=plain_ops.PlainOps(), **kw) == 0
    return out


def _worst(case, out, index, reqs):
    got = traces.collect(out, index, case.vocab)
    return traces.worst_error(got, {r: case.logits(t) for r, t in reqs.items()})


# -- configuration and spec -----------------------------------------------------------------
def test_config_is_read_and_written_back(putelix_case):
    arch = architecture_of(putelix_case.config)
    cfg = arch.config_cls.from_dict(putelix_case.config)
    assert arch.name == "Putelix"
    assert arch.config_cls.from_dict(cfg.to_dict()) == cfg
    assert cfg.width == putelix_case.config["width"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=8), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "one decay per head"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "fit"),
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "mask"),
    (lambda c: c.pop("max_positions"), "max_positions"),
])
def test_config_errors(change, message):
    cfg = copy.deepcopy(uc.CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).config_cls.from_dict(cfg)


def test_spec_has_one_page_group_and_a_state_per_layer(putelix_cases):
    case = putelix_cases["case_a"]
    arch = architecture_of(case.config)
    model = Model(arch.build_spec(arch.config_cls.from_dict(case.config)))
    groups = {(g.kv_heads, g.head_dim, g.planes): len(g.entries) for g in model.cache_groups}
    assert groups == {(2, 16, 2): 2, (3, 8, 2): 1}          # normed keys and values, two planes
    assert sorted(g.chunk for g in model.cache_groups) == [24, 37]
    assert model.state_shapes == {0: (3 * 8 * 12,), 1: (2 * 16 * 8,), 2: (3 * 8 * 12,)}
    assert model.blocks[2].feed_forward is None and model.blocks[2].norm2 is None
    assert model.spec.max_positions == 300
    names = set(model.tensor_requests())
    assert "l2.norm2" not in names and "l1.mlp.shared.sg" in names and "l1.mlp.router.b" in names


def test_checkpoint_problems_are_listed(putelix_cases, tmp_path):
    case = putelix_cases["case_a"]
    raw = dict(read_safetensors(case.dir + "/model.safetensors"))
    del raw["l1.mix.left.rel"]
    raw["l0.mix.right.norm"] = raw["l0.mix.right.norm"][:5].contiguous()
    (tmp_path / "m").mkdir()
    import shutil
    shutil.copy(case.dir + "/config.json", tmp_path / "m" / "config.json")
    write_safetensors(tmp_path / "m" / "model.safetensors", raw)
    arch = architecture_of(case.config)
    model = Model(arch.build_spec(arch.config_cls.from_dict(case.config)))
    with pytest.raises(WeightError) as err:
        load_checkpoint(tmp_path / "m", model)
    assert err.value.missing == ["l1.mix.left.rel"] and "l0.mix.right.norm" in err.value.wrong_shape


def test_rows_of_the_distance_table_come_from_the_tensor(putelix_cases, tmp_path):
    """Another number of rows than the initialisation's default loads and changes the logits."""
    case = putelix_cases["case_b"]
    raw = dict(read_safetensors(case.dir + "/model.safetensors"))
    g = torch.Generator().manual_seed(3)
    raw["l0.mix.left.rel"] = torch.randn(9, 1, generator=g)
    (tmp_path / "m").mkdir()
    import shutil
    shutil.copy(case.dir + "/config.json", tmp_path / "m" / "config.json")
    write_safetensors(tmp_path / "m" / "model.safetensors", raw)
    model, _ = load_model(tmp_path / "m", "float32", "cpu")
    rn = Runner(model, num_pages=4, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    toks = case.tokens(20, 4)
    got = rn.step([StepEntry("a", toks, want=[19])]).logits[0]
    want = plain_putelix.forward(case.config, plain_putelix.prepare(raw), toks)[19]
    assert (got.double() - want).abs().max() < TOL
    assert (want - case.logits(toks)[19]).abs().max() > 1e-3


# -- the plain implementation's own sanity and the table the package expands ----------------
def test_distance_buckets():
    rows = [plain_putelix.distance_bucket(n, 32, 200) for n in range(400)]
    assert rows[:16] == list(range(16)) and rows[16] == 16 and rows[199] == 31 and rows[399] == 31
    assert all(b >= a for a, b in zip(rows, rows[1:]))
    first_31 = rows.index(31)
    assert math.log(first_31 / 16) / math.log(200 / 16) * 16 >= 15 > \
        math.log((first_31 - 1) / 16) / math.log(200 / 16) * 16
    for B, far in ((32, 200), (10, 20), (6, 5), (14, 30), (2, 9)):
        assert distance_buckets(300, B, far) == [plain_putelix.distance_bucket(n, B, far)
                                                 for n in range(300)]


def test_plain_routing_breaks_ties_by_index_and_weights_the_chosen_only():
    z = torch.tensor([[1.0, 3.0, 3.0, -2.0, 3.0]], dtype=torch.float64)
    idx, wt = plain_putelix.route(z, 2)
    assert idx.tolist() == [[1, 2]] and torch.allclose(wt, torch.tensor([[0.5, 0.5]], dtype=torch.float64))
    idx, wt = plain_putelix.route(torch.tensor([[0.0, 2.0, 1.0]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 2]] and abs(float(wt[0, 0]) - 1 / (1 + math.exp(-1.0))) < 1e-12


def test_plain_prefix_property_and_chunks(putelix_case):
    """Causality; and a key outside the query's chunk changes nothing in the attention half."""
    toks = putelix_case.tokens(60, 5)
    full, part = putelix_case.logits(toks), putelix_case.logits(toks[:9])
    assert (full[:9] - part).abs().max() < 1e-9
    m = putelix_case.config["layers"][0]["mixer"]["left"]
    w = putelix_case.plain
    g = torch.Generator().manual_seed(8)
    h = torch.randn(2 * m["mask"]["size"] + 3, putelix_case.config["width"], generator=g,
                    dtype=torch.float64)
    out = plain_putelix.chunk_attention(h, w, "l0.mix.left.", m, 1e-6)
    c = m["mask"]["size"]
    alone = plain_putelix.chunk_attention(h[c:], w, "l0.mix.left.", m, 1e-6)
    assert (out[c:] - alone).abs().max() < 1e-10            # chunks start at multiples of c


# -- the engine with plain kernels -------------------------------------------------------------
@pytest.mark.parametrize("driver", ["whole", "tail", "portions"])
def test_cuts_agree_with_the_plain_model(putelix_case, tmp_path, driver):
    reqs = {f"r{i}": putelix_case.tokens(n, 50 + i) for i, n in enumerate((1, 19, 58))}
    if driver == "whole":
        steps, index = traces.whole(reqs)
    elif driver == "tail":
        steps, index = traces.tail_one_by_one(reqs, tail=12)
    else:
        steps, index = traces.portions(reqs, sizes=(7, 2, 16, 3, 2, 5))
    out = _replay(putelix_case, steps, tmp_path, max_tokens=96)
    err, where = _worst(putelix_case, out, index, reqs)
    assert err < TOL, (err, where)


def test_mixed_batches_reuse_pages_and_slots(putelix_case, tmp_path):
    reqs = {f"r{i}": putelix_case.tokens(n, 70 + i) for i, n in
            enumerate((33, 5, 18, 52, 3, 26))}
    steps, index, peak = traces.mixed(reqs, seed=3, max_live=3, sizes=(1, 2, 5, 1, 17, 3, 1, 9))
    out = _replay(putelix_case, steps, tmp_path, max_tokens=peak, max_requests=3)
    err, where = _worst(putelix_case, out, index, reqs)
    assert sum(len(v) for v in index.values()) > 20 and err < TOL, (err, where)


def test_a_slot_is_cleared_for_its_next_owner(putelix_cases):
    case = putelix_cases["case_a"]
    model, _ = load_model(case.dir, "float32", "cpu")
    rn = Runner(model, num_pages=6, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    a, b = case.tokens(30, 1), case.tokens(17, 2)
    rn.step([StepEntry("a", a)])
    rn.close("a")
    rn.step([StepEntry("b", b[:10]), ])
    res = rn.step([StepEntry("b", b[10:], want=[6])])
    assert (res.logits[0].double() - case.logits(b)[16]).abs().max() < TOL
    rn.manager.check()


def test_pages_of_passed_chunks_are_given_back(putelix_cases):
    """A request far longer than the pool holds runs in portions, because the pages of the
    chunks behind it are given back as it goes; its logits are the plain model's."""
    case = putelix_cases["case_a"]                    # chunks of 24 and 37 positions, pages of 16
    model, _ = load_model(case.dir, "float32", "cpu")
    rn = Runner(model, num_pages=6, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    toks = case.tokens(230, 17)
    want, at = case.logits(toks), 0
    for n in (20, 13, 2, 19, 1, 1, 20, 7, 20, 20, 3, 20, 1, 20, 20, 20, 2, 20, 1):
        res = rn.step([StepEntry("a", toks[at:at + n], want=[n - 1])])
        assert (res.logits[0].double() - want[at + n - 1]).abs().max() < TOL, at
        at += n
        assert all(6 - rn.manager.pages_free(g) <= 5 for g in range(len(model.cache_groups)))
    assert at == 230
    rn.manager.check()
    rn.close("a")
    assert all(rn.manager.pages_free(g) == 6 for g in range(len(model.cache_groups)))


def test_the_parts_under_an_arrangement_that_adds(putelix_cases):
    """The new parts in another design: norms BEFORE the sublayers (x += pair(norm1(x));
    x += ff(norm2(x))).  The paired mixer then forms its output itself and adds it, the norm
    normalises rows for the parts, the dense feed-forward adds into the stream."""
    import dataclasses
    from hetero_serve_b200.parts.spec import LayerSpec
    case = putelix_cases["case_a"]
    arch = architecture_of(case.config)
    spec = arch.build_spec(arch.config_cls.from_dict(case.config))
    first = spec.layers[0]
    spec = dataclasses.replace(spec, layers=(LayerSpec("pre_norm", dict(first.parts)),),
                               schedule=spec.schedule[:1])
    model = Model(spec)
    model.bind({n: case.raw[n] for n in model.tensor_requests()}, torch.float32, "cpu")
    rn = Runner(model, num_pages=4, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    toks = case.tokens(40, 3)
    rn.step([StepEntry("a", toks[:13])])
    got = rn.step([StepEntry("a", toks[13:], want=[0, 26])]).logits.double()
    w, cfg = case.plain, case.config
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(toks)] + w["pos"][:40]
    h = plain_putelix.rms_norm(x, w["l0.norm1"], eps)
    x = x + plain_putelix.paired_mixer(h, w, "l0.mix.", cfg["layers"][0]["mixer"], eps)
    x = x + plain_putelix.dense_feed_forward(plain_putelix.rms_norm(x, w["l0.norm2"], eps), w,
                                             "l0.mlp.")
    want = plain_putelix.rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    assert (got - want[[13, 39]]).abs().max() < TOL
