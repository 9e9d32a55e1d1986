"""Putelix through the engine on the GPU: the step function, the paged cache of normed keys and
values, the state slots and the CUDA kernels against the plain implementation
(tests/plain_putelix.py), in both precisions; then greedy generation through the Python entry
point and its scheduler."""

import io
import subprocess
import sys

import pytest
import torch

import plain_putelix
import putelix_cases as uc
import traces
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.replay import replay
from hetero_serve_b200.engine.step import Runner, StepEntry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# relative root-mean-square error of a row of logits: float32 sums of a few hundred terms;
# bfloat16 rounds the rows the projections read and the cache rows to 8 bits
TOL = {"float32": 2e-5, "bfloat16": 6e-2}


def _replay(case, dtype, steps, tmp_path, max_tokens, **kw):
    out = tmp_path / f"out_{dtype}"
    out.mkdir(exist_ok=True)
    assert replay(model_dir=case.dir, dtype=dtype, out_dir=out, max_tokens=max_tokens,
                  lines=traces.lines_of(steps), report=io.StringIO(), device=DEV, **kw) == 0
    return out


def _worst(case, dtype, out, index, reqs):
    """float32: the largest error.  bfloat16: rounding the rows the router reads can change
    which expert a token picks where two logits nearly tie, and such a token is then far from
    the plain model while nothing is wrong; so one row in twenty may be, and the error at that
    rank and three times the median have to stay under the tolerance."""
    got = traces.collect(out, index, case.vocab)
    errs = sorted(((uc.rms_error(torch.as_tensor(row), case.logits(reqs[rid], dtype)[p]),
                    (rid, p)) for (rid, p), row in got.items()), reverse=True)
    if dtype == "float32":
        return errs[0][0], errs[0][1], len(errs)
    k = len(errs) // 20
    return max(errs[k][0], 3 * errs[len(errs) // 2][0]), errs[k][1], len(errs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("driver", ["whole", "tail", "portions"])
def test_cuts_agree_with_the_plain_model(putelix_case, tmp_path, dtype, driver):
    reqs = {f"r{i}": putelix_case.tokens(n, 150 + i) for i, n in enumerate((1, 2, 23, 70, 131))}
    if driver == "whole":
        steps, index = traces.whole(reqs)
    elif driver == "tail":
        steps, index = traces.tail_one_by_one(reqs, tail=40)
    else:
        steps, index = traces.portions(reqs, sizes=(24, 7, 2, 16, 3, 2, 31, 5, 2, 9))
    out = _replay(putelix_case, dtype, steps, tmp_path, max_tokens=192)
    err, where, n = _worst(putelix_case, dtype, out, index, reqs)
    assert n > 4 and err < TOL[dtype], (err, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(putelix_case, tmp_path, dtype):
    reqs = {f"r{i}": putelix_case.tokens(n, 170 + i) for i, n in
            enumerate((90, 9, 64, 23, 70, 3, 55, 31, 2))}
    steps, index, peak = traces.mixed(reqs, seed=2)
    out = _replay(putelix_case, dtype, steps, tmp_path, max_tokens=peak, max_requests=4)
    err, where, n = _worst(putelix_case, dtype, out, index, reqs)
    assert n > 40 and err < TOL[dtype], (err, where)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_prompt_portions_on_the_tile_kernels(putelix_cases, tmp_path, dtype):
    """Sizes the tile kernels take and prompts long enough for them (200 and 150 tokens at
    once, then portions of 70 beside single tokens): several chunks a prompt, the sorted
    experts, the tensor-core linears."""
    from hetero_serve_b200.kernels import CudaOps
    case = putelix_cases["case_c"]
    reqs = {"a": case.tokens(200, 301), "b": case.tokens(150, 302), "c": case.tokens(9, 303)}
    steps, index = traces.whole(reqs)
    more, index2 = traces.portions({"d": case.tokens(160, 304)}, sizes=(70, 2, 70, 1, 17))
    ops = CudaOps(DEV)
    out = _replay(case, dtype, steps, tmp_path, max_tokens=384, ops=ops)
    err, where, n = _worst(case, dtype, out, index, reqs)
    assert n > 200 and err < TOL[dtype], (err, where)
    if dtype == "bfloat16":
        assert ops._moe_need and any(v[0] for v in ops._moe_need.values())   # the sorted path ran
    out2 = _replay(case, dtype, more, tmp_path, max_tokens=192, ops=ops)
    err, where, n = _worst(case, dtype, out2, index2, {"d": case.tokens(160, 304)})
    assert err < TOL[dtype], (err, where)


def _runner(case, dtype="float32", pages=16, slots=4, **kw):
    model, _ = load_model(case.dir, dtype, DEV)
    return Runner(model, num_pages=pages, page_size=16, max_requests=slots, dtype=model.dtype,
                  device=DEV, **kw)


def test_a_request_alone_and_in_a_batch(putelix_case):
    """The logits of a request do not depend on its neighbours in the batch, nor on the slot
    and pages it got: in float32 they are the same bits."""
    case = putelix_case
    a, b, c = case.tokens(45, 1), case.tokens(20, 2), case.tokens(33, 3)
    alone = _runner(case)
    want = alone.step([StepEntry("a", a[:30], want=[29])]).logits.clone()
    want2 = alone.step([StepEntry("a", a[30:], want=[0, 14])]).logits.clone()
    rn = _runner(case)
    rn.step([StepEntry("c", c)])                  # takes the first slot and pages
    got = rn.step([StepEntry("b", b[:7]), StepEntry("a", a[:30], want=[29]),
                   StepEntry("c", [5])]).logits.clone()
    rn.close("c")
    got2 = rn.step([StepEntry("a", a[30:], want=[0, 14]), StepEntry("b", b[7:])]).logits
    assert torch.equal(got, want) and torch.equal(got2, want2)
    assert uc.rms_error(got2[1].cpu(), case.logits(a)[44]) < TOL["float32"]


def test_freed_slots_and_pages_start_clean(putelix_cases):
    case = putelix_cases["case_a"]
    rn = _runner(case, pages=5, slots=1)
    for seed, n in ((4, 70), (5, 41), (6, 80)):
        t = case.tokens(n, seed)
        rn.step([StepEntry("x", t[:n // 2])])
        res = rn.step([StepEntry("x", t[n // 2:], want=[n - n // 2 - 1])])
        assert uc.rms_error(res.logits[0].cpu(), case.logits(t)[n - 1]) < TOL["float32"], seed
        rn.close("x")
    rn.manager.check()


def test_long_decoding(putelix_cases):
    """Single-token steps across many chunk and page borders."""
    case = putelix_cases["case_a"]
    t = case.tokens(260, 9)
    rn = _runner(case, pages=20)
    rn.step([StepEntry("d", t[:12])])
    want = case.logits(t)
    chunk = case.config["layers"][0]["mixer"]["left"]["mask"]["size"]
    for i in range(12, 260):
        res = rn.step([StepEntry("d", [t[i]], want=[0])])
        if i % chunk in (0, 1, chunk - 1) or i % 16 == 0 or i > 250:
            assert uc.rms_error(res.logits[0].cpu(), want[i]) < TOL["float32"], i


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_captured_steps_equal_eager_steps(putelix_cases, dtype):
    """The same steps through CUDA graphs (sizes rounded up to a class, padding rows, the state
    restored after the run that precedes a capture) and launched one by one."""
    case = putelix_cases["case_c"]
    a, b = case.tokens(140, 401), case.tokens(30, 402)
    eager, graphs = _runner(case, dtype, pages=24), _runner(case, dtype, pages=24, cuda_graphs=True)
    plan = [[("a", a[:100], [99])], [("a", a[100:120], [0, 19]), ("b", b[:1], [0])],
            [("a", a[120:121], [0]), ("b", b[1:2], [0])], [("a", a[121:122], [0]), ("b", b[2:3], [0])],
            [("a", a[122:140], [17]), ("b", b[3:4], [0])], [("a2", a[:100], [99])]]
    for step in plan:
        want = eager.step([StepEntry(r, t, w) for r, t, w in step]).logits.clone()
        got = graphs.step([StepEntry(r, t, w) for r, t, w in step]).logits.clone()
        for i in range(want.shape[0]):
            assert uc.rms_error(got[i].cpu(), want[i].cpu()) < (2e-2 if dtype == "bfloat16" else 1e-5), step[0][0]
    assert uc.rms_error(want[0].cpu(), case.logits(a, dtype)[99]) < TOL[dtype] * 3


def _greedy(case, prompt, n):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        row = plain_putelix.forward(case.config, case.plain, toks)[-1]
        top = torch.topk(row, 2).values
        margins.append(float(top[0] - top[1]))
        out.append(int(row.argmax()))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(putelix_case, graphs):
    """Prompts of unequal length, cut into portions by a small token budget, decoded side by
    side by the scheduler (with and without CUDA graphs: the recurrent state must survive the
    capture); the tokens are the plain model's greedy tokens."""
    from hetero_serve_b200 import LLMEngine
    case = putelix_case
    prompts = [case.tokens(n, 200 + n) for n in (37, 5, 18)]
    eng = LLMEngine(case.dir, dtype="float32", num_blocks=24, max_batch=4, max_prefill_tokens=16,
                    policy="mixed", cuda_graphs=graphs, device=DEV)
    got = eng.generate(prompts, max_new_tokens=10)
    for p, g in zip(prompts, got):
        want, margins = _greedy(case, p, 10)
        for i, (a, b, m) in enumerate(zip(g, want, margins)):
            if m < 1e-3:
                break                                         # a close call: stop comparing
            assert a == b, (len(p), i, g, want)
    eng.runner.manager.check()


def test_command_line_runs_a_preset():
    out = subprocess.run([sys.executable, "-m", "hetero_serve_b200", "--model", "putelix-tiny",
                          "--random-prompts", "2:12", "--max-new-tokens", "4"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
