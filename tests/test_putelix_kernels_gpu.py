"""The kernels of the Putelix parts, each alone, against its plain twin (tests/plain_ops.py,
float64 on the CPU): root-mean-square norms (also of a sublayer's output, of a pair of outputs),
the query/key preparation and attention with a distance bias, a score cap and a chunked mask,
lightning attention, the routing by the largest logits, silu-gated experts, the gated
activation, and the new epilogues of the linear kernels."""

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, I32, F64 = torch.float32, torch.bfloat16, torch.int32, torch.float64


@pytest.fixture(scope="module")
def ops():
    from hetero_serve_b200.kernels import CudaOps
    return CudaOps(DEV)


@pytest.fixture(scope="module")
def plain():
    return plain_ops.PlainOps()


def rnd(*shape, seed=0, std=1.0, dtype=F32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def dev(*ts):
    out = tuple(t.to(DEV).contiguous() for t in ts)
    return out if len(out) > 1 else out[0]


def ints(*v):
    return torch.tensor(v, dtype=I32)


def close(got, want, tol):
    """Largest difference, relative for entries above 1 (bfloat16 rounds in proportion)."""
    want = want.double()
    err = ((got.detach().cpu().double() - want).abs() / (1.0 + want.abs())).max().item()
    assert err <= tol, err


# -- norms ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype, tol", [(F32, 3e-6), (BF16, 2e-2)])
@pytest.mark.parametrize("width", [5, 100, 1030])
def test_rms_norm(ops, plain, dtype, tol, width):
    x, w = rnd(9, width, seed=1, std=3.0), rnd(width, seed=2)
    gate = rnd(9, width + 7, seed=3)
    rows = ints(7, 0, 3, 3)
    for sel, n in ((None, 9), (rows, 4)):
        for one_plus, g in ((False, None), (True, None), (False, gate)):
            want = torch.zeros(n, width, dtype=F64)
            plain.rms_norm(want, x, w, 1e-5, sel, one_plus=one_plus, gate=g, gate_offset=4)
            got = torch.zeros(n, width, dtype=dtype, device=DEV)
            ops.rms_norm(got, dev(x), dev(w), 1e-5, None if sel is None else dev(sel),
                         one_plus=one_plus, gate=None if g is None else dev(g), gate_offset=4)
            close(got, want, tol)


@pytest.mark.parametrize("width", [6, 96, 2049])
def test_rms_norm_add(ops, plain, width):
    """One output, a pair of outputs side by side (with another eps inside), the pair without
    the norm around it; the copy in the compute type; a large eps so that it shows."""
    x = rnd(7, width, seed=4)
    a, b = rnd(7, width, seed=5, std=0.01), rnd(7, width, seed=6, std=5.0)
    w, wa, wb = rnd(width, seed=7), rnd(width, seed=8), rnd(width, seed=9)
    for kw in (dict(), dict(b=b, wa=wa, wb=wb, mix=0.5), dict(b=b, wa=wa, wb=wb, mix=0.3, eps_in=2e-3)):
        for weight in (w, None):
            want = x.double().clone()
            plain.rms_norm_add(want, a, weight, 1e-4, **kw)
            got, h = dev(x.clone()), torch.zeros(7, width, dtype=BF16, device=DEV)
            ops.rms_norm_add(got, dev(a), None if weight is None else dev(weight), 1e-4, h=h,
                             **{k: (dev(v) if isinstance(v, torch.Tensor) else v)
                                for k, v in kw.items()})
            close(got, want, 2e-5)
            assert torch.equal(h.cpu(), got.cpu().to(BF16))
    # a row's result does not depend on its neighbours
    alone = dev(x[3:4].clone())
    ops.rms_norm_add(alone, dev(a[3:4]), dev(w), 1e-4, b=dev(b[3:4]), wa=dev(wa), wb=dev(wb))
    both = dev(x.clone())
    ops.rms_norm_add(both, dev(a), dev(w), 1e-4, b=dev(b), wa=dev(wa), wb=dev(wb))
    assert torch.equal(alone[0], both[3])


def test_cast_rows(ops):
    for n in (1, 7, 4096 + 3):
        x = rnd(n, seed=n)
        out = torch.zeros(n, dtype=BF16, device=DEV)
        ops.cast_rows(out, dev(x))
        assert torch.equal(out.cpu(), x.to(BF16))


# -- the new epilogues of the linear kernels ---------------------------------------------------
@pytest.mark.parametrize("act", ["relu2", "silu"])
@pytest.mark.parametrize("dtype, M, tol", [(F32, 5, 2e-5), (F32, 300, 2e-5), (BF16, 3, 4e-2),
                                           (BF16, 40, 4e-2), (BF16, 300, 4e-2)])
def test_linear_activations(ops, plain, act, dtype, M, tol):
    a, w, bias = rnd(M, 64, seed=1).to(dtype), rnd(96, 64, seed=2, std=0.2).to(dtype), rnd(96, seed=3)
    res = rnd(M, 96, seed=4)
    want = torch.zeros(M, 96, dtype=F64)
    plain.linear(want, a, w, bias, act=act, residual=res)
    got = torch.zeros(M, 96, dtype=F32, device=DEV)
    ops.linear(got, dev(a), dev(w), dev(bias), act=act, residual=dev(res))
    close(got, want, tol)
    got2 = torch.zeros(M, 96, dtype=dtype, device=DEV)
    ops.linear(got2, dev(a), dev(w), None, act=act)
    want2 = torch.zeros(M, 96, dtype=F64)
    plain.linear(want2, a, w, None, act=act)
    close(got2, want2, tol if dtype == F32 else 8e-2)


@pytest.mark.parametrize("M", [3, 40, 300])
@pytest.mark.parametrize("N", [5, 6, 518])
def test_linear_with_few_or_odd_output_columns(ops, plain, M, N):
    """Router logits (a handful of experts) and the mixer's fused projection (a width that is
    no multiple of 4) as float32 outputs of bfloat16 products."""
    a, w, bias = rnd(M, 64, seed=5).to(BF16), rnd(N, 64, seed=6, std=0.2).to(BF16), rnd(N, seed=7)
    for b in (bias, None):
        want = torch.zeros(M, N, dtype=F64)
        plain.linear(want, a, w, b)
        got = torch.full((M, N), float("nan"), dtype=F32, device=DEV)
        ops.linear(got, dev(a), dev(w), None if b is None else dev(b))
        close(got, want, 2e-5)


# -- attention with a distance bias, a cap and chunks -------------------------------------------
class Pages:
    """A request's pages scattered over a pool whose unused rows are NaN."""

    def __init__(self, n_req, max_pos, page, G, D, dtype, seed=0):
        self.page, self.G, self.D = page, G, D
        per = -(-max_pos // page)
        self.num = n_req * per + 5
        g = torch.Generator().manual_seed(seed)
        order = torch.randperm(self.num, generator=g)[:n_req * per]
        self.table = order.view(n_req, per).to(I32)
        self.pool = torch.full((self.num, 2, G, page, D), float("nan"), dtype=dtype)


def _attend(ops, plain, *, T_pos, T_req, pages, proj, wq, wk, bias, H, scale, cap, chunk, window,
            dtype, q_off, k_off, v_off, g_off, n_new):
    """Prepare (normed queries, pages) and attend for the last ``n_new`` tokens' worth of rows,
    on the twin and on the kernels; all rows are prepared (they fill the pages)."""
    G, D, page = pages.G, pages.D, pages.page
    n = proj.shape[0]
    kw = dict(q_off=q_off, k_off=k_off, v_off=v_off, eps=1e-5, writes=True, n_heads=H,
              n_kv_heads=G, head_dim=D, page_size=page, status=None)
    q_want = torch.zeros(n, H * D, dtype=F64)
    pool_want = pages.pool.double().clone()
    plain.qk_prepare(q_want, pool_want, proj, wq, wk, pages.table, T_pos, T_req, **kw)
    status = torch.zeros(1, dtype=I32, device=DEV)
    kw["status"] = status
    q_got = torch.zeros(n, H * D, dtype=dtype, device=DEV)
    pool_got = dev(pages.pool.clone())
    table, pos, req, proj_d = dev(pages.table, T_pos, T_req, proj)
    ops.qk_prepare(q_got, pool_got, proj_d, None if wq is None else dev(wq),
                   None if wk is None else dev(wk), table, pos, req, **kw)
    akw = dict(gate_offset=g_off, n_heads=H, n_kv_heads=G, head_dim=D, page_size=page,
               scale=scale, cap=cap, chunk=chunk, window=window)
    want = torch.zeros(n, H * D, dtype=F64)
    plain.biased_attention(want, q_want, pool_want, pages.table, T_pos, T_req, bias=bias,
                           gate=proj if g_off is not None else None, status=None,
                           **dict(akw, gate_offset=g_off or 0))
    got = torch.zeros(n, H * D, dtype=dtype, device=DEV)
    ops.biased_attention(got, q_got, pool_got, table, pos, req,
                         bias=None if bias is None else dev(bias),
                         gate=proj_d if g_off is not None else None, status=status,
                         **dict(akw, gate_offset=g_off or 0))
    assert int(status.item()) == 0
    return got, want, q_got, q_want, pool_got, pool_want


@pytest.mark.parametrize("dtype, tol", [(F32, 2e-5), (BF16, 6e-2)])
@pytest.mark.parametrize("H, G, D, chunk, window, page", [(4, 2, 16, 24, 0, 16), (3, 1, 40, 7, 0, 16),
                                                          (2, 2, 64, 0, 0, 8), (6, 3, 8, 50, 9, 16),
                                                          (2, 1, 256, 33, 0, 4)])
def test_prepare_and_attention(ops, plain, dtype, tol, H, G, D, chunk, window, page):
    """Two requests of unequal length with scattered pages, every position a query, a padding
    row in between; norms over the whole projections, values = the keys as projected."""
    lens = (70, 23)
    pos = torch.cat([torch.arange(lens[0]), ints(0), torch.arange(lens[1])]).to(I32)
    req = torch.cat([torch.zeros(lens[0]), -torch.ones(1), torch.ones(lens[1])]).to(I32)
    n = pos.shape[0]
    stride = 5 + H * D + G * D + H + 3
    proj = rnd(n, stride, seed=11)
    wq, wk = rnd(H * D, seed=12) + 1.5, rnd(G * D, seed=13) + 1.5
    n_dist = max(chunk, window) or 128
    bias = rnd(H, n_dist, seed=14)
    pages = Pages(2, 80, page, G, D, dtype, seed=H)
    got, want, qg, qw, pg, pw = _attend(
        ops, plain, T_pos=pos, T_req=req, pages=pages, proj=proj, wq=wq, wk=wk, bias=bias, H=H,
        scale=0.4, cap=6.0, chunk=chunk, window=window, dtype=dtype, q_off=5, k_off=5 + H * D,
        v_off=None, g_off=5 + H * D + G * D, n_new=n)
    live = req >= 0
    close(qg[live], qw[live], tol)
    filled = ~torch.isnan(pw)
    assert torch.equal(torch.isnan(pg.cpu().float()), ~filled)     # the same rows were written
    close(torch.nan_to_num(pg.float()), torch.nan_to_num(pw), tol)
    close(got[live], want[live], tol)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("chunk, window", [(24, 0), (0, 19), (40, 11)])
def test_one_large_key_at_every_edge(ops, plain, dtype, chunk, window):
    """One key with a score far above the others, the query at every distance from it: the
    output is that key's value exactly while the key is visible (same chunk, inside the
    window) and has nothing of it one position later.  No norms, no cap, no bias: the edge
    alone decides."""
    H, G, D, page, L = 2, 1, 16, 16, 100
    for key_at in (0, 15, 16, 23, 24, 47, 48, 71):
        proj = rnd(L, H * D + 2 * G * D, seed=20 + key_at, std=0.05)
        proj[:, :H * D] = 0.0
        proj[:, :H * D:D] = 1.0                                 # every query: e_0 per head
        proj[key_at, H * D] = 60.0                              # the key's first entry
        proj[key_at, H * D + G * D:] = 7.0                      # its value (a separate projection)
        pos, req = torch.arange(L, dtype=I32), torch.zeros(L, dtype=I32)
        pages = Pages(1, L, page, G, D, dtype, seed=key_at)
        got, want, *_ = _attend(ops, plain, T_pos=pos, T_req=req, pages=pages, proj=proj, wq=None,
                                wk=None, bias=None, H=H, scale=1.0, cap=0.0, chunk=chunk,
                                window=window, dtype=dtype, q_off=0, k_off=H * D,
                                v_off=H * D + G * D, g_off=None, n_new=L)
        for i in range(key_at, L):
            seen = (chunk == 0 or i // chunk == key_at // chunk) and (window == 0 or i - key_at < window)
            v = got[i].float().abs().max().item()
            assert (v > 6.9) == seen, (key_at, i, v)
        close(got, want, 1e-4 if dtype == F32 else 5e-2)


@pytest.mark.parametrize("dtype, tol", [(F32, 3e-5), (BF16, 6e-2)])
def test_a_far_key_among_hundreds_and_the_bias(ops, plain, dtype, tol):
    """No chunk: 700 keys over many pages, one of them large, then the same scores with a bias
    that prefers another distance; single queries (decoding) at the end of the context."""
    H, G, D, page, L = 2, 2, 32, 16, 700
    proj = rnd(L, H * D + G * D + H, seed=31, std=0.3)
    proj[37, H * D:H * D + G * D] *= 12.0
    pos, req = torch.arange(L, dtype=I32), torch.zeros(L, dtype=I32)
    bias = torch.zeros(H, 1024)
    bias[:, 500] = 25.0
    for b in (None, bias):
        pages = Pages(1, L, page, G, D, dtype, seed=3)
        got, want, *_ = _attend(ops, plain, T_pos=pos, T_req=req, pages=pages, proj=proj,
                                wq=torch.ones(H * D), wk=torch.ones(G * D), bias=b, H=H, scale=1.0,
                                cap=30.0, chunk=0, window=0, dtype=dtype, q_off=0, k_off=H * D,
                                v_off=None, g_off=H * D + G * D, n_new=L)
        close(got[600:], want[600:], tol)


@pytest.mark.parametrize("H, G, D, chunk, window", [(4, 2, 16, 24, 0), (2, 1, 64, 96, 0),
                                                    (3, 3, 32, 0, 0), (2, 2, 128, 200, 70),
                                                    (6, 2, 64, 7, 0), (2, 1, 48, 0, 33)])
def test_prompt_portions_on_the_tensor_cores(ops, plain, H, G, D, chunk, window):
    """The step's work list: portions of 150 and 131 queries that start in the middle of a
    context (and of a chunk) as tiles on the tensor cores, a request bringing three tokens and
    one bringing one on the CUDA cores; all against the twin, which knows no lists."""
    page = 16
    starts, news = (37, 0, 90, 11), (150, 131, 3, 1)
    pos = torch.cat([torch.arange(s + n) for s, n in zip(starts, news)]).to(I32)
    req = torch.cat([torch.full((s + n,), r) for r, (s, n) in enumerate(zip(starts, news))]).to(I32)
    n = pos.shape[0]
    stride = H * D + G * D + H
    proj = rnd(n, stride, seed=15, std=0.6)
    wq, wk = rnd(H * D, seed=16) * 0.2 + 1.2, rnd(G * D, seed=17) * 0.2 + 1.2
    bias = rnd(H, max(chunk, window) or 256, seed=18)
    pages = Pages(4, 200, page, G, D, BF16, seed=D)
    # every token is prepared (the context fills the pages); the step's own tokens are queries
    kw = dict(q_off=0, k_off=H * D, v_off=None, eps=1e-5, writes=True, n_heads=H, n_kv_heads=G,
              head_dim=D, page_size=page)
    q_want, pool_want = torch.zeros(n, H * D, dtype=F64), pages.pool.double().clone()
    plain.qk_prepare(q_want, pool_want, proj, wq, wk, pages.table, pos, req, status=None, **kw)
    status = torch.zeros(1, dtype=I32, device=DEV)
    q_all = torch.zeros(n, H * D, dtype=BF16, device=DEV)
    pool_got = dev(pages.pool.clone())
    ops.qk_prepare(q_all, pool_got, dev(proj), dev(wq), dev(wk), dev(pages.table), dev(pos),
                   dev(req), status=status, **kw)
    # the step: the last `new` tokens of every request, flat and in request order
    sel = torch.cat([torch.nonzero(req == r).flatten()[-m:] for r, m in enumerate(news)])
    T = sel.shape[0]
    akw = dict(bias=bias, gate_offset=H * D + G * D, n_heads=H, n_kv_heads=G, head_dim=D,
               page_size=page, scale=0.35, cap=9.0, chunk=chunk, window=window)
    want = torch.zeros(T, H * D, dtype=F64)
    plain.biased_attention(want, q_want[sel], pool_want, pages.table, pos[sel], req[sel],
                           gate=proj[sel], status=None, **akw)
    plan = ops.make_plan([(r, r, s, m) for r, (s, m) in enumerate(zip(starts, news))], T, page)
    assert plan.tile_cap == 4 and plan.decode_cap == 4
    got = torch.full((T, H * D), float("nan"), dtype=BF16, device=DEV)
    # the pages that lie wholly before the first key a request's first query sees have been
    # given back: the kernels must not look them up
    freed = pages.table.clone()
    for r, s0 in enumerate(starts):
        lo = s0 // chunk * chunk if chunk else 0
        if window:
            lo = max(lo, s0 - window + 1)
        freed[r, :lo // page] = -1
    ops.biased_attention(got, q_all[dev(sel)].contiguous(), pool_got, dev(freed),
                         dev(pos[sel]), dev(req[sel]), gate=dev(proj[sel]), status=status,
                         plan=plan, **dict(akw, bias=dev(bias)))
    assert int(status.item()) == 0
    close(got, want, 5e-2)
    # and the same rows through the CUDA-core kernel alone
    slow = torch.zeros(T, H * D, dtype=BF16, device=DEV)
    ops.biased_attention(slow, q_all[dev(sel)].contiguous(), pool_got, dev(pages.table),
                         dev(pos[sel]), dev(req[sel]), gate=dev(proj[sel]), status=status,
                         **dict(akw, bias=dev(bias)))
    close(got, slow.cpu().double(), 4e-2)


def test_attention_rows_do_not_depend_on_the_batch(ops, plain):
    """The same token alone and among others, its pages elsewhere: the same bits."""
    H, G, D, page = 4, 2, 16, 16
    proj = rnd(60, H * D + G * D + H, seed=41)
    pos, req = torch.arange(60, dtype=I32), torch.zeros(60, dtype=I32)
    outs = []
    for seed in (1, 2):
        pages = Pages(1, 60, page, G, D, F32, seed=seed)
        got, *_ = _attend(ops, plain, T_pos=pos, T_req=req, pages=pages, proj=proj,
                          wq=torch.ones(H * D), wk=torch.ones(G * D), bias=None, H=H, scale=0.5,
                          cap=5.0, chunk=24, window=0, dtype=F32, q_off=0, k_off=H * D, v_off=None,
                          g_off=H * D + G * D, n_new=60)
        outs.append(got.cpu())
    assert torch.equal(outs[0], outs[1])


# -- lightning attention ---------------------------------------------------------------------------
@pytest.mark.parametrize("H, D, V", [(2, 16, 16), (3, 8, 12), (1, 20, 5), (2, 64, 64), (1, 200, 33),
                                     (2, 128, 128)])
def test_lightning_in_portions_and_slots(ops, plain, H, D, V):
    """Two requests in two slots (not in slot order), a first step with portions of unequal
    length, then portions of 1 to 3 tokens; against the whole sequences on the twin."""
    lens = (37, 18)
    stride = 3 + 2 * H * D + H * V + 2
    q_off, k_off, v_off = 3, 3 + H * D, 3 + 2 * H * D
    seqs = [rnd(n, stride, seed=50 + i) for i, n in enumerate(lens)]
    decay = torch.tensor([0.997, 0.6, 1.0][:H], dtype=F32)
    kw = dict(q_off=q_off, k_off=k_off, v_off=v_off, heads=H, dim=D, vdim=V, act="silu")
    want = []
    state_w = torch.zeros(4, H * D * V, dtype=F64)
    for i, s in enumerate(seqs):
        o = torch.zeros(s.shape[0], H * V, dtype=F64)
        plain.lightning_recurrence(o, state_w, s, decay, ints(0), ints(s.shape[0]), ints(3 - 2 * i),
                                   **kw)
        want.append(o)
    state = torch.full((4, H * D * V), 0.0, dtype=F32, device=DEV)
    state[0] = float("nan")                       # slots nobody uses
    state[2] = float("nan")
    done = [0, 0]
    got = [torch.zeros(n, H * V) for n in lens]
    sizes = [(20, 5), (1, 3), (2, 1), (3, 2), (1, 1), (10, 6)]
    for sz in sizes:
        rows, starts, ns = [], [], []
        for r in (1, 0):                          # request 1 first in the batch
            n = min(sz[r], lens[r] - done[r])
            starts.append(sum(ns))
            ns.append(n)
            rows.append(seqs[r][done[r]:done[r] + n])
        proj = dev(torch.cat(rows))
        o = torch.full((proj.shape[0], H * V), float("nan"), dtype=F32, device=DEV)
        ops.lightning_recurrence(o, state, proj, dev(decay), dev(ints(*starts)), dev(ints(*ns)),
                                 dev(ints(1, 3)), **kw)
        for k, r in enumerate((1, 0)):
            got[r][done[r]:done[r] + ns[k]] = o[starts[k]:starts[k] + ns[k]].cpu()
            done[r] += ns[k]
    assert done == list(lens)
    for r in range(2):
        scale = want[r].abs().max().item()
        close(got[r], want[r], 3e-6 * max(1.0, scale))
    close(state[3], state_w[3], 3e-6 * max(1.0, state_w.abs().max().item()))
    assert torch.isnan(state[0]).all() and torch.isnan(state[2]).all()


@pytest.mark.parametrize("H, D, V", [(2, 64, 64), (1, 128, 32), (3, 16, 24), (1, 200, 36)])
def test_lightning_many_tokens_a_step(ops, plain, H, D, V):
    """Steps of many tokens activate their rows in a pass of their own and stream them; the
    bits are those of the few-token path.  Portions of 100 and 70 tokens, then 90 and 3."""
    stride = 2 * H * D + H * V + 5
    kw = dict(q_off=5, k_off=5 + H * D, v_off=5 + 2 * H * D, heads=H, dim=D, vdim=V, act="silu")
    decay = torch.tensor([0.997, 0.8, 0.5][:H])
    seqs = [rnd(190, stride, seed=70), rnd(73, stride, seed=71)]
    outs, states = [], []
    for bulk_from in (64, 10 ** 9):
        ops.lightning_bulk_rows = bulk_from
        state = torch.zeros(2, H * D * V, device=DEV)
        got = [torch.zeros(190, H * V), torch.zeros(73, H * V)]
        for (a0, a1), (b0, b1) in (((0, 100), (0, 70)), ((100, 190), (70, 73))):
            proj = dev(torch.cat([seqs[0][a0:a1], seqs[1][b0:b1]]))
            o = torch.zeros(proj.shape[0], H * V, device=DEV)
            ops.lightning_recurrence(o, state, proj, dev(decay), dev(ints(0, a1 - a0)),
                                     dev(ints(a1 - a0, b1 - b0)), dev(ints(1, 0)), **kw)
            got[0][a0:a1], got[1][b0:b1] = o[:a1 - a0].cpu(), o[a1 - a0:].cpu()
        outs.append(got)
        states.append(state.cpu())
    ops.lightning_bulk_rows = 64
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert torch.equal(states[0], states[1])
    want = torch.zeros(190, H * V, dtype=F64)
    plain.lightning_recurrence(want, torch.zeros(1, H * D * V, dtype=F64), seqs[0], decay, ints(0),
                               ints(190), ints(0), **kw)
    close(outs[0][0], want, 1e-5)


def test_lightning_long_decoding_is_bit_equal_to_one_portion(ops):
    """300 single-token steps against one portion of 300: the same chain of operations."""
    H, D, V, n = 2, 32, 24, 300
    proj = dev(rnd(n, 2 * H * D + H * V, seed=61, std=0.7))
    decay = dev(torch.tensor([0.997, 0.9]))
    kw = dict(q_off=0, k_off=H * D, v_off=2 * H * D, heads=H, dim=D, vdim=V, act="silu")
    s1 = torch.zeros(1, H * D * V, device=DEV)
    o1 = torch.zeros(n, H * V, device=DEV)
    ops.lightning_recurrence(o1, s1, proj, decay, dev(ints(0)), dev(ints(n)), dev(ints(0)), **kw)
    s2 = torch.zeros(1, H * D * V, device=DEV)
    o2 = torch.zeros(n, H * V, device=DEV)
    for t in range(n):
        ops.lightning_recurrence(o2[t:t + 1], s2, proj[t:t + 1].contiguous(), decay, dev(ints(0)),
                                 dev(ints(1)), dev(ints(0)), **kw)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


# -- routing and experts ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("E, top", [(5, 2), (2, 1), (3, 3), (64, 6)])
def test_route_top(ops, plain, dtype, E, top):
    """The largest logits with a bias that changes the order, ties by the lower index, weights
    by the softmax over the chosen; also with the logits handed in."""
    T, width = 9, 40
    h = rnd(T, width, seed=71).to(dtype)
    w = rnd(E, width, seed=72, std=0.3)
    w[E - 1] = w[0]                                              # a tie in every row
    bias = rnd(E, seed=73)
    bias[E - 1] = bias[0]
    req = ints(0, 0, 1, -1, 1, 2, 2, 2, 2)
    for b in (bias, None):
        for z in (None, h.float() @ w.t()):
            wi, ww = torch.zeros(T, top, dtype=I32), torch.zeros(T, top, dtype=F64)
            plain.moe_route_top(wi, ww, h, w, b, req, top=top, z=z)
            gi = torch.full((T, top), -7, dtype=I32, device=DEV)
            gw = torch.zeros(T, top, dtype=F32, device=DEV)
            ops.moe_route_top(gi, gw, dev(h), dev(w), None if b is None else dev(b), dev(req),
                              top=top, z=None if z is None else dev(z))
            live = req >= 0
            assert torch.equal(gi.cpu()[live], wi[live]) and (gi.cpu()[~live] == -7).all()
            close(gw[live], ww[live], 1e-5)
            if E > 1 and top < E:
                assert not ((gi.cpu()[live] == E - 1).any() and not (gi.cpu()[live] == 0).any())


@pytest.mark.parametrize("dtype, T, tol", [(F32, 7, 3e-5), (BF16, 7, 5e-2), (BF16, 200, 8e-2)])
def test_silu_experts(ops, plain, dtype, T, tol):
    """silu(gate) * up through both expert paths (a product per pair; sorted tiles)."""
    width, ff, E, top = 64, 96, 6, 2
    h = rnd(T, width, seed=81).to(dtype)
    wg, wu = rnd(E, ff, width, seed=82, std=0.2).to(dtype), rnd(E, ff, width, seed=83, std=0.2).to(dtype)
    wd = rnd(E, width, ff, seed=84, std=0.2).to(dtype)
    g = torch.Generator().manual_seed(85)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(I32)
    wt = torch.softmax(rnd(T, top, seed=86), 1)
    req = torch.zeros(T, dtype=I32)
    x = rnd(T, width, seed=87)
    want = x.double().clone()
    plain.moe_experts(want, None, h, wg, wu, wd, idx, wt, req, limit=0.0, act="silu")
    got = dev(x.clone())
    y = torch.zeros(T * top, ff, device=DEV)
    ops.moe_experts(got, y, dev(h), dev(wg), dev(wu), dev(wd), dev(idx), dev(wt), dev(req),
                    limit=0.0, act="silu")
    close(got, want, tol)


@pytest.mark.parametrize("dtype, tol", [(F32, 1e-5), (BF16, 3e-2)])
def test_gated_act(ops, plain, dtype, tol):
    T, ff, width = 6, 37, 50
    gu, h, ws = rnd(T, 2 * ff, seed=91).to(dtype), rnd(T, width, seed=92).to(dtype), \
        rnd(width, seed=93, std=0.3).to(dtype)
    for w_s in (ws, None):
        want = torch.zeros(T, ff, dtype=F64)
        plain.gated_act(want, gu, h, w_s, None, act="silu")
        got = torch.zeros(T, ff, dtype=dtype, device=DEV)
        ops.gated_act(got, dev(gu), dev(h), None if w_s is None else dev(w_s),
                      dev(torch.zeros(T, dtype=I32)), act="silu")
        close(got, want, tol)
