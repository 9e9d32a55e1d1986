"""The kernels of the Pedorax parts, each alone, against its plain twin (tests/plain_ops.py,
float64 on the CPU): the norm without statistics, rotary pairs, the block-diagonal linear,
attention over a shared latent with a sink, the gated delta rule, the routed experts."""

import math

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32


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
    err = (got.detach().cpu().double() - want.double()).abs().max().item()
    assert err <= tol, err


# -- norm, scale, rotation, block-diagonal linear ----------------------------------------------
@pytest.mark.parametrize("dtype, tol", [(F32, 2e-6), (BF16, 1e-2)])
def test_dyt_norm(ops, plain, dtype, tol):
    x, w, b = rnd(9, 100, seed=1, std=2.0), rnd(100, seed=2), rnd(100, seed=3)
    rows = ints(7, 0, 3, 3)
    for sel, n in ((None, 9), (rows, 4)):
        want = torch.zeros(n, 100, dtype=torch.float64)
        plain.dyt_norm(want, x, w, b, 0.7, sel)
        got = torch.zeros(n, 100, dtype=dtype, device=DEV)
        ops.dyt_norm(got, dev(x), dev(w), dev(b), 0.7, None if sel is None else dev(sel))
        close(got, want, tol)


def test_scale(ops):
    t = rnd(5, 333, seed=4)
    got = dev(t.clone())
    ops.scale_(got, -0.375)
    close(got, t.double() * -0.375, 1e-7)


def test_rotary_pairs_far_positions(ops, plain):
    """Three vectors a row, rotated on their first 6 of 10 entries, at positions up to 2e5:
    the angle must not lose accuracy with the position."""
    buf = rnd(6, 64, seed=5)
    pos, req = ints(0, 1, 777, 65536, 199999, 12), ints(0, 0, 1, 1, 2, -1)
    freq = torch.pow(torch.tensor(500.0, dtype=torch.float64), -2.0 * torch.arange(3) / 6)
    want = buf.double().clone()
    plain.rotary_pairs(want, pos, req, freq, n_vec=3, vec_stride=14, offset=5, dims=6)
    got = dev(buf.clone())
    ops.rotary_pairs(got, dev(pos), dev(req), dev(freq.float()), n_vec=3, vec_stride=14,
                     offset=5, dims=6)
    close(got, want, 5e-6)
    assert torch.equal(got[5].cpu(), buf[5])                       # a padding row is left alone
    untouched = [c for c in range(64) if not any(5 + 14 * v <= c < 11 + 14 * v for v in range(3))]
    assert torch.equal(got[:5, untouched].cpu(), buf[:5, untouched])


@pytest.mark.parametrize("wdt, odt, tol", [(F32, F32, 1e-5), (BF16, F32, 1e-5), (BF16, BF16, 7e-2)])
def test_grouped_linear_on_slices(ops, plain, wdt, odt, tol):
    T, groups, k, n = 11, 3, 10, 37
    a = rnd(T, 50, seed=6)
    w = rnd(groups, k, n, seed=7).to(wdt)
    want = torch.zeros(T, groups * n, dtype=torch.float64)
    plain.grouped_linear(want, a, w, a_offset=4, a_group_stride=15)
    got = torch.zeros(T, groups * n, dtype=odt, device=DEV)
    ops.grouped_linear(got, dev(a), dev(w), a_offset=4, a_group_stride=15)
    close(got, want, tol)


@pytest.mark.parametrize("odt, tol", [(F32, 3e-2), (BF16, 8e-2)])
@pytest.mark.parametrize("T, groups, k, n", [(150, 3, 64, 40), (64, 2, 32, 200), (129, 1, 96, 64)])
def test_grouped_linear_on_the_tensor_cores(ops, plain, odt, tol, T, groups, k, n):
    """Many tokens in bfloat16 with the weights also given n-major: tiles on the tensor cores;
    the input is rounded to bfloat16 there, which bounds the agreement."""
    a = rnd(T, 20 + groups * (k + 12) + T % 2, seed=8)      # an odd row length: no 16-byte loads
    w = rnd(groups, k, n, seed=9, std=0.3).to(BF16)
    want = torch.zeros(T, groups * n, dtype=torch.float64)
    plain.grouped_linear(want, a, w, a_offset=20, a_group_stride=k + 12)
    got = torch.zeros(T, groups * n, dtype=odt, device=DEV)
    w_nk = w.transpose(1, 2).contiguous()
    ops.grouped_linear(got, dev(a), dev(w), a_offset=20, a_group_stride=k + 12, w_nk=dev(w_nk))
    close(got, want, tol)
    exact = torch.zeros(T, groups * n, dtype=F32, device=DEV)
    ops.grouped_linear(exact, dev(a), dev(w), a_offset=20, a_group_stride=k + 12)
    close(exact, want, 1e-4)
    assert (got.float() - exact).abs().max() > 0          # the other kernel did run


# -- attention over a shared latent ---------------------------------------------------------------
class Latent:
    """A cache of two requests on scattered pages, filled through latent_append."""

    def __init__(self, ops, plain, lens, rank, rot, cache_dtype, seed=0, page_size=16, pages=64):
        self.rank, self.rot, self.ps = rank, rot, page_size
        W = rank + rot
        g = torch.Generator().manual_seed(seed)
        order = torch.randperm(pages, generator=g).tolist()
        max_pages = max(-(-n // page_size) for n in lens) + 1
        self.table = torch.full((len(lens), max_pages), -1, dtype=I32)
        for r, n in enumerate(lens):
            for i in range(-(-n // page_size)):
                self.table[r, i] = order.pop()
        self.pool = torch.zeros(pages, 1, 1, page_size, W, dtype=cache_dtype)
        self.pool_dev = dev(self.pool.clone())
        self.lens = lens

    def append(self, ops, plain, proj, pos, req, norm_w, c_offset, eps=1e-5):
        plain.latent_append(self.pool, proj, norm_w, self.table, pos, req, c_offset=c_offset,
                            rank=self.rank, rot_dim=self.rot, eps=eps, page_size=self.ps,
                            status=None)
        status = torch.zeros(1, dtype=I32, device=DEV)
        ops.latent_append(self.pool_dev, dev(proj), dev(norm_w), dev(self.table), dev(pos),
                          dev(req), c_offset=c_offset, rank=self.rank, rot_dim=self.rot, eps=eps,
                          page_size=self.ps, status=status)
        assert int(status.item()) == 0


def _fill(ops, plain, lens, rank, rot, cache_dtype, seed, boost=None):
    lat = Latent(ops, plain, lens, rank, rot, cache_dtype, seed)
    pos = torch.cat([torch.arange(n) for n in lens]).to(I32)
    req = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(I32)
    proj = rnd(len(pos), 3 + rank + rot, seed=seed + 1)
    if boost is not None:                     # one key far larger than the others, per request
        start = 0
        for r, n in enumerate(lens):
            if boost < n:
                proj[start + boost, 3 + rank:] *= 6.0
            start += n
    lat.append(ops, plain, proj, pos, req, rnd(rank, seed=seed + 2).abs() + 0.5, c_offset=3)
    return lat


def _attend(ops, plain, lat, queries, heads, sink, scale, seed, boost_q=None):
    """queries: (request, position) pairs; returns (got, want) [n, heads * rank]."""
    rank, rot = lat.rank, lat.rot
    n = len(queries)
    pos, req = ints(*[p for _, p in queries]), ints(*[r for r, _ in queries])
    qa = rnd(n, heads * rank, seed=seed, std=0.3)
    stride = rot + 5
    qr = rnd(n, 2 + heads * stride, seed=seed + 1, std=0.3)
    if boost_q is not None:
        qr *= boost_q
    want = torch.zeros(n, heads * rank, dtype=torch.float64)
    plain.latent_attention(want, qa, qr, lat.pool, lat.table, pos, req, sink, n_heads=heads,
                           rank=rank, rot_dim=rot, qr_head_stride=stride, qr_offset=2,
                           scale=scale, page_size=lat.ps, status=None)
    got = torch.zeros(n, heads * rank, dtype=F32, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    ops.latent_attention(got, dev(qa), dev(qr), lat.pool_dev, dev(lat.table), dev(pos), dev(req),
                         dev(sink), n_heads=heads, rank=rank, rot_dim=rot, qr_head_stride=stride,
                         qr_offset=2, scale=scale, page_size=lat.ps, status=status)
    assert int(status.item()) == 0
    return got, want


@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("cache_dtype, tol", [(F32, 2e-5), (BF16, 2e-5)])
@pytest.mark.parametrize("rank, rot, heads", [(24, 8, 3), (72, 4, 11), (130, 16, 1)])
def test_latent_attention_random(ops, plain, cache_dtype, tol, rank, rot, heads, splits):
    """The cache rows are rounded once (by the append, the same in twin and kernel); behind
    that both sides are exact, so the tolerance does not depend on the cache type."""
    lat = _fill(ops, plain, (70, 33), rank, rot, cache_dtype, seed=10)
    close(lat.pool_dev, lat.pool.double(), 4e-2 if cache_dtype == BF16 else 2e-6)
    lat.pool = lat.pool_dev.cpu().clone()          # attend over the very rows the kernel wrote
    queries = [(0, 0), (0, 1), (0, 15), (0, 16), (0, 31), (0, 32), (0, 69), (1, 0), (1, 32),
               (1, 17)]
    ops.latent_splits = splits          # one block a token, or its keys split over several
    try:
        got, want = _attend(ops, plain, lat, queries, heads, rnd(heads, seed=3), 0.2, seed=20)
    finally:
        ops.latent_splits = None
    close(got, want, tol)


@pytest.mark.parametrize("where", [0, 5, 15, 16, 17, 31, 32, 33, 63, 64, 500, 698, 699])
def test_latent_attention_finds_one_key_among_hundreds(ops, plain, where):
    """Position `where` carries a key several times larger than all others and the query
    points along it: nearly all weight must land there, wherever it lies (first tokens, page
    and tile borders, far back, the newest key)."""
    lat = _fill(ops, plain, (700,), 16, 8, F32, seed=30, boost=where)
    rows = lat.pool.view(-1, 16, 24)
    key = rows[int(lat.table[0, where // 16]), where % 16]
    n = 1
    qa = torch.zeros(n, 16)
    qr = torch.zeros(n, 2 + 13)
    qr[0, 2:10] = key[16:] * 2.0
    sink = torch.tensor([-3.0])
    pos, req = ints(699), ints(0)
    want = torch.zeros(n, 16, dtype=torch.float64)
    plain.latent_attention(want, qa, qr, lat.pool, lat.table, pos, req, sink, n_heads=1, rank=16,
                           rot_dim=8, qr_head_stride=13, qr_offset=2, scale=1.0, page_size=16,
                           status=None)
    got = torch.zeros(n, 16, dtype=F32, device=DEV)
    ops.latent_attention(got, dev(qa), dev(qr), lat.pool_dev, dev(lat.table), dev(pos), dev(req),
                         dev(sink), n_heads=1, rank=16, rot_dim=8, qr_head_stride=13, qr_offset=2,
                         scale=1.0, page_size=16, status=torch.zeros(1, dtype=I32, device=DEV))
    close(got, want, 2e-5)
    assert (want[0] - key[:16].double()).abs().max() < 0.05      # the test's premise
    if where > 0:                  # and a query one position before the key must not see it
        got2 = torch.zeros(n, 16, dtype=F32, device=DEV)
        ops.latent_attention(got2, dev(qa), dev(qr), lat.pool_dev, dev(lat.table),
                             dev(ints(where - 1)), dev(req), dev(sink), n_heads=1, rank=16,
                             rot_dim=8, qr_head_stride=13, qr_offset=2, scale=1.0, page_size=16,
                             status=torch.zeros(1, dtype=I32, device=DEV))
        assert (got2[0].cpu().double() - key[:16].double()).abs().max() > 0.3


def test_latent_rotations_fused_into_append_and_attention(ops, plain):
    """The key part turns as it is written, the query parts as they are read: the same as
    rotating both beforehand with rotary_pairs."""
    rank, rot, heads, dims = 24, 12, 3, 8
    lens = (45, 20)
    freq = torch.pow(torch.tensor(300.0, dtype=torch.float64), -2.0 * torch.arange(dims // 2) / dims)
    f32 = freq.float()
    lat = Latent(ops, plain, lens, rank, rot, F32, seed=44)
    pos = torch.cat([torch.arange(n) for n in lens]).to(I32)
    req = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(I32)
    proj = rnd(len(pos), 3 + rank + rot, seed=45)
    norm_w = rnd(rank, seed=46).abs() + 0.5
    # expected: rotate first with the twin of rotary_pairs, then the plain append
    turned = proj.double().clone()
    plain.rotary_pairs(turned, pos, req, freq, n_vec=1, vec_stride=rot, offset=3 + rank, dims=dims)
    want_pool = torch.zeros_like(lat.pool, dtype=torch.float64)
    plain.latent_append(want_pool, turned, norm_w, lat.table, pos, req, c_offset=3, rank=rank,
                        rot_dim=rot, eps=1e-5, page_size=16, status=None)
    status = torch.zeros(1, dtype=I32, device=DEV)
    ops.latent_append(lat.pool_dev, dev(proj), dev(norm_w), dev(lat.table), dev(pos), dev(req),
                      c_offset=3, rank=rank, rot_dim=rot, eps=1e-5, page_size=16, status=status,
                      freq=dev(f32), rot_dims=dims)
    close(lat.pool_dev, want_pool, 3e-6)
    lat.pool = lat.pool_dev.cpu().clone()
    n = 4
    qpos, qreq = ints(44, 7, 19, 0), ints(0, 0, 1, 1)
    qa, qr = rnd(n, heads * rank, seed=47, std=0.3), rnd(n, 2 + heads * (rot + 5), seed=48, std=0.3)
    qr_turned = qr.double().clone()
    plain.rotary_pairs(qr_turned, qpos, qreq, freq, n_vec=heads, vec_stride=rot + 5, offset=2, dims=dims)
    sink = rnd(heads, seed=49)
    want = torch.zeros(n, heads * rank, dtype=torch.float64)
    plain.latent_attention(want, qa, qr_turned, lat.pool, lat.table, qpos, qreq, sink,
                           n_heads=heads, rank=rank, rot_dim=rot, qr_head_stride=rot + 5,
                           qr_offset=2, scale=0.3, page_size=16, status=None)
    got = torch.zeros(n, heads * rank, dtype=F32, device=DEV)
    ops.latent_attention(got, dev(qa), dev(qr), lat.pool_dev, dev(lat.table), dev(qpos), dev(qreq),
                         dev(sink), n_heads=heads, rank=rank, rot_dim=rot, qr_head_stride=rot + 5,
                         qr_offset=2, scale=0.3, page_size=16, status=status, freq=dev(f32),
                         rot_dims=dims)
    close(got, want, 2e-5)
    assert int(status.item()) == 0


@pytest.mark.parametrize("rank, rot, heads", [(32, 8, 3), (48, 16, 8), (272, 24, 5), (16, 4, 70)])
def test_latent_attention_prompt_portions_on_the_tensor_cores(ops, plain, rank, rot, heads):
    """A step's plan sends a portion of 150 tokens (two tiles, the second one short) to the
    tensor-core kernel and two single tokens of another request to the CUDA-core kernel; the
    queries are rounded to bfloat16 there, which bounds the agreement.  Ranks above 256 run
    with eight warps a block; 70 heads put one token's heads into two blocks."""
    lat = _fill(ops, plain, (200, 33), rank, rot, BF16, seed=50)
    lat.pool = lat.pool_dev.cpu().clone()
    host_batch = [("a", 0, 50, 150), ("b", 1, 31, 2)]
    n = 152
    pos = torch.cat([torch.arange(50, 200), torch.arange(31, 33)]).to(I32)
    req = torch.cat([torch.zeros(150), torch.ones(2)]).to(I32)
    plan = ops.make_plan(host_batch, n, 16)
    assert plan.tile_cap == 2 and plan.decode_cap == 2
    stride = rot + 5
    qa = rnd(n, heads * rank, seed=51, std=0.3)
    qr = rnd(n, 2 + heads * stride, seed=52, std=0.3)
    sink = rnd(heads, seed=53)
    want = torch.zeros(n, heads * rank, dtype=torch.float64)
    plain.latent_attention(want, qa, qr, lat.pool, lat.table, pos, req, sink, n_heads=heads,
                           rank=rank, rot_dim=rot, qr_head_stride=stride, qr_offset=2, scale=0.2,
                           page_size=16, status=None)
    got = torch.full((n, heads * rank), 7.0, dtype=F32, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    before = ops.launches
    ops.latent_attention(got, dev(qa), dev(qr), lat.pool_dev, dev(lat.table), dev(pos), dev(req),
                         dev(sink), n_heads=heads, rank=rank, rot_dim=rot, qr_head_stride=stride,
                         qr_offset=2, scale=0.2, page_size=16, status=status, plan=plan)
    assert ops.launches - before >= 2 and int(status.item()) == 0
    close(got[150:], want[150:], 2e-5)                       # the single tokens: float32 queries
    close(got[:150], want[:150], 2e-2)


def test_latent_attention_sink_takes_weight_without_a_value(ops, plain):
    lat = _fill(ops, plain, (40,), 24, 8, F32, seed=40)
    queries = [(0, 0), (0, 39)]
    none = torch.full((2,), -1e4)
    got0, want0 = _attend(ops, plain, lat, queries, 2, none, 0.3, seed=41)
    close(got0, want0, 2e-5)
    big = torch.tensor([2.0, 9.0])
    got1, want1 = _attend(ops, plain, lat, queries, 2, big, 0.3, seed=41)
    close(got1, want1, 2e-5)
    # the sink only rescales: same direction, smaller norm; at position 0 the factor is known
    a, b = got0[0, :24].cpu().double(), got1[0, :24].cpu().double()
    f = float(a @ b / (a @ a))
    assert 0 < f < 1 and (b - f * a).abs().max() < 1e-5
    assert got1[:, 24:].norm() < got1[:, :24].norm() * 0.2        # the larger sink takes more


# -- the gated delta rule ----------------------------------------------------------------------------
def _delta_weights(shape, seed):
    H, HK, D, V = shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"]
    C = 2 * HK * D + H * V
    return dict(conv_w=rnd(C, shape["taps"], seed=seed, std=0.6),
                a2=rnd(shape["a_rank"], H * D, seed=seed + 1, std=0.5),
                dt_bias=rnd(H * D, seed=seed + 2, std=0.5), a_log=rnd(H, seed=seed + 3) - 1.0,
                g2=rnd(shape["g_rank"], H * V, seed=seed + 4, std=0.5),
                norm_w=rnd(V, seed=seed + 5).abs() + 0.5)


def _delta_run(o_ops, shape, w, proj, state, portions, slots, device):
    """Run requests (rows of `proj` one after another) through prepare / recurrence / finish
    in the given portions: portions[i] lists, per step, how many tokens request i brings."""
    H, HK, D, V = shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"]
    lens = [sum(p) for p in portions]
    starts = [sum(lens[:i]) for i in range(len(lens))]
    out = torch.zeros(sum(lens), H * V, dtype=torch.float64 if device == "cpu" else F32,
                      device=device)
    done = [0] * len(lens)
    mv = (lambda t: t.to(device).contiguous())
    wd = {k: mv(v) for k, v in w.items()}
    for step in range(max(len(p) for p in portions)):
        rows, tok_req, rs, rl, sl = [], [], [], [], []
        for r, p in enumerate(portions):
            n = p[step] if step < len(p) else 0
            if n == 0:
                continue
            rs.append(len(rows))
            rows += list(range(starts[r] + done[r], starts[r] + done[r] + n))
            tok_req += [len(rl)] * n
            rl.append(n)
            sl.append(slots[r])
            done[r] += n
        T = len(rows)
        pr = mv(proj[rows])
        f = dict(dtype=pr.dtype, device=device)
        qn, kn = torch.zeros(T, HK * D, **f), torch.zeros(T, HK * D, **f)
        vv, beta = torch.zeros(T, H * V, **f), torch.zeros(T, H, **f)
        decay, o = torch.zeros(T, H * D, **f), torch.zeros(T, H * V, **f)
        tq, a, b, c = mv(ints(*tok_req)), mv(ints(*rs)), mv(ints(*rl)), mv(ints(*sl))
        o_ops.delta_prepare(qn, kn, vv, beta, decay, pr, wd["conv_w"], wd["a2"], wd["dt_bias"],
                            wd["a_log"], state, tq, a, b, c, shape)
        o_ops.delta_recurrence(o, state, qn, kn, vv, beta, decay, a, b, c, shape)
        fin = torch.zeros(T, H * V, dtype=out.dtype, device=device)
        o_ops.delta_finish(fin, o, pr, wd["g2"], wd["norm_w"], tq, 1e-5, shape)
        out[rows] = fin
    return out


@pytest.mark.parametrize("shape", [
    dict(heads=4, kv_heads=2, dim=12, vdim=20, taps=4, a_rank=5, g_rank=3),
    dict(heads=2, kv_heads=1, dim=72, vdim=40, taps=3, a_rank=2, g_rank=9),     # 16 lanes a column
    dict(heads=3, kv_heads=3, dim=8, vdim=8, taps=1, a_rank=4, g_rank=4),       # no history
    dict(heads=1, kv_heads=1, dim=200, vdim=5, taps=2, a_rank=3, g_rank=3),
    dict(heads=2, kv_heads=2, dim=10, vdim=6, taps=2, a_rank=3, g_rank=2),      # rows not 16-byte
    dict(heads=1, kv_heads=1, dim=300, vdim=40, taps=2, a_rank=3, g_rank=2),    # two tokens a chunk
])
def test_delta_rule_in_portions_equals_the_whole(ops, plain, shape):
    """Two requests in slots 2 and 0 of three, cut into portions shorter than the convolution's
    history (1, 2, 3 tokens) beside longer ones, against the twin fed each request whole."""
    H, HK, D, V = shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"]
    C = 2 * HK * D + H * V
    width = C + H + shape["a_rank"] + shape["g_rank"]
    w = _delta_weights(shape, 50)
    portions = [[1, 2, 1, 3, 9, 1, 1, 17], [6, 1, 1, 2, 30]]
    n = sum(map(sum, portions))
    proj = rnd(n, width, seed=60, std=1.5)
    per_slot = H * D * V + (shape["taps"] - 1) * C
    state_c = torch.zeros(3, per_slot, dtype=torch.float64)
    want = _delta_run(plain, shape, {k: v.double() for k, v in w.items()}, proj.double(), state_c,
                      [[sum(p)] for p in portions], [2, 0], "cpu")
    state_g = torch.zeros(3, per_slot, dtype=F32, device=DEV)
    got = _delta_run(ops, shape, w, proj, state_g, portions, [2, 0], DEV)
    close(got, want, 3e-5)
    close(state_g, state_c, 3e-5)
    assert state_g[1].abs().max() == 0                       # the slot nobody owns is untouched


def test_delta_rule_long_decoding(ops, plain):
    shape = dict(heads=2, kv_heads=2, dim=16, vdim=24, taps=4, a_rank=4, g_rank=4)
    C = 2 * 2 * 16 + 2 * 24
    w = _delta_weights(shape, 70)
    n = 400
    proj = rnd(n, C + 2 + 8, seed=71, std=1.5)
    per_slot = 2 * 16 * 24 + 3 * C
    state_c = torch.zeros(1, per_slot, dtype=torch.float64)
    want = _delta_run(plain, shape, {k: v.double() for k, v in w.items()}, proj.double(), state_c,
                      [[n]], [0], "cpu")
    state_g = torch.zeros(1, per_slot, dtype=F32, device=DEV)
    got = _delta_run(ops, shape, w, proj, state_g, [[40] + [1] * 360], [0], DEV)
    close(got, want, 5e-5)
    close(state_g, state_c, 5e-5)


def test_delta_finish_writes_the_compute_type(ops, plain):
    shape = dict(heads=2, kv_heads=1, dim=8, vdim=12, taps=2, a_rank=3, g_rank=5)
    C = 2 * 8 + 2 * 12
    proj, o = rnd(7, C + 2 + 3 + 5, seed=80), rnd(7, 24, seed=81)
    w = _delta_weights(shape, 82)
    req = ints(0, 0, 0, 1, 1, 1, 1)
    want = torch.zeros(7, 24, dtype=torch.float64)
    plain.delta_finish(want, o, proj, w["g2"], w["norm_w"], req, 1e-6, shape)
    got = torch.zeros(7, 24, dtype=BF16, device=DEV)
    ops.delta_finish(got, dev(o), dev(proj), dev(w["g2"]), dev(w["norm_w"]), dev(req), 1e-6, shape)
    close(got, want, 2e-2)


# -- routed experts ----------------------------------------------------------------------------------
@pytest.mark.parametrize("E, top, groups, keep", [(12, 4, 3, 2), (8, 1, 1, 1), (6, 3, 6, 4),
                                                   (64, 8, 8, 3)])
@pytest.mark.parametrize("hdt", [F32, BF16])
def test_route(ops, plain, E, top, groups, keep, hdt):
    T, width = 37, 50
    h = rnd(T, width, seed=90).to(hdt)
    wr = rnd(E, width, seed=91, std=0.4)
    req = torch.zeros(T, dtype=I32)
    req[5] = -1
    wi, ww = torch.zeros(T, top, dtype=I32), torch.zeros(T, top, dtype=torch.float64)
    plain.moe_route(wi, ww, h, wr, req, top=top, n_groups=groups, keep=keep)
    gi = torch.full((T, top), -7, dtype=I32, device=DEV)
    gw = torch.zeros(T, top, dtype=F32, device=DEV)
    ops.moe_route(gi, gw, dev(h), dev(wr), dev(req), top=top, n_groups=groups, keep=keep)
    gi, gw = gi.cpu(), gw.cpu()
    assert (gi[5] == -7).all()
    for t in range(T):
        if t == 5:
            continue
        a = dict(zip(wi[t].tolist(), ww[t].tolist()))
        b = dict(zip(gi[t].tolist(), gw[t].tolist()))
        assert a.keys() == b.keys(), t
        assert max(abs(a[k] - b[k]) for k in a) < 1e-5
        assert gw[t, 0] >= gw[t, -1]                            # largest score first
    # the same choice when the logits are handed in (formed elsewhere as one matrix product)
    z = (h.double() @ wr.double().T).float()
    gi2 = torch.full((T, top), -7, dtype=I32, device=DEV)
    gw2 = torch.zeros(T, top, dtype=F32, device=DEV)
    ops.moe_route(gi2, gw2, dev(h), dev(wr), dev(req), top=top, n_groups=groups, keep=keep,
                  z=dev(z))
    keep_rows = [t for t in range(T) if t != 5]
    assert torch.equal(gi2.cpu()[keep_rows].sort(-1).values, gi[keep_rows].sort(-1).values)
    assert (gw2.cpu()[keep_rows].sort(-1).values - gw[keep_rows].sort(-1).values).abs().max() < 1e-5


def test_route_bars_the_best_expert_of_a_weak_group(ops):
    """Expert 0 has the largest score of all, but its group's two best sum to less than the
    other groups' and only one group is kept."""
    width = 8
    h = torch.zeros(1, width)
    h[0, 0] = 1.0
    wr = torch.zeros(6, width)
    wr[:, 0] = torch.tensor([3.0, -9.0, 2.0, 2.5, 0.1, 0.2])
    gi = torch.zeros(1, 2, dtype=I32, device=DEV)
    gw = torch.zeros(1, 2, dtype=F32, device=DEV)
    ops.moe_route(gi, gw, dev(h), dev(wr), dev(ints(0)), top=2, n_groups=3, keep=1)
    assert gi.cpu().tolist() == [[3, 2]]
    s3, s2 = 1 / (1 + math.exp(-2.5)), 1 / (1 + math.exp(-2.0))
    assert abs(gw[0, 0].item() - s3 / (s3 + s2)) < 1e-6


@pytest.mark.parametrize("dt, tol", [(F32, 2e-5), (BF16, 2e-5)])
def test_experts(ops, plain, dt, tol):
    """A limit low enough to clip many gates and ups; the inputs are rounded to the compute
    type before both sides see them, so the tolerance is that of float32 sums."""
    T, width, ff, E, top = 19, 40, 28, 5, 3
    h = rnd(T, width, seed=100).to(dt)
    wg, wu = rnd(E, ff, width, seed=101, std=0.4).to(dt), rnd(E, ff, width, seed=102, std=0.4).to(dt)
    wd = rnd(E, width, ff, seed=103, std=0.3).to(dt)
    g = torch.Generator().manual_seed(104)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(I32)
    wts = torch.rand(T, top, generator=g)
    req = torch.zeros(T, dtype=I32)
    req[3] = -1
    x = rnd(T, width, seed=105)
    want = x.double().clone()
    plain.moe_experts(want, None, h, wg, wu, wd, idx, wts, req, limit=0.8)
    got = dev(x.clone())
    y = torch.zeros(T * top, ff, dtype=F32, device=DEV)
    ops.moe_experts(got, y, dev(h), dev(wg), dev(wu), dev(wd), dev(idx), dev(wts), dev(req),
                    limit=0.8)
    close(got, want, tol)
    assert torch.equal(got[3].cpu(), x[3])


@pytest.mark.parametrize("T, width, ff, E, top", [(300, 64, 96, 7, 3), (90, 160, 32, 4, 3)])
def test_experts_sorted_by_expert_on_the_tensor_cores(ops, plain, T, width, ff, E, top):
    """Enough pairs for the sorted path: segments longer and shorter than a tile, an expert
    nobody picks, padding tokens.  Both sides see the same bfloat16 inputs; the kernel also
    rounds the activations to bfloat16, which bounds the agreement."""
    h = rnd(T, width, seed=110).to(BF16)
    wg, wu = rnd(E, ff, width, seed=111, std=0.3).to(BF16), rnd(E, ff, width, seed=112, std=0.3).to(BF16)
    wd = rnd(E, width, ff, seed=113, std=0.3).to(BF16)
    g = torch.Generator().manual_seed(114)
    idx = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(T)]).to(I32)
    idx[idx == 2] = E - 1                                  # expert 2 stays without tokens
    idx[:40] = torch.tensor([0, 1, 3][:top], dtype=I32)    # a long segment for expert 0
    wts = torch.rand(T, top, generator=g)
    req = torch.zeros(T, dtype=I32)
    req[[3, 77]] = -1
    x = rnd(T, width, seed=115)
    want = x.double().clone()
    plain.moe_experts(want, None, h, wg, wu, wd, idx, wts, req, limit=1.5)
    got = dev(x.clone())
    y = torch.zeros(T * top, ff, dtype=F32, device=DEV)
    assert ops.sorted_experts
    before = ops.launches
    ops.moe_experts(got, y, dev(h), dev(wg), dev(wu), dev(wd), dev(idx), dev(wts), dev(req),
                    limit=1.5)
    assert ops.launches - before == 4                      # sort, two tile kernels, combine
    scale = (want - x.double()).abs().max().item()
    close(got, want, 1e-2 * scale)
    assert torch.equal(got[3].cpu(), x[3]) and torch.equal(got[77].cpu(), x[77])
    ops.sorted_experts, ops._moe_need = False, {}
    try:
        rows = dev(x.clone())
        ops.moe_experts(rows, y, dev(h), dev(wg), dev(wu), dev(wd), dev(idx), dev(wts), dev(req),
                        limit=1.5)
    finally:
        ops.sorted_experts, ops._moe_need = True, {}
    close(rows, want, 1e-4 * scale)
