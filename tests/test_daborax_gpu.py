"""The Daborax decoder on the GPU against the plain implementation in ``plain_daborax`` (float64, whole sequences, no
cache): every mechanism's kernels alone, then small random models of several shapes through trace replay in four
cuttings and both precisions with pools that hold exactly what a trace needs, then long decoding and greedy
generation through the engine's entry point and scheduler.  Sizes are chosen so that nothing that could be confused
is equal (key and value sizes, heads and groups, state and head sizes, windows no multiple of the page size), and so
that values which a model may happen to make 1 or equal are also something else somewhere."""

import copy

import numpy as np
import pytest
import torch

import cuttings
import plain_daborax as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
F64 = torch.float64


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def rel_err(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


@pytest.fixture(scope="module")
def ops():
    from tokasaurus_b200.kernels import ops as o
    return o


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("H", [6, 33, 320])
def test_sinusoidal_positions(ops, H):
    from tokasaurus_b200.parts import SinusoidalPositions

    pos = [0, 1, 2, 17, 500, 4095, 3, 100000]
    x0 = torch.randn(len(pos), H)
    x = x0.to(DEV)
    ops.add_sinusoid(x, i32(pos), SinusoidalPositions(H).inv_freq().to(DEV))
    want = x0.double().clone()
    for r, p in enumerate(pos):
        want[r] += plain.position_vectors(1, H, start=p)[0]
    assert float((x.cpu().double() - want).abs().max()) < 5e-7  # angles in float64: only the float32 sum is rounded


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [24, 200, 1056])
def test_output_norm_with_scale_and_residual_add(ops, dtype, H):
    g = torch.Generator().manual_seed(H)
    x, y = torch.randn(5, H, generator=g) * 3, torch.randn(5, H, generator=g) * 0.2
    w, ls, b = torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.1
    for bias in (None, b):
        yb = y.double() if bias is None else y.double() + bias.double()
        want = x.double() + 0.6 * plain.rms_norm(yb, w.double(), 1e-6) * ls.double()
        xd = x.to(DEV)
        h = torch.empty(5, H, dtype=DT[dtype], device=DEV) if dtype == "bfloat16" else None
        ops.scaled_norm_add(xd, y.to(DEV), w.to(DEV), ls.to(DEV), 0.6, 1e-6, h, None if bias is None else bias.to(DEV))
        assert rel_err(xd.cpu(), want) < 1e-6
        if h is not None:
            assert rel_err(h.float().cpu(), want) < TOL[dtype]
    xd = x.to(DEV)
    ops.scaled_norm_add(xd, y.to(DEV), w.to(DEV), None, 1.0, 1e-6)  # no layer scale, multiplier 1
    assert rel_err(xd.cpu(), x.double() + plain.rms_norm(y.double(), w.double(), 1e-6)) < 1e-6
    sl = torch.randn(3, 5, H, generator=g) * 0.2  # float32 slices of a split product instead
    xd = x.to(DEV)
    ops.scaled_norm_add(xd, sl.to(DEV), w.to(DEV), ls.to(DEV), 0.6, 1e-6, None, b.to(DEV))
    want = x.double() + 0.6 * plain.rms_norm(sl.double().sum(0) + b.double(), w.double(), 1e-6) * ls.double()
    assert rel_err(xd.cpu(), want) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_gated_unit(ops, dtype):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(9, 2 * 52, generator=g) * 2).to(DT[dtype])
    for limit in (1.0, 2.5):
        gg, uu = gu[:, :52].double().clamp(max=limit), gu[:, 52:].double().clamp(-limit, limit)
        want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
        out = torch.empty(9, 52, dtype=DT[dtype], device=DEV)
        ops.clamped_glu(gu.to(DEV), out, limit, 1.702)
        assert rel_err(out.float().cpu(), want) < TOL[dtype]
    assert float(gu.abs().max()) > 2.5  # both limits cut something
    # gate and up columns interleaved in groups of 8 (the layout of the stacked weights in bfloat16): 56 features
    gu = (torch.randn(9, 2 * 56, generator=g) * 2).to(DT[dtype])
    gg, uu = gu[:, :56].double().clamp(max=1.5), gu[:, 56:].double().clamp(-1.5, 1.5)
    mixed = torch.stack([gu[:, :56].reshape(9, 7, 8), gu[:, 56:].reshape(9, 7, 8)], dim=2).reshape(9, 112).contiguous()
    out = torch.empty(9, 56, dtype=DT[dtype], device=DEV)
    ops.clamped_glu(mixed.to(DEV), out, 1.5, 1.702, interleave=8)
    assert rel_err(out.float().cpu(), gg * torch.sigmoid(1.702 * gg) * (uu + 1)) < TOL[dtype]


@pytest.mark.parametrize("M,K,inner", [(300, 192, 200), (128, 64, 40), (1000, 512, 1024)])
def test_clamped_unit_in_the_tensor_core_product(ops, M, K, inner):
    """The gated tcgen05 product with the clamped unit as its epilogue against the plain statement."""
    g = torch.Generator().manual_seed(M)
    a = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    wg, wu = (torch.randn(inner, K, generator=g) * 0.1).to(torch.bfloat16), (torch.randn(inner, K, generator=g) * 0.1).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops.gemm_tcgen05_clamped(a.to(DEV), ops.interleave_gate_up(wg.to(DEV), wu.to(DEV)), status, 0.9, 1.702)
    gg = (a.double() @ wg.double().T).clamp(max=0.9)
    uu = (a.double() @ wu.double().T).clamp(-0.9, 0.9)
    assert int(status.item()) == 0
    assert float(((a.double() @ wg.double().T) > 0.9).double().mean()) > 0.05  # the limit cuts something
    assert rel_err(got.float().cpu(), gg * torch.sigmoid(1.702 * gg) * (uu + 1)) < TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,groups", [(96, 1), (96, 3), (520, 2)])
def test_gated_norm_in_parts(ops, dtype, width, groups):
    g = torch.Generator().manual_seed(width + groups)
    wide = torch.randn(6, 2 * width + 5, generator=g)
    y, gate = wide[:, 3:3 + width], wide[:, width + 5:]
    w = torch.rand(width, generator=g) + 0.5
    wd = wide.to(DEV)
    yd, gd = wd[:, 3:3 + width], wd[:, width + 5:]
    out = torch.empty(6, width, dtype=DT[dtype], device=DEV)
    ops.gated_group_norm(yd, gd, w.to(DEV), out, groups, 1e-5, gate_first=True)
    v = (y.double() * plain.silu(gate.double())).reshape(6, groups, -1)
    assert rel_err(out.float().cpu(), plain.rms_norm(v, None, 1e-5).reshape(6, width) * w.double()) < TOL[dtype]
    ops.gated_group_norm(yd, gd, w.to(DEV), out, groups, 1e-5, gate_first=False)
    v = plain.rms_norm(y.double().reshape(6, groups, -1), None, 1e-5).reshape(6, width)
    assert rel_err(out.float().cpu(), v * w.double() * torch.sigmoid(gate.double())) < TOL[dtype]


def walk_defines(ops, dim, vdim):
    return ops.decay_recurrence_defines(dim, vdim)


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_convolution_step_sizes_and_carried_inputs(ops, taps):
    """Two requests side by side, fed in portions of 1, 2 and more tokens; then their slots are handed to others, zeroed
    as the cache manager zeroes them."""
    C, H, pre = 44, 3, 7  # channels, heads; the convolved columns start at column `pre` of the projections
    g = torch.Generator().manual_seed(taps)
    w, b = torch.randn(C, taps, generator=g) * 0.5, torch.randn(C, generator=g)
    dt_bias, a_log = torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.5
    lens = {0: 23, 1: 9}
    proj = {s: torch.randn(n, pre + C + H, generator=g) for s, n in lens.items()}
    proj[0][5, pre + C] = 40.0  # a step size beyond the range where exp() of it is finite in float32
    defines = walk_defines(ops, 8, 8)
    state = torch.zeros(3, 11 + (taps - 1) * C, device=DEV)
    state[:, :11] = 7.0  # what lies before the carried inputs is not this kernel's
    slots = {0: 2, 1: 0}
    for rnd in range(2):
        got = {s: [] for s in lens}
        got_dt = {s: [] for s in lens}
        at = {s: 0 for s in lens}
        portions = {0: [2, 1, 5, 1, 2, 12], 1: [1, 1, 2, 5]}
        for step in range(6):
            rows, tseq, qs, ql, sl = [], [], [], [], []
            for s in lens:
                if step < len(portions[s]):
                    n = portions[s][step]
                    qs.append(len(tseq)); ql.append(n); sl.append(slots[s])
                    rows.append(proj[s][at[s]:at[s] + n]); tseq += [len(qs) - 1] * n
            pj = torch.cat(rows).to(DEV)
            T = pj.shape[0]
            xbc, dd = torch.empty(T, C, device=DEV), torch.empty(T, 2 * H, device=DEV)
            ops.ssm_prep(pj, pre, C, w.to(DEV), b.to(DEV), state, 11, i32(tseq), i32(sl), i32(qs), i32(ql), len(qs), xbc,
                         pre + C, H, dt_bias.to(DEV), a_log.to(DEV), dd, defines)
            k = 0
            for s in lens:
                if step < len(portions[s]):
                    n = portions[s][step]
                    got[s].append(xbc[qs[k]:qs[k] + n].cpu()); got_dt[s].append(dd[qs[k]:qs[k] + n].cpu())
                    at[s] += n; k += 1
        for s, n in lens.items():
            u = proj[s].double()
            want = plain.silu(plain.causal_conv(u[:, pre:pre + C], w.double(), b.double()))
            assert rel_err(torch.cat(got[s]), want) < 1e-5, (taps, s, rnd)
            dt = plain.softplus(u[:, pre + C:] + dt_bias.double())
            want_dd = torch.cat([dt, torch.exp(-torch.exp(a_log.double()) * dt)], dim=1)
            assert rel_err(torch.cat(got_dt[s]), want_dd) < 1e-5
        assert float((state[:, :11] - 7.0).abs().max()) == 0.0
        # other requests take the slots over
        proj = {s: torch.randn(n, pre + C + H, generator=g) for s, n in lens.items()}
        slots = {0: 0, 1: 2}
        state[:, 11:] = 0.0


@pytest.mark.parametrize("heads,groups,dim,vdim", [(4, 2, 24, 40), (2, 2, 64, 16), (1, 1, 7, 130), (6, 1, 128, 64), (3, 3, 10, 300), (2, 1, 200, 36)])
def test_decay_walk_in_portions(ops, heads, groups, dim, vdim):
    """Both forms (a decay per head, silu on the inputs; decays and key scales per token with a skip term and shared
    q and k per group) over two requests in portions down to one token, against the whole sequences, with every build
    of the walk that the head size allows (8, 16, 32 threads a column)."""
    defines = walk_defines(ops, dim, vdim)
    builds = ops.decay_walk_modules(dim, vdim)
    import itertools
    chosen = itertools.cycle(builds)  # a request's steps go through different builds: the state's layout is one
    monkey = pytest.MonkeyPatch()
    monkey.setattr(ops, "_walk_defines", lambda *a: next(chosen))
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lens = {0: 70, 1: 19}
    portions = {0: [2, 33, 1, 1, 17, 16], 1: [1, 2, 16]}
    n_state = heads * dim * vdim
    for form in ("per_head", "per_token"):
        G = heads if form == "per_head" else groups
        q = {s: torch.randn(n, G * dim, generator=g) for s, n in lens.items()}
        k = {s: torch.randn(n, G * dim, generator=g) * 0.5 for s, n in lens.items()}
        v = {s: torch.randn(n, heads * vdim, generator=g) for s, n in lens.items()}
        decay = torch.rand(heads, generator=g) * 0.5 + 0.5
        decay[0] = 0.999
        dd = {s: torch.cat([torch.rand(n, heads, generator=g) * 2, torch.rand(n, heads, generator=g) * 0.4 + 0.6], dim=1)
              for s, n in lens.items()}
        skip = torch.randn(heads, generator=g)
        state = torch.zeros(4, n_state + 13, device=DEV)
        state[:, n_state:] = 5.0
        slots = {0: 3, 1: 1}
        got = {s: [] for s in lens}
        at = {s: 0 for s in lens}
        for step in range(6):
            live = [s for s in lens if step < len(portions[s])]
            ql = [portions[s][step] for s in live]
            qs = [int(x) for x in np.concatenate([[0], np.cumsum(ql)[:-1]])]
            cat = lambda d: torch.cat([d[s][at[s]:at[s] + n] for s, n in zip(live, ql)]).to(DEV)  # noqa: E731
            T = sum(ql)
            out = torch.empty(T, heads * vdim, device=DEV)
            if form == "per_head":
                # q, k and v as column slices of one tensor with something behind them, SiLU applied in place
                wide = torch.cat([cat(q), cat(k), cat(v), torch.full((T, 3), 9.0, device=DEV)], dim=1)
                ops.silu_cols(wide, wide.shape[1] - 3, defines)
                assert float((wide[:, -3:] - 9.0).abs().max()) == 0.0
                ops.decay_walk(wide[:, :G * dim], wide[:, G * dim:2 * G * dim], wide[:, 2 * G * dim:-3], 1, None, decay.to(DEV),
                               None, state, out, i32([slots[s] for s in live]), i32(qs), i32(ql), len(live), heads, dim, vdim)
            else:
                ops.decay_walk(cat(q), cat(k), cat(v), heads // groups, cat(dd), None, skip.to(DEV), state, out,
                               i32([slots[s] for s in live]), i32(qs), i32(ql), len(live), heads, dim, vdim)
            for s, a, n in zip(live, qs, ql):
                got[s].append(out[a:a + n].cpu())
                at[s] += n
        for s, n in lens.items():
            if form == "per_head":
                want = plain.decayed_linear_attention(plain.silu(q[s].double()).reshape(n, heads, dim),
                                                      plain.silu(k[s].double()).reshape(n, heads, dim),
                                                      plain.silu(v[s].double()).reshape(n, heads, vdim), decay.double())
                S = None
            else:
                # the plain scan takes raw step sizes: give it dt and A so that exp(-exp(A) dt) is the decay drawn above
                dt = dd[s][:, :heads].double()
                a_log = torch.zeros(heads, dtype=F64)
                dec = dd[s][:, heads:].double()
                want = torch.zeros(n, heads, vdim, dtype=F64)
                S = torch.zeros(heads, dim, vdim, dtype=F64)
                gi = torch.arange(heads) // (heads // groups)
                for t in range(n):
                    B, Cq = k[s][t].double().reshape(groups, dim)[gi], q[s][t].double().reshape(groups, dim)[gi]
                    x = v[s][t].double().reshape(heads, vdim)
                    S = dec[t][:, None, None] * S + dt[t][:, None, None] * B[:, :, None] * x[:, None, :]
                    want[t] = torch.einsum("hnp,hn->hp", S, Cq) + skip.double()[:, None] * x
                del a_log
            assert rel_err(torch.cat(got[s]), want.reshape(n, -1)) < 2e-5, (form, s)
            if S is not None:  # the state left in the slot: S^T per head
                left = state[slots[s], :n_state].cpu().reshape(heads, vdim, dim)
                assert rel_err(left, S.transpose(1, 2)) < 2e-5
        assert float((state[:, n_state:] - 5.0).abs().max()) == 0.0
    monkey.undo()


def paged(n_tokens, page, seed):
    """A block table of scattered pages for one request."""
    n_pages = -(-n_tokens // page)
    perm = np.random.default_rng(seed).permutation(n_pages + 5)[:n_pages]
    return [int(p) for p in perm], n_pages + 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim,page,heads,kv", [(64, 48, 16, 6, 2), (24, 40, 8, 3, 3), (20, 6, 16, 4, 1), (128, 128, 16, 2, 1), (32, 16, 16, 20, 1)])
def test_sink_attention_window_edges(ops, dtype, dim, vdim, page, heads, kv):
    """One made-up key that a probe query scores far above all others, with a value that stands out, at a page's first
    and last slot: seen from the position just inside the window and not from the one just outside, inside a portion
    and as single tokens; the cap holds the probe's score down to what the formula says; the sink takes its share."""
    window, n = 37, 150
    g = torch.Generator().manual_seed(dim + page)
    qkv_w = (heads + kv) * dim + kv * vdim
    sinks = torch.randn(heads, generator=g)
    scale, cap = 0.3, 6.0
    for far_at in (page * 3, page * 4 - 1, page * 5 + 2):
        raw = torch.randn(n, qkv_w, generator=g)
        bias = torch.randn(qkv_w, generator=g) * 0.3
        probe = torch.randn(dim, generator=g)
        rows_inside, rows_outside = far_at + window - 1, far_at + window
        for r in (rows_inside, rows_outside):
            raw[r, :heads * dim] = (probe * 3).repeat(heads) - bias[:heads * dim]
        raw[far_at, heads * dim:(heads + kv) * dim] = (probe * 3).repeat(kv) - bias[heads * dim:(heads + kv) * dim]
        raw[far_at, (heads + kv) * dim:] = 50.0
        x = raw.double() + bias.double()
        q = plain.rms_norm(x[:, :heads * dim].reshape(n, heads, dim), None, 1e-6)
        k = plain.rms_norm(x[:, heads * dim:(heads + kv) * dim].reshape(n, kv, dim), None, 1e-6)
        v = x[:, (heads + kv) * dim:].reshape(n, kv, vdim)
        want = plain.window_sink_attention(q, k, v, sinks.double(), scale, cap, window).reshape(n, heads * vdim)
        assert float(want[rows_inside].abs().max()) > 3 * float(want[rows_outside].abs().max())
        table, n_pages = paged(n, page, far_at)
        for cut in ([n], [rows_inside - 3, 5, n - rows_inside - 2], [rows_inside] + [1] * (n - rows_inside)):
            cache = torch.full((n_pages, kv, page, dim + vdim), float("nan"), dtype=DT[dtype], device=DEV)
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            got, at = [], 0
            for m in cut:
                pos = list(range(at, at + m))
                qd = torch.empty(m, heads * dim, dtype=DT[dtype], device=DEV)
                need = -(-(at + m) // page)
                ops.sink_attn_prep(raw[at:at + m].to(DEV), bias.to(DEV), True, 1e-6, qd, cache, i32(pos), i32([0] * m),
                                   i32([0, need]), i32(table[:need]), heads, kv, dim, vdim, page, True, status)
                out = torch.empty(m, heads * vdim, dtype=DT[dtype], device=DEV)
                ops.attn_sink(qd, out, cache, i32([0] * m), i32(pos), i32([0, need]), i32(table[:need]), None, m,
                              sinks.to(DEV), heads, kv, dim, vdim, page, scale, cap, window, status)
                got.append(out.float().cpu())
                if ops.can_use_attn_sink_tc(DT[dtype], dim, vdim):
                    # the same on the tensor cores: as a portion and, if it is one token, as a single token; beside a
                    # second request of one token (the first request's first token once more, from its own page)
                    out2 = torch.full((m + 1, heads * vdim), float("nan"), dtype=DT[dtype], device=DEV)
                    q2 = torch.cat([qd, qd[:1] if at == 0 else q_first])
                    if at == 0:
                        q_first = qd[:1].clone()
                    ops.attn_sink_tc(q2, out2, cache, i32([0, m]), i32([m, 1]), i32([at + m, 1]), i32([0, need, need + 1]),
                                     i32(table[:need] + table[:1]), 2, sinks.to(DEV), heads, kv, dim, vdim, page, scale, cap,
                                     window, status, portions=m > 1)
                    assert rel_err(out2[:m].float().cpu(), want[at:at + m]) < 3e-2, ("tensor cores", far_at, cut[:2], at)
                    assert rel_err(out2[m:].float().cpu(), want[:1]) < 3e-2
                at += m
            got = torch.cat(got)
            assert int(status.item()) == 0
            assert rel_err(got, want) < (3e-5 if dtype == "float32" else 3e-2), (far_at, cut[:2])
    # without a cap, without a sink, without a window, without the unit norm
    raw = torch.randn(40, qkv_w, generator=g)
    q, k = raw[:, :heads * dim].double().reshape(40, heads, dim), raw[:, heads * dim:(heads + kv) * dim].double().reshape(40, kv, dim)
    v = raw[:, (heads + kv) * dim:].double().reshape(40, kv, vdim)
    want = plain.window_sink_attention(q, k, v, torch.full((heads,), -1e30, dtype=F64), scale / dim ** 0.5, None, None)
    table, n_pages = paged(40, page, 1)
    cache = torch.zeros((n_pages, kv, page, dim + vdim), dtype=DT[dtype], device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    qd = torch.empty(40, heads * dim, dtype=DT[dtype], device=DEV)
    pos, need = list(range(40)), -(-40 // page)
    ops.sink_attn_prep(raw.to(DEV), None, False, 1e-6, qd, cache, i32(pos), i32([0] * 40), i32([0, need]), i32(table), heads,
                       kv, dim, vdim, page, True, status)
    rows = [39, 0, 17]
    out = torch.empty(3, heads * vdim, dtype=DT[dtype], device=DEV)
    ops.attn_sink(qd, out, cache, i32([0] * 40), i32(pos), i32([0, need]), i32(table), i32(rows), 3, None, heads, kv, dim,
                  vdim, page, scale / dim ** 0.5, None, None, status)
    assert rel_err(out.float().cpu(), want.reshape(40, -1)[rows]) < (3e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("window", [None, 130])
def test_sink_attention_single_tokens_over_several_blocks(ops, window):
    """Three requests that bring one token each at contexts of 300, 70 and 1: with so few requests a request's keys are
    shared out among several blocks (one of them gets the sink, some get no keys at all) and put together afterwards."""
    dim, vdim, heads, kv, page = 32, 48, 6, 2, 16
    g = torch.Generator().manual_seed(9)
    sinks = torch.randn(heads, generator=g) + 1
    lens = [300, 70, 1]
    qkv_w = (heads + kv) * dim + kv * vdim
    n_pages = sum(-(-n // page) for n in lens)
    cache = torch.full((n_pages, kv, page, dim + vdim), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    perm = [int(x) for x in np.random.default_rng(3).permutation(n_pages)]
    tables, want, last_q = [], [], []
    for n in lens:
        raw = torch.randn(n, qkv_w, generator=g)
        table, perm = perm[:-(-n // page)], perm[-(-n // page):]
        tables.append(table)
        qd = torch.empty(n, heads * dim, dtype=torch.bfloat16, device=DEV)
        ops.sink_attn_prep(raw.to(DEV), None, True, 1e-6, qd, cache, i32(list(range(n))), i32([0] * n), i32([0, len(table)]),
                           i32(table), heads, kv, dim, vdim, page, True, status)
        last_q.append(qd[-1:])
        x = raw.double()
        q = plain.rms_norm(x[:, :heads * dim].reshape(n, heads, dim), None, 1e-6)
        k = plain.rms_norm(x[:, heads * dim:(heads + kv) * dim].reshape(n, kv, dim), None, 1e-6)
        v = x[:, (heads + kv) * dim:].reshape(n, kv, vdim)
        want.append(plain.window_sink_attention(q, k, v, sinks.double(), 0.35, 20.0, window).reshape(n, -1)[-1])
    indptr = [0] + [int(x) for x in np.cumsum([len(t) for t in tables])]
    out = torch.full((3, heads * vdim), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attn_sink_tc(torch.cat(last_q), out, cache, i32([0, 1, 2]), i32([1, 1, 1]), i32(lens), i32(indptr),
                     i32(sum(tables, [])), 3, sinks.to(DEV), heads, kv, dim, vdim, page, 0.35, 20.0, window, status, portions=False)
    assert int(status.item()) == 0
    assert rel_err(out.float().cpu(), torch.stack(want)) < 3e-2


# ------------------------------------------------------------------------------------------------ whole models
def ssm(heads, vdim, state, groups, norm_groups, conv):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv))


def lin(heads, dim, vdim, decay):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay))


def att(heads, kv_heads, dim, vdim, window, scale, softcap):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=window),
                                             scale=scale, softcap=softcap))


def ff(inner, limit):
    return dict(kind="dense", ff=inner, limit=limit)


def shared(layer, j):
    return dict(copy.deepcopy(layer), weights_of=j)


A0, A1, A2 = dict(att(6, 3, 24, 40, 23, 0.4, 8.0), mlp=ff(72, 1.5)), dict(ssm(4, 24, 20, 2, 3, 3), mlp=None), \
    dict(lin(3, 16, 40, [0.7, 0.95, 0.999]), mlp=ff(56, 0.8))
B0, B1, B2 = dict(ssm(3, 20, 48, 1, 1, 5), mlp=ff(80, 1.0)), dict(lin(2, 40, 12, [0.5, 0.99]), mlp=None), \
    dict(att(4, 4, 16, 8, 200, 0.25, 30.0), mlp=ff(48, 2.0))
C0, C1, C2 = dict(lin(5, 8, 24, [0.999, 0.9, 0.8, 0.6, 0.3]), mlp=ff(96, 1.0)), dict(att(8, 1, 32, 16, 16, 0.18, 3.0), mlp=ff(64, 1.0)), \
    dict(ssm(6, 16, 16, 3, 2, 2), mlp=ff(40, 3.0))

D0, D1 = dict(lin(2, 24, 24, [0.9, 0.97]), mlp=ff(64, 1.0)), dict(ssm(2, 40, 24, 2, 1, 4), mlp=ff(32, 1.2))
E0, E1, E2 = dict(att(4, 2, 16, 16, 40, 0.3, 10.0), mlp=ff(48, 1.0)), dict(att(2, 2, 32, 8, 9, 0.2, 25.0), mlp=None), \
    dict(att(3, 1, 16, 32, 70, 0.25, 15.0), mlp=ff(40, 1.0))

MODELS = {
    # no attention at all: no pages, only slots
    "d": dict(page=16, lengths=[90, 20, 47, 3, 61],
              config=dict(architecture="Daborax", vocab=89, width=80, norm=dict(eps=1e-6), embedding=dict(scale=4.0),
                          residual_mult=0.8, layers=[D0, D1, shared(D0, 0)])),
    # only attention, of three shapes and windows: three cache groups, no slots' state
    "e": dict(page=8, lengths=[120, 33, 75, 9, 50],
              config=dict(architecture="Daborax", vocab=101, width=64, norm=dict(eps=1e-5), embedding=dict(scale=2.0),
                          residual_mult=0.9, layers=[E0, E1, E2, shared(E1, 1)])),
    # attention first with a window that is no multiple of the page size, a layer without a feed-forward, both kinds
    # of state, two layers that run with earlier layers' tensors
    "a": dict(page=8, lengths=[100, 37, 64, 5, 81, 1, 50],
              config=dict(architecture="Daborax", vocab=151, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.5),
                          residual_mult=0.6, layers=[A0, A1, A2, shared(A1, 1), shared(A0, 0)])),
    # a state space first: one group, one norm group, five taps; as many key/value heads as heads; a window longer than
    # most requests; multiplier 1 and embedding scale 1
    "b": dict(page=16, lengths=[130, 70, 33, 16, 97],
              config=dict(architecture="Daborax", vocab=97, width=64, norm=dict(eps=1e-6), embedding=dict(scale=1.0),
                          residual_mult=1.0, layers=[B0, B1, B2, shared(B2, 2)])),
    # a window of exactly one page, one key/value head for eight heads, a low cap, the same layer three times over
    "c": dict(page=16, lengths=[300, 150, 40, 210, 33, 64],
              config=dict(architecture="Daborax", vocab=113, width=128, norm=dict(eps=1e-6), embedding=dict(scale=9.0),
                          residual_mult=0.5, layers=[C0, C1, C2, shared(C0, 0), shared(C1, 1), shared(C0, 0)])),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from safetensors import safe_open
    from safetensors.torch import save_file
    from tokasaurus_b200.weights import write_model_folder

    root = tmp_path_factory.mktemp("daborax_models")
    out = {}
    for name, spec in MODELS.items():
        folder = write_model_folder(root / name, spec["config"], seed=23 + len(out), std=0.12, norm_init="uniform")
        w = {}
        with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
            for k in f.keys():
                w[k] = f.get_tensor(k)
        g = torch.Generator().manual_seed(5)
        for k in w:  # vectors that are no norm weights: signs and sizes of their own
            tail = k.split(".mix.")[-1] if ".mix." in k else ""
            if tail in ("q.b", "k.b", "v.b", "o.b", "conv.b", "D", "dt_bias"):
                w[k] = (torch.randn(w[k].shape, generator=g) * 0.5).to(w[k].dtype)
            elif tail == "sink":
                w[k] = (torch.randn(w[k].shape, generator=g) * 2 + 1).to(w[k].dtype)
            elif tail == "conv":
                w[k] = (torch.randn(w[k].shape, generator=g) * 0.6).to(w[k].dtype)
            elif tail == "A_log":
                w[k] = (torch.rand(w[k].shape, generator=g) * 3 - 3).to(w[k].dtype)  # decays from a few tokens to hundreds
            elif k.endswith(".ls1") or k.endswith(".ls2"):
                w[k] = (torch.randn(w[k].shape, generator=g) * 0.5).to(w[k].dtype)
        save_file(w, str(folder / "model.safetensors"))
        V = spec["config"]["vocab"]
        reqs = {f"{name}{i}": cuttings.random_tokens(n, V, 40 + i) for i, n in enumerate(spec["lengths"])}
        w64 = {k: v.to(F64) for k, v in w.items()}
        want = {rid: plain.forward(spec["config"], w64, t).numpy() for rid, t in reqs.items()}
        out[name] = dict(folder=folder, config=spec["config"], weights=w64, reqs=reqs, want=want, page=spec["page"])
    return out


def windows_of(config):
    return sorted({l["mixer"]["mask"]["size"] for l in config["layers"] if l["type"] == "attention"})


def pool_tokens(steps, config, page):
    """Tokens of page pool a trace needs when pages behind a window come back after every step (the largest need over
    the model's windows: every windowed group gets a pool of this size)."""
    peak = 0
    for window in windows_of(config):
        held = {}
        for st in steps:
            during = 0
            names = {e["id"] for e in st["entries"]}
            for e in st["entries"]:
                before = held.get(e["id"], 0)
                after = before + len(e["tokens"])
                during += -(-after // page) - max(0, before - window + 1) // page
                held[e["id"]] = after
            idle = sum(-(-n // page) - max(0, n - window + 1) // page for rid, n in held.items() if rid not in names)
            peak = max(peak, during + idle)
            for rid in st["end"]:
                held.pop(rid, None)
    return peak * page


def check_logits(got, m, dtype, what):
    """Every position within 3e-5 (float32) or 4e-2 (bfloat16) of the logits' scale, mean over the vocabulary taken off."""
    for rid, ref in m["want"].items():
        scale = float(np.sqrt((ref ** 2).mean()))
        tol = (3e-5 if dtype == "float32" else 4e-2) * scale
        d = got[rid] - ref
        err = np.sqrt(((d - d.mean(axis=1, keepdims=True)) ** 2).mean(axis=1))
        bad = np.nonzero(err > tol)[0]
        assert bad.size == 0, (f"{dtype} {what}: request {rid}: first wrong token at position {bad[0]} "
                               f"(error {err[bad[0]]:.3g}, tolerance {tol:.3g}); {bad.size} of {len(err)} over it")


CUTS = dict(whole=cuttings.whole, prefix_then_single=cuttings.prefix_then_single,
            changing_portions=cuttings.changing_portions, mixed=cuttings.mixed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("which", list(MODELS))
def test_cuttings_match_plain(models, which, cut, dtype):
    """Whole prompts, prompts then single tokens, portions of changing size down to one and two tokens, and up to four
    requests side by side in four slots, in a pool that holds exactly what the trace needs: pages and slots are used
    again, and a later request must see nothing of an earlier one's state."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    m = models[which]
    steps = CUTS[cut](m["reqs"])
    rp = TraceReplayer(str(m["folder"]), dtype, pool_tokens(steps, m["config"], m["page"]), page_size=m["page"], max_requests=4)
    cache = rp.runner.cache
    owners, slots, outs = {}, {}, []
    for st in steps:
        outs.append(rp.run_step(st))
        cache.check()
        for rid, rc in cache.requests.items():
            slots.setdefault(rc.slot, set()).add(rid)
            for gi in range(len(cache.groups)):
                for p in rc.live_pages(gi):
                    owners.setdefault((gi, p), set()).add(rid)
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]
    check_logits(cuttings.collect(steps, outs), m, dtype, cut)
    if cut == "mixed":
        assert not cache.groups or any(len(v) > 1 for v in owners.values()), "no page was used by two requests"
        assert any(len(v) > 1 for v in slots.values()), "no slot was used by two requests"


def test_layer_by_layer(models):
    """The residual stream after every layer call, float32, one prompt in one step."""
    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.trace import TraceReplayer

    for which, m in models.items():
        rid, toks = next(iter(m["reqs"].items()))
        want = []
        plain.forward(m["config"], m["weights"], toks, want)
        rp = TraceReplayer(str(m["folder"]), "float32", 512, page_size=m["page"], max_requests=2)
        rp.runner.cache.admit(rid)
        rp.runner.cache.ensure_capacity(rid, len(toks))
        got = []
        rp.runner.step([StepEntry(rid, toks, 0, list(range(len(toks))))], layer_outputs=got)
        assert len(got) == len(want)
        for i, (a, b) in enumerate(zip(got, want)):
            assert rel_err(a.cpu(), b) < 1e-4, (which, i)  # float32 sums of up to a few hundred terms a value


def test_edges_and_state_show_in_the_logits(models):
    """The comparisons above would not notice a window off by one, a lost tap, a left-out sink, another decay or a cap
    that is not applied if those carried no weight: on the plain implementation, changing each moves the logits by
    hundreds of times the tolerance of the float32 comparisons."""
    m = models["a"]
    rid, toks = max(m["reqs"].items(), key=lambda kv: len(kv[1]))
    ref = m["want"][rid]
    tol = 1e-3 * float(np.sqrt((ref ** 2).mean()))

    def moved(config, weights=None):
        d = plain.forward(config, weights or m["weights"], toks).numpy() - ref
        return float(np.sqrt((d ** 2).mean(axis=1)).max())

    for key, change in (("mask", lambda mx: mx["mask"].update(size=mx["mask"]["size"] + 1)),
                        ("softcap", lambda mx: mx.update(softcap=None)),
                        ("decay", lambda mx: mx.update(decay=[d * 0.98 for d in mx["decay"]])),
                        ("norm_groups", lambda mx: mx.update(norm_groups=1))):
        cfg = copy.deepcopy(m["config"])
        for l in cfg["layers"]:
            if key in l["mixer"]:
                change(l["mixer"])
        assert moved(cfg) > 3 * tol, key
    for name, f in (("l1.mix.conv", lambda t: t.index_fill(1, torch.tensor([0]), 0.0)),   # the oldest tap
                    ("l0.mix.sink", lambda t: t - 30.0),                                  # a sink that counts for nothing
                    ("l1.mix.dt_bias", lambda t: t + 0.3), ("l1.mix.D", lambda t: t * 0), ("l0.mix.k.b", lambda t: t * 0),
                    ("l0.ls1", lambda t: t * 1.1)):
        w = dict(m["weights"])
        w[name] = f(w[name].clone())
        assert moved(m["config"], w) > 3 * tol, name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_windows(models, dtype):
    """A short prompt, then 150 tokens one by one: every window passes over decoded tokens several times, pages come
    back behind it, and the states are carried 150 steps."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    for which in ("a", "c", "d", "e"):
        m = models[which]
        toks = cuttings.random_tokens(160, m["config"]["vocab"], 7)
        want = plain.forward(m["config"], m["weights"], toks).numpy()
        steps = cuttings.prefix_then_single({"long": toks}, tail=150)
        rp = TraceReplayer(str(m["folder"]), dtype, pool_tokens(steps, m["config"], m["page"]), page_size=m["page"], max_requests=4)
        got = cuttings.collect(steps, [rp.run_step(st) for st in steps])
        check_logits(got, dict(want={"long": want}), dtype, "long decoding")


def plain_greedy(m, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        out.append(int(plain.forward(m["config"], m["weights"], ids)[-1].argmax()))
        ids.append(out[-1])
    return out


@pytest.mark.parametrize("which", ["a", "d", "e"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(models, graphs, which):
    """Greedy generation in float32 through ``Engine.generate``: the scheduler admits, cuts prompts into portions,
    decodes (from CUDA graphs or kernel by kernel) and frees; five requests in three slots, so slots are handed on.
    Also for a model without any pages and for one without any state."""
    from tokasaurus_b200.engine.engine import Engine

    m = models[which]
    V = m["config"]["vocab"]
    prompts = [cuttings.random_tokens(n, V, 300 + n) for n in (30, 3, 41, 17, 9)]
    n_new = 10
    want = [plain_greedy(m, p, n_new) for p in prompts]
    eng = Engine(model=str(m["folder"]), dtype="float32", page_size=m["page"], kv_cache_num_tokens=512,
                 max_tokens_per_forward=24, max_seqs_per_forward=3, allocator_sanity_checks=True, use_cudagraphs=graphs)
    outs = eng.generate(prompts, max_num_tokens=n_new, ignore_eos=True)
    assert [o.completion_ids for o in outs] == want
    cache = eng.runner.cache
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]


def test_command_line_generates(models, tmp_path):
    """``toka model=<folder>`` picks the model class from config.json and generates."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    m = models["b"]
    prompt = cuttings.random_tokens(12, m["config"]["vocab"], 1)
    toka = Path(__file__).resolve().parent.parent / "bin" / "toka"
    r = subprocess.run([sys.executable, str(toka), f"model={m['folder']}", "dtype=float32", "page_size=16",
                        "kv_cache_num_tokens=256", "max_num_tokens=6", "ignore_eos=T", f"prompt_ids={json.dumps(prompt)}"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = plain_greedy(m, prompt, 6)
    assert json.loads(r.stdout.strip().splitlines()[-1])["completion_ids"] == want
