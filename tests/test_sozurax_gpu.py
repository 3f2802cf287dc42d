"""The Sozurax decoder on the GPU against the plain implementation in ``plain_sozurax`` (float64, whole sequences,
no cache): every mechanism's kernels alone, then small random models of several shapes through trace replay in four
cuttings and both precisions with pools that hold exactly what a trace needs, then greedy generation through the
engine's entry point and scheduler.  Sizes are chosen so that nothing that could be confused is equal: key and
value sizes of a head, latent ranks of queries and keys, rotated and rotary sizes, windows that are no multiple of
the page size, one and several chosen experts, layers without a feed-forward."""

import numpy as np
import pytest
import torch

import cuttings
import plain_sozurax as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def rel_err(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


@pytest.fixture(scope="module")
def ops():
    from tokasaurus_b200.kernels import ops as o
    return o


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [40, 321, 1024])
def test_layer_norm_with_residual_add(ops, dtype, H):
    g = torch.Generator().manual_seed(H)
    x = torch.randn(7, H, generator=g) * 3 + 1.5
    d = (torch.randn(7, H, generator=g)).to(DT[dtype])
    w, b = torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g)
    want_x = x.double() + d.double()
    want = plain.layer_norm(want_x, w.double(), b.double(), 1e-5)
    xd, out = x.to(DEV), torch.empty(7, H, dtype=DT[dtype], device=DEV)
    ops.add_layernorm(xd, d.to(DEV), w.to(DEV), b.to(DEV), 1e-5, out)
    assert rel_err(xd.cpu(), want_x) < 1e-6
    assert rel_err(out.float().cpu(), want) < TOL[dtype]
    # float32 slices of a split product instead
    sl = torch.randn(3, 7, H, generator=g)
    xd = x.to(DEV)
    ops.add_layernorm(xd, sl.to(DEV), w.to(DEV), b.to(DEV), 1e-5, out)
    assert rel_err(out.float().cpu(), plain.layer_norm(x.double() + sl.double().sum(0), w.double(), b.double(), 1e-5)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_short_conv_in_portions_and_slots(ops, dtype, taps):
    """Two requests fed in portions of unequal sizes (one, two and more tokens), side by side, in slots 2 and 0 of
    4; then another request in a slot that was used before and zeroed."""
    H = 72
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(H, taps, generator=g)
    seqs = [torch.randn(n, H, generator=g).to(DT[dtype]) for n in (19, 11)]
    want = [plain.input_conv(s.double(), w.double()) for s in seqs]
    carry = torch.zeros(4, taps - 1, H, device=DEV)
    carry[1] = 7.0  # another request's slot: must stay as it is
    slots = [2, 0]
    cuts = [[3, 1, 2, 1, 1, 6, 5], [1, 1, 4, 2, 3]]
    at = [0, 0]
    got = [[], []]
    step = 0
    while any(a < len(s) for a, s in zip(at, seqs)):
        rows, tseq, start, qlen, slot, who = [], [], [], [], [], []
        for r in (0, 1):
            if at[r] < len(seqs[r]) and step < len(cuts[r]):
                n = cuts[r][step]
                start.append(len(rows))
                rows += [seqs[r][at[r] + k] for k in range(n)]
                tseq += [len(who)] * n
                qlen.append(n)
                slot.append(slots[r])
                who.append((r, n))
                at[r] += n
        step += 1
        h = torch.stack(rows).to(DEV)
        out = torch.empty_like(h)
        ops.short_conv(h, out, w.to(DEV), carry, i32(tseq), i32(slot), i32(start), i32(qlen), len(who))
        o = out.float().cpu()
        for (r, n), s0 in zip(who, start):
            got[r].append(o[s0:s0 + n])
    for r in (0, 1):
        assert rel_err(torch.cat(got[r]), want[r]) < TOL[dtype]
    assert bool((carry[1] == 7.0).all())
    carry[2].zero_()  # what the cache manager does when it hands the slot to a new request
    h = seqs[1][:5].to(DEV)
    out = torch.empty_like(h)
    ops.short_conv(h, out, w.to(DEV), carry, i32([0] * 5), i32([2]), i32([0]), i32([5]), 1)
    assert rel_err(out.float().cpu(), want[1][:5]) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_norm_and_conv_in_one_kernel(ops, dtype):
    """Steps of single tokens: the fused kernel against norm then convolution, token after token, with padding rows."""
    H, taps, B = 96, 4, 3
    g = torch.Generator().manual_seed(3)
    w, b, cw = torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g), torch.randn(H, taps, generator=g)
    xs = torch.randn(6, B, H, generator=g) * 2
    carry = torch.zeros(5, taps - 1, H, device=DEV)
    slot = i32([4, 1, 3])
    normed = plain.layer_norm(xs.double(), w.double(), b.double(), 1e-6)
    if dtype == "bfloat16":
        normed = normed.to(torch.bfloat16).double()
    want = torch.stack([plain.input_conv(normed[:, r], cw.double()) for r in range(B)], dim=1)
    for t in range(6):
        x = torch.cat([xs[t], torch.zeros(1, H)]).to(DEV)  # one padding row
        out = torch.full((B + 1, H), 99.0, dtype=DT[dtype], device=DEV)
        ops.add_layernorm_conv1(x, None, w.to(DEV), b.to(DEV), 1e-6, cw.to(DEV), carry, i32([0, 1, 2, -1]), slot, out)
        assert rel_err(out[:B].float().cpu(), want[t]) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("F", [56, 640])
def test_polynorm(ops, dtype, F):
    g = torch.Generator().manual_seed(F)
    z = torch.randn(5, F, generator=g) * 1.7
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    out = torch.empty(5, F, dtype=DT[dtype], device=DEV)
    ops.polynorm(z.to(DEV), coef.to(DEV), 1e-6, out)
    assert rel_err(out.float().cpu(), plain.polynorm(z.double(), coef.double(), 1e-6)) < TOL[dtype]


def plain_recurrence(q_raw, f_raw, v, fb, low, nw, heads, dim, vdim, eps):
    T = q_raw.shape[0]
    q = plain.silu(q_raw).view(T, heads, dim)
    f = (low + (1 - low) * torch.sigmoid(f_raw + fb)).view(T, heads, dim)
    v = v.view(T, heads, vdim)
    S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    out = torch.zeros(T, heads, vdim, dtype=torch.float64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return plain.rms_norm(out, nw, eps).reshape(T, heads * vdim), S


@pytest.mark.parametrize("heads,dim,vdim", [(3, 24, 40), (2, 64, 16), (1, 7, 130), (2, 128, 128)])
def test_gated_recurrence_in_portions(ops, heads, dim, vdim):
    """A request's recurrence in portions (17 tokens, then one, two, ... tokens) beside a second request that starts
    later, against the recurrence over the whole sequences; the state that is left is S transposed."""
    g = torch.Generator().manual_seed(dim)
    T = [45, 23]
    C = heads * (2 * dim + vdim)
    raw = [torch.randn(t, C, generator=g) for t in T]
    fb, low = torch.randn(heads * dim, generator=g), torch.rand(heads * dim, generator=g) * 0.9
    nw = torch.rand(vdim, generator=g) + 0.5
    want = []
    for r in raw:
        d = r.double()
        want.append(plain_recurrence(d[:, :heads * dim], d[:, heads * dim:2 * heads * dim], d[:, 2 * heads * dim:], fb.double(),
                                     low.double(), nw.double(), heads, dim, vdim, 1e-6))
    state = torch.zeros(3, heads, vdim, dim, device=DEV)
    slots = [2, 0]
    portions = [[17, 1, 2, 1, 20, 4], [0, 0, 3, 1, 16, 3]]
    at, got = [0, 0], [[], []]
    for step in range(6):
        rows, start, qlen, slot, who = [], [], [], [], []
        for r in (0, 1):
            n = portions[r][step]
            if n:
                start.append(sum(x.shape[0] for x in rows))
                rows.append(raw[r][at[r]:at[r] + n])
                qlen.append(n)
                slot.append(slots[r])
                who.append((r, n))
                at[r] += n
        qfv = torch.cat(rows).to(DEV)
        out = torch.empty(qfv.shape[0], heads * vdim, device=DEV)
        ops.gated_recurrence(qfv, state, fb.to(DEV), low.to(DEV), nw.to(DEV), out, i32(slot), i32(start), i32(qlen),
                             len(who), heads, dim, vdim, 1e-6)
        o = out.cpu()
        for (r, n), s0 in zip(who, start):
            got[r].append(o[s0:s0 + n])
    for r in (0, 1):
        assert rel_err(torch.cat(got[r]), want[r][0]) < 3e-5
        assert rel_err(state[slots[r]].cpu().transpose(1, 2), want[r][1]) < 3e-5
    assert bool((state[1] == 0).all())


def latent_reference(q_abs, q_rot, rows, p, window, scale):
    """One query at position p over cached rows [n, rank + rot] (float64)."""
    R = q_abs.shape[-1]
    lo = max(0, p - window + 1) if window else 0
    keys = rows[lo:p + 1]
    s = (keys[:, :R] @ q_abs.T + keys[:, R:] @ q_rot.T) * scale  # [n, heads]
    w = torch.softmax(s, dim=0)
    return w.T @ keys[:, :R]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot,page", [(40, 8, 8), (36, 6, 16), (128, 16, 16)])
def test_latent_attention_window_edges(ops, dtype, rank, rot, page):
    """One request of 150 cached rows in scattered pages.  One row far back gets a key that a probe query scores far
    above all others: queries for which it is the oldest visible row must return (nearly) that row, queries one
    position later must not see it.  Checked for queries inside a portion and for single tokens, with the far row at
    a page's first and last slot."""
    heads, window, n, scale = 3, 37, 150, 0.3
    g = torch.Generator().manual_seed(rank)
    rows = (torch.randn(n, rank + rot, generator=g) * 0.5).to(DT[dtype])
    probe = torch.randn(rank + rot, generator=g)
    probe = probe / probe.norm()
    n_pages = 24
    perm = torch.randperm(n_pages, generator=g)[: -(-n // page)].tolist()
    for far in (page * 3, page * 4 - 1, 77):
        r = rows.clone()
        r[far] = (probe * 6).to(DT[dtype])
        cache = torch.zeros(n_pages, 1, page, rank + rot, dtype=DT[dtype], device=DEV)
        for j in range(n):
            cache[perm[j // page], 0, j % page] = r[j].to(DEV)
        r64 = r.double()
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        # a portion of queries at positions far + window - 3 .. far + window + 2, then the same as single tokens
        pos = list(range(far + window - 3, min(n, far + window + 3)))
        q = torch.randn(len(pos), heads, rank + rot, generator=g) * 0.3 + probe * 8
        q = q.to(DT[dtype])
        for single in (False, True):
            T = len(pos)
            out = torch.empty(T, heads, rank, dtype=DT[dtype], device=DEV)
            qd = q.to(DEV)
            if single:  # every query a request of its own that shares the pages (tables repeat)
                tseq, indptr = list(range(T)), [k * len(perm) for k in range(T + 1)]
                ids = perm * T
            else:
                tseq, indptr, ids = [0] * T, [0, len(perm)], perm
            ops.latent_attn(qd[:, :, :rank], qd[:, :, rank:], out, cache, i32(tseq), i32(pos), i32(indptr), i32(ids), None, T,
                            page, scale, window, status)
            assert int(status.item()) == 0
            o = out.float().cpu().double()
            for k, p in enumerate(pos):
                want = latent_reference(q[k, :, :rank].double(), q[k, :, rank:].double(), r64, p, window, scale)
                assert rel_err(o[k], want) < TOL[dtype], (far, p, single)
                sees = p - far < window
                near_far = float((o[k] - r64[far, :rank]).abs().max()) < 0.05 * float(r64[far, :rank].abs().max())
                assert near_far == sees, (far, p, single, sees)


@pytest.mark.parametrize("rank,rot,page,heads", [(40, 8, 8, 3), (128, 16, 16, 6), (176, 16, 16, 20)])
def test_latent_attention_window_edges_on_the_tensor_cores(ops, rank, rot, page, heads):
    """The same made-up far row through the tensor-core kernels as the latent mixer calls them in bfloat16: the cached
    rows as keys and as values of one shared head, single tokens through the split-key kernel and a portion through
    the tiled kernel, rows of 48, 144 and 192 values, 20 query heads on the one row."""
    from types import SimpleNamespace
    from tokasaurus_b200.parts.attention import plan_attention

    window, n, scale, Dk = 37, 150, 0.3, rank + rot
    g = torch.Generator().manual_seed(rank + 1)
    probe = torch.randn(Dk, generator=g)
    probe = probe / probe.norm()
    n_pages = 24
    perm = torch.randperm(n_pages, generator=g)[: -(-n // page)].tolist()
    for far in (page * 3, page * 4 - 1, 77):
        r = (torch.randn(n, Dk, generator=g) * 0.5).to(torch.bfloat16)
        r[far] = (probe * 6).to(torch.bfloat16)
        cache = torch.zeros(n_pages, 1, page, Dk, dtype=torch.bfloat16, device=DEV)
        for j in range(n):
            cache[perm[j // page], 0, j % page] = r[j].to(DEV)
        r64 = r.double()
        pos = list(range(far + window - 3, min(n, far + window + 3)))
        T = len(pos)
        q = (torch.randn(T, heads, Dk, generator=g) * 0.3 + probe * 8).to(torch.bfloat16)
        q2 = q.view(T, heads * Dk).to(DEV)
        for single in (False, True):
            if single:
                lens_q, lens_kv = [1] * T, [p + 1 for p in pos]
                indptr, ids = [k * len(perm) for k in range(T + 1)], perm * T
            else:
                lens_q, lens_kv, indptr, ids = [T], [pos[-1] + 1], [0, len(perm)], perm
            host = SimpleNamespace(seq_q_len=np.asarray(lens_q, dtype=np.int32), seq_kv_len=np.asarray(lens_kv, dtype=np.int32))
            plan = plan_attention(host, window, blocks_per_item=(heads + 15) // 16, query_tile=64)
            c = i32(plan["counts"])
            n_items, n_dec, n_tiles = (int(x) for x in plan["counts"][:3])
            out = torch.zeros(T, heads * Dk, dtype=torch.bfloat16, device=DEV)
            q_start = list(range(T)) if single else [0]
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            if single:
                assert n_dec == T and n_tiles == 0
                ops.attn_decode_mma(q2, cache, cache, i32(q_start), i32(lens_kv), i32(indptr), i32(ids), i32(plan["items"]),
                                    c[0:1], n_items, i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], n_dec, out,
                                    heads, 1, Dk, page, scale, window, item_entry=i32(plan["item_entry"]), status=status)
            else:
                assert n_tiles >= 1 and n_dec == 0
                ops.attn_prefill_mma(q2, out, cache, cache, i32(q_start), i32(lens_q), i32(lens_kv), i32(indptr), i32(ids),
                                     i32(plan["tiles"]), c[2:3], n_tiles, heads, 1, Dk, page, scale, window, status)
            assert int(status.item()) == 0
            o = out.view(T, heads, Dk)[:, :, :rank].float().cpu().double()
            for k, p in enumerate(pos):
                want = latent_reference(q[k, :, :rank].double(), q[k, :, rank:].double(), r64, p, window, scale)
                assert rel_err(o[k], want) < TOL["bfloat16"], (far, p, single)
                sees = p - far < window
                near_far = float((o[k] - r64[far, :rank]).abs().max()) < 0.05 * float(r64[far, :rank].abs().max())
                assert near_far == sees, (far, p, single, sees)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_rows_are_normed_rotated_and_paged(ops, dtype):
    """latent_prep + rotate_pairs against the plain norm and interleaved rotation, tokens of two requests at
    positions that straddle pages; only the first rot_dims values of the rotated part turn."""
    rank, rot, rot_dims, q_rank, page, base = 24, 10, 6, 20, 4, 5000.0
    g = torch.Generator().manual_seed(5)
    pos = [0, 1, 2, 3, 4, 30, 31, 32]
    tseq = [0, 0, 0, 0, 0, 1, 1, 1]
    T = len(pos)
    proj = torch.randn(T, q_rank + rank + rot, generator=g)
    qw, kw = torch.rand(q_rank, generator=g) + 0.5, torch.rand(rank, generator=g) + 0.5
    inv = (base ** (-2.0 * torch.arange(rot_dims // 2, dtype=torch.float64) / rot_dims)).float()
    cache = torch.zeros(12, 1, page, rank + rot, dtype=DT[dtype], device=DEV)
    cq = torch.empty(T, q_rank, dtype=DT[dtype], device=DEV)
    tables = [[5, 2], [-1] * 7 + [9, 0]]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.latent_prep(proj.to(DEV), 0, q_rank, qw.to(DEV), cq, q_rank, rank, rot, rot_dims, kw.to(DEV), inv.to(DEV), cache,
                    i32(pos), i32(tseq), i32([0, 2, 11]), i32(tables[0] + tables[1]), page, 1e-6, status, DT[dtype])
    assert int(status.item()) == 0
    d = proj.double()
    assert rel_err(cq.float().cpu(), plain.rms_norm(d[:, :q_rank], qw.double(), 1e-6)) < TOL[dtype]
    c = plain.rms_norm(d[:, q_rank:q_rank + rank], kw.double(), 1e-6)
    kr = plain.rotate_interleaved(d[:, q_rank + rank:], torch.tensor(pos), base, rot_dims)
    for t in range(T):
        row = cache[tables[tseq[t]][pos[t] // page], 0, pos[t] % page].float().cpu()
        assert rel_err(row[:rank], c[t]) < TOL[dtype]
        assert rel_err(row[rank:], kr[t]) < TOL[dtype]
        assert rel_err(row[rank + rot_dims:], d[t, q_rank + rank + rot_dims:]) < TOL[dtype]
    heads, dim = 3, 8
    q = torch.randn(T, heads * (dim + rot), generator=g).to(DT[dtype])
    qd = q.to(DEV)
    ops.rotate_pairs(qd, heads, dim + rot, dim, rot, rot_dims, inv.to(DEV), i32(pos), i32(tseq), rank)
    q3 = q.double().view(T, heads, dim + rot)
    want = q3.clone()
    want[..., dim:] = plain.rotate_interleaved(q3[..., dim:], torch.tensor(pos), base, rot_dims)
    assert rel_err(qd.float().cpu().view(T, heads, dim + rot), want) < TOL[dtype]
    # the same into the tail of wider rows (the layout the tensor-core attention reads)
    wide = torch.zeros(T, heads * (rank + rot), dtype=DT[dtype], device=DEV)
    ops.rotate_pairs(q.to(DEV), heads, dim + rot, dim, rot, rot_dims, inv.to(DEV), i32(pos), i32(tseq), rank,
                     out=wide, out_head_stride=rank + rot, out_off=rank)
    assert rel_err(wide.float().cpu().view(T, heads, rank + rot)[..., rank:], want[..., dim:]) < TOL[dtype]
    assert float(wide.view(T, heads, rank + rot)[..., :rank].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,T", [(5, 2, 37), (8, 1, 3), (3, 3, 150), (16, 4, 1)])
def test_routed_experts_kernels(ops, dtype, E, top, T):
    W, F = 48, 24
    g = torch.Generator().manual_seed(E * 100 + T)
    h = torch.randn(T, W, generator=g).to(DT[dtype])
    p = {"router": torch.randn(E, W, generator=g), "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        p[f"e{e}.gate"] = (torch.randn(F, W, generator=g) * 0.3).to(DT[dtype])
        p[f"e{e}.up"] = (torch.randn(F, W, generator=g) * 0.3).to(DT[dtype])
        p[f"e{e}.down"] = (torch.randn(W, F, generator=g) * 0.3).to(DT[dtype])
    want = plain.routed_ff(h.double(), {k: v.double() for k, v in p.items()}, E, top, False)
    hd = h.to(DEV)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    ops.moe_route(hd, p["router"].to(DEV), p["router.b"].to(DEV), None, top, idx, wts)
    logits = h.double() @ p["router"].double().T + p["router.b"].double()
    tv, ti = torch.topk(logits, top, dim=-1)
    assert torch.equal(idx.cpu().long(), ti)
    assert rel_err(wts.cpu(), torch.softmax(tv, -1)) < 1e-5
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(T * top, dtype=torch.int32, device=DEV)
    place = torch.empty(T * top, dtype=torch.int32, device=DEV)
    ops.moe_order(idx, E, offsets, order, place)
    off = offsets.cpu().tolist()
    assert off[0] == 0 and off[-1] == T * top
    assert sorted(order.cpu().tolist()) == list(range(T * top))
    flat = idx.cpu().view(-1)
    for e in range(E):
        assert all(int(flat[a]) == e for a in order.cpu()[off[e]:off[e + 1]].tolist())
    gu = torch.stack([torch.cat([p[f"e{e}.gate"], p[f"e{e}.up"]]) for e in range(E)]).to(DEV)
    dn = torch.stack([p[f"e{e}.down"] for e in range(E)]).to(DEV)
    act = torch.empty(T * top, F, dtype=DT[dtype], device=DEV)
    ops.moe_gemm(hd, gu, act, offsets, order, top, gated=True)
    y = torch.empty(T * top, W, dtype=torch.float32, device=DEV)
    ops.moe_gemm(act, dn, y, offsets, None, top, gated=False)
    out = torch.empty(T, W, dtype=DT[dtype], device=DEV)
    ops.moe_combine(y, place, wts, None, out)
    assert rel_err(out.float().cpu(), want) < TOL[dtype]


@pytest.mark.parametrize("E,top,T,shared", [(5, 2, 700, True), (3, 1, 1100, False), (9, 3, 260, True)])
def test_routed_experts_on_the_tensor_cores(ops, E, top, T, shared):
    """The part itself in bfloat16 with enough rows for the gathered tcgen05 products (spans of 128-row tiles, one
    expert's weights a tile), against the plain statement; inner size and width are no multiples of the tiles."""
    from tokasaurus_b200.engine.runtime import Runtime
    from tokasaurus_b200.parts import GatedMLP, RoutedExperts

    W, F = 136, 88
    g = torch.Generator().manual_seed(E + T)
    p = {"router": torch.randn(E, W, generator=g), "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        for n, shape in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F))):
            p[f"e{e}.{n}"] = (torch.randn(shape, generator=g) * 0.2).to(torch.bfloat16)
    if shared:
        for n, shape in (("gate", (48, W)), ("up", (48, W)), ("down", (W, 48))):
            p[f"shared.{n}"] = (torch.randn(shape, generator=g) * 0.2).to(torch.bfloat16)
    part = RoutedExperts(W, F, E, top, "router", "router.b", lambda e: (f"e{e}.gate", f"e{e}.up", f"e{e}.down"),
                         GatedMLP(W, 48, "shared.gate", "shared.up", "shared.down") if shared else None)
    assert T * top >= part.TENSOR_CORE_PAIRS_MIN
    part.bind({k: v.to(DEV) for k, v in p.items()}, Runtime.make(DEV, "bfloat16"))
    assert part.w_gate_up_tc is not None
    h = torch.randn(T, W, generator=g).to(torch.bfloat16)
    got = part.forward(None, h.to(DEV))
    if got.dim() == 3:
        got = got.sum(0)
    want = plain.routed_ff(h.double(), {k: v.double() for k, v in p.items()}, E, top, shared)
    assert rel_err(got.float().cpu(), want) < TOL["bfloat16"]


# ------------------------------------------------------------------------------------------------ whole models
def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, rot_dims=None, base=10000.0, kv_from=None, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, mask=dict(size=window),
             rot=dict(base=base, dims=rot_dim if rot_dims is None else rot_dims),
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def recurrent(heads, dim, vdim):
    return dict(type="hgrn2", mixer=dict(heads=heads, dim=dim, vdim=vdim))


def moe(ff, experts, top, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


MODELS = {
    # twenty query heads on one cached row (two tiles of sixteen in the tensor-core kernels), a window of several
    # key tiles, prompts longer than it, a reader with a narrower window and another head count
    "c": dict(page=16, lengths=[300, 150, 40, 210, 33, 64],
              config=dict(architecture="Sozurax", vocab=113, width=128, norm=dict(eps=1e-6), embedding=dict(scale=2.0),
                          canon=dict(taps=2),
                          layers=[dict(latent(20, 16, 16, 16, 48, 32, 200, base=2000.0), mlp=dict(kind="dense", ff=96)),
                                  dict(recurrent(4, 16, 32), mlp=None),
                                  dict(latent(17, 8, 16, 24, 48, 40, 130, base=2000.0, kv_from=0), mlp=moe(64, 4, 2, shared=64))])),
    # latent attention first, windows no multiple of the page size, a reader of another layer's rows without a
    # feed-forward, one chosen expert without a shared expert, rotary on fewer values than the rotated part holds
    "a": dict(page=8, lengths=[100, 37, 64, 5, 81, 1, 50],
              config=dict(architecture="Sozurax", vocab=151, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.5),
                          canon=dict(taps=3),
                          layers=[dict(latent(5, 24, 8, 16, 40, 56, 23, rot_dims=6), mlp=dict(kind="dense", ff=136)),
                                  dict(recurrent(3, 24, 40), mlp=moe(40, 5, 1)),
                                  dict(latent(2, 16, 8, 48, 40, 24, 23, rot_dims=6, kv_from=0), mlp=None),
                                  dict(recurrent(2, 20, 12), mlp=moe(24, 6, 2, shared=56))])),
    # a recurrence first, rows of 42 values (no 16-byte multiple), five taps, a window of one page and one longer than
    # most requests, three chosen experts, a reader of another layer's rows with a wider window than that layer's own
    "b": dict(page=16, lengths=[130, 70, 33, 16, 97],
              config=dict(architecture="Sozurax", vocab=97, width=64, norm=dict(eps=1e-6), embedding=dict(scale=1.0),
                          canon=dict(taps=5),
                          layers=[dict(recurrent(1, 64, 64), mlp=dict(kind="dense", ff=80)),
                                  dict(latent(3, 20, 6, 20, 36, 36, 16, base=500.0), mlp=moe(16, 4, 3, shared=32)),
                                  dict(latent(4, 8, 6, 8, 36, 16, 90, base=500.0), mlp=moe(32, 3, 2)),
                                  dict(latent(3, 20, 6, 20, 36, 36, 29, base=500.0, kv_from=1), mlp=dict(kind="dense", ff=48))])),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from safetensors import safe_open
    from safetensors.torch import save_file
    from tokasaurus_b200.weights import write_model_folder

    root = tmp_path_factory.mktemp("sozurax_models")
    out = {}
    for name, spec in MODELS.items():
        folder = write_model_folder(root / name, spec["config"], seed=17 + len(name), std=0.12, norm_init="uniform")
        w = {}
        with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
            for k in f.keys():
                w[k] = f.get_tensor(k)
        # a forget gate's lower bound lies in [0, 1): above 1 the state would grow without bound
        for k in w:
            if k.endswith(".mix.lower"):
                w[k] = ((w[k].float() - 0.5) * 0.9).to(w[k].dtype)
        save_file(w, str(folder / "model.safetensors"))
        V = spec["config"]["vocab"]
        reqs = {f"{name}{i}": cuttings.random_tokens(n, V, 40 + i) for i, n in enumerate(spec["lengths"])}
        want = {rid: plain.forward(spec["config"], w, t).numpy() for rid, t in reqs.items()}
        out[name] = dict(folder=folder, config=spec["config"], weights=w, reqs=reqs, want=want, page=spec["page"])
    return out


def windows_of(config):
    return sorted({l["mixer"]["mask"]["size"] for l in config["layers"] if l["type"] == "latent_attention"})


def pool_tokens(steps, config, page):
    """Tokens of page pool a trace needs when pages behind a window come back after every step (the largest need
    over the model's windows: every windowed group gets a pool of this size)."""
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
    """float32: every position within 3e-5 of the logits' scale.  bfloat16: rounding has a tail (a router's close
    call moves one token's experts), so a position may pass 4e-2 of the scale by up to half, one in fifty of a
    request's positions at most (at least one)."""
    for rid, ref in m["want"].items():
        scale = float(np.sqrt((ref ** 2).mean()))
        tol = (3e-5 if dtype == "float32" else 4e-2) * scale
        d = got[rid] - ref
        err = np.sqrt(((d - d.mean(axis=1, keepdims=True)) ** 2).mean(axis=1))
        bad = np.nonzero(err > tol)[0]
        allowed = 0 if dtype == "float32" else max(1, len(err) // 50)
        far = np.nonzero(err > 1.5 * tol)[0]
        assert bad.size <= allowed and far.size == 0, (
            f"{dtype} {what}: request {rid}: first wrong token at position {bad[0]} "
            f"(error {err[bad[0]]:.3g}, tolerance {tol:.3g}); {bad.size} of {len(err)} over it, {far.size} over 1.5 times it")


CUTS = dict(whole=cuttings.whole, prefix_then_single=cuttings.prefix_then_single,
            changing_portions=cuttings.changing_portions, mixed=cuttings.mixed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("which", list(MODELS))
def test_cuttings_match_plain(models, which, cut, dtype):
    """Whole prompts, prompts then single tokens, portions of changing size down to one and two tokens, and up to
    four requests side by side in four slots, in a pool that holds exactly what the trace needs: pages and slots are
    used again, and a later request must see nothing of an earlier one's state."""
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
            for p in rc.live_pages(0):
                owners.setdefault(p, set()).add(rid)
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]
    check_logits(cuttings.collect(steps, outs), m, dtype, cut)
    if cut == "mixed":
        assert any(len(v) > 1 for v in owners.values()), "no page was used by two requests"
        assert any(len(v) > 1 for v in slots.values()), "no slot was used by two requests"


def test_cuttings_with_the_tensor_core_expert_products(models, monkeypatch):
    """The same in bfloat16 with the gathered tcgen05 expert products used from 24 (token, choice) pairs on, so that
    portions of prompts go through them and single tokens beside them do not."""
    from tokasaurus_b200.engine.trace import TraceReplayer
    from tokasaurus_b200.parts import RoutedExperts

    monkeypatch.setattr(RoutedExperts, "TENSOR_CORE_PAIRS_MIN", 24)
    for which in MODELS:
        m = models[which]
        for cut in ("whole", "mixed"):
            steps = CUTS[cut](m["reqs"])
            rp = TraceReplayer(str(m["folder"]), "bfloat16", pool_tokens(steps, m["config"], m["page"]), page_size=m["page"],
                               max_requests=4)
            check_logits(cuttings.collect(steps, [rp.run_step(st) for st in steps]), m, "bfloat16", cut)


def test_windows_taps_and_state_show_in_the_logits(models):
    """The comparisons above would not notice a window off by one, a lost tap or a state that is not carried if those
    carried no weight: on the plain implementation, changing each moves the logits by hundreds of times the tolerance
    of the float32 comparisons (the bfloat16 ones are coarser; for them the edges of a window are shown with a made-up
    key in ``test_latent_attention_window_edges``)."""
    m = models["a"]
    rid, toks = max(m["reqs"].items(), key=lambda kv: len(kv[1]))
    ref = m["want"][rid]
    tol = 1e-3 * float(np.sqrt((ref ** 2).mean()))  # a hundred times what the float32 comparisons allow, taken three times below

    def moved(config, weights=None):
        d = plain.forward(config, weights or m["weights"], toks).numpy() - ref
        return float(np.sqrt((d ** 2).mean(axis=1)).max())

    import copy
    wider = copy.deepcopy(m["config"])
    for l in wider["layers"]:
        if l["type"] == "latent_attention":
            l["mixer"]["mask"]["size"] += 1
    assert moved(wider) > 3 * tol
    w2 = dict(m["weights"])
    w2["l1.canon1"] = w2["l1.canon1"].clone()
    w2["l1.canon1"][:, 0] = 0  # the oldest tap of one convolution
    assert moved(m["config"], w2) > 3 * tol
    w3 = dict(m["weights"])
    w3["l1.mix.lower"] = torch.zeros_like(w3["l1.mix.lower"])  # another decay of one recurrence
    assert moved(m["config"], w3) > 3 * tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_windows(models, dtype):
    """A short prompt, then 150 tokens one by one: every window passes over decoded tokens several times, pages come
    back behind it, and the recurrent state is carried 150 steps."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    m = models["a"]
    V = m["config"]["vocab"]
    toks = cuttings.random_tokens(160, V, 7)
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


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(models, graphs):
    """Greedy generation in float32 through ``Engine.generate``: the scheduler admits, cuts prompts into portions,
    decodes (from CUDA graphs or kernel by kernel) and frees; five requests in three slots, so slots are handed on."""
    from tokasaurus_b200.engine.engine import Engine

    m = models["a"]
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
