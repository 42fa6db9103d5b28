"""Sunesun (windowed attention whose values are its keys, routed experts, hyper-connected residual streams, looped
layers) on the GPU engine against the plain oracle of tests/sunesun_oracle.py: every mechanism alone, then whole models
under every way of feeding them."""
import math

import pytest
import torch

import sunesun_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 0.15
PAGE = 32


def _mixer(heads=6, kv_heads=3, dim=24, rot_dims=10, window=37, softcap=15.0, scaling=True, **kw):
    rot = {"base": 5000.0, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 6.0, "original": 64, "fast": 8.0, "slow": 1.5}
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": 1.0 / math.sqrt(dim), "rot": rot}
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    m.update(kw)
    return m


def _moe(experts=12, top=3, count=3, keep=2, ff=40):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def _cfg_a():
    """Sizes unlike powers of two: 6 / 3 heads of 24 with 10 rotated dimensions, a window of 37 (no multiple of the page),
    3 streams, 12 experts in 3 groups; a layer without feed-forward; layer 3 runs layer 1's weights; one layer has one
    key/value head, no soft cap and no frequency scaling, another as many key/value heads as heads and one expert group."""
    return {"architecture": "Sunesun", "width": 88, "vocab": 277, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7},
            "residual_mult": 0.6, "streams": 3, "layers": [
                {"type": "attention", "mixer": _mixer(), "mlp": _moe()},
                {"type": "attention", "mixer": _mixer(heads=4, kv_heads=1, dim=40, rot_dims=40, window=5, softcap=0, scaling=False),
                 "mlp": _moe(experts=5, top=2, count=1, keep=1, ff=24)},
                {"type": "attention", "mixer": _mixer(heads=3, kv_heads=3, dim=16, rot_dims=4, window=64), "mlp": None},
                {"type": "attention", "mixer": _mixer(heads=4, kv_heads=1, dim=40, rot_dims=40, window=5, softcap=0, scaling=False),
                 "mlp": _moe(experts=5, top=2, count=1, keep=1, ff=24), "weights_of": 1},
                {"type": "attention", "mixer": _mixer(heads=2, kv_heads=2, dim=32, rot_dims=32, window=0), "mlp": _moe(experts=4, top=4, count=4, keep=4)},
            ]}


def _cfg_plain():
    """No streams at all (the plain residual sum with its multiplier), one stream with weights is covered by _cfg_one."""
    c = _cfg_a()
    del c["streams"]
    c["layers"] = c["layers"][:2]
    return c


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    from dllama_b200.models.layered import write_random_model
    d = str(tmp_path_factory.mktemp("sunesun") / "a")
    cfg = _cfg_a()
    tensors = write_random_model(d, cfg, seed=3)
    g = torch.Generator().manual_seed(4)
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (150, 70, 5, 33)]
    want = [O.model_logits(tensors, cfg, r) for r in reqs]
    return d, cfg, tensors, reqs, want


def _engine(path, dtype="float32", max_rows=256, n_slots=4, seq=256, n_pages=None, **kw):
    from dllama_b200.models import registry
    return registry.engine_for_dir(path, max_rows=max_rows, n_slots=n_slots, max_seq_len=seq, n_pages=n_pages, dtype=dtype, **kw)


def _replay(eng, reqs, steps, free_when_done=True):
    fed, slot, got = {}, {}, {i: [] for i in range(len(reqs))}
    for step in steps:
        toks, pos, slots, owner = [], [], [], []
        for i, n in step:
            if i not in slot:
                slot[i], fed[i] = eng.alloc_slot(), 0
            toks += reqs[i][fed[i]:fed[i] + n]
            pos += list(range(fed[i], fed[i] + n))
            slots += [slot[i]] * n
            owner += [i] * n
            fed[i] += n
        lg = eng.forward(toks, pos, slots).cpu()
        for r, i in enumerate(owner):
            got[i].append(lg[r])
        for i, _ in step:
            if free_when_done and fed[i] == len(reqs[i]) and i in slot:
                eng.free_slot(slot.pop(i))
    return {i: torch.stack(v) for i, v in got.items() if v}


def _assert_close(got, want, tol, what="", flips=False):
    """flips: a bf16 run against the exact oracle.  Operand rounding moves router scores by about a hundredth, and with a
    dozen experts a good part of the tokens has its last chosen and first unchosen expert closer than that: such a token
    takes another expert than the oracle and lands far off, with the tokens that attend to it.  So bf16 runs are held to
    the oracle in the bulk (median, and three rows in four within the tolerance) and, row by row and tightly, to the bf16
    run of the whole prompt (_assert_same); row-by-row exactness against the oracle is the f32 runs' part."""
    err = O.logit_error(got, want[:got.shape[0]])
    assert float(err.median()) < tol / 4, f"{what}: median error {float(err.median()):.3e}"
    if flips:
        over = int((err > tol).sum())
        assert over <= max(2, got.shape[0] // 4), f"{what}: {over} of {got.shape[0]} rows over {tol}"
    else:
        assert float(err.max()) < tol, f"{what}: worst row {int(err.argmax())} error {float(err.max()):.3e}"


def _assert_same(got, ref, what, tol=0.02):
    """Two runs of the same engine type on the same tokens, fed differently: equal up to summation order (one row in fifty
    may differ: a routing tie within that noise)."""
    err = O.logit_error(got, ref[:got.shape[0]])
    over = int((err > tol).sum())
    assert over <= got.shape[0] // 50, f"{what}: {over} rows differ, worst row {int(err.argmax())} by {float(err.max()):.3e}"


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S,dim", [(1, 40), (2, 72), (4, 333), (5, 4500), (8, 64), (11, 96), (16, 50)])
def test_hyper_connection_write_read_and_both_at_once(S, dim):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(S * 100 + dim)
    M = 7
    x0 = torch.randn(M, S, dim, generator=g)
    y = torch.randn(M, dim, generator=g)
    mix, w_in, w_out, nw = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(dim, generator=g)
    copies = [x0[:, s].double() for s in range(S)]
    new = O.hyper_write(copies, mix.double(), w_out.double(), 0.3, y.double())
    want_x = torch.stack(new, 1)
    want_h = O.rms_weighted(O.hyper_read(new, w_in.double()), nw.double(), 1e-5)
    c = lambda t: t.cuda().contiguous()
    # write and read in one launch
    x, h = c(x0.reshape(M, S * dim)), torch.zeros(M, dim, device="cuda")
    L.hyper_step(x, M, S, dim, y=c(y), mix=c(mix), w_out=c(w_out), mult=0.3, h=h, w_in=c(w_in), norm_w=c(nw), eps=1e-5)
    assert torch.allclose(x.cpu().double().view(M, S, dim), want_x, atol=1e-5, rtol=1e-5)
    assert torch.allclose(h.cpu().double(), want_h, atol=2e-5, rtol=2e-5)
    # the same as two launches
    x2, h2 = c(x0.reshape(M, S * dim)), torch.zeros(M, dim, device="cuda")
    L.hyper_step(x2, M, S, dim, y=c(y), mix=c(mix), w_out=c(w_out), mult=0.3)
    L.hyper_step(x2, M, S, dim, h=h2, w_in=c(w_in), norm_w=c(nw), eps=1e-5)
    assert torch.equal(x2, x) and torch.allclose(h2, h, atol=1e-6, rtol=1e-6)
    # gathered rows, plain sum of the copies (the model's last norm)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    h3 = torch.zeros(3, dim, device="cuda")
    L.hyper_step(x, 3, S, dim, h=h3, norm_w=c(nw), eps=1e-5, rows=rows)
    want3 = O.rms_weighted(sum(new), nw.double(), 1e-5)[[5, 0, 5]]
    assert torch.allclose(h3.cpu().double(), want3, atol=2e-5, rtol=2e-5)


def test_interleaved_rotary_with_scaled_frequencies():
    from dllama_b200.models.layered import interpolated_rotary
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(1)
    M, H, d = 9, 3, 20
    for rot in ({"base": 700.0, "dims": 12, "scaling": {"factor": 5.0, "original": 40, "fast": 6.0, "slow": 1.2}},
                {"base": 10000.0, "dims": 20}):
        x0 = torch.randn(M, H, d, generator=g)
        pos = torch.tensor([0, 1, 2, 40, 41, 1000, 7, 8, 9], dtype=torch.int32)
        cos, sin = O.rotary_table(rot, 1001)
        want = O.rotate_interleaved(x0.double(), cos[pos.long()], sin[pos.long()])
        f, mag = interpolated_rotary(rot["base"], rot["dims"], rot.get("scaling"))
        x = x0.reshape(M, H * d).cuda().contiguous()
        L.rope_rows(x, M, H, d, 0, rot["dims"], f.cuda(), pos.cuda(), interleaved=True, mag=mag)
        assert torch.allclose(x.cpu().double().view(M, H, d), want, atol=1e-5, rtol=1e-5)


def _attention_case(ctype, H, G, d, rd, window, softcap, n_ctx, queries, boost, tc=False):
    """Fill a paged cache through the writer with random keys, make ONE key per query dominate (scaled so that its
    score stands out), and compare with the oracle's softmax over exactly the visible positions.
    queries: list of (position, boosted position)."""
    from dllama_b200.models.layered import interpolated_rotary
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(n_ctx + d)
    rot = {"base": 900.0, "dims": rd}
    f, mag = interpolated_rotary(rot["base"], rd, None)
    n_pages = (n_ctx + PAGE - 1) // PAGE
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages].to(torch.int32)          # pages out of order
    bt = torch.zeros(2, n_pages, dtype=torch.int32)
    bt[1] = perm
    cache = torch.full((n_pages + 3, G, PAGE, d + rd), 77.0, dtype=ctype).cuda()       # stale lines everywhere
    k = torch.randn(n_ctx, G, d, generator=g) * 0.3
    q = torch.randn(len(queries), H, d, generator=g) * 0.3
    rep = H // G
    cos, sin = O.rotary_table(rot, n_ctx)
    for n, (p, b) in enumerate(queries):            # query n at position p: every head points at (rotated) key b
        for h in range(H):
            kb = O.rotate_interleaved(k[b:b + 1].double(), cos[b:b + 1], sin[b:b + 1])[0, h // rep]
            # a query that the rotation at p turns into boost * key b
            qq = (kb * boost / (kb.norm() ** 2)).float()
            inv = O.rotate_interleaved(qq.view(1, 1, d).double(), cos[p:p + 1], -sin[p:p + 1])[0, 0]
            q[n, h] = inv.float()
    kd = k.reshape(n_ctx, G * d).cuda().contiguous()
    pos_all = torch.arange(n_ctx, dtype=torch.int32).cuda()
    slot_all = torch.ones(n_ctx, dtype=torch.int32).cuda()
    L.window_kv_write(kd, n_ctx, G, d, rd, f.cuda(), mag, pos_all, slot_all, bt.cuda(), cache)
    qd = q.reshape(len(queries), H * d).cuda().contiguous()
    qpos = torch.tensor([p for p, _ in queries], dtype=torch.int32).cuda()
    L.rope_rows(qd, len(queries), H, d, 0, rd, f.cuda(), qpos, interleaved=True, mag=mag)
    # the writer turns queries too (into a scratch cache here): the same numbers as the stand-alone rotation
    q2 = q.reshape(len(queries), H * d).cuda().contiguous()
    L.window_kv_write(torch.zeros(len(queries), G * d, device="cuda"), len(queries), G, d, rd, f.cuda(), mag, qpos,
                      torch.zeros(len(queries), dtype=torch.int32, device="cuda"), bt.cuda(), torch.zeros_like(cache), q=q2, q_heads=H)
    assert torch.allclose(q2, qd, atol=1e-5, rtol=1e-5)
    out = torch.zeros(len(queries), H * d, device="cuda")
    qslot = torch.ones(len(queries), dtype=torch.int32).cuda()
    scale = 1.0
    if tc:
        L.window_attention_tiles(qd, out, H, G, d, rd, scale, softcap, window, qpos, qslot, bt.cuda(), cache,
                                 [[i] for i in range(len(queries))])
    else:
        L.window_attention(qd, out, len(queries), H, G, d, rd, scale, softcap, window, qpos, qslot, bt.cuda(), cache)
    # oracle on the values the cache holds (rounded to its type)
    kr = O.rotate_interleaved(k.double(), cos, sin).to(ctype).double()
    kv = k.to(ctype).double()
    qr = torch.stack([O.rotate_interleaved(q[n:n + 1].double(), cos[p:p + 1], sin[p:p + 1])[0] for n, (p, _) in enumerate(queries)])
    want = torch.zeros(len(queries), H, d, dtype=torch.float64)
    seen = []
    for n, (p, b) in enumerate(queries):
        first = max(0, p - window + 1) if window else 0
        for h in range(H):
            sc = kr[first:p + 1, h // rep] @ qr[n, h] * scale
            if softcap:
                sc = softcap * torch.tanh(sc / softcap)
            pr = torch.softmax(sc, 0)
            want[n, h] = pr @ kv[first:p + 1, h // rep]
        seen.append(first <= b <= p)
        if seen[-1]:                                  # the boosted key really dominates where it is visible
            assert float(pr[b - first]) > 0.9
    got = out.cpu().double().view(len(queries), H, d)
    tol = 2e-5 if ctype == torch.float32 and not tc else 2e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), (got - want).abs().max()
    return seen


WINDOW = 41
WINDOW_QUERIES = [  # (position, boosted key): at distance 0, WINDOW - 1 (the last one seen) and WINDOW (the first one not seen)
    (0, 0), (1, 0), (5, 5), (40, 0), (41, 0), (41, 1), (42, 1), (42, 2), (63, 23), (63, 22), (64, 24), (64, 23),
    (95, 55), (96, 56), (96, 55), (200, 160), (200, 159), (200, 199), (200, 200), (255, 215), (255, 214), (255, 31), (255, 0)]


@pytest.mark.parametrize("ctype", [torch.float32, torch.bfloat16])
def test_window_attention_sees_exactly_its_window(ctype):
    seen = _attention_case(ctype, H=6, G=2, d=24, rd=8, window=WINDOW, softcap=50.0, n_ctx=256, queries=WINDOW_QUERIES, boost=25.0)
    assert seen == [0 <= p - b < WINDOW for p, b in WINDOW_QUERIES] and seen.count(False) == 9
    # window a multiple of the page, one key/value head per head, everything rotated; window 1: only itself
    _attention_case(ctype, H=3, G=3, d=16, rd=16, window=32, softcap=0.0, n_ctx=130,
                    queries=[(31, 0), (32, 0), (32, 1), (64, 32), (64, 33), (129, 98), (129, 97)], boost=20.0)
    _attention_case(ctype, H=2, G=1, d=8, rd=2, window=1, softcap=0.0, n_ctx=70, queries=[(0, 0), (33, 32), (33, 33), (69, 69)], boost=20.0)
    # no window: a key hundreds of positions back
    _attention_case(ctype, H=8, G=2, d=32, rd=32, window=0, softcap=30.0, n_ctx=600, queries=[(599, 0), (599, 3), (300, 299), (32, 31)], boost=25.0)


def test_window_attention_on_the_tensor_cores_sees_exactly_its_window():
    seen = _attention_case(torch.bfloat16, H=6, G=2, d=32, rd=8, window=WINDOW, softcap=50.0, n_ctx=256, queries=WINDOW_QUERIES, boost=25.0, tc=True)
    assert seen == [0 <= p - b < WINDOW for p, b in WINDOW_QUERIES]
    _attention_case(torch.bfloat16, H=3, G=3, d=16, rd=16, window=32, softcap=0.0, n_ctx=130,
                    queries=[(31, 0), (32, 0), (32, 1), (64, 32), (64, 33), (129, 98), (129, 97)], boost=20.0, tc=True)
    _attention_case(torch.bfloat16, H=8, G=2, d=64, rd=64, window=0, softcap=30.0, n_ctx=600, queries=[(599, 0), (599, 3), (300, 299), (32, 31)], boost=25.0, tc=True)
    _attention_case(torch.bfloat16, H=16, G=2, d=128, rd=16, window=100, softcap=0.0, n_ctx=300, queries=[(299, 200), (299, 199), (150, 51), (99, 0), (100, 0)], boost=25.0, tc=True)


def test_window_attention_tiles_of_rows_on_the_tensor_cores():
    """Tiles of consecutive rows of one sequence (prompt portions) against the per-row kernel on the same cache."""
    from dllama_b200.models.layered import interpolated_rotary
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(8)
    for H, G, d, rd, window, cap in ((6, 2, 32, 8, 41, 25.0), (6, 3, 48, 48, 33, 0.0), (8, 1, 64, 16, 0, 30.0), (2, 2, 96, 32, 64, 0.0)):
        n_ctx = 200
        f, mag = interpolated_rotary(3000.0, rd, {"factor": 3.0, "original": 32, "fast": 4.0, "slow": 1.0})
        n_pages = (n_ctx + PAGE - 1) // PAGE
        bt = torch.arange(n_pages, dtype=torch.int32).flip(0).view(1, n_pages).cuda().contiguous()
        cache = torch.full((n_pages, G, PAGE, d + rd), 5.0, dtype=torch.bfloat16).cuda()
        k = (torch.randn(n_ctx, G * d, generator=g)).cuda()
        q = (torch.randn(n_ctx, H * d, generator=g)).cuda()
        pos, slot = torch.arange(n_ctx, dtype=torch.int32).cuda(), torch.zeros(n_ctx, dtype=torch.int32).cuda()
        L.window_kv_write(k, n_ctx, G, d, rd, f.cuda(), mag, pos, slot, bt, cache)
        L.rope_rows(q, n_ctx, H, d, 0, rd, f.cuda(), pos, interleaved=True, mag=mag)
        want, got = torch.zeros(n_ctx, H * d, device="cuda"), torch.zeros(n_ctx, H * d, device="cuda")
        scale = 1.0 / math.sqrt(d)
        L.window_attention(q, want, n_ctx, H, G, d, rd, scale, cap, window, pos, slot, bt, cache)
        rq = L.window_tc_rows(H, G)
        for start in (0, 3):           # tiles that begin at a page border and off it; a short tail
            rows = list(range(start, n_ctx))
            tiles = [rows[i:i + rq] for i in range(0, len(rows), rq)]
            got.zero_()
            L.window_attention_tiles(q, got, H, G, d, rd, scale, cap, window, pos, slot, bt, cache, tiles)
            assert torch.allclose(got[start:], want[start:], atol=2e-2, rtol=2e-2), (H, G, d, (got[start:] - want[start:]).abs().max())
        # single rows (decoding) whose pages are shared by several CTAs, more CTAs than pages included
        for n_splits in (2, 3, 16):
            rows = [199, 0, 31, 32, 100]
            got.zero_()
            L.window_attention_tiles(q, got, H, G, d, rd, scale, cap, window, pos, slot, bt, cache, [[r] for r in rows], n_splits=n_splits)
            assert torch.allclose(got[rows], want[rows], atol=2e-2, rtol=2e-2), (H, G, d, n_splits, (got[rows] - want[rows]).abs().max())


@pytest.mark.parametrize("E,top,count,keep", [(12, 3, 3, 2), (10, 4, 2, 1), (5, 2, 1, 1), (16, 16, 4, 4), (6, 2, 6, 3), (64, 6, 8, 4), (3, 1, 1, 1)])
def test_routing_picks_the_best_experts_of_the_best_groups(E, top, count, keep):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(E * 7 + top)
    M = 37
    z = torch.randn(M, E, generator=g) * 2
    sel = torch.zeros(M, top, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(M, top, device="cuda")
    L.moe_select(z.cuda(), M, E, top, count, keep, sel, wgt)
    s = torch.sigmoid(z.double())
    r = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}}
    for m in range(M):
        want = O.route(s[m], r)
        assert sel[m].tolist() == want, (m, sel[m].tolist(), want)
        assert torch.allclose(wgt[m].cpu().double(), s[m][want], atol=1e-6)


def test_routing_can_drop_the_single_best_expert():
    """A group holding the best expert and a poor second loses to a group with two good ones (sum of the two largest)."""
    from dllama_b200.ops import layers as L
    z = torch.tensor([[4.0, -6.0, -6.0, 1.5, 1.4, -6.0]])           # groups of 3: 0.98 + 0.002 < 0.82 + 0.80
    sel, wgt = torch.zeros(1, 2, dtype=torch.int32, device="cuda"), torch.zeros(1, 2, device="cuda")
    L.moe_select(z.cuda(), 1, 6, 2, 2, 1, sel, wgt)
    assert sel[0].tolist() == [3, 4]
    assert torch.allclose(wgt.cpu(), torch.sigmoid(z[0, 3:5]).view(1, 2), atol=1e-6)


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,W,ff,E,top", [(1, 88, 40, 5, 2), (7, 72, 24, 4, 4), (70, 160, 56, 12, 3), (300, 288, 104, 8, 3)])
def test_expert_products_both_forms(wdtype, M, W, ff, E, top):
    """The per-pair form (any weights) and, for bf16 weights, the grouped tensor-core form against the oracle."""
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(M + W)
    up = (torch.randn(E, ff, W, generator=g) / math.sqrt(W)).to(wdtype)
    down = (torch.randn(E, W, ff, generator=g) / math.sqrt(ff)).to(wdtype)
    router = (torch.randn(E, W, generator=g) * 2 / math.sqrt(W)).to(wdtype)
    h = torch.randn(M, W, generator=g)
    rx = wdtype == torch.bfloat16
    hr = h.to(wdtype).double()
    w = {"router": router.double()}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = up[e].double(), down[e].double()
    spec = {"router": {"experts": E, "top": top, "groups": {"count": 1, "keep": 1}}}
    want = O.routed_experts(hr, w, spec)
    z = (hr @ router.double().T).float().cuda()
    sel, wgt = torch.zeros(M, top, dtype=torch.int32, device="cuda"), torch.zeros(M, top, device="cuda")
    L.moe_select(z, M, E, top, 1, 1, sel, wgt)
    act, y = torch.zeros(M * top, ff, device="cuda"), torch.zeros(M, W, device="cuda")
    L.moe_rows(up.cuda(), down.cuda(), h.cuda(), M, top, sel, wgt, act, y, rx)
    tol = 2e-5 if not rx else 3e-2
    scale = float(want.abs().max())
    assert float((y.cpu().double() - want).abs().max()) < tol * max(scale, 1.0)
    if rx:
        grouped = L.MoeGrouped(up.cuda(), down.cuda(), top, max_rows=M)
        y2 = torch.zeros(M, W, device="cuda")
        grouped.run(h.cuda(), M, sel, wgt, y2)
        assert float((y2.cpu().double() - want).abs().max()) < tol * max(scale, 1.0)
        assert float((y2 - y).abs().max()) < tol * max(scale, 1.0)


# ---------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompts_match_the_oracle(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    got = _replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], tol, f"request {i}", flips=dtype == "bfloat16")


def test_residual_stream_after_every_layer(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    res = []
    O.model_logits(tensors, cfg, reqs[3], residual_out=res)
    eng.layer_probe = []
    s = eng.alloc_slot()
    lg = eng.forward(reqs[3], list(range(len(reqs[3]))), [s] * len(reqs[3])).cpu()
    assert len(eng.layer_probe) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(eng.layer_probe, res)):
        assert torch.allclose(a.double().cpu(), b, atol=2e-4, rtol=2e-4), f"after layer {i}"
    _assert_close(lg, want[3], F32_TOL, "probed run")


@pytest.mark.parametrize("variant", ["plain", "one_stream", "two_streams"])
def test_other_numbers_of_streams(tmp_path, variant):
    from dllama_b200.models.layered import write_random_model
    cfg = _cfg_plain()
    if variant == "one_stream":
        cfg["streams"] = 1
    elif variant == "two_streams":
        cfg["streams"] = 2
        cfg["residual_mult"] = 1.0
        cfg["embedding"] = {"scale": 1.0}
    tensors = write_random_model(str(tmp_path / "m"), cfg, seed=11)
    assert ("l0.hc1.mix" in tensors) == (variant != "plain")
    g = torch.Generator().manual_seed(2)
    req = torch.randint(0, cfg["vocab"], (45,), generator=g).tolist()
    want = O.model_logits(tensors, cfg, req)
    eng = _engine(str(tmp_path / "m"))
    got = _replay(eng, [req], [[(0, 20)], [(0, 2)], [(0, 1)], [(0, 22)]])
    _assert_close(got[0], want, F32_TOL, variant)


def test_a_looped_layer_may_come_before_the_layer_whose_weights_it_runs(tmp_path):
    from dllama_b200.models.layered import write_random_model
    cfg = _cfg_plain()
    cfg["streams"] = 2
    cfg["layers"] = [{**cfg["layers"][1], "weights_of": 1}, cfg["layers"][1], cfg["layers"][0]]
    tensors = write_random_model(str(tmp_path / "m"), cfg, seed=13)
    assert "l0.mix.q" not in tensors and "l1.mix.q" in tensors
    req = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
    got = _replay(_engine(str(tmp_path / "m")), [req], [[(0, 33)], [(0, 7)]])
    _assert_close(got[0], O.model_logits(tensors, cfg, req), F32_TOL, "forward reference")


def test_prefill_then_token_by_token(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    steps = [[(0, 105)]] + [[(0, 1)]] * 45 + [[(1, 1)]] * 70        # the windows of 5 and 37 pass over decoded tokens
    got = _replay(eng, reqs, steps)
    _assert_close(got[0], want[0], F32_TOL, "prompt + decoded")
    _assert_close(got[1], want[1], F32_TOL, "decoded from the start")


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_portions_of_every_size(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    bf = dtype == "bfloat16"
    whole = _replay(eng, reqs, [[(0, 150)], [(1, 70)]])
    sizes = [2, 30, 1, 31, 2, 2, 33, 3, 32, 5, 2, 7]                # cuts before, at and after page borders and window edges
    assert sum(sizes) == 150
    for what, i, steps in (("portions", 0, [[(0, n)] for n in sizes]), ("two tokens at a time", 1, [[(1, 2)]] * 35),
                           ("portions of the window's size", 0, [[(0, 37)], [(0, 38)], [(0, 75)]])):
        got = _replay(eng, reqs, steps)
        _assert_close(got[i], want[i], tol, what, flips=bf)
        _assert_same(got[i], whole[i], what, 0.02 if bf else 1e-4)


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_mixed_batches_equal_each_request_alone(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    steps = [[(0, 3), (2, 1)], [(0, 40), (1, 2), (2, 1)], [(1, 30), (0, 1), (2, 2)], [(0, 1), (1, 1), (2, 1), (3, 20)],
             [(3, 13), (0, 64), (1, 5)], [(0, 1), (1, 32)], [(0, 40)]]
    got = _replay(eng, reqs, steps)
    assert got[0].shape[0] == 150 and got[1].shape[0] == 70 and got[2].shape[0] == 5 and got[3].shape[0] == 33
    whole = _replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], tol, f"request {i} in mixed batches", flips=dtype == "bfloat16")
        _assert_same(got[i], whole[i], f"request {i} in mixed batches against alone", 0.02 if dtype == "bfloat16" else 1e-4)


def test_pages_and_slots_are_reused_cleanly(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, max_rows=160, n_slots=1, seq=160, n_pages=5)
    for order in ([0, 2, 1, 3, 0], [3, 1]):
        for i in order:
            n = len(reqs[i])
            got = _replay(eng, reqs, [[(i, n // 2)], [(i, n - n // 2)]] if n > 1 else [[(i, n)]])
            _assert_close(got[i], want[i], F32_TOL, f"request {i} after reuse")
    assert len(eng.pages.free_pages) == 5 and len(eng.pages.free_slots) == 1
    eng2 = _engine(path, "bfloat16", max_rows=80, n_slots=2, seq=160, n_pages=6)     # two live requests share a small pool
    got = _replay(eng2, reqs, [[(1, 20), (3, 33)], [(1, 50)], [(2, 5), (0, 64)], [(0, 64)], [(0, 22)]])
    whole = _replay(_engine(path, "bfloat16"), reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], BF16_TOL, f"request {i} in the shared pool", flips=True)
        _assert_same(got[i], whole[i], f"request {i} in the shared pool against alone")


def test_long_decoding(model_a):
    path, cfg, tensors, reqs, want = model_a
    g = torch.Generator().manual_seed(21)
    seq = torch.randint(0, cfg["vocab"], (230,), generator=g).tolist()
    ref = O.model_logits(tensors, cfg, seq)
    eng = _engine(path)
    got = _replay(eng, [seq], [[(0, 6)]] + [[(0, 1)]] * 224)
    _assert_close(got[0], ref, F32_TOL, "224 decoded tokens")


def test_a_far_token_reaches_the_end_only_through_the_unwindowed_layer(tmp_path):
    """One token far back is changed: with every window shorter than the distance the last logits stay, with one
    unwindowed layer they move -- in the engine as in the oracle."""
    from dllama_b200.models.layered import write_random_model
    for window, moves in ((24, False), (0, True)):
        cfg = {"architecture": "Sunesun", "width": 64, "vocab": 97, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
               "residual_mult": 1.0, "streams": 2, "layers": [
                   {"type": "attention", "mixer": _mixer(heads=2, kv_heads=1, dim=32, rot_dims=16, window=window), "mlp": _moe(4, 2, 2, 1, 32)},
                   {"type": "attention", "mixer": _mixer(heads=2, kv_heads=1, dim=32, rot_dims=16, window=window), "mlp": None, "weights_of": 0}]}
        cfg["layers"][1]["mlp"] = cfg["layers"][0]["mlp"]
        d = str(tmp_path / f"w{window}")
        tensors = write_random_model(d, cfg, seed=5)
        g = torch.Generator().manual_seed(6)
        a = torch.randint(0, 97, (120,), generator=g).tolist()
        b = list(a)
        b[10] = (a[10] + 1) % 97
        eng = _engine(d)
        ga, gb = _replay(eng, [a, b], [[(0, 120)], [(1, 100)]] + [[(1, 1)]] * 20)
        wa, wb = O.model_logits(tensors, cfg, a), O.model_logits(tensors, cfg, b)
        _assert_close(ga := _replay(eng, [a], [[(0, 120)]])[0], wa, F32_TOL, "a")
        _assert_close(gb := _replay(eng, [b], [[(0, 100)]] + [[(0, 1)]] * 20)[0], wb, F32_TOL, "b")
        diff = float((ga[-1] - gb[-1]).abs().max())
        assert (diff > 1e-3) == moves, (window, diff)
        assert (float((wa[-1] - wb[-1]).abs().max()) > 1e-3) == moves


def test_greedy_generation_through_the_batching_loop(model_a, tmp_path):
    """The framework's own entry point: requests submitted to BatchEngine, batches formed by the C++ scheduler (prompt
    portions of 16 rows beside decoding rows), device greedy pick."""
    from dllama_b200.formats import tfile
    from dllama_b200.serving.batch_engine import BatchEngine, GenerationRequest
    from dllama_b200.text import native as T
    path, cfg, tensors, reqs, want = model_a
    tp = str(tmp_path / "t.t")
    tfile.write_synthetic_tokenizer(tp, cfg["vocab"])
    tok = T.Tokenizer(tp)
    eng = _engine(path, max_rows=32, n_slots=3, seq=128)
    be = BatchEngine(eng, tok, prefill_chunk=16)
    prompts = [reqs[1][:40], reqs[2], reqs[3][:20], reqs[0][:7], reqs[0][50:53]]
    n_new = 6
    rs = [be.submit(GenerationRequest(prompt_tokens=p, max_tokens=n_new, temperature=0.0)) for p in prompts]
    be.start()
    for r in rs:
        r.result(timeout=120)
    be.stop()
    assert be.n_errors == 0
    for r, p in zip(rs, prompts):
        seq = list(p)
        for _ in range(len(r.tokens)):
            seq.append(int(O.model_logits(tensors, cfg, seq)[-1].argmax()))
        assert r.tokens == seq[len(p):], (p, r.tokens, seq[len(p):])
        assert len(r.tokens) == n_new or tok.is_eos(r.tokens[-1])
    assert be.sched.stats()["free_slots"] == 3


def test_the_command_line_serves_the_model_directory(model_a):
    from dllama_b200.cli.app import build_engine
    from dllama_b200.ops import quant
    path, cfg, tensors, reqs, want = model_a
    eng = build_engine(path, 0, 1, 64, 2, 128, quant.F32, "cuda", dtype="float32")
    assert type(eng).__name__ == "LayerListEngine" and eng.h.vocab_size == cfg["vocab"] and eng.cfg.residual == "hyper"
    s = eng.alloc_slot()
    lg = eng.prefill(s, reqs[2])
    _assert_close(lg.cpu(), want[2][-1:], F32_TOL, "prefill() of the engine surface")


# ---------------------------------------------------------------------------------------------------------------------
# random configurations: sizes, layer lists and schedules drawn from a seed (f32, row by row against the oracle)
# ---------------------------------------------------------------------------------------------------------------------
def _random_config(rng):
    import json
    layers = []
    for i in range(rng.randint(1, 4)):
        own = [j for j in range(i) if "weights_of" not in layers[j]]
        if own and rng.random() < 0.3:
            j = rng.choice(own)
            layers.append({**json.loads(json.dumps(layers[j])), "weights_of": j})
            continue
        G, rep = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 5, 8])
        dim = rng.choice([16, 24, 48, 64, 80, 96, 128])
        rd = rng.choice([d for d in (0, 2, 8, 16, 24, 64, dim) if d <= dim])
        m = _mixer(heads=G * rep, kv_heads=G, dim=dim, rot_dims=rd, window=rng.choice([0, 1, 2, 7, 31, 32, 33, 65, 100]),
                   softcap=rng.choice([0, 5.0, 50.0]), scaling=bool(rd) and rng.random() < 0.7)
        mlp = None
        if rng.random() < 0.85:
            count, per = rng.choice([1, 2, 4]), rng.choice([1, 2, 3])
            keep = rng.randint(1, count)
            mlp = _moe(experts=count * per, top=rng.randint(1, keep * per), count=count, keep=keep, ff=rng.choice([16, 40, 130]))
        layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Sunesun", "width": rng.choice([64, 100, 136, 192]), "vocab": rng.choice([97, 300, 513]),
           "norm": {"eps": 1e-5}, "embedding": {"scale": rng.choice([1.0, 2.5])}, "residual_mult": rng.choice([1.0, 0.4]), "layers": layers}
    streams = rng.choice([0, 1, 2, 3, 4, 8])
    if streams:
        cfg["streams"] = streams
    return cfg


def _random_schedule(rng, lens):
    left, steps, live, pending = list(lens), [], [], list(range(len(lens)))
    while pending or live:
        while pending and len(live) < 3 and (not live or rng.random() < 0.7):
            live.append(pending.pop(0))
        step = []
        for i in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue                                                # a request sits a step out
            n = min(left[i], rng.choice([1, 1, 1, 2, 3, 17, 32, 33, 64, 90]))
            step.append((i, n))
            left[i] -= n
            if left[i] == 0:
                live.remove(i)
        if step:
            steps.append(step)
    return steps


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5])
def test_random_configurations_and_schedules(tmp_path, seed):
    import random
    from dllama_b200.models.layered import write_random_model
    rng = random.Random(seed)
    cfg = _random_config(rng)
    tensors = write_random_model(str(tmp_path / "m"), cfg, seed=seed)
    g = torch.Generator().manual_seed(seed)
    lens = [rng.choice([1, 5, 40, 70, 130]) for _ in range(4)]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    want = [O.model_logits(tensors, cfg, r) for r in reqs]
    n_pages = 3 * (max(lens) + 64) // PAGE
    eng = _engine(str(tmp_path / "m"), max_rows=n_pages * PAGE, n_slots=3, seq=n_pages * PAGE, n_pages=n_pages)
    got = _replay(eng, reqs, _random_schedule(rng, lens))
    for i in got:
        assert got[i].shape[0] == lens[i]
        _assert_close(got[i], want[i], F32_TOL, f"seed {seed}, request {i}: {cfg['layers']}")
    assert len(eng.pages.free_pages) == n_pages and len(eng.pages.free_slots) == 3
    eng.close()
    # the same model in bf16: fed in the schedule or whole, a row comes out the same
    eng = _engine(str(tmp_path / "m"), "bfloat16", max_rows=n_pages * PAGE, n_slots=3, seq=n_pages * PAGE, n_pages=n_pages)
    got = _replay(eng, reqs, _random_schedule(random.Random(seed + 100), lens))
    whole = _replay(eng, reqs, [[(i, n)] for i, n in enumerate(lens)])
    for i in got:
        _assert_same(got[i], whole[i], f"seed {seed}, request {i} in bf16", tol=0.03)
