"""Layer-list models (Mamba-2 and latent-attention mixers) on the GPU engine against the plain oracle of
tests/layered_oracle.py: every mechanism alone, then whole models under every way of feeding them (whole prompts, token
by token, portions down to two tokens, mixed batches, reused pages and slots, long decoding, the batching loop)."""
import math
import os

import pytest
import torch

import layered_oracle as O

pytestmark = pytest.mark.gpu

# bf16: operands of every product are rounded to 8 bits of mantissa, so single rows of a small model differ by several
# per cent from exact arithmetic; a fault (a missed key, a lost state) shows as an error of order one
F32_TOL, BF16_TOL = 2e-4, 0.15


def _cfg_a():
    """Sizes unlike any power of two: 3 and 5 heads, groups of 1 and of `heads`, one and three norm parts, 2 and 4 taps,
    attention first, a feed-forward behind a recurrent layer, two layers reading another layer's cache."""
    att = lambda **kw: {"heads": 3, "dim": 20, "rot_dim": 12, "vdim": 28, "q_rank": 36, "kv_rank": 44, "scale": 0.19,
                        "rot": {"base": 3000.0, "dims": 12}, **kw}
    return {"architecture": "Ribivik", "width": 72, "vocab": 301, "norm": {"eps": 1e-6}, "logit_softcap": 11.0, "layers": [
        {"type": "latent_attention", "mixer": att(), "mlp": {"kind": "dense", "ff": 100}},
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 52},
         "mixer": {"heads": 5, "vdim": 12, "state": 24, "groups": 1, "conv": 2, "norm_groups": 1}},
        {"type": "latent_attention", "mixer": att(kv_from=0), "mlp": None},
        {"type": "mamba2", "mlp": None,
         "mixer": {"heads": 3, "vdim": 40, "state": 8, "groups": 3, "conv": 4, "norm_groups": 3}},
        {"type": "latent_attention", "mixer": att(kv_from=0, heads=2, q_rank=16), "mlp": {"kind": "dense", "ff": 64}},
    ]}


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    from dllama_b200.models.layered import write_random_model
    d = str(tmp_path_factory.mktemp("layered") / "a")
    cfg = _cfg_a()
    tensors = write_random_model(d, cfg, seed=5)
    g = torch.Generator().manual_seed(9)
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (150, 70, 5, 33)]
    want = [O.model_logits(tensors, cfg, r) for r in reqs]
    return d, cfg, tensors, reqs, want


def _engine(path, dtype="float32", max_rows=256, n_slots=4, seq=256, n_pages=None):
    from dllama_b200.models import registry
    return registry.engine_for_dir(path, max_rows=max_rows, n_slots=n_slots, max_seq_len=seq, n_pages=n_pages, dtype=dtype)


def _replay(eng, reqs, steps, free_when_done=True):
    """steps: list of lists of (request index, token count).  Returns per request the logits of every position fed."""
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


def _assert_close(got, want, tol, what=""):
    err = O.logit_error(got, want[:got.shape[0]])
    assert float(err.max()) < tol, f"{what}: worst row {int(err.argmax())} error {float(err.max()):.3e}"
    assert float(err.median()) < tol / 4, f"{what}: median error {float(err.median()):.3e}"


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_dense_products_shapes_and_epilogues(wdtype):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(1)
    for (M, N, K) in [(1, 37, 50), (3, 64, 96), (8, 130, 72), (9, 37, 50), (70, 65, 33), (200, 128, 256)]:
        w = torch.randn(N, K, generator=g).to(wdtype).cuda()
        x = torch.randn(M + 2, K + 3, generator=g).cuda()[:, :K]              # strided rows
        aux = torch.randn(M, N, generator=g).cuda()
        for rx in (False, True):
            xr = (x[:M].bfloat16() if rx else x[:M]).double()
            ref = xr @ w.double().T
            for epi, fn in [(L.DENSE_STORE, lambda a: a), (L.DENSE_RELU2, lambda a: a.clamp(min=0) ** 2),
                            (L.DENSE_SIGMOID_MUL, lambda a: aux.double() * torch.sigmoid(a)),
                            (L.DENSE_SOFTCAP, lambda a: 7.0 * torch.tanh(a / 7.0))]:
                y = torch.full((M + 1, N + 5), -3.0, device="cuda")
                L.dense(w, x, y, M, rx, epi=epi, aux=aux if epi == L.DENSE_SIGMOID_MUL else None, param=7.0)
                want = fn(ref)
                assert torch.allclose(y[:M, :N].double(), want, rtol=2e-4, atol=2e-4 * float(want.abs().max())), (M, N, K, rx, epi)
                assert float(y[M:].max()) == -3.0 and float(y[:, N:].max()) == -3.0       # nothing written outside


def test_dense_products_on_the_tensor_cores():
    """bf16 operands through the tcgen05 GEMM on pre-tiled images: sizes that are no multiples of the 128 x 128 tiles,
    row counts around the 256-row activation tile, every element-wise op."""
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(8)
    for (M, N, K) in [(33, 130, 200), (256, 128, 128), (257, 384, 72), (700, 257, 640)]:
        w = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
        x = torch.randn(M + 1, K + 5, generator=g).cuda()[:, :K]
        aux = torch.randn(M, N, generator=g).cuda()
        ncap = (M + 7) // 8 * 8
        wh = L.make_wh(w)
        xh = torch.zeros(L.xh_bytes(K, ncap), dtype=torch.uint8, device="cuda")
        L.xh_from_rows(x, M, K, ncap, xh)
        ref = x[:M].bfloat16().double() @ w.double().T
        for epi, fn in [(L.DENSE_STORE, lambda a: a), (L.DENSE_RELU2, lambda a: a.clamp(min=0) ** 2),
                        (L.DENSE_SIGMOID_MUL, lambda a: aux.double() * torch.sigmoid(a)),
                        (L.DENSE_SOFTCAP, lambda a: 9.0 * torch.tanh(a / 9.0))]:
            y = torch.full((M + 1, N + 3), -3.0, device="cuda")
            L.dense_tc(wh, N, K, xh, ncap, y, M, epi=epi, aux=aux if epi == L.DENSE_SIGMOID_MUL else None, param=9.0)
            want = fn(ref)
            assert torch.allclose(y[:M, :N].double(), want, rtol=2e-4, atol=2e-4 * float(want.abs().max())), (M, N, K, epi)
            assert float(y[M:].max()) == -3.0 and float(y[:, N:].max()) == -3.0
        y2 = torch.zeros(M, N, device="cuda")
        L.dense(w, x, y2, M, True)                                   # the two paths agree to accumulation order
        L.dense_tc(wh, N, K, xh, ncap, y, M)
        assert torch.allclose(y[:M, :N], y2, rtol=1e-4, atol=1e-4 * float(ref.abs().max()))


def test_dense_per_head_products():
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(2)
    H, N, K = 5, 14, 22
    for M in (2, 40):
        w = torch.randn(H, N, K, generator=g).cuda()
        x = torch.randn(M, H * (K + 6), generator=g).cuda()                   # each head's K values inside a wider head slot
        y = torch.zeros(M, H * N, device="cuda")
        L.dense_heads(w, x, y, M, False, K + 6, N)
        want = torch.einsum("mhk,hnk->mhn", x.view(M, H, K + 6)[:, :, :K].double(), w.double()).reshape(M, H * N)
        assert torch.allclose(y.double(), want, rtol=1e-4, atol=1e-4)


def test_rms_norm_variants():
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(3)
    M, dim, eps = 7, 90, 1e-3
    x, gate = torch.randn(M, dim, generator=g).cuda(), torch.randn(M, dim, generator=g).cuda()
    w = torch.randn(dim, generator=g).cuda() * 0.2
    y = torch.zeros(M, dim, device="cuda")
    L.rms_norm(x, y, M, dim, eps, w=w, plus_one=True)
    assert torch.allclose(y.double(), O.norm_around_zero(x.double(), w.double(), eps), atol=1e-5)
    L.rms_norm(x, y, M, dim, eps, w=w)
    assert torch.allclose(y.double(), O.norm_plain(x.double(), w.double(), eps), atol=1e-5)
    L.rms_norm(x, y, M, dim, eps, w=w, groups=3, gate=gate)
    v = x.double() * (gate.double() * torch.sigmoid(gate.double()))
    assert torch.allclose(y.double(), O.norm_in_parts(v, w.double(), 3, eps), atol=1e-5)
    base = torch.randn(M, dim, generator=g).cuda()
    acc = base.clone()
    L.rms_norm(x, acc, M, dim, eps, w=w, plus_one=True, accumulate=True)
    assert torch.allclose(acc.double(), base.double() + O.norm_around_zero(x.double(), w.double(), eps), atol=1e-5)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device="cuda")
    L.rms_norm(x, y, 3, dim, eps, rows=rows)
    assert torch.allclose(y[:3].double(), O.rms_unit(x[[6, 0, 3]].double(), eps), atol=1e-5)
    wide = torch.randn(2, 5000, generator=g).cuda()                          # wider than the register-cached path takes
    yw = torch.zeros(2, 5000, device="cuda")
    L.rms_norm(wide, yw, 2, 5000, eps)
    assert torch.allclose(yw.double(), O.rms_unit(wide.double(), eps), atol=1e-5)
    z = x.clone()
    L.rms_norm(z, z, M, dim, eps, w=w)                                        # in place
    assert torch.allclose(z.double(), O.norm_plain(x.double(), w.double(), eps), atol=1e-5)


def test_rotary_on_a_slice_of_each_head():
    from dllama_b200.ops import layers as L
    from dllama_b200.models.layered import rotary_frequencies
    g = torch.Generator().manual_seed(4)
    M, H, hs, off, dims = 6, 3, 26, 10, 12
    x = torch.randn(M, H * hs, generator=g).cuda()
    pos = torch.tensor([0, 1, 31, 32, 1000, 70000], dtype=torch.int32, device="cuda")
    want = x.double().cpu().view(M, H, hs).clone()
    want[..., off:] = O.rotate_half_layout(want[..., off:], pos.cpu(), 5000.0, dims)
    L.rope_rows(x, M, H, hs, off, dims, rotary_frequencies(5000.0, dims).cuda(), pos)
    assert torch.allclose(x.double().cpu().view(M, H, hs), want, atol=2e-6)


@pytest.mark.parametrize("ctype", [torch.float32, torch.bfloat16])
def test_latent_attention_sees_exactly_the_keys_up_to_its_position(ctype):
    """One key is made to stand out (its latent is the query direction, scaled): the output must be that key's latent
    when it is at or before the query's position -- first token, far back among hundreds, last of a page, first of the
    next, the query's own position -- and must ignore it one place after the query (stale lines of a page's earlier
    owner).  Pages are scattered over the pool."""
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(6)
    H, r, rot, n_ctx, n_pages = 3, 40, 8, 420, 20
    perm = torch.randperm(n_pages, generator=g)
    table = torch.zeros(2, n_pages, dtype=torch.int32)
    table[1, :14] = perm[:14].int()
    for qpos, kpos in [(0, 0), (5, 0), (400, 0), (400, 3), (31, 31), (32, 31), (32, 32), (33, 32), (400, 223), (400, 224),
                       (400, 399), (400, 400), (63, 64), (400, 401), (31, 32)]:
        cache = torch.zeros(n_pages, 32, r + rot)
        lines = torch.randn(n_ctx, r + rot, generator=g) * 0.3
        direction = torch.randn(r + rot, generator=g)
        direction /= direction.norm()
        lines[kpos] = direction * 6.0
        for t in range(n_ctx):                                                 # also lines past the query: must stay unseen
            cache[int(table[1, t // 32]), t % 32] = lines[t]
        cache = cache.to(ctype).cuda()
        q_lat = (direction[:r] * 40.0).repeat(H, 1) * torch.tensor([1.0, 0.5, 0.25])[:, None]
        q = torch.zeros(1, H * (4 + rot))
        q.view(1, H, 4 + rot)[0, :, 4:] = direction[r:] * 40.0
        out = torch.zeros(1, H * r, device="cuda")
        pos = torch.tensor([qpos], dtype=torch.int32, device="cuda")
        slot = torch.tensor([1], dtype=torch.int32, device="cuda")
        L.latent_attention(q_lat.reshape(1, H * r).cuda(), q.cuda(), 4 + rot, 4, out, 1, H, r, rot, 0.5, pos, slot, table.cuda(), cache)
        seen = cache.double().cpu()[table[1, torch.arange(qpos + 1) // 32].long(), torch.arange(qpos + 1) % 32]
        for h in range(H):
            qv = torch.cat([q_lat[h], q.view(1, H, 4 + rot)[0, h, 4:]]).double()
            p = torch.softmax(seen @ qv * 0.5, dim=0)
            want = p @ seen[:, :r]
            assert torch.allclose(out.cpu().double().view(H, r)[h], want, atol=2e-5, rtol=1e-4), (qpos, kpos, h)
        if kpos <= qpos:
            assert float(p[kpos]) > 0.9                                        # the test's premise: that key dominates
        if ctype == torch.bfloat16:
            # the tensor-core kernel (queries and probabilities rounded to bf16), alone and with the pages split over CTAs
            rows = torch.tensor([0], dtype=torch.int32, device="cuda")
            for n_splits in (1, 3):
                part = torch.zeros(L.latent_tc_partial_floats(1, n_splits, r), device="cuda")
                out2 = torch.full((1, H * r), 7.0, device="cuda")
                L.latent_attention(q_lat.reshape(1, H * r).cuda(), q.cuda(), 4 + rot, 4, out2, 1, H, r, rot, 0.5, pos, slot,
                                   table.cuda(), cache, tiles=(rows, 1, 1, n_splits, part))
                assert torch.allclose(out2, out, atol=3e-2, rtol=3e-2), (qpos, kpos, n_splits)


def test_latent_attention_tiles_of_several_rows_on_the_tensor_cores():
    """Row tiles of one sequence (rows x heads stacked on the MMA's M dimension), tiles with fewer rows than the tile
    holds, rows of two sequences in one batch in scrambled order, against the per-row kernel."""
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(16)
    for H, r, rot, rq in [(3, 40, 8, 10), (16, 512, 64, 2), (5, 96, 16, 6), (32, 64, 32, 1), (16, 512, 64, 4), (3, 40, 8, 16), (40, 32, 8, 1)]:
        n_pages = 12
        cache = (torch.randn(n_pages, 32, r + rot, generator=g) * 0.5).to(torch.bfloat16).cuda()
        table = torch.stack([torch.randperm(n_pages, generator=g)[:6], torch.randperm(n_pages, generator=g)[:6]]).int().cuda()
        # sequence 0: positions 90..120 (31 rows), sequence 1: positions 0..12; rows interleaved in the batch
        rows0, rows1 = list(range(0, 62, 2)), list(range(1, 27, 2))
        M = 62
        pos = torch.zeros(M, dtype=torch.int32)
        slot = torch.zeros(M, dtype=torch.int32)
        pos[rows0], slot[rows0] = torch.arange(90, 121, dtype=torch.int32), 0
        pos[rows1], slot[rows1] = torch.arange(0, 13, dtype=torch.int32), 1
        pos[27:62:2], slot[27:62:2] = 0, 1                                       # filler rows, not in any tile
        hd = 4 + rot
        q_lat = torch.randn(M, H * r, generator=g).cuda() * 0.3
        q = torch.randn(M, H * hd, generator=g).cuda() * 0.3
        want = torch.zeros(M, H * r, device="cuda")
        L.latent_attention(q_lat, q, hd, 4, want, M, H, r, rot, 0.2, pos.cuda(), slot.cuda(), table, cache)
        tiles = []
        for rows in (rows0, rows1):
            for i in range(0, len(rows), rq):
                part = rows[i:i + rq]
                tiles.append(part + [-1] * (rq - len(part)))
        tr = torch.tensor(tiles, dtype=torch.int32).cuda()
        for n_splits in (1, 2):
            got = torch.zeros(M, H * r, device="cuda")
            part = torch.zeros(L.latent_tc_partial_floats(len(tiles), n_splits, r), device="cuda")
            L.latent_attention(q_lat, q, hd, 4, got, M, H, r, rot, 0.2, pos.cuda(), slot.cuda(), table, cache,
                               tiles=(tr, len(tiles), rq, n_splits, part))
            live = rows0 + rows1
            assert torch.allclose(got[live], want[live], atol=2e-2, rtol=2e-2), (H, r, rq, n_splits)
            assert float(got[27:62:2].abs().max()) == 0.0


def test_latent_cache_writer_norms_rotates_and_places_lines():
    from dllama_b200.ops import layers as L
    from dllama_b200.models.layered import rotary_frequencies
    g = torch.Generator().manual_seed(7)
    r, rot, M = 20, 6, 5
    kv = torch.randn(M, r + rot, generator=g).cuda()
    w = (1 + 0.1 * torch.randn(r, generator=g)).cuda()
    pos = torch.tensor([0, 31, 32, 95, 64], dtype=torch.int32, device="cuda")
    slot = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device="cuda")
    table = torch.tensor([[7, 2, 0, 0], [1, 5, 3, 0]], dtype=torch.int32, device="cuda")
    cache = torch.zeros(8, 32, r + rot, device="cuda")
    L.latent_kv_write(kv, M, w, 1e-5, r, rot, rot, rotary_frequencies(777.0, rot).cuda(), pos, slot, table, cache)
    for m, (page, line) in enumerate([(7, 0), (7, 31), (2, 0), (3, 31), (3, 0)]):
        want = torch.cat([O.norm_plain(kv[m, :r].double().cpu(), w.double().cpu(), 1e-5),
                          O.rotate_half_layout(kv[m:m + 1, r:].double().cpu(), pos[m:m + 1].cpu(), 777.0, rot)[0]])
        assert torch.allclose(cache[page, line].double().cpu(), want, atol=2e-6), m
    assert int((cache.abs().sum(-1) > 0).sum()) == M


def _one_layer_engine(tmp_path, layer, width=48, dtype="float32"):
    from dllama_b200.models.layered import write_random_model
    cfg = {"architecture": "Ribivik", "width": width, "vocab": 64, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": [layer]}
    tensors = write_random_model(str(tmp_path), cfg, seed=11)
    return _engine(str(tmp_path), dtype=dtype, max_rows=128, n_slots=3, seq=160), tensors, cfg


def _run_mixer(eng, h, portions, slot):
    """Feed h [T, width] through layer 0's mixer in the given portions; returns its output [T, width]."""
    out, at = [], 0
    for n in portions:
        eng.set_batch([0] * n, list(range(at, at + n)), [slot] * n, [])
        eng.hn[:n] = h[at:at + n]
        eng.begin_sublayer()
        eng.layers[0].mixer.forward(eng.hn, eng.y, n)
        out.append(eng.y[:n].clone())
        at += n
    return torch.cat(out)


@pytest.mark.parametrize("groups,parts,taps,state", [(1, 1, 4, 20), (4, 2, 2, 16), (2, 4, 3, 64), (2, 1, 1, 128), (1, 2, 4, 32)])
def test_mamba2_mixer_alone_whole_and_in_portions(tmp_path, groups, parts, taps, state):
    """state 20 runs the scan with the state in shared memory, 16 / 32 / 64 / 128 the one with the state in registers"""
    layer = {"type": "mamba2", "mlp": None,
             "mixer": {"heads": 4, "vdim": 12, "state": state, "groups": groups, "conv": taps, "norm_groups": parts}}
    eng, tensors, cfg = _one_layer_engine(tmp_path, layer)
    h = torch.randn(90, 48, generator=torch.Generator().manual_seed(12))
    want = O.mamba2(h.double(), O.sub(tensors, "l0.mix."), layer["mixer"], 1e-5)
    s0 = eng.alloc_slot()
    got = _run_mixer(eng, h.cuda(), [90], s0)
    assert torch.allclose(got.double().cpu(), want, atol=3e-4, rtol=1e-3)
    s1 = eng.alloc_slot()
    got = _run_mixer(eng, h.cuda(), [2, 1, 1, 3, 40, 1, 2, 33, 1, 1, 1, 2, 2], s1)     # the state and the carried inputs cross every cut
    assert torch.allclose(got.double().cpu(), want, atol=3e-4, rtol=1e-3)
    got = _run_mixer(eng, h.cuda(), [1] * 90, s0)                                        # same slot again: starts from zeros at position 0
    assert torch.allclose(got.double().cpu(), want, atol=3e-4, rtol=1e-3)


@pytest.mark.parametrize("state,groups", [(16, 1), (64, 2), (128, 4)])
def test_mamba2_chunk_parallel_scan(tmp_path, state, groups):
    """Portions of 256 rows and more run the recurrence in chunks of 128 rows in parallel (two passes): a long portion
    from position 0, one that continues a state, two sequences of unequal length in one batch, chunk tails of 1 row."""
    from dllama_b200.models.layered import write_random_model
    layer = {"type": "mamba2", "mlp": None,
             "mixer": {"heads": 4, "vdim": 12, "state": state, "groups": groups, "conv": 4, "norm_groups": 2}}
    cfg = {"architecture": "Ribivik", "width": 48, "vocab": 64, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": [layer]}
    tensors = write_random_model(str(tmp_path), cfg, seed=17)
    eng = _engine(str(tmp_path), max_rows=700, n_slots=3, seq=1024)
    assert eng._chunk_scratch is not None
    h = torch.randn(641, 48, generator=torch.Generator().manual_seed(18))
    want = O.mamba2(h.double(), O.sub(tensors, "l0.mix."), layer["mixer"], 1e-5)
    s0 = eng.alloc_slot()
    got = _run_mixer(eng, h.cuda(), [641], s0)                                   # 5 chunks of 128 + a chunk of 1
    assert eng._n_chunks == 6
    assert torch.allclose(got.double().cpu(), want, atol=3e-4, rtol=1e-3)
    s1 = eng.alloc_slot()
    got = _run_mixer(eng, h.cuda(), [3, 300, 1, 337], s1)                        # token-by-token kernel, chunked, again, chunked
    assert torch.allclose(got.double().cpu(), want, atol=3e-4, rtol=1e-3)
    # two sequences in one batch, rows interleaved; slot s0 starts again at 0, a third slot continues later
    s2 = eng.alloc_slot()
    _run_mixer(eng, h.cuda(), [50], s2)
    rows_a, rows_b = list(range(0, 600, 2)), list(range(1, 601, 2))[:291]
    M = 600
    toks, pos, slots = [0] * M, [0] * M, [0] * M
    hin = torch.zeros(M, 48)
    for i, m in enumerate(rows_a):
        pos[m], slots[m], hin[m] = i, s0, h[i]
    for i, m in enumerate(rows_b):
        pos[m], slots[m], hin[m] = 50 + i, s2, h[50 + i]
    fill = sorted(set(range(M)) - set(rows_a) - set(rows_b))                      # the rest: a third sequence
    for i, m in enumerate(fill):
        pos[m], slots[m], hin[m] = 641 + i, s1, h[i]
    eng.set_batch(toks, pos, slots, [])
    eng.hn[:M] = hin.cuda()
    eng.begin_sublayer()
    eng.layers[0].mixer.forward(eng.hn, eng.y, M)
    y = eng.y[:M].double().cpu()
    assert torch.allclose(y[rows_a], want[:300], atol=3e-4, rtol=1e-3)
    assert torch.allclose(y[rows_b], want[50:341], atol=3e-4, rtol=1e-3)


def test_latent_attention_mixer_alone_whole_and_in_portions(tmp_path):
    layer = {"type": "latent_attention", "mlp": None,
             "mixer": {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 14, "q_rank": 18, "kv_rank": 22, "scale": 0.3,
                       "rot": {"base": 100.0, "dims": 6}}}
    eng, tensors, cfg = _one_layer_engine(tmp_path, layer)
    h = torch.randn(100, 48, generator=torch.Generator().manual_seed(13))
    want, _ = O.latent_attention(h.double(), O.sub(tensors, "l0.mix."), layer["mixer"], 1e-5)
    s0 = eng.alloc_slot()
    assert torch.allclose(_run_mixer(eng, h.cuda(), [100], s0).double().cpu(), want, atol=2e-4, rtol=1e-3)
    s1 = eng.alloc_slot()
    assert torch.allclose(_run_mixer(eng, h.cuda(), [31, 2, 1, 30, 2, 34], s1).double().cpu(), want, atol=2e-4, rtol=1e-3)


# ---------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompts_match_the_oracle(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    got = _replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], tol, f"request {i}")


def test_residual_stream_after_every_layer(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    res = []
    O.model_logits(tensors, cfg, reqs[3], residual_out=res)
    eng.layer_probe = []
    s = eng.alloc_slot()
    eng.forward(reqs[3], list(range(len(reqs[3]))), [s] * len(reqs[3]))
    for i, (a, b) in enumerate(zip(eng.layer_probe, res)):
        assert torch.allclose(a.double().cpu(), b, atol=1e-4, rtol=1e-4), f"after layer {i}"


def test_prefill_then_token_by_token(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    steps = [[(0, 105)]] + [[(0, 1)]] * 45 + [[(1, 1)]] * 70                      # request 1 is decoded from its first token
    got = _replay(eng, reqs, steps)
    _assert_close(got[0], want[0], F32_TOL, "prompt + decoded")
    _assert_close(got[1], want[1], F32_TOL, "decoded from the start")


def test_portions_of_every_size(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    sizes = [2, 30, 1, 31, 2, 2, 33, 3, 32, 5, 2, 7]                              # cuts before, at and after page borders
    assert sum(sizes) == 150
    got = _replay(eng, reqs, [[(0, n)] for n in sizes])
    _assert_close(got[0], want[0], F32_TOL, "portions")
    got = _replay(eng, reqs, [[(1, 2)]] * 35)
    _assert_close(got[1], want[1], F32_TOL, "two tokens at a time")


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_mixed_batches_equal_each_request_alone(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    steps = [[(0, 3), (2, 1)], [(0, 40), (1, 2), (2, 1)], [(1, 30), (0, 1), (2, 2)], [(0, 1), (1, 1), (2, 1), (3, 20)],
             [(3, 13), (0, 64), (1, 5)], [(0, 1), (1, 32)], [(0, 40)]]
    got = _replay(eng, reqs, steps)
    assert got[0].shape[0] == 150 and got[1].shape[0] == 70 and got[2].shape[0] == 5 and got[3].shape[0] == 33
    for i in got:
        _assert_close(got[i], want[i], tol, f"request {i} in mixed batches")


def test_pages_and_slots_are_reused_cleanly(model_a):
    """A pool that holds one long request at a time and a single slot: every request inherits the pages, the slot and
    the recurrent state of the one before it, longer or shorter."""
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, max_rows=160, n_slots=1, seq=160, n_pages=5)
    for order in ([0, 2, 1, 3, 0], [3, 1]):
        for i in order:
            n = len(reqs[i])
            got = _replay(eng, reqs, [[(i, n // 2)], [(i, n - n // 2)]] if n > 1 else [[(i, n)]])
            _assert_close(got[i], want[i], F32_TOL, f"request {i} after reuse")
    assert len(eng.pages.free_pages) == 5 and len(eng.pages.free_slots) == 1
    eng2 = _engine(path, max_rows=80, n_slots=2, seq=160, n_pages=6)                 # two live requests share a small pool
    got = _replay(eng2, reqs, [[(1, 20), (3, 33)], [(1, 50)], [(2, 5), (0, 64)], [(0, 64)], [(0, 22)]])
    for i in got:
        _assert_close(got[i], want[i], F32_TOL, f"request {i} in the shared pool")


def test_long_decoding(model_a):
    path, cfg, tensors, reqs, want = model_a
    g = torch.Generator().manual_seed(21)
    seq = torch.randint(0, cfg["vocab"], (230,), generator=g).tolist()
    ref = O.model_logits(tensors, cfg, seq)
    eng = _engine(path)
    got = _replay(eng, [seq], [[(0, 6)]] + [[(0, 1)]] * 224)
    _assert_close(got[0], ref, F32_TOL, "224 decoded tokens")


def test_a_sequence_cannot_jump(model_a):
    path, *_ = model_a
    eng = _engine(path)
    s = eng.alloc_slot()
    eng.forward([1, 2, 3], [0, 1, 2], [s] * 3)
    with pytest.raises(ValueError):
        eng.forward([4], [5], [s])                     # the recurrent state is at position 3
    with pytest.raises(ValueError):
        eng.forward([4, 5], [3, 5], [s, s])


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
    # sampled rows go through the device sampler of the engine's own library
    a = be.submit(GenerationRequest(prompt_tokens=[3, 4, 5], max_tokens=5, temperature=0.9, top_p=0.9, seed=5))
    b = be.submit(GenerationRequest(prompt_tokens=[3, 4, 5], max_tokens=5, temperature=0.9, top_p=0.9, seed=5))
    be._stop.clear()
    be.start()
    a.result(timeout=60), b.result(timeout=60)
    be.stop()
    assert a.tokens == b.tokens and len(a.tokens) >= 1


def test_the_command_line_serves_a_model_directory(model_a, tmp_path, capsys):
    from dllama_b200.cli.app import build_engine
    from dllama_b200.ops import quant
    path, cfg, tensors, reqs, want = model_a
    eng = build_engine(path, 0, 1, 64, 2, 128, quant.F32, "cuda", dtype="float32")
    assert type(eng).__name__ == "LayerListEngine" and eng.h.vocab_size == cfg["vocab"]
    s = eng.alloc_slot()
    lg = eng.prefill(s, reqs[2])
    _assert_close(lg.cpu(), want[2][-1:], F32_TOL, "prefill() of the engine surface")


def test_the_http_server_serves_a_model_directory(tmp_path):
    """`dllama-api`'s native front end (C++ HTTP server and scheduler) on the layer-list engine: concurrent greedy
    and sampled chat completions, the same seed twice, a streamed answer."""
    import json
    import threading
    import urllib.request
    from dllama_b200.formats import tfile
    from dllama_b200.models.layered import example_config, write_random_model
    from dllama_b200.serving import api_types as A
    from dllama_b200.serving.native_server import NativeApiServer
    from dllama_b200.text import native as T
    d = str(tmp_path / "m")
    write_random_model(d, example_config(width=128, vocab=1024, blocks=3, heads=4), seed=23)
    tp = str(tmp_path / "t.t")
    tfile.write_synthetic_tokenizer(tp, 1024)
    tok = T.Tokenizer(tp)
    eng = _engine(d, "bfloat16", max_rows=64, n_slots=6, seq=256)
    srv = NativeApiServer(eng, tok, "m", A.InferenceParams(messages=[], temperature=0.0, top_p=0.9, seed=1), host="127.0.0.1",
                          port=0, verbose=False)
    srv.start()

    def post(body):
        req = urllib.request.Request(f"http://127.0.0.1:{srv.port}/v1/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"}, method="POST")
        with urllib.request.urlopen(req, timeout=120) as r:
            return r.read().decode("utf-8")

    try:
        out = {}
        texts = ["hello world", "the of and hello world token model fast " * 3, "token"]
        ts = [threading.Thread(target=lambda i=i: out.__setitem__(i, json.loads(post(
            {"messages": [{"role": "user", "content": texts[i]}], "max_tokens": 5})))) for i in range(3)]
        [t.start() for t in ts]
        [t.join(timeout=200) for t in ts]
        sampled = [json.loads(post({"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 1.0,
                                    "top_p": 0.95, "seed": 7})) for _ in range(2)]
        again = json.loads(post({"messages": [{"role": "user", "content": texts[0]}], "max_tokens": 5}))
        assert len(out) == 3 and srv.stats()["engine_errors"] == 0
        for r in list(out.values()) + sampled:
            assert r["object"] == "chat.completion" and r["usage"]["completion_tokens"] >= 1
        assert sampled[0]["choices"][0]["message"]["content"] == sampled[1]["choices"][0]["message"]["content"]
        assert again["choices"][0]["message"]["content"] == out[0]["choices"][0]["message"]["content"]
        raw = post({"messages": [{"role": "user", "content": texts[0]}], "max_tokens": 5, "stream": True})
        streamed = "".join(json.loads(e[6:])["choices"][0]["delta"].get("content", "")
                           for e in raw.split("\r\n\r\n") if e.startswith("data: {"))
        assert streamed == out[0]["choices"][0]["message"]["content"]
        st = srv.stats()
        assert st["running"] == 0 and st["waiting"] == 0 and st["free_slots"] == 6
    finally:
        srv.close()
        eng.close()
