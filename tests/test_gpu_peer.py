"""The peer exchange kernels with every rank played by one process on one GPU (one launch hosts
all ranks' CTAs, so the waits between ranks resolve inside a single resident grid), and the
expert window of the device-routed plan.  The same kernels run one rank per process over
NVLink in tests/test_gpu_tp.py::test_two_ranks_over_peer_memory when two GPUs are visible."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import trellis_ref as ref
from strix_trellis_b200 import native as N, synthetic
from strix_trellis_b200.peer import PeerGroup
from strix_trellis_b200.runtime import Context, MoePlan
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sum_is_rank_ordered_and_identical_on_every_rank(ctx, world):
    g = PeerGroup(ctx, 4 << 20, rank=0, world=world, local_ranks=world)
    count = 8 * 4096
    region = g.reserve(world * count * 8)
    rng = np.random.default_rng(70 + world)
    for turn in range(5):  # parities alternate; regions are reused
        parts = (rng.normal(size=(world, count)) * 10.0 ** rng.integers(-3, 4, (world, count))).astype(np.float32)
        rows = [dev(parts[r].copy()) for r in range(world)]
        g.sum_rows(rows, region)
        torch.cuda.synchronize()
        want = np.zeros(count, np.float32)
        for r in range(world):
            want = want + parts[r]
        for r in range(world):
            assert host(rows[r]).tobytes() == want.tobytes(), (turn, r)
    assert ctx.device_status() == 0
    g.close()


@pytest.mark.parametrize("tagged", [False, True])
def test_gather_uneven_column_blocks_and_row_blocks(ctx, tagged):
    world = 4
    g = PeerGroup(ctx, 8 << 20, rank=0, world=world, local_ranks=world)
    rng = np.random.default_rng(5)
    # column blocks of uneven width (an LM head whose block count does not divide by the ranks)
    widths, rows = [384, 256, 256, 128], 3
    col_at = [0, 384, 640, 896]
    region = g.reserve(rows * 1024 * (8 if tagged else 4))
    for turn in range(3):
        blocks = [rng.normal(size=(rows, w)).astype(np.float32) for w in widths]
        outs = [torch.zeros((rows, 1024), device="cuda") for _ in range(world)]
        g.gather([rows] * world, [0] * world,
                 [dict(blocks=[dev(b) for b in blocks], results=outs, widths=widths, col_at=col_at, total_cols=1024,
                       region=region)], tagged=tagged)
        torch.cuda.synchronize()
        want = np.concatenate(blocks, axis=1)
        for r in range(world):
            assert host(outs[r]).tobytes() == want.tobytes(), (turn, r)
    # row blocks of three matrices at once (token rows, route ids, scores); narrow ones are 6 words wide
    per, model, k = 5, 256, 6
    regions = [g.reserve(world * per * w * (8 if tagged else 4)) for w in (model, k, k)]
    xs = [rng.normal(size=(per, model)).astype(np.float32) for _ in range(world)]
    ids = [rng.integers(0, 1000, (per, k)).astype(np.int32) for _ in range(world)]
    sc = [rng.random((per, k)).astype(np.float32) for _ in range(world)]
    res = [[torch.zeros((world * per, w), dtype=t, device="cuda") for _ in range(world)]
           for w, t in ((model, torch.float32), (k, torch.int32), (k, torch.float32))]
    mats = [dict(blocks=[dev(b) for b in src], results=res[m], widths=[w] * world, col_at=[0] * world, total_cols=w,
                 region=regions[m]) for m, (src, w) in enumerate(((xs, model), (ids, k), (sc, k)))]
    g.gather([per] * world, [r * per for r in range(world)], mats, tagged=tagged)
    torch.cuda.synchronize()
    for r in range(world):
        assert host(res[0][r]).tobytes() == np.concatenate(xs).tobytes()
        assert host(res[1][r]).tobytes() == np.concatenate(ids).tobytes()
        assert host(res[2][r]).tobytes() == np.concatenate(sc).tobytes()
    assert ctx.device_status() == 0
    g.close()


def test_routed_rows_reach_the_home_rank(ctx):
    world, per, k, width, experts = 4, 3, 4, 256, 16
    tokens = world * per
    g = PeerGroup(ctx, 8 << 20, rank=0, world=world, local_ranks=world)
    region = g.reserve(per * k * width * 4)
    rng = np.random.default_rng(11)
    ids = np.stack([rng.choice(experts, k, replace=False) for _ in range(tokens)]).astype(np.int32)
    valid = np.ones(tokens, np.int32)
    valid[4] = 0  # an invalid token: nobody sends its rows
    each = [rng.normal(size=(tokens * k, width)).astype(np.float32) for _ in range(world)]  # rank r's rows
    each_d, ids_d, valid_d = [dev(e) for e in each], dev(ids), dev(valid)
    own = experts // world
    # exchange 1 of this group: parity 1
    g.return_routes([e.data_ptr() for e in each_d], [ids_d.data_ptr()] * world, [valid_d.data_ptr()] * world,
                    [r * own for r in range(world)], [own] * world, tokens, per, k, width, region)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    for home in range(world):
        landed = host(g.view(home, region + per * k * width * 4, (per, k, width)))
        for t in range(per):
            token = home * per + t
            if not valid[token]:
                continue
            for s in range(k):
                owner = ids[token, s] // own
                assert landed[t, s].tobytes() == each[owner][token * k + s].tobytes(), (home, t, s)
    g.close()


def test_expert_windows_recombine_to_the_single_rank_block(ctx):
    """Two plans whose banks are the two halves of the expert ids, on the same tokens: the union
    of the rows they compute, combined in slot order, is the single-bank plan's output bit for
    bit; submit() with a window yields that rank's contribution; a row with an id outside the
    id space or a duplicate is invalid on both and comes out NaN."""
    model, inter, n_exp, tokens, top_k = 512, 256, 8, 7, 4
    layers = [dict(gate=synthetic.make_layer(model, inter, 2 + e % 2, 9300 + 3 * e, sigma=0.5),
                   up=synthetic.make_layer(model, inter, 2, 9301 + 3 * e, sigma=0.5),
                   down=synthetic.make_layer(inter, model, 3, 9302 + 3 * e, sigma=0.5)) for e in range(n_exp)]
    ws = [tuple(ctx.prepare(l[k]) for k in ("gate", "up", "down")) for l in layers]
    x = synthetic.make_activations(tokens, model, seed=9311)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=9312)
    ids = ids.astype(np.int64)
    scores[2, 1] = 0.0
    ids[5, 3] = ids[5, 0]      # duplicate id
    ids[6, 2] = n_exp + 3      # outside the id space
    xd, idd, scd = dev(x), dev(ids.astype(np.uint32).view(np.int32)), dev(scores)
    y_full = torch.zeros((tokens, model), device="cuda")
    full = MoePlan(ctx, ws, xd, y_full, idd, scd, device_routed=True)
    full.submit()
    torch.cuda.synchronize()
    want = host(y_full)
    assert np.isnan(want[5]).all() and np.isnan(want[6]).all() and np.isfinite(want[:5]).all()

    halves, rows, contributions = [], torch.zeros((tokens, top_k, model), device="cuda"), []
    for r in range(2):
        y = torch.zeros((tokens, model), device="cuda")
        p = MoePlan(ctx, ws[4 * r:4 * r + 4], xd, y, idd, scd, device_routed=True)
        N.check(ctx.lib.strix_b200_moe_plan_set_window(p.handle, 4 * r, n_exp), "window")
        N.check(ctx.lib.strix_b200_moe_plan_projections(p.handle), "projections")
        each, valid = N.vp(), N.vp()
        N.check(ctx.lib.strix_b200_moe_plan_rows(p.handle, C.byref(each), C.byref(valid)), "rows")
        torch.cuda.synchronize()
        from strix_trellis_b200.peer import _Raw
        mine = torch.as_tensor(_Raw(each.value, tokens * top_k * model * 4), device="cuda").view(torch.float32).view(
            tokens, top_k, model)
        ok = torch.as_tensor(_Raw(valid.value, tokens * 4), device="cuda").view(torch.int32)
        assert host(ok).tolist() == [1, 1, 1, 1, 1, 0, 0]
        owned = torch.from_numpy((ids // 4 == r) & (np.arange(tokens)[:, None] < 5)).cuda()
        rows[owned] = mine[owned]
        p.submit()  # with a window: this rank's contribution
        torch.cuda.synchronize()
        contributions.append(host(y))
        halves.append((p, ok.clone()))
    y = torch.zeros((tokens, model), device="cuda")
    sd = N.stream_desc(torch.cuda.current_stream().cuda_stream)
    N.check(ctx.lib.strix_b200_moe_combine_rows(ctx.handle, rows.data_ptr(), scd.data_ptr(), halves[0][1].data_ptr(),
                                                tokens, top_k, model, y.data_ptr(), model, 1.0, 0.0, C.byref(sd)),
            "combine_rows")
    torch.cuda.synchronize()
    got = host(y)
    assert got[:5].tobytes() == want[:5].tobytes()
    assert np.isnan(got[5:]).all()
    # the two contributions add up to the block within float32 rounding of one add
    np.testing.assert_allclose(contributions[0][:5] + contributions[1][:5], want[:5], rtol=2e-6, atol=1e-6)
    assert ctx.device_status() == 0
    full.close()
    for p, _ in halves:
        p.close()
    for t in ws:
        for w in t:
            w.close()


def test_gather_descriptor_rules(ctx):
    """What the gather refuses: a region that does not fit the arena, a block that sticks out of
    the matrix, and -- for tagged words -- odd widths or a missing result."""
    world = 2
    g = PeerGroup(ctx, 1 << 20, rank=0, world=world, local_ranks=world)
    region = g.reserve(4 * 256 * 8)
    blocks = [torch.zeros((4, 128), device="cuda") for _ in range(world)]
    outs = [torch.zeros((4, 256), device="cuda") for _ in range(world)]
    good = dict(blocks=blocks, results=outs, widths=[128, 128], col_at=[0, 128], total_cols=256, region=region)
    g.gather([4, 4], [0, 0], [good], tagged=True)
    torch.cuda.synchronize()
    bad = [dict(good, region=(1 << 20) + 4096),                 # outside the arena
           dict(good, col_at=[0, 192]),                         # second block sticks out
           dict(good, widths=[127, 128]),                       # odd width with tagged words
           dict(good, results=[None, None])]                    # tagged words are of no use in place
    for spec in bad:
        with pytest.raises(N.StrixError):
            g.gather([4, 4], [0, 0], [spec], tagged=True)
    with pytest.raises(N.StrixError):
        g.set_wait_polls(0)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    g.close()
