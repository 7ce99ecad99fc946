"""The device-side expert-parallel plan (static shapes, no host synchronisation) checked on CPU: every rank
builds its plan from all ranks' routing tables; emulating dispatch / expert compute / combine with the plan
arrays must reproduce the dense mixture-of-experts result."""
import torch

from axolotl_b200.parallel.ep import ExpertParallelGroup


def _group(rank, world, E, cf=None):
    g = ExpertParallelGroup.__new__(ExpertParallelGroup)
    g.device, g.size, g.rank, g.E, g.E_local = torch.device("cpu"), world, rank, E, E // world
    g.fused, g.dedup, g.overflow = False, True, None
    g.capacity_factor = cf if cf is not None else float(world)
    return g


def _run(world, E, T, k, H, cf=None, seed=0):
    torch.manual_seed(seed)
    xs = [torch.randn(T, H) for _ in range(world)]
    idxs = [torch.stack([torch.randperm(E)[:k] for _ in range(T)]) for _ in range(world)]
    ws = [torch.rand(T, k) for _ in range(world)]
    We = torch.randn(E, H, H) * 0.1                       # expert e: y = x @ We[e]
    all_idx = torch.cat([i.reshape(-1) for i in idxs]).to(torch.int32)
    all_w = torch.cat([w.reshape(-1) for w in ws])
    outs = [torch.zeros(T, H) for _ in range(world)]
    dws = [torch.zeros(T * k) for _ in range(world)]
    groups = []
    for r in range(world):
        g = _group(r, world, E, cf)
        groups.append(g)
        p = g._plan_from_tables(all_idx, all_w, idxs[r], H)
        lay = p.lay
        nb = int(lay.n_blocks)
        assert nb <= lay.max_blocks
        # DISPATCH: padded rows pull their token from the source rank
        rows = torch.zeros(lay.max_rows, H)
        for i in range(lay.max_rows):
            sr = int(p.pad_src_rank[i])
            if sr >= 0:
                assert int(p.pad_src_row[i]) == int(p.pad_src_slot[i]) // k
                rows[i] = xs[sr][int(p.pad_src_row[i])]
                if g.dedup:
                    assert int(p.need[sr * T + int(p.pad_src_row[i])]) == 1
        # experts by block
        ys = torch.zeros_like(rows)
        for b in range(nb):
            e = int(lay.blk_expert[b]) + r * g.E_local
            ys[b * 128:(b + 1) * 128] = rows[b * 128:(b + 1) * 128] @ We[e]
        # every used row sits inside the segment of its expert
        for i in range(lay.max_rows):
            if int(p.pad_src_rank[i]) >= 0:
                e_loc = int(all_idx[int(p.pad_src_rank[i]) * T * k + int(p.pad_src_slot[i])]) - r * g.E_local
                assert int(lay.seg_start[e_loc]) <= i < int(lay.seg_start[e_loc]) + int(lay.seg_rows[e_loc])
                assert i < nb * 128
        # COMBINE: weighted rows back to (source rank, token); per-slot scalars back to (source rank, slot)
        for i in range(lay.max_rows):
            sr = int(p.pad_src_rank[i])
            if sr >= 0:
                outs[sr][int(p.pad_src_row[i])] += float(p.pad_weight[i]) * ys[i]
                dws[sr][int(p.pad_src_slot[i])] += 1.0
        if g.dedup:
            dest = idxs[r].reshape(-1) // g.E_local
            for s_ in range(T * k):
                assert int(p.sent[int(dest[s_]) * T + s_ // k]) == 1
    for r in range(world):
        ref = torch.zeros(T, H)
        for t in range(T):
            for j in range(k):
                ref[t] += ws[r][t, j] * (xs[r][t] @ We[int(idxs[r][t, j])])
        assert torch.allclose(outs[r], ref, atol=1e-4), r
        assert torch.equal(dws[r], torch.ones(T * k))          # every slot was computed exactly once
    return groups


def test_device_plan_reproduces_dense_moe_world4():
    groups = _run(world=4, E=8, T=37, k=2, H=16)
    assert all(int(g.overflow) == 0 for g in groups)


def test_device_plan_single_rank_and_uneven_load():
    _run(world=1, E=4, T=50, k=3, H=8)
    _run(world=2, E=6, T=200, k=1, H=8, seed=3)


def test_device_plan_flags_overflow_instead_of_failing_silently():
    torch.manual_seed(1)
    world, E, T, k = 4, 8, 64, 2
    g = _group(0, world, E, cf=0.25)                      # far too small on purpose
    all_idx = torch.randint(0, 2, (world * T * k,), dtype=torch.int32)   # everything goes to rank 0's experts
    p = g._plan_from_tables(all_idx, torch.ones(world * T * k), all_idx[: T * k].reshape(T, k), 8)
    assert int(g.overflow) == 1 and int(p.lay.n_blocks) <= p.lay.max_blocks
    assert g.take_overflow() and g.capacity_factor == 0.375 and int(g.overflow) == 0 and not g.take_overflow()
    g.overflow += 1
    try:
        g.check_overflow()
        raise AssertionError("no error raised")
    except RuntimeError as e:
        assert "AXB_EP_CAPACITY" in str(e)
