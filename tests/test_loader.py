"""Packed file -> device pipeline: exact-size arena, streamed copies, kernel layouts built in place, per-rank shards,
pooling of matrices that were built one by one. The loaded matrices must decode and multiply exactly like matrices
built tensor by tensor from the same file."""
import numpy as np
import pytest
import torch

from oracle import cbl_oracle as orc


def _file(tmp_path, specs, seed=0):
    from quantexperiments_b200 import packed
    g = torch.Generator().manual_seed(seed)
    mats, raw = {}, {}
    for name, (R, C, K, d, G, M) in specs.items():
        tags = torch.randint(0, K, (R, C // d), generator=g)
        table = torch.randn(G * K, d, generator=g).half()
        rs = (torch.rand(R, generator=g) + 0.1).half()
        rb = torch.randint(0, G, (R,), generator=g) if G > 1 else None
        rm = torch.randint(0, M, (R,), generator=g) if M > 1 else None
        mats[name] = packed.pack_matrix(tags, table, rs, d=d, K=K, G=G, M=M, seed=7, row_book=rb, row_mask=rm)
        raw[name] = (tags, table, rs, rb, rm)
    packed.save(tmp_path / "m.safetensors", mats, base_model="test/base")
    return tmp_path / "m.safetensors", raw


SPECS = {"a.q": (256, 896, 4096, 8, 1, 1), "a.gate": (640, 1024, 4096, 8, 1, 1), "b.masks": (100, 264, 4096, 8, 1, 4),
         "c.small_book": (33, 64, 256, 4, 2, 1)}


def test_plan_is_computed_from_metadata_alone(tmp_path):
    from quantexperiments_b200 import loader, packed
    path, _ = _file(tmp_path, SPECS)
    pf = packed.PackedFile(path)
    plan = loader.plan_arena(pf, layouts=("l8", "x16", "t16"))
    assert set(plan) == set(SPECS)
    assert plan["a.q"]["tags"] == 256 * (896 // 8 * 12 // 32) * 4 and plan["a.q"]["table"] == 65536 and plan["a.q"]["row_scale"] == 512
    assert {"l8", "x16", "t16"} <= set(plan["a.q"])
    # four column orders: the batch-1 layout groups the rows by order (each order padded to 32 row positions), the
    # activation-stationary layout needs a single order
    assert "l8" in plan["b.masks"] and "x16" not in plan["b.masks"] and "t16" in plan["b.masks"] and "perms" in plan["b.masks"]
    assert plan["b.masks"]["l8"] >= 5 * 3 * 128 * 4 + 65536 + 16
    assert not {"l8", "x16", "t16"} & set(plan["c.small_book"]) and "row_book" in plan["c.small_book"]
    assert all(v % loader.ALIGN == 0 for p in plan.values() for v in p.values())
    half = loader.plan_arena(pf, ["a.gate"], layouts=("l8",), rank=1, world=2, kinds={"a.gate": "col"})
    assert half["a.gate"]["tags"] == plan["a.gate"]["tags"] // 2
    with pytest.raises(ValueError):
        loader.plan_arena(pf, ["a.q"], layouts=("tiles",))


@pytest.mark.gpu
def test_streamed_load_matches_matrices_built_one_by_one(tmp_path):
    from quantexperiments_b200 import loader, packed
    from quantexperiments_b200.linear import PackedLinear
    path, raw = _file(tmp_path, SPECS)
    pf = packed.PackedFile(path)
    lins = loader.load_linears(path, layouts=("l8", "x16", "t16"))
    assert list(lins) == list(SPECS)
    plan = loader.plan_arena(pf, layouts=("l8", "x16", "t16"))
    assert lins.stats["arena_bytes"] == sum(sum(p.values()) for p in plan.values()) == lins.arena.off
    lo, hi = lins.arena.buf.data_ptr(), lins.arena.buf.data_ptr() + lins.arena.buf.numel()
    g = torch.Generator(device="cuda").manual_seed(1)
    for name, (R, C, K, d, G, M) in SPECS.items():
        lin = lins[name]
        tags, table, rs, rb, rm = raw[name]
        ref = orc.decode_tensors(tags.numpy(), table.numpy(), rs.numpy(), None if rb is None else rb.numpy(),
                                 None if rm is None else rm.numpy(), orc.seeded_perms(C, M, 7), K)
        assert np.array_equal(lin.dense().cpu().numpy(), ref), name
        for t in (lin.dm.tags, lin.dm.table, lin.dm.row_scale):
            assert lo <= t.data_ptr() < hi and t.data_ptr() % loader.ALIGN == 0
        if d != 8:
            continue
        for lay in (lin._l8, lin._t16, getattr(lin, "_x16", None)):
            if lay is not None:
                assert lo <= lay.words.data_ptr() < hi
        assert lin._t16 is not None and (M > 1 or (lin._l8 is not None and lin._x16 is not None))
        one = PackedLinear.from_packed(pf, name)
        for n in (1, 5, 12, 40, 100):
            x = torch.randn(n, C, device="cuda", generator=g).bfloat16()
            y, y1 = lin(x), one(x)
            assert orc.max_rel_err(y.float().cpu().numpy(), (x.float() @ torch.from_numpy(ref).cuda().T).cpu().numpy()) < 1e-2
            assert (y.float() - y1.float()).abs().max() <= 2e-2 * y1.float().abs().max()


@pytest.mark.gpu
def test_rank_shards_and_pooling(tmp_path):
    from quantexperiments_b200 import loader, packed
    from quantexperiments_b200.linear import PackedLinear
    path, raw = _file(tmp_path, SPECS)
    pf = packed.PackedFile(path)
    kinds = {"a.q": "col", "a.gate": "row"}
    full = {n: PackedLinear.from_packed(pf, n).dense() for n in kinds}
    for rank in range(2):
        lins = loader.load_linears(pf, list(kinds), layouts=("l8",), rank=rank, world=2, kinds=kinds)
        assert torch.equal(lins["a.q"].dense(), full["a.q"][rank * 128:(rank + 1) * 128])
        assert torch.equal(lins["a.gate"].dense(), full["a.gate"][:, rank * 512:(rank + 1) * 512])
        x = torch.randn(512, device="cuda").bfloat16()
        y = lins["a.gate"](x[None])[0]
        ref = full["a.gate"][:, rank * 512:(rank + 1) * 512] @ x.float()
        assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    # an input shard of a matrix with several column orders keeps orders that name positions of the full activation
    # vector: the ranks' partial products (1, 5 and 100 tokens: table lookups, row tiles, wide decode + GEMM) add up
    masks_full = PackedLinear.from_packed(pf, "b.masks")
    Cm = masks_full.C
    for T in (1, 5, 100):
        xm = torch.randn(T, Cm, device="cuda").bfloat16()
        want = xm.float() @ masks_full.dense().T
        got = torch.zeros_like(want)
        for rank in range(3):                            # 33 chunks: three ranks of 11
            sh = loader.load_linears(pf, ["b.masks"], rank=rank, world=3, kinds={"b.masks": "row"})["b.masks"]
            assert sh.wide and sh.in_features == Cm and sh.C < Cm
            y = torch.empty(T, sh.R, device="cuda", dtype=torch.float32)
            got += sh.forward_into(xm, y)
            with pytest.raises(ValueError):
                sh.dense()
        assert (got - want).abs().max() <= 2e-3 * want.abs().max(), T
    # matrices built tensor by tensor, then pooled: same answers, new addresses inside one buffer, second call is a no-op
    built = [PackedLinear.from_packed(pf, n) for n in ("a.q", "a.gate", "b.masks")]
    x = torch.randn(1, 896, device="cuda").bfloat16()
    before = built[0](x).clone()
    old = built[0].l8.words.data_ptr()
    n = loader.pool_layouts(built)
    assert n > 0 and built[0].l8.words.data_ptr() != old
    assert torch.equal(built[0](x), before) or (built[0](x).float() - before.float()).abs().max() <= 1e-2 * before.float().abs().max()
    assert torch.equal(built[2].dense(), PackedLinear.from_packed(pf, "b.masks").dense())
    assert loader.pool_layouts(built) == 0
