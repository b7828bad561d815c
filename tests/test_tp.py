"""Tensor-parallel sharding: host-side index arithmetic on CPU ranks (gloo, world size 2) and the
sharded kernels on one GPU (ranks emulated one after another)."""
import os
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import cbl_oracle as orc
from quantexperiments_b200 import tp


def _file_tensors(m):
    t = {"tags": torch.from_numpy(m["words"][0]), "table": torch.from_numpy(m["table"][0]), "row_scale": torch.from_numpy(m["row_scale"])}
    if m["books"] == 2:
        t["tags2"], t["table2"] = torch.from_numpy(m["words"][1]), torch.from_numpy(m["table"][1])
    if m["row_mask"] is not None:
        t["row_mask"] = torch.from_numpy(m["row_mask"])
    meta = {"R": m["R"], "C": m["C"], "d": m["d"], "K": m["K"], "G": 1, "M": m["M"]}
    return t, meta, torch.from_numpy(m["perms"])


def _oracle_decode(t, meta, perms_global, c0=0):
    """fp32 decode of a shard by the oracle; a column shard of a matrix with column orders is returned
    in the shard's own chunk order (its activations are gathered through perms_global[:, c0:c1])."""
    bits = int(meta["K"]).bit_length() - 1
    nch = meta["C"] // meta["d"]
    tags = orc.unpack_bits(t["tags"].numpy(), bits, nch)
    ident = np.arange(meta["C"])[None]
    if "tags2" in t:
        tags2 = orc.unpack_bits(t["tags2"].numpy(), bits, nch)
        return orc.additive_decode(t["table"].numpy(), t["table2"].numpy(), tags, tags2, t["row_scale"].numpy())
    return orc.decode_tensors(tags, t["table"].numpy(), t["row_scale"].numpy(), None, None, ident, meta["K"])


def _rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for books, M in ((1, 1), (2, 1), (1, 4)):
            m = orc.synth_matrix(32, 768, seed=5 + books + M, books=books, M=M)
            t, meta, perms = _file_tensors(m)
            wfull = orc.synth_decode(m)
            x = torch.randn(3, 768, generator=torch.Generator().manual_seed(1)).bfloat16().float()
            yfull = orc.linear_ref(x.numpy(), wfull)
            # column-parallel: rows split, outputs concatenated by all_gather
            r0, r1 = tp.row_range(meta["R"], rank, world)
            ts, ms = tp.shard_rows(t, meta, r0, r1)
            assert ts["tags"].shape[0] == r1 - r0 and ms["R"] == r1 - r0
            y_loc = torch.from_numpy(yfull[:, r0:r1].copy())
            parts = [torch.empty_like(y_loc) for _ in range(world)]
            dist.all_gather(parts, y_loc)
            assert np.allclose(torch.cat(parts, 1).numpy(), yfull)
            if M == 1:
                w_loc = _oracle_decode(ts, ms, perms)
                assert np.array_equal(w_loc, wfull[r0:r1])
            # row-parallel: columns split at chunk boundaries, partial products summed by all_reduce
            c0, c1 = tp.col_range(meta["C"], meta["d"], rank, world)
            ts, ms, ps = tp.shard_cols(t, meta, c0, c1, perms if M > 1 else None)
            assert ms["C"] == c1 - c0 and ts["tags"].shape[1] == orc.words_per_row((c1 - c0) // 8, 12)
            u_loc = _oracle_decode(ts, ms, perms)            # chunk order of the shard
            if M == 1:
                assert np.array_equal(u_loc, wfull[:, c0:c1])
                part = orc.linear_ref(x.numpy()[:, c0:c1], u_loc)
            else:
                # y[b, r] = sum_c u[r, c] * x[b, perms[mask[r]][c0 + c]]: gather the full x per row's order
                rm = t["row_mask"].numpy().astype(np.int64)
                xg = x.numpy()[:, ps.numpy()[rm]]            # [B, R, Cs]
                part = np.einsum("brc,rc->br", xg, u_loc).astype(np.float32)
            y = torch.from_numpy(part.copy())
            dist.all_reduce(y)
            assert orc.max_rel_err(y.numpy(), yfull) < 1e-5, (books, M)
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_sharding_on_two_cpu_ranks(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_unaligned_column_ranges_are_repacked():
    m = orc.synth_matrix(6, 8 * 10, seed=2)          # 10 chunks of 12 bits: ranges not word aligned
    t, meta, _ = _file_tensors(m)
    ts, ms, _ = tp.shard_cols(t, meta, 24, 56)       # chunks 3..6
    tags = orc.unpack_bits(ts["tags"].numpy(), 12, 4)
    assert np.array_equal(tags, m["tags"][0][:, 3:7])
    with pytest.raises(ValueError):
        tp.shard_cols(t, meta, 4, 16)
    with pytest.raises(ValueError):
        tp.row_range(10, 0, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("books,M", [(1, 1), (2, 1), (1, 16), (2, 16)])
def test_sharded_linears_on_one_gpu(world, books, M):
    R, C = 2304 * 2 if M == 1 else 256, 1024
    m = orc.synth_matrix(R, C, seed=world + books + M, books=books, M=M)
    t, meta, perms = _file_tensors(m)
    wfull = orc.synth_decode(m)
    for B in (1, 5, 80 if M == 1 else 150):          # one token: the table-lookup kernel; 150 tokens with column orders: wide decode + tensor-core GEMM
        x = torch.randn(B, C, generator=torch.Generator().manual_seed(B)).bfloat16()
        yfull = orc.linear_ref(x.float().numpy(), wfull)
        cols = [tp.ColumnParallelLinear(t, meta, perms if M > 1 else None, r, world)(x.cuda()) for r in range(world)]
        ycat = torch.cat(cols, 1).float().cpu().numpy()
        assert orc.max_rel_err(ycat, yfull) < 1e-3 + 2.0 ** -8
        acc = torch.zeros(B, R, device="cuda")
        for r in range(world):
            rp = tp.RowParallelLinear(t, meta, perms if M > 1 else None, r, world)
            xin = x.cuda() if M > 1 else x[:, rp.c0:rp.c1].contiguous().cuda()
            part = rp.partial(xin)
            assert part.dtype == torch.float32
            acc += part
        tol = 1e-3 if (B <= 64 or books == 1) else 1e-2      # >64 tokens with two books: the sum of the two codewords is rounded to 16 bits before the product
        assert orc.max_rel_err(acc.cpu().numpy(), yfull) < tol, (world, books, M, B)


def test_vllm_plugin_registers_the_method_and_pickles():
    pytest.importorskip("vllm")
    import pickle
    from quantexperiments_b200.vllm_ext import plugin
    cfg = plugin.ShapeQuantConfig.from_config({"packed_file": "x.packed", "bmax": 32, "layout": "tile", "tune": True})
    assert cfg.get_name() == "shapequant" and cfg.bmax == 32 and cfg.get_min_capability() == 100
    assert pickle.loads(pickle.dumps(cfg)).packed_file == "x.packed"
    with pytest.raises(ValueError):
        plugin.ShapeQuantConfig("x.packed", embed_head="packed")
    from quantexperiments_b200.vllm_ext import core
    names = {"model.layers.3.self_attn.q_proj", "model.layers.3.self_attn.k_proj", "model.layers.3.self_attn.v_proj"}
    assert core.packed_pieces("model.layers.3.self_attn.qkv_proj", names) == sorted(names, key=lambda n: "qkv".index(n[-6]))
    assert core.packed_pieces("model.layers.3.mlp.down_proj", names) is None
    with pytest.raises(ValueError):
        core.packed_pieces("model.layers.3.self_attn.qkv_proj", {"model.layers.3.self_attn.q_proj"})


@pytest.mark.gpu
def test_vllm_layer_shards_under_tensor_parallelism(tmp_path):
    pytest.importorskip("vllm")
    from quantexperiments_b200 import packed
    from quantexperiments_b200.vllm_ext import plugin
    g = torch.Generator().manual_seed(0)
    K, d = 4096, 8
    mats, ref = {}, {}
    for name, R, C in (("model.layers.0.self_attn.q_proj", 2048, 512), ("model.layers.0.self_attn.k_proj", 256, 512),
                       ("model.layers.0.self_attn.v_proj", 256, 512), ("model.layers.0.self_attn.o_proj", 512, 2048)):
        tags = torch.randint(0, K, (R, C // d), generator=g)
        table = torch.randn(K, d, generator=g).half()
        rs = (torch.rand(R, generator=g) * 0.02 + 0.01).half()
        mats[name] = packed.pack_matrix(tags, table, rs, d=d, K=K, seed=1)
        ref[name] = orc.decode_tensors(tags.numpy(), table.numpy(), rs.numpy(), None, None, np.arange(C)[None], K)
    packed.save(tmp_path / "m.packed", mats, base_model="test/base")
    pf = packed.PackedFile(tmp_path / "m.packed")
    world = 2
    qkv = [n for n in mats if n.endswith(("q_proj", "k_proj", "v_proj"))]
    x = torch.randn(5, 512, generator=g).bfloat16()
    outs = [plugin.build_shards(pf, qkv, input_size_per_partition=512, output_partition_sizes=[1024, 128, 128], input_size=512,
                                output_size=2560, rank=r, world=world, device="cuda", bmax=32).forward(x.cuda()).float().cpu()
            for r in range(world)]
    for i, (name, off, n) in enumerate(zip(qkv, (0, 1024, 1152), (1024, 128, 128))):
        full = orc.linear_ref(x.float().numpy(), ref[name])
        got = torch.cat([o[:, off:off + n] for o in outs], 1).numpy()
        assert orc.max_rel_err(got, full) < 1e-3 + 2.0 ** -8, name
    xo = torch.randn(5, 2048, generator=g).bfloat16()
    acc = 0
    for r in range(world):
        ps = plugin.build_shards(pf, ["model.layers.0.self_attn.o_proj"], input_size_per_partition=1024, output_partition_sizes=[512],
                                 input_size=2048, output_size=512, rank=r, world=world, device="cuda", bmax=32)
        acc = acc + ps.forward(xo[:, r * 1024:(r + 1) * 1024].contiguous().cuda().float()).cpu()
    assert orc.max_rel_err(acc.numpy(), orc.linear_ref(xo.float().numpy(), ref["model.layers.0.self_attn.o_proj"])) < 1e-3 + 2.0 ** -7


def _peer_rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        arena = tp.PeerArena(32 << 20)
        for R, C, books, M in ((3584, 1024, 1, 1), (2304, 4096, 1, 1), (2560, 1024, 2, 16)):
            m = orc.synth_matrix(R, C, seed=R + C, books=books, M=M)
            t, meta, perms = _file_tensors(m)
            wfull = orc.synth_decode(m)
            rp = tp.RowParallelLinear(t, meta, perms if M > 1 else None, rank, world)
            rp.attach(arena)
            g = torch.Generator().manual_seed(1)
            for it in range(3):
                x = torch.randn(C, generator=g).bfloat16()
                xin = x.cuda() if M > 1 else x[rp.c0:rp.c1].contiguous().cuda()      # column orders index the full vector
                y = rp.forward_fused(xin, torch.empty(R, device="cuda"))
                assert rp.fused.status()
                yref = orc.linear_ref(x.float().numpy()[None], wfull)[0]
                assert orc.max_rel_err(y.cpu().numpy(), yref) < 1e-3
                ys = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(ys, y)
                assert all(torch.equal(ys[0], v) for v in ys)        # rank-ordered sum: identical bits everywhere
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.gpu
def test_fused_row_parallel_product_over_peer_memory(tmp_path):
    """Needs two GPUs in the box: two processes, partial sums exchanged through peer pointers by the finish kernel."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29500 + (os.getpid() % 2000) + 7
    mp.spawn(_peer_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
