"""Writes tests/golden/*.npz by RUNNING the reference implementation (package `shapequant`,
imported read-only from a checkout given by --ref). The fixtures pin the CPU oracle
(oracle/cbl_oracle.py) and, through it, the CUDA kernels.

    python tests/golden/make_golden.py --ref /path/to/QuantExperiments

Every array is produced by reference code; inputs come from seeded CPU torch generators in the
style of the reference's own test helpers (tests/test_kernels.py:14-24, tests/test_packed.py:11-15).
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    from shapequant import codebook as cb
    from shapequant import masks as mk
    from shapequant import packed

    # 1. bit stream: round trips for the reference's own bit widths (tests/test_packed.py:18-24) + 12
    out = {}
    for bits in (1, 8, 10, 12, 13, 14, 16):
        g = torch.Generator().manual_seed(bits)
        v = torch.randint(0, 1 << bits, (70, 37), generator=g)
        w = packed.pack_bits(v, bits)
        assert torch.equal(packed.unpack_bits(w, bits, 37), v)
        out[f"vals_{bits}"] = v.numpy().astype(np.int32)
        out[f"words_{bits}"] = w.numpy()
    # layout known answers (tests/test_packed.py:27-35), produced by the reference packer
    out["kat_a_vals"] = np.array([[1, 1, 0, 0]], dtype=np.int32)
    out["kat_a_words"] = packed.pack_bits(torch.tensor([[1, 1, 0, 0]]), 10).numpy()
    out["kat_b_vals"] = np.array([[0, 0, 0, 0b1111111111]], dtype=np.int32)
    out["kat_b_words"] = packed.pack_bits(torch.tensor([[0, 0, 0, 0b1111111111]]), 10).numpy()
    np.savez_compressed(HERE / "bits.npz", **out)

    # 2. seeded column orders + CRC (shapequant/masks.py:334-342, packed.py:93-94)
    out = {}
    cases = [(64, 4, 7), (64, 1, 3), (896, 16, 1), (3584, 16, 1), (5120, 16, 12345)]
    out["cases"] = np.array(cases, dtype=np.int64)
    for C, M, seed in cases:
        p = mk.seeded_perms(C, M, torch.Generator(device="cpu").manual_seed(seed))
        out[f"crc_{C}_{M}_{seed}"] = np.array([packed.perm_crc(p)], dtype=np.int64)
        if C <= 896:
            out[f"perms_{C}_{M}_{seed}"] = p.numpy().astype(np.int32)
        else:   # large ones: first/last rows only (the CRC covers the rest)
            out[f"perms_{C}_{M}_{seed}_row1"] = p[1].numpy().astype(np.int32)
            out[f"perms_{C}_{M}_{seed}_rowlast"] = p[-1].numpy().astype(np.int32)
    np.savez_compressed(HERE / "perms.npz", **out)

    # 3. decode_tensors over the (G, M, K, d) grid of tests/test_packed.py:38 plus the benchmark
    #    format (d = 8, K = 4096) with and without column orders
    out = {}
    grid = [(1, 1, 64, 4), (4, 1, 32, 4), (1, 8, 64, 4), (4, 8, 16, 4), (1, 1, 4096, 8), (1, 16, 4096, 8),
            (2, 4, 256, 8)]
    out["grid"] = np.array(grid, dtype=np.int64)
    for i, (G, M, K, d) in enumerate(grid):
        g = torch.Generator().manual_seed(100 + i)
        R, C = (24, 64) if K < 4096 else (20, 896)
        bits = K.bit_length() - 1
        tags = torch.randint(0, K, (R, C // d), generator=g)
        table = (torch.randn(G * K, d, generator=g) * 0.7).half()
        rs = (torch.rand(R, generator=g) * 0.03 + 1e-3).half()
        rb = torch.randint(0, G, (R,), generator=g).to(torch.uint8) if G > 1 else None
        rm = torch.randint(0, M, (R,), generator=g).to(torch.uint8) if M > 1 else None
        seed = 1000 + i
        perms = mk.seeded_perms(C, M, torch.Generator(device="cpu").manual_seed(seed))
        words = packed.pack_bits(tags, bits)
        w = packed.decode_tensors(packed.unpack_bits(words, bits, C // d), table, rs, rb, rm, perms, K)
        out[f"words_{i}"] = words.numpy()
        out[f"table_{i}"] = table.numpy()
        out[f"rs_{i}"] = rs.numpy()
        if rb is not None:
            out[f"rb_{i}"] = rb.numpy()
        if rm is not None:
            out[f"rm_{i}"] = rm.numpy()
        out[f"seed_{i}"] = np.array([seed, R, C], dtype=np.int64)
        out[f"w_{i}"] = w.numpy()
    np.savez_compressed(HERE / "decode.npz", **out)

    # 4. CodebookMatrix decode with padding and a column permutation (shapequant/codebook.py:277-289)
    out = {}
    g = torch.Generator().manual_seed(5)
    w = torch.randn(16, 100, generator=g) * (torch.rand(16, 1, generator=g) + 0.2)   # 100 % 8 != 0
    perm = torch.randperm(100, generator=torch.Generator().manual_seed(0))
    cm, _ = cb.compress(w, 8, 64, iters=3, max_fit_chunks=10_000, seed=3, perm=perm)
    out.update(idx=cm.idx.numpy().astype(np.int32), codebook=cm.codebook.numpy(), row_scale=cm.row_scale.numpy(),
               pad=np.array([cm.pad, cm.cols], dtype=np.int64), perm=perm.numpy().astype(np.int32),
               decoded=cb.decode(cm).numpy())
    # 5. assign (shapequant/codebook.py:58-71): nearest codeword of random chunks
    x = torch.randn(300, 8, generator=g)
    book = torch.randn(256, 8, generator=g).half()
    i, e = cb.assign(x, book)
    out.update(assign_x=x.numpy(), assign_book=book.numpy(), assign_idx=i.numpy().astype(np.int32), assign_err=e.numpy())
    np.savez_compressed(HERE / "codebook.npz", **out)

    # 6. two summed d = 8 books: the dense formula of tests/test_proto_runs.py:135-144 evaluated by
    #    torch exactly as written there, and masks._decode_multi (shapequant/masks.py:193-200)
    out = {}
    g = torch.Generator().manual_seed(0)
    R, C, K = 24, 512, 4096
    A = (torch.randn(K, 8, generator=g) * 0.5).half()
    B = (torch.randn(K, 8, generator=g) * 0.3).half()
    ta = torch.randint(0, K, (R, C // 8), generator=g)
    tb = torch.randint(0, K, (R, C // 8), generator=g)
    rs = (torch.rand(R, generator=g) * 0.02 + 0.01).half()
    dense = ((A.float()[ta] + B.float()[tb]).reshape(R, C) * rs.float()[:, None])
    idx = torch.arange(C)[None].expand(R, C)
    multi = mk._decode_multi([A, B], [ta.reshape(-1), tb.reshape(-1)], R, C, rs.float(), idx, None, 1)
    assert torch.equal(dense, multi)
    out.update(A=A.numpy(), B=B.numpy(), ta=ta.numpy().astype(np.int32), tb=tb.numpy().astype(np.int32),
               rs=rs.numpy(), dense=dense.numpy())
    np.savez_compressed(HERE / "additive.npz", **out)

    # 7. the packed linear's outputs: PackedLinear.dense() and the fp32 product the reference's GPU tests
    #    compare against (tests/test_kernels.py:30-35), plus stored_bytes (kernels/gemv.py:172-175)
    from shapequant.kernels.gemv import PackedLinear
    out = {}
    g = torch.Generator().manual_seed(0)
    R, C, K, d, M = 48, 896, 4096, 8, 16
    tags = torch.randint(0, K, (R, C // d), generator=g)
    table = torch.randn(K, d, generator=g).half()
    rs = (torch.rand(R, generator=g) * 0.02 + 0.01).half()
    rm = torch.randint(0, M, (R,), generator=g)
    perms = mk.seeded_perms(C, M, torch.Generator().manual_seed(1))
    lin = PackedLinear(packed.pack_bits(tags, 12), table, rs, None, rm, perms, K, d)
    x = torch.randn(3, C, generator=g).bfloat16()
    dense = lin.dense()
    y = x.float() @ dense.T
    out.update(words=lin.words.numpy(), table=table.numpy(), rs=rs.numpy(), rm=rm.numpy().astype(np.uint8),
               x=x.float().numpy(), y=y.numpy(), dense_sum=np.array([dense.double().sum().item()]),
               stored_bytes=np.array([lin.stored_bytes()], dtype=np.int64))
    np.savez_compressed(HERE / "linear.npz", **out)

    # 8. block-32 formats of the embedding and the head (packed.py:33-41, 134-160; kernels/proto_formats.py:464-471):
    #    4-bit embedding pack + row decode, 8-bit head pack + row decode, incl. an all-zero block and an outlier block
    from shapequant.kernels import proto_formats as pfm
    out = {}
    g = torch.Generator().manual_seed(0)
    w = torch.randn(24, 128, generator=g) * 0.02
    w[3, 32:64] = 0.0
    w[5, 7] = 1.5
    w = w.bfloat16().float()
    q4, s4 = packed.q4_embed_pack(w)
    ids = torch.tensor([0, 3, 5, 23, 3])
    q8, s8, deq8 = pfm.q8_pack(w)
    out.update(w=w.numpy(), q4=q4.numpy(), s4=s4.numpy(), ids=ids.numpy(), rows4=packed.q4_embed_rows(q4, s4, ids).numpy(),
               q8=q8.numpy(), s8=s8.numpy(), deq8=deq8.numpy(), rows8=packed.q8_rows(q8, s8, 2, 9).numpy())
    np.savez_compressed(HERE / "blockq.npz", **out)

    # 9. the snap of compress() (shapequant/codebook.py:237-274) with and without weights, and the weighted branch of
    #    assign (codebook.py:52-55): matrix, weights and the fitted codebook in, tags / row scales / errors out
    out = {}
    g = torch.Generator().manual_seed(9)
    w = torch.randn(48, 200, generator=g) * (torch.rand(48, 1, generator=g) + 0.1)
    h = torch.rand(200, generator=g) + 0.05
    perm = torch.randperm(200, generator=torch.Generator().manual_seed(1))
    for tag, kw in (("plain", {}), ("weighted", dict(col_weight=h, row_weighted=True, perm=perm))):
        cm, stats = cb.compress(w, 8, 256, iters=3, max_fit_chunks=10_000, seed=4, **kw)
        out.update({f"{tag}_idx": cm.idx.numpy().astype(np.int32), f"{tag}_codebook": cm.codebook.numpy(),
                    f"{tag}_row_scale": cm.row_scale.numpy(), f"{tag}_mse": np.array([stats["normalized_chunk_mse"]], dtype=np.float64)})
    x = torch.randn(500, 8, generator=g)
    wt = torch.rand(500, 8, generator=g) * 2
    wt[7] = 0.0
    book = torch.randn(4096, 8, generator=g).half()
    i, e = cb.assign(x, book, wt=wt)
    i0, e0 = cb.assign(x, book)
    out.update(w=w.numpy(), h=h.numpy(), perm=perm.numpy().astype(np.int32), x=x.numpy(), wt=wt.numpy(), book=book.numpy(),
               widx=i.numpy().astype(np.int32), werr=e.numpy(), idx=i0.numpy().astype(np.int32), err=e0.numpy())
    np.savez_compressed(HERE / "snap.npz", **out)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
