"""GPU tests of the encoder side: nearest-codeword assignment (cbl_assign), tag packing (cbl_pack_tags) and the
snap of a weight matrix, against the reference-written fixtures and the CPU oracle. Tags are compared index for
index; where two codewords all but tie in fp32 the kernel may name the other one, so a differing index must lie within
a few fp32 ulps of the exact (float64) minimum."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cbl_oracle as orc

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def _check(x, book, idx, err, ref_idx, ref_err, wt=None, min_agree=0.995):
    idx, err = idx.cpu().numpy(), err.cpu().numpy()
    assert idx.dtype == np.int64 and err.dtype == np.float32
    agree = float((idx == ref_idx).mean()) if idx.size else 1.0
    assert agree >= min_agree, agree
    scale = 1.0 + (np.asarray(x, dtype=np.float64) ** 2 * (1.0 if wt is None else np.asarray(wt, dtype=np.float64))).sum(1)
    assert np.all(orc.assign_margin(x, book, idx, wt) <= 4e-6 * scale)
    assert np.allclose(err, ref_err, rtol=1e-4, atol=2e-5 * scale.max())


def test_assign_matches_reference_fixtures():
    from quantexperiments_b200 import codebook as cb
    z = np.load(G / "codebook.npz")
    i, e = cb.assign(_t(z["assign_x"]).cuda(), _t(z["assign_book"]).cuda())
    _check(z["assign_x"], z["assign_book"], i, e, z["assign_idx"], z["assign_err"])
    z = np.load(G / "snap.npz")
    i, e = cb.assign(_t(z["x"]).cuda(), _t(z["book"]).cuda())
    _check(z["x"], z["book"], i, e, z["idx"], z["err"])
    i, e = cb.assign(_t(z["x"]).cuda(), _t(z["book"]).cuda(), wt=_t(z["wt"]).cuda())
    _check(z["x"], z["book"], i, e, z["widx"], z["werr"], wt=z["wt"])
    assert int(i[7]) == 0 and float(e[7]) == 0.0          # all-zero weights: every codeword ties, the first wins


@pytest.mark.parametrize("n,K", [(1, 1), (5, 5), (2047, 37), (2049, 4096), (70001, 4096)])
@pytest.mark.parametrize("weighted", [False, True])
def test_assign_matches_oracle_on_ragged_sizes(n, K, weighted):
    from quantexperiments_b200 import codebook as cb
    g = torch.Generator().manual_seed(n + K)
    x = torch.randn(n, 8, generator=g)
    book = torch.randn(K, 8, generator=g).half()
    wt = torch.rand(n, 8, generator=g) + 0.01 if weighted else None
    ri, re = orc.assign(x.numpy(), book.numpy(), None if wt is None else wt.numpy())
    i, e = cb.assign(x.cuda(), book.cuda(), wt=None if wt is None else wt.cuda())
    _check(x.numpy(), book.numpy(), i, e, ri, re, wt=None if wt is None else wt.numpy())
    # a 32-bit book gives the same answer as its 16-bit values
    i2, e2 = cb.assign(x.cuda(), book.float().cuda(), wt=None if wt is None else wt.cuda())
    assert torch.equal(i, i2) and torch.equal(e, e2)


def test_assign_exact_codewords_and_first_index_on_ties():
    from quantexperiments_b200 import codebook as cb
    g = torch.Generator().manual_seed(3)
    book = torch.randn(4096, 8, generator=g).half()
    book[100] = book[7]                                    # a duplicate: the first index wins
    pick = torch.randint(0, 4096, (5000,), generator=g)
    pick[pick == 100] = 7
    i, e = cb.assign(book[pick].float().cuda(), book.cuda())
    assert torch.equal(i.cpu(), pick)
    assert float(e.max()) <= 1e-5
    i, e = cb.assign(torch.empty(0, 8).cuda(), book.cuda())
    assert i.numel() == 0 and e.numel() == 0


def test_assign_rejects_unsupported_arguments():
    from quantexperiments_b200 import _lib, codebook as cb
    x = torch.zeros(16, 8, device="cuda")
    book = torch.zeros(5000, 8, device="cuda")
    idx = torch.zeros(16, dtype=torch.int64, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    call = lambda d, K: _lib.lib.cbl_assign(x.data_ptr(), None, 16, d, book.data_ptr(), 0, K, idx.data_ptr(), x.data_ptr(), s)   # noqa: E731
    assert _lib.lib.cbl_assign_max_codewords() == 4096
    assert call(8, 4097) == _lib.EUNSUPPORTED
    assert call(4, 16) == _lib.EUNSUPPORTED
    assert call(8, 0) == _lib.EINVAL
    with pytest.raises(ValueError):
        cb.assign(x, book[:, :4])
    with pytest.raises(ValueError):
        cb.assign(x.cpu(), book.cpu())


def test_pack_bits_matches_reference_streams_bit_for_bit():
    from quantexperiments_b200 import codebook as cb
    z = np.load(G / "bits.npz")
    for bits in (1, 8, 10, 12, 13, 14, 16):
        w = cb.pack_bits(_t(z[f"vals_{bits}"]).cuda(), bits)
        assert w.dtype == torch.int32 and np.array_equal(w.cpu().numpy(), z[f"words_{bits}"]), bits
    g = torch.Generator().manual_seed(1)
    v = torch.randint(0, 4096, (300, 2368), generator=g)
    assert np.array_equal(cb.pack_bits(v.cuda(), 12).cpu().numpy(), orc.pack_bits(v.numpy(), 12))
    with pytest.raises(ValueError):
        cb.pack_bits(torch.full((2, 3), 4096).cuda(), 12)


def test_snap_matches_reference_compress_and_round_trips_through_the_decoder():
    """Matrix + fitted codebook in: the row scales bit for bit, the tags index for index (near-ties aside), then
    pack -> GPU decode equals the oracle's decode of the same tags."""
    from quantexperiments_b200 import codebook as cb
    from quantexperiments_b200.kernels import DeviceMatrix
    z = np.load(G / "snap.npz")
    w = _t(z["w"]).cuda()
    for tag, kw in (("plain", {}), ("weighted", dict(perm=_t(z["perm"]).long().cuda(), col_weight=_t(z["h"]).cuda(), row_weighted=True))):
        s = cb.snap(w, _t(z[f"{tag}_codebook"]).cuda(), **kw)
        assert np.array_equal(s["row_scale"].cpu().numpy(), z[f"{tag}_row_scale"])
        o = orc.snap(z["w"], z[f"{tag}_codebook"], perm=z["perm"] if kw else None, col_weight=z["h"] if kw else None, row_weighted=bool(kw))
        _check(o["chunks"], z[f"{tag}_codebook"], s["idx"].reshape(-1), s["err"], z[f"{tag}_idx"].reshape(-1), o["err"], wt=o["wt"], min_agree=0.999)
        assert abs(s["stats"]["normalized_chunk_mse"] - float(z[f"{tag}_mse"][0])) < 1e-5
    # self-hosting: snap a matrix against a 4096-word book, pack 12-bit tags, decode on the GPU
    g = torch.Generator().manual_seed(5)
    wm = torch.randn(96, 256, generator=g) * (torch.rand(96, 1, generator=g) + 0.5)
    book = torch.randn(4096, 8, generator=g).half()
    s = cb.snap(wm.cuda(), book.cuda())
    words = cb.pack_bits(s["idx"], 12)
    dm = DeviceMatrix(words, book.cuda(), s["row_scale"], K=4096, d=8, C=256, device="cuda")
    ref = orc.codebook_decode(s["idx"].cpu().numpy(), book.numpy(), s["row_scale"].cpu().numpy(), 0, 256, None)
    assert np.array_equal(dm.dequant(dtype=torch.float32).cpu().numpy(), ref)
    rel = float((dm.dequant(dtype=torch.float32).cpu() - wm).pow(2).mean() / wm.pow(2).mean())
    assert rel < 0.5                                       # random book, random matrix: the snap still halves the energy
    # the container's own decode takes the same path
    assert np.array_equal(cb.decode(s.cm).cpu().numpy(), ref)


def test_codebook_matrix_decode_with_padding_and_permutation_matches_the_reference_fixture():
    """decode(CodebookMatrix) on the GPU against the reference's decode of the same container (64-word book, rows of
    100 columns padded to 104, a column permutation): bit for bit, padding stripped, permutation undone."""
    from quantexperiments_b200 import codebook as cb
    z = np.load(G / "codebook.npz")
    pad, cols = (int(v) for v in z["pad"])
    cm = cb.CodebookMatrix(_t(z["idx"]).long(), _t(z["codebook"]), _t(z["row_scale"]), pad, cols, _t(z["perm"]).long())
    assert cm.K == 64 and cm.d == 8
    w = cb.decode(cm)
    assert w.shape == (16, 100) and np.array_equal(w.cpu().numpy(), z["decoded"])
    plain = cb.decode(cb.CodebookMatrix(cm.idx, cm.codebook, cm.row_scale, pad, cols, None))
    assert np.array_equal(plain.cpu().numpy()[:, z["perm"]], plain.cpu().numpy()[:, z["perm"]])
    inv = np.argsort(z["perm"])
    assert np.array_equal(plain.cpu().numpy()[:, inv], z["decoded"])                      # the permutation is what differs
    # a book whose size is not a power of two: 48 of the 64 words
    small = cb.CodebookMatrix(cm.idx % 48, cm.codebook[:48], cm.row_scale, pad, cols, None)
    ref = orc.codebook_decode((z["idx"] % 48), z["codebook"][:48], z["row_scale"], pad, cols, None)
    assert np.array_equal(cb.decode(small).cpu().numpy(), ref)
