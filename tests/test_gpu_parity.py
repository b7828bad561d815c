"""GPU parity tests: every kernel, called through the C ABI, against the CPU oracle and the
reference-generated fixtures. Decoded weights are compared bit for bit; products against an fp32
matmul on the reference-decoded weights with max|got - ref| / max|ref| <= 1e-3 for fp32 outputs
(16-bit outputs add their own rounding of at most half an ulp: 2^-8 for bf16, 2^-11 for fp16, of the element's magnitude)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cbl_oracle as orc

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"
TOL = 1e-3


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def _dm(m, device="cuda"):
    from quantexperiments_b200.kernels import DeviceMatrix
    two = m["books"] == 2
    return DeviceMatrix(_t(m["words"][0]), _t(m["table"][0]), _t(m["row_scale"]), None,
                        None if m["row_mask"] is None else _t(m["row_mask"]), None if m["M"] == 1 else _t(m["perms"]),
                        K=m["K"], d=m["d"], C=m["C"], device=device, tags2=_t(m["words"][1]) if two else None,
                        table2=_t(m["table"][1]) if two else None)


def _l8_counters(ws):
    """The partial-sum slots (160 x 4096 64-bit words) and the status word of a batch-1 work space: zero between calls."""
    return ws[:160 * 4096 * 8 + 256]


def _lib_mod():
    from quantexperiments_b200 import _lib
    return _lib


def _out_tol(dtype):
    return TOL + {torch.float32: 0.0, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}[dtype]


# ------------------------------------------------------------------------------------------ decode
def test_decode_matches_reference_fixtures_bit_for_bit():
    from quantexperiments_b200.kernels import DeviceMatrix
    z = np.load(G / "decode.npz")
    for i, (Gb, M, K, d) in enumerate(z["grid"]):
        seed, R, C = (int(v) for v in z[f"seed_{i}"])
        rb = _t(z[f"rb_{i}"]) if f"rb_{i}" in z else None
        rm = _t(z[f"rm_{i}"]) if f"rm_{i}" in z else None
        perms = _t(orc.seeded_perms(C, int(M), seed)) if M > 1 else None
        dm = DeviceMatrix(_t(z[f"words_{i}"]), _t(z[f"table_{i}"]), _t(z[f"rs_{i}"]), rb, rm, perms, K=int(K), d=int(d), C=C)
        w = dm.dequant(dtype=torch.float32)
        assert torch.equal(w.cpu(), _t(z[f"w_{i}"])), f"case {i}: G={Gb} M={M} K={K} d={d}"
        bits = int(K).bit_length() - 1
        assert np.array_equal(dm.unpack().cpu().numpy(), orc.unpack_bits(z[f"words_{i}"], bits, C // int(d)))


def test_product_of_every_format_in_the_reference_grid():
    """Formats outside d = 8 / 12-bit tags / one book per matrix (the reference's (G, M, K, d) grid, written by its own
    decoder): the generic product and PackedLinear's dispatch to it, 1 / 3 / 9 tokens, against an fp32 matmul on the
    reference-decoded weights."""
    from quantexperiments_b200.kernels import DeviceMatrix
    from quantexperiments_b200.linear import PackedLinear
    z = np.load(G / "decode.npz")
    seen_generic = 0
    for i, (Gb, M, K, d) in enumerate(z["grid"]):
        seed, R, C = (int(v) for v in z[f"seed_{i}"])
        rb = _t(z[f"rb_{i}"]) if f"rb_{i}" in z else None
        rm = _t(z[f"rm_{i}"]) if f"rm_{i}" in z else None
        perms = _t(orc.seeded_perms(C, int(M), seed)) if M > 1 else None
        dm = DeviceMatrix(_t(z[f"words_{i}"]), _t(z[f"table_{i}"]), _t(z[f"rs_{i}"]), rb, rm, perms, K=int(K), d=int(d), C=C)
        w = z[f"w_{i}"]
        lin = PackedLinear(_t(z[f"words_{i}"]).cuda(), _t(z[f"table_{i}"]).cuda(), _t(z[f"rs_{i}"]).cuda(), None if rb is None else rb.cuda(),
                           None if rm is None else rm.cuda(), (perms if perms is not None else torch.arange(C)[None]).cuda(), int(K), int(d))
        seen_generic += not dm.fast
        for T in (1, 3, 9):
            x = torch.randn(T, C, generator=torch.Generator().manual_seed(T + i)).bfloat16()
            yref = orc.linear_ref(x.float().numpy(), w)
            y = dm.gemv_generic(x.cuda(), torch.empty(T, R, device="cuda")).cpu().numpy()
            assert orc.max_rel_err(y, yref) < TOL, (i, T)
            y2 = lin(x.cuda()).float().cpu().numpy()
            assert orc.max_rel_err(y2, yref) < TOL + 2.0 ** -8, (i, T)
        if not dm.fast:
            y1 = lin.gemv(x[0].cuda()).float().cpu().numpy()
            assert orc.max_rel_err(y1, yref[0]) < TOL + 2.0 ** -8
    assert seen_generic >= 2
    # two summed books in a format the fast kernels do not run (d = 4, 8-bit tags)
    m = orc.synth_matrix(96, 64, seed=12, d=4, bits=8, books=2, M=3)
    dm = DeviceMatrix(_t(m["words"][0]), _t(m["table"][0]), _t(m["row_scale"]), None, _t(m["row_mask"]), _t(m["perms"]), K=256, d=4, C=64,
                      tags2=_t(m["words"][1]), table2=_t(m["table"][1]))
    x = torch.randn(5, 64, generator=torch.Generator().manual_seed(1))
    assert orc.max_rel_err(dm.gemv_generic(x.cuda()).cpu().numpy(), orc.linear_ref(x.numpy(), orc.synth_decode(m))) < TOL
    assert _lib_mod().lib.cbl_gemv_generic(None, None, 0, 1, 0, None, 0, 0, None) == _lib_mod().EINVAL


def test_two_book_decode_matches_reference_fixture():
    from quantexperiments_b200.kernels import DeviceMatrix
    z = np.load(G / "additive.npz")
    ta, tb = orc.pack_bits(z["ta"], 12), orc.pack_bits(z["tb"], 12)
    dm = DeviceMatrix(_t(ta), _t(z["A"]), _t(z["rs"]), K=4096, d=8, C=512, tags2=_t(tb), table2=_t(z["B"]))
    assert torch.equal(dm.dequant(dtype=torch.float32).cpu(), _t(z["dense"]))


@pytest.mark.parametrize("R,C,books,M", [(40, 512, 1, 1), (33, 1024, 2, 4), (100, 3584, 1, 16), (4864, 896, 1, 1)])
def test_decode_16bit_outputs_are_one_rounding_of_the_fp32_decode(R, C, books, M):
    m = orc.synth_matrix(R, C, seed=R + C, books=books, M=M)
    dm, ref = _dm(m), orc.synth_decode(m)
    assert torch.equal(dm.dequant(dtype=torch.float32).cpu(), _t(ref))
    assert torch.equal(dm.dequant(dtype=torch.float16).cpu(), _t(orc.round_to(ref, "f16")))
    assert torch.equal(dm.dequant(dtype=torch.bfloat16).cpu(), orc.round_to(ref, "bf16"))


def test_decode_row_range_into_a_larger_scratch_leaves_the_rest_untouched():
    m = orc.synth_matrix(70, 256, seed=5)
    dm, ref = _dm(m), orc.synth_decode(m)
    buf = torch.full((70 * 256 + 100,), float("nan"), dtype=torch.float16, device="cuda")
    got = dm.dequant(buf, rows=(13, 61))
    assert got.shape == (48, 256)
    assert torch.equal(got.cpu(), _t(orc.round_to(ref[13:61], "f16")))
    assert torch.isnan(buf[48 * 256:]).all()
    assert dm.dequant(rows=(7, 7)).shape == (0, 256)


def test_decode_rejects_unsupported_arguments():
    from quantexperiments_b200 import _lib
    m = orc.synth_matrix(8, 64, seed=1)
    dm = _dm(m)
    with pytest.raises(_lib.CblError):
        dm.dequant(rows=(0, 9))
    with pytest.raises(ValueError):
        dm.dequant(dtype=torch.int32)


def test_packed_file_decodes_on_the_gpu_exactly(tmp_path):
    from quantexperiments_b200 import packed
    g = torch.Generator().manual_seed(3)
    R, C, K, d, M = 24, 128, 4096, 8, 4
    tags = torch.randint(0, K, (R, C // d), generator=g)
    table = torch.randn(K, d, generator=g).half()
    rs = torch.rand(R, generator=g).half()
    rm = torch.randint(0, M, (R,), generator=g)
    packed.save(tmp_path / "q.safetensors", {"m": packed.pack_matrix(tags, table, rs, d=d, K=K, M=M, seed=5, row_mask=rm)},
                base_model="test/base")
    pf = packed.PackedFile(tmp_path / "q.safetensors")
    ref = orc.decode_tensors(tags.numpy(), table.numpy(), rs.numpy(), None, rm.numpy(), orc.seeded_perms(C, M, 5), K)
    assert torch.equal(pf.decode("m").cpu(), _t(ref))
    assert torch.equal(pf.local_tags("m").cpu(), tags)
    w = packed.decode_tensors(tags, table, rs, None, rm, pf.perms("m"), K)
    assert torch.equal(w.cpu(), _t(ref))


# ------------------------------------------------------------------------------------------ small-batch product
@pytest.mark.parametrize("R,C", [(512, 3584), (300, 18944), (256, 4864), (128, 256), (17, 896)])
@pytest.mark.parametrize("books,M", [(1, 1), (1, 16), (2, 1), (2, 16)])
def test_small_batch_product_matches_fp32_matmul(R, C, books, M):
    from quantexperiments_b200.kernels import T16Matrix
    m = orc.synth_matrix(R, C, seed=R * 7 + C + books + M, books=books, M=M)
    dm, ref = _dm(m), orc.synth_decode(m)
    t16 = T16Matrix(dm)
    g = torch.Generator().manual_seed(R)
    for B in (1, 4, 8, 13, 64):
        x = torch.randn(B, C, generator=g).bfloat16()
        yref = orc.linear_ref(x.float().numpy(), ref)
        y = torch.full((B, R), float("nan"), device="cuda")
        t16.run(x.cuda(), y)
        assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL, (B, orc.max_rel_err(y.cpu().numpy(), yref))
    x = torch.randn(5, C, generator=g).half()
    yref = orc.linear_ref(x.float().numpy(), ref)
    for dt in (torch.bfloat16, torch.float16):
        y = t16.run(x.cuda(), torch.empty(5, R, dtype=dt, device="cuda"))
        assert orc.max_rel_err(y.float().cpu().numpy(), yref) < _out_tol(dt)


def test_small_batch_product_writes_a_column_slice_and_nothing_else():
    from quantexperiments_b200.kernels import T16Matrix
    m = orc.synth_matrix(48, 512, seed=9)
    dm, ref = _dm(m), orc.synth_decode(m)
    x = torch.randn(6, 512, generator=torch.Generator().manual_seed(2)).bfloat16()
    wide = torch.full((6, 200), float("nan"), device="cuda")
    T16Matrix(dm).run(x.cuda(), wide[:, 100:148])
    yref = orc.linear_ref(x.float().numpy(), ref)
    assert orc.max_rel_err(wide[:, 100:148].cpu().numpy(), yref) < TOL
    assert torch.isnan(wide[:, :100]).all() and torch.isnan(wide[:, 148:]).all()


def test_small_batch_product_is_deterministic_and_survives_outliers():
    from quantexperiments_b200.kernels import T16Matrix
    m = orc.synth_matrix(256, 3584, seed=4)
    dm, ref = _dm(m), orc.synth_decode(m)
    t16 = T16Matrix(dm)
    x = torch.randn(8, 3584, generator=torch.Generator().manual_seed(0)).half()
    x[:, ::97] = 5536.0           # magnitudes that overflow fp16 products summed in half precision
    ys = [t16.run(x.cuda()).clone() for _ in range(3)]
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[1], ys[2])
    y = t16.run(x.cuda(), torch.empty(8, 256, device="cuda"))
    assert torch.isfinite(y).all()
    assert orc.max_rel_err(y.cpu().numpy(), orc.linear_ref(x.float().numpy(), ref)) < TOL


# ------------------------------------------------------------------------------------------ batch-1 product
@pytest.mark.parametrize("R,C,books", [(4864, 896, 1), (3584, 3584, 1), (2051, 1024, 1), (512, 3584, 1), (2304, 1000 * 8, 2),
                                        (4, 64, 1), (1030, 72, 2)])
def test_batch1_product_matches_fp32_matmul(R, C, books):
    from quantexperiments_b200.kernels import L8Matrix
    m = orc.synth_matrix(R, C, seed=R + 3 * C + books, books=books)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    g = torch.Generator().manual_seed(C)
    for it in range(3):           # repeated calls: the shared work space must return to zero every time
        x = torch.randn(C, generator=g).bfloat16()
        yref = orc.linear_ref(x.float().numpy()[None], ref)[0]
        y = torch.full((R,), float("nan"), device="cuda")
        l8.run(x.cuda(), y)
        assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL, (it, orc.max_rel_err(y.cpu().numpy(), yref))
    for dt in (torch.bfloat16, torch.float16):
        y = l8.run(x.cuda(), torch.empty(R, dtype=dt, device="cuda"))
        assert orc.max_rel_err(y.float().cpu().numpy(), yref) < _out_tol(dt)
    from quantexperiments_b200.kernels import l8_workspace
    assert int(_l8_counters(l8_workspace(dm.device, R)).count_nonzero()) == 0


def test_batch1_product_survives_outliers_and_extreme_scales():
    from quantexperiments_b200.kernels import L8Matrix
    m = orc.synth_matrix(2048, 3584, seed=8)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    x = torch.randn(3584, generator=torch.Generator().manual_seed(1))
    x[::97] = 5536.0
    for xs in (x.half(), (x * 1e30).bfloat16(), (x * 1e-20).bfloat16()):
        yref = orc.linear_ref(xs.float().numpy()[None], ref)[0]
        y = l8.run(xs.cuda(), torch.empty(2048, device="cuda"))
        assert torch.isfinite(y).all()
        assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL


@pytest.mark.parametrize("R,C,books,M", [(2304, 1024, 2, 16), (1000, 520, 1, 3), (4100, 896, 1, 16), (37, 64, 2, 2), (20, 128, 1, 16)])
def test_batch1_product_with_column_orders_matches_fp32_matmul(R, C, books, M):
    """Rows grouped by column order, one table per (tile, order) built from the permuted activations:
    y[r] = rs[r] * sum_j <table[tag[r, j]], x[perm_{m_r}[8j .. 8j+7]]> (shapequant/kernels/gemv.py:3)."""
    from quantexperiments_b200.kernels import L8Matrix, l8_workspace
    m = orc.synth_matrix(R, C, seed=R + C + M, books=books, M=M)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    assert l8.Rpad % 32 == 0 and l8.seg_off[-1] == l8.Rpad
    g = torch.Generator().manual_seed(R)
    for it in range(2):
        x = torch.randn(C, generator=g).bfloat16()
        yref = orc.linear_ref(x.float().numpy()[None], ref)[0]
        y = l8.run(x.cuda(), torch.full((R,), float("nan"), device="cuda"))
        assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL
    assert int(_l8_counters(l8_workspace(dm.device, R)).count_nonzero()) == 0


def test_batch1_product_is_bit_reproducible_and_flags_non_finite_inputs():
    """Blocks that share rows meet in integer accumulators, so the arrival order cannot change a bit: repeated
    calls and graph replays return identical outputs (the reference tests its ticket-ordered split-K the same way,
    tests/test_batched_runs.py:41-68).  A NaN anywhere in x makes every output NaN, as it would in a matmul."""
    from quantexperiments_b200.kernels import L8Group, L8Matrix
    m = orc.synth_matrix(1024, 18944, seed=77)           # few rows, many tiles: every row is summed over ~100 blocks
    l8 = L8Matrix(_dm(m))
    x = torch.randn(18944, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    y0 = l8.run(x, torch.empty(1024, device="cuda")).clone()
    for it in range(5):
        assert torch.equal(l8.run(x, torch.empty(1024, device="cuda")), y0)
    assert orc.max_rel_err(y0.cpu().numpy(), orc.linear_ref(x.float().cpu().numpy()[None], orc.synth_decode(m))[0]) < TOL
    s = torch.cuda.Stream()
    y = torch.empty(1024, device="cuda")
    with torch.cuda.stream(s):
        l8.run(x, y)
        s.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            l8.run(x, y)
        for it in range(3):
            y.fill_(0)
            gr.replay()
            s.synchronize()
            assert torch.equal(y, y0)
    xn = x.clone()
    xn[12345] = float("nan")
    assert torch.isnan(l8.run(xn, torch.empty(1024, device="cuda"))).all()
    assert torch.equal(l8.run(x, torch.empty(1024, device="cuda")), y0)      # and the work space is clean afterwards


def test_full_size_shapes_by_linearity_and_agreement_between_kernels():
    """At the benchmark's largest shapes the oracle is too slow to run whole; check size-independent
    properties: W(x1 + x2) = W x1 + W x2, the two kernels agree, and a sample of rows matches the oracle."""
    from quantexperiments_b200.kernels import DeviceMatrix, L8Matrix, T16Matrix
    for R, C in ((18944, 3584), (3584, 18944)):
        g = torch.Generator(device="cuda").manual_seed(R)
        W = (C // 8 * 12 + 31) // 32
        words = torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g)
        table = torch.randn(4096, 8, device="cuda", generator=g).half()
        rs = (torch.rand(R, device="cuda", generator=g) * 0.02 + 0.01).half()
        dm = DeviceMatrix(words, table, rs, K=4096, d=8, C=C)
        l8, t16 = L8Matrix(dm), T16Matrix(dm)
        x1 = torch.randn(C, device="cuda", generator=g).half().float()
        x2 = torch.randn(C, device="cuda", generator=g).half().float()
        f = lambda x: l8.run(x, torch.empty(R, device="cuda"))
        ya, yb, yab = f(x1), f(x2), f((x1 + x2).half().float())
        scale = float(yab.abs().max())
        x12 = (x1 + x2).half().float()
        assert float((f(x12) - yab).abs().max()) == 0.0 or float((f(x12) - yab).abs().max()) / scale < 1e-5
        lin_err = float((ya + yb - f(x1 + x2)).abs().max()) / scale
        assert lin_err < TOL
        yt = t16.run(x12[None], torch.empty(1, R, device="cuda"))[0]
        assert float((yt - yab).abs().max()) / scale < TOL
        rows = torch.randint(0, R, (64,), generator=torch.Generator().manual_seed(0))
        tags = orc.unpack_bits(words[rows.cuda()].cpu().numpy(), 12, C // 8)
        wref = orc.decode_tensors(tags, table.cpu().numpy(), rs[rows.cuda()].cpu().numpy(), None, None, np.arange(C)[None], 4096)
        assert torch.equal(dm.dequant(rows=(int(rows[0]), int(rows[0]) + 1)).cpu()[0], _t(wref[0]))
        yref = orc.linear_ref(x12.cpu().numpy()[None], wref)[0]
        assert float(np.abs(yab[rows.cuda()].cpu().numpy() - yref).max()) / scale < TOL


# ------------------------------------------------------------------------------------------ prefill product
@pytest.mark.parametrize("R,C,T,books", [(256, 64, 128, 1), (512, 896, 300, 1), (300, 1024, 77, 1), (4864, 896, 513, 1),
                                         (1024, 3584, 2048, 1), (259, 72, 1, 1), (512, 1024, 300, 2), (300, 5120, 700, 2)])
def test_prefill_product_matches_fp32_matmul(R, C, T, books):
    from quantexperiments_b200.kernels import L8Matrix
    m = orc.synth_matrix(R, C, seed=R + C + T, books=books)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    X = torch.randn(T, C, generator=torch.Generator().manual_seed(T)).bfloat16()
    yref = orc.linear_ref(X.float().numpy(), ref)
    Y = torch.full((T, R), float("nan"), device="cuda")
    l8.gemm(X.cuda(), Y)
    l8.status()
    assert orc.max_rel_err(Y.cpu().numpy(), yref) < TOL
    for dt in (torch.bfloat16, torch.float16):
        Y = l8.gemm(X.cuda(), torch.empty(T, R, dtype=dt, device="cuda"))
        assert orc.max_rel_err(Y.float().cpu().numpy(), yref) < _out_tol(dt)
    if books == 1:
        Y = torch.full((T, R), float("nan"), device="cuda")
        l8.gemm(X.cuda(), Y, two_sm=True)        # pairs of thread blocks (tcgen05 cta_group::2) above 256 tokens
        l8.status()
        assert orc.max_rel_err(Y.cpu().numpy(), yref) < TOL


def test_prefill_product_writes_a_column_slice_and_survives_outliers():
    from quantexperiments_b200.kernels import L8Matrix
    m = orc.synth_matrix(256, 512, seed=12)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    X = torch.randn(100, 512, generator=torch.Generator().manual_seed(3)).bfloat16()
    X[:, ::61] = 5536.0
    X[7] *= 1e30
    X[9] *= 1e-25
    yref = orc.linear_ref(X.float().numpy(), ref)
    wide = torch.full((100, 777), float("nan"), device="cuda")       # odd row stride: the scalar store path
    l8.gemm(X.cuda(), wide[:, 300:556])
    got = wide[:, 300:556].cpu().numpy()
    assert np.isfinite(got).all()
    for t in range(100):          # per token: scales differ by 55 orders of magnitude
        assert orc.max_rel_err(got[t], yref[t]) < TOL
    assert torch.isnan(wide[:, :300]).all() and torch.isnan(wide[:, 556:]).all()
    wide16 = torch.full((100, 768), float("nan"), device="cuda", dtype=torch.bfloat16)   # aligned slice: vector stores
    l8.gemm(X.cuda(), wide16[:, 256:512])
    assert torch.isnan(wide16[:, :256]).all() and torch.isnan(wide16[:, 512:]).all()
    for t in range(100):
        assert orc.max_rel_err(wide16[t, 256:512].float().cpu().numpy(), yref[t]) < _out_tol(torch.bfloat16)


# ------------------------------------------------------------------------------------------ call surfaces
def test_packed_linear_matches_reference_fixture_and_dispatches_by_token_count():
    from quantexperiments_b200.linear import PackedLinear
    z = np.load(G / "linear.npz")
    R, C, K, d, M = 48, 896, 4096, 8, 16
    lin = PackedLinear(_t(z["words"]).cuda(), _t(z["table"]).cuda(), _t(z["rs"]).cuda(), None, _t(z["rm"]).cuda(),
                       _t(orc.seeded_perms(C, M, 1)).cuda(), K, d)
    assert lin.stored_bytes() == int(z["stored_bytes"][0])
    assert float(lin.dense().double().sum()) == float(z["dense_sum"][0])
    x = _t(z["x"]).cuda()
    y = lin(x)                                    # 3 tokens -> small-batch kernel
    assert orc.max_rel_err(y.cpu().numpy(), z["y"]) < TOL
    y1 = lin(x[:1])                               # 1 token -> batch-1 path
    assert orc.max_rel_err(y1.cpu().numpy(), z["y"][:1]) < TOL
    xb = torch.randn(2, 40, C, device="cuda", dtype=torch.bfloat16)      # 80 tokens, column orders -> decode + library GEMM
    yb = lin(xb)
    ref = xb.float().reshape(80, C) @ lin.dense().T
    assert yb.shape == (2, 40, R) and orc.max_rel_err(yb.float().reshape(80, R).cpu().numpy(), ref.cpu().numpy()) < 1e-2
    assert lin(x[:0]).shape == (0, R)
    with pytest.raises(ValueError):
        PackedLinear(_t(z["words"]), _t(z["table"]), _t(z["rs"]), None, None, None, K, d)      # CPU tensors


def test_runs_lin_and_runs_batch_write_into_caller_buffers_and_capture_in_a_graph():
    from quantexperiments_b200.linear import PackedLinear, RunsBatch, RunsLin
    m = orc.synth_matrix(2304, 896, seed=21)
    ref = orc.synth_decode(m)
    lin = PackedLinear(_t(m["words"][0]).cuda(), _t(m["table"][0]).cuda(), _t(m["row_scale"]).cuda(), None, None,
                       torch.arange(896)[None].cuda(), 4096, 8)
    rl, rb = RunsLin(lin), RunsBatch(lin, bmax=32)
    x = torch.randn(896, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0)).bfloat16()
    X = torch.randn(32, 896, device="cuda").bfloat16()
    y, Y = torch.empty(2304, device="cuda", dtype=torch.bfloat16), torch.empty(32, 2304, device="cuda", dtype=torch.bfloat16)
    rl.run(x, y)
    rb.run(X, Y, 32)
    torch.cuda.synchronize()
    y0, Y0 = y.clone(), Y.clone()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        rl.run(x, y)
        rb.run(X, Y, 32)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            rl.run(x, y)
            rb.run(X, Y, 32)
        y.zero_(), Y.zero_()
        g.replay()
        s.synchronize()
    assert orc.max_rel_err(y.float().cpu().numpy(), orc.linear_ref(x.float().cpu().numpy()[None], ref)[0]) < _out_tol(torch.bfloat16)
    assert torch.equal(Y, Y0)
    assert orc.max_rel_err(y.float().cpu().numpy(), y0.float().cpu().numpy()) < 1e-2
    with pytest.raises(ValueError):
        rb.run(X.float(), Y, 32)


def test_packed_shards_and_custom_op(tmp_path):
    from quantexperiments_b200 import packed
    from quantexperiments_b200.vllm_ext import core
    g = torch.Generator().manual_seed(0)
    C, K, d = 512, 4096, 8
    mats, refs = {}, []
    for name, R in (("l.q_proj", 2048), ("l.k_proj", 64), ("l.v_proj", 64)):
        tags = torch.randint(0, K, (R, C // d), generator=g)
        table = torch.randn(K, d, generator=g).half()
        rs = (torch.rand(R, generator=g) * 0.02 + 0.01).half()
        mats[name] = packed.pack_matrix(tags, table, rs, d=d, K=K, seed=1)
        refs.append(orc.decode_tensors(tags.numpy(), table.numpy(), rs.numpy(), None, None, np.arange(C)[None], K))
    packed.save(tmp_path / "m.safetensors", mats, base_model="test/base")
    pf = packed.PackedFile(tmp_path / "m.safetensors")
    ps = core.PackedShards.from_packed(pf, list(mats), dev="cuda", bmax=32)
    wref = np.concatenate(refs)
    assert ps.R == 2176 and ps.C == C and ps.nbytes() > 0
    assert torch.equal(ps.dense().cpu(), _t(wref.astype(np.float16)))
    h = core.register(ps)
    for M in (1, 5, 32, 100):
        x = torch.randn(M, C, device="cuda", dtype=torch.bfloat16)
        y = torch.ops.shapequant.linear(x, h)
        assert y.shape == (M, 2176) and y.dtype == torch.bfloat16
        ref = orc.linear_ref(x.float().cpu().numpy(), wref)
        assert orc.max_rel_err(y.float().cpu().numpy(), ref) < (_out_tol(torch.bfloat16) if M <= 32 else 1e-2)
    assert torch.ops.shapequant.linear(torch.empty(0, C, device="cuda", dtype=torch.bfloat16), h).shape == (0, 2176)
    # opaque to the compiler, like the reference's op (fullgraph trace through the fake implementation)
    fn = torch.compile(lambda t: torch.ops.shapequant.linear(t, h) * 2, backend="aot_eager", fullgraph=True)
    x = torch.randn(3, C, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(fn(x), torch.ops.shapequant.linear(x, h) * 2)


@pytest.mark.parametrize("shapes,C", [([(3584, 1), (512, 1), (512, 1)], 896), ([(2304, 1), (2304, 2)], 512), ([(260, 1)], 64),
                                      ([(128, 1), (128, 1), (128, 1), (4100, 1)], 1024)])
def test_grouped_batch1_launch_matches_fp32_matmul(shapes, C):
    from quantexperiments_b200.kernels import L8Group, L8Matrix
    ms = [orc.synth_matrix(R, C, seed=R + i + books, books=books) for i, (R, books) in enumerate(shapes)]
    grp = L8Group([L8Matrix(_dm(m)) for m in ms])
    g = torch.Generator().manual_seed(C)
    for it in range(2):
        x = torch.randn(C, generator=g).bfloat16()
        ys = [torch.full((m["R"],), float("nan"), device="cuda") for m in ms]
        grp.run(x.cuda(), ys)
        for m, y in zip(ms, ys):
            yref = orc.linear_ref(x.float().numpy()[None], orc.synth_decode(m))[0]
            assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL
    with pytest.raises(ValueError):
        grp.run(x.cuda(), ys[:-1] + [ys[-1].double()] if len(ys) > 1 else [])


def test_peer_reduce_entry_point_with_one_rank_and_graph_replay():
    """cbl_gemv_l8_ar with world = 1 (the rank is its own only peer): same result as the plain product,
    and a captured graph can be replayed because the call number lives in the work space."""
    import ctypes
    from quantexperiments_b200 import _lib
    from quantexperiments_b200.kernels import L8Matrix
    m = orc.synth_matrix(3584, 896, seed=31)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    ws = torch.zeros(_lib.lib.cbl_gemv_l8_ar_workspace_bytes(3584), dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(ws.data_ptr())
    st = l8.struct()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(896, generator=g).bfloat16().cuda()
    y = torch.empty(3584, device="cuda")

    def call():
        rc = _lib.lib.cbl_gemv_l8_ar(ctypes.byref(st), x.data_ptr(), _lib.BF16, y.data_ptr(), _lib.F32, ptrs, 0, 1,
                                     torch.cuda.current_stream().cuda_stream)
        assert rc == _lib.OK

    for it in range(3):
        x.copy_(torch.randn(896, generator=g).bfloat16())
        y.fill_(float("nan"))
        call()
        yref = orc.linear_ref(x.float().cpu().numpy()[None], ref)[0]
        assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        call()
        s.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            call()
            call()
        for it in range(3):
            x.copy_(torch.randn(896, generator=g).bfloat16().cuda())
            y.fill_(float("nan"))
            gr.replay()
            s.synchronize()
            yref = orc.linear_ref(x.float().cpu().numpy()[None], ref)[0]
            assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL
    rmax = (3584 + 31) // 32 * 32 + 32 * 16                              # rows of a sum buffer (row positions incl. padding)
    ctl = ws[2 * rmax * 4 + 32:].view(torch.int32)[:3].cpu().tolist()
    assert ctl[0] == 0 and ctl[1] == 3 + 1 + 6 and ctl[2] == 0           # status, completed calls (capture itself runs nothing), ticket
    assert int(_l8_counters(ws[2 * rmax * 4 + 64:]).count_nonzero()) == 0   # the product's slots are zero again


def test_peer_reduce_reports_a_missing_peer_instead_of_hanging():
    """A rank whose peer never publishes its word: the finish kernel's wait is bounded, the call returns,
    the status query reports the time-out and the context keeps working (no fault, no hang)."""
    import ctypes
    import time
    from quantexperiments_b200 import _lib
    from quantexperiments_b200.kernels import L8Matrix
    lib = _lib.lib
    m = orc.synth_matrix(2048, 256, seed=3)
    dm, ref = _dm(m), orc.synth_decode(m)
    l8 = L8Matrix(dm)
    n = lib.cbl_gemv_l8_ar_workspace_bytes(2048)
    ws = torch.zeros(2 * n + 512, dtype=torch.uint8, device="cuda")
    off = (n + 255) // 256 * 256
    ptrs = (ctypes.c_void_p * 2)(ws.data_ptr(), ws.data_ptr() + off)       # "rank 1" is never launched
    x = torch.randn(256, generator=torch.Generator().manual_seed(0)).bfloat16().cuda()
    y = torch.full((2048,), 7.0, device="cuda")
    st = l8.struct()
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    assert lib.cbl_gemv_l8_ar(ctypes.byref(st), x.data_ptr(), _lib.BF16, y.data_ptr(), _lib.F32, ptrs, 0, 2, stream) == _lib.OK
    assert lib.cbl_gemv_l8_ar_status(ctypes.c_void_p(ws.data_ptr()), 2048, stream) == _lib.ETIMEOUT
    assert time.time() - t0 < 60
    assert torch.equal(y, torch.full_like(y, 7.0))                       # the output was left untouched
    assert lib.cbl_gemv_l8_ar_status(ctypes.c_void_p(ws.data_ptr()), 2048, stream) == _lib.OK      # cleared
    # the device is fine: an ordinary product right after
    yref = orc.linear_ref(x.float().cpu().numpy()[None], ref)[0]
    y2 = l8.run(x, torch.empty(2048, device="cuda"))
    assert orc.max_rel_err(y2.cpu().numpy(), yref) < TOL
    # and the SAME work space is good for the next calls (as a single rank): nothing of the failed call lingers
    one = (ctypes.c_void_p * 1)(ws.data_ptr())
    for it in range(2):
        y.fill_(float("nan"))
        assert lib.cbl_gemv_l8_ar(ctypes.byref(st), x.data_ptr(), _lib.BF16, y.data_ptr(), _lib.F32, one, 0, 1, stream) == _lib.OK
        assert lib.cbl_gemv_l8_ar_status(ctypes.c_void_p(ws.data_ptr()), 2048, stream) == _lib.OK
        assert orc.max_rel_err(y.cpu().numpy(), yref) < TOL


@pytest.mark.parametrize("C", [5120, 27648])
def test_qwen32b_shaped_rows_with_two_books_and_sixteen_column_orders(C):
    """Row samples of the 32B-shaped matrices (hidden 5120, SwiGLU 27648): two summed books and 16 seeded
    column orders per matrix: decode bit-exact, decode batches 1..64 and a 300-token prefill within tolerance."""
    from quantexperiments_b200.kernels import L8Matrix, T16Matrix
    from quantexperiments_b200.linear import PackedLinear
    R = 320
    m = orc.synth_matrix(R, C, seed=C, books=2, M=16)
    dm, ref = _dm(m), orc.synth_decode(m)
    assert torch.equal(dm.dequant(dtype=torch.float32).cpu(), _t(ref))
    t16 = T16Matrix(dm)
    g = torch.Generator().manual_seed(C)
    for B in (1, 32, 64):
        x = torch.randn(B, C, generator=g).bfloat16()
        y = t16.run(x.cuda(), torch.empty(B, R, device="cuda"))
        assert orc.max_rel_err(y.cpu().numpy(), orc.linear_ref(x.float().numpy(), ref)) < TOL
    # one column order: the table-lookup and tensor-core prefill paths with two books
    m1 = orc.synth_matrix(2304, C, seed=C + 1, books=2, M=1)
    dm1, ref1 = _dm(m1), orc.synth_decode(m1)
    l8 = L8Matrix(dm1)
    x = torch.randn(300, C, generator=g).bfloat16()
    yref = orc.linear_ref(x.float().numpy(), ref1)
    y1 = l8.run(x[0].cuda(), torch.empty(2304, device="cuda"))
    assert orc.max_rel_err(y1.cpu().numpy(), yref[0]) < TOL
    Y = l8.gemm(x.cuda(), torch.empty(300, 2304, device="cuda"))
    l8.status()
    assert orc.max_rel_err(Y.cpu().numpy(), yref) < TOL
    # the module dispatches 300 tokens of a 16-order matrix to decode + library GEMM
    lin = PackedLinear(_t(m["words"][0]).cuda(), _t(m["table"][0]).cuda(), _t(m["row_scale"]).cuda(), None, _t(m["row_mask"]).cuda(),
                       _t(m["perms"]).cuda(), 4096, 8, words2=_t(m["words"][1]).cuda(), table2=_t(m["table"][1]).cuda())
    yl = lin(x.cuda())
    assert orc.max_rel_err(yl.float().cpu().numpy(), orc.linear_ref(x.float().numpy(), ref)) < 1e-2


# ------------------------------------------------------------------------------------------ two-phase prefill
@pytest.mark.parametrize("R,C,T,books,M", [(300, 264, 70, 1, 1), (1000, 520, 300, 2, 1), (520, 1032, 257, 1, 4), (260, 264, 65, 2, 3),
                                            (777, 3584, 1100, 1, 1), (2, 8, 1, 1, 1)])
def test_two_phase_prefill_matches_fp32_matmul(R, C, T, books, M):
    """cbl_decode_raw + cbl_gemm_dense (decode once into a 16-bit scratch, TMA-fed tcgen05 GEMM) for one or two
    books and for several column orders, fp32 and 16-bit outputs."""
    from quantexperiments_b200.kernels import DenseStack
    m = orc.synth_matrix(R, C, seed=R + C + T, books=books, M=M)
    dm = _dm(m)
    w = torch.from_numpy(orc.synth_decode(m)).cuda()
    g = torch.Generator(device="cuda").manual_seed(T)
    for xdt in (torch.bfloat16, torch.float16, torch.float32):
        X = torch.randn(T, C, device="cuda", generator=g).to(xdt)
        ref = X.float() @ w.t()
        for ydt in (torch.float32, torch.bfloat16):
            Y = dm.gemm_dense(X, torch.full((T, R), 7.0, device="cuda", dtype=ydt))
            err = (Y.float() - ref).abs().max() / ref.abs().max()
            assert err <= _out_tol(ydt), (xdt, ydt, float(err))
    DenseStack.status("cuda")


def test_two_phase_prefill_stacks_pieces_writes_a_column_slice_and_survives_outliers():
    from quantexperiments_b200.kernels import DenseStack
    C, T = 520, 200
    ms = [orc.synth_matrix(R, C, seed=40 + i, books=1 + (i == 1), M=1 + 2 * (i == 2)) for i, R in enumerate((300, 129, 260))]
    dms = [_dm(m) for m in ms]
    w = torch.cat([torch.from_numpy(orc.synth_decode(m)) for m in ms]).cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    X = torch.randn(T, C, device="cuda", generator=g)
    X[5, 17] = 3.0e4                      # an outlier token: its own power-of-two scale keeps the others exact
    X[9] *= 1e-6
    X = X.bfloat16()
    ref = X.float() @ w.t()
    wide = torch.full((T, 689 + 16), 5.0, device="cuda", dtype=torch.bfloat16)
    st = DenseStack(dms)
    assert st.R == 689
    st.gemm(X, wide[:, 8:8 + 689])
    assert (wide[:, :8] == 5.0).all() and (wide[:, 8 + 689:] == 5.0).all()
    got = wide[:, 8:8 + 689].float()
    for t in (0, 5, 9, 199):              # per token: every token is scaled by its own power of two
        assert (got[t] - ref[t]).abs().max() / ref[t].abs().max() <= _out_tol(torch.bfloat16), t
    # twice in a row (the two scratch buffers alternate) and from a non-contiguous activation view
    Xw = torch.randn(T, C + 24, device="cuda", generator=g).bfloat16()
    y1 = st.gemm(Xw[:, 8:8 + C])
    y2 = st.gemm(Xw[:, 8:8 + C])
    assert torch.equal(y1, y2)
    assert (y1.float() - Xw[:, 8:8 + C].float() @ w.t()).abs().max() / ref.abs().max() <= _out_tol(torch.bfloat16)
    DenseStack.status("cuda")


def test_two_phase_prefill_back_to_back_matrices_on_alternating_scratches():
    """The documented call sequence through the C ABI: decode A -> gemm A -> decode B -> gemm B -> decode A ... on TWO
    scratch buffers (cbl_decode_raw starts writing before earlier work of the stream has finished, so a scratch is
    never reused by the very next decode)."""
    import ctypes
    from quantexperiments_b200 import _lib
    lib = _lib.lib
    T, C = 130, 520
    ms = [orc.synth_matrix(R, C, seed=40 + i) for i, R in enumerate((300, 520, 260, 300))]
    dms = [_dm(m) for m in ms]
    X = torch.randn(T, C, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)).bfloat16()
    ld = (C + 7) // 8 * 8
    scr = [torch.empty(lib.cbl_dense_scratch_bytes(520, C), dtype=torch.uint8, device="cuda") for _ in range(2)]
    stage = torch.zeros(lib.cbl_gemm_stage_bytes(T, C) + 16, dtype=torch.uint8, device="cuda")
    ys = [torch.empty(T, m["R"], device="cuda") for m in ms]
    s = torch.cuda.current_stream().cuda_stream
    for rep in range(3):
        for i, (dm, y) in enumerate(zip(dms, ys)):
            sc = scr[i & 1]
            assert lib.cbl_decode_raw(ctypes.byref(dm.struct()), sc.data_ptr(), s) == _lib.OK
            assert lib.cbl_gemm_dense(sc.data_ptr(), dm.R, C, dm.row_scale.data_ptr(), X.data_ptr(), _lib.BF16, T, X.stride(0), y.data_ptr(),
                                      _lib.F32, y.stride(0), stage.data_ptr(), stage.data_ptr() + stage.numel() - 16, s) == _lib.OK
    torch.cuda.synchronize()
    assert int(stage[-16:].view(torch.int32)[0]) == 0
    for m, y in zip(ms, ys):
        assert orc.max_rel_err(y.cpu().numpy(), orc.linear_ref(X.float().cpu().numpy(), orc.synth_decode(m))) < TOL


def test_two_phase_prefill_rejects_unsupported_arguments():
    from quantexperiments_b200 import _lib
    import ctypes
    m = orc.synth_matrix(64, 64, seed=1, d=4, bits=10)
    dm = _dm(m)
    t = torch.zeros(64 * 64, device="cuda", dtype=torch.float16)
    s = torch.cuda.current_stream().cuda_stream
    assert _lib.lib.cbl_decode_raw(ctypes.byref(dm.struct()), t.data_ptr(), s) == _lib.EUNSUPPORTED
    assert _lib.lib.cbl_decode_raw(None, t.data_ptr(), s) == _lib.EINVAL
    assert _lib.lib.cbl_gemm_dense(t.data_ptr(), 64, 60, t.data_ptr(), t.data_ptr(), 1, 4, 64, t.data_ptr(), 1, 64, t.data_ptr(), t.data_ptr(), s) == _lib.EINVAL
    assert _lib.lib.cbl_gemm_dense(t.data_ptr(), 64, 64, t.data_ptr(), t.data_ptr(), 1, 4, 64, t.data_ptr(), 1, 32, t.data_ptr(), t.data_ptr(), s) == _lib.EINVAL
    assert _lib.lib.cbl_dense_scratch_bytes(3, 12) == 3 * 16 * 2


# ------------------------------------------------------------------------------------------ a few dozen tokens, weight rows as M
@pytest.mark.parametrize("Rs,C,B,books", [((300,), 264, 5, 1), ((1000, 129), 520, 32, 1), ((260, 130, 130), 1032, 17, 2),
                                         ((3584, 512, 512), 3584, 32, 1), ((130,), 64, 1, 1), ((520, 520), 4104, 40, 1)])
def test_rows_as_m_product_matches_fp32_matmul(Rs, C, B, books):
    """cbl_gemm_rows_multi: grouped matrices, k-split launches (few row tiles) and whole-k launches, one and two
    books, ragged row counts, more than 32 tokens as several launches; outputs are column slices of one buffer."""
    from quantexperiments_b200.kernels import L8Group, L8Matrix
    ms = [orc.synth_matrix(R, C, seed=R + C + B + i, books=books) for i, R in enumerate(Rs)]
    l8s = [L8Matrix(_dm(m)) for m in ms]
    w = torch.cat([torch.from_numpy(orc.synth_decode(m)) for m in ms]).cuda()
    g = torch.Generator(device="cuda").manual_seed(B)
    X = torch.randn(B, C, device="cuda", generator=g)
    X[0, 3] = 2.0e4
    X = X.bfloat16()
    ref = X.float() @ w.t()
    grp = L8Group(l8s)
    for ydt in (torch.float32, torch.bfloat16, torch.float16):
        Y = torch.full((B, sum(Rs) + 8), 3.0, device="cuda", dtype=ydt)
        ys, o = [], 0
        for R in Rs:
            ys.append(Y[:, o:o + R])
            o += R
        for _ in range(2):              # the work space is left zero: a second call gives the same result
            grp.gemm_rows(X, ys)
            got = Y[:, :sum(Rs)].float()
            for t in range(B):
                assert (got[t] - ref[t]).abs().max() / ref[t].abs().max() <= _out_tol(ydt), (ydt, t)
            assert (Y[:, sum(Rs):] == 3.0).all()
    l8s[0].status()


def test_rows_as_m_product_rejects_unsupported_arguments():
    from quantexperiments_b200 import _lib
    from quantexperiments_b200.kernels import L8Matrix
    import ctypes
    l8 = L8Matrix(_dm(orc.synth_matrix(64, 64, seed=2)))
    st = (_lib.L8 * 1)(l8.struct_c())
    t = torch.zeros(1 << 16, device="cuda", dtype=torch.float16)
    ys = (ctypes.c_void_p * 1)(t.data_ptr())
    s = torch.cuda.current_stream().cuda_stream
    call = lambda n, ntok, ldy: _lib.lib.cbl_gemm_rows_multi(st, n, t.data_ptr(), 1, ntok, 64, ys, 1, ldy, t.data_ptr(), t.data_ptr(), s)   # noqa: E731
    assert call(1, 33, 64) == _lib.EUNSUPPORTED
    assert call(5, 4, 64) == _lib.EUNSUPPORTED
    assert call(1, 0, 64) == _lib.EINVAL
    assert call(1, 4, 32) == _lib.EINVAL
    assert _lib.lib.cbl_gemm_rows_max_tokens() == 32
    assert _lib.lib.cbl_gemm_rows_workspace_bytes(128) == 32 * 128 * 4 + 16



# ------------------------------------------------------------------------------------------ 16..32 tokens, activations stationary
@pytest.mark.parametrize("R,C,books", [(300, 264, 1), (2304, 896, 1), (129, 8200, 1), (640, 4104, 2), (1100, 3584, 1), (64, 128, 2)])
def test_activation_stationary_product_matches_fp32_matmul(R, C, books):
    """cbl_gemv_x16: ragged rows and columns, one and two books, whole-k launches and launches whose columns are
    split over several blocks (few rows, many columns); the output is a column slice; the work space is left zero."""
    from quantexperiments_b200.kernels import X16Matrix
    m = orc.synth_matrix(R, C, seed=R + C + books, books=books)
    xm = X16Matrix(_dm(m))
    w = torch.from_numpy(orc.synth_decode(m)).cuda()
    g = torch.Generator(device="cuda").manual_seed(R)
    for B in (1, 16, 17, 32):
        X = torch.randn(B, C, device="cuda", generator=g)
        X[0, 3] = 2.0e4
        X = X.bfloat16()
        ref = X.float() @ w.t()
        for ydt in (torch.float32, torch.bfloat16):
            Y = torch.full((B, R + 8), 3.0, device="cuda", dtype=ydt)
            for _ in range(2):
                xm.run(X, Y[:, :R])
                got = Y[:, :R].float()
                for t in range(B):
                    assert (got[t] - ref[t]).abs().max() / ref[t].abs().max() <= _out_tol(ydt), (B, ydt, t)
                assert (Y[:, R:] == 3.0).all()
    assert (xm.ws == 0).all()


def test_activation_stationary_product_rejects_unsupported_arguments():
    from quantexperiments_b200 import _lib
    from quantexperiments_b200.kernels import X16Matrix
    import ctypes
    xm = X16Matrix(_dm(orc.synth_matrix(64, 64, seed=2)))
    st = xm.struct()
    t = torch.zeros(1 << 16, device="cuda", dtype=torch.float16)
    s = torch.cuda.current_stream().cuda_stream
    call = lambda B, ldy: _lib.lib.cbl_gemv_x16(ctypes.byref(st), t.data_ptr(), B, t.data_ptr(), 1, ldy, xm.ws.data_ptr(), s)   # noqa: E731
    assert call(33, 64) == _lib.EUNSUPPORTED
    assert call(0, 64) == _lib.EINVAL
    assert call(4, 32) == _lib.EINVAL
    assert _lib.lib.cbl_gemv_x16_workspace_bytes(100) == 32 * 128 * 4 + 2 * 4
    assert _lib.lib.cbl_x16_bytes(100, 264, 2) == 2 * 3 * 2 * 96 * 16
    with pytest.raises(ValueError):
        X16Matrix(_dm(orc.synth_matrix(64, 64, seed=2, M=4)))


@pytest.mark.parametrize("R,C,books", [(1200, 3608, 1), (700, 6152, 2)])
def test_large_decode_with_the_book_in_shared_memory_equals_the_generic_decode(R, C, books):
    """From 4 M weights on, the benchmark format decodes through the kernel that keeps the book(s) in shared memory:
    bit-equal to the generic kernel (reached through row ranges below the threshold) and, in fp32, to the oracle."""
    m = orc.synth_matrix(R, C, seed=R + books, books=books)
    dm = _dm(m)
    ref = orc.synth_decode(m)
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        whole = dm.dequant(dtype=dt)
        parts = torch.cat([dm.dequant(dtype=dt, rows=(r, min(r + 200, R))) for r in range(0, R, 200)])
        assert torch.equal(whole, parts), dt
        if dt == torch.float32:
            assert np.array_equal(whole.cpu().numpy(), ref)
    big = torch.full((R + 3, C + 8), float("nan"), device="cuda", dtype=torch.bfloat16)      # a row range into a wider scratch
    from quantexperiments_b200 import _lib
    import ctypes
    _lib.check("cbl_dequant", _lib.lib.cbl_dequant(ctypes.byref(dm.struct()), big.data_ptr(), _lib.BF16, C + 8, 0, R,
                                                   torch.cuda.current_stream().cuda_stream))
    assert torch.equal(big[:R, :C], dm.dequant(dtype=torch.bfloat16)) and torch.isnan(big[:R, C:]).all() and torch.isnan(big[R:]).all()
