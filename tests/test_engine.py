"""GPU tests of the decode-step operators and the engine built on them, against a plain torch fp32
restatement of one Qwen2 decode step (weights decoded by the CPU oracle). The restatement rounds to the
model's 16-bit type at the same places as the reference engine (shapequant/kernels/decode_e2e.py:63-309),
so the operator tests are tight (a 16-bit ulp) and the end-to-end logits agree to 2e-2 of their range."""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import cbl_oracle as orc

pytestmark = pytest.mark.gpu


def _lib():
    from quantexperiments_b200 import _lib
    return _lib


def _dt(t):
    from quantexperiments_b200.kernels import _dt
    return _dt(t)


def _s():
    return torch.cuda.current_stream().cuda_stream


def _dense(lin) -> torch.Tensor:
    """fp32 [R, C] weight of a PackedLinear from the oracle's decode of its file-layout tensors."""
    dm = lin.dm
    tags = orc.unpack_bits(dm.tags.cpu().numpy(), dm.bits, dm.nch)
    perms = dm.perms.cpu().numpy() if dm.M > 1 else np.arange(dm.C)[None]
    mask = dm.row_mask.cpu().numpy() if dm.M > 1 else None
    if dm.books == 2:
        tb = orc.unpack_bits(dm.tags2.cpu().numpy(), dm.bits, dm.nch)
        u = orc.additive_decode(dm.table.cpu().numpy(), dm.table2.cpu().numpy(), tags, tb, dm.row_scale.cpu().numpy())
        idx = perms[mask.astype(np.int64)] if mask is not None else np.broadcast_to(perms[:1], u.shape)
        w = np.empty_like(u)
        np.put_along_axis(w, idx, u, axis=1)
    else:
        w = orc.decode_tensors(tags, dm.table.cpu().numpy(), dm.row_scale.cpu().numpy(), None, mask, perms, dm.K)
    return torch.from_numpy(w).cuda()


# ------------------------------------------------------------------------------------------- operators
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H", [(1, 3584), (5, 512), (3, 1000)])
def test_add_rmsnorm(dtype, B, H):
    L = _lib()
    g = torch.Generator(device="cuda").manual_seed(B * H)
    h = torch.randn(B, H, device="cuda", generator=g) * 3
    add = torch.randn(B, H, device="cuda", generator=g).to(dtype)
    w = (torch.randn(H, device="cuda", generator=g) * 0.1 + 1).to(dtype)
    x = torch.empty(B, H, device="cuda", dtype=dtype)
    h0 = h.clone()
    L.check("cbl_add_rmsnorm", L.lib.cbl_add_rmsnorm(h.data_ptr(), add.data_ptr(), H, w.data_ptr(), _dt(dtype), 1e-6, B, H, x.data_ptr(), _s()))
    hr = h0 + add.float()
    assert torch.equal(h, hr)
    xr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert ((x.float() - xr).abs() <= xr.abs() * ulp * 1.01 + 1e-6).all()
    # without an addend the residual is left as it is
    L.check("cbl_add_rmsnorm", L.lib.cbl_add_rmsnorm(h.data_ptr(), None, 0, w.data_ptr(), _dt(dtype), 1e-6, B, H, x.data_ptr(), _s()))
    assert torch.equal(h, hr)


def _rope_ref(x, p, theta, dtype):
    """x [..., HD] fp32 (already rounded to dtype), position p -> rotated, rounded to dtype (fp32 values)."""
    HD = x.shape[-1]
    i = torch.arange(HD // 2, device=x.device, dtype=torch.float32)
    inv = 1.0 / torch.pow(torch.tensor(theta, device=x.device), 2 * i / HD)
    ang = float(p) * inv
    c, s = torch.cos(ang).to(dtype).float(), torch.sin(ang).to(dtype).float()
    x1, x2 = x[..., :HD // 2], x[..., HD // 2:]
    return torch.cat([(x1 * c - x2 * s).to(dtype).float(), (x2 * c + x1 * s).to(dtype).float()], -1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rope_and_cache_write_decode_and_prefill_forms(dtype):
    L = _lib()
    NH, NKV, HD, max_len, B = 6, 2, 128, 40, 3
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, (NH + 2 * NKV) * HD + 8, device="cuda", generator=g).to(dtype)       # padded rows: ld > width
    bias = (torch.randn((NH + 2 * NKV) * HD, device="cuda", generator=g) * 0.1).to(dtype)
    pos = torch.tensor([0, 7, 39], dtype=torch.int32, device="cuda")
    qo = torch.zeros(B, NH * HD, device="cuda", dtype=dtype)
    kc = torch.zeros(B, NKV, max_len, HD, device="cuda", dtype=dtype)
    vc = torch.zeros(B, NKV, HD, max_len, device="cuda", dtype=dtype)          # values are cached dimension-major
    L.check("cbl_rope_kv", L.lib.cbl_rope_kv(qkv.data_ptr(), _dt(dtype), qkv.stride(0), bias.data_ptr(), pos.data_ptr(), 0, 0, B, NH, NKV, HD, 1e6,
                                             max_len, qo.data_ptr(), kc.data_ptr(), vc.data_ptr(), _s()))
    xb = (qkv[:, :(NH + 2 * NKV) * HD].float() + bias.float()).to(dtype).float()
    tol = dict(rtol=2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10, atol=1e-3)
    for b in range(B):
        p = int(pos[b])
        q = _rope_ref(xb[b, :NH * HD].view(NH, HD), p, 1e6, dtype)
        k = _rope_ref(xb[b, NH * HD:(NH + NKV) * HD].view(NKV, HD), p, 1e6, dtype)
        v = xb[b, (NH + NKV) * HD:].view(NKV, HD)
        torch.testing.assert_close(qo[b].float().view(NH, HD), q, **tol)
        torch.testing.assert_close(kc[b, :, p].float(), k, **tol)
        assert torch.equal(vc[b, :, :, p].float(), v)
        untouched = torch.ones(max_len, dtype=torch.bool, device="cuda")
        untouched[p] = False
        assert not kc[b][:, untouched].any() and not vc[b][:, :, untouched].any()
    # prefill form: rows are consecutive positions of one sequence
    kc.zero_(), vc.zero_()
    L.check("cbl_rope_kv", L.lib.cbl_rope_kv(qkv.data_ptr(), _dt(dtype), qkv.stride(0), None, None, 4, 1, B, NH, NKV, HD, 1e6, max_len,
                                             qo.data_ptr(), kc.data_ptr(), vc.data_ptr(), _s()))
    x0 = qkv[:, :(NH + 2 * NKV) * HD].float()
    for r in range(B):
        k = _rope_ref(x0[r, NH * HD:(NH + NKV) * HD].view(NKV, HD), 4 + r, 1e6, dtype)
        torch.testing.assert_close(kc[1, :, 4 + r].float(), k, **tol)
    assert not kc[0].any() and not kc[2].any()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("NH,NKV,B,max_len,nsplit,poss", [
    (28, 4, 1, 2304, 74, [2047]), (28, 4, 3, 320, 9, [0, 1, 299]), (8, 8, 2, 64, 1, [31, 63]), (40, 8, 2, 4096, 4, [4095, 100]),
    (4, 2, 4, 128, 7, [5, 64, 127, 33])])
def test_decode_attention_matches_softmax_attention(dtype, NH, NKV, B, max_len, nsplit, poss):
    L = _lib()
    HD = 128
    g = torch.Generator(device="cuda").manual_seed(NH * B + max_len)
    q = torch.randn(B, NH * HD, device="cuda", generator=g).to(dtype)
    kc = torch.randn(B, NKV, max_len, HD, device="cuda", generator=g).to(dtype)
    vc = torch.randn(B, NKV, HD, max_len, device="cuda", generator=g).to(dtype)          # dimension-major value cache
    pos = torch.tensor(poss, dtype=torch.int32, device="cuda")
    out = torch.zeros(B, NH * HD, device="cuda", dtype=dtype)
    ws = torch.full((L.lib.cbl_attn_decode_workspace_bytes(B, NH, nsplit),), 0xFF, dtype=torch.uint8, device="cuda")      # NaN patterns: nothing stale is read
    assert nsplit <= L.lib.cbl_attn_decode_max_splits()
    for _ in range(2):          # the work space is reusable as it is left
        L.check("cbl_attn_decode", L.lib.cbl_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), _dt(dtype), B, NH, NKV, HD,
                                                         max_len, HD ** -0.5, out.data_ptr(), ws.data_ptr(), nsplit, _s()))
    torch.cuda.synchronize()
    rep = NH // NKV
    for b in range(B):
        n = poss[b] + 1
        k = kc[b, :, :n].float().repeat_interleave(rep, 0)          # [NH, n, HD]
        v = vc[b, :, :, :n].float().transpose(1, 2).repeat_interleave(rep, 0)
        sc = torch.einsum("hd,hnd->hn", q[b].float().view(NH, HD), k) * HD ** -0.5
        ref = torch.einsum("hn,hnd->hd", torch.softmax(sc, -1), v)
        err = (out[b].float().view(NH, HD) - ref).abs().max() / ref.abs().max()
        # the probabilities enter the tensor-core value product rounded to the 16-bit type, the output is rounded once more
        assert err <= 2 * (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11) + 1e-4, (b, float(err))


def test_decode_attention_clamps_positions_beyond_the_cache():
    """pos = max_len (a caller that stepped one past the cache) reads nothing outside it: the result is the attention
    over the whole cache, exactly what pos = max_len - 1 gives."""
    L = _lib()
    NH, NKV, HD, max_len, B = 8, 2, 128, 96, 2
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn(B, NH * HD, device="cuda", generator=g).bfloat16()
    kc = torch.randn(B, NKV, max_len, HD, device="cuda", generator=g).bfloat16()
    vc = torch.randn(B, NKV, HD, max_len, device="cuda", generator=g).bfloat16()
    ws = torch.zeros(L.lib.cbl_attn_decode_workspace_bytes(B, NH, 3), dtype=torch.uint8, device="cuda")
    outs = []
    for p in ([max_len - 1, max_len - 1], [max_len, max_len + 1000]):
        pos = torch.tensor(p, dtype=torch.int32, device="cuda")
        out = torch.zeros(B, NH * HD, device="cuda", dtype=torch.bfloat16)
        L.check("cbl_attn_decode", L.lib.cbl_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), _dt(torch.bfloat16), B, NH, NKV,
                                                         HD, max_len, HD ** -0.5, out.data_ptr(), ws.data_ptr(), 3, _s()))
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


def test_decode_attention_rejects_too_many_slices_and_odd_shapes():
    L = _lib()
    t = torch.zeros(16, device="cuda")
    args = lambda NH, NKV, HD, max_len, ns: (t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 2, 1, NH, NKV, HD, max_len, 1.0,  # noqa: E731
                                             t.data_ptr(), t.data_ptr(), ns, _s())
    assert L.lib.cbl_attn_decode(*args(4, 2, 128, 4096, 129)) == L.EUNSUPPORTED  # at most 128 slices
    assert L.lib.cbl_attn_decode(*args(4, 2, 128, 100, 1)) == L.EINVAL           # cache length not a multiple of 32
    assert L.lib.cbl_attn_decode(*args(4, 2, 64, 128, 1)) == L.EUNSUPPORTED
    assert L.lib.cbl_attn_decode(*args(18, 2, 128, 128, 1)) == L.EUNSUPPORTED    # 9 query heads per kv head
    assert L.lib.cbl_attn_decode(*args(5, 2, 128, 128, 1)) == L.EUNSUPPORTED


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_mul_embed_head_and_argmax(dtype):
    L = _lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    B, I = 3, 1000
    gu = (torch.randn(B, 2 * I + 8, device="cuda", generator=g) * 3).to(dtype)
    out = torch.empty(B, I, device="cuda", dtype=dtype)
    L.check("cbl_silu_mul", L.lib.cbl_silu_mul(gu.data_ptr(), _dt(dtype), gu.stride(0), B, I, out.data_ptr(), _s()))
    a = gu[:, :I].float()
    ref = ((a * torch.sigmoid(a)).to(dtype).float() * gu[:, I:2 * I].float()).to(dtype)
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10          # the kernel's exp may differ from torch's in the last place
    assert ((out.float() - ref.float()).abs() <= ref.float().abs() * ulp + 1e-6).all()
    # embedding rows (token ids wrap around the table like the reference's `% rows`)
    V, H = 777, 264
    E = torch.randn(V, H, device="cuda", generator=g).to(dtype)
    tok = torch.tensor([5, 776, 777 + 3], dtype=torch.int64, device="cuda")
    h = torch.empty(3, H, device="cuda")
    L.check("cbl_embed_rows", L.lib.cbl_embed_rows(E.data_ptr(), _dt(dtype), V, H, tok.data_ptr(), 3, h.data_ptr(), _s()))
    assert torch.equal(h, E[[5, 776, 3]].float())
    # head for every supported batch, fp32 and 16-bit logits
    for Bh in (1, 2, 5, 8):
        x = torch.randn(Bh, H, device="cuda", generator=g).to(dtype)
        for ldt in (torch.float32, dtype):
            lg = torch.zeros(Bh, V + 3, device="cuda", dtype=ldt)
            L.check("cbl_head_gemv", L.lib.cbl_head_gemv(E.data_ptr(), x.data_ptr(), _dt(dtype), Bh, V, H, lg.data_ptr(), _dt(ldt), lg.stride(0), _s()))
            ref = x.float() @ E.float().t()
            tol = 1e-4 + (0.0 if ldt == torch.float32 else (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11))
            assert (lg[:, :V].float() - ref).abs().max() / ref.abs().max() <= tol
            assert not lg[:, V:].any()
    assert L.lib.cbl_head_gemv(E.data_ptr(), E.data_ptr(), _dt(dtype), 9, V, H, h.data_ptr(), 0, V, _s()) == L.EUNSUPPORTED
    # argmax: first of equal maxima, position counter advanced
    lg = torch.randn(4, 5000, device="cuda", generator=g)
    lg[1, 4321] = 50.0
    lg[2, 77] = lg[2, 4000] = 60.0
    lg[3] = -float("inf")
    tk = torch.zeros(4, dtype=torch.int64, device="cuda")
    pos = torch.tensor([0, 10, 20, 30], dtype=torch.int32, device="cuda")
    L.check("cbl_argmax", L.lib.cbl_argmax(lg.data_ptr(), 0, lg.stride(0), 4, 5000, tk.data_ptr(), pos.data_ptr(), _s()))
    assert tk.tolist() == [int(lg[0].argmax()), 4321, 77, 0]
    assert pos.tolist() == [1, 11, 21, 31]


def _rand_lin(R, C, g, books=1):
    from quantexperiments_b200.linear import PackedLinear
    W = (C // 8 * 12 + 31) // 32
    mk = lambda: torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g)      # noqa: E731
    tb = lambda: torch.randn(4096, 8, device="cuda", generator=g).half()                                         # noqa: E731
    rs = ((torch.rand(R, device="cuda", generator=g) * 0.5 + 0.75) / math.sqrt(C * books)).half()
    kw = dict(words2=mk(), table2=tb()) if books == 2 else {}
    return PackedLinear(mk(), tb(), rs, None, None, torch.arange(C, device="cuda")[None], 4096, 8, **kw)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("books", [1, 2])
def test_fused_epilogues_equal_the_product_followed_by_the_operator(dtype, books):
    """cbl_gemv_l8_silu_mul / _add_norm / _rope_kv against cbl_gemv_l8_multi + the separate operators."""
    import ctypes
    from quantexperiments_b200.kernels import L8Group, l8_workspace
    L = _lib()
    g = torch.Generator(device="cuda").manual_seed(21 + books)
    dtc, s = _dt(dtype), _s()
    ws = l8_workspace(torch.device("cuda", 0), 0, 4 * L.lib.cbl_gemv_l8_workspace_bytes(8192)).data_ptr()
    # gate | up -> silu * up   (row count not a multiple of 4: padded accumulator rows)
    C, I = 520, 2050
    gate, up = _rand_lin(I, C, g, books), _rand_lin(I, C, g, books)
    x = torch.randn(C, device="cuda", generator=g).to(dtype)
    grp = L8Group([gate.l8, up.l8])
    ygu = torch.empty(2 * I, device="cuda", dtype=dtype)
    grp.run(x, [ygu[:I], ygu[I:]])
    ref = torch.empty(1, I, device="cuda", dtype=dtype)
    L.check("cbl_silu_mul", L.lib.cbl_silu_mul(ygu.data_ptr(), dtc, 2 * I, 1, I, ref.data_ptr(), s))
    out = torch.zeros(I, device="cuda", dtype=dtype)
    # the product's partial sums meet in memory in any order, so two runs may differ in the last place of the
    # 16-bit product; everything after it is the same arithmetic
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11

    def close(a, b, n=4):
        a, b = a.float(), b.float()
        return bool(((a - b).abs() <= n * ulp * b.abs().max()).all()) and float((a - b).abs().mean()) <= 0.05 * ulp * float(b.abs().max())

    for _ in range(2):          # the work space is left zero: a second call gives the same result
        L.check("cbl_gemv_l8_silu_mul", L.lib.cbl_gemv_l8_silu_mul(grp._structs, x.data_ptr(), dtc, out.data_ptr(), None, None, dtc, ws, s))
        assert close(out, ref[0])
    # the two products themselves on request, and the reference-named surface RunsLin.run(x, y, epi=...)
    ykeep = torch.zeros(2 * I, device="cuda", dtype=dtype)
    L.check("cbl_gemv_l8_silu_mul", L.lib.cbl_gemv_l8_silu_mul(grp._structs, x.data_ptr(), dtc, out.data_ptr(), ykeep.data_ptr(),
                                                                ykeep.data_ptr() + I * ykeep.element_size(), dtc, ws, s))
    assert torch.equal(ykeep, ygu)                    # products are bit-reproducible: the fused launch rounds the same sums
    from quantexperiments_b200.linear import RunsLin
    rg, ru = RunsLin(gate), RunsLin(up)
    y2, o2 = torch.zeros(2 * I, device="cuda", dtype=dtype), torch.zeros(I, device="cuda", dtype=dtype)
    rg.run(x, y2, epi={"mode": 2, "up": ru, "out": o2})
    assert torch.equal(y2, ygu) and torch.equal(o2, out)
    with pytest.raises(ValueError):
        rg.run(x, y2, epi={"mode": 2, "up": ru, "out": o2, "perms": torch.zeros(1, I)})
    # down -> add + norm   (R = 3584: four finish blocks in one cluster; and a single-block case)
    for R, Cd in ((3584, 1032), (520, 264), (8192, 64)):
        down = _rand_lin(R, Cd, g, books)
        xd = torch.randn(Cd, device="cuda", generator=g).to(dtype)
        h0 = torch.randn(1, R, device="cuda", generator=g) * 2
        w = (torch.randn(R, device="cuda", generator=g) * 0.1 + 1).to(dtype)
        y = down.l8.run(xd, torch.empty(R, device="cuda", dtype=dtype))
        h_ref, x_ref = h0.clone(), torch.empty(1, R, device="cuda", dtype=dtype)
        L.check("cbl_add_rmsnorm", L.lib.cbl_add_rmsnorm(h_ref.data_ptr(), y.data_ptr(), R, w.data_ptr(), dtc, 1e-6, 1, R, x_ref.data_ptr(), s))
        h, xo = h0.clone(), torch.zeros(R, device="cuda", dtype=dtype)
        st = (L.L8 * 1)(down.l8.struct())
        L.check("cbl_gemv_l8_add_norm", L.lib.cbl_gemv_l8_add_norm(st, xd.data_ptr(), dtc, h.data_ptr(), w.data_ptr(), 1e-6, xo.data_ptr(), None, dtc, ws, s))
        assert close(h, h_ref[0]) and close(xo, x_ref[0])
        if R >= 2048:               # the same through RunsLin.run(x, y, epi={mode 1}): h_out = h_in + y, out = norm(h_out) * w, y kept
            hi, ho = h0[0].clone(), torch.zeros(R, device="cuda")
            yk, ok = torch.zeros(R, device="cuda", dtype=dtype), torch.zeros(R, device="cuda", dtype=dtype)
            RunsLin(down).run(xd, yk, epi={"mode": 1, "h_in": hi, "h_out": ho, "w": w, "eps": 1e-6, "out": ok, "src": yk})
            assert torch.equal(yk, y) and torch.equal(hi, h0[0]) and torch.equal(ho, h.reshape(-1)) and torch.equal(ok, xo)
    assert L.lib.cbl_gemv_l8_add_norm_max_rows() == 8192
    # q | k | v -> bias, rotary, cache write
    NH, NKV, HD, max_len, Cq = 6, 2, 128, 24, 264
    q, k, v = _rand_lin(NH * HD, Cq, g, books), _rand_lin(NKV * HD, Cq, g, books), _rand_lin(NKV * HD, Cq, g, books)
    xq = torch.randn(Cq, device="cuda", generator=g).to(dtype)
    bias = (torch.randn((NH + 2 * NKV) * HD, device="cuda", generator=g) * 0.1).to(dtype)
    grp = L8Group([q.l8, k.l8, v.l8])
    yqkv = torch.empty(1, (NH + 2 * NKV) * HD, device="cuda", dtype=dtype)
    grp.run(xq, [yqkv[0, :NH * HD], yqkv[0, NH * HD:(NH + NKV) * HD], yqkv[0, (NH + NKV) * HD:]])
    for with_bias in (True, False):
        pos = torch.tensor([17], dtype=torch.int32, device="cuda")
        bp = bias.data_ptr() if with_bias else None
        q_ref, kc_ref, vc_ref = (torch.zeros(1, NH * HD, device="cuda", dtype=dtype), torch.zeros(1, NKV, max_len, HD, device="cuda", dtype=dtype),
                                 torch.zeros(1, NKV, HD, max_len, device="cuda", dtype=dtype))
        L.check("cbl_rope_kv", L.lib.cbl_rope_kv(yqkv.data_ptr(), dtc, yqkv.stride(0), bp, pos.data_ptr(), 0, 0, 1, NH, NKV, HD, 1e6, max_len,
                                                 q_ref.data_ptr(), kc_ref.data_ptr(), vc_ref.data_ptr(), s))
        qo, kc, vc = torch.zeros_like(q_ref), torch.zeros_like(kc_ref), torch.zeros_like(vc_ref)
        L.check("cbl_gemv_l8_rope_kv", L.lib.cbl_gemv_l8_rope_kv(grp._structs, xq.data_ptr(), dtc, bp, pos.data_ptr(), NH, NKV, HD, 1e6, max_len,
                                                                 qo.data_ptr(), kc.data_ptr(), vc.data_ptr(), dtc, ws, s))
        assert close(qo, q_ref) and close(kc, kc_ref) and close(vc, vc_ref)
        assert kc[0, :, 17].any() and vc[0, :, :, 17].any()
    # shapes the fused forms refuse
    assert L.lib.cbl_gemv_l8_rope_kv(grp._structs, xq.data_ptr(), dtc, None, pos.data_ptr(), NH + 1, NKV, HD, 1e6, max_len, qo.data_ptr(),
                                     kc.data_ptr(), vc.data_ptr(), dtc, ws, s) == L.EINVAL
    seg = (ctypes.c_int32 * (L.L8_MAX_ORDERS + 1))(0, 8224)
    big = (L.L8 * 1)(L.L8(8196, 64, 1, 1, 8224, 1, 1, 0, 16, 16, None, 16, None, None, None, None, seg, 0))
    assert L.lib.cbl_gemv_l8_add_norm(big, xq.data_ptr(), dtc, h.data_ptr(), w.data_ptr(), 1e-6, xo.data_ptr(), None, dtc, ws, s) == L.EUNSUPPORTED


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_block32_embedding_rows_and_head_match_the_oracle(dtype):
    """cbl_embed_rows_q4 (exact) and cbl_head_gemv_q8 (fp32 matmul on the oracle's dequantized weights)."""
    from quantexperiments_b200.engine import Q4Embed, Q8Head
    L = _lib()
    g = torch.Generator().manual_seed(4)
    V, H = 777, 1056
    w = (torch.randn(V, H, generator=g) * 0.02).to(dtype).float()
    w[5, 64:96] = 0.0
    w[9, 3] = 2.0
    q4, s4 = orc.q4_embed_pack(w.numpy())
    emb = Q4Embed(torch.from_numpy(q4).cuda(), torch.from_numpy(s4).cuda(), dtype)
    tok = torch.tensor([5, 776, 777 + 9, 0], dtype=torch.int64, device="cuda")
    h = torch.empty(4, H, device="cuda")
    L.check("cbl_embed_rows_q4", L.lib.cbl_embed_rows_q4(emb.q.data_ptr(), emb.sc.data_ptr(), V, H, tok.data_ptr(), 4, h.data_ptr(), _s()))
    ref = orc.q4_embed_rows(q4, s4, np.array([5, 776, 9, 0]))
    assert np.array_equal(h.cpu().numpy(), ref)
    assert np.array_equal(emb.rows(torch.tensor([5, 776, 9, 0], device="cuda")).cpu().numpy(), ref)
    q8, s8, deq = orc.q8_pack(w.numpy())
    head = Q8Head(torch.from_numpy(q8).cuda(), torch.from_numpy(s8).cuda())
    assert head.nbytes() == V * H + V * H // 32 * 2
    wd = torch.from_numpy(deq).cuda()
    for B in (1, 3, 8, 11):             # more than 8 sequences: several passes
        x = torch.randn(B, H, generator=g).to(dtype).cuda()
        lgv = torch.zeros(B, V, device="cuda")
        head.run(x, lgv)
        r = x.float() @ wd.t()
        assert (lgv - r).abs().max() / r.abs().max() <= 1e-5          # int8 weights and 16-bit activations are exact in the fp16 MMAs
    # a 16-bit logits buffer with a wider row stride, through the C ABI
    x = torch.randn(2, H, generator=g).to(dtype).cuda()
    lg = torch.zeros(2, V + 3, device="cuda", dtype=dtype)
    sc = torch.empty(L.lib.cbl_head_q8_scratch_bytes(2, H), dtype=torch.uint8, device="cuda")
    L.check("cbl_head_gemv_q8", L.lib.cbl_head_gemv_q8(head.q.data_ptr(), head.sc.data_ptr(), x.data_ptr(), _dt(dtype), 2, V, H, lg.data_ptr(),
                                                       _dt(dtype), lg.stride(0), sc.data_ptr(), _s()))
    r = x.float() @ wd.t()
    assert (lg[:, :V].float() - r).abs().max() / r.abs().max() <= (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11) + 1e-5
    assert not lg[:, V:].any()
    assert L.lib.cbl_head_gemv_q8(head.q.data_ptr(), head.sc.data_ptr(), x.data_ptr(), _dt(dtype), 9, V, H, lg.data_ptr(), _dt(dtype), lg.stride(0),
                                  sc.data_ptr(), _s()) == L.EUNSUPPORTED
    assert L.lib.cbl_embed_rows_q4(emb.q.data_ptr(), emb.sc.data_ptr(), V, 40, tok.data_ptr(), 4, h.data_ptr(), _s()) == L.EINVAL


# ------------------------------------------------------------------------------------------- the engine
class _RefModel:
    """One Qwen2 decode step in plain torch (fp32 math, 16-bit rounding where the engine rounds)."""

    def __init__(self, eng):
        self.e, self.c, self.dt = eng, eng.cfg, eng.dtype
        self.W = [{n: _dense(L[n]) for n in ("q", "k", "v", "o", "gate", "up", "down")} for L in eng.layers]
        self.k = [[] for _ in eng.layers]      # per layer: list of [NKV, HD] per position
        self.v = [[] for _ in eng.layers]

    def r(self, x):
        return x.to(self.dt).float()

    def norm(self, h, w):
        return self.r(h * torch.rsqrt(h.pow(2).mean() + self.c.eps) * w.float())

    def step(self, tok: int, p: int) -> torch.Tensor:
        e, c = self.e, self.c
        NH, NKV, HD = c.n_heads, c.n_kv, c.head_dim
        from quantexperiments_b200.engine import Q4Embed, Q8Head
        from quantexperiments_b200.packed import q8_rows
        h = e.embed.rows(torch.tensor([tok], device="cuda"))[0] if isinstance(e.embed, Q4Embed) else e.embed[tok].float()
        for li, (L, W) in enumerate(zip(e.layers, self.W)):
            x = self.norm(h, L["ln1"])
            q, k, v = self.r(W["q"] @ x), self.r(W["k"] @ x), self.r(W["v"] @ x)
            if L.get("bq") is not None:
                q, k, v = self.r(q + L["bq"].float()), self.r(k + L["bk"].float()), self.r(v + L["bv"].float())
            q = _rope_ref(q.view(NH, HD), p, c.rope_theta, self.dt)
            self.k[li].append(_rope_ref(k.view(NKV, HD), p, c.rope_theta, self.dt))
            self.v[li].append(v.view(NKV, HD))
            K = torch.stack(self.k[li], 1).repeat_interleave(NH // NKV, 0)      # [NH, n, HD]
            V = torch.stack(self.v[li], 1).repeat_interleave(NH // NKV, 0)
            sc = torch.einsum("hd,hnd->hn", q, K) * HD ** -0.5
            ao = self.r(torch.einsum("hn,hnd->hd", torch.softmax(sc, -1), V).reshape(-1))
            h = h + self.r(W["o"] @ ao)
            x = self.norm(h, L["ln2"])
            g, u = self.r(W["gate"] @ x), self.r(W["up"] @ x)
            act = self.r(self.r(g * torch.sigmoid(g)) * u)
            h = h + self.r(W["down"] @ act)
        x = self.norm(h, e.final_norm)
        wh = q8_rows(e.lm_head.q, e.lm_head.sc) if isinstance(e.lm_head, Q8Head) else e.lm_head.w.float()
        return wh @ x


def _small_cfg(max_len=96):
    from quantexperiments_b200.engine import Cfg
    return Cfg(hidden=512, n_heads=4, n_kv=2, head_dim=128, inter=2048, vocab=1000, layers=2, rope_theta=1e6, eps=1e-6, max_len=max_len)


@pytest.mark.parametrize("dtype,books,M", [(torch.bfloat16, 1, 1), (torch.float16, 1, 1), (torch.bfloat16, 2, 4)])
def test_engine_steps_match_the_torch_restatement(dtype, books, M):
    from quantexperiments_b200.engine import random_engine
    eng = random_engine(_small_cfg(), seed=5, dtype=dtype, books=books, M=M)
    ref = _RefModel(eng)
    toks = [3, 999, 17, 256, 42, 7]
    eng.reset(toks[0])
    for p, t in enumerate(toks):
        eng.tok.fill_(t)
        eng.step()
        lr = ref.step(t, p)
        err = (eng.logits[0] - lr).abs().max() / lr.abs().max()
        assert err <= 2e-2, (p, float(err))
        assert int(eng.pos[0]) == p + 1
        assert int(eng.tok[0]) == int(eng.logits[0].argmax())
    eng.check()
    assert eng.fused == (M == 1)
    if eng.fused:
        # the same steps with every operator as its own kernel
        lg = eng.logits.clone()
        eng.fused = False
        eng.reset(toks[0])
        for t in toks:
            eng.tok.fill_(t)
            eng.step()
        assert (eng.logits - lg).abs().max() / lg.abs().max() <= 2e-2      # 16-bit roundings flip with the order of the partial sums


def test_engine_graph_replay_prefill_and_batched_engine_agree():
    from quantexperiments_b200.engine import Qwen2BatchEngine, generate, random_engine
    eng = random_engine(_small_cfg(max_len=160), seed=9)
    prompt = torch.randint(0, 1000, (70,), generator=torch.Generator().manual_seed(1)).tolist()      # > 64 tokens: the GEMM path
    # eager token-by-token feed of the prompt, then greedy continuation
    eng.reset(prompt[0])
    for i, t in enumerate(prompt):
        eng.tok.fill_(t)
        eng.step()
    lg_feed = eng.logits[0].clone()
    cont = [int(eng.tok[0])]
    for _ in range(7):
        eng.step()
        cont.append(int(eng.tok[0]))
    # batched prefill + CUDA-graph replay gives the same logits (to rounding) and the same greedy tokens
    eng.reset(0)
    lg_pre = eng.prefill(prompt)
    assert int(eng.pos[0]) == len(prompt)
    assert (lg_pre - lg_feed).abs().max() / lg_feed.abs().max() <= 2e-2
    out = generate(eng, prompt, 8, graph=True)
    agree = sum(a == b for a, b in zip(out, cont))
    assert agree >= 6, (out, cont)          # near-ties may flip a late token; the logits test above is the strict one
    eng.check()
    # batched engine on the same weights: every sequence fed the same tokens reproduces the batch-1 logits
    B = 3
    beng = Qwen2BatchEngine(eng, B)
    beng.reset(prompt[0])
    for t in prompt[:12]:
        beng.tok.fill_(t)
        beng.step()
    eng.reset(prompt[0])
    for t in prompt[:12]:
        eng.tok.fill_(t)
        eng.step()
    for b in range(B):
        assert (beng.logits[b] - eng.logits[0]).abs().max() / eng.logits[0].abs().max() <= 2e-2
    assert beng.pos.tolist() == [12] * B
    # twenty sequences: the products run on the tensor-core kernel with the weight rows as the M side
    b20 = Qwen2BatchEngine(eng, 20)
    assert b20.stages[0]["qkv"].rows is not None
    b20.reset(prompt[0])
    for t in prompt[:12]:
        b20.tok.fill_(t)
        b20.step()
    for b in (0, 7, 19):
        assert (b20.logits[b] - eng.logits[0]).abs().max() / eng.logits[0].abs().max() <= 2e-2
    b20.check()
    # sequences at different positions: prefill two prompts of different lengths, then step both
    beng.reset(0)
    beng.prefill(prompt[:40], 0)
    beng.prefill(prompt[:9], 1)
    beng.prefill(prompt[:1], 2)
    beng.step()
    assert beng.pos.tolist() == [41, 10, 2]
    eng.reset(0)
    eng.prefill(prompt[:9])
    eng.step()
    assert (beng.logits[1] - eng.logits[0]).abs().max() / eng.logits[0].abs().max() <= 2e-2
    beng.check()


def test_engine_with_the_8bit_head_and_the_4bit_embedding():
    from quantexperiments_b200.engine import Q4Embed, Q8Head, Qwen2BatchEngine, random_engine
    eng = random_engine(_small_cfg(), seed=6, head="q8", embed="q4")
    assert isinstance(eng.embed, Q4Embed) and isinstance(eng.lm_head, Q8Head)
    ref = _RefModel(eng)
    toks = [3, 999, 17, 256]
    eng.reset(toks[0])
    for p, t in enumerate(toks):
        eng.tok.fill_(t)
        eng.step()
        lr = ref.step(t, p)
        assert (eng.logits[0] - lr).abs().max() / lr.abs().max() <= 2e-2, p
    lg1 = eng.logits[0].clone()
    # prompt path and batched engine on the same formats
    eng.reset(0)
    lgp = eng.prefill(toks)
    assert (lgp - lg1).abs().max() / lg1.abs().max() <= 2e-2
    b6 = Qwen2BatchEngine(eng, 6)
    b6.reset(toks[0])
    for t in toks:
        b6.tok.fill_(t)
        b6.step()
    for b in range(6):
        assert (b6.logits[b] - lg1).abs().max() / lg1.abs().max() <= 2e-2
    assert eng.weight_bytes() < random_engine(_small_cfg(), seed=6).weight_bytes()


def test_engine_rejects_unsupported_shapes():
    from quantexperiments_b200.engine import Cfg, random_engine
    with pytest.raises(ValueError):
        random_engine(Cfg(hidden=256, n_heads=4, n_kv=2, head_dim=64, inter=512, vocab=100, layers=1, max_len=32))
    eng = random_engine(_small_cfg(max_len=32), seed=1)
    with pytest.raises(ValueError):
        eng.prefill(list(range(40)))


@pytest.mark.parametrize("feed", ["prefill", "steps"])
def test_engine_logits_match_a_hugging_face_qwen2_with_reference_decoded_weights(feed):
    """The pin of the decode engine, as the reference pins its own (tests/test_runtime.py:18-89): a tiny random Hugging
    Face Qwen2 (CPU, fp32, eager attention) whose block linears are codebook matrices decoded by the reference wrote
    the logits of 14 positions into tests/golden/engine_hf.npz; the same model, rebuilt here in the packed format from
    the same seeds, must reproduce them (relative error of the logit vectors < 2e-2, the reference's bound), fed
    either as one batched prefill per prefix or token by token through the decode step."""
    import sys
    from pathlib import Path
    gold = Path(__file__).resolve().parent / "golden"
    sys.path.insert(0, str(gold))
    import tiny_qwen2 as tq
    from quantexperiments_b200.engine import Cfg, DecodeEngine, DenseHead
    from quantexperiments_b200.linear import PackedLinear
    z = np.load(gold / "engine_hf.npz")
    tokens, want = [int(t) for t in z["tokens"]], torch.from_numpy(z["logits"])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()          # noqa: E731
    st = tq.small_tensors()
    layers = []
    for li in range(tq.NL):
        L = {"ln1": t(st[f"ln1_{li}"]), "ln2": t(st[f"ln2_{li}"]), "bq": t(st[f"bq_{li}"]), "bk": t(st[f"bk_{li}"]), "bv": t(st[f"bv_{li}"])}
        for n in tq.LINEARS:
            m = tq.matrix(li, n)
            L[n] = PackedLinear(t(m["words"][0]), t(m["table"][0]), t(m["row_scale"]), None, None, t(m["perms"]).long(), 4096, 8)
        layers.append(L)
    cfg = Cfg(hidden=tq.H, n_heads=tq.NH, n_kv=tq.NKV, head_dim=tq.HD, inter=tq.I, vocab=tq.V, layers=tq.NL, rope_theta=tq.THETA,
              eps=tq.EPS, max_len=tq.MAX_LEN)
    eng = DecodeEngine(cfg, t(st["embed"]), layers, t(st["final_norm"]), DenseHead(t(st["head"])))
    got = []
    if feed == "prefill":
        for n in range(1, len(tokens) + 1):               # the logits of position n - 1 = last position of the prefix of n tokens
            eng.reset(0)
            got.append(eng.prefill(torch.tensor(tokens[:n], device="cuda"), 0).float().cpu())
    else:
        eng.reset(tokens[0])
        for i, tok in enumerate(tokens):
            eng.tok.fill_(tok)                            # teacher forcing: the step reads tok at pos, leaves the logits, advances pos
            eng.step()
            got.append(eng.logits[0].float().cpu().clone())
    eng.check()
    got = torch.stack(got)
    rel = float((got - want).norm() / want.norm())
    assert rel < 2e-2, rel
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() >= 0.9
