"""CPU-only tests: host-side format code against the reference-generated fixtures, and that the C-ABI
library loads and exports every symbol include/cbl.h declares (no compute calls without a GPU)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from quantexperiments_b200 import _lib, packed

ROOT = Path(__file__).resolve().parent.parent
G = ROOT / "tests" / "golden"


def test_library_exports_every_declared_symbol():
    hdr = (ROOT / "include" / "cbl.h").read_text()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(cbl_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 15
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), f"libcbl.so lacks {name}"
    assert declared == set(_lib.SIGNATURES), "ctypes signatures and header disagree"


def test_library_identity_and_status_strings():
    assert _lib.lib.cbl_built_for_sm() == 100
    assert _lib.lib.cbl_version() >= 100
    assert _lib.lib.cbl_status_string(0) == b"ok"
    assert b"unsupported" in _lib.lib.cbl_status_string(_lib.EUNSUPPORTED)


def test_size_queries_match_the_layout_arithmetic():
    lib = _lib.lib
    # t16: [books][ntile][nsuper][3][32] uint4, nsuper = ceil(C/8/64)
    assert lib.cbl_t16_bytes(224, 3584, 1) == 224 * 7 * 3 * 32 * 16
    assert lib.cbl_t16_bytes(10, 896, 2) == 2 * 10 * 2 * 3 * 32 * 16
    # l8: [ntile][3][Rpad] words
    assert lib.cbl_l8_bytes(3584, 3584, 1) == 56 * 3 * 3584 * 4
    assert lib.cbl_l8_bytes(4863, 896, 2) == 2 * 14 * 3 * 4864 * 4
    assert lib.cbl_prep_x_bytes(3, 896, 16) == 16 * 8 * 1024 * 2 + 16 * 8 * 4
    # batch-1 layout: rows padded to 32 positions; work space = int64 + fp32 sums per position, counters, status
    assert lib.cbl_l8r_bytes(3584, 3584, 1) == 56 * 3 * 3584 * 4
    assert lib.cbl_l8r_bytes(4864 + 32, 896, 2) == 2 * 14 * 3 * 4896 * 4
    assert lib.cbl_book_frag_bytes() == 65536 + 16
    # work space: 160 partial-sum slots of 4096 64-bit words, 64 control words, fp32 sums per (padded) row
    assert lib.cbl_gemv_l8_workspace_bytes(18944) == 160 * 4096 * 8 + 256 + (18944 + 512) * 4
    assert lib.cbl_gemv_l8_static_max_rows() == 65536


def _l8_shape(R, C, books=1, seg=None):
    Rpad = (R + 31) // 32 * 32 if seg is None else seg[-1]
    seg = seg or [0, Rpad]
    arr = (ctypes.c_int32 * (_lib.L8_MAX_ORDERS + 1))(*(seg + [0] * (_lib.L8_MAX_ORDERS + 1 - len(seg))))
    return _lib.L8(R, C, books, books * (-(-(C // 8) // 8)), Rpad, 1, len(seg) - 1, 0, None, None, None, None, None, None, None, None, arr, 0)


@pytest.mark.parametrize("shapes,sms", [
    ([(3584, 3584), (512, 3584), (512, 3584)], 148), ([(18944, 3584), (18944, 3584)], 148), ([(3584, 18944)], 148),
    ([(4864, 896)], 148), ([(4, 64)], 148), ([(27648, 5120, 2), (27648, 5120, 2)], 148), ([(3584, 3584)], 20),
    ([(5120, 5120, 2, [0, 320, 672, 960, 1312, 1600, 1952, 2240, 2592, 2880, 3232, 3520, 3872, 4160, 4512, 4800, 5152])], 148),
    ([(70000, 128)], 132)])
def test_batch1_work_split_covers_every_row_and_tile_exactly_once(shapes, sms):
    """The host plan of the table-lookup product: rectangles (row positions x tiles) that partition every
    (matrix, column order); at most 4096 rows per block; one wave of blocks."""
    lib = _lib.lib
    mats = [_l8_shape(*sh) for sh in shapes]
    arr = (_lib.L8 * len(mats))(*mats)
    out = np.zeros((160, 8), np.int32)
    nb = ctypes.c_int32(0)
    assert lib.cbl_gemv_l8_plan(arr, len(mats), sms, out.ctypes.data, ctypes.byref(nb)) == _lib.OK
    assert 1 <= nb.value <= min(sms, 160)
    cover = [np.zeros((m.Rpad // 32, m.ntile), np.int32) for m in mats]
    parts = {}
    for mi, order, part, splits, row0, rows, t0, t1 in out[:nb.value]:
        m = mats[mi]
        assert rows > 0 and rows % 32 == 0 and row0 % 32 == 0 and rows <= 4096 and 0 <= t0 < t1 <= m.ntile
        assert m.seg_off[order] <= row0 and row0 + rows <= m.seg_off[order + 1]      # one column order per block
        cover[mi][row0 // 32:(row0 + rows) // 32, t0:t1] += 1
        parts.setdefault(part, []).append((mi, row0, rows, splits))
    for c in cover:
        assert (c == 1).all()
    for part, blocks in parts.items():                # the blocks of a part share rows and know how many they are
        assert len({b[:3] for b in blocks}) == 1 and all(b[3] == len(blocks) for b in blocks)
    assert len(parts) <= 160                          # one arrival counter each
    firsts = sorted(min(i for i, row in enumerate(out[:nb.value]) if row[2] == part) for part in parts)
    assert firsts == sorted(set(firsts))


def test_batch1_work_split_rejects_what_it_cannot_place():
    lib = _lib.lib
    out = np.zeros((160, 8), np.int32)
    nb = ctypes.c_int32(0)
    m = (_lib.L8 * 1)(_l8_shape(70000, 128))
    assert lib.cbl_gemv_l8_plan(m, 1, 8, out.ctypes.data, ctypes.byref(nb)) == _lib.EUNSUPPORTED    # 18 row parts of <= 4096 rows need 18 blocks
    assert lib.cbl_gemv_l8_plan(None, 1, 8, out.ctypes.data, ctypes.byref(nb)) == _lib.EINVAL
    bad = _l8_shape(64, 64)
    bad.rot = 0
    assert lib.cbl_gemv_l8_plan((_lib.L8 * 1)(bad), 1, 8, out.ctypes.data, ctypes.byref(nb)) == _lib.EINVAL


def test_null_and_bad_arguments_are_rejected_without_a_device():
    lib = _lib.lib
    p = _lib.Packed(R=4, C=16, d=8, bits=12, G=1, M=1, books=1, W=1)
    assert lib.cbl_dequant(ctypes.byref(p), None, _lib.F32, 16, 0, 4, None) == _lib.EINVAL
    assert lib.cbl_gemv_l8(None, None, 0, None, 0, None, None) == _lib.EINVAL
    assert lib.cbl_prep_x(None, _lib.BF16, 1, 8, 8, None, 1, None, None) == _lib.EINVAL


def test_host_pack_bits_matches_reference_fixtures():
    z = np.load(G / "bits.npz")
    for bits in (1, 8, 10, 12, 13, 14, 16):
        v = torch.from_numpy(z[f"vals_{bits}"].astype(np.int64))
        w = packed.pack_bits(v, bits)
        assert w.dtype == torch.int32 and np.array_equal(w.numpy(), z[f"words_{bits}"])
        assert torch.equal(packed.unpack_bits(w, bits, v.shape[1]), v)
    with pytest.raises(ValueError):
        packed.pack_bits(torch.tensor([[1 << 12]]), 12)


def test_host_column_orders_and_crc_match_reference_fixtures():
    z = np.load(G / "perms.npz")
    for C, M, seed in z["cases"]:
        p = packed.seeded_perms(int(C), int(M), torch.Generator(device="cpu").manual_seed(int(seed)))
        assert packed.perm_crc(p) == int(z[f"crc_{C}_{M}_{seed}"][0])


def test_packed_file_round_trip_metadata(tmp_path):
    g = torch.Generator().manual_seed(0)
    R, C, K, d, M = 12, 64, 4096, 8, 4
    tags = torch.randint(0, K, (R, C // d), generator=g)
    table = torch.randn(K, d, generator=g).half()
    rs = torch.rand(R, generator=g).half()
    rm = torch.randint(0, M, (R,), generator=g)
    t, meta = packed.pack_matrix(tags, table, rs, d=d, K=K, M=M, seed=11, row_mask=rm)
    # storage bits: tags + table + scales + row_mask bytes + 32 for the seed (reference formula)
    assert meta["bits"] == R * 3 * 32 + K * d * 16 + R * 16 + R * 8 + 32
    summary = packed.save(tmp_path / "q.safetensors", {"model.layers.0.mlp.up_proj": (t, meta)}, base_model="test/base")
    assert summary["format"] == packed.FORMAT and summary["matrices"] == 1
    pf = packed.PackedFile(tmp_path / "q.safetensors")
    tt = pf.tensors("model.layers.0.mlp.up_proj")
    assert set(tt) == {"tags", "table", "row_scale", "row_mask"}
    assert torch.equal(packed.unpack_bits(tt["tags"], 12, C // d), tags)
    assert pf.perms("model.layers.0.mlp.up_proj").shape == (M, C)
    pf.meta["model.layers.0.mlp.up_proj"]["perm_crc"] ^= 1
    with pytest.raises(RuntimeError):
        pf.perms("model.layers.0.mlp.up_proj")


def test_device_matrix_refuses_cpu():
    from quantexperiments_b200.kernels import DeviceMatrix
    with pytest.raises(ValueError):
        DeviceMatrix(torch.zeros(2, 3, dtype=torch.int32), torch.zeros(4096, 8), torch.ones(2), K=4096, d=8, device="cpu")


def test_engine_sampling_helper_and_config_defaults():
    """Host logic of the decode engine that needs no GPU: the config defaults are the Qwen2.5-7B shape of the
    reference's Cfg (shapequant/kernels/decode_e2e.py:313-327) and the sampler keeps the reference's top-k / top-p
    rules (shapequant/runtime.py:202-214)."""
    import torch
    from quantexperiments_b200.engine import Cfg, _sample
    c = Cfg()
    assert (c.hidden, c.n_heads, c.n_kv, c.head_dim, c.inter, c.vocab, c.layers) == (3584, 28, 4, 128, 18944, 152064, 28)
    logits = torch.tensor([0.1, 2.0, -1.0, 1.9, 0.0])
    g = torch.Generator().manual_seed(0)
    assert _sample(logits, 1.0, 1.0, 1, g) == 1                     # top-k 1 = argmax
    assert _sample(logits, 1e-4, 1.0, 0, g) == 1                    # vanishing temperature = argmax
    assert _sample(logits, 1.0, 0.01, 0, g) == 1                    # a tiny nucleus keeps only the best token
    picks = {_sample(logits, 1.0, 1.0, 2, g) for _ in range(64)}
    assert picks == {1, 3}                                          # top-k 2: only the two best are ever drawn
    a = [_sample(logits, 1.0, 0.9, 0, torch.Generator().manual_seed(5)) for _ in range(3)]
    b = [_sample(logits, 1.0, 0.9, 0, torch.Generator().manual_seed(5)) for _ in range(3)]
    assert a == b                                                   # seeded draws repeat
