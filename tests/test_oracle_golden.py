"""Pins the CPU oracle (oracle/cbl_oracle.py) against fixtures produced by running the reference
implementation (tests/golden/make_golden.py). Bit-exact for integers and decoded weights."""
from pathlib import Path

import numpy as np
import pytest

from oracle import cbl_oracle as orc

G = Path(__file__).resolve().parent / "golden"


def test_pack_unpack_matches_reference_for_every_bit_width():
    z = np.load(G / "bits.npz")
    for bits in (1, 8, 10, 12, 13, 14, 16):
        v, w = z[f"vals_{bits}"], z[f"words_{bits}"]
        got = orc.pack_bits(v, bits)
        assert got.dtype == np.int32 and got.shape == w.shape
        assert np.array_equal(got, w)
        assert np.array_equal(orc.unpack_bits(w, bits, v.shape[1]), v)


def test_bit_layout_known_answers():
    z = np.load(G / "bits.npz")
    # value 1 at index 0 -> bit 0; value 1 at index 1 with 10-bit tags -> bit 10
    assert np.array_equal(orc.pack_bits(z["kat_a_vals"], 10), z["kat_a_words"])
    assert int(orc.pack_bits(z["kat_a_vals"], 10)[0, 0]) == (1 | (1 << 10))
    # a tag straddling the word boundary: index 3 occupies stream bits 30..39
    w = orc.pack_bits(z["kat_b_vals"], 10).view(np.uint32)
    assert np.array_equal(w.view(np.int32), z["kat_b_words"])
    assert int(w[0, 0]) == 0b11 << 30 and int(w[0, 1]) == 0b11111111


def test_pack_rejects_out_of_range():
    with pytest.raises(ValueError):
        orc.pack_bits(np.array([[4096]]), 12)


def test_seeded_column_orders_and_crc():
    z = np.load(G / "perms.npz")
    for C, M, seed in z["cases"]:
        p = orc.seeded_perms(int(C), int(M), int(seed))
        assert p.shape == (M, C) and np.array_equal(p[0], np.arange(C))
        assert orc.perm_crc(p) == int(z[f"crc_{C}_{M}_{seed}"][0])
        if C <= 896:
            assert np.array_equal(p, z[f"perms_{C}_{M}_{seed}"])
        else:
            assert np.array_equal(p[1], z[f"perms_{C}_{M}_{seed}_row1"])
            assert np.array_equal(p[-1], z[f"perms_{C}_{M}_{seed}_rowlast"])


def test_decode_tensors_is_bit_exact_over_the_format_grid():
    z = np.load(G / "decode.npz")
    for i, (Gb, M, K, d) in enumerate(z["grid"]):
        seed, R, C = (int(v) for v in z[f"seed_{i}"])
        bits = int(K).bit_length() - 1
        tags = orc.unpack_bits(z[f"words_{i}"], bits, C // int(d))
        rb = z[f"rb_{i}"] if f"rb_{i}" in z else None
        rm = z[f"rm_{i}"] if f"rm_{i}" in z else None
        perms = orc.seeded_perms(C, int(M), seed)
        w = orc.decode_tensors(tags, z[f"table_{i}"], z[f"rs_{i}"], rb, rm, perms, int(K))
        assert w.dtype == np.float32
        assert np.array_equal(w, z[f"w_{i}"]), f"case {i}: G={Gb} M={M} K={K} d={d}"


def test_codebook_decode_with_padding_and_permutation():
    z = np.load(G / "codebook.npz")
    pad, cols = (int(v) for v in z["pad"])
    w = orc.codebook_decode(z["idx"], z["codebook"], z["row_scale"], pad, cols, z["perm"])
    assert w.shape == (16, 100) and np.array_equal(w, z["decoded"])


def test_assign_matches_reference():
    z = np.load(G / "codebook.npz")
    idx, err = orc.assign(z["assign_x"], z["assign_book"])
    assert np.array_equal(idx, z["assign_idx"])
    assert np.allclose(err, z["assign_err"], rtol=1e-5, atol=1e-6)


def test_weighted_assign_and_snap_match_reference():
    """Both branches of assign on a 4096-word book, and the snap of compress() (row scales, chunking with padding,
    weight normalisation, permutation) against what the reference produced from the same matrix and codebook."""
    z = np.load(G / "snap.npz")
    idx, err = orc.assign(z["x"], z["book"])
    assert np.array_equal(idx, z["idx"]) and np.allclose(err, z["err"], rtol=1e-5, atol=1e-6)
    idx, err = orc.assign(z["x"], z["book"], z["wt"])
    assert np.array_equal(idx, z["widx"]) and np.allclose(err, z["werr"], rtol=1e-5, atol=1e-6)
    assert np.all(orc.assign_margin(z["x"], z["book"], z["widx"], z["wt"]) < 1e-4)
    s = orc.snap(z["w"], z["plain_codebook"])
    assert np.array_equal(s["row_scale"], z["plain_row_scale"]) and np.array_equal(s["idx"], z["plain_idx"])
    assert abs(float(s["err"].mean()) - float(z["plain_mse"][0])) < 1e-6
    s = orc.snap(z["w"], z["weighted_codebook"], perm=z["perm"], col_weight=z["h"], row_weighted=True)
    assert np.array_equal(s["row_scale"], z["weighted_row_scale"]) and np.array_equal(s["idx"], z["weighted_idx"])
    assert abs(float(s["err"].mean()) - float(z["weighted_mse"][0])) < 1e-6


def test_additive_two_book_decode_is_bit_exact():
    z = np.load(G / "additive.npz")
    w = orc.additive_decode(z["A"], z["B"], z["ta"], z["tb"], z["rs"])
    assert np.array_equal(w, z["dense"])


def test_linear_reference_product_and_stored_bytes():
    z = np.load(G / "linear.npz")
    R, C, K, d, M = 48, 896, 4096, 8, 16
    tags = orc.unpack_bits(z["words"], 12, C // d)
    w = orc.decode_tensors(tags, z["table"], z["rs"], None, z["rm"], orc.seeded_perms(C, M, 1), K)
    assert float(w.astype(np.float64).sum()) == float(z["dense_sum"][0])
    y = orc.linear_ref(z["x"], w)
    assert orc.max_rel_err(y, z["y"]) < 1e-6
    stored = z["words"].nbytes + z["table"].nbytes + z["rs"].nbytes
    assert stored == int(z["stored_bytes"][0])


def test_synth_matrix_round_trip():
    m = orc.synth_matrix(20, 128, seed=3, M=4)
    assert np.array_equal(orc.unpack_bits(m["words"][0], 12, 16), m["tags"][0])
    w = orc.synth_decode(m)
    assert w.shape == (20, 128) and np.isfinite(w).all()
    t = __import__("torch")
    y = orc.cpu_linear_torch(t.from_numpy(m["words"][0]), t.from_numpy(m["table"][0]), t.from_numpy(m["row_scale"]),
                             t.ones(1, 128), 12, 8).numpy()
    m1 = orc.synth_matrix(20, 128, seed=3, M=1)
    assert np.allclose(y[0], orc.synth_decode(m1).sum(1), rtol=1e-5, atol=1e-6)


def test_block32_embedding_and_head_formats_match_the_reference_fixture():
    """4-bit embedding / 8-bit head pack + row decode (incl. an all-zero block and an outlier) against arrays written
    by the reference's q4_embed_pack / q4_embed_rows / q8_pack / q8_rows; the host packers agree with the oracle."""
    import torch
    from quantexperiments_b200 import packed
    f = np.load(G / "blockq.npz")
    q4, s4 = orc.q4_embed_pack(f["w"])
    assert np.array_equal(q4, f["q4"]) and np.array_equal(s4, f["s4"])
    assert np.array_equal(orc.q4_embed_rows(f["q4"], f["s4"], f["ids"]), f["rows4"])
    q8, s8, deq8 = orc.q8_pack(f["w"])
    assert np.array_equal(q8, f["q8"]) and np.array_equal(s8, f["s8"]) and np.array_equal(deq8, f["deq8"])
    assert np.array_equal(orc.q8_rows(f["q8"], f["s8"], 2, 9), f["rows8"])
    w = torch.from_numpy(f["w"])
    hq4, hs4 = packed.q4_embed_pack(w)
    hq8, hs8 = packed.q8_pack(w)
    assert np.array_equal(hq4.numpy(), f["q4"]) and np.array_equal(hs4.numpy(), f["s4"])
    assert np.array_equal(hq8.numpy(), f["q8"]) and np.array_equal(hs8.numpy(), f["s8"])
    assert np.array_equal(packed.q4_embed_rows(hq4, hs4, torch.from_numpy(f["ids"])).numpy(), f["rows4"])
    assert np.array_equal(packed.q8_rows(hq8, hs8, 2, 9).numpy(), f["rows8"])

