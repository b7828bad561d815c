"""CPU oracle for the codebook-linear path. TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
module; the product package never does (it fails loudly when its CUDA library is missing).

Every function restates, in numpy / CPU torch, one piece of the reference project
(angryslavemerchant/QuantExperiments, package `shapequant`) and cites the file:line it follows.
The restatement is pinned against fixtures produced by running the reference itself
(tests/golden/make_golden.py writes them; tests/test_oracle_golden.py checks them).

Format recap (shapequant/packed.py:1-27): an [R, C] weight is cut into nch = C/d chunks per row;
chunk j of row r stores a log2(K)-bit tag into a table of G*K fp16 codewords of d values; tags
form a little-endian bit stream per row, padded to whole 32-bit words; each row has an fp16
scale, optionally a codebook id (row_book) and a column-order id (row_mask); column orders are
regenerated from a seed.
"""

from __future__ import annotations

import math
import zlib

import numpy as np
import torch


# --------------------------------------------------------------------------- bit stream

def words_per_row(n: int, bits: int) -> int:
    """W = ceil(n * bits / 32) (shapequant/packed.py:64)."""
    return (n * bits + 31) // 32


def pack_bits(vals: np.ndarray, bits: int) -> np.ndarray:
    """[R, n] ints in [0, 2^bits) -> [R, W] int32, little-endian bit stream per row
    (shapequant/packed.py:61-77). Value j occupies stream bits [j*bits, (j+1)*bits)."""
    vals = np.asarray(vals)
    R, n = vals.shape
    if n and (int(vals.min()) < 0 or int(vals.max()) >= (1 << bits)):
        raise ValueError(f"values out of range for {bits} bits")
    W = words_per_row(n, bits)
    out = np.zeros((R, W + 1), dtype=np.uint64)
    v = vals.astype(np.uint64)
    pos = np.arange(n, dtype=np.int64) * bits
    wi = pos >> 5
    sh = (pos & 31).astype(np.uint64)
    lo = (v << sh) & np.uint64(0xFFFFFFFF)
    hi = (v << sh) >> np.uint64(32)          # bits <= 16 and sh <= 31: fits in 64 bits
    for j in range(n):                        # several values share a word: accumulate in order
        out[:, wi[j]] |= lo[:, j]
        out[:, wi[j] + 1] |= hi[:, j]
    return out[:, :W].astype(np.uint32).view(np.int32)


def unpack_bits(words: np.ndarray, bits: int, n: int) -> np.ndarray:
    """Inverse of pack_bits: [R, W] int32 -> [R, n] int64 (shapequant/packed.py:80-90)."""
    w = np.asarray(words).view(np.uint32).astype(np.uint64)
    R, W = w.shape
    w = np.concatenate([w, np.zeros((R, 1), dtype=np.uint64)], axis=1)
    pos = np.arange(n, dtype=np.int64) * bits
    wi = pos >> 5
    sh = (pos & 31).astype(np.uint64)
    both = w[:, wi] | (w[:, wi + 1] << np.uint64(32))
    return ((both >> sh) & np.uint64((1 << bits) - 1)).astype(np.int64)


# --------------------------------------------------------------------------- column orders

def seeded_perms(C: int, M: int, seed: int) -> np.ndarray:
    """[M, C] int64 column orders: identity, then M-1 draws of torch's CPU randperm; M draws
    are consumed and the first is discarded (shapequant/masks.py:334-342, called with
    torch.Generator('cpu').manual_seed(seed) at shapequant/packed.py:123,236)."""
    if M <= 1:
        return np.arange(C, dtype=np.int64)[None]
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    rand = [torch.randperm(C, generator=gen) for _ in range(M)]
    rand[0] = torch.arange(C)
    return torch.stack(rand).numpy().astype(np.int64)


def perm_crc(perms: np.ndarray) -> int:
    """CRC32 over the int64 little-endian bytes of the orders (shapequant/packed.py:93-94)."""
    return zlib.crc32(np.ascontiguousarray(perms, dtype=np.int64).tobytes())


# --------------------------------------------------------------------------- decode

def decode_tensors(local_tags, table, row_scale, row_book, row_mask, perms, K: int) -> np.ndarray:
    """Reference decode of a packed matrix (shapequant/packed.py:259-270):
    u[r, j*d:(j+1)*d] = fp32(table[row_book[r]*K + tag[r, j]]) * fp32(row_scale[r]);
    w[r, perms[row_mask[r]][c]] = u[r, c]. Returns fp32 [R, C]."""
    tags = np.asarray(local_tags, dtype=np.int64)
    table = np.asarray(table, dtype=np.float16)
    R, nch = tags.shape
    d = table.shape[1]
    C = nch * d
    if row_book is not None:
        tags = tags + np.asarray(row_book, dtype=np.int64)[:, None] * K
    u = table.astype(np.float32)[tags].reshape(R, C) * np.asarray(row_scale, dtype=np.float16).astype(np.float32)[:, None]
    perms = np.asarray(perms, dtype=np.int64)
    idx = perms[np.asarray(row_mask, dtype=np.int64)] if row_mask is not None else np.broadcast_to(perms[:1], (R, C))
    w = np.empty_like(u)
    np.put_along_axis(w, idx, u, axis=1)
    return w


def codebook_decode(idx, codebook, row_scale, pad: int, cols: int, perm=None) -> np.ndarray:
    """CodebookMatrix decode (shapequant/codebook.py:277-289): gather, strip the zero padding of
    the last chunk, scale rows, undo the single column permutation (w_out = w[:, inverse(perm)])."""
    idx = np.asarray(idx, dtype=np.int64)
    rows = idx.shape[0]
    w = np.asarray(codebook, dtype=np.float16).astype(np.float32)[idx.reshape(-1)].reshape(rows, -1)
    if pad:
        w = w[:, :cols]
    w = w * np.asarray(row_scale, dtype=np.float16).astype(np.float32)[:, None]
    if perm is not None:
        perm = np.asarray(perm, dtype=np.int64)
        inv = np.empty_like(perm)
        inv[perm] = np.arange(perm.size)
        w = w[:, inv]
    return w


def additive_decode(A, B, ta, tb, row_scale) -> np.ndarray:
    """Two summed d = 8 books: (fp32(A[ta]) + fp32(B[tb])) rounded to fp32, then times
    fp32(row_scale) (tests/test_proto_runs.py:135-144; shapequant/masks.py:193-200)."""
    A = np.asarray(A, dtype=np.float16).astype(np.float32)
    B = np.asarray(B, dtype=np.float16).astype(np.float32)
    R = np.asarray(ta).shape[0]
    s = (A[np.asarray(ta, dtype=np.int64)] + B[np.asarray(tb, dtype=np.int64)]).reshape(R, -1)
    return s * np.asarray(row_scale, dtype=np.float16).astype(np.float32)[:, None]


def round_to(w: np.ndarray, dtype: str) -> np.ndarray:
    """One round-to-nearest-even of the fp32 decode to the storage dtype the GPU dequant writes
    (shapequant/kernels/cuda_dequant.py:27-31 for fp16; batched_runs.py:873-881 for bf16)."""
    if dtype == "f32":
        return w.astype(np.float32)
    if dtype == "f16":
        return w.astype(np.float16)
    if dtype == "bf16":
        return torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).to(torch.bfloat16)
    raise ValueError(dtype)


# --------------------------------------------------------------------------- assign (format definition)

def assign(x: np.ndarray, codebook: np.ndarray, wt: np.ndarray | None = None) -> tuple[np.ndarray, np.ndarray]:
    """Nearest codeword per chunk: argmin of c_sq - 2 x.c, or with per-element weights argmin of
    [-2 w x, w] . [c, c^2] (shapequant/codebook.py:40-71, both branches). Returns (idx int64 [n], err fp32 [n])."""
    xt = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    c = torch.from_numpy(np.asarray(codebook, dtype=np.float16).astype(np.float32))
    if wt is None:
        c_sq = (c * c).sum(1)
        d2 = torch.addmm(c_sq[None, :], xt, c.T, alpha=-2.0)
        m, i = d2.min(dim=1)
        return i.numpy(), (m + (xt * xt).sum(1)).clamp_min(0).numpy()
    w = torch.from_numpy(np.ascontiguousarray(wt, dtype=np.float32))
    a = torch.cat([-2.0 * w * xt, w], dim=1)
    b = torch.cat([c, c * c], dim=1)
    m, i = (a @ b.T).min(dim=1)
    return i.numpy(), (m + (w * xt * xt).sum(1)).clamp_min(0).numpy()


def assign_margin(x: np.ndarray, codebook: np.ndarray, idx: np.ndarray, wt: np.ndarray | None = None) -> np.ndarray:
    """In float64: (weighted) squared distance to codeword idx[i] minus the smallest distance to any codeword, per
    chunk. Zero where idx is the exact nearest; a few fp32 ulps of the distances where two codewords all but tie."""
    x64 = np.asarray(x, dtype=np.float64)
    c64 = np.asarray(codebook, dtype=np.float16).astype(np.float64)
    w64 = np.ones_like(x64) if wt is None else np.asarray(wt, dtype=np.float64)
    out = np.empty(x64.shape[0])
    for s in range(0, x64.shape[0], 4096):
        df = x64[s:s + 4096, None, :] - c64[None, :, :]
        d2 = (w64[s:s + 4096, None, :] * df * df).sum(-1)
        out[s:s + 4096] = d2[np.arange(d2.shape[0]), np.asarray(idx[s:s + 4096], dtype=np.int64)] - d2.min(1)
    return out


def snap(w: np.ndarray, codebook: np.ndarray, d: int = 8, perm: np.ndarray | None = None, col_weight: np.ndarray | None = None,
         row_weighted: bool = False) -> dict:
    """compress() after the codebook fit (shapequant/codebook.py:237-274): permute, row-normalise by the fp16 rms,
    chunk with zero padding, weights h_c (* row_scale^2) normalised to mean 1 with padding weight 0, assign."""
    wt_ = torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32))
    rows, cols = wt_.shape
    if perm is not None:
        wt_ = wt_[:, torch.from_numpy(np.asarray(perm, dtype=np.int64))]
    rms = wt_.pow(2).mean(dim=1).sqrt()
    row_scale = torch.where(rms == 0, torch.ones_like(rms), rms).to(torch.float16)
    wn = wt_ / row_scale.to(torch.float32)[:, None]
    pad = (-cols) % d
    chunks = torch.nn.functional.pad(wn, (0, pad)).reshape(-1, d)
    wts = None
    if col_weight is not None or row_weighted:
        h = torch.ones(cols) if col_weight is None else torch.from_numpy(np.asarray(col_weight, dtype=np.float32))
        if perm is not None and col_weight is not None:
            h = h[torch.from_numpy(np.asarray(perm, dtype=np.int64))]
        full = h[None, :].expand(rows, cols)
        if row_weighted:
            full = full * row_scale.to(torch.float32).pow(2)[:, None]
        full = full / full.mean()
        wts = torch.nn.functional.pad(full.contiguous(), (0, pad)).reshape(-1, d).numpy()
    idx, err = assign(chunks.numpy(), codebook, wts)
    return {"idx": idx.reshape(rows, -1), "row_scale": row_scale.numpy(), "err": err, "chunks": chunks.numpy(), "wt": wts}


# --------------------------------------------------------------------------- linear

def linear_ref(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = fp32(x) @ w^T in fp32 on the reference-decoded weights: the reference tests' oracle
    (tests/test_kernels.py:30-35 `lin.dense() @ x.float()`). x [B, C] or [C]."""
    xt = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    wt = torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32))
    return (xt @ wt.T).numpy()


def max_rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got - ref| / max|ref| (tests/test_kernels.py:35)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


# --------------------------------------------------------------------------- the reference's CPU path, for timing

def cpu_linear_torch(words_t: torch.Tensor, table_t: torch.Tensor, rs_t: torch.Tensor, x_t: torch.Tensor,
                     bits: int, d: int) -> torch.Tensor:
    """The reference's CPU execution of one packed linear, op for op in CPU torch so that it uses
    the host's cores the same way: unpack_bits (shapequant/packed.py:80-90, 64 rows per step),
    decode (packed.py:259-270 with G = M = 1), then `x.float() @ W.T` (kernels/gemv.py:164-170).
    Used only as the benchmark's timed CPU baseline."""
    R, W = words_t.shape
    n = (W * 32) // bits
    C = x_t.shape[-1]
    n = C // d
    out = torch.empty(R, n, dtype=torch.int64)
    wordpos = torch.arange(32)
    bitpos = torch.arange(bits)
    for a in range(0, R, 64):
        w = words_t[a:a + 64].to(torch.int64) & 0xFFFFFFFF
        stream = ((w[..., None] >> wordpos) & 1).reshape(w.shape[0], W * 32)[:, : n * bits]
        out[a:a + 64] = (stream.view(-1, n, bits) << bitpos).sum(-1)
    u = table_t.float()[out].reshape(R, C) * rs_t.float()[:, None]
    return x_t.float() @ u.T


# --------------------------------------------------------------------------- block-32 embedding / head formats

def q4_embed_pack(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """4-bit block-32 embedding (shapequant/packed.py:134-148): per block of 32 columns s = fp16(max|w| / 7)
    (clamped below at 1e-8 before the division; an fp16 zero becomes 1), n = clamp(round(w / s), -8, 7) + 8, two
    nibbles per byte with the even column in the low nibble. Returns (q uint8 [V, C/2], scale fp16 [V, C/32])."""
    w = np.asarray(w, dtype=np.float32)
    V, C = w.shape
    b = w.reshape(V, C // 32, 32)
    k = (np.maximum(np.abs(b).max(-1), np.float32(1e-8)) / np.float32(7.0)).astype(np.float16).astype(np.float32)
    k = np.where(k == 0, np.float32(1.0), k)
    n = (np.clip(np.rint(b / k[..., None]), -8, 7) + 8).astype(np.uint8).reshape(V, C // 2, 2)
    return (n[..., 0] | (n[..., 1] << 4)).astype(np.uint8), k.astype(np.float16)


def q4_embed_rows(q: np.ndarray, sc: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """fp32 rows of a 4-bit block-32 embedding (shapequant/packed.py:151-155): (nibble - 8) * scale."""
    b = np.asarray(q)[np.asarray(ids)]
    n = np.stack([b & 15, b >> 4], -1).reshape(b.shape[0], -1).astype(np.float32) - 8
    return (n.reshape(b.shape[0], -1, 32) * np.asarray(sc)[np.asarray(ids)].astype(np.float32)[..., None]).reshape(b.shape[0], -1)


def q8_pack(w: np.ndarray) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """8-bit block-32 head (shapequant/kernels/proto_formats.py:464-471): s = fp16(max|w| / 127) per block of 32 (same
    clamps as the 4-bit format), n = clamp(round(w / s), -127, 127). Returns (q int8 [R, C], scale fp16 [R, C/32],
    dequantized fp32 [R, C])."""
    w = np.asarray(w, dtype=np.float32)
    R, C = w.shape
    b = w.reshape(R, C // 32, 32)
    k = (np.maximum(np.abs(b).max(-1), np.float32(1e-8)) / np.float32(127.0)).astype(np.float16).astype(np.float32)
    k = np.where(k == 0, np.float32(1.0), k)
    n = np.clip(np.rint(b / k[..., None]), -127, 127)
    return n.reshape(R, C).astype(np.int8), k.astype(np.float16), (n * k[..., None]).reshape(R, C).astype(np.float32)


def q8_rows(q: np.ndarray, sc: np.ndarray, s: int = 0, e: int | None = None) -> np.ndarray:
    """fp32 rows s:e of an 8-bit block-32 matrix (shapequant/packed.py:158-160)."""
    b = np.asarray(q)[s:e]
    return (b.astype(np.float32).reshape(b.shape[0], -1, 32) * np.asarray(sc)[s:e].astype(np.float32)[..., None]).reshape(b.shape[0], -1)


def synth_matrix(R: int, C: int, seed: int, *, d: int = 8, bits: int = 12, books: int = 1, M: int = 1):
    """Seeded synthetic matrix in the benchmark's format (random tags, N(0,1) fp16 book(s),
    positive fp16 row scales), generated like the reference tests' `_lin` helpers
    (tests/test_kernels.py:14-24): CPU torch generator, then packed. Returns a dict of numpy
    arrays: tags [books, R, nch], words [books, R, W] int32, table [books, K, d] fp16,
    row_scale [R] fp16, row_mask [R] uint8 or None, perms [M, C] int64, seed_perm."""
    g = torch.Generator().manual_seed(seed)
    K = 1 << bits
    nch = C // d
    tags = torch.randint(0, K, (books, R, nch), generator=g)
    table = torch.randn(books, K, d, generator=g).half()
    rs = (torch.rand(R, generator=g) * 0.02 + 0.01).half()
    rm = torch.randint(0, M, (R,), generator=g).to(torch.uint8).numpy() if M > 1 else None
    perms = seeded_perms(C, M, seed + 1)
    tg = tags.numpy()
    words = np.stack([pack_bits(tg[b], bits) for b in range(books)])
    return dict(tags=tg, words=words, table=table.numpy(), row_scale=rs.numpy(), row_mask=rm, perms=perms,
                seed_perm=seed + 1, R=R, C=C, d=d, bits=bits, K=K, M=M, books=books)


def synth_decode(m: dict) -> np.ndarray:
    """fp32 reference decode of a synth_matrix(): single book -> decode_tensors; two books ->
    additive formula followed by the same column-order scatter."""
    if m["books"] == 1:
        return decode_tensors(m["tags"][0], m["table"][0], m["row_scale"], None, m["row_mask"], m["perms"], m["K"])
    u = additive_decode(m["table"][0], m["table"][1], m["tags"][0], m["tags"][1], m["row_scale"])
    R, C = u.shape
    idx = m["perms"][m["row_mask"].astype(np.int64)] if m["row_mask"] is not None else np.broadcast_to(m["perms"][:1], (R, C))
    w = np.empty_like(u)
    np.put_along_axis(w, idx, u, axis=1)
    return w
