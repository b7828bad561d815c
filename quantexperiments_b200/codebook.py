"""Encoder side of the format on the GPU: snap every chunk of a weight matrix to its nearest codeword and pack
the tags. Mirrors the reference's names and argument meaning:

    assign(x, codebook, batch, wt)      shapequant/codebook.py:58-71
    chunk_rows(w, d)                    shapequant/codebook.py:212-218
    snap(w, codebook, ...)              the part of compress() after the codebook fit, shapequant/codebook.py:237-274
    pack_bits(vals, bits)               shapequant/packed.py:60-77

The codebook fit itself (k-means) stays with the reference's trainer. CUDA tensors only; there is no CPU path."""

from __future__ import annotations

import torch

from . import _lib
from ._lib import lib
from .kernels import _dt, _stream


def assign(x: torch.Tensor, codebook: torch.Tensor, batch: int = 65536, wt: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Index of the nearest codeword and its (weighted) squared error, per chunk: (idx int64 [n], err fp32 [n]).
    `batch` is accepted for call compatibility; the kernel streams the chunks and never forms a distance matrix."""
    if x.device.type != "cuda" or codebook.device != x.device:
        raise ValueError("assign needs CUDA tensors on one device (no CPU path)")
    if x.dim() != 2 or codebook.dim() != 2 or x.shape[1] != codebook.shape[1]:
        raise ValueError("x [n, d] and codebook [K, d] must agree in d")
    if wt is not None and wt.shape != x.shape:
        raise ValueError("wt must have x's shape")
    x = x.to(torch.float32).contiguous()
    wt = None if wt is None else wt.to(device=x.device, dtype=torch.float32).contiguous()
    book = codebook.contiguous()
    if book.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        book = book.to(torch.float32)
    n, d = x.shape
    idx = torch.empty(n, dtype=torch.int64, device=x.device)
    err = torch.empty(n, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check("cbl_assign", lib.cbl_assign(x.data_ptr(), None if wt is None else wt.data_ptr(), n, d, book.data_ptr(), _dt(book.dtype),
                                                book.shape[0], idx.data_ptr(), err.data_ptr(), _stream()))
    return idx, err


def chunk_rows(w: torch.Tensor, d: int) -> tuple[torch.Tensor, int]:
    """[R, C] -> [R * ceil(C / d), d], each row zero-padded to a multiple of d; returns (chunks, pad)."""
    rows, cols = w.shape
    pad = (-cols) % d
    if pad:
        w = torch.nn.functional.pad(w, (0, pad))
    return w.reshape(rows * ((cols + pad) // d), d), pad


def pack_bits(vals: torch.Tensor, bits: int) -> torch.Tensor:
    """[R, n] ints in [0, 2^bits) -> [R, W] int32 on the GPU (little-endian bit stream per row)."""
    if vals.device.type != "cuda":
        raise ValueError("pack_bits needs a CUDA tensor (no CPU path)")
    R, n = vals.shape
    if vals.numel() and (int(vals.min()) < 0 or int(vals.max()) >= (1 << bits)):
        raise ValueError(f"values out of range for {bits} bits")
    v = vals.to(torch.int64).contiguous()
    out = torch.empty(R, (n * bits + 31) // 32, dtype=torch.int32, device=vals.device)
    with torch.cuda.device(vals.device):
        _lib.check("cbl_pack_tags", lib.cbl_pack_tags(v.data_ptr(), R, n, bits, out.data_ptr(), _stream()))
    return out


def snap(w: torch.Tensor, codebook: torch.Tensor, *, d: int = 8, perm: torch.Tensor | None = None,
         col_weight: torch.Tensor | None = None, row_weighted: bool = False) -> dict:
    """Row-normalise, chunk and snap a weight matrix against a fitted codebook (stored at 16 bits, as the reference
    snaps against what is stored). Returns idx [R, C/d] int64, row_scale fp16 [R], pad, err [R * C/d] and the
    reference's two statistics. Weighting follows the reference: `col_weight` h (length C, original column
    order) and `row_weighted` (factor row_scale^2), normalised to mean 1, padding weight 0."""
    if w.device.type != "cuda":
        raise ValueError("snap needs a CUDA tensor (no CPU path)")
    w = w.to(torch.float32)
    rows, cols = w.shape
    if perm is not None:
        w = w[:, perm]
    rms = w.pow(2).mean(dim=1).sqrt()
    row_scale = torch.where(rms == 0, torch.ones_like(rms), rms).to(torch.float16)
    wn = w / row_scale.to(torch.float32)[:, None]
    chunks, pad = chunk_rows(wn, d)
    wt = None
    if col_weight is not None or row_weighted:
        h = torch.ones(cols, device=w.device) if col_weight is None else col_weight.to(w.device, torch.float32)
        if perm is not None and col_weight is not None:
            h = h[perm]
        full = h[None, :].expand(rows, cols)
        if row_weighted:
            full = full * row_scale.to(torch.float32).pow(2)[:, None]
        full = full / full.mean()
        wt, _ = chunk_rows(full.contiguous(), d)
    book = codebook.to(torch.float16)
    idx, err = assign(chunks, book, wt=wt)
    used = torch.unique(idx).numel()
    return {"idx": idx.reshape(rows, -1), "codebook": book, "row_scale": row_scale, "pad": pad, "cols": cols, "perm": perm, "err": err,
            "stats": {"codebook_usage": used / book.shape[0], "normalized_chunk_mse": float(err.mean())}}
