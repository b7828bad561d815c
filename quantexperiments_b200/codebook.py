"""Encoder side of the format on the GPU: snap every chunk of a weight matrix to its nearest codeword and pack
the tags. Mirrors the reference's names and argument meaning:

    CodebookMatrix, decode(cm)          shapequant/codebook.py:17-32, 277-289
    assign(x, codebook, batch, wt)      shapequant/codebook.py:58-71
    chunk_rows(w, d)                    shapequant/codebook.py:212-218
    snap(w, codebook, ...)              the part of compress() after the codebook fit, shapequant/codebook.py:237-274
    pack_bits(vals, bits)               shapequant/packed.py:60-77

The codebook fit itself (k-means) stays with the reference's trainer. CUDA tensors only; there is no CPU path."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import lib
from .kernels import DeviceMatrix, _dt, _stream


@dataclass
class CodebookMatrix:
    """One matrix in codebook form, field for field the reference's container: tags idx int64 [R, ceil(C / d)],
    codebook fp16 [K, d], row_scale fp16 [R], `pad` zero columns appended to reach a multiple of d, the original
    row length `cols`, and an optional column permutation `perm` [cols] that was applied before chunking."""
    idx: torch.Tensor
    codebook: torch.Tensor
    row_scale: torch.Tensor
    pad: int
    cols: int
    perm: torch.Tensor | None = None

    @property
    def d(self) -> int:
        return self.codebook.shape[1]

    @property
    def K(self) -> int:
        return self.codebook.shape[0]


def decode(cm: CodebookMatrix, device="cuda") -> torch.Tensor:
    """Dense fp32 [R, cols] weights of a CodebookMatrix, decoded on the GPU bit for bit like the reference:
    w = fp32(codebook)[idx] * fp32(row_scale), padding columns dropped, the permutation undone
    (w_out[:, perm[c]] = w[:, c]).  The tags are packed into the file layout's bit stream on the way."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise ValueError("decode runs on a CUDA device (no CPU path)")
    K, d = cm.K, cm.d
    bits = max(1, (K - 1).bit_length())
    if bits > 16 or d > 16:
        raise ValueError(f"K={K}, d={d}: the decode kernel reads tags of at most 16 bits and chunks of at most 16 values")
    idx = cm.idx.to(dev)
    R, nch = idx.shape
    if nch * d != cm.cols + cm.pad:
        raise ValueError("idx, cols and pad disagree")
    book = cm.codebook.to(dev, torch.float16)
    if K != 1 << bits:                                  # the bit stream addresses a power-of-two table
        book = torch.cat([book, torch.zeros((1 << bits) - K, d, dtype=torch.float16, device=dev)])
    words = pack_bits(idx, bits)
    C = nch * d
    perms = mask = None
    if cm.perm is not None:
        ext = torch.cat([cm.perm.to(dev, torch.int64), torch.arange(cm.cols, C, device=dev)])     # padding columns stay where they are
        perms, mask = torch.stack([ext, ext]), torch.zeros(R, dtype=torch.uint8, device=dev)     # the kernel takes column orders per row
    dm = DeviceMatrix(words, book, cm.row_scale, None, mask, perms, K=1 << bits, d=d, C=C, device=dev)
    w = dm.dequant(dtype=torch.float32)
    return w[:, :cm.cols].contiguous() if cm.pad else w



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


@dataclass
class Snapped:
    """Result of snap(): the matrix in codebook form, the per-chunk (weighted) squared errors in chunk order and the
    two statistics the reference's compress() reports."""
    cm: CodebookMatrix
    err: torch.Tensor
    stats: dict

    def __getitem__(self, key):                         # dict-style access to the container's fields
        return getattr(self, key) if key in ("err", "stats", "cm") else getattr(self.cm, key)


def _fp16_row_rms(w: torch.Tensor) -> torch.Tensor:
    """Per-row scale of the format: the root mean square of the row in fp32, stored as fp16; an all-zero row gets 1.
    (The order of operations is the format's definition - square, mean, root - so that scales agree bit for bit.)"""
    rms = w.pow(2).mean(dim=1).sqrt()
    rms[rms == 0] = 1.0
    return rms.to(torch.float16)


def _chunk_weights(shape: tuple, d: int, scale16: torch.Tensor, perm, col_weight, row_weighted: bool) -> torch.Tensor | None:
    """Per-element weights of the weighted snap, chunked like the matrix: the column weights (given in the original
    column order, so permuted along with the columns) times, optionally, the squared row scale; normalised to mean 1
    over the real elements, zero on padding."""
    if col_weight is None and not row_weighted:
        return None
    rows, cols = shape
    dev = scale16.device
    wt = torch.ones(rows, cols, device=dev)
    if col_weight is not None:
        h = col_weight.to(dev, torch.float32)
        wt = wt * (h[perm] if perm is not None else h)[None, :]
    if row_weighted:
        wt = wt * scale16.to(torch.float32).square()[:, None]
    return chunk_rows((wt / wt.mean()).contiguous(), d)[0]


def snap(w: torch.Tensor, codebook: torch.Tensor, *, d: int = 8, perm: torch.Tensor | None = None,
         col_weight: torch.Tensor | None = None, row_weighted: bool = False) -> Snapped:
    """The part of the reference's compress() that follows the codebook fit: permute the columns (optional), divide
    every row by its fp16 RMS, cut into chunks of d and snap each chunk to the nearest word of `codebook` (taken at
    fp16, the precision it is stored at), optionally under per-element weights.  Returns the CodebookMatrix with the
    errors and statistics; result["idx"], ["row_scale"], ... read the container's fields."""
    if w.device.type != "cuda":
        raise ValueError("snap needs a CUDA tensor (no CPU path)")
    w32 = w.to(torch.float32)
    cols = w32.shape[1]
    if perm is not None:
        w32 = w32.index_select(1, perm.to(w32.device))
    scale16 = _fp16_row_rms(w32)
    chunks, pad = chunk_rows(w32 / scale16.to(torch.float32)[:, None], d)
    book16 = codebook.to(torch.float16)
    idx, err = assign(chunks, book16, wt=_chunk_weights(tuple(w32.shape), d, scale16, perm, col_weight, row_weighted))
    cm = CodebookMatrix(idx.view(w32.shape[0], -1), book16, scale16, pad, cols, perm)
    stats = {"codebook_usage": torch.unique(idx).numel() / book16.shape[0], "normalized_chunk_mse": float(err.mean())}
    return Snapped(cm, err, stats)
