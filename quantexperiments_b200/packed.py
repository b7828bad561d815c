"""The packed on-disk format, host side: bit streams, column orders, the safetensors reader.

Mirrors the public names of the reference's shapequant/packed.py (pack_bits, unpack_bits, perm_crc,
pack_matrix, save, PackedFile, decode_tensors) for the parts that describe block linears; the file
format itself ("shapequant-stack-v1", shapequant/packed.py:1-27) is unchanged, so files written by
either side load in the other. Decoding runs on the GPU through libcbl; there is no CPU decode here.
"""

from __future__ import annotations

import json
import math
import zlib
from pathlib import Path

import torch

FORMAT = "shapequant-stack-v1"


def words_per_row(n: int, bits: int) -> int:
    return (n * bits + 31) // 32


def pack_bits(vals: torch.Tensor, bits: int) -> torch.Tensor:
    """[R, n] ints in [0, 2^bits) -> [R, W] int32, little-endian bit stream per row, rows padded to
    whole words (same layout as shapequant/packed.py:61-77). Host-side, offline."""
    R, n = vals.shape
    W = words_per_row(n, bits)
    if n and (int(vals.min()) < 0 or int(vals.max()) >= (1 << bits)):
        raise ValueError(f"values out of range for {bits} bits")
    v = vals.to(torch.int64).cpu()
    pos = torch.arange(n, dtype=torch.int64) * bits
    wi, sh = pos >> 5, pos & 31
    shifted = v << sh                       # < 2^47: low part goes to word wi, the rest to wi + 1
    out = torch.zeros(R, W + 1, dtype=torch.int64)
    out.scatter_add_(1, wi.expand(R, n), shifted & 0xFFFFFFFF)      # disjoint bit ranges: add == or
    out.scatter_add_(1, (wi + 1).expand(R, n), shifted >> 32)
    out = out[:, :W]
    return torch.where(out >= (1 << 31), out - (1 << 32), out).to(torch.int32)


def unpack_bits(words: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    """Inverse of pack_bits: [R, W] int32 -> [R, n] int64 on words' device
    (shapequant/packed.py:80-90). CUDA tensors are unpacked by the library's kernel."""
    if words.is_cuda:
        from .kernels import DeviceMatrix
        return DeviceMatrix.tags_only(words, bits, n).unpack().to(torch.int64)
    w = words.to(torch.int64) & 0xFFFFFFFF
    w = torch.nn.functional.pad(w, (0, 1))
    pos = torch.arange(n, dtype=torch.int64) * bits
    wi, sh = pos >> 5, pos & 31
    both = w[:, wi] | ((w[:, wi + 1] & 0xFFFF) << 32)
    return (both >> sh) & ((1 << bits) - 1)


def seeded_perms(C: int, M: int, gen: torch.Generator) -> torch.Tensor:
    """[M, C] int64 column orders: identity followed by M - 1 draws of torch's CPU randperm; all M
    draws are consumed and the first is replaced (the single source of the draw order in the
    reference is shapequant/masks.py:334-342; the file stores only the seed)."""
    if M <= 1:
        return torch.arange(C)[None]
    rand = [torch.randperm(C, generator=gen) for _ in range(M)]
    rand[0] = torch.arange(C)
    return torch.stack(rand)


def perm_crc(perms: torch.Tensor) -> int:
    return zlib.crc32(perms.to(torch.int64).cpu().numpy().tobytes())


def pack_matrix(tags: torch.Tensor, table: torch.Tensor, row_scale: torch.Tensor, *, d: int, K: int, G: int = 1,
                M: int = 1, seed: int = 0, row_book: torch.Tensor | None = None,
                row_mask: torch.Tensor | None = None) -> tuple[dict, dict]:
    """Tensors + metadata of one matrix in the file layout, from LOCAL tags [R, C/d] (the
    reference's pack_matrix takes its quantizer's Fit object, shapequant/packed.py:97-131; the
    resulting tensors and metadata keys are the same)."""
    if K & (K - 1):
        raise ValueError(f"K={K} is not a power of two")
    R, nch = tags.shape
    C = nch * d
    if table.shape != (G * K, d):
        raise ValueError(f"table shape {tuple(table.shape)} != ({G * K}, {d})")
    b = int(math.log2(K))
    t = {"tags": pack_bits(tags, b), "table": table.to(torch.float16).cpu().contiguous(),
         "row_scale": row_scale.to(torch.float16).cpu().contiguous()}
    if G > 1:
        t["row_book"] = row_book.to(torch.uint8).cpu()
    if M > 1:
        t["row_mask"] = row_mask.to(torch.uint8).cpu()
    perms = seeded_perms(C, M, torch.Generator(device="cpu").manual_seed(seed))
    meta = {"R": R, "C": C, "d": d, "K": K, "G": G, "M": M, "seed": seed, "perm_crc": perm_crc(perms),
            "bits": sum(x.numel() * x.element_size() * 8 for x in t.values()) + 32}
    return t, meta


def save(path, packed: dict[str, tuple[dict, dict]], *, base_model: str, extra: dict | None = None) -> dict:
    """Write {name: (tensors, meta)} to one safetensors file (block linears only; the reference's
    optional aux section, shapequant/packed.py:186-214, is not written)."""
    from safetensors.torch import save_file
    tensors, metas = {}, {}
    for name, (t, m) in packed.items():
        for k, v in t.items():
            tensors[f"{name}.{k}"] = v
        metas[name] = m
    total_bits = sum(m["bits"] for m in metas.values())
    numel = sum(m["R"] * m["C"] for m in metas.values())
    summary = {"format": FORMAT, "base_model": base_model, "matrices": len(metas), "bits": total_bits,
               "numel": numel, "bpw": total_bits / max(numel, 1), **(extra or {})}
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    save_file(tensors, str(path), metadata={"summary": json.dumps(summary), "matrices": json.dumps(metas)})
    return summary


class PackedFile:
    """Read access to a packed file: metadata, raw tensors, column orders, GPU decode
    (same surface as shapequant/packed.py:217-256)."""

    def __init__(self, path):
        from safetensors import safe_open
        self.f = safe_open(str(path), framework="pt", device="cpu")
        md = self.f.metadata()
        self.summary = json.loads(md["summary"])
        if self.summary.get("format") != FORMAT:
            raise ValueError(f"{path}: format {self.summary.get('format')!r} != {FORMAT}")
        self.meta = json.loads(md["matrices"])
        self.aux = json.loads(md["aux"]) if "aux" in md else None

    def tensors(self, name: str) -> dict:
        m = self.meta[name]
        keys = ["tags", "table", "row_scale"] + (["row_book"] if m["G"] > 1 else []) \
            + (["row_mask"] if m["M"] > 1 else [])
        return {k: self.f.get_tensor(f"{name}.{k}") for k in keys}

    def perms(self, name: str) -> torch.Tensor:
        m = self.meta[name]
        p = seeded_perms(m["C"], m["M"], torch.Generator(device="cpu").manual_seed(m["seed"]))
        if perm_crc(p) != m["perm_crc"]:
            raise RuntimeError(f"{name}: regenerated column orders do not match the file (torch RNG changed?)")
        return p

    def local_tags(self, name: str, device="cuda") -> torch.Tensor:
        m = self.meta[name]
        return unpack_bits(self.f.get_tensor(f"{name}.tags").to(device), int(math.log2(m["K"])), m["C"] // m["d"])

    def matrix(self, name: str, device="cuda"):
        """The matrix as a kernels.DeviceMatrix (file layout resident on `device`)."""
        from .kernels import DeviceMatrix
        m = self.meta[name]
        t = self.tensors(name)
        return DeviceMatrix(t["tags"], t["table"], t["row_scale"], t.get("row_book"), t.get("row_mask"),
                            self.perms(name) if m["M"] > 1 else None, K=m["K"], d=m["d"], C=m["C"], device=device)

    def decode(self, name: str, device="cuda") -> torch.Tensor:
        """Dense float32 [R, C] weight in the original row and column order, decoded on the GPU."""
        return self.matrix(name, device).dequant(dtype=torch.float32)


# ---- the reference's block-32 formats of embedding and head (aux section of a packed file, shapequant/packed.py:33-41):
# every run of 32 columns shares one fp16 scale = largest magnitude / qmax (a run of zeros gets scale 1), values are
# round(w / scale) clamped to the code range.  The arithmetic below is the format's definition; fixtures written by the
# reference's packers (tests/golden/blockq.npz) pin it bit for bit.
_BLOCK = 32


def _block32_codes(w: torch.Tensor, qmax: float, lo: int, hi: int, max_elems: int = 1 << 26) -> tuple[torch.Tensor, torch.Tensor]:
    """(codes int32 [R, C], scale fp16 [R, C / 32]) of a matrix, a slab of rows at a time so that the fp32 temporaries
    stay below max_elems elements whatever the vocabulary size."""
    R, C = w.shape
    if C % _BLOCK:
        raise ValueError(f"{C} columns are not a multiple of {_BLOCK}")
    codes = torch.empty(R, C, dtype=torch.int32, device=w.device)
    scale = torch.empty(R, C // _BLOCK, dtype=torch.float16, device=w.device)
    slab = max(1, max_elems // C)
    for r0 in range(0, R, slab):
        blocks = w[r0:r0 + slab].to(torch.float32).unflatten(1, (C // _BLOCK, _BLOCK))
        s16 = (blocks.abs().amax(dim=2).clamp_min(1e-8) / qmax).to(torch.float16)
        s16[s16 == 0] = 1.0                               # a scale that underflows fp16: the codes are all zero anyway
        scale[r0:r0 + slab] = s16
        codes[r0:r0 + slab] = torch.round(blocks / s16.to(torch.float32).unsqueeze(2)).clamp_(lo, hi).flatten(1).to(torch.int32)
    return codes, scale


def q8_pack(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [R, C] -> (q int8 [R, C], scale fp16 [R, C/32]): the reference's 8-bit block-32 head, codes in -127..127
    (shapequant/kernels/proto_formats.py:464-471; aux.lm_head of shapequant/packed.py:38-39)."""
    codes, scale = _block32_codes(w, 127.0, -127, 127)
    return codes.to(torch.int8), scale


def q4_embed_pack(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [V, C] -> (q uint8 [V, C/2], scale fp16 [V, C/32]): the reference's 4-bit block-32 embedding
    (shapequant/packed.py:134-148), codes -8..7 stored with an offset of 8, the even column in the low nibble."""
    codes, scale = _block32_codes(w, 7.0, -8, 7)
    nib = (codes + 8).to(torch.uint8)
    return nib[:, 0::2] | (nib[:, 1::2] << 4), scale


def _block32_expand(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 values of block-32 codes [n, C] (any integer or float type) under their scales [n, C / 32]."""
    return (codes.to(torch.float32).unflatten(1, (-1, _BLOCK)) * scale.to(torch.float32).unsqueeze(2)).flatten(1)


def q4_embed_rows(q: torch.Tensor, sc: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """fp32 [len(ids), C] rows of a 4-bit block-32 embedding (shapequant/packed.py:151-155); on a CUDA device the
    engine uses cbl_embed_rows_q4 instead."""
    packed_rows = q[ids]
    nib = torch.empty(packed_rows.shape[0], 2 * packed_rows.shape[1], dtype=torch.int16, device=q.device)
    nib[:, 0::2] = packed_rows & 15
    nib[:, 1::2] = packed_rows >> 4
    return _block32_expand(nib - 8, sc[ids])


def q8_rows(q: torch.Tensor, sc: torch.Tensor, s: int = 0, e: int | None = None) -> torch.Tensor:
    """fp32 rows s:e of an 8-bit block-32 matrix (shapequant/packed.py:158-160)."""
    return _block32_expand(q[s:e], sc[s:e])


def decode_tensors(local_tags, table, row_scale, row_book, row_mask, perms, K: int) -> torch.Tensor:
    """Decode from unpacked parts on the GPU (argument order of shapequant/packed.py:259-270):
    local_tags [R, nch], table [G*K, d] fp16, row_scale [R], row_book / row_mask [R] or None,
    perms [M, C]. Tensors are moved to the current CUDA device if needed."""
    from .kernels import DeviceMatrix
    R, nch = local_tags.shape
    d = table.shape[1]
    bits = int(math.log2(K))
    M = perms.shape[0] if (row_mask is not None and perms is not None) else 1
    dm = DeviceMatrix(pack_bits(local_tags.cpu(), bits), table, row_scale, row_book, row_mask if M > 1 else None,
                      perms if M > 1 else None, K=K, d=d, C=nch * d, device="cuda")
    return dm.dequant(dtype=torch.float32)
