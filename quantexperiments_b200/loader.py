"""Packed file -> device, as a pipeline: every matrix of a packed safetensors file is streamed through two pinned
staging buffers into ONE exact-size arena per device and re-laid out for the kernels there.

    plan  = plan_arena(pf, names, layouts, rank, world, kinds)      # bytes per matrix, from the metadata alone
    lins  = load_linears(path, device="cuda", layouts=("l8",))       # {name: PackedLinear}, arena in lins.arena

While the copy engine moves matrix i to the device and the repack kernels of matrix i - 1 run, the host reads
matrix i + 1 from the file into the other staging buffer. Column orders are regenerated from the stored seed and
checked against the stored CRC (`PackedFile.perms`). With world > 1 each rank keeps its row range ("col" kind,
output sharded) or column range ("row" kind, input sharded) of every matrix, cut before the copy; an input shard of a
matrix with several column orders keeps `perms[:, c0:c1]` and reads the full activation vector (`PackedLinear.wide`).

Everything a matrix needs on the device (file-order tags for the dense decode, tables, scales, kernel layouts)
lies back to back in the arena, 256-byte aligned, instead of one caching-allocator block per tensor: the
reference pools its tile words after loading for the same reason (shapequant/vllm_ext/core.py:630-670, 8.20 GiB
held for 7.38 GiB of data before pooling); `pool_layouts` does that for matrices that were built one by one.
Replaces shapequant/packed.py:217-256 (PackedFile as used by the runtime loaders) + core.py:630-670.

No load-time cache of the re-laid-out tags is kept on disk: the repack kernels rewrite a matrix at HBM speed
(microseconds), reading the same bytes back from a cache file would take longer than producing them."""

from __future__ import annotations

import math

import torch

from . import packed as pk
from . import tp
from ._lib import lib
from .kernels import L8Matrix, T16Matrix, X16Matrix
from .linear import PackedLinear

ALIGN = 256
LAYOUTS = ("l8", "t16", "x16")


def _al(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


class Arena:
    """One device allocation handed out in 256-byte aligned pieces, in order."""

    def __init__(self, nbytes: int, device):
        self.buf = torch.empty(max(nbytes, ALIGN), dtype=torch.uint8, device=device)
        self.off = 0

    def take(self, nbytes: int) -> torch.Tensor:
        if self.off + nbytes > self.buf.numel():
            raise RuntimeError(f"arena of {self.buf.numel()} bytes is too small: the plan and the loader disagree")
        v = self.buf[self.off:self.off + nbytes]
        self.off += _al(nbytes)
        return v


def _shard_meta(m: dict, kind: str | None, rank: int, world: int) -> tuple[int, int]:
    """(R, C) of the rank's piece."""
    R, C = m["R"], m["C"]
    if world > 1 and kind == "col":
        r0, r1 = tp.row_range(R, rank, world)
        R = r1 - r0
    elif world > 1 and kind == "row":
        c0, c1 = tp.col_range(C, m["d"], rank, world)
        C = c1 - c0
    return R, C


def _t16_tiles(R: int, M: int, row_mask: torch.Tensor | None) -> int:
    if M == 1 or row_mask is None:
        return -(-R // 16)
    counts = torch.bincount(row_mask.to(torch.int64).flatten(), minlength=M)
    return int(sum(-(-int(c) // 16) for c in counts if int(c) > 0))


def _l8_positions(R: int, M: int, row_mask: torch.Tensor | None) -> int:
    """Row positions of the batch-1 layout: every column order padded to a multiple of 32 rows."""
    if M == 1 or row_mask is None:
        return (R + 31) // 32 * 32
    counts = torch.bincount(row_mask.to(torch.int64).flatten(), minlength=M)
    return int(sum((int(c) + 31) // 32 * 32 for c in counts))


def matrix_bytes(m: dict, R: int, C: int, layouts, ntile16: int, rpad8: int | None = None) -> dict:
    """Aligned device bytes of one matrix piece: file-order tensors and each requested layout."""
    bits = int(math.log2(m["K"]))
    W = pk.words_per_row(C // m["d"], bits)
    out = {"tags": _al(R * W * 4), "table": _al(m["G"] * m["K"] * m["d"] * 2), "row_scale": _al(R * 2)}
    if m["G"] > 1:
        out["row_book"] = _al(R)
    if m["M"] > 1:
        out["row_mask"] = _al(R)
        out["perms"] = _al(m["M"] * C * 4)
    fast = m["d"] == 8 and m["K"] == 4096 and m["G"] == 1
    for lay in layouts:
        if lay not in LAYOUTS:
            raise ValueError(f"unknown layout {lay!r}")
        if not fast or (lay == "x16" and m["M"] > 1) or (lay == "l8" and m["M"] > L8Matrix.MAX_ORDERS):
            continue
        if lay == "l8":
            rp = rpad8 if rpad8 is not None else (R + 31) // 32 * 32
            out["l8"] = _al(max(lib.cbl_l8r_bytes(rp, C, 1), 16)) + _al(lib.cbl_book_frag_bytes())
        elif lay == "x16":
            out["x16"] = _al(max(lib.cbl_x16_bytes(R, C, 1), 16))
        else:
            out["t16"] = _al(max(lib.cbl_t16_bytes(ntile16, C, 1), 16))
    return out


def plan_arena(pf: pk.PackedFile, names=None, layouts=("l8",), rank: int = 0, world: int = 1, kinds: dict | None = None) -> dict:
    """{name: {part: bytes}} for the rank's pieces, from the file's metadata (plus the row masks of matrices with
    several column orders when the row-tile layout is requested: its tile count depends on them)."""
    names = list(pf.meta) if names is None else list(names)
    plan = {}
    for name in names:
        m = pf.meta[name]
        kind = (kinds or {}).get(name)
        R, C = _shard_meta(m, kind, rank, world)
        mask = None
        if m["M"] > 1 and ("t16" in layouts or "l8" in layouts):
            mask = pf.f.get_tensor(f"{name}.row_mask")
            if world > 1 and kind == "col":
                r0, r1 = tp.row_range(m["R"], rank, world)
                mask = mask[r0:r1]
        plan[name] = matrix_bytes(m, R, C, layouts, _t16_tiles(R, m["M"], mask), _l8_positions(R, m["M"], mask))
    return plan


class LoadedLinears(dict):
    """{name: PackedLinear} plus the arena that holds their tensors and what the load moved."""
    arena: Arena
    stats: dict


def load_linears(path_or_file, names=None, device="cuda", layouts=("l8",), rank: int = 0, world: int = 1,
                 kinds: dict | None = None) -> LoadedLinears:
    """Stream the matrices `names` (default: all) of a packed file onto `device`; see the module text."""
    pf = path_or_file if isinstance(path_or_file, pk.PackedFile) else pk.PackedFile(path_or_file)
    dev = torch.device(device)
    if dev.type != "cuda":
        raise ValueError("load_linears targets a CUDA device; there is no CPU path")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    names = list(pf.meta) if names is None else list(names)
    plan = plan_arena(pf, names, layouts, rank, world, kinds)
    file_parts = ("tags", "table", "row_scale", "row_book", "row_mask", "perms")
    total = sum(sum(p.values()) for p in plan.values())
    stage_bytes = max([sum(v for k, v in p.items() if k in file_parts) for p in plan.values()] + [ALIGN])
    out = LoadedLinears()
    with torch.cuda.device(dev):
        arena = Arena(total, dev)
        pinned = [torch.empty(stage_bytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        copied = [None, None]                       # event: the staging buffer's last copy has left it
        copy_stream = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream()
        copy_stream.wait_stream(main)               # the arena's allocation is ordered before the first copy
        h2d = 0
        for i, name in enumerate(names):
            m = pf.meta[name]
            kind = (kinds or {}).get(name)
            t = pf.tensors(name)
            perms = pf.perms(name) if m["M"] > 1 else None
            meta = dict(m)
            if world > 1 and kind == "col":
                t, meta = tp.shard_rows(t, m, *tp.row_range(m["R"], rank, world))
            elif world > 1 and kind == "row":
                t, meta, perms = tp.shard_cols(t, m, *tp.col_range(m["C"], m["d"], rank, world), perms=perms)
            if perms is not None:
                t = dict(t, perms=perms.to(torch.int32))
            t["tags"] = t["tags"].to(torch.int32)
            t["table"], t["row_scale"] = t["table"].to(torch.float16), t["row_scale"].to(torch.float16)
            for k in ("row_book", "row_mask"):
                if k in t:
                    t[k] = t[k].to(torch.uint8)
            buf = pinned[i % 2]
            if copied[i % 2] is not None:
                copied[i % 2].synchronize()
            views, off = {}, 0
            for k in file_parts:
                if k not in t:
                    continue
                src = t[k].contiguous()
                nb = src.numel() * src.element_size()
                if _al(nb) != plan[name][k]:
                    raise RuntimeError(f"{name}.{k}: {nb} bytes in the file, {plan[name][k]} planned")
                buf[off:off + nb].view(src.dtype).view(src.shape).copy_(src)        # file (page cache) -> pinned
                dst = arena.take(nb)
                with torch.cuda.stream(copy_stream):
                    dst.copy_(buf[off:off + nb], non_blocking=True)
                views[k] = dst.view(src.dtype).view(src.shape)
                off += _al(nb)
                h2d += nb
            ev = torch.cuda.Event()
            ev.record(copy_stream)
            copied[i % 2] = ev
            main.wait_event(ev)
            C = meta["C"]
            # an input shard of a matrix with several column orders keeps orders that name positions of the full vector
            wide = m["C"] if (world > 1 and kind == "row" and m["M"] > 1) else None
            lin = PackedLinear(views["tags"], views["table"], views["row_scale"], views.get("row_book"), views.get("row_mask"),
                               views["perms"] if "perms" in views else torch.empty((1, C), device="meta"), meta["K"], meta["d"], x_cols=wide)
            for lay in layouts:
                if lay not in plan[name]:
                    continue
                if lay == "l8":
                    lin._l8 = L8Matrix(lin.dm, alloc=arena.take)
                elif lay == "x16":
                    lin._x16 = X16Matrix(lin.dm, alloc=arena.take)
                else:
                    lin._t16 = T16Matrix(lin.dm, alloc=arena.take)
            out[name] = lin
        torch.cuda.current_stream().synchronize()
        copy_stream.synchronize()
    if arena.off != total:
        raise RuntimeError(f"arena plan {total} bytes, used {arena.off}: the plan and the loader disagree")
    out.arena = arena
    out.stats = {"arena_bytes": total, "h2d_bytes": h2d, "matrices": len(names), "staging_bytes": 2 * stage_bytes}
    return out


def pool_layouts(linears) -> int:
    """Move the kernel layouts (and file-order tensors) of PackedLinears that were built one by one into one exact-size
    buffer per device and repoint them; the per-tensor allocations are released. Call before capturing CUDA graphs
    that use these matrices: single-matrix launchers and L8Group read the pointers at every call, but a captured
    graph, a PeerReduceGemv or a decode engine built earlier keeps the old addresses (build those afterwards).
    Returns the bytes now pooled."""
    lins = [l for l in linears if not getattr(l, "_pooled", False)]
    pooled = 0
    for dev in {l.dm.device for l in lins}:
        slots = []
        for l in (x for x in lins if x.dm.device == dev):
            objs = [l.dm] + [o for o in (l._l8, l._t16, getattr(l, "_x16", None)) if o is not None]
            for o in objs:
                for attr in ("tags", "tags2", "table", "table2", "row_scale", "row_book", "row_mask", "perms", "words", "words_c", "frag", "frag2",
                             "row_index", "tile_rows", "tile_mask"):
                    v = getattr(o, attr, None)
                    if isinstance(v, torch.Tensor):
                        slots.append((o, attr, v))
            l._pooled = True
        with torch.cuda.device(dev):
            arena = Arena(sum(_al(v.numel() * v.element_size()) for _, _, v in slots), dev)
            for o, attr, v in slots:
                new = arena.take(v.numel() * v.element_size()).view(v.dtype).view(v.shape)
                new.copy_(v)
                setattr(o, attr, new)
        pooled += arena.buf.numel()
    return pooled
