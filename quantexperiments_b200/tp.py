"""Tensor-parallel sharding of packed matrices (new design: the reference refuses tensor parallelism,
shapequant/vllm_ext/plugin.py:198-199).

Column-parallel linears (q, k, v, gate, up) split the OUTPUT rows: every row carries its own tags,
scale and column-order id, so a rank keeps a contiguous row range plus a full copy of the book(s).
Row-parallel linears (o, down) split the INPUT dimension at chunk boundaries: a rank keeps, for every
row, the tags of its chunk range (re-packed into its own bit stream), all row scales and the book(s),
and produces partial outputs that are summed across ranks (NCCL all-reduce over NVLink).

With several column orders (M > 1) a chunk range of a row-parallel matrix reads activations at
arbitrary global columns; the shard then keeps perms[:, c0:c1] (global indices) and is fed the FULL
activation vector (all-gathered by the caller), see RowParallelLinear.

The shard_* functions work on the file-layout tensors (CPU or GPU) and are pure index arithmetic, so
they are tested on CPU ranks; the linears launch the CUDA kernels."""

from __future__ import annotations

import math

import torch

from .packed import pack_bits, unpack_bits


def row_range(R: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of a column-parallel shard. R must split evenly (vLLM's rule); a KV projection with fewer
    heads than ranks is replicated by the caller instead (rank // (world // n_kv_heads))."""
    if R % world:
        raise ValueError(f"{R} rows do not split evenly over {world} ranks")
    n = R // world
    return rank * n, (rank + 1) * n


def col_range(C: int, d: int, rank: int, world: int) -> tuple[int, int]:
    """Columns of a row-parallel shard, cut at chunk boundaries."""
    nch = C // d
    if nch % world:
        raise ValueError(f"{nch} chunks do not split evenly over {world} ranks")
    n = nch // world
    return rank * n * d, (rank + 1) * n * d


def shard_rows(t: dict, meta: dict, r0: int, r1: int) -> tuple[dict, dict]:
    """File-layout tensors + metadata of rows [r0, r1) of a matrix (tags, row_scale, row_book,
    row_mask sliced; table and column orders unchanged)."""
    out = {"tags": t["tags"][r0:r1].contiguous(), "table": t["table"], "row_scale": t["row_scale"][r0:r1].contiguous()}
    for k in ("row_book", "row_mask"):
        if k in t:
            out[k] = t[k][r0:r1].contiguous()
    for k in ("tags2", "table2"):
        if k in t:
            out[k] = t[k][r0:r1].contiguous() if k == "tags2" else t[k]
    m = dict(meta, R=r1 - r0)
    return out, m


def _slice_stream(words: torch.Tensor, bits: int, nch: int, j0: int, j1: int) -> torch.Tensor:
    """Bit stream of chunks [j0, j1) of every row. Word-aligned ranges are sliced in place (all
    Qwen2.5 shapes at TP 2/4/8); anything else goes through unpack + pack."""
    n = j1 - j0
    if (j0 * bits) % 32 == 0 and ((n * bits) % 32 == 0 or j1 == nch):
        w0 = j0 * bits // 32
        return words[:, w0:w0 + (n * bits + 31) // 32].contiguous()
    tags = unpack_bits(words.cpu(), bits, nch)[:, j0:j1]
    return pack_bits(tags, bits).to(words.device)


def shard_cols(t: dict, meta: dict, c0: int, c1: int, perms: torch.Tensor | None = None) -> tuple[dict, dict, torch.Tensor | None]:
    """File-layout tensors + metadata of input columns [c0, c1) (chunk aligned) of a matrix, and the
    shard's column orders (global activation indices) when the matrix has several."""
    d, K = meta["d"], meta["K"]
    if c0 % d or c1 % d:
        raise ValueError("column ranges must be cut at chunk boundaries")
    bits = int(math.log2(K))
    nch = meta["C"] // d
    out = {"tags": _slice_stream(t["tags"], bits, nch, c0 // d, c1 // d), "table": t["table"], "row_scale": t["row_scale"]}
    if "tags2" in t:
        out["tags2"] = _slice_stream(t["tags2"], bits, nch, c0 // d, c1 // d)
        out["table2"] = t["table2"]
    for k in ("row_book", "row_mask"):
        if k in t:
            out[k] = t[k]
    m = dict(meta, C=c1 - c0)
    p = None if perms is None else perms[:, c0:c1].contiguous()
    return out, m, p


class PeerArena:
    """One symmetric-memory allocation per rank, mapped into every rank of `group`, carved into
    sub-buffers at identical offsets on all ranks (take() must be called in the same order everywhere).
    Used by the row-parallel linears that sum their partial outputs through peer pointers."""

    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.nbytes, self.used = nbytes, 0
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)                   # every rank's buffer is zero before anyone uses a peer's

    def take(self, nbytes: int) -> list[int]:
        """Per-rank addresses of a fresh zeroed sub-buffer (256-byte aligned)."""
        off = (self.used + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise ValueError("peer arena exhausted")
        self.used = off + nbytes
        return [p + off for p in self.ptrs]


class PeerReduceGemv:
    """Batch-1 product of one row-parallel shard fused with the sum over ranks through peer memory
    (cbl_gemv_l8_ar): run(x_slice, y) leaves the full y on every rank. All ranks must create these
    objects, and call run(), in the same order."""

    def __init__(self, l8, arena: PeerArena):
        import ctypes
        from ._lib import lib
        self.l8, self.rank, self.world = l8, arena.rank, arena.world
        ptrs = arena.take(lib.cbl_gemv_l8_ar_workspace_bytes(l8.R))
        self.ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.own = ptrs[self.rank]
        self._struct = l8.struct()

    def status(self) -> bool:
        """Synchronises the stream; False if a bounded wait of a run() since the last query expired (a peer's word or
        a staged copy never arrived: that call's output is invalid, later calls are correct again)."""
        from . import _lib
        from .kernels import _stream
        with torch.cuda.device(self.l8.device):
            rc = _lib.lib.cbl_gemv_l8_ar_status(self.own, self.l8.R, _stream())
        if rc not in (_lib.OK, _lib.ETIMEOUT):
            _lib.check("cbl_gemv_l8_ar_status", rc)
        return rc == _lib.OK

    def run(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """x: this rank's activation slice [C_local]; for a matrix with column orders the FULL activation vector (the
        shard's column orders hold global indices)."""
        import ctypes
        from . import _lib
        from .kernels import _dt, _stream
        xv, yv = x.reshape(-1), y.reshape(-1)
        wide_ok = self.l8.M > 1 and xv.numel() >= self.l8.C
        if (xv.numel() != self.l8.C and not wide_ok) or not xv.is_contiguous() or yv.numel() != self.l8.R or not yv.is_contiguous():
            raise ValueError("x must be this rank's contiguous activation slice and y a contiguous [R] vector")
        with torch.cuda.device(self.l8.device):
            _lib.check("cbl_gemv_l8_ar", _lib.lib.cbl_gemv_l8_ar(ctypes.byref(self._struct), xv.data_ptr(), _dt(xv.dtype), yv.data_ptr(),
                                                               _dt(y.dtype), self.ptrs, self.rank, self.world, _stream()))
        return y


class ColumnParallelLinear:
    """Rank-local part of a column-parallel packed linear: y_local [..., R / world] = x . W[r0:r1]^T.
    No communication; the caller gathers or consumes the sharded output."""

    def __init__(self, t: dict, meta: dict, perms: torch.Tensor | None, rank: int, world: int, device="cuda"):
        from .linear import PackedLinear
        r0, r1 = row_range(meta["R"], rank, world)
        ts, ms = shard_rows(t, meta, r0, r1)
        self.r0, self.r1 = r0, r1
        p = perms if perms is not None else torch.arange(meta["C"])[None]
        self.lin = PackedLinear(ts["tags"].to(device), ts["table"].to(device), ts["row_scale"].to(device),
                                ts["row_book"].to(device) if "row_book" in ts else None,
                                ts["row_mask"].to(device) if "row_mask" in ts else None, p.to(device), ms["K"], ms["d"],
                                words2=ts["tags2"].to(device) if "tags2" in ts else None,
                                table2=ts["table2"].to(device) if "table2" in ts else None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.lin(x)

    __call__ = forward


class RowParallelLinear:
    """Rank-local part of a row-parallel packed linear plus the sum over ranks:
    y = sum_ranks x[..., c0:c1] . W[:, c0:c1]^T. `x` is the rank's slice [..., C / world] when the
    matrix has one column order, or the full [..., C] vector when it has several (the shard's column
    orders index the full vector). reduce=False returns the partial product (for callers that
    reduce themselves, e.g. vLLM's RowParallelLinear)."""

    def __init__(self, t: dict, meta: dict, perms: torch.Tensor | None, rank: int, world: int, device="cuda", group=None,
                 arena: "PeerArena | None" = None):
        from .linear import PackedLinear
        self.rank, self.fused = rank, None
        c0, c1 = col_range(meta["C"], meta["d"], rank, world)
        multi = meta["M"] > 1
        ts, ms, ps = shard_cols(t, meta, c0, c1, perms if multi else None)
        self.c0, self.c1, self.group, self.world, self.multi = c0, c1, group, world, multi
        self.R, self.C_full = meta["R"], meta["C"]
        self.lin = PackedLinear(ts["tags"].to(device), ts["table"].to(device), ts["row_scale"].to(device),
                                ts["row_book"].to(device) if "row_book" in ts else None, ts["row_mask"].to(device) if multi else None,
                                ps.to(device) if multi else torch.arange(c1 - c0)[None].to(device), ms["K"], ms["d"],
                                words2=ts["tags2"].to(device) if "tags2" in ts else None,
                                table2=ts["table2"].to(device) if "table2" in ts else None, x_cols=meta["C"] if multi else None)
        if multi:       # column orders: every kernel gathers x through perms[:, c0:c1] from the full vector
            self.dm = self.lin.dm

    def partial(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 partial product [..., R] of this rank's column range."""
        lead = x.shape[:-1]
        n = math.prod(lead)
        y = torch.empty(n, self.R, dtype=torch.float32, device=x.device)
        self.lin.forward_into(x.reshape(n, self.lin.in_features), y)    # one token: table lookups; <= 64: row tiles; more: decode + GEMM
        return y.reshape(*lead, self.R)

    @property
    def l8_multi(self):
        """The batch-1 layout of a shard with column orders (at most 16 of them), built on first use."""
        from .kernels import L8Matrix
        return self.lin.l8 if self.lin.dm.M <= L8Matrix.MAX_ORDERS else None

    def attach(self, arena: "PeerArena") -> None:
        """Reserve this matrix's peer work space (call on every rank, in the same order)."""
        if self.multi:
            if self.l8_multi is None:
                raise ValueError("the fused path runs matrices with at most 16 column orders")
            self.fused = PeerReduceGemv(self.l8_multi, arena)
            return
        if not self.lin.use_l8():
            raise ValueError("the fused path runs matrices with at least 2048 rows")
        self.fused = PeerReduceGemv(self.lin.l8, arena)

    def forward_fused(self, x: torch.Tensor, y: torch.Tensor | None = None) -> torch.Tensor:
        """One token: product + sum over ranks through peer memory (no collective library call)."""
        if getattr(self, "fused", None) is None:
            raise ValueError("attach() a peer arena first")
        if y is None:
            y = torch.empty(self.R, dtype=x.dtype, device=x.device)
        return self.fused.run(x, y)

    def forward(self, x: torch.Tensor, reduce: bool = True) -> torch.Tensor:
        """Partials are kept in fp32 through the all-reduce and rounded to x's dtype once."""
        y = self.partial(x)
        if reduce and self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(y, group=self.group)
        return y.to(x.dtype)

    __call__ = forward

