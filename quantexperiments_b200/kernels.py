"""Device-side matrices and kernel launchers over libcbl (thin, allocation-aware Python).

DeviceMatrix  the file layout resident on the GPU: dense decode, tag unpacking
T16Matrix     row-tile re-layout + tensor-core product for batches up to 64 (column orders and
              two summed books supported)
L8Matrix      column-tile re-layout + batch-1 product by activation-side tables

All launches go to torch's current CUDA stream; outputs can be caller-provided so that steady-state
calls allocate nothing (CUDA-graph capturable)."""

from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from ._lib import lib

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise ValueError(f"dtype {t} is not supported (float32, float16, bfloat16)") from None


class DeviceMatrix:
    """One packed matrix in the file layout on a CUDA device (tags int32 [R, W], table fp16
    [G*K, d], row_scale fp16 [R], optional row_book / row_mask uint8 [R], perms int32 [M, C];
    optional second tag plane + table for two summed books)."""

    def __init__(self, tags, table, row_scale, row_book=None, row_mask=None, perms=None, *, K: int, d: int,
                 C: int | None = None, device="cuda", tags2=None, table2=None, x_cols: int | None = None):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("DeviceMatrix lives on a CUDA device; there is no CPU path")
        self.device = dev
        self.K, self.d = int(K), int(d)
        self.bits = int(math.log2(K))
        if 1 << self.bits != K:
            raise ValueError(f"K={K} is not a power of two")
        self.tags = tags.to(dev, torch.int32).contiguous()
        dev = self.device = self.tags.device          # normalised ("cuda" -> "cuda:0")
        self.R, self.W = self.tags.shape
        self.table = table.to(dev, torch.float16).contiguous()
        if self.table.shape[1] != d or self.table.shape[0] % K:
            raise ValueError(f"table shape {tuple(self.table.shape)} does not fit K={K}, d={d}")
        self.G = self.table.shape[0] // K
        self.row_scale = row_scale.to(dev, torch.float16).contiguous()
        self.row_book = None if row_book is None else row_book.to(dev, torch.uint8).contiguous()
        if self.G > 1 and self.row_book is None:
            raise ValueError("G > 1 needs row_book")
        self.M = 1 if (perms is None or row_mask is None) else int(perms.shape[0])
        self.row_mask = row_mask.to(dev, torch.uint8).contiguous() if self.M > 1 else None
        self.perms = perms.to(dev, torch.int32).contiguous() if self.M > 1 else None
        self.C = int(C) if C is not None else (int(perms.shape[1]) if perms is not None else (self.W * 32 // self.bits) * d)
        if self.C % d or self.W * 32 < (self.C // d) * self.bits:
            raise ValueError(f"C={self.C} does not fit d={d}, W={self.W}, bits={self.bits}")
        self.nch = self.C // d
        self.books = 1 if tags2 is None else 2
        self.tags2 = None if tags2 is None else tags2.to(dev, torch.int32).contiguous()
        self.table2 = None if table2 is None else table2.to(dev, torch.float16).contiguous()
        if self.books == 2 and (self.table2 is None or self.tags2.shape != self.tags.shape or self.G != 1):
            raise ValueError("two summed books need tags2 and table2 of matching shape and G = 1")
        # A column shard (tensor parallelism) of a matrix with several column orders keeps orders that name positions
        # of the FULL activation vector: x_cols is that vector's length (None: the activations are C long).
        self.x_cols = None if x_cols is None or int(x_cols) == self.C else int(x_cols)
        if self.x_cols is not None and (self.M == 1 or self.x_cols < self.C):
            raise ValueError("x_cols (wider activations than columns) needs several column orders and x_cols >= C")

    @classmethod
    def tags_only(cls, words: torch.Tensor, bits: int, n: int) -> "DeviceMatrix":
        """A matrix with a dummy one-value table, for unpacking a tag stream."""
        dev = words.device
        return cls(words, torch.zeros(1 << bits, 1, dtype=torch.float16, device=dev),
                   torch.ones(words.shape[0], dtype=torch.float16, device=dev), K=1 << bits, d=1, C=n, device=dev)

    def struct(self) -> _lib.Packed:
        return _lib.Packed(self.R, self.C, self.d, self.bits, self.G, self.M, self.books, self.W, _ptr(self.tags),
                           _ptr(self.tags2), _ptr(self.table), _ptr(self.table2), _ptr(self.row_scale),
                           _ptr(self.row_book), _ptr(self.row_mask), _ptr(self.perms))

    def stored_bytes(self) -> int:
        """Bytes a product must stream: tags, tables, row scales (the definition of the reference's
        PackedLinear.stored_bytes, shapequant/kernels/gemv.py:172-175)."""
        ts = [self.tags, self.table, self.row_scale, self.tags2, self.table2]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def dequant(self, out: torch.Tensor | None = None, dtype: torch.dtype = torch.float32,
                rows: tuple[int, int] | None = None) -> torch.Tensor:
        """Dense [r1 - r0, C] decode, bit-exact with the reference decode (fp32) or one rounding of
        it (fp16 / bf16). `out` may be a larger flat scratch buffer (its first (r1-r0)*C elements are used)."""
        if self.x_cols is not None:
            raise ValueError("a column shard whose column orders index the full activation vector has no [R, C] decode "
                             "(its weights are positions of that vector: gemm_dense decodes it x_cols wide)")
        r0, r1 = rows if rows is not None else (0, self.R)
        n = (r1 - r0) * self.C
        if out is None:
            res = torch.empty(r1 - r0, self.C, dtype=dtype, device=self.device)
        else:
            if out.numel() < n or not out.is_contiguous() or out.device != self.device:
                raise ValueError("out must be a contiguous buffer on the matrix's device with room for the rows")
            res = out.view(-1)[:n].view(r1 - r0, self.C)
        with torch.cuda.device(self.device):
            _lib.check("cbl_dequant", lib.cbl_dequant(ctypes.byref(self.struct()), res.data_ptr(), _dt(res.dtype),
                                                      self.C, r0, r1, _stream()))
        return res

    def gemm_dense(self, X: torch.Tensor, Y: torch.Tensor | None = None) -> torch.Tensor:
        """Y [T, R] = X [T, C] . W^T through the two-phase path (see DenseStack).  A shard with x_cols takes X
        [T, x_cols]: it is decoded once into a zeroed 16-bit scratch as wide as the activation vector (its orders name
        positions of that vector) and multiplied over all x_cols columns - every rank multiplies the full width, its rows
        being 1 / world dense, so for such shards this path buys tensor-core speed on long inputs, not a per-rank saving."""
        if self.x_cols is None:
            return DenseStack([self]).gemm(X, Y)
        _need_fast(self)
        T, Cx = X.shape[0], self.x_cols
        if X.dim() != 2 or X.shape[1] != Cx or X.stride(1) != 1 or X.device != self.device:
            raise ValueError("X must be [T, x_cols] with unit column stride on the matrix's device")
        if Y is None:
            Y = torch.empty(T, self.R, dtype=X.dtype, device=self.device)
        if Y.shape != (T, self.R) or Y.stride(1) != 1:
            raise ValueError("Y must be [T, R] with unit column stride")
        if T == 0 or self.R == 0:
            return Y
        key = (self.device.index, _stream())
        need = lib.cbl_dense_scratch_bytes(self.R, Cx)
        pair = DenseStack._scratch.setdefault(key, [None, None, 0])     # the two alternating scratches of the device and stream
        pair[2] ^= 1
        sc = pair[pair[2]]
        if sc is None or sc.numel() < need:
            sc = pair[pair[2]] = torch.empty(need, dtype=torch.uint8, device=self.device)
        nst = lib.cbl_gemm_stage_bytes(T, Cx) + 16
        st = DenseStack._stage.get(key)
        if st is None or st.numel() < nst:
            st = DenseStack._stage[key] = torch.zeros(nst, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            sc[:need].zero_()
            s = _stream()
            _lib.check("cbl_decode_raw_wide", lib.cbl_decode_raw_wide(ctypes.byref(self.struct()), sc.data_ptr(), Cx, s))
            _lib.check("cbl_gemm_dense", lib.cbl_gemm_dense(sc.data_ptr(), self.R, Cx, self.row_scale.data_ptr(), X.data_ptr(), _dt(X.dtype), T,
                                                            X.stride(0), Y.data_ptr(), _dt(Y.dtype), Y.stride(0), st.data_ptr(),
                                                            st.data_ptr() + st.numel() - 16, s))
        return Y

    @property
    def fast(self) -> bool:
        """The format the table-lookup and tensor-core kernels execute (d = 8, 12-bit tags, one book per matrix)."""
        return self.d == 8 and self.bits == 12 and self.G == 1

    def gemv_generic(self, X: torch.Tensor, Y: torch.Tensor | None = None) -> torch.Tensor:
        """Y [T, R] = X [T, C] . W^T for any format the layout holds (any d, tag width, books per matrix, column orders):
        the correctness path for formats outside the benchmark's; fp32 accumulate."""
        if X.dim() == 1:
            X = X[None]
        width = self.x_cols if self.x_cols is not None else self.C
        if X.dim() != 2 or X.shape[1] != width or X.stride(1) != 1 or X.device != self.device:
            raise ValueError("X must be [T, C] with unit column stride on the matrix's device")
        T = X.shape[0]
        if Y is None:
            Y = torch.empty(T, self.R, dtype=X.dtype, device=self.device)
        if Y.shape != (T, self.R) or Y.stride(1) != 1:
            raise ValueError("Y must be [T, R] with unit column stride")
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_generic", lib.cbl_gemv_generic(ctypes.byref(self.struct()), X.data_ptr(), _dt(X.dtype), T, X.stride(0) if T > 1 else width,
                                                                Y.data_ptr(), _dt(Y.dtype), Y.stride(0) if T > 1 else self.R, _stream()))
        return Y

    def unpack(self, plane: int = 0) -> torch.Tensor:
        out = torch.empty(self.R, self.nch, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check("cbl_unpack_tags", lib.cbl_unpack_tags(ctypes.byref(self.struct()), plane, out.data_ptr(), _stream()))
        return out


def _need_fast(dm: DeviceMatrix) -> None:
    if dm.d != 8 or dm.bits != 12 or dm.G != 1:
        raise ValueError(f"the product kernels execute d=8, 12-bit tags, one codebook per matrix "
                         f"(got d={dm.d}, bits={dm.bits}, G={dm.G})")


def _alloc_i32(n: int, device, alloc=None) -> torch.Tensor:
    """n int32 elements on `device`: from `alloc` (a loader's arena: alloc(nbytes) -> uint8 view) or the caching allocator."""
    if alloc is None:
        return torch.empty(n, dtype=torch.int32, device=device)
    return alloc(n * 4).view(torch.int32)


class T16Matrix:
    """Row-tile layout: rows grouped by column order into tiles of 16; run() multiplies a batch."""

    BMAX = 64

    def __init__(self, dm: DeviceMatrix, alloc=None):
        _need_fast(dm)
        self.dm, self.R, self.C, self.M, self.books, self.device = dm, dm.R, dm.C, dm.M, dm.books, dm.device
        # tiles: rows of one column order, padded with -1 to whole tiles (the reference groups rows
        # by order the same way, shapequant/kernels/proto_runs.py:380-388)
        if dm.M > 1:
            mask = dm.row_mask.cpu().to(torch.int64)
            rows, tmask = [], []
            for m in range(dm.M):
                r = torch.nonzero(mask == m).flatten()
                if r.numel() == 0:
                    continue
                pad = (-r.numel()) % 16
                rows.append(torch.cat([r, torch.full((pad,), -1, dtype=torch.int64)]))
                tmask += [m] * ((r.numel() + pad) // 16)
            tile_rows = torch.cat(rows) if rows else torch.empty(0, dtype=torch.int64)
            self.tile_mask = torch.tensor(tmask, dtype=torch.int32, device=dm.device)
        else:
            pad = (-dm.R) % 16
            tile_rows = torch.cat([torch.arange(dm.R), torch.full((pad,), -1, dtype=torch.int64)])
            self.tile_mask = None
        self.tile_rows = tile_rows.to(torch.int32).to(dm.device).contiguous()
        self.ntile = self.tile_rows.numel() // 16
        self.nsuper = -(-dm.nch // 64)
        nbytes = lib.cbl_t16_bytes(self.ntile, dm.C, dm.books)
        self.words = _alloc_i32(max(nbytes, 16) // 4, dm.device, alloc)
        with torch.cuda.device(dm.device):
            _lib.check("cbl_repack_t16", lib.cbl_repack_t16(ctypes.byref(dm.struct()), self.tile_rows.data_ptr(), self.ntile,
                                                            self.words.data_ptr(), _stream()))
        self._xp: dict[int, torch.Tensor] = {}

    def struct(self) -> _lib.T16:
        dm = self.dm
        return _lib.T16(self.R, self.C, self.books, self.M, self.ntile, self.nsuper, _ptr(self.words), _ptr(self.tile_rows),
                        _ptr(self.tile_mask), _ptr(dm.table), _ptr(dm.table2), _ptr(dm.row_scale))

    def nbytes(self) -> int:
        return self.words.numel() * 4 + self.tile_rows.numel() * 4

    def xp_buffer(self, B: int) -> torch.Tensor:
        """Staging buffer for the fp16 (permuted, padded) activations of a batch of B; cached per
        padded batch size so that repeated calls allocate nothing."""
        nb = -(-B // 8)
        buf = self._xp.get(nb)
        if buf is None:
            buf = self._xp[nb] = torch.empty(lib.cbl_prep_x_bytes(B, self.C, self.M) // 2, dtype=torch.float16, device=self.device)
        return buf

    def run(self, X: torch.Tensor, Y: torch.Tensor | None = None, B: int | None = None, wide: bool = False) -> torch.Tensor:
        """Y [B, R] = X [B, C] . W^T. X f16 / bf16 / f32 with unit column stride; Y f16 / bf16 / f32
        with unit column stride (e.g. a column slice of a wider output; its row stride is passed on).
        wide=True (matrices with column orders only): X is wider than C and the column orders index
        into the wide rows (a tensor-parallel input shard that reads the full activation vector)."""
        if X.dim() == 1:
            X = X[None]
        B = X.shape[0] if B is None else B
        if B < 1 or B > self.BMAX:
            raise ValueError(f"batch {B} outside 1..{self.BMAX}")
        if wide and self.M == 1:
            raise ValueError("wide activations need column orders")
        if (X.shape[-1] != self.C and not wide) or X.stride(-1) != 1 or X.device != self.device:
            raise ValueError("X must be [B, C] with unit column stride on the matrix's device")
        if Y is None:
            Y = torch.empty(B, self.R, dtype=X.dtype, device=self.device)
        if Y.shape[-1] != self.R or Y.stride(-1) != 1:
            raise ValueError("Y must be [B, R] with unit column stride")
        ldy = Y.stride(0) if Y.dim() == 2 else self.R
        xp = self.xp_buffer(B)
        with torch.cuda.device(self.device):
            s = _stream()
            _lib.check("cbl_prep_x", lib.cbl_prep_x(X.data_ptr(), _dt(X.dtype), B, self.C, X.stride(0), _ptr(self.dm.perms), self.M,
                                                    xp.data_ptr(), s))
            _lib.check("cbl_gemv_t16", lib.cbl_gemv_t16(ctypes.byref(self.struct()), xp.data_ptr(), B, Y.data_ptr(), _dt(Y.dtype),
                                                        ldy, s))
        return Y

    def prep(self, X: torch.Tensor, B: int) -> torch.Tensor:
        """Stage a batch of activations once for several matrices that share it and its column orders
        (q|k|v, gate|up): returns the staging buffer to pass to run_prepped()."""
        xp = self.xp_buffer(B)
        with torch.cuda.device(self.device):
            _lib.check("cbl_prep_x", lib.cbl_prep_x(X.data_ptr(), _dt(X.dtype), B, self.C, X.stride(0), _ptr(self.dm.perms), self.M,
                                                    xp.data_ptr(), _stream()))
        return xp

    def run_prepped(self, xp: torch.Tensor, Y: torch.Tensor, B: int) -> torch.Tensor:
        """The product alone, on activations staged by prep() of a matrix with the same input size and column orders."""
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_t16", lib.cbl_gemv_t16(ctypes.byref(self.struct()), xp.data_ptr(), B, Y.data_ptr(), _dt(Y.dtype),
                                                        Y.stride(0) if Y.dim() == 2 else self.R, _stream()))
        return Y


class X16Matrix:
    """Activation-stationary layout for 16..32 tokens (one column order): a warp keeps its 128 columns of the
    batch in registers and walks over the weight rows on mma.sync.  d = 8, 12-bit tags, G = 1, M = 1."""

    BMAX = 32

    def __init__(self, dm: DeviceMatrix, alloc=None):
        _need_fast(dm)
        if dm.M != 1:
            raise ValueError("the x16 layout needs a single column order")
        self.dm, self.R, self.C, self.books, self.device = dm, dm.R, dm.C, dm.books, dm.device
        self.nkr, self.nrb = -(-dm.nch // 16), -(-dm.R // 64)
        nbytes = lib.cbl_x16_bytes(dm.R, dm.C, dm.books)
        self.words = _alloc_i32(max(nbytes, 16) // 4, dm.device, alloc)
        self.ws = torch.zeros(max(lib.cbl_gemv_x16_workspace_bytes(dm.R), 16) // 4, dtype=torch.int32, device=dm.device)
        with torch.cuda.device(dm.device):
            _lib.check("cbl_repack_x16", lib.cbl_repack_x16(ctypes.byref(dm.struct()), self.words.data_ptr(), _stream()))
        self._xp: dict[int, torch.Tensor] = {}

    def struct(self) -> _lib.X16:
        dm = self.dm
        return _lib.X16(self.R, self.C, self.books, self.nkr, self.nrb, _ptr(self.words), _ptr(dm.table), _ptr(dm.table2),
                        _ptr(dm.row_scale))

    def nbytes(self) -> int:
        return self.words.numel() * 4

    def xp_buffer(self, B: int) -> torch.Tensor:
        nb = -(-B // 8)
        buf = self._xp.get(nb)
        if buf is None:
            buf = self._xp[nb] = torch.empty(lib.cbl_prep_x_bytes(B, self.C, 1) // 2, dtype=torch.float16, device=self.device)
        return buf

    def prep(self, X: torch.Tensor, B: int) -> torch.Tensor:
        """Stage a batch once for several matrices with the same input size (q|k|v, gate|up)."""
        xp = self.xp_buffer(B)
        with torch.cuda.device(self.device):
            _lib.check("cbl_prep_x", lib.cbl_prep_x(X.data_ptr(), _dt(X.dtype), B, self.C, X.stride(0), None, 1, xp.data_ptr(), _stream()))
        return xp

    def run_prepped(self, xp: torch.Tensor, Y: torch.Tensor, B: int) -> torch.Tensor:
        if B < 1 or B > self.BMAX:
            raise ValueError(f"batch {B} outside 1..{self.BMAX}")
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_x16", lib.cbl_gemv_x16(ctypes.byref(self.struct()), xp.data_ptr(), B, Y.data_ptr(), _dt(Y.dtype),
                                                        Y.stride(0) if Y.dim() == 2 else self.R, self.ws.data_ptr(), _stream()))
        return Y

    def run(self, X: torch.Tensor, Y: torch.Tensor | None = None, B: int | None = None) -> torch.Tensor:
        """Y [B, R] = X [B, C] . W^T for B <= 32; X and Y with unit column stride."""
        if X.dim() == 1:
            X = X[None]
        B = X.shape[0] if B is None else B
        if X.shape[-1] != self.C or X.stride(-1) != 1 or X.device != self.device:
            raise ValueError("X must be [B, C] with unit column stride on the matrix's device")
        if Y is None:
            Y = torch.empty(B, self.R, dtype=X.dtype, device=self.device)
        if Y.shape[-1] != self.R or Y.stride(-1) != 1:
            raise ValueError("Y must be [B, R] with unit column stride")
        return self.run_prepped(self.prep(X, B), Y, B)


class DenseStack:
    """Matrices that multiply the same activations (q|k|v, gate|up, or a single matrix), for many tokens or
    for matrices with several column orders: every matrix is decoded ONCE into a 16-bit scratch shared by
    all stacks of the device and stream (rows stacked in order), then one TMA-fed tensor-core GEMM writes
    Y [T, sum R]. d = 8, 12-bit tags, G = 1; one or two books; any number of column orders."""

    _scratch: dict = {}
    _stage: dict = {}

    def __init__(self, dms: list):
        for dm in dms:
            _need_fast(dm)
        if len({dm.C for dm in dms}) != 1 or len({dm.device for dm in dms}) != 1:
            raise ValueError("stacked matrices share the input size and the device")
        self.dms, self.C, self.device = dms, dms[0].C, dms[0].device
        self.R = sum(dm.R for dm in dms)
        self.row_scale = dms[0].row_scale if len(dms) == 1 else torch.cat([dm.row_scale for dm in dms])
        self.ld = (self.C + 7) // 8 * 8

    def gemm(self, X: torch.Tensor, Y: torch.Tensor | None = None) -> torch.Tensor:
        if X.dim() != 2 or X.shape[1] != self.C or X.stride(1) != 1 or X.device != self.device:
            raise ValueError("X must be [T, C] with unit column stride on the matrices' device")
        T = X.shape[0]
        if Y is None:
            Y = torch.empty(T, self.R, dtype=X.dtype, device=self.device)
        if Y.shape != (T, self.R) or Y.stride(1) != 1:
            raise ValueError("Y must be [T, sum R] with unit column stride")
        if T == 0 or self.R == 0:
            return Y
        key = (self.device.index, _stream())
        need = lib.cbl_dense_scratch_bytes(self.R, self.C)
        # two scratch buffers alternate: the decode of this stack may run beside the GEMM of the previous one
        pair = DenseStack._scratch.setdefault(key, [None, None, 0])
        pair[2] ^= 1
        sc = pair[pair[2]]
        if sc is None or sc.numel() < need:
            sc = pair[pair[2]] = torch.empty(need, dtype=torch.uint8, device=self.device)
        need = lib.cbl_gemm_stage_bytes(T, self.C) + 16
        st = DenseStack._stage.get(key)
        if st is None or st.numel() < need:
            st = DenseStack._stage[key] = torch.zeros(need, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            s, row = _stream(), 0
            for dm in self.dms:
                _lib.check("cbl_decode_raw", lib.cbl_decode_raw(ctypes.byref(dm.struct()), sc.data_ptr() + row * self.ld * 2, s))
                row += dm.R
            _lib.check("cbl_gemm_dense", lib.cbl_gemm_dense(sc.data_ptr(), self.R, self.C, self.row_scale.data_ptr(), X.data_ptr(), _dt(X.dtype),
                                                            T, X.stride(0), Y.data_ptr(), _dt(Y.dtype), Y.stride(0), st.data_ptr(),
                                                            st.data_ptr() + st.numel() - 16, s))
        return Y

    @classmethod
    def status(cls, device) -> None:
        """Synchronises and raises CblError if a bounded device-side wait of an earlier gemm() expired."""
        device = torch.device(device)
        key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
        st = cls._stage.get(key)
        if st is not None:
            torch.cuda.synchronize(device)
            if int(st[-16:].view(torch.int32)[0]) != 0:
                raise _lib.CblError("cbl_gemm_dense", _lib.ETIMEOUT, "a bounded device-side wait expired")


_WORKSPACES: dict[tuple, torch.Tensor] = {}
_RETIRED: list[torch.Tensor] = []       # outgrown work spaces stay alive: a captured graph may still point at them


def l8_workspace(device: torch.device, R: int, nbytes: int = 0) -> torch.Tensor:
    """Zero-initialised work space shared by every L8 product on (device, current stream): the kernels
    leave it zero. Products that may overlap on the device (different streams) get distinct buffers.
    16 MB to begin with (a launch needs 5.3 MB of partial-sum slots plus 4 bytes per output row); a larger request
    gets a new buffer and the old one is kept, so pointers handed out earlier (CUDA graphs) stay valid."""
    key = (device.index, _stream())
    need = max(lib.cbl_gemv_l8_workspace_bytes(R), nbytes)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _RETIRED.append(ws)
        ws = _WORKSPACES[key] = torch.zeros(max(need, 16 << 20), dtype=torch.uint8, device=device)
    return ws


class L8Matrix:
    """Column-tile layouts of one matrix.

    The batch-1 layout (tags rotated by row position, rows grouped by column order; any number of column
    orders up to 16) is built at construction and read by run() / L8Group.run().  The column-ordered variant
    that the tensor-core products read (gemm(), L8Group.gemm_rows(); one column order) is built on first use,
    so a matrix that only ever sees one token keeps a single copy of its tags."""

    MAX_ORDERS = _lib.L8_MAX_ORDERS

    def __init__(self, dm: DeviceMatrix, alloc=None):
        _need_fast(dm)
        if dm.M > self.MAX_ORDERS:
            raise ValueError(f"the table-lookup product supports at most {self.MAX_ORDERS} column orders (got {dm.M})")
        self.dm, self.R, self.C, self.M, self.books, self.device = dm, dm.R, dm.C, dm.M, dm.books, dm.device
        self.ntile = dm.books * (-(-dm.nch // 8))
        self._alloc = alloc
        # row positions: rows of one column order are contiguous, every order padded to a multiple of 32 rows
        # (the reference groups rows by order the same way, shapequant/kernels/proto_runs.py:380-388)
        if dm.M > 1:
            mask = dm.row_mask.cpu().to(torch.int64)
            parts, seg = [], [0]
            for m in range(dm.M):
                r = torch.nonzero(mask == m).flatten()
                pad = (-r.numel()) % 32
                parts.append(torch.cat([r, torch.full((pad,), -1, dtype=torch.int64)]))
                seg.append(seg[-1] + r.numel() + pad)
            self.row_index = torch.cat(parts).to(torch.int32).to(dm.device).contiguous()
            self.seg_off = seg
        else:
            self.row_index = None
            self.seg_off = [0, (dm.R + 31) // 32 * 32]
        self.Rpad = self.seg_off[-1]
        nbytes = lib.cbl_l8r_bytes(self.Rpad, dm.C, dm.books)
        self.words = _alloc_i32(max(nbytes, 16) // 4, dm.device, alloc)
        self.frag = _alloc_i32(lib.cbl_book_frag_bytes() // 4, dm.device, alloc)
        self.frag2 = _alloc_i32(lib.cbl_book_frag_bytes() // 4, dm.device, alloc) if dm.books == 2 else None
        self.words_c = None                     # column-ordered variant, see struct_c()
        with torch.cuda.device(dm.device):
            _lib.check("cbl_repack_l8r", lib.cbl_repack_l8r(ctypes.byref(dm.struct()), _ptr(self.row_index), self.Rpad,
                                                            self.words.data_ptr(), _stream()))
            _lib.check("cbl_repack_book", lib.cbl_repack_book(dm.table.data_ptr(), self.frag.data_ptr(), _stream()))
            if dm.books == 2:
                _lib.check("cbl_repack_book", lib.cbl_repack_book(dm.table2.data_ptr(), self.frag2.data_ptr(), _stream()))
            # the exponent that scales the kernel's tables, read back once so that no launch has to fetch it
            e = ctypes.c_int32(0)
            _lib.check("cbl_book_norm_exp", lib.cbl_book_norm_exp(self.frag.data_ptr(), ctypes.byref(e), _stream()))
            self.book_exp, self.book_exp2 = e.value, 0
            if dm.books == 2:
                _lib.check("cbl_book_norm_exp", lib.cbl_book_norm_exp(self.frag2.data_ptr(), ctypes.byref(e), _stream()))
                self.book_exp2 = e.value

    def struct(self) -> _lib.L8:
        """The batch-1 layout (rot = 1)."""
        dm = self.dm
        seg = (ctypes.c_int32 * (_lib.L8_MAX_ORDERS + 1))(*(self.seg_off + [0] * (_lib.L8_MAX_ORDERS + 1 - len(self.seg_off))))
        return _lib.L8(self.R, self.C, self.books, self.ntile, self.Rpad, 1, self.M, self.book_exp, _ptr(self.words), _ptr(self.frag),
                       _ptr(self.frag2), _ptr(dm.row_scale), _ptr(dm.table), _ptr(dm.table2), _ptr(self.row_index),
                       _ptr(dm.perms), seg, self.book_exp2)

    def struct_c(self) -> _lib.L8:
        """The column-ordered layout (rot = 0) of the tensor-core products; built on first use."""
        dm = self.dm
        if dm.M != 1:
            raise ValueError("the tensor-core products on the column-tile layout support one column order (M = 1)")
        if self.words_c is None:
            nbytes = lib.cbl_l8_bytes(dm.R, dm.C, dm.books)
            self.words_c = _alloc_i32(max(nbytes, 16) // 4, dm.device, None)
            with torch.cuda.device(dm.device):
                _lib.check("cbl_repack_l8", lib.cbl_repack_l8(ctypes.byref(dm.struct()), self.words_c.data_ptr(), _stream()))
        seg = (ctypes.c_int32 * (_lib.L8_MAX_ORDERS + 1))()
        return _lib.L8(self.R, self.C, self.books, self.ntile, (self.R + 3) // 4 * 4, 0, 1, 0, _ptr(self.words_c), _ptr(self.frag),
                       _ptr(self.frag2), _ptr(dm.row_scale), _ptr(dm.table), _ptr(dm.table2), None, None, seg, 0)

    def nbytes(self) -> int:
        n = self.words.numel() * 4 + self.frag.numel() * 4 * self.books
        n += self.words_c.numel() * 4 if self.words_c is not None else 0
        return n + (self.row_index.numel() * 4 if self.row_index is not None else 0)

    def run_static(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """y [R] = W . x using the scratch array built into the library instead of a work-space tensor:
        for hosts that must not allocate (at most 65536 rows; calls must not overlap on the GPU). Both
        x and y are caller tensors; nothing is allocated here."""
        if self.R > lib.cbl_gemv_l8_static_max_rows():
            raise ValueError(f"{self.R} rows exceed the built-in scratch ({lib.cbl_gemv_l8_static_max_rows()} rows)")
        x, yv = x.reshape(-1), y.reshape(-1)
        if x.numel() != self.C or not x.is_contiguous() or yv.numel() != self.R or not yv.is_contiguous():
            raise ValueError("x must be a contiguous [C] vector and y a contiguous [R] vector")
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_l8_static", lib.cbl_gemv_l8_static(ctypes.byref(self.struct()), x.data_ptr(), _dt(x.dtype),
                                                                    yv.data_ptr(), _dt(y.dtype), _stream()))
        return y

    def static_status(self) -> None:
        """Synchronises and raises CblError if a run_static() product gave up on a bounded device-side wait."""
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_l8_static_status", lib.cbl_gemv_l8_static_status(_stream()))

    _stage: dict = {}

    def gemm(self, X: torch.Tensor, Y: torch.Tensor | None = None, two_sm: bool = False) -> torch.Tensor:
        """Y [T, R] = X [T, C] . W^T on the tensor cores (prefill). X f16 / bf16 / f32 with unit column
        stride; Y f16 / bf16 / f32 with unit column stride (its row stride is passed through).
        two_sm selects the cta_group::2 variant (pairs of thread blocks per tile)."""
        if self.books != 1 and two_sm:
            raise ValueError("the two-SM variant executes one book per matrix")
        if X.dim() != 2 or X.shape[1] != self.C or X.stride(1) != 1 or X.device != self.device:
            raise ValueError("X must be [T, C] with unit column stride on the matrix's device")
        T = X.shape[0]
        if Y is None:
            Y = torch.empty(T, self.R, dtype=X.dtype, device=self.device)
        if Y.shape != (T, self.R) or Y.stride(1) != 1:
            raise ValueError("Y must be [T, R] with unit column stride")
        if T == 0:
            return Y
        need = lib.cbl_gemm_stage_bytes(T, self.C)
        key = (self.device.index, _stream())
        st = L8Matrix._stage.get(key)
        if st is None or st.numel() < need:
            st = L8Matrix._stage[key] = torch.empty(need, dtype=torch.uint8, device=self.device)
        ws = l8_workspace(self.device, self.R)
        with torch.cuda.device(self.device):
            fn = lib.cbl_gemm_l8_2sm if two_sm else lib.cbl_gemm_l8
            _lib.check("cbl_gemm_l8", fn(ctypes.byref(self.struct_c()), X.data_ptr(), _dt(X.dtype), T, X.stride(0), Y.data_ptr(),
                                         _dt(Y.dtype), Y.stride(0), st.data_ptr(), ws.data_ptr() + ws.numel() - 16, _stream()))
        return Y

    def status(self, workspace: torch.Tensor | None = None) -> None:
        """Synchronises and raises CblError if a bounded device-side wait of an earlier run() expired."""
        ws = workspace if workspace is not None else l8_workspace(self.device, self.R)
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_l8_status", lib.cbl_gemv_l8_status(ws.data_ptr(), self.R, _stream()))

    def run(self, x: torch.Tensor, y: torch.Tensor | None = None, workspace: torch.Tensor | None = None, wide: bool = False) -> torch.Tensor:
        """y [R] = W . x for x [C] (f16 / bf16 / f32, contiguous).  wide=True (matrices with column orders only): x is
        longer than C and the column orders index into it (a tensor-parallel input shard reading the full vector)."""
        x = x.reshape(-1)
        if wide and self.M == 1:
            raise ValueError("wide activations need column orders")
        if (x.numel() != self.C and not wide) or not x.is_contiguous() or x.device != self.device:
            raise ValueError("x must be a contiguous [C] vector on the matrix's device")
        if y is None:
            y = torch.empty(self.R, dtype=x.dtype, device=self.device)
        yv = y.reshape(-1)
        if yv.numel() != self.R or not yv.is_contiguous():
            raise ValueError("y must be a contiguous [R] vector")
        ws = workspace if workspace is not None else l8_workspace(self.device, self.R)
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_l8", lib.cbl_gemv_l8(ctypes.byref(self.struct()), x.data_ptr(), _dt(x.dtype), yv.data_ptr(),
                                                      _dt(y.dtype), ws.data_ptr(), _stream()))
        return y


class L8Group:
    """Up to four column-tile matrices that read the same activation vector (q|k|v, gate|up), run as
    one launch: run(x, ys) writes each matrix's output into its own contiguous vector."""

    MAX = 4

    def __init__(self, mats: list[L8Matrix]):
        if not 1 <= len(mats) <= self.MAX:
            raise ValueError(f"a group holds 1..{self.MAX} matrices")
        if len({m.C for m in mats}) != 1 or len({m.device for m in mats}) != 1:
            raise ValueError("grouped matrices share the input size and the device")
        self.mats, self.C, self.device = mats, mats[0].C, mats[0].device
        self.Rs = [m.R for m in mats]
        self._built = None
        self._built_c = None                    # column-ordered variants, built on first use (gemm_rows)
        self._ys = (ctypes.c_void_p * len(mats))()
        self.ws_bytes = sum(lib.cbl_gemv_l8_workspace_bytes(m.R) for m in mats)
        self.rows_ws_bytes = lib.cbl_gemm_rows_workspace_bytes(sum((m.R + 3) // 4 * 4 for m in mats))
        self._rows_stage: dict = {}

    @property
    def _structs(self):
        """The matrices' batch-1 descriptors; rebuilt when a matrix's buffers have moved (loader.pool_layouts)."""
        key = tuple(m.words.data_ptr() for m in self.mats)
        if self._built is None or self._built[0] != key:
            self._built = (key, (_lib.L8 * len(self.mats))(*[m.struct() for m in self.mats]))
        return self._built[1]

    @property
    def _structs_c(self):
        """The matrices' column-ordered descriptors (the tensor-core products); the layout is built on first use."""
        if self._built_c is None:
            self._built_c = (_lib.L8 * len(self.mats))(*[m.struct_c() for m in self.mats])
        return self._built_c

    def gemm_rows(self, X: torch.Tensor, ys: list[torch.Tensor]) -> list[torch.Tensor]:
        """A few dozen tokens on the tensor cores with the weight rows as the M side: ys[i] [B, R_i] = X [B, C] . W_i^T.
        The outputs share one row stride (column slices of one stacked buffer, or equal-width tensors). More than
        32 tokens run as several launches of up to 32."""
        B = X.shape[0]
        nmax = lib.cbl_gemm_rows_max_tokens()
        if B > nmax:
            for b0 in range(0, B, nmax):
                self.gemm_rows(X[b0:b0 + nmax], [y[b0:b0 + nmax] for y in ys])
            return ys
        if X.dim() != 2 or X.shape[1] != self.C or X.stride(1) != 1 or X.device != self.device or B < 1:
            raise ValueError("X must be [B, C] with unit column stride on the matrices' device")
        if len(ys) != len(self.mats) or len({y.dtype for y in ys}) != 1:
            raise ValueError("one output per matrix, one dtype")
        ldy = ys[0].stride(0) if B > 1 else max(m.R for m in self.mats)
        for i, (y, R) in enumerate(zip(ys, self.Rs)):
            if y.shape != (B, R) or y.stride(1) != 1 or (B > 1 and y.stride(0) != ldy):
                raise ValueError("outputs must be [B, R_i] with unit column stride and a common row stride")
            self._ys[i] = y.data_ptr()
        key = _stream()
        st = self._rows_stage.get(key)
        if st is None:
            st = self._rows_stage[key] = torch.empty(lib.cbl_gemm_stage_bytes(lib.cbl_gemm_rows_max_tokens(), self.C), dtype=torch.uint8,
                                                     device=self.device)
        ws = l8_workspace(self.device, 0, self.rows_ws_bytes)
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemm_rows_multi", lib.cbl_gemm_rows_multi(self._structs_c, len(self.mats), X.data_ptr(), _dt(X.dtype), B, X.stride(0),
                                                                      self._ys, _dt(ys[0].dtype), ldy, st.data_ptr(), ws.data_ptr(), _stream()))
        return ys

    def run(self, x: torch.Tensor, ys: list[torch.Tensor]) -> list[torch.Tensor]:
        x = x.reshape(-1)
        if x.numel() != self.C or not x.is_contiguous() or x.device != self.device:
            raise ValueError("x must be a contiguous [C] vector on the matrices' device")
        if len(ys) != len(self.mats):
            raise ValueError("one output vector per matrix")
        dt = ys[0].dtype
        for i, (y, R) in enumerate(zip(ys, self.Rs)):
            if y.numel() != R or not y.is_contiguous() or y.dtype != dt:
                raise ValueError("outputs must be contiguous [R_i] vectors of one dtype")
            self._ys[i] = y.data_ptr()
        ws = l8_workspace(self.device, 0, self.ws_bytes)
        with torch.cuda.device(self.device):
            _lib.check("cbl_gemv_l8_multi", lib.cbl_gemv_l8_multi(self._structs, len(self.mats), x.data_ptr(), _dt(x.dtype), self._ys,
                                                                  _dt(dt), ws.data_ptr(), _stream()))
        return ys
