"""The packed-linear call surfaces of the reference, backed by libcbl.

PackedLinear   mirrors shapequant/kernels/gemv.py:107-175 (from_packed, gemv, dense, forward, stored_bytes);
               more than 64 tokens run the fused decode + tcgen05 GEMM (the role of shapequant/kernels/runs_gemm.py:471-514)
RunsLin        mirrors shapequant/kernels/decode_e2e.py:405-443 (run(x, y) into a caller-provided buffer)
runs_linear    mirrors shapequant/runtime.py:41-51
RunsBatch      mirrors shapequant/kernels/batched_runs.py:680-771 (run(X, Y, B))

Differences that a caller can observe: the product kernels execute the benchmark format (d = 8,
12-bit tags, one 4096-entry book per matrix, optionally a second summed book and seeded column
orders) instead of the reference's d = 4 fast path, accumulate in fp32 throughout (no table
pre-scaling against fp16 overflow is needed), and apply column orders inside the kernels: callers
pass the plain activation vector, not permuted copies.
"""

from __future__ import annotations

import math

import torch

from .kernels import DeviceMatrix, L8Matrix, T16Matrix

# rows from which the batch-1 product uses activation-side tables instead of codeword lookups; with several column
# orders every order needs its own tables, so the rule applies to the rows per order (measured on B200: a table build
# costs as much as the lookups of ~1300 rows)
L8_MIN_ROWS = 2048
L8_MIN_ROWS_PER_ORDER = 1536
# tokens from which the two-phase path runs (decode the matrix once into a 16-bit scratch + TMA-fed tensor-core
# GEMM). Measured on B200 it beats the kernel that decodes weight tiles on the fly at every token count above the
# small-batch kernel's 64 (12.1 vs 20.6 ms for the 196 Qwen2.5-7B matrices at 128 tokens, 30 vs 36 ms at 2048).
DENSE_MIN_TOKENS = 65
# tokens from which (up to 64) matrices with one column order run on the tensor-core kernel that takes the weight
# rows as the M side (its cost does not grow with the token count; the mma.sync kernel wins below: 18944 x 3584 pair
# 66 us at any count against 49 / 63 / 132 us at 8 / 16 / 32 tokens)
ROWS_MIN_TOKENS = 17
# 9..16 tokens, one column order: the activation-stationary mma.sync kernel (18944 x 3584 pair 45 us at any count up to
# 16, against 72-75 us for the row-tile kernel at 12 / 16 tokens and 64 us for the rows-as-M kernel; up to 8 tokens the
# row-tile kernel is as fast inside a step: 3.26 / 3.60 ms for the 196-matrix set at 4 / 8 tokens against 3.40 / 3.61)
X16_MIN_TOKENS, X16_MAX_TOKENS = 9, 16


def _is_capturing() -> bool:
    return torch.cuda.is_current_stream_capturing()


class PackedLinear(torch.nn.Module):
    """A block linear run from packed tensors: one token -> batch-1 kernel, up to 64 tokens -> the
    small-batch tensor-core kernel, more -> fused decode + tcgen05 GEMM. Constructor arguments follow the
    reference (words, table, row_scale, row_book, row_mask, perms, K, d, bias)."""

    def __init__(self, words, table, row_scale, row_book, row_mask, perms, K: int, d: int, bias=None,
                 words2=None, table2=None, x_cols: int | None = None):
        super().__init__()
        dev = words.device
        if dev.type != "cuda":
            raise ValueError("PackedLinear needs CUDA tensors (no CPU path)")
        C = perms.shape[1] if perms is not None else None
        has_mask = row_mask is not None and perms is not None and perms.shape[0] > 1
        self.dm = DeviceMatrix(words, table, row_scale, row_book, row_mask if has_mask else None,
                               perms if has_mask else None, K=K, d=d, C=C, device=dev, tags2=words2, table2=table2, x_cols=x_cols)
        # x_cols: this is a column shard (tensor parallelism) of a matrix with several column orders; its orders name
        # positions of the full activation vector of that length, which forward() then expects
        self.wide = self.dm.x_cols is not None
        self.in_features = self.dm.x_cols if self.wide else self.dm.C
        self.R, self.C, self.K, self.d, self.W = self.dm.R, self.dm.C, K, d, self.dm.W
        self.bits, self.nch, self.has_mask = self.dm.bits, self.dm.nch, has_mask
        self.bias = bias
        self._t16: T16Matrix | None = None
        self._l8: L8Matrix | None = None

    @classmethod
    def from_packed(cls, pf, name: str, device="cuda", bias=None, **kw):
        m = pf.meta[name]
        t = pf.tensors(name)
        return cls(t["tags"].to(device), t["table"].to(device), t["row_scale"].to(device),
                   t["row_book"].to(device) if "row_book" in t else None,
                   t["row_mask"].to(device) if "row_mask" in t else None,
                   pf.perms(name).to(device), m["K"], m["d"], bias=bias, **kw)

    # lazily built kernel layouts (a second copy of the tags in the kernel's order)
    @property
    def t16(self) -> T16Matrix:
        if self._t16 is None:
            self._t16 = T16Matrix(self.dm)
        return self._t16

    @property
    def l8(self) -> L8Matrix:
        if self._l8 is None:
            self._l8 = L8Matrix(self.dm)
        return self._l8

    @property
    def x16(self):
        if getattr(self, "_x16", None) is None:
            from .kernels import X16Matrix
            self._x16 = X16Matrix(self.dm)
        return self._x16

    def small_batch(self, n: int):
        """The kernel layout that multiplies n <= 64 tokens by this matrix (prep / run_prepped / run / xp_buffer): the
        activation-stationary one for 2..16 tokens and one column order, else the row-tile one."""
        return self.x16 if (self.dm.M == 1 and X16_MIN_TOKENS <= n <= X16_MAX_TOKENS) else self.t16

    @property
    def rows_group(self):
        if getattr(self, "_rows_group", None) is None:
            from .kernels import L8Group
            self._rows_group = L8Group([self.l8])
        return self._rows_group

    def use_l8(self) -> bool:
        """One token runs on the table-lookup kernel (any number of column orders up to its limit)."""
        if not self.dm.fast:
            return False
        if self.dm.M == 1:
            return self.R >= L8_MIN_ROWS
        return self.dm.M <= L8Matrix.MAX_ORDERS and self.R >= L8_MIN_ROWS_PER_ORDER * self.dm.M

    def use_gemm(self) -> bool:
        """The tensor-core kernel that decodes weight tiles on the fly executes one column order (one or two
        books); matrices with several orders take the two-phase path at every token count above 64."""
        return self.dm.M == 1

    def gemv(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [C] (fp16 / bf16 / fp32, contiguous) -> y [R] in x's dtype (or `out`'s)."""
        if not self.dm.fast:            # any d / tag width / several books per matrix: the generic product
            y = out if out is not None else torch.empty(self.R, dtype=x.dtype, device=x.device)
            self.dm.gemv_generic(x.reshape(1, -1), y.reshape(1, -1))
            return y
        if self.use_l8():
            return self.l8.run(x, out, wide=self.wide)
        y = out if out is not None else torch.empty(self.R, dtype=x.dtype, device=x.device)
        self.t16.run(x.reshape(1, -1), y.reshape(1, -1), 1, wide=self.wide)
        return y

    def dense(self) -> torch.Tensor:
        """fp32 [R, C] reference-exact decode."""
        return self.dm.dequant(dtype=torch.float32)

    def forward_into(self, x2: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """y [n, R] (any of fp32 / fp16 / bf16, unit column stride) = x2 [n, C] . W^T, dispatched by n."""
        n = x2.shape[0]
        if n == 0:
            return y
        if not self.dm.fast:
            # formats outside d = 8 / 12-bit tags / one book per matrix: the generic product (a warp per row), which is
            # what the reference's own kernel is for them; a correctness path, whatever the token count
            self.dm.gemv_generic(x2 if x2.stride(1) == 1 else x2.contiguous(), y)
            return y
        if n == 1 and self.use_l8() and y.is_contiguous():
            self.l8.run(x2[0].contiguous(), y[0], wide=self.wide)
        elif X16_MIN_TOKENS <= n <= X16_MAX_TOKENS and self.dm.M == 1:
            self.x16.run(x2 if x2.stride(1) == 1 else x2.contiguous(), y)
        elif n <= T16Matrix.BMAX and (n < ROWS_MIN_TOKENS or self.dm.M > 1):
            self.t16.run(x2.contiguous(), y, n, wide=self.wide)
        elif n <= T16Matrix.BMAX:
            self.rows_group.gemm_rows(x2 if x2.stride(1) == 1 else x2.contiguous(), [y])
        elif self.use_gemm() and n < DENSE_MIN_TOKENS:
            self.l8.gemm(x2 if x2.stride(1) == 1 else x2.contiguous(), y)
        else:
            # many tokens, or several column orders: decode once into the shared 16-bit scratch, then the TMA-fed GEMM
            self.dm.gemm_dense(x2 if x2.stride(1) == 1 else x2.contiguous(), y)
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        n = math.prod(lead)
        y = self.forward_into(x.reshape(n, self.in_features), torch.empty(n, self.R, dtype=x.dtype, device=x.device))
        y = y.reshape(*lead, self.R)
        return y if self.bias is None else y + self.bias

    def stored_bytes(self) -> int:
        return self.dm.stored_bytes()


class RunsLin:
    """Engine linear: run(x, y) writes y [R] (or [B, R]) into a caller-provided buffer; no allocation
    and no host synchronisation in run(), so a decode step can be captured in one CUDA graph."""

    def __init__(self, lin: PackedLinear):
        self.lin, self.R, self.C = lin, lin.R, lin.C
        self.perms = lin.dm.perms
        if lin.use_l8():
            lin.l8          # build the layouts now, not inside a captured region
        else:
            lin.t16.xp_buffer(1)

    def run(self, x: torch.Tensor, y: torch.Tensor, epi: dict | None = None):
        """y = W . x.  `epi` asks for the operator that follows the product in a decode step to run with it, as the
        reference's run kernel does for its last blocks (shapequant/kernels/proto_runs.py:223-287, 505-520):
            dict(mode=1, h_in, h_out, w, eps, out)   h_out = h_in + y;  out = RMSNorm(h_out) * w
            dict(mode=2, out)                        this matrix is `gate`, epi["up"] a second RunsLin on the same x:
                                                     y = [gate.x | up.x] (2R values), out = silu(gate.x) * (up.x)
        (`src` of the reference's dict is this launch's own y and is accepted and ignored; `perms`, the M permuted
        copies of `out`, must be None: column orders are applied inside the next product here.)  h_in / h_out are the
        fp32 residual stream; y, w and out are in the model's 16-bit type.  One token, one column order."""
        if epi is None:
            if x.dim() == 1 or x.shape[0] == 1:
                self.lin.gemv(x.reshape(-1), y.reshape(-1))
            else:
                self.lin.t16.run(x, y, wide=self.lin.wide)
            return y
        import ctypes
        from . import _lib
        from .kernels import L8Group, _dt, _stream, l8_workspace
        if epi.get("perms") is not None:
            raise ValueError("epi['perms']: permuted copies of the output are not produced here (the next product applies its column orders itself)")
        if not self.lin.use_l8() or self.lin.dm.M != 1 or x.numel() != self.C:
            raise ValueError("fused epilogues run one token through the table-lookup kernel (one column order, at least 2048 rows)")
        mode, out = epi.get("mode"), epi["out"]
        xv = x.reshape(-1)
        if y.dtype not in (torch.float16, torch.bfloat16) or out.dtype != y.dtype:
            raise ValueError("fused epilogues write the model's 16-bit type")
        with torch.cuda.device(self.lin.dm.device):
            if mode == 1:
                h_in, h_out = epi["h_in"], epi.get("h_out", epi["h_in"])
                if h_in.dtype != torch.float32 or h_out.dtype != torch.float32:
                    raise ValueError("the residual stream is fp32")
                if h_out.data_ptr() != h_in.data_ptr():
                    h_out.copy_(h_in)
                st = (_lib.L8 * 1)(self.lin.l8.struct())
                ws = l8_workspace(self.lin.dm.device, self.R)
                _lib.check("cbl_gemv_l8_add_norm", _lib.lib.cbl_gemv_l8_add_norm(st, xv.data_ptr(), _dt(xv.dtype), h_out.data_ptr(), epi["w"].data_ptr(),
                                                                                 float(epi.get("eps", 1e-6)), out.data_ptr(), y.data_ptr(), _dt(y.dtype),
                                                                                 ws.data_ptr(), _stream()))
            elif mode == 2:
                up = epi["up"]
                if up.R != self.R or up.C != self.C or y.numel() != 2 * self.R:
                    raise ValueError("mode 2: `up` has this matrix's shape and y holds gate | up (2 R values)")
                grp = self._pair if getattr(self, "_pair", None) is not None and self._pair[0] is up else None
                if grp is None:
                    self._pair = grp = (up, L8Group([self.lin.l8, up.lin.l8]))
                yv = y.reshape(-1)
                ws = l8_workspace(self.lin.dm.device, 0, grp[1].ws_bytes)
                _lib.check("cbl_gemv_l8_silu_mul", _lib.lib.cbl_gemv_l8_silu_mul(grp[1]._structs, xv.data_ptr(), _dt(xv.dtype), out.data_ptr(),
                                                                                 yv.data_ptr(), yv.data_ptr() + self.R * yv.element_size(), _dt(y.dtype),
                                                                                 ws.data_ptr(), _stream()))
            else:
                raise ValueError("epi['mode'] is 1 (add + RMSNorm) or 2 (silu * up)")
        return y

    def nbytes(self) -> int:
        return self.lin.stored_bytes()


def runs_linear(pf, name: str, dev="cuda", **_ignored) -> RunsLin:
    """One packed matrix of a PackedFile as an engine linear (keyword arguments that tune the
    reference's launch geometry are accepted and ignored)."""
    m = pf.meta[name]
    if m["d"] != 8 or m["K"] != 4096 or m["G"] != 1:
        raise ValueError(f"{name}: the kernels execute d=8, K=4096, G=1 (d={m['d']}, K={m['K']}, G={m['G']})")
    return RunsLin(PackedLinear.from_packed(pf, name, device=dev))


class RunsBatch:
    """Batched launcher for one matrix: run(X [B, C], Y [B, R]) for any B <= bmax. X fp16 or bf16
    contiguous; Y fp16 / bf16 with unit column stride, e.g. a column slice of a wider stacked output
    (its row stride is passed through)."""

    def __init__(self, lin: PackedLinear | RunsLin, bmax: int = 32, **_ignored):
        self.lin = lin.lin if isinstance(lin, RunsLin) else lin
        if bmax > T16Matrix.BMAX:
            raise ValueError(f"bmax {bmax} over {T16Matrix.BMAX}")
        self.R, self.C, self.bmax = self.lin.R, self.lin.C, bmax
        for b in range(1, bmax + 1):
            self.lin.small_batch(b).xp_buffer(b)

    def run(self, X: torch.Tensor, Y: torch.Tensor, B: int | None = None) -> torch.Tensor:
        B = X.shape[0] if B is None else B
        ok = (torch.float16, torch.bfloat16)
        if not (B <= self.bmax and X.is_contiguous() and X.dtype in ok and Y.dtype in ok):
            raise ValueError("RunsBatch.run: B <= bmax, X contiguous, X and Y fp16 or bf16")
        if Y.stride(-1) != 1 or Y.shape[-1] != self.R:
            raise ValueError("RunsBatch.run: Y must be [B, R] with unit column stride")
        return self.lin.t16.run(X, Y, B, wide=True) if self.lin.wide else self.lin.small_batch(B).run(X, Y, B)
