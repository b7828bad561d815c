"""vLLM-free serving layer: stacked packed pieces (q|k|v, gate|up) behind one forward(), a handle
registry and the `shapequant::linear` torch custom op.

Mirrors shapequant/vllm_ext/core.py of the reference: PackedShards (:212-486: from_packed, forward,
dense, nbytes, R, C), register (:622-624) and linear_op with its fake implementation (:693-702), so
that vLLM's LinearMethod.apply can stay `torch.ops.shapequant.linear(x, handle)`.

Dispatch on the number of tokens M: 1 -> batch-1 kernel per piece, <= bmax -> small-batch
tensor-core kernel per piece, each writing its column slice of the stacked output; larger ->
the fused decode + tcgen05 GEMM per piece into its slice (pieces with several column orders: decode
to x's 16-bit dtype into a shared scratch followed by a library GEMM)."""

from __future__ import annotations


import torch

from ..kernels import DenseStack, L8Group, T16Matrix
from ..linear import DENSE_MIN_TOKENS, L8_MIN_ROWS, ROWS_MIN_TOKENS, PackedLinear

BMAX = T16Matrix.BMAX

# vLLM fuses some HF projections into one layer; the packed file keeps the HF pieces
STACKED = {"self_attn.qkv_proj": ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"),
           "mlp.gate_up_proj": ("mlp.gate_proj", "mlp.up_proj")}
def packed_pieces(prefix: str, names) -> list[str] | None:
    """Packed matrix names (model.layers.N.<kind>) that make up the vLLM layer at `prefix`: the HF pieces of a fused
    projection, in order.  None when the layer is not a block linear or none of its pieces is in the file; an error
    when only some are (the rule of shapequant/vllm_ext/core.py:127-142)."""
    parts = prefix.split(".")
    if "layers" not in parts:
        return None
    at = len(parts) - 1 - parts[::-1].index("layers")           # the last "layers" component
    if at + 2 >= len(parts) or not parts[at + 1].isdigit():
        return None
    layer, kind = parts[at + 1], ".".join(parts[at + 2:])
    wanted = [f"model.layers.{layer}.{piece}" for piece in STACKED.get(kind, (kind,))]
    present = [name for name in wanted if name in names]
    if len(present) == len(wanted):
        return wanted
    if present:
        raise ValueError(f"{prefix}: only some of its pieces are packed ({wanted})")
    return None


class PackedShards:
    def __init__(self, lins: list[PackedLinear], *, bmax: int = BMAX, **_ignored):
        if not lins:
            raise ValueError("no pieces")
        C = {lin.C for lin in lins}
        if len(C) != 1:
            raise ValueError(f"stacked pieces disagree on the input size: {sorted(C)}")
        if bmax > BMAX:
            raise ValueError(f"bmax {bmax} over {BMAX}")
        self.lins = lins
        self.C = C.pop()
        self.Rs = [lin.R for lin in lins]
        self.R = sum(self.Rs)
        self.offs = [sum(self.Rs[:i]) for i in range(len(lins))]
        self.bmax = self.cross = bmax
        self.device = lins[0].dm.device
        self.sq_name = ""
        self.stack = DenseStack([lin.dm for lin in lins])     # many tokens / several column orders: decode once, one GEMM
        # Kernel layouts are second copies of the tags in a kernel's order: each is built when its token-count class
        # is first used (or by prepare()), so a layer that only ever decodes keeps one extra copy, not three.
        self.group = self.rows = None
        self._one_order = all(lin.dm.M == 1 for lin in lins) and len(lins) <= L8Group.MAX
        self._ready: set = set()
        self.prepare(1)

    def _class_of(self, M: int) -> str:
        if M == 1:
            return "one"
        if M <= self.cross:
            return "rows" if (M >= ROWS_MIN_TOKENS and self._one_order and len({lin.dm.books for lin in self.lins}) == 1) else f"small{M}"
        return "many"

    def prepare(self, M: int) -> None:
        """Build whatever forward() needs for M tokens (kernel layouts, staging buffers).  forward() calls it on
        first use; call it yourself for every token count a CUDA graph will replay, before capturing."""
        cls = self._class_of(M)
        if cls in self._ready:
            return
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"PackedShards.prepare({M}) must run before the stream is captured (layouts are allocated on first use)")
        if cls == "one":
            if self._one_order and self.R >= L8_MIN_ROWS:
                self.group = L8Group([lin.l8 for lin in self.lins])       # all pieces in one launch
            else:
                for lin in self.lins:
                    lin.l8 if lin.use_l8() else lin.small_batch(1).xp_buffer(1)
        elif cls == "rows":
            self.rows = self.group if self.group is not None else L8Group([lin.l8 for lin in self.lins])
            self.rows._structs_c                                      # (built by the first gemm_rows otherwise)
        elif cls.startswith("small"):
            for lin in self.lins:
                lin.small_batch(M).xp_buffer(M)
        self._ready.add(cls)

    @classmethod
    def from_packed(cls, pf, names: list[str], dev="cuda", **kw) -> "PackedShards":
        return cls([PackedLinear.from_packed(pf, n, device=dev) for n in names], **kw)

    def nbytes(self) -> int:
        n = 0
        for lin in self.lins:
            n += lin.stored_bytes()
            n += lin._t16.nbytes() if lin._t16 is not None else 0
            n += lin._x16.nbytes() if getattr(lin, "_x16", None) is not None else 0
            n += lin._l8.nbytes() if lin._l8 is not None else 0
        return n

    def dense(self) -> torch.Tensor:
        """fp16 [R, C] (testing)."""
        return torch.cat([lin.dm.dequant(dtype=torch.float16) for lin in self.lins])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [..., C] -> [..., R] in x's dtype."""
        shp = x.shape
        x2 = x.reshape(-1, self.C)
        M = x2.shape[0]
        if M == 0:
            y = x2.new_empty(0, self.R)
        elif M <= self.cross:
            self.prepare(M)
            xin = x2 if x2.dtype in (torch.float16, torch.bfloat16) else x2.to(torch.bfloat16)
            y = self._small(xin.contiguous(), M)
        else:
            xin = x2 if x2.dtype in (torch.float16, torch.bfloat16) else x2.to(torch.bfloat16)
            y = self._large(xin.contiguous())
        return y.to(x.dtype).view(*shp[:-1], self.R)

    def _small(self, x: torch.Tensor, M: int) -> torch.Tensor:
        y = torch.empty(M, self.R, dtype=x.dtype, device=x.device)
        if M == 1 and self.group is not None:
            self.group.run(x[0], [y[0, off:off + R] for off, R in zip(self.offs, self.Rs)])
            return y
        if self._class_of(M) == "rows":
            self.rows.gemm_rows(x, [y[:, off:off + R] for off, R in zip(self.offs, self.Rs)])
            return y
        for lin, off, R in zip(self.lins, self.offs, self.Rs):
            if M == 1 and lin.use_l8():
                lin.l8.run(x[0], y[0, off:off + R])
            else:
                lin.small_batch(M).run(x, y[:, off:off + R], M)
        return y

    def _large(self, x: torch.Tensor) -> torch.Tensor:
        y = torch.empty(x.shape[0], self.R, dtype=x.dtype, device=x.device)
        if x.shape[0] >= DENSE_MIN_TOKENS or not all(lin.use_gemm() for lin in self.lins):
            return self.stack.gemm(x, y)                  # all pieces decoded once, one TMA-fed tcgen05 GEMM over the stacked rows
        for lin, off, R in zip(self.lins, self.offs, self.Rs):
            lin.l8.gemm(x, y[:, off:off + R])             # fused decode + tcgen05 GEMM straight into the column slice
        return y


# ------------------------------------------------------------------ torch custom op

_REGISTRY: list = []


def register(ps) -> int:
    _REGISTRY.append(ps)
    return len(_REGISTRY) - 1


@torch.library.custom_op("shapequant::linear", mutates_args=())
def linear_op(x: torch.Tensor, handle: int) -> torch.Tensor:
    return _REGISTRY[handle].forward(x)


@linear_op.register_fake
def _(x: torch.Tensor, handle: int) -> torch.Tensor:
    return x.new_empty(*x.shape[:-1], _REGISTRY[handle].R)
