"""Decode engine for Qwen2-architecture models whose block linears are packed codebook matrices.

Mirrors the reference's engine surface: `Cfg`, `DecodeEngine` (step / reset / capture / generate /
time_tokens / weight_bytes; shapequant/kernels/decode_e2e.py:313-327, 507-768), `Qwen2BatchEngine`
(B sequences per step sharing a batch-1 engine's weights, shapequant/runtime_batch.py:27-180),
`random_engine` (decode_e2e.py:770-817), and `start` / `generate` / `bench` (shapequant/runtime.py:166-280).

One step = embedding row, then per layer: add + RMSNorm, q|k|v, rotary + cache write, grouped-query
attention over the cache, o, add + RMSNorm, gate|up, silu * up, down; final norm, output head, greedy
argmax. The residual stream is fp32, activations are rounded to the model's 16-bit type between
operators. Every operator is a libcbl kernel launched on the current stream into preallocated
buffers, so a step is captured in one CUDA graph. Prompts run through `prefill`: the same operators
over all prompt tokens at once, the linears on the tcgen05 GEMM, causal attention by torch's
scaled_dot_product_attention (a library call: the only one on this path besides the batched head).
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import lib
from .kernels import DenseStack, L8Group, _dt, _stream
from .linear import DENSE_MIN_TOKENS, ROWS_MIN_TOKENS, PackedLinear, RunsLin

NAMES = ("q", "k", "v", "o", "gate", "up", "down")


@dataclass
class Cfg:
    hidden: int = 3584
    n_heads: int = 28
    n_kv: int = 4
    head_dim: int = 128
    inter: int = 18944
    vocab: int = 152064
    layers: int = 28
    rope_theta: float = 1e6
    eps: float = 1e-6
    max_len: int = 512


def _lin(obj) -> PackedLinear:
    return obj.lin if isinstance(obj, RunsLin) else obj


class DenseHead:
    """16-bit weight [V, H]: run(x [B, H], logits [B, V] fp32). Up to 8 sequences stream the weight once
    through the library's own kernel; larger batches are a plain library GEMM."""

    def __init__(self, w: torch.Tensor):
        if w.dtype not in (torch.float16, torch.bfloat16) or w.device.type != "cuda":
            raise ValueError("the head weight must be a CUDA fp16 / bf16 tensor")
        self.w = w.contiguous()
        self.R, self.C = w.shape
        self.perms = None

    def run(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        B = x.shape[0]
        if B <= lib.cbl_head_gemv_max_batch():
            _lib.check("cbl_head_gemv", lib.cbl_head_gemv(self.w.data_ptr(), x.data_ptr(), _dt(self.w.dtype), B, self.R, self.C,
                                                          logits.data_ptr(), _dt(logits.dtype), logits.stride(0), _stream()))
        else:
            logits.copy_(x @ self.w.t())

    def nbytes(self) -> int:
        return self.w.numel() * 2


class Q8Head:
    """The reference's 8-bit block-32 head (Q8Lin, shapequant/kernels/decode_e2e.py:385-402): q int8 [V, H], scale fp16
    [V, H/32]; run(x [B, H], logits [B, V] fp32). Up to 8 sequences per pass over the weights (more run as several passes)."""

    def __init__(self, q: torch.Tensor, sc: torch.Tensor):
        if q.dtype != torch.int8 or sc.dtype != torch.float16 or q.device.type != "cuda" or q.shape[1] % 32:
            raise ValueError("the 8-bit head is int8 [V, H] + fp16 [V, H/32] on a CUDA device, H a multiple of 32")
        self.q, self.sc = q.contiguous(), sc.contiguous()
        self.R, self.C = q.shape
        self.perms = None
        self._scratch = torch.empty(lib.cbl_head_q8_scratch_bytes(lib.cbl_head_gemv_q8_max_batch(), self.C), dtype=torch.uint8, device=q.device)

    @classmethod
    def from_weight(cls, w: torch.Tensor, dev="cuda") -> "Q8Head":
        from .packed import q8_pack
        q, sc = q8_pack(w.to(dev))
        return cls(q, sc)

    def run(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        nmax = lib.cbl_head_gemv_q8_max_batch()
        for b0 in range(0, x.shape[0], nmax):
            xb, lb = x[b0:b0 + nmax], logits[b0:b0 + nmax]
            _lib.check("cbl_head_gemv_q8", lib.cbl_head_gemv_q8(self.q.data_ptr(), self.sc.data_ptr(), xb.data_ptr(), _dt(x.dtype), xb.shape[0],
                                                                self.R, self.C, lb.data_ptr(), _dt(logits.dtype), logits.stride(0),
                                                                self._scratch.data_ptr(), _stream()))

    def nbytes(self) -> int:
        return self.q.numel() + self.sc.numel() * 2


class Q4Embed:
    """The reference's 4-bit block-32 token embedding (Q4Embed, shapequant/kernels/decode_e2e.py:370-382): q uint8
    [V, H/2], scale fp16 [V, H/32]. `dtype` names the model's activation type (the rows themselves decode to fp32)."""

    def __init__(self, q: torch.Tensor, sc: torch.Tensor, dtype=torch.bfloat16):
        if q.dtype != torch.uint8 or sc.dtype != torch.float16 or q.device.type != "cuda":
            raise ValueError("the 4-bit embedding is uint8 [V, H/2] + fp16 [V, H/32] on a CUDA device")
        self.q, self.sc, self.dtype = q.contiguous(), sc.contiguous(), dtype
        self.shape = (q.shape[0], q.shape[1] * 2)
        self.device = q.device

    @classmethod
    def from_weight(cls, w: torch.Tensor, dev="cuda", dtype=None) -> "Q4Embed":
        from .packed import q4_embed_pack
        q, sc = q4_embed_pack(w.to(dev))
        return cls(q, sc, dtype if dtype is not None else (w.dtype if w.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16))

    def rows(self, ids: torch.Tensor) -> torch.Tensor:
        from .packed import q4_embed_rows
        return q4_embed_rows(self.q, self.sc, ids)

    def nbytes(self) -> int:
        return self.q.numel() + self.sc.numel() * 2


class _Stage:
    """Linears that read the same input and write column slices of one [B, sum R] buffer (q|k|v, gate|up,
    or a single matrix). One token and one column order: one grouped table-lookup launch."""

    def __init__(self, lins: list, out: torch.Tensor):
        self.lins = [_lin(l) for l in lins]
        self.out, self.B = out, out.shape[0]
        self.offs, o = [], 0
        for l in self.lins:
            self.offs.append(o)
            o += l.R
        assert o == out.shape[1]
        self.group = self.rows = None
        one_order = all(l.dm.M == 1 for l in self.lins) and len(self.lins) <= L8Group.MAX and len({l.dm.books for l in self.lins}) == 1
        if self.B == 1 and one_order:
            self.group = L8Group([l.l8 for l in self.lins])
            self.ys = [out[0, o:o + l.R] for o, l in zip(self.offs, self.lins)]
        elif self.B >= ROWS_MIN_TOKENS and one_order:
            # a few dozen sequences: the tensor-core kernel with the weight rows as the M side, all matrices in one launch
            self.rows = L8Group([l.l8 for l in self.lins])
            self.ys = [out[:, o:o + l.R] for o, l in zip(self.offs, self.lins)]
        else:
            for l in self.lins:
                l.small_batch(self.B).xp_buffer(self.B)
            # one staging pass of the activations serves every matrix of the stage when they share the column orders
            p0 = self.lins[0].dm.perms
            self.share = all(l.dm.M == self.lins[0].dm.M and (l.dm.perms is p0 or (p0 is not None and l.dm.perms is not None
                                                                                     and torch.equal(l.dm.perms, p0)))
                             for l in self.lins)

    def run(self, x: torch.Tensor) -> None:
        if self.group is not None:
            self.group.run(x[0], self.ys)
        elif self.rows is not None:
            self.rows.gemm_rows(x, self.ys)
        elif self.share:
            xp = self.lins[0].small_batch(self.B).prep(x, self.B)
            for o, l in zip(self.offs, self.lins):
                l.small_batch(self.B).run_prepped(xp, self.out[:, o:o + l.R], self.B)
        else:
            for o, l in zip(self.offs, self.lins):
                l.forward_into(x, self.out[:, o:o + l.R])


class DecodeEngine:
    """layers: list of dicts with ln1, ln2 (16-bit [hidden]), q, k, v, o, gate, up, down (PackedLinear or
    RunsLin), bq, bk, bv (16-bit bias or None). B sequences advance together, each with its own cache and
    position. step() reads tok [B] at pos [B], writes logits [B, vocab] (fp32), tok (greedy next), pos += 1."""

    def __init__(self, cfg: Cfg, embed: torch.Tensor, layers: list, final_norm: torch.Tensor, lm_head, dev="cuda", B: int = 1,
                 attn_split: int | None = None):
        if cfg.head_dim != 128 or cfg.n_heads % cfg.n_kv or cfg.n_heads // cfg.n_kv > 8:
            raise ValueError("attention shape not supported: head_dim 128, at most 8 query heads per kv head")
        if not 1 <= B <= 64:
            raise ValueError(f"B = {B} outside 1..64")
        dev = torch.device(dev)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self.cfg, self.embed, self.layers, self.final_norm, self.lm_head, self.B, self.dev = cfg, embed, layers, final_norm, lm_head, B, dev
        self.dtype = dt = embed.dtype
        self.vocab_rows = embed.shape[0]
        if dt not in (torch.float16, torch.bfloat16):
            raise ValueError("the model's activation type is fp16 or bf16")
        H, NH, NKV, HD, I = cfg.hidden, cfg.n_heads, cfg.n_kv, cfg.head_dim, cfg.inter
        a = dict(dtype=dt, device=dev)
        self.h = torch.zeros(B, H, dtype=torch.float32, device=dev)
        self.x16 = torch.zeros(B, H, **a)
        self.yqkv = torch.zeros(B, (NH + 2 * NKV) * HD, **a)
        self.qr, self.ao = torch.zeros(B, NH * HD, **a), torch.zeros(B, NH * HD, **a)
        self.yo, self.yd = torch.zeros(B, H, **a), torch.zeros(B, H, **a)
        self.ygu, self.act = torch.zeros(B, 2 * I, **a), torch.zeros(B, I, **a)
        self.logits = torch.zeros(B, lm_head.R, dtype=torch.float32, device=dev)
        # caches: keys [layer][seq][kv][position][dim], values dimension-major [layer][seq][kv][dim][position] (what the
        # attention kernel's tensor-core value product reads directly); positions padded to a multiple of 32
        self.cache_len = (cfg.max_len + 31) // 32 * 32
        self.kc = torch.zeros(len(layers), B, NKV, self.cache_len, HD, **a)
        self.vc = torch.zeros(len(layers), B, NKV, HD, self.cache_len, **a)
        self.tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(B, dtype=torch.int32, device=dev)
        # attention slices: about four blocks (of four warps) per SM, at least 128 positions per slice at full length
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        ns = attn_split if attn_split is not None else max(1, (4 * sms) // (NKV * B))
        self.nsplit = max(1, min(ns, max(1, self.cache_len // 128), lib.cbl_attn_decode_max_splits()))
        self.att_ws = torch.zeros(lib.cbl_attn_decode_workspace_bytes(B, NH, self.nsplit), dtype=torch.uint8, device=dev)
        self.biases = []
        for L in layers:
            bs = [L.get("bq"), L.get("bk"), L.get("bv")]
            if all(b is None for b in bs):
                self.biases.append(None)
            else:
                sizes = (NH * HD, NKV * HD, NKV * HD)
                self.biases.append(torch.cat([b.to(**a) if b is not None else torch.zeros(n, **a) for b, n in zip(bs, sizes)]))
        self.stages = []
        for L in layers:
            self.stages.append({"qkv": _Stage([L["q"], L["k"], L["v"]], self.yqkv), "o": _Stage([L["o"]], self.yo),
                                "gu": _Stage([L["gate"], L["up"]], self.ygu), "down": _Stage([L["down"]], self.yd)})
        # prompts: q|k|v and gate|up as stacked two-phase GEMMs (decode once, one launch over the stacked rows)
        self.stacks = [{"qkv": DenseStack([_lin(L[n]).dm for n in ("q", "k", "v")]), "gu": DenseStack([_lin(L[n]).dm for n in ("gate", "up")])}
                       for L in layers]
        self.graph = None
        self.only_linears = False
        # one token, one column order everywhere: the operator that follows a product runs on its fp32 sums (one small kernel)
        self.fused = B == 1 and all(st.group is not None for S in self.stages for st in S.values()) and H <= lib.cbl_gemv_l8_add_norm_max_rows()

    # -- operators (thin wrappers over the C ABI; all on the current stream)
    def _embed(self, tok, rows: int, h) -> None:
        if isinstance(self.embed, Q4Embed):
            _lib.check("cbl_embed_rows_q4", lib.cbl_embed_rows_q4(self.embed.q.data_ptr(), self.embed.sc.data_ptr(), self.vocab_rows, self.cfg.hidden,
                                                                  tok.data_ptr(), rows, h.data_ptr(), _stream()))
        else:
            _lib.check("cbl_embed_rows", lib.cbl_embed_rows(self.embed.data_ptr(), _dt(self.dtype), self.vocab_rows, self.cfg.hidden, tok.data_ptr(),
                                                            rows, h.data_ptr(), _stream()))

    def _addnorm(self, h, add, w, x, rows: int) -> None:
        _lib.check("cbl_add_rmsnorm", lib.cbl_add_rmsnorm(h.data_ptr(), None if add is None else add.data_ptr(),
                                                          0 if add is None else add.stride(0), w.data_ptr(), _dt(self.dtype),
                                                          self.cfg.eps, rows, self.cfg.hidden, x.data_ptr(), _stream()))

    def _rope(self, yqkv, bias, pos, pos0: int, seq0: int, rows: int, qr, kc, vc) -> None:
        c = self.cfg
        _lib.check("cbl_rope_kv", lib.cbl_rope_kv(yqkv.data_ptr(), _dt(self.dtype), yqkv.stride(0), None if bias is None else bias.data_ptr(),
                                                  None if pos is None else pos.data_ptr(), pos0, seq0, rows, c.n_heads, c.n_kv, c.head_dim,
                                                  c.rope_theta, self.cache_len, qr.data_ptr(), kc.data_ptr(), vc.data_ptr(), _stream()))

    def _silu(self, ygu, act, rows: int) -> None:
        _lib.check("cbl_silu_mul", lib.cbl_silu_mul(ygu.data_ptr(), _dt(self.dtype), ygu.stride(0), rows, self.cfg.inter, act.data_ptr(),
                                                    _stream()))

    def step(self) -> None:
        """One greedy decode step of all B sequences (graph-capturable)."""
        c, B, dtc = self.cfg, self.B, _dt(self.dtype)
        with torch.cuda.device(self.dev):
            if self.only_linears:          # product-only timing: the same linears in the same order, nothing else
                for S in self.stages:
                    S["qkv"].run(self.x16)
                    S["o"].run(self.ao)
                    S["gu"].run(self.x16)
                    S["down"].run(self.act)
                return
            s = _stream()
            self._embed(self.tok, B, self.h)
            if self.fused:
                self._step_fused(s)
                return
            add = None
            for li, (L, S) in enumerate(zip(self.layers, self.stages)):
                self._addnorm(self.h, add, L["ln1"], self.x16, B)
                S["qkv"].run(self.x16)
                self._rope(self.yqkv, self.biases[li], self.pos, 0, 0, B, self.qr, self.kc[li], self.vc[li])
                _lib.check("cbl_attn_decode", lib.cbl_attn_decode(self.qr.data_ptr(), self.kc[li].data_ptr(), self.vc[li].data_ptr(),
                                                                  self.pos.data_ptr(), dtc, B, c.n_heads, c.n_kv, c.head_dim, self.cache_len,
                                                                  c.head_dim ** -0.5, self.ao.data_ptr(), self.att_ws.data_ptr(), self.nsplit, s))
                S["o"].run(self.ao)
                self._addnorm(self.h, self.yo, L["ln2"], self.x16, B)
                S["gu"].run(self.x16)
                self._silu(self.ygu, self.act, B)
                S["down"].run(self.act)
                add = self.yd
            self._addnorm(self.h, add, self.final_norm, self.x16, B)
            self.lm_head.run(self.x16, self.logits)
            _lib.check("cbl_argmax", lib.cbl_argmax(self.logits.data_ptr(), _dt(self.logits.dtype), self.logits.stride(0), B, self.logits.shape[1],
                                                    self.tok.data_ptr(), self.pos.data_ptr(), s))

    def _pieces(self, li: int, stack: str, names, x, y) -> None:
        """Prompt tokens through stacked linears: one stacked two-phase GEMM for long prompts (or several column
        orders), else piece by piece into column slices of y."""
        L = self.layers[li]
        if x.shape[0] >= DENSE_MIN_TOKENS or (x.shape[0] > 64 and any(_lin(L[n]).dm.M > 1 for n in names)):
            self.stacks[li][stack].gemm(x, y)
            return
        o = 0
        for n in names:
            l = _lin(L[n])
            l.forward_into(x, y[:, o:o + l.R])
            o += l.R

    def _step_fused(self, s: int) -> None:
        """Batch-1 layers, each product followed by its step operator on the fp32 sums: q|k|v + rotary + cache
        write, attention, o + add + norm, gate|up + silu * up, down + add + norm (of the next layer)."""
        from .kernels import l8_workspace
        c, dtc = self.cfg, _dt(self.dtype)
        ws = l8_workspace(self.dev, 0, max(st.group.ws_bytes for S in self.stages for st in S.values())).data_ptr()
        x, act, ao, h = self.x16.data_ptr(), self.act.data_ptr(), self.ao.data_ptr(), self.h.data_ptr()
        self._addnorm(self.h, None, self.layers[0]["ln1"], self.x16, 1)
        n = len(self.layers)
        for li, (L, S) in enumerate(zip(self.layers, self.stages)):
            bias = self.biases[li]
            kc, vc = self.kc[li], self.vc[li]
            _lib.check("cbl_gemv_l8_rope_kv", lib.cbl_gemv_l8_rope_kv(S["qkv"].group._structs, x, dtc, None if bias is None else bias.data_ptr(),
                                                                      self.pos.data_ptr(), c.n_heads, c.n_kv, c.head_dim, c.rope_theta, self.cache_len,
                                                                      self.qr.data_ptr(), kc.data_ptr(), vc.data_ptr(), dtc, ws, s))
            _lib.check("cbl_attn_decode", lib.cbl_attn_decode(self.qr.data_ptr(), kc.data_ptr(), vc.data_ptr(), self.pos.data_ptr(), dtc, 1,
                                                              c.n_heads, c.n_kv, c.head_dim, self.cache_len, c.head_dim ** -0.5, ao,
                                                              self.att_ws.data_ptr(), self.nsplit, s))
            _lib.check("cbl_gemv_l8_add_norm", lib.cbl_gemv_l8_add_norm(S["o"].group._structs, ao, dtc, h, L["ln2"].data_ptr(), c.eps, x, None, dtc, ws, s))
            _lib.check("cbl_gemv_l8_silu_mul", lib.cbl_gemv_l8_silu_mul(S["gu"].group._structs, x, dtc, act, None, None, dtc, ws, s))
            w_next = self.layers[li + 1]["ln1"] if li + 1 < n else self.final_norm
            _lib.check("cbl_gemv_l8_add_norm", lib.cbl_gemv_l8_add_norm(S["down"].group._structs, act, dtc, h, w_next.data_ptr(), c.eps, x, None, dtc, ws, s))
        self.lm_head.run(self.x16, self.logits)
        _lib.check("cbl_argmax", lib.cbl_argmax(self.logits.data_ptr(), _dt(self.logits.dtype), self.logits.stride(0), 1, self.logits.shape[1],
                                                self.tok.data_ptr(), self.pos.data_ptr(), s))

    @torch.no_grad()
    def prefill(self, ids, seq: int = 0) -> torch.Tensor:
        """Run a whole prompt of sequence `seq` from position 0: fills its cache, leaves pos[seq] = len(ids) and
        tok[seq] = the greedy next token; returns the last position's logits [vocab] (fp32)."""
        c = self.cfg
        ids = torch.as_tensor(ids, dtype=torch.int64, device=self.dev).reshape(-1)
        T = ids.numel()
        if not 1 <= T <= c.max_len:
            raise ValueError(f"prompt of {T} tokens outside 1..max_len {c.max_len}")
        if T > 65535:
            raise ValueError("prompts are prefilled in one pass of at most 65535 tokens")
        H, NH, NKV, HD, I = c.hidden, c.n_heads, c.n_kv, c.head_dim, c.inter
        a = dict(dtype=self.dtype, device=self.dev)
        with torch.cuda.device(self.dev):
            h = torch.empty(T, H, dtype=torch.float32, device=self.dev)
            x = torch.empty(T, H, **a)
            yqkv, qr = torch.empty(T, (NH + 2 * NKV) * HD, **a), torch.empty(T, NH * HD, **a)
            yo, ygu, act, yd = torch.empty(T, H, **a), torch.empty(T, 2 * I, **a), torch.empty(T, I, **a), torch.empty(T, H, **a)
            self._embed(ids, T, h)
            add = None
            for li, L in enumerate(self.layers):
                self._addnorm(h, add, L["ln1"], x, T)
                self._pieces(li, "qkv", ("q", "k", "v"), x, yqkv)
                kc, vc = self.kc[li], self.vc[li]
                self._rope(yqkv, self.biases[li], None, 0, seq, T, qr, kc, vc)
                q4 = qr.view(T, NH, HD).transpose(0, 1)[None]
                v4 = yqkv[:, (NH + NKV) * HD:].view(T, NKV, HD).transpose(0, 1)[None]         # the values as projected (+ bias below)
                if self.biases[li] is not None:
                    v4 = (v4 + self.biases[li][(NH + NKV) * HD:].view(1, NKV, 1, HD)).to(self.dtype)
                ao = torch.nn.functional.scaled_dot_product_attention(q4, kc[seq, :, :T][None], v4, is_causal=True, enable_gqa=True)
                ao = ao[0].transpose(0, 1).reshape(T, NH * HD)
                _lin(L["o"]).forward_into(ao, yo)
                self._addnorm(h, yo, L["ln2"], x, T)
                self._pieces(li, "gu", ("gate", "up"), x, ygu)
                self._silu(ygu, act, T)
                _lin(L["down"]).forward_into(act, yd)
                add = yd
            hl, xl = h[T - 1:T].clone(), torch.empty(1, H, **a)
            self._addnorm(hl, yd[T - 1:T], self.final_norm, xl, 1)
            lg = self.logits[seq:seq + 1]
            self.lm_head.run(xl, lg)
            _lib.check("cbl_argmax", lib.cbl_argmax(lg.data_ptr(), _dt(lg.dtype), lg.stride(0), 1, lg.shape[1], self.tok[seq:].data_ptr(), None,
                                                    _stream()))
            self.pos[seq] = T
        return lg[0].clone()

    def reset(self, tok=0) -> None:
        if isinstance(tok, int):
            self.tok.fill_(tok)
        else:
            self.tok.copy_(torch.as_tensor(tok, dtype=torch.int64))
        self.pos.zero_()

    def capture(self):
        """Capture one step as a CUDA graph (two eager steps first: they advance the state, reset afterwards)."""
        st = torch.cuda.Stream(device=self.dev)
        st.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(st):
            for _ in range(2):
                self.step()
        torch.cuda.current_stream(self.dev).wait_stream(st)
        torch.cuda.synchronize(self.dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=st):      # the warm-up stream: its work spaces exist already
            self.step()
        return self.graph

    def check(self) -> None:
        """Synchronises; raises if a bounded device-side wait of a prompt product expired during the calls so far."""
        torch.cuda.synchronize(self.dev)
        DenseStack.status(self.dev)

    @torch.no_grad()
    def generate(self, n: int, tok=0) -> list:
        """Greedy-decode n tokens from `tok` at position 0 (eager steps; for checks). B = 1: a list of ints,
        else a list of B lists."""
        if n > self.cfg.max_len:
            raise ValueError(f"{n} steps from position 0 would run past max_len {self.cfg.max_len}")
        self.reset(tok)
        out = []
        for _ in range(n):
            self.step()
            out.append(self.tok.tolist())
        return [o[0] for o in out] if self.B == 1 else [list(s) for s in zip(*out)]

    @torch.no_grad()
    def time_tokens(self, n: int = 128, reps: int = 3, start: int = 0) -> float:
        """Seconds per step, averaged over n graph replays from position `start` (median of reps). The cache
        below `start` is used as it is (decode speed does not depend on its values)."""
        assert start + n <= self.cfg.max_len
        if self.graph is None:
            self.capture()
        ts = []
        for _ in range(reps):
            self.reset()
            self.pos.fill_(start)
            torch.cuda.synchronize(self.dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                self.graph.replay()
            b.record()
            torch.cuda.synchronize(self.dev)
            ts.append(a.elapsed_time(b) / 1e3 / n)
        return sorted(ts)[len(ts) // 2]

    def weight_bytes(self) -> int:
        """Stored bytes a step reads: the packed block linears (tags, books, scales) and the head."""
        return sum(_lin(L[n]).stored_bytes() for L in self.layers for n in NAMES) + self.lm_head.nbytes()


class Qwen2BatchEngine(DecodeEngine):
    """B sequences per step on the weights of a batch-1 engine (its own caches, positions and buffers)."""

    def __init__(self, eng: DecodeEngine, B: int, *, nsplit: int | None = None, **_ignored):
        super().__init__(eng.cfg, eng.embed, eng.layers, eng.final_norm, eng.lm_head, dev=eng.dev, B=B, attn_split=nsplit)
        self.eng = eng


def random_engine(cfg: Cfg, *, seed: int = 0, dev="cuda", dtype=torch.bfloat16, B: int = 1, books: int = 1, M: int = 1,
                  bias: bool = True, head: str = "16", embed: str = "16") -> DecodeEngine:
    """A random-init model of the given architecture with every block linear in the packed format (d = 8,
    12-bit tags, one 4096-entry book per matrix; `books` = 2 adds a second summed book, M > 1 seeded column
    orders). Stand-in for a real checkpoint: tags uniform, books ~N(0, 1), row scales ~0.02 / sqrt(books),
    embedding and head ~N(0, 0.02), norm weights 1 +- 0.1, q/k/v biases ~N(0, 0.1). head = "16" (the model's 16-bit
    type) or "q8" (the reference's 8-bit block-32 head), embed = "16" or "q4" (its 4-bit block-32 embedding)."""
    dev = torch.device(dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    H, NH, NKV, HD, I = cfg.hidden, cfg.n_heads, cfg.n_kv, cfg.head_dim, cfg.inter

    def lin(R, C):
        W = (C // 8 * 12 + 31) // 32
        words = torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device=dev, generator=g)
        table = torch.randn(4096, 8, device=dev, generator=g).half()
        rs = ((torch.rand(R, device=dev, generator=g) * 0.5 + 0.75) / math.sqrt(C * books)).half()
        kw = {}
        if books == 2:
            kw = dict(words2=torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device=dev, generator=g),
                      table2=torch.randn(4096, 8, device=dev, generator=g).half())
        if M > 1:
            from .packed import seeded_perms
            perms = seeded_perms(C, M, torch.Generator().manual_seed(seed + R + C)).to(dev)
            mask = torch.randint(0, M, (R,), dtype=torch.int32, device=dev, generator=g)
        else:
            perms, mask = torch.arange(C, device=dev)[None], None
        return PackedLinear(words, table, rs, None, mask, perms, 4096, 8, **kw)

    def vec(n, s, base=0.0):
        return (torch.randn(n, device=dev, generator=g) * s + base).to(dtype)

    layers = []
    for _ in range(cfg.layers):
        L = {"ln1": vec(H, 0.1, 1.0), "ln2": vec(H, 0.1, 1.0), "q": lin(NH * HD, H), "k": lin(NKV * HD, H), "v": lin(NKV * HD, H),
             "o": lin(H, NH * HD), "gate": lin(I, H), "up": lin(I, H), "down": lin(H, I)}
        if bias:
            L.update(bq=vec(NH * HD, 0.1), bk=vec(NKV * HD, 0.1), bv=vec(NKV * HD, 0.1))
        layers.append(L)
    we = (torch.randn(cfg.vocab, H, device=dev, generator=g) * 0.02).to(dtype)
    wh = (torch.randn(cfg.vocab, H, device=dev, generator=g) * 0.02).to(dtype)
    if head not in ("16", "q8") or embed not in ("16", "q4"):
        raise ValueError("head is '16' or 'q8', embed is '16' or 'q4'")
    emb = Q4Embed.from_weight(we, dev, dtype) if embed == "q4" else we
    hd = Q8Head.from_weight(wh, dev) if head == "q8" else DenseHead(wh)
    return DecodeEngine(cfg, emb, layers, vec(H, 0.1, 1.0), hd, dev=dev, B=B)


# ------------------------------------------------------------------------------------------- runtime helpers
@torch.no_grad()
def start(eng: DecodeEngine, prompt, seq: int = 0) -> torch.Tensor:
    """Fresh context for sequence `seq`: run `prompt` from position 0 (batched prefill). Returns the last
    position's fp32 logits; afterwards tok[seq] = greedy next token, pos[seq] = len(prompt)."""
    return eng.prefill(prompt, seq)


def _sample(logits: torch.Tensor, temperature: float, top_p: float, top_k: int, gen) -> int:
    """One token id drawn from softmax(logits / temperature) restricted to the top_k largest logits and to the nucleus
    whose probability first reaches top_p (the usual temperature / top-k / top-p sampler; the same choices as the
    reference's, shapequant/runtime.py:203-213)."""
    scaled = logits.to(torch.float32) / max(temperature, 1e-6)
    order = torch.argsort(scaled, descending=True)
    keep = torch.ones(order.numel(), dtype=torch.bool, device=scaled.device)     # in sorted order
    if 0 < top_k < order.numel():
        keep[top_k:] = False
    if top_p < 1.0:
        probs = torch.softmax(scaled[order].masked_fill(~keep, float("-inf")), 0)
        before = probs.cumsum(0) - probs                    # mass strictly ahead of each candidate
        keep &= before <= top_p
    probs = torch.softmax(scaled[order].masked_fill(~keep, float("-inf")), 0)
    return int(order[torch.multinomial(probs, 1, generator=gen)])


@torch.no_grad()
def generate(eng: DecodeEngine, prompt, n: int, graph: bool = True, *, temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0,
             seed: int | None = None, stop_ids=()) -> list:
    """Continue `prompt` by up to n tokens on a batch-1 engine. temperature 0: greedy (the step's own argmax),
    else sampled with top-k / top-p. Stops after a token in stop_ids (included)."""
    if eng.B != 1:
        raise ValueError("generate() drives a batch-1 engine")
    if len(prompt) + n > eng.cfg.max_len:
        raise ValueError("prompt + n exceeds max_len")
    if graph and eng.graph is None:
        eng.capture()
    gen = None
    if temperature > 0:
        gen = torch.Generator(device=eng.dev)
        gen.manual_seed(seed if seed is not None else torch.seed() % (2 ** 63))
    stop_ids = set(stop_ids or ())
    eng.reset(0)
    logits = start(eng, prompt)
    out = []
    while True:
        if temperature > 0:
            t = _sample(logits, temperature, top_p, top_k, gen)
            eng.tok.fill_(t)
        else:
            t = int(eng.tok[0])
        out.append(t)
        if len(out) >= n or t in stop_ids:
            break
        if graph:
            eng.graph.replay()
        else:
            eng.step()
        logits = eng.logits[0]
    return out


@torch.no_grad()
def bench(eng: DecodeEngine, pp: int = 512, tg: int = 128, reps: int = 3) -> dict:
    """Prompt tokens/s of one prefill of `pp` tokens and generated tokens/s over `tg` graph-replayed steps
    that follow it (all B sequences; median of reps)."""
    res = {}
    if pp:
        ids = torch.randint(0, eng.cfg.vocab, (pp,), device=eng.dev)
        ts = []
        for _ in range(reps + 1):
            torch.cuda.synchronize(eng.dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.prefill(ids, 0)
            b.record()
            torch.cuda.synchronize(eng.dev)
            ts.append(a.elapsed_time(b) / 1e3)
        ts = sorted(ts[1:])
        res.update(pp=pp, pp_tok_s=pp / ts[len(ts) // 2])
    if tg:
        res.update(tg=tg, tg_tok_s=eng.B / eng.time_tokens(tg, reps, start=pp))
    return res
