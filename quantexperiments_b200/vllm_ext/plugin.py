"""vLLM quantization method "shapequant" on the B200 kernels: the block linears of a packed codebook
file run through `torch.ops.shapequant.linear`; everything else is stock vLLM.

Mirrors shapequant/vllm_ext/plugin.py of the reference (ShapeQuantConfig :53-160,
ShapeQuantLinearMethod :191-235, register :363-372) for the linear path, and adds what the reference
refuses (`NotImplementedError("tensor parallelism is not supported")`, :198-199): under tensor
parallelism create_weights() keeps only this rank's rows (column-parallel layers:
`output_partition_sizes`) or chunk range (row-parallel layers: `input_size_per_partition`) of every
piece; vLLM's RowParallelLinear performs the all-reduce after apply(), as for any other method.

The packed lm_head / embedding methods of the reference (`embed_head: "packed"`) are outside this
path: only `embed_head: "bf16"` (stock vLLM layers) is accepted.

Checkpoint layout and `quantization_config` keys are the reference's:
  "quantization_config": {"quant_method": "shapequant", "packed_file": "shapequant.packed", ...}
Keys that tune the reference's launch geometry (layout, large, chunk_mb, xs, warps, tune, compact)
are accepted and ignored."""

from __future__ import annotations

import os
from typing import Any

import torch

from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization import register_quantization_config
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig, QuantizeMethodBase

from .. import tp
from ..linear import PackedLinear
from . import core


def _resolve(file: str) -> str:
    """Where the packed file lives: an existing absolute path as given; else a file of the model vLLM is loading -
    inside its local directory, or fetched from its hub repository at the configured revision."""
    path = os.path.abspath(file) if os.path.isabs(file) else None
    if path and os.path.exists(path):
        return path
    from vllm.config import get_current_vllm_config
    model_cfg = get_current_vllm_config().model_config
    if os.path.isdir(model_cfg.model):
        return os.path.join(model_cfg.model, file)
    from huggingface_hub import hf_hub_download
    return hf_hub_download(repo_id=model_cfg.model, filename=file, revision=getattr(model_cfg, "revision", None))


def _tp() -> tuple[int, int]:
    try:
        from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size
        return get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
    except Exception:
        return 0, 1


@register_quantization_config("shapequant")
class ShapeQuantConfig(QuantizationConfig):
    def __init__(self, packed_file: str, bmax: int = core.BMAX, embed_head: str = "bf16", **ignored):
        super().__init__()
        if embed_head != "bf16":
            raise ValueError(f"embed_head {embed_head!r}: only 'bf16' (stock vLLM embedding and head) is supported")
        self.packed_file = packed_file
        self.bmax = min(int(os.environ.get("SHAPEQUANT_BMAX", bmax)), core.BMAX)
        self.embed_head = embed_head
        self.ignored = dict(ignored)
        self._pf = None

    def __repr__(self) -> str:
        return f"ShapeQuantConfig(packed_file={self.packed_file!r}, bmax={self.bmax}, embed_head={self.embed_head!r})"

    def __getstate__(self):
        # vLLM builds the config in its front-end process and pickles it into the engine process:
        # the open file handle stays behind
        d = dict(self.__dict__)
        d["_pf"] = None
        return d

    @classmethod
    def get_name(cls) -> str:
        return "shapequant"

    @classmethod
    def get_supported_act_dtypes(cls) -> list[torch.dtype]:
        return [torch.bfloat16, torch.float16]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100

    @staticmethod
    def get_config_filenames() -> list[str]:
        return []

    @classmethod
    def from_config(cls, config: dict[str, Any]) -> "ShapeQuantConfig":
        keys = ("layout", "large", "chunk_mb", "xs", "warps", "tune", "compact")
        return cls(packed_file=config["packed_file"], bmax=int(config.get("bmax", core.BMAX)),
                   embed_head=config.get("embed_head", "bf16"), **{k: config[k] for k in keys if k in config})

    @property
    def pf(self):
        if self._pf is None:
            from ..packed import PackedFile
            self._pf = PackedFile(_resolve(self.packed_file))
        return self._pf

    def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> QuantizeMethodBase | None:
        if not isinstance(layer, LinearBase):
            return None
        pieces = core.packed_pieces(prefix, self.pf.meta)
        if pieces is None:
            return UnquantizedLinearMethod()
        return ShapeQuantLinearMethod(self, prefix, pieces)


def build_shards(pf, pieces: list[str], *, input_size_per_partition: int, output_partition_sizes: list[int],
                 input_size: int, output_size: int, rank: int, world: int, device, bmax: int) -> core.PackedShards:
    """This rank's PackedShards for the vLLM layer made of `pieces` (testable without vLLM).
    Column-parallel layers: every piece keeps rows [rank * R/world, (rank+1) * R/world); row-parallel
    layers: every piece keeps the chunk range of `input_size_per_partition` columns."""
    lins = []
    split_in = input_size_per_partition != input_size
    split_out = sum(output_partition_sizes) != output_size
    if split_in and split_out:
        raise ValueError("a layer split along both dimensions is not a tensor-parallel linear")
    for name, part in zip(pieces, output_partition_sizes if len(output_partition_sizes) == len(pieces) else [None] * len(pieces)):
        m = pf.meta[name]
        t = pf.tensors(name)
        perms = pf.perms(name) if m["M"] > 1 else None
        if split_out:
            if m["R"] % world or (part is not None and part != m["R"] // world):
                raise ValueError(f"{name}: {m['R']} rows do not split over {world} ranks as vLLM expects ({part})")
            r0, r1 = tp.row_range(m["R"], rank, world)
            t, m = tp.shard_rows(t, m, r0, r1)
        elif split_in:
            if m["M"] > 1:
                raise ValueError(f"{name}: column orders with a row-parallel split need the full activation vector")
            c0, c1 = tp.col_range(m["C"], m["d"], rank, world)
            if c1 - c0 != input_size_per_partition:
                raise ValueError(f"{name}: chunk range {c1 - c0} != vLLM partition {input_size_per_partition}")
            t, m, _ = tp.shard_cols(t, m, c0, c1)
        p = perms if perms is not None else torch.arange(m["C"])[None]
        lins.append(PackedLinear(t["tags"].to(device), t["table"].to(device), t["row_scale"].to(device),
                                 t["row_book"].to(device) if "row_book" in t else None,
                                 t["row_mask"].to(device) if "row_mask" in t else None, p.to(device), m["K"], m["d"]))
    return core.PackedShards(lins, bmax=bmax)


class ShapeQuantLinearMethod(LinearMethodBase):
    def __init__(self, cfg: ShapeQuantConfig, prefix: str, pieces: list[str]):
        self.cfg, self.prefix, self.pieces = cfg, prefix, pieces

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs):
        rank, world = _tp()
        dev = torch.device("cuda", torch.cuda.current_device())
        ps = build_shards(self.cfg.pf, self.pieces, input_size_per_partition=input_size_per_partition,
                          output_partition_sizes=output_partition_sizes, input_size=input_size, output_size=output_size,
                          rank=rank, world=world, device=dev, bmax=self.cfg.bmax)
        ps.sq_name = self.prefix
        if ps.C != input_size_per_partition or ps.R != sum(output_partition_sizes):
            raise ValueError(f"{self.prefix}: packed pieces are [{ps.R}, {ps.C}], vLLM partition is "
                             f"[{sum(output_partition_sizes)}, {input_size_per_partition}]")
        layer.sq_handle = core.register(ps)
        layer.sq_shards = ps            # keeps the kernels' tensors alive with the module

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        return None

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        y = torch.ops.shapequant.linear(x, layer.sq_handle)
        return y if bias is None else y + bias


def register() -> None:
    """vllm.general_plugins entry point: importing this module registers the config."""
    return None
