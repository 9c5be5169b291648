"""Model side of the second-generation stack: loads the checkpoint and tokenizer, then lets three plugin families shape
the model: where its storage first lives (``InitPlugin``), which parameters train (``PeftPlugin``) and which kernels
its layers run on (``KernelPlugin``).

``ModelEngine(model_path, init_config={"name": "init_on_meta"}, peft_config={"name": "lora", "rank": 8},
kernel_config={"name": "auto", "include_kernels": ["fp8_linear"]})``.

* init: ``init_on_default`` (build on the host, move), ``init_on_meta`` (no storage until the checkpoint fills it),
  ``init_on_rank0`` (rank 0 reads the files, the other ranks allocate and receive a broadcast: one reader per node
  instead of one per GPU);
* peft: ``lora`` (``rank``, ``alpha``, ``target``, ``use_rslora``, ``use_dora``, ``pissa_init``, ``quantization_bit``),
  ``freeze`` (``trainable_layers``);
* kernels: ``auto`` applies every registered kernel switch or those named in ``include_kernels``.  The tcgen05 GEMM
  behind every ``nn.Linear`` is always on (``models.build_model``); ``fp8_linear`` moves the projections to the
  row-wise scaled float8 GEMM.

Reference: ``v1/core/model_engine.py:42-160``, ``v1/plugins/model_plugins/{initialization,peft}.py``,
``v1/plugins/model_plugins/kernels/{interface,registry}.py`` (whose registered kernels are NPU ones)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn

from .plugin import Plugin


class InitPlugin(Plugin):
    """``InitPlugin(name)(path, dtype, device) -> model``."""


class PeftPlugin(Plugin):
    """``PeftPlugin(name)(model, config: dict, is_train) -> model``."""


class KernelPlugin(Plugin):
    """``KernelPlugin(name)(model, include_kernels=None) -> model``."""


def _dist():
    import torch.distributed as dist
    return dist if dist.is_available() and dist.is_initialized() else None


@InitPlugin("init_on_default").register(replace=True)
def _init_default(path: str, dtype, device):
    from ..utils import checkpoint_io
    return checkpoint_io.from_pretrained(path, dtype=dtype, device=device)


@InitPlugin("init_on_meta").register(replace=True)
def _init_meta(path: str, dtype, device):
    from ..utils import checkpoint_io
    return checkpoint_io.from_pretrained(path, dtype=dtype, device=device, init="meta")


@InitPlugin("init_on_rank0").register(replace=True)
def _init_rank0(path: str, dtype, device):
    from ..models.configuration import HybridConfig
    from ..models.modeling_hybrid import build_model
    from ..utils import checkpoint_io
    dist = _dist()
    if dist is None or dist.get_world_size() == 1:
        return _init_meta(path, dtype, device)
    if dist.get_rank() == 0:
        model = checkpoint_io.from_pretrained(path, dtype=dtype, device=device, init="meta")
    else:
        cfg = HybridConfig.from_pretrained(path)
        with torch.device("meta"):
            model = build_model(cfg).to(dtype or torch.bfloat16)
        model = model.to_empty(device=device if device is not None else "cpu")
        if getattr(cfg, "tie_word_embeddings", False):
            model.lm_head.weight = model.get_input_embeddings().weight
    for _, t in sorted(model.state_dict(keep_vars=True).items()):        # same order on every rank
        dist.broadcast(t.data, src=0)
    return model


@PeftPlugin("lora").register(replace=True)
def _peft_lora(model: nn.Module, config: dict, is_train: bool = True):
    from ..train.adapters import apply_lora
    apply_lora(model, rank=int(config.get("rank", config.get("r", 8))), alpha=config.get("alpha", config.get("lora_alpha")),
               target=config.get("target", config.get("target_modules", "all")),
               use_rslora=bool(config.get("use_rslora", False)), use_dora=bool(config.get("use_dora", False)),
               pissa_init=bool(config.get("pissa_init", False)), pissa_iter=int(config.get("pissa_iter", 0)))
    if config.get("quantization_bit"):
        from ..train.qlora import quantize_adapter_bases
        quantize_adapter_bases(model, int(config["quantization_bit"]), config.get("quantization_type", "nf4"))
    if not is_train:
        for p in model.parameters():
            p.requires_grad_(False)
    return model


@PeftPlugin("freeze").register(replace=True)
def _peft_freeze(model: nn.Module, config: dict, is_train: bool = True):
    from ..train.adapters import freeze_all_but_last
    freeze_all_but_last(model, int(config.get("trainable_layers", config.get("freeze_trainable_layers", 2))))
    return model


KERNELS: Dict[str, Callable[[nn.Module], int]] = {}


def register_kernel(name: str):
    """Registers ``fn(model) -> number of modules switched`` under ``name`` for ``KernelPlugin("auto")``."""
    def deco(fn):
        KERNELS[name] = fn
        return fn
    return deco


@register_kernel("own_linear")
def _kernel_linear(model: nn.Module) -> int:
    from ..ops.gemm import use_own_linear
    return int(use_own_linear(model) or 0)


@register_kernel("fp8_linear")
def _kernel_fp8(model: nn.Module) -> int:
    from ..ops.fp8 import use_fp8_linear
    return int(use_fp8_linear(model) or 0)


@KernelPlugin("auto").register(replace=True)
def _kernels_auto(model: nn.Module, include_kernels: Optional[List[str]] = None):
    names = list(include_kernels) if include_kernels else ["own_linear"]
    unknown = [n for n in names if n not in KERNELS]
    if unknown:
        raise ValueError(f"unknown kernels {unknown}; registered: {sorted(KERNELS)}")
    model.applied_kernels = {n: KERNELS[n](model) for n in names}
    return model


class ModelEngine:
    """``.model``, ``.tokenizer`` and ``.renderer`` of a run."""

    def __init__(self, model_path: str, *, template: Optional[str] = None, cutoff_len: int = 2048,
                 dtype: Optional[torch.dtype] = None, device=None, is_train: bool = True,
                 init_config: Optional[dict] = None, peft_config: Optional[dict] = None,
                 kernel_config: Optional[dict] = None):
        from ..data.formats import load_tokenizer
        from .rendering import Renderer
        self.model_path, self.is_train = model_path, is_train
        self.tokenizer = load_tokenizer(model_path)
        self.renderer = Renderer(self.tokenizer, template or "default", cutoff_len)
        init = (init_config or {}).get("name", "init_on_default")
        model = InitPlugin(init)(model_path, dtype, device)
        if peft_config:
            model = PeftPlugin(peft_config["name"])(model, peft_config, is_train)
        if kernel_config:
            model = KernelPlugin(kernel_config.get("name", "auto"))(model,
                                                                     include_kernels=kernel_config.get("include_kernels"))
        self.model = model.train() if is_train else model.eval()

    def trainable_parameters(self) -> int:
        return sum(p.numel() for p in self.model.parameters() if p.requires_grad)
