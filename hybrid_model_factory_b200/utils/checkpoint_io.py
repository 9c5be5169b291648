"""HF-style checkpoint I/O: ``config.json`` + safetensors shards (``model-0000i-of-0000n.safetensors``
with ``model.safetensors.index.json``) of at most ``max_shard_size``.

Tensor names are the HF names of the reference project's checkpoints.  Two conversions are
applied at the boundary so that in-memory modules can use fused layouts:
  * MoE experts: stacked ``experts.gate_up_proj [E, 2F, D]`` / ``experts.down_proj [E, D, F]``  <->
    ``experts.{e}.gate_proj|up_proj|down_proj.weight``;
  * nothing else is renamed (``A_log``, ``dt_bias``, conv weights ``[C, 1, K]`` are stored as is).
Reference: ``train/trainer_utils.py:80-122`` (``SaveShardMixin``), ``priming/hybridize_model.py:216-332``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterator, List, Optional, Tuple

import torch

_UNITS = {"KB": 10 ** 3, "MB": 10 ** 6, "GB": 10 ** 9, "KIB": 2 ** 10, "MIB": 2 ** 20, "GIB": 2 ** 30}


def parse_size(size) -> int:
    if isinstance(size, int):
        return size
    m = re.fullmatch(r"\s*([\d.]+)\s*([A-Za-z]+)\s*", str(size))
    if not m:
        raise ValueError(f"cannot parse size '{size}'")
    return int(float(m.group(1)) * _UNITS[m.group(2).upper()])


# -- expert name conversion --------------------------------------------------------------------
_EXPERT_RE = re.compile(r"^(.*\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def to_hf_names(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for name, t in state.items():
        if name.endswith(".experts.gate_up_proj"):
            base = name[: -len(".gate_up_proj")]
            F = t.shape[1] // 2
            for e in range(t.shape[0]):
                out[f"{base}.{e}.gate_proj.weight"] = t[e, :F].contiguous()
                out[f"{base}.{e}.up_proj.weight"] = t[e, F:].contiguous()
        elif name.endswith(".experts.down_proj"):
            base = name[: -len(".down_proj")]
            for e in range(t.shape[0]):
                out[f"{base}.{e}.down_proj.weight"] = t[e].contiguous()
        else:
            out[name] = t
    return out


def from_hf_names(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    groups: Dict[str, Dict[Tuple[int, str], torch.Tensor]] = {}
    for name, t in state.items():
        m = _EXPERT_RE.match(name)
        if m:
            groups.setdefault(m.group(1), {})[(int(m.group(2)), m.group(3))] = t
        else:
            out[name] = t
    for base, parts in groups.items():
        E = max(e for e, _ in parts) + 1
        if all((e, "gate_proj") in parts and (e, "up_proj") in parts for e in range(E)):
            out[f"{base}.gate_up_proj"] = torch.stack(
                [torch.cat([parts[(e, "gate_proj")], parts[(e, "up_proj")]], dim=0) for e in range(E)])
        if all((e, "down_proj") in parts for e in range(E)):
            out[f"{base}.down_proj"] = torch.stack([parts[(e, "down_proj")] for e in range(E)])
    return out


# -- save ----------------------------------------------------------------------------------------
def shard_state_dict(state: Dict[str, torch.Tensor], max_shard_size) -> List[Dict[str, torch.Tensor]]:
    limit = parse_size(max_shard_size)
    shards, cur, cur_size = [], {}, 0
    for name, t in state.items():
        n = t.numel() * t.element_size()
        if cur and cur_size + n > limit:
            shards.append(cur)
            cur, cur_size = {}, 0
        cur[name] = t
        cur_size += n
    if cur:
        shards.append(cur)
    return shards


def save_state_dict(state: Dict[str, torch.Tensor], path: str, max_shard_size="5GB") -> List[str]:
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    # tied tensors are written once
    seen, dedup = {}, {}
    for name, t in state.items():
        key = (t.data_ptr(), t.numel(), t.dtype)
        if key in seen and t.numel() > 0:
            continue
        seen[key] = name
        dedup[name] = t.detach().to("cpu").contiguous()
    shards = shard_state_dict(dedup, max_shard_size)
    files = []
    if len(shards) == 1:
        fn = "model.safetensors"
        save_file(shards[0], os.path.join(path, fn), metadata={"format": "pt"})
        return [fn]
    index = {"metadata": {"total_size": sum(t.numel() * t.element_size() for t in dedup.values())}, "weight_map": {}}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
        files.append(fn)
        for name in sh:
            index["weight_map"][name] = fn
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=2)
    return files


def save_pretrained(model: torch.nn.Module, path: str, max_shard_size="5GB", dtype: Optional[torch.dtype] = None) -> None:
    os.makedirs(path, exist_ok=True)
    state = {k: (v.to(dtype) if dtype is not None and v.is_floating_point() else v) for k, v in model.state_dict().items()}
    if getattr(getattr(model, "config", None), "tie_word_embeddings", False):
        state.pop("lm_head.weight", None)
    save_state_dict(to_hf_names(state), path, max_shard_size)
    if hasattr(model, "config") and hasattr(model.config, "save_pretrained"):
        model.config.save_pretrained(path)


# -- load ----------------------------------------------------------------------------------------
def checkpoint_files(path: str) -> List[str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return sorted(set(json.load(f)["weight_map"].values()))
    if os.path.exists(os.path.join(path, "model.safetensors")):
        return ["model.safetensors"]
    return sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))


def iter_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    from safetensors import safe_open
    for fn in checkpoint_files(path):
        with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
            for name in f.keys():
                yield name, f.get_tensor(name)


def load_state_dict(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of a checkpoint directory under this package's names; matrices stored as quantised integers (this
    package's group-wise format of ``hmf export --quantize int8|int4``, or the GPTQ / AWQ layouts) are expanded to
    bf16 on the way in."""
    state = dict(iter_tensors(path))
    if any(k.endswith(".qzeros") for k in state):
        from .quant_loaders import expand_quantized_state
        quant_cfg = None
        cfg_path = os.path.join(path, "config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                quant_cfg = json.load(f).get("quantization_config")
        state = expand_quantized_state(state, quant_cfg)
    if any(k.endswith(".qweight") for k in state):
        from .export import dequantize_state
        state = dequantize_state(state)
    return from_hf_names(state)


def load_state_dict_into(model: torch.nn.Module, path: str, strict: bool = False) -> Tuple[List[str], List[str]]:
    """Copies checkpoint tensors into existing parameters *in place* (views into flat optimizer
    buffers stay valid).  Returns ``(missing, unexpected)`` key lists."""
    state = load_state_dict(path)
    own = dict(model.state_dict(keep_vars=True))
    missing = [k for k in own if k not in state]
    unexpected = [k for k in state if k not in own]
    if getattr(getattr(model, "config", None), "tie_word_embeddings", False) and "lm_head.weight" in missing:
        missing.remove("lm_head.weight")
    with torch.no_grad():
        for k, t in state.items():
            if k in own:
                if own[k].shape != t.shape:
                    raise ValueError(f"shape mismatch for {k}: checkpoint {tuple(t.shape)} vs model {tuple(own[k].shape)}")
                own[k].data.copy_(t.to(own[k].dtype))
    if strict and (missing or unexpected):
        raise KeyError(f"missing={missing[:8]} unexpected={unexpected[:8]}")
    return missing, unexpected


def from_pretrained(path: str, dtype: Optional[torch.dtype] = None, device=None, allow_missing: bool = False,
                    init: str = "default", **config_overrides):
    """Builds the model named by ``config.json`` and loads its weights.

    A parameter of the model that the checkpoint does not hold raises ``KeyError`` unless ``allow_missing`` is set
    (a converted or adapter-wrapped checkpoint whose names do not match would otherwise leave random weights in
    place without a sound); checkpoint tensors that the model does not own are reported with a warning.  Both lists
    are kept in ``model._load_report``.

    ``init="meta"`` builds the module tree without storage, allocates it directly in the target dtype on the target
    device and fills it from the checkpoint: no random initialisation and no fp32 copy in host memory (an 8B model
    otherwise passes through 32 GB of it).  Every parameter must then come from the checkpoint."""
    from ..models.configuration import HybridConfig
    from ..models.modeling_hybrid import build_model
    cfg = HybridConfig.from_pretrained(path, **config_overrides)
    dt = dtype or getattr(torch, str(cfg.torch_dtype).replace("torch.", ""), torch.bfloat16)
    if init == "meta":
        with torch.device("meta"):
            model = build_model(cfg).to(dt)
        model = model.to_empty(device=device if device is not None else "cpu")
        if getattr(cfg, "tie_word_embeddings", False) and hasattr(model, "lm_head"):
            model.lm_head.weight = model.get_input_embeddings().weight       # allocation un-ties shared parameters
        allow_missing = False
    elif init == "default":
        model = build_model(cfg).to(dt)
        if device is not None:
            model = model.to(device)
    else:
        raise ValueError(f"init must be 'default' or 'meta', not {init!r}")
    missing, unexpected = load_state_dict_into(model, path)
    model._load_report = {"missing": missing, "unexpected": unexpected}
    if missing and not allow_missing:
        raise KeyError(f"{path}: {len(missing)} model parameters are not in the checkpoint (first: {missing[:6]}); "
                       f"pass allow_missing=True to keep their initial values")
    if unexpected:
        import warnings
        warnings.warn(f"{path}: {len(unexpected)} checkpoint tensors match no model parameter "
                      f"(first: {unexpected[:6]})", stacklevel=2)
    return model
