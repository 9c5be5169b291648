"""``hmf export CKPT OUT [--dtype bf16|fp16|fp32] [--max-shard-size 5GB] [--merge-lora --lora-alpha A]
[--quantize int8|int4 --group-size G] [--ollama --template NAME]``: re-shard / cast a checkpoint, fold LoRA (DoRA)
adapters into the base weights, store the large matrices as group-wise quantised integers (dequantised again by
``checkpoint_io`` when the checkpoint is loaded), write an Ollama ``Modelfile``.
Reference: ``train/tuner.py:115-200`` (``export_model``)."""
from __future__ import annotations

import argparse
import json
import os
import shutil

import torch

from . import checkpoint_io

DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
          "fp32": torch.float32, "float32": torch.float32}


def merge_lora_state(state: dict, alpha: float = None, use_rslora: bool = False) -> dict:
    """Folds ``<name>.lora_A / lora_B (/ magnitude)`` into ``<name>.base.weight`` and renames it ``<name>.weight``."""
    out, groups = {}, {}
    for k, v in state.items():
        for tail in (".lora_A", ".lora_B", ".magnitude", ".base.weight", ".base.bias"):
            if k.endswith(tail):
                groups.setdefault(k[:-len(tail)], {})[tail] = v
                break
        else:
            out[k] = v
    for name, g in groups.items():
        w = g[".base.weight"].float()
        if ".lora_A" in g:
            rank = g[".lora_A"].shape[0]
            a = float(alpha) if alpha is not None else 2.0 * rank
            scaling = a / (rank ** 0.5 if use_rslora else rank)
            w = w + (g[".lora_B"].float() @ g[".lora_A"].float()) * scaling
        if ".magnitude" in g:
            w = w * (g[".magnitude"].float()[:, None] / w.norm(dim=1, keepdim=True).clamp_min(1e-12))
        out[name + ".weight"] = w.to(g[".base.weight"].dtype)
        if ".base.bias" in g:
            out[name + ".bias"] = g[".base.bias"]
    return out


def quantize_state(state: dict, bits: int = 8, group_size: int = 128, min_numel: int = 1 << 16) -> dict:
    """Symmetric group-wise integer quantisation of every 2-D floating-point matrix with at least ``min_numel``
    elements whose inner size divides into groups: ``<name>`` becomes ``<name>.qweight`` (int8; two 4-bit values per
    byte for ``bits=4``) + ``<name>.qscales`` (fp16, one per group) + ``<name>.qmeta`` (``[bits, group, rows, cols]``)."""
    assert bits in (4, 8)
    qmax = 2 ** (bits - 1) - 1
    out = {}
    for k, v in state.items():
        if not (v.dim() == 2 and v.is_floating_point() and v.numel() >= min_numel and v.shape[1] % group_size == 0
                and "embed" not in k and "lm_head" not in k):
            out[k] = v
            continue
        g = v.float().reshape(v.shape[0], -1, group_size)
        scale = g.abs().amax(-1, keepdim=True).clamp_min(1e-8) / qmax
        q = torch.clamp(torch.round(g / scale), -qmax - 1, qmax).to(torch.int8).reshape(v.shape)
        if bits == 4:
            q = ((q[:, 0::2] & 0xF) | (q[:, 1::2] << 4)).to(torch.int8)
        out[k + ".qweight"], out[k + ".qscales"] = q.contiguous(), scale.squeeze(-1).to(torch.float16)
        out[k + ".qmeta"] = torch.tensor([bits, group_size, v.shape[0], v.shape[1]], dtype=torch.int64)
    return out


def interchange_quantize_state(state: dict, method: str, bits: int = 4, group_size: int = 128,
                               min_numel: int = 1 << 16) -> dict:
    """Round-to-nearest 4-bit weights in the GPTQ or AWQ tensor layout (``<layer>.qweight / .qzeros / .scales``), for
    the ``.weight`` of every 2-D matrix that :func:`quantize_state` would take and whose outputs divide by 8."""
    from .quant_loaders import pack_awq, pack_gptq
    pack = pack_gptq if method == "gptq" else pack_awq
    out = {}
    for k, v in state.items():
        if not (k.endswith(".weight") and v.dim() == 2 and v.is_floating_point() and v.numel() >= min_numel
                and v.shape[1] % group_size == 0 and v.shape[0] % 8 == 0 and "embed" not in k and "lm_head" not in k
                and "norm" not in k):
            out[k] = v
            continue
        for suffix, t in pack(v, bits, group_size).items():
            out[k[:-len("weight")] + suffix] = t.contiguous()
    return out


def dequantize_state(state: dict, dtype: torch.dtype = torch.bfloat16) -> dict:
    """Inverse of :func:`quantize_state` (tensors without the quantised triple pass through)."""
    out = {}
    for k, v in state.items():
        if k.endswith(".qscales") or k.endswith(".qmeta"):
            continue
        if not k.endswith(".qweight"):
            out[k] = v
            continue
        name = k[:-len(".qweight")]
        bits, group, rows, cols = (int(x) for x in state[name + ".qmeta"])
        q = v
        if bits == 4:
            lo = ((q << 4).to(torch.int8) >> 4)             # sign-extend the low nibble
            hi = q >> 4
            q = torch.stack([lo, hi], dim=-1).reshape(rows, cols)
        w = q.float().reshape(rows, -1, group) * state[name + ".qscales"].float()[..., None]
        out[name] = w.reshape(rows, cols).to(dtype)
    return out


def write_ollama_modelfile(dst: str, template_name: str = None) -> str:
    """``Modelfile`` beside the exported weights: chat format and stop strings of the chosen template."""
    from ..data.formats import get_template
    t = get_template(template_name)
    user = t.user_fmt.replace("{content}", "{{ .Prompt }}")
    system = t.system_fmt.replace("{content}", "{{ .System }}")
    lines = ["FROM .", "", 'TEMPLATE """{{ if .System }}' + system + "{{ end }}" + user + '{{ .Response }}"""']
    if t.default_system:
        lines += ["", 'SYSTEM """' + t.default_system + '"""']
    for stop in getattr(t, "stop_words", None) or []:
        lines.append(f'PARAMETER stop "{stop}"')
    path = os.path.join(dst, "Modelfile")
    with open(path, "w", encoding="utf-8") as fh:
        fh.write("\n".join(lines) + "\n")
    return path


def export(src: str, dst: str, dtype: str = None, max_shard_size="5GB", merge_lora: bool = False, lora_alpha=None,
           use_rslora: bool = False, quantize: str = None, group_size: int = 128, ollama: bool = False,
           template: str = None) -> str:
    os.makedirs(dst, exist_ok=True)
    state = checkpoint_io.load_state_dict(src)
    if merge_lora:
        state = merge_lora_state(state, lora_alpha, use_rslora)
    if dtype:
        dt = DTYPES[dtype]
        state = {k: (v.to(dt) if v.is_floating_point() else v) for k, v in state.items()}
    if quantize in ("gptq", "awq"):
        state = interchange_quantize_state(state, quantize, 4, group_size)
    elif quantize:
        state = quantize_state(state, 4 if quantize == "int4" else 8, group_size)
    checkpoint_io.save_state_dict(state, dst, max_shard_size)
    for name in os.listdir(src):
        if name.endswith((".json", ".txt", ".model", ".jinja")) and not name.endswith("index.json"):
            shutil.copy(os.path.join(src, name), os.path.join(dst, name))
    if (dtype or quantize in ("gptq", "awq")) and os.path.exists(os.path.join(dst, "config.json")):
        with open(os.path.join(dst, "config.json")) as f:
            cfg = json.load(f)
        if dtype:
            cfg["torch_dtype"] = str(DTYPES[dtype]).replace("torch.", "")
        if quantize == "gptq":
            cfg["quantization_config"] = {"quant_method": "gptq", "bits": 4, "group_size": group_size,
                                          "desc_act": False, "sym": False, "checkpoint_format": "gptq"}
        elif quantize == "awq":
            cfg["quantization_config"] = {"quant_method": "awq", "bits": 4, "group_size": group_size,
                                          "zero_point": True, "version": "gemm"}
        with open(os.path.join(dst, "config.json"), "w") as f:
            json.dump(cfg, f, indent=2)
    if ollama:
        write_ollama_modelfile(dst, template)
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hmf export")
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--dtype", default=None, choices=sorted(DTYPES))
    ap.add_argument("--max-shard-size", default="5GB")
    ap.add_argument("--merge-lora", action="store_true")
    ap.add_argument("--lora-alpha", type=float, default=None)
    ap.add_argument("--use-rslora", action="store_true")
    ap.add_argument("--quantize", default=None, choices=["int8", "int4", "gptq", "awq"])
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--ollama", action="store_true")
    ap.add_argument("--template", default=None)
    a = ap.parse_args(argv)
    print(export(a.src, a.dst, a.dtype, a.max_shard_size, a.merge_lora, a.lora_alpha, a.use_rslora, a.quantize,
                 a.group_size, a.ollama, a.template))
    return 0
