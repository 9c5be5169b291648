"""Readers for checkpoints whose linear layers were quantised after training by GPTQ or AWQ: the packed integers are
expanded to bf16 matrices while the checkpoint is loaded, so every kernel of this package sees an ordinary weight.
(Training and serving here run in bf16 / fp8; the integer formats are an interchange format, not a compute format.)

Layouts, for a linear layer with ``in`` inputs and ``out`` outputs, ``bits`` in {2, 4, 8}, ``per = 32 // bits``:

=========  ==========================  ==========================  ====================  ==========================
format     ``qweight`` (int32)         ``qzeros`` (int32)          ``scales`` (fp16)     value of W[in, out]
=========  ==========================  ==========================  ====================  ==========================
GPTQ       ``[in / per, out]``, rows   ``[groups, out / per]``,    ``[groups, out]``     ``(q - (z + 1)) * s`` with
           packed low bits first       columns packed in order                           group ``g_idx[in]``
AWQ        ``[in, out / per]``,        ``[groups, out / per]``,    ``[groups, out]``     ``(q - z) * s`` with group
           columns packed in the       same column order                                 ``in // group_size``
           order 0,2,4,6,1,3,5,7
=========  ==========================  ==========================  ====================  ==========================

The module weight is ``W.T`` (``[out, in]``).  The reference reaches these formats through ``transformers``'
quantiser classes (``model/model_utils/quantization.py:85-165``, methods ``gptq`` and ``awq``) and keeps the integers
for the library's kernels; this package expands them once at load time."""
from __future__ import annotations

from typing import Dict, Optional

import torch

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)            # nibble i of a packed word holds column AWQ_ORDER[i]


def _unpack(words: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """int32 words -> integers of ``bits`` bits, expanded along ``dim`` (low bits first)."""
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int32) * bits
    w = words.to(torch.int32)
    if dim == 0:
        out = (w[:, None, :] >> shifts[None, :, None]) & ((1 << bits) - 1)
        return out.reshape(w.shape[0] * per, w.shape[1])
    out = (w[:, :, None] >> shifts[None, None, :]) & ((1 << bits) - 1)
    return out.reshape(w.shape[0], w.shape[1] * per)


def _pack(vals: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    per = 32 // bits
    v = vals.to(torch.int64) & ((1 << bits) - 1)
    shifts = torch.arange(per, dtype=torch.int64) * bits
    if dim == 0:
        words = (v.reshape(-1, per, v.shape[1]) << shifts[None, :, None]).sum(1)
    else:
        words = (v.reshape(v.shape[0], -1, per) << shifts[None, None, :]).sum(2)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)          # two's complement into int32
    return words.to(torch.int32)


def _awq_natural(cols: torch.Tensor, bits: int) -> torch.Tensor:
    """Undo AWQ's column interleave (defined for 4 bits: eight values per word)."""
    if bits != 4:
        return cols
    inverse = torch.tensor([AWQ_ORDER.index(j) for j in range(8)])
    return cols.reshape(cols.shape[0], -1, 8)[:, :, inverse].reshape(cols.shape)


def dequantize_gptq(qweight, qzeros, scales, g_idx: Optional[torch.Tensor], bits: int,
                    dtype: torch.dtype = torch.bfloat16, zero_offset: int = 1) -> torch.Tensor:
    """Module weight ``[out, in]`` of a GPTQ layer.  ``zero_offset`` is 1 for the original format (zeros stored minus
    one) and 0 for the ``gptq_v2`` checkpoint format."""
    q = _unpack(qweight, bits, dim=0)                                      # [in, out]
    z = _unpack(qzeros, bits, dim=1)[:, :q.shape[1]] + zero_offset         # [groups, out]
    n_in = q.shape[0]
    if g_idx is None:
        group = n_in // scales.shape[0]
        g_idx = torch.arange(n_in) // group
    g = g_idx.long()
    w = (q - z[g]).float() * scales.float()[g]
    return w.t().contiguous().to(dtype)


def dequantize_awq(qweight, qzeros, scales, bits: int, group_size: int,
                   dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Module weight ``[out, in]`` of an AWQ (GEMM layout) layer."""
    q = _awq_natural(_unpack(qweight, bits, dim=1), bits)                  # [in, out]
    z = _awq_natural(_unpack(qzeros, bits, dim=1), bits)                   # [groups, out]
    n_in = q.shape[0]
    group = group_size if group_size > 0 else n_in
    g = torch.arange(n_in) // group
    w = (q - z[g]).float() * scales.float()[g]
    return w.t().contiguous().to(dtype)


def _affine_groups(w_in_out: torch.Tensor, bits: int, group_size: int):
    """Asymmetric round-to-nearest per (group of inputs, output): integers, zeros, scales."""
    n_in, n_out = w_in_out.shape
    group = group_size if group_size > 0 else n_in
    g = w_in_out.float().reshape(n_in // group, group, n_out)
    lo, hi = g.amin(1), g.amax(1)
    qmax = (1 << bits) - 1
    scales = ((hi - lo) / qmax).clamp_min(1e-8).to(torch.float16)
    zeros = torch.clamp(torch.round(-lo / scales.float()), 0, qmax).to(torch.int32)
    q = torch.clamp(torch.round(g / scales.float()[:, None]) + zeros[:, None], 0, qmax).to(torch.int32)
    return q.reshape(n_in, n_out), zeros, scales


def pack_gptq(weight: torch.Tensor, bits: int = 4, group_size: int = 128) -> Dict[str, torch.Tensor]:
    """Round-to-nearest quantisation of a module weight ``[out, in]`` written in the GPTQ layout (no error
    compensation: this is the packer of ``hmf export --quantize gptq`` and of the tests, not the GPTQ algorithm)."""
    q, zeros, scales = _affine_groups(weight.t(), bits, group_size)
    group = group_size if group_size > 0 else weight.shape[1]
    return {"qweight": _pack(q, bits, dim=0), "qzeros": _pack(zeros - 1, bits, dim=1), "scales": scales,
            "g_idx": (torch.arange(weight.shape[1]) // group).to(torch.int32)}


def pack_awq(weight: torch.Tensor, bits: int = 4, group_size: int = 128) -> Dict[str, torch.Tensor]:
    """Round-to-nearest quantisation of a module weight ``[out, in]`` written in the AWQ GEMM layout."""
    q, zeros, scales = _affine_groups(weight.t(), bits, group_size)

    def interleave(cols):
        if bits != 4:
            return cols
        return cols.reshape(cols.shape[0], -1, 8)[:, :, torch.tensor(AWQ_ORDER)].reshape(cols.shape)

    return {"qweight": _pack(interleave(q), bits, dim=1), "qzeros": _pack(interleave(zeros), bits, dim=1),
            "scales": scales}


def detect_method(state: Dict[str, torch.Tensor], quant_config: Optional[dict] = None) -> Optional[str]:
    """``"gptq"``, ``"awq"`` or ``None`` for a state dict, from the checkpoint's ``quantization_config`` when it has
    one, else from the tensor shapes (GPTQ packs inputs, AWQ packs outputs)."""
    name = next((k[:-len(".qzeros")] for k in state if k.endswith(".qzeros")), None)
    if name is None:
        return None
    method = str((quant_config or {}).get("quant_method", "")).lower()
    if method in ("gptq", "awq"):
        return method
    return "gptq" if state[name + ".qweight"].shape[1] == state[name + ".scales"].shape[1] else "awq"


def expand_quantized_state(state: Dict[str, torch.Tensor], quant_config: Optional[dict] = None,
                           dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Replaces every ``<layer>.qweight / .qzeros / .scales (/ .g_idx)`` group by ``<layer>.weight``."""
    method = detect_method(state, quant_config)
    if method is None:
        return state
    cfg = quant_config or {}
    out = {}
    for k, v in state.items():
        if k.endswith((".qzeros", ".scales", ".g_idx")) and k.rsplit(".", 1)[0] + ".qweight" in state:
            continue
        if not k.endswith(".qweight") or k[:-len(".qweight")] + ".qzeros" not in state:
            out[k] = v
            continue
        name = k[:-len(".qweight")]
        qz, sc = state[name + ".qzeros"], state[name + ".scales"]
        if method == "gptq":
            bits = int(cfg.get("bits", 0)) or 32 * qz.shape[1] // sc.shape[1]   # zeros: 32 / bits columns per word
            offset = 0 if str(cfg.get("checkpoint_format", "gptq")).lower() == "gptq_v2" else 1
            out[name + ".weight"] = dequantize_gptq(v, qz, sc, state.get(name + ".g_idx"), bits, dtype, offset)
        else:
            bits = int(cfg.get("bits", 0) or cfg.get("w_bit", 0)) or 32 * v.shape[1] // sc.shape[1]
            n_in = v.shape[0]
            group = int(cfg.get("group_size", 0) or cfg.get("q_group_size", 0)) or n_in // sc.shape[0]
            out[name + ".weight"] = dequantize_awq(v, qz, sc, bits, group, dtype)
    return out
