"""Adapters on a quantised base (QLoRA): the frozen base weights of the adapted linear layers are held as 4-bit or
8-bit codes with one scale per block of inputs, and expanded block by block whenever a layer runs; only the low-rank
adapters (bf16) train.  An 8B model's projections then take about 4.5 GB instead of 15 GB.

* ``nf4``: 4-bit codes index a fixed table of 16 levels (the quantiles of a standard normal distribution, rescaled to
  [-1, 1], as published with QLoRA); a block's scale is its largest magnitude.
* ``int8`` / ``int4``: symmetric integers.

The matrix product neither stores the expanded weight for the backward pass nor needs a weight gradient: the backward
pass expands the codes again and returns ``dy @ W`` only.

Reference: ``model/model_utils/quantization.py:166-229`` (``quantization_bit`` with ``quantization_method: bnb | hqq |
eetq`` hands the base model to those libraries' 4 / 8-bit layers); here the layer is this package's own and the
expansion is plain tensor arithmetic.  Double quantisation of the scales is not reproduced (scales are bf16)."""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F

NF4_LEVELS = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
              -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
              0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
              0.7229568362236023, 1.0)


class _FrozenQuantMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        ctx.layer = layer
        return F.linear(x, layer.dequantize(x.dtype))

    @staticmethod
    def backward(ctx, dy):
        return dy @ ctx.layer.dequantize(dy.dtype), None


class QuantizedLinear(nn.Module):
    """Frozen ``y = x W^T + b`` with ``W`` stored as codes.  ``weight`` expands the whole matrix (what adapter
    initialisation and merging read); ``forward`` does the same per call without keeping it."""

    def __init__(self, linear: nn.Linear, bits: int = 4, quant_type: str = "nf4", block_size: int = 64):
        super().__init__()
        if bits not in (4, 8):
            raise ValueError(f"quantization_bit must be 4 or 8, not {bits}")
        if bits == 8:
            quant_type = "int"
        if quant_type not in ("nf4", "int"):
            raise ValueError(f"unknown quantisation type '{quant_type}' (nf4, int)")
        w = linear.weight.detach()
        self.out_features, self.in_features = w.shape
        if self.in_features % block_size:
            raise ValueError(f"{self.in_features} inputs do not divide into blocks of {block_size}")
        self.bits, self.quant_type, self.block_size = bits, quant_type, block_size
        self.compute_dtype = w.dtype
        blocks = w.float().reshape(self.out_features, -1, block_size)
        absmax = blocks.abs().amax(-1, keepdim=True).clamp_min(1e-12)
        if quant_type == "nf4":
            levels = torch.tensor(NF4_LEVELS, device=w.device)
            edges = (levels[1:] + levels[:-1]) / 2                       # nearest level = bucket between midpoints
            codes = torch.bucketize(blocks / absmax, edges).to(torch.uint8)
            scales = absmax
        else:
            qmax = 2 ** (bits - 1) - 1
            scales = absmax / qmax
            codes = (torch.clamp(torch.round(blocks / scales), -qmax - 1, qmax) + (qmax + 1)).to(torch.uint8)
        codes = codes.reshape(self.out_features, self.in_features)
        if bits == 4:
            codes = (codes[:, 0::2] << 4) | codes[:, 1::2]
        self.register_buffer("qweight", codes.contiguous())
        self.register_buffer("scales", scales.squeeze(-1).to(torch.bfloat16))
        self.bias = None if linear.bias is None else nn.Parameter(linear.bias.detach().clone(), requires_grad=False)

    def dequantize(self, dtype: torch.dtype = None) -> torch.Tensor:
        q = self.qweight
        if self.bits == 4:
            q = torch.stack([q >> 4, q & 0xF], dim=-1).reshape(self.out_features, self.in_features)
        if self.quant_type == "nf4":
            vals = torch.tensor(NF4_LEVELS, device=q.device, dtype=torch.float32)[q.long()]
        else:
            vals = q.float() - float(2 ** (self.bits - 1))
        w = vals.reshape(self.out_features, -1, self.block_size) * self.scales.float().unsqueeze(-1)
        return w.reshape(self.out_features, self.in_features).to(dtype or self.compute_dtype)

    @property
    def weight(self) -> torch.Tensor:
        return self.dequantize()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = _FrozenQuantMatmul.apply(x, self)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def to_linear(self) -> nn.Linear:
        lin = nn.Linear(self.in_features, self.out_features, bias=self.bias is not None, device=self.qweight.device,
                        dtype=self.compute_dtype)
        with torch.no_grad():
            lin.weight.copy_(self.dequantize())
            if self.bias is not None:
                lin.bias.copy_(self.bias)
        return lin

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, {self.quant_type}{self.bits}, block={self.block_size}"


def quantize_adapter_bases(model: nn.Module, bits: int = 4, quant_type: str = "nf4", block_size: int = 64) -> List[str]:
    """Replaces the frozen base of every ``LoRALinear`` whose input width divides into blocks by a ``QuantizedLinear``
    (run after ``apply_lora``: PiSSA has already taken its share out of the base weight by then).  Returns their
    names."""
    from .adapters import LoRALinear
    done = []
    for name, m in model.named_modules():
        if isinstance(m, LoRALinear) and isinstance(m.base, nn.Linear) and m.base.in_features % block_size == 0:
            m.base = QuantizedLinear(m.base, bits, quant_type, block_size)
            done.append(name)
    return done


def quantized_bytes(model: nn.Module) -> int:
    return sum(m.qweight.numel() + 2 * m.scales.numel() for m in model.modules() if isinstance(m, QuantizedLinear))
