"""Muon (momentum + Newton-Schulz orthogonalisation) for the 2-D hidden weights, AdamW for everything else
(embeddings, ``lm_head``, norms, gates, biases).  Same interface as ``FlatAdamW`` so the trainer can swap them.
Gradients are averaged over all ranks with one all-reduce per parameter bucket (no state sharding: Muon needs the
whole matrix).  Reference: the vendored ``third_party/muon/muon.py`` selected by ``use_muon``
(``train/trainer_utils.py:257-605``).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def newton_schulz(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal polar factor of ``G`` (bf16 on the GPU)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.to(torch.bfloat16 if G.is_cuda else torch.float32)
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-1, -2)
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.transpose(-1, -2)
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    if transposed:
        X = X.transpose(-1, -2)
    return X.to(G.dtype)


class Muon:
    def __init__(self, named_params, lr: float = 2e-2, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5, adam_lr_ratio: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: float = 0.0, dp_size: int = 1):
        named = [(n, p) for n, p in named_params if p.requires_grad]
        is_matrix = lambda n, p: p.dim() == 2 and "embed_tokens" not in n and "lm_head" not in n  # noqa: E731
        self.muon_params: List[torch.nn.Parameter] = [p for n, p in named if is_matrix(n, p)]
        self.adam_params: List[torch.nn.Parameter] = [p for n, p in named if not is_matrix(n, p)]
        self.params = self.muon_params + self.adam_params
        self.lr, self.momentum, self.nesterov, self.ns_steps = lr, momentum, nesterov, ns_steps
        self.adam_lr_ratio, self.betas, self.eps, self.weight_decay = adam_lr_ratio, betas, eps, weight_decay
        self.max_grad_norm, self.dp_size = max_grad_norm, max(1, dp_size)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.step_count = 0
        self.buf = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.muon_params}
        self.m = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.adam_params}
        self.v = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.adam_params}
        self._norm: Optional[torch.Tensor] = None

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None

    def _reduce(self) -> None:
        if self.world > 1:
            for p in self.params:
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                dist.all_reduce(p.grad)
                p.grad.div_(self.dp_size)      # SP ranks hold partial sums of one sample, DP ranks are averaged

    def grad_norm(self) -> torch.Tensor:
        return self._norm if self._norm is not None else torch.zeros(())

    def step(self, lr: Optional[float] = None) -> None:
        lr = self.lr if lr is None else lr
        self._reduce()
        grads = [p.grad for p in self.params if p.grad is not None]
        self._norm = torch.sqrt(sum((g.float() ** 2).sum() for g in grads)) if grads else torch.zeros(())
        scale = 1.0
        if self.max_grad_norm > 0:
            scale = float(torch.clamp(self.max_grad_norm / (self._norm + 1e-6), max=1.0))
        self.step_count += 1
        b1, b2 = self.betas
        for p in self.muon_params:
            if p.grad is None:
                continue
            g = p.grad.float() * scale
            buf = self.buf[id(p)]
            buf.mul_(self.momentum).add_(g)
            upd = g.add(buf, alpha=self.momentum) if self.nesterov else buf
            upd = newton_schulz(upd, self.ns_steps).float()
            upd = upd * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
            p.data.mul_(1 - lr * self.weight_decay).add_(upd.to(p.dtype), alpha=-lr)
        alr = lr * self.adam_lr_ratio
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        for p in self.adam_params:
            if p.grad is None:
                continue
            g = p.grad.float() * scale
            m, v = self.m[id(p)], self.v[id(p)]
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            wd = 0.0 if (p.dim() < 2 or getattr(p, "_no_weight_decay", False)) else self.weight_decay
            p.data.mul_(1 - alr * wd).add_(upd.to(p.dtype), alpha=-alr)

    def state_dict(self) -> dict:
        return {"step": self.step_count, "buf": [self.buf[id(p)] for p in self.muon_params],
                "m": [self.m[id(p)] for p in self.adam_params], "v": [self.v[id(p)] for p in self.adam_params]}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for p, t in zip(self.muon_params, sd["buf"]):
            self.buf[id(p)].copy_(t)
        for p, m, v in zip(self.adam_params, sd["m"], sd["v"]):
            self.m[id(p)].copy_(m)
            self.v[id(p)].copy_(v)
