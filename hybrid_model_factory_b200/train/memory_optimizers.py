"""Memory-saving optimizers selected by the fine-tuning arguments: GaLore and APOLLO (Adam moments kept in a
rank-``r`` subspace of each weight matrix), BAdam (block-coordinate Adam: one block of layers trains at a time),
Adam-mini (one second moment per block of a tensor instead of per element) and LoRA+ (a larger learning rate for the
LoRA ``B`` matrices).  They share the trainer-facing interface of ``FlatAdamW`` / ``Muon``:
``zero_grad()``, ``step(lr)``, ``grad_norm()``, ``state_dict()``, ``load_state_dict()``.

The reference wires external packages for these (``train/trainer_utils.py:257-605``: ``galore_torch``,
``apollo_torch``, ``badam``, ``adam_mini``, LoRA+ parameter groups); here they are written out against the same
hyper-parameters (``hparams/finetuning_args.py:91-98, 266-392, 498``).
"""
from __future__ import annotations

import math
import re
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class _PerParamOptimizer:
    """Gradient averaging over ranks, global-norm clipping and state (de)serialisation; subclasses give the
    per-parameter update."""

    def __init__(self, named_params, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.0, dp_size: int = 1):
        self.named: List[Tuple[str, torch.nn.Parameter]] = [(n, p) for n, p in named_params if p.requires_grad]
        assert self.named, "no trainable parameters"
        self.params = [p for _, p in self.named]
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm, self.dp_size = max_grad_norm, max(1, dp_size)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.step_count = 0
        self.state: Dict[str, Dict[str, torch.Tensor]] = {n: {} for n, _ in self.named}
        self._norm: Optional[torch.Tensor] = None

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None

    def grad_norm(self) -> torch.Tensor:
        return self._norm if self._norm is not None else torch.zeros(())

    def _active(self, name: str, p: torch.nn.Parameter) -> bool:
        return True

    def _decay(self, p: torch.nn.Parameter) -> float:
        return 0.0 if (p.dim() < 2 or getattr(p, "_no_weight_decay", False)) else self.weight_decay

    def step(self, lr: Optional[float] = None) -> None:
        lr = self.lr if lr is None else lr
        live = [(n, p) for n, p in self.named if p.grad is not None and self._active(n, p)]
        if self.world > 1:
            for _, p in live:
                dist.all_reduce(p.grad)
                p.grad.div_(self.dp_size)
        sq = [(p.grad.float() ** 2).sum() for _, p in live]
        self._norm = torch.sqrt(torch.stack(sq).sum()) if sq else torch.zeros(())
        scale = 1.0
        if self.max_grad_norm > 0 and sq:
            scale = float(torch.clamp(self.max_grad_norm / (self._norm + 1e-6), max=1.0))
        self.step_count += 1
        for n, p in live:
            self._update(n, p, p.grad.float() * scale, lr)

    # Adam on a tensor ``g`` with moments stored under ``key`` of the parameter's state; returns the update direction
    def _adam(self, st: Dict[str, torch.Tensor], g: torch.Tensor, key: str = "") -> torch.Tensor:
        b1, b2 = self.betas
        if "m" + key not in st:
            st["m" + key], st["v" + key] = torch.zeros_like(g), torch.zeros_like(g)
            st["t" + key] = torch.zeros((), dtype=torch.long)
        st["t" + key] += 1
        t = int(st["t" + key])
        m, v = st["m" + key], st["v" + key]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        return (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + self.eps)

    def _apply(self, p: torch.nn.Parameter, upd: torch.Tensor, lr: float) -> None:
        p.data.mul_(1 - lr * self._decay(p)).add_(upd.to(p.dtype), alpha=-lr)

    def _update(self, name: str, p: torch.nn.Parameter, g: torch.Tensor, lr: float) -> None:
        self._apply(p, self._adam(self.state[name], g), lr)

    def state_dict(self) -> dict:
        return {"step": self.step_count, "state": {n: dict(s) for n, s in self.state.items()}}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for n, s in sd["state"].items():
            if n in self.state:
                self.state[n] = {k: v.clone() for k, v in s.items()}


def _matches(name: str, targets: Sequence[str]) -> bool:
    return "all" in targets or any(t in name for t in targets)


class ProjectedAdamW(_PerParamOptimizer):
    """GaLore (``mode="galore"``): the gradient of a target matrix is projected on the top-``rank`` singular
    subspace (recomputed every ``update_interval`` steps), Adam runs there and the update is projected back and
    scaled.  APOLLO (``mode="apollo"``): Adam runs in a random (or SVD) ``rank``-dimensional sketch only to estimate a
    per-channel (or per-tensor) scaling of the raw gradient, which then steps the weight like SGD with
    Adam-like step sizes.  Non-target parameters take plain AdamW."""

    def __init__(self, named_params, lr: float, mode: str = "galore", rank: int = 16, update_interval: int = 200,
                 scale: float = 0.25, proj_type: str = "std", proj: str = "svd", scale_type: str = "channel",
                 targets: Sequence[str] = ("all",), seed: int = 0, **kw):
        super().__init__(named_params, lr, **kw)
        assert mode in ("galore", "apollo")
        self.mode, self.rank, self.interval, self.scale = mode, rank, max(1, update_interval), scale
        self.proj_type, self.proj, self.scale_type = proj_type, (proj if mode == "apollo" else "svd"), scale_type
        self.targets = tuple(targets)
        self.seed = seed

    def _is_target(self, name: str, p) -> bool:
        return p.dim() == 2 and min(p.shape) > self.rank and _matches(name, self.targets)

    def _left(self, p) -> bool:
        """Project the rows (``P^T G``, left) or the columns (``G Q``, right)?  ``std`` picks the short side."""
        if self.proj_type == "left":
            return True
        if self.proj_type == "right":
            return False
        short_rows = p.shape[0] <= p.shape[1]
        return short_rows if self.proj_type == "std" else not short_rows       # reverse_std

    def _projector(self, name: str, p, g: torch.Tensor) -> torch.Tensor:
        st = self.state[name]
        n_upd = int(st.get("n_proj", torch.zeros(())))
        if "P" in st and (int(st["t"]) if "t" in st else 0) % self.interval != 0:
            return st["P"]
        left = self._left(p)
        if self.proj == "random":
            gen = torch.Generator(device="cpu").manual_seed(self.seed + 7919 * n_upd + hash(name) % 65521)
            dim = g.shape[0] if left else g.shape[1]
            P = (torch.randn(dim, self.rank, generator=gen) / math.sqrt(self.rank)).to(g.device, g.dtype)
        else:
            U, _, Vh = torch.linalg.svd(g, full_matrices=False)
            P = U[:, :self.rank] if left else Vh[:self.rank].t()
        st["P"], st["n_proj"] = P.contiguous(), torch.tensor(n_upd + 1)
        return st["P"]

    def _update(self, name, p, g, lr):
        if not self._is_target(name, p):
            return super()._update(name, p, g, lr)
        st = self.state[name]
        P = self._projector(name, p, g)
        left = self._left(p)
        low = P.t() @ g if left else g @ P                       # [r, n] or [m, r]
        step_low = self._adam(st, low)
        if self.mode == "galore":
            upd = (P @ step_low if left else step_low @ P.t()) * self.scale
        else:
            if self.scale_type == "tensor":
                s = step_low.norm() / (low.norm() + 1e-8)
            else:                                                  # one factor per channel of the unprojected side
                dim = 0 if left else 1
                s = step_low.norm(dim=dim, keepdim=True) / (low.norm(dim=dim, keepdim=True) + 1e-8)
            upd = g * s * math.sqrt(self.scale)
        self._apply(p, upd, lr)


class BlockAdamW(_PerParamOptimizer):
    """BAdam: the layers are partitioned into blocks; only the active block receives updates (and holds Adam
    moments), and the active block changes every ``switch_interval`` steps (``ascending`` / ``descending`` /
    ``random`` / ``fixed``).  ``mode="ratio"`` instead updates a fixed fraction of every matrix's rows (``adjacent``:
    a contiguous band that moves, ``scatter``: a random subset redrawn at every switch).  Call
    ``apply_requires_grad()`` after a switch to stop autograd from computing gradients of frozen blocks."""

    LAYER_RE = re.compile(r"layers\.(\d+)\.")

    def __init__(self, named_params, lr: float, mode: str = "layer", switch_mode: str = "ascending",
                 switch_interval: int = 50, start_block: Optional[int] = None, update_ratio: float = 0.05,
                 mask_mode: str = "adjacent", seed: int = 0, **kw):
        super().__init__(named_params, lr, **kw)
        self.mode, self.switch_mode, self.switch_interval = mode, switch_mode, max(1, switch_interval)
        self.update_ratio, self.mask_mode = update_ratio, mask_mode
        ids = sorted({int(m.group(1)) for n, _ in self.named for m in [self.LAYER_RE.search(n)] if m})
        self.blocks: List[Optional[int]] = ids + [None]           # ``None``: everything outside the layer stack
        self.gen = torch.Generator().manual_seed(seed)
        self.active = (start_block if start_block is not None else
                       (len(self.blocks) - 1 if switch_mode == "descending" else 0)) % len(self.blocks)
        self.masks: Dict[str, torch.Tensor] = {}

    def _block_of(self, name: str) -> Optional[int]:
        m = self.LAYER_RE.search(name)
        return int(m.group(1)) if m else None

    def _active(self, name, p) -> bool:
        return self.mode == "ratio" or self._block_of(name) == self.blocks[self.active]

    def apply_requires_grad(self) -> None:
        if self.mode == "layer":
            for n, p in self.named:
                p.requires_grad_(self._active(n, p))

    def _switch(self) -> None:
        n = len(self.blocks)
        if self.switch_mode == "ascending":
            self.active = (self.active + 1) % n
        elif self.switch_mode == "descending":
            self.active = (self.active - 1) % n
        elif self.switch_mode == "random":
            self.active = int(torch.randint(0, n, (1,), generator=self.gen))
        self.masks.clear()
        for s in self.state.values():       # the moments belong to the block that just went inactive
            s.clear()

    def _row_mask(self, name: str, p) -> torch.Tensor:
        if name not in self.masks:
            rows = p.shape[0]
            k = max(1, int(round(rows * self.update_ratio)))
            mask = torch.zeros(rows, dtype=torch.bool)
            if self.mask_mode == "scatter":
                mask[torch.randperm(rows, generator=self.gen)[:k]] = True
            else:
                start = (self.step_count // self.switch_interval * k) % rows
                mask[(torch.arange(k) + start) % rows] = True
            self.masks[name] = mask.to(p.device)
        return self.masks[name]

    def step(self, lr: Optional[float] = None) -> None:
        super().step(lr)
        if self.step_count % self.switch_interval == 0 and self.switch_mode != "fixed":
            self._switch()

    def _update(self, name, p, g, lr):
        if self.mode == "ratio" and p.dim() >= 2:
            mask = self._row_mask(name, p)
            upd = torch.zeros_like(g)
            upd[mask] = self._adam(self.state[name], g[mask])
            p.data[mask] = (p.data[mask].float() * (1 - lr * self._decay(p)) - lr * upd[mask]).to(p.dtype)
            return
        super()._update(name, p, g, lr)


class AdamMini(_PerParamOptimizer):
    """Adam-mini: the first moment stays per element; the second moment is one scalar per block of the tensor — per
    attention head for q/k projections, per output row for the other matrices, per tensor for vectors;
    embeddings and the output head keep the element-wise second moment."""

    def __init__(self, named_params, lr: float, head_dim: int = 128, **kw):
        super().__init__(named_params, lr, **kw)
        self.head_dim = head_dim

    def _blocks(self, name: str, p) -> Optional[Tuple[int, ...]]:
        """Shape the gradient is viewed in; the mean of ``g^2`` is taken over the last axis."""
        if "embed" in name or "lm_head" in name:
            return None
        if p.dim() < 2:
            return (1, p.numel())
        if re.search(r"\b(q_proj|k_proj)\b", name) and p.shape[0] % self.head_dim == 0:
            return (p.shape[0] // self.head_dim, self.head_dim * p.shape[1])
        return (p.shape[0], p[0].numel())

    def _update(self, name, p, g, lr):
        shape = self._blocks(name, p)
        if shape is None:
            return super()._update(name, p, g, lr)
        st = self.state[name]
        b1, b2 = self.betas
        gb = g.reshape(shape)
        if "m" not in st:
            st["m"], st["v"] = torch.zeros_like(gb), torch.zeros(shape[0], 1, device=g.device, dtype=g.dtype)
            st["t"] = torch.zeros((), dtype=torch.long)
        st["t"] += 1
        t = int(st["t"])
        st["m"].mul_(b1).add_(gb, alpha=1 - b1)
        st["v"].mul_(b2).add_((gb * gb).mean(dim=1, keepdim=True), alpha=1 - b2)
        upd = (st["m"] / (1 - b1 ** t)) / ((st["v"] / (1 - b2 ** t)).sqrt() + self.eps)
        self._apply(p, upd.reshape(p.shape), lr)


class LoraPlusAdamW(_PerParamOptimizer):
    """LoRA+: ``lora_B`` matrices step with ``lr * lr_ratio``, LoRA embeddings with ``lr_embedding``."""

    def __init__(self, named_params, lr: float, lr_ratio: float = 16.0, lr_embedding: float = 1e-6, **kw):
        super().__init__(named_params, lr, **kw)
        self.lr_ratio, self.lr_embedding, self.base_lr = lr_ratio, lr_embedding, lr

    def _update(self, name, p, g, lr):
        if "lora_embedding_B" in name or ("embed" in name and "lora" in name):
            lr = self.lr_embedding * (lr / self.base_lr if self.base_lr else 1.0)
        elif "lora_B" in name or p.dim() == 1:
            lr = lr * self.lr_ratio
        super()._update(name, p, g, lr)


def build_optimizer(name: str, model: torch.nn.Module, lr: float, trainable=None, **kw):
    """``name``: ``galore`` | ``apollo`` | ``badam`` | ``adam_mini`` | ``loraplus``; ``kw`` carries the
    optimizer-specific arguments plus ``betas``, ``eps``, ``weight_decay``, ``max_grad_norm``, ``dp_size``."""
    ids = None if trainable is None else {id(p) for p in trainable}
    named = [(n, p) for n, p in model.named_parameters() if ids is None or id(p) in ids]
    if name in ("galore", "apollo"):
        return ProjectedAdamW(named, lr, mode=name, **kw)
    if name == "badam":
        return BlockAdamW(named, lr, **kw)
    if name == "adam_mini":
        return AdamMini(named, lr, **kw)
    if name == "loraplus":
        return LoraPlusAdamW(named, lr, **kw)
    raise ValueError(f"unknown optimizer {name!r}")
