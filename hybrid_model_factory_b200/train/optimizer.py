"""Flat-buffer AdamW with ZeRO-style sharding.

All trainable parameters live in one contiguous buffer (``flat_param``) and their gradients in
another (``flat_grad``); ``param.data`` / ``param.grad`` are views, so autograd accumulates
straight into the flat gradient and the optimizer touches memory with one fused kernel
(``csrc/kernels/elementwise.cu``: ``adamw_kernel``) instead of one launch per tensor.

With a process group the optimizer states are sharded (ZeRO-1/2 semantics, the configuration
the reference project trains its 8B/128K model with, ``examples/deepspeed/ds_z2_config.json``):

    backward -> reduce-scatter(flat_grad)  -> each rank: grad-norm partial, AdamW on its shard
             -> all-gather(flat_param)

Sequence-parallel ranks hold partial gradients of the same sample, data-parallel replicas hold
gradients of different samples: the reduction is a SUM over everything followed by a division
by the number of data-parallel replicas, folded into the kernel's ``grad_scale``.
Gradient clipping uses the global norm computed on the device (no host synchronisation).
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..utils.profiling import phase


class FlatAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: float = 0.0, group=None, dp_size: int = 1,
                 state_dtype: Optional[torch.dtype] = None, grad_dtype: Optional[torch.dtype] = None,
                 master_weights: bool = False):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        assert self.params, "no trainable parameters"
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.dp_size = max(1, dp_size)
        self.step_count = 0
        p0 = self.params[0]
        self.device, self.dtype = p0.device, p0.dtype
        assert all(p.dtype == self.dtype and p.device == self.device for p in self.params), \
            "all trainable parameters must share one dtype and device"
        self.grad_dtype = grad_dtype or self.dtype
        self.state_dtype = state_dtype or self.dtype
        # no_weight_decay parameters (A_log, dt_bias, D, norms, biases) are handled by a per-element mask-free
        # trick: they are placed in a second segment of the flat buffer that steps with weight_decay = 0.
        decay = [p for p in self.params if not getattr(p, "_no_weight_decay", False) and p.dim() >= 2]
        no_decay = [p for p in self.params if getattr(p, "_no_weight_decay", False) or p.dim() < 2]
        self.params = decay + no_decay
        align = 128 * self.world
        # every parameter starts on a 16-byte boundary of the flat buffers (8 elements also covers fp32): the kernels
        # read weights 16 bytes at a time, and a [4]-element gate vector must not shift what follows it
        pad8 = lambda n: (n + 7) // 8 * 8  # noqa: E731
        n_decay = sum(pad8(p.numel()) for p in decay)
        self.n_decay = (n_decay + align - 1) // align * align
        n_rest = sum(pad8(p.numel()) for p in no_decay)
        self.n_total = self.n_decay + (n_rest + align - 1) // align * align
        self.flat_param = torch.zeros(self.n_total, device=self.device, dtype=self.dtype)
        self.flat_grad = torch.zeros(self.n_total, device=self.device, dtype=self.grad_dtype)
        off = 0
        for i, p in enumerate(self.params):
            if i == len(decay):
                off = self.n_decay
            n = p.numel()
            self.flat_param[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat_param[off:off + n].view(p.shape)
            p.grad = self.flat_grad[off:off + n].view(p.shape) if self.grad_dtype == self.dtype else None
            p._flat_offset = off
            off += pad8(n)
        self.shard = self.n_total // self.world
        lo = self.rank * self.shard
        self._shard_slice = slice(lo, lo + self.shard)
        self.exp_avg = torch.zeros(self.shard, device=self.device, dtype=self.state_dtype)
        self.exp_avg_sq = torch.zeros(self.shard, device=self.device, dtype=self.state_dtype)
        self.master = self.flat_param[self._shard_slice].float().clone() if master_weights else None
        self.norm_sq = torch.zeros(1, device=self.device, dtype=torch.float32)
        self._fp32_grad_params = self.grad_dtype != self.dtype

    # -- gradient plumbing --------------------------------------------------------------
    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        if not self._fp32_grad_params:
            for p in self.params:
                if p.grad is None or p.grad.data_ptr() != self.flat_grad.data_ptr() + p._flat_offset * self.flat_grad.element_size():
                    p.grad = self.flat_grad[p._flat_offset:p._flat_offset + p.numel()].view(p.shape)

    def _collect_grads(self) -> None:
        """When gradients are kept in another dtype than the parameters (fp32 accumulation), copy
        ``p.grad`` into the flat buffer."""
        if not self._fp32_grad_params:
            return
        for p in self.params:
            if p.grad is not None:
                self.flat_grad[p._flat_offset:p._flat_offset + p.numel()].add_(p.grad.reshape(-1).to(self.grad_dtype))
                p.grad = None

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last step (device tensor)."""
        return self.norm_sq.sqrt() / self.dp_size

    # -- step ---------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> None:
        self._collect_grads()
        lr = self.lr if lr is None else lr
        self.step_count += 1
        if self.world > 1:
            gshard = torch.empty(self.shard, device=self.device, dtype=self.grad_dtype)
            with phase("zero_grad_reduce_scatter"):
                dist.reduce_scatter_tensor(gshard, self.flat_grad, group=self.group) if self.flat_grad.is_cuda else \
                    self._cpu_reduce_scatter(gshard)
        else:
            gshard = self.flat_grad
        pshard = self.flat_param[self._shard_slice]
        self.norm_sq.zero_()
        use_kernel = pshard.is_cuda and _lib.kernels_available()
        if use_kernel:
            from ..ops import cuda_ops
            cuda_ops.grad_sumsq(gshard, self.norm_sq)
        else:
            self.norm_sq += gshard.float().pow(2).sum()
        if self.world > 1:
            dist.all_reduce(self.norm_sq, group=self.group)
        gscale = 1.0 / self.dp_size
        b1, b2 = self.betas
        # the shard may straddle the decay / no-decay boundary: step the two pieces separately
        lo = self.rank * self.shard
        pieces = []
        cut = min(max(self.n_decay - lo, 0), self.shard)
        if cut > 0:
            pieces.append((0, cut, self.weight_decay))
        if cut < self.shard:
            pieces.append((cut, self.shard, 0.0))
        for a, b, wd in pieces:
            if use_kernel:
                cuda_ops.adamw_step(pshard[a:b], gshard[a:b], self.exp_avg[a:b], self.exp_avg_sq[a:b], lr=lr, beta1=b1,
                                    beta2=b2, eps=self.eps, weight_decay=wd, step=self.step_count,
                                    master=None if self.master is None else self.master[a:b], norm_sq=self.norm_sq,
                                    max_norm=self.max_grad_norm, grad_scale=gscale)
            else:
                self._torch_adamw(pshard[a:b], gshard[a:b], self.exp_avg[a:b], self.exp_avg_sq[a:b], lr, wd, gscale,
                                  None if self.master is None else self.master[a:b])
        if self.world > 1:
            if self.flat_param.is_cuda:
                with phase("zero_param_all_gather"):
                    dist.all_gather_into_tensor(self.flat_param, pshard.clone(), group=self.group)
            else:
                parts = [torch.empty_like(pshard) for _ in range(self.world)]
                dist.all_gather(parts, pshard.clone(), group=self.group)
                self.flat_param.copy_(torch.cat(parts))

    def _cpu_reduce_scatter(self, out: torch.Tensor) -> None:
        buf = self.flat_grad.clone()
        dist.all_reduce(buf, group=self.group)
        out.copy_(buf[self._shard_slice])

    def _torch_adamw(self, p, g, m, v, lr, wd, gscale, master) -> None:
        b1, b2 = self.betas
        scale = gscale
        if self.max_grad_norm and self.max_grad_norm > 0:
            nrm = self.norm_sq.sqrt() * gscale
            scale = scale * torch.clamp(self.max_grad_norm / (nrm + 1e-6), max=1.0)
        gf = g.float() * scale
        mf = m.float().mul_(b1).add_(gf, alpha=1 - b1)
        vf = v.float().mul_(b2).addcmul_(gf, gf, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        pf = (master if master is not None else p.float())
        pf = pf * (1 - lr * wd) - lr * (mf / bc1) / ((vf / bc2).sqrt() + self.eps)
        m.copy_(mf)
        v.copy_(vf)
        if master is not None:
            master.copy_(pf)
        p.copy_(pf)

    # -- checkpointing ------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "master": self.master, "rank": self.rank, "world": self.world, "shard": self.shard}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["shard"] == self.shard, "optimizer shard layout changed"
        self.step_count = int(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])


def cosine_lr(step: int, base_lr: float, warmup: int, total: int, min_ratio: float = 0.0) -> float:
    if warmup > 0 and step < warmup:
        return base_lr * (step + 1) / warmup
    if total <= warmup:
        return base_lr
    t = min(1.0, (step - warmup) / max(1, total - warmup))
    return base_lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t)))


def wsd_lr(step: int, base_lr: float, warmup: int, total: int, decay_frac: float = 0.1, min_ratio: float = 0.0) -> float:
    """Warmup-stable-decay schedule (reference: ``train/trainer_utils.py:608-646``)."""
    if warmup > 0 and step < warmup:
        return base_lr * (step + 1) / warmup
    decay_steps = int(total * decay_frac)
    if step < total - decay_steps:
        return base_lr
    t = (step - (total - decay_steps)) / max(1, decay_steps)
    return base_lr * (min_ratio + (1 - min_ratio) * (1 - t))


def get_lr(kind: str, step: int, base_lr: float, warmup: int, total: int) -> float:
    if kind in ("cosine", "cosine_with_min_lr"):
        return cosine_lr(step, base_lr, warmup, total)
    if kind in ("wsd", "warmup_stable_decay"):
        return wsd_lr(step, base_lr, warmup, total)
    if kind == "linear":
        if warmup > 0 and step < warmup:
            return base_lr * (step + 1) / warmup
        return base_lr * max(0.0, (total - step) / max(1, total - warmup))
    if warmup > 0 and step < warmup:  # constant / constant_with_warmup
        return base_lr * (step + 1) / warmup
    return base_lr
