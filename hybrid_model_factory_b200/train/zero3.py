"""ZeRO stage 3: parameters, gradients and optimizer states are all sharded over the ranks; a unit's full
parameters exist only while that unit computes.

A *unit* is one decoder layer (or any module handed to ``Zero3Engine``); everything outside the units (embedding,
final norm, output head) forms one more unit.  Each unit owns a flat shard ``[n_pad / world]`` of its parameters.

* before the unit's forward a hook all-gathers the shards into a full flat buffer and points the parameters at views
  of it; after a forward that records no autograd graph (the first pass of a checkpointed layer, inference) the
  buffer is dropped again.  When a graph is recorded (the recompute pass inside backward, or training without
  checkpointing) the buffer stays until every parameter of the unit has received its gradient;
* then the unit's gradients are flattened, reduce-scattered (summed over ranks) into the shard's gradient and freed,
  and the full parameters are dropped;
* ``step()`` runs AdamW on the shards only (fused kernel on the GPU).  With ``offload_optimizer=True`` the two
  moments and the fp32 master copy live in pinned host memory and stream through the GPU one unit at a time.

With per-layer activation checkpointing the peak parameter memory is one layer plus the outside unit.  The reference
gets the same behaviour from DeepSpeed ZeRO-3 (+ CPU offload) configs (``examples/deepspeed/ds_z3_config.json``,
``ds_z3_offload_config.json``; ``hparams/parser.py:170-212`` checks the combinations).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib


def _all_gather_flat(out: torch.Tensor, shard: torch.Tensor, group) -> None:
    if out.is_cuda:
        dist.all_gather_into_tensor(out, shard, group=group)
    else:
        parts = list(out.chunk(dist.get_world_size(group)))
        dist.all_gather(parts, shard, group=group)


def _reduce_scatter_flat(out: torch.Tensor, full: torch.Tensor, rank: int, group) -> None:
    if full.is_cuda:
        dist.reduce_scatter_tensor(out, full, group=group)
    else:       # gloo has no reduce-scatter: all-reduce and keep this rank's part
        dist.all_reduce(full, group=group)
        out.copy_(full.chunk(dist.get_world_size(group))[rank])


class _Unit:
    def __init__(self, name: str, module_or_params, world: int, rank: int, group, align: int = 128, replica_group=None):
        self.name, self.world, self.rank, self.group = name, world, rank, group
        self.replica_group = replica_group
        if isinstance(module_or_params, torch.nn.Module):
            self.params = [p for p in module_or_params.parameters() if p.requires_grad]
        else:
            self.params = [p for p in module_or_params if p.requires_grad]
        p0 = self.params[0]
        self.device, self.dtype = p0.device, p0.dtype
        self.shapes = [p.shape for p in self.params]
        self.numels = [p.numel() for p in self.params]
        # weight-decayed tensors first, so a shard is stepped as (at most) two contiguous pieces
        order = sorted(range(len(self.params)), key=lambda i: self._no_decay(self.params[i]))
        self.params = [self.params[i] for i in order]
        self.shapes = [self.shapes[i] for i in order]
        self.numels = [self.numels[i] for i in order]
        # every parameter starts on a 16-byte boundary of the flat buffer (the kernels read weights 16 bytes at a time)
        self.slots = [(k + 7) // 8 * 8 for k in self.numels]
        self.n_decay = sum(n for p, n in zip(self.params, self.slots) if not self._no_decay(p))
        n = sum(self.slots)
        self.n_pad = (n + align * world - 1) // (align * world) * (align * world)
        self.shard_len = self.n_pad // world
        full = torch.zeros(self.n_pad, device=self.device, dtype=self.dtype)
        off = 0
        for p, k, slot in zip(self.params, self.numels, self.slots):
            full[off:off + k].copy_(p.data.reshape(-1))
            off += slot
        self.shard = full[rank * self.shard_len:(rank + 1) * self.shard_len].clone()
        self.grad_shard: Optional[torch.Tensor] = None
        self.full: Optional[torch.Tensor] = None
        self.pending = 0
        self._empty = torch.empty(0, device=self.device, dtype=self.dtype)
        self.release()
        for p in self.params:
            p.register_post_accumulate_grad_hook(self._on_grad)

    @staticmethod
    def _no_decay(p) -> bool:
        return bool(getattr(p, "_no_weight_decay", False) or p.dim() < 2)

    # -- parameters ---------------------------------------------------------------------------------
    def materialize(self) -> None:
        if self.full is not None:
            return
        self.full = torch.empty(self.n_pad, device=self.device, dtype=self.dtype)
        if self.world > 1:
            _all_gather_flat(self.full, self.shard, self.group)
        else:
            self.full.copy_(self.shard)
        off = 0
        for p, k, shp, slot in zip(self.params, self.numels, self.shapes, self.slots):
            p.data = self.full[off:off + k].view(shp)
            off += slot

    def release(self) -> None:
        self.full = None
        for p in self.params:
            p.data = self._empty

    # -- gradients ----------------------------------------------------------------------------------
    def expect_grads(self) -> None:
        self.pending = len(self.params)

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        self.pending -= 1
        if self.pending == 0:
            self.reduce_grads()

    def reduce_grads(self) -> None:
        """All parameters of the unit have their gradient: flatten, reduce-scatter, free."""
        flat = torch.zeros(self.n_pad, device=self.device, dtype=self.dtype)
        off = 0
        for p, k, slot in zip(self.params, self.numels, self.slots):
            if p.grad is not None:
                flat[off:off + k].copy_(p.grad.reshape(-1))
                p.grad = None
            off += slot
        if self.world > 1:
            out = torch.empty(self.shard_len, device=self.device, dtype=self.dtype)
            _reduce_scatter_flat(out, flat, self.rank, self.group)
        else:
            out = flat
        if self.replica_group is not None:      # MiCS: the same shard lives in every replica group
            dist.all_reduce(out, group=self.replica_group)
        self.grad_shard = out if self.grad_shard is None else self.grad_shard.add_(out)
        self.release()


def mics_groups(shard_size: int):
    """MiCS layout: parameters are sharded inside groups of ``shard_size`` consecutive ranks and replicated across the
    groups.  Returns ``(shard_group, replica_group)`` of the calling rank (collective: every rank creates every
    group).  The reference forces this layout through DeepSpeed's ``mics_shard_size`` (``model/loader.py:185-208``)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    assert world % shard_size == 0, "mics_shard_size must divide the world size"
    shard = replica = None
    for g in range(world // shard_size):
        ranks = list(range(g * shard_size, (g + 1) * shard_size))
        grp = dist.new_group(ranks)
        if rank in ranks:
            shard = grp
    for i in range(shard_size):
        ranks = list(range(i, world, shard_size))
        grp = dist.new_group(ranks)
        if rank in ranks:
            replica = grp
    return shard, (replica if world > shard_size else None)


class Zero3Engine:
    """Shards ``model`` in place.  ``units``: the modules to shard separately (default: ``model.model.layers``)."""

    def __init__(self, model: torch.nn.Module, units: Optional[Sequence[torch.nn.Module]] = None, group=None,
                 lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.0, dp_size: Optional[int] = None, offload_optimizer: bool = False,
                 state_dtype: torch.dtype = torch.float32, replica_group=None):
        self.model, self.group, self.replica_group = model, group, replica_group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        n_rep = dist.get_world_size(replica_group) if replica_group is not None else 1
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.dp_size = self.world * n_rep if dp_size is None else max(1, dp_size)
        self.offload = offload_optimizer
        if units is None:
            units = list(model.model.layers)
        self.units: List[_Unit] = []
        inside = set()
        for i, m in enumerate(units):
            if any(p.requires_grad for p in m.parameters()):
                u = _Unit(f"unit{i}", m, self.world, self.rank, group, replica_group=replica_group)
                self.units.append(u)
                inside.update(id(p) for p in u.params)
                m.register_forward_pre_hook(self._pre(u))
                m.register_forward_hook(self._post(u))
        rest = [p for p in model.parameters() if p.requires_grad and id(p) not in inside]
        self.outer: Optional[_Unit] = None
        if rest:
            self.outer = _Unit("outer", rest, self.world, self.rank, group, replica_group=replica_group)
            self.units.append(self.outer)
            model.register_forward_pre_hook(self._pre(self.outer))
            model.register_forward_hook(self._post(self.outer))
        dev = self.units[0].device
        host = dict(device="cpu", pin_memory=torch.cuda.is_available()) if offload_optimizer else dict(device=dev)
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        for u in self.units:
            master = u.shard.detach().float().to(host["device"])
            if host.get("pin_memory"):
                master = master.pin_memory()
            self.state[u.name] = {"m": torch.zeros(u.shard_len, dtype=state_dtype, **host),
                                  "v": torch.zeros(u.shard_len, dtype=state_dtype, **host), "master": master}
        self.step_count = 0
        self._norm = torch.zeros((), device=dev)

    def _pre(self, u: _Unit):
        def hook(_m, _args):
            u.materialize()
            if torch.is_grad_enabled():
                u.expect_grads()
        return hook

    def _post(self, u: _Unit):
        def hook(_m, _args, _out):
            if not torch.is_grad_enabled():
                u.release()
        return hook

    # -- trainer interface ------------------------------------------------------------------------
    def zero_grad(self) -> None:
        for u in self.units:
            u.grad_shard = None
            for p in u.params:
                p.grad = None

    def grad_norm(self) -> torch.Tensor:
        return self._norm

    def parameter_bytes_resident(self) -> int:
        """Bytes of full (gathered) parameters alive right now (the shards are not counted)."""
        return sum(u.full.numel() * u.full.element_size() for u in self.units if u.full is not None)

    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> None:
        lr = self.lr if lr is None else lr
        for u in self.units:            # units whose backward never completed (unused parameters) are flushed here
            if u.full is not None and u.pending != 0 and any(p.grad is not None for p in u.params):
                u.reduce_grads()
            elif u.full is not None and not torch.is_grad_enabled():
                u.release()
        dev = self.units[0].device
        sq = torch.zeros((), device=dev, dtype=torch.float32)
        for u in self.units:
            if u.grad_shard is not None:
                sq += u.grad_shard.float().pow(2).sum()
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        gscale = 1.0 / self.dp_size
        self._norm = sq.sqrt() * gscale
        scale = gscale
        if self.max_grad_norm > 0:
            scale = scale * float(torch.clamp(self.max_grad_norm / (self._norm + 1e-6), max=1.0))
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        fused = (not self.offload) and dev.type == "cuda" and _lib.kernels_available()
        for u in self.units:
            if u.grad_shard is None:
                continue
            st = self.state[u.name]
            if fused:       # the flat fused AdamW kernel of the ZeRO-2 optimizer, one launch per decay class
                from ..ops import cuda_ops
                lo = u.rank * u.shard_len
                cut = min(max(u.n_decay - lo, 0), u.shard_len)
                for a, b_, wd in ((0, cut, self.weight_decay), (cut, u.shard_len, 0.0)):
                    if b_ > a:
                        cuda_ops.adamw_step(u.shard[a:b_], u.grad_shard[a:b_], st["m"][a:b_], st["v"][a:b_], lr=lr,
                                            beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd, step=self.step_count,
                                            master=st["master"][a:b_], norm_sq=sq, max_norm=self.max_grad_norm,
                                            grad_scale=gscale)
                u.grad_shard = None
                continue
            m, v, master = (st[k].to(u.device, non_blocking=True) if self.offload else st[k] for k in ("m", "v", "master"))
            g = u.grad_shard.float() * scale
            mf = m.float().mul_(b1).add_(g, alpha=1 - b1)
            vf = v.float().mul_(b2).addcmul_(g, g, value=1 - b2)
            # decayed tensors come first in the flat layout; this shard covers [lo, lo + shard_len)
            lo = u.rank * u.shard_len
            cut = min(max(u.n_decay - lo, 0), u.shard_len)
            upd = (mf / bc1) / ((vf / bc2).sqrt() + self.eps)
            pf = master.float()
            if cut > 0 and self.weight_decay:
                pf[:cut].mul_(1 - lr * self.weight_decay)
            pf.add_(upd, alpha=-lr)
            u.shard.copy_(pf)
            for k, t in (("m", mf), ("v", vf), ("master", pf)):
                st[k].copy_(t, non_blocking=self.offload)
            u.grad_shard = None
        if self.offload and torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    # -- whole-model access (checkpoint save / load) -----------------------------------------------------
    def gather_full_state(self) -> None:
        """Materialises every unit (e.g. before ``save_pretrained``); ``release_all`` undoes it."""
        for u in self.units:
            u.materialize()

    def release_all(self) -> None:
        for u in self.units:
            u.release()

    def reshard_from_full(self) -> None:
        """After weights were copied into the materialised parameters (``gather_full_state`` + a checkpoint load):
        re-slices every unit's shard and fp32 master copy from them."""
        for u in self.units:
            assert u.full is not None, "reshard_from_full needs gather_full_state() first"
            lo = u.rank * u.shard_len if u.world > 1 else 0
            u.shard.copy_(u.full[lo:lo + u.shard_len])
            st = self.state.get(u.name)
            if st is not None and st.get("master") is not None:
                st["master"].copy_(u.shard.detach().float())

    def state_dict(self) -> dict:
        return {"step": self.step_count, "rank": self.rank, "world": self.world,
                "shards": {u.name: u.shard.detach().cpu() for u in self.units},
                "state": {n: {k: t.detach().cpu() for k, t in s.items()} for n, s in self.state.items()}}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "ZeRO-3 shards are tied to (rank, world)"
        self.step_count = sd["step"]
        for u in self.units:
            u.shard.copy_(sd["shards"][u.name])
            for k, t in sd["state"][u.name].items():
                self.state[u.name][k].copy_(t)
