"""Expert-parallel load balancing: hot experts get replicas, and the physical copies are packed onto the ranks so
that every rank sees about the same number of routed tokens.

* ``balance(load, num_physical, num_ranks)`` -> ``EPLBPlan``: replicas are handed out greedily to the expert with the
  largest load per replica; the physical copies are then placed longest-first onto the least-loaded rank that still has
  a free slot (every rank holds ``num_physical / num_ranks`` slots).
* ``remap(indices, plan)``: logical routing ids -> physical slot ids; a token picks among an expert's replicas by its
  position, so the split is even and needs no communication.
* ``shard_experts_balanced(block, ep, plan)``: each rank keeps the weights of the physical slots placed on it; from
  then on the ordinary expert-parallel paths (``parallel/ep.py``, ``parallel/ep_fused.py``) run unchanged on physical
  ids.  ``LoadTracker`` accumulates the routing counts a new plan is computed from.

Reference: the serving side relies on vLLM's expert-parallel load balancer for its MoE models
(``vllm-inference/src/primed_vllm/models/hybridqwen3_moe.py``, ``enable_eplb``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch


@dataclass
class EPLBPlan:
    phys2log: torch.Tensor        # [P] logical expert held by each physical slot; slot p lives on rank p // (P / ranks)
    log2phys: torch.Tensor        # [E, max_replicas] physical slots of each expert, padded with -1
    replicas: torch.Tensor        # [E] number of physical copies
    num_ranks: int

    @property
    def slots_per_rank(self) -> int:
        return self.phys2log.numel() // self.num_ranks

    def rank_load(self, load: torch.Tensor) -> torch.Tensor:
        """Tokens each rank receives under this plan for the logical ``load [E]``."""
        per_copy = load.double() / self.replicas.double()
        out = torch.zeros(self.num_ranks, dtype=torch.float64)
        out.index_add_(0, torch.arange(self.phys2log.numel()) // self.slots_per_rank, per_copy[self.phys2log])
        return out


def balance(load: torch.Tensor, num_physical: int, num_ranks: int) -> EPLBPlan:
    load = load.detach().double().cpu().clamp_min(0)
    E = load.numel()
    if num_physical < E or num_physical % num_ranks:
        raise ValueError(f"{num_physical} physical slots: need at least {E} and a multiple of {num_ranks} ranks")
    reps = torch.ones(E, dtype=torch.long)
    for _ in range(num_physical - E):                     # the next replica goes where a copy carries the most
        reps[int(torch.argmax(load / reps))] += 1
    copies = [(float(load[e] / reps[e]), e) for e in range(E) for _ in range(int(reps[e]))]
    copies.sort(key=lambda c: (-c[0], c[1]))
    per = num_physical // num_ranks
    rank_slots: List[List[int]] = [[] for _ in range(num_ranks)]
    rank_load = [0.0] * num_ranks
    for w, e in copies:
        # least-loaded rank with a free slot; among equals prefer one that does not hold this expert yet
        cands = [r for r in range(num_ranks) if len(rank_slots[r]) < per]
        r = min(cands, key=lambda r: (rank_load[r], e in rank_slots[r], r))
        rank_slots[r].append(e)
        rank_load[r] += w
    phys2log = torch.tensor([e for slots in rank_slots for e in slots], dtype=torch.long)
    max_rep = int(reps.max())
    log2phys = torch.full((E, max_rep), -1, dtype=torch.long)
    fill = [0] * E
    for p, e in enumerate(phys2log.tolist()):
        log2phys[e, fill[e]] = p
        fill[e] += 1
    return EPLBPlan(phys2log, log2phys, reps, num_ranks)


def identity_plan(num_experts: int, num_ranks: int) -> EPLBPlan:
    return EPLBPlan(torch.arange(num_experts), torch.arange(num_experts)[:, None].clone(),
                    torch.ones(num_experts, dtype=torch.long), num_ranks)


def remap(indices: torch.Tensor, plan: EPLBPlan) -> torch.Tensor:
    """``indices [T, k]`` logical -> physical.  Replica choice: ``(token + column) mod replicas``."""
    dev = indices.device
    T, k = indices.shape
    reps = plan.replicas.to(dev)[indices]
    pick = (torch.arange(T, device=dev)[:, None] + torch.arange(k, device=dev)[None]) % reps
    return plan.log2phys.to(dev)[indices, pick]


def shard_experts_balanced(moe_block, ep, plan: EPLBPlan) -> None:
    """Keeps the weights of this rank's physical slots (from the FULL, unsharded expert weights) and makes the block
    route on physical ids."""
    per = plan.slots_per_rank
    mine = plan.phys2log[ep.rank * per:(ep.rank + 1) * per].to(moe_block.experts.gate_up_proj.device)
    moe_block.experts.gate_up_proj.data = moe_block.experts.gate_up_proj.data[mine].contiguous()
    moe_block.experts.down_proj.data = moe_block.experts.down_proj.data[mine].contiguous()
    moe_block.expert_parallel_group = ep
    moe_block.num_local_experts = per
    moe_block.eplb_plan = plan


class LoadTracker:
    """Running count of routed tokens per expert (one row per MoE layer)."""

    def __init__(self, num_layers: int, num_experts: int):
        self.counts = torch.zeros(num_layers, num_experts, dtype=torch.float64)

    def update(self, layer: int, indices: torch.Tensor) -> None:
        self.counts[layer] += torch.bincount(indices.reshape(-1).cpu(), minlength=self.counts.shape[1]).double()

    def plans(self, num_physical: int, num_ranks: int) -> List[EPLBPlan]:
        return [balance(row, num_physical, num_ranks) for row in self.counts]
