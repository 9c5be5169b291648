"""Ray launch of a training run (``ray: true`` / ``USE_RAY=1``): one Ray actor per rank, placed by a placement group
with one GPU bundle per worker, each running the ordinary training workflow under a ``torch.distributed``
rendezvous that the driver hands out (reference: ``train/tuner.py:203-291``, ``train/trainer_utils.py:869-953``).

The driver
  1. connects to (or starts) Ray and checks that the cluster has ``ray_num_workers`` GPUs;
  2. reserves a placement group (``PACK`` by default: fill nodes, so sequence-parallel groups of consecutive ranks
     share NVLink) and orders its bundles so that rank 0 lives on the node of ``master_addr``;
  3. starts one actor per bundle with ``RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT`` in its
     environment and calls ``run_exp(config)`` on all of them; the first failure is re-raised on the driver.
Ray is imported lazily: the module loads (and its planning helpers are testable) without it.
"""
from __future__ import annotations

import os
import socket
from typing import Any, Dict, List, Optional


def find_available_port() -> int:
    with socket.socket() as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def worker_env(rank: int, world: int, master_addr: str, master_port: int, base: Optional[Dict[str, str]] = None) -> Dict[str, str]:
    env = dict(base or {})
    env.update({"RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": master_addr,
                "MASTER_PORT": str(master_port), "LOCAL_RANK": "0", "LOCAL_WORLD_SIZE": "1"})
    return env


def order_bundles(bundle_nodes: List[str], master_addr: Optional[str]) -> List[int]:
    """Bundle indices in rank order: bundles on the master's node first, then node by node (ranks that share a node
    are consecutive)."""
    nodes: List[str] = []
    for n in bundle_nodes:
        if n not in nodes:
            nodes.append(n)
    if master_addr in nodes:
        nodes.remove(master_addr)
        nodes.insert(0, master_addr)
    return [i for n in nodes for i, b in enumerate(bundle_nodes) if b == n]


class RayWorker:
    """Body of the Ray actor: fixes the visible device, then runs the training workflow of this process' rank."""

    def __init__(self, env: Dict[str, str]):
        os.environ.update(env)
        try:
            import ray
            ids = ray.get_runtime_context().get_accelerator_ids().get("GPU", [])
            if os.environ.get("RAY_EXPERIMENTAL_NOSET_CUDA_VISIBLE_DEVICES") and ids:
                os.environ["LOCAL_RANK"] = str(ids[0])     # Ray left every GPU visible: pick the assigned one
        except Exception:
            pass

    def node_ip(self) -> str:
        import ray
        return ray.util.get_node_ip_address()

    def train(self, config: Any):
        from .train.workflow import run_exp
        tr = run_exp(config)
        return {"global_step": int(tr.global_step), "rank": int(os.environ.get("RANK", "0"))}


def launch(config: Any, num_workers: int, master_addr: Optional[str] = None, master_port: Optional[int] = None,
           resources_per_worker: Optional[Dict[str, float]] = None, placement_strategy: str = "PACK",
           ray_init_kwargs: Optional[dict] = None) -> List[dict]:
    import ray
    from ray.util.placement_group import placement_group
    from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy
    if not ray.is_initialized():
        ray.init(**(ray_init_kwargs or {}))
    total = int(ray.cluster_resources().get("GPU", 0))
    if num_workers > total:
        raise ValueError(f"the Ray cluster has {total} GPUs, fewer than ray_num_workers={num_workers}")
    bundle = dict(resources_per_worker or {"GPU": 1, "CPU": 8})
    pg = placement_group([dict(bundle) for _ in range(num_workers)], strategy=placement_strategy)
    ray.get(pg.ready())
    Actor = ray.remote(RayWorker)

    def start(idx: int, env: Dict[str, str]):
        return Actor.options(num_cpus=bundle.get("CPU", 1), num_gpus=bundle.get("GPU", 0),
                             scheduling_strategy=PlacementGroupSchedulingStrategy(
                                 placement_group=pg, placement_group_bundle_index=idx)).remote(env)
    # first pass: one probe actor per bundle tells where the bundle landed
    probes = [start(i, {}) for i in range(num_workers)]
    nodes = ray.get([p.node_ip.remote() for p in probes])
    for p in probes:
        ray.kill(p)
    if master_addr is not None and master_addr not in nodes:
        raise ValueError(f"master_addr {master_addr} is not a node of the placement group ({sorted(set(nodes))})")
    order = order_bundles(nodes, master_addr)
    addr = master_addr or nodes[order[0]]
    port = int(master_port or find_available_port())
    base = {k: v for k, v in os.environ.items() if k.startswith(("HMF_", "NCCL_", "CUDA_", "TORCH_", "RECORD_VRAM"))}
    workers = [start(order[r], worker_env(r, num_workers, addr, port, base)) for r in range(num_workers)]
    try:
        return ray.get([w.train.remote(config) for w in workers])
    finally:
        ray.shutdown()
