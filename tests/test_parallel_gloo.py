"""Expert, Ulysses and pipeline parallelism and the mesh layout on CPU ranks (gloo)."""
import copy

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks
from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import SparseMoeBlock, build_model
from hybrid_model_factory_b200.parallel import mesh


def test_mesh_coordinates_and_groups():
    dims = mesh.MeshDims(pp=2, dp=2, sp=2, tp=2)
    assert mesh.coords(13, dims) == {"pp": 1, "dp": 1, "sp": 0, "tp": 1}
    tp_groups = mesh.group_ranks(dims, "tp")
    assert [0, 1] in tp_groups and len(tp_groups) == 8
    assert [0, 2] in mesh.group_ranks(dims, "sp") and [0, 8] in mesh.group_ranks(dims, "pp")
    all_ranks = sorted(r for g in mesh.group_ranks(dims, "dp") for r in g)
    assert all_ranks == list(range(16))


def _moe_cfg():
    return HybridConfig("hybrid_qwen3_moe", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                        num_attention_heads=2, num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2,
                        moe_intermediate_size=16, hybrid_override_pattern="*")


def _ep_worker(rank, world):
    from hybrid_model_factory_b200.parallel.ep import EPContext, shard_experts
    torch.manual_seed(0)
    ref = SparseMoeBlock(_moe_cfg())
    blk = copy.deepcopy(ref)
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(6 + rank, 32, generator=g)          # different token counts per rank
    xr = x.clone().requires_grad_(True)
    out_ref, _ = ref(xr)
    out_ref.sum().backward()
    shard_experts(blk, EPContext.from_group(None))
    xe = x.clone().requires_grad_(True)
    out, _ = blk(xe)
    out.sum().backward()
    assert torch.allclose(out, out_ref, atol=1e-5)
    assert torch.allclose(xe.grad, xr.grad, atol=1e-5)
    # expert weight gradients: each rank holds the gradient of its experts from all ranks' tokens
    full = ref.experts.down_proj.grad.clone()
    dist.all_reduce(full)
    per = 4 // world
    assert torch.allclose(blk.experts.down_proj.grad, full[rank * per:(rank + 1) * per], atol=1e-5)


def test_expert_parallel_matches_local_experts():
    run_ranks(_ep_worker, 2)


def _eplb_worker(rank, world):
    """Skewed routing: the hot expert is replicated, the ranks' loads even out, the output does not change."""
    from hybrid_model_factory_b200.parallel.ep import EPContext
    from hybrid_model_factory_b200.parallel.eplb import balance, shard_experts_balanced
    torch.manual_seed(0)
    ref = SparseMoeBlock(_moe_cfg())
    blk = copy.deepcopy(ref)
    g = torch.Generator().manual_seed(20 + rank)
    x = torch.randn(9, 32, generator=g)
    out_ref, _ = ref(x)
    plan = balance(torch.tensor([100.0, 5.0, 5.0, 10.0]), num_physical=6, num_ranks=world)
    shard_experts_balanced(blk, EPContext.from_group(None), plan)
    assert blk.experts.gate_up_proj.shape[0] == 3
    out, _ = blk(x)
    assert torch.allclose(out, out_ref, atol=1e-5)


def test_expert_load_balancer():
    from hybrid_model_factory_b200.parallel.eplb import LoadTracker, balance, identity_plan, remap
    load = torch.tensor([100.0, 5.0, 5.0, 10.0, 40.0, 0.0, 20.0, 20.0])
    plan = balance(load, num_physical=12, num_ranks=4)
    assert plan.replicas.sum() == 12 and plan.replicas[0] >= 3 and plan.replicas[5] == 1
    assert sorted(plan.phys2log.tolist()) == sorted(sum(([e] * int(r) for e, r in enumerate(plan.replicas)), []))
    before = identity_plan(8, 4).rank_load(load)
    after = plan.rank_load(load)
    assert after.max() < 0.6 * before.max() and abs(after.sum() - load.sum()) < 1e-6
    idx = torch.randint(0, 8, (64, 2))
    phys = remap(idx, plan)
    assert torch.equal(plan.phys2log[phys], idx)                       # every physical id serves the routed expert
    hot = phys[idx == 0]
    assert len(set(hot.tolist())) == int(plan.replicas[0])             # all replicas of the hot expert are used
    tr = LoadTracker(2, 8)
    tr.update(0, idx)
    tr.update(1, torch.zeros(10, 2, dtype=torch.long))
    plans = tr.plans(12, 4)
    assert plans[1].replicas[0] == 5                                   # all spare slots go to the only busy expert
    run_ranks(_eplb_worker, 2)


def _ulysses_worker(rank, world):
    from hybrid_model_factory_b200.ops import reference as R
    from hybrid_model_factory_b200.parallel.sp import init_sp_group, zigzag_split
    from hybrid_model_factory_b200.parallel.ulysses import ulysses_attention
    g = torch.Generator().manual_seed(0)
    B, T, H, Hkv, D = 2, 32, 4, 2, 8
    q, k, v = torch.randn(B, T, H, D, generator=g), torch.randn(B, T, Hkv, D, generator=g), torch.randn(B, T, Hkv, D, generator=g)
    do = torch.randn(B, T, H, D, generator=g)
    full = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o_ref = R.attention(*full, causal=True)
    o_ref.backward(do)
    sp = init_sp_group(world)
    loc = [zigzag_split(t, rank, world).clone().requires_grad_(True) for t in (q, k, v)]
    o = ulysses_attention(*loc, sp)
    o.backward(zigzag_split(do, rank, world))
    assert torch.allclose(o, zigzag_split(o_ref, rank, world), atol=1e-5)
    for a, b in zip(loc, full):
        assert torch.allclose(a.grad, zigzag_split(b.grad, rank, world), atol=1e-5)


def test_ulysses_attention_matches_single_rank():
    run_ranks(_ulysses_worker, 2)


def _pp_worker(rank, world):
    from hybrid_model_factory_b200.parallel.pp import PipelineStage, partition_layers
    assert partition_layers(5, 2) == [(0, 3), (3, 5)]
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=4,
                       num_attention_heads=2, num_key_value_heads=2, head_dim=16, hybrid_override_pattern="*-GDN-M2-*")
    model = build_model(cfg).eval()
    ids = torch.randint(0, 64, (1, 9), generator=torch.Generator().manual_seed(3))
    ref = model.generate(ids, max_new_tokens=5)[:, 9:]
    stage = PipelineStage(model)
    out = stage.generate(ids, max_new_tokens=5)
    assert torch.equal(out, ref), (rank, out, ref)


def test_pipeline_parallel_generation_matches_single_rank():
    run_ranks(_pp_worker, 2)


# -- ZeRO-3 ---------------------------------------------------------------------------------------------------------
def _zero3_worker(rank, world, offload, checkpointing, mics=0):
    import copy
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.train.zero3 import Zero3Engine, mics_groups
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN-M2")
    model = build_model(cfg)
    ref = copy.deepcopy(model)
    if checkpointing:
        model.gradient_checkpointing_enable()
    total = sum(p.numel() for p in model.parameters())
    groups = {}
    if mics:
        shard_group, replica_group = mics_groups(mics)
        groups = dict(group=shard_group, replica_group=replica_group)
    eng = Zero3Engine(model, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, offload_optimizer=offload, **groups)
    if mics:
        assert eng.world == mics and eng.dp_size == world
    assert eng.parameter_bytes_resident() == 0 and all(p.numel() == 0 for p in model.parameters())
    decay = [p for p in ref.parameters() if p.dim() >= 2 and not getattr(p, "_no_weight_decay", False)]
    rest = [p for p in ref.parameters() if not (p.dim() >= 2 and not getattr(p, "_no_weight_decay", False))]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}], lr=1e-2)
    g = torch.Generator().manual_seed(1)
    peak = 0
    for step in range(3):
        ids = torch.randint(0, 64, (2 * world, 12), generator=g)
        # reference: the whole batch on one process
        opt.zero_grad()
        ref.train()
        ref(input_ids=ids, labels=ids).loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        # ZeRO-3: every rank takes its slice of the batch
        eng.zero_grad()
        model.train()
        mine = ids[rank * 2:(rank + 1) * 2]
        loss = model(input_ids=mine, labels=mine).loss
        peak = max(peak, eng.parameter_bytes_resident())
        loss.backward()
        assert eng.parameter_bytes_resident() == 0           # every unit was reduced and released
        eng.step()
    if checkpointing:       # never more than the outer unit plus one layer at a time
        assert peak < total * 4 * 0.8, (peak, total * 4)
    eng.gather_full_state()
    for (n, p), q in zip(model.named_parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=2e-4, rtol=1e-3), (n, float((p - q).abs().max()))
    eng.release_all()
    sd = eng.state_dict()
    eng.load_state_dict(sd)
    assert sd["step"] == 3


@pytest.mark.parametrize("offload,checkpointing", [(False, True), (True, True), (False, False)])
def test_zero3_matches_single_process_adamw(offload, checkpointing):
    run_ranks(_zero3_worker, 2, offload, checkpointing)


def test_zero3_mics_shards_inside_groups_of_two():
    """Four ranks, parameters sharded over pairs and replicated across the two pairs (MiCS)."""
    run_ranks(_zero3_worker, 4, False, True, 2)


def _sp_workflow_worker(rank, world, out_dir, ref_losses):
    """`hmf train` with sequence_parallel_size = world: every rank takes its zig-zag share of each sample; the logged
    losses equal the single-process run of the same configuration."""
    import json
    import os
    from hybrid_model_factory_b200.train.workflow import run_exp
    tiny = {"model_type": "hybrid_qwen3", "vocab_size": 259, "hidden_size": 32, "intermediate_size": 64,
            "num_hidden_layers": 3, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
            "hybrid_override_pattern": "*-GDN-M2", "torch_dtype": "float32"}
    cfg = {"model_name_or_path": json.dumps(tiny), "stage": "pt", "synthetic": True, "cutoff_len": 64, "max_steps": 3,
           "output_dir": os.path.join(out_dir, "sp"), "bf16": False, "pure_bf16": False, "learning_rate": 1e-3,
           "lr_scheduler_type": "constant", "per_device_train_batch_size": 1, "sequence_parallel_size": world,
           "logging_steps": 1, "seed": 7}
    tr = run_exp(cfg)
    assert tr.global_step == 3 and tr.sp is not None and tr.sp.size == world
    if rank == 0:
        log = [json.loads(l)["loss"] for l in open(os.path.join(out_dir, "sp", "trainer_log.jsonl"))]
        assert all(abs(a - b) < 2e-3 for a, b in zip(log, ref_losses)), (log, ref_losses)


def test_training_workflow_under_sequence_parallelism(tmp_path):
    import json
    import os
    from hybrid_model_factory_b200.train.workflow import run_exp
    tiny = {"model_type": "hybrid_qwen3", "vocab_size": 259, "hidden_size": 32, "intermediate_size": 64,
            "num_hidden_layers": 3, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
            "hybrid_override_pattern": "*-GDN-M2", "torch_dtype": "float32"}
    cfg = {"model_name_or_path": json.dumps(tiny), "stage": "pt", "synthetic": True, "cutoff_len": 64, "max_steps": 3,
           "output_dir": str(tmp_path / "one"), "bf16": False, "pure_bf16": False, "learning_rate": 1e-3,
           "lr_scheduler_type": "constant", "per_device_train_batch_size": 1, "logging_steps": 1, "seed": 7}
    run_exp(cfg)
    ref = [json.loads(l)["loss"] for l in open(os.path.join(str(tmp_path / "one"), "trainer_log.jsonl"))]
    run_ranks(_sp_workflow_worker, 2, str(tmp_path), ref)
