"""Reference arm of ``bench.py``: trains the reference project's own ``HybridQwen3ForCausalLM`` on the headline
configuration (GDN-primed Qwen3-8B, 128K tokens, bf16 AdamW, sequence parallelism over all ranks) and prints
the same JSON line as the repo's arm.

What runs is the reference's code, unmodified, imported from ``baseline/_ref/hmf`` (a plain copy of its
``training/src/hmf`` tree; the package is pure Python, so the copy is the install):

* model: ``hmf.model.hybrid_zoo.models.hybrid_qwen3`` (``modeling_hybrid_qwen3.py:1328``) with the
  ``*-GDN`` pattern; Gated DeltaNet through ``fla`` (``layers/gated_deltanet/gdn.py:463-473``), softmax
  attention through flash-attn 2;
* one GPU: ``attn_implementation="flash_attention_2"`` and the reference's liger patch
  (``hybrid_qwen3/liger_kernel_patch.py:33-85``: fused linear + cross entropy, RMSNorm, RoPE, SwiGLU), without
  which the 128K x 151936 logits do not fit;
* several GPUs: ``apply_sequence_parallel`` (``model/model_utils/sequence_parallel.py:145-204``, zig-zag ring
  attention), the zig-zag gather / scatter path of its GDN layer, its sequence-parallel data split
  (``data/data_utils.py::preprocess_sp_dataset``) and its sequence-parallel loss (``train/pt/trainer.py:162-195``);
* gradient checkpointing per decoder layer (the model's own ``gradient_checkpointing_enable``), as in the repo's arm.

What is replaced, because the packages are absent offline: the HF ``Trainer`` + DeepSpeed ZeRO-2 engine.  The arm
runs the same sequence by hand: forward, loss, backward, a SUM all-reduce of the bf16 gradients over all ranks
(what ZeRO-2's reduce-scatter + all-gather moves), gradient clipping at 1.0, fused ``torch.optim.AdamW`` on bf16
parameters.  Packages the reference imports at module top but never executes on this path are registered as empty
stand-ins (listed in the output under ``stubs``); nothing under ``baseline/_ref`` is edited.
"""
from __future__ import annotations

import importlib.machinery
import os
import shutil
import sys
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(ROOT, "_ref")
REF_SRC = os.environ.get("HMF_REFERENCE_SRC", "/root/reference/training/src/hmf")


def ensure_installed() -> str:
    """Copies the reference's Python package next to this file if it is not there yet; returns '' or the reason
    it could not."""
    dst = os.path.join(REF_DIR, "hmf")
    if os.path.isdir(dst):
        return ""
    if not os.path.isdir(REF_SRC):
        return f"reference source not found at {REF_SRC} and no copy under baseline/_ref"
    os.makedirs(REF_DIR, exist_ok=True)
    shutil.copytree(REF_SRC, dst)
    return ""


class _Empty(types.ModuleType):
    def __getattr__(self, key):
        if key.startswith("__"):
            raise AttributeError(key)
        return None


def _stub(name: str, package: bool) -> None:
    m = _Empty(name)
    if package:
        m.__path__ = []
    m.__spec__ = importlib.machinery.ModuleSpec(name, None, is_package=package)
    sys.modules[name] = m


def install_shims() -> list:
    """Makes the reference's model code importable on this image.  Returns what was stubbed or shimmed."""
    notes = []
    # The reference pins flash-linear-attention 0.4.1, whose gated delta rule is Triton only.  The 0.5.1 on this image
    # routes the backward through a TileLang kernel by default on sm_90 and later; switch that backend off (the
    # library's own variable) so that the Triton path the reference was written against runs.
    if os.environ.setdefault("FLA_TILELANG", "0") == "0":
        notes.append("FLA_TILELANG=0 (fla 0.5.1 TileLang backend off: reference pins fla 0.4.1, Triton)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import liger_kernel.transformers.monkey_patch  # noqa: F401  (before the peft stand-in, so liger sees no peft)
    # hmf/model/__init__.py imports the loader, which pulls peft / trl / accelerate / omegaconf; the model classes
    # do not need it.  Register the package without running its __init__.
    pkg = types.ModuleType("hmf.model")
    pkg.__path__ = [os.path.join(REF_DIR, "hmf", "model")]
    pkg.__spec__ = importlib.machinery.ModuleSpec("hmf.model", None, is_package=True)
    pkg.__spec__.submodule_search_locations = pkg.__path__
    sys.modules["hmf.model"] = pkg
    notes.append("hmf.model.__init__ (loader: peft/trl/accelerate/omegaconf) not executed")
    for name, is_pkg in [("deepspeed", True), ("mamba_ssm", True), ("mamba_ssm.ops", True),
                         ("mamba_ssm.ops.triton", True), ("mamba_ssm.ops.triton.layernorm_gated", False),
                         ("mamba_ssm.ops.triton.ssd_combined", False),
                         ("mamba_ssm.ops.triton.selective_state_update", False), ("yunchang", True),
                         ("yunchang.kernels", False), ("peft", True), ("peft.utils", False)]:
        try:
            __import__(name)
        except Exception:
            _stub(name, is_pkg)
            notes.append(name)
    # transformers 5.5 (this image) validates layer_types against a fixed list; the reference (written for 5.3)
    # stores its pattern symbols there
    import transformers.configuration_utils as cu
    cu.ALLOWED_LAYER_TYPES = tuple(cu.ALLOWED_LAYER_TYPES) + ("*", "GDN", "GKA", "M2", "BMF", "SWA")
    notes.append("transformers ALLOWED_LAYER_TYPES extended with the pattern symbols")
    # ring_flash_attn's HF adapter imports a name transformers 5.5 no longer has
    import transformers.modeling_flash_attention_utils as mfu
    if not hasattr(mfu, "is_flash_attn_greater_or_equal_2_10"):
        mfu.is_flash_attn_greater_or_equal_2_10 = lambda: True
        notes.append("transformers.modeling_flash_attention_utils.is_flash_attn_greater_or_equal_2_10 shim")
    return notes


def _reference_config(args, seq_len: int):
    from hmf.model.hybrid_zoo.models.hybrid_qwen3.configuration_hybrid_qwen3 import HybridQwen3Config
    syms = args.pattern.split("-")
    pattern = "-".join(syms[i % len(syms)] for i in range(args.layers))
    return HybridQwen3Config(
        vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=args.layers,
        num_attention_heads=32, num_key_value_heads=8, head_dim=128, hidden_act="silu",
        max_position_embeddings=max(seq_len, 40960), rms_norm_eps=1e-6, use_cache=False, tie_word_embeddings=False,
        rope_parameters={"rope_type": "default", "rope_theta": 1000000.0}, attention_bias=False,
        hybrid_override_pattern=pattern)


def _run(args, clock_sampler_cls, t_start: float) -> dict:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    stubs = install_shims()
    import hmf  # noqa: F401
    from hmf.model.hybrid_zoo.models.hybrid_qwen3.modeling_hybrid_qwen3 import HybridQwen3ForCausalLM

    S, sp = args.seq_len, world
    torch.manual_seed(0)
    cfg = _reference_config(args, S)
    group = None
    if sp > 1:
        from hmf.model.model_utils.sequence_parallel import apply_sequence_parallel
        margs = types.SimpleNamespace(sequence_parallel_size=sp, sequence_parallel_mode="zigzag-ring")
        group = apply_sequence_parallel(margs)
        attn_impl = "sequence_parallel_attention"
    else:
        attn_impl = "flash_attention_2"
    liger = sp == 1
    if liger:
        # class-level patch before the model is built, as the reference's loader does (model/loader.py, liger_kernel.py)
        from hmf.model.hybrid_zoo.models.hybrid_qwen3.liger_kernel_patch import apply_liger_kernel_to_hybridqwen3
        apply_liger_kernel_to_hybridqwen3(rope=True, cross_entropy=False, fused_linear_cross_entropy=True,
                                          rms_norm=True, swiglu=True)
    with torch.device(dev):
        model = HybridQwen3ForCausalLM._from_config(cfg, attn_implementation=attn_impl, dtype=torch.bfloat16)
    model = model.to(dev).to(torch.bfloat16)
    model.sequence_parallel_group = group

    def set_group(module):                     # train/pt/workflow.py:35-39
        module.sequence_parallel_group = group
        for child in module.children():
            set_group(child)
    set_group(model)
    model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": True})
    model.config.use_cache = False
    model.train()
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=1e-5, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, fused=True)

    def make_batch(seed: int):
        g = torch.Generator().manual_seed(1000 + seed)
        ids = torch.randint(0, cfg.vocab_size, (S,), generator=g)
        if sp == 1:
            b = {"input_ids": ids[None].clone(), "labels": ids[None].clone()}
        else:
            from hmf.data.data_utils import preprocess_sp_dataset
            labels = torch.cat([ids[1:], torch.tensor([-100])])          # shifted before the split (sequence_parallel.py)
            pos = torch.arange(S)
            pick = lambda t: torch.as_tensor(preprocess_sp_dataset(t.tolist(), sp, "zigzag-ring")[rank])[None]
            b = {"input_ids": pick(ids), "labels": pick(labels), "position_ids": pick(pos)}
        return {k: v.pin_memory() for k, v in b.items()}

    loss_fct = torch.nn.CrossEntropyLoss(reduction="sum")

    def train_step(batch) -> float:
        inputs = {k: v.to(dev, non_blocking=True) for k, v in batch.items()}
        opt.zero_grad(set_to_none=True)
        if sp == 1:
            loss = model(**inputs, use_cache=False).loss
        else:                                   # train/pt/trainer.py:162-195
            out = model(**inputs, use_cache=False)
            logits = out["logits"]
            labels = inputs["labels"].view(-1)
            loss = loss_fct(logits.view(-1, logits.shape[-1]), labels)
            dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
            n = (labels != -100).sum()
            dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
            loss = loss / n
        loss.backward()
        if world > 1:
            grads = [p.grad for p in params if p.grad is not None]
            for i in range(0, len(grads), 64):
                flat = torch.cat([g.reshape(-1) for g in grads[i:i + 64]])
                dist.all_reduce(flat)
                off = 0
                for g in grads[i:i + 64]:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
        torch.nn.utils.clip_grad_norm_(params, 1.0, foreach=True)
        opt.step()
        return float(loss.item())

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_batches = 4
    batches = [make_batch(i) for i in range(n_batches)]
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())
    if sp > 1:                                  # train/pt/trainer.py:151-159: one no-grad forward before the first step
        model.eval()
        with torch.no_grad():
            model(**{k: v.to(dev) for k, v in batches[0].items()}, use_cache=False)
        model.train()
    w0 = time.perf_counter()
    for i in range(args.warmup):
        train_step(batches[i % n_batches])
    sync()
    warm_s = (time.perf_counter() - w0) / max(args.warmup, 1)
    left = args.time_budget - (time.perf_counter() - t_start) - 20.0
    steps_t = torch.tensor([max(1, min(args.steps, int(left / max(warm_s, 1e-6))))], device=dev)
    if world > 1:
        dist.all_reduce(steps_t, op=dist.ReduceOp.MIN)
    steps = int(steps_t)
    sampler = clock_sampler_cls(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t0 = time.perf_counter()
    ev0.record()
    last = 0.0
    for i in range(steps):
        last = train_step(batches[i % n_batches])
    ev1.record()
    sync()
    host_s = time.perf_counter() - t0
    t = torch.tensor([ev0.elapsed_time(ev1), host_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = float(t[0]) / steps
    out = {"impl": "reference", "metric": "train tok/s (128K ctx, SP 1/2/4/8)", "value": S / (ms_per_step / 1e3),
           "unit": "tokens/s", "n_gpus": world, "steps": steps, "steps_requested": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
           "config": {"model": f"reference HybridQwen3ForCausalLM ({args.layers} layers, pattern {args.pattern} tiled, "
                               "hidden 4096, SwiGLU 12288, 32/8 heads x 128, vocab 151936)",
                      "global_batch": 1, "seq_len": S, "parallelism": f"sp{world}", "same_config": True,
                      "attention": attn_impl, "liger_kernel": liger, "activation_checkpointing": "per layer",
                      "optimizer_note": "fused torch AdamW on bf16 parameters, bf16 gradient all-reduce over all ranks, "
                                        "clip 1.0 (stands in for DeepSpeed ZeRO-2, which is not installed)",
                      "stubs": stubs, "l2": "working set per step far exceeds the 126 MB L2 (no flush needed)"},
           "clocks": clocks,
           "e2e": {"value": S * steps / float(t[1]), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": 4, "last_loss": last},
           "gpu_launches": 0}
    return out


def run(args, clock_sampler_cls, t_start: float) -> dict:
    """Returns the JSON-able result of the reference run, or ``{"unavailable": why}``."""
    base = {"impl": "reference", "n_gpus": args.gpus}
    why = ensure_installed()
    if why:
        base["unavailable"] = why
        return base
    try:
        return _run(args, clock_sampler_cls, t_start)
    except BaseException as e:  # noqa: BLE001  (an out-of-memory error at one N must not lose the line)
        if isinstance(e, KeyboardInterrupt):
            raise
        msg = f"{type(e).__name__}: {e}".replace("\n", " ")
        base["unavailable"] = f"reference run failed at N={args.gpus}: {msg[:600]}"
        return base
