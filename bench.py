"""Headline benchmark: training tokens/s of GDN-primed Qwen3-8B (36 layers, every other layer Gated
DeltaNet) at 128K context, bf16 AdamW, sequence parallelism over all N GPUs (SP = N, batch 1,
synthetic uniform-random token ids, random-init weights).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

ONE timed region of K optimizer steps through ``Trainer.train_step``, the call a user of the
framework makes.  Every step copies its inputs from pinned host memory to the device and reads the
loss back to the host.  The region is bracketed twice: by CUDA events on the launching stream
(``value``, maximum over ranks) and by the host clock around synchronised boundaries (``e2e``).
The process keeps to a wall-clock budget (``--time-budget`` seconds, default 780): when the warm-up
steps show that K steps would not fit, fewer steps are timed and the line says so (``steps`` is the
number actually timed, ``steps_requested`` what was asked).
``--impl reference`` runs (or reports why it cannot run) the unmodified reference project.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
T_START = time.perf_counter()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=int(os.environ.get("HMF_BENCH_SEQ_LEN", 131072)))
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--pattern", default="*-GDN")
    ap.add_argument("--ref-child", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--time-budget", type=float, default=float(os.environ.get("HMF_BENCH_BUDGET_S", 780)),
                    help="wall-clock seconds the whole process may take; fewer steps are timed if K would not fit")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.proc, self.idx = None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_reference(args):
    """Runs the reference arm in a child process per rank, so that a crash inside one of its native dependencies
    (which ends the process, not a Python exception) still yields the one-line ``unavailable`` report."""
    rank0 = int(os.environ.get("RANK", "0")) == 0
    if not args.ref_child:
        cmd = [sys.executable, os.path.abspath(__file__), "--ref-child"] + sys.argv[1:]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        line = next((ln for ln in reversed(proc.stdout.splitlines()) if ln.startswith("{")), None)
        if rank0:
            if line is not None:
                print(line, flush=True)
            else:
                err = [ln for ln in proc.stderr.splitlines() if "rror" in ln and not ln.startswith("frame")]
                why = (err[-1] if err else proc.stderr[-300:]).strip()
                print(json.dumps({"impl": "reference", "n_gpus": args.gpus,
                                  "unavailable": f"reference process ended with code {proc.returncode}: {why[:500]}"}),
                      flush=True)
            sys.stderr.write(proc.stderr[-4000:])
        return
    from baseline.reference_arm import run as run_ref
    out = run_ref(args, ClockSampler, T_START)
    if rank0:
        print(json.dumps(out), flush=True)
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    import torch
    import torch.distributed as dist

    from hybrid_model_factory_b200.models.configuration import qwen3_8b_config
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.ops import _lib
    from hybrid_model_factory_b200.parallel.sp import zigzag_split
    from hybrid_model_factory_b200.train.trainer import Trainer, TrainingArguments

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)

    S, sp = args.seq_len, world
    cfg = qwen3_8b_config(args.pattern, num_hidden_layers=args.layers, max_position_embeddings=max(S, 40960))
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = build_model(cfg)
    torch.set_default_dtype(torch.float32)
    model = model.to(torch.bfloat16)
    targs = TrainingArguments(output_dir="", learning_rate=1e-5, max_steps=10 ** 6, warmup_steps=0,
                              lr_scheduler_type="constant", sequence_parallel_size=sp, max_grad_norm=1.0,
                              logging_steps=0)
    trainer = Trainer(model, targs, device=dev)

    def make_batch(seed: int, pinned: bool):
        g = torch.Generator().manual_seed(1000 + seed)
        ids = torch.randint(0, cfg.vocab_size, (1, S), generator=g)
        labels = torch.roll(ids, -1, dims=1)
        labels[:, -1] = -100
        pos = torch.arange(S)[None]
        if sp > 1:
            ids, labels, pos = (zigzag_split(t, rank, sp).contiguous() for t in (ids, labels, pos))
        b = {"input_ids": ids, "labels": labels, "position_ids": pos}
        if pinned:
            b = {k: v.pin_memory() for k, v in b.items()}
        b["labels_shifted"] = True
        return b

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fit_steps(sec_per_step: float, done_s: float) -> int:
        """Number of timed steps that fit what is left of the wall-clock budget (same answer on every rank)."""
        left = args.time_budget - done_s - 20.0                 # 20 s for the report and the teardown
        n = max(1, min(args.steps, int(left / max(sec_per_step, 1e-6))))
        t = torch.tensor([n], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return int(t)

    from hybrid_model_factory_b200.utils import profiling
    n_batches = 4                                               # distinct pinned batches, cycled
    batches = [make_batch(i, True) for i in range(n_batches)]
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values() if hasattr(v, "numel"))
    warm_t0 = time.perf_counter()
    for i in range(args.warmup):
        float(trainer.train_step(batches[i % n_batches]).item())
    sync()
    warm_s = (time.perf_counter() - warm_t0) / max(args.warmup, 1)
    transport = "none" if trainer.sp is None else type(trainer.sp.transport).__name__
    if world > 1:
        # a device-side wait of the peer-memory state chain that ran out leaves a status code: fall back to the NCCL
        # transport on every rank and warm up again, so that the timed steps are valid either way
        code = torch.tensor([_lib.read_status(reset=True)[0]], device=dev)
        dist.all_reduce(code, op=dist.ReduceOp.MAX)
        if int(code) != 0 and trainer.sp is not None:
            from hybrid_model_factory_b200.parallel.sp import StateTransport
            trainer.sp.transport = StateTransport(trainer.sp.group, trainer.sp.ranks)
            transport = "StateTransport (peer chain reported a timeout during warm-up)"
            for i in range(args.warmup):
                float(trainer.train_step(batches[i % n_batches]).item())
            sync()
    steps = fit_steps(warm_s, time.perf_counter() - T_START)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    profiling.enable_phases(True)
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t0 = time.perf_counter()
    ev0.record()
    last = 0.0
    for i in range(steps):
        last = float(trainer.train_step(batches[i % n_batches]).item())   # H2D of the inputs, D2H of the loss
    ev1.record()
    sync()
    host_s = time.perf_counter() - t0
    ms = ev0.elapsed_time(ev1)
    launches = _lib.launch_count() - launches0
    t = torch.tensor([ms, host_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t[0]) / steps
    e2e = {"value": S * steps / float(t[1]), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4, "last_loss": last,
           "note": "same steps as `value`; host clock around synchronised boundaries, max over ranks"}
    phases = {k: round(v["total_ms"] / steps, 3) for k, v in profiling.PHASES.summary().items()}
    profiling.enable_phases(False)
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.read_status()
    if rank == 0:
        value = S / (ms_per_step / 1e3)
        out = {"metric": "train tok/s (128K ctx, SP 1/2/4/8)", "value": value, "unit": "tokens/s", "n_gpus": world,
               "steps": steps, "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
               "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
               "config": {"model": f"GDN-primed Qwen3-8B ({args.layers} layers, pattern {args.pattern} tiled, hidden 4096, "
                                   "SwiGLU 12288, 32/8 heads x 128, vocab 151936)",
                          "global_batch": 1, "seq_len": S, "parallelism": f"sp{world}",
                          "optimizer": "AdamW bf16 states, ZeRO-sharded over all ranks, grad clip 1.0",
                          "activation_checkpointing": (
                              f"per layer; {len(trainer.unchecked_layers)} of {args.layers} layers keep their "
                              "activations instead (they fit in the memory left free after the first step)"),
                          "sp_state_transport": transport,
                          "l2": "working set per step far exceeds the 126 MB L2 (no flush needed)"},
               "memory_gib": {"peak_allocated": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
                              "peak_reserved": round(torch.cuda.max_memory_reserved() / 2 ** 30, 1)},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "phase_ms_per_step": phases, "kernel_status": list(status),
               "impl": "ours"}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
