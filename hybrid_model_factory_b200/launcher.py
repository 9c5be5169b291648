"""Command dispatch and multi-process launch.

``hmf train cfg.yaml`` re-executes itself under ``torch.distributed.run`` when more than one GPU is
visible (or ``FORCE_TORCHRUN=1``), with static rendezvous from ``MASTER_ADDR`` / ``MASTER_PORT`` /
``NNODES`` / ``NODE_RANK`` / ``NPROC_PER_NODE`` or elastic c10d rendezvous when ``RDZV_ID`` is set
(``MAX_RESTARTS``, ``MIN_NNODES``, ``MAX_NNODES``).  Reference: ``launcher.py:41-259``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from typing import List

VERSION = "0.1.0"

USAGE = """usage: hmf <command> [args]

  prime-init CONFIG.yaml         stage 0: initialise a hybrid (or L2A) model from a Transformer checkpoint
  prime-unfuse CKPT [OUT]        convert a fused stage-1 checkpoint to the standard hybrid layout
  select-layers rank CSV --M N | variants SRC DST   which layers to replace: ranking from per-layer benchmark
                                 scores, or one sliding-window variant of the checkpoint per layer
  reassemble-vlm TEXT_CKPT VL_CKPT OUT   put a distilled text backbone back into its VL wrapper
  convert-qwen-gdn SRC OUT [--pattern P] convert a Qwen3-Next / Qwen3.5-MoE checkpoint to the hybrid layout
  train CONFIG.yaml [k=v ...]    run a training stage (pt | sft | hkd | dpo | kto | rm)
  train-multinode CONFIG.yaml    same, expecting NNODES / NODE_RANK / MASTER_ADDR in the environment
                                 (USE_RAY=1: Ray actors instead of torchrun; USE_V1=1: the second-generation SFT stack)
  preprocess --config CFG.yaml   tokenise (and SP-split) datasets into `tokenized_path`, sharded and parallel
  eval CKPT --task T_split ...   multiple-choice benchmark evaluation (few-shot, accuracy per category)
  export CKPT OUT [--dtype D] [--merge-lora] [--quantize int8|int4|gptq|awq] [--ollama]
                                 re-shard / cast a checkpoint, fold adapters in, quantise, write an Ollama Modelfile
  serve CKPT [--tp N --port P] [--draft-model D]
                                 OpenAI-compatible server on the native engine (--tp N: tensor parallel over N GPUs)
  api CKPT                       alias of serve
  chat CKPT                      interactive chat in the terminal
  bench-serve CKPT|CONFIG ...    serving benchmark (continuous batching workload)
  env                            print the environment
  version                        print the version
"""


def _visible_gpus() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def torchrun_command(script_args: List[str]) -> List[str]:
    nproc = int(os.environ.get("NPROC_PER_NODE", str(max(1, _visible_gpus()))))
    nnodes = os.environ.get("NNODES", "1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", str(nproc)]
    if os.environ.get("RDZV_ID"):
        lo, hi = os.environ.get("MIN_NNODES", nnodes), os.environ.get("MAX_NNODES", nnodes)
        cmd += ["--nnodes", f"{lo}:{hi}", "--rdzv-id", os.environ["RDZV_ID"], "--rdzv-backend", "c10d",
                "--rdzv-endpoint", f"{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{os.environ.get('MASTER_PORT', '29500')}",
                "--max-restarts", os.environ.get("MAX_RESTARTS", "0")]
    else:
        cmd += ["--nnodes", nnodes, "--node-rank", os.environ.get("NODE_RANK", "0"),
                "--master-addr", os.environ.get("MASTER_ADDR", "127.0.0.1"),
                "--master-port", os.environ.get("MASTER_PORT", "29500")]
    return cmd + ["-m", "hybrid_model_factory_b200.launcher", "--worker", "train"] + script_args


def serve_command(tp: int, server_args: List[str]) -> List[str]:
    """torchrun command line of a tensor-parallel server on this node (rank 0 serves HTTP, the others follow)."""
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes", "1", "--nproc-per-node", str(tp),
            "--master-addr", os.environ.get("MASTER_ADDR", "127.0.0.1"),
            "--master-port", os.environ.get("MASTER_PORT", "29500"),
            "-m", "hybrid_model_factory_b200.serving.api_server"] + list(server_args)


def launch(argv: List[str]) -> int:
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(USAGE)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "version":
        print(f"hybrid-model-factory (B200 native) {VERSION}")
        return 0
    if cmd == "env":
        from .utils.env import print_env
        print_env()
        return 0
    if cmd == "prime-init":
        from .priming.hybridize_model import main as prime_main
        prime_main(rest[0])
        return 0
    if cmd == "prime-unfuse":
        from .priming.fused_to_standard import unfuse_checkpoint
        print(unfuse_checkpoint(rest[0], rest[1] if len(rest) > 1 else None))
        return 0
    if cmd == "convert-qwen-gdn":
        from .priming.convert_qwen_gdn import main as convert_main
        return convert_main(rest)
    if cmd == "select-layers":
        from .priming.layer_selection import main as select_main
        return select_main(rest)
    if cmd == "reassemble-vlm":
        from .priming.reassemble_vlm import reassemble_vlm
        reassemble_vlm(rest[0], rest[1], rest[2])
        return 0
    if cmd == "train" and os.environ.get("USE_V1", "0") == "1":
        # the second-generation stack (data engine, resumable batch generator, token-weighted trainer)
        from .v1.launcher import main as v1_main
        return v1_main(rest)
    if cmd in ("train", "train-multinode") and os.environ.get("USE_RAY", "0") == "1":
        # Ray placement-group launch: one actor per GPU (RAY_NUM_WORKERS, default: every GPU of the cluster)
        from .launcher_ray import launch as ray_launch
        n = int(os.environ.get("RAY_NUM_WORKERS", "0")) or max(1, _visible_gpus())
        ray_launch(rest, n, os.environ.get("MASTER_ADDR"), int(os.environ["MASTER_PORT"]) if "MASTER_PORT" in os.environ else None)
        return 0
    if cmd in ("train", "train-multinode"):
        multi = (_visible_gpus() > 1 or os.environ.get("FORCE_TORCHRUN", "0") == "1" or cmd == "train-multinode")
        if multi and "WORLD_SIZE" not in os.environ:
            return subprocess.call(torchrun_command(rest))
        from .train.workflow import run_exp
        run_exp(rest)
        return 0
    if cmd == "preprocess":
        from .data.sharded_preprocess import main as prep_main
        return prep_main(rest)
    if cmd == "eval":
        from .train.evaluate import main as eval_main
        return eval_main(rest)
    if cmd == "export":
        from .utils.export import main as export_main
        return export_main(rest)
    if cmd in ("serve", "api"):
        if "--tp" in rest and "WORLD_SIZE" not in os.environ:       # tensor parallel: one process per GPU under torchrun
            i = rest.index("--tp")
            tp, rest = int(rest[i + 1]), rest[:i] + rest[i + 2:]
            if tp > 1:
                return subprocess.call(serve_command(tp, rest))
        from .serving.api_server import main as serve_main
        return serve_main(rest)
    if cmd == "chat":
        from .serving.chat import main as chat_main
        return chat_main(rest)
    if cmd == "bench-serve":
        from .serving.bench_serve import main as bench_main
        return bench_main(rest)
    print(f"unknown command '{cmd}'\n\n{USAGE}")
    return 2


def main() -> None:
    argv = sys.argv[1:]
    if argv[:2] == ["--worker", "train"]:
        from .train.workflow import run_exp
        run_exp(argv[2:])
        return
    sys.exit(launch(argv))


if __name__ == "__main__":
    main()
