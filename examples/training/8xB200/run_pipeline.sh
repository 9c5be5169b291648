#!/bin/bash
# Priming pipeline on one node with 8 B200 GPUs: stage 0 (Transformer -> fused hybrid), stage 1 (layer-wise
# distillation, 8K context), unfuse, stage 2 (long-context training at 128K with 8-way sequence parallelism).
# Run from the repository root after `python -c "import __graft_entry__ as g; g.build()"` (builds the CUDA libraries
# in-tree).  To resume, comment out the stages that have finished.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")/../../.."
EX=examples/priming
TOK=examples/tokenization

# stage 0: weight surgery, a few minutes on the CPU
python -m hybrid_model_factory_b200.cli prime-init $EX/stage0/qwen3_8b_gdn.yaml

# 8K pre-training data for stage 1 (restartable: finished shards are skipped)
python -m hybrid_model_factory_b200.cli preprocess --config $TOK/sft.yaml --num-shards 64 --workers 32

# stage 1: only the student mixers train; 8 data-parallel ranks, optimizer state sharded over them
python -m hybrid_model_factory_b200.cli train $EX/stage1/hqwen3_8b_gdn.yaml

# fused two-stream checkpoint -> standard hybrid layout
python -m hybrid_model_factory_b200.cli prime-unfuse ./models/qwen3_8b_gdn-fused/stage1/final ./models/hqwen3_8b_gdn

# 128K blocks, written directly in the zig-zag layout of 8-way sequence parallelism
python -m hybrid_model_factory_b200.cli preprocess --config $TOK/pretraining_sp.yaml --num-shards 64 --workers 32

# stage 2: long-context training, one 128K sample per step split over the 8 GPUs
python -m hybrid_model_factory_b200.cli train $EX/stage2/hqwen3_8b_gdn_long_ctx.yaml

echo "stage 0 (fused):      ./models/qwen3_8b_gdn-fused"
echo "stage 1 (distilled):  ./models/hqwen3_8b_gdn"
echo "stage 2 (long ctx):   see output_dir of $EX/stage2/hqwen3_8b_gdn_long_ctx.yaml"
echo "serve it:             python -m hybrid_model_factory_b200.cli serve <stage-2 dir>/final --tp 8"
