"""The training workflows end to end on a GPU, in bf16 and at kernel-sized shapes (head dimension 128): pre-training
with resume, stage-1 distillation of a fused model, LoRA / DoRA fine-tuning, preference training, fp8 linears.  Each
run is a few steps of a small model; the point is that every stage reaches the native kernels without tripping."""
import json
import os

import pytest
import torch

from hybrid_model_factory_b200.train.workflow import run_exp

pytestmark = pytest.mark.gpu

SMALL = {"model_type": "hybrid_qwen3", "vocab_size": 512, "hidden_size": 512, "intermediate_size": 1024,
         "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
         "hybrid_override_pattern": "*-GDN", "torch_dtype": "bfloat16"}


def _launches():
    from hybrid_model_factory_b200.ops import _lib
    return _lib.launch_count()


def _run(tmp_path, name, model=None, **cfg):
    base = {"model_name_or_path": json.dumps(model or SMALL), "synthetic": True, "cutoff_len": 512, "max_steps": 2,
            "output_dir": str(tmp_path / name), "bf16": True, "pure_bf16": True, "learning_rate": 1e-3,
            "lr_scheduler_type": "constant", "per_device_train_batch_size": 1, "logging_steps": 1}
    base.update(cfg)
    before = _launches()
    tr = run_exp(base)
    torch.cuda.synchronize()
    from hybrid_model_factory_b200.ops import _lib
    _lib.assert_status_ok()
    assert _launches() > before, "no native kernel ran"
    log = [json.loads(l) for l in open(os.path.join(base["output_dir"], "trainer_log.jsonl"))]
    assert log and all(l["loss"] == l["loss"] for l in log), log          # finite losses
    return tr, log


@pytest.mark.parametrize("pattern", ["*-GDN", "M2-GKA", "SWA-*"])
def test_pretraining_steps_and_resume(tmp_path, pattern):
    model = dict(SMALL, hybrid_override_pattern=pattern, swa_config={"window_size": 128})
    tr, _ = _run(tmp_path, "pt", model, stage="pt", max_steps=3, save_steps=2)
    assert tr.global_step == 3 and tr.unchecked_layers == [0, 1]           # both layers fit: no recompute after step 1
    tr2, _ = _run(tmp_path, "pt", model, stage="pt", max_steps=4, save_steps=2,
                  model_name_or_path=os.path.join(str(tmp_path / "pt"), "checkpoint-2"))
    assert tr2.global_step == 4


@pytest.mark.parametrize("pattern,learn", [("*DA-GDN*", "gdn"), ("GKA*-*DA", "gka"), ("M2*-*DA", "mamba")])
def test_stage1_distillation_of_a_fused_model(tmp_path, pattern, learn):
    tr, log = _run(tmp_path, "hkd", dict(SMALL, hybrid_override_pattern=pattern), stage="hkd",
                   hybrid_learnable_params=learn, hybrid_lw_distill_target="all", learning_rate=1e-2)
    names = [n for n, p in tr.model.named_parameters() if p.requires_grad]
    assert names and log[0]["loss"] > 0


def test_sft_with_dora_adapters_and_dft_loss(tmp_path):
    data = tmp_path / "data"
    data.mkdir()
    recs = [{"instruction": f"say {i} " * 20, "input": "", "output": f"{i} " * 40} for i in range(8)]
    (data / "toy.json").write_text(json.dumps(recs))
    (data / "dataset_info.json").write_text(json.dumps({"toy": {"file_name": "toy.json"}}))
    tr, _ = _run(tmp_path, "sft", stage="sft", synthetic=False, dataset="toy", dataset_dir=str(data), template="default",
                 cutoff_len=256, finetuning_type="lora", lora_rank=8, use_dora=True, use_dft_loss=True)
    # the adapters are folded back into the weights when the run ends: the saved model has the ordinary layout
    assert not any("lora_" in n or n.endswith("magnitude") for n, _ in tr.model.named_parameters())
    from hybrid_model_factory_b200.utils import checkpoint_io
    assert checkpoint_io.from_pretrained(os.path.join(str(tmp_path / "sft"), "final"), device="cuda") is not None


def test_fp8_linears_train(tmp_path):
    tr, log = _run(tmp_path, "fp8", dict(SMALL, num_hidden_layers=4, hybrid_override_pattern="*-GDN-*-GDN"), stage="pt",
                   fp8=True, max_steps=3)
    assert tr.global_step == 3
