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


def _prefs(tmp_path, stage):
    rows = ([{"instruction": f"question number {i} " * 6, "chosen": "a good and long answer " * 8, "rejected": "bad " * 5}
             for i in range(8)] if stage in ("dpo", "rm") else
            [{"instruction": f"q{i} " * 10, "output": "answer " * 12, "kto_tag": i % 2 == 0} for i in range(8)])
    (tmp_path / "dataset_info.json").write_text(json.dumps({"d": {"file_name": "d.json", "ranking": stage in ("dpo", "rm")}}))
    (tmp_path / "d.json").write_text(json.dumps(rows))


@pytest.mark.parametrize("stage", ["dpo", "rm", "kto"])
def test_preference_stages(tmp_path, stage):
    _prefs(tmp_path, stage)
    tr, _ = _run(tmp_path, stage, stage=stage, synthetic=False, dataset="d", dataset_dir=str(tmp_path), template="default",
                 cutoff_len=384, per_device_train_batch_size=2)
    assert tr.global_step == 2


def test_ppo_stage(tmp_path):
    _run(tmp_path, "rm_ckpt", stage="pt", max_steps=1, cutoff_len=256)
    base = {"model_name_or_path": json.dumps(SMALL), "synthetic": True, "cutoff_len": 64, "bf16": True, "pure_bf16": True,
            "learning_rate": 1e-4, "lr_scheduler_type": "constant", "per_device_train_batch_size": 2}
    tr = run_exp(dict(base, stage="ppo", max_steps=2, output_dir=str(tmp_path / "ppo"),
                      reward_model=os.path.join(str(tmp_path / "rm_ckpt"), "final"), ppo_epochs=1, ppo_max_new_tokens=4,
                      ppo_prompt_len=16))
    assert len(tr.stats) == 2 and all(v == v for v in tr.stats[-1].values())


@pytest.mark.parametrize("extra", [{"use_muon": True}, {"use_galore": True, "galore_rank": 16}, {"use_adam_mini": True},
                                   {"deepspeed": "z3"}, {"finetuning_type": "oft", "lora_target": "q_proj,o_proj",
                                                         "oft_block_size": 32}],
                         ids=["muon", "galore", "adam_mini", "zero3", "oft"])
def test_optimizer_options(tmp_path, extra):
    extra = dict(extra)
    if extra.get("deepspeed") == "z3":
        js = tmp_path / "ds_z3.json"
        js.write_text(json.dumps({"zero_optimization": {"stage": 3}}))
        extra["deepspeed"] = str(js)
    tr, _ = _run(tmp_path, "opt", stage="pt", max_steps=3, **extra)
    assert tr.global_step == 3


def test_neat_packing_and_prediction(tmp_path):
    data = tmp_path / "data"
    data.mkdir()
    recs = [{"instruction": f"say {i} " * (3 + i), "input": "", "output": f"{i} " * (5 + 2 * i)} for i in range(12)]
    (data / "toy.json").write_text(json.dumps(recs))
    (data / "dataset_info.json").write_text(json.dumps({"toy": {"file_name": "toy.json"}}))
    common = dict(synthetic=False, dataset="toy", dataset_dir=str(data), template="default")
    tr, _ = _run(tmp_path, "pack", stage="sft", cutoff_len=256, packing=True, neat_packing=True, **common)
    assert tr.global_step == 2
    out = str(tmp_path / "pred")
    run_exp({"model_name_or_path": os.path.join(str(tmp_path / "pack"), "final"), "stage": "sft", "do_train": False,
             "do_predict": True, "eval_dataset": "toy", "dataset_dir": str(data), "template": "default", "cutoff_len": 128,
             "max_new_tokens": 8, "do_sample": False, "output_dir": out, "bf16": True, "pure_bf16": True})
    assert os.path.exists(os.path.join(out, "generated_predictions.jsonl"))
