"""End-to-end training workflows on CPU with tiny models: config parsing, data pipeline, pt / sft / hkd
stages, checkpoint save + auto-resume."""
import json
import os

import pytest
import torch

from hybrid_model_factory_b200.config.parser import get_train_args, read_args
from hybrid_model_factory_b200.data import loader as L
from hybrid_model_factory_b200.data.formats import ByteTokenizer, get_template
from hybrid_model_factory_b200.train.workflow import run_exp

TINY = {"model_type": "hybrid_qwen3", "vocab_size": 259, "hidden_size": 32, "intermediate_size": 64,
        "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
        "hybrid_override_pattern": "*-GDN", "torch_dtype": "float32"}


def test_read_args_overrides(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text("stage: pt\nlearning_rate: 1.0e-4\nsynthetic: true\nmax_steps: 3\n")
    d = read_args([str(p), "learning_rate=5e-5", "--cutoff_len", "64", "bf16=false", "pure_bf16=false"])
    assert d["learning_rate"] == 5e-5 and d["cutoff_len"] == 64 and d["stage"] == "pt"
    with pytest.raises(ValueError):
        get_train_args({"stage": "nope", "synthetic": True, "max_steps": 1})
    with pytest.raises(ValueError):
        get_train_args({"stage": "pt", "synthetic": True, "max_steps": 1, "bogus_key": 1})


def test_sp_split_and_processors():
    tok = ByteTokenizer()
    rows = L.process_pretrain([{"text": "hello world " * 20}], tok, 32)
    assert all(len(r["input_ids"]) == 32 for r in rows) and len(rows) >= 7
    sup = L.process_supervised([{"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}],
                                 "system": ""}], tok, get_template("default"), 64)
    assert sup[0]["labels"].count(-100) > 0 and sup[0]["labels"][-1] == tok.eos_token_id
    row = {"input_ids": list(range(16)), "labels": list(range(16)), "position_ids": list(range(16))}
    shards = L.sp_split(L.shift_labels(row), 2)
    assert shards[0]["input_ids"] == [0, 1, 2, 3, 12, 13, 14, 15] and shards[1]["position_ids"] == [4, 5, 6, 7, 8, 9, 10, 11]
    assert shards[0]["labels"][:4] == [1, 2, 3, 4] and shards[0]["labels"][-1] == -100
    packed = L.pack_supervised(sup * 3, 64, 0)
    assert len(packed) <= 3 and len(packed[0]["input_ids"]) == 64


def test_pt_train_save_resume(tmp_path):
    out = str(tmp_path / "run")
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "pt", "synthetic": True, "cutoff_len": 32,
           "max_steps": 4, "save_steps": 2, "output_dir": out, "bf16": False, "pure_bf16": False,
           "learning_rate": 1e-3, "lr_scheduler_type": "constant", "per_device_train_batch_size": 2}
    tr = run_exp(cfg)
    assert tr.global_step == 4
    log = [json.loads(l) for l in open(os.path.join(out, "trainer_log.jsonl"))]
    assert len(log) == 4 and log[-1]["loss"] < log[0]["loss"] + 0.5
    assert os.path.exists(os.path.join(out, "checkpoint-4", "model.safetensors"))
    assert os.path.exists(os.path.join(out, "final", "config.json"))
    # auto-resume: the same output dir continues from the last checkpoint
    cfg2 = dict(cfg, max_steps=6, model_name_or_path=os.path.join(out, "checkpoint-4"))
    tr2 = run_exp(cfg2)
    assert tr2.global_step == 6


def test_sft_on_json_dataset(tmp_path):
    data = tmp_path / "data"
    data.mkdir()
    recs = [{"instruction": f"say {i}", "input": "", "output": f"{i} " * 3} for i in range(16)]
    (data / "toy.json").write_text(json.dumps(recs))
    (data / "dataset_info.json").write_text(json.dumps({"toy": {"file_name": "toy.json"}}))
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "sft", "dataset": "toy", "dataset_dir": str(data),
           "cutoff_len": 48, "max_steps": 3, "output_dir": str(tmp_path / "sft"), "bf16": False, "pure_bf16": False,
           "per_device_train_batch_size": 2, "template": "default"}
    tr = run_exp(cfg)
    assert tr.global_step == 3


def test_hkd_stage_only_student_trains(tmp_path):
    fused = dict(TINY, hybrid_override_pattern="*DA-GDN*")
    cfg = {"model_name_or_path": json.dumps(fused), "stage": "hkd", "synthetic": True, "cutoff_len": 32, "max_steps": 2,
           "output_dir": str(tmp_path / "hkd"), "bf16": False, "pure_bf16": False, "hybrid_learnable_params": "gdn",
           "hybrid_lw_distill_target": "all", "learning_rate": 1e-2, "lr_scheduler_type": "constant"}
    tr = run_exp(cfg)
    names = [n for n, p in tr.model.named_parameters() if p.requires_grad]
    assert names and all("gdn" in n for n in names)
    log = [json.loads(l) for l in open(os.path.join(str(tmp_path / "hkd"), "trainer_log.jsonl"))]
    assert log[0]["loss"] > 0


def test_zero_config_reads_deepspeed_style_json(tmp_path):
    import json
    from hybrid_model_factory_b200.train.workflow import zero_config
    p = tmp_path / "ds_z3_offload.json"
    p.write_text(json.dumps({"zero_optimization": {"stage": 3, "offload_optimizer": {"device": "cpu"}}}))
    assert zero_config(str(p)) == {"zero_stage": 3, "offload_optimizer": True}
    p.write_text(json.dumps({"zero_optimization": {"stage": 2}}))
    assert zero_config(str(p)) == {"zero_stage": 2, "offload_optimizer": False}
    assert zero_config(None) == {}


def test_preference_feedback_and_tool_data_processing(tmp_path):
    import json
    import torch
    from hybrid_model_factory_b200.config.hparams import DataArguments
    from hybrid_model_factory_b200.data.formats import ByteTokenizer, DatasetAttr, convert_alpaca, convert_sharegpt, get_template
    from hybrid_model_factory_b200.data.loader import (IGNORE_INDEX, collate, get_dataset, process_feedback,
                                                       process_pairwise, process_unsupervised)
    tok, tpl = ByteTokenizer(), get_template("qwen3")
    pair = convert_alpaca({"instruction": "2+2?", "chosen": "4", "rejected": "five"}, DatasetAttr("p", "p", ranking=True))
    assert pair["chosen"]["content"] == "4" and pair["messages"][-1]["role"] == "user"
    rows = process_pairwise([pair], tok, tpl, 256)
    r = rows[0]
    assert r["chosen_input_ids"][:10] == r["rejected_input_ids"][:10]                       # the shared prompt
    n_prompt = sum(l == IGNORE_INDEX for l in r["chosen_labels"])
    assert bytes(r["chosen_labels"][n_prompt:n_prompt + 1]) == b"4"
    assert sum(l != IGNORE_INDEX for l in r["rejected_labels"]) > sum(l != IGNORE_INDEX for l in r["chosen_labels"])
    b = collate(rows * 2, pad_id=0)
    assert set(b) == {"chosen_input_ids", "chosen_labels", "rejected_input_ids", "rejected_labels"}
    assert b["chosen_input_ids"].shape[0] == 2 and b["rejected_labels"].dtype == torch.long
    fb = convert_alpaca({"instruction": "hi", "output": "yo", "kto_tag": False}, DatasetAttr("k", "k"))
    rows = process_feedback([fb], tok, tpl, 128)
    assert rows[0]["kto_tags"] == 0 and collate(rows)["kto_tags"].tolist() == [0]
    # tool calls: function / observation turns, tool list in the system prompt
    conv = convert_sharegpt({"conversations": [
        {"from": "human", "value": "weather in Paris?"},
        {"from": "function_call", "value": json.dumps({"name": "get_weather", "arguments": {"city": "Paris"}})},
        {"from": "observation", "value": json.dumps({"temp": 21})},
        {"from": "gpt", "value": "21 degrees."}], "tools": json.dumps([{"name": "get_weather"}])}, DatasetAttr("t", "t", "sharegpt"))
    assert [m["role"] for m in conv["messages"]] == ["user", "function", "observation", "assistant"]
    msgs, system = tpl.normalise(conv["messages"], "", conv["tools"])
    assert [m["role"] for m in msgs] == ["user", "assistant", "user", "assistant"]
    assert "<tool_call>" in msgs[1]["content"] and "<tool_response>" in msgs[2]["content"] and "<tools>" in system
    text = bytes(t for p, r_ in tpl.encode_multiturn(tok, conv["messages"]) for t in p + r_).decode()
    assert "<tool_call>" in text and "get_weather" in text
    un = process_unsupervised([conv], tok, tpl, 512)[0]
    assert bytes(un["labels"]).decode().startswith("21 degrees.")
    # end to end through get_dataset with a ranking dataset from dataset_info.json
    (tmp_path / "dataset_info.json").write_text(json.dumps({"prefs": {"file_name": "prefs.json", "ranking": True}}))
    (tmp_path / "prefs.json").write_text(json.dumps([{"instruction": f"q{i}", "chosen": "good", "rejected": "bad"}
                                                     for i in range(4)]))
    ds = get_dataset(DataArguments(dataset="prefs", dataset_dir=str(tmp_path), template="qwen3", cutoff_len=128), tok,
                     stage="dpo")
    assert len(ds) == 4 and "rejected_labels" in ds[0]


@pytest.mark.parametrize("extra", [
    {"use_galore": True, "galore_rank": 4, "galore_update_interval": 2},
    {"use_adam_mini": True},
    {"finetuning_type": "oft", "lora_target": "q_proj,o_proj", "oft_block_size": 16},
    {"deepspeed": "z3"},
    {"finetuning_type": "lora", "lora_rank": 4, "quantization_bit": 4, "neftune_noise_alpha": 5.0,
     "report_to": "tensorboard", "logging_steps": 1},
    {"mixture_of_depths": "convert", "mod_capacity": 0.5},
])
def test_training_options_run_end_to_end(tmp_path, extra):
    """`hmf train` configurations beyond the default optimizer: each runs a few steps, lowers the loss and saves a
    loadable final checkpoint."""
    from hybrid_model_factory_b200.utils import checkpoint_io
    out = str(tmp_path / "run")
    extra = dict(extra)
    if extra.get("deepspeed") == "z3":
        js = tmp_path / "ds_z3.json"
        js.write_text(json.dumps({"zero_optimization": {"stage": 3}}))
        extra["deepspeed"] = str(js)
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "pt", "synthetic": True, "cutoff_len": 32,
           "max_steps": 6, "output_dir": out, "bf16": False, "pure_bf16": False, "learning_rate": 3e-3,
           "lr_scheduler_type": "constant", "per_device_train_batch_size": 2, **extra}
    tr = run_exp(cfg)
    assert tr.global_step == 6
    log = [json.loads(l) for l in open(os.path.join(out, "trainer_log.jsonl"))]
    assert log[-1]["loss"] < log[0]["loss"] + 0.2, [r["loss"] for r in log]
    model = checkpoint_io.from_pretrained(os.path.join(out, "final"))
    assert all(p.numel() > 0 and torch.isfinite(p).all() for p in model.parameters())
    assert not any("oft" in n or "lora" in n for n, _ in model.named_parameters())
    assert not any("qweight" in n for n in model.state_dict())
    if extra.get("report_to") == "tensorboard":
        from hybrid_model_factory_b200.utils.tensorboard_writer import read_scalars
        runs = os.path.join(out, "runs")
        scalars = list(read_scalars(os.path.join(runs, os.listdir(runs)[0])))
        assert sum(t == "train/loss" for t, _, _ in scalars) == 6
    if extra.get("mixture_of_depths"):
        assert hasattr(model.model.layers[1], "mod_router")


def test_dpo_stage_on_a_ranking_dataset(tmp_path):
    (tmp_path / "dataset_info.json").write_text(json.dumps({"prefs": {"file_name": "prefs.json", "ranking": True}}))
    (tmp_path / "prefs.json").write_text(json.dumps(
        [{"instruction": f"question {i}", "chosen": "a good answer", "rejected": "bad"} for i in range(8)]))
    out = str(tmp_path / "run")
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "dpo", "dataset": "prefs", "dataset_dir": str(tmp_path),
           "template": "qwen3", "cutoff_len": 96, "max_steps": 3, "output_dir": out, "bf16": False, "pure_bf16": False,
           "learning_rate": 1e-3, "lr_scheduler_type": "constant", "per_device_train_batch_size": 2}
    tr = run_exp(cfg)
    assert tr.global_step == 3
    log = [json.loads(l) for l in open(os.path.join(out, "trainer_log.jsonl"))]
    assert all(torch.isfinite(torch.tensor(r["loss"])) for r in log)


@pytest.mark.parametrize("stage", ["rm", "kto"])
def test_rm_and_kto_stages(tmp_path, stage):
    rows = ([{"instruction": f"q{i}", "chosen": "good answer", "rejected": "bad"} for i in range(8)] if stage == "rm" else
            [{"instruction": f"q{i}", "output": "answer", "kto_tag": i % 2 == 0} for i in range(8)])
    (tmp_path / "dataset_info.json").write_text(json.dumps({"d": {"file_name": "d.json", "ranking": stage == "rm"}}))
    (tmp_path / "d.json").write_text(json.dumps(rows))
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": stage, "dataset": "d", "dataset_dir": str(tmp_path),
           "template": "qwen3", "cutoff_len": 96, "max_steps": 2, "output_dir": str(tmp_path / "run"), "bf16": False,
           "pure_bf16": False, "learning_rate": 1e-3, "lr_scheduler_type": "constant", "per_device_train_batch_size": 2}
    assert run_exp(cfg).global_step == 2


def test_ppo_stage_with_a_reward_model_checkpoint(tmp_path):
    rm_out, ppo_out = str(tmp_path / "rm"), str(tmp_path / "ppo")
    base = {"model_name_or_path": json.dumps(TINY), "synthetic": True, "cutoff_len": 24, "bf16": False, "pure_bf16": False,
            "learning_rate": 1e-3, "lr_scheduler_type": "constant", "per_device_train_batch_size": 2}
    run_exp(dict(base, stage="pt", max_steps=1, output_dir=rm_out))          # any checkpoint serves as the scorer here
    tr = run_exp(dict(base, stage="ppo", max_steps=2, output_dir=ppo_out, reward_model=os.path.join(rm_out, "final"),
                      ppo_epochs=1, ppo_max_new_tokens=4, ppo_prompt_len=8))
    assert len(tr.stats) == 2 and {"score", "kl", "policy_loss"} <= set(tr.stats[-1])
    assert os.path.exists(os.path.join(ppo_out, "final", "value_head.pt"))


def test_launcher_commands_and_torchrun_command(tmp_path, monkeypatch, capsys):
    from hybrid_model_factory_b200 import launcher
    assert launcher.launch(["version"]) == 0 and "B200" in capsys.readouterr().out
    assert launcher.launch(["env"]) == 0 and "torch" in capsys.readouterr().out.lower()
    assert launcher.launch(["no-such-command"]) == 2
    monkeypatch.setenv("NPROC_PER_NODE", "4")
    monkeypatch.setenv("MASTER_PORT", "29611")
    cmd = launcher.torchrun_command(["cfg.yaml"])
    assert cmd[1:3] == ["-m", "torch.distributed.run"] and "--master-port" in cmd and cmd[-1] == "cfg.yaml"
    assert cmd[cmd.index("--nproc-per-node") + 1] == "4" and cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"
    monkeypatch.setenv("RDZV_ID", "job7")
    monkeypatch.setenv("MIN_NNODES", "1")
    monkeypatch.setenv("MAX_NNODES", "2")
    monkeypatch.setenv("MAX_RESTARTS", "3")
    el = launcher.torchrun_command(["cfg.yaml"])
    assert el[el.index("--nnodes") + 1] == "1:2" and el[el.index("--rdzv-id") + 1] == "job7"
    assert el[el.index("--max-restarts") + 1] == "3" and el[el.index("--rdzv-endpoint") + 1] == "127.0.0.1:29611"
    monkeypatch.delenv("RDZV_ID")
    sc = launcher.serve_command(4, ["ckpt", "--port", "8123"])
    assert sc[sc.index("--nproc-per-node") + 1] == "4" and sc[-3:] == ["ckpt", "--port", "8123"]
    assert "hybrid_model_factory_b200.serving.api_server" in sc
    # single-process training through the command line entry
    y = tmp_path / "c.yaml"
    y.write_text("model_name_or_path: '%s'\nstage: pt\nsynthetic: true\ncutoff_len: 16\nmax_steps: 1\noutput_dir: %s\n"
                 "bf16: false\npure_bf16: false\n" % (json.dumps(TINY), tmp_path / "out"))
    assert launcher.launch(["train", str(y)]) == 0
    assert os.path.exists(tmp_path / "out" / "final" / "config.json")


def test_sharded_preprocess_four_phases(tmp_path):
    from hybrid_model_factory_b200.config.hparams import DataArguments
    from hybrid_model_factory_b200.data import sharded_preprocess as SPP
    from hybrid_model_factory_b200.data.loader import ListDataset, get_dataset
    (tmp_path / "dataset_info.json").write_text(json.dumps({"docs": {"file_name": "docs.json", "formatting": "text",
                                                                     "columns": {"prompt": "text"}}}))
    (tmp_path / "docs.json").write_text(json.dumps([{"text": f"document number {i} " * 12} for i in range(40)]))
    out = str(tmp_path / "tok")
    da = DataArguments(dataset="docs", dataset_dir=str(tmp_path), cutoff_len=64, tokenized_path=out)
    path = SPP.run(da, None, stage="pt", sp_size=1, num_shards=3, workers=2)
    ds = ListDataset.load(path)
    assert len(ds) > 10 and all(len(ds[i]["input_ids"]) == 64 for i in range(len(ds)))
    # the same corpus through the single-process path holds the same number of tokens (up to one block per shard)
    single = get_dataset(DataArguments(dataset="docs", dataset_dir=str(tmp_path), cutoff_len=64), ByteTokenizer(), "pt")
    assert abs(len(single) - len(ds)) <= 3
    # sequence-parallel layout: rows come in groups of sp_size, labels pre-shifted
    out2 = str(tmp_path / "tok_sp")
    da2 = DataArguments(dataset="docs", dataset_dir=str(tmp_path), cutoff_len=64, tokenized_path=out2)
    ds2 = ListDataset.load(SPP.run(da2, None, stage="pt", sp_size=2, num_shards=2, workers=2))
    assert ds2.labels_shifted and len(ds2) % 2 == 0 and len(ds2[0]["input_ids"]) == 32
    # command line entry
    y = tmp_path / "c.yaml"
    y.write_text("model_name_or_path: '%s'\nstage: pt\ndataset: docs\ndataset_dir: %s\ncutoff_len: 64\n"
                 "tokenized_path: %s\nmax_steps: 1\noutput_dir: %s\n" % (json.dumps(TINY), tmp_path, tmp_path / "tok_cli",
                                                                         tmp_path / "o"))
    assert SPP.main(["--config", str(y), "--num-shards", "2", "--workers", "2"]) == 0
    assert os.path.exists(tmp_path / "tok_cli" / "dataset.pt")


def test_every_chat_template_encodes_a_two_turn_conversation():
    from hybrid_model_factory_b200.data.formats import TEMPLATES, Template, register_template
    tok = ByteTokenizer()
    msgs = [{"role": "user", "content": "first question"}, {"role": "assistant", "content": "first answer"},
            {"role": "user", "content": "second question"}, {"role": "assistant", "content": "second answer"}]
    assert len(TEMPLATES) >= 24
    for name, tpl in TEMPLATES.items():
        pairs = tpl.encode_multiturn(tok, msgs, "be exact")
        assert len(pairs) == 2, name
        text = bytes(t for p, r in pairs for t in p + r if t < 256).decode(errors="ignore")
        for piece in ("first question", "first answer", "second question", "second answer"):
            assert piece in text, (name, piece)
        if name != "empty":
            assert text.index("be exact") < text.index("first question"), name           # system prompt comes first
        prompt2 = bytes(t for t in pairs[1][0] if t < 256).decode(errors="ignore")
        assert "be exact" not in prompt2, name                                            # and only once
        rows = L.process_supervised([{"messages": msgs, "system": ""}], tok, tpl, 512)
        lab = [t for t in rows[0]["labels"] if t != -100 and t < 256]
        assert "first answer" in bytes(lab).decode(errors="ignore") and "question" not in bytes(lab).decode(errors="ignore")
    register_template(Template("my_format", user_fmt="Q: {content}\\nA:", assistant_fmt=" {content}\\n"))
    with pytest.raises(ValueError):
        register_template(Template("qwen3"))


def test_multiple_choice_evaluator(tmp_path, capsys):
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.train import evaluate as E
    from hybrid_model_factory_b200.utils import checkpoint_io
    root = tmp_path / "evaluation" / "toy"
    root.mkdir(parents=True)
    (root / "mapping.json").write_text(json.dumps({"algebra": {"name": "algebra", "category": "STEM"},
                                                   "history": {"name": "world history", "category": "Humanities"}}))
    letters = "ABCD"

    def make(n, off):
        return [{"question": f"question {i} #{letters[(i + off) % 4]}", "A": "one", "B": "two", "C": "three", "D": "four",
                 "answer": letters[(i + off) % 4]} for i in range(n)]
    for subj, off in (("algebra", 0), ("history", 1)):
        (root / f"{subj}.json").write_text(json.dumps({"train": make(6, off + 2), "test": make(8, off)}))

    class Oracle(torch.nn.Module):
        """Reads the letter after the last '#' of the prompt: a perfect model for this toy task."""
        def __init__(self, always=None):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(1))
            self.always = always

        def forward(self, ids, logits_to_keep=1):
            out = torch.zeros(ids.shape[0], 1, 259)
            for b, row in enumerate(ids.tolist()):
                pos = max(i for i, t in enumerate(row) if t == ord("#"))
                out[b, 0, ord(self.always) if self.always else row[pos + 1]] = 5.0
            return type("O", (), {"logits": out})()
    tok, tpl = ByteTokenizer(), get_template("qwen3")
    args = E.EvaluationArguments(task="toy_test", task_dir=str(tmp_path / "evaluation"), n_shot=3, batch_size=4,
                                 save_dir=str(tmp_path / "res"))
    res = E.Evaluator(Oracle(), tok, tpl, args).evaluate()
    assert res["Average"] == 100.0 and res["STEM"] == 100.0 and res["subject/history"] == 100.0
    assert json.load(open(tmp_path / "res" / "results.json"))["algebra"]["1"] == "B"
    assert "Average" in open(tmp_path / "res" / "results.log").read()
    res_a = E.Evaluator(Oracle(always="A"), tok, tpl, args).evaluate()
    assert res_a["Average"] == 25.0
    # few-shot prompt: header once, three solved exemplars, then the open question
    ev = E.Evaluator(Oracle(), tok, tpl, args)
    msgs = ev.eval_template.format_example(make(1, 0)[0], make(3, 2), "algebra")
    assert len(msgs) == 8 and msgs[0]["content"].startswith("The following are multiple choice questions")
    assert msgs[1]["content"] in letters and msgs[-2]["content"].endswith("Answer:")
    # a real (untrained) checkpoint through the command line
    cfg = HybridConfig(**TINY)
    checkpoint_io.save_pretrained(build_model(cfg), str(tmp_path / "ckpt"))
    assert E.main([str(tmp_path / "ckpt"), "--task", "toy_test", "--task-dir", str(tmp_path / "evaluation"), "--n-shot", "1",
                   "--template", "qwen3"]) == 0
    assert "Average" in capsys.readouterr().out
    # the same through a YAML file; an unknown key is refused
    (tmp_path / "eval.yaml").write_text(f"task: toy_test\ntask_dir: {tmp_path / 'evaluation'}\nn_shot: 1\ntemplate: qwen3\n")
    assert E.main([str(tmp_path / "ckpt"), "--config", str(tmp_path / "eval.yaml")]) == 0
    assert "Average" in capsys.readouterr().out
    (tmp_path / "bad.yaml").write_text("task: toy_test\nshots: 1\n")
    with pytest.raises(ValueError, match="unknown keys"):
        E.main([str(tmp_path / "ckpt"), "--config", str(tmp_path / "bad.yaml")])


def test_example_configs_parse():
    """Every file under examples/ is accepted by the parser it is meant for."""
    import glob
    from hybrid_model_factory_b200.models.patterns import is_fused, parse_override_pattern
    from hybrid_model_factory_b200.priming.hybridize_model import load_config, verify_hybrid_config
    from hybrid_model_factory_b200.train.workflow import zero_config
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    stage0 = sorted(glob.glob(os.path.join(root, "priming", "stage0", "*.yaml")))
    assert len(stage0) >= 4
    for path in stage0:
        cfg = load_config(path)
        verify_hybrid_config(cfg, 36)
        assert any(is_fused(s) for s in parse_override_pattern(cfg.hybrid_override_pattern).values()), path
    train = sorted(glob.glob(os.path.join(root, "priming", "stage[12]", "*.yaml")) +
                   glob.glob(os.path.join(root, "tokenization", "*.yaml")))
    assert len(train) >= 6
    for path in train:
        model_args, data_args, run_args, ft_args, _ = get_train_args([path])
        assert ft_args.stage in ("pt", "sft", "hkd", "dpo") and data_args.cutoff_len >= 4096, path
    # the L2A research example: construction pattern of 36 routed layers, training with the sparsity term
    l2a = load_config(os.path.join(root, "research", "L2A", "construct_qwen3_8b.yaml"))
    verify_hybrid_config(l2a, 36)
    assert set(parse_override_pattern(l2a.hybrid_override_pattern).values()) == {"L2A"} and l2a.l2a["sliding_window"] == 4095
    _, data_args, _, ft_args, _ = get_train_args([os.path.join(root, "research", "L2A", "train_l2a_qwen3_8b.yaml")])
    assert ft_args.lambda_reg == 1e-8 and data_args.cutoff_len == 131072
    pipeline = open(os.path.join(root, "training", "8xB200", "run_pipeline.sh")).read()
    for rel in ("priming/stage0/qwen3_8b_gdn.yaml", "priming/stage1/hqwen3_8b_gdn.yaml",
                "priming/stage2/hqwen3_8b_gdn_long_ctx.yaml", "tokenization/pretraining_sp.yaml"):
        assert os.path.basename(rel) in pipeline and os.path.exists(os.path.join(root, rel)), rel
    stages = {os.path.basename(p): zero_config(p) for p in glob.glob(os.path.join(root, "zero", "*.json"))}
    assert stages["ds_z3_offload_config.json"] == {"zero_stage": 3, "offload_optimizer": True}
    assert stages["ds_z3_mics_config.json"]["mics_shard_size"] == 8 and stages["ds_z2_config.json"]["zero_stage"] == 2


def test_text_metrics_and_do_predict(tmp_path):
    from hybrid_model_factory_b200.train import predict as P
    a, b = "the cat sat on the mat".split(), "the cat lay on the mat".split()
    assert P.rouge_n(a, a, 1) == 1.0 and abs(P.rouge_n(a, b, 1) - 5 / 6) < 1e-9
    assert abs(P.rouge_n(a, b, 2) - 3 / 5) < 1e-9 and abs(P.rouge_l(a, b) - 5 / 6) < 1e-9
    assert P.bleu4(a, a) == 1.0 and 0 < P.bleu4(a, b) < 1 and P.bleu4(["x"], a) == 0.0
    assert P.bleu4(a[:3], a) < P.bleu4(a, a)                                 # brevity penalty
    m = P.text_metrics(["hello world", "abc"], ["hello world", "abd"])
    assert m["predict_exact_match"] == 50.0 and m["predict_rouge-l"] > 50.0
    # through the workflow: an untrained tiny model generates for two prompts of a sharegpt file
    (tmp_path / "dataset_info.json").write_text(json.dumps({"qa": {"file_name": "qa.json", "formatting": "sharegpt"}}))
    (tmp_path / "qa.json").write_text(json.dumps([
        {"conversations": [{"from": "human", "value": f"question {i}"}, {"from": "gpt", "value": f"answer {i}"}]}
        for i in range(2)]))
    out = str(tmp_path / "pred")
    metrics = run_exp({"model_name_or_path": json.dumps(TINY), "stage": "sft", "do_train": False, "do_predict": True,
                       "eval_dataset": "qa", "dataset_dir": str(tmp_path), "template": "qwen3", "cutoff_len": 128,
                       "max_new_tokens": 5, "do_sample": False, "output_dir": out, "bf16": False, "pure_bf16": False})
    assert set(metrics) == {"predict_exact_match", "predict_rouge-1", "predict_rouge-2", "predict_rouge-l", "predict_bleu-4"}
    lines = [json.loads(l) for l in open(os.path.join(out, "generated_predictions.jsonl"))]
    assert len(lines) == 2 and lines[0]["label"].startswith("answer 0") and "question 0" in lines[0]["prompt"]
    assert os.path.exists(os.path.join(out, "predict_results.json"))


def test_held_out_loss_during_training(tmp_path):
    (tmp_path / "dataset_info.json").write_text(json.dumps({"docs": {"file_name": "docs.json", "formatting": "text",
                                                                     "columns": {"prompt": "text"}}}))
    (tmp_path / "docs.json").write_text(json.dumps([{"text": "abc abc abc " * 30} for _ in range(24)]))
    out = str(tmp_path / "run")
    tr = run_exp({"model_name_or_path": json.dumps(TINY), "stage": "pt", "dataset": "docs", "dataset_dir": str(tmp_path),
                  "cutoff_len": 32, "val_size": 0.1, "eval_steps": 3, "max_steps": 6, "output_dir": out, "bf16": False,
                  "pure_bf16": False, "learning_rate": 3e-3, "lr_scheduler_type": "constant",
                  "per_device_train_batch_size": 2, "per_device_eval_batch_size": 2})
    log = [json.loads(l) for l in open(os.path.join(out, "trainer_log.jsonl"))]
    evals = [r["eval_loss"] for r in log if "eval_loss" in r]
    assert len(evals) == 2 and evals[1] < evals[0] and abs(tr.last_eval_loss - evals[1]) < 1e-9
