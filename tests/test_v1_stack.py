"""Second-generation stack: data engine index, renderer, resumable batch generator, token-weighted trainer."""
import json

import torch

from hybrid_model_factory_b200.data.formats import ByteTokenizer
from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model
from hybrid_model_factory_b200.v1 import BatchGenerator, DataEngine, Renderer, SFTTrainerV1, V1TrainingArguments


def _records(n, tag="q"):
    return [{"instruction": f"{tag} {i}?", "input": "", "output": "answer " + "x" * (i % 7)} for i in range(n)]


def _engine(tmp_path):
    a, b = tmp_path / "a.json", tmp_path / "b.jsonl"
    a.write_text(json.dumps(_records(10, "a")))
    b.write_text("\n".join(json.dumps({"conversations": [{"from": "human", "value": f"b {i}"},
                                                          {"from": "gpt", "value": f"reply {i}"}]}) for i in range(6)))
    info = tmp_path / "mix.yaml"
    info.write_text("alpaca_part:\n  path: a.json\n  converter: alpaca\n  size: 12\n"
                    "share_part:\n  path: b.jsonl\n  converter: sharegpt\n  weight: 0.5\n")
    return DataEngine(str(info))


def test_data_engine_index_and_conversion(tmp_path):
    eng = _engine(tmp_path)
    assert len(eng) == 12 + 3                                    # size resamples, weight scales
    s = eng[0]
    assert s["_dataset_name"] == "alpaca_part" and [m["role"] for m in s["messages"]] == ["user", "assistant"]
    assert s["messages"][0]["loss_weight"] == 0.0 and s["messages"][1]["loss_weight"] == 1.0
    assert eng[10]["messages"][0]["content"] == "a 0?"           # wrapped around after 10 records
    last = eng[[13, 14]]
    assert [x["_dataset_name"] for x in last] == ["share_part"] * 2
    rnd = Renderer(ByteTokenizer(), "default", cutoff_len=64).process_samples([s])[0]
    assert len(rnd["input_ids"]) == len(rnd["labels"]) and any(l != -100 for l in rnd["labels"])
    assert rnd["labels"][0] == -100                              # the prompt carries no loss


def test_batch_generator_resumes_exactly(tmp_path):
    eng = _engine(tmp_path)
    rnd = Renderer(ByteTokenizer(), "default", cutoff_len=64)
    for strategy, kw in (("normal", {}), ("padding_free", {}), ("dynamic", {"token_budget": 150})):
        gen = BatchGenerator(eng, rnd, micro_batch_size=2, global_batch_size=4, strategy=strategy, seed=3, **kw)
        first = [next(gen) for _ in range(2)]
        state = json.loads(json.dumps(gen.state_dict()))         # must survive JSON
        rest = list(gen)
        gen2 = BatchGenerator(eng, rnd, micro_batch_size=2, global_batch_size=4, strategy=strategy, seed=3, **kw)
        gen2.load_state_dict(state)
        rest2 = list(gen2)
        assert len(rest) == len(rest2) and len(rest) >= 1, strategy
        for a, b in zip(rest, rest2):
            assert len(a) == len(b)
            for ma, mb in zip(a, b):
                assert torch.equal(ma["input_ids"], mb["input_ids"]) and torch.equal(ma["labels"], mb["labels"])
        if strategy == "normal":
            assert len(first[0]) == 2 and first[0][0]["input_ids"].shape[0] == 2
        else:
            mb = first[0][0]
            assert mb["input_ids"].shape[0] == 1 and mb["cu_seqlens"][-1] == mb["input_ids"].shape[1]
        if strategy == "dynamic":
            assert all(sum(m["input_ids"].numel() for m in step) <= 150 for step in first + rest)
    # the two data-parallel ranks of one epoch see disjoint samples of equal count
    g0 = BatchGenerator(eng, rnd, 1, 2, dp_rank=0, dp_size=2, seed=1)
    g1 = BatchGenerator(eng, rnd, 1, 2, dp_rank=1, dp_size=2, seed=1)
    assert len(g0._indices()) == len(g1._indices()) and not set(g0._indices()) & set(g1._indices())
    g0.set_epoch(1)
    assert g0._indices() != BatchGenerator(eng, rnd, 1, 2, dp_rank=0, dp_size=2, seed=1)._indices()


def test_v1_trainer_token_weighting_and_resume(tmp_path):
    torch.manual_seed(0)
    eng = _engine(tmp_path)
    rnd = Renderer(ByteTokenizer(), "default", cutoff_len=48)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=259, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN")

    def make(strategy, micro, out):
        torch.manual_seed(1)
        model = build_model(cfg)
        args = V1TrainingArguments(output_dir=str(out), micro_batch_size=micro, global_batch_size=4, max_steps=3,
                                   learning_rate=1e-3, lr_scheduler="constant", bf16=False,
                                   batching_strategy=strategy)
        return SFTTrainerV1(args, model, rnd, eng, device=torch.device("cpu")), model

    # the same four samples as one micro-batch of 4 or four micro-batches of 1: same step (token-weighted loss)
    t4, m4 = make("normal", 4, tmp_path / "o4")
    t1, m1 = make("normal", 1, tmp_path / "o1")
    l4 = t4.train_step(next(t4.generator))
    l1 = t1.train_step(next(t1.generator))
    assert abs(l4 - l1) < 1e-4
    for (n, a), (_, b) in zip(m4.named_parameters(), m1.named_parameters()):
        assert torch.allclose(a, b, atol=2e-5), n
    # packed rows with checkpointing on: runs, finite loss
    tp, _ = make("padding_free", 2, tmp_path / "op")
    assert tp.train_step(next(tp.generator)) > 0
    # checkpoint after one step, resume, and both continue identically
    ta, _ = make("normal", 2, tmp_path / "oa")
    ta.train_step(next(ta.generator))
    ta.save_checkpoint(str(tmp_path / "ck"))
    la = ta.train_step(next(ta.generator))
    tb, _ = make("normal", 2, tmp_path / "ob")
    tb.load_checkpoint(str(tmp_path / "ck"))
    assert tb.global_step == 1
    lb = tb.train_step(next(tb.generator))
    assert abs(la - lb) < 1e-5
    ta.fit()
    assert ta.global_step == 3


def test_v1_launcher_runs_from_yaml(tmp_path):
    """``USE_V1=1 hmf train cfg.yaml``: loads a checkpoint, trains two steps on a dataset description, saves a model
    that loads again."""
    from hybrid_model_factory_b200.utils import checkpoint_io
    from hybrid_model_factory_b200.v1.launcher import main
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=259, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN")
    checkpoint_io.save_pretrained(build_model(cfg), str(tmp_path / "model"))
    _engine(tmp_path)                                            # writes mix.yaml and its data files
    out = tmp_path / "out"
    (tmp_path / "run.yaml").write_text(
        f"model: {tmp_path / 'model'}\ntrain_dataset: {tmp_path / 'mix.yaml'}\noutput_dir: {out}\n"
        "micro_batch_size: 2\nglobal_batch_size: 4\nmax_steps: 2\nbf16: false\ncutoff_len: 48\n"
        "batching_strategy: padding_free\nlearning_rate: 1.0e-3\n")
    assert main([str(tmp_path / "run.yaml"), "lr_scheduler=constant"]) == 0
    again = checkpoint_io.from_pretrained(str(out), dtype=torch.float32)
    assert again.config.num_hidden_layers == 2
    import pytest
    with pytest.raises(ValueError, match="unknown configuration keys"):
        (tmp_path / "bad.yaml").write_text(f"model: {tmp_path / 'model'}\ntrain_dataset: x\nno_such_key: 1\n")
        main([str(tmp_path / "bad.yaml")])


def test_plugins_register_by_name_and_serve_the_data_engine(tmp_path):
    """A plugin family keeps functions by name; a user converter and a user batching strategy are found by the data
    engine and the batch generator through their names."""
    import pytest
    from hybrid_model_factory_b200.v1 import BatchingStrategy, DataConverter, Plugin

    class Greeter(Plugin):
        def twice(self, who):
            return self(who) + " " + self["again"](who)

    @Greeter("hello").register()
    def _hello(who):
        return f"hello {who}"

    @Greeter("hello").register("again")
    def _again(who):
        return f"again {who}"

    assert Greeter("hello")("x") == "hello x" and Greeter("hello").again("x") == "again x"
    assert Greeter("hello").twice("y") == "hello y again y"
    assert Greeter.names() == ["hello"] and "hello" not in DataConverter.names()   # tables are per family
    with pytest.raises(ValueError, match="already has"):
        Greeter("hello").register()(_hello)
    with pytest.raises(KeyError, match="no '__call__'"):
        Greeter("nobody")("x")
    with pytest.raises(ValueError, match="needs a name"):
        Greeter().register()

    @DataConverter("question_answer").register(replace=True)
    def _qa(rec):
        return {"messages": [{"role": "user", "content": rec["q"], "loss_weight": 0.0},
                             {"role": "assistant", "content": rec["a"], "loss_weight": 1.0}]}

    (tmp_path / "qa.jsonl").write_text("\n".join(json.dumps({"q": f"q{i}", "a": f"a{i}"}) for i in range(8)))
    (tmp_path / "qa.yaml").write_text("qa:\n  path: qa.jsonl\n  converter: question_answer\n")
    eng = DataEngine(str(tmp_path / "qa.yaml"))
    assert len(eng) == 8 and eng[3]["messages"][1]["content"] == "a3"

    @BatchingStrategy("one_row_each").register(replace=True)
    def _one_each(rows, gen):
        from hybrid_model_factory_b200.v1.batching import packed_collate
        return [packed_collate([r]) for r in rows]

    rnd = Renderer(ByteTokenizer(), "default", cutoff_len=64)
    gen = BatchGenerator(eng, rnd, micro_batch_size=2, global_batch_size=4, strategy="one_row_each", shuffle=False)
    step = next(gen)
    assert len(step) == 4 and all(len(mb["cu_seqlens"]) == 2 for mb in step)
    with pytest.raises(ValueError, match="unknown batching strategy"):
        BatchGenerator(eng, rnd, strategy="no_such_strategy")


def test_model_engine_plugins_and_launcher_sections(tmp_path):
    """Init / peft / kernel plugins: meta loading equals default loading, LoRA leaves only adapters trainable, an unknown
    kernel name is refused, and a YAML with the three sections trains and saves a model in the ordinary layout."""
    import pytest
    from hybrid_model_factory_b200.utils import checkpoint_io
    from hybrid_model_factory_b200.v1 import ModelEngine, register_kernel
    from hybrid_model_factory_b200.v1.launcher import main
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=259, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN")
    checkpoint_io.save_pretrained(build_model(cfg), str(tmp_path / "model"))
    ids = torch.randint(0, 259, (1, 9))
    a = ModelEngine(str(tmp_path / "model"), dtype=torch.float32, is_train=False)
    b = ModelEngine(str(tmp_path / "model"), dtype=torch.float32, is_train=False, init_config={"name": "init_on_meta"})
    c = ModelEngine(str(tmp_path / "model"), dtype=torch.float32, is_train=False, init_config={"name": "init_on_rank0"})
    with torch.no_grad():
        ref = a.model(input_ids=ids).logits
        assert torch.allclose(b.model(input_ids=ids).logits, ref, atol=1e-6)
        assert torch.allclose(c.model(input_ids=ids).logits, ref, atol=1e-6)
    seen = []

    @register_kernel("count_layers")
    def _count(model):
        seen.append(len(model.model.layers))
        return len(model.model.layers)
    lora = ModelEngine(str(tmp_path / "model"), dtype=torch.float32, peft_config={"name": "lora", "rank": 2},
                       kernel_config={"name": "auto", "include_kernels": ["own_linear", "count_layers"]})
    names = [n for n, p in lora.model.named_parameters() if p.requires_grad]
    assert names and all("lora_" in n for n in names) and lora.trainable_parameters() < 4000
    assert seen == [2] and lora.model.applied_kernels["count_layers"] == 2
    frozen = ModelEngine(str(tmp_path / "model"), dtype=torch.float32, peft_config={"name": "freeze", "trainable_layers": 1})
    assert 0 < frozen.trainable_parameters() < sum(p.numel() for p in frozen.model.parameters())
    with pytest.raises(ValueError, match="unknown kernels"):
        ModelEngine(str(tmp_path / "model"), dtype=torch.float32, kernel_config={"include_kernels": ["no_such"]})
    _engine(tmp_path)
    out = tmp_path / "out"
    (tmp_path / "run.yaml").write_text(
        f"model: {tmp_path / 'model'}\ntrain_dataset: {tmp_path / 'mix.yaml'}\noutput_dir: {out}\n"
        "micro_batch_size: 2\nglobal_batch_size: 4\nmax_steps: 2\nbf16: false\ncutoff_len: 48\nlearning_rate: 1.0e-3\n"
        "init_config:\n  name: init_on_meta\npeft_config:\n  name: lora\n  rank: 2\nkernel_config:\n  name: auto\n")
    assert main([str(tmp_path / "run.yaml"), "lr_scheduler=constant"]) == 0
    again = checkpoint_io.from_pretrained(str(out), dtype=torch.float32)          # strict: no adapter tensors left
    assert not any("lora" in n for n, _ in again.named_parameters())


def test_v1_sampler_streams_and_answers_a_dataset(tmp_path):
    import asyncio
    from hybrid_model_factory_b200.utils import checkpoint_io
    from hybrid_model_factory_b200.v1 import ModelEngine
    from hybrid_model_factory_b200.v1.sampler import Sampler
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=259, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN")
    checkpoint_io.save_pretrained(build_model(cfg), str(tmp_path / "model"))
    me = ModelEngine(str(tmp_path / "model"), dtype=torch.float32, is_train=False, init_config={"name": "init_on_meta"})
    s = Sampler(me, max_new_tokens=6, max_num_seqs=4, max_model_len=256, block_size=8, num_blocks=64)
    s.params["ignore_eos"] = True
    msgs = [{"role": "user", "content": "hello there"}]
    whole = s.chat(msgs)

    async def collect():
        return [p async for p in s.generate(msgs)]
    pieces = asyncio.run(collect())
    assert "".join(pieces) == whole and len(pieces) >= 1
    rows = [{"messages": [{"role": "user", "content": "a"}, {"role": "assistant", "content": "gold"}]},
            {"messages": [{"role": "user", "content": "hello there"}]}]
    out = s.batch_infer(rows)
    assert out[0]["label"] == "gold" and out[1]["label"] is None and out[1]["prediction"] == whole
