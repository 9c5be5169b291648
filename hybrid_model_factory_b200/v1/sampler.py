"""Generation for the second-generation stack: a sampler wraps a ``ModelEngine`` and the native serving engine and
answers chat messages one conversation at a time (streamed piece by piece) or a whole dataset in batches.

Reference: ``v1/core/base_sampler.py:23-67`` (``generate`` as an async generator of text pieces, ``batch_infer`` over
a dataset) and ``v1/samplers/cli_sampler.py`` (terminal loop); the reference's engine is Hugging Face ``generate`` with
a streamer thread, here it is ``serving/engine.py`` (continuous batching, so ``batch_infer`` runs all rows together)."""
from __future__ import annotations

from typing import AsyncGenerator, Iterable, List, Optional

from ..serving.engine import SamplingParams, ServingEngine


class Sampler:
    def __init__(self, model_engine, max_new_tokens: int = 256, temperature: float = 0.0, top_p: float = 1.0,
                 max_num_seqs: int = 16, max_model_len: int = 8192, **engine_kwargs):
        self.me = model_engine
        self.tokenizer, self.renderer = model_engine.tokenizer, model_engine.renderer
        self.engine = ServingEngine(model_engine.model, max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                                    **engine_kwargs)
        self.params = dict(max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p,
                           eos_token_id=getattr(self.tokenizer, "eos_token_id", None), ignore_eos=False)

    def _prompt_ids(self, messages: List[dict], tools: Optional[str] = None) -> List[int]:
        tpl = self.renderer.template
        system = next((m["content"] for m in messages if m["role"] == "system"), "")
        turns = [m for m in messages if m["role"] != "system"]
        if tools or any(m["role"] in ("function", "observation") for m in turns):
            turns, system = tpl.normalise(turns, system, tools or "")
        pairs = tpl.encode_multiturn(self.tokenizer, turns + [{"role": "assistant", "content": ""}], system)
        ids: List[int] = []
        for i, (p, r) in enumerate(pairs):
            ids += p + (r if i < len(pairs) - 1 else [])
        return ids

    async def generate(self, messages: List[dict], tools: Optional[str] = None) -> AsyncGenerator[str, None]:
        """Text pieces of the answer as they are decoded (whole characters only)."""
        rid = self.engine.add_request(self._prompt_ids(messages, tools), SamplingParams(**self.params))
        toks, sent = [], 0
        while not self.engine.requests[rid].finished:
            for r, tok, _ in self.engine.step():
                if r == rid:
                    toks.append(tok)
            text = self.tokenizer.decode(toks)
            if text.endswith("�") and not self.engine.requests[rid].finished:
                continue
            if len(text) > sent:
                yield text[sent:]
                sent = len(text)

    def chat(self, messages: List[dict], tools: Optional[str] = None) -> str:
        out = self.engine.generate([self._prompt_ids(messages, tools)], SamplingParams(**self.params))[0]
        return self.tokenizer.decode(out)

    def batch_infer(self, dataset: Iterable[dict]) -> List[dict]:
        """Every sample's ``messages`` up to its last user turn is answered; returns the samples with ``prediction``
        (and ``label``: the sample's own last assistant turn, when it has one)."""
        rows = list(dataset)
        prompts, labels = [], []
        for s in rows:
            msgs = s["messages"]
            has_answer = bool(msgs) and msgs[-1]["role"] == "assistant"
            labels.append(msgs[-1]["content"] if has_answer else None)
            prompts.append(self._prompt_ids(msgs[:-1] if has_answer else msgs))
        outs = self.engine.generate(prompts, SamplingParams(**self.params))
        return [dict(s, prediction=self.tokenizer.decode(o), label=l) for s, o, l in zip(rows, outs, labels)]


def cli(model_path: str, template: Optional[str] = None, **kw) -> int:
    """Terminal loop: ``exit`` leaves, ``clear`` forgets the conversation."""
    import asyncio
    from .model_engine import ModelEngine
    sampler = Sampler(ModelEngine(model_path, template=template, is_train=False,
                                  init_config={"name": "init_on_meta"}), **kw)
    history: List[dict] = []

    async def answer() -> str:
        pieces = []
        async for piece in sampler.generate(history):
            print(piece, end="", flush=True)
            pieces.append(piece)
        print()
        return "".join(pieces)
    while True:
        try:
            text = input("User: ")
        except EOFError:
            return 0
        if text.strip() == "exit":
            return 0
        if text.strip() == "clear":
            history.clear()
            continue
        history.append({"role": "user", "content": text})
        print("Assistant: ", end="")
        history.append({"role": "assistant", "content": asyncio.run(answer())})
