"""OpenAI-compatible HTTP front end on the native engine: ``/v1/models``, ``/v1/completions``,
``/v1/chat/completions`` (optionally SSE streaming) and ``/metrics``.  One background thread drives
``engine.step()``; handlers enqueue requests and wait on per-request queues.
Reference surface: ``api/app.py:69-133`` and ``vllm serve`` as used in ``docs/Inference.md``."""
from __future__ import annotations

import argparse
import asyncio
import json
import threading
import time
import uuid
from typing import Dict, List, Optional

import torch

from ..data.formats import get_template, load_tokenizer
from ..utils import checkpoint_io
from .engine import SamplingParams, ServingEngine


class ControlChannel:
    """Rank 0 of a tensor-parallel server tells the other ranks what it is about to do: a small object broadcast on a
    gloo group before every engine step (new requests, stop).  The engine itself is deterministic given the same
    request stream, so this is all the followers need to stay in lock-step.

    Rank 0 broadcasts at least every 50 ms, also when idle, so the channel doubles as a heartbeat: the group's
    timeout (``HMF_TP_CONTROL_TIMEOUT_S``, default 120 s) ends a follower whose rank 0 has gone, and rank 0's send to
    a follower that has gone fails the same way, instead of either side waiting for gloo's default half hour."""

    def __init__(self, timeout_s: Optional[float] = None):
        import datetime
        import os
        import torch.distributed as dist
        self.dist = dist
        timeout_s = timeout_s or float(os.environ.get("HMF_TP_CONTROL_TIMEOUT_S", "120"))
        self.group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
        self.rank = dist.get_rank()

    def broadcast(self, msg=None):
        box = [msg]
        self.dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]


def _params_to_dict(p: SamplingParams) -> dict:
    """Every field: a follower that sampled with other settings than rank 0 would pick other tokens, finish its
    requests at other steps and leave the ranks' collectives unmatched."""
    import dataclasses
    return dataclasses.asdict(p)


class EngineLoop:
    """Runs ``engine.step()`` in a thread and routes new tokens to per-request asyncio queues.  With a
    ``ControlChannel`` (tensor parallelism) every step is announced to the follower ranks first."""

    def __init__(self, engine: ServingEngine, control: Optional[ControlChannel] = None):
        self.engine, self.control = engine, control
        self.lock = threading.Lock()
        self.pending: List[tuple] = []
        self.queues: Dict[int, tuple] = {}
        self.wake = threading.Event()
        self.stop = False
        self.error: Optional[BaseException] = None
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def submit(self, prompt: List[int], params: SamplingParams, loop) -> tuple:
        q: asyncio.Queue = asyncio.Queue()
        with self.lock:
            self.pending.append((list(prompt), params, q, loop))
        self.wake.set()
        return None, q

    def shutdown(self, timeout: float = 20.0) -> None:
        """Stops the serving thread (which also releases the follower ranks) and drops the engine's captured graphs."""
        self.stop = True
        self.wake.set()
        self.thread.join(timeout=timeout)
        self.engine.close()

    def _run(self):
        try:
            if self.engine.device.type == "cuda":       # a new thread starts on device 0
                torch.cuda.set_device(self.engine.device)
            self._loop()
        except BaseException as e:      # an engine failure must not leave handlers and follower ranks waiting for ever
            self.error = e
            self.stop = True
            if self.control is not None:
                try:
                    self.control.broadcast({"add": [], "stop": True})
                except Exception:
                    pass
            with self.lock:
                waiting = list(self.queues.values()) + [(q, loop) for _, _, q, loop in self.pending]
                self.queues.clear()
                self.pending = []
            for q, loop in waiting:
                loop.call_soon_threadsafe(q.put_nowait, (None, True))
            import logging
            logging.getLogger(__name__).exception("engine thread stopped: %r", e)

    def _loop(self):
        while True:
            with self.lock:
                new, self.pending = self.pending, []
            stop = self.stop
            if self.control is not None:
                self.control.broadcast({"add": [(p, _params_to_dict(sp)) for p, sp, _, _ in new], "stop": stop})
            if stop:
                return
            for prompt, params, q, loop in new:
                self.queues[self.engine.add_request(prompt, params)] = (q, loop)
            busy = self.engine.has_unfinished()
            results = self.engine.step() if busy else []
            for rid, tok, done in results:
                entry = self.queues.get(rid)
                if entry:
                    q, loop = entry
                    loop.call_soon_threadsafe(q.put_nowait, (tok, done))
                    if done:
                        self.queues.pop(rid, None)
            if not busy:
                self.wake.wait(timeout=0.05)
                self.wake.clear()


def follow(engine: ServingEngine, control: ControlChannel) -> int:
    """Loop of the tensor-parallel ranks other than 0: replay rank 0's request stream and step with it.  Returns the
    number of engine steps taken; the engine's captured graphs are released on the way out (they pin the NCCL
    communicator, see ``ServingEngine.close``)."""
    steps = 0
    while True:
        msg = control.broadcast()
        if msg["stop"]:
            engine.close()
            return steps
        for prompt, params in msg["add"]:
            engine.add_request(prompt, SamplingParams(**params))
        if engine.has_unfinished():
            engine.step()
            steps += 1


def create_app(engine: ServingEngine, tokenizer, model_name: str = "hybrid", template: Optional[str] = None,
               control: Optional[ControlChannel] = None):
    from fastapi import FastAPI
    from fastapi.responses import JSONResponse, StreamingResponse
    app = FastAPI(title="hybrid-model-factory (B200 native) server")
    loop_runner = EngineLoop(engine, control)
    tpl = get_template(template)

    def params_from(body: dict) -> SamplingParams:
        return SamplingParams(max_new_tokens=int(body.get("max_tokens", 64)), temperature=float(body.get("temperature", 0.0)),
                              top_k=int(body.get("top_k", 0)), top_p=float(body.get("top_p", 1.0)),
                              min_p=float(body.get("min_p", 0.0)),
                              repetition_penalty=float(body.get("repetition_penalty", 1.0)),
                              speculative_tokens=int(body.get("speculative_tokens", 0)),
                              eos_token_id=getattr(tokenizer, "eos_token_id", None),
                              ignore_eos=bool(body.get("ignore_eos", False)))

    async def run(prompt_ids: List[int], body: dict, chat: bool):
        if loop_runner.error is not None:
            return JSONResponse({"error": repr(loop_runner.error)}, status_code=500)
        rid, q = loop_runner.submit(prompt_ids, params_from(body), asyncio.get_running_loop())
        created, cid = int(time.time()), f"cmpl-{uuid.uuid4().hex[:12]}"
        if body.get("stream"):
            async def gen():
                toks, sent = [], 0          # incremental detokenisation: a character may span several tokens
                while True:
                    tok, done = await q.get()
                    if tok is None:         # the engine thread failed
                        yield "data: " + json.dumps({"error": repr(loop_runner.error)}) + "\n\n"
                        return
                    toks.append(tok)
                    full = tokenizer.decode(toks)
                    if not done and full.endswith("\ufffd"):
                        continue            # incomplete multi-byte character: wait for the rest
                    text, sent = full[sent:], len(full)
                    delta = {"delta": {"content": text}} if chat else {"text": text}
                    yield "data: " + json.dumps({"id": cid, "created": created, "model": model_name,
                                                 "choices": [{"index": 0, **delta, "finish_reason": "length" if done else None}]}) + "\n\n"
                    if done:
                        yield "data: [DONE]\n\n"
                        return
            return StreamingResponse(gen(), media_type="text/event-stream")
        toks = []
        while True:
            tok, done = await q.get()
            if tok is None:                 # the engine thread failed
                return JSONResponse({"error": repr(loop_runner.error)}, status_code=500)
            toks.append(tok)
            if done:
                break
        text = tokenizer.decode(toks)
        choice = {"index": 0, "finish_reason": "length"}
        choice.update({"message": {"role": "assistant", "content": text}} if chat else {"text": text})
        return JSONResponse({"id": cid, "object": "chat.completion" if chat else "text_completion", "created": created,
                             "model": model_name, "choices": [choice],
                             "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": len(toks),
                                       "total_tokens": len(prompt_ids) + len(toks)}})

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "local"}]}

    @app.post("/v1/completions")
    async def completions(body: dict):
        prompt = body.get("prompt", "")
        ids = prompt if isinstance(prompt, list) and prompt and isinstance(prompt[0], int) else tokenizer.encode(
            prompt if isinstance(prompt, str) else prompt[0], add_special_tokens=False)
        return await run(list(ids), body, chat=False)

    @app.post("/v1/chat/completions")
    async def chat(body: dict):
        msgs = body.get("messages", [])
        system = next((m["content"] for m in msgs if m["role"] == "system"), "")
        turns = [m for m in msgs if m["role"] != "system"] + [{"role": "assistant", "content": ""}]
        pairs = tpl.encode_multiturn(tokenizer, turns, system)
        ids: List[int] = []
        for i, (p, r) in enumerate(pairs):
            ids += p + (r if i < len(pairs) - 1 else [])
        return await run(ids, body, chat=True)

    @app.post("/v1/score/evaluation")
    async def score(body: dict):
        """Reward-model scores of ``messages`` (a list of texts): the value head at each text's last token.  Needs a
        checkpoint trained with ``stage: rm`` (it carries ``v_head``); reference: ``api/app.py`` ``/v1/score/evaluation``.
        Runs on the serving thread's model between engine steps (texts are short; no paged cache is involved)."""
        model = engine.model
        if not hasattr(model, "v_head"):
            return JSONResponse({"error": "this checkpoint has no value head (train it with stage: rm)"}, status_code=400)
        texts = body.get("messages", [])
        max_len = int(body.get("max_length", 1024))
        rows = [tokenizer.encode(t, add_special_tokens=False)[:max_len] or [0] for t in texts]
        from ..train.preference import reward_scores
        scores = []
        with torch.no_grad():
            for ids in rows:            # one text at a time: no padding, so the last token is the last position
                t = torch.tensor([ids], dtype=torch.long, device=engine.device)
                scores.append(float(reward_scores(model, t)[0]))
        return {"id": f"scoreval-{uuid.uuid4().hex[:12]}", "object": "score.evaluation", "model": model_name,
                "scores": scores}

    @app.get("/metrics")
    async def metrics():
        return engine.request_metrics()

    app.state.loop_runner = loop_runner
    return app


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hmf serve")
    ap.add_argument("model")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--enable-prefix-caching", action="store_true")
    ap.add_argument("--template", default=None)
    ap.add_argument("--draft-model", default=None,
                    help="checkpoint of a small model with the same vocabulary: proposes tokens for requests that set "
                         "speculative_tokens, where their own n-grams offer none")
    ap.add_argument("--hf-overrides", default=None, help='JSON, e.g. {"gka_overrides": {"num_iter": 10}}')
    args = ap.parse_args(argv)
    overrides = json.loads(args.hf_overrides) if args.hf_overrides else {}
    import os
    world, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    model = checkpoint_io.from_pretrained(args.model, device=device, **overrides)
    tp = control = None
    if world > 1:       # launched by torchrun: tensor parallel over all ranks, rank 0 serves HTTP
        import torch.distributed as dist
        from ..parallel.tp import TPContext, shard_model
        if device.type == "cuda":
            torch.cuda.set_device(device)
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
        tp = TPContext(dist.group.WORLD)
        if device.type == "cuda":
            tp.enable_fused_gemm(max_m=256, max_n=8192)
        shard_model(model, tp)
        torch.manual_seed(0)           # stochastic sampling must draw the same numbers on every rank
        control = ControlChannel()
    draft = checkpoint_io.from_pretrained(args.draft_model, device=device) if args.draft_model else None
    engine = ServingEngine(model, max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
                           max_model_len=args.max_model_len, enable_prefix_caching=args.enable_prefix_caching, tp=tp,
                           draft_model=draft)
    if device.type == "cuda":
        # capture the decode graphs here, on the main thread and on every rank at the same time; the serving thread
        # then only replays them
        engine.warmup(args.max_model_len, every_length=True)
    if control is not None and control.rank != 0:
        follow(engine, control)
        return 0
    import uvicorn
    app = create_app(engine, load_tokenizer(args.model), model_name=args.model, template=args.template, control=control)
    try:
        uvicorn.run(app, host=args.host, port=args.port)
    finally:
        app.state.loop_runner.shutdown(timeout=5)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
