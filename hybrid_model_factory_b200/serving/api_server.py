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


def _params_from_dict(d: dict) -> SamplingParams:
    d = dict(d)
    d["stop_token_ids"] = tuple(d.get("stop_token_ids") or ())
    return SamplingParams(**d)


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
        self.rid_of: Dict[int, int] = {}          # id(queue) -> request id, once the serving thread has admitted it
        self.aborts: List[int] = []               # id(queue) of requests to end before the next step
        self.sent: Dict[int, int] = {}            # request id -> log-probability entries handed out so far
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

    def abort(self, q) -> None:
        """Ends the request that feeds ``q`` before the next engine step (all tensor-parallel ranks with it)."""
        with self.lock:
            self.aborts.append(id(q))
        self.wake.set()

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
                loop.call_soon_threadsafe(q.put_nowait, (None, True, None))
            import logging
            logging.getLogger(__name__).exception("engine thread stopped: %r", e)

    def _loop(self):
        while True:
            with self.lock:
                new, self.pending = self.pending, []
                wanted, self.aborts = self.aborts, []
            # a request aborted before it was admitted is simply not added
            new = [n for n in new if id(n[2]) not in wanted]
            abort_rids = [self.rid_of[k] for k in wanted if k in self.rid_of]
            stop = self.stop
            if self.control is not None:
                self.control.broadcast({"add": [(p, _params_to_dict(sp)) for p, sp, _, _ in new], "stop": stop,
                                        "abort": abort_rids})
            if stop:
                return
            for rid in abort_rids:
                self.engine.abort(rid)
                entry = self.queues.pop(rid, None)
                if entry:
                    self.rid_of.pop(id(entry[0]), None)
            for prompt, params, q, loop in new:
                rid = self.engine.add_request(prompt, params)
                self.queues[rid] = (q, loop)
                self.rid_of[id(q)] = rid
            busy = self.engine.has_unfinished()
            results = self.engine.step() if busy else []
            for rid, tok, done in results:
                entry = self.queues.get(rid)
                if entry:
                    q, loop = entry
                    req = self.engine.requests[rid]
                    reason = req.finish_reason if done else None
                    lp = None
                    if req.params.logprobs > 0:                 # the entry of this token: results arrive in order
                        k = self.sent.get(rid, 0)
                        lp, self.sent[rid] = req.logprobs[k] if k < len(req.logprobs) else None, k + 1
                    loop.call_soon_threadsafe(q.put_nowait, (tok, reason or done, lp))
                    if done:
                        self.queues.pop(rid, None)
                        self.rid_of.pop(id(q), None)
                        self.sent.pop(rid, None)
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
        for rid in msg.get("abort", ()):
            engine.abort(rid)
        for prompt, params in msg["add"]:
            engine.add_request(prompt, _params_from_dict(params))
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
                              ignore_eos=bool(body.get("ignore_eos", False)),
                              stop_token_ids=tuple(int(t) for t in body.get("stop_token_ids") or ()),
                              logprobs=logprobs_wanted(body))

    def logprobs_wanted(body: dict) -> int:
        """Completions: ``logprobs: k``.  Chat: ``logprobs: true`` with ``top_logprobs: k``."""
        lp = body.get("logprobs")
        if lp is True:
            return max(1, int(body.get("top_logprobs") or 1))
        return int(lp or 0)

    def logprobs_json(c, chat: bool):
        if not c.lps:
            return None
        word = lambda t: tokenizer.decode([t])  # noqa: E731
        if chat:
            return {"content": [{"token": word(t), "logprob": lp, "top_logprobs": [{"token": word(i), "logprob": v}
                                                                                   for i, v in top]}
                                for t, (lp, top) in c.lps]}
        return {"tokens": [word(t) for t, _ in c.lps], "token_logprobs": [lp for _, (lp, _) in c.lps],
                # (tokens that decode to the same string share a key: the likeliest one keeps it)
                "top_logprobs": [{word(i): v for i, v in reversed(top)} for _, (_, top) in c.lps]}

    def stops_of(body: dict) -> List[str]:
        stop = body.get("stop") or []
        return [s for s in ([stop] if isinstance(stop, str) else list(stop)) if s]

    class Choice:
        """One generated sequence: collects tokens from its queue, cuts the text at the first stop string (and has
        the engine drop the request then), and holds back text that may still turn into a stop string."""

        def __init__(self, index: int, q, stops: List[str]):
            self.index, self.q, self.stops = index, q, stops
            self.toks: List[int] = []
            self.text, self.sent, self.reason, self.failed = "", 0, None, False
            self.lps: List[tuple] = []                 # (token, (logprob, [(token, logprob)])) when asked for
            self.hold = max((len(s) for s in stops), default=1) - 1

        async def advance(self) -> str:
            """Waits for the next token; returns the text that may be shown now ('' if none yet)."""
            tok, done, lp = await self.q.get()
            if lp is not None:
                self.lps.append((tok, lp))
            if tok is None:
                self.failed, self.reason = True, "error"
                return ""
            self.toks.append(tok)
            full = tokenizer.decode(self.toks)
            cut = min((full.find(s) for s in self.stops if s in full), default=-1)
            if cut >= 0:
                self.text, self.reason = full[:cut], "stop"
                if not done:
                    loop_runner.abort(self.q)
            elif done:
                self.text, self.reason = full, (done if isinstance(done, str) else "length")
            elif full.endswith("\ufffd"):
                return ""                   # incomplete multi-byte character: wait for the rest
            else:
                self.text = full
            upto = len(self.text) if self.reason else max(self.sent, len(self.text) - self.hold)
            out, self.sent = self.text[self.sent:upto], upto
            return out

    async def run(prompt_ids: List[int], body: dict, chat: bool):
        if loop_runner.error is not None:
            return JSONResponse({"error": repr(loop_runner.error)}, status_code=500)
        n = max(1, int(body.get("n", 1)))
        ev_loop = asyncio.get_running_loop()
        choices = [Choice(i, loop_runner.submit(prompt_ids, params_from(body), ev_loop)[1], stops_of(body))
                   for i in range(n)]
        created, cid = int(time.time()), f"cmpl-{uuid.uuid4().hex[:12]}"

        async def drain(c: Choice, sink=None):
            while c.reason is None:
                piece = await c.advance()
                if sink is not None and (piece or c.reason):
                    await sink.put((c, piece))

        if body.get("stream"):
            async def gen():
                sink: asyncio.Queue = asyncio.Queue()
                tasks = [asyncio.ensure_future(drain(c, sink)) for c in choices]
                live = n
                try:
                    while live:
                        c, piece = await sink.get()
                        if c.failed:
                            yield "data: " + json.dumps({"error": repr(loop_runner.error)}) + "\n\n"
                            return
                        delta = {"delta": {"content": piece}} if chat else {"text": piece}
                        yield "data: " + json.dumps({"id": cid, "created": created, "model": model_name,
                                                     "choices": [{"index": c.index, **delta,
                                                                  "finish_reason": c.reason}]}) + "\n\n"
                        live -= c.reason is not None
                    yield "data: [DONE]\n\n"
                finally:
                    # a client that went away (the generator is closed early) must not keep its requests decoding
                    for t in tasks:
                        t.cancel()
                    for c in choices:
                        if c.reason is None:
                            loop_runner.abort(c.q)
            return StreamingResponse(gen(), media_type="text/event-stream")
        await asyncio.gather(*[drain(c) for c in choices])
        if any(c.failed for c in choices):
            return JSONResponse({"error": repr(loop_runner.error)}, status_code=500)
        out = []
        for c in choices:
            item = {"index": c.index, "finish_reason": c.reason, "logprobs": logprobs_json(c, chat)}
            item.update({"message": {"role": "assistant", "content": c.text}} if chat else {"text": c.text})
            out.append(item)
        done_toks = sum(len(c.toks) for c in choices)
        return JSONResponse({"id": cid, "object": "chat.completion" if chat else "text_completion", "created": created,
                             "model": model_name, "choices": out,
                             "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": done_toks,
                                       "total_tokens": len(prompt_ids) + done_toks}})

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "local"}]}

    @app.post("/v1/completions")
    async def completions(body: dict):
        prompt = body.get("prompt", "")
        ids = prompt if isinstance(prompt, list) and prompt and isinstance(prompt[0], int) else tokenizer.encode(
            prompt if isinstance(prompt, str) else prompt[0], add_special_tokens=False)
        return await run(list(ids), body, chat=False)

    def chat_turns(msgs: List[dict]) -> List[dict]:
        """OpenAI chat messages -> the template's roles: ``tool`` results become observations, assistant turns that
        carry ``tool_calls`` become function turns (a JSON list of ``{name, arguments}``)."""
        turns = []
        for m in msgs:
            if m["role"] == "system":
                continue
            if m["role"] == "tool":
                turns.append({"role": "observation", "content": m.get("content") or ""})
            elif m["role"] == "assistant" and m.get("tool_calls"):
                calls = []
                for c in m["tool_calls"]:
                    fn = c.get("function", c)
                    args = fn.get("arguments", {})
                    calls.append({"name": fn["name"], "arguments": json.loads(args) if isinstance(args, str) else args})
                turns.append({"role": "function", "content": json.dumps(calls, ensure_ascii=False)})
            else:
                content = m.get("content") or ""
                if isinstance(content, list):           # content parts: the text ones
                    content = "".join(p.get("text", "") for p in content if p.get("type", "text") == "text")
                turns.append({"role": m["role"], "content": content})
        return turns

    @app.post("/v1/chat/completions")
    async def chat(body: dict):
        msgs = body.get("messages", [])
        system = next((m["content"] for m in msgs if m["role"] == "system"), "")
        turns = chat_turns(msgs)
        tools = body.get("tools") or []
        if tools or any(t["role"] in ("function", "observation") for t in turns):
            turns, system = tpl.normalise(turns, system, json.dumps([t.get("function", t) for t in tools],
                                                                    ensure_ascii=False) if tools else "")
        pairs = tpl.encode_multiturn(tokenizer, turns + [{"role": "assistant", "content": ""}], system)
        ids: List[int] = []
        for i, (p, r) in enumerate(pairs):
            ids += p + (r if i < len(pairs) - 1 else [])
        resp = await run(ids, body, chat=True)
        if tools and not body.get("stream") and getattr(resp, "status_code", 200) == 200:
            data = json.loads(resp.body)                # answers that call tools: structured calls instead of text
            for choice in data["choices"]:
                text, calls = tpl.extract_tool_calls(choice["message"]["content"])
                if calls:
                    choice["message"]["content"] = text or None
                    choice["message"]["tool_calls"] = [
                        {"id": f"call_{uuid.uuid4().hex[:16]}", "type": "function",
                         "function": {"name": c["name"], "arguments": json.dumps(c["arguments"], ensure_ascii=False)}}
                        for c in calls]
                    choice["finish_reason"] = "tool_calls"
            return JSONResponse(data)
        return resp

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
    model = checkpoint_io.from_pretrained(args.model, device=device, init="meta", **overrides)
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
    draft = checkpoint_io.from_pretrained(args.draft_model, device=device, init="meta") if args.draft_model else None
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
