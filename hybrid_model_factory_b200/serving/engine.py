"""Native serving engine: continuous batching with chunked prefill over paged K/V and slot-indexed
recurrent state.

Each ``step()`` asks the native scheduler for a batch (decodes first, then prefill chunks), runs
  * one batched decode forward for all running requests (slot-indexed decode kernels: paged GQA
    attention, fused GDN recurrent step, Mamba2 state update, conv1d update), and
  * one forward per scheduled prefill chunk through the training-path kernels with the slot's state
    as the initial state (``SlotCache``),
samples one token per request that reached the end of its known tokens, and returns the new tokens.

This replaces what the reference obtains from vLLM (scheduler, hybrid KV-cache manager, model
runner; ``vllm-inference/src/primed_vllm`` + ``docs/Inference.md``).
"""
from __future__ import annotations

import ctypes
import itertools
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..layers.attention import Attention
from ..layers.gdn import GatedDeltaNet
from ..layers.gka import GatedKalmaNet
from ..layers.mamba2 import Mamba2
from ..ops import _lib
from ..ops import functional as F_ops
from ..ops import gemm as gemm_ops
from ..ops import reference as R
from .cache import ServingState, SlotCache
from .scheduler import NativeScheduler, ScheduledSeq

c_int, c_ll, c_float = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    speculative_tokens: int = 0       # greedy requests: up to this many drafted tokens are verified per step (drafts
    #                                   come from the request's own text: the continuation of its latest repeated n-gram)
    eos_token_id: Optional[int] = None
    ignore_eos: bool = True
    stop_token_ids: tuple = ()        # generation ends after any of these tokens (the token is part of the output)
    logprobs: int = 0                 # > 0: keep the log-probability of every emitted token and of the k likeliest ones


@dataclass
class RequestState:
    req_id: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    arrival: float = 0.0
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    finished: bool = False
    finish_reason: Optional[str] = None                 # "length" | "stop" (end-of-sequence or stop token) | "abort"
    logprobs: List[tuple] = field(default_factory=list)  # per emitted token: (its logprob, [(token, logprob)] of the top k)
    ngram_index: dict = field(default_factory=dict)     # speculative decoding: n-gram -> end of its latest occurrence
    ngram_upto: int = 0
    draft_cache: Any = None                             # draft model: its cache over the first `draft_upto` tokens
    draft_upto: int = 0


def sample_tokens(logits: torch.Tensor, params: List[SamplingParams], histories=None,
                  generator: Optional[torch.Generator] = None) -> List[int]:
    """One token per row of ``logits [rows, V]``: temperature, top-k, top-p, min-p and repetition penalty
    (``histories[row]`` = token ids seen so far) for the whole batch in one kernel (``csrc/kernels/sampler.cu``) on
    the GPU, the same procedure in PyTorch elsewhere.  Rows with ``temperature <= 0`` take the arg-max."""
    rows, V = logits.shape
    pen = [p.repetition_penalty for p in params]
    use_kernel = logits.is_cuda and _lib.kernels_available() and logits.dtype in (torch.bfloat16, torch.float32)
    if histories is not None and any(x != 1.0 for x in pen):
        logits = logits.clone()
        n_max = max(1, max(len(h) for h in histories))
        ids = torch.zeros(rows, n_max, dtype=torch.long)
        for r, h in enumerate(histories):
            ids[r, :len(h)] = torch.as_tensor(list(h), dtype=torch.long)
        n_ids = torch.tensor([len(h) for h in histories], dtype=torch.int32)
        if use_kernel:
            ids, n_ids = ids.to(logits.device), n_ids.to(logits.device)
            pt = torch.tensor(pen, dtype=torch.float32, device=logits.device)
            lg = logits if logits.stride(1) == 1 else logits.contiguous()
            _lib.check(_lib.kernels().hmf_repetition_penalty(_lib.ptr(lg), c_int(int(lg.dtype == torch.bfloat16)),
                                                             c_ll(lg.stride(0)), c_int(rows), _lib.ptr(ids), c_int(n_max),
                                                             _lib.ptr(n_ids), _lib.ptr(pt), _lib.stream_ptr(lg.device)),
                       "repetition_penalty")
            logits = lg
        else:
            for r, h in enumerate(histories):
                if pen[r] != 1.0 and len(h):
                    idx = torch.as_tensor(sorted(set(h)), dtype=torch.long, device=logits.device)
                    v = logits[r, idx].float()
                    logits[r, idx] = torch.where(v > 0, v / pen[r], v * pen[r]).to(logits.dtype)
    u = torch.rand(rows, generator=generator)
    if use_kernel:
        par = torch.tensor([[p.temperature, p.top_p, p.min_p, float(u[i])] for i, p in enumerate(params)],
                           dtype=torch.float32, device=logits.device)
        topk = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=logits.device)
        out = torch.empty(rows, dtype=torch.long, device=logits.device)
        lg = logits if logits.stride(1) == 1 else logits.contiguous()
        _lib.check(_lib.kernels().hmf_sample(_lib.ptr(lg), c_int(int(lg.dtype == torch.bfloat16)), c_ll(lg.stride(0)),
                                             c_int(rows), c_int(V), _lib.ptr(par), _lib.ptr(topk), _lib.ptr(out),
                                             _lib.stream_ptr(lg.device)), "sample")
        return out.tolist()
    out = []
    for r, (row, p) in enumerate(zip(logits.float(), params)):
        if p.temperature <= 0:
            out.append(int(row.argmax()))
            continue
        pr = torch.exp((row - row.max()) / p.temperature)
        keep = torch.ones_like(pr, dtype=torch.bool)
        if p.top_k and p.top_k < V:
            keep &= pr >= torch.topk(pr, p.top_k).values[-1]
        if p.min_p > 0:
            keep &= pr >= p.min_p
        if 0 < p.top_p < 1:
            srt, order = torch.sort(torch.where(keep, pr, torch.zeros_like(pr)), descending=True)
            cum = torch.cumsum(srt, 0)
            n_keep = int((cum < p.top_p * cum[-1]).sum()) + 1
            mask = torch.zeros_like(keep)
            mask[order[:n_keep]] = True
            keep &= mask
        pr = torch.where(keep, pr, torch.zeros_like(pr))
        cdf = torch.cumsum(pr, 0)
        out.append(int(torch.searchsorted(cdf, u[r].to(cdf.device) * cdf[-1], right=True).clamp(max=V - 1)))
    return out


class ServingEngine:
    def __init__(self, model, *, block_size: int = 64, num_blocks: Optional[int] = None, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 8192, enable_prefix_caching: bool = False, max_model_len: int = 32768,
                 gpu_memory_utilization: float = 0.85, tp=None, use_cuda_graphs: bool = True,
                 whole_prompts: bool = True, draft_model=None):
        self.model = model.eval()
        # speculative decoding: a small model of the same vocabulary proposes tokens where the request's own n-grams
        # offer none (it runs with the plain per-request cache of `models/cache.py`, not the paged one)
        self.draft_model = None if draft_model is None else draft_model.eval()
        self.cfg = model.config
        self.device = next(model.parameters()).device
        self.tp = tp
        self.block_size = block_size
        has_ssm = any(not isinstance(l.seq_mixer, Attention) for l in model.model.layers)
        n_attn = sum(isinstance(l.seq_mixer, Attention) for l in model.model.layers)
        if num_blocks is None:
            num_blocks = self._plan_blocks(n_attn, block_size, max_num_seqs, max_model_len, gpu_memory_utilization)
        snapshots = max_num_seqs if (enable_prefix_caching and has_ssm) else 0
        # one extra block and one extra slot absorb the padding rows of a bucketed (graph-captured) decode batch
        # ... and one more slot holds the recurrent state of a request while its drafted tokens are verified
        self._spec_slots = min(max_num_seqs, 8)       # requests whose drafts are verified in the same step
        self.state = ServingState(model, num_blocks + 1, block_size, max_num_seqs, snapshots + 1 + self._spec_slots,
                                  self.device, dtype=next(model.parameters()).dtype)
        self._pad_block, self._pad_slot = num_blocks, max_num_seqs + snapshots
        self._spec_slot = max_num_seqs + snapshots + 1
        self.spec_ngram = (4, 2)          # longest / shortest n-gram looked up for a draft
        self.sched = NativeScheduler(num_blocks, block_size, max_num_seqs, max_num_seqs, max_num_batched_tokens,
                                     enable_prefix_caching, snapshots, require_snapshot=has_ssm,
                                     whole_prompts=whole_prompts)
        self.prefix_caching = enable_prefix_caching
        self.requests: Dict[int, RequestState] = {}
        self._ids = itertools.count()
        self._cuda = self.device.type == "cuda" and _lib.kernels_available()
        self._layer_cache: Dict[int, dict] = {}
        self.max_blocks_per_seq = (max_model_len + block_size - 1) // block_size
        self.stats = {"steps": 0, "decode_tokens": 0, "prefill_tokens": 0, "graph_replays": 0, "decode_steps": 0, "packed_prefills": 0,
                      "spec_steps": 0, "spec_drafted": 0, "spec_accepted": 0, "spec_model_drafts": 0,
                      "decode_s": 0.0, "prefill_s": 0.0, "decode_gpu_s": 0.0}
        has_moe = any(hasattr(l.mlp, "experts") for l in model.model.layers)
        # B'MOJO-F layers decode request by request through the layer itself (bounded window state per request)
        self.packed_prefill = True      # several requests' prefill pieces of one step share a forward
        self.status_check_steps = 64    # tensor parallelism: how often the kernels' wait-status block is read
        # MoE layers: the bf16 expert path sorts and pads its rows on the device with static shapes (`ops/moe.py`), so
        # the decode step stays capturable; other dtypes take a per-expert loop with a host read and run eagerly
        moe_ok = not has_moe or next(model.parameters()).dtype == torch.bfloat16
        self._use_graphs = bool(use_cuda_graphs and self._cuda and moe_ok and not self.state.bmojo_layers)
        self._graphs: Dict[tuple, dict] = {}
        self._tables: Dict[int, torch.Tensor] = {}
        self._timed_replay = False
        self._events = ((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                        if self._cuda else None)

    def _plan_blocks(self, n_attn, block_size, max_seqs, max_len, util) -> int:
        need = max_seqs * ((max_len + block_size - 1) // block_size)
        if self.device.type != "cuda" or n_attn == 0:
            return max(need if n_attn else 8, 8)
        free, total = torch.cuda.mem_get_info(self.device)
        a = next(l.seq_mixer for l in self.model.model.layers if isinstance(l.seq_mixer, Attention))
        per_block = 2 * block_size * a.num_kv_heads * a.head_dim * 2 * n_attn
        budget = int(free - (1 - util) * total)
        return int(max(64, min(need, budget // max(per_block, 1))))

    # -- request API -----------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        rid = next(self._ids)
        self.requests[rid] = RequestState(rid, list(prompt), params, arrival=time.perf_counter())
        self.sched.add_request(rid, list(prompt), params.max_new_tokens)
        return rid

    def has_unfinished(self) -> bool:
        return any(not r.finished for r in self.requests.values())

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> List[List[int]]:
        ids = [self.add_request(p, params) for p in prompts]
        while any(not self.requests[i].finished for i in ids):
            self.step()
        return [self.requests[i].output for i in ids]

    # -- one engine step -------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> List[tuple]:
        batch = self.sched.step()
        if not batch:
            return []
        self.stats["steps"] += 1
        decodes = [s for s in batch if s.is_decode and self._at_frontier(s)]
        prefills = [s for s in batch if s not in decodes]
        results = []
        # speculative decoding: the requests with a usable draft are verified together in one packed forward (several
        # tokens each); the others share the batched decode step below
        decodes, verified = self._speculate(decodes)
        for s, toks in verified:
            for t in toks:
                self.sched.advance(s.req_id, 1)
                res = self._emit(s.req_id, int(t))
                results.append(res)
                self.stats["decode_tokens"] += 1
                if res[2]:
                    break
        t0 = time.perf_counter()
        if decodes:
            # longest contexts first: the attention kernel's CTAs are issued in row order, so the long rows start early
            # and the short ones fill the last wave instead of the other way round
            decodes.sort(key=lambda s: -s.start_pos)
            logits = self._decode_forward(decodes)
            reqs = [self.requests[s.req_id] for s in decodes]
            hist = [r.prompt + r.output for r in reqs] if any(r.params.repetition_penalty != 1.0 for r in reqs) else None
            toks = self._sample(logits, [r.params for r in reqs], hist)
            if self._timed_replay:      # the sampled ids were read back, so the replay has finished
                self.stats["decode_gpu_s"] += self._events[0].elapsed_time(self._events[1]) * 1e-3
                self._timed_replay = False
            for row, (s, t) in enumerate(zip(decodes, toks)):
                self.sched.advance(s.req_id, 1)
                self._note_logprobs(s.req_id, logits[row], int(t))
                results.append(self._emit(s.req_id, int(t)))
            self.stats["decode_tokens"] += len(decodes)
            self.stats["decode_steps"] += 1
            self.stats["decode_s"] += time.perf_counter() - t0
        t0 = time.perf_counter()
        packed = None
        if len(prefills) > 1 and self.packed_prefill and not self.state.bmojo_layers:
            # the pieces of several requests as ONE row with sample boundaries: embeddings, norms, MLPs and the
            # vocabulary projection run once for all of them, every mixer once per piece with that request's cache
            for s in prefills:
                if s.restore_from >= 0:
                    self.state.copy_slot(s.restore_from, s.slot)
            packed = self._prefill_forward_packed(prefills)
            self.stats["packed_prefills"] += 1
        for i, s in enumerate(prefills):
            req = self.requests[s.req_id]
            tokens = (req.prompt + req.output)[s.start_pos:s.start_pos + s.num_tokens]
            if packed is not None:
                logits = packed[i:i + 1]
            else:
                if s.restore_from >= 0:
                    self.state.copy_slot(s.restore_from, s.slot)
                logits = self._prefill_forward(s, tokens)
            self.sched.advance(s.req_id, s.num_tokens)
            self.stats["prefill_tokens"] += s.num_tokens
            end = s.start_pos + s.num_tokens
            if self.prefix_caching and self.state.ssm and end % self.block_size == 0 and end < len(req.prompt):
                snap = self.sched.register_snapshot(s.req_id, end)
                if snap >= 0:
                    self.state.copy_slot(s.slot, snap)
            if end >= len(req.prompt) + len(req.output):
                hist = [req.prompt + req.output] if req.params.repetition_penalty != 1.0 else None
                tok = self._sample(logits[-1:], [req.params], hist)[0]
                self._note_logprobs(s.req_id, logits[-1], int(tok))
                results.append(self._emit(s.req_id, int(tok)))
        if prefills:
            self.stats["prefill_s"] += time.perf_counter() - t0
        if (self.tp is not None and self.tp.size > 1 and self._cuda
                and self.stats["steps"] % self.status_check_steps == 0):
            self.check_kernel_status()
        return results

    def check_kernel_status(self, status_reader=None) -> None:
        """Raises ``KernelError`` when a device-side wait ran out since the last check (a late or missing peer in a
        fused GEMM + reduction): such a kernel returns and the step goes on with partial sums, so the tokens produced
        since then are not valid.  Read every ``status_check_steps`` steps of a tensor-parallel engine (one small
        device-to-host read)."""
        code, block, detail, count = (status_reader or _lib.read_status)()
        if code != 0:
            raise _lib.KernelError(
                f"engine step {self.stats['steps']}: a device-side wait ran out (code={code} block={block} "
                f"detail={detail:#x} count={count}); HMF_TP_FUSED=0 selects the NCCL reductions")

    # -- speculative decoding ----------------------------------------------------------------------
    def _draft(self, req: "RequestState", seq: List[int], k: int) -> List[int]:
        """Continuation of the latest earlier occurrence of the sequence's last n tokens (longest n first).  The
        request keeps an index ``n-gram -> end of its latest occurrence`` that grows with the sequence, so a lookup
        costs a few dictionary reads whatever the context length."""
        hi, lo = self.spec_ngram
        index, upto = req.ngram_index, req.ngram_upto
        for e in range(max(upto, lo), len(seq)):              # n-grams that end before the last token
            for n in range(lo, min(hi, e) + 1):
                index[tuple(seq[e - n:e])] = e
        req.ngram_upto = len(seq)
        for n in range(min(hi, len(seq) - 1), lo - 1, -1):
            e = index.get(tuple(seq[-n:]))
            if e is not None:
                return seq[e:e + k]
        if self.draft_model is not None:
            return self._draft_with_model(req, seq, k)
        return []

    @torch.no_grad()
    def _draft_with_model(self, req: "RequestState", seq: List[int], k: int) -> List[int]:
        """``k`` greedy tokens of the draft model after ``seq``.  The draft's cache is kept at the verified prefix: it
        first reads the tokens verified since its last turn, a snapshot is taken, the drafts are generated, and the
        snapshot becomes the request's cache again (the next turn reads whatever part of the drafts was accepted)."""
        from ..models.cache import HybridCache
        cache = req.draft_cache if req.draft_cache is not None else HybridCache()
        dev = next(self.draft_model.parameters()).device
        if len(seq) - 1 > req.draft_upto:
            ids = torch.tensor([seq[req.draft_upto:len(seq) - 1]], dtype=torch.long, device=dev)
            self.draft_model(input_ids=ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
            req.draft_upto = len(seq) - 1
        keep = cache.snapshot()
        tok, out = seq[-1], []
        for _ in range(k):
            ids = torch.tensor([[tok]], dtype=torch.long, device=dev)
            logits = self.draft_model(input_ids=ids, past_key_values=cache, use_cache=True).logits[0, -1]
            tok = int(logits.argmax())
            out.append(tok)
        req.draft_cache = keep
        self.stats["spec_model_drafts"] += 1
        return out

    def _speculate(self, decodes: List[ScheduledSeq]):
        """Verifies drafted tokens for the decoding requests that have some.  Returns ``(plain, verified)``: the
        requests left to the ordinary decode step, and ``(request, tokens to emit)`` pairs (accepted drafts + the
        model's own next token).

        Each request's drafts run as one piece of ``1 + k`` tokens, exactly like a prefill continuation, all pieces of
        the step packed into one forward; the greedy targets of every position come out of it.  Attention needs no undo
        (cache entries after the accepted prefix are overwritten later).  The recurrent state does: it is copied to a
        spare slot first, and after a rejection it is restored and advanced again over the accepted prefix only (one
        more packed forward for all rejected requests), which is what starting from the state "after ``num_accepted``
        tokens" means for a recurrence (reference: ``num_accepted_tokens`` in
        ``vllm-inference/src/primed_vllm/layers/gdn/ops/fused_recurrent_gqa.py:24-154``)."""
        plain, cand = [], []
        for s in decodes:
            req = self.requests[s.req_id]
            p = req.params
            drafts: List[int] = []
            if (p.speculative_tokens > 0 and p.temperature <= 0 and p.repetition_penalty == 1.0
                    and not self.state.bmojo_layers and len(cand) < self._spec_slots):
                seq = req.prompt + req.output
                capacity = len(self.sched.block_table(s.req_id)) * self.block_size
                k = min(p.speculative_tokens, capacity - 1 - s.start_pos, p.max_new_tokens - len(req.output) - 1)
                drafts = self._draft(req, seq, k) if k > 0 else []
            if drafts:
                cand.append((s, [(req.prompt + req.output)[s.start_pos]] + drafts))
            else:
                plain.append(s)
        if not cand:
            return plain, []
        has_state = bool(self.state.ssm)
        if has_state:
            for j, (s, _) in enumerate(cand):
                self.state.copy_slot(s.slot, self._spec_slot + j)
        logits, cu = self._pieces_forward(cand)
        params = [self.requests[s.req_id].params for s, toks in cand for _ in toks]
        targets = self._sample(logits, params)
        verified, redo = [], []
        for j, (s, toks) in enumerate(cand):
            mine, drafts = targets[cu[j]:cu[j + 1]], toks[1:]
            n_acc = 0
            while n_acc < len(drafts) and drafts[n_acc] == mine[n_acc]:
                n_acc += 1
            if n_acc < len(drafts) and has_state:
                self.state.copy_slot(self._spec_slot + j, s.slot)
                redo.append((s, toks[:n_acc + 1]))
            self.stats["spec_drafted"] += len(drafts)
            self.stats["spec_accepted"] += n_acc
            for i in range(n_acc + 1):
                self._note_logprobs(s.req_id, logits[cu[j] + i], int(mine[i]))
            verified.append((s, mine[:n_acc + 1]))
        if redo:
            self._pieces_forward(redo, want_logits=False)
        self.stats["spec_steps"] += 1
        return plain, verified

    def _pieces_forward(self, items, want_logits: bool = True):
        """One packed forward over ``(request, tokens)`` pieces, each continuing its request at ``start_pos`` with the
        request's caches.  Returns ``(logits of every position, piece boundaries)``."""
        toks, pos, cu, caches = [], [], [0], []
        for s, t in items:
            toks += t
            pos += list(range(s.start_pos, s.start_pos + len(t)))
            cu.append(len(toks))
            caches.append(SlotCache(self.state, s.slot, self.sched.block_table(s.req_id), s.start_pos, None))
        ids = torch.tensor([toks], dtype=torch.long, device=self.device)
        pid = torch.tensor([pos], dtype=torch.long, device=self.device)
        h, _ = self.model.model(ids, position_ids=pid, cu_seqlens=cu, sample_caches=caches)
        return (self._logits(h[0]) if want_logits else None), cu

    def close(self) -> None:
        """Drops the captured decode graphs.  A graph that holds NCCL kernels (tensor parallelism) keeps its
        communicator busy: the process group cannot shut down while such a graph exists, and an engine that is only
        unreachable (it sits in a reference cycle with its serving thread) still counts.  Call this before
        ``destroy_process_group``."""
        self._graphs.clear()
        if self._cuda:
            torch.cuda.synchronize(self.device)

    def _at_frontier(self, s: ScheduledSeq) -> bool:
        req = self.requests[s.req_id]
        return s.start_pos == len(req.prompt) + len(req.output) - 1

    def _emit(self, rid: int, tok: int):
        req = self.requests[rid]
        now = time.perf_counter()
        if req.first_token_time is None:
            req.first_token_time = now
        req.output.append(tok)
        self.sched.append_token(rid, tok)
        p = req.params
        stopped = (not p.ignore_eos and p.eos_token_id is not None and tok == p.eos_token_id) or \
            (bool(p.stop_token_ids) and tok in p.stop_token_ids)
        done = stopped or len(req.output) >= p.max_new_tokens
        if done:
            self._retire(req, "stop" if stopped else "length", now)
        return (rid, tok, done)

    def _note_logprobs(self, rid: int, row: torch.Tensor, tok: int) -> None:
        """Log-probabilities of the model's distribution (before temperature / penalties) for a token about to be
        emitted, when the request asked for them."""
        req = self.requests[rid]
        k = req.params.logprobs
        if k <= 0:
            return
        lp = torch.log_softmax(row.float(), dim=-1)
        top = lp.topk(min(k, lp.numel()))
        req.logprobs.append((float(lp[tok]), list(zip(top.indices.tolist(), top.values.tolist()))))

    def _retire(self, req: "RequestState", reason: str, now: float) -> None:
        req.finished, req.finish_time, req.finish_reason = True, now, reason
        req.draft_cache = None
        del req.logprobs[len(req.output):]          # (a verify step may have scored tokens past the end)
        self.sched.finish(req.req_id)
        self._tables.pop(req.req_id, None)
        self.state.side.pop(req.req_id, None)

    def abort(self, req_id: int) -> bool:
        """Ends a request between steps (a stop string seen by the caller, a client that went away): its blocks and
        state slot are free for the next step.  Under tensor parallelism every rank has to abort the same request
        before the same step (the API server sends it through the control channel).  Returns whether it was live."""
        req = self.requests.get(req_id)
        if req is None or req.finished:
            return False
        self._retire(req, "abort", time.perf_counter())
        return True

    # -- sampling ------------------------------------------------------------------------------
    def _sample(self, logits: torch.Tensor, params: List[SamplingParams], histories=None) -> List[int]:
        if all(p.temperature <= 0 for p in params):
            if self._cuda and logits.is_cuda:
                ids = torch.empty(logits.shape[0], dtype=torch.long, device=logits.device)
                lg = logits.contiguous()
                _lib.check(_lib.kernels().hmf_argmax(_lib.ptr(lg), c_int(int(lg.dtype == torch.bfloat16)), _lib.ptr(ids),
                                                     c_int(lg.shape[0]), c_int(lg.shape[1]), c_ll(lg.stride(0)),
                                                     _lib.stream_ptr(lg.device)), "argmax")
                if lg.dtype not in (torch.bfloat16, torch.float32):
                    ids = lg.float().argmax(-1)
                return ids.tolist()
            return logits.float().argmax(-1).tolist()
        return sample_tokens(logits, params, histories)

    # -- prefill (per request chunk) -------------------------------------------------------------
    def _prefill_forward(self, s: ScheduledSeq, tokens: List[int]) -> torch.Tensor:
        ids = torch.tensor([tokens], dtype=torch.long, device=self.device)
        pos = torch.arange(s.start_pos, s.start_pos + len(tokens), device=self.device)[None]
        side = self.state.side_cache(s.req_id) if self.state.bmojo_layers else None
        if side is not None:
            side.seqlen_offset = s.start_pos
        cache = SlotCache(self.state, s.slot, self.sched.block_table(s.req_id), s.start_pos, side)
        h, _ = self.model.model(ids, position_ids=pos, past_key_values=cache, use_cache=True)
        return self._logits(h[0, -1:])

    def _prefill_forward_packed(self, pieces: List[ScheduledSeq]) -> torch.Tensor:
        """One forward for the prefill pieces of several requests; returns the logits at each piece's last token."""
        toks, pos, cu, caches = [], [], [0], []
        for s in pieces:
            req = self.requests[s.req_id]
            t = (req.prompt + req.output)[s.start_pos:s.start_pos + s.num_tokens]
            toks += t
            pos += list(range(s.start_pos, s.start_pos + len(t)))
            cu.append(len(toks))
            caches.append(SlotCache(self.state, s.slot, self.sched.block_table(s.req_id), s.start_pos, None))
        ids = torch.tensor([toks], dtype=torch.long, device=self.device)
        pid = torch.tensor([pos], dtype=torch.long, device=self.device)
        h, _ = self.model.model(ids, position_ids=pid, cu_seqlens=cu, sample_caches=caches)
        last = torch.tensor([c - 1 for c in cu[1:]], dtype=torch.long, device=self.device)
        return self._logits(h[0, last])

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.model.lm_head(h)
        if self.tp is not None:
            logits = self.tp.gather_logits(logits)
        return logits

    # -- batched decode ----------------------------------------------------------------------------
    def _decode_forward(self, seqs: List[ScheduledSeq]) -> torch.Tensor:
        """Batched single-token forward.  On the GPU the whole step (embedding to logits) is captured once per
        (batch bucket, KV split count) in a CUDA graph and replayed from static input buffers."""
        Rn = len(seqs)
        last = []
        for s in seqs:
            rq = self.requests[s.req_id]
            n = len(rq.prompt)
            last.append(rq.prompt[s.start_pos] if s.start_pos < n else rq.output[s.start_pos - n])
        pos = [s.start_pos for s in seqs]
        slots = [s.slot for s in seqs]
        tables = [self._table(s.req_id, s.start_pos) for s in seqs] if self.state.kv else None
        max_len = max(pos) + 1
        if not self._use_graphs:
            inp = self._decode_inputs(Rn, max(len(t) for t in tables) if tables else 1)
            self._fill_inputs(inp, last, pos, slots, tables)
            inp["req_ids"] = [s.req_id for s in seqs]
            return self._decode_body(inp, self._splits_for(Rn, max_len))
        Rb = 1
        while Rb < Rn:
            Rb *= 2
        Rb = min(Rb, max(self.sched.max_num_seqs, Rn))
        splits = self._splits_for(Rb, max_len)
        key = (Rb, splits)
        g = self._graphs.get(key)
        if g is None:
            try:
                g = self._capture(Rb, splits, last, pos, slots, tables)
            except Exception as e:      # an op that cannot be captured (host sync in a fallback path): run eagerly
                import warnings
                warnings.warn(f"CUDA graph capture of the decode step failed ({e}); continuing without graphs")
                self._use_graphs = False
                torch.cuda.synchronize(self.device)
                self.state.clear_slot(self._pad_slot)
                return self._decode_forward(seqs)
            self._graphs[key] = g
        self._fill_inputs(g["inp"], last, pos, slots, tables)
        ev = self._events
        ev[0].record()
        g["graph"].replay()
        ev[1].record()
        self._timed_replay = True
        self.stats["graph_replays"] += 1
        return g["logits"][:Rn]

    def _table(self, rid: int, pos: int):
        """Block table of a decoding request, re-read from the scheduler only when a new block was appended."""
        t = self._tables.get(rid)
        if t is None or pos // self.block_size >= len(t):
            t = torch.from_numpy(self.sched.block_table_array(rid))
            self._tables[rid] = t
        return t

    def warmup(self, max_len: Optional[int] = None, every_length: bool = False) -> int:
        """Captures the decode graphs of every batch bucket up front: for the shortest and the longest context, or
        (``every_length``) for every KV split count a context between them can select, so that nothing is captured
        later (a server replays from a thread other than the one that captured)."""
        if not self._use_graphs:
            return 0
        longest = max_len or self.max_blocks_per_seq * self.block_size
        lengths = {1, longest}
        if every_length:
            ml = 512
            while ml < longest:
                lengths.add(ml)
                ml *= 2
        n, rows = 0, 1
        while True:
            rows = min(rows, self.sched.max_num_seqs)
            for ml in sorted(lengths):
                key = (rows, self._splits_for(rows, ml))
                if key not in self._graphs:
                    tables = [[self._pad_block]] * rows if self.state.kv else None
                    self._graphs[key] = self._capture(rows, key[1], [0] * rows, [0] * rows, [self._pad_slot] * rows, tables)
                    n += 1
            if rows >= self.sched.max_num_seqs:
                return n
            rows *= 2

    def _splits_for(self, rows: int, max_len: int) -> int:
        """KV splits of the paged attention kernel: enough CTAs for two waves over the SMs on long contexts."""
        if max_len <= 1024 or not self.state.kv:
            return 1
        a = next(l.seq_mixer for l in self.model.model.layers if isinstance(l.seq_mixer, Attention))
        ctas = rows * a.num_kv_heads
        sp = 1
        while sp < 64 and ctas * sp < 148 and sp * 256 < max_len:
            sp *= 2
        if sp == 1 and max_len >= 4096:
            # long contexts: two splits balance rows of unequal length better (17.2 against 17.75 ms per decode step of
            # the serving workload; four splits, with the kernel's one-split-per-2048-tokens rule, gave 17.4 ms)
            sp = 2
        return sp

    def _decode_inputs(self, rows: int, mb: int) -> dict:
        dev = self.device
        pin = dev.type == "cuda"
        host = {"ids": torch.zeros(rows, dtype=torch.long, pin_memory=pin),
                "pos": torch.zeros(rows, dtype=torch.long, pin_memory=pin),
                "slots": torch.zeros(rows, dtype=torch.int32, pin_memory=pin),
                "bt": torch.zeros(rows, mb, dtype=torch.int32, pin_memory=pin)}
        d = {k: torch.zeros_like(v, device=dev) for k, v in host.items()}
        d.update(host=host, rows=rows, mb=mb)
        return d

    def _fill_inputs(self, inp: dict, last, pos, slots, tables) -> None:
        h, Rn, rows = inp["host"], len(last), inp["rows"]
        h["ids"][:Rn] = torch.tensor(last, dtype=torch.long)
        h["pos"][:Rn] = torch.tensor(pos, dtype=torch.long)
        h["slots"][:Rn] = torch.tensor(slots, dtype=torch.int32)
        if Rn < rows:                       # padding rows: token 0 at position 0 of the spare slot / block
            h["ids"][Rn:] = 0
            h["pos"][Rn:] = 0
            h["slots"][Rn:] = self._pad_slot
        if tables is not None:
            bt = h["bt"]
            bt.fill_(self._pad_block)
            for i, t in enumerate(tables):
                bt[i, :len(t)] = t if isinstance(t, torch.Tensor) else torch.tensor(t, dtype=torch.int32)
        for k in ("ids", "pos", "slots", "bt"):
            inp[k].copy_(h[k], non_blocking=True)

    def _capture(self, rows: int, splits: int, last, pos, slots, tables) -> dict:
        inp = self._decode_inputs(rows, self.max_blocks_per_seq)
        # warm-up on the padding slot only (real state must not advance twice): lazy initialisation, workspaces
        n = len(last)
        self._fill_inputs(inp, [0] * n, [0] * n, [self._pad_slot] * n, None if tables is None else [[self._pad_block]] * n)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._decode_body(inp, splits)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            logits = self._decode_body(inp, splits)
        self.state.clear_slot(self._pad_slot)
        return {"graph": graph, "inp": inp, "logits": logits}

    def _decode_body(self, inp: dict, splits: int) -> torch.Tensor:
        m = self.model.model
        ids, pos, slots = inp["ids"], inp["pos"], inp["slots"]
        Rn = ids.shape[0]
        x = m.embed_tokens(ids)                                    # [R, Dm]
        cos, sin = m.rotary_emb(pos[:, None])                        # [R, 1, rot]
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        meta = None
        if self.state.kv:
            bs = self.block_size
            bt = inp["bt"]
            slot_map = (bt[torch.arange(Rn, device=bt.device), pos // bs].to(torch.long) * bs + pos % bs)
            meta = {"bt": bt, "mb": bt.shape[1], "slot_map": slot_map.contiguous(), "lens": (pos + 1).to(torch.int32),
                    "splits": splits}
        res, pending = x, None
        for i, layer in enumerate(m.layers):
            h, res = self._add_norm(pending, res, layer.input_layernorm)
            mixer = layer.seq_mixer
            if isinstance(mixer, Attention):
                y = self._attn_decode(i, mixer, h, cos, sin, meta)
            elif isinstance(mixer, GatedDeltaNet):
                y = self._gdn_decode(i, mixer, h, slots)
            elif isinstance(mixer, Mamba2):
                y = self._mamba_decode(i, mixer, h, cos, sin, slots)
            elif isinstance(mixer, GatedKalmaNet):
                y = self._gka_decode(i, mixer, h, slots)
            elif i in self.state.bmojo_layers:
                y = self._bmojo_decode(mixer, h, pos, cos, sin, inp["req_ids"])
            else:
                raise NotImplementedError(type(mixer).__name__)
            h2, res = self._add_norm(y, res, layer.post_attention_layernorm)
            pending = self._mlp_decode(i, layer.mlp, h2)
        h, _ = self._add_norm(pending, res, m.norm)
        return self._logits(h)

    def _add_norm(self, y, res, norm):
        """``res + y`` followed by RMSNorm, in one kernel on the GPU.  Returns ``(normed, new residual)``."""
        if y is None:
            return norm(res), res
        if self._cuda and res.dtype == torch.bfloat16 and not getattr(norm, "zero_centered", False):
            return F_ops.fused_add_rms_norm(y, res, norm.weight, norm.variance_epsilon)
        res = res + y
        return norm(res), res

    def _mlp_decode(self, i, mlp, h):
        from ..layers.common import MLP
        if not (self._cuda and isinstance(mlp, MLP) and h.dtype == torch.bfloat16 and mlp.gate_proj.bias is None):
            y = mlp(h)                       # (under TP the MLP's forward hook reduces the partial sums)
            return y[0] if isinstance(y, tuple) else y
        c = self._layer_cache.setdefault(("mlp", i), {})
        if not c:
            c["w_gu"] = torch.cat([mlp.gate_proj.weight, mlp.up_proj.weight], dim=0).contiguous()
        gu = gemm_ops.linear(h, c["w_gu"])
        Fi = gu.shape[-1] // 2
        a = torch.empty(h.shape[0], Fi, device=h.device, dtype=h.dtype)
        _lib.check(_lib.kernels().hmf_swiglu_packed(_lib.ptr(gu), _lib.ptr(a), c_ll(h.shape[0]), c_int(Fi),
                                                    c_ll(gu.stride(0)), _lib.stream_ptr(h.device)), "swiglu_packed")
        return self._row_linear(a, mlp.down_proj)

    def _row_linear(self, x, lin):
        """Output projection of a mixer / MLP: under TP the weight is a row-parallel shard and the partial sums
        are reduced inside the GEMM kernel (peer memory) or by NCCL."""
        if self.tp is None or self.tp.size == 1:
            return lin(x)
        if lin.bias is None:
            return self.tp.linear_allreduce(x, lin.weight)
        return self.tp.all_reduce(lin(x))

    def _attn_decode(self, i, mx: Attention, h, cos, sin, meta):
        Rn = h.shape[0]
        fused = (self._cuda and mx.head_dim == 128 and h.dtype == torch.bfloat16 and not mx.gated
                 and cos.shape[-1] % 2 == 0)
        gate = None
        if fused:
            c = self._layer_cache.setdefault(("attn", i), {})
            if not c:
                c["w"] = torch.cat([mx.q_proj.weight, mx.k_proj.weight, mx.v_proj.weight], dim=0).contiguous()
                c["b"] = (torch.cat([mx.q_proj.bias, mx.k_proj.bias, mx.v_proj.bias]).contiguous()
                          if mx.q_proj.bias is not None else None)
            qkv = gemm_ops.linear(h, c["w"], c["b"])
            kc, vc = self.state.kv[i]
            q = torch.empty(Rn, mx.num_heads, mx.head_dim, device=h.device, dtype=h.dtype)
            qn = mx.q_norm
            cs, sn = cos.reshape(Rn, -1).contiguous(), sin.reshape(Rn, -1).contiguous()
            _lib.check(_lib.kernels().hmf_qkv_norm_rope_append(
                _lib.ptr(qkv), c_ll(qkv.stride(0)), _lib.ptr(qn.weight if qn is not None else None),
                _lib.ptr(mx.k_norm.weight if qn is not None else None),
                c_float(qn.variance_epsilon if qn is not None else 0.0),
                c_int(int(getattr(qn, "zero_centered", False)) if qn is not None else 0), _lib.ptr(cs), _lib.ptr(sn),
                c_int(cs.shape[-1]), _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(meta["slot_map"]), c_int(Rn),
                c_int(mx.num_heads), c_int(mx.num_kv_heads), c_int(mx.head_dim), _lib.stream_ptr(h.device)),
                "qkv_norm_rope_append")
            k = v = None
        else:
            q = mx.q_proj(h)
            if mx.gated:
                q = q.view(Rn, mx.num_heads, 2 * mx.head_dim)
                q, gate = q[..., :mx.head_dim], q[..., mx.head_dim:].reshape(Rn, -1)
            q = q.reshape(Rn, 1, mx.num_heads, mx.head_dim)
            k = mx.k_proj(h).view(Rn, 1, mx.num_kv_heads, mx.head_dim)
            v = mx.v_proj(h).view(Rn, mx.num_kv_heads, mx.head_dim)
            if mx.q_norm is not None:
                q, k = mx.q_norm(q), mx.k_norm(k)
            q, k = F_ops.apply_rope(q, cos, sin)[:, 0], F_ops.apply_rope(k, cos, sin)[:, 0]
        beta = (getattr(mx.config, "rope_scaling", None) or {}).get("llama_4_scaling_beta")
        if beta:        # query temperature beyond the original context (see ``Attention.forward``); position = length - 1
            old = float(mx.config.rope_scaling.get("original_max_position_embeddings") or 0) or float("inf")
            pos = meta["lens"].to(torch.float32) - 1.0
            q = q * (1.0 + float(beta) * torch.log1p(torch.floor(pos / old))).view(Rn, 1, 1).to(q.dtype)
        kc, vc = self.state.kv[i]
        window = mx.sliding_window or 0
        if self._cuda and mx.head_dim == 128 and q.dtype == torch.bfloat16:
            K = _lib.kernels()
            q = q.contiguous()
            if k is not None:
                k, v = k.contiguous(), v.contiguous()
                _lib.check(K.hmf_cache_append(_lib.ptr(k), _lib.ptr(v), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(meta["slot_map"]),
                                              c_ll(Rn), c_int(mx.num_kv_heads), c_int(mx.head_dim), c_ll(k.stride(0)),
                                              c_ll(v.stride(0)), _lib.stream_ptr(h.device)), "cache_append")
            splits = meta["splits"]
            o = torch.empty(Rn, mx.num_heads, mx.head_dim, device=h.device, dtype=h.dtype)
            po = torch.empty(Rn, mx.num_heads, splits, mx.head_dim, device=h.device, dtype=torch.float32)
            pml = torch.empty(Rn, mx.num_heads, splits, 2, device=h.device, dtype=torch.float32)
            if self.block_size % 64 == 0 and self.block_size <= 256:
                # tcgen05 kernel: K/V tiles by TMA straight from the paged cache, accumulators in tensor memory
                _lib.check(K.hmf_paged_attention_decode_tc(
                    _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(meta["bt"]), _lib.ptr(meta["lens"]), _lib.ptr(o),
                    _lib.ptr(po), _lib.ptr(pml), c_int(Rn), c_int(mx.num_heads), c_int(mx.num_kv_heads),
                    c_int(mx.head_dim), c_int(self.block_size), c_int(kc.shape[0]), c_int(meta["mb"]), c_int(splits),
                    c_int(window), c_float(mx.scaling), _lib.stream_ptr(h.device)), "paged_attention_decode_tc")
            else:
                _lib.check(K.hmf_paged_attention_decode(
                    _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(meta["bt"]), _lib.ptr(meta["lens"]), _lib.ptr(o),
                    _lib.ptr(po), _lib.ptr(pml), c_int(Rn), c_int(mx.num_heads), c_int(mx.num_kv_heads),
                    c_int(mx.head_dim), c_int(self.block_size), c_int(meta["mb"]), c_int(splits), c_int(window),
                    c_float(mx.scaling), _lib.stream_ptr(h.device)), "paged_attention_decode")
        else:
            kc.view(-1, *kc.shape[2:])[meta["slot_map"]] = k
            vc.view(-1, *vc.shape[2:])[meta["slot_map"]] = v
            outs = []
            bs = self.block_size
            for r in range(Rn):
                L = int(meta["lens"][r])
                p_ = torch.arange(L, device=h.device)
                flat = meta["bt"][r].long()[p_ // bs] * bs + p_ % bs
                kk, vv = kc.view(-1, *kc.shape[2:])[flat][None], vc.view(-1, *vc.shape[2:])[flat][None]
                outs.append(R.attention(q[r][None, None], kk, vv, scale=mx.scaling, window=window or None)[0, 0])
            o = torch.stack(outs)
        o = o.reshape(Rn, -1)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self._row_linear(o, mx.o_proj)

    def _bmojo_decode(self, mixer, h, pos, cos, sin, req_ids):
        """B'MOJO-F: one call of the layer per request with that request's window cache."""
        outs = []
        for r, rid in enumerate(req_ids):
            side = self.state.side_cache(rid)
            side.seqlen_offset = int(pos[r])
            cache = SlotCache(self.state, -1, [], int(pos[r]), side)
            y, _, _ = mixer(h[r:r + 1, None], position_embeddings=(cos[r:r + 1], sin[r:r + 1]),
                            position_ids=pos[r:r + 1, None], past_key_values=cache, use_cache=True)
            outs.append(y[:, 0])
        out = torch.cat(outs, dim=0)
        return self.tp.all_reduce(out) if self.tp is not None and self.tp.size > 1 else out

    def _conv_update(self, i, x_cat, weight, bias, slots):
        e = self.state.ssm[i]
        if self._cuda and x_cat.dtype == torch.bfloat16:
            from ..ops import cuda_ops
            y, _ = cuda_ops.causal_conv1d_update(x_cat, e["conv"], weight, bias, "silu", slots)
            return y
        st = e["conv"][slots.long()]
        y, new = R.causal_conv1d_update(x_cat, st, weight, bias, "silu")
        e["conv"][slots.long()] = new.to(e["conv"].dtype)
        return y

    def _packed(self, key, mods):
        """Several projections of the same input as ONE weight (rows concatenated, padded with zero rows to whole
        128-row tiles so the decode GEMM kernel takes it; the reference merges the input projections of its serving
        layers the same way, ``vllm-inference/src/primed_vllm/layers/gdn/primed_gdn_layer.py``).  The modules' own
        weights become views of the packed tensor, so nothing is held twice.  Every projection starts at a multiple of
        8 output columns: with one decoding request the slices of the product are handed to kernels as they are, and
        those read 16 bytes at a time.  ``{"w": None}`` when the modules are not plain linears of one kind."""
        c = self._layer_cache.get(key)
        if c is None:
            plain = all(isinstance(m, torch.nn.Linear) for m in mods)
            if (not plain or len({m.weight.dtype for m in mods}) != 1
                    or any(m.weight.shape[0] % 8 for m in mods[:3])):      # q, k, v are read as one contiguous block
                c = {"w": None}
            else:
                sizes = [m.weight.shape[0] for m in mods]
                offs, n = [], 0
                for sz in sizes:
                    offs.append(n)
                    n += (sz + 7) // 8 * 8
                w0 = mods[0].weight
                W = torch.zeros((n + 127) // 128 * 128, w0.shape[1], dtype=w0.dtype, device=w0.device)
                b = None
                if any(m.bias is not None for m in mods):       # zero where a projection has no bias
                    b = torch.zeros(W.shape[0], dtype=w0.dtype, device=w0.device)
                for m, sz, off in zip(mods, sizes, offs):
                    W[off:off + sz].copy_(m.weight.detach())
                    m.weight.data = W[off:off + sz]
                    if m.bias is not None:
                        b[off:off + sz] = m.bias.detach()
                c = {"w": W, "b": b, "sizes": sizes, "offs": offs}
            self._layer_cache[key] = c
        return c

    def _layer_consts(self, i, mixer):
        c = self._layer_cache.get(i)
        if c is None:
            if isinstance(mixer, (GatedDeltaNet, GatedKalmaNet)):
                convs = [mixer.q_conv1d, mixer.k_conv1d] + ([mixer.v_conv1d] if getattr(mixer, "use_v_conv", True) else [])
                w = torch.cat([cv.weight for cv in convs], dim=0).squeeze(1).contiguous()
                b = None
                if convs[0].bias is not None:
                    b = torch.cat([cv.bias for cv in convs]).contiguous()
                c = {"w": w, "b": b}
            else:
                c = {"w": mixer.conv1d.weight.squeeze(1).contiguous(), "b": mixer.conv1d.bias}
            self._layer_cache[i] = c
        return c

    def _gdn_decode(self, i, mx: GatedDeltaNet, h, slots):
        Rn = h.shape[0]
        c = self._layer_consts(i, mx)
        pk = {"w": None}
        if mx.kv_proj_rank is None:
            pk = self._packed(("in", i), [mx.q_proj, mx.k_proj, mx.v_proj, mx.gk_proj, mx.b_proj]
                              + ([mx.g_proj] if mx.use_gate else []))
        gate = None
        if pk["w"] is not None:         # one GEMM for every projection of the layer input
            z = gemm_ops.linear(h, pk["w"], pk["b"])
            sz, of = pk["sizes"], pk["offs"]
            part = [z[:, o:o + n_] for o, n_ in zip(of, sz)]
            qkv = z[:, :sz[0] + sz[1] + sz[2]]          # q, k, v are multiples of 8 wide: no padding between them
            a_in, b_in = part[3], part[4]
            gate = part[5] if mx.use_gate else None
        else:
            qkv = torch.cat([mx.q_proj(h), mx.k_proj(h), mx.v_proj(h)], dim=-1)
            a_in, b_in = mx.gk_proj(h), mx.b_proj(h)
        qkv = self._conv_update(i, qkv, c["w"], c["b"], slots)
        q, k, v = torch.split(qkv, [mx.query_dim, mx.key_dim, mx.value_dim], dim=-1)
        g, beta = R.gdn_gating(a_in, b_in, mx.A_log, mx.dt_bias, 2.0 if mx.allow_neg_eigval else 1.0)
        H, D = mx.expanded_num_heads, mx.head_dim
        st = self.state.ssm[i]["state"]
        if self._cuda and D == 128 and h.dtype == torch.bfloat16 and mx.kv_proj_rank is None:
            o = torch.empty(Rn, H, D, device=h.device, dtype=h.dtype)
            # keep the contiguous copies alive until the launch (a temporary's block would be reused)
            q, k, v, g, beta = q.contiguous(), k.contiguous(), v.contiguous(), g.float().contiguous(), beta.float().contiguous()
            _lib.check(_lib.kernels().hmf_gdn_decode(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g), _lib.ptr(beta), _lib.ptr(st), _lib.ptr(slots),
                _lib.ptr(o), c_int(Rn), c_int(H), c_int(mx.num_q_heads), c_int(mx.num_k_heads), c_int(mx.num_v_heads),
                c_int(D), c_int(D), c_float(D ** -0.5), c_int(1), _lib.stream_ptr(h.device)), "gdn_decode")
        else:
            from ..layers.common import repeat_heads
            qh = repeat_heads(q.reshape(Rn, 1, mx.num_q_heads, D), mx.num_q_groups)
            kh, vh = mx._expand_kv(k[:, None], v[:, None])
            s0 = st[slots.long()]
            o, sT = R.gated_delta_rule_recurrent(qh, kh, vh, g[:, None], beta[:, None], initial_state=s0)
            st[slots.long()] = sT
            o = o[:, 0].to(h.dtype)
        if mx.use_gate:
            o = mx.o_norm(o, (gate if gate is not None else mx.g_proj(h)).reshape(Rn, H, D))
        else:
            o = mx.o_norm(o)
        return self._row_linear(o.reshape(Rn, -1), mx.o_proj)

    def _mamba_decode(self, i, mx: Mamba2, h, cos, sin, slots):
        Rn = h.shape[0]
        c = self._layer_consts(i, mx)
        # the projection's rows padded to whole 128-row tiles, so the decode GEMM kernel takes it
        pk = self._packed(("in", i), [mx.in_proj]) if (self._cuda and h.dtype == torch.bfloat16) else {"w": None}
        zx = gemm_ops.linear(h, pk["w"], pk["b"]) if pk["w"] is not None else mx.in_proj(h)
        z, xBC, dt = torch.split(zx if zx.shape[-1] == mx.in_proj_valid else zx[:, :mx.in_proj_valid],
                                 [mx.d_inner, mx.conv_dim, mx.nheads], dim=-1)
        rope = mx.use_pos_emb and cos is not None
        if (self._cuda and h.dtype == torch.bfloat16 and mx.headdim == 128 and mx.d_xb % 128 == 0
                and (not rope or cos.shape[-1] % 2 == 0)):
            # split + B/C norms + rotary + concatenation in one pass, written as the contiguous convolution input
            cs = sn = None
            if rope:
                cs, sn = cos.reshape(Rn, -1).contiguous(), sin.reshape(Rn, -1).contiguous()
            bn = mx.B_norm
            xin = xBC
            xBC = torch.empty(Rn, mx.conv_dim, device=h.device, dtype=h.dtype)
            _lib.check(_lib.kernels().hmf_heads_norm_rope(
                _lib.ptr(xin), c_ll(xin.stride(0)), _lib.ptr(xBC), c_ll(xBC.stride(0)), c_int(mx.d_xb // 128),
                c_int(mx.d_xb // 128), c_int(mx.d_inner // 128), _lib.ptr(bn.weight if bn is not None else None),
                _lib.ptr(mx.C_norm.weight if bn is not None else None),
                c_float(bn.variance_epsilon if bn is not None else 0.0),
                c_int(int(getattr(bn, "zero_centered", False)) if bn is not None else 0), _lib.ptr(cs), _lib.ptr(sn),
                c_int(cs.shape[-1] if rope else 0), c_int(Rn), _lib.stream_ptr(h.device)), "heads_norm_rope")
        else:
            xBC = mx._norm_rope(xBC[:, None], (cos, sin))[:, 0].contiguous()
        xBC = self._conv_update(i, xBC, c["w"], c["b"], slots)
        st = self.state.ssm[i]["state"]
        Hx = mx.d_xb // mx.headdim
        packed = self._cuda and h.dtype == torch.bfloat16 and mx.d_state in (128, 256)
        if not packed:
            x, Bm, Cm = torch.split(xBC, [mx.d_xb, mx.d_xb, mx.d_inner], dim=-1)
            A = -torch.exp(mx.A_log.float())
            dtp = F.softplus(dt.float() + mx.dt_bias.float())
        if self._cuda and h.dtype == torch.bfloat16 and mx.d_state in (128, 256):
            # x / B / C are read straight from the convolution output, dt from the projection output
            if "A_log" not in c:
                c["A_log"], c["dt_bias"], c["D"] = (mx.A_log.float().contiguous(), mx.dt_bias.float().contiguous(),
                                                   mx.D.float().contiguous())
            y = torch.empty(Rn, mx.nheads, mx.headdim, device=h.device, dtype=h.dtype)
            xBC = xBC if xBC.is_contiguous() else xBC.contiguous()
            _lib.check(_lib.kernels().hmf_ssd_decode_packed(
                _lib.ptr(xBC), c_ll(xBC.stride(0)), c_int(0), c_int(mx.d_xb), c_int(2 * mx.d_xb), _lib.ptr(dt),
                c_ll(dt.stride(0)), _lib.ptr(c["dt_bias"]), _lib.ptr(c["A_log"]), _lib.ptr(c["D"]), _lib.ptr(st),
                _lib.ptr(slots), _lib.ptr(y), c_int(Rn), c_int(mx.nheads), c_int(Hx), c_int(Hx), c_int(mx.headdim),
                c_int(mx.d_state), _lib.stream_ptr(h.device)), "ssd_decode_packed")
        elif self._cuda and h.dtype == torch.bfloat16:
            y = torch.empty(Rn, mx.nheads, mx.headdim, device=h.device, dtype=h.dtype)
            # keep the contiguous copies alive until the launch (a temporary's block would be reused)
            x, dtp, A, Bm, Cm, Dp = (x.contiguous(), dtp.contiguous(), A.contiguous(), Bm.contiguous(), Cm.contiguous(),
                                     mx.D.float().contiguous())
            _lib.check(_lib.kernels().hmf_ssd_decode(
                _lib.ptr(x), _lib.ptr(dtp), _lib.ptr(A), _lib.ptr(Bm), _lib.ptr(Cm), _lib.ptr(Dp), _lib.ptr(st),
                _lib.ptr(slots), _lib.ptr(y), c_int(Rn), c_int(mx.nheads), c_int(Hx), c_int(Hx), c_int(mx.headdim),
                c_int(mx.d_state), _lib.stream_ptr(h.device)), "ssd_decode")
        else:
            from ..layers.common import repeat_heads
            xh = repeat_heads(x.reshape(Rn, 1, Hx, mx.headdim), mx.num_kv_groups)[:, 0]
            Bh = repeat_heads(Bm.reshape(Rn, 1, Hx, mx.d_state), mx.num_kv_groups)[:, 0]
            Ch = Cm.reshape(Rn, mx.ngroups, mx.d_state)
            s0 = st[slots.long()]
            y, sT = R.selective_state_update(s0, xh, dtp, A, Bh, Ch, mx.D)
            st[slots.long()] = sT
            y = y.to(h.dtype)
        zg = z.reshape(Rn, mx.nheads, mx.headdim)
        y = F_ops.gated_rms_norm(y, zg, mx.norm.weight.view(mx.nheads, mx.headdim), mx.norm.eps, norm_before_gate=False)
        return self._row_linear(y.reshape(Rn, mx.d_inner), mx.out_proj)

    def _gka_decode(self, i, mx: GatedKalmaNet, h, slots):
        """GKA decode: conv update + token-level solve and GLA update on the slot states."""
        from ..layers.common import repeat_heads
        Rn = h.shape[0]
        c = self._layer_consts(i, mx)
        e = self.state.ssm[i]
        pk = {"w": None}
        if mx.kv_proj_rank is None:
            names = (["q_proj", "k_proj", "v_proj", "a_proj"] + (["b_proj"] if mx.use_beta_gate else [])
                     + (["alpha_proj"] if mx.use_alpha_connection else []) + (["g_proj"] if mx.use_gate else []))
            pk = self._packed(("in", i), [getattr(mx, n) for n in names])
        pre = {}
        if pk["w"] is not None:         # one GEMM for every projection of the layer input
            z = gemm_ops.linear(h, pk["w"], pk["b"])
            pre = {n_: z[:, o:o + sz_] for n_, o, sz_ in zip(names, pk["offs"], pk["sizes"])}
            nconv = pk["sizes"][0] + pk["sizes"][1] + (pk["sizes"][2] if mx.use_v_conv else 0)
            parts = [pre["q_proj"], pre["k_proj"]] + ([pre["v_proj"]] if mx.use_v_conv else [])
            xin = z[:, :nconv]
        else:
            parts = [mx.q_proj(h), mx.k_proj(h)] + ([mx.v_proj(h)] if mx.use_v_conv else [])
            xin = torch.cat(parts, dim=-1)
        proj = lambda n: pre[n] if n in pre else getattr(mx, n)(h)  # noqa: E731
        x = self._conv_update(i, xin, c["w"], c["b"], slots)
        outs = torch.split(x, [p.shape[-1] for p in parts], dim=-1)
        q, k = outs[0], outs[1]
        v = outs[2] if mx.use_v_conv else proj("v_proj")
        D = mx.head_dim
        H = mx.expanded_num_heads
        if self._cuda and D == 128 and h.dtype == torch.bfloat16 and mx.kv_proj_rank is None:
            # fused kernel: norms, gates, covariance update, Chebyshev solve, GLA update and read-out
            beta = torch.sigmoid(proj("b_proj")).float().contiguous() if mx.use_beta_gate else None
            alpha = torch.sigmoid(proj("alpha_proj")).float().contiguous() if mx.use_alpha_connection else None
            g = (-mx.A_log.float().exp() * F.softplus(proj("a_proj").float() + mx.dt_bias.float())).contiguous()
            qc, kc_, vc_ = q.contiguous(), k.contiguous(), v.contiguous()
            o = torch.empty(Rn, H, D, device=h.device, dtype=h.dtype)
            _lib.check(_lib.kernels().hmf_gka_decode(
                _lib.ptr(qc), _lib.ptr(kc_), _lib.ptr(vc_), _lib.ptr(g), _lib.ptr(beta), _lib.ptr(alpha),
                _lib.ptr(e["state_kk"]), _lib.ptr(e["state"]), _lib.ptr(slots), _lib.ptr(o), c_int(Rn), c_int(H),
                c_int(mx.num_q_heads), c_int(mx.num_k_heads), c_int(mx.num_v_heads), c_int(D), c_float(mx.gla_scale),
                c_float(mx.ridge_strength), c_int(mx.num_iter), c_int(int(mx.use_forgetting_gate_kk)),
                _lib.stream_ptr(h.device)), "gka_decode")
            o = mx.o_norm(o, proj("g_proj").reshape(Rn, H, D)) if mx.use_gate else mx.o_norm(o)
            return self._row_linear(o.reshape(Rn, -1), mx.o_proj)
        q = repeat_heads(q.reshape(Rn, 1, mx.num_q_heads, D), mx.num_q_groups)
        k, v = mx._expand_kv(k[:, None], v[:, None])
        eps = 1e-6
        q = q.float() / (torch.linalg.vector_norm(q.float(), dim=-1, keepdim=True) + eps)
        k = k.float() / (torch.linalg.vector_norm(k.float(), dim=-1, keepdim=True) + eps)
        v = v.float()
        if mx.use_beta_gate:
            beta = torch.sigmoid(proj("b_proj")).float()[:, None]
            k, v = (beta[..., None] + eps) * k, (beta[..., None] + eps) * v
        alpha = torch.sigmoid(proj("alpha_proj")).float()[:, None] if mx.use_alpha_connection else None
        g = (-mx.A_log.float().exp() * F.softplus(proj("a_proj").float() + mx.dt_bias.float()))[:, None]
        gk = g if mx.use_forgetting_gate_kk else None
        sl = slots.long()
        o, (h_kk, h_kv) = R.gka_forward(q, k, v, alpha, g, gk, scale=mx.gla_scale, ridge_ratio=mx.ridge_strength,
                                        num_iter=mx.num_iter, initial_state=(e["state_kk"][sl], e["state"][sl]),
                                        recurrent=True)
        if h_kk is not None:
            e["state_kk"][sl] = h_kk
        e["state"][sl] = h_kv
        o = o[:, 0].to(h.dtype)
        H = mx.expanded_num_heads
        o = mx.o_norm(o, proj("g_proj").reshape(Rn, H, D)) if mx.use_gate else mx.o_norm(o)
        return self._row_linear(o.reshape(Rn, -1), mx.o_proj)

    # -- metrics ---------------------------------------------------------------------------------------
    def request_metrics(self) -> dict:
        done = [r for r in self.requests.values() if r.finished]
        ttft = sorted((r.first_token_time - r.arrival) * 1e3 for r in done if r.first_token_time)
        out_tokens = sum(len(r.output) for r in done)
        return {"finished": len(done), "output_tokens": out_tokens,
                "p50_ttft_ms": ttft[len(ttft) // 2] if ttft else None,
                "mean_ttft_ms": sum(ttft) / len(ttft) if ttft else None, **self.sched.stats(), **self.stats}
