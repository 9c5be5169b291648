"""Decoder-only hybrid language models.

One generic implementation serves every family of the reference zoo (HybridQwen3 / Qwen2 /
Llama / Ministral3 / Qwen3-MoE, Qwen3-Next-HMF, Qwen3.5-MoE-HMF text); the family only fixes
configuration defaults (``models/configuration.py``).  Each decoder layer is chosen by the
``hybrid_override_pattern`` symbol at its index.  Module and parameter names follow the HF
checkpoints of the reference project (``model.layers.N.{self_attn,gdn,gka,mamba,bmojo_f,swa}``,
``input_layernorm``, ``post_attention_layernorm``, ``mlp.{gate,up,down}_proj``, ``model.norm``,
``lm_head``) so its safetensors load unchanged.

Reference: ``models/hybrid_qwen3/modeling_hybrid_qwen3.py:424-1396``,
``models/hybrid_qwen3_moe/modeling_hybrid_qwen3_moe.py:329-386, 1412-1492``,
``models/qwen3_next_hmf/modeling_qwen3_next_hmf.py:128-145, 233-407``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint  # noqa: F401

from ..utils.checkpointing import layer_checkpoint

from ..layers.attention import Attention, SlidingWindowAttention
from ..layers.bmojo import BMojoLayer
from ..layers.common import MLP, RMSNorm, RotaryEmbedding
from ..layers.gdn import GatedDeltaNetLayer
from ..layers.gka import GatedKalmaNetLayer
from ..layers.mamba2 import Mamba2Layer
from ..ops import functional as F_ops
from ..ops import moe as moe_ops
from ..parallel.sp import reduce_loss
from .cache import HybridCache
from .configuration import HybridConfig
from .patterns import FUSED_SYMBOLS, MIXER_ATTR, is_fused, unfuse_symbol


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    past_key_values: Optional[HybridCache] = None
    hidden_states: Optional[torch.Tensor] = None
    aux_loss: Optional[torch.Tensor] = None
    num_tokens: Optional[torch.Tensor] = None


# ----------------------------------------------------------------------------------------
# MoE feed-forward
# ----------------------------------------------------------------------------------------
class SparseMoeBlock(nn.Module):
    """Top-k routed SwiGLU experts (+ optional shared expert with a sigmoid gate).

    Expert weights are stacked: ``experts.gate_up_proj [E, 2F, Dm]`` and ``experts.down_proj
    [E, Dm, F]``; ``utils.checkpoint_io`` converts to / from the per-expert HF names
    (``experts.{e}.{gate,up,down}_proj.weight``).  With an expert-parallel group the experts are
    sharded over ranks and tokens travel by all-to-all (``parallel/ep.py``)."""

    def __init__(self, config: HybridConfig):
        super().__init__()
        self.num_experts, self.top_k = int(config.num_experts), int(config.num_experts_per_tok)
        self.norm_topk_prob = bool(config.norm_topk_prob)
        Dm, Fi = config.hidden_size, int(config.moe_intermediate_size)
        self.gate = nn.Linear(Dm, self.num_experts, bias=False)
        self.experts = nn.Module()
        self.experts.gate_up_proj = nn.Parameter(torch.empty(self.num_experts, 2 * Fi, Dm))
        self.experts.down_proj = nn.Parameter(torch.empty(self.num_experts, Dm, Fi))
        nn.init.normal_(self.experts.gate_up_proj, std=config.initializer_range)
        nn.init.normal_(self.experts.down_proj, std=config.initializer_range)
        sh = int(getattr(config, "shared_expert_intermediate_size", 0) or 0)
        if sh > 0:
            self.shared_expert = MLP(Dm, sh)
            self.shared_expert_gate = nn.Linear(Dm, 1, bias=False)
        else:
            self.shared_expert = None
        self.expert_parallel_group = None
        self.fused_ep = None            # parallel.ep_fused.FusedExpertParallel (grouped GEMM kernels, inference)
        self.eplb_plan = None           # parallel.eplb.EPLBPlan: replicated hot experts, routing on physical slots

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        logits = self.gate(flat)
        weights, indices = moe_ops.router(logits, self.top_k, self.norm_topk_prob)
        if self.eplb_plan is not None:
            from ..parallel.eplb import remap
            indices = remap(indices, self.eplb_plan)
        out = moe_ops.experts_forward(flat, self.experts.gate_up_proj, self.experts.down_proj, weights.to(flat.dtype),
                                      indices, ep=self.expert_parallel_group, fused=self.fused_ep)
        if self.shared_expert is not None:
            out = out + torch.sigmoid(self.shared_expert_gate(flat)) * self.shared_expert(flat)
        return out.reshape(shape), logits


def load_balancing_loss(router_logits: List[torch.Tensor], num_experts: int, top_k: int) -> torch.Tensor:
    """Switch-style auxiliary loss ``E * sum_e f_e * P_e`` over all MoE layers
    (reference: ``hybrid_qwen3_moe/modeling_hybrid_qwen3_moe.py:1412-1492``)."""
    if not router_logits:
        return torch.zeros(())
    logits = torch.cat([l.float() for l in router_logits], dim=0)
    probs = torch.softmax(logits, dim=-1)
    _, sel = torch.topk(probs, top_k, dim=-1)
    mask = F.one_hot(sel, num_experts).float()  # [T, k, E]
    tokens_per_expert = mask.mean(dim=0)  # [k, E]
    router_prob = probs.mean(dim=0)  # [E]
    return (tokens_per_expert * router_prob[None]).sum() * num_experts


# ----------------------------------------------------------------------------------------
# decoder layers
# ----------------------------------------------------------------------------------------
def _native_window(config: HybridConfig, layer_idx: int):
    """Window of an attention layer that the *base* architecture itself runs as sliding-window attention (its weights
    stay under ``self_attn``); ``HybridConfig`` works out which layers those are."""
    window = getattr(config, "sliding_window", None)
    return int(window) if window and layer_idx in (getattr(config, "native_window_layers", None) or ()) else None


def _make_mixer(symbol: str, config: HybridConfig, layer_idx: int) -> nn.Module:
    if symbol == "*":
        return Attention(config, layer_idx, gated=bool(config.gated_attention),
                         sliding_window=_native_window(config, layer_idx))
    if symbol == "SWA":
        return SlidingWindowAttention(config, layer_idx)
    if symbol == "M2":
        return Mamba2Layer(config, layer_idx)
    if symbol == "GDN":
        return GatedDeltaNetLayer(config, layer_idx)
    if symbol == "GKA":
        return GatedKalmaNetLayer(config, layer_idx)
    if symbol == "BMF":
        return BMojoLayer(config, layer_idx)
    if symbol == "L2A":
        from ..layers.l2a import L2AAttention
        return L2AAttention(config, layer_idx)
    raise ValueError(f"no mixer for layer symbol '{symbol}'")


class DecoderLayer(nn.Module):
    """Pre-norm residual block: ``x + mixer(norm(x))`` then ``x + mlp(norm(x))``."""

    def __init__(self, config: HybridConfig, layer_idx: int, symbol: str):
        super().__init__()
        self.symbol, self.layer_idx = symbol, layer_idx
        zc = bool(config.zero_centered_norm)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, zc)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, zc)
        setattr(self, MIXER_ATTR[symbol], _make_mixer(symbol, config, layer_idx))
        if config.layer_is_moe(layer_idx):
            self.mlp = SparseMoeBlock(config)
        else:
            self.mlp = MLP(config.hidden_size, config.intermediate_size, bias=bool(config.mlp_bias))
        self.is_moe = isinstance(self.mlp, SparseMoeBlock)

    @property
    def seq_mixer(self) -> nn.Module:
        return getattr(self, MIXER_ATTR[self.symbol])

    def _mlp(self, x):
        if self.is_moe:
            return self.mlp(x)
        return self.mlp(x), None

    def forward(self, hidden_states, position_embeddings=None, position_ids=None, past_key_values=None,
                use_cache=False, **kwargs):
        residual = hidden_states
        h = self.input_layernorm(hidden_states)
        if self.symbol == "L2A":        # the router reads the residual stream after the local attention
            kwargs = dict(kwargs, residual=residual)
        cu = kwargs.pop("cu_seqlens", None)
        caches = kwargs.pop("sample_caches", None)
        if cu is not None and (len(cu) > 2 or caches is not None):
            # packed samples (batch of one row): the mixer runs once per sample on its slice, so neither attention
            # nor recurrent state crosses a sample boundary.  `sample_caches` (serving: the prefill pieces of several
            # requests in one forward) gives every sample its own cache
            parts = []
            mixer = self.seq_mixer
            # inference: the projections that read the layer input run ONCE on the packed row (one GEMM each instead of
            # one per sample), and so does the output projection afterwards; the samples only differ in the mixer core
            pre_all, out_name = {}, None
            if caches is not None and not torch.is_grad_enabled() and hasattr(mixer, "INPUT_PROJECTIONS"):
                for n in mixer.INPUT_PROJECTIONS:
                    m = getattr(mixer, n, None)
                    if isinstance(m, nn.Linear):
                        pre_all[n] = m(h)
                # (a mixer with forward hooks -- tensor parallelism sums its partial outputs there -- must return its
                # finished output, so its output projection stays inside)
                if isinstance(getattr(mixer, mixer.OUTPUT_PROJECTION, None), nn.Linear) and not mixer._forward_hooks:
                    out_name = mixer.OUTPUT_PROJECTION
            for j, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
                pe = None if position_embeddings is None else tuple(t[:, a:b] for t in position_embeddings)
                kw = dict(kwargs)
                if "residual" in kw:
                    kw["residual"] = kw["residual"][:, a:b]
                if pre_all:
                    kw["pre_proj"] = {n: y[:, a:b] for n, y in pre_all.items()}
                if out_name:
                    kw["defer_out_proj"] = True
                pkv = None if caches is None else caches[j]
                parts.append(mixer(h[:, a:b], position_embeddings=pe,
                                   position_ids=None if position_ids is None else position_ids[:, a:b],
                                   past_key_values=pkv, use_cache=pkv is not None, **kw)[0])
            h = torch.cat(parts, dim=1)
            if out_name:
                h = getattr(mixer, out_name)(h)
        else:
            h, _, _ = self.seq_mixer(h, position_embeddings=position_embeddings, position_ids=position_ids,
                                     past_key_values=past_key_values, use_cache=use_cache, **kwargs)
        norm = self.post_attention_layernorm
        if not torch.is_grad_enabled() and h.is_cuda and h.dtype == torch.bfloat16 and not norm.zero_centered:
            normed, residual = F_ops.fused_add_rms_norm(h, residual, norm.weight, norm.variance_epsilon)   # one pass
        else:
            residual = residual + h
            normed = norm(residual)
        h, router_logits = self._mlp(normed)
        return residual + h, router_logits


class FusedDecoderLayer(nn.Module):
    """Stage-1 (distillation) layer: a student mixer and a teacher mixer share the norms and the
    MLP and process two streams.  Symbols ``X*`` (student ``X``, teacher attention), ``*DA`` (the
    same attention on both streams) and ``GDN>GKA`` (teacher GDN, student GKA).  Teacher outputs are
    detached.  Returns ``(student_out, teacher_out, student_mixer_out, teacher_mixer_out,
    student_mlp_out, teacher_mlp_out)``
    (reference: ``modeling_hybrid_qwen3.py:668-1128``)."""

    def __init__(self, config: HybridConfig, layer_idx: int, symbol: str):
        super().__init__()
        self.symbol, self.layer_idx = symbol, layer_idx
        zc = bool(config.zero_centered_norm)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, zc)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, zc)
        self.student_symbol = FUSED_SYMBOLS[symbol]
        self.teacher_symbol = "GDN" if symbol == "GDN>GKA" else "*"
        setattr(self, MIXER_ATTR[self.teacher_symbol], _make_mixer(self.teacher_symbol, config, layer_idx))
        if symbol != "*DA":
            setattr(self, MIXER_ATTR[self.student_symbol], _make_mixer(self.student_symbol, config, layer_idx))
        if config.layer_is_moe(layer_idx):
            self.mlp = SparseMoeBlock(config)
        else:
            self.mlp = MLP(config.hidden_size, config.intermediate_size, bias=bool(config.mlp_bias))
        self.is_moe = isinstance(self.mlp, SparseMoeBlock)

    @property
    def seq_mixer(self):
        return getattr(self, MIXER_ATTR[self.student_symbol])

    @property
    def teacher_mixer(self):
        return getattr(self, MIXER_ATTR[self.teacher_symbol])

    def _stream(self, mixer, hidden_states, **kw):
        residual = hidden_states
        mixer_out, _, _ = mixer(self.input_layernorm(hidden_states), **kw)
        h = residual + mixer_out
        m = self.mlp(self.post_attention_layernorm(h))
        mlp_out = m[0] if self.is_moe else m
        return h + mlp_out, mlp_out, mixer_out

    def forward(self, hidden_states, attention_hidden_states=None, position_embeddings=None, position_ids=None,
                past_key_values=None, use_cache=False, **kwargs):
        kw = dict(position_embeddings=position_embeddings, position_ids=position_ids, past_key_values=None,
                  use_cache=False)
        if attention_hidden_states is None:
            attention_hidden_states = hidden_states
        s_out, s_mlp, s_mix = self._stream(self.seq_mixer, hidden_states, **kw)
        if self.symbol == "*DA":
            t_out, t_mlp, t_mix = self._stream(self.teacher_mixer, attention_hidden_states, **kw)
            return s_out, t_out.detach(), s_mix, t_mix.detach(), s_mlp, t_mlp.detach()
        with torch.no_grad():
            t_out, t_mlp, t_mix = self._stream(self.teacher_mixer, attention_hidden_states, **kw)
        return s_out, t_out, s_mix, t_mix, s_mlp, t_mlp


# ----------------------------------------------------------------------------------------
# model
# ----------------------------------------------------------------------------------------
class HybridModel(nn.Module):
    def __init__(self, config: HybridConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, padding_idx=config.pad_token_id)
        layers = []
        for i, sym in enumerate(config.pattern):
            layers.append(FusedDecoderLayer(config, i, sym) if is_fused(sym) else DecoderLayer(config, i, sym))
        self.layers = nn.ModuleList(layers)
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, bool(config.zero_centered_norm))
        rot_dim = int(config.head_dim * float(config.partial_rotary_factor or 1.0))
        self.rotary_emb = RotaryEmbedding(rot_dim, config.rope_theta, config.rope_scaling,
                                          config.max_position_embeddings)
        self.gradient_checkpointing = False
        # indices of layers that keep their activations although checkpointing is on (they fit in memory: see
        # `Trainer.plan_recompute`); every rank of a sequence-parallel group must hold the same set
        self.checkpoint_skip = frozenset()
        self.sequence_parallel_group = None

    @staticmethod
    def _ckpt_anchor(h: torch.Tensor) -> torch.Tensor:
        """Zero-size tensor that requires grad: keeps a checkpointed layer in the autograd graph even when
        its activations do not require grad (frozen embeddings)."""
        return torch.empty(0, device=h.device, dtype=h.dtype, requires_grad=True)

    @property
    def has_fused_layers(self) -> bool:
        return any(isinstance(l, FusedDecoderLayer) for l in self.layers)

    def forward(self, input_ids=None, position_ids=None, past_key_values=None, use_cache=False, inputs_embeds=None,
                **kwargs):
        """``cu_seqlens`` (keyword): boundaries ``[0, e_1, ..., T]`` of the samples packed into the (single) row, or a
        list with one such list per row when the batch has one row; every sequence mixer then treats the samples
        independently (``data/collator.py``)."""
        h = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        B, T = h.shape[0], h.shape[1]
        cu = kwargs.get("cu_seqlens")
        if cu is not None:
            if len(cu) and isinstance(cu[0], (list, tuple)):
                if B != 1 and any(len(c) > 2 for c in cu):
                    raise ValueError("packed samples (cu_seqlens) need a batch of one row; collate rows one by one")
                cu = list(cu[0])
            kwargs["cu_seqlens"] = [int(c) for c in cu]
        if position_ids is None:
            off = past_key_values.seqlen_offset if past_key_values is not None else 0
            position_ids = torch.arange(off, off + T, device=h.device).expand(B, T)
        pos_emb = self.rotary_emb(position_ids)
        pos_emb = (pos_emb[0].to(h.dtype), pos_emb[1].to(h.dtype))
        router_logits = []
        for li, layer in enumerate(self.layers):
            if isinstance(layer, FusedDecoderLayer):
                h = layer(h, h, position_embeddings=pos_emb, position_ids=position_ids)[0]
                continue
            if self.gradient_checkpointing and self.training and li not in self.checkpoint_skip:
                pk = {"cu_seqlens": kwargs["cu_seqlens"]} if kwargs.get("cu_seqlens") is not None else {}
                if layer.is_moe:
                    h, rl = layer_checkpoint(
                        lambda a, c, s_, p_, _d, layer=layer, pk=pk: layer(a, (c, s_), p_, None, False, **pk),
                        h, pos_emb[0], pos_emb[1], position_ids, self._ckpt_anchor(h), key=li)
                else:
                    (h,) = layer_checkpoint(
                        lambda a, c, s_, p_, _d, layer=layer, pk=pk: layer(a, (c, s_), p_, None, False, **pk)[0],
                        h, pos_emb[0], pos_emb[1], position_ids, self._ckpt_anchor(h), key=li)
                    rl = None
            else:
                h, rl = layer(h, position_embeddings=pos_emb, position_ids=position_ids,
                              past_key_values=past_key_values, use_cache=use_cache, **kwargs)
            if rl is not None:
                router_logits.append(rl)
        if past_key_values is not None:
            past_key_values.update_offset(T)
        if kwargs.get("sample_caches") is not None:
            for c, a, b in zip(kwargs["sample_caches"], kwargs["cu_seqlens"][:-1], kwargs["cu_seqlens"][1:]):
                c.update_offset(b - a)
        return self.norm(h), router_logits


class HybridForCausalLM(nn.Module):
    """Language-model head on top of :class:`HybridModel` with a fused linear + cross-entropy
    loss (the ``[T, vocab]`` logits are never materialised during training)."""

    config_class = HybridConfig

    def __init__(self, config: HybridConfig):
        super().__init__()
        self.config = config
        self.model = HybridModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.sequence_parallel_group = None
        self.apply(self._init_weights)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def _init_weights(self, m):
        std = self.config.initializer_range
        if isinstance(m, nn.Linear):
            if not getattr(m, "_keep_init", False):
                nn.init.normal_(m.weight, mean=0.0, std=std)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=std)

    # -- HF-style conveniences ------------------------------------------------------------
    def get_input_embeddings(self):
        return self.model.embed_tokens

    def gradient_checkpointing_enable(self, *_, **__):
        self.model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.model.gradient_checkpointing = False

    def num_parameters(self, only_trainable: bool = False) -> int:
        seen, total = set(), 0
        for p in self.parameters():
            if id(p) in seen or (only_trainable and not p.requires_grad):
                continue
            seen.add(id(p))
            total += p.numel()
        return total

    def forward(self, input_ids=None, labels=None, position_ids=None, past_key_values=None, use_cache=False,
                labels_shifted: bool = False, logits_to_keep: Optional[int] = None, return_logits: Optional[bool] = None,
                inputs_embeds=None, **kwargs) -> CausalLMOutput:
        if use_cache and past_key_values is None:
            past_key_values = HybridCache()
        h, router_logits = self.model(input_ids, position_ids=position_ids, past_key_values=past_key_values,
                                      use_cache=use_cache, inputs_embeds=inputs_embeds, **kwargs)
        out = CausalLMOutput(past_key_values=past_key_values, hidden_states=h)
        if labels is not None:
            sp = self.sequence_parallel_group
            if labels_shifted or (sp is not None and sp.size > 1):
                hs, ys = h, labels
            else:
                hs, ys = h[:, :-1], labels[:, 1:]
            loss_sum, n = F_ops.linear_cross_entropy(hs.reshape(-1, hs.shape[-1]), self.lm_head.weight, ys.reshape(-1))
            out.loss, out.num_tokens = reduce_loss(loss_sum, n, sp)
            if router_logits and self.config.router_aux_loss_coef:
                out.aux_loss = load_balancing_loss(router_logits, self.config.num_experts,
                                                   self.config.num_experts_per_tok).to(out.loss.device)
                out.loss = out.loss + self.config.router_aux_loss_coef * out.aux_loss
            if getattr(self.config, "mixture_of_depths", None) and self.training:
                from .mod import mod_aux_loss
                aux = mod_aux_loss(self)            # (terms of checkpointed layers carry no graph and are left out)
                if aux is not None:
                    out.loss = out.loss + float(getattr(self.config, "mod_aux_loss_coef", 0.01)) * aux
        want_logits = return_logits if return_logits is not None else labels is None
        if want_logits:
            hk = h if not logits_to_keep else h[:, -logits_to_keep:]
            out.logits = self.lm_head(hk)
        return out

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 16, temperature: float = 0.0,
                 top_k: int = 0, eos_token_id: Optional[int] = None, past_key_values: Optional[HybridCache] = None):
        """Greedy / temperature sampling with the hybrid cache (prefill, then one token per step)."""
        was_training = self.training
        self.eval()
        cache = past_key_values if past_key_values is not None else HybridCache()
        out = self(input_ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
        tokens = [input_ids]
        finished = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        for _ in range(max_new_tokens):
            logits = out.logits[:, -1].float()
            if temperature and temperature > 0:
                logits = logits / temperature
                if top_k:
                    kth = torch.topk(logits, top_k, dim=-1).values[:, -1:]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                nxt = torch.multinomial(torch.softmax(logits, dim=-1), 1)
            else:
                nxt = logits.argmax(dim=-1, keepdim=True)
            if eos_token_id is not None:
                nxt = torch.where(finished[:, None], torch.full_like(nxt, eos_token_id), nxt)
                finished |= nxt[:, 0] == eos_token_id
            tokens.append(nxt)
            if eos_token_id is not None and bool(finished.all()):
                break
            out = self(nxt, past_key_values=cache, use_cache=True, logits_to_keep=1)
        if was_training:
            self.train()
        return torch.cat(tokens, dim=1)


def _family(name: str, model_type: str):
    def __init__(self, config: HybridConfig):
        HybridForCausalLM.__init__(self, config)
    cls = type(name, (HybridForCausalLM,), {"__init__": __init__, "model_type": model_type,
                                             "__doc__": f"{model_type} family (see HybridForCausalLM)."})
    return cls


HybridQwen3ForCausalLM = _family("HybridQwen3ForCausalLM", "hybrid_qwen3")
HybridQwen2ForCausalLM = _family("HybridQwen2ForCausalLM", "hybrid_qwen2")
HybridLlamaForCausalLM = _family("HybridLlamaForCausalLM", "hybrid_llama")
HybridMinistral3ForCausalLM = _family("HybridMinistral3ForCausalLM", "hybrid_ministral3")
HybridQwen3MoeForCausalLM = _family("HybridQwen3MoeForCausalLM", "hybrid_qwen3_moe")
Qwen3NextHMFForCausalLM = _family("Qwen3NextHMFForCausalLM", "qwen3_next_hmf")
Qwen3_5MoeHMFForCausalLM = _family("Qwen3_5MoeHMFForCausalLM", "qwen3_5_moe_hmf_text")

MODEL_CLASSES = {
    "hybrid_qwen3": HybridQwen3ForCausalLM, "hybrid_qwen2": HybridQwen2ForCausalLM,
    "hybrid_llama": HybridLlamaForCausalLM, "hybrid_ministral3": HybridMinistral3ForCausalLM,
    "hybrid_qwen3_moe": HybridQwen3MoeForCausalLM, "qwen3_next_hmf": Qwen3NextHMFForCausalLM,
    "qwen3_5_moe_hmf_text": Qwen3_5MoeHMFForCausalLM, "qwen3_5_moe_hmf": Qwen3_5MoeHMFForCausalLM,
}


def build_model(config: HybridConfig) -> HybridForCausalLM:
    """Builds the model class of ``config.model_type``; every ``nn.Linear`` in it is re-classed to the layer that runs
    its three GEMMs on the library's tcgen05 kernel (bf16 CUDA tensors; other tensors take ``F.linear``)."""
    from ..ops.gemm import use_own_linear
    model = MODEL_CLASSES.get(config.model_type, HybridForCausalLM)(config)
    mod = getattr(config, "mixture_of_depths", None)
    if isinstance(mod, dict):                       # a checkpoint saved with routed layers: same routers, then load
        from .mod import apply_mixture_of_depths
        apply_mixture_of_depths(model, **mod)
    use_own_linear(model)
    return model
