"""PPO stage (RLHF): rollouts from the policy, scores from a reward model, per-token KL penalty against a frozen
reference policy, generalised advantage estimation, clipped policy and value losses, adaptive KL coefficient.

The policy is a ``HybridForCausalLM`` with a scalar value head on the final hidden state.  Rollouts use the model's
own ``generate`` (hybrid cache: K/V for attention layers, recurrent state for the SSM layers).  Hyper-parameters
follow the reference's arguments (``hparams/finetuning_args.py:203-223``: ``ppo_buffer_size``, ``ppo_epochs``,
``ppo_score_norm``, ``ppo_target``, ``ppo_whiten_rewards``); its trainer wraps ``trl``'s ``PPOTrainer``
(``train/ppo/trainer.py``), which is not a dependency here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.nn.functional as F


@dataclass
class PPOConfig:
    learning_rate: float = 1e-6
    ppo_epochs: int = 4
    ppo_buffer_size: int = 1
    mini_batch_size: int = 4
    max_new_tokens: int = 32
    temperature: float = 1.0
    top_k: int = 0
    gamma: float = 1.0
    lam: float = 0.95
    cliprange: float = 0.2
    cliprange_value: float = 0.2
    vf_coef: float = 0.1
    init_kl_coef: float = 0.2
    ppo_target: Optional[float] = 6.0        # adaptive KL control towards this KL per sequence; None: fixed
    kl_horizon: int = 10000
    ppo_score_norm: bool = False
    ppo_whiten_rewards: bool = False
    max_grad_norm: float = 1.0
    eos_token_id: Optional[int] = None
    pad_token_id: int = 0


class ValueHead(torch.nn.Module):
    def __init__(self, hidden_size: int):
        super().__init__()
        self.summary = torch.nn.Linear(hidden_size, 1)
        torch.nn.init.zeros_(self.summary.weight)
        torch.nn.init.zeros_(self.summary.bias)

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.summary(hidden.float().to(self.summary.weight.dtype)).squeeze(-1).float()


def _whiten(x: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    n = mask.sum().clamp(min=1)
    mean = (x * mask).sum() / n
    var = (((x - mean) ** 2) * mask).sum() / n
    out = (x - mean) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mean


def gae(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float, lam: float):
    """Advantages and returns over the response tokens (``[B, R]`` tensors, ``mask`` 1 on real tokens)."""
    B, R = rewards.shape
    adv = torch.zeros_like(rewards)
    last = torch.zeros(B, device=rewards.device)
    for t in reversed(range(R)):
        nxt = values[:, t + 1] if t + 1 < R else torch.zeros(B, device=rewards.device)
        nxt = nxt * (mask[:, t + 1] if t + 1 < R else 0.0)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lam * last * (mask[:, t + 1] if t + 1 < R else 0.0)
        adv[:, t] = last
    adv = adv * mask
    return adv, adv + values * mask


class PPOTrainer:
    """``reward_fn(full_ids [B, P+R], response_mask [B, R]) -> scores [B]``; ``ref_model`` defaults to a frozen
    snapshot of the policy's initial weights' log-probabilities (computed without gradient before the updates)."""

    def __init__(self, model, reward_fn: Callable, config: Optional[PPOConfig] = None, ref_model=None,
                 optimizer: Optional[torch.optim.Optimizer] = None):
        self.model, self.reward_fn, self.cfg, self.ref_model = model, reward_fn, config or PPOConfig(), ref_model
        dev = next(model.parameters()).device
        self.value_head = ValueHead(model.config.hidden_size).to(dev)
        params = [p for p in model.parameters() if p.requires_grad] + list(self.value_head.parameters())
        self.optimizer = optimizer or torch.optim.AdamW(params, lr=self.cfg.learning_rate, weight_decay=0.0)
        self.params = params
        self.kl_coef = self.cfg.init_kl_coef
        self.score_mean, self.score_var, self.score_n = 0.0, 1.0, 0
        self.stats: List[Dict[str, float]] = []

    # -- pieces ---------------------------------------------------------------------------------
    def _forward(self, model, ids: torch.Tensor, n_prompt: int, with_values: bool):
        """Log-probabilities of the response tokens (and values at the positions that emit them)."""
        hidden, _ = model.model(ids)
        h = hidden[:, n_prompt - 1:-1]
        logits = model.lm_head(h).float()
        logp = torch.gather(F.log_softmax(logits, -1), 2, ids[:, n_prompt:].unsqueeze(-1)).squeeze(-1)
        return logp, (self.value_head(h) if with_values else None), logits

    @torch.no_grad()
    def rollout(self, prompts: torch.Tensor) -> Dict[str, torch.Tensor]:
        c = self.cfg
        ids = self.model.generate(prompts, max_new_tokens=c.max_new_tokens, temperature=c.temperature, top_k=c.top_k,
                                  eos_token_id=c.eos_token_id)
        P = prompts.shape[1]
        resp = ids[:, P:]
        mask = torch.ones_like(resp, dtype=torch.float32)
        if c.eos_token_id is not None:      # tokens after the first EOS are padding
            after = (resp == c.eos_token_id).float().cumsum(-1) - (resp == c.eos_token_id).float()
            mask = (after == 0).float()
        was_training = self.model.training
        self.model.eval()
        logp, values, _ = self._forward(self.model, ids, P, True)
        ref_logp = self._forward(self.ref_model, ids, P, False)[0] if self.ref_model is not None else logp.clone()
        self.model.train(was_training)
        scores = self.reward_fn(ids, mask).float()
        if c.ppo_score_norm:                # running mean / variance of the raw scores
            for s in scores.tolist():
                self.score_n += 1
                d = s - self.score_mean
                self.score_mean += d / self.score_n
                self.score_var += (d * (s - self.score_mean) - self.score_var) / self.score_n
            scores = (scores - self.score_mean) / max(self.score_var, 1e-8) ** 0.5
        kl = (logp - ref_logp) * mask
        rewards = -self.kl_coef * kl
        last = mask.sum(-1).long().clamp(min=1) - 1
        rewards[torch.arange(ids.shape[0]), last] += scores
        if c.ppo_whiten_rewards:
            rewards = _whiten(rewards, mask, shift_mean=False) * mask
        adv, returns = gae(rewards, values, mask, c.gamma, c.lam)
        adv = _whiten(adv, mask) * mask
        return {"ids": ids, "n_prompt": torch.tensor(P), "mask": mask, "logp": logp, "values": values, "adv": adv,
                "returns": returns, "scores": scores, "kl": kl.sum(-1)}

    def loss(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        c = self.cfg
        mask = batch["mask"]
        n = mask.sum().clamp(min=1)
        logp, values, logits = self._forward(self.model, batch["ids"], int(batch["n_prompt"]), True)
        ratio = torch.exp(logp - batch["logp"])
        pg = torch.max(-batch["adv"] * ratio, -batch["adv"] * ratio.clamp(1 - c.cliprange, 1 + c.cliprange))
        v_clip = batch["values"] + (values - batch["values"]).clamp(-c.cliprange_value, c.cliprange_value)
        vf = 0.5 * torch.max((values - batch["returns"]) ** 2, (v_clip - batch["returns"]) ** 2)
        pg_loss, vf_loss = (pg * mask).sum() / n, (vf * mask).sum() / n
        probs = torch.softmax(logits, -1)
        entropy = ((torch.logsumexp(logits, -1) - (probs * logits).sum(-1)) * mask).sum() / n
        return {"loss": pg_loss + c.vf_coef * vf_loss, "policy_loss": pg_loss.detach(), "value_loss": vf_loss.detach(),
                "entropy": entropy.detach(), "clipfrac": (((ratio - 1).abs() > c.cliprange).float() * mask).sum() / n}

    # -- one PPO step: collect ``ppo_buffer_size`` rollouts, optimise ``ppo_epochs`` over mini-batches ----------------
    def step(self, prompt_batches: List[torch.Tensor]) -> Dict[str, float]:
        c = self.cfg
        buffer = [self.rollout(p) for p in prompt_batches[:max(1, c.ppo_buffer_size)]]
        agg: Dict[str, float] = {}
        n_updates = 0
        self.model.train()
        for _ in range(c.ppo_epochs):
            for roll in buffer:
                B = roll["ids"].shape[0]
                perm = torch.randperm(B, device=roll["ids"].device)
                for i in range(0, B, c.mini_batch_size):
                    idx = perm[i:i + c.mini_batch_size]
                    mb = {k: (v[idx] if v.dim() > 0 and v.shape[0] == B else v) for k, v in roll.items()}
                    out = self.loss(mb)
                    self.optimizer.zero_grad(set_to_none=True)
                    out["loss"].backward()
                    if c.max_grad_norm > 0:
                        torch.nn.utils.clip_grad_norm_(self.params, c.max_grad_norm)
                    self.optimizer.step()
                    n_updates += 1
                    for k, v in out.items():
                        agg[k] = agg.get(k, 0.0) + float(v.detach())
        stats = {k: v / max(n_updates, 1) for k, v in agg.items()}
        kl = float(torch.cat([r["kl"] for r in buffer]).mean())
        stats["kl"], stats["kl_coef"] = kl, self.kl_coef
        stats["score"] = float(torch.cat([r["scores"] for r in buffer]).mean())
        if c.ppo_target is not None:        # proportional controller on the KL coefficient
            err = max(-0.2, min(0.2, kl / c.ppo_target - 1.0))
            n_seq = sum(r["ids"].shape[0] for r in buffer)
            self.kl_coef *= 1.0 + err * n_seq / c.kl_horizon
        self.stats.append(stats)
        return stats


def reward_model_fn(reward_model, score_row: int = 0) -> Callable:
    """Reward function backed by a model trained by the ``rm`` stage (``train/preference.py``): the score is the
    value head applied to the hidden state of the last real token (a model without a value head is scored by one
    row of its output head)."""
    @torch.no_grad()
    def fn(ids: torch.Tensor, resp_mask: torch.Tensor) -> torch.Tensor:
        h = reward_model.model(ids)[0].float()
        P = ids.shape[1] - resp_mask.shape[1]
        last = P + resp_mask.sum(-1).long().clamp(min=1) - 1
        h_last = h[torch.arange(ids.shape[0], device=ids.device), last]
        if hasattr(reward_model, "v_head"):
            return reward_model.v_head(h_last.to(reward_model.v_head.weight.dtype)).squeeze(-1).float()
        return h_last @ reward_model.lm_head.weight[score_row].float()
    return fn
