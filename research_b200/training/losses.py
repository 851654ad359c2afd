"""Loss functions returning ``(loss, metrics)``: pre-training / SFT cross-entropy, GRPO
(sequence-mean log-prob x advantage), GRPO with PPO clipping, GRPO with ratio masking, PPO.

API of the reference (rollouts/training/losses.py:28-466). One deliberate difference: the
reference scores position t against token t because callers pass ``labels = input_ids.clone()``
and nothing shifts (training/grpo.py:511, loops/sft_loop.py:193). Here every loss takes
NEXT-token targets: ``shift_labels`` turns ``labels[b, t]`` into the target of position t-1 and
the loss mask is shifted with it, which is the standard causal-LM objective.

Each loss exists in two forms sharing one implementation: ``*_loss(logits, batch)`` for API
parity, and ``*_from_logprobs(logprobs, entropy, batch)`` which consumes per-token log-probs
produced by the fused lm_head kernel (no ``[B,T,V]`` log-softmax is ever materialised).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

LossOutput = tuple[torch.Tensor, dict[str, float]]


def compute_group_advantages(rewards: list[float], group_indices: list[int], normalize_std: bool = False) -> torch.Tensor:
    """advantage = reward - mean(reward of the same prompt group) [/ std of the group]."""
    r = torch.tensor(rewards, dtype=torch.float32)
    g = torch.tensor(group_indices)
    adv = torch.zeros_like(r)
    for gi in torch.unique(g):
        m = g == gi
        gr = r[m]
        a = gr - gr.mean()
        if normalize_std and gr.numel() > 1:
            sd = gr.std()
            if sd > 1e-6:
                a = a / sd
        adv[m] = a
    return adv


def shift_labels(labels: torch.Tensor, loss_mask: torch.Tensor | None = None, ignore_index: int = -100):
    """Next-token targets: position t predicts ``labels[t+1]``; the last position has no target."""
    tgt = torch.full_like(labels, ignore_index)
    tgt[..., :-1] = labels[..., 1:]
    if loss_mask is None:
        return tgt, None
    m = torch.zeros_like(loss_mask)
    m[..., :-1] = loss_mask[..., 1:]
    return tgt, m


def compute_entropy(logits: torch.Tensor, loss_mask: torch.Tensor | None = None) -> torch.Tensor:
    lp = F.log_softmax(logits.float(), dim=-1)
    ent = -(lp.exp() * lp).sum(-1)
    if loss_mask is None:
        return ent.mean()
    return (ent * loss_mask).sum() / loss_mask.sum().clamp(min=1)


def get_per_token_logprobs(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """log p(target) per position; positions with target < 0 give 0."""
    lp = F.log_softmax(logits.float(), dim=-1)
    safe = targets.clamp(min=0)
    out = lp.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    return torch.where(targets >= 0, out, torch.zeros_like(out))


def seq_mean(per_token: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return (per_token * mask).sum(-1) / mask.sum(-1).clamp(min=1)


def get_seq_logprobs(logits: torch.Tensor, labels: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
    tgt, m = shift_labels(labels, loss_mask)
    return seq_mean(get_per_token_logprobs(logits, tgt), m)


# ------------------------------------------------------------------ from per-token log-probs
def _masked_mean(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return (x * mask).sum() / mask.sum().clamp(min=1)


def ce_from_logprobs(logprobs, entropy, batch) -> LossOutput:
    mask = batch["shift_mask"]
    loss = -_masked_mean(logprobs, mask)
    return loss, {"loss": loss.item(), "perplexity": float(torch.exp(loss.detach()).clamp(max=1e9)),
                  "num_tokens": float(mask.sum())}


def grpo_from_logprobs(logprobs, entropy, batch) -> LossOutput:
    mask, adv = batch["shift_mask"], batch["advantages"]
    seq_lp = seq_mean(logprobs, mask)
    loss = -(seq_lp * adv).mean()
    ent = _masked_mean(entropy, mask).item() if entropy is not None else 0.0
    return loss, {"pg_loss": loss.item(), "entropy": ent, "avg_logprob": seq_lp.mean().item(),
                  "avg_advantage": adv.mean().item()}


def grpo_clipped_from_logprobs(logprobs, entropy, batch, clip_range: float = 0.2, entropy_coef: float = 0.0) -> LossOutput:
    mask, adv, old = batch["shift_mask"], batch["advantages"], batch["old_logprobs"]
    seq_lp = seq_mean(logprobs, mask)
    log_ratio = seq_lp - old
    ratio = log_ratio.exp()
    pg = torch.max(-ratio * adv, -ratio.clamp(1 - clip_range, 1 + clip_range) * adv).mean()
    ent = _masked_mean(entropy, mask) if entropy is not None else torch.zeros((), device=pg.device)
    loss = pg - entropy_coef * ent
    with torch.no_grad():
        clipped = (ratio < 1 - clip_range) | (ratio > 1 + clip_range)
        metrics = {"pg_loss": pg.item(), "entropy": float(ent), "clipfrac": clipped.float().mean().item(),
                   "approx_kl": ((ratio - 1) - log_ratio).mean().item(), "avg_ratio": ratio.mean().item(),
                   "avg_logprob": seq_lp.mean().item(), "avg_advantage": adv.mean().item()}
    return loss, metrics


def grpo_masked_from_logprobs(logprobs, entropy, batch, ratio_low: float = 0.1, ratio_high: float = 10.0,
                              kl_coef: float = 0.0) -> LossOutput:
    mask, adv, old = batch["shift_mask"], batch["advantages"], batch["old_logprobs"]
    seq_lp = seq_mean(logprobs, mask)
    log_ratio = seq_lp - old
    ratio = log_ratio.exp()
    low, high = ratio < ratio_low, ratio > ratio_high
    keep = ~(low | high)
    pg = -(ratio[keep] * adv[keep]).sum() / keep.sum() if keep.sum() > 0 else seq_lp.sum() * 0.0
    loss = pg
    if kl_coef > 0 and (~keep).sum() > 0:
        loss = pg + kl_coef * log_ratio[~keep].sum() / (~keep).sum()
    ent = _masked_mean(entropy, mask).item() if entropy is not None else 0.0
    return loss, {"pg_loss": float(pg.detach()), "entropy": ent, "masked_frac": (~keep).float().mean().item(),
                  "masked_low_frac": low.float().mean().item(), "masked_high_frac": high.float().mean().item(),
                  "mismatch_kl": (ratio - log_ratio - 1).mean().item(), "avg_ratio": ratio.mean().item(),
                  "avg_logprob": seq_lp.mean().item(), "avg_advantage": adv.mean().item()}


def ppo_from_logprobs(logprobs, entropy, batch, clip_range: float = 0.2) -> LossOutput:
    """Token-level PPO: per-token ratios against ``old_token_logprobs`` and per-token advantages."""
    mask = batch["shift_mask"]
    old = batch["old_token_logprobs"]
    adv = batch["token_advantages"] if "token_advantages" in batch else batch["advantages"][:, None].expand_as(logprobs)
    ratio = (logprobs - old).exp()
    per_tok = torch.max(-ratio * adv, -ratio.clamp(1 - clip_range, 1 + clip_range) * adv)
    loss = _masked_mean(per_tok, mask)
    return loss, {"pg_loss": loss.item(), "avg_ratio": _masked_mean(ratio, mask).item()}


# ------------------------------------------------------------------ from logits (API parity)
def _with_shift(batch: dict) -> dict:
    if "shift_mask" in batch:
        return batch
    labels = batch["labels"]
    mask = batch.get("loss_mask")
    if mask is None:
        mask = (labels != -100).float()
    tgt, m = shift_labels(labels, mask.float())
    return {**batch, "targets": tgt, "shift_mask": m}


def _lp_ent(logits, batch, need_entropy=True):
    b = _with_shift(batch)
    lp = get_per_token_logprobs(logits, torch.where(b["shift_mask"] > 0, b["targets"], torch.full_like(b["targets"], -1)))
    ent = None
    if need_entropy:
        l32 = F.log_softmax(logits.float(), -1)
        ent = -(l32.exp() * l32).sum(-1)
    return lp, ent, b


def pretrain_loss(logits: torch.Tensor, batch: dict) -> LossOutput:
    lp, _, b = _lp_ent(logits, batch, False)
    return ce_from_logprobs(lp, None, b)


def sft_loss(logits: torch.Tensor, batch: dict) -> LossOutput:
    lp, _, b = _lp_ent(logits, batch, False)
    return ce_from_logprobs(lp, None, b)


def grpo_loss(logits: torch.Tensor, batch: dict) -> LossOutput:
    lp, ent, b = _lp_ent(logits, batch)
    return grpo_from_logprobs(lp, ent.detach(), b)


def grpo_loss_clipped(logits, batch, clip_range: float = 0.2, entropy_coef: float = 0.0) -> LossOutput:
    lp, ent, b = _lp_ent(logits, batch)
    return grpo_clipped_from_logprobs(lp, ent if entropy_coef else ent.detach(), b, clip_range, entropy_coef)


def grpo_loss_masked(logits, batch, ratio_low: float = 0.1, ratio_high: float = 10.0, kl_coef: float = 0.0) -> LossOutput:
    lp, ent, b = _lp_ent(logits, batch)
    return grpo_masked_from_logprobs(lp, ent.detach(), b, ratio_low, ratio_high, kl_coef)


def ppo_loss(logits, batch, clip_range: float = 0.2) -> LossOutput:
    lp, ent, b = _lp_ent(logits, batch, False)
    return ppo_from_logprobs(lp, None, b, clip_range)


LOGPROB_LOSSES = {"ce": ce_from_logprobs, "sft": ce_from_logprobs, "pretrain": ce_from_logprobs,
                  "grpo": grpo_from_logprobs, "grpo_clipped": grpo_clipped_from_logprobs,
                  "grpo_masked": grpo_masked_from_logprobs, "ppo": ppo_from_logprobs}
