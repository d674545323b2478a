"""Token sampling from fp32 logits: greedy, temperature, top-k / top-p / min-p, repetition / presence /
frequency penalties, per-request seeded generators, optional log-probabilities.

Counterpart of vllm/v1/sample/sampler.py:17-270 and ops/topk_topp_sampler.py:170-262. Random draws use
the exponential-race form ``argmax(p / Exp(1))`` so that no host synchronisation is needed; the
all-greedy batch (the latency benchmarks) takes a single argmax kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import ops
from ..sampling_params import SamplingParams


@dataclass
class SamplerOutput:
    token_ids: torch.Tensor                      # [B] int32 (device)
    logprobs: Optional[list] = None              # per request: dict token -> logprob (top-n + sampled)


def apply_penalties(logits: torch.Tensor, params: Sequence[SamplingParams], prompt_tokens: Sequence[Sequence[int]],
                    output_tokens: Sequence[Sequence[int]], guided=None) -> torch.Tensor:
    """Edits the logits rows in place. ``guided(sp, generated tokens)`` returns the token ids a structured-output
    constraint allows next (None: the request has no such constraint)."""
    V = logits.shape[1]
    for i, sp in enumerate(params):
        if not sp.needs_penalties:
            continue
        allowed_next = guided(sp, output_tokens[i]) if guided is not None else None
        if allowed_next is not None:
            # regex / JSON-schema constraint (vllm/v1/structured_output: the grammar bitmask applied to the logits)
            keep = torch.as_tensor([t for t in allowed_next if 0 <= t < V], dtype=torch.long, device=logits.device)
            masked = torch.full_like(logits[i], float("-inf"))
            masked[keep] = logits[i, keep]
            logits[i] = masked
        out_ids = torch.as_tensor(list(output_tokens[i]), dtype=torch.long, device=logits.device)
        if sp.repetition_penalty != 1.0:
            seen = torch.as_tensor(list(prompt_tokens[i]) + list(output_tokens[i]), dtype=torch.long, device=logits.device)
            seen = seen[seen < V].unique()
            row = logits[i, seen]
            logits[i, seen] = torch.where(row > 0, row / sp.repetition_penalty, row * sp.repetition_penalty)
        if out_ids.numel() and (sp.frequency_penalty != 0.0 or sp.presence_penalty != 0.0):
            counts = torch.bincount(out_ids[out_ids < V], minlength=V).to(logits.dtype)
            logits[i] -= sp.frequency_penalty * counts
            logits[i] -= sp.presence_penalty * (counts > 0).to(logits.dtype)
        # logit bias, allowed-token and bad-word masks, minimum length
        # (vllm/v1/sample/sampler.py ``apply_logits_bias`` / ``apply_allowed_token_ids`` / ``apply_bad_words``,
        # vllm/v1/sample/logits_processor.py ``MinTokensLogitsProcessor``)
        if sp.logit_bias:
            ids = torch.as_tensor([t for t in sp.logit_bias if 0 <= t < V], dtype=torch.long, device=logits.device)
            vals = torch.as_tensor([sp.logit_bias[int(t)] for t in ids.tolist()], dtype=logits.dtype, device=logits.device)
            logits[i, ids] += vals
        if sp.allowed_token_ids is not None:
            keep = torch.as_tensor([t for t in sp.allowed_token_ids if 0 <= t < V], dtype=torch.long, device=logits.device)
            masked = torch.full_like(logits[i], float("-inf"))
            masked[keep] = logits[i, keep]
            logits[i] = masked
        if sp.bad_words_token_ids:
            hist = list(output_tokens[i])
            for word in sp.bad_words_token_ids:
                prefix, last = word[:-1], word[-1]
                # the last token of a bad word is banned when the tokens generated so far end with its prefix
                if 0 <= last < V and (not prefix or (len(hist) >= len(prefix) and hist[-len(prefix):] == list(prefix))):
                    logits[i, last] = float("-inf")
        if sp.guided_choice_token_ids:
            # constrained to one of several token sequences: only the tokens that continue a still-possible
            # choice are allowed; a completed choice that is a prefix of a longer one may also end (EOS)
            hist = list(output_tokens[i])
            n = len(hist)
            alive = [c for c in sp.guided_choice_token_ids if len(c) >= n and list(c[:n]) == hist]
            allowed = {int(c[n]) for c in alive if len(c) > n and 0 <= c[n] < V}
            if any(len(c) == n for c in alive) and sp.eos_token_id is not None:
                allowed.add(int(sp.eos_token_id))
            if allowed:
                keep = torch.as_tensor(sorted(allowed), dtype=torch.long, device=logits.device)
                masked = torch.full_like(logits[i], float("-inf"))
                masked[keep] = logits[i, keep]
                logits[i] = masked
        if sp.min_tokens > 0 and len(output_tokens[i]) < sp.min_tokens:
            stops = [t for t in ([sp.eos_token_id] if sp.eos_token_id is not None else []) + list(sp.stop_token_ids)
                     if 0 <= t < V]
            if stops:
                logits[i, torch.as_tensor(stops, dtype=torch.long, device=logits.device)] = float("-inf")
    return logits


def _filter_top_k_top_p(logits: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor) -> torch.Tensor:
    """Sort-based joint top-k / top-p mask (ascending sort, as in the reference)."""
    V = logits.shape[1]
    if bool((top_k < V).any()) or bool((top_p < 1.0).any()):
        sorted_logits, idx = logits.sort(dim=-1, descending=False)
        kth = sorted_logits.gather(1, (V - top_k.clamp(max=V)).unsqueeze(1).long())
        sorted_logits = sorted_logits.masked_fill(sorted_logits < kth, float("-inf"))
        probs = sorted_logits.softmax(dim=-1)
        cum = probs.cumsum(dim=-1)
        mask = cum <= (1.0 - top_p).unsqueeze(1)
        mask[:, -1] = False
        sorted_logits = sorted_logits.masked_fill(mask, float("-inf"))
        logits = torch.empty_like(logits).scatter_(1, idx, sorted_logits)
    if bool((min_p > 0).any()):
        probs = logits.softmax(dim=-1)
        thresh = probs.max(dim=-1, keepdim=True).values * min_p.unsqueeze(1)
        logits = logits.masked_fill(probs < thresh, float("-inf"))
    return logits


_MASK64 = (1 << 64) - 1


class Sampler:
    """On a GPU a batch that is not all-greedy is sampled by one launch of the fused kernel
    (``ops.sample``: temperature, top-k / top-p / min-p and the draw, no sort); on the CPU, and as the
    oracle of that kernel, the sort-based PyTorch path below is used."""

    def __init__(self, seed: int = 0, use_fused_kernel: bool = True):
        import random
        self._rng = random.Random(seed)      # row seeds of unseeded requests; identical on every TP rank
        self.use_fused_kernel = use_fused_kernel
        self.vocab_provider = None           # () -> list of token byte strings; set by the model runner
        self._trie = None

    def _guided(self, sp: SamplingParams, generated) -> Optional[list]:
        """Allowed next tokens under the request's regex / JSON-schema constraint."""
        from ..engine import structured
        pattern = structured.constraint_pattern(sp)
        if pattern is None:
            return None
        if self._trie is None:
            if self.vocab_provider is None:
                raise RuntimeError("structured output needs the tokenizer's vocabulary on the worker")
            self._trie = structured.TokenTrie(self.vocab_provider())
        fsm = structured.get_fsm(pattern, self._trie, sp.eos_token_id)
        allowed = fsm.allowed_tokens(fsm.state_after(generated))
        # a dead end (only reachable if a token outside the mask was forced in): let the request end
        return allowed if allowed else ([sp.eos_token_id] if sp.eos_token_id is not None else None)

    def _row_seeds(self, params: Sequence[SamplingParams], output_tokens) -> list[int]:
        seeds = []
        for i, sp in enumerate(params):
            if sp.seed is None:
                seeds.append(self._rng.getrandbits(64))
            else:       # a seeded request repeats: the draw depends on (seed, position) only
                n = len(output_tokens[i]) if output_tokens is not None else 0
                seeds.append(((sp.seed + 1) * 0x9E3779B97F4A7C15 + (n + 1) * 0xD1B54A32D192ED03) & _MASK64)
        return seeds

    def _sample_fused(self, logits: torch.Tensor, params: Sequence[SamplingParams], output_tokens) -> torch.Tensor:
        packed = ops.pack_sample_params(
            [0.0 if sp.greedy else sp.temperature for sp in params], [sp.top_k for sp in params],
            [sp.top_p for sp in params], [sp.min_p for sp in params], self._row_seeds(params, output_tokens))
        return ops.sample(logits, packed.pin_memory().to(logits.device, non_blocking=True))

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                 generators: Sequence[Optional[torch.Generator]], prompt_tokens=None, output_tokens=None,
                 needs_penalties: Optional[Sequence[bool]] = None) -> SamplerOutput:
        """``needs_penalties``: per request, whether its logits have to be edited (the caller may have cached what
        ``SamplingParams.needs_penalties`` works out from a dozen fields)."""
        B, V = logits.shape
        want_logprobs = any(sp.logprobs is not None for sp in params)
        # reported log-probabilities are the model's own: taken before penalties, logit bias and masks touch the
        # logits (vllm/v1/sample/sampler.py:36-47 computes its raw_logprobs first as well)
        raw_logprobs = torch.log_softmax(logits.float(), dim=-1) if want_logprobs else None
        if any(needs_penalties) if needs_penalties is not None else any(sp.needs_penalties for sp in params):
            logits = apply_penalties(logits.clone(), params, prompt_tokens, output_tokens, guided=self._guided)
        if all(sp.greedy for sp in params):
            ids = ops.argmax(logits)
        elif logits.is_cuda and self.use_fused_kernel:
            ids = self._sample_fused(logits, params, output_tokens)
        else:
            dev = logits.device
            temp = torch.tensor([1.0 if sp.greedy else sp.temperature for sp in params], dtype=torch.float32, device=dev)
            top_k = torch.tensor([V if sp.top_k <= 0 else min(sp.top_k, V) for sp in params], dtype=torch.long, device=dev)
            top_p = torch.tensor([sp.top_p for sp in params], dtype=torch.float32, device=dev)
            min_p = torch.tensor([sp.min_p for sp in params], dtype=torch.float32, device=dev)
            scaled = _filter_top_k_top_p(logits / temp.unsqueeze(1), top_k, top_p, min_p)
            probs = scaled.softmax(dim=-1)
            noise = torch.empty_like(probs)
            for i, g in enumerate(generators):
                noise[i].exponential_(generator=g)
            sampled = (probs / noise).argmax(dim=-1)
            greedy = torch.tensor([sp.greedy for sp in params], dtype=torch.bool, device=dev)
            ids = torch.where(greedy, logits.argmax(dim=-1), sampled).to(torch.int32)
        lp_out = None
        if want_logprobs:
            lp_out = []
            ids_l = ids.long()
            for i, sp in enumerate(params):
                if sp.logprobs is None:
                    lp_out.append(None)
                    continue
                row = raw_logprobs[i]
                d = {int(ids_l[i]): float(row[ids_l[i]])}
                if sp.logprobs > 0:
                    vals, toks = row.topk(min(sp.logprobs, V))
                    d.update({int(t): float(v) for t, v in zip(toks.tolist(), vals.tolist())})
                lp_out.append(d)
        return SamplerOutput(ids, lp_out)
