"""Offline inference API: ``LLM(model, tensor_parallel_size=..., ...).generate(prompts, sampling_params)``.

Counterpart of vllm/entrypoints/llm.py:162-471 and the ``_run_engine`` loop at :1404-1446. Keyword
arguments are the reference's engine flags that TokenWeave runs use (``tensor_parallel_size``,
``enforce_eager``, ``enable_chunked_prefill``, ``max_num_batched_tokens``, ``disable_custom_all_reduce``,
``enable_prefix_caching``, ``load_format``, ``max_model_len``, ``gpu_memory_utilization``, ``seed``,
``dtype``...), plus ``tokenweave_*`` options.
"""
from __future__ import annotations

import itertools
from typing import Any, Optional, Sequence, Union

from ..config import EngineArgs, ModelConfig
from ..engine.llm_engine import LLMEngine
from ..outputs import BeamSearchOutput, BeamSearchSequence, ClassificationOutput, PoolingOutput, RequestOutput
from ..sampling_params import BeamSearchParams, SamplingParams
from ..utils.logging import init_logger

logger = init_logger(__name__)

PromptType = Union[str, list[int], dict]


class LLM:
    def __init__(self, model: Union[str, ModelConfig] = "tiny-llama", tokenizer: Optional[str] = None,
                 tensor_parallel_size: int = 1, dtype: str = "auto", seed: int = 0, **kwargs: Any):
        if "no_enable_prefix_caching" in kwargs:
            kwargs["enable_prefix_caching"] = not kwargs.pop("no_enable_prefix_caching")
        kwargs.pop("trust_remote_code", None)
        kwargs.pop("tokenizer_mode", None)
        self.engine_args = EngineArgs(model=model, tokenizer=tokenizer, tensor_parallel_size=tensor_parallel_size,
                                      dtype=dtype, seed=seed, **kwargs)
        self.llm_engine = LLMEngine.from_engine_args(self.engine_args)
        self._counter = itertools.count()

    def get_tokenizer(self):
        return self.llm_engine.tokenizer

    # ---- generation ---------------------------------------------------------------------------
    def generate(self, prompts: Union[PromptType, Sequence[PromptType], None] = None,
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 prompt_token_ids: Optional[Sequence[list[int]]] = None, use_tqdm: bool = False,
                 lora_request=None, priority: Optional[Sequence[int]] = None) -> list[RequestOutput]:
        """Generate completions; results come back in prompt order. A prompt is text, a list of token
        ids, or ``{"prompt": ..., "prompt_token_ids": [...]}``. ``lora_request``: a
        :class:`tokenweave_b200.lora.LoRARequest` for all prompts, or one (or None) per prompt.
        ``priority``: one integer per prompt (lower runs first) under ``scheduling_policy="priority"``."""
        if prompts is None:
            if prompt_token_ids is None:
                raise ValueError("give prompts or prompt_token_ids")
            prompts = [list(p) for p in prompt_token_ids]
        elif isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        prompts = list(prompts)
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt (or a single one for all)")
        loras = lora_request if isinstance(lora_request, (list, tuple)) else [lora_request] * len(prompts)
        if len(loras) != len(prompts):
            raise ValueError("one LoRARequest per prompt (or a single one for all)")
        prios = list(priority) if priority is not None else [0] * len(prompts)
        if len(prios) != len(prompts):
            raise ValueError("one priority per prompt")
        ids = []
        for p, sp, lr, pr in zip(prompts, sampling_params, loras, prios):
            rid = str(next(self._counter))
            self.llm_engine.add_request(rid, p, sp, lora_request=lr, priority=int(pr))
            ids.append(rid)
        return self._run_engine(ids, use_tqdm)

    def _run_engine(self, request_ids: list[str], use_tqdm: bool = False) -> list[RequestOutput]:
        final: dict[str, RequestOutput] = {}
        bar = None
        if use_tqdm:
            from tqdm import tqdm
            bar = tqdm(total=len(request_ids), desc="Processed prompts")
        while self.llm_engine.has_unfinished_requests():
            for out in self.llm_engine.step(final_only=True):
                if out.finished:
                    final[out.request_id] = out
                    if bar is not None:
                        bar.update(1)
        if bar is not None:
            bar.close()
        return [final[r] for r in request_ids if r in final]

    # ---- beam search ------------------------------------------------------------------------
    def beam_search(self, prompts: Sequence[PromptType], params: "BeamSearchParams") -> list["BeamSearchOutput"]:
        """Beam search driven from the host, one engine step per generated position: every live beam
        asks for one token with the ``2 * beam_width`` best log-probabilities, the expansions are
        ranked by cumulative log-probability, beams that emit EOS retire to the finished set
        (vllm/entrypoints/llm.py ``LLM.beam_search``). With ``enable_prefix_caching`` the shared
        prefixes of the beams are not recomputed."""
        tok = self.get_tokenizer()
        eos = getattr(tok, "eos_token_id", None) if tok is not None else None
        if eos is None:
            eos = self.llm_engine.eos_token_id
        width = params.beam_width
        step_sp = SamplingParams(temperature=0.0, max_tokens=1, logprobs=2 * width, ignore_eos=True, detokenize=False)
        results = []
        for prompt in prompts:
            ids = self.llm_engine.tokenize_prompt(prompt)
            live = [BeamSearchSequence(tokens=list(ids), cum_logprob=0.0)]
            done: list[BeamSearchSequence] = []
            for _ in range(params.max_tokens):
                if not live:
                    break
                outs = self.generate(prompt_token_ids=[b.tokens for b in live], sampling_params=step_sp)
                cand = []
                for beam, out in zip(live, outs):
                    lps = out.outputs[0].logprobs[0]
                    for t, lp in lps.items():
                        seq = BeamSearchSequence(tokens=beam.tokens + [int(t)], cum_logprob=beam.cum_logprob + float(lp))
                        if int(t) == eos and not params.ignore_eos:
                            done.append(seq)
                        else:
                            cand.append(seq)
                cand.sort(key=lambda s: s.cum_logprob, reverse=True)
                live = cand[:width]
            done.extend(live)

            def score(s: BeamSearchSequence) -> float:
                n = len(s.tokens) - len(ids)
                if s.tokens[-1] == eos:
                    n -= 1
                return s.cum_logprob / (max(n, 1) ** params.length_penalty)

            best = sorted(done, key=score, reverse=True)[:width]
            for s in best:
                s.text = tok.decode(s.tokens[len(ids):]) if tok is not None else None
            results.append(BeamSearchOutput(sequences=best))
        return results

    # ---- pooling ------------------------------------------------------------------------------
    def encode(self, prompts: Union[PromptType, Sequence[PromptType]], normalize: bool = False) -> list["PoolingOutput"]:
        """Last-token pooling of the final-norm hidden state (the default pooler of decoder-only models in
        the reference, vllm/model_executor/layers/pooler.py ``PoolingType.LAST``): one vector per prompt."""
        if isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        prompts = list(prompts)
        outs = self.generate(prompts, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, detokenize=False,
                                                     pooling=True))
        res = []
        for o in outs:
            vec = o.pooled
            if normalize:
                vec = vec / vec.norm().clamp_min(1e-12)
            res.append(PoolingOutput(request_id=o.request_id, prompt_token_ids=o.prompt_token_ids, data=vec))
        return res

    def embed(self, prompts: Union[PromptType, Sequence[PromptType]]) -> list["PoolingOutput"]:
        """L2-normalised :meth:`encode` (``LLM.embed`` of the reference)."""
        return self.encode(prompts, normalize=True)

    def classify(self, prompts: Union[PromptType, Sequence[PromptType]]) -> list["ClassificationOutput"]:
        """Class probabilities for checkpoints with a sequence-classification head (``score.weight`` of the
        ``*ForSequenceClassification`` layouts): the head is applied to the last token's final-norm hidden
        state and soft-maxed (``LLM.classify`` of the reference, pooler ``PoolingType.LAST`` + softmax)."""
        import torch
        head = self._classifier_head()
        res = []
        for o in self.encode(prompts):
            probs = torch.softmax(o.data.float() @ head.t(), dim=-1)
            res.append(ClassificationOutput(o.request_id, o.prompt_token_ids, probs.tolist()))
        return res

    def _classifier_head(self):
        head = getattr(self, "_score_head", None)
        if head is None:
            from ..models.loader import iter_checkpoint
            path = self.llm_engine.config.model.path
            if path is not None:
                for name, tensor in iter_checkpoint(path):
                    if name in ("score.weight", "classifier.weight"):
                        head = tensor.float()
                        break
            if head is None:
                raise ValueError("classify() needs a checkpoint with a sequence-classification head (score.weight)")
            self._score_head = head
        return head

    def score(self, text_1: Union[PromptType, Sequence[PromptType]], text_2: Union[PromptType, Sequence[PromptType]]) -> list[float]:
        """Cosine similarity of the embeddings of ``text_1`` and ``text_2`` (one-to-many or pairwise), the
        embedding-model branch of the reference's ``LLM.score``."""
        one = lambda x: isinstance(x, (str, dict)) or (isinstance(x, list) and x and isinstance(x[0], int))  # noqa: E731
        a = [text_1] if one(text_1) else list(text_1)
        b = [text_2] if one(text_2) else list(text_2)
        if len(a) == 1 and len(b) > 1:
            a = a * len(b)
        if len(a) != len(b):
            raise ValueError("score() takes one-to-many or equally long lists")
        ea, eb = self.embed(a), self.embed(b)
        return [float((x.data * y.data).sum()) for x, y in zip(ea, eb)]

    # ---- utilities ------------------------------------------------------------------------------
    def collective_rpc(self, method: str, *args, **kwargs) -> list[Any]:
        return self.llm_engine.core.executor.collective_rpc(method, *args, **kwargs)

    def start_profile(self) -> None:
        self.collective_rpc("profile", True)

    def stop_profile(self) -> None:
        self.collective_rpc("profile", False)

    def chat(self, messages, sampling_params: Optional[SamplingParams] = None, add_generation_prompt: bool = True,
             use_tqdm: bool = False) -> list[RequestOutput]:
        """Chat completion: ``messages`` is one conversation (a list of ``{"role", "content"}`` dicts) or a
        list of conversations. Uses the tokenizer's chat template when it has one, else a plain
        ``role: content`` transcript (vllm/entrypoints/llm.py ``LLM.chat``)."""
        tok = self.get_tokenizer()
        if tok is None:
            raise ValueError("chat() needs a tokenizer")
        convs = [messages] if messages and isinstance(messages[0], dict) else list(messages)
        prompts = []
        for conv in convs:
            if hasattr(tok, "apply_chat_template") and getattr(tok, "chat_template", None):
                prompts.append(tok.apply_chat_template(conv, tokenize=False, add_generation_prompt=add_generation_prompt))
            else:
                text = "".join(f"{m['role']}: {m['content']}\n" for m in conv)
                prompts.append(text + ("assistant: " if add_generation_prompt else ""))
        return self.generate(prompts, sampling_params, use_tqdm=use_tqdm)

    def sleep(self, level: int = 1) -> None:
        """Release GPU memory between uses: the KV cache is dropped, and at level 1 the weights move to
        pinned host memory (level 2 discards them). Counterpart of ``LLM.sleep`` / the cumem allocator of
        the reference (vllm/device_allocator/cumem.py); here tensors are moved, not unmapped."""
        if self.llm_engine.has_unfinished_requests():
            raise RuntimeError("cannot sleep with requests in flight")
        self.reset_prefix_cache()           # the KV contents do not survive
        self.collective_rpc("sleep", level)

    def reset_prefix_cache(self) -> bool:
        core = self.llm_engine.core
        if not hasattr(core.scheduler, "kv"):
            # the scheduler lives in the core process: it drops its prefix cache there
            return bool(core.rpc_core("reset_prefix_cache"))
        return core.scheduler.kv.pool.reset_prefix_cache()

    def wake_up(self) -> None:
        self.collective_rpc("wake_up")

    def save_sharded_state(self, path: str) -> None:
        """Write every rank's already-sharded parameters to ``path/rank_<r>.safetensors`` so that a later
        start can skip resharding (vllm/v1/worker/gpu_worker.py:273-285)."""
        self.collective_rpc("save_sharded_state", path)

    def shutdown(self) -> None:
        self.llm_engine.shutdown()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass
