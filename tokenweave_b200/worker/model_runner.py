"""Model runner: turns the scheduler's decision for one step into device inputs, runs the model and
samples.

Counterpart of vllm/v1/worker/gpu_model_runner.py:532-746 (input preparation incl. the TokenWeave split
metadata) and :1117-1380 (execute_model). Request state (token ids, block ids, sampling parameters,
generators) is cached on the worker so a running request costs a few integers per step on the wire.
All integer inputs of a step are packed into pinned staging memory and reach the device in two
``non_blocking`` copies (token ids; attention metadata).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .. import envs, ops
from ..config import EngineConfig
from ..layers.attention import AttentionMetadata, build_attention_metadata
from ..layers.sampler import Sampler
from ..models.decoder import DecoderModel, StepInput
from ..parallel.state import broadcast_from_last_stage, get_tp
from ..sampling_params import SamplingParams
from ..tokenweave.config import TokenWeavePlanner
from ..utils.logging import init_logger
from .split_metadata import split_batch

logger = init_logger(__name__)


@dataclass
class NewRequestData:
    req_id: str
    token_ids: list[int]             # prompt (+ outputs generated before a preemption)
    num_prompt_tokens: int
    sampling_params: SamplingParams
    block_ids: list[int]
    lora_request: Optional[object] = None        # tokenweave_b200.lora.LoRARequest


@dataclass
class StepData:
    """What the scheduler sends to the workers for one step (picklable)."""
    step_id: int
    new_requests: list[NewRequestData] = field(default_factory=list)
    # (req_id, num_computed_tokens, num_new_tokens, block ids appended since the last step)
    scheduled: list[tuple[str, int, int, list[int]]] = field(default_factory=list)
    finished_req_ids: list[str] = field(default_factory=list)
    preempted_req_ids: list[str] = field(default_factory=list)
    total_num_tokens: int = 0


@dataclass
class StepResult:
    req_ids: list[str]
    sampled_token_ids: list[Optional[int]]
    logprobs: Optional[list] = None
    device_time_ms: Optional[float] = None
    # request id -> [(prompt position, {token id: log-probability})] for the prompt positions of this step
    prompt_logprobs: Optional[dict] = None
    pooled: Optional[dict] = None        # request id -> final-norm hidden state (host fp32) of pooling requests


@dataclass
class _CachedRequest:
    token_ids: list[int]
    num_prompt_tokens: int
    sampling_params: SamplingParams
    block_ids: list[int]
    generator: Optional[torch.Generator] = None
    lora_id: int = 0
    # fixed for the life of a request (its sampling parameters do not change once it is with the workers); read
    # for every request on every step, so not recomputed from the dozen fields behind them each time
    needs_penalties: bool = False
    plain_greedy: bool = False        # greedy, no logits edits, no log-probabilities: the argmax kernel suffices

    def __post_init__(self):
        sp = self.sampling_params
        self.needs_penalties = bool(sp.needs_penalties)
        self.plain_greedy = bool(sp.greedy and not self.needs_penalties and sp.logprobs is None)
        self._blocks_np = np.empty(max(16, 2 * len(self.block_ids)), dtype=np.int32)
        self._blocks_n = 0

    def block_array(self) -> np.ndarray:
        """``block_ids`` as an int32 array that grows with the list (block-table rows are filled from it on every
        step; converting the list each time was a visible share of a decode step's host time)."""
        n = len(self.block_ids)
        if n > self._blocks_n:
            if n > self._blocks_np.size:
                grown = np.empty(2 * n, dtype=np.int32)
                grown[:self._blocks_n] = self._blocks_np[:self._blocks_n]
                self._blocks_np = grown
            self._blocks_np[self._blocks_n:n] = self.block_ids[self._blocks_n:n]
            self._blocks_n = n
        return self._blocks_np[:n]


class ModelRunner:
    def __init__(self, config: EngineConfig, device: torch.device):
        self.config = config
        self.device = device
        self.tp = get_tp()
        self.model: Optional[DecoderModel] = None
        self.requests: dict[str, _CachedRequest] = {}
        self.sampler = Sampler(seed=config.seed)
        self.sampler.vocab_provider = self._token_bytes       # structured output: built on first use
        self.block_size = config.cache.block_size
        self.max_tokens = config.scheduler.max_num_batched_tokens
        tw = config.tokenweave
        self.planner = TokenWeavePlanner(
            config.model.architecture, self.tp.world_size, tw.mode, tw.config_path, tw.overlap_threshold,
            tw.fuse_only_ctas, tw.split_offset, tw.attention_ctas, tw.mlp_ctas,
            force_overlap=tw.force_overlap)
        pin = device.type == "cuda"
        self._ids_host = torch.zeros(self.max_tokens, dtype=torch.int32, pin_memory=pin)
        self._ids_dev = torch.zeros(self.max_tokens, dtype=torch.int32, device=device)
        self._meta_host = [torch.zeros(1 << 20, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.h2d_bytes_last_step = 0
        self.d2h_bytes_last_step = 0
        self.timing_events = None
        self.capture_logits = False          # tests: keep the fp32 logits of every step
        self.captured_logits: list = []
        self.lora = None                     # LoRAManager when the engine was built with enable_lora
        self.capture_hidden = False          # pooling requests: keep the final-norm hidden row of every sampled position
        self.captured_hidden: dict = {}
        self._want_pooled = False            # this step samples for a request with SamplingParams.pooling
        from ..ops.reference import longrope_offset
        self._longrope_offset = longrope_offset(config.model.rope_scaling, config.model.max_model_len)
        self._h2d_done = torch.cuda.Event() if pin else None   # guards reuse of the pinned staging buffers
        # CUDA graphs: a step whose shape signature has been seen before is replayed from a captured graph
        self.use_graphs = bool(tw.use_cuda_graphs) and pin and self.tp.pp_size == 1    # stage hand-offs are not captured
        self._meta_dev = [torch.zeros(1 << 20, dtype=torch.int32, device=device) if self.use_graphs else None
                          for _ in range(2)]
        # logits rows per step: one per sequence, plus one per draft token under speculative decoding
        k_spec = config.speculative.num_speculative_tokens if config.speculative is not None else 0
        n_rows = max(config.scheduler.max_num_seqs, 1) * (1 + k_spec)
        self._rows_dev = torch.zeros(n_rows, dtype=torch.long, device=device)
        self._rows_host = torch.zeros(n_rows, dtype=torch.long, pin_memory=pin)
        # the word kernels OR their error codes into travels to the host with the sampled ids of every step
        self._status_src = (lambda: ops.status_word(device)) if pin else None
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=pin)
        self._graphs: dict = {}
        self._graph_seen: dict = {}
        self._graph_pool = None
        self.graph_replays = 0

    # ---- set-up -----------------------------------------------------------------------------
    def load_model(self, embedding_parallel: bool = False, weights_pool=None) -> None:
        """``weights_pool``: optional allocation context for the parameters only (sleep mode); activation
        buffers, the rotary table and the symmetric staging buffer stay in ordinary memory."""
        import contextlib
        from ..models.registry import build_model
        t0 = time.monotonic()
        with (weights_pool if weights_pool is not None else contextlib.nullcontext()):
            self.model = build_model(self.config, self.device, embedding_parallel)
        self.model.setup_runtime(self.max_tokens, self.config.tokenweave,
                                 disable_custom_all_reduce=self.config.parallel.disable_custom_all_reduce)
        if self.config.enable_lora:
            from ..lora import LoRAManager
            self.lora = LoRAManager(self.model, self.config.max_loras)
            self.model.rt.lora = self.lora
        logger.info("model %s ready on %s in %.1fs (%.2f GB of weights on this rank)", self.config.model.name,
                    self.device, time.monotonic() - t0,
                    sum(p.numel() * p.element_size() for p in self.model.parameters()) / 1e9)

    def init_kv_cache(self, num_blocks: int) -> None:
        self.model.init_kv_cache(num_blocks, self.block_size)

    def release_graphs(self) -> None:
        """Drop every captured CUDA graph and the pool they allocate from."""
        if self._graphs:
            torch.cuda.synchronize()
        self._graphs.clear()
        self._graph_seen.clear()
        self._graph_pool = None

    def _token_bytes(self) -> list:
        """Bytes every vocabulary entry contributes to the text, from the same tokenizer the front end uses."""
        from ..engine.structured import token_bytes_table
        from ..engine.tokenizer import load_tokenizer
        cfg = self.config
        tok = load_tokenizer(cfg.tokenizer or (cfg.model.path if cfg.model.path else "byte"))
        return token_bytes_table(tok, cfg.model.vocab_size)

    # ---- one step ---------------------------------------------------------------------------
    def _update_states(self, step: StepData) -> None:
        for rid in step.finished_req_ids:
            self.requests.pop(rid, None)
        for rid in step.preempted_req_ids:
            self.requests.pop(rid, None)
        for nr in step.new_requests:
            gen = None
            sp = nr.sampling_params
            if sp.seed is not None:
                gen = torch.Generator(device=self.device)
                gen.manual_seed(sp.seed)
            lora_id = 0
            if nr.lora_request is not None:
                if self.lora is None:
                    raise RuntimeError("a request names a LoRA adapter but the engine was built without enable_lora")
                self.lora.ensure_loaded(nr.lora_request)
                lora_id = nr.lora_request.lora_int_id
            self.requests[nr.req_id] = _CachedRequest(list(nr.token_ids), nr.num_prompt_tokens, sp, list(nr.block_ids), gen,
                                                      lora_id)

    def _build_metadata(self, entries, tokens_base: int, positions: np.ndarray, slots: np.ndarray,
                        tables: dict[int, list[int]], which: int) -> AttentionMetadata:
        """entries: list of (seq_index, q_len, kv_len) laid out back to back starting at row tokens_base."""
        q_lens = [e[1] for e in entries]
        kv_lens = [e[2] for e in entries]
        n = sum(q_lens)
        max_blocks = max((len(tables[e[0]]) for e in entries), default=1)
        if self.use_graphs:
            max_blocks = (max_blocks + 15) // 16 * 16      # fewer distinct graph signatures
        bt = np.zeros((len(entries), max(1, max_blocks)), dtype=np.int32)
        for i, e in enumerate(entries):
            t = tables[e[0]]
            bt[i, : len(t)] = t
        return build_attention_metadata(q_lens, kv_lens, positions[tokens_base:tokens_base + n],
                                        slots[tokens_base:tokens_base + n], bt, self.device, self._meta_host[which],
                                        self._meta_dev[which])

    def _signature(self, step_in: StepInput, n_logits: int, greedy: bool):
        parts = [step_in.plan, n_logits, greedy]
        for m in (step_in.meta, step_in.meta0, step_in.meta1):
            if m is None:
                parts.append(None)
                continue
            a = self.model.layers[0].attn
            splits = ops.decode_plan(m.num_single, a.hq, a.hkv, a.head_dim, self.block_size,
                                     min(m.max_kv_len, a.window) if a.window > 0 else m.max_kv_len,
                                     self.model.rt.sm_count, a.window <= 0 and a.softcap <= 0)
            parts.append((m.num_actual_tokens, m.num_seqs, m.num_tiles, m.num_single, m.block_table.shape[1], splits))
        return tuple(parts)

    def _forward_and_logits(self, step_in: StepInput, n_logits: int, greedy: bool):
        hidden = self.model(step_in)
        if n_logits == 0:
            return None, None
        rows = hidden.index_select(0, self._rows_dev[:n_logits])
        if self.capture_hidden or self._want_pooled:
            self._last_hidden_rows = rows
        logits = self.model.compute_logits(rows)
        return logits, (ops.argmax(logits) if greedy else None)

    def _run_graphed(self, sig, step_in: StepInput, n_logits: int, greedy: bool):
        """Eager on the first sight of a signature (which also warms every kernel up), then captured and replayed.
        A capture costs a device synchronisation plus tens of milliseconds, so it has to pay for itself: steps that
        are all single-token rows (decode) or one prefill of one sequence repeat for many steps and are captured on
        their second sight; steps that mix prefill chunks with decode rows rarely come back with the same shape and
        are captured only after ``TW_GRAPH_MIXED_SIGHTS`` (4) sights (a throughput run with chunked prefill lost 15 % to captures of shapes
        that were never replayed)."""
        entry = self._graphs.get(sig)
        if entry is None:
            seen = self._graph_seen.get(sig, 0)
            self._graph_seen[sig] = seen + 1
            metas = [m for m in (step_in.meta, step_in.meta0, step_in.meta1) if m is not None]
            steady = all(m.num_tiles == 0 or (m.num_single == 0 and m.num_seqs == 1) for m in metas)
            if seen < (1 if steady else envs.TW_GRAPH_MIXED_SIGHTS) or len(self._graphs) >= 64:
                return self._forward_and_logits(step_in, n_logits, greedy)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                out = self._forward_and_logits(step_in, n_logits, greedy)
            entry = (graph, out)
            self._graphs[sig] = entry
        entry[0].replay()
        self.graph_replays += 1
        return entry[1]

    @torch.inference_mode()
    def execute_model(self, step: StepData) -> StepResult:
        self._update_states(step)
        if not step.scheduled:
            return StepResult([], [])
        T = step.total_num_tokens
        assert T <= self.max_tokens, f"step of {T} tokens exceeds max_num_batched_tokens={self.max_tokens}"
        if self._h2d_done is not None:
            self._h2d_done.synchronize()      # the previous step's copies have left the staging buffers
        ids = self._ids_host.numpy()
        positions = np.empty(T, dtype=np.int32)
        slots = np.empty(T, dtype=np.int32)
        q_lens, kv_lens, tables = [], [], {}
        logits_rows, sample_reqs = [], []
        row = 0
        bs = self.block_size
        spec: dict[str, list[int]] = {}          # request -> drafts verified in this step
        row_lora: list[int] = []                 # adapter id of every token row (0 = none)
        prompt_lp_jobs: list[tuple[str, int, int, int]] = []     # (request, first row, first position, rows)
        for b, (rid, computed, n_new, new_blocks, *rest) in enumerate(step.scheduled):
            req = self.requests[rid]
            req.block_ids.extend(new_blocks)
            drafts = list(rest[0]) if rest and rest[0] else []
            if n_new == 1 and not drafts and req.sampling_params.prompt_logprobs is None:
                # decode fast path (most rows of a serving step): scalars only, no array temporaries
                ids[row] = req.token_ids[computed]
                positions[row] = computed
                slots[row] = req.block_ids[computed // bs] * bs + computed % bs
                q_lens.append(1)
                kv_lens.append(computed + 1)
                tables[b] = req.block_array()
                if computed + 1 >= len(req.token_ids):
                    logits_rows.append(row)
                    sample_reqs.append(rid)
                if self.lora is not None:
                    row_lora.append(req.lora_id)
                row += 1
                continue
            n_base = n_new - len(drafts)             # tokens of the request itself; the drafts follow them
            ids[row:row + n_base] = req.token_ids[computed:computed + n_base]
            if drafts:
                ids[row + n_base:row + n_new] = drafts
                spec[rid] = drafts
            pos = np.arange(computed, computed + n_new, dtype=np.int32)
            positions[row:row + n_new] = pos
            blocks = req.block_array()
            slots[row:row + n_new] = blocks[pos // bs] * bs + pos % bs
            q_lens.append(n_new)
            kv_lens.append(computed + n_new)
            tables[b] = blocks
            if computed + n_base >= len(req.token_ids):
                # one logits row at the request's last own token, and one after every draft
                for k in range(len(drafts) + 1):
                    logits_rows.append(row + n_base - 1 + k)
                    sample_reqs.append(rid)
            if self.lora is not None:
                row_lora.extend([req.lora_id] * n_new)
            if req.sampling_params.prompt_logprobs is not None and computed < req.num_prompt_tokens - 1:
                # rows of prompt positions p whose successor p + 1 is still a prompt token
                n_pl = min(computed + n_base, req.num_prompt_tokens - 1) - computed
                prompt_lp_jobs.append((rid, row, computed, n_pl))
            row += n_new
        if self.lora is not None:
            self.lora.set_batch(row_lora)

        if self._longrope_offset and T and int(positions[:T].max()) > self._longrope_offset:
            # LongRoPE: a step that reaches beyond the original window rotates all its tokens with the "long"
            # factors, which sit behind the "short" rows of the rotary table (slots were computed above)
            positions = positions + np.int32(self._longrope_offset)
        plan = self.planner.plan(T)
        ids_dev = self._ids_dev[:T]
        ids_dev.copy_(self._ids_host[:T], non_blocking=True)
        h2d = T * 4
        if plan.overlap:
            first, second = split_batch(q_lens, kv_lens, plan.split)
            meta0 = self._build_metadata(first, 0, positions, slots, tables, 0)
            meta1 = self._build_metadata(second, plan.split, positions, slots, tables, 1)
            step_in = StepInput(ids_dev, plan, meta0=meta0, meta1=meta1)
        else:
            entries = [(b, q_lens[b], kv_lens[b]) for b in range(len(q_lens))]
            step_in = StepInput(ids_dev, plan, meta=self._build_metadata(entries, 0, positions, slots, tables, 0))
        for m in (step_in.meta, step_in.meta0, step_in.meta1):
            if m is not None:
                h2d += 4 * (2 * m.num_actual_tokens + 2 * m.num_seqs + 1 + m.block_table.numel() + 2 * m.num_tiles + 3 * m.num_single)

        if self._h2d_done is not None:
            self._h2d_done.record()
        ev = None
        if self.timing_events is not None:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        if self.tp.pp_size > 1 and not self.tp.is_last_stage:
            # an inner pipeline stage: run the local layers (the model hands its output to the next stage); the
            # sampled tokens come back from the last stage with the rest of the step's result
            self.model(step_in)
            if ev is not None:
                ev[1].record()
                self.timing_events.append(ev)
            self.h2d_bytes_last_step, self.d2h_bytes_last_step = h2d, 0
            result = broadcast_from_last_stage(None)
            for rid, tok in zip(result.req_ids, result.sampled_token_ids):
                if tok is not None:
                    self.requests[rid].token_ids.extend(list(tok) if isinstance(tok, (list, tuple)) else [int(tok)])
            return result
        n_logits = len(logits_rows)
        reqs = [self.requests[r] for r in sample_reqs]
        greedy = bool(reqs) and all(r.plain_greedy for r in reqs)
        if n_logits:
            self._rows_host[:n_logits] = torch.as_tensor(logits_rows, dtype=torch.long)
            self._rows_dev[:n_logits].copy_(self._rows_host[:n_logits], non_blocking=True)
        lora_active = self.lora is not None and self.lora.active      # row gathers of a step are not graph-stable
        self._want_pooled = any(r.sampling_params.pooling for r in reqs)
        if (self.use_graphs and not self.capture_logits and not self.capture_hidden and not lora_active
                and not self._want_pooled):
            logits, greedy_ids = self._run_graphed(self._signature(step_in, n_logits, greedy), step_in, n_logits, greedy)
        else:
            logits, greedy_ids = self._forward_and_logits(step_in, n_logits, greedy)
        sampled: dict[str, int] = {}
        lp = None
        d2h = 0
        prompt_lp = self._prompt_logprobs(prompt_lp_jobs) if prompt_lp_jobs else None
        pooled = None
        if logits_rows and self._want_pooled:
            host_rows = self._last_hidden_rows.detach().float().cpu()
            pooled = {rid: host_rows[i].clone() for i, (rid, r) in enumerate(zip(sample_reqs, reqs))
                      if r.sampling_params.pooling}
        if logits_rows:
            if self.capture_hidden:
                rows = self._last_hidden_rows.detach().float().cpu()
                for rid, row in zip(sample_reqs, rows):
                    self.captured_hidden.setdefault(rid, row.clone())
            if self.capture_logits:
                self.captured_logits.append((list(sample_reqs), logits.detach().float().cpu().clone()))
            if greedy_ids is not None:
                from ..layers.sampler import SamplerOutput
                out = SamplerOutput(greedy_ids)
            else:
                # the token history is copied only for the requests whose logits it edits (penalties, masks);
                # everyone else gets its LENGTH (seeded draws depend on the position), not a copy of its tokens:
                # slicing every prompt on every step cost milliseconds per decode step of a full batch
                prompts_h, outputs_h = [], []
                for r in reqs:
                    n_p = r.num_prompt_tokens
                    if r.needs_penalties:
                        prompts_h.append(r.token_ids[:n_p])
                        outputs_h.append(r.token_ids[n_p:])
                    else:
                        prompts_h.append(())
                        outputs_h.append(range(len(r.token_ids) - n_p))
                out = self.sampler(logits, [r.sampling_params for r in reqs], [r.generator for r in reqs],
                                   prompts_h, outputs_h, [r.needs_penalties for r in reqs])
            if ev is not None:
                ev[1].record()
            if self._status_src is not None:
                self._status_host.copy_(self._status_src(), non_blocking=True)
            toks = out.token_ids.tolist()            # the device -> host synchronisation point of the step
            d2h = len(toks) * 4
            if self._status_src is not None:
                d2h += 4
                self._raise_on_device_status()
            lp = out.logprobs
            i = 0
            while i < len(toks):
                rid = sample_reqs[i]
                drafts = spec.get(rid)
                if drafts:
                    # speculative decoding: rows i .. i + len(drafts) are the model's choices after the last
                    # sampled token and after every draft; keep the confirmed drafts and one more token
                    from ..engine.spec_decode import accept_greedy
                    emitted = accept_greedy(drafts, toks[i:i + len(drafts) + 1])
                    sampled[rid] = emitted
                    self.requests[rid].token_ids.extend(emitted)
                    i += len(drafts) + 1
                else:
                    sampled[rid] = int(toks[i])
                    self.requests[rid].token_ids.append(int(toks[i]))
                    i += 1
        elif ev is not None:
            ev[1].record()
        if ev is not None:
            self.timing_events.append(ev)
        self.h2d_bytes_last_step, self.d2h_bytes_last_step = h2d, d2h
        req_ids = [s[0] for s in step.scheduled]
        lp_by_req = dict(zip(sample_reqs, lp)) if lp is not None else None
        result = StepResult(req_ids, [sampled.get(r) for r in req_ids],
                            [lp_by_req.get(r) for r in req_ids] if lp_by_req is not None else None,
                            prompt_logprobs=prompt_lp, pooled=pooled)
        if self.tp.pp_size > 1:
            result = broadcast_from_last_stage(result)       # every stage's scheduler sees the same result
        return result

    def _raise_on_device_status(self) -> None:
        """Called right after the step's device -> host synchronisation: a kernel that gave up on a bounded
        wait (a peer that never signalled, a tile flag that never came) has left un-reduced data behind, so
        the step's tokens must not be emitted. The word is sticky (kernels OR into it), so a failure in a
        step that sampled nothing is seen at the next step that does."""
        code = int(self._status_host[0])
        if code != 0:
            raise ops.KernelStatusError(code)

    def _prompt_logprobs(self, jobs: list[tuple[str, int, int, int]]) -> dict:
        """Log-probabilities of the prompt tokens computed in this step: the final-norm hidden rows of the
        step are still in the staging buffer; they go through the LM head in blocks of 512 rows (a block of
        fp32 logits over a 128k vocabulary is 256 MB), and only the chosen and top-k entries leave the device
        (vllm/v1/worker/gpu_model_runner.py ``_get_prompt_logprobs_dict``)."""
        hidden = self.model.rt.hidden
        out: dict[str, list] = {}
        for rid, row0, pos0, n in jobs:
            req = self.requests[rid]
            k = int(req.sampling_params.prompt_logprobs)
            targets = torch.as_tensor(req.token_ids[pos0 + 1: pos0 + 1 + n], dtype=torch.long, device=hidden.device)
            items = out.setdefault(rid, [])
            for b in range(0, n, 512):
                e = min(n, b + 512)
                lsm = torch.log_softmax(self.model.compute_logits(hidden[row0 + b: row0 + e]).float(), dim=-1)
                chosen = lsm.gather(1, targets[b:e, None]).squeeze(1).tolist()
                if k > 0:
                    top_v, top_i = lsm.topk(min(k, lsm.shape[1]), dim=-1)
                    top_v, top_i = top_v.tolist(), top_i.tolist()
                tg = targets[b:e].tolist()
                for j in range(e - b):
                    d = {int(tg[j]): float(chosen[j])}
                    if k > 0:
                        for t, v in zip(top_i[j], top_v[j]):
                            d.setdefault(int(t), float(v))
                    items.append((pos0 + b + j + 1, d))
        return out
