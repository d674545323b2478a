"""Cutting one step's batch of tokens into the two subsets of the overlap schedule.

Counterpart of vllm/v1/worker/gpu_model_runner.py:618-680: requests are laid out back to back; subset 0
takes tokens ``[0, split)``, subset 1 the rest. A request that straddles the cut appears in both
subsets: its head in subset 0 with ``kv_len`` reduced by the tail length, its tail in subset 1 with the
full ``kv_len``. Causality across the cut holds because subset 0's keys are written to the paged cache
(same stream) before subset 1's attention reads them.
"""
from __future__ import annotations

from typing import Sequence


def split_batch(q_lens: Sequence[int], kv_lens: Sequence[int], split: int):
    """Returns (subset0, subset1); each is a list of ``(seq_index, q_len, kv_len)``."""
    first, second = [], []
    start = 0
    for b, (ql, kv) in enumerate(zip(q_lens, kv_lens)):
        end = start + ql
        if end <= split:
            first.append((b, ql, kv))
        elif start >= split:
            second.append((b, ql, kv))
        else:
            tail = end - split
            first.append((b, ql - tail, kv - tail))
            second.append((b, tail, kv))
        start = end
    return first, second
