"""Replay capacity buckets: ``ReplayBucketPolicy`` (crates/inference-executor-core/src/replay.rs:4-88),
``GQAReplayBucketPolicy`` and ``GQAReplayShape``
(crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:11-96)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import abi


class ReplayBucketPolicy:
    def __init__(self, max_capacity: int):
        count = C.c_uint32()
        abi.call("kh_replay_buckets", max_capacity, None, 0, C.byref(count))
        arr = (C.c_uint32 * count.value)()
        abi.call("kh_replay_buckets", max_capacity, arr, count.value, C.byref(count))
        self._max = max_capacity
        self._buckets = list(arr)

    def max_capacity(self) -> int:
        return self._max

    def buckets(self) -> list[int]:
        return self._buckets

    def capacity(self, active: int) -> int:
        out = C.c_uint32()
        abi.call("kh_replay_capacity", self._max, active, C.byref(out))
        return out.value

    def capacity_allow_zero(self, active: int) -> int:
        return 0 if active == 0 else self.capacity(active)


class GQAReplayBucketPolicy:
    def __init__(self, max_tokens: int, max_map_task_templates: int):
        self.q_token_ranges = ReplayBucketPolicy(max_tokens)
        self.map_task_templates = ReplayBucketPolicy(max_map_task_templates)

    def max_tokens(self) -> int:
        return self.q_token_ranges.max_capacity()

    def max_map_task_templates(self) -> int:
        return self.map_task_templates.max_capacity()

    def capacity(self, num_active_q_token_ranges: int, num_active_map_task_templates: int) -> tuple[int, int]:
        return (self.q_token_ranges.capacity(num_active_q_token_ranges),
                self.map_task_templates.capacity(num_active_map_task_templates))


@dataclass(frozen=True)
class GQAReplayShape:
    num_tokens: int
    num_total_tokens: int
    num_q_token_tiles: int
    num_total_q_token_tiles: int
    num_sdpa_map_task_templates: int
    num_total_sdpa_map_task_templates: int
    reduce_sdpa_partial_outputs: bool

    @staticmethod
    def new(*args) -> "GQAReplayShape":
        shape = GQAReplayShape(*args)
        shape.validate()
        return shape

    @staticmethod
    def from_c(s: abi.ReplayShapeC) -> "GQAReplayShape":
        return GQAReplayShape(s.num_tokens, s.num_total_tokens, s.num_q_token_tiles, s.num_total_q_token_tiles,
                              s.num_sdpa_map_task_templates, s.num_total_sdpa_map_task_templates,
                              bool(s.reduce_sdpa_partial_outputs))

    def validate(self) -> None:
        ok = (self.num_tokens > 0 and self.num_tokens <= self.num_total_tokens
              and 0 < self.num_q_token_tiles <= self.num_tokens
              and self.num_q_token_tiles <= self.num_total_q_token_tiles
              and self.num_sdpa_map_task_templates >= self.num_q_token_tiles
              and self.num_sdpa_map_task_templates <= self.num_total_sdpa_map_task_templates)
        if not ok:
            raise abi.InvalidArgument(1, f"invalid GQA replay shape {self}")
