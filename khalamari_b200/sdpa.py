"""Backend SDPA capability registry: ``Config``, ``MapKernelKind``, ``ExecutionVariant``, ``Registry``
(crates/inference-backend-metal/src/components/gqa/sdpa.rs)."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

from . import abi
from .device import Dtype


class MapKernelKind(enum.IntEnum):
    SlicedKv = 0
    QTokensPerHead = 1
    QHeadsPerToken = 2
    QTokensAndHeads = 3


@dataclass(frozen=True)
class Config:
    """``sdpa::Config`` (sdpa.rs:219-241)."""

    io_dtype: Dtype
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    tokens_per_page: int

    def to_c(self) -> abi.SdpaConfig:
        return abi.SdpaConfig(int(self.io_dtype), self.num_q_heads, self.num_kv_heads, self.head_dim,
                              self.tokens_per_page)

    def validate(self) -> None:
        abi.call("kh_sdpa_config_validate", C.byref(self.to_c()))

    def q_heads_per_kv_head(self) -> int:
        return self.num_q_heads // self.num_kv_heads


@dataclass(frozen=True)
class MapThreadBlockConstants:
    max_q_tokens: int
    max_q_heads: int
    kv_tokens_per_iteration: int
    required_threads: int


@dataclass(frozen=True)
class ReduceThreadBlockConstants:
    max_q_tokens: int
    max_q_heads: int
    required_threads: int


@dataclass(frozen=True)
class ExecutionVariant:
    """``ExecutionVariant`` (sdpa.rs:49-57), flattened: ``kind`` and ``thread_block`` are ``map.*``."""

    kind: MapKernelKind
    thread_block: MapThreadBlockConstants
    tokens_per_page: int
    reduce: ReduceThreadBlockConstants

    @staticmethod
    def from_c(v: abi.ExecutionVariantC) -> "ExecutionVariant":
        return ExecutionVariant(
            MapKernelKind(v.kind),
            MapThreadBlockConstants(v.max_q_tokens, v.max_q_heads, v.kv_tokens_per_iteration, v.required_threads),
            v.tokens_per_page,
            ReduceThreadBlockConstants(v.reduce_max_q_tokens, v.reduce_max_q_heads, v.reduce_required_threads))

    def to_c(self) -> abi.ExecutionVariantC:
        tb, rd = self.thread_block, self.reduce
        return abi.ExecutionVariantC(int(self.kind), tb.max_q_tokens, tb.max_q_heads, tb.kv_tokens_per_iteration,
                                     tb.required_threads, self.tokens_per_page, rd.max_q_tokens, rd.max_q_heads,
                                     rd.required_threads)

    @staticmethod
    def sliced_kv(config: Config, kv_tokens_per_iteration: int, required_threads: int,
                  max_q_heads: int) -> "ExecutionVariant":
        out = abi.ExecutionVariantC()
        abi.call("kh_variant_sliced_kv", C.byref(config.to_c()), kv_tokens_per_iteration, required_threads,
                 max_q_heads, C.byref(out))
        return ExecutionVariant.from_c(out)

    @staticmethod
    def sliced_q(config: Config, kind: MapKernelKind, max_q_tokens: int, kv_tokens_per_iteration: int,
                 max_q_heads: int) -> "ExecutionVariant":
        out = abi.ExecutionVariantC()
        abi.call("kh_variant_sliced_q", C.byref(config.to_c()), int(kind), max_q_tokens, kv_tokens_per_iteration,
                 max_q_heads, C.byref(out))
        return ExecutionVariant.from_c(out)

    @staticmethod
    def sliced_q_per_head(config: Config, max_q_tokens: int, kv_tokens_per_iteration: int,
                          max_q_heads: int) -> "ExecutionVariant":
        return ExecutionVariant.sliced_q(config, MapKernelKind.QTokensPerHead, max_q_tokens,
                                         kv_tokens_per_iteration, max_q_heads)

    def supports(self, config: Config) -> bool:
        out = C.c_int32()
        abi.call("kh_variant_supports", C.byref(self.to_c()), C.byref(config.to_c()), C.byref(out))
        return bool(out.value)


class Registry:
    """``Registry`` (sdpa.rs:243-302): static capability filtering only."""

    def __init__(self, config: Config, variants: list[ExecutionVariant] | None = None):
        config.validate()
        self._config = config
        if variants is None:
            count = C.c_uint32()
            arr = (abi.ExecutionVariantC * 8)()
            abi.call("kh_registry_variants", C.byref(config.to_c()), arr, 8, C.byref(count))
            variants = [ExecutionVariant.from_c(arr[i]) for i in range(count.value)]
        else:
            if not variants:
                raise abi.InvalidArgument(1, "GQA SDPA registry requires an execution variant")
            if not all(v.supports(config) for v in variants):
                raise abi.InvalidArgument(1, "GQA SDPA registry contains an unsupported execution variant")
        self._variants = list(variants)

    @staticmethod
    def from_variants(config: Config, variants: list[ExecutionVariant]) -> "Registry":
        return Registry(config, variants)

    def config(self) -> Config:
        return self._config

    def variants(self) -> list[ExecutionVariant]:
        return self._variants

    def max_q_tokens_per_map_task(self) -> int:
        return max(v.thread_block.max_q_tokens for v in self._variants)
