"""The GQA component seam: ``GQA.prepare`` and ``GQA.record_sdpa``
(crates/inference-executor-metal/src/attn/gqa/backend.rs:255-286 and 438-542), limited to attention.

``GQAAttention`` owns what the reference's gated / ungated GQA layer owners own for this path: the SDPA
selector, the batch metadata buffers and the partial-state scratch
(crates/inference-executor-metal/src/attn/gqa/scratch.rs:49-83). The caller owns Q, the KV page pool, the
request page table and the output, as the executor does in the reference."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import abi, sdpa, sliced_kv, sliced_q
from .batch_metadata import GQAMetadataBuffers
from .device import Buffer, Device, Dtype, PinnedArray, Stream
from .replay import GQAReplayBucketPolicy, GQAReplayShape
from .request_page_table import GQAPageTableLayout
from .selector import RequestShape, Selection, Selector, SelectorPolicy


@dataclass(frozen=True)
class GQACore:
    """The fields of ``GQACore`` this path reads (crates/inference-executor-core/src/attn/gqa/core.rs:4-41)."""

    head_dim: int
    num_q_heads: int
    num_kv_heads: int
    scale: float

    def validate(self) -> None:
        if self.head_dim <= 0 or self.num_q_heads <= 0 or self.num_kv_heads <= 0:
            raise abi.InvalidArgument(1, "GQA core dimensions must be positive")
        if self.num_q_heads % self.num_kv_heads != 0:
            raise abi.InvalidArgument(1, "GQA Q heads must be a multiple of KV heads")
        if not self.scale > 0.0:
            raise abi.InvalidArgument(1, "GQA scale must be positive")


class GQAAttention:
    def __init__(self, device: Device, core: GQACore, io_dtype: Dtype, page_bytes: int,
                 page_table_layout: GQAPageTableLayout, max_tokens: int,
                 policy: SelectorPolicy = SelectorPolicy.B200, selector: Selector | None = None,
                 kv_dtype: Dtype | None = None):
        """``kv_dtype``: element type of the K/V pages; ``io_dtype`` (default) or ``Dtype.Fp8E4M3FN``, the
        reference's cache format (decoded on load, components/gqa/sdpa/sliced_kv.rs:118)."""
        core.validate()
        self.device = device
        self.core = core
        self.io_dtype = io_dtype
        self.kv_dtype = io_dtype if kv_dtype is None else kv_dtype
        self.page_bytes = page_bytes
        self.layout = page_table_layout
        elem = self.kv_dtype.item_size()
        self.tokens_per_page = page_bytes // (2 * core.num_kv_heads * core.head_dim * elem)
        self.sdpa_config = sdpa.Config(io_dtype, core.num_q_heads, core.num_kv_heads, core.head_dim,
                                       self.tokens_per_page)
        if selector is None:
            selector = Selector.for_lookup(self.sdpa_config, max_tokens, page_table_layout)
            selector.set_policy(policy, device.sm_count())
        self.selector = selector
        limits = selector.limits()
        self.limits = limits
        self.metadata = GQAMetadataBuffers(device, limits.max_tokens, limits.max_map_task_templates)
        self.policy = GQAReplayBucketPolicy(limits.max_tokens, limits.max_map_task_templates)
        states = limits.partial_state_group_capacity * core.num_q_heads
        self.partial_exp_sums = Buffer.new_zeroed(device, states * 4)
        self.partial_max_logits = Buffer.new_zeroed(device, states * 4)
        self.partial_output = Buffer.new_zeroed(device, states * core.head_dim * 4)
        # arrival counters of the fused map + reduce launch: one per (Q-token tile, KV head, Q-head range);
        # zero here, and every launch leaves them zero
        self.arrival_counters = Buffer.new_zeroed(device, max(limits.max_tokens, 1) * core.num_q_heads * 4)
        # False: map and reduce as two launches, the reference's form and the faster one on a saturated memory
        # system; True: one launch whose last-arriving CTA of a partial range merges it
        self.fused = False
        self._computes = {}
        self.selection: Selection | None = None

    # -- GQA::prepare (backend.rs:255-286) ---------------------------------------------------------
    def prepare(self, req_slots, token_indices, cu_tokens, num_total_tokens: int | None = None,
                stream: Stream | None = None, selection: Selection | None = None) -> GQAReplayShape:
        num_tokens = int(cu_tokens[-1]) if len(cu_tokens) else 0
        if num_tokens <= 0:
            raise abi.InvalidArgument(1, "GQA replay requires active tokens")
        # the page table's shape is known here: a slot or a context beyond it must not reach the kernels
        capacity = self.layout.num_blocks * self.layout.num_page_ids_per_block * self.tokens_per_page
        for r, slot in enumerate(req_slots):
            if not 0 <= int(slot) < self.layout.num_req_slots:
                raise abi.InvalidArgument(1, f"GQA request slot {int(slot)} out of range: num_req_slots="
                                             f"{self.layout.num_req_slots}")
            context = int(token_indices[r]) + int(cu_tokens[r + 1]) - int(cu_tokens[r])
            if context > capacity:
                raise abi.InvalidArgument(1, f"GQA request context of {context} tokens exceeds the page table's "
                                             f"{capacity} tokens per request")
        if num_total_tokens is None:
            # the executor records token capacities in replay buckets; a Q-tile capacity (bucketed by the selector)
            # can never exceed it
            num_total_tokens = self.policy.q_token_ranges.capacity(num_tokens)
        if selection is None:
            shapes = RequestShape.from_batch(list(token_indices), list(cu_tokens))
            selection = self.selector.select(shapes, self.policy, num_total_tokens)
        self.selection = selection
        return self.metadata.update(req_slots, token_indices, cu_tokens, selection, stream)

    def select_partitioned(self, variant, kv_slice, direct_output, token_indices, cu_tokens,
                           num_total_tokens=None) -> Selection:
        shapes = RequestShape.from_batch(list(token_indices), list(cu_tokens))
        total = self.policy.q_token_ranges.capacity(int(cu_tokens[-1])) if num_total_tokens is None else num_total_tokens
        return self.selector.select_partitioned(variant, kv_slice, direct_output, shapes, self.policy, total)

    def _sliced_kv(self, shape: GQAReplayShape, execution):
        key = ("kv", execution, shape.num_total_tokens, shape.num_total_sdpa_map_task_templates)
        if key not in self._computes:
            config = sliced_kv.Config(self.core.num_q_heads, self.core.num_kv_heads, self.core.head_dim,
                                      self.core.scale, self.page_bytes, self.layout, self.io_dtype, self.kv_dtype)
            self._computes[key] = sliced_kv.Compute(
                self.device, config, execution,
                sliced_kv.Shape(shape.num_total_tokens, shape.num_total_sdpa_map_task_templates))
        return self._computes[key]

    def _sliced_q(self, shape: GQAReplayShape, execution, direct: bool):
        key = ("q", execution, direct, shape.num_total_tokens, shape.num_total_q_token_tiles,
               shape.num_total_sdpa_map_task_templates)
        if key not in self._computes:
            config = sliced_q.Config(self.core.num_q_heads, self.core.num_kv_heads, self.core.head_dim,
                                     self.core.scale, self.page_bytes, self.io_dtype, self.layout, self.kv_dtype)
            self._computes[key] = sliced_q.Compute(
                self.device, config, execution,
                sliced_q.Shape(shape.num_total_tokens, shape.num_total_q_token_tiles,
                               shape.num_total_sdpa_map_task_templates), direct)
        return self._computes[key]

    # -- GQA::record_sdpa (backend.rs:438-542) -----------------------------------------------------
    def record_replay(self, stream: Stream, q: Buffer, kv_pages: Buffer, page_ids: Buffer, output: Buffer,
                      gqa_layer_index: int = 0) -> int:
        """``record_sdpa`` in the form a replay program records it (EM/replay.rs:21-74): grids sized by the
        recorded capacities (``num_total_*``), active counts read on the device from the metadata's count words.
        Capture this call into a CUDA graph; ``prepare`` on the same stream then retargets every later launch of
        the graph, as long as the batch stays in the same replay bucket (same ``GQAReplayShape`` totals)."""
        stream.bind_active_counts(self.metadata.active_counts())
        try:
            return self.record_sdpa(stream, q, kv_pages, page_ids, output, gqa_layer_index, capacities=True)
        finally:
            stream.bind_active_counts(None)

    def record_sdpa(self, stream: Stream, q: Buffer, kv_pages: Buffer, page_ids: Buffer, output: Buffer,
                    gqa_layer_index: int = 0, after_map=None, capacities: bool = False) -> int:
        """Enqueues the selected branch on ``stream`` and returns how many kernels it launched. ``after_map``,
        when given, is called between the map and the reduce launch (a timing hook: record an event there)."""
        meta = self.metadata
        shape = meta.replay_shape()
        if capacities:
            shape = GQAReplayShape(shape.num_total_tokens, shape.num_total_tokens, shape.num_total_q_token_tiles,
                                   shape.num_total_q_token_tiles, shape.num_total_sdpa_map_task_templates,
                                   shape.num_total_sdpa_map_task_templates, shape.reduce_sdpa_partial_outputs)
        execution = meta.variant()
        if execution.kind == sdpa.MapKernelKind.SlicedKv:
            compute = self._sliced_kv(shape, execution)
            map_buffers = sliced_kv.MapBuffers(
                q, kv_pages, meta.req_slots(), page_ids, meta.sdpa_map_task_templates(), self.partial_exp_sums,
                self.partial_max_logits, self.partial_output)
            reduce_buffers = sliced_kv.ReduceBuffers(
                self.partial_exp_sums, self.partial_max_logits, self.partial_output, meta.cu_sdpa_partial_outputs(),
                output)
            if self.fused:
                compute.invoke_map_reduce(stream, map_buffers, reduce_buffers, self.arrival_counters, gqa_layer_index,
                                          shape.num_tokens, shape.num_sdpa_map_task_templates)
                return 1
            compute.invoke_map(stream, map_buffers, gqa_layer_index, shape.num_tokens,
                               shape.num_sdpa_map_task_templates)
            if after_map is not None:
                after_map()
            compute.invoke_reduce(stream, reduce_buffers, shape.num_tokens)
            return 2
        if meta.direct_output():
            compute = self._sliced_q(shape, execution, True)
            compute.invoke_direct(stream, sliced_q.DirectBuffers(
                q, kv_pages, meta.req_slots(), page_ids, meta.visible_kv_token_ranges(), meta.q_token_ranges(),
                meta.sdpa_map_task_templates(), output), gqa_layer_index, shape.num_tokens, shape.num_q_token_tiles)
            return 1
        compute = self._sliced_q(shape, execution, False)
        map_buffers = sliced_q.MapBuffers(
            q, kv_pages, meta.req_slots(), page_ids, meta.visible_kv_token_ranges(), meta.q_token_ranges(),
            meta.sdpa_map_task_templates(), self.partial_output, self.partial_exp_sums, self.partial_max_logits)
        reduce_buffers = sliced_q.ReduceBuffers(
            self.partial_output, self.partial_exp_sums, self.partial_max_logits, meta.q_token_ranges(),
            meta.cu_sdpa_partial_outputs(), output)
        if self.fused:
            compute.invoke_map_reduce(stream, map_buffers, reduce_buffers, self.arrival_counters, gqa_layer_index,
                                      shape.num_tokens, shape.num_q_token_tiles, shape.num_sdpa_map_task_templates)
            return 1
        compute.invoke_map(stream, map_buffers, gqa_layer_index, shape.num_tokens, shape.num_q_token_tiles,
                           shape.num_sdpa_map_task_templates)
        if after_map is not None:
            after_map()
        compute.invoke_reduce(stream, reduce_buffers, shape.num_q_token_tiles)
        return 2

    # -- end-to-end call with host buffers -----------------------------------------------------------
    def attend_host(self, stream: Stream, q_host: PinnedArray, out_host: PinnedArray, q_dev: Buffer, out_dev: Buffer,
                    kv_pages: Buffer, page_ids: Buffer, req_slots, token_indices, cu_tokens,
                    gqa_layer_index: int = 0, selection: Selection | None = None) -> tuple[int, int, int]:
        """One attention call the way a host-side caller issues it: plan the batch, copy this step's Q and
        metadata to the device, run attention over the resident KV pages, and copy the output back. Returns
        (kernel launches, host->device bytes, device->host bytes). The caller synchronises ``stream``."""
        num_tokens = int(cu_tokens[-1])
        row = self.core.num_q_heads * self.core.head_dim * self.io_dtype.item_size()
        stream.write(q_dev, 0, q_host.ptr, num_tokens * row)  # first: the copy runs while the host plans the batch
        self.prepare(req_slots, token_indices, cu_tokens, num_tokens, stream, selection)
        launches = self.record_sdpa(stream, q_dev, kv_pages, page_ids, out_dev, gqa_layer_index)
        stream.read(out_dev, 0, out_host.ptr, num_tokens * row)
        return launches, num_tokens * row + self.metadata.upload_bytes(), num_tokens * row


class HostPipeline:
    """Attention calls with host buffers, two steps in flight.

    A step is what a host-side caller issues per batch: copy Q from page-locked host memory, plan the batch
    (selector + metadata, on the host, while the copy runs), run map + reduce over the resident KV pages, copy
    the output back. ``submit`` enqueues one step and returns without waiting; the Q copy of a step and the output
    copy of the step before run on two copy streams while kernels run on the compute stream (``ReplaySubmission``
    handles in the
    reference, metal/stream/submission.rs:41-101: a caller may hold several submissions and wait for each). Two
    slots of device Q / output buffers and batch metadata alternate; ``submit`` first waits for the step that used
    the slot two submissions ago, so at most two steps are in flight. ``wait(ticket)`` blocks until that step's
    output is in its host buffer."""

    SLOTS = 2

    def __init__(self, attention: GQAAttention, compute_stream: Stream):
        from .device import Event

        self.attention = attention
        self.compute = compute_stream
        self.copy = Stream(attention.device)      # device -> host: outputs
        self.copy_in = Stream(attention.device)   # host -> device: Q rows of the next step, beside this step's kernels
        core = attention.core
        limits = attention.limits
        row = core.num_q_heads * core.head_dim * attention.io_dtype.item_size()
        capacity = attention.policy.q_token_ranges.capacity(limits.max_tokens)
        self.row_bytes = row
        self.q = [Buffer.new_zeroed(attention.device, capacity * row) for _ in range(self.SLOTS)]
        self.out = [Buffer.new_zeroed(attention.device, capacity * row) for _ in range(self.SLOTS)]
        self.metadata = [attention.metadata] + [
            GQAMetadataBuffers(attention.device, limits.max_tokens, limits.max_map_task_templates)
            for _ in range(self.SLOTS - 1)]
        self.q_ready = [Event(attention.device) for _ in range(self.SLOTS)]
        self.kernels_done = [Event(attention.device) for _ in range(self.SLOTS)]
        self.copied = [Event(attention.device) for _ in range(self.SLOTS)]
        self.in_flight = [False] * self.SLOTS
        self.submitted = 0
        self._decode_variant = None

    def submit(self, q_host: PinnedArray, out_host: PinnedArray, kv_pages: Buffer, page_ids: Buffer, req_slots,
               token_indices, cu_tokens, gqa_layer_index: int = 0, partition: int | None = None):
        """Enqueues one step. ``partition``: force split-KV slices of that many tokens (the selector still runs,
        through ``select_partitioned``); None lets the selector choose. Returns (ticket, kernel launches,
        host->device bytes, device->host bytes). ``q_host`` may be reused once ``submit`` returns the ticket of
        the step after next; ``out_host`` is valid after ``wait(ticket)``."""
        attention = self.attention
        slot = self.submitted % self.SLOTS
        if self.in_flight[slot]:
            self.copied[slot].synchronize()  # the slot's buffers and its metadata host block are free again
        num_tokens = int(cu_tokens[-1])
        nbytes = num_tokens * self.row_bytes
        self.copy_in.write(self.q[slot], 0, q_host.ptr, nbytes)  # runs while the host plans the batch
        attention.metadata = self.metadata[slot]
        selection = None
        if partition:
            if self._decode_variant is None:  # (the registry does not change: looked up once)
                self._decode_variant = next(v for v in attention.selector.variants()
                                            if v.kind == 0 and v.thread_block.max_q_tokens == 1)
            selection = attention.select_partitioned(self._decode_variant, partition, False, token_indices, cu_tokens,
                                                     num_tokens)
        # the metadata block follows the Q rows on the copy stream: the compute stream carries kernels only, so the
        # kernels of consecutive steps run back to back
        attention.prepare(req_slots, token_indices, cu_tokens, num_tokens, self.copy_in, selection)
        self.copy_in.record_event(self.q_ready[slot])
        self.compute.wait_event(self.q_ready[slot])
        launches = attention.record_sdpa(self.compute, self.q[slot], kv_pages, page_ids, self.out[slot],
                                         gqa_layer_index)
        self.compute.record_event(self.kernels_done[slot])
        self.copy.wait_event(self.kernels_done[slot])
        self.copy.read(self.out[slot], 0, out_host.ptr, nbytes)
        self.copy.record_event(self.copied[slot])
        # the next user of this slot's device buffers is two steps away and ordered by `copied` on the host
        self.in_flight[slot] = True
        ticket = self.submitted
        self.submitted += 1
        return ticket, launches, nbytes + attention.metadata.upload_bytes(), nbytes

    def wait(self, ticket: int) -> None:
        if ticket < self.submitted - self.SLOTS:
            return  # its slot has been reused, which waited for it
        self.copied[ticket % self.SLOTS].synchronize()

    def drain(self) -> None:
        for slot in range(self.SLOTS):
            if self.in_flight[slot]:
                self.copied[slot].synchronize()
                self.in_flight[slot] = False


class MixedBatchAttention:
    """A batch that mixes decode requests (one new token) with prefill / verify requests (several), as one call.

    The reference selects ONE execution variant per batch (``Selector::select``, attn/gqa/sdpa.rs:278-380): in a
    mixed batch the decode rows then ride the wide Q tiles chosen for the prefill rows (128-row tensor-memory tiles
    with 8 valid rows). Here the two kinds are recorded back to back on the same stream as two selections - the
    decode requests through the SlicedKv map + reduce, the others through the sliced-Q kernels - each writing its
    own rows of the one output buffer: two kernels (pairs) in one recorded sequence rather than two task kinds in
    one grid, because the tensor-memory kernel and the warp-level decode kernel want different block shapes,
    register budgets and shared-memory layouts. The split needs the decode requests to form one contiguous run at
    the start or the end of the batch (their Q rows and output rows are then one slice of the buffers); any other
    order falls back to the reference's single selection."""

    def __init__(self, device: Device, core: GQACore, io_dtype: Dtype, page_bytes: int,
                 page_table_layout: GQAPageTableLayout, max_tokens: int, max_decode_tokens: int | None = None,
                 policy: SelectorPolicy = SelectorPolicy.B200, kv_dtype: Dtype | None = None):
        self.device = device
        self._args = (core, io_dtype, page_bytes, page_table_layout)
        self._policy = policy
        self._kv_dtype = kv_dtype
        self.max_tokens = max_tokens
        self.max_decode_tokens = max_decode_tokens or min(max_tokens, 256)
        self.core = core
        self.io_dtype = io_dtype
        self._parts = {}
        self.plan = None  # list of (attention, first flat token, token count)

    def _part(self, name: str, max_tokens: int) -> GQAAttention:
        if name not in self._parts:
            core, io_dtype, page_bytes, layout = self._args
            self._parts[name] = GQAAttention(self.device, core, io_dtype, page_bytes, layout, max_tokens, self._policy,
                                             kv_dtype=self._kv_dtype)
        return self._parts[name]

    def prepare(self, req_slots, token_indices, cu_tokens, stream: Stream | None = None) -> None:
        n = len(req_slots)
        q_lens = [int(cu_tokens[r + 1]) - int(cu_tokens[r]) for r in range(n)]
        decode = [r for r in range(n) if q_lens[r] == 1]
        split = None
        if decode and len(decode) < n and len(decode) <= self.max_decode_tokens:
            if decode == list(range(n - len(decode), n)):
                split = n - len(decode)          # the others first, then the decode run
                parts = [("wide", 0, split), ("decode", split, n)]
            elif decode == list(range(len(decode))):
                split = len(decode)
                parts = [("decode", 0, split), ("wide", split, n)]
        if split is None:
            whole = self._part("whole", self.max_tokens)
            whole.prepare(req_slots, token_indices, cu_tokens, int(cu_tokens[-1]), stream)
            self.plan = [(whole, 0, int(cu_tokens[-1]))]
            return
        self.plan = []
        for name, begin, end in parts:
            part = self._part(name, self.max_decode_tokens if name == "decode" else self.max_tokens)
            first = int(cu_tokens[begin])
            # token capacity = the part's own token count: its Q and output rows are a slice of the caller's buffers
            part.prepare(list(req_slots[begin:end]), list(token_indices[begin:end]),
                         [int(c) - first for c in cu_tokens[begin:end + 1]], int(cu_tokens[end]) - first, stream)
            self.plan.append((part, first, int(cu_tokens[end]) - first))

    def record_sdpa(self, stream: Stream, q: Buffer, kv_pages: Buffer, page_ids: Buffer, output: Buffer,
                    gqa_layer_index: int = 0, between=None) -> int:
        """Enqueues every part of the plan on ``stream``; returns the kernels launched. ``between`` (a timing hook)
        is called after each part."""
        row = self.core.num_q_heads * self.core.head_dim * self.io_dtype.item_size()
        launches = 0
        for part, first, count in self.plan:
            q_view = Buffer.wrap(self.device, q.ref.ptr + first * row, count * row)
            out_view = Buffer.wrap(self.device, output.ref.ptr + first * row, count * row)
            launches += part.record_sdpa(stream, q_view, kv_pages, page_ids, out_view, gqa_layer_index)
            if between is not None:
                between()
        return launches


def combine_partials(device: Device, stream: Stream, num_partials: int, num_rows: int, head_dim: int,
                     exp_sums: Buffer, max_logits: Buffer, partial_output: Buffer, out_dtype: Dtype, output: Buffer,
                     out_exp_sums: Buffer | None = None, out_max_logits: Buffer | None = None) -> None:
    """LSE merge of ``num_partials`` triples per row (``kh_combine_partials``): the reducer's formula
    (docs/gqa_sdpa_selection.md:443-460) applied to partials that may come from other GPUs."""
    null = abi.BufferRef()
    abi.call("kh_combine_partials", device.handle, stream.handle, num_partials, num_rows, head_dim, exp_sums.ref,
             max_logits.ref, partial_output.ref, int(out_dtype), output.ref,
             out_exp_sums.ref if out_exp_sums else null, out_max_logits.ref if out_max_logits else null)
