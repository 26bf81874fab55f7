"""Sharding of the attention path over the GPUs of one node. The reference runs on one device and has no
counterpart; what is reused from it is the reducer's partial-state merge
(docs/gqa_sdpa_selection.md:443-460), which is associative and therefore also merges partials of different GPUs.

Two shardings:

* many requests (decode, verify, mixed batches): requests are independent units. ``assign_requests`` bins them
  by context length; every rank owns the pages, block tables, Q rows and outputs of its requests and runs the
  single-GPU path. No collective.
* one very long sequence: ``split_context`` gives every rank a contiguous token range whose boundaries fall on
  page boundaries; the rank holds only those pages. Each rank runs the single-GPU split-KV map over its range and
  merges its own partials into one record per call (``record_floats`` f32: exp sums, max logits, normalised
  output); one all-gather brings the records of all ranks into local memory and every rank merges them
  (``kh_combine_packed_partials``). The collective moves ``world * record`` bytes (16.5 KB per rank at
  Hq16/D256) and no kernel reads another GPU's memory."""
from __future__ import annotations

import numpy as np

from . import abi
from .device import Buffer, Device, Dtype, Stream


# -- rank arithmetic (pure host logic) --------------------------------------------------------------------
def assign_requests(contexts, world: int) -> list:
    """Longest-first greedy binning of request indices by context length: the next longest request goes to the
    rank with the least total context so far (lowest rank on ties). Returns ``world`` lists of request indices,
    each in ascending order."""
    if world <= 0:
        raise abi.InvalidArgument(1, "world size must be positive")
    order = sorted(range(len(contexts)), key=lambda i: (-int(contexts[i]), i))
    load = [0] * world
    bins = [[] for _ in range(world)]
    for index in order:
        rank = min(range(world), key=lambda r: (load[r], r))
        bins[rank].append(index)
        load[rank] += int(contexts[index])
    return [sorted(b) for b in bins]


def split_context(context_len: int, world: int, tokens_per_page: int) -> list:
    """Token ranges ``[begin, end)`` of one sequence, one per rank, contiguous in token order, every boundary a
    multiple of the page size, pages divided as evenly as possible. A rank gets an empty range when the
    sequence has fewer pages than there are ranks."""
    if world <= 0 or tokens_per_page <= 0 or context_len < 0:
        raise abi.InvalidArgument(1, "split_context needs a positive world size and page size")
    pages = -(-context_len // tokens_per_page)
    ranges = []
    for rank in range(world):
        begin = min((rank * pages // world) * tokens_per_page, context_len)
        end = min(((rank + 1) * pages // world) * tokens_per_page, context_len)
        ranges.append((begin, end))
    return ranges


def record_floats(num_rows: int, head_dim: int) -> int:
    """f32 count of one rank's record: ``[exp sums: rows][max logits: rows][output: rows x head_dim]``."""
    return num_rows * (head_dim + 2)


def pack_record(exp_sums, max_logits, output) -> np.ndarray:
    output = np.asarray(output, dtype=np.float32)
    rows, _ = output.shape
    return np.concatenate([np.asarray(exp_sums, dtype=np.float32).reshape(rows),
                           np.asarray(max_logits, dtype=np.float32).reshape(rows), output.reshape(-1)])


def unpack_records(packed, num_records: int, num_rows: int, head_dim: int):
    """Returns (exp_sums [n, rows], max_logits [n, rows], outputs [n, rows, D]) views of gathered records."""
    records = np.asarray(packed, dtype=np.float32).reshape(num_records, record_floats(num_rows, head_dim))
    return (records[:, :num_rows], records[:, num_rows:2 * num_rows],
            records[:, 2 * num_rows:].reshape(num_records, num_rows, head_dim))


def empty_record(num_rows: int, head_dim: int) -> np.ndarray:
    """Record of a rank that holds no token of the sequence: weight zero in the merge."""
    return pack_record(np.zeros(num_rows, np.float32), np.full(num_rows, -np.inf, np.float32),
                       np.zeros((num_rows, head_dim), np.float32))


def gather_records(local_record, group=None):
    """All-gathers one record per rank (a 1-D f32 torch tensor, CPU for gloo or CUDA for NCCL) into a
    ``[world * record]`` tensor in local memory; rank order. With no process group the record is returned alone."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return local_record.clone()
    world = dist.get_world_size(group)
    gathered = torch.empty(world * local_record.numel(), dtype=local_record.dtype, device=local_record.device)
    dist.all_gather_into_tensor(gathered, local_record, group=group)
    return gathered


# -- exchange over peer memory ----------------------------------------------------------------------------
class PeerExchange:
    """One rank's end of the peer-memory exchange (``kh_peer_exchange_*``): an inbox every other rank of the node
    writes its merged rows into, and the mapped inboxes of the others. ``combine`` is ONE kernel launch: local
    merge of this rank's partials, rows stored into every inbox over NVLink, flags, a bounded wait for the other
    ranks' rows, final merge into ``output``. Every rank must call it the same number of times.

    ``connect`` exchanges the CUDA IPC handles of the inboxes through ``torch.distributed`` (host side, once)."""

    def __init__(self, device: Device, rank: int, world: int, num_rows: int, head_dim: int):
        import ctypes as C

        self.device, self.rank, self.world, self.rows, self.head_dim = device, rank, world, num_rows, head_dim
        size = C.c_uint64()
        abi.call("kh_peer_exchange_inbox_bytes", world, num_rows, head_dim, C.byref(size))
        self.inbox = Buffer.new_zeroed(device, size.value)
        self.handle = None
        self._imported = []

    def export_handle(self) -> bytes:
        import ctypes as C
        raw = (C.c_uint8 * 64)()
        abi.call("kh_ipc_export", self.device.handle, self.inbox.ref, raw)
        return bytes(raw)

    def attach(self, inbox_pointers) -> None:
        """``inbox_pointers[r]``: device address of rank r's inbox as this process sees it (own entry: the local
        buffer)."""
        import ctypes as C
        pointers = (C.c_void_p * self.world)(*[C.c_void_p(int(ptr)) for ptr in inbox_pointers])
        handle = C.c_void_p()
        abi.call("kh_peer_exchange_create", self.device.handle, self.rank, self.world, self.rows, self.head_dim, pointers,
                 C.byref(handle))
        self.handle = handle

    def connect(self, group=None) -> None:
        import ctypes as C

        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, self.export_handle(), group=group)
        pointers = []
        for r, raw in enumerate(handles):
            if r == self.rank:
                pointers.append(self.inbox.ref.ptr)
                continue
            mapped = C.c_void_p()
            abi.call("kh_ipc_import", self.device.handle, (C.c_uint8 * 64).from_buffer_copy(raw), C.byref(mapped))
            self._imported.append(mapped)
            pointers.append(mapped.value)
        self.attach(pointers)
        dist.barrier(group=group)  # every rank has mapped every inbox before the first kernel writes into one

    def combine(self, stream: Stream, num_partials: int, exp_sums: Buffer, max_logits: Buffer, partial_output: Buffer,
                out_dtype: Dtype, output: Buffer) -> None:
        null = abi.BufferRef()
        abi.call("kh_peer_exchange_combine", self.handle, stream.handle, num_partials,
                 exp_sums.ref if num_partials else null, max_logits.ref if num_partials else null,
                 partial_output.ref if num_partials else null, int(out_dtype), output.ref)

    def close(self) -> None:
        if self.handle:
            abi.call("kh_peer_exchange_destroy", self.handle)
            self.handle = None
        for mapped in self._imported:
            abi.call("kh_ipc_close", self.device.handle, mapped)
        self._imported = []


# -- one long sequence over several GPUs ----------------------------------------------------------------
class SplitKvDecode:
    """Decode attention of ONE sequence whose KV pages are split in token order over the ranks of ``group``.

    Every rank constructs it with its own page pool and block table holding only its token range (as local
    tokens ``0 .. local_len``), and the same Q row. ``record_step`` enqueues: local map, local merge into this
    rank's record, all-gather of the records, merge of the gathered records into ``output`` (every rank ends
    with the full result). All launches and the collective go to torch's current stream."""

    def __init__(self, device: Device, attention, world: int, group=None, peer_exchange: "PeerExchange | None" = None):
        """``peer_exchange``: when given, ``record_step`` is the local map plus ONE exchange-and-merge kernel over
        peer memory; otherwise local merge, NCCL all-gather of the records and a merge of the gathered records."""
        import torch

        self.peer_exchange = peer_exchange
        self.torch = torch
        self.device = device
        self.attention = attention
        self.world = world
        self.group = group
        core = attention.core
        self.rows = core.num_q_heads
        self.head_dim = core.head_dim
        floats = record_floats(self.rows, self.head_dim)
        self.local_record = torch.zeros(floats, dtype=torch.float32, device="cuda")
        self.gathered = torch.zeros(world * floats, dtype=torch.float32, device="cuda")
        base = self.local_record.data_ptr()
        self._sums = Buffer.wrap(device, base, self.rows * 4)
        self._maxes = Buffer.wrap(device, base + self.rows * 4, self.rows * 4)
        self._out = Buffer.wrap(device, base + 2 * self.rows * 4, self.rows * self.head_dim * 4)
        self._gathered = Buffer.wrap(device, self.gathered.data_ptr(), world * floats * 4)
        self._empty = torch.from_numpy(empty_record(self.rows, self.head_dim)).to("cuda")
        self.local_len = 0

    def prepare(self, req_slot: int, local_len: int, partition: int | None = None) -> None:
        """Plans the local map over ``local_len`` tokens (all visible to the one query token)."""
        self.local_len = int(local_len)
        if self.local_len == 0:
            return
        attention = self.attention
        token_indices, cu_tokens = [self.local_len - 1], [0, 1]
        selection = None
        if partition:
            variant = next(v for v in attention.selector.variants()
                           if v.kind == 0 and v.thread_block.max_q_tokens == 1)
            selection = attention.select_partitioned(variant, partition, False, token_indices, cu_tokens)
        attention.prepare([req_slot], token_indices, cu_tokens, selection=selection)
        if attention.metadata.direct_output():
            raise abi.InvalidArgument(1, "split-KV decode needs partial outputs; the selection is a direct one")

    def record_local(self, stream: Stream, q: Buffer, kv_pages: Buffer, page_ids: Buffer,
                     gqa_layer_index: int = 0) -> int:
        """Local map + local merge into this rank's record. Returns the kernels launched."""
        from . import sdpa, sliced_kv
        from .gqa import combine_partials

        if self.local_len == 0:
            self.local_record.copy_(self._empty, non_blocking=True)
            return 0
        attention = self.attention
        meta = attention.metadata
        shape = meta.replay_shape()
        execution = meta.variant()
        if execution.kind != sdpa.MapKernelKind.SlicedKv:
            raise abi.InvalidArgument(1, "split-KV decode runs the SlicedKv map")
        compute = attention._sliced_kv(shape, execution)
        compute.invoke_map(stream, sliced_kv.MapBuffers(
            q, kv_pages, meta.req_slots(), page_ids, meta.sdpa_map_task_templates(), attention.partial_exp_sums,
            attention.partial_max_logits, attention.partial_output), gqa_layer_index, shape.num_tokens,
            shape.num_sdpa_map_task_templates)
        combine_partials(self.device, stream, shape.num_sdpa_map_task_templates, self.rows, self.head_dim,
                         attention.partial_exp_sums, attention.partial_max_logits, attention.partial_output,
                         Dtype.Float32, self._out, self._sums, self._maxes)
        return 2

    def record_step(self, stream: Stream, q: Buffer, kv_pages: Buffer, page_ids: Buffer, output: Buffer,
                    gqa_layer_index: int = 0) -> int:
        import torch.distributed as dist

        if self.peer_exchange is not None:
            return self._record_step_over_peer_memory(stream, q, kv_pages, page_ids, output, gqa_layer_index)
        launches = self.record_local(stream, q, kv_pages, page_ids, gqa_layer_index)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.local_record, group=self.group)
        else:
            self.gathered.copy_(self.local_record, non_blocking=True)
        abi.call("kh_combine_packed_partials", self.device.handle, stream.handle, self.world, self.rows,
                 self.head_dim, self._gathered.ref, int(self.attention.io_dtype), output.ref)
        return launches + 1

    def _record_step_over_peer_memory(self, stream: Stream, q: Buffer, kv_pages: Buffer, page_ids: Buffer,
                                      output: Buffer, gqa_layer_index: int) -> int:
        from . import sdpa, sliced_kv

        attention = self.attention
        if self.local_len == 0:
            self.peer_exchange.combine(stream, 0, attention.partial_exp_sums, attention.partial_max_logits,
                                       attention.partial_output, attention.io_dtype, output)
            return 1
        meta = attention.metadata
        shape = meta.replay_shape()
        execution = meta.variant()
        if execution.kind != sdpa.MapKernelKind.SlicedKv:
            raise abi.InvalidArgument(1, "split-KV decode runs the SlicedKv map")
        compute = attention._sliced_kv(shape, execution)
        compute.invoke_map(stream, sliced_kv.MapBuffers(
            q, kv_pages, meta.req_slots(), page_ids, meta.sdpa_map_task_templates(), attention.partial_exp_sums,
            attention.partial_max_logits, attention.partial_output), gqa_layer_index, shape.num_tokens,
            shape.num_sdpa_map_task_templates)
        self.peer_exchange.combine(stream, shape.num_sdpa_map_task_templates, attention.partial_exp_sums,
                                   attention.partial_max_logits, attention.partial_output, attention.io_dtype, output)
        return 2
