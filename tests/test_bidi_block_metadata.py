"""Metadata of a BiDi-block proposal step (CPU): the reference's own goldens for ``build_metal_metadata``
(crates/inference-executor-metal/src/attn/bidi_block_gqa/metadata.rs:377-443), restated."""
import numpy as np
import pytest

from khalamari_b200 import abi
from khalamari_b200.bidi_block_sdpa import build_metadata

MAXU = 0xFFFFFFFF


def test_metadata_materializes_tiled_history_and_block_partials():
    # metadata.rs:378-402: two requests (slots 3, 7), block size 3, variant sliced_q_per_head(.., 8, 16, 2)
    # (8 Q tokens per range, 16 KV tokens per iteration), template capacity 8
    meta = build_metadata([3, 7], [11, 12, 13, 20, 21, 22], [0, 0, 0, 3, 3, 3], [11, 11, 11, 20, 20, 20], 3, 8, 16, 8)
    shape = meta.replay_shape
    assert shape.num_tokens == 6 and shape.num_q_token_tiles == 2
    assert shape.num_total_sdpa_map_task_templates == 8
    assert meta.visible_kv_token_ranges.tolist() == [0, 11, 0, 11, 0, 11, 3, 20, 3, 20, 3, 20]
    assert meta.q_token_ranges.tolist() == [0, 3, 3, 6]
    assert meta.cu_sdpa_partial_outputs.tolist() == [0, 2, 5]
    assert meta.req_slots.tolist() == [3, 3, 3, 7, 7, 7]
    templates = meta.sdpa_map_task_templates.reshape(-1, 3).tolist()
    # range 0: one history task then the block's slot; range 1: 17 history tokens = two iterations = two tasks
    assert templates[:5] == [[0, 0, 11], [MAXU] * 3, [1, 3, 19], [1, 19, 20], [MAXU] * 3]
    assert all(t == [MAXU] * 3 for t in templates[5:]) and len(templates) == 8


def test_long_history_is_partitioned_without_growing_static_scratch():
    # metadata.rs:404-421: one request, block of 6 at position 262,144, full history, capacity 16
    anchor = 262_144
    meta = build_metadata([1], list(range(anchor, anchor + 6)), [0] * 6, [anchor] * 6, 6, 8, 16, 16)
    block_task = int(meta.cu_sdpa_partial_outputs[1]) - 1
    history = meta.sdpa_map_task_templates.reshape(-1, 3)[:block_task]
    assert history[0][1] == 0 and history[-1][2] == anchor
    assert all(history[i][2] == history[i + 1][1] for i in range(len(history) - 1))
    assert meta.cu_sdpa_partial_outputs.tolist() == [0, 16]
    assert meta.replay_shape.num_total_sdpa_map_task_templates == 16


def test_q_tile_uses_history_union_and_preserves_per_query_masks():
    # metadata.rs:423-441: one request (slot 3), block of 3 at position 20, windows 0..20, 1..20, 2..20: the tasks
    # cover the union, the per-token visible ranges keep each token's own window
    meta = build_metadata([3], [20, 21, 22], [0, 1, 2], [20, 20, 20], 3, 8, 16, 8)
    assert meta.replay_shape.num_q_token_tiles == 1
    assert meta.visible_kv_token_ranges.tolist() == [0, 20, 1, 20, 2, 20]
    first = meta.sdpa_map_task_templates.reshape(-1, 3)[0]
    assert first[1] == 0 and first[2] <= 20


def test_later_ranges_win_ties_and_the_budget_is_respected():
    # allocate_history_kv_splits (metadata.rs:341-367): 3 ranges of 4 iterations each, capacity 8 -> 5 history
    # templates: one each, then the two spare ones go to the LAST ranges
    begins, ends = [0] * 6, [64] * 6
    meta = build_metadata([0, 1, 2], [64, 65] * 3, begins, ends, 2, 2, 16, 8)
    cu = meta.cu_sdpa_partial_outputs.tolist()
    assert [cu[i + 1] - cu[i] - 1 for i in range(3)] == [1, 2, 2]
    assert cu[-1] == 8


def test_builder_rejects_what_the_reference_asserts():
    with pytest.raises(abi.InvalidArgument, match="power of two"):
        build_metadata([0], [5, 6], [0, 0], [5, 5], 2, 8, 16, 6)
    with pytest.raises(abi.InvalidArgument, match="two TaskTemplates per Q-token range"):
        build_metadata([0, 1, 2], [5] * 3, [0] * 3, [5] * 3, 1, 8, 16, 4)
    with pytest.raises(abi.InvalidArgument, match="history range must not be empty"):
        build_metadata([0], [5, 6], [3, 3], [3, 3], 2, 8, 16, 8)
