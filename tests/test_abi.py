"""The C-ABI library loads on a machine without a GPU and exports every declared symbol."""
import ctypes as C

import pytest

import __graft_entry__ as entry
from khalamari_b200 import abi


def test_every_declared_symbol_is_exported_and_bound():
    handle = abi.lib()
    declared = entry.declared_symbols()
    assert len(declared) >= 55
    for name in declared:
        assert hasattr(handle, name), name
    bound = set(abi.PROTOTYPES) | set(abi._SPECIAL)
    assert set(declared) == bound, set(declared) ^ bound


def test_version_and_error_message_plumbing():
    assert b"sm_100a" in abi.lib().kh_version()
    with pytest.raises(abi.InvalidArgument, match="config is null"):
        abi.call("kh_sdpa_config_validate", None)
    assert "config is null" in abi.last_error()


def test_struct_sizes_match_the_header():
    assert C.sizeof(abi.BufferRef) == 16
    assert C.sizeof(abi.SdpaConfig) == 20
    assert C.sizeof(abi.ExecutionVariantC) == 36
    assert C.sizeof(abi.PageTableLayoutC) == 16
    assert C.sizeof(abi.SlicedKvConfigC) == 44
    assert C.sizeof(abi.SlicedQConfigC) == 44
    assert C.sizeof(abi.MapTaskTemplateC) == 12
    assert C.sizeof(abi.SelectorLimitsC) == 16


def test_device_open_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    handle = C.c_void_p()
    with pytest.raises(abi.KhError) as info:
        abi.call("kh_device_open", 0, C.byref(handle))
    assert info.value.code == 7  # Unavailable: there is no CPU fallback


def test_page_table_index_formula():
    # (((slot * L) + layer) * B + block) * n  (request_page_table.rs:151-156)
    from khalamari_b200.request_page_table import GQAPageTableLayout
    layout = GQAPageTableLayout(4, 3, 6, 2)
    assert layout.bytes() == 4 * 3 * 6 * 2 * 4
    assert layout.start_index(1, 2, 5) == (((1 * 3) + 2) * 6 + 5) * 2
    with pytest.raises(abi.InvalidArgument, match="block out of range"):
        layout.start_index(1, 2, 6)
    with pytest.raises(abi.InvalidArgument):
        GQAPageTableLayout(0, 1, 1, 1).validate()
