"""Child process of test_gpu_guards.py: makes a bounded wait inside the map kernel run out, on the measurement
build of the library (``KH_GQA_LIBRARY=measure``), and prints one JSON line with what the host saw.

The switch (``KH_GQA_DEBUG`` bit 8192, honoured only by that build) makes the stream warp announce the bytes of a
task's first stage without issuing the copy. Nothing is in flight for that stage, so the consumers' wait can only
end by its poll limit; the limit is lowered to 4,096 polls for the one call. No fault, no trap, no endless loop:
the kernel returns by itself and the context stays usable, which the second half of the run checks."""
import json
import os
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for path in (ROOT, ROOT / "tests"):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))


def main(tile: str) -> None:
    assert os.environ.get("KH_GQA_LIBRARY") == "measure", "this worker runs on the measurement build only"
    from helpers import DeviceCase, assert_within_contract, make_case
    from khalamari_b200 import abi
    from khalamari_b200.device import Device

    device = Device(0)
    if tile == "decode":
        case = make_case(71, "bf16", 64, 8, 128, [900, 1500], [1, 1])
        run = DeviceCase(device, case)
    else:  # 16 tokens x 8 heads = 128-row tiles: the tcgen05 / tensor-memory instance
        case = make_case(72, "bf16", 16, 2, 128, [300, 40], [24, 19])
        run = DeviceCase(device, case, max_tokens=64)
    run.attention.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    report = {"tile": tile}
    os.environ["KH_GQA_DEBUG"] = "8192"
    device.set_wait_limit(4096)
    run.attention.record_sdpa(run.stream, run.q, run.kv_pages, run.page_ids, run.output, case.layer_index)
    os.environ.pop("KH_GQA_DEBUG")
    device.set_wait_limit(0)
    try:
        report["status_word"] = device.check(run.stream)
        report["aborted_code"] = 0
        report["message"] = ""
    except abi.KhError as error:
        report["aborted_code"] = error.code
        report["message"] = str(error)
        word = re.search(r"status word 0x([0-9a-fA-F]+)", str(error))
        report["status_word"] = int(word.group(1), 16) if word else 0
    report["clean_word_after"] = device.check(run.stream)
    out = run.run(fused=False)
    try:
        assert_within_contract(out, case.oracle_output(), "call after an aborted one")
        report["next_call_within_contract"] = True
    except AssertionError as error:
        report["next_call_within_contract"] = False
        report["next_call_error"] = str(error)
    print(json.dumps(report), flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "decode")
