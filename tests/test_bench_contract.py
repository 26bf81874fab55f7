"""The reference arm of ``bench.py`` runs on the CPU: its JSON line carries the keys the bench contract names."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [line for line in out.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "GQA decode KV-read GB/s" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["n_gpus"] == 1
    assert line["value"] > 0 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the same `config` object as the GPU arm prints, so that the two lines describe one configuration
    import bench
    spec = bench.WORKLOADS["c2"]
    assert line["config"] == bench.workload_config(spec, bench.contexts_for(spec, 0), 1)
    assert "requests" in line["cpu_baseline"]["sample"]


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}
    import os
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=120, cwd=ROOT,
                         env={**os.environ, **env})
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_several_gpus_share_the_job_by_longest_first_binning():
    """At N GPUs the bench bins the job's requests (64 per GPU) over the ranks with ``split_kv.assign_requests``:
    every request lands on exactly one rank and the ranks' byte loads differ by less than one request."""
    import bench
    spec = bench.WORKLOADS["c2"]
    for world in (2, 4, 8):
        shares = [bench.contexts_for(spec, rank, world) for rank in range(world)]
        job = sorted(ctx for rank in range(world) for ctx in bench.contexts_for(spec, rank))
        assert sorted(ctx for share in shares for ctx in share) == job
        loads = [sum(share) for share in shares]
        assert max(loads) - min(loads) <= spec["hi"]
    assert bench.contexts_for(spec, 0, 1) == bench.contexts_for(spec, 0)
