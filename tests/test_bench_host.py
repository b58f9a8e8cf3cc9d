"""Host-side pieces of bench.py that need no GPU: the workload description, the rule that picks the captured
DRAM traffic of the instantiation a shard runs, the bounded CPU sample, and the whole reference arm
(`--impl reference`: the CPU oracle timed on the host's cores), run as the driver runs it."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from mamba_trainer_b200 import synthetic  # noqa: E402


def test_workload_description_names_the_workload_and_nothing_of_a_model():
    w = synthetic.WORKLOADS[4]
    cfg = bench.workload_config(w, 8, 4)
    assert cfg["workload"] == "cfg4_mimo2_scaling_bf16" and "model" not in cfg
    assert cfg["global_batch"] == 64 and cfg["seq_len"] == 16384 and cfg["rank"] == 2      # strong: the batch is not multiplied
    assert "8 shard(s)" in cfg["sharding"]
    assert bench.workload_config(synthetic.WORKLOADS[1], 4, 1)["global_batch"] == 4 * synthetic.WORKLOADS[1].batch


def test_traffic_follows_the_instantiation_the_shard_runs():
    """Stripes are cut in time when there are more of them than SMs but fewer than six per SM: the N = 4 and
    N = 8 shards of the scaling workload on 148 SMs, not the N = 1 and N = 2 ones."""
    w = synthetic.WORKLOADS[4]
    table = bench.NCU_TRAFFIC_BYTES_PER_TOKEN_HEAD[w.name]
    for batch, want in ((64, "whole"), (32, "whole"), (16, "split"), (8, "split"), (4, "whole")):
        assert bench.traffic_per_token_head(w.scaled(batch=batch), 148) == table[want], batch
    assert table["split"] > table["whole"] > w.bytes_per_token_head() * 0  # the hand-over adds traffic
    assert bench.traffic_per_token_head(synthetic.WORKLOADS[3], 148) is None   # no capture, no figure


def test_cpu_sample_is_bounded_and_says_what_it_is():
    w = synthetic.WORKLOADS[4]
    sw, note = bench.cpu_sample_shape(w)
    assert sw.batch * sw.seq * sw.heads <= 2 * 4096 * 16 and "flatters the CPU" in note
    whole, note1 = bench.cpu_sample_shape(synthetic.WORKLOADS[1])
    assert whole is synthetic.WORKLOADS[1] and note1 == "the whole workload"


def test_measured_peak_comes_from_the_drivers_file_when_it_is_there():
    peak, kind = bench.measured_peaks()
    if (ROOT / "MEASURED_PEAKS.json").exists():
        assert kind == "measured" and peak == float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"])
    else:
        assert (peak, kind) == (6650.0, "fallback")


def test_reference_arm_prints_one_line_with_the_contracts_keys():
    """`bench.py --impl reference` on the smallest bf16 workload (it runs whole on the CPU)."""
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--config", "1", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == bench.UNIT
    assert d["higher_is_better"] is True and d["value"] > 0 and d["vs_baseline"] is None
    assert d["config"]["workload"] == "cfg1_siso_trapezoid_bf16"
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "whole workload" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": bench.UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
