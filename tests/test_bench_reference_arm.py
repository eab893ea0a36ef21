"""`bench.py --impl reference` is CPU-only code (the reference's own PSO step on the host cores when
oracle/build_ref.py has installed it under oracle/_ref, else the oracle's restatement): run it on the
small workload and check the JSON contract of the line it prints."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    res = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "pso_ackley_1e4x500", "--steps", "1", "--warmup", "1"],
        capture_output=True, text=True, timeout=600, cwd=ROOT,
    )
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "pso_generations_per_s" and line["unit"] == "gens/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["gpu_launches"] == 0
    installed = (ROOT / "oracle" / "_ref" / "evox" / "__init__.py").exists()
    assert line["cpu_baseline"]["kind"] == ("reference" if installed else "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["n_gpus"] == 0 and line["reference_class"] == "cpu"
    assert line["e2e"] == {"value": line["value"], "unit": "gens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"] == "pso_ackley_1e4x500"
