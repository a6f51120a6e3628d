"""bench.py's arithmetic and its CPU (reference) arm, without a GPU."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_algorithmic_bytes_match_the_checkpoint_layout():
    sys.path.insert(0, str(ROOT))
    import bench

    # packed weight + packed zeros + fp16 scales + g_idx + x + y, M = 1
    assert bench.algorithmic_bytes(4096, 14336) == 29_360_128 + 229_376 + 917_504 + 16_384 + 8_192 + 28_672 == 30_560_256
    assert bench.algorithmic_bytes(14336, 4096) == 30_601_216
    assert bench.STEP_BYTES == 32 * (2 * 30_560_256 + 30_601_216) == 2_935_095_296


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "w4a16_m1_gemv_hbm_gbs" and line["unit"] == "GB/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
