"""The overlapped exchange of the column-sharded GEMM on two GPUs: every rank multiplies its column block and pushes
finished row blocks into the other rank's copy of the full product (symmetric memory, dtn_push_block) while it
multiplies the rest. The full product on every rank must equal, bit for bit, the one assembled by an all-gather of the
separately computed blocks. Runs `bench.py --gpus 2 --all-gather` (one process per GPU, NCCL) and reads its line;
skipped on a box with one GPU."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_gathered_product_equals_gemm_plus_all_gather(cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    done = subprocess.run([sys.executable, str(ROOT / 'bench.py'), '--gpus', '2', '--all-gather', '--steps', '3'], env=env,
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line['n_gpus'] == 2 and line['overlapped_failure'] is None, line
    assert line['overlapped_result_identical'] is True
    assert line['overlapped_ms'] < line['gemm_then_all_gather_ms']
