"""Results must not depend on a kernel being launched for the first time in a process (cold
instruction caches, one-time set-up on the host, recycled device memory): a race that only a
slow first launch exposes shows up as a checksum that differs between fresh processes."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parents[1]


def test_fresh_processes_agree_bit_for_bit(cuda):
    lines = []
    for _ in range(4):
        proc = subprocess.run([sys.executable, str(REPO / "tests" / "cold_start_case.py")], cwd=REPO,
                              capture_output=True, text=True, timeout=300)
        assert proc.returncode == 0, proc.stderr[-2000:]
        lines.append(proc.stdout.strip().splitlines()[-1])
    assert len(set(lines)) == 1, lines
    assert lines[0].split()[-1].endswith("="), f"graph replay differs from the eager forward: {lines[0]}"
