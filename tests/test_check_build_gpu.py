"""The checking build of the kernels (-DTL_CHECK=1, TENSORLINE_B200_CHECK=1) in place of a memory checker: every
kernel that indexes block tables or pages checks slot, page index and page number against the bounds its launcher
states, records a violation and sends the access to the sink page.  Here the replay schedules and the kernel tests
run once under that build and must report nothing, and the checker itself is shown to catch entries outside its
bounds (tests/check_build_cases.py).  Each runs in a process of its own: the switch is read at import."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def run(args, timeout=1500):
    env = dict(os.environ, TENSORLINE_B200_CHECK="1", PYTHONPATH=str(ROOT))
    return subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_checker_catches_entries_outside_its_bounds_and_redirects_them():
    proc = run(["tests/check_build_cases.py"])
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    lines = proc.stdout.splitlines()
    assert lines[-1] == "ok" and sum(l.startswith("caught:") for l in lines) == 8, proc.stdout


def test_replay_schedules_and_kernel_tests_report_nothing_under_the_checking_build():
    proc = run(["-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
                "tests/test_replay_gpu.py", "tests/test_kernels_gpu.py", "tests/test_parts_gpu.py"])
    tail = proc.stdout[-3000:] + proc.stderr[-2000:]
    assert proc.returncode == 0, tail
    assert " passed" in proc.stdout and "failed" not in proc.stdout.splitlines()[-1], tail
