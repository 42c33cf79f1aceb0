"""The checked build (-DB200MOE_DEBUG) on a GPU: range checks record a bad index and skip the access."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_checked_build_records_and_skips_bad_index():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    env = {**os.environ, "B200MOE_DEBUG": "1"}
    subprocess.run([sys.executable, "-m", "b200moe.build"], check=True, cwd=ROOT, env=env)
    done = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_debug_worker.py")], cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "checked build ok" in done.stdout
