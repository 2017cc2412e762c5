"""The example scripts run end to end on a machine without a GPU (tiny random-init models)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,expect", [
    ("simple_generate.py", "["),
    ("engine_generate.py", "batch == single: [True, True, True]"),
    ("nvfp4_generate.py", "lossless: True"),
    ("tree_generate.py", "tokens/round"),
])
def test_example_runs(script, expect):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script)], capture_output=True, text=True,
                       timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert expect in r.stdout
