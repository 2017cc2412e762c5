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


def test_ar_decode_baseline_script_runs_on_cpu():
    """The stand-alone autoregressive baseline (engine and reference-engine arms) on a small model."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench", "ar_decode_baseline.py"), "--model", "small",
                        "--prompt-len", "12", "--new", "6"], capture_output=True, text=True, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout[r.stdout.index("{"):])
    for arm in ("engine", "llm"):
        assert out[arm]["output_tokens"] == 6 and out[arm]["decode_tokens_per_s"] > 0
