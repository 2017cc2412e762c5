"""The ``jetspec`` import alias: reference import lines resolve to this framework, and the alias steps aside
when a real ``jetspec`` package is on the path."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code: str, extra_path=()):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, *extra_path]))
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT)


def test_reference_import_lines_resolve_here():
    code = (
        "from jetspec import LLM, SamplingParams, RandomTreeDrafter, load_draft_head, DraftHeadTreeDrafter\n"
        "from jetspec.inference_engine import JetSpecEngine, SamplingParams as SP2\n"
        "from jetspec.tree import get_algorithm, list_algorithms, build_ancestor_matrix, tree_accept\n"
        "from jetspec.draft_head_adapter import GraphedDraftHead, CompiledDraftHead\n"
        "import jetspec, jetspec_b200\n"
        "assert jetspec is jetspec_b200 and SP2 is SamplingParams\n"
        "assert JetSpecEngine.__module__.startswith('jetspec_b200') and 'accum_logp' in list_algorithms()\n"
        "print('ok', SamplingParams(0.0, 64).max_new_tokens)\n")
    r = _run(code)
    assert r.returncode == 0 and r.stdout.strip() == "ok 64", r.stdout + r.stderr


def test_alias_steps_aside_for_another_jetspec_package(tmp_path):
    pkg = tmp_path / "jetspec"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("WHO = 'the other package'\n")
    (pkg / "sub.py").write_text("X = 7\n")
    r = _run("import jetspec; from jetspec.sub import X; print(jetspec.WHO, X)", extra_path=[str(tmp_path)])
    assert r.returncode == 0 and r.stdout.strip() == "the other package 7", r.stdout + r.stderr
