"""Runs the unmodified reference package on the benchmark configuration.

Filled in by :func:`run_reference`; prints the same JSON line as ``bench.py`` with
``"impl": "reference"``, or ``{"impl": "reference", "unavailable": "<why>"}``.
"""
import json


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}))
