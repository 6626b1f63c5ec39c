"""Run a piece of a test in a fresh Python process.

Two kinds of test code never run inside the pytest process itself: anything that imports vLLM's
compiled extension (its static initialisers abort the interpreter when an op schema is already
defined, which no ``except`` can catch), and anything that defines or overrides ``torch.ops``
entries (registrations outlive the test and change what later tests call)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_PRELUDE = f"import sys; sys.path.insert(0, {ROOT!r})\n"


def run_isolated(code: str, timeout: int = 600) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, "-c", _PRELUDE + code], capture_output=True, text=True, timeout=timeout,
                          cwd=ROOT)


def check_isolated(code: str, timeout: int = 600) -> str:
    """Runs the snippet; the test fails with the child's output unless it exits 0."""
    r = run_isolated(code, timeout)
    assert r.returncode == 0, f"child exited {r.returncode}\n--- stdout\n{r.stdout[-4000:]}\n--- stderr\n{r.stderr[-4000:]}"
    return r.stdout


_vllm_state = {}


def require_vllm_ops(*op_names: str) -> None:
    """Skips the calling test unless vLLM's compiled ops import cleanly in a fresh process and
    define every op named (e.g. "_moe_C.topk_softmax").  Probed once per test session."""
    key = tuple(op_names)
    if key not in _vllm_state:
        probe = "import torch, vllm._custom_ops\n" + "".join(f"torch.ops.{n}\n" for n in op_names)
        try:
            r = run_isolated(probe, timeout=300)
            _vllm_state[key] = (r.returncode, (r.stderr or "")[-300:])
        except subprocess.TimeoutExpired:
            _vllm_state[key] = (-1, "timed out")
    rc, err = _vllm_state[key]
    if rc != 0:
        pytest.skip(f"vLLM's compiled ops do not load in a fresh process here (exit {rc}): {err.strip()[-200:]}")
