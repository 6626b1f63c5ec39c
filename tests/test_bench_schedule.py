"""The benchmark's step schedule must be the same on every rank: ranks that run different numbers
of steps issue different numbers of collectives and stop matching."""
import argparse
import importlib
import inspect
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _args(**kw):
    d = dict(warmup=3, steps=10, passes=5)
    d.update(kw)
    return argparse.Namespace(**d)


def test_schedule_depends_on_the_command_line_only(monkeypatch):
    bench = importlib.import_module("bench")
    base = bench.step_schedule(_args())
    for rank in ("0", "3", "7"):
        monkeypatch.setenv("RANK", rank)
        monkeypatch.setenv("LOCAL_RANK", rank)
        monkeypatch.setenv("WORLD_SIZE", "8")
        assert bench.step_schedule(_args()) == base
    src = inspect.getsource(bench.step_schedule)
    for forbidden in ("time.", "clocks", "rank", "environ", "random"):
        assert forbidden not in src.split('"""')[-1], f"step_schedule must not look at {forbidden}"
    timed = [n for phase, n in base if phase == "timed"]
    assert timed == [10] * 5
    assert bench.step_schedule(_args(warmup=0))[0] == ("warmup", 3)  # at least three warm-up steps


def test_run_loop_has_no_rank_local_step_condition():
    """The loop that executes the schedule contains no `while`: every step count comes from the
    schedule."""
    bench = importlib.import_module("bench")
    src = inspect.getsource(bench._run_ours)
    assert "while " not in src
    assert "for phase, n in step_schedule(args)" in src
