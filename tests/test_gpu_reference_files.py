"""The reference project's own test files, unmodified, run against this library.

`python -m oracle.make_ref` stages tests/testing.py, tests/test_router.py, tests/test_expert.py and
tests/test_mlp.py of the reference under oracle/_ref/tests.  They import the three operators as
``omni_moe.ops.triton.triton_omni_*_func`` - which here resolves to this library's alias package - and
benchmark them beside their in-file PyTorch mirrors.  As shipped, their numerical check is optional and never
fails (tests/testing.py:249,290-297: a mismatch is printed); this runner switches it on for every forward test
and makes a mismatch fatal:

* where the file itself validates (router forward) the reference's own tolerance applies (bf16: 1e-3 / 1e-3);
* the other forward tests (expert, MLP) compare bf16 outputs with the bf16 PyTorch mirror at rtol 2e-2 and an
  absolute tolerance of 2e-2 of the output's scale (the mirror rounds to bf16 between its own steps, so the
  reference's 1e-3 is not reachable by any implementation there - which is why the file leaves it off);
* the backward tests run as they are (benchmarks without a check).
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TESTS = os.path.join(ROOT, "oracle", "_ref", "tests")

_RUNNER = r"""
import inspect, sys
ref_tests, root = sys.argv[1], sys.argv[2]
sys.path[:0] = [ref_tests, root]
import torch
import testing                      # the reference's harness, unmodified

failures = []
reference_check = testing._assert_allclose


def scale_check(out, ref, rtol=2e-2, atol_of_scale=2e-2):
    outs, refs = testing._flatten_tensors(out), testing._flatten_tensors(ref)
    assert len(outs) == len(refs), "output structure differs from the baseline"
    for o, r in zip(outs, refs):
        assert o.shape == r.shape and o.dtype == r.dtype, (o.shape, r.shape, o.dtype, r.dtype)
        o, r = o.float(), r.float()
        atol = atol_of_scale * float(r.abs().max())
        bad = (o - r).abs() > atol + rtol * r.abs()
        assert not bool(bad.any()), f"{int(bad.sum())}/{bad.numel()} elements outside rtol={rtol} atol={atol:.3g}"


mode = {"check": None}


def strict(out, ref, *, rtol, atol):
    try:
        if mode["check"] == "reference":
            reference_check(out, ref, rtol=rtol, atol=atol)
        else:
            scale_check(out, ref)
    except Exception as e:          # the harness swallows it and prints; remember it
        failures.append(str(e))
        raise


run_as_shipped = testing.run_benchmarks


def run_benchmarks(impls, factory, *, flops, config=None, validate=False):
    caller = inspect.stack()[1].function
    failures.clear()
    if validate:
        mode["check"] = "reference"
    elif "forward" in caller:
        mode["check"], validate = "scale", True
    results = run_as_shipped(impls, factory, flops=flops, config=config, validate=validate)
    if failures:
        raise AssertionError(f"{caller}: output differs from the PyTorch baseline: {failures[0]}")
    print(f"[strict] {caller}: validated={validate} ({mode['check']})")
    return results


testing._assert_allclose = strict
testing.run_benchmarks = run_benchmarks
import pytest
sys.exit(pytest.main(["-x", "-q", "-s", "-p", "no:cacheprovider"] + sys.argv[3:]))
"""


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF_TESTS, "testing.py")),
                    reason="oracle/_ref is empty: run `python -m oracle.make_ref` where the reference project is checked out")
@pytest.mark.parametrize("name", ["test_router.py", "test_expert.py", "test_mlp.py"])
def test_reference_test_file_runs_unmodified(name, tmp_path):
    runner = tmp_path / "run_reference_tests.py"
    runner.write_text(_RUNNER)
    r = subprocess.run([sys.executable, str(runner), REF_TESTS, ROOT, os.path.join(REF_TESTS, name)],
                       capture_output=True, text=True, timeout=1500, cwd=str(tmp_path))
    tail = r.stdout[-4000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "skipped" not in r.stdout.splitlines()[-1], tail
    assert "[strict]" in r.stdout and "validated=True" in r.stdout, tail
