"""Runs the C++ front-end programs built by tests/cpp/build.py.

own_*  programs come from tests/cpp/*.cpp; ref_* programs are the reference project's own sample
and unit-test sources compiled unchanged against include/fusilli*.h (they can only be built where
the reference checkout is present, and travel as built programs).
"""
import importlib.util
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("cpp_build", os.path.join(HERE, "cpp", "build.py"))
cpp_build = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(cpp_build)

OWN, REF_DEVICE, REF_HOST = cpp_build.expected_programs()  # OWN also holds host_execute_latency (no test cases)


def _run(name, tmp_path, required):
    exe = os.path.join(cpp_build.OUT, name)
    if not os.path.exists(exe):
        if required:
            cpp_build.build(only=name)
        else:
            pytest.skip("not built: the reference checkout was not present at build time")
    env = dict(os.environ, FUSILLI_CACHE_DIR=str(tmp_path))
    p = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, "%s failed\n%s\n%s" % (name, p.stdout[-3000:], p.stderr[-3000:])
    assert " 0 failure(s)" in p.stdout


def test_own_host_program(tmp_path):
    _run("own_test_frontend_host", tmp_path, required=True)


@pytest.mark.parametrize("name", REF_HOST)
def test_reference_host_tests(name, tmp_path):
    _run(name, tmp_path, required=False)


@pytest.mark.gpu
def test_host_cost_of_execute_with_and_without_the_launch_cache(tmp_path):
    """std::chrono around 1000 back-to-back executes of a 1x1 convolution plan; the cached run must
    not be slower on the host than the run that re-encodes its tensor maps on every call."""
    import json
    exe = os.path.join(cpp_build.OUT, "own_host_execute_latency")
    if not os.path.exists(exe):
        cpp_build.build(only="own_host_execute_latency")
    res = {}
    for cache in ("1", "0"):
        env = dict(os.environ, FUSILLI_CACHE_DIR=str(tmp_path))
        if cache == "0":
            env["FUSILLI_B200_NO_LAUNCH_CACHE"] = "1"
        p = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
        assert p.returncode == 0, p.stdout + p.stderr
        res[cache] = json.loads(p.stdout.strip().splitlines()[-1])
    print("host us per execute:", res)
    assert res["1"]["launch_cache"] is True and res["0"]["launch_cache"] is False
    assert res["1"]["host_us_per_execute"] <= res["0"]["host_us_per_execute"] * 1.25


@pytest.mark.gpu
def test_own_device_program(tmp_path):
    _run("own_test_frontend_device", tmp_path, required=True)


@pytest.mark.gpu
@pytest.mark.parametrize("name", REF_DEVICE)
def test_reference_samples(name, tmp_path):
    _run(name, tmp_path, required=False)
