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

OWN, REF_DEVICE, REF_HOST = cpp_build.expected_programs()


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
def test_own_device_program(tmp_path):
    _run("own_test_frontend_device", tmp_path, required=True)


@pytest.mark.gpu
@pytest.mark.parametrize("name", REF_DEVICE)
def test_reference_samples(name, tmp_path):
    _run(name, tmp_path, required=False)
