"""The reference's own API tests for the hot path (test/mlu_op_gtest/api_gtest/src/gtest/
get_indice_pairs/*.cpp and indice_convolution_forward/*.cpp: 102 status-code cases), compiled
unchanged from the reference tree against this library's headers and shared library by
tests/api_gtest/build_ref_api_gtest.py, must all pass: source compatibility of the drop-in
boundary, and the reference's own expectations of every argument check."""
import importlib.util
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _binary(pkg):
    spec = importlib.util.spec_from_file_location("build_ref_api_gtest",
                                                  os.path.join(HERE, "api_gtest", "build_ref_api_gtest.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    exe = mod.build()
    if exe is None:
        pytest.skip("the reference tree is absent and no prebuilt binary travelled with the repository")
    return exe


def _run(exe, extra_env):
    env = dict(os.environ, MLUOP_MIN_LOG_LEVEL="3", **extra_env)
    r = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=600)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    assert "[  PASSED  ] 102 test cases." in r.stdout, tail


def test_reference_api_tests_pass_on_a_host_only_handle(pkg):
    _run(_binary(pkg), {"MLUOP_B200_HOST_ONLY_HANDLE": "1", "CUDA_VISIBLE_DEVICES": ""})


@pytest.mark.gpu
def test_reference_api_tests_pass_on_the_gpu(pkg):
    _run(_binary(pkg), {})
