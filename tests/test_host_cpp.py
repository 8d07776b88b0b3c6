"""Runs the C++ test programs of the host layer (cgadimpl_b200/host/tests/*.cpp): plain main()
executables in the style of the reference's own tests, built by cgadimpl_b200.host.build."""
import os
import subprocess

import pytest

from cgadimpl_b200.host import build as host_build

BIN = os.path.join(os.path.dirname(host_build.__file__), "build")


@pytest.fixture(scope="module", autouse=True)
def built():
    host_build.build()


def _run(name, timeout=600):
    r = subprocess.run([os.path.join(BIN, name)], capture_output=True, text=True, timeout=timeout)
    out = r.stdout + r.stderr
    assert r.returncode == 0, f"{name} failed (exit {r.returncode}):\n{out}"
    assert "all passed" in out, out
    return out


def test_host_layer_without_gpu():
    out = _run("test_host_cpu")
    assert out.count("[PASS]") >= 9 and "[FAIL]" not in out


@pytest.mark.gpu
def test_reference_gradient_checks_on_gpu():
    out = _run("test_core_ops_gpu")
    assert "[FAIL]" not in out and "Testing: RMSNorm " in out


@pytest.mark.gpu
def test_graph_api_parity_on_gpu():
    out = _run("test_rmsnorm_graph_gpu")
    assert "[FAIL]" not in out


@pytest.mark.gpu
def test_cuda_graph_capture_of_the_layer_stack():
    out = _run("test_graph_capture_gpu")
    assert "[FAIL]" not in out


@pytest.mark.gpu
def test_nn_module_and_optimizers_on_gpu():
    out = _run("test_nn_optim_gpu")
    assert "[FAIL]" not in out


@pytest.mark.gpu
def test_activation_checkpointing_across_the_stack():
    out = _run("test_checkpoint_gpu")
    assert "[FAIL]" not in out and out.count("[PASS]") >= 6
