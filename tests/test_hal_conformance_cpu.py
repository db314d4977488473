"""The HAL contract check of oracle/ref_shim.cpp (the eight cases of the reference's parameterised
conformance suite, tests/cpp/hal_conformance/test_hal_conformance.cpp:96-269 of the reference) run
against the reference's own CPU backend: it must pass there, which pins the check itself before the
GPU test applies it to this repository's backend classes."""
import pytest

from oracle import ref_runtime

pytestmark = pytest.mark.skipif(not ref_runtime.available(), reason="the reference build (oracle/_ref) is not present")


def test_reference_cpu_backend_meets_the_contract():
    failed, report = ref_runtime.hal_conformance("cpu")
    assert failed == 0, report
    assert len(report) == 8 and all(line.startswith("ok ") for line in report)


def test_unknown_backend_fails_every_case():
    failed, report = ref_runtime.hal_conformance("no_such_backend")
    assert failed == 8 and report[0].startswith("FAIL ")


def test_cnn_builder_emits_the_reference_golden_graph():
    """nn::Sequential{Conv2d, Relu, MaxPool2d, Flatten, Linear} at the shape of the reference's own
    golden (tests/cpp/nn/testdata/cnn_forward_expected.txt): conv2d -> relu -> max_pool2d -> reshape ->
    matmul -> add."""
    text = ref_runtime.nn_graph_text("cnn", 8, 1, 8, 4, 1, True, 0, "cpu")
    ops = [line.split("=")[1].split("(")[0].strip() for line in text.splitlines() if line.startswith("%")]
    assert ops == ["graph_input"] * 5 + ["conv2d", "relu", "max_pool2d", "reshape", "matmul", "add"]
    assert "float32[8,4,8,8]" in text and "target_shape=shape[8,64]" in text and "float32[8,1]" in text
