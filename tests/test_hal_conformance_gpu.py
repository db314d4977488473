"""The reference's HAL conformance cases (tests/cpp/hal_conformance/test_hal_conformance.cpp:96-269 of
the reference) applied to this repository's C++ classes, B200Backend / B200Allocator / B200Stream /
B200Event / B200Backend::compile, as the reference's BackendRegistry hands them out under the name
"cuda": name round trip, device count, stream and event creation, an unrecorded event reports
complete, record -> wait -> synchronize, a 64-byte aligned allocation that survives host -> device ->
host through Backend::copy, device-to-device copies, and compile() of an op without a kernel
returning kUnimplemented with the op's name."""
import pytest

from oracle import ref_runtime

pytestmark = pytest.mark.gpu

if not ref_runtime.available():
    pytest.skip("oracle/_ref (the reference build) is not present", allow_module_level=True)


def test_b200_backend_classes_meet_the_hal_contract():
    ref_runtime.load_b200_backend()
    assert ref_runtime.has_backend("cuda")
    failed, report = ref_runtime.hal_conformance("cuda")
    assert failed == 0, report
    assert len(report) == 8 and all(line.startswith("ok ") for line in report)
