"""Generates tests/golden/ref_cpu_cases.npz: outputs of the UNMODIFIED reference CPU backend
(oracle/_ref, built by oracle/build_ref.sh from the reference's own sources) for every
reference-native case of tests/cases.py, plus a checksum of each case's inputs so that a drift
of the seeded generator is detected; and tests/golden/plans/case_<name>.plan for cases.PLAN_CASES.  Run where the reference is present:

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import ref_runtime  # noqa: E402
import cases  # noqa: E402


def input_digest(case) -> str:
    h = hashlib.sha256()
    for a in case.inputs:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()[:16]


def main():
    out = {}
    for case in cases.CASES:
        if case.new_op:
            continue
        if case.expected().size == 0:
            continue
        comp = ref_runtime.Compiled(case.ir_text("cpu"), "cpu")
        (res,) = comp.run(case.inputs)
        comp.close()
        out[case.name] = res
        out["digest__" + case.name] = np.frombuffer(input_digest(case).encode(), dtype=np.uint8)
        print(f"{case.name:40s} {res.shape}")
    path = os.path.join(ROOT, "tests", "golden", "ref_cpu_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
    # executable plans of a few single-op graphs, derived by the reference for backend "cuda" with
    # this repository's plugin loaded (backend_lowering must find the kernel registrations)
    ref_runtime.load_b200_backend()
    for name in cases.PLAN_CASES:
        text = ref_runtime.plan_text(cases.CASES_BY_NAME[name].ir_text("cuda"), "cuda")
        with open(os.path.join(ROOT, "tests", "golden", "plans", "case_" + name + ".plan"), "w") as f:
            f.write(text)
        print("plan", name)


if __name__ == "__main__":
    main()
