"""Generates tests/golden/ref_cpu_fullsize.npz: what the reference CPU backend computes for a slab
of each workload at its benchmark size (the MLP whole; the first 16 rows of GELU(A.B + bias) at
8192^3 in bf16 and fp32; sample 0 of the batch-32 conv stack; sequence 0 of the batch-8 transformer
block; sample 0 of the batch-16 Mamba block).  Rows and samples are independent on this path, so the
full-size GPU result must agree with the slab on those rows; the inputs are regenerated from their
seeds by the tests (frame_public_b200/configs.py), only the slab outputs are stored.  The Mamba
slab keeps a subset of its 2048 rows (MAMBA_ROWS) to stay small.

gelu, silu, softplus, bias_add and mamba_scan are not reference ops: their CPU kernels are this
repository's (loaded into the reference process), everything else is the unmodified reference.  For
the fp32 GEMM slab the script also evaluates tanh-GELU as a composition of reference-native ops
(mul, add, square, tanh with constant tensors as inputs) and checks that the two agree within the
fp32 tier.

Run where the reference is present:  python tests/golden/make_fullsize_golden.py
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_runtime  # noqa: E402
from oracle import frame_oracle as fo  # noqa: E402
from frame_public_b200 import configs, irtext  # noqa: E402

MAMBA_ROWS = np.unique(np.concatenate([np.arange(0, 64), np.arange(64, 2048, 16), np.arange(1984, 2048)]))


def gelu_composition_text(rows, n):
    """matmul -> add -> tanh-GELU from reference-native ops only; the three constants are inputs."""
    g = irtext.IrGraph("cpu")
    f = "float32"
    va, vb, vbias = g.input(f, (rows, n)), g.input(f, (n, n)), g.input(f, (rows, n))
    c_half, c_one, c_k, c_c = (g.input(f, (rows, n)) for _ in range(4))
    x = g.add(g.matmul(va, vb), vbias)
    x3 = g.mul(g.unary("square", x), x)
    inner = g.mul(c_k, g.add(x, g.mul(c_c, x3)))
    out = g.mul(g.mul(c_half, x), g.add(c_one, g.unary("tanh", inner)))
    g.output(out)
    return g.text()


def main():
    ref_runtime.load_b200_backend()
    out = {}
    for key, (builder, kw) in configs.FULL_BUILDERS.items():
        t0 = time.time()
        full = builder(**kw)
        ins = configs.slab_inputs(key, full.inputs)
        comp = ref_runtime.Compiled(configs.slab_graph(key), "cpu")
        t1 = time.time()
        (res,) = comp.run(ins)
        t2 = time.time()
        comp.close()
        if key == "mamba":
            res = res[MAMBA_ROWS]
        out[key] = res
        print(f"{key:12s} slab out {res.shape} inputs {t1 - t0:.1f}s cpu {t2 - t1:.1f}s", flush=True)
        if key == "gemm_f32":
            r, n = configs.GEMM_SLAB_ROWS, kw["n"]
            consts = [np.full((r, n), v, np.float32) for v in (0.5, 1.0, 0.7978845608028654, 0.044715)]
            comp = ref_runtime.Compiled(gelu_composition_text(r, n), "cpu")
            (alt,) = comp.run(ins + consts)
            comp.close()
            assert fo.all_close(res, alt, fo.DT_F32, rtol=1e-5, atol=1e-6), fo.max_err(res, alt)
            print("gemm_f32: gelu kernel agrees with the composition of reference ops", fo.max_err(res, alt))
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "ref_cpu_fullsize.npz"),
                        mamba_rows=MAMBA_ROWS.astype(np.int32), **out)


if __name__ == "__main__":
    main()
