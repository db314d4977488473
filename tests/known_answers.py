"""Loads tests/golden/reference_known_answers.json into (op, dtype, inputs, attrs, expected)."""
import json
import os

import numpy as np

from oracle import frame_oracle as fo

HERE = os.path.dirname(os.path.abspath(__file__))
DT = {"float32": fo.DT_F32, "bfloat16": fo.DT_BF16}


def _tensor(spec, dtype):
    if "fill" in spec:
        arr = np.full(spec["shape"], spec["fill"], dtype=np.float32)
    else:
        arr = np.asarray(spec["data"], dtype=np.float32).reshape(spec["shape"])
    return fo.from_accum(arr, dtype)


def load():
    with open(os.path.join(HERE, "golden", "reference_known_answers.json")) as f:
        doc = json.load(f)
    out = []
    for c in doc["cases"]:
        dt = DT[c["dtype"]]
        ins = [_tensor(t, dt) for t in c["inputs"]]
        exp = _tensor(c["expected"], dt)
        out.append((c["cite"], c["op"], dt, ins, c.get("attrs", {}), exp, c.get("expected_bits")))
    return out


def oracle_eval(op, dt, ins, attrs):
    if op == "matmul":
        return fo.matmul(ins[0], ins[1], dt)
    if op == "conv2d":
        return fo.conv2d(ins[0], ins[1], ins[2] if len(ins) > 2 else None, tuple(attrs["stride"]),
                         tuple(attrs["padding"]), attrs["groups"], dt)
    if op == "max_pool2d":
        return fo.max_pool2d(ins[0], tuple(attrs["kernel"]), tuple(attrs["stride"]),
                             tuple(attrs["padding"]), dt)
    if op == "softmax":
        return fo.softmax(ins[0], dt)
    if op == "layer_norm":
        return fo.layer_norm(ins[0], ins[1], ins[2], attrs["eps"], dt)
    if op == "selective_scan":
        return fo.selective_scan(*ins, dtype=dt)
    if op == "fused_elementwise_internal":
        return fo.fused_elementwise(ins, attrs["ops"], attrs["arities"], dt)
    raise KeyError(op)
