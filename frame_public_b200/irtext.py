"""Builds Frame IR text (the reference's deterministic text serialisation, one node per line:
`%<id> = <op>(%<in>, ...) {<attr>=<value>, ...} : <dtype>[<shape>]@<backend>:<index>`,
include/frame/ir/serialization.h:1-60 of the reference) from Python, with the shape rules of
the op schemas on the compiled-graph path.  The text is what the reference's `ir::parse_text`
reads; it is how the harness hands graphs to the reference pipeline without a C++ build step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

DTYPE_NAMES = {0: "float32", 1: "float64", 2: "float16", 3: "bfloat16", 4: "int8", 5: "int16",
               6: "int32", 7: "int64", 8: "uint8", 9: "bool"}
DTYPE_CODES = {v: k for k, v in DTYPE_NAMES.items()}


@dataclass(frozen=True)
class Value:
    id: int
    dtype: str
    shape: tuple


def _fmt_double(v: float) -> str:
    s = repr(float(v))
    if s in ("inf", "-inf", "nan"):
        return s
    if "." not in s and "e" not in s and "E" not in s:
        s += ".0"
    return s


def _fmt_attr(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if isinstance(v, float):
        return _fmt_double(v)
    if isinstance(v, str):
        return '"' + v.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n") + '"'
    if isinstance(v, Shape):
        return "shape[" + ",".join(str(d) for d in v.dims) + "]"
    if isinstance(v, DTypeAttr):
        return f"dtype({v.name})"
    if isinstance(v, (list, tuple)):
        if len(v) > 0 and isinstance(v[0], float):
            return "[" + ", ".join(_fmt_double(e) for e in v) + "]"
        return "[" + ", ".join(str(int(e)) for e in v) + "]"
    raise TypeError(f"unsupported attribute value {v!r}")


@dataclass(frozen=True)
class Shape:
    dims: tuple


@dataclass(frozen=True)
class DTypeAttr:
    name: str


class DoubleList(list):
    """A kDoubleArray attribute (forces the double formatting even for integral values)."""


def conv_out(size: int, k: int, stride: int, pad: int) -> int:
    return (size + 2 * pad - k) // stride + 1


class IrGraph:
    def __init__(self, backend: str = "cpu", device: int = 0):
        self.backend = backend
        self.device = device
        self.lines: List[str] = []
        self.next_id = 0
        self.inputs: List[Value] = []
        self.outputs: List[Value] = []

    def _type(self, dtype: str, shape: Sequence[int]) -> str:
        return f"{dtype}[{','.join(str(int(d)) for d in shape)}]@{self.backend}:{self.device}"

    def input(self, dtype: str, shape: Sequence[int]) -> Value:
        v = Value(self.next_id, dtype, tuple(int(d) for d in shape))
        self.next_id += 1
        self.lines.append(f"%{v.id} = graph_input() : {self._type(dtype, shape)}")
        self.inputs.append(v)
        return v

    def node(self, op: str, inputs: Sequence[Value], attrs: Dict[str, object], dtype: str,
             shape: Sequence[int]) -> Value:
        v = Value(self.next_id, dtype, tuple(int(d) for d in shape))
        self.next_id += 1
        args = ", ".join(f"%{i.id}" for i in inputs)
        attr_txt = ""
        if attrs:
            parts = []
            for k in sorted(attrs):
                val = attrs[k]
                if isinstance(val, DoubleList):
                    parts.append(f"{k}=[" + ", ".join(_fmt_double(e) for e in val) + "]")
                else:
                    parts.append(f"{k}={_fmt_attr(val)}")
            attr_txt = " {" + ", ".join(parts) + "}"
        self.lines.append(f"%{v.id} = {op}({args}){attr_txt} : {self._type(dtype, shape)}")
        return v

    def output(self, v: Value) -> None:
        self.outputs.append(v)

    def text(self) -> str:
        return "\n".join(self.lines + [f"graph_output(%{v.id})" for v in self.outputs]) + "\n"

    # ---- ops on the path (shape rules of the reference's schemas) -------------------------------
    def matmul(self, a: Value, b: Value) -> Value:
        assert len(a.shape) == 2 and len(b.shape) == 2 and a.shape[1] == b.shape[0]
        return self.node("matmul", [a, b], {}, a.dtype, (a.shape[0], b.shape[1]))

    def binary(self, op: str, a: Value, b: Value) -> Value:
        assert a.shape == b.shape, (op, a.shape, b.shape)
        return self.node(op, [a, b], {}, a.dtype, a.shape)

    def add(self, a, b):
        return self.binary("add", a, b)

    def mul(self, a, b):
        return self.binary("mul", a, b)

    def unary(self, op: str, x: Value) -> Value:
        return self.node(op, [x], {}, x.dtype, x.shape)

    def softmax(self, x: Value) -> Value:
        return self.node("softmax", [x], {}, x.dtype, x.shape)

    def layer_norm(self, x: Value, gamma: Value, beta: Value, eps: float = 1e-5) -> Value:
        return self.node("layer_norm", [x, gamma, beta], {"eps": float(eps)}, x.dtype, x.shape)

    def selective_scan(self, x, a, b, c, d) -> Value:
        return self.node("selective_scan", [x, a, b, c, d], {}, x.dtype, x.shape)

    def conv2d(self, x: Value, w: Value, bias=None, stride=(1, 1), padding=(0, 0), groups=1) -> Value:
        n, _, h, wd = x.shape
        cout, _, kh, kw = w.shape
        shape = (n, cout, conv_out(h, kh, stride[0], padding[0]), conv_out(wd, kw, stride[1], padding[1]))
        ins = [x, w] + ([bias] if bias is not None else [])
        return self.node("conv2d", ins, {"stride": list(stride), "padding": list(padding),
                                         "groups": int(groups)}, x.dtype, shape)

    def conv1d(self, x: Value, w: Value, bias=None, stride=1, padding=0, groups=1) -> Value:
        n, _, l = x.shape
        cout, _, k = w.shape
        ins = [x, w] + ([bias] if bias is not None else [])
        return self.node("conv1d", ins, {"stride": int(stride), "padding": int(padding),
                                         "groups": int(groups)}, x.dtype,
                         (n, cout, conv_out(l, k, stride, padding)))

    def max_pool2d(self, x: Value, kernel=(2, 2), stride=(2, 2), padding=(0, 0)) -> Value:
        n, c, h, w = x.shape
        shape = (n, c, conv_out(h, kernel[0], stride[0], padding[0]),
                 conv_out(w, kernel[1], stride[1], padding[1]))
        return self.node("max_pool2d", [x], {"kernel": list(kernel), "stride": list(stride),
                                             "padding": list(padding)}, x.dtype, shape)

    def reshape(self, x: Value, shape) -> Value:
        return self.node("reshape", [x], {"target_shape": Shape(tuple(shape))}, x.dtype, shape)

    def transpose(self, x: Value, perm) -> Value:
        return self.node("transpose", [x], {"perm": list(perm)}, x.dtype,
                         tuple(x.shape[p] for p in perm))

    def slice(self, x: Value, axis: int, start: int, stop: int) -> Value:
        shape = list(x.shape)
        shape[axis] = stop - start
        return self.node("slice", [x], {"axis": axis, "start": start, "stop": stop}, x.dtype, shape)

    def concat(self, xs, axis: int) -> Value:
        shape = list(xs[0].shape)
        shape[axis] = sum(v.shape[axis] for v in xs)
        return self.node("concat", list(xs), {"axis": axis}, xs[0].dtype, shape)

    def sum(self, x: Value, axes, keepdims: bool = False) -> Value:
        axes = [a % len(x.shape) for a in axes]
        shape = [d for i, d in enumerate(x.shape) if i not in axes]
        return self.node("sum", [x], {"axes": list(axes)}, x.dtype, shape)

    def constant(self, values, shape, dtype: str) -> Value:
        return self.node("constant", [], {"value": DoubleList(float(v) for v in values),
                                          "shape": Shape(tuple(shape)), "dtype": DTypeAttr(dtype)},
                         dtype, shape)

    # ---- new ops (registered by this repository's plugin, not part of the reference) -----------
    def bias_add(self, x: Value, bias: Value) -> Value:
        assert bias.shape == (x.shape[-1],)
        return self.node("bias_add", [x, bias], {}, x.dtype, x.shape)

    def mamba_scan(self, u, delta, A, B, C, D, z=None) -> Value:
        ins = [u, delta, A, B, C, D] + ([z] if z is not None else [])
        return self.node("mamba_scan", ins, {}, u.dtype, u.shape)
