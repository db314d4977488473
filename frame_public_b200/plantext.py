"""Reads the line-oriented plan text (the serialised ops::ExecutablePlan) on the Python side, to
account for the algorithmic work of each step: FLOPs of contractions, bytes moved by everything
else (every distinct input read once + the output written once, at the tensors' dtypes)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

ITEMSIZE = {0: 4, 1: 8, 2: 2, 3: 2, 4: 1, 5: 2, 6: 4, 7: 8, 8: 1, 9: 1}


@dataclass
class Slot:
    dtype: int
    dims: Tuple[int, ...]

    @property
    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * ITEMSIZE[self.dtype]


@dataclass
class PlanStep:
    op: str
    inputs: List[int]
    outputs: List[int]
    attrs: Dict[str, str] = field(default_factory=dict)


@dataclass
class Plan:
    slots: Dict[int, Slot]
    steps: List[PlanStep]
    inputs: List[int]
    outputs: List[int]
    arena_bytes: int


def parse(text: str) -> Plan:
    slots: Dict[int, Slot] = {}
    steps: List[PlanStep] = []
    inputs: List[int] = []
    outputs: List[int] = []
    arena = 0
    for line in text.splitlines():
        tok = line.split()
        if not tok:
            continue
        if tok[0] == "plan":
            arena = int(tok[2].split("=")[1])
        elif tok[0] == "in":
            idx, dtype, rank = int(tok[1]), int(tok[2]), int(tok[3])
            slots[idx] = Slot(dtype, tuple(int(t) for t in tok[4:4 + rank]))
            inputs.append(idx)
        elif tok[0] == "step":
            op = tok[1]
            nin = int(tok[2].split("=")[1])
            ins = [int(t) for t in tok[3:3 + nin]]
            pos = 3 + nin
            nout = int(tok[pos].split("=")[1])
            pos += 1
            outs = []
            for _ in range(nout):
                slot, dtype, _off, rank = int(tok[pos]), int(tok[pos + 1]), int(tok[pos + 2]), int(tok[pos + 3])
                dims = tuple(int(t) for t in tok[pos + 4:pos + 4 + rank])
                slots[slot] = Slot(dtype, dims)
                outs.append(slot)
                pos += 4 + rank
            steps.append(PlanStep(op, ins, outs))
        elif tok[0] == "attr":
            steps[-1].attrs[tok[1]] = line.split(" ", 3)[3] if len(tok) > 3 else ""
        elif tok[0] == "out":
            outputs.append(int(tok[1]))
    return Plan(slots, steps, inputs, outputs, arena)


def step_work(plan: Plan, index: int) -> Tuple[float, float]:
    """(algorithmic FLOPs, algorithmic bytes) of one step as the reference graph states it."""
    s = plan.steps[index]
    ins = [plan.slots[i] for i in s.inputs]
    outs = [plan.slots[o] for o in s.outputs]
    nbytes = float(sum(t.nbytes for t in {i: plan.slots[i] for i in s.inputs}.values()) + sum(t.nbytes for t in outs))
    flops = 0.0
    if s.op == "matmul":
        m, k = ins[0].dims
        n = ins[1].dims[1]
        flops = 2.0 * m * n * k
    elif s.op == "conv2d":
        cout, cpg, kh, kw = ins[1].dims
        flops = 2.0 * outs[0].numel * cpg * kh * kw
    elif s.op == "conv1d":
        cout, cpg, k = ins[1].dims
        flops = 2.0 * outs[0].numel * cpg * k
    return flops, nbytes


def attention_fan_work(plan: Plan) -> Tuple[float, float]:
    """(FLOPs, bytes) of all `matmul -> softmax -> matmul` chains of the plan together: the work of
    the single attention_fan launch that replaces them.  Bytes: each head's q, k, v read and its
    result written once."""
    producer = {o: i for i, s in enumerate(plan.steps) for o in s.outputs}
    flops = nbytes = 0.0
    for i, s in enumerate(plan.steps):
        if s.op != "softmax":
            continue
        scores = producer.get(s.inputs[0])
        values = next((j for j, t in enumerate(plan.steps) if t.op == "matmul" and t.inputs[0] == s.outputs[0]), None)
        if scores is None or values is None or plan.steps[scores].op != "matmul":
            continue
        flops += step_work(plan, scores)[0] + step_work(plan, values)[0]
        q, kt = (plan.slots[k] for k in plan.steps[scores].inputs)
        v = plan.slots[plan.steps[values].inputs[1]]
        o = plan.slots[plan.steps[values].outputs[0]]
        nbytes += q.nbytes + kt.nbytes + v.nbytes + o.nbytes
    return flops, nbytes
