"""SSA programs for fused pointwise kernels.

A `Program` is what the library's `twg_fused_compile` consumes: a straight-line list of
(opcode, a, b, imm) over f32 / bool values (include/twg.h, TwgFusedOpcode).  This module knows how
ATen pointwise ops map to opcodes and keeps the emission order canonical - inputs in first-use
order, then the operations in graph order with each scalar constant emitted right before its use,
then the outputs - so that equal subgraphs always produce equal programs (and hit the kernels the
library instantiates ahead of time).

It replaces the reference's HighIR -> LowIR lowering (python/torch_webgpu/compiler/high_ir.py,
low_ir.py), whose only fusion is the peephole ADD,RELU -> FUSED_ADD_RELU (high_ir.py:108-120).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

aten = torch.ops.aten

# TwgFusedOpcode
INPUT_F32, INPUT_BOOL, CONST_F32, ADD, MUL, RELU, SILU, GELU_ERF, GELU_TANH, ABS = range(10)
EQ, NE, LT, LE, GT, GE, AND, OUTPUT = range(10, 18)

F32, BOOL = "f32", "bool"

UNARY_OPS = {
    aten.relu.default: RELU,
    aten.silu.default: SILU,
    aten.abs.default: ABS,
}
COMPARE_OPS = {}
for _name, _code in (("eq", EQ), ("ne", NE), ("lt", LT), ("le", LE), ("gt", GT), ("ge", GE)):
    _packet = getattr(aten, _name)
    COMPARE_OPS[_packet.Tensor] = _code
    COMPARE_OPS[_packet.Scalar] = _code
BINARY_OPS = {
    aten.add.Tensor: ADD,
    aten.add.Scalar: ADD,
    aten.mul.Tensor: MUL,
    aten.mul.Scalar: MUL,
}
OTHER_OPS = {aten.gelu.default, aten.bitwise_and.Tensor, aten.logical_and.default}


def supported_targets():
    return set(UNARY_OPS) | set(COMPARE_OPS) | set(BINARY_OPS) | OTHER_OPS


@dataclass
class Program:
    instrs: list = field(default_factory=list)   # (opcode, a, b, imm)
    types: list = field(default_factory=list)    # F32 / BOOL per value
    inputs: list = field(default_factory=list)   # external keys, slot order
    outputs: list = field(default_factory=list)  # (value index, type), slot order

    def _emit(self, opcode: int, a: int = 0, b: int = 0, imm: float = 0.0, ty: str | None = None) -> int:
        self.instrs.append((opcode, a, b, float(imm)))
        self.types.append(ty)
        return len(self.instrs) - 1

    def add_input(self, key, ty: str) -> int:
        slot = len(self.inputs)
        self.inputs.append(key)
        return self._emit(INPUT_BOOL if ty == BOOL else INPUT_F32, slot, 0, 0.0, ty)

    def const(self, value: float) -> int:
        return self._emit(CONST_F32, 0, 0, float(value), F32)

    def op(self, opcode: int, a: int, b: int = 0, imm: float = 0.0) -> int:
        if opcode in (ADD, MUL):
            assert self.types[a] == F32 and self.types[b] == F32
            ty = F32
        elif opcode in (RELU, SILU, GELU_ERF, GELU_TANH, ABS):
            assert self.types[a] == F32
            ty = F32
        elif EQ <= opcode <= GE:
            assert self.types[a] == F32 and self.types[b] == F32
            ty = BOOL
        elif opcode == AND:
            assert self.types[a] == BOOL and self.types[b] == BOOL
            ty = BOOL
        else:
            raise ValueError(f"unknown opcode {opcode}")
        return self._emit(opcode, a, b, imm, ty)

    def add_output(self, value: int) -> int:
        slot = len(self.outputs)
        self.outputs.append((value, self.types[value]))
        self._emit(OUTPUT, value, slot, 0.0, None)
        return slot

    def columns(self):
        """The four parallel lists `torch.ops.webgpu.compile_fused` takes."""
        return ([i[0] for i in self.instrs], [i[1] for i in self.instrs], [i[2] for i in self.instrs],
                [i[3] for i in self.instrs])

    def out_dtypes(self):
        # c10::ScalarType codes, which is what an `int[]` schema argument can carry
        scalar_type_bool, scalar_type_float = 11, 6
        return [scalar_type_bool if ty == BOOL else scalar_type_float for _, ty in self.outputs]

    def __str__(self) -> str:
        names = {INPUT_F32: "input_f32", INPUT_BOOL: "input_bool", CONST_F32: "const", ADD: "add", MUL: "mul",
                 RELU: "relu", SILU: "silu", GELU_ERF: "gelu_erf", GELU_TANH: "gelu_tanh", ABS: "abs", EQ: "eq",
                 NE: "ne", LT: "lt", LE: "le", GT: "gt", GE: "ge", AND: "and", OUTPUT: "output"}
        return "\n".join(f"  v{i} = {names[o]}(a={a}, b={b}, imm={imm})" for i, (o, a, b, imm) in enumerate(self.instrs))
