"""`webgpu_backend`: the torch.compile entry point (reference:
python/torch_webgpu/compiler/webgpu_compiler.py:22-62).

The reference lowers FX -> HighIR -> LowIR, runs the lowered program once at compile time,
prints it and then returns the *unfused* `gm.forward`; it accepts only graphs without inputs.
This backend keeps the entry point and does the job for real:

  1. dynamo's graph is normalised to ATen ops with `aot_autograd`, so `a + b`, `torch.add`,
     `operator.add`, `F.relu` ... all arrive as the same few overloads, with FakeTensor metadata;
  2. maximal runs of supported pointwise ops over one iteration shape are cut out of the graph
     (`partition`), each becomes one SSA program (`program.Program`) and one call to
     `torch.ops.webgpu.run_fused` - one kernel, no intermediate tensor touches HBM;
  3. a group whose only output is a bool mask consumed by masked_select of one of the group's own
     inputs becomes `torch.ops.webgpu.run_fused_select`: the mask travels as one bit per element
     in scratch memory instead of as a bool tensor (possible when dynamo keeps masked_select in
     the graph, see `webgpu_backend`);
  4. everything else (views, copies, ops the library has no fused form for) stays in the graph
     and runs through the dispatcher on the same device - there is no CPU fallback.
"""
from __future__ import annotations

import operator
from typing import Callable, List

import torch
from torch import fx
from torch._dynamo import register_backend
from torch._dynamo.backends.common import aot_autograd

from . import program as P

aten = torch.ops.aten

# Set by tests / users to watch what the backend did with the last graph it compiled.
last_compile_report: dict = {}


def _val(node):
    return node.meta.get("val") if isinstance(node, fx.Node) else None


def _is_webgpu_tensor(v) -> bool:
    return isinstance(v, torch.Tensor) and v.device.type == "webgpu"


def _dtype_tag(v):
    if v.dtype == torch.float32:
        return P.F32
    if v.dtype == torch.bool:
        return P.BOOL
    return None


def _fusible(node: fx.Node) -> bool:
    if node.op != "call_function" or node.target not in P.supported_targets():
        return False
    out = _val(node)
    if not _is_webgpu_tensor(out) or _dtype_tag(out) is None:
        return False
    t = node.target
    for arg in node.args:
        if isinstance(arg, fx.Node):
            v = _val(arg)
            if not _is_webgpu_tensor(v) or _dtype_tag(v) is None:
                return False
        elif not isinstance(arg, (int, float, bool)):
            return False
    tensor_args = [a for a in node.args if isinstance(a, fx.Node)]
    if t in P.UNARY_OPS or t is aten.gelu.default:
        return _dtype_tag(_val(tensor_args[0])) == P.F32
    if t in P.BINARY_OPS or t in P.COMPARE_OPS:
        return all(_dtype_tag(_val(a)) == P.F32 for a in tensor_args) and out.dtype in (torch.float32, torch.bool)
    if t in (aten.bitwise_and.Tensor, aten.logical_and.default):
        return len(tensor_args) == 2 and all(_dtype_tag(_val(a)) == P.BOOL for a in tensor_args)
    return False


def partition(graph: fx.Graph) -> list[list[fx.Node]]:
    """Split the graph's fusible nodes into groups that can each become one kernel.

    One group is open at a time.  A fusible node joins it when it iterates over the same shape;
    a different shape closes the group, and so does any other node that reads a value the open
    group produces (the value has to exist before that node runs).  Nodes that do not touch the
    group pass by without closing it, so independent ops in between do not break a chain.
    """
    groups: list[list[fx.Node]] = []
    open_group: list[fx.Node] = []
    open_shape = None

    def close():
        nonlocal open_group, open_shape
        if open_group:
            groups.append(open_group)
        open_group, open_shape = [], None

    for node in graph.nodes:
        if _fusible(node):
            shape = tuple(_val(node).shape)
            if open_group and shape != open_shape:
                close()
            open_group.append(node)
            open_shape = shape
        elif open_group and any(inp in open_group for inp in node.all_input_nodes):
            close()
    close()
    return [g for g in groups if len(g) >= 2]


def build_program(group: list[fx.Node]):
    """SSA program of a group plus the fx nodes that feed it and the group nodes it must output."""
    prog = P.Program()
    value_of: dict[fx.Node, int] = {}
    in_group = set(group)

    # external inputs, in first-use order
    for node in group:
        for arg in node.args:
            if isinstance(arg, fx.Node) and arg not in in_group and arg not in value_of:
                value_of[arg] = prog.add_input(arg, _dtype_tag(_val(arg)))

    def operand(arg) -> int:
        if isinstance(arg, fx.Node):
            return value_of[arg]
        return prog.const(float(arg))

    for node in group:
        t = node.target
        if t in P.UNARY_OPS:
            value_of[node] = prog.op(P.UNARY_OPS[t], operand(node.args[0]))
        elif t is aten.gelu.default:
            approximate = node.kwargs.get("approximate", node.args[1] if len(node.args) > 1 else "none")
            value_of[node] = prog.op(P.GELU_TANH if approximate == "tanh" else P.GELU_ERF, operand(node.args[0]))
        elif t in P.BINARY_OPS:
            a, b = operand(node.args[0]), operand(node.args[1])
            alpha = node.kwargs.get("alpha", node.args[2] if len(node.args) > 2 else 1)
            value_of[node] = prog.op(P.BINARY_OPS[t], a, b, float(alpha) if P.BINARY_OPS[t] == P.ADD else 0.0)
        elif t in P.COMPARE_OPS:
            a, b = operand(node.args[0]), operand(node.args[1])
            value_of[node] = prog.op(P.COMPARE_OPS[t], a, b)
        else:  # bitwise_and / logical_and on bool
            value_of[node] = prog.op(P.AND, operand(node.args[0]), operand(node.args[1]))

    out_nodes = [n for n in group if any(u not in in_group for u in n.users)]
    for n in out_nodes:
        prog.add_output(value_of[n])
    return prog, list(prog.inputs), out_nodes


def select_pattern(group: list[fx.Node], inputs: list, out_nodes: list[fx.Node]):
    """If the group's single output is a bool mask whose only consumer is
    masked_select(x, mask) with x one of the group's own f32 inputs of the same shape, return
    (masked_select node, index of x among the inputs): the pair can run as one fused select."""
    if len(out_nodes) != 1:
        return None
    mask = out_nodes[0]
    users = list(mask.users)
    if len(users) != 1 or users[0].op != "call_function" or users[0].target is not aten.masked_select.default:
        return None
    sel = users[0]
    if len(sel.args) != 2 or sel.args[1] is not mask or sel.args[0] not in inputs:
        return None
    mv = _val(mask)
    if mv.dtype != torch.bool:
        return None
    for node in inputs:
        v = _val(node)
        if v.dtype != torch.float32 or tuple(v.shape) != tuple(mv.shape):
            return None
    return sel, inputs.index(sel.args[0])


class FusedSelectKernel:
    """Callable placed in the rewritten graph: predicate (written as one bit per element) and the
    compaction that reads those bits, in place of a bool mask tensor followed by masked_select."""

    def __init__(self, prog: P.Program, src_index: int):
        self.program = prog
        self.src_index = src_index
        self.handle = torch.ops.webgpu.compile_fused(*prog.columns())
        self.kind = "aot" if torch.ops.webgpu.fused_kind(self.handle) == 0 else "nvrtc"
        self.__name__ = f"webgpu_fused_select_{len(prog.instrs)}"

    def __call__(self, *inputs):
        return torch.ops.webgpu.run_fused_select(self.handle, list(inputs), self.src_index)


class FusedKernel:
    """Callable placed in the rewritten graph: one launch of a compiled program."""

    def __init__(self, prog: P.Program):
        self.program = prog
        self.handle = torch.ops.webgpu.compile_fused(*prog.columns())
        self.kind = "aot" if torch.ops.webgpu.fused_kind(self.handle) == 0 else "nvrtc"
        self.out_dtypes = prog.out_dtypes()
        self.__name__ = f"webgpu_fused_{len(prog.instrs)}"

    def __call__(self, *inputs):
        return torch.ops.webgpu.run_fused(self.handle, list(inputs), self.out_dtypes)


def fuse_graph(gm: fx.GraphModule, options: dict | None = None) -> fx.GraphModule:
    options = options or {}
    graph = gm.graph
    kernels = []
    for group in partition(graph):
        prog, inputs, out_nodes = build_program(group)
        if not out_nodes:
            continue
        pattern = select_pattern(group, inputs, out_nodes) if options.get("fuse_select", True) else None
        if pattern is not None:
            sel, src_index = pattern
            kernel = FusedSelectKernel(prog, src_index)
            kernels.append(kernel)
            with graph.inserting_after(sel):
                call = graph.call_function(kernel, tuple(inputs))
            call.meta = dict(sel.meta)
            sel.replace_all_uses_with(call)
            graph.erase_node(sel)
            for n in reversed(group):
                graph.erase_node(n)
            continue
        kernel = FusedKernel(prog)
        kernels.append(kernel)
        with graph.inserting_after(group[-1]):
            call = graph.call_function(kernel, tuple(inputs))
        prev = call
        for slot, n in enumerate(out_nodes):
            with graph.inserting_after(prev):
                item = graph.call_function(operator.getitem, (call, slot))
            item.meta = dict(n.meta)
            n.replace_all_uses_with(item)
            prev = item
        for n in reversed(group):
            graph.erase_node(n)
    graph.lint()
    gm.recompile()
    last_compile_report.clear()
    last_compile_report.update(
        fused_kernels=len(kernels),
        kinds=[k.kind for k in kernels],
        fused_selects=sum(isinstance(k, FusedSelectKernel) for k in kernels),
        instructions=[len(k.program.instrs) for k in kernels],
        programs=[str(k.program) for k in kernels],
        remaining_ops=[str(n.target) for n in graph.nodes if n.op == "call_function" and not isinstance(n.target, (FusedKernel, FusedSelectKernel))
                       and n.target is not operator.getitem],
    )
    return gm


@register_backend
def webgpu_backend(gm: fx.GraphModule, example_inputs: List[torch.Tensor], **kwargs) -> Callable:
    """torch.compile(fn, backend=webgpu_backend[, options={"fuse_select": False}]).

    masked_select has a data-dependent output shape, so dynamo cuts the graph in front of it unless
    `torch._dynamo.config.capture_dynamic_output_shape_ops = True`.  With that flag set, a mask that
    feeds nothing but masked_select of one of the chain's own inputs is never written as a bool
    tensor: the fused kernel writes it as one bit per element into scratch memory and the compaction
    reads the bits (webgpu::run_fused_select; 0.75 ms against 0.83 ms for the three-input silu chain
    over 2^28 elements on B200).  `options={"fuse_select": False}` keeps the bool tensor and the
    plain masked_select; without the dynamo flag the graph break leaves no other choice.
    """
    options = dict(kwargs.pop("options", None) or {})

    def fw_compiler(graph_module: fx.GraphModule, _example_inputs):
        return fuse_graph(graph_module, options).forward

    return aot_autograd(fw_compiler=fw_compiler)(gm, example_inputs, **kwargs)
