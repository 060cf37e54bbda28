"""The graph passes of buddy_mlir_b200/graph_pass.py against buddy-mlir's own graph classes
and its own quantisation passes: a small graph is built by hand, quantised by the reference
(weight_only_channel_wise / w8a8_channel_wise,
frontend/Python/graph/transform/quantization/passes.py:37-63), and the matmul that comes out
must become the external call of this library, with the graph's edges and index lists intact.

Needs a buddy-mlir checkout (BUDDY_MLIR_ROOT, or a `reference` directory beside the
repository); its graph package imports the MLIR Python bindings at module level, which are
not needed to build and rewrite graphs, so they are stood in for by empty modules."""
import importlib.abc
import importlib.machinery
import os
import sys
import types
from unittest import mock

import pytest

from buddy_mlir_b200 import graph_pass

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("BUDDY_MLIR_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
FRONTEND = os.path.join(REF, "frontend", "Python")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(FRONTEND, "graph")),
                                reason="needs a buddy-mlir checkout for its graph classes")


class _NoBindings(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Answers `import buddy_mlir...` with an empty stand-in module."""

    def find_spec(self, name, path, target=None):
        if name == "buddy_mlir" or name.startswith("buddy_mlir."):
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = mock.MagicMock(name=spec.name)
        m.__path__, m.__name__, m.__spec__ = [], spec.name, spec
        return m

    def exec_module(self, module):
        pass


@pytest.fixture(scope="module")
def bc():
    """buddy.compiler.graph of the checkout (frontend/Python is installed under that name)."""
    finder = _NoBindings()
    sys.meta_path.insert(0, finder)
    saved = {k: sys.modules.get(k) for k in ("buddy", "buddy.compiler")}
    top, comp = types.ModuleType("buddy"), types.ModuleType("buddy.compiler")
    top.__path__, comp.__path__ = [], [FRONTEND]
    top.compiler = comp
    sys.modules["buddy"], sys.modules["buddy.compiler"] = top, comp
    try:
        import buddy.compiler.graph as g
        import buddy.compiler.graph.transform.quantization as q
        yield types.SimpleNamespace(graph=g, ops=g.operation, quant=q)
    finally:
        sys.meta_path.remove(finder)
        for k in [k for k in sys.modules
                  if k in ("buddy", "buddy_mlir") or k.startswith("buddy.") or k.startswith("buddy_mlir.")]:
            sys.modules.pop(k)
        for k, v in saved.items():
            if v is not None:
                sys.modules[k] = v


def build(bc, with_plain_matmul=False):
    """y = (x @ w) [@ x2 when with_plain_matmul]: w is a parameter, x and x2 are inputs."""
    g, ops = bc.graph, bc.ops
    graph = g.Graph({}, "forward")
    f32 = g.TensorDType.Float32

    def add(cls, name, args, shape, kind=g.NodeType.OtherNode):
        op = cls()
        op._name = name
        for a in args:
            op.add_argument(a)
            op.add_parent(a)
            graph.node_table[a].add_children(name)
        op.tensor_meta = {"shape": list(shape), "dtype": f32}
        graph.add_node(op, kind)
        return op
    add(ops.PlaceholderOp, "w", [], (64, 32), g.NodeType.FakeNode)
    add(ops.PlaceholderOp, "x", [], (4, 64), g.NodeType.InputNode)
    add(ops.MatmulOp, "mm", ["x", "w"], (4, 32))
    last = "mm"
    if with_plain_matmul:
        add(ops.PlaceholderOp, "x2", [], (32, 8), g.NodeType.InputNode)
        add(ops.MatmulOp, "mm2", ["mm", "x2"], (4, 8))
        last = "mm2"
    add(ops.OutputOp, "output", [last], (4, 8) if with_plain_matmul else (4, 32))
    return graph


def check_edges(graph):
    """Every argument that names a node is a parent, every parent lists the node as a child,
    and the parameter / input index lists point at placeholders."""
    for node in graph.body:
        for a in node.args:
            if isinstance(a, str) and a in graph.node_table:
                assert a in node._parents, (node.name, a)
        for p in node._parents:
            assert p in graph.node_table and node.name in graph.node_table[p]._children, (node.name, p)
        for c in node._children:
            assert c in graph.node_table and node.name in graph.node_table[c]._parents, (node.name, c)
    assert [graph.body[i].name for i in graph._inputs] == [n.name for n in graph.body if n.name in ("x", "x2")]
    assert sorted(graph.body[i].name for i in graph._fake_params) == ["scaler_w", "w"]


def test_weight_only_matmul_becomes_the_int8_gemv_call(bc):
    graph = build(bc, with_plain_matmul=True)
    bc.quant.weight_only_channel_wise(graph)
    assert isinstance(graph.node_table["mm"], bc.ops.MatmulOp) and "dequantized_w" in graph.node_table
    assert graph_pass.replace_dequant_matmul_with_b200(graph, bc.ops) == 1
    call = graph.node_table["mm"]
    assert isinstance(call, bc.ops.CallExternalOp)
    assert call.call_func_name == "buddy_gemv_w8_f32"
    assert list(call.args) == ["x", "w", "scaler_w"] and call._args_index == [0, 0, 0]
    assert call.tensor_meta["shape"] == [4, 32]
    assert "dequantized_w" not in graph.node_table                  # the chain went with its only consumer
    assert graph.node_table["w"].tensor_meta["dtype"] == bc.graph.TensorDType.Int8
    assert isinstance(graph.node_table["mm2"], bc.ops.MatmulOp)     # activation x activation: untouched
    assert list(graph.node_table["mm2"].args) == ["mm", "x2"]
    check_edges(graph)
    assert graph_pass.replace_dequant_matmul_with_b200(graph, bc.ops) == 0     # idempotent


def test_w8a8_matmul_becomes_the_integer_tensor_core_call(bc):
    graph = build(bc)
    bc.quant.w8a8_channel_wise(graph)
    assert isinstance(graph.node_table["mm"], bc.ops.QuantizedMatmulOp)
    assert graph_pass.replace_quantized_matmul_with_b200(graph, bc.ops) == 1
    call = graph.node_table["mm"]
    assert isinstance(call, bc.ops.CallExternalOp) and call.call_func_name == "buddy_matmul_w8a8_f32"
    assert list(call.args) == ["x", "w", "scaler_w"]
    assert call._op_type == bc.ops.OpType.Unfusable
    assert list(graph.node_table["output"].args) == ["mm"]
    check_edges(graph)


def test_a_dequantisation_with_another_consumer_stays(bc):
    graph = build(bc)
    bc.quant.weight_only_channel_wise(graph)
    # a second consumer of the dequantised weight (say, a tied embedding read)
    extra = bc.ops.MulOp()
    extra._name = "other_use"
    extra.add_argument("dequantized_w")
    extra.add_parent("dequantized_w")
    extra.tensor_meta = {"shape": [64, 32], "dtype": bc.graph.TensorDType.Float32}
    graph.node_table["dequantized_w"].add_children("other_use")
    graph.body.insert(len(graph.body) - 1, extra)
    graph.node_table["other_use"] = extra
    assert graph_pass.replace_dequant_matmul_with_b200(graph, bc.ops) == 1
    assert "dequantized_w" in graph.node_table
    assert graph.node_table["dequantized_w"]._children == ["other_use"]
    check_edges(graph)
