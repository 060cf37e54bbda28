"""Graph passes that hand buddy-mlir graph operations to this library's per-op
external kernels (the `_mlir_ciface_buddy_*` symbols of buddy_b200_memref.h).

They are written against buddy-mlir's own graph classes and are meant to live
next to `frontend/Python/graph/transform/runtime_matmul_replace.py:27-55`, whose
shape they follow: an operation is replaced by a `CallExternalOp`
(`frontend/Python/graph/operation.py:714-736`) that the frontend lowers to a
`func.call` with `llvm.emit_c_interface`, so the linked library's
`_mlir_ciface_<call_func_name>` receives MemRef descriptors.

    replace_quantized_matmul_with_b200   QuantizedMatmulOp (the w8a8 graphs,
                                         transform/quantization/passes.py:54-140)
                                         -> buddy_matmul_w8a8_f32
    replace_dequant_matmul_with_b200     cast(int8 weight) * scaler -> MatmulOp
                                         (the weight-only graphs) -> buddy_gemv_w8_f32

Registration, like the RNG group (`frontend/Python/frontend.py:55-61,1373-1396`):

    EXTERNAL_CALL_TRANSFORM_GROUPS["b200"] = (replace_quantized_matmul_with_b200,
                                              replace_dequant_matmul_with_b200)
    EXTERNAL_CALL_GROUP_LIBS["b200"] = "libbuddy_b200_kernels"

`ops` is the module that defines the graph's operation classes; inside the
buddy-mlir tree that is `buddy.compiler.graph.operation` (the default).
"""


def _operation_module(ops):
    if ops is not None:
        return ops
    from buddy.compiler.graph import operation      # the installed name of frontend/Python/graph
    return operation


def _swap_in(graph, old, new, arg_names):
    """`new` takes the place, the name and the consumers of `old`; its producers are arg_names."""
    new._arguments = list(arg_names)
    new._parents = []
    for name in arg_names:
        if name in graph.node_table and name not in new._parents:
            new._parents.append(name)
    new._children = list(old._children)
    for name in old._parents:            # producers that no longer feed this node
        if name not in new._parents and name in graph.node_table:
            producer = graph.node_table[name]
            producer._children = [c for c in producer._children if c != old.name]
    for name in new._parents:
        producer = graph.node_table[name]
        if new.name not in producer._children:
            producer._children.append(new.name)
    graph._body[graph._body.index(old)] = new
    graph.node_table[new.name] = new


def _drop_unused(graph, nodes):
    """Remove nodes nobody consumes any more (a dequantisation whose matmul was replaced, and the
    cast that fed it), keeping the index lists of inputs and parameters consistent."""
    params = [graph._body[i] for i in graph._fake_params]
    inputs = [graph._body[i] for i in graph._inputs]
    pending = list(nodes)
    while pending:
        node = pending.pop()
        if node.name not in graph.node_table or node._children:
            continue
        if node in params or node in inputs:
            continue
        for name in node._parents:
            producer = graph.node_table.get(name)
            if producer is not None:
                producer._children = [c for c in producer._children if c != node.name]
                pending.append(producer)
        graph._body.remove(node)
        graph.node_table.pop(node.name)
    where = {id(n): i for i, n in enumerate(graph._body)}
    graph._fake_params = [where[id(n)] for n in params]
    graph._inputs = [where[id(n)] for n in inputs]


def _external_call(ops, old, func_name, n_args):
    meta = old.tensor_meta
    call = ops.CallExternalOp(call_func_name=func_name, args=[], args_index=[0] * n_args,
                              tensor_meta={"shape": meta.get("shape", []), "dtype": meta.get("dtype", "float32")},
                              name=old.name)
    call._op_type = ops.OpType.Unfusable
    return call


def replace_quantized_matmul_with_b200(graph, ops=None):
    """QuantizedMatmulOp(activation, int8 weight, weight scale) -> buddy_matmul_w8a8_f32.
    The arguments map one to one (`frontend/Python/ops/linalg.py:12797-12803`); the kernel is
    bit-identical to the lowering it replaces.  QuantizedAddMMOp keeps its own lowering (the
    external kernel takes no bias).  Returns the number of operations replaced."""
    ops = _operation_module(ops)
    count = 0
    for op in list(graph.body):
        if isinstance(op, ops.QuantizedMatmulOp):
            call = _external_call(ops, op, "buddy_matmul_w8a8_f32", 3)
            _swap_in(graph, op, call, list(op.args[:3]))
            count += 1
    return count


def replace_dequant_matmul_with_b200(graph, ops=None):
    """MatmulOp(activation, dequantized_<w>) with dequantized_<w> = cast(<w>) * scaler_<w>
    (what WeightOnlyQuantization leaves behind, transform/quantization/weight_only_channel_wise.py:366-461)
    -> buddy_gemv_w8_f32(activation, <w>, scaler_<w>).  The dequantisation chain is removed when
    nothing else consumes it.  Returns the number of operations replaced."""
    ops = _operation_module(ops)
    count, orphans = 0, []
    for op in list(graph.body):
        if not isinstance(op, ops.MatmulOp) or len(op.args) < 2:
            continue
        dequant = graph.node_table.get(op.args[1])
        if not isinstance(dequant, ops.MulOp) or not dequant.name.startswith("dequantized_"):
            continue
        weight = dequant.name[len("dequantized_"):]
        scaler = "scaler_" + weight
        if weight not in graph.node_table or scaler not in graph.node_table:
            continue
        call = _external_call(ops, op, "buddy_gemv_w8_f32", 3)
        _swap_in(graph, op, call, [op.args[0], weight, scaler])
        orphans.append(dequant)
        count += 1
    _drop_unused(graph, orphans)
    return count
