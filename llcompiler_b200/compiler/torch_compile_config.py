"""Decomposition table and operator-support test for the torch.compile backend.

Same role as llcompiler/compiler/torch_compile_config.py: LLC_DECOMPOSITIONS is the
reference's table (:12-28) unchanged; the support test (:71-132) is answered by the
importer's translator registry instead of a hand-kept dict, so the two cannot drift.
"""
import torch
from torch.fx.passes.operator_support import OperatorSupport

from ..importer.fx_translate import TORCH_FUNCTION_TRANSLATE, target_name

aten = torch.ops.aten

LLC_DECOMPOSITIONS = {
    aten.addmm,
    aten.expand,
    aten._unsafe_view,
    aten.transpose,
    aten.add,
    aten.mul,
    aten.sub,
    aten.div,
    aten.threshold_backward,
    aten.native_batch_norm_backward,
    aten.masked_fill,
    aten._softmax,
    aten.where,
    aten.squeeze.dim,
    aten.squeeze.dims,
}


class LLCOperatorSupport(OperatorSupport):
    def is_node_supported(self, submodules, node: torch.fx.Node) -> bool:
        if node.op in ("placeholder", "output"):
            return False
        if node.op != "call_function":
            return node.op == "get_attr"
        return target_name(node.target) in TORCH_FUNCTION_TRANSLATE


def unsupported_nodes(gm: torch.fx.GraphModule):
    return sorted({target_name(n.target) for n in gm.graph.nodes
                   if n.op == "call_function" and target_name(n.target) not in TORCH_FUNCTION_TRANSLATE})
