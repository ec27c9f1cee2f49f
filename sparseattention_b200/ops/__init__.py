from .functional import build_hierarchical_logits, build_parent_nodes, hierarchical_attention
from .topology import build_tree_topology, generate_span_input_Y

__all__ = ["build_parent_nodes", "hierarchical_attention", "build_tree_topology", "generate_span_input_Y",
           "build_hierarchical_logits"]
