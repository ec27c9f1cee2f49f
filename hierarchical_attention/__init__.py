"""Drop-in import name: `from hierarchical_attention import HierarchicalAttention, ...` keeps working
for code written against the reference package; everything is served by sparseattention_b200."""
from sparseattention_b200 import (HierarchicalAttention, __version__, build_hierarchical_logits, build_parent_nodes,
                                  build_tree_topology, generate_span_input_Y, hierarchical_attention)

__all__ = ["HierarchicalAttention", "build_tree_topology", "generate_span_input_Y", "build_parent_nodes",
           "hierarchical_attention", "build_hierarchical_logits", "__version__"]
