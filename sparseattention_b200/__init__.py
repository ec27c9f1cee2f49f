"""hsa_b200: hierarchical sparse attention for NVIDIA B200 (sm_100a).

Same public surface as the reference project's `hierarchical_attention` package
(hierarchical_attention/__init__.py:3-17); the device work is done by libhsa_b200.so.
"""
__version__ = "0.1.0"

from .modules import HierarchicalAttention
from .ops import (build_hierarchical_logits, build_parent_nodes, build_tree_topology, generate_span_input_Y,
                  hierarchical_attention)

__all__ = [
    "HierarchicalAttention",
    "build_tree_topology",
    "generate_span_input_Y",
    "build_parent_nodes",
    "hierarchical_attention",
    "build_hierarchical_logits",       # the logits op of the reference's first prototype (Hierarchical_Attention_Triton.py:456)
    "__version__",
]
