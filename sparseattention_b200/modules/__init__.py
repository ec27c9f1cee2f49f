from .attention import HierarchicalAttention

__all__ = ["HierarchicalAttention"]
