"""Mirror of the reference's ``layers`` package (the fused layers only)."""
from .edgeconv_layer import EdgeConv
from .gatconv_layer import GATConv, GATConv_fusescatter, GATConv_stash
from .gmmconv_layer import GMMConv, GMMConv_stash

__all__ = ["GATConv", "GATConv_stash", "GATConv_fusescatter", "EdgeConv", "GMMConv", "GMMConv_stash"]
