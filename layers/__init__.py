"""Reference-style import path: ``from layers.gatconv_layer import GATConv``."""
from ae_mlsys_gnn_b200.layers import *  # noqa: F401,F403
