"""Reference-style import path: ``from operators.fused_gat import fused_gat_op``."""
from ae_mlsys_gnn_b200.operators import *  # noqa: F401,F403
