"""Reference-style import path for ae_mlsys_gnn_b200.operators.fused_gmmconv."""
from ae_mlsys_gnn_b200.operators import fused_gmmconv as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
