"""Reference-style import path for ae_mlsys_gnn_b200.operators.u_add_v."""
from ae_mlsys_gnn_b200.operators import u_add_v as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
