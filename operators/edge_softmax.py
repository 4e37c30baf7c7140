"""Reference-style import path for ae_mlsys_gnn_b200.operators.edge_softmax."""
from ae_mlsys_gnn_b200.operators import edge_softmax as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
