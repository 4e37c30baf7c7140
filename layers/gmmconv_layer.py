"""Reference-style import path for ae_mlsys_gnn_b200.layers.gmmconv_layer."""
from ae_mlsys_gnn_b200.layers import gmmconv_layer as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
