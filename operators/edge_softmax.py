from ae_mlsys_gnn_b200.operators.edge_softmax import *  # noqa: F401,F403
from ae_mlsys_gnn_b200.operators import edge_softmax as _impl
globals().update({k: v for k, v in vars(_impl).items() if not k.startswith('__')})
