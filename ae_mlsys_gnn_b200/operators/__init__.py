"""Mirror of the reference's ``operators`` package."""
from . import dense
from .csr2csc import csr2csc, sparsetrans
from .edge_softmax import csr_edge_softmax
from .fused_edgeconv import fused_edgeconv_op
from .fused_gat import fused_gat_fusescatter, fused_gat_op, fused_gat_stash_op
from .fused_gmmconv import GaussianCp, GmmConvFuse, GmmConvFuseEb, GmmConvStash
from .knn import knn_graph
from .mhspmm import csrmhspmm
from .spmm import coo_sddmm, csr_sddmm, csrspmm
from .u_add_v import u_add_v_op

__all__ = [
    "csr2csc", "sparsetrans", "csr_edge_softmax", "fused_edgeconv_op", "fused_gat_op",
    "fused_gat_stash_op", "fused_gat_fusescatter", "GmmConvFuse", "GmmConvFuseEb",
    "GmmConvStash", "GaussianCp", "csrmhspmm", "knn_graph", "csrspmm", "csr_sddmm", "coo_sddmm", "u_add_v_op",
]
