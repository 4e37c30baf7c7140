"""B200-native (sm_100a) fused GNN sparse kernels behind the ``operators`` /
``layers`` API of mlsysAE2022/ae_mlsys_gnn.

``ae_mlsys_gnn_b200.operators`` and ``ae_mlsys_gnn_b200.layers`` mirror the
reference's modules of the same names; the top-level ``operators`` and ``layers``
packages of this repository re-export them so that reference-style imports
(``from operators.fused_gat import fused_gat_op``) keep working.
"""
__version__ = "0.1.0"
