"""sga_b200: selective gradient accumulation training on B200 (sm_100a).

Plugin axes (score / selection / optimizer / backend), the flat ``--sga-*``
configuration, shadow and trace capture, offline fused replay and the
residual-aware AdamW of the reference framework, on hand-written CUDA kernels
that fuse compute with NVLink peer-memory collectives.
"""
__version__ = "0.1.0"
