"""lvar_b200: B200 (sm_100a) kernels for the sparse-attention hot path of VAR / Infinity
next-scale prediction - dense, block-sparse and column-sparse attention, attention column sums
(KV-importance scores) and the mask / index construction between them.

Importing the package does not load the CUDA library; ``lvar_b200.kernels`` and
``lvar_b200.sparse_attn_ops`` do, and raise if it is missing.
"""

__version__ = "0.1.0"
