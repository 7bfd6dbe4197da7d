"""CPU restatement of the reference's sparse-attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is shipped or measured as the product: it is imported by ``tests/``,
by ``__graft_entry__.smoke()`` (as the checker) and by ``bench.py`` (CPU baseline / reference arm).
Every function cites the file and lines of the reference project (Weepingchestnut/Lvar, paths relative
to its root) whose arithmetic it follows.

Parity status: pinned.  ``tests/golden/make_golden.py`` imports the reference's own Python functions
(``naive_dense_colsum_attn``, ``reference_blocksums``, ``reference_sparse_o``, the SparVAR index
builders, the CSLA mask builder's arithmetic) and stores their outputs on seeded inputs under
``tests/golden/``; ``tests/test_oracle_golden.py`` checks this package against those files.
Third-party arithmetic on the path that no reference test pins (``torch.topk``, ``flex_attention``) is defined
here: top-k is a stable descending sort (lower index wins a tie, the one thing PyTorch leaves open) and
block-sparse attention is a dense masked fp32 softmax; the GPU tests run both PyTorch operators, the reference's
Triton attention kernels (``baseline/_ref``) and its CUDA index kernels (``build_ref.py`` -> ``oracle/_ref``) on
the same device and compare them with these definitions and with the product's kernels.
"""
