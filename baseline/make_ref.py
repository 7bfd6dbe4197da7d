"""Puts the reference's own Python sources for this path where the GPU runs can reach them.

    python baseline/make_ref.py /path/to/Lvar

The GPU box has no reference checkout, so the files that are run there for CONTEXT (never on the product
path) are copied, unmodified, into the git-ignored folder ``baseline/_ref/``:

* ``kernels/sparse_attn/`` - the operator module, its config and the three Triton kernels (dense attention,
  dense attention + column sums, column-sparse attention): the only kernels of the reference that can run on a
  B200.  ``bench.py`` times them next to this package's kernels (``extra.reference_triton_us``).
* ``models/sparvar/sparse_attn.py`` and ``sparse_attn_layer_counter.py`` - the reference's CS4A policy class,
  which ``tests/test_gpu_reference_dropin.py`` runs over THIS package's operator modules.

Nothing under ``baseline/_ref/`` is committed or imported by the package.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
FILES = [
    "kernels/__init__.py",
    "kernels/sparse_attn/__init__.py",
    "kernels/sparse_attn/sparse_attn_config.py",
    "kernels/sparse_attn/sparse_attn_ops.py",
    "kernels/sparse_attn/triton/__init__.py",
    "kernels/sparse_attn/triton/attn_dense.py",
    "kernels/sparse_attn/triton/attn_dense_colsum.py",
    "kernels/sparse_attn/triton/attn_csp.py",
    "models/sparvar/sparse_attn.py",
    "models/sparvar/sparse_attn_layer_counter.py",
]


def make(ref: Path) -> Path:
    for rel in FILES:
        src = ref / rel
        if not src.exists():
            raise FileNotFoundError(f"{src} is missing from the reference checkout")
        dst = DEST / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python baseline/make_ref.py /path/to/Lvar")
    print(make(Path(sys.argv[1])))
