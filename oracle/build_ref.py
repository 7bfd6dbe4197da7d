"""Builds the reference's own index kernels into ``oracle/_ref/`` (test infrastructure, git-ignored).

    python oracle/build_ref.py /path/to/Lvar

``kernels/chipmunk/csrc/indexed_io/mask_to_indices.cu`` and ``topk_indices.cu`` are plain CUDA + torch
extension sources without the Hopper-only parts of the reference's attention kernels, so they compile for
sm_100a as they are.  They are compiled from the checkout in place, together with ``ref_kernels/binding.cpp``
(this repository's own few lines of pybind11), into ``oracle/_ref/lvar_ref_indexed_io.so``.  The GPU tests load
that file when it exists and compare this package's kernels and the CPU oracle with it; nothing else uses it.
The reference's attention kernels (``csrc/attn/*.cu``) need ThunderKittens and wgmma and are not buildable here.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
NAME = "lvar_ref_indexed_io"
SOURCES = ["kernels/chipmunk/csrc/indexed_io/mask_to_indices.cu", "kernels/chipmunk/csrc/indexed_io/topk_indices.cu"]


def build(ref: Path, verbose: bool = False) -> Path:
    from torch.utils.cpp_extension import load
    srcs = [ref / s for s in SOURCES]
    for s in srcs:
        if not s.exists():
            raise FileNotFoundError(f"{s} is missing from the reference checkout")
    build_dir = DEST / "build"
    build_dir.mkdir(parents=True, exist_ok=True)
    load(name=NAME, sources=[str(s) for s in srcs] + [str(HERE / "ref_kernels" / "binding.cpp")],
         extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3"], extra_cflags=["-O2"],
         build_directory=str(build_dir), is_python_module=False, verbose=verbose)
    built = build_dir / f"{NAME}.so"
    out = DEST / f"{NAME}.so"
    out.write_bytes(built.read_bytes())
    shutil.rmtree(build_dir, ignore_errors=True)  # objects and ninja files: only the library is kept
    return out


def load_built():
    """The built module, or None when ``oracle/_ref`` does not hold it."""
    path = DEST / f"{NAME}.so"
    if not path.exists():
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/build_ref.py /path/to/Lvar")
    print(build(Path(sys.argv[1]), verbose=True))
