"""The shared library loads without a GPU and exports every entry point the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "lvar_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lvar_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported_and_bound():
    from lvar_b200 import _lib
    names = _declared()
    assert len(names) >= 13
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/lvar_b200.h but not exported"
    assert sorted(_lib.exported_symbols()) == names, "ctypes bindings and header disagree"


def test_version_config_and_error_string():
    from lvar_b200 import _lib
    assert _lib.version().count(".") == 2
    assert _lib.kernel_config_attn()["bm"] == 256
    assert isinstance(_lib.lib.lvar_last_error(), bytes)


def test_argument_struct_layout_matches_header():
    """Field order of the ctypes mirror follows the C struct (names in declaration order)."""
    from lvar_b200._lib import AttnArgs
    text = (ROOT / "include" / "lvar_b200.h").read_text()
    start = text.index("typedef struct lvar_attn_args {") + len("typedef struct lvar_attn_args {")
    body = text[start:text.index("} lvar_attn_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = decl.split()[-1] if "," not in decl else None
        if names is None:
            first, *rest = decl.split(",")
            fields.append(first.split()[-1].lstrip("*"))
            fields.extend(r.strip().lstrip("*") for r in rest)
        else:
            fields.append(names.lstrip("*"))
    assert fields == [f[0] for f in AttnArgs._fields_]
