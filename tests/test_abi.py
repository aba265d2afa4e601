"""The C-ABI library builds, loads, and exports every symbol include/itb.h declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "itb.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(itb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from inferred_thoughts_b200 import build
    so = build.build()
    lib = ctypes.CDLL(str(so))
    names = declared_symbols()
    assert len(names) > 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_create_fails_loudly_without_a_device():
    import torch  # only to learn whether a device is present
    if torch.cuda.is_available():
        return
    from inferred_thoughts_b200 import host
    try:
        host.B200Ops(0)
    except RuntimeError as e:
        assert "itb_create failed" in str(e)
    else:
        raise AssertionError("itb_create succeeded with no CUDA device")


def test_dims_struct_matches_header_order():
    from inferred_thoughts_b200 import host
    text = (ROOT / "include" / "itb.h").read_text()
    body = text[text.index("typedef struct {\n    uint32_t n_layer"):text.index("} itb_model_dims;")]
    names = re.findall(r"\b([a-z_]+)(?=[,;])", body)
    assert names == [n for n, _ in host.ModelDims._fields_]
