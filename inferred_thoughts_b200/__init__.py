"""Importable name of the package directory `inferred-thoughts_b200/` (a hyphen cannot be imported): this package's
search path IS that directory, so `inferred_thoughts_b200.host`, `.build` and `.configs` are the files there."""
from pathlib import Path

__path__ = [str(Path(__file__).resolve().parent.parent / "inferred-thoughts_b200")]
__all__ = ["build", "host", "configs"]
