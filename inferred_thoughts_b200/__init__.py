"""Importable alias of the package directory `inferred-thoughts_b200/` (a hyphen cannot be imported)."""
from pathlib import Path

__path__ = [str(Path(__file__).resolve().parent.parent / "inferred-thoughts_b200")]
exec(compile((Path(__path__[0]) / "__init__.py").read_text(), str(Path(__path__[0]) / "__init__.py"), "exec"))
