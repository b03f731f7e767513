"""Puts the reference's own CPU implementation of the path next to the oracle, where the benchmark's
CPU arm and the tests can import it on a machine that has no reference checkout.

    python -m oracle.build_ref [/path/to/fp4-post]

TEST INFRASTRUCTURE ONLY.  The two pure-Python modules the path lives in (src/Metis/Metis/quant.py and
src/Metis/Metis/bitlinear.py of decisivemoments/fp4-post: torch is their only import) are copied,
unmodified, from the checkout into oracle/_ref/Metis/Metis/.  That folder is a build output like a
compiled .so: it is listed in .gitignore and never committed.  Without a checkout the call is a
no-op and reports so; callers then fall back to the restated oracle (oracle/metis_layer.py).
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
DEFAULT_CHECKOUT = Path("/root/reference")
FILES = ("src/Metis/Metis/quant.py", "src/Metis/Metis/bitlinear.py")


def build(checkout: Path | str | None = None) -> Path | None:
    """Copy the reference modules; returns the output folder, or None when there is no checkout."""
    root = Path(checkout) if checkout else DEFAULT_CHECKOUT
    if not all((root / f).exists() for f in FILES):
        return OUT if available() else None
    pkg = OUT / "Metis" / "Metis"
    pkg.mkdir(parents=True, exist_ok=True)
    for f in FILES:
        shutil.copyfile(root / f, pkg / Path(f).name)
    (OUT / "Metis" / "__init__.py").write_text("")
    (pkg / "__init__.py").write_text("from .bitlinear import BitLinear\n")
    return OUT


def available() -> bool:
    return all((OUT / "Metis" / "Metis" / Path(f).name).exists() for f in FILES)


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference checkout found: nothing copied")
