"""The Python bindings name every exported C launcher with as many arguments as its declaration
has: a list that is one short makes ctypes pass the rest unconverted, which crashes the process
instead of raising."""

from __future__ import annotations

import re
from pathlib import Path

from tinyserve_b200.kernels import ops

CSRC = Path(ops.__file__).resolve().parent.parent / "csrc"


def test_signatures_match_the_c_declarations() -> None:
    source = "".join(f.read_text() for f in sorted(CSRC.glob("*.cu")))
    for name, sig in ops._SIGNATURES.items():
        m = re.search(r'extern "C" int ' + name + r"\s*\(([^)]*)\)", source)
        assert m, f"{name} is bound but not declared in csrc"
        params = [a for a in m.group(1).split(",") if a.strip()]
        assert len(params) == len(sig), f"{name}: {len(params)} parameters in C, {len(sig)} in the binding"
