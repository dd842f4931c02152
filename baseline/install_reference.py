"""Place the upstream engine, unmodified, under ``baseline/_ref`` so that ``bench.py --impl reference``
can import it.

    python baseline/install_reference.py <path of an upstream checkout>

Upstream is pure Python (its ``pyproject.toml`` needs the ``hatchling`` backend only to pack a wheel),
and ``pip install --no-index --no-build-isolation`` fails where hatchling is not installed. What pip
would have put into the target folder is reproduced by hand instead: the package folder
``src/tinyserve`` copied byte for byte, and a ``tinyserve-<version>.dist-info/METADATA`` beside it,
which is all that ``importlib.metadata.version("tinyserve")`` in upstream's ``__init__.py`` asks for.
Nothing of upstream is edited, and nothing of this repository is imported on that path.
"""

from __future__ import annotations

import re
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def install(checkout: Path) -> Path:
    src = checkout / "src" / "tinyserve"
    if not (src / "engine.py").is_file():
        raise FileNotFoundError(f"{checkout} is not an upstream checkout (no src/tinyserve/engine.py)")
    text = (checkout / "pyproject.toml").read_text(encoding="utf-8")
    version = re.search(r'^version\s*=\s*"([^"]+)"', text, re.M)
    if version is None:
        raise ValueError("no version in upstream's pyproject.toml")
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.mkdir(parents=True)
    shutil.copytree(src, TARGET / "tinyserve", ignore=shutil.ignore_patterns("__pycache__"))
    info = TARGET / f"tinyserve-{version.group(1)}.dist-info"
    info.mkdir()
    (info / "METADATA").write_text(f"Metadata-Version: 2.1\nName: tinyserve\nVersion: {version.group(1)}\n",
                                   encoding="utf-8")
    (info / "INSTALLER").write_text("baseline/install_reference.py\n", encoding="utf-8")
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(f"upstream placed in {install(Path(sys.argv[1]))}")
