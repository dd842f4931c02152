"""Makes the golden logits of ``tests/golden/``: the UPSTREAM engine's own model code
(princemittalr/tinyserve, ``src/tinyserve``) run on the CPU in float32 on the tiny random
models of ``tests/tiny_configs.py``.

    python tests/golden/make_golden.py --upstream-src <path to upstream>/src

Upstream's package asks ``importlib.metadata`` for its installed version
(src/tinyserve/__init__.py:3-5); it is not installed here, so that one lookup is answered
with a constant. Nothing else of upstream is altered. For each tiny model the script writes
``tiny_<name>.safetensors`` holding the token ids, upstream's ``Qwen3.forward`` logits
``[T, vocab]`` float32, the model's weights themselves (``w.<tensor name>``, float32: a few
hundred KB), and their checksum. A test re-makes the weights from the same seed; if this torch
build draws the same values it uses those (which also pins the random-weights mode), otherwise it
falls back on the stored ones, so the comparison with upstream's logits always runs.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.metadata as md
import sys
import tempfile
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from tiny_configs import TINIES, random_prompt, write_tiny  # noqa: E402

PROMPT_LEN = {"A": 33, "B": 40, "C": 21}


def weights_checksum(folder: Path) -> str:
    from safetensors import safe_open

    h = hashlib.sha256()
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        for name in sorted(f.keys()):
            h.update(name.encode())
            h.update(f.get_tensor(name).float().numpy().tobytes())
    return h.hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--upstream-src", required=True, type=Path)
    args = ap.parse_args()
    sys.path.insert(0, str(args.upstream_src))
    orig = md.version
    md.version = lambda name: "0.0.0" if name == "tinyserve" else orig(name)
    from tinyserve.config import ModelConfig
    from tinyserve.model import Qwen3
    from tinyserve.weights import load_weights

    for name, (cfg_dict, _, seed) in TINIES.items():
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_tiny(Path(tmp), name, torch.float32)
            cfg = ModelConfig.from_file(folder / "config.json")
            model = Qwen3(cfg, load_weights(folder, cfg, torch.float32, "cpu"))
            ids = random_prompt(PROMPT_LEN[name], cfg_dict["vocab_size"], 100 + seed)
            logits = model.forward(torch.tensor(ids))
            digest = weights_checksum(folder)
            stored = {}
            with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
                for tensor_name in f.keys():
                    stored["w." + tensor_name] = f.get_tensor(tensor_name).float().contiguous()
        save_file(
            {"token_ids": torch.tensor(ids, dtype=torch.int32), "logits": logits.float().contiguous(), **stored},
            str(HERE / f"tiny_{name}.safetensors"),
            metadata={"weights_sha256": digest, "seed": str(seed), "source": "upstream Qwen3.forward, float32, CPU"},
        )
        print(name, tuple(logits.shape), float(logits.abs().max()), digest[:12])


if __name__ == "__main__":
    main()
