"""Model registry: which class serves a model folder.

A folder with `params.json` is a reference-format checkpoint (`Transformer`); a folder with `config.json` names its design in
the key "architecture", looked up in ARCHITECTURES.  `load_model` is what the command-line tools call.
"""
import json
from pathlib import Path
from typing import Any, Callable, Dict, Union

import torch

ARCHITECTURES: Dict[str, Callable[..., Any]] = {}


def register(name: str, loader: Callable[..., Any]) -> None:
    ARCHITECTURES[name] = loader


def _layered(*a: Any, **k: Any) -> Any:
    from .layered import LayeredTransformer
    return LayeredTransformer.from_folder(*a, **k)


def _reference_format(*a: Any, **k: Any) -> Any:
    from .transformer import Transformer
    return Transformer.from_folder(*a, **k)


register("Fesenex", _layered)
register("Taruvik", _layered)
register("Lotazen", _layered)
register("Viladra", _layered)
register("transformer", _reference_format)


def architecture_of(folder: Union[Path, str]) -> str:
    folder = Path(folder)
    if (folder / "params.json").exists():
        return "transformer"
    with open(folder / "config.json", "r") as f:
        arch = json.load(f).get("architecture")
    if arch not in ARCHITECTURES:
        raise ValueError(f"{folder}: unknown architecture {arch!r} (known: {sorted(ARCHITECTURES)})")
    return arch


def load_model(folder: Union[Path, str], max_batch_size: int = 1, device: Union[torch.device, str] = "cuda", dtype: Any = None, **kwargs: Any) -> Any:
    return ARCHITECTURES[architecture_of(folder)](folder, max_batch_size=max_batch_size, device=device, dtype=dtype, **kwargs)
