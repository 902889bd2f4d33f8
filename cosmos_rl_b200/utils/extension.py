"""Extension points for workloads that are not Hugging Face language models: how to get a tokenizer, how to resolve
a model name to a config without a ``config.json``, and custom parallelisation plans per model type
(``register_tokenizer_loader`` / ``register_local_model_config`` / ``register_parallelism_strategy`` in
cosmos_rl/utils/util.py and policy/model/base.py; used by tools/gym_example)."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

_TOKENIZER_LOADERS: Dict[str, Callable[[str], Any]] = {}
_LOCAL_CONFIGS: Dict[str, Callable[[str], Dict[str, Any]]] = {}
_PARALLELISM: Dict[str, Callable] = {}


def register_tokenizer_loader(prefix, loader: Callable[[str], Any]) -> None:
    """``loader(model_name_or_path)`` is used for model names starting with ``prefix``, or, when ``prefix`` is a
    callable, for names it returns true for (the reference's ``predicate`` form). Return None for no tokenizer."""
    _TOKENIZER_LOADERS[prefix] = loader


def clear_tokenizer_loaders() -> None:
    _TOKENIZER_LOADERS.clear()


def load_tokenizer(name_or_path: str):
    for prefix, fn in _TOKENIZER_LOADERS.items():
        try:
            hit = bool(prefix(name_or_path)) if callable(prefix) else (name_or_path or "").startswith(prefix)
        except Exception:  # noqa: BLE001  (a predicate that cannot judge this name does not match it)
            hit = False
        if hit:
            return fn(name_or_path), True
    return None, False


def register_local_model_config(prefix: str, fn: Callable[[str], Dict[str, Any]]) -> None:
    """``fn(model_name_or_path) -> dict`` in config.json form (must contain ``model_type``)."""
    _LOCAL_CONFIGS[prefix] = fn


def local_model_config(name_or_path: str) -> Optional[Dict[str, Any]]:
    for prefix, fn in _LOCAL_CONFIGS.items():
        if (name_or_path or "").startswith(prefix):
            return dict(fn(name_or_path))
    return None


def register_parallelism_strategy(model_type: str):
    """Decorator: ``fn(model, parallel_dims, config)`` is applied by the trainer after the model is materialised
    (attach tensor-parallel objects, expert groups, custom sharding)."""
    def deco(fn):
        _PARALLELISM[model_type] = fn
        return fn
    return deco


def parallelism_strategy(model_type: str) -> Optional[Callable]:
    return _PARALLELISM.get(model_type)
