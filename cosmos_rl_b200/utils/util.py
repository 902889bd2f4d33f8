"""Helpers under the names user scripts of the reference import from ``cosmos_rl.utils.util``
(cosmos_rl/utils/util.py:64-1528): tokenizer set-up with registered loaders, ``call_setup`` for both ``setup``
signatures, data loading, small numeric helpers, MFU. Each is written on this package's own functions."""
from __future__ import annotations

import base64
import functools
import importlib.util
import inspect
import json
import os
import random
import struct
import time
import warnings
from typing import Any, Callable, Dict, List, Optional

import torch

from .extension import clear_tokenizer_loaders, load_tokenizer, register_tokenizer_loader  # noqa: F401
from .logging import logger
from .misc import peak_flops, str2dtype


def str2torch_dtype(dtype_str: str) -> torch.dtype:
    return str2dtype(dtype_str)


def retry(func: Optional[Callable] = None, *, max_retry: int = 10, max_delay: float = 30.0):
    """Decorator (bare or with arguments): call again after an exception, with exponential back-off and jitter."""
    def deco(f):
        @functools.wraps(f)
        def wrapped(*a, **kw):
            delay = 1.0
            for attempt in range(max_retry + 1):
                try:
                    return f(*a, **kw)
                except Exception as e:  # noqa: BLE001
                    if attempt == max_retry:
                        raise
                    logger.warning("%s failed (%s); retry %d of %d", getattr(f, "__name__", f), e, attempt + 1, max_retry)
                    time.sleep(min(delay, max_delay) * (0.5 + random.random() / 2))
                    delay *= 2
        return wrapped
    return deco(func) if callable(func) else deco


@functools.lru_cache(maxsize=None)
def setup_tokenizer(model_name_or_path: str):
    """A registered loader's tokenizer when one matches, else the ``transformers`` tokenizer of a local folder (pad
    token defaulting to the end-of-sequence token); None for built-in architecture names, which have no vocabulary."""
    tok, handled = load_tokenizer(model_name_or_path)
    if handled:
        return tok
    if not os.path.isdir(model_name_or_path):
        return None
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(model_name_or_path, trust_remote_code=False)
    if getattr(tok, "pad_token_id", None) is None:
        tok.pad_token_id = tok.eos_token_id
    return tok


def call_setup(dataset_or_datapacker, config) -> None:
    """Call ``setup`` of a data set or data packer written for either signature: ``setup(config)`` or the older
    ``setup(config, tokenizer)``."""
    fn = getattr(dataset_or_datapacker, "setup", None)
    if fn is None:
        return
    params = [p for p in inspect.signature(fn).parameters.values()
              if p.name != "self" and p.kind == p.POSITIONAL_OR_KEYWORD]
    required = sum(1 for p in params if p.default is inspect.Parameter.empty)
    if required <= 1:
        fn(config)
    elif required == 2:
        warnings.warn(f"{type(dataset_or_datapacker).__name__}.setup(config, tokenizer) is the older signature",
                      DeprecationWarning, stacklevel=2)
        fn(config, setup_tokenizer(config.policy.model_name_or_path))
    else:
        raise TypeError(f"{type(dataset_or_datapacker).__name__}.setup must take (config) or (config, tokenizer)")


def load_data_from_disk_or_hf(data_name: str, data_subset: Optional[str] = None, revision: Optional[str] = None):
    """Rows of a local data set (json / jsonl / parquet / a saved ``datasets`` folder); there is no hub access here."""
    from ..tools.dataset.common import load_rows
    return load_rows(data_name, data_subset, None)


def read_json_file(path: str):
    with open(path) as f:
        return json.load(f)


def write_json_file(data, path: str) -> None:
    with open(path, "w") as f:
        json.dump(data, f, indent=4)


def list_to_b64(lst: List[int]) -> str:
    return base64.b64encode(struct.pack(f"{len(lst)}i", *lst)).decode()


def b64_to_list(s: str) -> List[int]:
    raw = base64.b64decode(s)
    return list(struct.unpack(f"{len(raw) // 4}i", raw))


def basename_from_modelpath(path: str) -> str:
    return os.path.basename(os.path.normpath(path))


def is_master_rank(parallel_dims, global_rank: int) -> bool:
    return global_rank == 0


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    m = mask.to(values.dtype)
    if axis is None:
        return (values * m).sum() / m.sum().clamp_min(1e-8)
    return (values * m).sum(axis) / m.sum(axis).clamp_min(1e-8)


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[index]`` without materialising the full log-softmax in the input dtype."""
    lse = torch.logsumexp(logits.float(), dim=-1)
    return logits.gather(-1, index[..., None])[..., 0].float() - lse


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    lsm = torch.log_softmax(logits.float(), dim=-1)
    return -(lsm.exp() * lsm).sum(-1)


def entropy_from_logits_with_chunking(logits: torch.Tensor, chunk_size: int = 2048) -> torch.Tensor:
    flat = logits.reshape(-1, logits.shape[-1])
    out = torch.cat([entropy_from_logits(flat[i:i + chunk_size]) for i in range(0, flat.shape[0], chunk_size)])
    return out.view(logits.shape[:-1])


def get_device_flops(dtype: torch.dtype, num_gpus: int) -> int:
    name = {torch.bfloat16: "bf16", torch.float16: "bf16", torch.float32: "tf32"}.get(dtype, "bf16")
    try:
        return int(peak_flops(name) * num_gpus)
    except Exception:  # noqa: BLE001
        return int(peak_flops("bf16") * num_gpus)


def compute_mfu(model, n_tokens: int, iter_time: float, num_gpus: int, dtype: torch.dtype) -> Dict[str, float]:
    """Model FLOPs utilisation of one step from the model's own accounting (``get_nparams_and_flops``)."""
    seq = max(1, int(n_tokens))
    _, flops_per_token = model.get_nparams_and_flops(seq)
    achieved = flops_per_token * n_tokens / max(iter_time, 1e-9)
    return {"mfu": achieved / max(get_device_flops(dtype, num_gpus), 1), "tflops": achieved / 1e12}


def dynamic_import_module(path: str, attr: Optional[str] = None):
    """Import a Python file by path; with ``attr`` return that attribute, else the module's public names."""
    spec = importlib.util.spec_from_file_location(os.path.splitext(os.path.basename(path))[0], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if attr is not None:
        return getattr(mod, attr)
    return {k: v for k, v in vars(mod).items() if not k.startswith("_")}


def sanitize(obj):
    """JSON-friendly copy: tensors and numpy scalars become Python numbers / lists, unknown objects their ``str``."""
    if isinstance(obj, dict):
        return {str(k): sanitize(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [sanitize(v) for v in obj]
    if isinstance(obj, torch.Tensor):
        return obj.item() if obj.numel() == 1 else obj.tolist()
    if hasattr(obj, "item") and not isinstance(obj, (str, bytes)):
        try:
            return obj.item()
        except Exception:  # noqa: BLE001
            pass
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return str(obj)


def do_once(func):
    """Run the wrapped function on the first call only (later calls return the first result)."""
    done: Dict[str, Any] = {}

    @functools.wraps(func)
    def wrapped(*a, **kw):
        if "v" not in done:
            done["v"] = func(*a, **kw)
        return done["v"]
    return wrapped


def aggregate_report_data(reports: List[Dict[str, Any]]) -> Dict[str, Any]:
    """Per-replica step reports -> one: ``*_max`` and iteration time take the maximum, everything else the mean."""
    from ..dispatcher.status import PolicyStatusManager
    return PolicyStatusManager._aggregate_reports(reports)


def split_train_n_val_dataset(rows, test_size, seed: int = 0):
    """(train rows, validation rows): the last ``test_size`` rows (a count, or a fraction of the whole)."""
    rows = list(rows)
    n = test_size if isinstance(test_size, int) else int(len(rows) * float(test_size))
    n = max(0, min(n, len(rows)))
    return rows[:len(rows) - n], rows[len(rows) - n:]
