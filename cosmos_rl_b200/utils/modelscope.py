"""ModelScope hub access (cosmos_rl/utils/modelscope.py). Jobs of this package read data sets and checkpoints from
local folders; these entry points exist so scripts that import them load, and say what to do instead when called."""
from __future__ import annotations

import os


def if_use_modelscope(path: str) -> bool:
    return False


def modelscope_load_dataset(name: str, subset_name=None, split=None, **kw):
    if os.path.exists(name):
        from ..tools.dataset.common import load_rows
        return load_rows(name, subset_name, split)
    raise RuntimeError(f"data set {name!r} is not a local path and hub downloads are not available: download it "
                       f"beforehand and point train.train_policy.dataset.name (or local_dir) at the folder")
