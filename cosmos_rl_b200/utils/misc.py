"""Small helpers shared across the framework."""
from __future__ import annotations

import os
import random
import socket
from typing import Any, Dict, Optional

import numpy as np
import torch

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "float8_e4m3fn": torch.float8_e4m3fn, "fp8": torch.float8_e4m3fn,
}


def str2dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}") from None


def dtype2str(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


def seed_everything(seed: Optional[int]) -> None:
    if seed is None:
        return
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def rng_state() -> Dict[str, Any]:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def set_rng_state(st: Dict[str, Any]) -> None:
    random.setstate(st["python"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])


def free_port(host: str = "127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]


def local_ips() -> list:
    ips = ["127.0.0.1"]
    try:
        host_ip = socket.gethostbyname(socket.gethostname())
        if host_ip not in ips:
            ips.append(host_ip)
    except Exception:
        pass
    return ips


def env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def env_float(name: str, default: float) -> float:
    try:
        return float(os.environ.get(name, default))
    except ValueError:
        return default


def default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count())
    return torch.device("cpu")


# Peak dense tensor throughput (FLOP/s) used for MFU reports. The reference only knows H100 and A100
# (cosmos_rl/utils/util.py:524-533); B200 is added here.
PEAK_FLOPS = {
    "B200": {"bf16": 2.25e15, "fp8": 4.5e15, "fp32": 1.1e15},
    "H100": {"bf16": 1.979e15 / 2, "fp8": 1.979e15, "fp32": 0.989e15 / 2},
    "A100": {"bf16": 312e12, "fp32": 156e12},
}


def peak_flops(dtype: str = "bf16") -> float:
    name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else ""
    for key, tab in PEAK_FLOPS.items():
        if key in name:
            return tab.get(dtype, tab["bf16"])
    return PEAK_FLOPS["B200"][dtype]
