"""Wire format of an enqueue request: a little-endian u32 header length, a JSON header (reward names, metadata,
tensor dtype and shape), then the raw tensor bytes. Text-only requests carry no tensor
(reward_service/cosmos_rl_reward/utils/protocol.py)."""
from __future__ import annotations

import json
import struct
from typing import Any, Dict, List, Optional, Tuple

import torch

_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "uint8": torch.uint8,
           "int64": torch.int64}

ENQUEUE, PULL, PUSH, PING = "/api/reward/enqueue", "/api/reward/pull", "/api/reward/push", "/api/reward/ping"


def encode_request(reward_fns: List[str], metadata: Dict[str, Any], tensor: Optional[torch.Tensor] = None) -> bytes:
    head: Dict[str, Any] = {"reward_fns": reward_fns, "metadata": metadata}
    body = b""
    if tensor is not None:
        t = tensor.detach().cpu().contiguous()
        name = str(t.dtype).replace("torch.", "")
        if name not in _DTYPES:
            raise ValueError(f"unsupported tensor dtype {t.dtype}")
        head["tensor"] = {"dtype": name, "shape": list(t.shape)}
        body = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.uint8 else t.numpy().tobytes()
    h = json.dumps(head).encode()
    return struct.pack("<I", len(h)) + h + body


def decode_request(blob: bytes) -> Tuple[List[str], Dict[str, Any], Optional[torch.Tensor]]:
    if len(blob) < 4:
        raise ValueError("request shorter than its header length field")
    (n,) = struct.unpack("<I", blob[:4])
    if 4 + n > len(blob):
        raise ValueError("header length exceeds the request size")
    head = json.loads(blob[4:4 + n])
    tensor = None
    if "tensor" in head:
        dt = _DTYPES[head["tensor"]["dtype"]]
        shape = head["tensor"]["shape"]
        raw = torch.frombuffer(bytearray(blob[4 + n:]), dtype=torch.uint8)
        numel = 1
        for s in shape:
            numel *= int(s)
        if raw.numel() != numel * torch.empty((), dtype=dt).element_size():
            raise ValueError("tensor payload size does not match its declared shape")
        tensor = raw.view(dt).view(shape)
    return list(head["reward_fns"]), dict(head.get("metadata", {})), tensor
