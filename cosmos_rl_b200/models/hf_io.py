"""HF-compatible weight I/O: config resolution, safetensors loading with TP slicing and q/k/v, gate/up
fusion, and export back to the HF layout (<= 4 GB shards + ``model.safetensors.index.json``).
Reference behaviour: cosmos_rl/policy/model/gpt/__init__.py:573-673 (load),
cosmos_rl/policy/trainer/llm_trainer/llm_trainer.py:445-790 (export),
cosmos_rl/utils/multi_rank_weight_loader.py:34-300 (ranks split the files and broadcast tensors).
"""
from __future__ import annotations

import glob
import json
import os
import shutil
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils.logging import logger

MAX_SHARD_BYTES = 4 * 1024 ** 3


def load_hf_config(name_or_path: str, override: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """A dict in HF ``config.json`` form. Sources, in order: an explicit dict, ``<path>/config.json``,
    a built-in architecture name (``qwen2.5-7b``, ``qwen3-30b-a3b`` ...)."""
    if override:
        return dict(override)
    from ..utils.extension import local_model_config
    custom = local_model_config(name_or_path)
    if custom is not None:
        return custom
    if name_or_path and os.path.isdir(name_or_path) and os.path.exists(os.path.join(name_or_path, "config.json")):
        with open(os.path.join(name_or_path, "config.json")) as f:
            return json.load(f)
    key = (name_or_path or "").lower().split("/")[-1]
    from . import named_architectures
    archs = named_architectures()
    for k, args in archs.items():
        if k == key or k.replace("-", "") == key.replace("-", "").replace("_", "").replace("instruct", ""):
            return args.to_hf_config()
    raise FileNotFoundError(
        f"cannot resolve model {name_or_path!r}: not a local HF folder and not a built-in architecture "
        f"({sorted(archs)}); there is no network access to download it")


def has_safetensors(path: str) -> bool:
    return bool(glob.glob(os.path.join(path, "*.safetensors")))


def _index(path: str) -> Dict[str, str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return json.load(f)["weight_map"]
    from safetensors import safe_open
    out = {}
    for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with safe_open(fn, framework="pt") as f:
            for k in f.keys():
                out[k] = os.path.basename(fn)
    return out


def _tp_slice(name: str, t: torch.Tensor, tp: int, r: int, cfg) -> torch.Tensor:
    """Slice one HF tensor for tensor-parallel rank ``r``: column-parallel (rows of the weight) for
    q/k/v/gate/up/embed/lm_head, row-parallel (columns) for o/down; KV heads replicate when tp > n_kv."""
    if tp == 1:
        return t
    if any(s in name for s in ("q_proj", "gate_proj", "up_proj", "embed_tokens", "lm_head")) and t.dim() >= 1:
        return t.chunk(tp, dim=0)[r]
    if any(s in name for s in ("k_proj", "v_proj")):
        n_kv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
        if n_kv >= tp:
            return t.chunk(tp, dim=0)[r]
        rep = tp // n_kv
        return t.chunk(n_kv, dim=0)[r // rep]
    if any(s in name for s in ("o_proj", "down_proj")) and t.dim() == 2:
        return t.chunk(tp, dim=1)[r]
    return t


def load_hf_state(model, read, available, cfg: Dict[str, Any], tp: int = 1, r: int = 0) -> None:
    """Fill ``model`` (fused layout, TP rank ``r`` of ``tp``) from HF-named tensors served by ``read(name)``."""
    from .base import ModelRegistry
    mapper = ModelRegistry.mapper(cfg.get("model_type"))(cfg)
    mapper.ep_rank = getattr(getattr(model, "args", None), "ep_rank", 0)
    mapper.layer_offset = getattr(model, "layer_offset", 0)
    mapper.layer_map = getattr(model, "layer_map", None)
    missing = []
    with torch.no_grad():
        for name, p in model.named_parameters():
            if ".lora_" in name:               # adapters are not part of the base checkpoint
                continue
            if hasattr(mapper, "load_param") and mapper.load_param(name, p, read, available, tp, r):
                continue
            hf_names = mapper.hf_names(name)
            if not all(h in available for h in hf_names):
                if name.startswith("lm_head") and "model.embed_tokens.weight" in available:
                    hf_names = ["model.embed_tokens.weight"]
                else:
                    missing.append(name)
                    continue
            parts = [_tp_slice(h, read(h), tp, r, cfg) for h in hf_names]
            t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
            if tuple(t.shape) != tuple(p.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != model shape {tuple(p.shape)}")
            p.copy_(t.to(p.dtype))
    if missing:
        raise KeyError(f"parameters missing from checkpoint: {missing[:5]}{'...' if len(missing) > 5 else ''}")


_ST_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
              "I64": torch.int64, "I32": torch.int32, "U8": torch.uint8, "BOOL": torch.bool}


def load_hf_weights(model, path: str, parallel_dims=None, split_group=None) -> None:
    """Fill ``model`` (already on its device, fused layout) from an HF safetensors folder.

    ``split_group`` (default: the replica's dp_shard group when it has more than one rank): its ranks need the same
    tensors (same tensor- and pipeline-parallel coordinates), so the checkpoint FILES are divided between them; the
    owner of a file reads a tensor's bytes and broadcasts them, the others only read the file's header for shape and
    dtype. An 8-rank replica then reads the checkpoint once instead of eight times
    (cosmos_rl/utils/multi_rank_weight_loader.py:34-300 splits and broadcasts the same way)."""
    from safetensors import safe_open
    cfg = load_hf_config(path)
    tp = parallel_dims.tp if parallel_dims is not None else 1
    r = parallel_dims.tp_coord if parallel_dims is not None else 0
    index = _index(path)
    handles: Dict[str, Any] = {}
    if split_group is None and parallel_dims is not None and os.environ.get("COSMOS_B200_SPLIT_LOAD", "1") != "0":
        split_group = parallel_dims.group("dp_shard")
    n_split = dist.get_world_size(split_group) if (split_group is not None and dist.is_initialized()) else 1
    me = dist.get_rank(split_group) if n_split > 1 else 0
    files = sorted(set(index.values()))
    owner = {fn: i % n_split for i, fn in enumerate(files)}
    dev = next(model.parameters()).device
    # NCCL moves device tensors, gloo host tensors
    on_dev = n_split > 1 and dev.type == "cuda" and dist.get_backend(split_group) != "gloo"
    stats = {"read_bytes": 0, "recv_bytes": 0}
    model._hf_load_stats = stats

    def handle(fn):
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), framework="pt")
        return handles[fn]

    def read(hf_name: str) -> torch.Tensor:
        fn = index[hf_name]
        if n_split == 1:
            return handle(fn).get_tensor(hf_name)
        src = owner[fn]
        if src == me:
            t = handle(fn).get_tensor(hf_name)
            stats["read_bytes"] += t.numel() * t.element_size()
            t = t.to(dev) if on_dev else t.contiguous()
        else:
            sl = handle(fn).get_slice(hf_name)                    # header only: no tensor bytes are read here
            t = torch.empty(sl.get_shape(), dtype=_ST_DTYPES[sl.get_dtype()], device=dev if on_dev else "cpu")
            stats["recv_bytes"] += t.numel() * t.element_size()
        dist.broadcast(t, dist.get_global_rank(split_group, src), group=split_group)
        return t

    load_hf_state(model, read, index, cfg, tp, r)


def hf_state_dict(model, hf_config: Dict[str, Any]) -> Dict[str, torch.Tensor]:
    """HF-named tensors of an unsharded (tp = 1) model: fused parameters are split back."""
    from .base import ModelRegistry
    mapper = ModelRegistry.mapper(hf_config.get("model_type"))(hf_config)
    mapper.layer_offset = getattr(model, "layer_offset", 0)
    mapper.layer_map = getattr(model, "layer_map", None)
    a = model.args
    out: Dict[str, torch.Tensor] = {}
    if hasattr(model, "export_items"):
        return {k: v.detach() for k, v in model.export_items()}
    for name, p in model.named_parameters():
        if ".lora_" in name:
            continue
        for hf_name, piece in _split_fused(name, p.detach(), mapper, hf_config, getattr(a, "n_heads", 0),
                                           getattr(a, "n_kv_heads", 0), getattr(a, "head_dim", 0)):
            out[hf_name] = piece
    return out


def _split_fused(name: str, t: torch.Tensor, mapper, cfg, hq: int, hkv: int, d: int) -> List[Tuple[str, torch.Tensor]]:
    hf_names = mapper.hf_names(name)
    if hasattr(mapper, "export_tensor"):
        t = mapper.export_tensor(name, t)            # layouts that differ from the checkpoint's (a flattened convolution)
    if len(hf_names) == 1:
        return [(hf_names[0], t)]
    if len(hf_names) == 3:   # q, k, v
        sizes = [hq * d, hkv * d, hkv * d]
    else:                    # gate, up
        sizes = [t.shape[0] // 2, t.shape[0] // 2]
    return list(zip(hf_names, t.split(sizes, dim=0)))


def export_safetensors(model, hf_config: Dict[str, Any], output_dir: str, parallel_dims=None,
                       source_dir: Optional[str] = None) -> None:
    """Write the model in HF layout. With TP every rank participates in gathers; rank 0 writes."""
    from safetensors.torch import save_file
    from .base import ModelRegistry
    mapper = ModelRegistry.mapper(hf_config.get("model_type"))(hf_config)
    mapper.layer_offset = getattr(model, "layer_offset", 0)
    mapper.layer_map = getattr(model, "layer_map", None)
    tp = parallel_dims.tp if parallel_dims is not None else 1
    rank = parallel_dims.global_rank if parallel_dims is not None else 0
    writer = rank == 0
    if writer:
        os.makedirs(output_dir, exist_ok=True)
    a = getattr(model, "args", None)
    hq = getattr(a, "n_heads", 0) // tp          # only families with fused q / k / v projections need these
    hkv = max(1, getattr(a, "n_kv_heads", 0) // tp)
    d = getattr(a, "head_dim", 0)
    shard: Dict[str, torch.Tensor] = {}
    shard_bytes = 0
    files: List[Dict[str, torch.Tensor]] = []
    weight_map: Dict[str, str] = {}
    total = 0

    def flush():
        nonlocal shard, shard_bytes
        if shard:
            files.append(shard)
            shard, shard_bytes = {}, 0

    export_items = model.export_items() if hasattr(model, "export_items") else None
    named = export_items if export_items is not None else list(model.named_parameters())
    for name, p in named:
        if ".lora_" in name:                   # adapters are exported separately (adapter_model.safetensors)
            continue
        t = p.detach()
        pieces = _split_fused(name, t, mapper, hf_config, hq, hkv, d) if export_items is None else [(name, t)]
        for hf_name, piece in pieces:
            if tp > 1:
                g = parallel_dims.group("tp")
                if piece.dim() == 2 or "bias" in hf_name:
                    parts = [torch.empty_like(piece) for _ in range(tp)]
                    dist.all_gather(parts, piece.contiguous(), group=g)
                    dim = 1 if any(s in hf_name for s in ("o_proj", "down_proj")) else 0
                    n_kv = hf_config.get("num_key_value_heads") or hf_config["num_attention_heads"]
                    if any(s in hf_name for s in ("k_proj", "v_proj")) and n_kv < tp:
                        parts = parts[:: tp // n_kv]
                    piece = torch.cat(parts, dim=dim)
            if not writer:
                continue
            cpu = piece.to("cpu", copy=True).contiguous()
            nbytes = cpu.numel() * cpu.element_size()
            if shard_bytes + nbytes > MAX_SHARD_BYTES:
                flush()
            shard[hf_name] = cpu
            shard_bytes += nbytes
            total += nbytes
    flush()
    if not writer:
        return
    for i, tensors in enumerate(files):
        fn = f"{i:05d}.safetensors"
        save_file(tensors, os.path.join(output_dir, fn), metadata={"format": "pt"})
        for k in tensors:
            weight_map[k] = fn
    with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    with open(os.path.join(output_dir, "config.json"), "w") as f:
        json.dump(hf_config, f, indent=2)
    with open(os.path.join(output_dir, "generation_config.json"), "w") as f:
        json.dump({"do_sample": True}, f)
    if source_dir and os.path.isdir(source_dir):
        for fn in os.listdir(source_dir):
            if fn.endswith((".py", ".json", ".txt", ".model", ".tiktoken")) and not fn.startswith("model") \
                    and fn not in ("config.json", "generation_config.json"):
                shutil.copy(os.path.join(source_dir, fn), os.path.join(output_dir, fn))
    logger.info("exported %d tensors (%.2f GB) to %s", len(weight_map), total / 1e9, output_dir)
