"""Resharding planner for policy -> rollout weight synchronisation.

Each rank of each side describes what it holds as a list of *parts*: a rectangle ``[r0, r1) x [c0, c1)`` of a
globally named 2-D tensor (HF-level name; 1-D tensors are ``1 x n``), plus where that rectangle lives inside
the rank's flat parameter buffer (element offset and leading dimension). Fused parameters (qkv, gate_up)
simply contribute several parts. The plan for a destination rank is the list of rectangle copies
``(src rank, src offset, src ld) -> (dst offset, dst ld, rows, cols)`` obtained by intersecting its parts with
the source parts of the same name; identical source rectangles held by several ranks (data-parallel copies,
replicated KV heads) are used round-robin so every source GPU's NVLink egress is loaded equally.

This is the information the reference keeps in ``DimSliceInfo`` and ``ParallelizedShardMapper``
(cosmos_rl/utils/dim_slice_info.py:29-383, cosmos_rl/utils/parallelism_map.py:126-1535), reduced to
rectangle intersection, and emitted as a flat copy-descriptor table for ONE pull kernel instead of
per-tensor send/recv instruction lists.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple


@dataclass
class Part:
    key: str           # global tensor name
    r0: int
    r1: int
    c0: int
    c1: int
    off: int           # element offset of (r0, c0) inside the rank's flat buffer
    ld: int            # elements between consecutive rows in the local storage
    trainable: bool = True

    def to_list(self) -> list:
        return [self.key, self.r0, self.r1, self.c0, self.c1, self.off, self.ld, int(self.trainable)]

    @staticmethod
    def from_list(x: Sequence) -> "Part":
        return Part(x[0], x[1], x[2], x[3], x[4], x[5], x[6], bool(x[7]))


def shard_info(rank: int, parts: List[Part], total_elems: int, extra: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    d = {"rank": rank, "total": total_elems, "parts": [p.to_list() for p in parts]}
    if extra:
        d.update(extra)
    return d


def _slice(n: int, world: int, rank: int) -> Tuple[int, int]:
    per = n // world
    return rank * per, (rank + 1) * per


def gpt_parts(model, flat) -> List[Part]:
    """Parts of a dense decoder (:class:`cosmos_rl_b200.models.gpt.GPT`) given its flat storage."""
    a = model.args
    tp, r = a.tp_size, a.tp_rank
    d = a.head_dim
    Hq, Hkv = a.n_heads, a.n_kv_heads
    hq = Hq // tp
    kv_rep = max(1, tp // Hkv)          # ranks sharing one KV head when tp > n_kv
    hkv = max(1, Hkv // tp)
    kv_lo = (r // kv_rep) * hkv if tp > Hkv else r * hkv
    I = a.ffn_dim
    il0, il1 = _slice(I, tp, r)
    parts: List[Part] = []
    from ..models.base import ModelRegistry
    mapper = ModelRegistry.mapper(a.model_type)({"model_type": a.model_type})
    mapper.layer_offset = getattr(model, "layer_offset", 0)
    mapper.layer_map = getattr(model, "layer_map", None)

    def add(key, r0, r1, c0, c1, slot_off, row_in_local, col_in_local, ld, trainable):
        parts.append(Part(key, r0, r1, c0, c1, slot_off + row_in_local * ld + col_in_local, ld, trainable))

    for name, p in flat.params:
        slot = flat.by_name[name]
        tr = bool(p.requires_grad)
        hf = mapper.hf_names(name)
        if p.dim() == 1:
            n = p.shape[0]
            if "qkv_proj.bias" in name:
                add(hf[0], 0, 1, r * hq * d, (r + 1) * hq * d, slot.offset, 0, 0, n, tr)
                add(hf[1], 0, 1, kv_lo * d, (kv_lo + hkv) * d, slot.offset, 0, hq * d, n, tr)
                add(hf[2], 0, 1, kv_lo * d, (kv_lo + hkv) * d, slot.offset, 0, (hq + hkv) * d, n, tr)
            else:
                add(hf[0], 0, 1, 0, n, slot.offset, 0, 0, n, tr)
            continue
        rows, cols = p.shape
        if "qkv_proj.weight" in name:
            add(hf[0], r * hq * d, (r + 1) * hq * d, 0, cols, slot.offset, 0, 0, cols, tr)
            add(hf[1], kv_lo * d, (kv_lo + hkv) * d, 0, cols, slot.offset, hq * d, 0, cols, tr)
            add(hf[2], kv_lo * d, (kv_lo + hkv) * d, 0, cols, slot.offset, (hq + hkv) * d, 0, cols, tr)
        elif "gate_up_proj.weight" in name:
            il = rows // 2                 # local rows of each half (dense FFN, or the shared experts of an MoE block)
            add(hf[0], r * il, (r + 1) * il, 0, cols, slot.offset, 0, 0, cols, tr)
            add(hf[1], r * il, (r + 1) * il, 0, cols, slot.offset, il, 0, cols, tr)
        elif "o_proj.weight" in name:
            add(hf[0], 0, rows, r * hq * d, (r + 1) * hq * d, slot.offset, 0, 0, cols, tr)
        elif "down_proj.weight" in name:
            add(hf[0], 0, rows, r * cols, (r + 1) * cols, slot.offset, 0, 0, cols, tr)
        elif "embed_tokens" in name or "lm_head" in name:
            v0 = r * rows if tp > 1 else 0
            add(hf[0], v0, v0 + rows, 0, cols, slot.offset, 0, 0, cols, tr)
        else:
            add(hf[0], 0, rows, 0, cols, slot.offset, 0, 0, cols, tr)
    return parts


def whole_parts(flat, prefix: str = "") -> List[Part]:
    """Every parameter as one whole part under its own name: models that run data parallel only (diffusion
    transformers, action experts) have the same layout on the policy and the rollout side."""
    parts: List[Part] = []
    for name, p in flat.params:
        slot = flat.by_name[name]
        rows, cols = (1, p.numel()) if p.dim() <= 1 else (p.shape[0], p.numel() // p.shape[0])
        parts.append(Part(prefix + name, 0, rows, 0, cols, slot.offset, cols, bool(p.requires_grad)))
    return parts


def model_parts(model, flat) -> List[Part]:
    if hasattr(model, "shard_parts"):
        return model.shard_parts(flat)
    return gpt_parts(model, flat)


# ---------------------------------------------------------------------------------------------------
def build_plan(src_infos: List[Dict[str, Any]], dst_info: Dict[str, Any], trainable_only: bool = False
               ) -> List[List[int]]:
    """Copy descriptors for one destination rank:
    ``[src_rank, src_off, src_ld, dst_off, dst_ld, rows, cols]`` (offsets in elements)."""
    by_key: Dict[str, List[Tuple[int, Part]]] = {}
    for info in src_infos:
        for raw in info["parts"]:
            p = Part.from_list(raw)
            by_key.setdefault(p.key, []).append((info["rank"], p))
    load: Dict[int, int] = {}
    plan: List[List[int]] = []
    for raw in dst_info["parts"]:
        dp = Part.from_list(raw)
        if trainable_only and not dp.trainable:
            continue
        cands = by_key.get(dp.key)
        if not cands:
            raise KeyError(f"destination part {dp.key!r} has no source")
        # group identical source rectangles (duplicates across data-parallel ranks / replicated heads)
        groups: Dict[Tuple[int, int, int, int], List[Tuple[int, Part]]] = {}
        for rank, sp in cands:
            groups.setdefault((sp.r0, sp.r1, sp.c0, sp.c1), []).append((rank, sp))
        covered = 0
        for box, members in sorted(groups.items()):
            r0, r1 = max(dp.r0, box[0]), min(dp.r1, box[1])
            c0, c1 = max(dp.c0, box[2]), min(dp.c1, box[3])
            if r0 >= r1 or c0 >= c1:
                continue
            # least-loaded holder of this rectangle (ties broken starting at the destination's own rank)
            nm = len(members)
            rank, sp = min(members, key=lambda m: (load.get(m[0], 0), (m[0] - dst_info["rank"]) % max(nm, 1)))
            load[rank] = load.get(rank, 0) + (r1 - r0) * (c1 - c0)
            plan.append([rank, sp.off + (r0 - sp.r0) * sp.ld + (c0 - sp.c0), sp.ld,
                         dp.off + (r0 - dp.r0) * dp.ld + (c0 - dp.c0), dp.ld, r1 - r0, c1 - c0])
            covered += (r1 - r0) * (c1 - c0)
        want = (dp.r1 - dp.r0) * (dp.c1 - dp.c0)
        if covered != want:
            raise ValueError(f"part {dp.key!r} of rank {dst_info['rank']}: sources cover {covered} of {want} elements")
    return plan


def plan_for_rank(policy_infos: Optional[Dict[str, Any]], rollout_infos: Optional[Dict[str, Any]], role: str,
                  rank: int, trainable_only: bool = False):
    """Controller-side entry: the receive plan of a rollout rank, or for a policy rank the list of
    ``[dst_rank, descriptor]`` pairs in which it is the source (used by the send/recv transports)."""
    if not policy_infos or not rollout_infos:
        return []
    src, dst = policy_infos["ranks"], rollout_infos["ranks"]
    if role == "rollout":
        info = next(i for i in dst if i["rank"] == rank)
        return build_plan(src, info, trainable_only)
    out = []
    for info in dst:
        for desc in build_plan(src, info, trainable_only):
            if desc[0] == rank:
                out.append([info["rank"], desc])
    return out


def merge_descriptors(plan: List[List[int]]) -> List[List[int]]:
    """Fuse vertically adjacent rectangles of the same source with equal geometry (fewer, larger copies)."""
    out: List[List[int]] = []
    for d in sorted(plan, key=lambda x: (x[0], x[1])):
        if out:
            p = out[-1]
            if (p[0] == d[0] and p[2] == d[2] and p[4] == d[4] and p[6] == d[6]
                    and p[1] + p[5] * p[2] == d[1] and p[3] + p[5] * p[4] == d[3]):
                p[5] += d[5]
                continue
        out.append(list(d))
    return out


def interleave_sources(plan: List[List[int]], first: int = 0) -> List[List[int]]:
    """Order descriptors so that a pull draws on every source at once: the lists of the sources are merged by the
    fraction of each source's bytes already scheduled, starting with the ``first``-th source (callers pass the
    destination's rank so that two destinations do not start on the same source). A plan sorted by source makes every
    puller read one source at a time, and pullers that share a source then share its outgoing link."""
    by_src: Dict[int, List[List[int]]] = {}
    for d in plan:
        by_src.setdefault(d[0], []).append(d)
    srcs = sorted(by_src)
    if len(srcs) <= 1:
        return list(plan)
    srcs = srcs[first % len(srcs):] + srcs[:first % len(srcs)]
    total = {r: float(sum(d[5] * d[6] for d in by_src[r])) or 1.0 for r in srcs}
    done = {r: 0.0 for r in srcs}
    pos = {r: 0 for r in srcs}
    out: List[List[int]] = []
    while len(out) < len(plan):
        r = min((r for r in srcs if pos[r] < len(by_src[r])), key=lambda r: (done[r] / total[r], srcs.index(r)))
        d = by_src[r][pos[r]]
        pos[r] += 1
        done[r] += d[5] * d[6]
        out.append(d)
    return out
