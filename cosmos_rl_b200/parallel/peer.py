"""Python side of the peer-memory runtime (``csrc/peer.cu``).

``PeerBuffer`` owns a ``cudaMalloc`` allocation that is exposed to PyTorch as a tensor (zero copy) and can
be exported as a 64-byte CUDA IPC handle; ``open_peer`` maps another process's buffer. The handles travel
through whatever control channel connects the processes (``torch.distributed`` object collectives inside one
launch, the controller's key/value store between replicas).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import native

_SIGS_DONE = False


def _lib():
    global _SIGS_DONE
    L = native.lib()
    if not _SIGS_DONE:
        vp = ctypes.c_void_p
        L.b200_peer_alloc.argtypes = [ctypes.POINTER(vp), ctypes.c_ulonglong]
        L.b200_peer_free.argtypes = [vp]
        L.b200_peer_export.argtypes = [vp, ctypes.c_char_p]
        L.b200_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.b200_peer_close.argtypes = [vp]
        L.b200_can_access_peer.argtypes = [ctypes.c_int, ctypes.c_int]
        L.b200_flag_set.argtypes = [vp, ctypes.c_uint32, vp]
        L.b200_flag_wait.argtypes = [vp, ctypes.c_uint32, vp, ctypes.c_ulonglong, vp]
        for n in ("b200_peer_alloc", "b200_peer_free", "b200_peer_export", "b200_peer_open", "b200_peer_close",
                  "b200_can_access_peer", "b200_flag_set", "b200_flag_wait"):
            getattr(L, n).restype = ctypes.c_int
        _SIGS_DONE = True
    return L


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` holder so torch can wrap a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
                                         "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, dtype: torch.dtype, device: torch.device, owner=None) -> torch.Tensor:
    raw = torch.as_tensor(_RawCuda(ptr, nbytes, owner), device=device)
    return raw.view(dtype)


class PeerBuffer:
    _live: List["PeerBuffer"] = []

    def __init__(self, nbytes: int, device: torch.device):
        self.device = device
        self.nbytes = int(nbytes)
        p = ctypes.c_void_p()
        with torch.cuda.device(device):
            native.check(_lib().b200_peer_alloc(ctypes.byref(p), self.nbytes), "peer_alloc")
        self.ptr = p.value
        PeerBuffer._live.append(self)

    def tensor(self, dtype: torch.dtype) -> torch.Tensor:
        return tensor_from_ptr(self.ptr, self.nbytes, dtype, self.device, owner=self)

    def export(self) -> bytes:
        buf = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            native.check(_lib().b200_peer_export(self.ptr, buf), "peer_export")
        return buf.raw

    def free(self) -> None:
        if self.ptr:
            _lib().b200_peer_free(self.ptr)
            self.ptr = 0
            if self in PeerBuffer._live:
                PeerBuffer._live.remove(self)


def peer_allocator(device: torch.device):
    """An allocator for :class:`FlatParams` that places the buffer in exportable memory."""
    bufs: List[PeerBuffer] = []

    def alloc(n: int, dtype: torch.dtype, dev: torch.device) -> torch.Tensor:
        b = PeerBuffer(n * torch.empty((), dtype=dtype).element_size(), dev)
        bufs.append(b)
        t = b.tensor(dtype)
        t._peer_buffer = b
        return t

    alloc.buffers = bufs
    return alloc


class PeerMapping:
    """A remote buffer mapped into this process."""

    def __init__(self, handle: bytes, nbytes: int, device: torch.device):
        p = ctypes.c_void_p()
        with torch.cuda.device(device):
            native.check(_lib().b200_peer_open(handle, ctypes.byref(p)), "peer_open")
        self.ptr = p.value
        self.nbytes = nbytes
        self.device = device

    def tensor(self, dtype: torch.dtype) -> torch.Tensor:
        return tensor_from_ptr(self.ptr, self.nbytes, dtype, self.device, owner=self)

    def close(self) -> None:
        if self.ptr:
            _lib().b200_peer_close(self.ptr)
            self.ptr = 0


def flag_set(flag: torch.Tensor, value: int) -> None:
    native.check(_lib().b200_flag_set(flag.data_ptr(), value & 0xFFFFFFFF, native.stream()), "flag_set")


def flag_wait(flag_ptr: int, value: int, device: torch.device, limit_s: float = 2.0) -> None:
    st = native.status_word(device)
    native.check(_lib().b200_flag_wait(flag_ptr, value & 0xFFFFFFFF, st.data_ptr(), int(limit_s * 1e9),
                                       native.stream()), "flag_wait")
