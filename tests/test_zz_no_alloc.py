"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call it: a serving host that handed the
whole GPU to weights and KV cache at start-up, or a C caller without a device allocator. For them
``b200_paged_decode_static`` keeps the split-merge scratch inside the library. This test loads the shared
library with ctypes (not through the package's wrappers), runs the regular entry point with a scratch buffer
from torch and the static one without, and requires the same result on two calls in a row with different
inputs (the second call finds the first call's leftovers in the shared array). The file name sorts last so a
run that stops at the first failure has already executed every other test.
"""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cosmos_rl_b200", "ops",
                   "libb200rl.so")


@pytest.fixture(scope="module", autouse=True)
def _built_library():
    """Build the shared library when this file runs alone on a fresh tree (the object files are not tracked); the
    symbol is still reached through ctypes below, not through the package's wrappers."""
    from cosmos_rl_b200.ops import build
    path = build.build()
    assert os.path.samefile(path, LIB)


def _load():
    lib = ctypes.CDLL(LIB)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.b200_paged_decode.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, vp]
    lib.b200_paged_decode.restype = i
    lib.b200_paged_decode_static.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, vp]
    lib.b200_paged_decode_static.restype = i
    return lib


def _case(seed, B, hq, hkv, d, page_size, n_pages, max_pages):
    g = torch.Generator(device="cuda").manual_seed(seed)
    cache = torch.randn(n_pages, 2, hkv, page_size, d, device="cuda", generator=g).to(torch.bfloat16)
    q = torch.randn(B, hq, d, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.stack([torch.randperm(n_pages, device="cuda", generator=g)[:max_pages] for _ in range(B)]).to(torch.int32)
    lens = torch.randint(1, max_pages * page_size, (B,), device="cuda", generator=g).to(torch.int32)
    return q, cache, table.contiguous(), lens


def test_static_scratch_entry_matches_regular_entry_twice():
    assert os.path.exists(LIB), "libb200rl.so has not been built"
    lib = _load()
    stream = torch.cuda.current_stream().cuda_stream
    B, hq, hkv, d, P, n_pages, max_pages, nsplit = 6, 28, 4, 128, 16, 96, 12, 4
    for call, seed in enumerate((11, 12)):
        q, cache, table, lens = _case(seed, B, hq, hkv, d, P, n_pages, max_pages)
        scale = 1.0 / math.sqrt(d)
        ref = torch.empty_like(q)
        scratch = torch.empty(B * hq * nsplit * (d + 2), dtype=torch.float32, device="cuda")
        rc = lib.b200_paged_decode(q.data_ptr(), cache.data_ptr(), table.data_ptr(), lens.data_ptr(), ref.data_ptr(),
                                   scratch.data_ptr(), B, hq, hkv, d, P, max_pages, nsplit, scale, stream)
        assert rc == 0
        out = torch.full_like(q, float("nan"))
        rc = lib.b200_paged_decode_static(q.data_ptr(), cache.data_ptr(), table.data_ptr(), lens.data_ptr(),
                                          out.data_ptr(), B, hq, hkv, d, P, max_pages, nsplit, scale, stream)
        assert rc == 0, f"call {call}: rc={rc}"
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2), f"call {call}"


def test_static_scratch_entry_rejects_oversize():
    lib = _load()
    # 4096 * 64 * 16 * 130 floats is far beyond the 4 Mi float array: refused before anything is launched
    rc = lib.b200_paged_decode_static(None, None, None, None, None, 4096, 64, 8, 128, 16, 4, 16, 1.0, None)
    assert rc == -4
