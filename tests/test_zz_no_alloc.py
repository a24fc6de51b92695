"""The allocation-free MLA decode entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it: their memory pool belongs to
another runtime and is fully handed out at start-up, or they run on a latency-critical thread that must never
block on the driver's allocator.  ``omni_mla_decode_noalloc`` serves them by keeping the split-KV scratch in a
fixed array inside the library.  The test checks it against the regular entry point (caller-provided scratch)
on two consecutive calls, which also shows that leftovers of the first call in the shared array do no harm.
This file sorts last on purpose, so a run that stops at the first failure has already run every other test."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, cache2, bt, sl, H, bs, scale, splits, out, status):
    fn = lib.omni_mla_decode_noalloc
    fn.restype = ctypes.c_int
    return fn(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(cache2.data_ptr()), ctypes.c_int(cache2.stride(0)),
              ctypes.c_longlong(cache2.shape[0]), ctypes.c_void_p(bt.data_ptr()), ctypes.c_int(bt.stride(0)),
              ctypes.c_void_p(sl.data_ptr()), ctypes.c_void_p(0), ctypes.c_int(q.shape[0]), ctypes.c_int(H),
              ctypes.c_int(bs), ctypes.c_float(scale), ctypes.c_int(splits), ctypes.c_void_p(out.data_ptr()),
              ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_matches_regular_entry_point_twice():
    from omni_infer_b200.ops import _native as nat
    from omni_infer_b200.ops import attention as A

    lib = ctypes.CDLL(str(nat.lib_path()))          # the exported C symbol, not the Python wrapper
    torch.manual_seed(0)
    dev = "cuda"
    H, bs, scale = 128, 128, 1.0 / math.sqrt(192)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    for call, (lens, splits) in enumerate([([700, 300, 1], 4), ([129, 1024], 3)]):
        Bq = len(lens)
        max_blocks = (max(lens) + bs - 1) // bs + 1
        nb = Bq * max_blocks + 1
        cache = (torch.randn(nb, bs, 576, device=dev) * 0.5).bfloat16()
        bt = (torch.randperm(nb - 1, device=dev)[: Bq * max_blocks].int() + 1).view(Bq, max_blocks).contiguous()
        q = (torch.randn(Bq, H, 576, device=dev) * 0.5).bfloat16()
        sl = torch.tensor(lens, dtype=torch.int32, device=dev)
        want = A.mla_decode(q, cache, bt, sl, scale, num_splits=splits)      # regular path, caller scratch
        got = torch.empty(Bq, H, 512, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        rc = _call_noalloc(lib, q, cache.view(-1, 576), bt, sl, H, bs, scale, splits, got, status)
        assert rc == 0, f"call {call}: rc={rc}"
        torch.cuda.synchronize()
        # the property in the name: neither the driver nor torch's pool handed out memory for the call
        # (the very first call may still load the module lazily, so only the second one is held to it)
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_reserved() == reserved_before
        assert status.tolist()[0] == 0
        torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=2e-2)
        ref = A.mla_decode_ref(q, cache, bt, sl, scale)
        torch.testing.assert_close(got.float(), ref.float(), rtol=3e-2, atol=2e-2)


def test_noalloc_rejects_oversized_problem():
    from omni_infer_b200.ops import _native as nat

    lib = ctypes.CDLL(str(nat.lib_path()))
    dev = "cuda"
    q = torch.zeros(128, 128, 576, dtype=torch.bfloat16, device=dev)      # 128 * 8 * 128 parts > limit
    cache = torch.zeros(2, 128, 576, dtype=torch.bfloat16, device=dev)
    bt = torch.zeros(128, 2, dtype=torch.int32, device=dev)
    sl = torch.zeros(128, dtype=torch.int32, device=dev)
    out = torch.empty(128, 128, 512, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = _call_noalloc(lib, q, cache.view(-1, 576), bt, sl, 128, 128, 0.1, 8, out, status)
    assert rc == -100


def test_noalloc_single_split_has_no_size_limit():
    """One split never touches the built-in scratch, so a batch far above the split-KV limit is accepted."""
    from omni_infer_b200.ops import _native as nat
    from omni_infer_b200.ops import attention as A

    lib = ctypes.CDLL(str(nat.lib_path()))
    torch.manual_seed(1)
    dev = "cuda"
    Bq, H, bs, scale = 96, 128, 128, 1.0 / math.sqrt(192)      # 96 * 128 = 12288 parts > 8192
    cache = (torch.randn(Bq + 1, bs, 576, device=dev) * 0.5).bfloat16()
    bt = (torch.arange(Bq, device=dev, dtype=torch.int32) + 1).view(Bq, 1).contiguous()
    q = (torch.randn(Bq, H, 576, device=dev) * 0.5).bfloat16()
    sl = torch.full((Bq,), 100, dtype=torch.int32, device=dev)
    out = torch.empty(Bq, H, 512, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = _call_noalloc(lib, q, cache.view(-1, 576), bt, sl, H, bs, scale, 1, out, status)
    assert rc == 0
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    ref = A.mla_decode_ref(q, cache, bt, sl, scale)
    torch.testing.assert_close(out.float(), ref.float(), rtol=3e-2, atol=2e-2)
