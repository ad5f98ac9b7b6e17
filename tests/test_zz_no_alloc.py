"""The entry point that allocates nothing (turingserve_b200/csrc/no_alloc.h), called through its
exported C symbol the way a user without an allocator would: plain pointers in, result out.

Some callers of this library cannot allocate device memory at the moment they call it (a thread
inside a stream capture, a process with a fixed, policed memory budget).  For them
``ts_attention_decode_static`` keeps the split-key scratch in an array inside the library.  The
test checks it against the ordinary entry point, which takes its scratch from the caller, and
against a plain 32-bit attention over the same pages, on two calls in a row that share the array;
it checks that the device's free memory is the same before and after a call (what the driver
reports, so an allocation inside the library would show), and that a shape whose scratch would
not fit is refused instead of overrunning it.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, ctx, H=12, KVH=2, D=128, page=16):
    g = torch.Generator().manual_seed(seed)
    lens = [max(1, ctx - 37 * i) for i in range(B)]
    n_pages = [-(-l // page) for l in lens]
    total = sum(n_pages) + 1
    ids = (torch.randperm(total - 1, generator=g) + 1).tolist()
    bt = torch.zeros((B, max(n_pages)), dtype=torch.int32)
    for b in range(B):
        bt[b, : n_pages[b]] = torch.tensor([ids.pop() for _ in range(n_pages[b])], dtype=torch.int32)
    kc = torch.randn((total, KVH, page, D), generator=g).to(torch.bfloat16)
    vc = torch.randn((total, KVH, page, D), generator=g).to(torch.bfloat16)
    qkv = torch.randn((B, (H + 2 * KVH) * D), generator=g).to(torch.bfloat16)
    qs = torch.arange(B + 1, dtype=torch.int32)
    sl = torch.tensor(lens, dtype=torch.int32)
    return [t.cuda() for t in (qkv, kc, vc, bt, qs, sl)], (B, H, KVH, D, page)


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from turingserve_b200 import kernels
    kernels.use(None)
    ops = kernels.ops()
    lib = ctypes.CDLL(ops.lib_path)                      # the exported C symbol, no Python wrapper around it
    fn = lib.ts_attention_decode_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    lib.ts_last_error.restype = ctypes.c_char_p
    ref_fn = lib.ts_attention_decode
    ref_fn.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P]
    ref_fn.restype = I
    stream = torch.cuda.current_stream().cuda_stream
    scale = 128 ** -0.5
    from tests.twin_ops import paged_attention
    for call, (seed, B, ctx, nsplit, window) in enumerate(((1, 8, 2049, 16, 0), (2, 3, 700, 5, 300))):   # two calls in a row
        (qkv, kc, vc, bt, qs, sl), (B, H, KVH, D, page) = _case(seed, B, ctx)
        plain32 = torch.empty((B, H * D), dtype=torch.float32, device="cuda")
        paged_attention(plain32, qkv, kc, vc, bt, qs, sl, H, KVH, D, page, scale, window or None)
        want = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(B * H * nsplit * (D + 2), dtype=torch.float32, device="cuda")
        counters = torch.zeros(B * KVH, dtype=torch.int32, device="cuda")
        rc = ref_fn(want.data_ptr(), scratch.data_ptr(), counters.data_ptr(), qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                    bt.data_ptr(), qs.data_ptr(), sl.data_ptr(), B, bt.shape[1], H, KVH, D, page, scale, window, nsplit, stream)
        assert rc == 0, lib.ts_last_error()
        got = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]           # the driver's count: sees any allocation, not only torch's
        rc = fn(got.data_ptr(), qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), qs.data_ptr(), sl.data_ptr(),
                B, bt.shape[1], H, KVH, D, page, scale, window, nsplit, stream)
        assert rc == 0, lib.ts_last_error()
        torch.cuda.synchronize()
        if call > 0:                                         # the first call on a device may load the module's image
            assert torch.cuda.mem_get_info()[0] == free_before
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), atol=1e-2, rtol=1e-2)      # the attention tests' bound
        torch.testing.assert_close(got.float(), plain32, atol=1e-2, rtol=1e-2)
    # a shape whose scratch would not fit the fixed array is refused, nothing runs
    (qkv, kc, vc, bt, qs, sl), (B, H, KVH, D, page) = _case(3, 64, 300)
    out = torch.zeros((B, H * D), dtype=torch.bfloat16, device="cuda")
    rc = fn(out.data_ptr(), qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), qs.data_ptr(), sl.data_ptr(),
            B, bt.shape[1], H, KVH, D, page, scale, 0, 64, stream)
    assert rc < 0 and b"fixed array" in lib.ts_last_error()
    torch.cuda.synchronize()
    assert torch.all(out == 0)
