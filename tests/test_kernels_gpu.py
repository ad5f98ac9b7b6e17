"""Each CUDA kernel alone against its plain torch twin, at sizes other than the engine's test
models (shape grids after the reference's tests/kernels/test_kernels.py:22-154)."""

from __future__ import annotations

import dataclasses
import math

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests.twin_ops import TwinOps, paged_attention

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
DEFAULT_GEMM = "auto"
TOL = {torch.float32: dict(atol=2e-5, rtol=2e-5), torch.bfloat16: dict(atol=2e-2, rtol=2e-2)}


@pytest.fixture(scope="module")
def ops():
    from turingserve_b200 import kernels
    kernels.use(None)
    return kernels.ops()


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@dataclasses.dataclass
class FakeStep:
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    num_requests: int
    max_q_len: int
    max_seq_len: int
    num_decode: int = 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    for V, h in [(50, 64), (301, 80), (1000, 1536), (77, 30)]:
        table = _rand((V, h), dtype, 1)
        ids = torch.randint(0, V, (23,), dtype=torch.int32)
        out = torch.empty((23, h), dtype=dtype, device="cuda")
        ops.embedding(out, table.cuda(), ids.cuda())
        assert torch.equal(out.cpu(), table[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 7, 130])
@pytest.mark.parametrize("N", [64, 224, 1000, 1536, 4100])
def test_rmsnorm(ops, dtype, T, N):
    twin = TwinOps()
    x, r, w = _rand((T, N), dtype, 2), _rand((T, N), dtype, 3), (1 + 0.1 * _rand((N,), torch.float32, 4)).to(dtype)
    for eps in (1e-6, 1e-3):
        out = torch.empty((T, N), dtype=dtype, device="cuda")
        ops.rmsnorm(out, x.cuda(), w.cuda(), eps)
        ref = torch.empty_like(x)
        twin.rmsnorm(ref, x, w, eps)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **TOL[dtype])
        res = r.clone().cuda()
        ops.rmsnorm(out, x.cuda(), w.cuda(), eps, res)
        rref = r.clone()
        twin.rmsnorm(ref, x, w, eps, rref)
        assert torch.equal(res.cpu(), rref), "residual sum is a single rounding: must be exact"
        torch.testing.assert_close(out.cpu().float(), ref.float(), **TOL[dtype])
    if dtype == torch.bfloat16:                      # a scale stored in 32-bit stays 32-bit
        w32 = 1 + 0.1 * _rand((N,), torch.float32, 5)
        out = torch.empty((T, N), dtype=dtype, device="cuda")
        ops.rmsnorm(out, x.cuda(), w32.cuda(), 1e-6)
        ref = torch.empty_like(x)
        twin.rmsnorm(ref, x, w32, 1e-6)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    twin = TwinOps()
    for T, inter in [(1, 128), (33, 4864), (5, 1001), (2048, 96)]:
        gu = _rand((T, 2 * inter), dtype, 6, 3.0)
        out = torch.empty((T, inter), dtype=dtype, device="cuda")
        ops.silu_mul(out, gu.cuda())
        ref = torch.empty((T, inter), dtype=dtype)
        twin.silu_mul(ref, gu)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **TOL[dtype])
    for T, inter, group in [(3, 128, 64), (70, 8960, 64), (9, 96, 8), (5, 1024, 64)]:    # interleaved blocks
        gu = _rand((T, 2 * inter), dtype, 16, 3.0)
        out = torch.empty((T, inter), dtype=dtype, device="cuda")
        ops.silu_mul(out, gu.cuda(), group)
        ref = torch.empty((T, inter), dtype=dtype)
        twin.silu_mul(ref, gu, group)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 8, 17, 40, 100, 128, 300])
@pytest.mark.parametrize("inter,K,group", [(128, 64, 64), (8960, 1536, 64), (320, 200, 64), (96, 72, 0)])
def test_gated_linear(ops, monkeypatch, dtype, T, inter, K, group):
    """Gate/up product and activation as one operation: for a few bfloat16 tokens one kernel with
    the activation in its epilogue, otherwise product then activation; either way the result is
    that of the two steps with the product rounded to the model dtype in between."""
    twin = TwinOps()
    x, w = _rand((T, K), dtype, 30, 1.0), _rand((2 * inter, K), dtype, 31, 0.1)
    out = torch.full((T, inter), float("nan"), dtype=dtype, device="cuda")
    separate = []
    monkeypatch.setattr(ops, "silu_mul", lambda *a, _f=ops.silu_mul: (separate.append(1), _f(*a))[1])
    monkeypatch.setattr(ops, "fused_gate_tokens", 128)            # everything the fused kernel takes
    ops.gated_linear(out, x.cuda(), w.cuda(), None, group)
    # (more tokens than the few-token kernel takes: the kernel for pairs of SMs, where its schedule is the shorter)
    fused = dtype == torch.bfloat16 and group == 64 and (T <= 128 or ops.pair_wins(T, 2 * inter, K, 6.0 * T * inter))
    assert (not separate) == fused, "no activation kernel of its own exactly when a fused epilogue applies"
    monkeypatch.undo()
    ref = torch.empty((T, inter), dtype=dtype)
    twin.gated_linear(ref, x, w, None, group)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)       # as test_linear
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol)
    if fused and T <= 128 and ops.tc_splits(T, 2 * inter, K) == 1:       # same sums, same roundings: the same bits
        two = torch.empty((T, inter), dtype=dtype, device="cuda")
        gu = torch.empty((T, 2 * inter), dtype=dtype, device="cuda")
        ops.linear(gu, x.cuda(), w.cuda(), None)
        ops.silu_mul(two, gu, group)
        assert torch.equal(out, two)
    assert ops.tc_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KVH,D,rot", [(4, 2, 16, 16), (14, 2, 64, 64), (12, 2, 128, 128), (5, 5, 48, 48),
                                         (6, 3, 32, 16), (2, 1, 80, 0)])
@pytest.mark.parametrize("T", [37, 150])          # a few tokens: a warp per head; many: several heads per warp
def test_rope_kv_write(ops, dtype, H, KVH, D, rot, T):
    twin = TwinOps()
    page, pages = 8, 24
    qkv = _rand((T, (H + 2 * KVH) * D), dtype, 7)
    pos = torch.randint(0, 500, (T,), dtype=torch.int32)
    cos, sin = plain.rope_tables(max(rot, 2), 10000.0, 500)
    perm = torch.randperm(page * (pages - 1))[:T].to(torch.int32) + page
    slots = perm.clone()
    slots[5] = -1
    slots[20] = -1
    kc = _rand((pages, KVH, page, D), dtype, 8)
    vc = _rand((pages, KVH, page, D), dtype, 9)
    q_d, kc_d, vc_d = qkv.clone().cuda(), kc.clone().cuda(), vc.clone().cuda()
    ops.rope_kv_write(q_d, pos.cuda(), cos.cuda() if rot else None, sin.cuda() if rot else None, H, KVH, D, rot,
                      kc_d, vc_d, slots.cuda(), page)
    q_r, kc_r, vc_r = qkv.clone(), kc.clone(), vc.clone()
    twin.rope_kv_write(q_r, pos, cos, sin, H, KVH, D, rot, kc_r, vc_r, slots, page)
    tol = dict(atol=1e-6, rtol=1e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(q_d.cpu().float(), q_r.float(), **tol)
    torch.testing.assert_close(kc_d.cpu().float(), kc_r.float(), **tol)
    assert torch.equal(vc_d.cpu(), vc_r), "values are copied, not computed"
    # rotate only (a run that reads another run's cache)
    q_d2 = qkv.clone().cuda()
    ops.rope_kv_write(q_d2, pos.cuda(), cos.cuda() if rot else None, sin.cuda() if rot else None, H, KVH, D, rot,
                      None, None, slots.cuda(), page)
    torch.testing.assert_close(q_d2.cpu().float(), q_r.float(), **tol)


@pytest.mark.parametrize("T", [1, 3, 8, 16, 40, 128])
@pytest.mark.parametrize("H,KVH,K,bias,D", [(12, 2, 1536, True, 128), (4, 2, 192, True, 128), (5, 1, 200, False, 128),
                                            (28, 4, 3584, True, 128), (14, 2, 896, True, 64), (5, 1, 200, False, 64),
                                            (3, 3, 320, True, 64)])
def test_qkv_product_that_rotates_and_writes_the_cache_itself(ops, monkeypatch, T, H, KVH, K, bias, D):
    """The q/k/v product of a few tokens with heads of 128 or 64 finishes itself (split sums, bias,
    rotation, cache write in its epilogue): bit for bit what the product followed by the rotary
    kernel gives, in the q/k/v tensor and in the cache pages.  With heads of 64 a tile of 128 weight
    rows is two heads, and an odd number of heads leaves the last tile half empty."""
    page, pages = 16, 40
    N = (H + 2 * KVH) * D
    x = _rand((T, K), torch.bfloat16, 50, 1.0).cuda()
    w = _rand((N, K), torch.bfloat16, 51, 0.05).cuda()
    b = _rand((N,), torch.bfloat16, 52, 0.5).cuda() if bias else None
    pos = torch.randint(0, 600, (T,), dtype=torch.int32)
    cos, sin = plain.rope_tables(D, 1e6, 600)
    slots = (torch.randperm(page * (pages - 1))[:T].to(torch.int32) + page)
    if T > 2:
        slots[1] = -1
    kc0, vc0 = _rand((pages, KVH, page, D), torch.bfloat16, 53), _rand((pages, KVH, page, D), torch.bfloat16, 54)
    got = {}
    monkeypatch.setattr(ops, "pair_wins", lambda *a: False)       # (the many-row kernel has a test of its own)
    # fused with its splits as one thread-block cluster (where the split count allows), fused with
    # scratch and a ticket counter, and product and rotary kernel apart
    for fused, clusters in ((True, 1), ("ticket", 0), (False, 1)):
        monkeypatch.setattr(ops, "fused_qkv_tokens", 128 if fused else 0)
        ops.lib.ts_set_clusters(clusters)
        try:
            kc, vc = kc0.clone().cuda(), vc0.clone().cuda()
            out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            launches = ops.launches
            for _ in range(2):                                     # twice: the counters come back to zero
                q = ops.qkv_rope(out, x, w, b, pos.cuda(), cos.cuda(), sin.cuda(), H, KVH, D, D, kc, vc, slots.cuda(),
                                 page)
        finally:
            ops.lib.ts_set_clusters(1)
        if T <= 32:                                                 # above, one kernel only where the splits can be clusters
            assert (ops.launches - launches == 2) == bool(fused)
        got[fused] = (q.clone(), kc, vc)
    for other in ("ticket", False):
        for a, c in zip(got[True], got[other]):
            assert torch.equal(a, c)
    # rotate only (a run that reads another run's cache): no cache write
    monkeypatch.setattr(ops, "fused_qkv_tokens", 128)
    out = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
    q = ops.qkv_rope(out, x, w, b, pos.cuda(), cos.cuda(), sin.cuda(), H, KVH, D, D, None, None, slots.cuda(), page)
    assert torch.equal(q, got[True][0])
    assert ops.tc_status() == 0


def _page_ids(total, order, g):
    """Page numbers 1..total-1 in the order in which ``pop()`` hands them out: shuffled, one after
    the other, or in runs of one to six neighbours whose order among themselves is shuffled."""
    if order == "shuffled":
        return (torch.randperm(total - 1, generator=g) + 1).tolist()
    if order == "in_order":
        return list(range(total - 1, 0, -1))
    assert order == "runs"
    runs, at = [], 1
    while at < total:
        n = min(int(torch.randint(1, 7, (1,), generator=g)), total - at)
        runs.append(list(range(at, at + n)))
        at += n
    out = []
    for r in torch.randperm(len(runs), generator=g).tolist():
        out.extend(runs[r])
    return out[::-1]


def _paged_case(dtype, H, KVH, D, page, q_lens, prefixes, seed, window=None, needle=None, order="shuffled"):
    """Random q/k/v for several requests, laid into a paged cache."""
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    seq_lens = [q + p for q, p in zip(q_lens, prefixes)]
    n_pages = [-(-s // page) for s in seq_lens]
    total = sum(n_pages) + 1
    ids = _page_ids(total, order, g)
    W = max(n_pages + [1])
    bt = torch.zeros((B, W), dtype=torch.int32)
    kc = torch.zeros((total, KVH, page, D))
    vc = torch.zeros((total, KVH, page, D))
    T = sum(q_lens)
    qkv = torch.randn((T, (H + 2 * KVH) * D), generator=g)
    at = 0
    for b in range(B):
        mine = [ids.pop() for _ in range(n_pages[b])]
        bt[b, :len(mine)] = torch.tensor(mine, dtype=torch.int32)
        k = torch.randn((seq_lens[b], KVH, D), generator=g)
        v = torch.randn((seq_lens[b], KVH, D), generator=g)
        if needle is not None and needle < seq_lens[b]:
            # one far key lines up with the last query of every head: its value must come out
            last = at + q_lens[b] - 1
            G = H // KVH
            for kvh in range(KVH):
                q = qkv[last, kvh * G * D:(kvh * G + 1) * D]
                k[needle, kvh] = 100.0 * q / q.norm()
                for gi in range(G):
                    qkv[last, (kvh * G + gi) * D:(kvh * G + gi + 1) * D] = q
        for j in range(seq_lens[b]):
            kc[mine[j // page], :, j % page] = k[j]
            vc[mine[j // page], :, j % page] = v[j]
        at += q_lens[b]
    qs = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    return qkv.to(dtype), kc.to(dtype), vc.to(dtype), bt, qs, sl


def _poison_unwritten(kc, vc, bt, sl, page):
    """NaN in every cache row that holds no key of any request: what a pool that was never cleared
    may hold.  No such row may reach an output."""
    written = torch.zeros(kc.shape[0], page, dtype=torch.bool)
    for b in range(bt.shape[0]):
        for j in range(int(sl[b])):
            written[int(bt[b, j // page]), j % page] = True
    hole = ~written[:, None, :, None].expand_as(kc)
    kc[hole] = float("nan")
    vc[hole] = float("nan")


def _run_attention(ops, dtype, H, KVH, D, page, q_lens, prefixes, seed, window=None, needle=None, fast=True, tc=True,
                   tma=True, poison=False, order="shuffled"):
    qkv, kc, vc, bt, qs, sl = _paged_case(dtype, H, KVH, D, page, q_lens, prefixes, seed, window, needle, order)
    if poison:
        _poison_unwritten(kc, vc, bt, sl, page)
    T = qkv.shape[0]
    scale = D ** -0.5
    nd = 0
    while nd < len(q_lens) and q_lens[nd] == 1:
        nd += 1
    step = FakeStep(qs.cuda(), sl.cuda(), len(q_lens), max(q_lens), int(sl.max()), nd)
    out = torch.full((T, H * D), float("nan"), dtype=dtype, device="cuda")
    ops.use_fast_attention = fast
    tc_before = ops.use_tc_attention
    ops.use_tc_attention = tc and tc_before
    kernel_before = ops.decode_kernel
    ops.decode_kernel = "tma" if tma else "cp"
    try:
        ops.attention(out, qkv.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), step, H, KVH, D, page, scale, window)
    finally:
        ops.use_fast_attention = True
        ops.use_tc_attention = tc_before
        ops.decode_kernel = kernel_before
    assert ops.tc_status() == 0, "a tensor-core or TMA block gave up on a wait"
    ref = torch.empty((T, H * D), dtype=torch.float32)
    paged_attention(ref, qkv.float().nan_to_num(0.0), kc.float().nan_to_num(0.0), vc.float().nan_to_num(0.0), bt, qs, sl,
                    H, KVH, D, page, scale, window)
    return out.cpu().float(), ref, (qkv, kc, vc, bt, qs, sl)


ATT_TOL = {torch.float32: dict(atol=2e-5, rtol=1e-4), torch.bfloat16: dict(atol=1e-2, rtol=1e-2)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KVH,D,page", [(4, 2, 16, 16), (14, 2, 64, 16), (12, 2, 128, 16), (8, 8, 64, 8),
                                          (5, 5, 48, 4), (3, 1, 256, 16), (6, 1, 80, 32)])
def test_attention_decode(ops, dtype, H, KVH, D, page):
    lens = [1, 2, 15, 16, 17, 100, 1000, 0, 33, 64, 65, 257, 4000]
    for fast, tma in ((True, True), (True, False), (False, False)):
        out, ref, _ = _run_attention(ops, dtype, H, KVH, D, page, [1] * len(lens),
                                     [max(l - 1, 0) if l else -1 for l in lens], 11, fast=fast, tma=tma)
        torch.testing.assert_close(out, ref, **ATT_TOL[dtype])
        assert torch.all(out[7] == 0), "a padding row (context 0) gives zeros"


@pytest.mark.parametrize("B,ctx", [(1, 3000), (3, 700), (64, 90)])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_split_counts(ops, B, ctx, window):
    """Few requests with long contexts are cut into many key splits, many requests into one."""
    H, KVH, D, page = 12, 2, 128, 16
    lens = [max(ctx - 7 * i, 1 + i) for i in range(B)]
    assert ops.decode_splits(1, KVH, 3000) > 4 and ops.decode_splits(256, KVH, 90) == 1
    assert ops.decode_splits_tma(1, KVH, D, 3000) > 4 and ops.decode_splits_tma(256, KVH, D, 90) == 1
    for tma in (True, False):
        out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, [1] * B, [l - 1 for l in lens], 15,
                                     window=window, tma=tma)
        torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])


@pytest.mark.parametrize("H,KVH,D,page", [(12, 2, 128, 16), (14, 2, 64, 32), (16, 1, 128, 48), (9, 3, 64, 64), (7, 1, 128, 128)])
@pytest.mark.parametrize("nsplit,stages", [(1, 2), (1, 6), (3, 3), (7, 8), (20, 4), (40, 3), (128, 6)])
@pytest.mark.parametrize("window", [None, 1, 130])
def test_attention_decode_tma_rings(ops, monkeypatch, H, KVH, D, page, nsplit, stages, window):
    """The TMA decode kernel with every way its ring of stages and its split count can fall: more
    tiles than stages (stages reused several times), more splits than tiles (blocks that leave at
    once), contexts that end on and around tile and page edges, a window whose low edge cuts a
    tile, and a cache whose unwritten rows hold NaN.  More than 16 splits with a tile each merge in two
    levels (groups of 8, the last group smaller: 17 tiles are 8 + 8 + 1), and the launch is made twice:
    every ticket counter is back at zero."""
    if stages * 2 * 64 * D * 2 > 220 * 1024:
        pytest.skip("more stages than shared memory holds at this head size")
    lens = [1, 63, 64, 65, 128, 129, 1000, 1024, 1025, 2500, 16, 17]
    monkeypatch.setattr(ops, "decode_splits_tma", lambda *a: nsplit)
    monkeypatch.setattr(ops, "decode_stages", stages)
    # 2 to 8 splits merge as a thread-block cluster (some of whose blocks get no tile here and leave
    # early), or, switched off, through scratch and a ticket counter like the larger counts
    try:
        for clusters in ((1, 0) if 2 <= nsplit <= 8 else (1,)):
            ops.lib.ts_set_clusters(clusters)
            for _ in range(2):
                out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, [1] * len(lens), [l - 1 for l in lens],
                                             17, window=window, poison=True)
                assert torch.isfinite(out).all()
                torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
    finally:
        ops.lib.ts_set_clusters(1)


@pytest.mark.parametrize("B,H,KVH,page,D", [(1, 12, 2, 16, 128), (8, 12, 2, 16, 128), (4, 28, 4, 64, 128), (3, 5, 5, 32, 128),
                                            (2, 16, 1, 48, 128), (8, 14, 2, 16, 64), (3, 5, 5, 32, 64)])
@pytest.mark.parametrize("window", [None, 150])
def test_attention_decode_blocks_of_eight_warps(ops, monkeypatch, B, H, KVH, page, D, window):
    """Few requests whose keys the rule cuts into 16: the kernel then runs 8 splits of 8 warps, merged as
    one cluster a (request, kv head) or, where the clusters do not all fit the chip, by the ticket (8 x 2
    and 4 x 4 pairs here).  Contexts around the edges of its tiles of 128 keys and of its splits, a
    window, NaN in unwritten rows; against the reference and against the blocks of 4 warps."""
    monkeypatch.setattr(ops, "decode_splits", lambda *a: 16)
    lens = [2049, 1, 127, 128, 129, 1023, 1024, 1025, 2500, 5000, 300, 17][:B] if B > 1 else [2049]
    outs = []
    try:
        for wide in (2, 1, 0):
            ops.lib.ts_set_decode_wide(wide)
            out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, [1] * len(lens), [l - 1 for l in lens], 23,
                                         window=window, tma=False, poison=True)
            assert torch.isfinite(out).all()
            torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
            outs.append(out)
    finally:
        ops.lib.ts_set_decode_wide(2)
    torch.testing.assert_close(outs[0], outs[2], atol=4e-3, rtol=8e-3)     # one bfloat16 step
    torch.testing.assert_close(outs[1], outs[2], atol=4e-3, rtol=8e-3)


@pytest.mark.parametrize("H,KVH,D,page", [(12, 2, 128, 16), (14, 2, 64, 32), (16, 1, 128, 64), (9, 3, 64, 64)])
@pytest.mark.parametrize("nsplit", [1, 2, 3, 4, 8, 16, 24, 40, 128])
@pytest.mark.parametrize("window", [None, 1, 130])
def test_attention_decode_merge_of_splits(ops, monkeypatch, H, KVH, D, page, nsplit, window):
    """The cp.async decode kernel's two ways of merging its key splits: 2, 4, 8 or 16 splits as one
    thread-block cluster that reads its blocks' shared memory, and any count through scratch and a
    ticket counter.  More splits than tiles (blocks without a key), contexts on and around tile
    edges, a window, NaN in unwritten rows; the two ways agree to rounding."""
    monkeypatch.setattr(ops, "decode_splits", lambda *a: nsplit)
    # many requests, and one (clusters of 16 are used only while they are few)
    for lens in ([1, 63, 64, 65, 128, 129, 1000, 1024, 1025, 2500, 16, 17], [2500]):
        outs = []
        try:
            for clusters in (1, 0):
                ops.lib.ts_set_clusters(clusters)
                out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, [1] * len(lens),
                                             [l - 1 for l in lens], 19, window=window, tma=False, poison=True)
                assert torch.isfinite(out).all()
                torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
                outs.append(out)
        finally:
            ops.lib.ts_set_clusters(1)
        torch.testing.assert_close(outs[0], outs[1], atol=4e-3, rtol=8e-3)     # one bfloat16 step


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KVH,D,page", [(4, 2, 16, 16), (12, 2, 128, 16), (14, 2, 64, 8), (5, 5, 48, 16)])
@pytest.mark.parametrize("case", [[(1, 0)], [(15, 16)], [(16, 37)], [(17, 1000)], [(300, 0)],
                                  [(1, 5), (1, 99), (40, 0), (2, 31), (33, 64)]])
def test_attention_chunks(ops, dtype, H, KVH, D, page, case):
    for fast, tc in ((True, True), (True, False), (False, False)):
        out, ref, _ = _run_attention(ops, dtype, H, KVH, D, page, [c[0] for c in case], [c[1] for c in case], 12,
                                     fast=fast, tc=tc)
        torch.testing.assert_close(out, ref, **ATT_TOL[dtype])


@pytest.mark.parametrize("H,KVH,D", [(12, 2, 128), (28, 4, 128), (14, 2, 64), (4, 4, 64), (40, 2, 64)])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_long_portions(ops, H, KVH, D, window):
    """Portions of hundreds of tokens after long prefixes, several requests of different shape in
    one launch, group sizes that are no power of two (and one above 16)."""
    for tc in (True, False):
        out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, 16, [1, 1, 700, 65, 2, 130], [300, 0, 0, 1000, 77, 129],
                                     16, window=window, tc=tc)
        torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 24, 200])
def test_attention_window(ops, dtype, window):
    for H, KVH, D in [(6, 2, 32), (6, 2, 64)]:
        out, ref, _ = _run_attention(ops, dtype, H, KVH, D, 8, [1, 40, 7, 1], [99, 0, 90, 3], 13, window=window)
        torch.testing.assert_close(out, ref, **ATT_TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("needle", [0, 14, 15, 16, 17, 31, 32, 99, 511, 777])
def test_attention_needle(ops, dtype, needle):
    """One far key among hundreds carries all the weight: the output is that key's value
    (reference tests/kernels/test_kernels.py:135-154)."""
    H, KVH, D, page = 12, 2, 128, 16
    for tma in (True, False):
        out, ref, (qkv, kc, vc, bt, qs, sl) = _run_attention(ops, dtype, H, KVH, D, page, [1, 9], [899, 891], 14,
                                                           needle=needle, tma=tma)
        torch.testing.assert_close(out, ref, **ATT_TOL[dtype])
    for b in range(2):
        last = int(qs[b + 1]) - 1
        pg = int(bt[b, needle // page])
        for kvh in range(KVH):
            v = vc[pg, kvh, needle % page].float()
            got = out[last, kvh * (H // KVH) * D:(kvh * (H // KVH) + 1) * D]
            torch.testing.assert_close(got, v, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("page", [16, 64])
def test_attention_tensor_core_uneven_warps(ops, page):
    """A long portion whose last row tile ends in rows without a query: that warp masks every tile
    element by element and falls behind the other three, which already have the next tile's scores.
    A warp running ahead must not be counted among the rows that have finished the tile before
    (it once was: the product then read probabilities that the slow warp had not written yet,
    in some launches only, hence the repeats)."""
    H, KVH, D = 12, 2, 128
    q_lens, prefixes = [1, 2047], [2048, 0]
    qkv, kc, vc, bt, qs, sl = _paged_case(torch.bfloat16, H, KVH, D, page, q_lens, prefixes, 23)
    # small queries: flat scores, no row's maximum ever jumps, so nothing makes a fast warp wait for
    # the products of the tile before (as in a trained or N(0, 0.02) model; random queries hide it)
    qkv[:, : H * D] = (qkv[:, : H * D].float() * 0.02).to(qkv.dtype)
    step = FakeStep(qs.cuda(), sl.cuda(), 2, 2047, int(sl.max()), 1)
    ref = torch.empty((qkv.shape[0], H * D), dtype=torch.float32)
    paged_attention(ref, qkv.float(), kc.float(), vc.float(), bt, qs, sl, H, KVH, D, page, D ** -0.5, None)
    ref = ref.cuda()
    q_d, bt_d = qkv.cuda(), bt.cuda()
    copies = [(kc.cuda(), vc.cuda()) for _ in range(48)]          # rotated: keys and values come from DRAM, as in a model
    ops.use_tc_attention = True
    for i in range(96):
        out = torch.full((qkv.shape[0], H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        k_d, v_d = copies[i % len(copies)]
        ops.attention(out, q_d, k_d, v_d, bt_d, step, H, KVH, D, page, D ** -0.5, None)
        torch.testing.assert_close(out.float(), ref, **ATT_TOL[torch.bfloat16])
    assert ops.tc_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 300, 130), (65, 129, 257), (130, 70, 1000), (3, 1000, 48)])
def test_linear(ops, dtype, M, N, K):
    x, w, b = _rand((M + 5, K), dtype, 20), _rand((N, K), dtype, 21, 0.1), _rand((N,), dtype, 22)
    rows = torch.randperm(M + 5)[:M].to(torch.int32)
    ref = torch.nn.functional.linear(x.float(), w.float(), b.float())
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=5e-2, rtol=2e-2)
    for use_lib in ([False, True] if dtype == torch.bfloat16 else [False]):
        ops.use_library_gemm = use_lib
        ops.gemm_mode = "library"
        try:
            out = torch.empty((M + 5, N), dtype=dtype, device="cuda")
            ops.linear(out, x.cuda(), w.cuda(), b.cuda())
            torch.testing.assert_close(out.cpu().float(), ref, **tol)
            out32 = torch.empty((M, N), dtype=torch.float32, device="cuda")
            ops.linear(out32, x.cuda(), w.cuda(), None, rows.cuda())
            ref32 = torch.nn.functional.linear(x.float()[rows.long()], w.float())
            torch.testing.assert_close(out32.cpu(), ref32, atol=1e-4 if dtype == torch.float32 else 2e-3, rtol=1e-4)
        finally:
            ops.use_library_gemm = True
            ops.gemm_mode = DEFAULT_GEMM


@pytest.mark.parametrize("M", [1, 8, 17, 64, 128, 129, 300, 2048])
@pytest.mark.parametrize("N,K", [(128, 64), (1536, 1536), (200, 200), (2048, 8960), (17920, 1536), (1000, 72)])
def test_linear_tensor_core(ops, M, N, K):
    """The tcgen05 product in both orientations, with K split or not, against float64."""
    x, w, b = _rand((M, K), torch.bfloat16, 30, 1.0), _rand((N, K), torch.bfloat16, 31, 0.05), _rand((N,), torch.bfloat16, 32)
    ref = (x.double() @ w.double().T + b.double()).float()
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    ops.gemm_mode = "tc"
    try:
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        ops.linear(out, xd, wd, bd)
        torch.testing.assert_close(out.cpu().float(), ref, atol=3e-2, rtol=2e-2)
        out32 = torch.empty((M, N), dtype=torch.float32, device="cuda")
        ops.linear(out32, xd, wd, None)
        torch.testing.assert_close(out32.cpu(), ref - b.float(), atol=2e-3, rtol=1e-3)
        rows = torch.randperm(M)[: max(1, M // 2)].to(torch.int32)
        outr = torch.empty((rows.shape[0], N), dtype=torch.float32, device="cuda")
        ops.linear(outr, xd, wd, None, rows.cuda())
        torch.testing.assert_close(outr.cpu(), (ref - b.float())[rows.long()], atol=2e-3, rtol=1e-3)
        assert ops.tc_status() == 0, "a block of the tensor-core product gave up on a wait"
    finally:
        ops.gemm_mode = DEFAULT_GEMM


@pytest.mark.parametrize("M", [1, 3, 8, 17, 32])
@pytest.mark.parametrize("N,K", [(1536, 1536), (1536, 8960), (200, 72), (384, 136), (256, 4096), (202, 264)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_into_residual(ops, M, N, K, with_bias):
    """The few-token product that sums its K splits (a thread-block cluster, or one block) and adds
    itself to the residual rows in place: against the formula in 32 bits, and bit for bit against the
    path it replaces (product left unreduced, the norm kernel summing and adding) when both cut K alike."""
    from turingserve_b200.kernels import LazyProduct
    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16() if with_bias else None
    resid = torch.randn(M, N, generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(N, generator=g))
    h = x.float() @ w.float().t()
    if with_bias:
        h = h + bias.float()
    want = (h.bfloat16().float() + resid.float()).bfloat16()
    cu = lambda t: None if t is None else t.cuda()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    normed = torch.empty_like(out)
    before, cap = ops.max_splits, ops.fused_link_tokens
    try:
        ops.max_splits = 8
        ops.fused_link_tokens = 32                   # the kernel takes more tokens than the engine gives it
        r1 = resid.cuda()
        p = ops.linear(out, cu(x), cu(w), cu(bias), may_defer=True)
        assert isinstance(p, LazyProduct)
        ops.rmsnorm(normed, p, nw.cuda(), 1e-5, r1)
        y1 = normed.clone()
        assert ops.tc_status() == 0
        # a product of bfloat16 values summed in another order differs in its last bit at most
        torch.testing.assert_close(r1.cpu().float(), want.float(), atol=2e-2, rtol=1.6e-2)
        assert (r1.cpu() == want).float().mean() > 0.9
        if N % 8:                                    # (the path it replaces wants rows of a multiple of 8)
            return
        ops.fused_link_tokens = 0                    # the path it replaces
        r2 = resid.cuda()
        d = ops.linear(out, cu(x), cu(w), cu(bias), may_defer=True)
        assert not isinstance(d, LazyProduct)
        y2 = torch.empty_like(out)
        ops.rmsnorm(y2, d, nw.cuda(), 1e-5, r2)
        assert torch.equal(r1, r2), "same splits, same order of sums: the same bits"
        # (two norm kernels add a row's squares up in different orders: a value may differ by one step)
        torch.testing.assert_close(y1.float(), y2.float(), atol=3e-2, rtol=1.6e-2)
        assert (y1 == y2).float().mean() > 0.97
    finally:
        ops.max_splits, ops.fused_link_tokens = before, cap


@pytest.mark.parametrize("width", [0, 256, 192, 128])
@pytest.mark.parametrize("M,N,K,with_bias", [(256, 256, 64, False), (300, 520, 200, True), (129, 1000, 1536, True),
                                             (1100, 1536, 904, False), (2048, 2048, 1536, True)])
def test_linear_on_pairs_of_sms(ops, M, N, K, with_bias, width):
    """The many-row product whose tiles are computed by two SMs together, at every tile width, with ragged
    edges in all three sizes: against the formula in 32 bits.  More tiles than pairs of SMs (the last
    shape at width 128) makes blocks take several tiles, with both accumulators in use."""
    g = torch.Generator().manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16() if with_bias else None
    want = x.float() @ w.float().t()
    if with_bias:
        want = want + bias.float()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.lib.ts_set_pair_tile_width(width)
    try:
        assert ops.linear_pair(out, x.cuda(), w.cuda(), None if bias is None else bias.cuda(), ops.PAIR_PLAIN)
    finally:
        ops.lib.ts_set_pair_tile_width(0)
    assert ops.tc_status() == 0
    torch.testing.assert_close(out.cpu().float(), want, atol=3e-2, rtol=1.6e-2)
    assert (out.cpu() == want.bfloat16()).float().mean() > 0.9, "another order of sums moves the last bit at most"


@pytest.mark.parametrize("T,inter,K", [(129, 128, 64), (300, 320, 200), (700, 1280, 1536), (2048, 8960, 1536)])
def test_gated_linear_on_pairs_of_sms(ops, monkeypatch, T, inter, K):
    """Gate/up product of many rows with the activation in its epilogue: no product tensor, no activation
    kernel, and the result of the two steps with the product rounded to bfloat16 in between."""
    x, w = _rand((T, K), torch.bfloat16, 30, 1.0).cuda(), _rand((2 * inter, K), torch.bfloat16, 31, 0.1).cuda()
    two = torch.empty((T, inter), dtype=torch.bfloat16, device="cuda")
    monkeypatch.setattr(ops, "pair_wins", lambda *a: False)
    ops.gated_linear(two, x, w, None, 64)
    separate = []
    monkeypatch.setattr(ops, "pair_wins", lambda *a: True)
    monkeypatch.setattr(ops, "silu_mul", lambda *a, _f=ops.silu_mul: (separate.append(1), _f(*a))[1])
    out = torch.full((T, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gated_linear(out, x, w, None, 64)
    assert not separate
    assert ops.tc_status() == 0
    ref = torch.empty((T, inter), dtype=torch.bfloat16)
    TwinOps().gated_linear(ref, x.cpu(), w.cpu(), None, 64)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=3e-2, rtol=3e-2)
    # against the library product and the activation kernel: the sums differ in their order only
    torch.testing.assert_close(out.float(), two.float(), atol=3e-2, rtol=3e-2)
    assert (out == two).float().mean() > 0.9


@pytest.mark.parametrize("T", [65, 300, 1500])
@pytest.mark.parametrize("H,KVH,K,bias,D", [(12, 2, 1536, True, 128), (5, 1, 200, False, 128), (14, 2, 896, True, 64),
                                            (3, 3, 320, True, 64), (5, 1, 200, False, 64)])
def test_qkv_product_on_pairs_of_sms_rotates_and_writes_the_cache(ops, monkeypatch, T, H, KVH, K, bias, D):
    """The q/k/v product of many rows with bias, rotation and cache write in its epilogue: what the library
    product followed by the rotary kernel gives, in the q/k/v tensor and in the cache pages (slots of -1 are
    not written); tiles of 256 columns are two heads of 128 or four of 64, the last tile partly empty."""
    page, pages = 16, 120
    N = (H + 2 * KVH) * D
    x = _rand((T, K), torch.bfloat16, 50, 1.0).cuda()
    w = _rand((N, K), torch.bfloat16, 51, 0.05).cuda()
    b = _rand((N,), torch.bfloat16, 52, 0.5).cuda() if bias else None
    pos = torch.randint(0, 600, (T,), dtype=torch.int32).cuda()
    cos, sin = (t.cuda() for t in plain.rope_tables(D, 1e6, 600))
    slots = (torch.randperm(page * (pages - 1))[:T].to(torch.int32) + page)
    slots[1] = -1
    slots[T - 1] = -1
    slots = slots.cuda()
    kc0, vc0 = _rand((pages, KVH, page, D), torch.bfloat16, 53), _rand((pages, KVH, page, D), torch.bfloat16, 54)
    got = {}
    for pairs in (True, False):
        monkeypatch.setattr(ops, "pair_wins", lambda *a, _p=pairs: _p)
        kc, vc = kc0.clone().cuda(), vc0.clone().cuda()
        out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        launches = ops.launches
        q = ops.qkv_rope(out, x, w, b, pos, cos, sin, H, KVH, D, D, kc, vc, slots, page)
        if pairs:
            assert ops.launches - launches == 1
        got[pairs] = (q.clone(), kc, vc)
    assert ops.tc_status() == 0
    for a, c in zip(got[True], got[False]):
        torch.testing.assert_close(a.float(), c.float(), atol=3e-2, rtol=2e-2)
        assert (a == c).float().mean() > 0.9
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[slots[slots >= 0].long().cpu()] = False
    for cache, before in ((got[True][1], kc0), (got[True][2], vc0)):
        rows = cache.cpu().permute(0, 2, 1, 3).reshape(pages * page, KVH, D)
        assert torch.equal(rows[untouched], before.permute(0, 2, 1, 3).reshape(pages * page, KVH, D)[untouched])
    # rotate only (a run that reads another run's cache): no cache write
    monkeypatch.setattr(ops, "pair_wins", lambda *a: True)
    out = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
    q = ops.qkv_rope(out, x, w, b, pos, cos, sin, H, KVH, D, D, None, None, slots, page)
    assert torch.equal(q, got[True][0])


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("N,K", [(151936, 1536), (75800, 320)])
def test_linear_tensor_core_output_head(ops, M, N, K):
    """The output head's shape (turingserve/model/qwen2.py:94-99: hidden states times the whole
    vocabulary, 32-bit logits): at most 16 rows and so many outputs that the launch is several waves of
    blocks, which is where the kernel runs with three stages and two blocks to an SM.  One vocabulary
    that is no multiple of the tile's 128 rows.  Against float64, at every row and column."""
    x, w = _rand((M, K), torch.bfloat16, 33, 1.0), _rand((N, K), torch.bfloat16, 34, 0.05)
    assert -(-N // 128) >= 592
    xd, wd = x.cuda(), w.cuda()
    ref = (xd.double() @ wd.double().T).float()
    ops.gemm_mode = "auto"
    try:
        out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        ops.linear(out32, xd, wd, None)
        torch.testing.assert_close(out32, ref, atol=2e-3, rtol=1e-3)
        rows = torch.arange(M - 1, -1, -1, dtype=torch.int32, device="cuda")       # the head gathers its rows
        ops.linear(out32, xd, wd, None, rows)
        torch.testing.assert_close(out32, ref.flip(0), atol=2e-3, rtol=1e-3)
        out16 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        ops.linear(out16, xd, wd, None)
        torch.testing.assert_close(out16.float(), ref, atol=3e-2, rtol=2e-2)
        assert ops.tc_status() == 0
    finally:
        ops.gemm_mode = DEFAULT_GEMM


def test_work_buffers_outlive_the_graphs_that_captured_them(ops):
    """A product small enough for the first work buffer is captured in a graph; a larger one then makes
    the buffer grow.  The old buffer is set aside, not freed, so the graph's replay still computes the
    right thing (it reads and writes the old address)."""
    from turingserve_b200.kernels import Deferred
    M, N, K = 4, 1536, 8960
    x, w = _rand((M, K), torch.bfloat16, 50).cuda(), _rand((N, K), torch.bfloat16, 51, 0.05).cuda()
    nw = torch.ones(N, dtype=torch.bfloat16, device="cuda")
    ref = torch.nn.functional.linear(x.float(), w.float())
    ops.gemm_mode = "auto"
    out, normed = (torch.empty((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    if "partials" in ops._buffers:                         # start from a buffer of the first size
        ops._outgrown.append(ops._buffers.pop("partials"))

    def small():
        d = ops.linear(out, x, w, None, may_defer=True, lazy=False)
        assert isinstance(d, Deferred)
        ops.rmsnorm(normed, d, nw, 1e-6)

    small()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        small()
    before = ops._buffers["partials"]
    xb = _rand((128, K), torch.bfloat16, 52).cuda()       # ten splits of 128 x 1536 partial sums: twice the first buffer
    ob = torch.empty((128, N), dtype=torch.bfloat16, device="cuda")
    d = ops.linear(ob, xb, w, None, may_defer=True, lazy=False)
    assert isinstance(d, Deferred) and d.splits * 128 * N > before.numel()
    ops.materialize(d)
    assert ops._buffers["partials"] is not before and any(b is before for b in ops._outgrown)
    torch.cuda.empty_cache()
    junk = [torch.full((1 << 20,), float("nan"), device="cuda") for _ in range(8)]     # whoever gets freed blocks next
    normed.zero_()
    g.replay()
    torch.cuda.synchronize()
    want = torch.empty((M, N), dtype=torch.bfloat16)
    TwinOps().rmsnorm(want, ref.cpu().to(torch.bfloat16), nw.cpu(), 1e-6)
    torch.testing.assert_close(normed.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)
    assert all(torch.isnan(j).all() for j in junk)
    assert ops.tc_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 1536, 1536), (8, 1536, 8960), (64, 200, 264), (128, 4104, 72)])
def test_deferred_product_finished_by_the_norm(ops, M, N, K):
    """A few-token product may leave its split-K partial sums to the norm that consumes it; the
    result equals product, then residual add, then norm, each rounded where the separate kernels round."""
    from turingserve_b200.kernels import Deferred
    twin = TwinOps()
    x, w, b = _rand((M, K), torch.bfloat16, 40), _rand((N, K), torch.bfloat16, 41, 0.05), _rand((N,), torch.bfloat16, 42)
    res, nw = _rand((M, N), torch.bfloat16, 43), (1 + 0.1 * _rand((N,), torch.float32, 44)).to(torch.bfloat16)
    ops.gemm_mode = "tc"
    try:
        for bias in (None, b):
            for with_res in (True, False):
                out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
                d = ops.linear(out, x.cuda(), w.cuda(), None if bias is None else bias.cuda(), may_defer=True, lazy=False)
                assert isinstance(d, Deferred) and d.shape == (M, N)
                plain_out = ops.materialize(d).cpu()
                ref_lin = torch.nn.functional.linear(x.float(), w.float(), None if bias is None else bias.float())
                torch.testing.assert_close(plain_out.float(), ref_lin, atol=3e-2, rtol=2e-2)
                normed = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
                r_dev = res.clone().cuda() if with_res else None
                ops.rmsnorm(normed, d, nw.cuda(), 1e-6, r_dev)
                ref = torch.empty((M, N), dtype=torch.bfloat16)
                r_ref = res.clone() if with_res else None
                twin.rmsnorm(ref, plain_out, nw, 1e-6, r_ref)
                torch.testing.assert_close(normed.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)
                if with_res:
                    torch.testing.assert_close(r_dev.cpu().float(), r_ref.float(), atol=2e-2, rtol=1e-2)
        assert ops.tc_status() == 0
    finally:
        ops.gemm_mode = DEFAULT_GEMM


@pytest.mark.parametrize("H,KVH", [(14, 2), (3, 3), (16, 1)])
@pytest.mark.parametrize("page,order", [(16, "in_order"), (16, "shuffled"), (32, "runs"), (64, "shuffled"), (48, "shuffled")])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("tile", [64, 128])
def test_attention_tensor_core_portions_head_64(ops, H, KVH, page, order, window, tile):
    """The same kernel at head size 64 (one 64-column half per row of Q, K and V; the row's two softmax
    threads take 32 columns of the output each)."""
    D = 64
    ops.use_tc_attention = True
    ops.lib.ts_set_prefill_tile(tile)
    try:
        for q_lens, prefixes in (([300], [0]), ([1, 1, 700, 65, 2, 130], [300, 0, 0, 1000, 77, 129]), ([17, 40], [1000, 3])):
            out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, q_lens, prefixes, 31, window=window, order=order)
            torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
        if window is None:
            for needle in (0, 63, 64, 127, 128, 500):
                out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, [9, 130], [891, 770], 32, needle=needle,
                                             order=order)
                torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
        assert ops.tc_status() == 0, "a block of the tensor-core attention gave up on a wait"
    finally:
        ops.use_tc_attention = True
        ops.lib.ts_set_prefill_tile(0)


@pytest.mark.parametrize("H,KVH", [(12, 2), (28, 4), (5, 5), (40, 2)])
@pytest.mark.parametrize("page", [16, 32, 64, 128])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("order,tile", [("shuffled", 0), ("in_order", 64), ("runs", 128), ("shuffled", 128), ("in_order", 128)])
def test_attention_tensor_core_portions(ops, H, KVH, page, window, order, tile):
    """The tcgen05 prompt-portion kernel (head size 128): portions after prefixes, several requests,
    group sizes that are no power of two, a needle far back.  Pages smaller than a tile of keys are
    fetched as one box where they lie one after the other in the pool and page by page where they do
    not, so the pool is laid out shuffled, in order, and in short runs.  ``tile``: keys per tile, 64 or
    128, or 0 for what the launch's size chooses."""
    D = 128
    ops.use_tc_attention = True
    ops.lib.ts_set_prefill_tile(tile)
    try:
        for q_lens, prefixes in (([300], [0]), ([1, 1, 700, 65, 2, 130], [300, 0, 0, 1000, 77, 129]), ([17, 40], [1000, 3])):
            out, ref, _ = _run_attention(ops, torch.bfloat16, H, KVH, D, page, q_lens, prefixes, 21, window=window,
                                         order=order)
            torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
        if window is None:
            for needle in (0, 15, 16, 63, 64, 65, 127, 500):
                out, ref, (qkv, kc, vc, bt, qs, sl) = _run_attention(ops, torch.bfloat16, H, KVH, D, page, [9, 130], [891, 770],
                                                                   22, needle=needle, order=order)
                torch.testing.assert_close(out, ref, **ATT_TOL[torch.bfloat16])
        assert ops.tc_status() == 0, "a block of the tensor-core attention gave up on a wait"
    finally:
        ops.use_tc_attention = True
        ops.lib.ts_set_prefill_tile(0)
