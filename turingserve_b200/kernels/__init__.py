"""The CUDA kernels (sm_100a) behind one object, ``ops()``.

The library is built in-tree at the first call (``kernels.build``) and loaded with ctypes; every
function takes raw device pointers and the current CUDA stream.  There is no other backend: on a
machine without the library and without nvcc, or without a CUDA device, ``ops()`` raises.

Kernels and their reference counterparts (turingserve/ops/__init__.py:15-19 lists the op
namespace): embedding, rmsnorm (+residual), linear, rope fused with the cache write, paged
attention, silu*mul, sampling.  bfloat16 matrix products go to cuBLAS through ``torch.mm`` where
the reference uses ``F.linear`` (turingserve/ops/triton_ops.py:74-76), unless a hand-written
tensor-core kernel takes the shape; float32 products always use this library's FFMA kernel.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from turingserve_b200.kernels.build import build, library_path

_OPS = None

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16, not {dtype}") from None


class KernelError(RuntimeError):
    pass


class Deferred:
    """A product whose split-K partial sums still sit in scratch ([splits, M, N] float32): the norm
    that consumes it finishes the sum in its own kernel.  Quacks like a tensor as far as shape,
    dtype and device go; anything else must call ``ops().materialize`` first."""

    def __init__(self, part: torch.Tensor, splits: int, shape, dtype, bias, out: torch.Tensor) -> None:
        self.part, self.splits, self.shape, self.dtype, self.bias = part, splits, tuple(shape), dtype, bias
        self.device = part.device
        self.out = out                      # the buffer the finished product belongs in


class LazyProduct:
    """A few-token product that has not been launched yet: out = x @ w^T + bias.  The norm that gets it
    together with a residual launches it as ONE kernel that also sums its K splits (a thread-block
    cluster) and adds the result to the residual in place; any other consumer has it launched the
    ordinary way (``ops().materialize``, or as a ``Deferred``).  Shape, dtype and device as a tensor's."""

    def __init__(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, bias) -> None:
        self.out, self.x, self.w, self.bias = out, x, w, bias
        self.shape, self.dtype, self.device = tuple(out.shape), out.dtype, out.device


class CudaOps:
    """ctypes front of ``libturingserve_b200.so``."""

    ABI = 8
    UNSUPPORTED = -4            # a kernel's refusal of a shape or layout another kernel takes

    def __init__(self, lib_path: str) -> None:
        self.lib_path = lib_path
        self.lib = ctypes.CDLL(lib_path)
        self.lib.ts_last_error.restype = ctypes.c_char_p
        if self.lib.ts_abi_version() != self.ABI:
            raise KernelError(f"{lib_path} has ABI {self.lib.ts_abi_version()}, this package needs {self.ABI}")
        P, I, F = c_void_p, c_int, c_float
        sigs = {
            "ts_embedding": [P, P, P, I, I, I, I, P],
            "ts_gather_rows": [P, P, P, I, I, I, P],
            "ts_rmsnorm": [P, P, P, P, F, I, I, I, I, P],
            "ts_silu_mul": [P, P, I, I, I, P],
            "ts_silu_mul_ex": [P, P, I, I, I, I, P],
            "ts_linear_tc_gated": [P, P, P, I, I, I, P],
            "ts_linear_tc_resid": [P, P, P, P, I, I, I, I, P],
            "ts_linear_pair": [P, P, P, P, I, I, I, I, P],
            "ts_linear_pair_qkv": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
            "ts_linear_tc_qkv_rope": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
            "ts_rope_kv_write": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
            "ts_rope_kv_write_ex": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, I, P, P],
            "ts_attention_generic": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P],
            "ts_linear_simt": [P, P, P, P, P, I, I, I, I, I, P],
            "ts_attention_decode": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
            "ts_attention_decode_tma": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P],
            "ts_attention_prefill": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
            "ts_attention_prefill_tc": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P],
            "ts_linear_tc": [P, P, P, P, P, I, I, I, I, I, P],
            "ts_linear_tc_ex": [P, P, P, P, P, I, I, I, I, I, I, P, P],
            "ts_reduce_rmsnorm": [P, P, I, P, P, P, F, I, I, I, P],
            "ts_feed_tokens": [P, P, P, P, I, I, P],
            "ts_sample": [P, P, P, P, I, I, P, P],
            "ts_penalize": [P, P, P, P, I, I, P],
            "ts_sample_greedy": [P, P, I, I, P, P, P, P],
            "ts_clear_status": [P],
            "ts_decode_step": [P, I, I, P],
            "ts_decode_step_encode_map": [P, P, I, I],
            "ts_poke_status": [I, I, P],
        }
        for name, args in sigs.items():
            fn = getattr(self.lib, name)
            fn.argtypes = args
            fn.restype = c_int
        self.lib.ts_attention_decode_supported.argtypes = [I, I, I, I]
        self.lib.ts_attention_decode_supported.restype = c_int
        self.lib.ts_attention_decode_tma_supported.argtypes = [I, I, I, I, I]
        self.lib.ts_attention_decode_tma_supported.restype = c_int
        self.lib.ts_attention_decode_tma_status.argtypes = []
        self.lib.ts_attention_decode_tma_status.restype = c_int
        self.lib.ts_attention_decode_tma_blocks_per_sm.argtypes = [I, I]
        self.lib.ts_attention_decode_tma_blocks_per_sm.restype = c_int
        # decode attention: "tma" the kernel built for streaming many keys (pages of a multiple of 16
        # tokens), "cp" the one built for the shortest chain, "auto" by the step's streaming_decode
        self.decode_kernel = os.environ.get("TURINGSERVE_B200_DECODE_ATTENTION", "auto")
        self.decode_stages = int(os.environ.get("TURINGSERVE_B200_DECODE_STAGES", "3"))
        self.lib.ts_set_decode_tma_cluster_max.argtypes = [I]
        self.lib.ts_set_decode_tma_cluster_max.restype = None
        if "TURINGSERVE_B200_DECODE_TMA_CLUSTER" in os.environ:
            self.lib.ts_set_decode_tma_cluster_max(int(os.environ["TURINGSERVE_B200_DECODE_TMA_CLUSTER"]))
        # the "cp" kernel where the rule asks for 16 splits: 8 splits of 8 warps instead.  2: whenever those
        # blocks fit one per SM (merged as clusters where all clusters fit the chip, else by the ticket);
        # 1: only as clusters; 0: never
        self.lib.ts_set_pair_tile_width.argtypes = [I]
        self.lib.ts_set_pair_tile_width.restype = None
        self.lib.ts_set_decode_wide.argtypes = [I]
        self.lib.ts_set_decode_wide.restype = None
        self.lib.ts_set_decode_wide(int(os.environ.get("TURINGSERVE_B200_DECODE_WIDE", "2")))
        self.lib.ts_linear_tc_qkv_rope_scratch_floats.argtypes = [I, I, I]
        self.lib.ts_linear_tc_qkv_rope_scratch_floats.restype = ctypes.c_longlong
        self.lib.ts_sample_greedy_parts.argtypes = [I]
        self.lib.ts_sample_greedy_parts.restype = c_int
        self.lib.ts_rope_kv_write_fused_supported.argtypes = [I, I, I]
        self.lib.ts_rope_kv_write_fused_supported.restype = c_int
        self.lib.ts_linear_tc_supported.argtypes = [I, I, I]
        self.lib.ts_linear_tc_supported.restype = c_int
        self.lib.ts_linear_tc_status.argtypes = []
        self.lib.ts_linear_tc_status.restype = c_int
        # which bfloat16 products run on this library's tcgen05 kernel: "tc" all of them, "auto" those
        # with at most 128 rows (decode), "library" none (cuBLAS through torch.mm)
        self.gemm_mode = os.environ.get("TURINGSERVE_B200_GEMM", "auto")
        self.lib.ts_set_pdl.argtypes = [I]
        self.lib.ts_set_pdl.restype = None
        self.lib.ts_set_pdl(0 if os.environ.get("TURINGSERVE_B200_PDL", "1") == "0" else 1)
        self.lib.ts_set_clusters.argtypes = [I]
        self.lib.ts_set_clusters.restype = None
        self.lib.ts_set_clusters(0 if os.environ.get("TURINGSERVE_B200_CLUSTERS", "1") == "0" else 1)
        self.lib.ts_attention_prefill_tc_supported.argtypes = [I, I, I, I, I]
        self.lib.ts_attention_prefill_tc_supported.restype = c_int
        self.lib.ts_attention_prefill_tc_status.argtypes = []
        self.lib.ts_attention_prefill_tc_status.restype = c_int
        # prompt-portion attention on tcgen05 (head size 128, pages of a multiple of 16 tokens) or mma.sync
        self.use_tc_attention = os.environ.get("TURINGSERVE_B200_ATTENTION", "tc") == "tc"
        # its tiles of keys: 64 (two blocks an SM), 128 (one), 0 = by the size of the launch
        self.lib.ts_set_prefill_tile.argtypes = [I]
        self.lib.ts_set_prefill_tile.restype = None
        self.lib.ts_set_prefill_tile(int(os.environ.get("TURINGSERVE_B200_ATTENTION_TILE", "0")))
        self.lib.ts_attention_prefill_supported.argtypes = [I, I, I, I]
        self.lib.ts_attention_prefill_supported.restype = c_int
        for name, args in (("ts_decode_step_max_stages", [I]), ("ts_decode_step_blocks", [I, I]),
                           ("ts_decode_step_work_bytes", [I]), ("ts_decode_step_status", [])):
            getattr(self.lib, name).argtypes = args
            getattr(self.lib, name).restype = c_int
        self.lib.ts_attention_decode_scratch_floats.argtypes = [I, I, I, I]
        self.lib.ts_attention_decode_scratch_floats.restype = ctypes.c_longlong
        self._device_index = torch.cuda.current_device()
        self.num_sms = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        # work buffers by name; one that was outgrown is kept, not freed: a captured graph may still
        # hold its address
        self._buffers: dict[str, torch.Tensor] = {}
        self._outgrown: list[torch.Tensor] = []
        self._decode_slots: dict = {}
        self.use_fast_attention = True
        self.use_fused_step = True          # a whole decode step as one kernel where the model allows it
        self.use_library_gemm = True
        self.max_splits = 10        # (the fused reduce kernels load up to 16 partial sums in one go)
        self.launches = 0           # kernels of this library launched (graph replays add their share)

    # -- plumbing -----------------------------------------------------------------------------------
    def _stream(self) -> int:
        # the raw handle of the current stream: a tenth of the cost of building a torch.cuda.Stream
        # object for it, and every kernel launch asks
        return torch._C._cuda_getCurrentRawStream(self._device_index)

    def _buffer(self, name: str, numel: int, dtype: torch.dtype, device, floor: int = 0, zero: bool = False) -> torch.Tensor:
        """A work buffer of at least ``numel`` elements that lives as long as this object.  When a
        larger one is needed the old one is set aside, never freed: decode graphs captured earlier
        read and write it at its address on every replay."""
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < numel or buf.device != device:
            if buf is not None:
                self._outgrown.append(buf)
            make = torch.zeros if zero else torch.empty
            buf = self._buffers[name] = make(max(int(numel), floor), dtype=dtype, device=device)
        return buf

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            msg = self.lib.ts_last_error().decode(errors="replace")
            raise KernelError(f"{what} failed ({rc}): {msg}")

    # -- kernels ------------------------------------------------------------------------------------
    def embedding(self, out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
        T, h = out.shape
        self._check(self.lib.ts_embedding(_ptr(out), _ptr(table), _ptr(ids), T, h, table.shape[0],
                                          _code(out.dtype), self._stream()), "embedding")

    def gather_rows(self, out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor) -> None:
        S, w = out.shape
        self._check(self.lib.ts_gather_rows(_ptr(out), _ptr(x), _ptr(rows), S, w, _code(x.dtype),
                                            self._stream()), "gather_rows")

    # Up to this many tokens the output and down projections add themselves to the residual stream
    # (their K splits summed by a thread-block cluster) and the norm that follows reads the finished
    # rows: 1.437 -> 1.413 ms a decode step at batch 8, 1.753 -> 1.715 ms at batch 16, 1.966 -> 1.908 ms
    # at batch 32, 2.484 -> 2.402 ms at batch 64.  0: they leave partial sums for the norm kernel.
    fused_link_tokens = int(os.environ.get("TURINGSERVE_B200_FUSED_LINK_TOKENS", "64"))

    def _settle(self, x):
        """What the kernels that finish a split-K sum take: a product not yet launched is launched now,
        its partial sums left in scratch."""
        if isinstance(x, LazyProduct):
            return self.linear(x.out, x.x, x.w, x.bias, may_defer=True, lazy=False)
        return x

    def materialize(self, x):
        """A plain tensor for ``x``, running or finishing what was put off."""
        if isinstance(x, LazyProduct):
            return self.linear(x.out, x.x, x.w, x.bias)
        if not isinstance(x, Deferred):
            return x
        x.out.copy_(x.part[: x.splits].sum(0) if x.bias is None else x.part[: x.splits].sum(0) + x.bias.float())
        return x.out

    def rmsnorm(self, out, x, weight, eps: float, residual=None) -> None:
        """out = weight * norm(x), or of x + residual (which then holds the sum)."""
        if isinstance(x, LazyProduct):
            if residual is not None and self._into_residual(x, residual):
                x, residual = residual, None             # the sum is in place: what is left is a plain norm of it
            else:
                x = self._settle(x)
        self._rmsnorm(out, x, weight, eps, residual)

    def _into_residual(self, p: LazyProduct, residual: torch.Tensor) -> bool:
        """residual += product, in one kernel; False when that kernel does not take the shape."""
        M, N = p.shape
        K = p.w.shape[1]
        if not (residual.dtype == torch.bfloat16 and residual.is_contiguous() and tuple(residual.shape) == (M, N)):
            return False
        splits = min(self.tc_splits(M, N, K), 8)
        if M <= 16 and M > 4 * splits:
            # up to 16 tokens a block of the cluster sums its tokens one after the other: with few splits that
            # are many (0.5B shape, 16 tokens over 3 splits: 1.201 against 1.162 ms a step with the norm kernel)
            return False
        rc = self.lib.ts_linear_tc_resid(_ptr(residual), _ptr(p.x), _ptr(p.w), _ptr(p.bias), M, N, K, splits, self._stream())
        if rc == self.UNSUPPORTED:
            return False
        self._check(rc, "linear_tc_resid")
        return True

    def _rmsnorm(self, out, x, weight, eps: float, residual=None) -> None:
        if isinstance(x, Deferred):
            T, h = x.shape
            if h % 8 == 0 and h <= 16384 and x.dtype == torch.bfloat16:
                self._check(self.lib.ts_reduce_rmsnorm(
                    _ptr(out), _ptr(x.part), x.splits, _ptr(x.bias), _ptr(residual), _ptr(weight), float(eps), T, h,
                    _code(weight.dtype), self._stream()), "reduce_rmsnorm")
                return
            x = self.materialize(x)
        T, h = x.shape
        self._check(self.lib.ts_rmsnorm(_ptr(out), _ptr(x), _ptr(residual), _ptr(weight), float(eps), T, h,
                                        _code(x.dtype), _code(weight.dtype), self._stream()), "rmsnorm")

    def silu_mul(self, out, gu, group: int = 0) -> None:
        """out = silu(gate) * up.  ``group`` 0: gu = [gates | ups]; else gu comes in blocks of
        2 * group columns, group gates then the matching group ups."""
        T, inter = out.shape
        self._check(self.lib.ts_silu_mul_ex(_ptr(out), _ptr(gu), T, inter, group, _code(gu.dtype), self._stream()),
                    "silu_mul")

    GATE_GROUP = 64      # rows of gates, then of ups, in one 128-row tile of the few-token product
    # up to this many tokens the activation goes into the product's epilogue (the kernel takes 128; above
    # 16 tokens all four warps of its epilogue share the activation: 1.739 -> 1.688 ms a step at batch 24,
    # 1.857 -> 1.805 ms at batch 32; at batch 48 and 64 it is within half a percent of the kernel of its own)
    fused_gate_tokens = int(os.environ.get("TURINGSERVE_B200_FUSED_GATE_TOKENS", "32"))

    def gated_linear(self, out, x, w, bias, group: int) -> None:
        """out[T, I] = silu(g) * u with [g, u] = x @ w[2I, K]^T + bias, the rows of ``w`` (and
        ``bias``) laid out as ``silu_mul`` describes.  A few bfloat16 tokens and blocks of 64: one
        kernel, the activation in the product's epilogue; otherwise product, then activation."""
        T, inter = out.shape
        K = w.shape[1]
        use_tc = self.gemm_mode == "tc" or (self.gemm_mode == "auto" and T <= 128)
        if (x.dtype == torch.bfloat16 and use_tc and bias is None and group == self.GATE_GROUP and T <= self.fused_gate_tokens
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            rc = self.lib.ts_linear_tc_gated(_ptr(out), _ptr(x), _ptr(w), T, 2 * inter, K, self._stream())
            if rc != self.UNSUPPORTED:
                self._check(rc, "linear_tc_gated")
                return
        if (x.dtype == torch.bfloat16 and bias is None and group == self.GATE_GROUP and T > self.fused_gate_tokens
                and x.is_contiguous() and self.pair_wins(T, 2 * inter, K, 6.0 * T * inter)
                and self.linear_pair(out, x, w, None, self.PAIR_GATED)):
            return
        gu = torch.empty((T, 2 * inter), dtype=x.dtype, device=x.device)
        self.linear(gu, x, w, bias)
        self.silu_mul(out, gu, group)

    def rope_kv_write(self, qkv, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                      page_size):
        """Rotates q and k in place and writes k, v to the cache; returns the q/k/v tensor.  ``qkv`` may
        be a deferred product: the kernel then finishes its sum on the way."""
        qkv = self._settle(qkv)
        if isinstance(qkv, Deferred):
            d = qkv
            if (self.lib.ts_rope_kv_write_fused_supported(D, rotary_dim, _code(d.dtype))
                    and all(t is None or t.data_ptr() % 16 == 0 for t in (d.out, k_cache, v_cache, cos, sin))):
                self._check(self.lib.ts_rope_kv_write_ex(
                    _ptr(d.out), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), _ptr(slots),
                    d.shape[0], H, KVH, D, rotary_dim, page_size, _code(d.dtype), _ptr(d.part), d.splits,
                    _ptr(d.bias), self._stream()), "rope_kv_write")
                return d.out
            qkv = self.materialize(d)
        T = qkv.shape[0]
        self._check(self.lib.ts_rope_kv_write(
            _ptr(qkv), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), _ptr(slots),
            T, H, KVH, D, rotary_dim, page_size, _code(qkv.dtype), self._stream()), "rope_kv_write")
        return qkv

    # up to this many tokens the q/k/v product finishes itself (sum over its splits, bias, rotation,
    # cache write in its own epilogue) instead of leaving that to the rotary kernel (batch 24: 1.93
    # against 2.09 ms a step; batch 48: 2.12 against 2.27 ms, batch 64: 2.32 against 2.39 ms since the
    # block that finishes a token takes four pairs a thread)
    fused_qkv_tokens = int(os.environ.get("TURINGSERVE_B200_FUSED_QKV_TOKENS", "64"))

    def qkv_rope(self, out, x, w, bias, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                 page_size):
        """out[T, (H + 2 KVH) D] = x @ w^T + bias with q and k rotated, and the new keys and values
        written to the cache: one kernel for a few bfloat16 tokens with heads of 64 or 128 rotated over
        their full width, otherwise the product and then ``rope_kv_write``.  Returns the q/k/v tensor."""
        T, K = x.shape[0], w.shape[1]
        use_tc = self.gemm_mode == "tc" or (self.gemm_mode == "auto" and T <= 128)
        if (x.dtype == torch.bfloat16 and use_tc and T <= self.fused_qkv_tokens and D in (64, 128) and rotary_dim == D
                and cos is not None and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and self.lib.ts_linear_tc_supported(T, (H + 2 * KVH) * D, K)):
            splits = self.tc_splits(T, (H + 2 * KVH) * D, K)
            need = self.lib.ts_linear_tc_qkv_rope_scratch_floats(T, -(-(H + 2 * KVH) * D // 128), splits)
            qkv_part = self._buffer("qkv_part", need, torch.float32, x.device, floor=1 << 18)
            qkv_counters = self._buffer("qkv_counters", 4096, torch.int32, x.device, zero=True)
            if (H + 2 * KVH) * -(-T // 16) <= qkv_counters.numel():
                rc = self.lib.ts_linear_tc_qkv_rope(
                    _ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(qkv_part), _ptr(qkv_counters),
                    _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slots), _ptr(k_cache), _ptr(v_cache), T, H, KVH, D,
                    page_size, K, splits, self._stream())
                if rc != self.UNSUPPORTED:
                    self._check(rc, "linear_tc_qkv_rope")
                    return out
        if (self.pair_qkv and T > self.fused_qkv_tokens and x.dtype == torch.bfloat16 and D in (64, 128) and rotary_dim == D
                and cos is not None and cos.dtype == torch.float32 and x.is_contiguous()
                and self.pair_wins(T, (H + 2 * KVH) * D, K, 4.0 * T * (H + 2 * KVH) * D)):
            x = self.materialize(x)
            rc = self.lib.ts_linear_pair_qkv(
                _ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slots),
                _ptr(k_cache), _ptr(v_cache), T, H, KVH, D, page_size, K, self._stream())
            if rc != self.UNSUPPORTED:
                self._check(rc, "linear_pair_qkv")
                return out
        qkv = self.linear(out, x, w, bias, may_defer=True)
        return self.rope_kv_write(qkv, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots, page_size)

    def scratch(self, floats: int, device) -> torch.Tensor:
        """A float32 work buffer of at least ``floats`` elements, kept between calls."""
        return self._buffer("scratch", floats, torch.float32, device, floor=1 << 20)

    def decode_splits(self, num_requests: int, KVH: int, max_seq_len: int) -> int:
        """How many pieces each request's keys are cut into so that the launch fills the GPU
        (the cp.async decode kernel: two blocks per SM, pieces of at least 256 keys)."""
        want = -(-2 * self.num_sms // max(1, num_requests * KVH))
        return max(1, min(want, -(-max_seq_len // 256), 128))

    def decode_splits_tma(self, num_requests: int, KVH: int, D: int, max_seq_len: int) -> int:
        """The most pieces a request's keys may be cut into by the TMA decode kernel, which deals
        tiles of 64 keys out evenly over as many of them as get a tile: as many as one wave of
        blocks holds (the kernel itself uses fewer when the contexts are short)."""
        key = (D, self.decode_stages)
        if key not in self._decode_slots:
            self._decode_slots[key] = max(1, self.lib.ts_attention_decode_tma_blocks_per_sm(D, self.decode_stages))
        slots = self.num_sms * self._decode_slots[key]
        pairs = max(1, num_requests * KVH)
        tiles = max(1, -(-max_seq_len // 64))
        return max(1, min(slots // pairs, tiles, 128))

    def _decode_scratch(self, nd: int, H: int, KVH: int, D: int, nsplit: int, device):
        if nsplit <= 1:
            return None, None
        scratch = self.scratch(self.lib.ts_attention_decode_scratch_floats(nd, H, D, nsplit), device)
        # (one ticket counter per (request, kv head); the streaming kernel's two-level merge of more than 16
        # splits takes 16 more for each)
        return scratch, self._buffer("counters", nd * KVH * 17, torch.int32, device, floor=1 << 16, zero=True)

    def attention(self, out, qkv, k_cache, v_cache, block_tables, step, H, KVH, D, page_size, scale,
                  window) -> None:
        """Rows of requests with one token (the first ``step.num_decode`` requests) go to a
        split-key decode kernel when one takes the shape; the rest to the chunk kernels."""
        w = 0 if window is None else int(window)
        code = _code(qkv.dtype)
        B, nd = step.num_requests, 0
        width = block_tables.shape[1]
        streaming = self.decode_kernel == "tma"
        if self.decode_kernel == "auto":
            streaming = getattr(step, "streaming_decode", None)
            if streaming is None:
                streaming = step.num_decode * step.max_seq_len >= 98304
            # The other kernel is the faster one only while its blocks of 8 warps fit one per SM, eight to
            # a (request, kv head): from ten requests with two kv heads on, the streaming kernel wins at
            # every context (batch 12 x 2,048 keys: 12.3 against 18.7 us; batch 16 x 256 keys: 9.5 against 12.8)
            streaming = streaming or step.num_decode * KVH * 8 > self.num_sms
        if (self.use_fast_attention and streaming and step.num_decode > 0
                and self.lib.ts_attention_decode_tma_supported(H, KVH, D, page_size, code)):
            nd = step.num_decode
            nsplit = self.decode_splits_tma(nd, KVH, D, step.max_seq_len)
            scratch, counters = self._decode_scratch(nd, H, KVH, D, nsplit, qkv.device)
            rc = self.lib.ts_attention_decode_tma(
                _ptr(out), _ptr(scratch), _ptr(counters), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                _ptr(step.q_start), _ptr(step.seq_lens), nd, width, H, KVH, D, page_size, k_cache.shape[0],
                float(scale), w, nsplit, self.decode_stages, self._stream())
            if rc == self.UNSUPPORTED:          # e.g. key and value caches that no one tensor map spans
                nd = 0
            else:
                self._check(rc, "attention_decode_tma")
        if nd == 0 and self.use_fast_attention and step.num_decode > 0 and self.lib.ts_attention_decode_supported(H, KVH, D, code):
            nd = step.num_decode
            nsplit = self.decode_splits(nd, KVH, step.max_seq_len)
            scratch, counters = self._decode_scratch(nd, H, KVH, D, nsplit, qkv.device)
            self._check(self.lib.ts_attention_decode(
                _ptr(out), _ptr(scratch), _ptr(counters), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                _ptr(step.q_start), _ptr(step.seq_lens), nd, width, H, KVH, D, page_size, float(scale), w,
                nsplit, self._stream()), "attention_decode")
        if nd == B:
            return
        if (self.use_fast_attention and self.use_tc_attention
                and self.lib.ts_attention_prefill_tc_supported(H, KVH, D, page_size, code)):
            self._check(self.lib.ts_attention_prefill_tc(
                _ptr(out), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), block_tables.data_ptr() + 4 * nd * width,
                step.q_start.data_ptr() + 4 * nd, step.seq_lens.data_ptr() + 4 * nd, B - nd, width,
                step.max_q_len, H, KVH, D, page_size, k_cache.shape[0], float(scale), w, self._stream()),
                "attention_prefill_tc")
            return
        if self.use_fast_attention and self.lib.ts_attention_prefill_supported(H, KVH, D, code):
            self._check(self.lib.ts_attention_prefill(
                _ptr(out), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), block_tables.data_ptr() + 4 * nd * width,
                step.q_start.data_ptr() + 4 * nd, step.seq_lens.data_ptr() + 4 * nd, B - nd, width,
                step.max_q_len, H, KVH, D, page_size, float(scale), w, self._stream()), "attention_prefill")
            return
        self._check(self.lib.ts_attention_generic(
            _ptr(out), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), block_tables.data_ptr() + 4 * nd * width,
            step.q_start.data_ptr() + 4 * nd, step.seq_lens.data_ptr() + 4 * nd, B - nd, width,
            step.max_q_len, H, KVH, D, page_size, float(scale), w, code, self._stream()), "attention")

    def linear(self, out, x, w, bias=None, rows=None, may_defer: bool = False, lazy: bool = True):
        """out[M, N] = x[rows or all, :] @ w[N, K]^T + bias.  Returns ``out``; or, when ``may_defer``
        and the few-token tensor-core kernel takes the product, a ``LazyProduct`` (not launched yet:
        the norm that gets it with a residual launches it fused with the residual add) or a ``Deferred``
        whose sum the consuming norm finishes (``out`` is then left untouched)."""
        M, N = out.shape
        K = w.shape[1]
        x = self.materialize(x)
        use_tc = self.gemm_mode == "tc" or (self.gemm_mode == "auto" and M <= 128)
        if (may_defer and lazy and rows is None and use_tc and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and 0 < M <= self.fused_link_tokens and self.lib.ts_linear_tc_supported(M, N, K)
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return LazyProduct(out, x, w, bias)
        if x.dtype == torch.bfloat16 and (use_tc or self.use_library_gemm) and rows is not None:
            xg = torch.empty((M, K), dtype=x.dtype, device=x.device)
            self.gather_rows(xg, x, rows)
            x, rows = xg, None
        if (x.dtype == torch.bfloat16 and use_tc and self.lib.ts_linear_tc_supported(M, N, K)
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            splits = self.tc_splits(M, N, K)
            if may_defer and M <= 128 and N % 8 == 0 and out.dtype == torch.bfloat16:
                part = self.partial_scratch(splits * M * N, x.device)
                used = ctypes.c_int(0)
                self._check(self.lib.ts_linear_tc_ex(_ptr(out), _ptr(x), _ptr(w), None, _ptr(part), M, N, K, 0, splits,
                                                     1, ctypes.addressof(used), self._stream()), "linear_tc")
                return Deferred(part.view(-1)[: used.value * M * N].view(used.value, M, N), used.value, (M, N),
                                out.dtype, bias, out)
            scratch = self.scratch(splits * M * N, x.device) if splits > 1 else None
            self._check(self.lib.ts_linear_tc(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(scratch), M, N, K,
                                              1 if out.dtype == torch.float32 else 0, splits, self._stream()),
                        "linear_tc")
            if splits > 1:
                self.launches += 1
            return out
        if x.dtype == torch.bfloat16 and self.use_library_gemm:
            if out.dtype == torch.float32:
                torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
                if bias is not None:
                    out.add_(bias.float())
            elif bias is not None:
                torch.addmm(bias, x, w.t(), out=out)
            else:
                torch.mm(x, w.t(), out=out)
            return out
        self._check(self.lib.ts_linear_simt(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(rows), M, N, K,
                                            _code(x.dtype), _code(out.dtype), self._stream()), "linear")
        return out

    PAIR_PLAIN, PAIR_GATED = 0, 1
    # The many-row products whose epilogue saves a kernel (gate/up with the activation, q/k/v with rotation and
    # cache write) run on this library's kernel for pairs of SMs where its schedule is the shorter one; 0: never.
    # ("gated": the gate/up product only)
    pair_gemm = os.environ.get("TURINGSERVE_B200_PAIR_GEMM", "1") != "0"
    pair_qkv = os.environ.get("TURINGSERVE_B200_PAIR_GEMM", "1") not in ("0", "gated")

    def pair_wins(self, M: int, N: int, K: int, saved_bytes: float) -> bool:
        """Whether the pair kernel's schedule (rounds of 256 x 256 tiles over the pairs of SMs, 0.42 us a
        64-wide k-block: 79 us measured for 2,048 x 17,920 x 1,536, 353 us for 2,048 x 37,888 x 3,584) is shorter
        than the library product at 1.35 PFLOP/s followed by a kernel that moves ``saved_bytes`` at 5.5 TB/s
        (2,048 tokens of the 1.5B shape: 80 + 19 us; 544 tokens of the 14B shape: 113 + 9 us against 147)."""
        if not (self.pair_gemm and self.gemm_mode in ("auto", "tc")):
            return False
        tiles = -(-M // 256) * -(-N // 256)
        rounds = -(-tiles // max(1, self.num_sms // 2))
        pair_us = rounds * -(-K // 64) * 0.42 + 3.0
        library_us = 2.0 * M * N * K / 1.35e9 + 3.0 + saved_bytes / 5.5e6 + 2.0
        return pair_us < library_us

    def linear_pair(self, out, x, w, bias, epilogue: int) -> bool:
        """The many-row bfloat16 product on pairs of SMs.  ``epilogue`` PAIR_PLAIN: out[M, N] = x @ w^T + bias;
        PAIR_GATED: out[M, N / 2] = silu(g) * u, the rows of ``w`` in blocks of 64 gates and their 64 ups.
        False when the kernel does not take the shape."""
        M, K = x.shape
        N = w.shape[0]
        rc = self.lib.ts_linear_pair(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), M, N, K, epilogue, self._stream())
        if rc == self.UNSUPPORTED:
            return False
        self._check(rc, "linear_pair")
        return True

    def partial_scratch(self, floats: int, device) -> torch.Tensor:
        """The buffer deferred products leave their partial sums in (one deferred product at a time)."""
        return self._buffer("partials", floats, torch.float32, device, floor=1 << 20)

    def tc_splits(self, M: int, N: int, K: int) -> int:
        """Pieces K is cut into for a few-token product, so that about one tile lands on every SM."""
        if M > 128:
            return 1
        tiles = -(-N // 128)
        k_blocks = -(-K // 64)
        if tiles >= self.num_sms // 2:
            return 1
        # partial sums cost 8*M*N bytes per split (written, read back): keep that below the weights' 2*N*K
        traffic_cap = max(1, K // (4 * M))
        # every split is one more partial sum for the consuming kernel to fetch: at least four k-blocks
        # a split, ten splits at most (measured on the 1.5B shape at 8 tokens: 1.555 -> 1.501 ms a step
        # against twelve splits everywhere)
        return max(1, min(self.num_sms // tiles, max(2, k_blocks // 4), traffic_cap, self.max_splits))

    def tc_status(self) -> int:
        """0 when no tensor-core block (GEMM or attention) ever gave up on a wait (synchronises the device)."""
        return (int(self.lib.ts_linear_tc_status()) or int(self.lib.ts_attention_prefill_tc_status())
                or int(self.lib.ts_attention_decode_tma_status()) or int(self.lib.ts_decode_step_status()))

    STATUS_WORDS = 4            # what ts_sample* report beside the tokens: GEMM, prompt attention, TMA decode attention, fused decode step

    def fault_reported(self, status) -> str:
        """The engine found non-zero status words beside a step's tokens: a block of one of the
        kernels with bounded waits gave up, so the step's output cannot be trusted.  Takes the kernel
        concerned off the product path (its slower counterpart runs from the next step on), clears
        the words, and says what happened."""
        names = ("tensor-core product", "tensor-core prompt attention", "TMA decode attention", "fused decode step")
        hit = [f"{names[i]} (wait {int(v)})" for i, v in enumerate(status) if int(v)]
        if int(status[0]):
            self.gemm_mode = "library"
        if int(status[1]):
            self.use_tc_attention = False
        if int(status[2]):
            self.decode_kernel = "cp"
        if int(status[3]):
            self.use_fused_step = False
        self.lib.ts_clear_status(self._stream())
        return "a kernel gave up on a bounded wait: " + ", ".join(hit) + "; its fallback runs from now on"

    def feed_tokens(self, ids, rows, src, tokens, vocab: int) -> None:
        """ids[rows[i]] = tokens[src[i]] on the device (all int32)."""
        self._check(self.lib.ts_feed_tokens(_ptr(ids), _ptr(rows), _ptr(src), _ptr(tokens), rows.shape[0], vocab,
                                            self._stream()), "feed_tokens")

    def sample(self, out, logits, fparams, iparams, status_out=None) -> None:
        """``status_out``: STATUS_WORDS int32 that receive the kernels' status words (see fault_reported)."""
        S, V = logits.shape
        self._check(self.lib.ts_sample(_ptr(out), _ptr(logits), _ptr(fparams), _ptr(iparams), S, V,
                                       _ptr(status_out), self._stream()), "sample")

    def sample_greedy(self, out, logits, status_out=None) -> None:
        """Every row greedy: the draw without parameters, each row spread over many blocks."""
        S, V = logits.shape
        need = 2 * S * self.lib.ts_sample_greedy_parts(V)
        scratch = self._buffer("greedy_scratch", need, torch.int32, logits.device, floor=2 * 256 * 64)
        counters = self._buffer("greedy_counters", S, torch.int32, logits.device, floor=1024, zero=True)
        self._check(self.lib.ts_sample_greedy(_ptr(out), _ptr(logits), S, V, _ptr(scratch), _ptr(counters),
                                              _ptr(status_out), self._stream()), "sample_greedy")

    def penalize(self, logits, ids, meta, pen) -> None:
        S, V = logits.shape
        self._check(self.lib.ts_penalize(_ptr(logits), _ptr(ids), _ptr(meta), _ptr(pen), S, V,
                                         self._stream()), "penalize")


def ops():
    """The kernel object; builds and loads the CUDA library on first use.  Raises when there is
    no CUDA device or the library cannot be built: there is no fallback."""
    global _OPS
    if _OPS is None:
        if not torch.cuda.is_available():
            raise KernelError("turingserve_b200 needs a CUDA device (sm_100a); none is available")
        _OPS = CudaOps(build())
    return _OPS


def use(ops_object) -> None:
    """Install another object behind ``ops()`` (tests drive the engine's host logic with a plain
    torch twin of every kernel this way); ``use(None)`` goes back to the CUDA library."""
    global _OPS
    _OPS = ops_object


__all__ = ["CudaOps", "Deferred", "KernelError", "LazyProduct", "build", "library_path", "ops", "use"]
