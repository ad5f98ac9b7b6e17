"""Grouped-query softmax attention over the paged cache: fused q/k/v projection, position
encoding fused with the cache write, attention from the cache, output projection
(turingserve/model/qwen2.py:24-33,84-92; turingserve/ops/reference.py:50-57,94-111).

Each step writes the new keys and values first and then attends from the cache, so a prompt
portion and a single decoded token take the same path (turingserve/model/qwen2.py:88-90).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, CacheNeed, Mixer, ParamSpec, build, register


class Attention(Mixer):
    MAX_HEAD_DIM = 256          # the any-size attention kernel's limit; the faster ones take 64 and 128

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.KVH, self.D = int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        if self.H % self.KVH:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not 0 < self.D <= self.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {self.D}: the attention kernels take head sizes up to {self.MAX_HEAD_DIM}")
        self.scale = float(spec.scale)
        self.window = None if spec.window is None else int(spec.window)
        self.qkv_bias, self.out_bias = bool(spec.qkv_bias), bool(spec.out_bias)
        self.position = None if spec.position is None else build("position", spec.position, ctx)
        if self.position is not None and self.position.rotary_dim > self.D:
            raise ValueError("rotary_dim exceeds head_dim")
        self.q_dim, self.kv_dim = self.H * self.D, self.KVH * self.D
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"q_proj.weight": ParamSpec((self.q_dim, self.hidden)),
             "k_proj.weight": ParamSpec((self.kv_dim, self.hidden)),
             "v_proj.weight": ParamSpec((self.kv_dim, self.hidden)),
             "o_proj.weight": ParamSpec((self.hidden, self.q_dim))}
        if self.qkv_bias:
            p["q_proj.bias"] = ParamSpec((self.q_dim,))
            p["k_proj.bias"] = ParamSpec((self.kv_dim,))
            p["v_proj.bias"] = ParamSpec((self.kv_dim,))
        if self.out_bias:
            p["o_proj.bias"] = ParamSpec((self.hidden,))
        return p

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([t[f"{n}_proj.weight"] for n in "qkv"], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([t[f"{n}_proj.bias"] for n in "qkv"], dim=0).contiguous()
        self.w_o = t["o_proj.weight"].contiguous()
        if self.out_bias:
            self.b_o = t["o_proj.bias"].contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.KVH, self.D, self.window)

    def forward(self, x: torch.Tensor, step, cache, state=None) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        qkv = torch.empty((T, self.q_dim + 2 * self.kv_dim), dtype=x.dtype, device=x.device)
        grp = step.groups[cache.group]
        pos = self.position
        qkv = ops.qkv_rope(
            qkv, x, self.w_qkv, self.b_qkv, step.positions, None if pos is None else pos.cos,
            None if pos is None else pos.sin, self.H, self.KVH, self.D, 0 if pos is None else pos.rotary_dim,
            cache.k if cache.writable else None, cache.v if cache.writable else None,
            grp.slot_mapping, cache.page_size)
        attn = torch.empty((T, self.q_dim), dtype=x.dtype, device=x.device)
        ops.attention(attn, qkv, cache.k, cache.v, grp.block_tables, step, self.H, self.KVH, self.D,
                      cache.page_size, self.scale, self.window)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, attn, self.w_o, self.b_o, may_defer=True)


register("mixer", "attention", Attention)
