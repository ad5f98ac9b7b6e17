"""Each part of the model alone on the GPU against the plain function of the same formula, at
sizes of its own (not those of the tiny models)."""

from __future__ import annotations

import dataclasses

import pytest
import torch
import torch.nn.functional as F

from tests import plain_qwen2 as plain
from turingserve_b200.config.model_config import AttentionSpec, GatedMLPSpec, LayerSpec, RMSNormSpec, RotarySpec
from turingserve_b200.parts.base import BuildContext, build, build_block

pytestmark = pytest.mark.gpu
TOL = {torch.float32: dict(atol=1e-4, rtol=1e-4), torch.bfloat16: dict(atol=3e-2, rtol=3e-2)}


def close(got, ref, dtype):
    """float32: element-wise 1e-4.  bfloat16: the largest error against 2% of the largest reference
    value (products of a few hundred bfloat16 terms; an element near zero carries the same absolute
    error as its neighbours)."""
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, **TOL[dtype])
    else:
        err, scale = (got - ref).abs().max().item(), ref.abs().max().item()
        assert err <= 0.02 * scale, (err, scale)


def ctx(hidden, dtype):
    from turingserve_b200 import kernels
    kernels.use(None)
    kernels.ops()
    return BuildContext(hidden_size=hidden, dtype=dtype, device=torch.device("cuda"), max_positions=512)


def rnd(shape, dtype, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    norm = build("norm", RMSNormSpec(eps=3e-5), ctx(200, dtype))
    assert list(norm.parameters()) == ["weight"] and norm.parameters()["weight"].shape == (200,)
    w, x, r = 1 + rnd((200,), dtype, 1, 0.1), rnd((9, 200), dtype, 2), rnd((9, 200), dtype, 3)
    norm.load({"weight": w.cuda()})
    y = norm.forward(x.cuda())
    torch.testing.assert_close(y.cpu().float(), plain.rmsnorm(x.float(), w.float(), 3e-5), **TOL[dtype])
    res = r.clone().cuda()
    y = norm.forward(x.cuda(), res)
    s = (x + r)
    assert torch.equal(res.cpu(), s)
    torch.testing.assert_close(y.cpu().float(), plain.rmsnorm(s.float(), w.float(), 3e-5), **TOL[dtype])


def test_rotary_part_tables():
    rot = build("position", RotarySpec(theta=12345.0, rotary_dim=24, max_positions=300), ctx(64, torch.float32))
    cos, sin = plain.rope_tables(24, 12345.0, 300)
    assert rot.cos.shape == (300, 12)
    torch.testing.assert_close(rot.cos.cpu(), cos, atol=0, rtol=0)
    torch.testing.assert_close(rot.sin.cpu(), sin, atol=0, rtol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    ffn = build("feed_forward", GatedMLPSpec(intermediate_size=136), ctx(72, dtype))
    t = {"gate_proj.weight": rnd((136, 72), dtype, 1, 0.2), "up_proj.weight": rnd((136, 72), dtype, 2, 0.2),
         "down_proj.weight": rnd((72, 136), dtype, 3, 0.2)}
    assert set(ffn.parameters()) == set(t)
    ffn.load({k: v.cuda() for k, v in t.items()})
    x = rnd((11, 72), dtype, 4)
    from turingserve_b200 import kernels
    y = kernels.ops().materialize(ffn.forward(x.cuda()))
    ref = plain.mlp(x.float(), *(t[k].float() for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    close(y.cpu().float(), ref, dtype)


@dataclasses.dataclass
class _Group:
    block_tables: torch.Tensor
    slot_mapping: torch.Tensor


@dataclasses.dataclass
class _Step:
    positions: torch.Tensor
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    groups: list
    num_requests: int
    num_decode: int
    max_q_len: int
    max_seq_len: int


@dataclasses.dataclass
class _View:
    group: int
    k: torch.Tensor
    v: torch.Tensor
    page_size: int
    writable: bool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,rot", [(None, 64), (13, 32), (None, 0)])
def test_attention_part_two_portions(dtype, window, rot):
    """The attention mixer alone: a prompt in two portions through a paged cache, against the plain
    whole-sequence attention with the same projections."""
    from turingserve_b200 import kernels
    H, KVH, D, hid, page = 6, 2, 64, 40, 8
    pos_spec = RotarySpec(theta=5000.0, rotary_dim=rot, max_positions=512) if rot else None
    spec = AttentionSpec(num_heads=H, num_kv_heads=KVH, head_dim=D, scale=0.2, qkv_bias=True, out_bias=True,
                         position=pos_spec, window=window)
    att = build("mixer", spec, ctx(hid, dtype))
    assert att.cache_need().window == window and att.state_need() is None
    t = {"q_proj.weight": rnd((H * D, hid), dtype, 1, 0.3), "k_proj.weight": rnd((KVH * D, hid), dtype, 2, 0.3),
         "v_proj.weight": rnd((KVH * D, hid), dtype, 3, 0.3), "o_proj.weight": rnd((hid, H * D), dtype, 4, 0.1),
         "q_proj.bias": rnd((H * D,), dtype, 5, 0.1), "k_proj.bias": rnd((KVH * D,), dtype, 6, 0.1),
         "v_proj.bias": rnd((KVH * D,), dtype, 7, 0.1), "o_proj.bias": rnd((hid,), dtype, 8, 0.1)}
    assert set(att.parameters()) == set(t)
    att.load({k: v.cuda() for k, v in t.items()})
    T = 37
    x = rnd((T, hid), dtype, 9)
    f = {k: v.float() for k, v in t.items()}
    q = F.linear(x.float(), f["q_proj.weight"], f["q_proj.bias"]).view(T, H, D)
    k = F.linear(x.float(), f["k_proj.weight"], f["k_proj.bias"]).view(T, KVH, D)
    v = F.linear(x.float(), f["v_proj.weight"], f["v_proj.bias"]).view(T, KVH, D)
    if rot:
        cos, sin = plain.rope_tables(rot, 5000.0, T)
        ar = torch.arange(T)
        q = torch.cat([plain.apply_rope(q[..., :rot], ar, cos, sin), q[..., rot:]], -1)
        k = torch.cat([plain.apply_rope(k[..., :rot], ar, cos, sin), k[..., rot:]], -1)
    ref = F.linear(plain.attention(q, k, v, 0.2, window), f["o_proj.weight"], f["o_proj.bias"])
    pages = 8
    kc = torch.zeros((pages, KVH, page, D), dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    table = torch.tensor([[5, 2, 7, 1, 3]], dtype=torch.int32, device="cuda")
    outs = []
    for a, b in ((0, 21), (21, T)):
        n = b - a
        pos = torch.arange(a, b, dtype=torch.int32, device="cuda")
        slots = (table[0][(pos // page).long()] * page + pos % page).to(torch.int32)
        step = _Step(pos, torch.tensor([0, n], dtype=torch.int32, device="cuda"),
                     torch.tensor([b], dtype=torch.int32, device="cuda"), [_Group(table, slots)], 1, 0, n, b)
        y = att.forward(x[a:b].cuda(), step, _View(0, kc, vc, page, True), None)
        outs.append(kernels.ops().materialize(y).cpu().float())
    close(torch.cat(outs), ref, dtype)


def test_block_part_wires_the_four_parts():
    norm = RMSNormSpec(eps=1e-6)
    att = AttentionSpec(num_heads=2, num_kv_heads=1, head_dim=16, scale=0.25, qkv_bias=False, out_bias=False,
                        position=RotarySpec(theta=1e4, rotary_dim=16, max_positions=64))
    blk = build_block(LayerSpec(mixer=att, feed_forward=GatedMLPSpec(intermediate_size=48), mixer_norm=norm, ffn_norm=norm),
                      ctx(32, torch.float32))
    assert set(blk.parts()) == {"mixer_norm", "mixer", "ffn_norm", "feed_forward"}
    with pytest.raises(ValueError, match="arrangement"):
        build_block(LayerSpec(mixer=att, feed_forward=GatedMLPSpec(intermediate_size=48), mixer_norm=norm, ffn_norm=norm,
                              arrangement="post_norm"), ctx(32, torch.float32))
    with pytest.raises(ValueError, match="no mixer registered"):
        build("mixer", dataclasses.replace(att, kind="linear_attention"), ctx(32, torch.float32))
