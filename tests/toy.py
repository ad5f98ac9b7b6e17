"""A toy architecture defined entirely in the test-suite: it registers a mixer with per-request state
of its own (a running mean), a feed-forward that routes every token to one of several small
experts, a position encoding of its own (rotation by a fraction of the position), a position-free
attention layer, and a run schedule that names a layer twice and lets a run read another run's
cache; a block arrangement with a third norm (a part in a role the built-in arrangement does not
have) and a model class that scales its embeddings and caps its logits, registered with the
architecture.  Nothing under ``turingserve_b200`` knows about it; it is no model of anyone's.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from turingserve_b200.config.model_config import (
    AttentionSpec, GatedMLPSpec, LayerRun, LayerSpec, ModelConfig, RMSNormSpec, RotarySpec)
from turingserve_b200.config.registry import Architecture, LayerTensorNames, TensorNames, register_architecture
from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, FeedForward, Mixer, ParamSpec, StateNeed, build, register
from turingserve_b200.parts.model import DecoderModel

NAME = "ToyStateLM"


@dataclass(frozen=True)
class RunningMeanSpec:
    """y_t = W . mean(x_0 .. x_t): the state is the running sum and the count."""

    kind: str = "running_mean"


class RunningMeanMixer(Mixer):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.h = ctx.hidden_size
        self.w = None

    def parameters(self):
        return {"proj.weight": ParamSpec((self.h, self.h))}

    def load(self, t):
        self.w = t["proj.weight"]

    def state_need(self):
        return StateNeed((self.h + 1,), torch.float32)

    def forward(self, x, step, cache, state):
        slots = step.state_slots.tolist()
        out = torch.empty_like(x)
        at = 0
        for b, n in enumerate(step.q_lens):
            if step.seq_lens is not None and n == 0:
                continue
            st = state[slots[b]]
            if step.starts[b] == 0:
                st.zero_()                                   # the first portion of a request starts clean
            rows = x[at:at + n].float()
            sums = rows.cumsum(0) + st[: self.h]
            counts = st[self.h] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
            mean = (sums / counts[:, None]).to(x.dtype)
            out[at:at + n] = F.linear(mean.float(), self.w.float()).to(x.dtype)
            st[: self.h] = sums[-1]
            st[self.h] = counts[-1]
            at += n
        return out


register("mixer", "running_mean", RunningMeanMixer)


@dataclass(frozen=True)
class OneOfExpertsSpec:
    """y = p_e(x) . down_e(silu(gate_e(x)) * up_e(x)) for the expert e with the largest router logit;
    p = softmax of the router logits, in 32-bit."""

    num_experts: int
    intermediate_size: int
    kind: str = "one_of_experts"


class OneOfExperts(FeedForward):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.h, self.n, self.inter = ctx.hidden_size, int(spec.num_experts), int(spec.intermediate_size)
        self.t = None

    def parameters(self):
        p = {"router.weight": ParamSpec((self.n, self.h), compute_dtype=False)}
        for e in range(self.n):
            p[f"experts.{e}.gate_proj.weight"] = ParamSpec((self.inter, self.h))
            p[f"experts.{e}.up_proj.weight"] = ParamSpec((self.inter, self.h))
            p[f"experts.{e}.down_proj.weight"] = ParamSpec((self.h, self.inter))
        return p

    def load(self, t):
        self.t = t

    def forward(self, x):
        probs = F.linear(x.float(), self.t["router.weight"].float()).softmax(-1)       # 32-bit routing
        weight, choice = probs.max(-1)
        out = torch.zeros_like(x)
        for e in range(self.n):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            xe = x[rows]
            g = F.linear(xe, self.t[f"experts.{e}.gate_proj.weight"])
            u = F.linear(xe, self.t[f"experts.{e}.up_proj.weight"])
            y = F.linear(F.silu(g) * u, self.t[f"experts.{e}.down_proj.weight"])
            out[rows] = (y.float() * weight[rows, None]).to(x.dtype)
        return out


register("feed_forward", "one_of_experts", OneOfExperts)


@dataclass(frozen=True)
class SlowRotarySpec:
    """Rotate-half rotation whose angle is position / slowdown times the usual frequency."""

    theta: float
    rotary_dim: int
    max_positions: int
    slowdown: float
    kind: str = "slow_rope"


class SlowRotary:
    """What the attention mixer asks of a position encoding: rotary_dim and 32-bit cos / sin tables
    [positions, rotary_dim / 2] on the device."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.rotary_dim = int(spec.rotary_dim)
        n = min(int(spec.max_positions), ctx.max_positions) if ctx.max_positions else int(spec.max_positions)
        self.max_positions = n
        self.cos, self.sin = (t.to(ctx.device).contiguous()
                              for t in slow_tables(self.rotary_dim, float(spec.theta), n, float(spec.slowdown)))


def slow_tables(rot: int, theta: float, n: int, slowdown: float):
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    freqs = torch.outer(torch.arange(n).float() / slowdown, inv_freq)
    return freqs.cos(), freqs.sin()


register("position", "slow_rope", SlowRotary)


class SandwichBlock:
    """h += after(mixer(before(h))); h += ffn(norm(h)): a third norm, in a role of its own
    ("mixer_after_norm"), and residual adds done on the spot instead of deferred."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.before = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.after = build("norm", spec.mixer_after_norm, ctx)
        self.ffn_norm = build("norm", spec.ffn_norm, ctx)
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx)

    def parts(self):
        return {"mixer_norm": self.before, "mixer": self.mixer, "mixer_after_norm": self.after,
                "ffn_norm": self.ffn_norm, "feed_forward": self.feed_forward}

    @staticmethod
    def _tensor(x):
        ops = kernels.ops()
        return ops.materialize(x) if hasattr(ops, "materialize") else x

    def forward(self, h, residual, step, cache, state):
        assert residual is None
        a = self.mixer.forward(self.before.forward(h), step, cache, state)
        h = h + self.after.forward(self._tensor(a))
        h = h + self._tensor(self.feed_forward.forward(self.ffn_norm.forward(h)))
        return h, None


register("block", "sandwich", SandwichBlock)


class ScaledModel(DecoderModel):
    """The plain decoder with its embeddings multiplied by a constant and its logits capped by
    cap * tanh(logits / cap); both constants come from the configuration's extras."""

    def embed(self, step):
        return (super().embed(step).float() * float(self.cfg.extra("embedding_multiplier", 1.0))).to(self.dtype)

    def finish_logits(self, logits):
        cap = self.cfg.extra("logit_cap")
        return logits if cap is None else float(cap) * torch.tanh(logits / float(cap))


def parse_config(c: dict, gen=None) -> ModelConfig:
    h, heads, kv, d = c["width"], c["heads"], c["kv_heads"], c["head_size"]
    norm = RMSNormSpec(eps=c["eps"])
    dense = GatedMLPSpec(intermediate_size=c["ffn_width"])
    rope = RotarySpec(theta=c["theta"], rotary_dim=c.get("rotary_dim", d), max_positions=c["max_positions"])
    slow = SlowRotarySpec(theta=c["theta"], rotary_dim=c.get("rotary_dim", d), max_positions=c["max_positions"],
                          slowdown=c.get("slowdown", 1.0))
    ffns = c.get("ffns", ["dense"] * len(c["mixers"]))
    layers = []
    for kind, ffn_kind in zip(c["mixers"], ffns):
        if kind == "mean":
            mixer = RunningMeanSpec()
        else:
            position = None if kind == "nope" else (slow if kind == "slow" else rope)
            mixer = AttentionSpec(num_heads=heads, num_kv_heads=kv, head_dim=d, scale=c.get("scale", d ** -0.5),
                                  qkv_bias=False, out_bias=True, position=position,
                                  window=c.get("window") if kind == "window" else None)
        ffn = dense if ffn_kind == "dense" else OneOfExpertsSpec(c["experts"], c["expert_width"])
        if c.get("arrangement", "pre_norm") == "sandwich":
            layers.append(LayerSpec("sandwich", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    mixer_after_norm=RMSNormSpec(eps=10 * c["eps"]), ffn_norm=norm))
        else:
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm))
    schedule = tuple(LayerRun(l, f) for l, f in c.get("schedule", [(i, None) for i in range(len(layers))]))
    extras = tuple((k, c[k]) for k in ("embedding_multiplier", "logit_cap") if k in c)
    return ModelConfig(architecture=NAME, hidden_size=h, vocab_size=c["vocab"], layers=tuple(layers),
                       schedule=schedule, final_norm=norm, tie_word_embeddings=False,
                       max_position_embeddings=c["max_positions"], extras=extras)


def tensor_names(cfg: ModelConfig) -> TensorNames:
    layers = tuple(LayerTensorNames(mixer=f"blocks.{i}.mix.", feed_forward=f"blocks.{i}.ffn.",
                                    mixer_norm=f"blocks.{i}.norm_a.", ffn_norm=f"blocks.{i}.norm_b.",
                                    **({"mixer_after_norm": f"blocks.{i}.norm_mid."}
                                       if "mixer_after_norm" in cfg.layers[i].roles else {}))
                   for i in range(len(cfg.layers)))
    return TensorNames(embedding="embed.weight", lm_head="head.weight", final_norm="norm_out.", layers=layers)


_JSON: dict[int, dict] = {}


def to_config_json(cfg: ModelConfig) -> dict:
    return _JSON[id(cfg)]


def make(c: dict) -> ModelConfig:
    c = {"architectures": [NAME], **c}
    cfg = parse_config(c)
    _JSON[id(cfg)] = c
    return cfg


register_architecture(Architecture(NAME, parse_config, tensor_names, to_config_json, build_model=ScaledModel))


# -- a plain whole-sequence implementation of the toy model (for the tests only) ------------------------
def plain_forward(c: dict, w: dict, ids: list[int]) -> torch.Tensor:
    from tests import plain_qwen2 as plain
    x_ids = torch.as_tensor(ids, dtype=torch.long)
    T = len(ids)
    h = w["embed.weight"][x_ids] * c.get("embedding_multiplier", 1.0)
    sandwich = c.get("arrangement", "pre_norm") == "sandwich"
    d, H, KVH = c["head_size"], c["heads"], c["kv_heads"]
    rot = c.get("rotary_dim", d)
    cos, sin = plain.rope_tables(rot, c["theta"], T)
    slow_cos, slow_sin = slow_tables(rot, c["theta"], T, c.get("slowdown", 1.0))
    ffns = c.get("ffns", ["dense"] * len(c["mixers"]))
    pos = torch.arange(T)
    kept = []
    schedule = c.get("schedule", [(i, None) for i in range(len(c["mixers"]))])

    def rope(t, cs, sn):
        if rot == d:
            return plain.apply_rope(t, pos, cs, sn)
        return torch.cat([plain.apply_rope(t[..., :rot], pos, cs, sn), t[..., rot:]], dim=-1)

    def experts(x, p):
        probs = F.linear(x, w[p + "router.weight"]).softmax(-1)
        weight, choice = probs.max(-1)
        rows = []
        for t in range(x.shape[0]):
            e = f"{p}experts.{int(choice[t])}."
            rows.append(weight[t] * plain.mlp(x[t:t + 1], w[e + "gate_proj.weight"], w[e + "up_proj.weight"],
                                              w[e + "down_proj.weight"])[0])
        return torch.stack(rows)

    for layer, cache_from in schedule:
        p = f"blocks.{layer}."
        kind = c["mixers"][layer]
        x = plain.rmsnorm(h, w[p + "norm_a.weight"], c["eps"])
        if kind == "mean":
            mean = x.cumsum(0) / torch.arange(1, T + 1)[:, None]
            a = F.linear(mean, w[p + "mix.proj.weight"])
            kept.append(None)
        else:
            q = F.linear(x, w[p + "mix.q_proj.weight"]).view(T, H, d)
            k = F.linear(x, w[p + "mix.k_proj.weight"]).view(T, KVH, d)
            v = F.linear(x, w[p + "mix.v_proj.weight"]).view(T, KVH, d)
            if kind == "slow":
                q, k = rope(q, slow_cos, slow_sin), rope(k, slow_cos, slow_sin)
            elif kind != "nope":
                q, k = rope(q, cos, sin), rope(k, cos, sin)
            if cache_from is not None:
                k, v = kept[cache_from]
            kept.append((k, v))
            a = plain.attention(q, k, v, c.get("scale", d ** -0.5), c.get("window") if kind == "window" else None)
            a = F.linear(a, w[p + "mix.o_proj.weight"], w[p + "mix.o_proj.bias"])
        if sandwich:
            a = plain.rmsnorm(a, w[p + "norm_mid.weight"], 10 * c["eps"])
        h = h + a
        x = plain.rmsnorm(h, w[p + "norm_b.weight"], c["eps"])
        if ffns[layer] == "dense":
            h = h + plain.mlp(x, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
        else:
            h = h + experts(x, p + "ffn.")
    logits = F.linear(plain.rmsnorm(h, w["norm_out.weight"], c["eps"]), w["head.weight"]).float()
    if "logit_cap" in c:
        logits = c["logit_cap"] * torch.tanh(logits / c["logit_cap"])
    return logits


TOY = {"width": 48, "heads": 6, "kv_heads": 2, "head_size": 16, "rotary_dim": 8, "ffn_width": 72, "vocab": 211,
       "eps": 2e-5, "theta": 777.0, "max_positions": 300, "window": 9, "scale": 0.3,
       "mixers": ["rope", "mean", "window", "nope"],
       "schedule": [(0, None), (1, None), (2, None), (0, None), (3, None), (3, 4), (1, None)]}

# A second toy: a routed feed-forward in two of its layers and the slowed rotation in one.  Compared in
# 32-bit only: in bfloat16 a token whose two best router logits nearly tie may go to the other expert.
TOY_ROUTED = {"width": 40, "heads": 4, "kv_heads": 1, "head_size": 32, "ffn_width": 56, "vocab": 157,
              "eps": 1e-5, "theta": 5000.0, "max_positions": 200, "slowdown": 3.5, "experts": 3, "expert_width": 24,
              "mixers": ["slow", "mean", "rope"], "ffns": ["experts", "dense", "experts"]}

# A third toy: every layer in the arrangement with three norms, embeddings scaled and logits capped by
# the model class the architecture registers.
TOY_SANDWICH = {"width": 56, "heads": 2, "kv_heads": 2, "head_size": 24, "ffn_width": 88, "vocab": 173,
                "eps": 3e-6, "theta": 9000.0, "max_positions": 160, "arrangement": "sandwich",
                "embedding_multiplier": 7.5, "logit_cap": 1.5, "mixers": ["rope", "mean", "nope"]}
