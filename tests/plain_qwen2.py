"""A plain, slow Qwen2 decoder in PyTorch on the CPU: whole sequences, no cache, one function per
part.  It is the oracle of the test-suite and shares no code with ``turingserve_b200``: it reads
``config.json`` as a dict and the checkpoint as a dict of tensors by their Hugging Face names.

Written from the formulas of the reference (Muskanpandey0304/TuringServe); each function cites
the file and lines it restates.  ``tests/golden/make_golden.py`` compared it once with the
reference's own model code on tiny random models; ``tests/test_plain.py`` checks it against
those stored outputs.

Beyond the reference: a sliding window (the reference rejects ``use_sliding_window``,
turingserve/model/qwen2_config.py:40-41) and an explicit run schedule, both only to test the
engine's generality.  The window mask is the usual one: the query at position p sees keys
p-w+1 .. p.
"""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch
import torch.nn.functional as F
from safetensors.torch import load_file


# -- reading a model folder -------------------------------------------------------------------------
def read_folder(folder: str, dtype=torch.float32):
    """(config dict, {HF tensor name: tensor in ``dtype``})."""
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = {}
    for fn in sorted(os.listdir(folder)):
        if fn.endswith(".safetensors"):
            tensors.update(load_file(os.path.join(folder, fn)))
    return cfg, {k: v.to(dtype) for k, v in tensors.items()}


def sizes(cfg: dict) -> dict:
    """Sizes as turingserve/model/qwen2_config.py:52-63 derives them (plus an optional head_dim key)."""
    H, KVH = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or cfg["hidden_size"] // H
    rp = cfg.get("rope_parameters") or {}
    return dict(H=H, KVH=KVH, D=D, G=H // KVH, L=cfg["num_hidden_layers"],
                eps=float(cfg.get("rms_norm_eps", 1e-6)),
                theta=float(cfg.get("rope_theta", rp.get("rope_theta", 10000.0))),
                tied=bool(cfg.get("tie_word_embeddings", False)))


def layer_window(cfg: dict, layer: int) -> int | None:
    """Layers from ``max_window_layers`` on use the sliding window when it is switched on."""
    if not cfg.get("use_sliding_window"):
        return None
    return cfg["sliding_window"] if layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]) else None


# -- parts ----------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """turingserve/ops/reference.py:13-16: statistics in fp32, cast BEFORE the weight."""
    x32 = x.float()
    x32 = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    return w * x32.to(x.dtype)


def rope_tables(head_dim: int, theta: float, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """turingserve/model/layers.py:13-18."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = torch.outer(torch.arange(n).float(), inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, heads, D]; rotate-half, turingserve/ops/reference.py:31-42."""
    D = x.shape[-1]
    c = cos[positions].to(x.dtype)[:, None, :]
    s = sin[positions].to(x.dtype)[:, None, :]
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int | None = None) -> torch.Tensor:
    """q [T,H,D], k/v [T,KVH,D] of ONE whole sequence -> [T, H*D].
    turingserve/ops/reference.py:60-77 (Tq == Tk here, so the mask is j <= i)."""
    T, H, D = q.shape
    G = H // k.shape[1]
    qf = q.float().permute(1, 0, 2)
    kf = k.float().repeat_interleave(G, dim=1).permute(1, 0, 2)
    vf = v.float().repeat_interleave(G, dim=1).permute(1, 0, 2)
    scores = torch.matmul(qf, kf.transpose(1, 2)) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    allowed = j <= i
    if window is not None:
        allowed = allowed & (j > i - window)
    scores = scores.masked_fill(~allowed, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.matmul(p, vf).permute(1, 0, 2).reshape(T, H * D).to(q.dtype)


def mlp(x: torch.Tensor, gate_w, up_w, down_w) -> torch.Tensor:
    """turingserve/model/qwen2.py:35-36 with turingserve/ops/reference.py:26-28."""
    return F.linear(F.silu(F.linear(x, gate_w)) * F.linear(x, up_w), down_w)


def qkv_projection(x, w: dict, p: str, s: dict):
    """turingserve/model/qwen2.py:24-33 (fused there, loader.py:82-83; separate products here)."""
    T = x.shape[0]
    q = F.linear(x, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, s["H"], s["D"])
    k = F.linear(x, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, s["KVH"], s["D"])
    v = F.linear(x, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, s["KVH"], s["D"])
    return q, k, v


# -- the model --------------------------------------------------------------------------------------
@torch.inference_mode()
def forward(cfg: dict, w: dict, token_ids, schedule=None, return_hidden: bool = False):
    """Logits [T, V] (fp32) of one whole sequence.  Op order of turingserve/model/qwen2.py:38-61
    with the deferred residual add of :42-57; output head :94-99.

    ``schedule``: optional list of (layer, cache_from) pairs; default one run per layer.
    """
    s = sizes(cfg)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    T = ids.shape[0]
    pos = torch.arange(T)
    cos, sin = rope_tables(s["D"], s["theta"], T)
    scale = s["D"] ** -0.5
    runs = schedule if schedule is not None else [(i, None) for i in range(s["L"])]
    h = w["model.embed_tokens.weight"][ids]
    residual = None
    kept_kv: list = []
    hiddens = []
    for layer, cache_from in runs:
        p = f"model.layers.{layer}."
        if residual is None:
            residual = h
        else:
            residual = h + residual
        hiddens.append(residual)
        x = rmsnorm(residual, w[p + "input_layernorm.weight"], s["eps"])
        q, k, v = qkv_projection(x, w, p, s)
        q = apply_rope(q, pos, cos, sin)
        if cache_from is None:
            k = apply_rope(k, pos, cos, sin)
        else:
            k, v = kept_kv[cache_from]
        kept_kv.append((k, v))
        a = attention(q, k, v, scale, layer_window(cfg, layer))
        h = F.linear(a, w[p + "self_attn.o_proj.weight"])
        residual = h + residual
        x = rmsnorm(residual, w[p + "post_attention_layernorm.weight"], s["eps"])
        h = mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = rmsnorm(h + residual, w["model.norm.weight"], s["eps"])
    head = w["model.embed_tokens.weight"] if s["tied"] else w["lm_head.weight"]
    logits = F.linear(x, head).float()
    if return_hidden:
        return logits, hiddens + [x]
    return logits


@torch.inference_mode()
def greedy(cfg: dict, w: dict, prompt: list[int], max_new_tokens: int, eos_ids=()) -> list[int]:
    """Greedy continuation by running the whole sequence again for every token
    (what turingserve/simple_generate.py:10-31 computes with a cache)."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        tok = int(forward(cfg, w, ids)[-1].argmax())
        out.append(tok)
        ids.append(tok)
        if tok in eos_ids:
            break
    return out


# -- sampling ---------------------------------------------------------------------------------------
def _philox_first_word(c, k):
    """Philox4x32-10, first output word; c = 4 counters, k = 2 keys (numpy uint32 arrays/scalars)."""
    c0, c1, c2, c3 = (np.asarray(v, dtype=np.uint64) for v in c)
    k0, k1 = (np.uint64(v) for v in k)
    M0, M1, mask = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c0.astype(np.uint32)


def exponential_noise(seed: int, drawn: int, vocab: int) -> np.ndarray:
    """E ~ Exp(1) per vocabulary entry for a request's ``drawn``-th draw: the engine's
    counter-based stand-in for ``exponential_`` in turingserve/sampling/sampler.py:95-102."""
    seed &= (1 << 64) - 1
    i = np.arange(vocab, dtype=np.uint64)
    z = np.zeros(vocab, dtype=np.uint64)
    r = _philox_first_word((i, z + np.uint64(drawn & 0xFFFFFFFF), z + np.uint64(drawn >> 32), z),
                           (seed & 0xFFFFFFFF, seed >> 32))
    u = ((r >> np.uint32(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -np.log(u).astype(np.float32)


def penalize(logits: torch.Tensor, prompt_ids, output_ids, repetition, presence, frequency) -> torch.Tensor:
    """One row; turingserve/sampling/penalties.py:20-45."""
    V = logits.shape[0]
    counts = torch.zeros(V)
    for t in output_ids:
        counts[t] += 1
    seen = torch.zeros(V, dtype=torch.bool)
    seen[list(prompt_ids) + list(output_ids)] = True
    pen = torch.where(logits > 0, logits / repetition, logits * repetition)
    logits = torch.where(seen, pen, logits)
    logits = logits - frequency * counts
    return logits - presence * (counts > 0).float()


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """One row [V]; turingserve/sampling/sampler.py:45-65."""
    V = logits.shape[0]
    scaled = logits / temperature
    if top_k == -1 and top_p >= 1.0:
        return torch.softmax(scaled, dim=-1)
    sl, si = scaled.sort(descending=True)
    pos = torch.arange(V)
    k = V if top_k < 0 else top_k
    sl = sl.masked_fill(pos >= k, float("-inf"))
    probs = torch.softmax(sl, dim=-1)
    cum_before = probs.cumsum(-1) - probs
    sl = sl.masked_fill((cum_before >= top_p) & (pos > 0), float("-inf"))
    sp = torch.softmax(sl, dim=-1)
    out = torch.zeros_like(sp)
    out.scatter_(0, si, sp)
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, drawn: int):
    """One row -> (token, scores) with scores = probs / E; greedy when temperature < 1e-5
    (turingserve/sampling/sampler.py:87-104, turingserve/engine/sampling_params.py:45-47)."""
    if temperature < 1e-5:
        return int(logits.argmax()), None
    probs = filtered_probs(logits.float(), temperature, top_k, top_p)
    scores = probs / torch.from_numpy(exponential_noise(seed, drawn, logits.shape[0]))
    return int(scores.argmax()), scores
