"""Plain PyTorch twins of the CUDA kernels, one function per kernel, with the same call
signature as ``turingserve_b200.kernels.CudaOps``.

Two uses: (1) the ``-m gpu`` tests compare each kernel alone with its twin; (2) the CPU tests
install ``TwinOps()`` behind ``kernels.ops()`` to drive the engine's HOST logic (cache manager,
batch builder, step function, scheduler, replay) without a GPU.  The product never uses this file.

Formulas: turingserve/ops/reference.py (rmsnorm :13-23, silu_mul :26-28, rope :31-42,
linear :45-47, kv_write :50-57, attention :60-77,94-111), sampling as
turingserve/sampling/sampler.py:45-107.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from tests import plain_qwen2 as plain


class TwinOps:
    def embedding(self, out, table, ids):
        out.copy_(table[ids.long()])

    def gather_rows(self, out, x, rows):
        out.copy_(x[rows.long()])

    def rmsnorm(self, out, x, weight, eps, residual=None):
        if residual is not None:
            residual.copy_(x + residual)
            x = residual
        x32 = x.float()
        y = (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
        out.copy_((weight.float() * y.float()).to(x.dtype))

    def silu_mul(self, out, gu, group=0):
        i = gu.shape[-1] // 2
        if group:
            blocks = gu.reshape(gu.shape[0], i // group, 2, group)
            g, u = blocks[:, :, 0].reshape(-1, i), blocks[:, :, 1].reshape(-1, i)
        else:
            g, u = gu[..., :i], gu[..., i:]
        out.copy_(F.silu(g) * u)

    def gated_linear(self, out, x, w, bias, group):
        gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype)
        self.linear(gu, x, w, bias)
        self.silu_mul(out, gu, group)

    def qkv_rope(self, out, x, w, bias, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                 page_size):
        self.linear(out, x, w, bias)
        return self.rope_kv_write(out, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots, page_size)

    def rope_kv_write(self, qkv, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                      page_size):
        T = qkv.shape[0]
        pos = positions.long()
        qk = qkv[:, : (H + KVH) * D].view(T, H + KVH, D)
        if rotary_dim:
            half = rotary_dim // 2
            c = cos[pos].to(qkv.dtype).float()[:, None, :]
            s = sin[pos].to(qkv.dtype).float()[:, None, :]
            x1, x2 = qk[..., :half].float(), qk[..., half:rotary_dim].float()
            o1, o2 = x1 * c - x2 * s, x2 * c + x1 * s
            qk[..., :half] = o1.to(qkv.dtype)
            qk[..., half:rotary_dim] = o2.to(qkv.dtype)
        if k_cache is None:
            return qkv
        k = qkv[:, H * D:(H + KVH) * D].view(T, KVH, D)
        v = qkv[:, (H + KVH) * D:].view(T, KVH, D)
        m = slots >= 0
        sl = slots[m].long()
        k_cache[sl // page_size, :, sl % page_size, :] = k[m]
        v_cache[sl // page_size, :, sl % page_size, :] = v[m]
        return qkv

    def attention(self, out, qkv, k_cache, v_cache, block_tables, step, H, KVH, D, page_size, scale,
                  window):
        paged_attention(out, qkv, k_cache, v_cache, block_tables, step.q_start, step.seq_lens,
                        H, KVH, D, page_size, scale, window)

    def linear(self, out, x, w, bias=None, rows=None, may_defer=False):
        if rows is not None:
            x = x[rows.long()]
        y = F.linear(x.float(), w.float(), None if bias is None else bias.float())
        out.copy_(y.to(out.dtype))
        return out

    def materialize(self, x):
        return x

    def sample(self, out, logits, fparams, iparams):
        S = logits.shape[0]
        for r in range(S):
            row = logits[r].float().cpu()
            if not torch.isfinite(row).all():
                out[0, r], out[1, r] = 0, 1
                continue
            tok, _ = plain.sample(row, float(fparams[r, 0]), int(iparams[r, 0]), float(fparams[r, 1]),
                                  int(iparams[r, 1]), int(iparams[r, 2]))
            out[0, r], out[1, r] = tok, 0

    def penalize(self, logits, ids, meta, pen):
        ids = ids.tolist()
        for r in range(logits.shape[0]):
            a, b, c, d = (int(x) for x in meta[r, :4])
            if c > a:
                logits[r] = plain.penalize(logits[r].cpu(), ids[a:b], ids[b:c], float(pen[r, 0]),
                                           float(pen[r, 1]), float(pen[r, 2])).to(logits.device)
            for t in ids[c:d]:
                logits[r, t] = float("-inf")


def paged_attention(out, qkv, k_cache, v_cache, block_tables, q_start, seq_lens, H, KVH, D, page_size,
                    scale, window):
    """Attention from the paged cache for a flat batch (turingserve/ops/reference.py:94-111 with the
    bottom-right mask of :60-77, plus the window)."""
    qsl = q_start.tolist()
    G = H // KVH
    out.zero_()
    for b, seq_len in enumerate(seq_lens.tolist()):
        qs, qe = qsl[b], qsl[b + 1]
        if seq_len == 0 or qe == qs:
            continue
        Tq = qe - qs
        nb = -(-seq_len // page_size)
        blocks = block_tables[b, :nb].long()
        kk = k_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, D)[:seq_len].float()
        vv = v_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, D)[:seq_len].float()
        q = qkv[qs:qe, : H * D].view(Tq, H, D).float().permute(1, 0, 2)
        kf = kk.repeat_interleave(G, dim=1).permute(1, 0, 2)
        vf = vv.repeat_interleave(G, dim=1).permute(1, 0, 2)
        scores = torch.matmul(q, kf.transpose(1, 2)) * scale
        i = torch.arange(Tq, device=qkv.device)[:, None] + (seq_len - Tq)
        j = torch.arange(seq_len, device=qkv.device)[None, :]
        ok = j <= i
        if window:
            ok = ok & (j > i - window)
        scores = scores.masked_fill(~ok, float("-inf"))
        p = torch.softmax(scores, dim=-1)
        # keys of pages a window gave back may hold anything: they carry zero weight, keep them out
        vf = torch.where(ok.any(0)[None, :, None], vf, torch.zeros_like(vf))
        o = torch.matmul(p, vf).permute(1, 0, 2).reshape(Tq, H * D)
        out[qs:qe] = o.to(out.dtype)
