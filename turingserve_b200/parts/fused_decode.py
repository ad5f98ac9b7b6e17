"""A whole decode step as one kernel, for models whose layers are all of the kind the kernel is
written for.

``FusedDecodeStep.try_build(model, cache_views)`` looks at the parts the model was built from, not
at its name: every block a pre-norm block of an RMSNorm, an ``Attention`` mixer with heads of 128
rotated over their full width (or not rotated), another RMSNorm and a ``GatedMLP`` whose rows are
packed in blocks of 64; bfloat16; widths that are multiples of 64; a schedule that runs every layer
once with a cache of its own.  Anything else gives ``None`` and the step runs part by part
(``DecoderModel.forward``), which computes the same thing.

What the kernel does with these pointers is described in ``csrc/decode_step.cu``; the op order is
the decoder's, turingserve/model/qwen2.py:38-61,94-99.
"""

from __future__ import annotations

import ctypes
import os

import torch

from turingserve_b200 import kernels

MAX_TOKENS = 16
MAX_HIDDEN = 1536          # the in-kernel norm keeps a row of this many values in registers
MAX_GROUPS = 4
MAX_UNITS = 1024
MAX_PARTS = int(os.environ.get("TURINGSERVE_B200_STEP_PARTS", "16"))        # parts a product's K is cut into, at most
TICKETS = 4 * 512
HEAD_DIM = 128


class StepShape(ctypes.Structure):
    _fields_ = [("R", ctypes.c_int), ("KB", ctypes.c_int), ("S", ctypes.c_int), ("per", ctypes.c_int),
                ("rot", ctypes.c_int), ("pad", ctypes.c_int * 3)]


class StepLayer(ctypes.Structure):
    _fields_ = [("ln1_w", ctypes.c_void_p), ("ln2_w", ctypes.c_void_p), ("qkv_bias", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p), ("cos_t", ctypes.c_void_p),
                ("sin_t", ctypes.c_void_p), ("group", ctypes.c_int), ("window", ctypes.c_int)]


class StepArgs(ctypes.Structure):
    _fields_ = [("layers", ctypes.c_void_p), ("maps", ctypes.c_void_p),
                ("L", ctypes.c_int), ("T", ctypes.c_int), ("H", ctypes.c_int), ("KVH", ctypes.c_int),
                ("hidden", ctypes.c_int), ("inter", ctypes.c_int), ("V", ctypes.c_int), ("page", ctypes.c_int),
                ("norm_w_is_f32", ctypes.c_int), ("stages", ctypes.c_int), ("work_bytes", ctypes.c_int),
                ("lookahead", ctypes.c_int), ("attn_splits", ctypes.c_int),
                ("eps", ctypes.c_float), ("scale", ctypes.c_float),
                ("shape", StepShape * 5),
                ("ids", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("seq_lens", ctypes.c_void_p),
                ("block_tables", ctypes.c_void_p * MAX_GROUPS), ("slot_mapping", ctypes.c_void_p * MAX_GROUPS),
                ("table_width", ctypes.c_int * MAX_GROUPS), ("group_window", ctypes.c_int * MAX_GROUPS),
                ("num_groups", ctypes.c_int), ("num_pages", ctypes.c_int), ("l2_ahead", ctypes.c_int), ("pad1", ctypes.c_int),
                ("embedding", ctypes.c_void_p), ("final_norm_w", ctypes.c_void_p),
                ("resid", ctypes.c_void_p), ("qkv", ctypes.c_void_p), ("attn", ctypes.c_void_p),
                ("act", ctypes.c_void_p), ("logits", ctypes.c_void_p),
                ("attn_part", ctypes.c_void_p), ("ctrl", ctypes.c_void_p), ("tickets", ctypes.c_void_p),
                ("status", ctypes.c_void_p), ("trace", ctypes.c_void_p)]


def _cut(R: int, KB: int, blocks: int, splittable: bool) -> tuple[int, int]:
    """(parts, k-blocks a part) for a product of R tiles and KB k-blocks on ``blocks`` blocks: as many
    parts as give every block at most one unit, 16 at most, none shorter than two k-blocks."""
    if not splittable or R >= blocks:
        return 1, KB
    want = max(1, min(blocks // R, MAX_PARTS, max(1, KB // 2)))
    per = -(-KB // want)
    return -(-KB // per), per


class FusedDecodeStep:
    """Buffers, tensor maps and layer table of the one-kernel decode step for one model and cache."""

    enabled = os.environ.get("TURINGSERVE_B200_FUSED_STEP", "0") == "1"      # off until it beats the chain of kernels

    def __init__(self, model, views, lib, blocks: int, stages: int, work_bytes: int) -> None:
        self.model, self.lib, self.blocks, self.stages, self.work_bytes = model, lib, blocks, stages, work_bytes
        self.runs = 0                                                # steps this kernel has run (graph replays not counted)
        self.trace: torch.Tensor | None = None                       # set to an int64 [blocks, 5 L + 2, 8] tensor to record barrier times
        cfg = model.cfg
        dev = model.device
        att0 = model.blocks[0].mixer
        self.H, self.KVH = att0.H, att0.KVH
        self.hidden, self.inter, self.V = cfg.hidden_size, model.blocks[0].feed_forward.inter, cfg.vocab_size
        self.L = len(cfg.schedule)
        self.page = views[0].page_size
        self.num_pages = int(views[0].k.shape[0])
        self.eps = model.final_norm.eps
        self.scale = att0.scale
        self.lookahead = int(os.environ.get("TURINGSERVE_B200_STEP_LOOKAHEAD", "0"))
        self.l2_ahead = int(os.environ.get("TURINGSERVE_B200_STEP_L2_AHEAD", "1"))
        self.cooperative = os.environ.get("TURINGSERVE_B200_STEP_COOPERATIVE", "1") != "0"
        self.norm_w_is_f32 = 1
        # the kernel reads the norms' scales as 32-bit: converted once (the conversion is exact)
        self._scales = {}

        def scale32(norm) -> torch.Tensor:
            t = self._scales.get(id(norm))
            if t is None:
                t = self._scales[id(norm)] = norm.weight.float().contiguous()
            return t
        self._scale32 = scale32

        # tensor maps: per layer q/k/v, output, gate/up, down; then the head
        mats = []
        for r in range(self.L):
            b = model.blocks[cfg.schedule[r].layer]
            mats += [b.mixer.w_qkv, b.mixer.w_o, b.feed_forward.w_gate_up, b.feed_forward.w_down]
        mats.append(model.lm_head)
        host = ctypes.create_string_buffer(128 * len(mats))
        for i, w in enumerate(mats):
            rc = lib.ts_decode_step_encode_map(ctypes.byref(host, 128 * i), w.data_ptr(), w.shape[0], w.shape[1])
            if rc != 0:
                raise kernels.KernelError(f"decode step: tensor map {i}: {lib.ts_last_error().decode(errors='replace')}")
        self.maps = torch.frombuffer(bytearray(host.raw), dtype=torch.uint8).to(dev)
        self._mats = mats                                            # the maps hold their addresses

        layers = (StepLayer * self.L)()
        for r in range(self.L):
            b = model.blocks[cfg.schedule[r].layer]
            att, view = b.mixer, views[r]
            ly = layers[r]
            ly.ln1_w, ly.ln2_w = self._scale32(b.mixer_norm).data_ptr(), self._scale32(b.ffn_norm).data_ptr()
            ly.qkv_bias = None if att.b_qkv is None else att.b_qkv.data_ptr()
            ly.k_cache, ly.v_cache = view.k.data_ptr(), view.v.data_ptr()
            ly.cos_t = None if att.position is None else att.position.cos.data_ptr()
            ly.sin_t = None if att.position is None else att.position.sin.data_ptr()
            ly.group = view.group
            ly.window = 0 if att.window is None else int(att.window)
        self.layers = torch.frombuffer(bytearray(bytes(layers)), dtype=torch.uint8).to(dev)
        self.group_window = {views[r].group: (0 if model.blocks[cfg.schedule[r].layer].mixer.window is None
                                              else int(model.blocks[cfg.schedule[r].layer].mixer.window)) for r in range(self.L)}

        bf = torch.bfloat16
        n_qkv = (self.H + 2 * self.KVH) * HEAD_DIM
        self.resid = torch.zeros((MAX_TOKENS, self.hidden), dtype=torch.float32, device=dev)
        self.qkv = torch.zeros((MAX_TOKENS, n_qkv), dtype=torch.float32, device=dev)
        self.attn = torch.zeros((MAX_TOKENS, self.H * HEAD_DIM), dtype=bf, device=dev)
        self.act = torch.zeros((MAX_TOKENS, self.inter), dtype=bf, device=dev)
        self.attn_part = torch.empty((self.H // self.KVH) * blocks * (HEAD_DIM + 2) + 64, dtype=torch.float32, device=dev)
        self.ctrl = torch.zeros(16, dtype=torch.int32, device=dev)
        self.tickets = torch.zeros(TICKETS, dtype=torch.int32, device=dev)

        def shape(rows: int, k: int, splittable: bool) -> tuple[int, int, int, int]:
            R, KB = -(-rows // 128), k // 64
            S, per = _cut(R, KB, blocks, splittable)
            return R, KB, S, per
        self.shapes = [shape(n_qkv, self.hidden, True), shape(self.hidden, self.H * HEAD_DIM, True),
                       shape(2 * self.inter, self.hidden, False), shape(self.hidden, self.inter, True),
                       shape(self.V, self.hidden, False)]

    # -- can this model take the kernel? ----------------------------------------------------------------
    @classmethod
    def try_build(cls, model, views) -> FusedDecodeStep | None:
        from turingserve_b200.parts.attention import Attention
        from turingserve_b200.parts.block import PreNormBlock
        from turingserve_b200.parts.gated_mlp import GatedMLP
        from turingserve_b200.parts.rmsnorm import RMSNorm

        if not cls.enabled or model.dtype != torch.bfloat16 or model.device.type != "cuda":
            return None
        ops = kernels.ops()
        lib = getattr(ops, "lib", None)
        if lib is None or not hasattr(lib, "ts_decode_step"):
            return None
        cfg = model.cfg
        if type(model).embed is not _plain_model().embed or type(model).finish_logits is not _plain_model().finish_logits:
            return None                                              # a model class with hooks of its own
        if any(run.cache_from is not None for run in cfg.schedule) or len(cfg.schedule) != len(cfg.layers):
            return None
        if [run.layer for run in cfg.schedule] != list(range(len(cfg.layers))):
            return None
        first = model.blocks[0]
        if not isinstance(model.final_norm, RMSNorm) or model.final_norm.weight.dtype not in (torch.bfloat16, torch.float32):
            return None
        pages = set()
        for r, b in enumerate(model.blocks):
            if type(b) is not PreNormBlock or type(b.mixer) is not Attention or type(b.feed_forward) is not GatedMLP:
                return None
            if type(b.mixer_norm) is not RMSNorm or type(b.ffn_norm) is not RMSNorm:
                return None
            a, f, a0, f0 = b.mixer, b.feed_forward, first.mixer, first.feed_forward
            if (a.H, a.KVH, a.D, a.scale) != (a0.H, a0.KVH, a0.D, a0.scale) or f.inter != f0.inter:
                return None
            if a.D != HEAD_DIM or a.H // a.KVH > 16 or a.b_o is not None or f.bias or f.group != 64 or a.window is not None:
                return None
            if a.position is not None and (a.position.rotary_dim != HEAD_DIM or a.position.cos.dtype != torch.float32):
                return None
            for n in (b.mixer_norm, b.ffn_norm):
                if n.eps != model.final_norm.eps or n.weight.dtype != model.final_norm.weight.dtype:
                    return None
            v = views[r]
            if v is None or v.k is None or not v.writable or v.k.dtype != torch.bfloat16 or v.group >= MAX_GROUPS:
                return None
            pages.add(v.page_size)
        if len(pages) != 1 or (64 % next(iter(pages)) and next(iter(pages)) % 64) or cfg.hidden_size % 64 or first.feed_forward.inter % 64 or cfg.hidden_size > MAX_HIDDEN:
            return None
        stages = int(lib.ts_decode_step_max_stages(cfg.hidden_size))
        if stages < 3:
            return None
        stages = min(stages, int(os.environ.get("TURINGSERVE_B200_STEP_STAGES", "16")))
        blocks = int(lib.ts_decode_step_blocks(stages, cfg.hidden_size))
        if blocks < 8:
            return None
        me = cls(model, views, lib, blocks, stages, int(lib.ts_decode_step_work_bytes(cfg.hidden_size)))
        for R, KB, S, per in me.shapes[:2] + me.shapes[3:4]:
            if R * S > MAX_UNITS or R > 512:
                return None
        return me

    # -- one step -------------------------------------------------------------------------------------------
    def takes(self, step) -> bool:
        """Single-token requests only, at most 16 of them."""
        return (step.num_tokens == step.num_requests == step.num_decode and 1 <= step.num_tokens <= MAX_TOKENS
                and step.num_tokens * self.KVH <= min(self.blocks, 512))

    def run(self, step) -> torch.Tensor:
        """Logits [T, V] (32-bit) of every token of the step; new keys and values go into the cache."""
        T = step.num_tokens
        dev = self.model.device
        a = StepArgs()
        a.layers, a.maps = self.layers.data_ptr(), self.maps.data_ptr()
        a.L, a.T, a.H, a.KVH, a.hidden, a.inter, a.V, a.page = (self.L, T, self.H, self.KVH, self.hidden, self.inter,
                                                                self.V, self.page)
        a.norm_w_is_f32, a.stages, a.work_bytes, a.lookahead = self.norm_w_is_f32, self.stages, self.work_bytes, self.lookahead
        a.attn_splits = max(1, min(self.blocks // (T * self.KVH), -(-max(step.max_seq_len, 1) // 64), 128))
        a.eps, a.scale = self.eps, self.scale
        at = 0
        for k, (R, KB, S, per) in enumerate(self.shapes):
            sh = a.shape[k]
            sh.R, sh.KB, sh.S, sh.per = R, KB, S, per
            sh.rot = (self.blocks - at) % self.blocks
            at = (at + R * S) % self.blocks
        a.ids, a.positions, a.seq_lens = step.input_ids.data_ptr(), step.positions.data_ptr(), step.seq_lens.data_ptr()
        for g, grp in enumerate(step.groups):
            a.block_tables[g], a.slot_mapping[g] = grp.block_tables.data_ptr(), grp.slot_mapping.data_ptr()
            a.table_width[g] = grp.block_tables.shape[1]
            a.group_window[g] = self.group_window.get(g, 0)
        a.num_groups = len(step.groups)
        a.l2_ahead = self.l2_ahead
        a.num_pages = self.num_pages
        a.embedding, a.final_norm_w = self.model.embedding.data_ptr(), self._scale32(self.model.final_norm).data_ptr()
        logits = torch.empty((T, self.V), dtype=torch.float32, device=dev)
        a.resid, a.qkv, a.attn, a.act = (t.data_ptr() for t in (self.resid, self.qkv, self.attn, self.act))
        a.logits, a.attn_part = logits.data_ptr(), self.attn_part.data_ptr()
        a.ctrl, a.tickets = self.ctrl.data_ptr(), self.tickets.data_ptr()
        a.trace = None if self.trace is None else self.trace.data_ptr()
        ops = kernels.ops()
        rc = self.lib.ts_decode_step(ctypes.byref(a), self.blocks, 1 if self.cooperative else 0, ctypes.c_void_p(ops._stream()))
        ops._check(rc, "decode_step")
        self.runs += 1
        return logits


def _plain_model():
    from turingserve_b200.parts.model import DecoderModel
    return DecoderModel
