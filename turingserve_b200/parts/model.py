"""The decoder: embedding, the layers in schedule order, final norm, output head.

Op order as turingserve/model/qwen2.py:38-61 and :94-99.  The schedule is data
(``ModelConfig.schedule``): a layer may run twice, and a run may read an earlier run's cache.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.config.model_config import ModelConfig
from turingserve_b200.config.registry import TensorNames
from turingserve_b200.parts.base import BuildContext, ParamSpec, build, build_block


class DecoderModel:
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device, max_positions: int) -> None:
        self.cfg = cfg
        self.dtype = dtype
        self.device = torch.device(device)
        ctx = BuildContext(hidden_size=cfg.hidden_size, dtype=dtype, device=self.device,
                           max_positions=max_positions)
        self.blocks = [build_block(spec, ctx) for spec in cfg.layers]
        self.final_norm = build("norm", cfg.final_norm, ctx)
        self.embedding: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None

    # -- weights ---------------------------------------------------------------------------------
    def parameters(self, names: TensorNames) -> dict[str, ParamSpec]:
        """Every checkpoint tensor this model reads: full name -> spec."""
        c = self.cfg
        out = {names.embedding: ParamSpec((c.vocab_size, c.hidden_size))}
        if not c.tie_word_embeddings:
            out[names.lm_head] = ParamSpec((c.vocab_size, c.hidden_size))
        for block, ln in zip(self.blocks, names.layers):
            for role, part in block.parts().items():
                prefix = ln[role]
                for local, spec in part.parameters().items():
                    out[prefix + local] = spec
        for local, spec in self.final_norm.parameters().items():
            out[names.final_norm + local] = spec
        return out

    def load(self, names: TensorNames, tensors: dict[str, torch.Tensor]) -> None:
        """``tensors``: full name -> tensor on the device, already converted."""
        c = self.cfg
        self.embedding = tensors[names.embedding].contiguous()
        self.lm_head = self.embedding if c.tie_word_embeddings else tensors[names.lm_head].contiguous()
        for block, ln in zip(self.blocks, names.layers):
            for role, part in block.parts().items():
                prefix = ln[role]
                part.load({local: tensors[prefix + local] for local in part.parameters()})
        self.final_norm.load({local: tensors[names.final_norm + local]
                              for local in self.final_norm.parameters()})

    # -- what the cache manager has to provide -----------------------------------------------------
    def run_mixer(self, run_index: int):
        return self.blocks[self.cfg.schedule[run_index].layer].mixer

    # -- forward ---------------------------------------------------------------------------------------
    def forward(self, step, cache_views, states) -> torch.Tensor:
        """Hidden states [T, hidden] after the final norm.

        ``cache_views[r]`` / ``states[r]``: the cache view and the state tensor of run r (or None).
        """
        h = self.embed(step)
        residual = None
        for r, run in enumerate(self.cfg.schedule):
            h, residual = self.blocks[run.layer].forward(h, residual, step, cache_views[r], states[r])
        return self.final_norm.forward(h, residual)

    def embed(self, step) -> torch.Tensor:
        """The rows of the embedding table for the step's token ids, [T, hidden].  A model class that
        scales or adds to its embeddings overrides this."""
        h = torch.empty((step.num_tokens, self.cfg.hidden_size), dtype=self.dtype, device=self.device)
        kernels.ops().embedding(h, self.embedding, step.input_ids)
        return h

    def logits(self, hidden: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        """fp32 logits [S, V] of the hidden rows named by ``rows`` (int32 indices on the device; None: of
        every row, in order)."""
        count = hidden.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((count, self.cfg.vocab_size), dtype=torch.float32, device=self.device)
        kernels.ops().linear(out, hidden, self.lm_head, None, rows)
        return self.finish_logits(out)

    def finish_logits(self, logits: torch.Tensor) -> torch.Tensor:
        """What happens to the head's output before anyone sees it (nothing here; a cap or a scale in
        a model class that overrides this)."""
        return logits
