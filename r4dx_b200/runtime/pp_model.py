"""Pipeline-parallel text models for two ranks.

``LayerSplitTextModel`` (``--pp 2``): each rank holds the full-width weights of its half of the layers; prompts run as
a two-stage pipeline over prefill chunks, decode passes the residual rows from stage A to stage B, which runs the head.
For models whose weights do not fit one GPU, and for prefill throughput: both GPUs compute on different chunks at once.

``HybridPpTextModel`` (``--pp 2 --tp 2 --hybrid``): prompts of at least ``pp_min_rows`` tokens run through the pipeline
(no collectives inside the layers, whole GEMMs per GPU), then the per-layer state is resharded into the
tensor-parallel layout and decode continues tensor-parallel (lowest latency per token).  Short prompts and everything
after the prompt use the tensor-parallel model directly.

Every method is called on both ranks in the same order (the leader/follower facade ``TpTextModel`` broadcasts the
calls), and every method returns the same value on both ranks.

(reference: src/model/pp_model.cpp:441-513 pipelined prefill, src/model/hybrid_model.cpp + reshard_plan.h:1-18 the
prefill-then-reshard mode, src/model/tp_model.cpp:1271-1275 picks the facade from --pp / --hybrid / --pp-split /
--pp-min-rows.)
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..parallel.pp import LayerSplitDecode, PipelinePrefill, reshard_to_tp
from .text_model import LocalTextModel, ModelStateError, TextModel


def stage_of_layers(n_layers: int, split: int) -> Dict[int, int]:
    return {i: (0 if i < split else 1) for i in range(n_layers)}


class LayerSplitTextModel(TextModel):
    def __init__(self, stage, rank: int, split: int, global_config: ModelConfig, model_id: str = "r4dx-b200",
                 chunk: int = 1024, group=None):
        self.m = stage                       # this rank's layers (a HybridModel with a layer_range)
        self.rank, self.split, self.group = rank, split, group
        self.config = global_config
        self.model_id = model_id
        self.pp = PipelinePrefill(stage, rank, split, chunk=chunk, group=group)
        self.ls = LayerSplitDecode(stage, rank, group=group)
        self._ck = None
        self._row = torch.zeros(global_config.vocab_size, dtype=torch.float32, device=stage.device)

    @property
    def max_ctx(self) -> int:
        return self.m.max_ctx

    def position_count(self) -> int:
        return self.m.pos

    def tp_world(self) -> int:
        return 1

    def reset(self) -> None:
        self.m.reset()

    def save_checkpoint(self) -> None:
        self._ck = self.m.save_checkpoint()

    def restore_checkpoint(self) -> None:
        if self._ck is None:
            raise ModelStateError("no checkpoint saved")
        self.m.restore_checkpoint(self._ck)

    def has_checkpoint(self) -> bool:
        return self._ck is not None

    def prefill(self, ids: Sequence[int], embed_overrides=None) -> int:
        if embed_overrides is not None:
            raise NotImplementedError("embedding overrides (images, audio) with a layer split")
        return self.pp.prefill(torch.as_tensor(list(ids), dtype=torch.int32))

    def _share_row(self) -> torch.Tensor:
        """The head ran on stage B: its logits row goes to both ranks."""
        if self.rank == 1:
            self._row.copy_(self.m.buf.logits[0][:self._row.numel()])
        dist.broadcast(self._row, src=1, group=self.group)
        return self._row

    def last_logits(self) -> torch.Tensor:
        return self._share_row()

    def decode_step_greedy(self, token: int) -> int:
        return self.ls.step(int(token))

    def decode_step(self, token: int) -> torch.Tensor:
        self.ls.step(int(token))
        return self._share_row()


class HybridPpTextModel(LocalTextModel):
    """Tensor-parallel decode model (``self.m``) whose long prompts run through a two-stage pipeline first."""

    def __init__(self, tp_model, stage, rank: int, world: int, split: int, global_config: ModelConfig,
                 model_id: str = "r4dx-b200", chunk: int = 1024, min_rows: int = 512, group=None, drafter=None,
                 prefill_chunk: int = 0):
        super().__init__(tp_model, model_id=model_id, global_config=global_config, drafter=drafter, prefill_chunk=prefill_chunk)
        if world != 2:
            raise ValueError("the pipelined prefill has two stages: --hybrid needs exactly two ranks")
        self.stage, self.rank, self.world, self.split, self.group = stage, rank, world, split, group
        self.min_rows = min_rows
        self.pp = PipelinePrefill(stage, rank, split, chunk=chunk, group=group)
        self._full_row = torch.zeros(global_config.vocab_size, dtype=torch.float32, device=tp_model.device)
        self.pipelined_prompts = 0

    def prefill(self, ids: Sequence[int], embed_overrides=None) -> int:
        ids = list(ids)
        if len(ids) < self.min_rows or len(ids) > self.stage.max_ctx or self.m.pos != 0 or embed_overrides is not None \
                or self.drafter is not None:
            # short prompts, prompts beyond the stages' capacity, continuations of a cached prefix, multimodal rows and drafter
            # hooks: the tensor-parallel model
            return super().prefill(ids, embed_overrides)
        self._graph_active = False
        self.stage.reset()
        tok = self.pp.prefill(torch.as_tensor(ids, dtype=torch.int32))
        reshard_to_tp(self.config, self.stage, self.m, self.world, self.rank,
                      stage_of_layers(self.config.num_hidden_layers, self.split), group=self.group)
        # the prompt's last logits row lives on stage B: every rank keeps its vocabulary shard of it
        if self.rank == 1:
            self._full_row.copy_(self.stage.buf.logits[0][:self._full_row.numel()])
        dist.broadcast(self._full_row, src=1, group=self.group)
        c = self.m.cfg
        lo = c.vocab_shard_begin
        hi = min(lo + c.vocab_shard_size, self._full_row.numel())
        self.m.buf.logits[0][:hi - lo].copy_(self._full_row[lo:hi])
        self.m.buf.next_ids[:1].fill_(tok)
        self.pipelined_prompts += 1
        return tok
