"""The model facade the serving layer talks to, and its implementations.

``TextModel`` mirrors the reference's interface (reference: src/model/text_model.h:115-222): prefill,
greedy / sampled decode steps, speculative steps, reset, prompt checkpoint.  ``LocalTextModel`` wraps
one ``HybridModel`` (one GPU, or one rank of a tensor-parallel group -- every rank runs the same
calls in lockstep); ``FakeTextModel`` is a CPU stand-in whose logits are a pure function of the tokens
it was fed, used by the server tests (reference: tests/server/test_engine_recovery.cpp:1-30).
"""
from __future__ import annotations

import hashlib
from typing import Callable, List, Optional, Sequence

import torch

from ..config import ModelConfig
from .sampler import Rng, SampleParams, apply_repetition_penalty, sample_canonical


class ModelStateError(RuntimeError):
    """The model needs Reset() before the next call (a previous call failed half-way)."""


class TextModel:
    config: ModelConfig
    model_id: str = "r4dx-b200"

    # ---- state ----
    def position_count(self) -> int: raise NotImplementedError
    def reset(self) -> None: raise NotImplementedError
    def save_checkpoint(self) -> None: raise NotImplementedError
    def restore_checkpoint(self) -> None: raise NotImplementedError
    def has_checkpoint(self) -> bool: return False
    @property
    def max_ctx(self) -> int: raise NotImplementedError
    def tp_world(self) -> int: return 1
    def mtp_enabled(self) -> bool: return False
    def dflash_enabled(self) -> bool: return False
    def has_vision(self) -> bool: return False

    # ---- forward ----
    def prefill(self, ids: Sequence[int], embed_overrides=None) -> int:
        """Feeds the tokens; returns the greedy next token (logits of the last row via ``last_logits``).
        ``embed_overrides`` = (positions [M], rows [M, hidden]) replaces those tokens' input embeddings (images)."""
        raise NotImplementedError
    def last_logits(self) -> torch.Tensor: raise NotImplementedError
    def decode_step_greedy(self, token: int) -> int: raise NotImplementedError
    def decode_step(self, token: int) -> torch.Tensor: raise NotImplementedError

    def decode_step_sampled(self, token: int, params: SampleParams, rng: Rng, seen: Optional[Sequence[int]] = None) -> int:
        logits = self.decode_step(token).float().cpu()
        if params.repetition_penalty != 1.0 and seen:
            apply_repetition_penalty(logits, seen, params.repetition_penalty)
        return sample_canonical(logits, params, rng.next())

    def sample_from_last(self, params: SampleParams, rng: Rng, seen: Optional[Sequence[int]] = None) -> int:
        logits = self.last_logits().float().cpu().clone()
        if params.repetition_penalty != 1.0 and seen:
            apply_repetition_penalty(logits, seen, params.repetition_penalty)
        if params.greedy:
            return int(torch.argmax(logits))
        return sample_canonical(logits, params, rng.next())

    def decode_step_spec_greedy(self, token: int, k: int) -> List[int]:
        """Speculative round (drafter chosen at load): emitted tokens, at least one."""
        return [self.decode_step_greedy(token)]

    # ---- sampled speculation: sample-and-match -------------------------------------------------------------
    def draft_tokens(self, token: int, k: int) -> List[int]:
        """Up to k proposed continuations of ``token`` (no drafter: none)."""
        return []

    def window_logits(self, token: int, drafts: Sequence[int]) -> torch.Tensor:
        """Logits rows [1 + len(drafts), vocab] of the window [token, drafts...]; commits nothing."""
        raise NotImplementedError

    def commit_window(self, token: int, drafts: Sequence[int], n: int) -> None:
        """Commits the first n rows of the window that ``window_logits`` just ran."""
        raise NotImplementedError

    def decode_step_spec_sampled(self, token: int, k: int, params: SampleParams, rng: Rng,
                                 seen: Optional[Sequence[int]] = None) -> List[int]:
        """One speculative round under sampling.  Row i of the verify window is the target distribution after
        [.., token, d1..di]; one token is drawn per row with the request's generator and a draft is accepted only if the
        draw equals it - rejection sampling for a point-mass proposal, one draw per emitted token, so the stream is the
        same as plain sampled decode with the same seed (reference: src/model/model.h:559-581, docs/sampling.md:417-460)."""
        drafts = list(self.draft_tokens(token, k))
        if not drafts:
            return [self.decode_step_sampled(token, params, rng, seen)]
        rows = self.window_logits(token, drafts).float().cpu()
        hist = list(seen) if seen is not None else []
        emitted: List[int] = []
        for i in range(rows.shape[0]):
            lg = rows[i].clone()
            if params.repetition_penalty != 1.0 and hist:
                apply_repetition_penalty(lg, hist, params.repetition_penalty)
            t = int(torch.argmax(lg)) if params.greedy else sample_canonical(lg, params, rng.next())
            emitted.append(t)
            hist.append(t)
            if i >= len(drafts) or t != drafts[i]:
                break
        self.commit_window(token, drafts, len(emitted))
        return emitted


class LocalTextModel(TextModel):
    def __init__(self, model, model_id: str = "r4dx-b200", global_config: Optional[ModelConfig] = None, drafter=None,
                 prefill_chunk: int = 0):
        self.prefill_chunk = prefill_chunk
        self.m = model
        self.config = global_config or model.cfg
        self.model_id = model_id
        self._ck = None
        self.drafter = drafter
        self._graph_ready = False
        self._graph_active = False

    @property
    def max_ctx(self) -> int:
        return self.m.max_ctx

    def position_count(self) -> int:
        return self.m.pos

    def tp_world(self) -> int:
        return self.m.cfg.tp_world

    def mtp_enabled(self) -> bool:
        return self.drafter is not None and getattr(self.drafter, "kind", "") == "mtp"

    def reset(self) -> None:
        self.m.reset()
        self._graph_active = False
        if self.drafter is not None:
            self.drafter.reset()

    def save_checkpoint(self) -> None:
        self._graph_active = False
        self._ck = self.m.save_checkpoint()

    def restore_checkpoint(self) -> None:
        if self._ck is None:
            raise ModelStateError("no checkpoint saved")
        self._graph_active = False
        self.m.restore_checkpoint(self._ck)

    def has_checkpoint(self) -> bool:
        return self._ck is not None

    def prefill(self, ids: Sequence[int], embed_overrides=None, image_blocks=None) -> int:
        """``image_blocks``: [start, end) runs of image rows that attend to each other in both directions on sliding-window
        layers (the Gemma-style family); the chunk plan never cuts one."""
        self._graph_active = False
        t = torch.as_tensor(list(ids), dtype=torch.int32)
        hook = self.drafter.prefill_hook(t) if self.drafter is not None else None
        kw = {"image_blocks": image_blocks} if image_blocks else {}
        tok = self.m.prefill(t, chunk=self.prefill_chunk or None, hook=hook, embed_overrides=embed_overrides, **kw)
        if self.drafter is not None:
            self.drafter.after_prefill(t, tok)
        return tok

    def last_logits(self) -> torch.Tensor:
        n = self._last_row()
        return self.m.buf.logits[n]

    def _last_row(self) -> int:
        return 0

    def decode_step_greedy(self, token: int) -> int:
        """Graph replay when possible (tokens stay on the device between steps)."""
        m = self.m
        if not self._graph_ready:
            m.enable_graphs((1,))
            self._graph_ready = True
        if not self._graph_active:
            m.decode_begin(token)
            self._graph_active = True
        else:
            m.buf.ids[:1].fill_(token)
        m.decode_step_graph()
        return m._read_token(0)

    def decode_step(self, token: int) -> torch.Tensor:
        self._graph_active = False
        return self.m.decode_step_logits(token)

    def decode_step_spec_greedy(self, token: int, k: int) -> List[int]:
        if self.drafter is None:
            return [self.decode_step_greedy(token)]
        self._graph_active = False
        drafts = self.drafter.draft(token, k)
        self._window_graph(len(drafts) + 1)
        emitted = self.m.verify_window(token, drafts)
        self.drafter.after_verify(token, drafts, emitted)
        return emitted

    def _window_graph(self, T: int) -> None:
        """Captures the verify window of T rows once it has been used a few times with that size (windows shrink near the
        end of a request: those sizes stay eager)."""
        if T < 2 or not self.window_graphs or T in getattr(self.m, "_graphs", {T: None}):
            return
        seen = self.__dict__.setdefault("_window_uses", {})
        seen[T] = seen.get(T, 0) + 1
        if seen[T] == 3:
            self.m.enable_graphs((T,))

    window_graphs = True

    def draft_tokens(self, token: int, k: int) -> List[int]:
        return self.drafter.draft(token, k) if self.drafter is not None else []

    def window_logits(self, token: int, drafts: Sequence[int]) -> torch.Tensor:
        self._graph_active = False
        self._window_graph(len(drafts) + 1)
        return self.m.window_logits(token, list(drafts))

    def commit_window(self, token: int, drafts: Sequence[int], n: int) -> None:
        emitted_like = list(drafts[:n - 1]) + [0]          # the drafter only needs to know how many drafts were accepted
        self.m.commit_window(n)
        if self.drafter is not None:
            self.drafter.after_verify(token, list(drafts), emitted_like)


class FakeTextModel(TextModel):
    """Deterministic CPU model: the logits depend only on the token history."""

    def __init__(self, vocab: int = 256, max_ctx: int = 4096, fail_at_call: Optional[int] = None, eos: int = 0):
        self.config = ModelConfig(vocab_size=vocab, hidden_size=128, num_hidden_layers=0)
        self.vocab = vocab
        self._max_ctx = max_ctx
        self.history: List[int] = []
        self._ck: Optional[List[int]] = None
        self.calls = 0
        self.fail_at_call = fail_at_call
        self.needs_reset = False
        self.prefill_tokens = 0
        self.eos = eos

    @property
    def max_ctx(self) -> int:
        return self._max_ctx

    def position_count(self) -> int:
        return len(self.history)

    def _tick(self):
        if self.needs_reset:
            raise ModelStateError("call reset() first")
        self.calls += 1
        if self.fail_at_call is not None and self.calls == self.fail_at_call:
            self.needs_reset = True
            raise RuntimeError("injected model fault")

    def reset(self) -> None:
        self.history = []
        self.needs_reset = False

    def save_checkpoint(self) -> None:
        self._ck = list(self.history)

    def restore_checkpoint(self) -> None:
        if self._ck is None:
            raise ModelStateError("no checkpoint saved")
        self.history = list(self._ck)

    def has_checkpoint(self) -> bool:
        return self._ck is not None

    def _logits(self) -> torch.Tensor:
        h = hashlib.sha256(bytes(str(self.history[-8:]), "ascii")).digest()
        g = torch.Generator().manual_seed(int.from_bytes(h[:8], "little") % (2**63))
        return torch.randn(self.vocab, generator=g)

    def prefill(self, ids: Sequence[int], embed_overrides=None, image_blocks=None) -> int:
        self._tick()
        self.last_overrides = embed_overrides
        self.last_image_blocks = image_blocks
        self.history += list(ids)
        self.prefill_tokens += len(ids)
        return int(torch.argmax(self._logits()))

    def last_logits(self) -> torch.Tensor:
        return self._logits()

    def decode_step(self, token: int) -> torch.Tensor:
        self._tick()
        self.history.append(token)
        return self._logits()

    def decode_step_greedy(self, token: int) -> int:
        return int(torch.argmax(self.decode_step(token)))

    # speculation hooks: ``draft_fn(history, token, k)`` plays the drafter
    draft_fn = None

    def draft_tokens(self, token: int, k: int) -> List[int]:
        return list(self.draft_fn(list(self.history), token, k)) if self.draft_fn else []

    def window_logits(self, token: int, drafts: Sequence[int]) -> torch.Tensor:
        self._tick()
        if len(self.history) + 1 + len(drafts) > self._max_ctx:     # same rule as the device model's window
            raise ValueError("context overflow")
        keep = list(self.history)
        rows = []
        for t in [token] + list(drafts):
            self.history.append(t)
            rows.append(self._logits())
        self.history = keep
        self._window = [token] + list(drafts)
        return torch.stack(rows)

    def commit_window(self, token: int, drafts: Sequence[int], n: int) -> None:
        self.history += self._window[:n]
