"""Tensor-parallel model facade: one leader rank talks to the serving layer, every call runs on all ranks.

Rank 0 owns the tokenizer, the sampler, the HTTP front door and the engine.  Each ``TextModel`` call it
makes is first broadcast to the follower ranks over a host-side (gloo) group and then executed on every rank
inside ``RankGroup.run_collective``: lockstep fingerprint before the call (kind, rows, position, hash of the
tokens), error exchange after it, and for token-valued calls a comparison of the result across ranks.  A
failure anywhere leaves the group in NEEDS_RECOVERY; the next ``reset()`` drains and re-synchronises the
device communicator (``FusedComm.recover``) and the per-rank models, self-tests, and only then serves again.
A rank that is gone makes the host exchange fail: the group turns FATAL, which the server reports as
503 ``tp_fatal``.  Followers sit in ``follow()`` until the leader sends ``shutdown``.

Logits-valued calls (sampled decoding) return the full vocabulary row on every rank: the shards of the
vocabulary-parallel head are concatenated by an all-gather.

(reference: src/model/tp_model.h:317-351 ``RunCollective``: state check -> post to every rank -> wait ->
compare results -> recover; src/model/tp_model.cpp:1271-1275 chooses the facade at load.  There the ranks are
threads of one process and the post is a queue push; here they are processes and the post is a broadcast.)
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..parallel.tp_group import RankGroup, TpState, TpStateError
from .text_model import TextModel

# calls whose result every rank must agree on
_TOKEN_OPS = {"prefill", "decode_step_greedy", "decode_step_spec_greedy", "position_count"}
# calls that return logits (sharded on the device models)
_LOGITS_OPS = {"decode_step", "last_logits", "window_logits"}


class TpTextModel(TextModel):
    def __init__(self, local: TextModel, group: RankGroup, ctl_group=None, comm=None, data_group=None):
        self.local = local
        self.group = group
        self.ctl = ctl_group                  # host-side process group for the command broadcast (gloo)
        self.comm = comm                      # device communicator (None for host-only models)
        self.data_group = data_group          # device process group for the logits all-gather
        self.rank, self.world = group.rank, group.world
        self.config = local.config
        self.model_id = getattr(local, "model_id", "r4dx-b200")

    # ---- plumbing ---------------------------------------------------------------------------------
    def _post(self, op: str, args: tuple) -> None:
        box = [(op, args)]
        dist.broadcast_object_list(box, src=0, group=self.ctl)

    def _call(self, op: str, *args) -> Any:
        if self.rank != 0:
            raise TpStateError("only the leader rank drives the model; followers run follow()")
        if self.group.state is TpState.FATAL:
            raise TpStateError(f"tensor-parallel group is in a fatal state: {self.group.last_error}")
        self._post(op, args)
        return self._exec(op, args)

    def _tokens_of(self, op: str, args: tuple) -> Sequence[int]:
        if op == "prefill":
            return [int(t) for t in args[0]]
        if op in ("decode_step_greedy", "decode_step", "decode_step_spec_greedy"):
            return [int(args[0])]
        if op in ("window_logits", "commit_window"):
            return [int(args[0])] + [int(t) for t in args[1]]
        return ()

    def _full_logits(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenates the ranks' vocabulary shards (rank order = vocabulary order)."""
        cfg_local = getattr(getattr(self.local, "m", None), "cfg", None)    # the rank-local device model knows its shard
        if not t.is_cuda or self.world == 1 or cfg_local is None or getattr(cfg_local, "tp_world", 1) == 1:
            return t
        full = self.config.vocab_size
        rows = t.reshape(-1, t.shape[-1]).float().contiguous()
        parts = torch.empty(self.world, rows.shape[0], rows.shape[1], dtype=rows.dtype, device=rows.device)
        dist.all_gather_into_tensor(parts, rows, group=self.data_group)
        out = parts.permute(1, 0, 2).reshape(rows.shape[0], -1)[:, :full]
        return out.reshape(*t.shape[:-1], out.shape[-1]) if t.dim() > 1 else out[0]

    def _exec(self, op: str, args: tuple) -> Any:
        if op == "reset":
            return self._reset_all()
        fn = getattr(self.local, op)

        def run():
            r = fn(*args)
            if op in _LOGITS_OPS:
                r = self._full_logits(r)
            if self.comm is not None:
                self.comm.check_healthy()          # a wait that ran out must fail the call, not return a token
            return r

        toks = self._tokens_of(op, args)
        pos = self.local.position_count()
        res = self.group.run_collective(run, kind=op, rows=len(toks), pos=pos, tokens=toks)
        if op in _TOKEN_OPS:
            self.group.require_all_equal(res if not isinstance(res, list) else tuple(res), op)
        return res

    def _reset_all(self) -> None:
        def reset_fn():
            if self.comm is not None:
                self.comm.recover()
            self.local.reset()
        if self.group.state is TpState.NEEDS_RECOVERY:
            self.group.recover(reset_fn=reset_fn, self_test=lambda: self.local.position_count())
        else:
            self.group.run_collective(self.local.reset, kind="reset")

    # ---- follower side ------------------------------------------------------------------------------
    def follow(self) -> None:
        """Runs the leader's commands until ``shutdown`` (or until the host group breaks)."""
        while True:
            box: List[Any] = [None]
            try:
                dist.broadcast_object_list(box, src=0, group=self.ctl)
            except Exception as e:                      # the leader is gone
                self.group.state = TpState.FATAL
                self.group.last_error = f"command broadcast failed: {e}"
                return
            op, args = box[0]
            if op == "shutdown":
                return
            try:
                self._exec(op, args)
            except TpStateError:
                if self.group.state is TpState.FATAL:
                    return
            except Exception:                           # noqa: BLE001 -- already reported to the group; wait for reset
                pass

    def shutdown(self) -> None:
        if self.rank == 0 and self.world > 1 and self.group.state is not TpState.FATAL:
            try:
                self._post("shutdown", ())
            except Exception:                           # noqa: BLE001
                pass

    @property
    def fatal(self) -> Optional[str]:
        return self.group.last_error if self.group.state is TpState.FATAL else None

    @property
    def m(self):
        """The rank-local device model (weights, buffers) behind the facade."""
        return getattr(self.local, "m", None)

    # ---- TextModel interface (leader) ---------------------------------------------------------------
    def position_count(self) -> int: return self.local.position_count()
    def has_checkpoint(self) -> bool: return self.local.has_checkpoint()
    @property
    def max_ctx(self) -> int: return self.local.max_ctx
    def tp_world(self) -> int: return self.world
    def mtp_enabled(self) -> bool: return self.local.mtp_enabled()
    def dflash_enabled(self) -> bool: return self.local.dflash_enabled()
    def has_vision(self) -> bool: return self.local.has_vision()

    def reset(self) -> None: self._call("reset")
    def save_checkpoint(self) -> None: self._call("save_checkpoint")
    def restore_checkpoint(self) -> None: self._call("restore_checkpoint")

    def prefill(self, ids: Sequence[int], embed_overrides=None, image_blocks=None) -> int:
        ids = [int(t) for t in ids]
        if embed_overrides is not None:
            pos, rows = embed_overrides
            embed_overrides = (pos.cpu(), rows.detach().float().cpu())     # travels inside the command
            if image_blocks:
                return self._call("prefill", ids, embed_overrides, [tuple(b) for b in image_blocks])
            return self._call("prefill", ids, embed_overrides)
        return self._call("prefill", ids)

    def last_logits(self) -> torch.Tensor: return self._call("last_logits")
    def decode_step_greedy(self, token: int) -> int: return self._call("decode_step_greedy", int(token))
    def decode_step(self, token: int) -> torch.Tensor: return self._call("decode_step", int(token))

    def decode_step_spec_greedy(self, token: int, k: int) -> List[int]:
        return list(self._call("decode_step_spec_greedy", int(token), int(k)))

    def draft_tokens(self, token: int, k: int) -> List[int]:
        # drafters are deterministic functions of the fed tokens: every rank computes the same proposal locally
        return list(self._call("draft_tokens", int(token), int(k)))

    def window_logits(self, token: int, drafts: Sequence[int]) -> torch.Tensor:
        return self._call("window_logits", int(token), [int(t) for t in drafts])

    def commit_window(self, token: int, drafts: Sequence[int], n: int) -> None:
        self._call("commit_window", int(token), [int(t) for t in drafts], int(n))
