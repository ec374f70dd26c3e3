"""Batched decode over sequence slots (`--batch N` serving and the MoE throughput workload).

Every slot owns its recurrent state (GDN state, conv ring, write-once log) and a block table into one
shared paged-KV pool.  A slot is filled by a normal single-sequence prefill whose state tensors are the
slot's views; ``decode_batch`` then advances any subset of slots by one token in a single pass of the
layer stack: linears see B rows at once (tcgen05 GEMM for B > 8, the weight-streaming kernel otherwise),
the GDN step and the attention run one CTA column per sequence
(reference: src/model/model.cpp:3034-3288 DecodeBatch, src/server/batch_executor.h:1-50).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config import ModelConfig
from ..native import c_f32, c_int, c_ptr, register_cuda_sig
from ..ops import kernels as K
from .hybrid import CONV_RING, KV_BLOCK, MAX_ROWS, HybridModel

BF = torch.bfloat16
register_cuda_sig("r4dxb_gdn_decode_batch", c_int, [c_ptr] * 16 + [c_int, c_int, c_int, c_int, c_f32, c_ptr])
register_cuda_sig("r4dxb_attn_precore_batch", c_int, [c_ptr] * 10 + [c_int, c_ptr, c_ptr] + [c_int] * 5 + [c_f32, c_f32, c_int, c_ptr])
register_cuda_sig("r4dxb_attn_decode_batch", c_int, [c_ptr] * 5 + [c_int] + [c_ptr] * 6 + [c_int] * 6 + [c_ptr])


class PagedKvAllocator:
    """Free-list allocator of 16-token KV blocks shared by all slots; tables are filled on demand."""

    def __init__(self, num_blocks: int, slots: int, max_blocks_per_slot: int, device):
        self.free = list(range(num_blocks - 1, -1, -1))
        self.tables = torch.zeros(slots, max_blocks_per_slot, dtype=torch.int32, device=device)
        self.owned: List[List[int]] = [[] for _ in range(slots)]
        self.max_blocks = max_blocks_per_slot

    def ensure(self, slot: int, tokens: int) -> None:
        need = (tokens + KV_BLOCK - 1) // KV_BLOCK
        if need > self.max_blocks:
            raise ValueError("slot context overflow")
        own = self.owned[slot]
        if need > len(own):
            if need - len(own) > len(self.free):
                raise MemoryError("KV block pool exhausted")
            new = [self.free.pop() for _ in range(need - len(own))]
            self.tables[slot, len(own):need] = torch.tensor(new, dtype=torch.int32, device=self.tables.device)
            own += new

    def release(self, slot: int) -> None:
        self.free += reversed(self.owned[slot])
        self.owned[slot] = []

    def blocks_in_use(self) -> int:
        return sum(len(o) for o in self.owned)


class BatchModel:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, object], slots: int, slot_ctx: int, device: str = "cuda",
                 comm=None, pool_blocks: Optional[int] = None):
        self.cfg, self.slots, self.device = cfg, slots, torch.device(device)
        self.slot_ctx = ((slot_ctx + KV_BLOCK - 1) // KV_BLOCK) * KV_BLOCK
        self.base = HybridModel(cfg, weights, max_ctx=self.slot_ctx, device=device, comm=comm)
        b = self.base
        nblk = self.slot_ctx // KV_BLOCK
        self.alloc = PagedKvAllocator(pool_blocks or slots * nblk, slots, nblk + 1, self.device)
        Hkv, D = cfg.num_key_value_heads, cfg.head_dim
        Hv, Dg = cfg.linear_num_value_heads, cfg.linear_key_head_dim
        z = lambda *s, dtype=torch.float32: torch.zeros(*s, dtype=dtype, device=self.device)
        pool = (pool_blocks or slots * nblk) + 1
        self.kv = {i: z(pool, Hkv, 2, KV_BLOCK, D, dtype=torch.uint8) for i in b.kv}
        self.gdn_state = {i: z(slots, Hv, Dg, Dg) for i in b.gdn_state}
        self.ring = {i: z(slots, CONV_RING, cfg.conv_dim, dtype=BF) for i in b.ring}
        self.log_u = {i: z(slots, MAX_ROWS, Hv, Dg) for i in b.gdn_state}
        self.log_k = {i: z(slots, MAX_ROWS, Hv, Dg) for i in b.gdn_state}
        self.log_eg = {i: z(slots, MAX_ROWS, Hv) for i in b.gdn_state}
        self.n_replay = z(slots, dtype=torch.int32)
        self.pos = [0] * slots
        self.active = [False] * slots
        # drop the base model's private state: it only ever runs on slot views
        for i in b.kv:
            b.kv[i] = self.kv[i]
        self._rows = 0
        if cfg.is_moe:
            from .moe import MoeBlock
            er = getattr(comm, "expert_range", None) if comm is not None else None
            self.moe = {i: MoeBlock(cfg, weights, i, self.device, max(slots, 8), *(er or (0, cfg.num_experts)),
                                    share_from=b.moe.get(i)) for i in range(cfg.num_hidden_layers)}
        self._L = None

    # ---- slot lifecycle -------------------------------------------------------------------------------
    def _bind(self, slot: int) -> None:
        b = self.base
        for i in b.gdn_state:
            b.gdn_state[i], b.ring[i] = self.gdn_state[i][slot], self.ring[i][slot]
            b.log_u[i], b.log_k[i], b.log_eg[i] = self.log_u[i][slot], self.log_k[i][slot], self.log_eg[i][slot]
        b.block_table = self.alloc.tables[slot]
        b.pos, b.pending_rows = self.pos[slot], 0
        b._graphs.clear()

    def import_slot(self, slot: int, ids: Sequence[int]) -> int:
        """Prefills ``ids`` into a free slot; returns the greedy first token."""
        self.release_slot(slot)
        self.alloc.ensure(slot, len(ids) + 1)
        for d in (self.gdn_state, self.ring):
            for t in d.values():
                t[slot].zero_()
        self.pos[slot] = 0
        self._bind(slot)
        tok = self.base.prefill(torch.as_tensor(list(ids), dtype=torch.int32))
        self.last_prefill_logits = self.base.buf.logits[getattr(self.base, "last_row", 0)].float().clone()
        self.base.commit_pending()
        self.pos[slot] = self.base.pos
        self.n_replay[slot] = 0
        self.active[slot] = True
        return tok

    def position_slot(self, slot: int, pos: int) -> None:
        """Benchmark aid: marks ``slot`` active at position ``pos`` without a prefill (its KV blocks hold zeros, which cost
        the same to read; the recurrent state starts at zero)."""
        self.release_slot(slot)
        self.alloc.ensure(slot, pos + 1)
        self.pos[slot] = pos
        self.n_replay[slot] = 0
        self.active[slot] = True

    def release_slot(self, slot: int) -> None:
        self.alloc.release(slot)
        self.active[slot] = False

    # ---- one token for B slots ---------------------------------------------------------------------------
    def decode_batch(self, slots: Sequence[int], tokens: Sequence[int]) -> List[int]:
        from .. import native
        L = self._L = self._L or native.cuda()
        cfg, b, w = self.cfg, self.base, self.base.w
        B = len(slots)
        for s in slots:
            self.alloc.ensure(s, self.pos[s] + 1)
        dev = self.device
        ids = torch.tensor(list(tokens), dtype=torch.int32, device=dev)
        positions = torch.tensor([self.pos[s] for s in slots], dtype=torch.int32, device=dev)
        row_slot = torch.tensor(list(slots), dtype=torch.int32, device=dev)
        cb = b._chunk_buffers(max(B, MAX_ROWS + 1))
        x, h = cb["x"][:B], cb["h"][:B]
        st = torch.cuda.current_stream().cuda_stream
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        Hv, Hk, Dg = cfg.linear_num_value_heads, cfg.linear_num_key_heads, cfg.linear_key_head_dim
        G = Hq // max(1, Hkv)
        splits = max(1, min(16, 592 // max(1, Hkv * B)))        # about four CTAs per SM
        part_acc = torch.empty(B * splits * Hkv * G * D, dtype=torch.float32, device=dev)
        part_ml = torch.empty(B * splits * Hkv * G * 2, dtype=torch.float32, device=dev)

        def lin(name, inp, out, residual=None, fused=False):
            l = b.lin[name]
            if B > MAX_ROWS:
                return l.chunk(inp, cb["xh"], out, residual=residual, fused_silu_mul=fused)
            return l(inp, out=out, residual=residual, prologue=K.PRO_SILU_MUL if fused else K.PRO_NONE)

        K.embed_gather(ids, w["text.embed_tokens"], out=x)
        for i in range(cfg.num_hidden_layers):
            p = f"text.layers.{i}."
            K.rmsnorm(x, w[p + "input_layernorm"], cfg.rms_norm_eps, out=h)
            if cfg.is_attention_layer(i):
                pa = p + "attn."
                qg, kk, vv, q = cb["qg"][:B], cb["k"][:B], cb["v"][:B], cb["q"][:B]
                lin(pa + "qg", h, qg); lin(pa + "k", h, kk); lin(pa + "v", h, vv)
                qn, kn = w.get(pa + "q_norm"), w.get(pa + "k_norm")
                rc = L.r4dxb_attn_precore_batch(qg.data_ptr(), kk.data_ptr(), vv.data_ptr(), qn.data_ptr() if qn is not None else None,
                                                kn.data_ptr() if kn is not None else None, w[pa + "k_descale"].data_ptr(), w[pa + "v_descale"].data_ptr(),
                                                positions.data_ptr(), self.alloc.tables.data_ptr(), row_slot.data_ptr(),
                                                self.alloc.tables.shape[1], q.data_ptr(), self.kv[i].data_ptr(), B, Hq, Hkv, D,
                                                cfg.rotary_dim, cfg.rope_theta, cfg.rms_norm_eps, cfg.q_proj_dim // Hq, st)
                assert rc == 0, rc
                core = cb["core"][:B * cfg.q_dim].view(B, cfg.q_dim)
                rc = L.r4dxb_attn_decode_batch(q.data_ptr(), qg.data_ptr(), self.kv[i].data_ptr(), self.alloc.tables.data_ptr(),
                                               row_slot.data_ptr(), self.alloc.tables.shape[1], positions.data_ptr(),
                                               w[pa + "k_descale"].data_ptr(), w[pa + "v_descale"].data_ptr(), part_acc.data_ptr(),
                                               part_ml.data_ptr(), core.data_ptr(), B, Hq, Hkv, D, splits,
                                               1 if cfg.attn_output_gate else 0, st)
                assert rc == 0, rc
                lin(pa + "o", core, x, residual=x)
            else:
                pg = p + "gdn."
                mixed, z, ab = cb["mixed"][:B], cb["z"][:B], cb["ab"][:B]
                lin(pg + "in_proj_qkv", h, mixed); lin(pg + "in_proj_z", h, z)
                K.bf16_gemv(b.ab_w[i], h, out=ab)
                core = cb["core"][:B * cfg.value_dim].view(B, cfg.value_dim)
                rc = L.r4dxb_gdn_decode_batch(mixed.data_ptr(), z.data_ptr(), ab.data_ptr(), w[pg + "conv1d_weight"].data_ptr(),
                                              w[pg + "A_log"].data_ptr(), w[pg + "dt_bias"].data_ptr(), w[pg + "norm_weight"].data_ptr(),
                                              self.ring[i].data_ptr(), self.gdn_state[i].data_ptr(), self.log_u[i].data_ptr(),
                                              self.log_k[i].data_ptr(), self.log_eg[i].data_ptr(), positions.data_ptr(),
                                              self.n_replay.data_ptr(), row_slot.data_ptr(), core.data_ptr(), B, Hv, Hk, Dg,
                                              cfg.rms_norm_eps, st)
                assert rc == 0, rc
                lin(pg + "out_proj", core, x, residual=x)
            K.rmsnorm(x, w[p + "post_attention_layernorm"], cfg.rms_norm_eps, out=h)
            if cfg.is_moe:
                comm = b.comm
                if comm is not None and hasattr(comm, "moe_forward"):
                    comm.moe_forward(self.moe[i], h, x, B)
                else:
                    self.moe[i].forward(h, x, B)
            else:
                gu = cb["gate_up"][:B]
                lin(p + "mlp.gate_up", h, gu)
                lin(p + "mlp.down", gu, x, residual=x, fused=True)
        self.n_replay[row_slot.long()] = 1
        K.rmsnorm(x, w["text.final_norm"], cfg.rms_norm_eps, out=h)
        V = cfg.vocab_shard_size
        if B > MAX_ROWS:
            # many rows: the head runs on the tensor cores straight from its packed weights
            logits = b.lin["lm_head"].many(h[:B], out_f32=True)
        else:
            logits = torch.empty(B, V, dtype=torch.float32, device=dev)
            b.lin["lm_head"](h, out=logits)
        nxt, _ = K.argmax_rows(logits, cfg.vocab_shard_begin)
        for s in slots:
            self.pos[s] += 1
        self.last_logits = logits
        return nxt.tolist()
