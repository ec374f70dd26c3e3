"""Model configuration for the Qwen-style hybrid family (Gated DeltaNet + gated full attention).

Covers the dense hybrid (27B geometry), the tiny 4-layer test geometry and the hybrid MoE
variant (routed experts + shared expert).  ``shard(world, rank)`` returns the rank-local view for
tensor parallelism at world 1/2/4/8; unlike the reference, whose ``ModelConfig::Shard`` accepts
world 2 only (reference: src/model/model_config.h:211-266), KV heads are replicated when the
world exceeds the KV head count so that TP=8 works on 4 KV heads.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class ModelConfig:
    arch: str = "qwen_hybrid"          # qwen_hybrid | qwen_hybrid_moe | llama
    hidden_size: int = 0
    num_hidden_layers: int = 0
    layer_types: List[str] = field(default_factory=list)   # "linear_attention" | "full_attention" | "conv"
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    attn_output_gate: bool = True
    qk_norm: bool = True               # per-head RMSNorm of q and k before rope
    norm_zero_centered: bool = True    # checkpoint norm weights are w with scale (1 + w); False: plain scale w
    # Gemma-style blocks
    sandwich_norm: bool = False        # block outputs pass a second RMSNorm before they join the residual stream
    mlp_act: str = "silu"              # gate activation of the gated MLP: "silu" | "gelu_tanh"
    sliding_window: int = 0            # > 0: attention layers are windowed, except every ``sliding_global_every``-th one
    sliding_global_every: int = 6
    rope_local_theta: float = 1.0e4    # rope base of the windowed layers
    embed_scale: float = 1.0           # token embeddings are multiplied by this (sqrt(hidden) for Gemma)
    intermediate_size: int = 0
    partial_rotary_factor: float = 0.25
    rope_theta: float = 1.0e7
    mrope_interleaved: bool = True
    mrope_section: List[int] = field(default_factory=list)
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    rms_norm_eps: float = 1e-6
    vocab_size: int = 0
    tie_word_embeddings: bool = False
    mtp_num_hidden_layers: int = 0
    max_position_embeddings: int = 262144
    # MoE variant (0 experts = dense MLP in every layer)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    moe_router: str = "softmax"        # "softmax" | "sigmoid" (selection by sigmoid + per-expert bias, unbiased weights)
    moe_expert_bias: bool = False      # sigmoid router: a learned per-expert bias moves the selection only
    routed_scaling_factor: float = 1.0
    num_dense_layers: int = 0          # the first layers keep a dense gated MLP in a MoE model
    # short-conv layers ("conv" in layer_types): y = C * causal_fir(B * x), taps per channel
    short_conv_taps: int = 3
    # qwen4_exp extras (reference: docs/qwen4exp-plan.md 2.2-2.4): gated multi-stream residual, hashed n-gram embedding
    # layer, block-indexed sparse attention; all off (0 / empty) for the other families
    hc_count: int = 0                  # residual streams (4); 0 = the plain single-stream residual
    hc_lowrank: int = 0                # width of the gate's low-rank bottleneck (320)
    ple_layers: List[int] = field(default_factory=list)   # 0-indexed layers that add the n-gram embedding block first
    ple_embed_dim: int = 0             # ngram_heads * ngram_head_dim
    ple_conv_kernel: int = 4
    ple_conv_dilation: int = 3
    ngram_heads: int = 16              # half of them hash 2-grams, the other half 3-grams
    indexer_heads: int = 0             # > 0: attention layers select key blocks with an indexer (QSA)
    indexer_dim: int = 128
    indexer_ratio: int = 4             # tokens per key block
    indexer_budget: int = 2048         # selected tokens: the top budget / ratio complete blocks, plus the open tail
    gdn_gate_act: str = "silu"         # output gate of the GDN norm: "silu" | "sigmoid"
    final_norm: bool = True            # False: the stack ends in the final stream mixer, no norm before the head
    eos_token_id: int = -1             # n-gram history is cut at this token
    # tensor parallel view
    tp_world: int = 1
    tp_rank: int = 0
    kv_replicas: int = 1               # >1 when tp_world > global KV heads

    # ---- derived shapes (names follow reference src/model/model_config.h:76-96) ----
    @property
    def key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def conv_dim(self) -> int:
        return 2 * self.key_dim + self.value_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor + 0.5)

    @property
    def gdn_gqa(self) -> int:
        return self.linear_num_value_heads // max(1, self.linear_num_key_heads)

    @property
    def attn_gqa(self) -> int:
        return self.num_attention_heads // max(1, self.num_key_value_heads)

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def q_proj_dim(self) -> int:
        """Rows of the q projection: q|gate pairs per head when the output gate exists."""
        return self.q_dim * (2 if self.attn_output_gate else 1)

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def vocab_shard_size(self) -> int:
        return self.vocab_size // self.tp_world

    @property
    def vocab_shard_begin(self) -> int:
        return self.tp_rank * self.vocab_shard_size

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        return self.num_experts > 0 and i >= self.num_dense_layers

    def is_conv_layer(self, i: int) -> bool:
        return self.layer_types[i] == "conv"

    @property
    def conv_channels(self) -> int:
        """Channels of a short-conv mixer held by this rank (the hidden width split over the tensor-parallel ranks)."""
        return self.hidden_size // self.tp_world

    @property
    def has_conv_layers(self) -> bool:
        return any(t == "conv" for t in self.layer_types)

    def layer_window(self, i: int) -> int:
        """Sliding-window length of layer ``i`` (0 = global attention)."""
        if self.sliding_window <= 0 or (i + 1) % self.sliding_global_every == 0:
            return 0
        return self.sliding_window

    def layer_theta(self, i: int) -> float:
        return self.rope_local_theta if self.layer_window(i) > 0 else self.rope_theta

    def is_attention_layer(self, i: int) -> bool:
        return self.layer_types[i] == "full_attention"

    def num_attention_layers(self) -> int:
        return sum(1 for t in self.layer_types if t == "full_attention")

    @property
    def is_qwen4_exp(self) -> bool:
        return self.hc_count > 0

    @property
    def ngram_head_dim(self) -> int:
        return self.ple_embed_dim // max(1, self.ngram_heads)

    def validate(self) -> None:
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types length != num_hidden_layers")
        if self.hc_count:
            if self.hc_lowrank < 1 or self.ple_embed_dim % max(1, self.ngram_heads) or self.ngram_heads % 2:
                raise ValueError("qwen4_exp: hc_lowrank, ple_embed_dim / ngram_heads")
            if any(not 0 <= i < self.num_hidden_layers for i in self.ple_layers):
                raise ValueError("qwen4_exp: ple_layers out of range")
            if self.indexer_heads and (self.indexer_budget % self.indexer_ratio or self.indexer_dim % 32 or self.indexer_dim > 128
                                       or self.rotary_dim > self.indexer_dim):
                raise ValueError("qwen4_exp: indexer geometry")
            if self.gdn_gate_act not in ("silu", "sigmoid"):
                raise ValueError("gdn_gate_act")
        if self.num_attention_heads % max(1, self.num_key_value_heads):
            raise ValueError("attention heads not a multiple of KV heads")
        if self.linear_num_value_heads % max(1, self.linear_num_key_heads):
            raise ValueError("GDN value heads not a multiple of key heads")
        if self.hidden_size % 128:
            raise ValueError("hidden_size must be a multiple of 128 (trellis block)")

    # ---- tensor-parallel shard view --------------------------------------------------------
    def shard(self, world: int, rank: int) -> "ModelConfig":
        """Rank-local view: head counts and intermediate sizes of this rank's slices.

        vocab_size stays global; the lm_head width is ``vocab_shard_size``.  Contiguous head
        blocks per rank keep the GQA grouping intact.  When ``world`` exceeds the KV head count
        each KV head is replicated on ``world / kv_heads`` consecutive ranks.
        """
        if world not in (1, 2, 4, 8):
            raise ValueError(f"tp world {world} not in (1, 2, 4, 8)")
        if not 0 <= rank < world:
            raise ValueError("rank out of range")
        if self.tp_world != 1:
            raise ValueError("shard() must be called on the global config")
        if world == 1:
            return dataclasses.replace(self)
        if self.has_conv_layers and (self.hidden_size // world) % 128:
            raise ValueError("per-rank short-conv channels must stay a multiple of 128")
        c = dataclasses.replace(self, tp_world=world, tp_rank=rank)

        def div(v: int, what: str) -> int:
            if v % world:
                raise ValueError(f"{what}={v} not divisible by tp world {world}")
            return v // world

        c.num_attention_heads = div(self.num_attention_heads, "num_attention_heads")
        if self.num_key_value_heads >= world:
            c.num_key_value_heads = div(self.num_key_value_heads, "num_key_value_heads")
            c.kv_replicas = 1
        else:
            if world % self.num_key_value_heads:
                raise ValueError("tp world not a multiple of KV heads")
            c.num_key_value_heads = 1
            c.kv_replicas = world // self.num_key_value_heads
            if c.num_attention_heads * world // self.num_key_value_heads % c.kv_replicas:
                raise ValueError("query heads do not split evenly over replicated KV heads")
        c.linear_num_key_heads = div(self.linear_num_key_heads, "linear_num_key_heads")
        c.linear_num_value_heads = div(self.linear_num_value_heads, "linear_num_value_heads")
        c.intermediate_size = div(self.intermediate_size, "intermediate_size") if self.intermediate_size else 0
        if c.intermediate_size % 128:
            raise ValueError("per-rank intermediate_size must stay a multiple of 128")
        if self.vocab_size % (world * 16):
            raise ValueError("vocab shard must be a multiple of 16 rows")
        if self.shared_expert_intermediate_size:
            c.shared_expert_intermediate_size = div(self.shared_expert_intermediate_size, "shared expert")
        if self.has_conv_layers and self.num_experts:
            # the short-conv MoE family splits every expert's inner width over the ranks (all experts on every rank)
            c.moe_intermediate_size = div(self.moe_intermediate_size, "moe_intermediate_size")
            if c.moe_intermediate_size % 128:
                raise ValueError("per-rank moe_intermediate_size must stay a multiple of 128")
        return c

    def kv_head_of_rank(self) -> int:
        """Global index of the first KV head held by this rank."""
        if self.kv_replicas > 1:
            return self.tp_rank // self.kv_replicas
        return self.tp_rank * self.num_key_value_heads

    # ---- json ------------------------------------------------------------------------------
    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), sort_keys=True)

    @staticmethod
    def from_json(text: str) -> "ModelConfig":
        d = json.loads(text)
        if "text_config" in d:
            d = d["text_config"]
        known = {f.name for f in dataclasses.fields(ModelConfig)}
        cfg = ModelConfig(**{k: v for k, v in d.items() if k in known})
        if d.get("model_type") == "qwen4_exp" and "arch" not in d:
            from .quant.hf_import import config_from_hf      # the checkpoint's own key names (1-based ple_layer_ids, indexer_n_heads, ...)
            return config_from_hf(text)
        if not cfg.layer_types and cfg.num_hidden_layers:
            interval = int(d.get("full_attention_interval", 4))
            cfg.layer_types = ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                               for i in range(cfg.num_hidden_layers)]
        cfg.validate()
        return cfg


def _pattern(n_layers: int, interval: int = 4) -> List[str]:
    return ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n_layers)]


def tiny_hybrid_config() -> ModelConfig:
    """4-layer test geometry: layers 0-2 Gated DeltaNet, layer 3 gated full attention."""
    return ModelConfig(
        hidden_size=256, num_hidden_layers=4, layer_types=_pattern(4),
        num_attention_heads=4, num_key_value_heads=2, head_dim=64,
        intermediate_size=512, partial_rotary_factor=0.25, rope_theta=1.0e7,
        linear_num_key_heads=2, linear_num_value_heads=4,
        linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4,
        rms_norm_eps=1e-6, vocab_size=4096, mtp_num_hidden_layers=1)


def small_hybrid_config(layers: int = 4) -> ModelConfig:
    """Same per-layer shapes as the 27B geometry's kernels need (head_dim 256 / 128) but narrow."""
    return ModelConfig(
        hidden_size=1024, num_hidden_layers=layers, layer_types=_pattern(layers),
        num_attention_heads=8, num_key_value_heads=2, head_dim=256,
        intermediate_size=2048, linear_num_key_heads=4, linear_num_value_heads=8,
        linear_key_head_dim=128, linear_value_head_dim=128, vocab_size=8192, mtp_num_hidden_layers=1)


def qwen_hybrid_27b_config(layers: int = 64) -> ModelConfig:
    """Dense hybrid 27B geometry (reference: docs/architecture.md:85-142)."""
    return ModelConfig(
        hidden_size=5120, num_hidden_layers=layers, layer_types=_pattern(layers),
        num_attention_heads=24, num_key_value_heads=4, head_dim=256,
        intermediate_size=17408, linear_num_key_heads=16, linear_num_value_heads=48,
        linear_key_head_dim=128, linear_value_head_dim=128, vocab_size=248320,
        mtp_num_hidden_layers=1, mrope_section=[11, 11, 10])


def qwen_hybrid_moe_config(layers: int = 48) -> ModelConfig:
    """Hybrid MoE geometry: 512 routed experts, top-10, one shared expert."""
    return ModelConfig(
        arch="qwen_hybrid_moe", hidden_size=2048, num_hidden_layers=layers, layer_types=_pattern(layers),
        num_attention_heads=16, num_key_value_heads=2, head_dim=256,
        intermediate_size=0, linear_num_key_heads=16, linear_num_value_heads=32,
        linear_key_head_dim=128, linear_value_head_dim=128, vocab_size=151936,
        num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
        shared_expert_intermediate_size=512, mtp_num_hidden_layers=0)


def llama_config(hidden: int = 4096, layers: int = 32, heads: int = 32, kv_heads: int = 8, head_dim: int = 128,
                 intermediate: int = 14336, vocab: int = 128256, theta: float = 5.0e5) -> ModelConfig:
    """Llama-style dense decoder: every layer full attention, no q/k norm, no output gate, full-width NeoX rope,
    plain-scale RMSNorm (also the graph of the dense 33B family the reference serves in w8a16;
    reference: docs/nanbeige.md:1-90)."""
    return ModelConfig(
        arch="llama", hidden_size=hidden, num_hidden_layers=layers, layer_types=["full_attention"] * layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, attn_output_gate=False, qk_norm=False,
        norm_zero_centered=False, intermediate_size=intermediate, partial_rotary_factor=1.0, rope_theta=theta,
        vocab_size=vocab, mtp_num_hidden_layers=0)


def gemma_config(hidden: int = 3840, layers: int = 48, heads: int = 16, kv_heads: int = 8, head_dim: int = 256,
                 intermediate: int = 15360, vocab: int = 262144, window: int = 1024) -> ModelConfig:
    """Gemma-style dense decoder: sandwich norms, GeGLU, q/k norm, five sliding-window layers per global layer with
    their own rope base, scaled embeddings, tied head (reference: src/model/gemma_*.{h,cpp}, docs/gemma4-plan.md)."""
    import math
    return ModelConfig(
        arch="gemma", hidden_size=hidden, num_hidden_layers=layers, layer_types=["full_attention"] * layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, attn_output_gate=False, qk_norm=True,
        intermediate_size=intermediate, partial_rotary_factor=1.0, rope_theta=1.0e6, vocab_size=vocab,
        tie_word_embeddings=True, mtp_num_hidden_layers=0, sandwich_norm=True, mlp_act="gelu_tanh", sliding_window=window,
        sliding_global_every=6, rope_local_theta=1.0e4, embed_scale=math.sqrt(hidden))


def tiny_gemma_config() -> ModelConfig:
    c = gemma_config(hidden=256, layers=4, heads=4, kv_heads=2, head_dim=64, intermediate=512, vocab=4096, window=24)
    c.sliding_global_every = 2
    return c


def lfm2_moe_config(hidden: int = 2048, layers: int = 40, heads: int = 32, kv_heads: int = 8, head_dim: int = 64,
                    intermediate: int = 11776, experts: int = 64, top_k: int = 4, moe_intermediate: int = 1536,
                    dense_layers: int = 2, vocab: int = 128000, attention_layers=None) -> ModelConfig:
    """Short-conv + attention MoE decoder (defaults: the 24B-total / 2B-active geometry): most layers are gated short
    convolutions, every fourth one (i % 4 == 2) is grouped-query attention (head_dim 64, q/k norm, full rope); the first
    layers keep a dense SwiGLU MLP, the rest route over sigmoid-scored experts with a selection bias and no shared
    expert (reference: docs/lfm2-plan.md:12-57)."""
    if attention_layers is None:
        attention_layers = [i for i in range(layers) if i % 4 == 2]
    types = ["full_attention" if i in set(attention_layers) else "conv" for i in range(layers)]
    return ModelConfig(
        arch="lfm2_moe", hidden_size=hidden, num_hidden_layers=layers, layer_types=types,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, attn_output_gate=False, qk_norm=True,
        norm_zero_centered=False, intermediate_size=intermediate, partial_rotary_factor=1.0, rope_theta=1.0e6,
        vocab_size=vocab, tie_word_embeddings=True, mtp_num_hidden_layers=0, num_experts=experts,
        num_experts_per_tok=top_k, moe_intermediate_size=moe_intermediate, shared_expert_intermediate_size=0,
        norm_topk_prob=True, moe_router="sigmoid", moe_expert_bias=True, routed_scaling_factor=1.0,
        num_dense_layers=dense_layers, short_conv_taps=3, rms_norm_eps=1e-5)


def tiny_lfm2_config() -> ModelConfig:
    return lfm2_moe_config(hidden=256, layers=5, heads=4, kv_heads=2, head_dim=64, intermediate=512, experts=8, top_k=2,
                           moe_intermediate=128, dense_layers=1, vocab=4096, attention_layers=(2, 4))


def tiny_llama_config() -> ModelConfig:
    return llama_config(hidden=256, layers=3, heads=4, kv_heads=2, head_dim=64, intermediate=512, vocab=4096, theta=1.0e4)


def tiny_moe_config() -> ModelConfig:
    return ModelConfig(
        arch="qwen_hybrid_moe", hidden_size=256, num_hidden_layers=4, layer_types=_pattern(4),
        num_attention_heads=4, num_key_value_heads=2, head_dim=64,
        intermediate_size=0, linear_num_key_heads=2, linear_num_value_heads=4,
        linear_key_head_dim=64, linear_value_head_dim=64, vocab_size=4096,
        num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128,
        shared_expert_intermediate_size=128, mtp_num_hidden_layers=0)


def qwen4_exp_config(layers: int = 48) -> ModelConfig:
    """The 4-stream MoE geometry: GDN + block-indexed sparse attention, 512 experts top-10 + shared expert, gated
    multi-stream residual, one n-gram embedding layer (reference: docs/qwen4exp-plan.md 2.1-2.4)."""
    return ModelConfig(
        arch="qwen4_exp", hidden_size=2560, num_hidden_layers=layers, layer_types=_pattern(layers),
        num_attention_heads=24, num_key_value_heads=2, head_dim=256, intermediate_size=0,
        linear_num_key_heads=16, linear_num_value_heads=48, linear_key_head_dim=128, linear_value_head_dim=128,
        vocab_size=248320, num_experts=512, num_experts_per_tok=10, moe_intermediate_size=640,
        shared_expert_intermediate_size=640, mtp_num_hidden_layers=0, mrope_section=[11, 11, 10],
        hc_count=4, hc_lowrank=320, ple_layers=[1] if layers > 1 else [], ple_embed_dim=2560, ngram_heads=16,
        indexer_heads=4, indexer_dim=128, indexer_ratio=4, indexer_budget=2048, gdn_gate_act="sigmoid", final_norm=False,
        eos_token_id=248044)


def tiny_qwen4_exp_config() -> ModelConfig:
    """4 layers (GDN, GDN with the n-gram block, GDN, sparse attention) small enough for the CPU oracle; the indexer's
    budget is 16 tokens, so a prompt of a few dozen tokens already exercises the block selection."""
    return ModelConfig(
        arch="qwen4_exp", hidden_size=256, num_hidden_layers=4, layer_types=_pattern(4),
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=0,
        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64, linear_value_head_dim=64,
        vocab_size=4096, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128,
        shared_expert_intermediate_size=128, mtp_num_hidden_layers=0,
        hc_count=4, hc_lowrank=32, ple_layers=[1], ple_embed_dim=256, ngram_heads=16,
        indexer_heads=2, indexer_dim=64, indexer_ratio=4, indexer_budget=16, gdn_gate_act="sigmoid", final_norm=False,
        eos_token_id=7)
