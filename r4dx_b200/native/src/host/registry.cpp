// Machine-readable registry of the CUDA library's kernels: what each entry point computes, on which engine, and the
// geometry constraints as testable predicates, so a caller can ask whether a model's shapes are covered instead of
// restating the rules.  A constraint is a NECESSARY condition on one named parameter; strides, alignment and buffer sizes
// stay with the entry points, which still reject what they cannot run.
// (reference: third_party/libr4d/r4d.h:523-560 and r4d_registry.hip give its library the same kind of table.)
#include <cstdlib>
#include <cstring>

#include "r4dxb_registry.h"

namespace {

const R4dxbConstraint c0[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}, {"ksplit", R4DXB_C_IN, 0, "1 2 4 8"}};
const R4dxbConstraint c1[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"count", R4DXB_C_LE, 3, nullptr}, {"count", R4DXB_C_GE, 2, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}};
const R4dxbConstraint c2[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}};
const R4dxbConstraint c3[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"world", R4DXB_C_LE, 8, nullptr}, {"world", R4DXB_C_GE, 2, nullptr}, {"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}};
const R4dxbConstraint c4[] = {{"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}, {"tmax", R4DXB_C_IN, 0, "2 8"}};
const R4dxbConstraint c5[] = {{"world", R4DXB_C_LE, 8, nullptr}, {"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}};
const R4dxbConstraint c6[] = {{"K", R4DXB_C_DIV, 128, nullptr}};
const R4dxbConstraint c7[] = {{"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "0 3 4 5"}, {"tn", R4DXB_C_IN, 0, "16 32 64 128 256 512"}};
const R4dxbConstraint c8[] = {{"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}, {"tn", R4DXB_C_IN, 0, "128 256 512"}};
const R4dxbConstraint c9[] = {{"K", R4DXB_C_DIV, 8, nullptr}};
const R4dxbConstraint c10[] = {{"world", R4DXB_C_LE, 8, nullptr}, {"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}};
const R4dxbConstraint c11[] = {{"world", R4DXB_C_LE, 8, nullptr}, {"world", R4DXB_C_GE, 2, nullptr}, {"H", R4DXB_C_DIV, 8, nullptr}};
const R4dxbConstraint c13[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"world", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c14[] = {{"world", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c15[] = {{"N", R4DXB_C_DIV, 128, nullptr}, {"K", R4DXB_C_DIV, 128, nullptr}, {"kb", R4DXB_C_IN, 0, "3 4 5"}, {"tn", R4DXB_C_IN, 0, "16 32 64 128 256"}, {"E", R4DXB_C_LE, 1024, nullptr}};
const R4dxbConstraint c16[] = {{"K", R4DXB_C_DIV, 128, nullptr}};
const R4dxbConstraint c17[] = {{"E", R4DXB_C_LE, 1024, nullptr}};
const R4dxbConstraint c18[] = {{"N", R4DXB_C_DIV, 4, nullptr}, {"K", R4DXB_C_DIV, 8, nullptr}};
const R4dxbConstraint c19[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"group", R4DXB_C_IN, 0, "32 64 128"}};
const R4dxbConstraint c20[] = {{"T", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c21[] = {{"K", R4DXB_C_DIV, 2, nullptr}};
const R4dxbConstraint c22[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"K", R4DXB_C_DIV, 2, nullptr}};
const R4dxbConstraint c24[] = {{"T", R4DXB_C_LE, 64, nullptr}};
const R4dxbConstraint c25[] = {{"k", R4DXB_C_LE, 64, nullptr}};
const R4dxbConstraint c27[] = {{"T", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c28[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"D", R4DXB_C_IN, 0, "64 128"}};
const R4dxbConstraint c29[] = {{"D", R4DXB_C_IN, 0, "64 128"}};
const R4dxbConstraint c30[] = {{"D", R4DXB_C_IN, 0, "64 128"}};
const R4dxbConstraint c31[] = {{"D", R4DXB_C_DIV, 32, nullptr}};
const R4dxbConstraint c32[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"D", R4DXB_C_LE, 256, nullptr}, {"D", R4DXB_C_DIV, 16, nullptr}};
const R4dxbConstraint c33[] = {{"D", R4DXB_C_LE, 256, nullptr}};
const R4dxbConstraint c34[] = {{"D", R4DXB_C_IN, 0, "128 256"}};
const R4dxbConstraint c35[] = {{"D", R4DXB_C_IN, 0, "64 128 256"}, {"gqa", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c39[] = {{"k", R4DXB_C_LE, 16, nullptr}, {"E", R4DXB_C_LE, 1024, nullptr}};
const R4dxbConstraint c40[] = {{"k", R4DXB_C_LE, 16, nullptr}};
const R4dxbConstraint c43[] = {{"world", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c44[] = {{"world", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint c45[] = {{"H", R4DXB_C_LE, 16384, nullptr}};
const R4dxbConstraint c46[] = {{"H", R4DXB_C_DIV, 128, nullptr}};
const R4dxbConstraint c47[] = {{"kb", R4DXB_C_IN, 0, "3 4 5"}};
const R4dxbConstraint c53[] = {{"T", R4DXB_C_LE, 16, nullptr}, {"D", R4DXB_C_IN, 0, "64 128"}};
const R4dxbConstraint c54[] = {{"H", R4DXB_C_DIV, 16, nullptr}};
const R4dxbConstraint c55[] = {{"D", R4DXB_C_DIV, 32, nullptr}};

const R4dxbConstraint cx0[] = {{"D", R4DXB_C_DIV, 32, nullptr}};
const R4dxbConstraint cx1[] = {{"world", R4DXB_C_LE, 8, nullptr}};

const R4dxbConstraint cq0[] = {{"group_size", R4DXB_C_GE, 1, nullptr}};
const R4dxbConstraint cq1[] = {{"heads", R4DXB_C_LE, 16, nullptr}, {"heads", R4DXB_C_DIV, 2, nullptr}};
const R4dxbConstraint cq2[] = {{"kernel", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint cq3[] = {{"Di", R4DXB_C_DIV, 32, nullptr}, {"Di", R4DXB_C_LE, 128, nullptr}, {"Hi", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint cq4[] = {{"D", R4DXB_C_IN, 0, "64 128 256"}, {"gqa", R4DXB_C_LE, 16, nullptr}};
const R4dxbConstraint cq8[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"k", R4DXB_C_LE, 16, nullptr}, {"E", R4DXB_C_LE, 1024, nullptr}};
const R4dxbConstraint cq7[] = {{"D", R4DXB_C_IN, 0, "64 128"}, {"gate_act", R4DXB_C_IN, 0, "0 1"}};
const R4dxbConstraint cq6[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"hc", R4DXB_C_LE, 8, nullptr}};
const R4dxbConstraint cq5[] = {{"T", R4DXB_C_LE, 8, nullptr}, {"D", R4DXB_C_IN, 0, "64 128"}, {"gate_act", R4DXB_C_IN, 0, "0 1"}};

const R4dxbKernelInfo kKernels[] = {
    {"gdn_prefill_gate", "gdn", "gdn_prefill", "GDN prefill (conv, gates, scan, gated norm) with the norm's output gate chosen by the caller",
     "D 64 / 128", "bf16 rows, fp32 state", "simt", cq7, 2},
    {"gdn_decode_gate", "gdn", "gdn_decode_rows_le_8", "the GDN step with the norm's output gate chosen by the caller (silu or sigmoid)",
     "as gdn_decode_ab without the in-kernel a / b projections", "bf16 rows, fp32 state", "simt", cq5, 3},
    {"q4x_grouped_rmsnorm", "elementwise", "grouped_rmsnorm", "zero-centred RMSNorm over consecutive channel groups of a row (stream gate, n-gram layer)",
     "any group size", "bf16", "simt", cq0, 1},
    {"q4x_hc_gate", "gemm", "stream_gate", "the whole stream gate of up to 8 rows in two launches: statistics + [down; inject] product + silu, then up product + mix",
     "T <= 8, up to 8 streams", "bf16 in, bf16 block input, fp32 injection logits", "simt", cq6, 2},
    {"q4x_hc_mid", "elementwise", "stream_gate", "silu of the scaled low-rank product of the stream gate", "", "fp32 in, bf16 out", "simt", nullptr, 0},
    {"q4x_hc_mix", "elementwise", "stream_gate", "block input = mean over the streams of sigmoid(up) * normalised stream", "", "bf16 / fp32 in, bf16 out", "simt", nullptr, 0},
    {"q4x_hc_inject", "elementwise", "stream_gate", "every stream += block output * 2 sigmoid(inject / streams)", "", "bf16 in place", "simt", nullptr, 0},
    {"q4x_embed_repeat", "elementwise", "stream_embedding", "embedding rows repeated over the residual streams", "", "bf16", "simt", nullptr, 0},
    {"q4x_ngram_gather", "elementwise", "ngram_rows", "n-gram row ids hashed from the device token history and rows gathered from the device-resident table",
     "up to 16 heads, even", "int32 tokens, bf16 rows", "simt", cq1, 2},
    {"q4x_ple_gate_value", "elementwise", "ngram_layer", "per-stream gate from the normalised key projection and residual, times the value row", "", "fp32 products, bf16 out", "simt", nullptr, 0},
    {"q4x_ple_conv", "conv", "ngram_layer", "dilated depthwise causal conv over a position-keyed ring + silu + the layer's adds",
     "(kernel - 1) * dilation < 32", "bf16", "simt", cq2, 1},
    {"q4x_qsa_index", "attn", "block_index", "indexer queries normed + roped, raw keys by position, pooled block keys of completed blocks",
     "index dim a multiple of 32 up to 128", "fp32 projection in, bf16 out", "simt", cq3, 3},
    {"q4x_qsa_select", "attn", "block_select", "block scores and the exact top-k blocks by (score, recency) as ascending token lists",
     "index dim a multiple of 32 up to 128", "bf16 keys, fp32 scores, int32 lists", "simt", cq3, 3},
    {"q4x_qsa_attn", "attn", "sparse_paged_attention", "attention over each row's token list in the fp8 paged cache, split merge, output gate",
     "head_dim 64 / 128 / 256, up to 16 query heads per KV head", "bf16 q, fp8 cache, bf16 out", "simt", cq4, 2},
    {"trellis_gemv_ex", "gemm", "trellis_linear_rows_le_8", "y = svh * H128(Q * H128(suh * act(x))) (+ residual) for up to 8 rows; RMSNorm / SwiGLU / GeGLU prologues",
     "N, K multiples of 128; cluster split 1/2/4/8 of K; kb 3/4/5", "bf16 x, packed trellis words, bf16 y", "simt+bulk-copy", c0, 5},
    {"trellis_gemv_siblings", "gemm", "trellis_linear_rows_le_8", "2 or 3 weights of one K and bit width over the same rows in one launch",
     "as trellis_gemv_ex; no residual", "bf16 x, packed trellis words, bf16 y", "simt+bulk-copy", c1, 5},
    {"trellis_gemv_mma", "gemm", "trellis_linear_rows_le_8", "the same product with code values written to tensor memory and contracted by tcgen05.mma",
     "K / ksplit <= 6144", "bf16 x, packed trellis words, bf16 y", "tcgen05", c2, 4},
    {"trellis_gemv_allreduce", "gemm+collective", "row_parallel_linear_allreduce", "row-parallel product whose epilogue pushes (value, sequence) pairs to every peer and sums them in rank order",
     "world 2..8; hidden up to the symmetric buffer", "bf16 x, packed trellis words, bf16 y, fp32 pairs over NVLink", "simt+peer-stores", c3, 5},
    {"trellis_gemv_grouped", "gemm", "moe_experts_rows_le_16", "every local expert times its planned rows (8 rows per pass), SwiGLU prologue for the down projection",
     "experts <= 65535", "bf16 x, stacked trellis words", "simt+bulk-copy", c4, 4},
    {"moe_route_plan", "moe", "moe_route_rows_le_8", "router (softmax or sigmoid + bias) and routing plan of up to 8 rows in one launch",
     "T <= 8, k <= 16, E <= 1024", "fp32 logits, int32 ids / plan, fp32 weights", "simt", cq8, 3},
    {"trellis_gemv_grouped_pairs", "gemm", "moe_experts_rows_le_16", "the grouped expert product over a compact grid: only experts named by the call's routed pairs get CTAs",
     "pairs <= 65535", "bf16 x, stacked trellis words", "simt+bulk-copy", c4, 4},
    {"trellis_gemv_grouped_ep", "gemm+collective", "moe_experts_expert_parallel", "grouped experts over rows that arrive from peers; results pushed back to the owning rank",
     "world <= 8", "bf16 rows over NVLink", "simt+peer-stores", c5, 3},
    {"trellis_input", "quant", "trellis_input_transform", "xh = fp16(H128(suh * x)), optionally x = act(gate) * up",
     "K multiple of 128", "bf16 in, fp16 out", "simt", c6, 1},
    {"trellis_gemm", "gemm", "trellis_linear_rows_ge_16", "prefill product on tcgen05 with the output Hadamard in the epilogue",
     "token tiles 16..512", "fp16 xh (TMA), packed trellis words, bf16 y", "tcgen05", c7, 4},
    {"trellis_gemm_f8", "gemm", "trellis_linear_rows_ge_16_8bit", "the same product with e4m3 code values and e4m3 activations (one scale per row), kind::f8f6f4",
     "token tiles 128/256/512", "e4m3 xq + fp32 row scales, bf16 y", "tcgen05", c8, 4},
    {"quantize_rows_e4m3", "quant", "activation_quantizer", "fp16 rows -> e4m3 rows + one fp32 scale per row",
     "K multiple of 8", "fp16 in, e4m3 + fp32 out", "simt", c9, 1},
    {"trellis_gemm_rs", "gemm+collective", "row_parallel_gemm_reduce_scatter", "prefill product whose epilogue stores partial rows into their owners' receive buffers",
     "world <= 8", "fp16 xh, bf16 partial rows over NVLink", "tcgen05+peer-stores", c10, 4},
    {"tp_reduce_push", "collective", "reduce_and_all_gather_push", "owner sums the ranks' partial rows on the residual row and stores the result into every rank's copy",
     "H multiple of 8", "bf16 rows over NVLink", "simt+peer-stores", c11, 3},
    {"tp_wait", "collective", "bounded_wait", "lets the stream pass once a counter has reached its target; records a status code otherwise",
     "", "u32 counter", "simt", nullptr, 0},
    {"tp_allreduce_rows", "collective", "allreduce_rows_le_8", "all-reduce of up to 8 bf16 rows by the push protocol",
     "world <= 8", "bf16 rows, fp32 pairs over NVLink", "simt+peer-stores", c13, 2},
    {"tp_argmax_merge", "collective", "vocab_parallel_argmax", "(value, id) pairs pushed to every peer; lowest id wins ties",
     "world <= 8", "fp32 values, int32 ids", "simt+peer-stores", c14, 1},
    {"trellis_gemm_grouped", "gemm", "moe_experts_rows_gt_16", "grouped experts on tcgen05: a token tile is one expert's next rows",
     "E <= 1024 local experts", "fp16 sorted rows, stacked trellis words", "tcgen05", c15, 5},
    {"trellis_input_grouped", "quant", "moe_input_transform", "per-expert input signs + Hadamard for the planned pairs in expert order",
     "K multiple of 128", "bf16 in, fp16 out", "simt", c16, 1},
    {"moe_tiles", "moe", "moe_tile_list", "token tiles of a routing plan built on the device",
     "E <= 1024", "int32", "simt", c17, 1},
    {"linear_tc", "gemm", "plain_linear_rows_any", "y = act(x W^T + bias) + residual: dense bf16 / fp16 W by TMA, or w4a16 W widened by the decode warps",
     "dense: N % 4, K % 8; w4a16: N, K % 128, group 32/64/128", "bf16 / fp16 / w4a16, bf16 or fp32 y", "tcgen05", c18, 2},
    {"w4a16_gemv", "gemm", "w4a16_linear_rows_le_8", "group-quantised 4-bit head product",
     "rows * K * 2 <= 200 KB", "bf16 x, nibbles + fp16 scale / zero", "simt", c19, 2},
    {"w8a16_gemv", "gemm", "w8a16_linear_rows_le_8", "group-quantised 8-bit product",
     "", "bf16 x, u8 + fp16 scale", "simt", c20, 1},
    {"bf16_gemv", "gemm", "bf16_linear", "dense bf16 product, fp32 out (tiled above 8 rows)",
     "", "bf16", "simt", c21, 1},
    {"bf16_gemv_norm", "gemm", "bf16_linear_rows_le_8", "the same with the RMSNorm of the rows folded in",
     "", "bf16", "simt", c22, 2},
    {"argmax_rows", "sampling", "row_argmax", "two-stage argmax with an id offset; lowest id wins ties",
     "", "fp32 or bf16 logits", "simt", nullptr, 0},
    {"argmax_rows_static", "sampling", "row_argmax", "the same with its partials in a fixed device array (no caller scratch)",
     "rows <= 64", "fp32 or bf16 logits", "simt", c24, 1},
    {"topk_lse", "sampling", "topk_and_logsumexp", "top-k values / ids in canonical order and the row's log-sum-exp",
     "k <= 64", "fp32 logits", "simt", c25, 1},
    {"repetition_penalty", "sampling", "repetition_penalty", "in-place penalty over a token-seen mask",
     "", "fp32 logits", "simt", nullptr, 0},
    {"spec_accept", "sampling", "speculative_accept", "longest accepted draft prefix + emitted tokens of a verify window",
     "rows <= 8", "int32", "simt", c27, 1},
    {"gdn_decode_ab", "gdn", "gdn_step_rows_le_8", "conv + gates + delta-rule recurrence + gated norm with a write-once log; optional in-kernel a / b projections",
     "head dim 64 / 128", "bf16 activations, fp32 state", "simt", c28, 2},
    {"gdn_decode_batch", "gdn", "gdn_step_batched", "the same for B sequences, one row each",
     "head dim 64 / 128", "bf16 activations, fp32 state", "simt", c29, 1},
    {"gdn_prefill", "gdn", "gdn_chunk_scan", "chunked delta-rule scan (64-token chunks, triangular solve, TF32 mma.sync state recurrence) or the token loop",
     "chunked path: head dim 128, >= 128 rows", "bf16 activations, fp32 state", "mma.sync", c30, 1},
    {"attn_precore", "attn", "qk_norm_rope_kv_write", "per-head norms, partial rope, fp8 KV write into the paged cache",
     "D % 32", "bf16 in, e4m3 cache", "simt", c31, 1},
    {"attn_decode", "attn", "paged_decode_attention", "split-KV decode attention over the fp8 paged cache + combine",
     "rows <= 8, D <= 256", "bf16 q, e4m3 cache", "mma.sync", c32, 3},
    {"attn_decode_batch", "attn", "paged_decode_attention_batched", "the same for B sequences with per-slot block tables",
     "D <= 256", "bf16 q, e4m3 cache", "mma.sync", c33, 1},
    {"attn_prefill_tc", "attn", "paged_prefill_attention", "causal / windowed prefill attention with S, P and O in tensor memory",
     "head dim 128 / 256", "bf16 q, e4m3 cache", "tcgen05", c34, 1},
    {"attn_prefill_ex", "attn", "paged_prefill_attention", "the mma.sync kernel: other head dims and per-row key limits (image blocks)",
     "head dim 64 / 128 / 256, gqa <= 8", "bf16 q, e4m3 cache", "mma.sync", c35, 2},
    {"vit_attention", "attn", "vision_attention", "non-causal attention over variable-length image segments",
     "", "bf16", "simt", nullptr, 0},
    {"vit_rope", "attn", "vision_rope", "2-D rotary embedding of the fused qkv rows",
     "", "bf16", "simt", nullptr, 0},
    {"short_conv", "conv", "gated_short_conv", "C * causal_fir(B * x) over a position-keyed ring",
     "ring of 32 rows", "bf16", "simt", nullptr, 0},
    {"moe_router", "moe", "softmax_topk_router", "softmax top-k with optional renormalisation",
     "k <= 16, experts <= 1024", "fp32 logits", "simt", c39, 2},
    {"moe_router_sigmoid", "moe", "sigmoid_topk_router", "sigmoid scores with a selection bias",
     "k <= 16", "fp32 logits", "simt", c40, 1},
    {"moe_plan", "moe", "routing_plan", "pairs sorted by expert + per-expert offsets on the device",
     "", "int32", "simt", nullptr, 0},
    {"moe_combine", "moe", "expert_combine", "weighted sum of the pairs + gated shared expert + residual",
     "", "bf16", "simt", nullptr, 0},
    {"ep_dispatch", "collective", "expert_parallel_dispatch", "rows and routing pushed to the ranks that own the experts",
     "world <= 8", "bf16 rows over NVLink", "simt+peer-stores", c43, 1},
    {"ep_combine", "collective", "expert_parallel_combine", "waits (bounded) for the experts' rows and combines them",
     "world <= 8", "bf16 rows", "simt", c44, 1},
    {"rotate_residual", "quant", "residual_rotation", "x <- x Q or x Q^T (signs x block Hadamard x orthogonal mix)",
     "H / block <= 8, H <= 16384", "bf16 rows, fp32 signs / mix", "simt", c45, 1},
    {"rotate_rows", "quant", "block_hadamard", "in-place 128-wide Hadamard with optional signs",
     "H multiple of 128", "bf16", "simt", c46, 1},
    {"trellis_encode_tiles", "quant", "viterbi_encoder", "trellis search of 16x16 tiles, one CTA per tile",
     "kb 3/4/5", "fp32 values in, packed words out", "simt", c47, 1},
    {"rmsnorm_bf16", "elementwise", "rmsnorm", "RMSNorm (zero-centred, plain or weightless)",
     "", "bf16", "simt", nullptr, 0},
    {"add_rmsnorm_bf16", "elementwise", "norm_add", "normalise a branch output and add it to the residual stream",
     "", "bf16", "simt", nullptr, 0},
    {"layernorm_bf16", "elementwise", "layernorm", "LayerNorm with bias",
     "", "bf16", "simt", nullptr, 0},
    {"embed_gather_bf16", "elementwise", "embedding", "row gather",
     "", "bf16", "simt", nullptr, 0},
    {"silu_mul_bf16", "elementwise", "swiglu", "silu(gate) * up",
     "", "bf16", "simt", nullptr, 0},
    {"dflash_attention", "dflash", "drafter_block_attention", "bidirectional attention of the draft block over its ring and itself",
     "rows <= 16, head dim 64 / 128", "bf16", "simt", c53, 2},
    {"dflash_conv", "dflash", "drafter_conv", "two-tap conv with per-channel base and per-group dynamic kernels",
     "H multiple of 16", "bf16", "simt", c54, 1},
    {"dflash_norm_rope", "dflash", "drafter_norm_rope", "per-head RMSNorm + full-width NeoX rope",
     "D % 32", "bf16", "simt", c55, 1},
    {"attn_precore_batch", "attn", "qk_norm_rope_kv_write_batched", "the pre-core step for B sequences with per-slot block tables",
     "D % 32", "bf16 in, e4m3 cache", "simt", cx0, 1},
    {"residual_add_bf16", "elementwise", "residual_add", "res += delta",
     "", "bf16", "simt", nullptr, 0},
    {"bias_act_bf16", "elementwise", "bias_activation", "x = act(x + bias): none, tanh-GELU or erf-GELU",
     "", "bf16", "simt", nullptr, 0},
    {"ep_plan", "collective", "expert_parallel_plan", "waits (bounded) for the peers' routing, then plans the local experts' rows",
     "world <= 8", "int32", "simt", cx1, 1},
};
constexpr int kCount = static_cast<int>(sizeof(kKernels) / sizeof(kKernels[0]));

bool InSet(const char* set, long long v) {
  // `set` is a list of space-separated decimal words
  const char* p = set;
  while (*p) {
    char* end = nullptr;
    const long long w = strtoll(p, &end, 10);
    if (end == p) break;
    if (w == v) return true;
    p = end;
    while (*p == ' ') ++p;
  }
  return false;
}

}  // namespace

extern "C" {

int r4dxb_kernel_count(void) { return kCount; }

const R4dxbKernelInfo* r4dxb_kernel_at(int i) { return (i >= 0 && i < kCount) ? &kKernels[i] : nullptr; }

/* 1 when every constraint of kernel `name` whose key appears in `keys` holds for the given values (keys the kernel does
 * not constrain are ignored, constrained keys that are not given are not tested); 0 when one fails; -1 for an unknown name. */
int r4dxb_kernel_covers(const char* name, const char* const* keys, const long long* vals, int n) {
  for (int i = 0; i < kCount; ++i) {
    if (strcmp(kKernels[i].name, name) != 0) continue;
    for (int c = 0; c < kKernels[i].n_constraints; ++c) {
      const R4dxbConstraint& k = kKernels[i].constraints[c];
      for (int j = 0; j < n; ++j) {
        if (strcmp(keys[j], k.key) != 0) continue;
        const long long v = vals[j];
        bool ok = true;
        switch (k.op) {
          case R4DXB_C_EQ: ok = v == k.ival; break;
          case R4DXB_C_LE: ok = v <= k.ival; break;
          case R4DXB_C_GE: ok = v >= k.ival; break;
          case R4DXB_C_DIV: ok = k.ival != 0 && v % k.ival == 0; break;
          case R4DXB_C_IN: ok = InSet(k.sval, v); break;
          default: ok = false;
        }
        if (!ok) return 0;
      }
    }
    return 1;
  }
  return -1;
}

}  // extern "C"
