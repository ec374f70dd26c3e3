/* C ABI of libr4dxb_cuda.so: every entry point takes raw device pointers and a CUDA stream
 * handle, launches on that stream and returns 0 or an error code (a cudaError_t value, or one
 * of the R4DXB_* codes below).  Nothing on a launch path allocates or synchronises unless its
 * comment says so, so the decode step can be captured in a CUDA graph. */
#ifndef R4DXB_H_
#define R4DXB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define R4DXB_BAD_ARG 10001
#define R4DXB_UNSUPPORTED 10002
#define R4DXB_TOO_LARGE 10003

unsigned long long r4dxb_launch_count(void);
void r4dxb_launch_count_reset(void);

/* ---- elementwise / norms ------------------------------------------------------------------ */
int r4dxb_embed_gather_bf16(const int* ids, const void* table, void* out, int T, int H, int V, void* stream);
/* mode bit0: weight is zero-centred (1 + w); bit1: no weight */
int r4dxb_rmsnorm_bf16(const void* x, const void* w, void* out, int T, int H, float eps, int mode, void* stream);
/* res += delta (rounded to bf16 in place), out = rmsnorm(res) */
int r4dxb_add_rmsnorm_bf16(void* res, const void* delta, const void* w, void* out, int T, int H, float eps, int mode,
                           void* stream);
int r4dxb_layernorm_bf16(const void* x, const void* w, const void* b, void* out, int T, int H, float eps, void* stream);
int r4dxb_silu_mul_bf16(const void* gate_up, void* out, int T, int I, void* stream);
int r4dxb_residual_add_bf16(void* res, const void* delta, long long n, void* stream);
int r4dxb_bias_act_bf16(void* x, const void* bias, int T, int H, int act, void* stream);

/* Speculative-window acceptance (greedy or sample-and-match: next_ids = the target's pick per row):
 * out[0] = rows to commit, out[1..out[0]] = emitted tokens; n_replay (optional) receives out[0]. */
int r4dxb_spec_accept(const int* next_ids, const int* draft, int T, int* out, int* n_replay, void* stream);

/* ---- weight-streaming GEMMs for T <= 8 rows ------------------------------------------------- */
/* y[T,N] (bf16) = svh * H(Q . H(suh * x)) (+ residual), trellis-coded Q, kb in {3,4,5}.
 * ksplit in {1,2,4,8} CTAs share one 128-row block through a thread-block cluster. */
int r4dxb_trellis_gemv(const void* words, const void* suh, const void* svh, const void* x, void* y,
                       const void* residual, int T, int N, int K, int kb, int ksplit, void* stream);
/* logits[T,N] = x . dequant(wq)^T, asymmetric 4-bit groups of 32/64/128 along K; out_f32 selects
 * fp32 or bf16 output */
int r4dxb_dflash_norm_rope(void* x, const void* w, const int* positions, int T, int heads, int D, float theta, float eps,
                           void* stream);
int r4dxb_dflash_conv(const void* h, const void* base, const void* dyn, void* out, int T, int H, void* stream);
int r4dxb_dflash_attention(const void* q, const void* kb, const void* vb, const void* ring_k, const void* ring_v, void* out,
                           int T, int Hq, int Hkv, int D, int window, int lo, int n, void* stream);
int r4dxb_vit_rope(void* qkv, const int* pos_hw, int T, int H, int D, float theta, void* stream);
int r4dxb_vit_attention(const void* qkv, void* out, const int* cu_seqlens, int nseg, int T, int H, int D, void* stream);
int r4dxb_w8a16_gemv(const void* wq, const void* ws, const void* x, void* y, int T, int N, int K, int group, int out_f32,
                     void* stream);
int r4dxb_rotate_rows(void* x, const void* signs, long long T, int H, int mode, void* stream);
/* Residual-stream rotation in place on bf16 rows [T, H]: x <- x Q (inverse 0) or x Q^T (inverse 1),
 * Q = diag(signs) . blockdiag(Hadamard_B / sqrt(B)) . (mix (x) I_B); signs fp32 [H], mix fp32 [H/B, H/B], H/B <= 8. */
int r4dxb_rotate_residual(void* x, const float* signs, const float* mix, long long T, int H, int B, int inverse, void* stream);
int r4dxb_w4a16_gemv(const void* wq, const void* wsz, const void* x, void* y, int T, int N, int K, int group,
                     int out_f32, void* stream);
/* y[T,N] (fp32) = x[T,K] (bf16) . W[N,K]^T (bf16): small dense projections (gates, router) */
int r4dxb_bf16_gemv(const void* W, const void* x, float* y, int T, int N, int K, void* stream);
/* same for T <= 8 rows of the residual stream with the zero-centred RMSNorm folded in */
int r4dxb_bf16_gemv_norm(const void* W, const void* x, const void* norm_w, float eps, float* y, int T, int N, int K,
                         void* stream);

/* ---- sampling ------------------------------------------------------------------------------- */
/* row-wise argmax with ties to the lowest index; writes id + id_offset (int32) and the max (f32).
 * scratch: 2 * T * 256 * 4 bytes */
int r4dxb_argmax_rows(const void* logits, int is_f32, int T, int V, int id_offset, int* out_ids, float* out_vals,
                      void* scratch, void* stream);

/* row summary for exact host sampling: top-K (K <= 64) raw logits + ids (canonical order) and the log-sum-exp
 * of logits / temperature.  scratch: T * 128 * (2K + 2) * 4 bytes */
int r4dxb_topk_lse(const float* logits, int T, int V, int K, float temperature, int id_offset, float* out_vals, int* out_ids,
                   float* out_lse, void* scratch, void* stream);
/* HF repetition penalty on the distinct ids of `seen` */
int r4dxb_repetition_penalty(float* logits, int V, const int* seen, int n, float penalty, void* stream);

/* ---- Gated DeltaNet ------------------------------------------------------------------------- */
/* Fused decode / verify step (T <= 8 rows): conv1d ring + SiLU, L2 norm, gates, delta rule, gated
 * RMSNorm.  The base state is only written when *n_replay > 0 (commit of the previous call's
 * accepted rows); this call's rows go to the log.  D (= key = value head dim) in {64, 128}. */
/* The same step with the a / b projections computed in the kernel (ab_w [2H, K] bf16: a rows then b rows; x [T, K]
 * residual rows; in_norm_w [K] the layer's zero-centred input RMSNorm weight); ab_w == null reads `ab` instead. */
int r4dxb_gdn_decode_ab(const void* mixed, const void* z, const float* ab, const void* ab_w, const void* x,
                        const void* in_norm_w, int K, float in_eps, const void* conv_w, const float* A_log,
                        const float* dt_bias, const void* norm_w, void* ring, float* state, float* log_u, float* log_k,
                        float* log_eg, const int* positions, const int* n_replay, void* out, int T, int H, int Hk, int D,
                        float eps, void* stream);
int r4dxb_gdn_decode(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                     const float* dt_bias, const void* norm_w, void* ring, float* state, float* log_u, float* log_k,
                     float* log_eg, const int* positions, const int* n_replay, void* out, int T, int H, int Hk, int D,
                     float eps, void* stream);

/* ---- attention (fp8 e4m3 paged KV, 16-token blocks) ------------------------------------------ */
int r4dxb_attn_precore(const void* qg, const void* k, const void* v, const void* q_norm, const void* k_norm,
                       const float* k_descale, const float* v_descale, const int* positions, const int* block_table,
                       void* q_out, void* cache, int T, int Hq, int Hkv, int D, int rotary_dim, float theta, float eps,
                       int q_stride, void* stream);   /* q_norm / k_norm may be null (no per-head norm); q_stride 0 = 2D */
/* scratch: part_acc = splits*Hkv*G*D floats, part_ml = splits*Hkv*G*2 floats, G = Hq/Hkv*T */
int r4dxb_attn_decode(const void* q, const void* qg, const void* cache, const int* block_table, const int* positions,
                      const float* k_descale, const float* v_descale, float* part_acc, float* part_ml, void* out,
                      int T, int Hq, int Hkv, int D, int splits, int gated, void* stream);

/* Sibling projections in one launch of the weight-streaming kernel: `count` (2 or 3) trellis weights of the same K and
 * bit width read the same rows x through the same prologue; weight i writes y[i] [T, n[i]] (no residual). */
int r4dxb_trellis_gemv_siblings(int count, const void* const* words, const void* const* suh, const void* const* svh,
                                void* const* y, const int* n, const void* x, const void* norm_w, float eps, int prologue, int T,
                                int K, int kb, int ksplit, void* stream);

/* A/B switch: one-token steps use the warp-autonomous decode-attention kernel (default on); off = the window kernel
 * for every row count, which makes one-row and many-row calls bit-identical. */
void r4dxb_set_attn_decode_row(int on);

/* ---- trellis GEMM on tcgen05 / TMEM (T >= 16 rows) ------------------------------------------- */
/* xh = fp16(H128(suh * x)); mode 1 fuses silu(gate) * up over fused [T, 2K] rows */
int r4dxb_trellis_input(const void* in, const void* suh, void* out, int T, int K, int mode, void* stream);
/* y[T,N] bf16 from xh[T,K]; kb = 0: w is dense fp16 [N,K]; kb in {3,4,5}: packed trellis words.
 * tn: token tile 16/32/64/128/256.  *status (device int) becomes non-zero if a bounded wait ran out. */
long long r4dxb_trellis_encode_scratch_bytes(int kb, int ctas);
int r4dxb_trellis_encode_tiles(const float* vals, int ntiles, int kb, void* words, float* err, void* scratch, int ctas,
                               void* stream);
void r4dxb_set_gemm_decode_warps(int n);
int r4dxb_trellis_gemm_rs(const void* w, const void* svh, const void* xh, int T, int N, int K, int kb, int tn, int* status,
                          void* const* recv, void* const* cnt, int world, int rank, int rows_per_rank, void* stream);
int r4dxb_tp_reduce_push(void* const* x, void* const* xflag, const void* recv, const void* cnt, unsigned target, int world, int rank,
                         int rows_per_rank, int rows_own, int H, int spin_limit, int* status, void* stream);
int r4dxb_tp_wait(const void* flag, unsigned target, int spin_limit, int code, int* status, void* stream);
int r4dxb_trellis_gemm(const void* w, const void* svh, const void* xh, void* y, const void* residual, int T, int N, int K,
                       int kb, int tn, int* status, void* stream);

/* Plain linear on the same tensor-core kernel, any T: y[T,N] = x[T,K] W^T (+ bias[N] bf16) (+ residual[T,N] bf16).
 * kind 0: dense 16-bit W[N,K] (bf16 != 0: W and x bf16, else fp16); kind 1: w4a16 (w = nibbles [N][K/8] u32,
 * wsz = [N][K/group] fp16 scale | fp16 -(1024 + zero) << 16; x fp16; N, K multiples of 128).  Dense: N % 4 == 0,
 * K % 8 == 0.  out_f32 bit 0: y fp32; bits 8-15: activation after the bias (0 none, 1 tanh-GELU, 2 erf-GELU). */
int r4dxb_linear_tc(const void* w, const void* wsz, int kind, int group, int bf16, const void* x, void* y, int out_f32,
                    const void* bias, const void* residual, int T, int N, int K, int tn, int* status, void* stream);

/* 8-bit prefill product (opt-in): r4dxb_quantize_rows_e4m3 turns fp16 rows [T, K] into e4m3 rows + one fp32 scale per row
 * (scale = rowmax / 448); r4dxb_trellis_gemm_f8 multiplies them with e4m3 code values on tcgen05.mma kind::f8f6f4
 * (K per shared-memory slab 128, fp32 accumulate, row scale in the epilogue).  K a multiple of 128, tn 128 / 256 / 512. */
int r4dxb_quantize_rows_e4m3(const void* xh, void* xq, float* scale, int T, int K, void* stream);
int r4dxb_trellis_gemm_f8(const void* w, const void* svh, const void* xq, const float* x_scale, void* y, const void* residual,
                          int T, int N, int K, int kb, int tn, int* status, void* stream);

/* Grouped experts on the tensor cores: tile list of a routing plan (E <= 1024 local experts, tiles [2 * max_tiles]),
 * per-expert input transform of the planned pairs in expert order (xdiv: pairs per input row; mode as
 * r4dxb_trellis_input), and y[perm[p]] = svh[e] * H128(xh[p] Q_e^T) with one expert's next tn rows per token tile
 * (tn 16/32/64/128, max_tiles >= P / tn + E). */
int r4dxb_moe_tiles(const int* offsets, int E, int tn, int* tiles, int* ntiles, int max_tiles, void* stream);
int r4dxb_trellis_input_grouped(const void* in, const void* suh, void* out, const int* offsets, const int* perm, int E, int P,
                                int K, int xdiv, int mode, void* stream);
int r4dxb_trellis_gemm_grouped(const void* words, const void* svh, const void* xh, void* y, const int* offsets, const int* perm,
                               const int* tiles, const int* ntiles, int max_tiles, int P, int E, int N, int K, int kb, int tn,
                               int* status, void* stream);

/* ---- batched decode (B sequences, one new token each; per-sequence state indexed by slot) ---------- */
int r4dxb_gdn_decode_batch(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                           const float* dt_bias, const void* norm_w, void* ring, float* state, float* log_u, float* log_k,
                           float* log_eg, const int* positions, const int* n_replay, const int* row_slot, void* out, int B,
                           int H, int Hk, int D, float eps, void* stream);
int r4dxb_attn_precore_batch(const void* qg, const void* k, const void* v, const void* q_norm, const void* k_norm,
                             const float* k_descale, const float* v_descale, const int* positions, const int* block_tables,
                             const int* row_slot, int table_stride, void* q_out, void* cache, int B, int Hq, int Hkv, int D,
                             int rotary_dim, float theta, float eps, int q_stride, void* stream);
int r4dxb_attn_decode_batch(const void* q, const void* qg, const void* cache, const int* block_tables, const int* row_slot,
                            int table_stride, const int* positions, const float* k_descale, const float* v_descale,
                            float* part_acc, float* part_ml, void* out, int B, int Hq, int Hkv, int D, int splits, int gated,
                            void* stream);

/* ---- prefill (long chunks) ---------------------------------------------------------------------- */
/* GDN over T rows starting at position pos0: conv prep, register-resident recurrence, gated norm.
 * Commits the state (no log).  fp32 scratch: q,k [T,Hk,D], v,o [T,H,D], eg,beta [T,H]. */
int r4dxb_gdn_prefill(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                      const float* dt_bias, const void* norm_w, void* ring, float* state, float* q, float* k, float* v,
                      float* eg, float* beta, float* o, void* out, int T, int H, int Hk, int D, int pos0, float eps, float* ws,
                      void* stream);
long long r4dxb_gdn_chunk_ws_floats(int T, int H);
/* causal GQA attention of T query rows at positions pos0.. over the paged fp8 cache (rows already written) */
/* The same with per-row key limits: key_limit [T] int32 (-1 = none) lets row t also see keys up to that absolute position,
 * which must belong to this call (rows of an image block attend to the whole block on sliding-window layers). */
int r4dxb_attn_prefill_ex(const void* q, const void* qg, const void* cache, const int* block_table, const float* k_descale,
                          const float* v_descale, void* out, int T, int Hq, int Hkv, int D, int pos0, int flags,
                          const int* key_limit, void* stream);
int r4dxb_attn_prefill(const void* q, const void* qg, const void* cache, const int* block_table, const float* k_descale,
                       const float* v_descale, void* out, int T, int Hq, int Hkv, int D, int pos0, int gated, void* stream);

/* Same kernel with a fused activation producer: prologue 0 = x is the activation [T,K];
 * 1 = x is the residual stream and the activation is RMSNorm(x) with zero-centred weight norm_w;
 * 2 = x is fused [gate | up] rows [T,2K] and the activation is bf16(silu(gate) * up). */
int r4dxb_trellis_gemv_ex(const void* words, const void* suh, const void* svh, const void* x, void* y,
                          const void* residual, const void* norm_w, float eps, int prologue, int T, int N, int K, int kb,
                          int ksplit, void* stream);

/* ---- mixture of experts ---------------------------------------------------------------------------- */
int r4dxb_moe_router(const float* logits, int T, int E, int k, int renorm, int* ids, float* weights, void* stream);
int r4dxb_moe_router_sigmoid(const float* logits, const float* bias, int T, int E, int k, int renorm, float scale, int* ids,
                             float* weights, void* stream);
/* Gated short convolution: bcx [T, 3H] bf16 (B | C | x), w [H, L] bf16, ring [32, H] bf16 keyed by position & 31 */
int r4dxb_short_conv(const void* bcx, const void* w, void* ring, const int* positions, void* out, int T, int H, int L,
                     void* stream);
int r4dxb_moe_plan(const int* ids, int npairs, int E, int e_begin, int e_count, int* offsets, int* perm, void* stream);
int r4dxb_moe_combine(const void* y_pairs, const int* ids, const float* weights, const void* shared, const float* shared_gate,
                      const void* residual, void* out, int T, int H, int k, void* stream);
/* one launch for every local expert; experts' packed weights lie back to back; tmax in {2, 8} */
int r4dxb_trellis_gemv_grouped(const void* words, const void* suh, const void* svh, const void* x, void* y,
                               const int* offsets, const int* perm, int in_div, int pass, int tmax, int prologue,
                               int experts, int N, int K, int kb, int ksplit, void* stream);

/* Expert-parallel form: input rows arrive from peer GPUs (ready flags, double-buffered by the parity of the
 * device call counter *seq_ptr + 1) and, when ep_y is given, output rows go to the combine buffer of the rank
 * that owns the token (ep_y[rank]: [2][ep_P][N] bf16, ep_cnt[rank]: [2][ep_P] arrival counters). */
int r4dxb_trellis_gemv_grouped_ep(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                  const int* offsets, const int* perm, int in_div, int pass, int tmax, int prologue,
                                  int experts, int N, int K, int kb, int ksplit, const void* seq_ptr, const void* ready,
                                  long long x_par_stride, long long ready_par_stride, void* const* ep_y, void* const* ep_cnt,
                                  int ep_P, int world, int spin_limit, int* status, void* stream);
/* expert-parallel all-to-all around it (native/src/cuda/ep.cu) */
int r4dxb_ep_dispatch(void* const* meta, void* const* xrecv, void* const* xflag, const void* h, const int* ids,
                      const void* seq_ptr, int T, int k, int H, int P, int world, int rank, int experts_per_rank, void* stream);
int r4dxb_ep_plan(const void* meta_local, const void* seq_ptr, int world, int P, int e_begin, int e_count, int* offsets,
                  int* perm, int spin_limit, int* status, void* stream);
int r4dxb_ep_combine(const void* comb, void* ccount, void* seq_ptr, const int* ids, const float* weights, const void* shared,
                     const float* shared_gate, void* x, int T, int H, int k, int P, int blocks_per_row, int spin_limit,
                     int* status, void* stream);

/* ---- tensor parallel: collectives issued from inside the compute kernels ------------------------- */
/* Row-parallel trellis linear (T <= 8) + all-reduce over NVLink peer memory + residual, one kernel.
 * recv[p]: rank p's receive buffer, [2][world][8][N] (fp32 value, u32 sequence) pairs, zero-initialised and
 * peer-mapped; block_seq ([N/128] u32, zeros) and status (int) are this rank's own.  Every wait is bounded
 * by spin_limit polls; when one runs out *status becomes 100 + the rank that did not answer. */
int r4dxb_trellis_gemv_allreduce(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                 const void* residual, int prologue, int T, int N, int K, int kb, int ksplit,
                                 void* const* recv, void* block_seq, int* status, int world, int rank, int spin_limit,
                                 void* stream);

/* router (mode 0: softmax, 1: sigmoid + selection bias) and routing plan of T <= 8 rows in one launch; the same ids, weights,
 * offsets and perm as r4dxb_moe_router / r4dxb_moe_router_sigmoid followed by r4dxb_moe_plan */
int r4dxb_moe_route_plan(const float* logits, const float* bias, int T, int E, int k, int renorm, int mode, float scale, int* ids,
                         float* weights, int e_begin, int e_count, int* offsets, int* perm, void* stream);
/* grouped expert product over a compact grid: blockIdx.z runs over the call's `pairs` routed (row, slot) pairs (pair_ids =
 * their global expert ids) instead of every local expert; results equal r4dxb_trellis_gemv_grouped */
int r4dxb_trellis_gemv_grouped_pairs(const void* words, const void* suh, const void* svh, const void* x, void* y,
                                     const int* offsets, const int* perm, const int* pair_ids, int pairs, int e_begin,
                                     int in_div, int pass, int tmax, int prologue, int experts, int N, int K, int kb, int ksplit,
                                     void* stream);
/* GDN prefill with the output gate of its norm chosen by the caller (0 silu, 1 sigmoid) */
int r4dxb_gdn_prefill_gate(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                           const float* dt_bias, const void* norm_w, void* ring, float* state, float* q, float* k, float* v,
                           float* eg, float* beta, float* o, void* out, int T, int H, int Hk, int D, int pos0, float eps,
                           float* ws, int gate_act, void* stream);
/* GDN decode step with the output gate of its norm chosen by the caller: gate_act 0 = silu(z), 1 = sigmoid(z). */
int r4dxb_gdn_decode_gate(const void* mixed, const void* z, const float* ab, const void* conv_w, const float* A_log,
                          const float* dt_bias, const void* norm_w, void* ring, float* state, float* log_u, float* log_k,
                          float* log_eg, const int* positions, const int* n_replay, void* out, int T, int H, int Hk, int D,
                          float eps, int gate_act, void* stream);

/* ---- qwen4_exp family: gated multi-stream residual, n-gram embedding layer, block-selecting attention ------------- */
/* out = bf16(x * rsqrt(mean(x^2 over the group) + eps) * (1 + w)) for `groups` groups of `group_size` channels per row */
int r4dxb_q4x_grouped_rmsnorm(const void* x, const void* w, void* out, int rows, int groups, int group_size, float eps, void* stream);
/* mid [rows, lowrank] bf16 = silu(down / hc); down = the first `lowrank` columns of an fp32 product with `stride` columns */
int r4dxb_q4x_hc_mid(const float* down, void* mid, int rows, int lowrank, int stride, int hc, void* stream);
/* x [rows, hidden] = mean over the hc streams of sigmoid(up) * n;  n bf16 [rows, hc * hidden], up fp32 of the same shape */
int r4dxb_q4x_hc_mix(const void* n, const float* up, void* x, int rows, int hc, int hidden, void* stream);
/* h [rows, hc * hidden] += block_out [rows, hidden] * 2 sigmoid(inject / hc) per stream; inject = hc fp32 columns of a row of `stride` */
int r4dxb_q4x_hc_inject(void* h, const void* block_out, const float* inject, int rows, int hc, int hidden, int stride, void* stream);
/* the stream gate for T <= 8 rows in two launches (norm statistics, [down; inject] product, silu, up product, mix):
 * x [T, hidden] = the block input, injv [T, n_inject] fp32 = the raw injection logits (n_inject = 0: the final mixer) */
int r4dxb_q4x_hc_gate(const void* h, const void* norm_w, const void* w_down_inject, const void* w_up, void* mid, float* injv,
                      float* rstd, void* x, int T, int hc, int hidden, int lowrank, int n_inject, float eps, void* stream);
/* out [rows, hc * hidden] = embedding row of ids[r] repeated over the streams (ids outside the table give NaN rows) */
int r4dxb_q4x_embed_repeat(const void* table, const int* ids, void* out, int rows, int vocab, int hidden, int hc, void* stream);
/* n-gram rows of T tokens from the device-resident table: ids hashed from the device token history `hist` (indexed by
 * position; read for the two positions before the call, written for the call's rows) and gathered into emb [T, heads * head_dim] */
int r4dxb_q4x_ngram_gather(const int* ids, const int* positions, int* hist, const void* table, void* emb, int T, int heads,
                           int head_dim, long long table_rows, const long long* mult, const unsigned long long* primes,
                           const unsigned long long* offsets, long long eos, void* stream);
/* gated_value [rows, hc * hidden] = sigmoid(signed sqrt(<norm(key_proj), norm(h)> / sqrt(hidden))) * value, per stream */
int r4dxb_q4x_ple_gate_value(const float* key_proj, const void* h, const float* value, const void* norm_key, const void* norm_query,
                             void* gated_value, int rows, int hc, int hidden, float eps, void* stream);
/* h += gated_value + silu(dilated depthwise causal conv of gvn); ring [32, channels] holds gvn by position & 31 */
int r4dxb_q4x_ple_conv(const void* gvn, const void* gated_value, const void* conv_w, void* ring, void* h, const int* positions,
                       int rows, int channels, int kernel, int dilation, void* stream);
/* indexer prologue: queries normed + roped, raw keys stored by position, block keys of the blocks these rows complete */
int r4dxb_q4x_qsa_index(const float* qk, const void* q_norm, const void* k_norm, const int* positions, void* idx_q, void* raw_keys,
                        void* block_keys, int T, int Hi, int Di, int ratio, int rotary_dim, float theta, float eps, void* stream);
/* block scores + exact top-k selection (ties: the most recent block wins); sel_count[t] = -1 for rows that attend densely */
int r4dxb_q4x_qsa_select(const void* idx_q, const void* block_keys, const int* positions, float* scores, int* sel_tokens, int* sel_count,
                         int T, int Hi, int Di, int ratio, int topk, int nb_max, int stride, int sel_stride, void* stream);
/* attention over each row's token list (fp8 paged cache), split merge, sigmoid output gate */
int r4dxb_q4x_qsa_attn(const void* q, const void* qg, const void* cache, const int* block_table, const int* positions,
                       const int* sel_tokens, const int* sel_count, const float* k_descale, const float* v_descale, float* part_acc,
                       float* part_ml, void* out, int T, int Hq, int Hkv, int D, int sel_stride, int max_tokens, int nsplit, int gated,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* R4DXB_H_ */
