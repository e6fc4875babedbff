// kernels.h — every launcher of the CUDA kernel library (csrc/*.cu), as plain C declarations.
//
// The kernels are compiled for sm_100a.  Each launcher enqueues work on `stream` and returns at once:
// 0 on success, VM_ERR_UNSUPPORTED (-1) for a size or dtype the kernel does not take, VM_ERR_BAD_ARG (-2)
// for an argument that contradicts another, or a positive cudaError_t.  Pointers are device pointers
// unless a comment says otherwise.  `err` is an optional device int that kernels set to an error word
// (see VM_ERRWORD_*) instead of faulting; 0 means nothing happened.
//
// Activations are float32 or bfloat16 (`act_dtype`: VM_F32 / VM_BF16); the residual stream and all logits
// are float32.  The cache is paged: k/v pages are [n_pages, Hkv, VM_PAGE_TOKENS, D]; a block table
// int32 [B, max_blocks] names the page of every VM_PAGE_TOKENS-token block of each sequence (-1: none).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { VM_F32 = 0, VM_BF16 = 1 };
enum { VM_ERR_UNSUPPORTED = -1, VM_ERR_BAD_ARG = -2 };
// tokens per cache page: the one constant that the host's page bookkeeping and the kernels share
#define VM_PAGE_TOKENS 64
// which two values of a head a rotary position encoding turns together: (j, j + rot_dim/2) or (2j, 2j + 1)
enum { VM_PAIR_HALF_SPLIT = 0, VM_PAIR_INTERLEAVED = 1 };
// activations of the feed-forward kernels: x sigmoid(x); the tanh form of GELU; max(x, 0)^2
enum { VM_ACT_SILU = 0, VM_ACT_GELU_TANH = 1, VM_ACT_RELU_SQUARED = 2 };
// not elementwise, so no kernel that takes VM_ACT_* knows it: a polynomial of a token's row and its powers, each divided by its root
// mean square (vm_polynorm)
enum { VM_ACT_POLYNORM = 16 };
// gated experts: the clamped unit min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u) + 1); or silu(w g) (w u) with the routing weight w
// on the expert's input (it is then not applied to the output again, and the shared expert is gated in the same way, with w = 1); or the
// plain SiLU-gated unit silu(g) u whose OUTPUT takes the routing weight (the shared expert gated too, with weight 1)
enum { VM_GLU_NONE = 0, VM_GLU_CLAMPED = 1, VM_GLU_SILU_WEIGHTED_INPUT = 2, VM_GLU_SILU = 3 };
// how a router that scores all its outputs scores them: softmax over all of them, or the sigmoid of each alone
enum { VM_SCORE_SOFTMAX = 0, VM_SCORE_SIGMOID = 1 };
// error words a kernel may leave in `err`
enum { VM_ERRWORD_TOKEN_ID = 1, VM_ERRWORD_CACHE_WRITE = 2, VM_ERRWORD_CACHE_READ = 3, VM_ERRWORD_BARRIER_WAIT = 4 };

// ---- elementwise.cu
void vm_set_pdl(int on);                      // programmatic dependent launch for the decode chain (default on)
int vm_embed_gather(const void* table, int table_dtype, const int* tokens, float* out, int T, int hid, int vocab, int* err,
                    cudaStream_t stream);
int vm_embed_gather_scaled(const void* table, int table_dtype, const int* tokens, float* out, int T, int hid, int vocab, float scale, int* err,
                           cudaStream_t stream);      // the rows times `scale`
int vm_add_rmsnorm(float* h, const void* delta, const float* w, void* out, const int* rows, int n_out, int hid, float eps,
                   int act_dtype, cudaStream_t stream);
int vm_residual_add(float* h, const void* delta, long long n, int act_dtype, cudaStream_t stream);
int vm_swiglu(const void* gate_up, void* out, int T, int I, int act_dtype, cudaStream_t stream);
int vm_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream);
// out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i] for the activation `kind` (VM_ACT_*)
int vm_gated_activation(const void* gate_up, void* out, int T, int I, int kind, int act_dtype, cudaStream_t stream);

// ---- latent_cache.cu: the norms of a latent-attention layer's two down projections and the cache write of the key/value latent
// down float32 [T, ld]: columns [0, q_rank) and, if `pages` is given, [q_rank, q_rank + kv_rank); cq [T, q_rank] and the
// pages [n_pages, VM_PAGE_TOKENS, kv_rank] in the activation dtype
int vm_latent_norm_write(const float* down, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps, void* cq,
                         const int* positions, const int* seq_of_token, const int* block_table, int max_blocks, void* pages,
                         int n_pages, int T, int act_dtype, int* err, cudaStream_t stream);

// the same for a layer with rotary positions: rot_dim more columns behind the key/value latent (not normed, one key part shared by all heads)
// whose first rotary_dim values are turned by the token's position; pages [n_pages, VM_PAGE_TOKENS, kv_rank + rot_dim]
int vm_latent_rope_norm_write(const float* down, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps, void* cq,
                              const int* positions, const int* seq_of_token, const int* block_table, int max_blocks, void* pages, int n_pages,
                              int rot_dim, int rotary_dim, const float* inv_freq, int pairing, int T, int act_dtype, int* err, cudaStream_t stream);

// ---- sublayer.cu: a layer whose sublayers read the residual stream through a short causal convolution and are normed on their output
// out [T, hid] (activation dtype) = h + conv(h) over time per channel, taps float32 [hid, K]; the K - 1 last inputs of every sequence are
// kept in state [slot, state_stride] at state_offset (float32) and moved on by the step's tokens
int vm_input_conv(const float* h, const float* taps, float* state, long long state_stride, int state_offset, const int* positions,
                  const int* seq_of_token, const int* cu_tokens, const int* slots, void* out, int T, int B, int hid, int K, int one_token_each,
                  int act_dtype, cudaStream_t stream);
int vm_norm_residual_add(float* h, const void* y, long long ld, int y_dtype, const float* w, int T, int hid, float eps, cudaStream_t stream);
// one token per sequence: the same sum, then out = h + conv(h) of the next sublayer on the row just made, its kept inputs moved on
int vm_norm_residual_conv_step(float* h, const void* y, long long ld, int y_dtype, const float* w, int B, int hid, float eps, const float* taps,
                               float* state, long long state_stride, int state_offset, const int* slots, void* out, int K, int act_dtype,
                               cudaStream_t stream);
// a N(z) + b N(z^2) + c N(z^3) + e per token, N: division by the root mean square over the token's n values; coef float32 [4]
int vm_polynorm(const void* z, int z_dtype, const float* coef, void* out, int T, int n, float eps, int act_dtype, cudaStream_t stream);
int vm_rotate_slice(const void* src, long long src_ld, int src_head, int src_off, void* dst, long long dst_ld, int dst_head, int dst_off,
                    const int* positions, const float* inv_freq, int rotary_dim, int pairing, int width, int H, int T, int act_dtype,
                    cudaStream_t stream);
int vm_sigmoid_gate(void* x, const float* gate, long long gate_ld, int T, int cols, int act_dtype, cudaStream_t stream);

// ---- head_products.cu: per-head products of a step of few tokens (bfloat16): out[t, h, :N] = W_h x[t, h, :K], W_h = w + h * w_head stored
// [K, N] (k_by_n) or [N, K]; with [N, K] an optional gate (out *= sigmoid(gate[t, h * N + n]), float32 rows), with [K, N] an optional tail
// (out[t, h, N : N + tail] = x[t, h, K : K + tail], its first rotary_dim values turned by the token's position)
int vm_head_products_few(const void* x, long long x_ld, int x_head, const void* w, long long w_head, int k_by_n, void* out, long long out_ld,
                         int out_head, int T, int N, int K, int H, const float* gate, long long gate_ld, int tail, const int* positions,
                         const float* inv_freq, int rotary_dim, int pairing, cudaStream_t stream);

// ---- mlstm.cu: the matrix-memory recurrence with its output stage
// proj float32 [T, ld]: q | k | v | g | x_i | x_f (H*D, H*D, H*V, H*V, H, H columns); state float32, per slot and head S [D, V], n [D], m;
// out [T, H*V] in the activation dtype
int vm_mlstm_scan(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state,
                  const int* cu_tokens, const int* slots, void* out, int B, int H, int D, int V, float cap, float eps, int act_dtype,
                  cudaStream_t stream);

int vm_mlstm_scan_fits(int D, int V);      // 1 if vm_mlstm_scan takes heads of these sizes
// the same recurrence chunk by chunk (prompts): scratch of vm_mlstm_chunk_scratch_floats(T, B, H, D, V) floats
long long vm_mlstm_chunk_scratch_floats(int T, int B, int H, int D, int V);
int vm_mlstm_chunks(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state,
                    const int* cu_tokens, const int* slots, void* out, float* scratch, int T, int B, int H, int D, int V, float cap,
                    float eps, int act_dtype, cudaStream_t stream);
// one token per sequence (token s belongs to sequence s): scratch of B * H * (V + D + 1) floats
int vm_mlstm_step(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, float* state,
                  const int* cu_tokens, const int* slots, void* out, float* scratch, int B, int H, int D, int V, float cap, float eps,
                  int act_dtype, cudaStream_t stream);

// ---- routed_experts.cu: a routed feed-forward for few tokens
// x [T, hidden] in the activation dtype, or (norm_w given) the float32 residual stream, whose rows the kernels then norm themselves;
// residual given: the experts' result is added into it instead of being written to `out`
int vm_expert_router(const void* x, const float* norm_w, float eps, const float* w_router, const float* b_router, const float* w_gate, int T,
                     int hidden, int E, int top, int* chosen, float* weight, float* shared_gate, int act_dtype, cudaStream_t stream);
int vm_experts_few_tokens(const void* x, const float* norm_w, float eps, const void* w_up, const void* w_down, const void* w_up_shared,
                          const void* w_down_shared, int weight_dtype, const int* chosen, const float* weight, const float* shared_gate, int T,
                          int hidden, int ff, int ff_shared, int top, int act_kind, int act_kind_shared, void* act, void* out,
                          float* residual, int act_dtype, cudaStream_t stream);

// the same with gated experts and identity experts: E real experts; a chosen index >= E names one of the n_identity identity experts,
// whose result is the token's input row; glu: an expert's up matrix is [2 * ff, hidden] (gate rows first) and its activation
// min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1); act [T, vm_experts_act_cols(...)]
long long vm_experts_act_cols(int hidden, int ff, int ff_shared, int top, int n_identity);
int vm_experts_few_tokens_glu(const void* x, const float* norm_w, float eps, const void* w_up, const void* w_down, const void* w_up_shared,
                              const void* w_down_shared, int weight_dtype, const int* chosen, const float* weight, const float* shared_gate, int T,
                              int hidden, int ff, int ff_shared, int top, int act_kind, int act_kind_shared, int E, int n_identity, int glu,
                              float limit, float alpha, void* act, void* out, float* residual, int act_dtype, cudaStream_t stream);
// a router that scores all its n_out outputs: s = softmax(z); the choice goes by s + correction (null: none) among the outputs of the
// group_keep best of group_count equal groups of neighbours (a group's score: its largest choice score); weight = s * scale
int vm_expert_router_scored(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                            int n_out, int top, int group_count, int group_keep, float scale, int* chosen, float* weight, int act_dtype,
                            cudaStream_t stream);

int vm_expert_router_scores(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                            int n_out, int top, int group_count, int group_keep, float scale, int score_kind, int* chosen, float* weight, int act_dtype,
                            cudaStream_t stream);      // vm_expert_router_scored with the kind of score (VM_SCORE_*) as an argument
// the same with the number of a group's largest scores that make up the group's score (1: its largest; 2: the sum of its two largest)
int vm_expert_router_groups(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                            int n_out, int top, int group_count, int group_keep, int group_top, float scale, int score_kind, int* chosen,
                            float* weight, int act_dtype, cudaStream_t stream);

// ---- attention_biased.cu: windowed attention with kept first tokens and a learned bias by bucketed distance; keys of Dk, values of Dv
// qkv [T, ld]: H query heads and Hkv key heads of Dk, Hkv value heads of Dv; queries and keys get a unit-rms norm per head (weights wq, wk
// float32 [Dk]), queries in place, keys and values into the pages (kpages null: none written); v_first [T, Hkv * Dv] is blended into the
// values with the device float `lambda` ((1 - lambda) v + lambda v_first); v_keep [T, Hkv * Dv] receives the values as projected
int vm_qkv_prepare(void* qkv, int ld, const float* wq, const float* wk, float eps, const float* lambda, const void* v_first, void* v_keep,
                   const int* positions, const int* seq_of_token, const int* block_table, int max_blocks, void* kpages, void* vpages, int T, int H,
                   int Hkv, int Dk, int Dv, int n_pages, int act_dtype, int* err, cudaStream_t stream);
// rel float32 [rows, H], bucket_of int32 [far + 1] (distances beyond `far` read the last entry); both null: no bias.
// A query at position p sees keys j <= p with p - j < window (0: all) or j < keep_first.
int vm_attention_biased_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                                const int* positions, const int* seq_of_token, const float* rel, const int* bucket_of, int far, void* out,
                                int n_tokens, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages, int act_dtype,
                                int* err, cudaStream_t stream);

// The same attention with a sink and with values that may lie inside the key rows.  sink float32 [H] (null: none): exp(sink[h]) is one
// more term of head h's softmax denominator, without a key or a value, not scaled.  v_row_stride: elements between the value rows of
// neighbouring tokens in `vpages` (0: Dv); with vpages == kpages and v_row_stride == Dk a token's value is the first Dv values of its key row.
int vm_attention_sink_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                              const int* positions, const int* seq_of_token, const float* rel, const int* bucket_of, int far, const float* sink,
                              int v_row_stride, void* out, int n_tokens, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first,
                              int n_pages, int act_dtype, int* err, cudaStream_t stream);
int vm_attention_sink_prefill_fits(int Dk, int Dv, int values_in_keys);
int vm_attention_sink_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                                   const int* positions, const int* cu_tokens, int B, int n_tiles, const float* rel, const int* bucket_of, int far,
                                   int rel_rows, const float* sink, int v_row_stride, void* out, int H, int Hkv, int Dk, int Dv, float scale, int window,
                                   int keep_first, int n_pages, int* err, cudaStream_t stream);
int vm_attention_sink_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                                  const int* positions, const float* rel, const int* bucket_of, int far, const float* sink, int v_row_stride, void* out,
                                  int B, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages, int* err,
                                  cudaStream_t stream);

// ---- attention_biased_fast.cu: the same attention in bfloat16: prompts on mma.sync tiles (keys and values of the sizes that
// vm_attention_biased_prefill_fits names; n_tiles = sum over the sequences of ceil(new tokens / 64)), decode steps (token s is sequence s's)
int vm_attention_biased_prefill_fits(int Dk, int Dv);
int vm_attention_biased_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                     int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, const float* rel,
                                     const int* bucket_of, int far, int rel_rows, void* out, int H, int Hkv, int Dk, int Dv, float scale,
                                     int window, int keep_first, int n_pages, int* err, cudaStream_t stream);
int vm_attention_biased_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                    int max_blocks, const int* positions, const float* rel, const int* bucket_of, int far, void* out, int B, int H,
                                    int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages, int* err, cudaStream_t stream);

// ---- ssm.cu: a selective state-space mixer (short causal convolution, matrix-state recurrence, gated group norm)
long long vm_ssm_state_floats(int H, int P, int N, int G, int K);
long long vm_ssm_chunk_scratch_floats(int T, int n_chunks, int H, int P, int N);
// chunk_scratch given with n_chunks = sum over the sequences of ceil(new tokens / 64): prompts run chunk by chunk; one_token_each: decode steps
int vm_ssm_mixer(const void* proj, int ld, const float* taps, const float* conv_bias, const float* dt_bias, const float* A_log, const float* Dskip,
                 const float* norm_w, float eps, float* state, int state_floats, const int* positions, const int* seq_of_token, const int* cu_tokens,
                 const int* slots, void* xbc, float* y, void* out, float* chunk_scratch, int n_chunks, int one_token_each, int T, int B, int H, int P,
                 int N, int G, int K, int parts, int act_dtype, cudaStream_t stream);

// ---- rope_cache.cu
int vm_rope_kv_write(void* qkv, const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
                     const float* inv_freq, int rot_dim, int pairing, void* kpages, void* vpages, int T, int H, int Hkv, int D,
                     int n_pages, int act_dtype, int* err, cudaStream_t stream);

// ---- attention
int vm_attention_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                         int max_blocks, const int* positions, const int* seq_of_token, void* out, int n_tokens, int H, int Hkv,
                         int D, float scale, int window, int n_pages, int act_dtype, int* err, cudaStream_t stream);
int vm_attention_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                              int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H,
                              int Hkv, int D, float scale, int window, int n_pages, int* err, int groups, cudaStream_t stream);
int vm_attention_prefill_tc_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                 int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, void* out, int H,
                                 int Hkv, int D, float scale, int window, int n_pages, int* err, int groups, cudaStream_t stream);
// the warp-specialised tcgen05 kernel: host_cu_tokens [B + 1] (host memory) repeats cu_tokens, the launch is shaped from it
int vm_attention_prefill_ws_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                 int max_blocks, const int* positions, const int* cu_tokens, const int* host_cu_tokens, int B,
                                 void* out, int H, int Hkv, int D, float scale, int window, int n_pages, int* err, int groups,
                                 cudaStream_t stream);
long long vm_attention_decode_scratch_floats(int B, int H, int D, int n_splits);
int vm_attention_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                             int max_blocks, const int* positions, void* out, float* partial, int* counters, int B, int H,
                             int Hkv, int D, int n_splits, float scale, int window, int n_pages, int* err, cudaStream_t stream);

// ---- routed_experts_grouped.cu: the same feed-forward for many tokens (bfloat16), pairs grouped by expert on the device
long long vm_experts_grouped_rows(int T, int top, int E);
int vm_experts_grouped(const void* x, const void* w_up, const void* w_down, const int* chosen, const float* weight, const float* shared_y,
                       const float* shared_gate, int T, int hidden, int ff, int top, int E, int act_kind, int row_cap, int* row_of_pair,
                       int* token_of_row, int* expert_of_tile, void* act, float* y, void* out, cudaStream_t stream);
int vm_activation(const void* in, void* out, long long n, int kind, int act_dtype, cudaStream_t stream);
// the general form: gated and identity experts as in vm_experts_few_tokens_glu; x_sorted given: tcgen05 tiles of 128 rows, else mma.sync
// tiles of 64; gate_up bf16 [row_cap, 2 * ff] is scratch of the gated form
int vm_experts_grouped_glu(const void* x, const void* w_up, const void* w_down, const int* chosen, const float* weight, const float* shared_y,
                           const float* shared_gate, int T, int hidden, int ff, int top, int E, int n_identity, int act_kind, int glu, float limit,
                           float alpha, int row_cap, int* row_of_pair, int* token_of_row, int* expert_of_tile, void* x_sorted, void* act,
                           void* gate_up, float* y, void* out, int* err, cudaStream_t stream);
// the same with the experts' products on tcgen05: runs padded to tiles of 128 rows, x_sorted bf16 [row_cap, hidden] as one more scratch
long long vm_experts_grouped_rows_tiled(int T, int top, int E, int tile);
int vm_experts_grouped_tc(const void* x, const void* w_up, const void* w_down, const int* chosen, const float* weight, const float* shared_y,
                          const float* shared_gate, int T, int hidden, int ff, int top, int E, int act_kind, int row_cap, int* row_of_pair,
                          int* token_of_row, int* expert_of_tile, void* x_sorted, void* act, float* y, void* out, int* err,
                          cudaStream_t stream);

// ---- skinny_gemm.cu: weight-streaming products for few rows (bfloat16 weights [N, K])
// (err: the step's error word, may be null; the kernel for large weight matrices reports a wait that ran out there)
int vm_skinny_linear(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int N, int K, void* out,
                     int out_stride, int out_f32, float* residual_h, int* err, cudaStream_t stream);
// out[M, N] = act(A W^T) in bfloat16: the activation (VM_ACT_*) of the product as bfloat16 holds it (the first half of a two-matrix unit)
int vm_skinny_linear_act(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int N, int K, int act, void* out,
                         int out_stride, int* err, cudaStream_t stream);
int vm_skinny_swiglu(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int I, int K, void* out,
                     int* err, cudaStream_t stream);
int vm_skinny_gated(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int I, int K, int act, void* out,
                    int* err, cudaStream_t stream);      // vm_skinny_swiglu with the gate's activation (VM_ACT_*) as an argument
void vm_skinny_variant(int variant);       // 0 choose by size, 1 / 2 force one of the two kernels (tests, measurements)
int vm_skinny_qkv_rope(const void* A, int pro, const float* norm_w, float eps, const void* W, int M, int K, void* q_out,
                       const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
                       const float* inv_freq, int rot_dim, int pairing, void* kpages, void* vpages, int H, int Hkv, int D,
                       int n_pages, int* err, cudaStream_t stream);

// ---- tc_gemm.cu: tcgen05 + TMA products for many rows, with fused epilogues
int vm_tc_linear(const void* A, long long lda, const void* W, int M, int N, int K, void* out, int out_stride, int out_f32,
                 float* residual_h, int* err, cudaStream_t stream);
int vm_tc_swiglu(const void* A, long long lda, const void* W, int M, int I, int K, void* out, int* err, cudaStream_t stream);
// grouped: row tile t of A (128 rows) multiplies with rows [g * N, g * N + N) of the stacked W [groups * N, K], g = tile_group[t] (-1: unused)
int vm_tc_grouped_linear(const void* A, long long lda, const void* W, int M, int N, int K, int groups, const int* tile_group,
                         void* out, int out_stride, int out_f32, int act_kind, int* err, cudaStream_t stream);
int vm_tc_qkv_rope(const void* A, long long lda, const void* W, int M, int K, void* q_out, const int* positions,
                   const int* seq_of_token, const int* block_table, int max_blocks, const float* inv_freq, int rot_dim,
                   int pairing, void* kpages, void* vpages, int H, int Hkv, int D, int n_pages, int* err, cudaStream_t stream);

// ---- hyper.cu: several copies of the residual stream; an embedding with a table read by pairs of tokens
// Copy s of the stream is [T, hid] float32 at h + s * stride.  y (activation dtype, or null): every copy becomes
// sum_s mix[s, to] x_s + w_out[to] * y (mix float32 [S, S] indexed [from, to]).  out (activation dtype, or null) then gets
// rmsnorm(sum_s w_in[s] x_s) * norm_w.  At most 16 copies.
int vm_streams_step(float* h, long long stride, int S, const void* y, const float* mix, const float* w_out, const float* w_in, const float* norm_w,
                    float eps, void* out, int T, int hid, int act_dtype, cudaStream_t stream);
int vm_streams_sum_rows(float* h, long long stride, int S, const int* rows, int n_rows, int hid, cudaStream_t stream);   // copy 0 <- the sum, at `rows`
// out[t] = table[token] + pairs[(previous * mul_prev + token * mul_cur) mod buckets], row `buckets` for a sequence's first token;
// `last`: an int32 word per slot (last_stride words apart) that keeps the token before the next step's first one
int vm_embed_pairs(const void* table, const void* pairs, int table_dtype, const int* tokens, const int* positions, const int* seq_of_token,
                   const int* cu_tokens, const int* slots, int* last, long long last_stride, float* out, int T, int B, int hid, int vocab,
                   long long buckets, long long mul_prev, long long mul_cur, int one_token_each, int* err, cudaStream_t stream);

// ---- mixer_prep.cu: from an attention mixer's projections to its attention kernel (bias, short convolution over time with kept rows,
// norm over the whole projection, rotary positions, cache write), and gates, biases and joins behind it
// proj float32 [T, ld]: columns [0, H Dk) queries, then G Dk keys, then (unless the values are the keys) G Dv values; bias float32 [C]
// or null; taps float32 [C, K] or null (the K - 1 rows kept per sequence lie in state [slot, state_stride] at state_offset);
// q_norm [H Dk], k_norm [G Dk] or both null; inv_freq [rotary_dim / 2] or null.  q_out [T, H Dk] and the pages in the activation dtype.
int vm_mixer_prepare(const float* proj, int ld, const float* bias, const float* taps, int K, float* state, long long state_stride, int state_offset,
                     const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rotary_dim, int pairing, const int* positions,
                     const int* seq_of_token, const int* cu_tokens, const int* slots, const int* block_table, int max_blocks, void* q_out, void* kpages,
                     void* vpages, int n_pages, int T, int B, int H, int G, int Dk, int Dv, int values_are_keys, int one_token_each, int act_dtype,
                     int* err, cudaStream_t stream);
// x[t, c] *= sigmoid(g[t, c / per]), g float32 rows of stride ldg: one gate for every `per` neighbouring values (a head)
int vm_sigmoid_gate_heads(void* x, const float* g, int ldg, int T, int cols, int per, int act_dtype, cudaStream_t stream);
// out = ca f(a + bias_a) + cb f(b); f the identity or (wa, wb given) the RMS norm over the row with that weight; b null: the first term alone
int vm_join_rows(const void* a, const void* b, const float* bias_a, float ca, float cb, const float* wa, const float* wb, float eps, void* out, int T,
                 int cols, int act_dtype, cudaStream_t stream);

// ---- decayed_memory.cu: linear attention with a decaying matrix memory S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t
// proj float32 [T, ld] with queries at q_off ([H, Dk]), keys at k_off, values at v_off ([H, Dv]); z float32 [T, ldz] decay logits
// (a = sigmoid(z + z_bias)^(1 / tau), z_bias float32 [H, Dk] or null) or null with head_log_decay float32 [H]; inv_freq or null; the [H, Dk, Dv] memory of a sequence lies in
// state [slot, state_stride] at state_offset; o float32 [T, H Dv]
int vm_decayed_memory(const float* proj, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, float tau, const float* z_bias,
                      const float* head_log_decay, const float* inv_freq, int rotary_dim, int pairing, float q_scale, float k_scale, float* state, long long state_stride,
                      int state_offset, const int* positions, const int* cu_tokens, const int* slots, float* o, int T, int B, int H, int Dk, int Dv,
                      cudaStream_t stream);
// the same for prompts, chunk by chunk in three launches behind one that turns the queries and keys of `proj` in place (keys and values in multiples of 4 that fit the shared memory: the chunk's
// tokens, 64 / 32 / 16, or 0 where the sizes are not taken); n_chunks: sum over the step's sequences of ceil(tokens / chunk tokens)
int vm_decayed_memory_chunk_tokens(int Dk, int Dv);
long long vm_decayed_memory_scratch_floats(int T, int B, int H, int Dk, int Dv);
int vm_decayed_memory_chunked(float* proj, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, float tau, const float* z_bias,
                              const float* head_log_decay, const float* inv_freq, int rotary_dim, int pairing, float q_scale, float k_scale,
                              float* state, long long state_stride, int state_offset, const int* positions, const int* cu_tokens, const int* slots,
                              float* o, float* scratch, int n_chunks, int T, int B, int H, int Dk, int Dv, cudaStream_t stream);
// out[t, h] = o[t, h] / rms(o[t, h]) * w * silu(g[t, h]); w float32 [Dv] or null; g float32 rows of stride ldg
int vm_memory_output(const float* o, const float* g, int ldg, const float* w, float eps, void* out, int T, int H, int Dv, int act_dtype,
                     cudaStream_t stream);

// ---- sampling.cu
int vm_sample(const float* logits, long long row_stride, int R, int V, const float* temperature, const float* top_p,
              const long long* seed, const long long* stream_id, const long long* step, long long step_add, int* out,
              cudaStream_t stream);
int vm_decode_advance(const int* sampled, int* tokens, int* positions, int* ctx_len, long long* draw_step, int* history,
                      int* iteration, int B, cudaStream_t stream);

// ---- host_transfer.cu (no kernels)
void* vm_host_device_pointer(void* host);     // the address under which kernels reach pinned host memory, or null
void* vm_event_create(void);
int vm_event_destroy(void* event);
int vm_event_synchronize(void* event);
int vm_upload_record(void* dst, const void* src, long long nbytes, void* event, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
