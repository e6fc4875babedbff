// ops.h (internal) — the device operations the parts are made of: checked wrappers over the CUDA launchers and the
// library matrix product.  There is no other implementation: a missing device or a refused launch throws.
//
// Debugging switches, read once from the environment (the reference has VELOMIND_CUDA_SYNC and VELOMIND_FAIL_BACKEND for
// the same purposes: src/cuda/cuda_context.cu:115-118, src/cuda/ops/backend_error.h:31-51); both act on the host only:
//   VELOMIND_B200_SYNC=1        wait for the device after every launch, so that a CUDA error names the operation
//   VELOMIND_B200_FAIL_OP=name  the operation of that name throws after its launch (fault injection)
#pragma once

#include <cublas_v2.h>

#include <string>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

namespace vmb {
namespace ops {

struct Counters {
    long long own_launches = 0;     // this library's own kernels
    long long library_calls = 0;    // library matrix products (cuBLAS)
    long long h2d_bytes = 0;        // bytes of step inputs copied from pinned host memory
    long long d2h_bytes = 0;        // bytes of step results that reached the host
    long long tc_attention_calls = 0;
};
Counters& counters();

// per-operation device time (two events around every launch), switched on by OpTimes
struct OpTimes {
    OpTimes();
    ~OpTimes();
    std::string table();            // name, launches, milliseconds; the events are read here (synchronises)
};
bool op_times_active();
void op_time_begin(const char* name, cudaStream_t stream);
void op_time_end(const char* name, cudaStream_t stream);

bool sync_every_op();
void check(int status, const char* name, cudaStream_t stream);      // counts the launch; throws KernelError on a refusal
void cuda_check(cudaError_t e, const char* what);

inline int code(DType t) {
    if (t == DType::F32) return VM_F32;
    if (t == DType::BF16) return VM_BF16;
    throw KernelError(std::string("dtype ") + dtype_name(t) + " has no kernel (float32 and bfloat16 do)");
}

struct Timed {                      // brackets one launch with events when op times are on
    const char* name;
    cudaStream_t stream;
    Timed(const char* n, cudaStream_t s) : name(n), stream(s) { if (op_times_active()) op_time_begin(n, s); }
    ~Timed() { if (op_times_active()) op_time_end(name, stream); }
};

inline void embed_gather(const DeviceTensor& table, const int* tokens, float* out, int T, int hid, float scale, int* err, cudaStream_t s) {
    Timed t("embed_gather", s);
    check(vm_embed_gather_scaled(table.ptr, code(table.dtype), tokens, out, T, hid, static_cast<int>(table.rows()), scale, err, s), "embed_gather", s);
}

// what a sublayer reads: h + conv(h), a short causal convolution over time on every channel; the kept inputs live in the running
// schedule position's state area at `state_offset`
inline void input_conv(const float* h, const float* taps, int K, int state_offset, StepContext& ctx, void* out) {
    Timed t("input_conv", ctx.stream);
    if (K > 1 && (!ctx.state() || ctx.state_floats() < state_offset + (K - 1) * ctx.hidden))
        throw CacheError("input convolution: the cache holds no state area for this layer's kept inputs");
    check(vm_input_conv(h, taps, ctx.state(), ctx.state_floats(), state_offset, ctx.positions, ctx.seq_of_token, ctx.cu_tokens, ctx.slots, out, ctx.T, ctx.B,
                        ctx.hidden, K, ctx.one_token_each ? 1 : 0, code(ctx.act_dtype), ctx.stream),
          "input_conv", ctx.stream);
    if (!ctx.one_token_each && K > 1) ++counters().own_launches;      // two kernels
}

// h += rmsnorm(y) * w: the residual sum of a sublayer whose norm sits on its output
inline void norm_residual_add(float* h, const void* y, long long ld, DType y_dtype, const float* w, float eps, int T, int hid, cudaStream_t s) {
    Timed t("norm_residual_add", s);
    check(vm_norm_residual_add(h, y, ld, code(y_dtype), w, T, hid, eps, s), "norm_residual_add", s);
}

// a step of one token per sequence: that sum and the next sublayer's input convolution in one launch
inline void norm_residual_conv_step(float* h, const void* y, DType y_dtype, const float* w, float eps, const float* taps, int K, int state_offset,
                                    StepContext& ctx, void* out) {
    Timed t("norm_residual_conv_step", ctx.stream);
    if (K > 1 && (!ctx.state() || ctx.state_floats() < state_offset + (K - 1) * ctx.hidden))
        throw CacheError("input convolution: the cache holds no state area for this layer's kept inputs");
    check(vm_norm_residual_conv_step(h, y, ctx.hidden, code(y_dtype), w, ctx.B, ctx.hidden, eps, taps, ctx.state(), ctx.state_floats(), state_offset, ctx.slots,
                                     out, K, code(ctx.act_dtype), ctx.stream),
          "norm_residual_conv_step", ctx.stream);
}

inline void polynorm(const void* z, DType z_dtype, const float* coef, void* out, int T, int n, float eps, DType act, cudaStream_t s) {
    Timed t("polynorm", s);
    check(vm_polynorm(z, code(z_dtype), coef, out, T, n, eps, code(act), s), "polynorm", s);
}

inline void rotate_slice(const void* src, long long src_ld, int src_head, int src_off, void* dst, long long dst_ld, int dst_head, int dst_off,
                         const RotaryTable& rot, int width, int H, const StepContext& ctx) {
    Timed t("rotate_slice", ctx.stream);
    check(vm_rotate_slice(src, src_ld, src_head, src_off, dst, dst_ld, dst_head, dst_off, ctx.positions, rot.inv_freq, rot.inv_freq ? rot.rotary_dim : 0,
                          rot.pairing, width, H, ctx.T, code(ctx.act_dtype), ctx.stream),
          "rotate_slice", ctx.stream);
}

// the heads' products of a step of few tokens in bfloat16, with the gate or the rotated tail that follows them (csrc/head_products.cu)
inline void head_products_few(const void* x, long long x_ld, int x_head, const void* w, long long w_head, bool k_by_n, void* out, long long out_ld,
                              int out_head, int N, int K, int H, const float* gate, long long gate_ld, int tail, const RotaryTable* rot,
                              const StepContext& ctx) {
    Timed t("head_products_few", ctx.stream);
    const bool turns = tail > 0 && rot && rot->inv_freq;
    check(vm_head_products_few(x, x_ld, x_head, w, w_head, k_by_n ? 1 : 0, out, out_ld, out_head, ctx.T, N, K, H, gate, gate_ld, tail, ctx.positions,
                               turns ? rot->inv_freq : nullptr, turns ? rot->rotary_dim : 0, turns ? rot->pairing : 0, ctx.stream),
          "head_products_few", ctx.stream);
}

inline void sigmoid_gate(void* x, const float* gate, long long gate_ld, int T, int cols, DType act, cudaStream_t s) {
    Timed t("sigmoid_gate", s);
    check(vm_sigmoid_gate(x, gate, gate_ld, T, cols, code(act), s), "sigmoid_gate", s);
}

inline void add_rmsnorm(float* h, const void* delta, const float* weight, float eps, void* out, const int* rows, int n_out, int hid, DType act,
                        cudaStream_t s) {
    Timed t("add_rmsnorm", s);
    check(vm_add_rmsnorm(h, delta, weight, out, rows, n_out, hid, eps, code(act), s), "add_rmsnorm", s);
}

inline void residual_add(float* h, const void* delta, long long n, DType act, cudaStream_t s) {
    Timed t("residual_add", s);
    check(vm_residual_add(h, delta, n, code(act), s), "residual_add", s);
}

inline void swiglu(const void* gate_up, void* out, int T, int I, DType act, cudaStream_t s) {
    Timed t("swiglu", s);
    check(vm_swiglu(gate_up, out, T, I, code(act), s), "swiglu", s);
}

inline void gated_activation(const void* gate_up, void* out, int T, int I, int kind, DType act, cudaStream_t s) {
    Timed t("gated_activation", s);
    check(vm_gated_activation(gate_up, out, T, I, kind, code(act), s), "gated_activation", s);
}

inline void convert(const void* in, DType in_dtype, void* out, DType out_dtype, long long n, cudaStream_t s) {
    Timed t("convert", s);
    check(vm_convert(in, code(in_dtype), out, code(out_dtype), n, s), "convert", s);
}

inline void rope_kv_write(void* qkv, const StepContext& ctx, const KVView& kv, const RotaryTable& rot, int H, int Hkv, int D, DType act) {
    Timed t("rope_kv_write", ctx.stream);
    check(vm_rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width, rot.inv_freq, rot.rotary_dim, rot.pairing,
                           kv.owns ? kv.k_pages : nullptr, kv.owns ? kv.v_pages : nullptr, ctx.T, H, Hkv, D, kv.owns ? kv.n_pages : 0, code(act),
                           ctx.err, ctx.stream),
          "rope_kv_write", ctx.stream);
}

inline void latent_norm_write(const float* down, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps, void* cq,
                              const StepContext& ctx, const KVView& kv, bool write) {
    Timed t("latent_norm_write", ctx.stream);
    check(vm_latent_norm_write(down, ld, q_rank, kv_rank, wq, wkv, eps, cq, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width,
                               write ? kv.k_pages : nullptr, write ? kv.n_pages : 0, ctx.T, code(ctx.act_dtype), ctx.err, ctx.stream),
          "latent_norm_write", ctx.stream);
}

// the same with `rot_dim` more values per token behind the latent: the key part all heads share, turned by the token's position
inline void latent_rope_norm_write(const float* down, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps, void* cq,
                                   const StepContext& ctx, const KVView& kv, bool write, int rot_dim, const RotaryTable& rot) {
    Timed t("latent_norm_write", ctx.stream);
    check(vm_latent_rope_norm_write(down, ld, q_rank, kv_rank, wq, wkv, eps, cq, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width,
                                    write ? kv.k_pages : nullptr, write ? kv.n_pages : 0, rot_dim, rot.inv_freq ? rot.rotary_dim : 0, rot.inv_freq,
                                    rot.pairing, ctx.T, code(ctx.act_dtype), ctx.err, ctx.stream),
          "latent_norm_write", ctx.stream);
}

constexpr int MLSTM_SCAN_MAX_TOKENS = 8;
inline void mlstm_scan(const float* proj, int ld, const float* bias_i, const float* bias_f, const float* norm_w, const StepContext& ctx, void* out, int H,
                       int D, int V, float cap, float eps) {
    Timed t("mlstm_scan", ctx.stream);
    if (!ctx.state() || ctx.state_floats() != H * (D * V + D + 1)) throw CacheError("mlstm: the cache holds no state area of this layer's size");
    // Decode steps stream the state once; the smallest pieces go token by token; everything else chunk by chunk.  The choice
    // follows the step's capacity bucket alone, so that every step of a bucket asks for the same scratch.
    StepContext& c = const_cast<StepContext&>(ctx);
    if (ctx.one_token_each) {
        float* scratch = static_cast<float*>(c.take(static_cast<long long>(ctx.B_cap) * H * (V + D + 1), DType::F32));
        check(vm_mlstm_step(proj, ld, bias_i, bias_f, norm_w, ctx.state(), ctx.cu_tokens, ctx.slots, out, scratch, ctx.B, H, D, V, cap, eps,
                            code(ctx.act_dtype), ctx.stream),
              "mlstm_step", ctx.stream);
        ++counters().own_launches;      // two kernels
        c.give(scratch);
        return;
    }
    if (ctx.T_cap <= MLSTM_SCAN_MAX_TOKENS && vm_mlstm_scan_fits(D, V)) {
        check(vm_mlstm_scan(proj, ld, bias_i, bias_f, norm_w, ctx.state(), ctx.cu_tokens, ctx.slots, out, ctx.B, H, D, V, cap, eps, code(ctx.act_dtype),
                            ctx.stream),
              "mlstm_scan", ctx.stream);
        return;
    }
    float* scratch = static_cast<float*>(c.take(vm_mlstm_chunk_scratch_floats(ctx.T_cap, ctx.B_cap, H, D, V), DType::F32));
    check(vm_mlstm_chunks(proj, ld, bias_i, bias_f, norm_w, ctx.state(), ctx.cu_tokens, ctx.slots, out, scratch, ctx.T, ctx.B, H, D, V, cap, eps,
                          code(ctx.act_dtype), ctx.stream),
          "mlstm_chunks", ctx.stream);
    counters().own_launches += 3;       // four kernels
    c.give(scratch);
}

// (norm_w given: x is the float32 residual stream and the kernels norm its rows themselves; residual given: the result is added into it)
inline void expert_router(const void* x, const float* norm_w, float eps, const float* w_router, const float* b_router, const float* w_gate, int T,
                          int hidden, int E, int top, int* chosen, float* weight, float* shared_gate, DType act, cudaStream_t s) {
    Timed t("expert_router", s);
    check(vm_expert_router(x, norm_w, eps, w_router, b_router, w_gate, T, hidden, E, top, chosen, weight, shared_gate, code(act), s), "expert_router", s);
}

inline void experts_few_tokens(const void* x, const float* norm_w, float eps, const DeviceTensor& up, const DeviceTensor& down, const void* up_shared,
                               const void* down_shared, const int* chosen, const float* weight, const float* shared_gate, int T, int hidden, int ff,
                               int ff_shared, int top, int act_kind, int act_kind_shared, void* act, void* out, float* residual, DType act_dtype,
                               cudaStream_t s) {
    Timed t("experts_few_tokens", s);
    check(vm_experts_few_tokens(x, norm_w, eps, up.ptr, down.ptr, up_shared, down_shared, code(up.dtype), chosen, weight, shared_gate, T, hidden, ff,
                                ff_shared, top, act_kind, act_kind_shared, act, out, residual, code(act_dtype), s),
          "experts_few_tokens", s);
    ++counters().own_launches;          // two kernels
}

// the general forms: a router that scores all outputs, gated experts, identity experts (csrc/routed_experts.cu)
struct ExpertKind {
    int E = 0, n_identity = 0;          // real experts; identity experts behind them in the router's outputs
    int act_kind = VM_ACT_RELU_SQUARED;
    int glu = VM_GLU_NONE;              // gated experts: VM_GLU_CLAMPED, or VM_GLU_SILU_WEIGHTED_INPUT (the routing weight on the expert's input)
    float limit = 0.f, alpha = 0.f;
};

inline void expert_router_scored(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                                 int n_out, int top, int group_count, int group_keep, int group_top, float scale, int score_kind, int* chosen, float* weight,
                                 DType act, cudaStream_t s) {
    Timed t("expert_router", s);
    check(vm_expert_router_groups(x, norm_w, eps, w_router, correction, T, hidden, n_out, top, group_count, group_keep, group_top, scale, score_kind, chosen,
                                  weight, code(act), s),
          "expert_router", s);
}

inline void experts_few_tokens_glu(const void* x, const float* norm_w, float eps, const DeviceTensor& up, const DeviceTensor& down, const void* up_shared,
                                   const void* down_shared, const int* chosen, const float* weight, const float* shared_gate, int T, int hidden, int ff,
                                   int ff_shared, int top, int act_kind_shared, const ExpertKind& k, void* act, void* out, float* residual,
                                   DType act_dtype, cudaStream_t s) {
    Timed t("experts_few_tokens", s);
    check(vm_experts_few_tokens_glu(x, norm_w, eps, up.ptr, down.ptr, up_shared, down_shared, code(up.dtype), chosen, weight, shared_gate, T, hidden, ff,
                                    ff_shared, top, k.act_kind, act_kind_shared, k.E, k.n_identity, k.glu, k.limit, k.alpha, act, out, residual,
                                    code(act_dtype), s),
          "experts_few_tokens", s);
    ++counters().own_launches;          // two kernels
}

inline void experts_grouped_glu(const void* x, const DeviceTensor& up, const DeviceTensor& down, const int* chosen, const float* weight,
                                const float* shared_y, const float* shared_gate, int T, int hidden, int ff, int top, const ExpertKind& k, int row_cap,
                                int* row_of_pair, int* token_of_row, int* expert_of_tile, void* x_sorted, void* act, void* gate_up, float* y, void* out,
                                int* err, cudaStream_t s) {
    Timed t(x_sorted ? "experts_grouped_tc" : "experts_grouped", s);
    check(vm_experts_grouped_glu(x, up.ptr, down.ptr, chosen, weight, shared_y, shared_gate, T, hidden, ff, top, k.E, k.n_identity, k.act_kind,
                                 k.glu, k.limit, k.alpha, row_cap, row_of_pair, token_of_row, expert_of_tile, x_sorted, act, gate_up, y, out, err, s),
          "experts_grouped", s);
    counters().own_launches += (x_sorted ? 4 : 3) + (k.glu ? 1 : 0);
}

inline void qkv_prepare(void* qkv, int ld, const float* wq, const float* wk, float eps, const float* lambda, const void* v_first, void* v_keep,
                        const StepContext& ctx, const KVView& kv, int H, int Hkv, int Dk, int Dv) {
    Timed t("qkv_prepare", ctx.stream);
    check(vm_qkv_prepare(qkv, ld, wq, wk, eps, lambda, v_first, v_keep, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width,
                         kv.owns ? kv.k_pages : nullptr, kv.owns ? kv.v_pages : nullptr, ctx.T, H, Hkv, Dk, Dv, kv.owns ? kv.n_pages : 0,
                         code(ctx.act_dtype), ctx.err, ctx.stream),
          "qkv_prepare", ctx.stream);
}

// what the biased attention kernels need beside the sizes: the bias table, the distance table, the mask
struct BiasedMask {
    const float* rel = nullptr;         // device float32 [rows, H], or null: no bias
    const int* bucket_of = nullptr;     // device int32 [far + 1]
    int far = 0, rows = 0, window = 0, keep_first = 0;
    const float* sink = nullptr;        // device float32 [H], or null: exp(sink[h]) joins head h's softmax denominator
    int v_row_stride = 0;               // elements between neighbouring tokens' value rows (0: Dv); Dk with the key pool as value pool: values inside keys
};
// attention of the step's tokens over the cache with that mask and bias; keys of Dk, values of Dv; picks the kernel by shape and dtype
void attention_biased(StepContext& ctx, const void* q, int q_row_stride, const KVView& kv, void* out, int H, int Hkv, int Dk, int Dv, float scale,
                      const BiasedMask& mask);

// the state-space mixer's kernels over the running schedule position's state area
constexpr int SSM_CHUNKS_FROM_TOKENS = 64;      // a step's capacity from which prompts run chunk by chunk
inline void ssm_mixer(const void* proj, int ld, const float* taps, const float* conv_bias, const float* dt_bias, const float* A_log, const float* Dskip,
                      const float* norm_w, float eps, StepContext& ctx, void* out, int H, int P, int N, int G, int K, int parts) {
    Timed t("ssm_mixer", ctx.stream);
    if (!ctx.state() || ctx.state_floats() < vm_ssm_state_floats(H, P, N, G, K)) throw CacheError("ssm: the cache holds no state area of this layer's size");
    const long long C = static_cast<long long>(H) * P + 2ll * G * N;
    void* xbc = ctx.take_tokens(C, ctx.act_dtype);
    float* y = static_cast<float*>(ctx.take_tokens(static_cast<long long>(H) * P, DType::F32));
    // The choice follows the step's capacity bucket alone, so that every step of a bucket asks for the same scratch: decode steps and
    // the smallest pieces go token by token, everything else chunk by chunk (every sequence may end in a chunk that is not full).
    const bool chunks = !ctx.one_token_each && ctx.T_cap >= SSM_CHUNKS_FROM_TOKENS && P <= 128;
    float* scratch = nullptr;
    int n_chunks = 0;
    if (chunks) {
        scratch = static_cast<float*>(ctx.take(vm_ssm_chunk_scratch_floats(ctx.T_cap, ctx.T_cap / 64 + ctx.B_cap, H, P, N), DType::F32));
        for (int b = 0; b < ctx.B; ++b) n_chunks += (ctx.host_cu_tokens[b + 1] - ctx.host_cu_tokens[b] + 63) / 64;
    }
    check(vm_ssm_mixer(proj, ld, taps, conv_bias, dt_bias, A_log, Dskip, norm_w, eps, ctx.state(), ctx.state_floats(), ctx.positions, ctx.seq_of_token,
                       ctx.cu_tokens, ctx.slots, xbc, y, out, scratch, n_chunks, ctx.one_token_each ? 1 : 0, ctx.T, ctx.B, H, P, N, G, K, parts,
                       code(ctx.act_dtype), ctx.stream),
          "ssm_mixer", ctx.stream);
    counters().own_launches += ctx.one_token_each ? 2 : (chunks ? 5 : (K > 1 ? 3 : 2));
    ctx.give(scratch);
    ctx.give(y);
    ctx.give(xbc);
}

inline void activation(const void* in, void* out, long long n, int kind, DType act, cudaStream_t s) {
    Timed t("activation", s);
    check(vm_activation(in, out, n, kind, code(act), s), "activation", s);
}

inline void experts_grouped(const void* x, const DeviceTensor& up, const DeviceTensor& down, const int* chosen, const float* weight, const float* shared_y,
                            const float* shared_gate, int T, int hidden, int ff, int top, int E, int act_kind, int row_cap, int* row_of_pair,
                            int* token_of_row, int* expert_of_tile, void* act, float* y, void* out, cudaStream_t s) {
    Timed t("experts_grouped", s);
    check(vm_experts_grouped(x, up.ptr, down.ptr, chosen, weight, shared_y, shared_gate, T, hidden, ff, top, E, act_kind, row_cap, row_of_pair,
                             token_of_row, expert_of_tile, act, y, out, s),
          "experts_grouped", s);
    counters().own_launches += 3;       // four kernels
}

inline void experts_grouped_tc(const void* x, const DeviceTensor& up, const DeviceTensor& down, const int* chosen, const float* weight,
                               const float* shared_y, const float* shared_gate, int T, int hidden, int ff, int top, int E, int act_kind, int row_cap,
                               int* row_of_pair, int* token_of_row, int* expert_of_tile, void* x_sorted, void* act, float* y, void* out, int* err,
                               cudaStream_t s) {
    Timed t("experts_grouped_tc", s);
    check(vm_experts_grouped_tc(x, up.ptr, down.ptr, chosen, weight, shared_y, shared_gate, T, hidden, ff, top, E, act_kind, row_cap, row_of_pair,
                                token_of_row, expert_of_tile, x_sorted, act, y, out, err, s),
          "experts_grouped_tc", s);
    counters().own_launches += 4;       // five kernels
}

// out = x W^T.  x [T, K] (row stride ldx), W [N, K], out [T, N]; a library matrix product, as in the reference
// (src/cuda/ops/matmul.cu:87-126); float32 runs without any reduced-precision mode.
void linear(const void* x, DType x_dtype, long long ldx, const DeviceTensor& W, void* out, DType out_dtype, int T, cudaStream_t s);
// h[T, N] += x W^T with the float32 residual stream h as the product's own accumulator (x and W bfloat16): the sum happens in
// the library's float32 epilogue, and the kernel after it reads h alone.
void linear_residual(const void* x, long long ldx, const DeviceTensor& W, float* h, int T, cudaStream_t s);

// `batch` products with one stride per operand (the heads of an activation against the heads of a weight):
// out_b[T, N] = x_b[T, K] W_b^T with W_b [N, K] row-major (transposed = false), or x_b W_b with W_b [K, N] row-major (true).
// x, W and out have the same dtype (float32 or bfloat16); sums are float32.
void linear_batched(const void* x, long long ldx, long long stride_x, const void* W, long long stride_w, bool w_is_k_by_n, void* out, long long ldo,
                    long long stride_o, DType dtype, int T, int N, int K, int batch, cudaStream_t s);

// attention of the step's tokens over the cache; picks the kernel for the step's shape and dtype
void attention(StepContext& ctx, const void* q, int q_row_stride, const KVView& kv, void* out, int H, int Hkv, int D, float scale, int window);

// the weight-streaming products for few rows (bfloat16 weights)
extern int SKINNY_MAX_ROWS;        // beyond this many rows the library product takes over
extern int SKINNY_NORM_ROWS;       // up to this many rows the norm is fused into the product that follows it
extern int SKINNY_HEAD_MAX_ROWS;   // up to this many rows the head streams its table with the weight-streaming kernels
extern int SKINNY_MAX_ROWS_LARGE;  // the same limit for a part whose largest weight matrix has SKINNY_LARGE_WEIGHT_BYTES and more
extern long long SKINNY_LARGE_WEIGHT_BYTES;
// rows (of a step's capacity) up to which the weight-streaming kernels take a part whose largest weight matrix has `weight_bytes`
inline int skinny_max_rows(long long weight_bytes) {
    return weight_bytes >= SKINNY_LARGE_WEIGHT_BYTES && SKINNY_MAX_ROWS_LARGE < SKINNY_MAX_ROWS ? SKINNY_MAX_ROWS_LARGE : SKINNY_MAX_ROWS;
}
inline bool skinny_ok(int M, long long K, const DeviceTensor& W) { return M > 0 && M <= SKINNY_MAX_ROWS && K % 32 == 0 && W.dtype == DType::BF16; }

inline void skinny_linear(const void* x, const float* norm_w, float eps, const DeviceTensor& W, int M, void* out, int out_stride, bool out_f32,
                          float* residual, int* err, cudaStream_t s) {
    Timed t("skinny_linear", s);
    check(vm_skinny_linear(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, M, static_cast<int>(W.rows()), static_cast<int>(W.cols()), out, out_stride,
                           out_f32 ? 1 : 0, residual, err, s),
          "skinny_linear", s);
}

inline void skinny_linear_act(const void* x, const float* norm_w, float eps, const DeviceTensor& W, int M, int act, void* out, int out_stride, int* err,
                              cudaStream_t s) {
    Timed t("skinny_linear_act", s);
    check(vm_skinny_linear_act(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, M, static_cast<int>(W.rows()), static_cast<int>(W.cols()), act, out, out_stride, err, s),
          "skinny_linear_act", s);
}

inline void skinny_swiglu(const void* x, const float* norm_w, float eps, const DeviceTensor& W, int M, int I, void* out, int* err, cudaStream_t s) {
    Timed t("skinny_swiglu", s);
    check(vm_skinny_swiglu(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, M, I, static_cast<int>(W.cols()), out, err, s), "skinny_swiglu", s);
}

inline void skinny_gated(const void* x, const float* norm_w, float eps, const DeviceTensor& W, int M, int I, int act, void* out, int* err,
                         cudaStream_t s) {
    Timed t("skinny_gated", s);
    check(vm_skinny_gated(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, M, I, static_cast<int>(W.cols()), act, out, err, s), "skinny_gated", s);
}

inline void skinny_qkv_rope(const void* x, const float* norm_w, float eps, const DeviceTensor& W, void* q_out, const StepContext& ctx, const KVView& kv,
                            const RotaryTable& rot, int H, int Hkv, int D) {
    Timed t("skinny_qkv_rope", ctx.stream);
    check(vm_skinny_qkv_rope(x, norm_w ? 1 : 0, norm_w, eps, W.ptr, ctx.T, static_cast<int>(W.cols()), q_out, ctx.positions, ctx.seq_of_token,
                             kv.block_table, kv.table_width, rot.inv_freq, rot.rotary_dim, rot.pairing, kv.owns ? kv.k_pages : nullptr,
                             kv.owns ? kv.v_pages : nullptr, H, Hkv, D, kv.owns ? kv.n_pages : 0, ctx.err, ctx.stream),
          "skinny_qkv_rope", ctx.stream);
}

// the tcgen05 + TMA products for many rows
inline bool tc_fused_rows(const StepContext& ctx) { return ctx.fused_prefill_rows > 0 && ctx.T_cap >= ctx.fused_prefill_rows; }

inline void tc_linear(const void* x, long long ldx, const DeviceTensor& W, int M, void* out, int out_stride, bool out_f32, float* residual, int* err,
                      cudaStream_t s) {
    Timed t("tc_linear", s);
    check(vm_tc_linear(x, ldx, W.ptr, M, static_cast<int>(W.rows()), static_cast<int>(W.cols()), out, out_stride, out_f32 ? 1 : 0, residual, err, s),
          "tc_linear", s);
}

inline void tc_swiglu(const void* x, long long ldx, const DeviceTensor& W, int M, int I, void* out, int* err, cudaStream_t s) {
    Timed t("tc_swiglu", s);
    check(vm_tc_swiglu(x, ldx, W.ptr, M, I, static_cast<int>(W.cols()), out, err, s), "tc_swiglu", s);
}

inline void tc_qkv_rope(const void* x, long long ldx, const DeviceTensor& W, void* q_out, const StepContext& ctx, const KVView& kv,
                        const RotaryTable& rot, int H, int Hkv, int D) {
    Timed t("tc_qkv_rope", ctx.stream);
    check(vm_tc_qkv_rope(x, ldx, W.ptr, ctx.T, static_cast<int>(W.cols()), q_out, ctx.positions, ctx.seq_of_token, kv.block_table, kv.table_width,
                         rot.inv_freq, rot.rotary_dim, rot.pairing, kv.owns ? kv.k_pages : nullptr, kv.owns ? kv.v_pages : nullptr, H, Hkv, D,
                         kv.owns ? kv.n_pages : 0, ctx.err, ctx.stream),
          "tc_qkv_rope", ctx.stream);
}

inline void sample(const float* logits, long long row_stride, int R, int V, const float* temperature, const float* top_p, const long long* seed,
                   const long long* stream_id, const long long* step, long long step_add, int* out, cudaStream_t s) {
    Timed t("sample", s);
    check(vm_sample(logits, row_stride, R, V, temperature, top_p, seed, stream_id, step, step_add, out, s), "sample", s);
}

inline void decode_advance(const int* sampled, int* tokens, int* positions, int* ctx_len, long long* draw_step, int* history, int* iteration, int B,
                           cudaStream_t s) {
    Timed t("decode_advance", s);
    check(vm_decode_advance(sampled, tokens, positions, ctx_len, draw_step, history, iteration, B, s), "decode_advance", s);
}

// ---- several copies of the residual stream
inline void streams_step(float* h, const StepContext& ctx, const void* y, const float* mix, const float* w_out, const float* w_in, const float* norm_w,
                         float eps, void* out) {
    Timed t("streams_step", ctx.stream);
    check(vm_streams_step(h, ctx.stream_stride, ctx.streams, y, mix, w_out, w_in, norm_w, eps, out, ctx.T, ctx.hidden, code(ctx.act_dtype), ctx.stream),
          "streams_step", ctx.stream);
}
inline void streams_sum_rows(float* h, long long stride, int S, const int* rows, int n_rows, int hid, cudaStream_t s) {
    Timed t("streams_sum_rows", s);
    check(vm_streams_sum_rows(h, stride, S, rows, n_rows, hid, s), "streams_sum_rows", s);
}

// where the running part keeps its own floats of a sequence: the run's state area, from ctx.state_offset on
inline void need_state(const StepContext& ctx, long long floats, const char* who) {
    if (!ctx.state() || ctx.state_floats() < ctx.state_offset + floats) throw CacheError(std::string(who) + ": the cache holds no state area of this part's size");
}

inline void embed_pairs(const DeviceTensor& table, const DeviceTensor& pairs, long long buckets, long long mul_prev, long long mul_cur, StepContext& ctx,
                        float* out) {
    Timed t("embed_pairs", ctx.stream);
    need_state(ctx, 1, "embedding");
    check(vm_embed_pairs(table.ptr, pairs.ptr, code(table.dtype), ctx.tokens, ctx.positions, ctx.seq_of_token, ctx.cu_tokens, ctx.slots,
                         reinterpret_cast<int*>(ctx.state() + ctx.state_offset), ctx.state_floats(), out, ctx.T, ctx.B, ctx.hidden,
                         static_cast<int>(table.rows()), buckets, mul_prev, mul_cur, ctx.one_token_each ? 1 : 0, ctx.err, ctx.stream),
          "embed_pairs", ctx.stream);
    if (!ctx.one_token_each) ++counters().own_launches;
}

// what mixer_prepare needs beside the step: the projections' layout and the options
struct PrepareArgs {
    const float* bias = nullptr;        // float32 [C] or null
    const float* taps = nullptr;        // float32 [C, K] or null
    int K = 0;
    const float *q_norm = nullptr, *k_norm = nullptr;
    float eps = 0.f;
    RotaryTable rot;
    int H = 0, G = 0, Dk = 0, Dv = 0;
    bool values_are_keys = false;
};
inline void mixer_prepare(const float* proj, int ld, const PrepareArgs& a, StepContext& ctx, const KVView& kv, void* q_out) {
    Timed t("mixer_prepare", ctx.stream);
    const long long C = static_cast<long long>(a.H + a.G) * a.Dk + (a.values_are_keys ? 0 : static_cast<long long>(a.G) * a.Dv);
    if (a.taps && a.K > 1) need_state(ctx, (a.K - 1) * C, "attention");
    check(vm_mixer_prepare(proj, ld, a.bias, a.taps, a.K, ctx.state(), ctx.state_floats(), ctx.state_offset, a.q_norm, a.k_norm, a.eps, a.rot.inv_freq,
                           a.rot.rotary_dim, a.rot.pairing, ctx.positions, ctx.seq_of_token, ctx.cu_tokens, ctx.slots, kv.block_table, kv.table_width, q_out,
                           kv.owns ? kv.k_pages : nullptr, kv.owns ? kv.v_pages : nullptr, kv.owns ? kv.n_pages : 0, ctx.T, ctx.B, a.H, a.G, a.Dk, a.Dv,
                           a.values_are_keys ? 1 : 0, ctx.one_token_each ? 1 : 0, code(ctx.act_dtype), ctx.err, ctx.stream),
          "mixer_prepare", ctx.stream);
    if (a.taps && a.K > 1 && !ctx.one_token_each) ++counters().own_launches;
}
inline void sigmoid_gate_heads(void* x, const float* g, int ldg, int T, int cols, int per, DType act, cudaStream_t s) {
    Timed t("sigmoid_gate", s);
    check(vm_sigmoid_gate_heads(x, g, ldg, T, cols, per, code(act), s), "sigmoid_gate", s);
}
inline void join_rows(const void* a, const void* b, const float* bias_a, float ca, float cb, const float* wa, const float* wb, float eps, void* out, int T,
                      int cols, DType act, cudaStream_t s) {
    Timed t("join_rows", s);
    check(vm_join_rows(a, b, bias_a, ca, cb, wa, wb, eps, out, T, cols, code(act), s), "join_rows", s);
}

// linear attention with a decaying matrix memory over the running part's state
struct MemoryArgs {
    int q_off = 0, k_off = 0, v_off = 0;
    const float* z = nullptr;           // decay logits float32 [T, ldz], or null: head_log_decay
    int ldz = 0;
    float tau = 1.f;
    const float* z_bias = nullptr;      // float32 [H, Dk] added to the logits, or null
    const float* head_log_decay = nullptr;
    RotaryTable rot;
    float q_scale = 1.f, k_scale = 1.f;
    int H = 0, Dk = 0, Dv = 0;
};
bool memory_scan_forced();                      // debugging aid: VELOMIND_B200_MEMORY_SCAN=1 keeps prompts on the token-by-token kernel
constexpr int MEMORY_CHUNKS_FROM_TOKENS = 64;   // a step's capacity from which prompts run chunk by chunk
inline void decayed_memory(float* proj, int ld, const MemoryArgs& a, StepContext& ctx, float* o) {      // (prompts: q and k of `proj` are turned in place)
    Timed t("decayed_memory", ctx.stream);
    need_state(ctx, static_cast<long long>(a.H) * a.Dk * a.Dv, "decayed_memory");
    // The choice follows the step's capacity bucket alone, so that every step of a bucket asks for the same scratch: decode steps and
    // the smallest pieces go token by token, everything else chunk by chunk (every sequence may end in a chunk that is not full).
    const int C = vm_decayed_memory_chunk_tokens(a.Dk, a.Dv);
    if (C > 0 && !ctx.one_token_each && ctx.T_cap >= MEMORY_CHUNKS_FROM_TOKENS && !memory_scan_forced()) {
        float* scratch = static_cast<float*>(ctx.take(vm_decayed_memory_scratch_floats(ctx.T_cap, ctx.B_cap, a.H, a.Dk, a.Dv), DType::F32));
        int n_chunks = 0;
        for (int b = 0; b < ctx.B; ++b) n_chunks += (ctx.host_cu_tokens[b + 1] - ctx.host_cu_tokens[b] + C - 1) / C;
        check(vm_decayed_memory_chunked(proj, ld, a.q_off, a.k_off, a.v_off, a.z, a.ldz, a.tau, a.z_bias, a.head_log_decay, a.rot.inv_freq, a.rot.rotary_dim,
                                        a.rot.pairing, a.q_scale, a.k_scale, ctx.state(), ctx.state_floats(), ctx.state_offset, ctx.positions, ctx.cu_tokens,
                                        ctx.slots, o, scratch, n_chunks, ctx.T, ctx.B, a.H, a.Dk, a.Dv, ctx.stream),
              "decayed_memory", ctx.stream);
        counters().own_launches += a.rot.inv_freq ? 3 : 2;       // three kernels, and one that turns q and k
        ctx.give(scratch);
        return;
    }
    check(vm_decayed_memory(proj, ld, a.q_off, a.k_off, a.v_off, a.z, a.ldz, a.tau, a.z_bias, a.head_log_decay, a.rot.inv_freq, a.rot.rotary_dim, a.rot.pairing,
                            a.q_scale, a.k_scale, ctx.state(), ctx.state_floats(), ctx.state_offset, ctx.positions, ctx.cu_tokens, ctx.slots, o, ctx.T, ctx.B,
                            a.H, a.Dk, a.Dv, ctx.stream),
          "decayed_memory", ctx.stream);
}
inline void memory_output(const float* o, const float* g, int ldg, const float* w, float eps, void* out, int T, int H, int Dv, DType act, cudaStream_t s) {
    Timed t("memory_output", s);
    check(vm_memory_output(o, g, ldg, w, eps, out, T, H, Dv, code(act), s), "memory_output", s);
}

int sm_count();                     // streaming multiprocessors of the current device, asked once

}  // namespace ops
}  // namespace vmb
