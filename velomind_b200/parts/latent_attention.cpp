// Latent attention without positions, as a mixer: queries and keys/values both pass through a low-rank latent, and the
// key/value latent is all the cache keeps of a token.
//
//   c_q = rmsnorm(W_dq x) ;  q_h = W_uq,h c_q                       (heads h, `dim` values each)
//   c   = rmsnorm(W_dkv x)                                           (kv_rank values: the cached row)
//   k_h = W_uk,h c ;  v_h = W_uv,h c ;  score = scale (q_h . k_h) ;  causal softmax ;  out = W_o concat_h(sum_j p_j v_h,j)
//
// Since q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j and sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j), the up-projections move to
// the query's and the output's side: attention runs with one shared "key/value head", the latent itself, as key AND value,
// and keys and values are never made.  That is the multi-query form the attention kernels of this library already serve
// (query heads that share a kv head), so prompts and decode steps use the same kernels as grouped-query attention.
//
// A layer may read another run's latents (the schedule's `cache_of`): it then has no W_dkv of its own, and writes nothing.
//
// Options, each an argument:
//   rot_dim > 0 with a `position` part: every query head has rot_dim more values behind its `dim` unrotated ones, and W_dkv has rot_dim
//     more rows behind the latent's: one key part for all heads, not normed.  Both are turned by the token's position, and
//     score = scale (q_h . k_h + q_rot,h . k_rot).  A cache row is then [c | k_rot]: with the up-projection on the query's side the
//     query is [W_uk,h^T q_h | q_rot,h], the key the whole row, the value its first kv_rank values.
//   window > 0: a query sees itself and the window - 1 tokens before it; the cache gives older pages back.
//   sink: a learned number per head (tensor `sink`) whose exponential joins the softmax's denominator, without key or value.
//   gate: the heads' outputs are multiplied by sigmoid(W_g x) (tensor `g`, read from the layer's input) before W_o.
#include <algorithm>
#include <cmath>

#include "args.h"
#include "linear.h"

namespace vmb {

struct LatentOptions {
    int rot_dim = 0, window = 0;
    bool sink = false, gate = false;
    PartSpec position{"none", json::Value()};
};

class LatentAttention : public Mixer {
public:
    using Options = LatentOptions;
    LatentAttention(int hidden, int heads, int dim, int vdim, int q_rank, int kv_rank, double scale, double eps, bool own_latent, const Options& o)
        : hidden_(hidden), H_(heads), D_(dim), V_(vdim), Rq_(q_rank), Rkv_(kv_rank), R_(o.rot_dim), window_(o.window), own_(own_latent), sink_(o.sink),
          gate_(o.gate), scale_(scale > 0 ? static_cast<float>(scale) : static_cast<float>(1.0 / std::sqrt(static_cast<double>(dim + o.rot_dim)))),
          eps_(static_cast<float>(eps)), position_(build_part_as<Position>("position", o.position)) {
        if (R_ < 0 || window_ < 0) throw ConfigError("part 'latent_attention': rot_dim and window must not be negative");
    }
    bool plain() const { return R_ == 0 && window_ == 0 && !sink_; }      // the form the unbiased attention kernels serve

    WeightTable weight_specs() const override {
        WeightTable t;
        t["dq"].shape = {Rq_, hidden_};
        t["dq.norm"].shape = {Rq_};
        t["dq.norm"].init_ones = true;
        t["uq"].shape = {static_cast<long long>(H_) * (D_ + R_), Rq_};
        if (own_) {
            t["dkv"].shape = {Rkv_ + R_, hidden_};
            t["dkv.norm"].shape = {Rkv_};
            t["dkv.norm"].init_ones = true;
        }
        t["uk"].shape = {static_cast<long long>(H_) * D_, Rkv_};
        t["uv"].shape = {static_cast<long long>(H_) * V_, Rkv_};
        t["o"].shape = {hidden_, static_cast<long long>(H_) * V_};
        if (sink_) t["sink"].shape = {H_};
        if (gate_) t["g"].shape = {static_cast<long long>(H_) * V_, hidden_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        std::vector<const HostTensor*> down{&w.at("dq")};      // one product for everything that reads the layer's input
        if (own_) down.push_back(&w.at("dkv"));
        if (gate_) down.push_back(&w.at("g"));
        down_.bind(down, bc);
        if (sink_) sinks_ = bc.upload(w.at("sink"), DType::F32);
        rotary_ = position_->tables(bc);
        if (R_ > 0 && (!rotary_.inv_freq || rotary_.rotary_dim > R_)) throw ConfigError("part 'latent_attention': rot_dim needs a rotary position part of at most that size");
        q_norm_ = bc.upload(w.at("dq.norm"), DType::F32);
        if (own_) kv_norm_ = bc.upload(w.at("dkv.norm"), DType::F32);
        up_q_.bind({&w.at("uq")}, bc);
        up_k_ = bc.upload(w.at("uk"), bc.dtype);          // the per-head products want one dtype for both operands
        up_v_ = bc.upload(w.at("uv"), bc.dtype);
        out_.bind({&w.at("o")}, bc);
    }

    bool graph_safe() const override { return position_->graph_safe(); }

    CacheNeed cache_need() const override {
        CacheNeed n;
        n.kind = window_ > 0 ? CacheNeed::Window : CacheNeed::All;
        n.kv_heads = 1;
        n.key_dim = Rkv_ + R_;                             // the latent and, behind it, the rotated key part
        n.value_dim = 0;                                   // the latent is key and value at once
        n.window = window_;
        return n;
    }
    int down_cols() const { return Rq_ + (own_ ? Rkv_ + R_ : 0) + (gate_ ? H_ * V_ : 0); }
    int gate_col() const { return Rq_ + (own_ ? Rkv_ + R_ : 0); }

    // Few tokens (decode steps) in bfloat16: the weight-streaming products of this library, with the layer's norm taken into
    // the down-projection and the residual sum into the output projection.
    int max_rows() const {
        long long most = std::max(down_.weight.rows() * down_.weight.cols(), out_.weight.rows() * out_.weight.cols());
        most = std::max(most, up_q_.weight.rows() * up_q_.weight.cols());
        return std::min(ops::skinny_max_rows(2 * most), ops::SKINNY_NORM_ROWS);
    }

    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || !skinny(ctx)) return false;
        return true;
    }

    // few tokens in bfloat16: the weight-streaming products take the layer's three projections
    bool skinny(const StepContext& ctx) const {
        if (ctx.act_dtype != DType::BF16 || ctx.T_cap > max_rows()) return false;
        if (down_.weight.dtype != DType::BF16 || up_q_.weight.dtype != DType::BF16 || out_.weight.dtype != DType::BF16) return false;
        return hidden_ % 32 == 0 && Rq_ % 32 == 0 && (H_ * V_) % 32 == 0 && down_cols() % 8 == 0 && (H_ * (D_ + R_)) % 8 == 0 && hidden_ % 8 == 0;
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        KVView kv = ctx.kv();
        if (kv.owns != own_) throw ConfigError("a latent-attention layer and its schedule disagree about whose latents it reads");
        void* o = heads(ctx, h, nw, eps, kv, true);
        ops::skinny_linear(o, nullptr, 0.f, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        ctx.give(o);
    }

    // x [T, hidden] (or, with norm_w, the float32 stream whose rows the first product norms) -> the heads' gated outputs [T, H*V]
    void* heads(StepContext& ctx, const void* x, const float* norm_w, float eps, KVView kv, bool skinny_products) {
        const DType act = ctx.act_dtype;
        const int cols = down_cols();
        float* down = static_cast<float*>(ctx.take_tokens(cols, DType::F32));
        if (skinny_products) ops::skinny_linear(x, norm_w, eps, down_.weight, ctx.T, down, cols, true, nullptr, ctx.err, ctx.stream);
        else down_.apply(ctx, x, act, down, DType::F32, ctx.T, ctx.T_cap);
        void* cq = ctx.take_tokens(Rq_, act);
        ops::latent_rope_norm_write(down, cols, Rq_, Rkv_, static_cast<const float*>(q_norm_.ptr), own_ ? static_cast<const float*>(kv_norm_.ptr) : nullptr,
                                    eps_, cq, ctx, kv, own_, R_, rotary_);
        if (!gate_) {                                      // (nothing else reads the projections' float32 result)
            ctx.give(down);
            down = nullptr;
        }
        const long long q_cols = static_cast<long long>(H_) * (D_ + R_);
        void* q = ctx.take_tokens(q_cols, act);
        if (skinny_products) ops::skinny_linear(cq, nullptr, 0.f, up_q_.weight, ctx.T, q, static_cast<int>(q_cols), false, nullptr, ctx.err, ctx.stream);
        else up_q_.apply(ctx, cq, act, q, act, ctx.T, ctx.T_cap);
        ctx.give(cq);
        // few tokens: the heads' products in kernels of this library that take the rotation and the gate along
        const bool own_products = act == DType::BF16 && ctx.T_cap <= 32 && D_ * 8 * 4 <= 48 * 1024 && Rkv_ * 8 * 4 <= 48 * 1024;
        void* o = attend(ctx, q, kv, own_products, gate_ ? down + gate_col() : nullptr, cols);
        if (gate_ && !own_products) ops::sigmoid_gate(o, down + gate_col(), cols, ctx.T, H_ * V_, act, ctx.stream);
        ctx.give(down);
        return o;
    }

    // q [T, H*(D+R)] -> o [T, H*V] (a buffer the caller gives back); q is given back here.  own_products: the per-head products run in
    // this library's kernels for few tokens, which turn the query's rotated part and apply the gate (float32 rows of gate_ld) themselves.
    void* attend(StepContext& ctx, void* q, KVView kv, bool own_products, const float* gate, long long gate_ld) {
        const DType act = ctx.act_dtype;
        // the key up-projection on the query's side: qa_h = [W_uk,h^T q_h | turned q_rot,h]
        const int Dk = Rkv_ + R_, Dq = D_ + R_;
        void* qa = ctx.take_tokens(static_cast<long long>(H_) * Dk, act);
        if (own_products) {
            ops::head_products_few(q, static_cast<long long>(H_) * Dq, Dq, up_k_.ptr, static_cast<long long>(D_) * Rkv_, /*k_by_n=*/true, qa,
                                   static_cast<long long>(H_) * Dk, Dk, Rkv_, D_, H_, nullptr, 0, R_, &rotary_, ctx);
        } else {
            ops::linear_batched(q, static_cast<long long>(H_) * Dq, Dq, up_k_.ptr, static_cast<long long>(D_) * Rkv_, /*w_is_k_by_n=*/true, qa,
                                static_cast<long long>(H_) * Dk, Dk, act, ctx.T, Rkv_, D_, H_, ctx.stream);
            if (R_ > 0) ops::rotate_slice(q, static_cast<long long>(H_) * Dq, Dq, D_, qa, static_cast<long long>(H_) * Dk, Dk, Rkv_, rotary_, R_, H_, ctx);
        }
        ctx.give(q);
        void* att = ctx.take_tokens(static_cast<long long>(H_) * Rkv_, act);
        kv.v_pages = kv.k_pages;
        if (plain()) {
            ops::attention(ctx, qa, H_ * Rkv_, kv, att, H_, 1, Rkv_, scale_, 0);
        } else {
            ops::BiasedMask mask;                          // no bias table: the mask, the sink, and values that are the front of the key rows
            mask.window = window_;
            mask.sink = sink_ ? static_cast<const float*>(sinks_.ptr) : nullptr;
            mask.v_row_stride = Dk;
            ops::attention_biased(ctx, qa, H_ * Dk, kv, att, H_, 1, Dk, Rkv_, scale_, mask);
        }
        ctx.give(qa);
        // the value up-projection on the output's side: o_h = W_uv,h (sum_j p_j c_j)
        void* o = ctx.take_tokens(static_cast<long long>(H_) * V_, act);
        if (own_products)
            ops::head_products_few(att, static_cast<long long>(H_) * Rkv_, Rkv_, up_v_.ptr, static_cast<long long>(V_) * Rkv_, /*k_by_n=*/false, o,
                                   static_cast<long long>(H_) * V_, V_, V_, Rkv_, H_, gate, gate_ld, 0, nullptr, ctx);
        else
            ops::linear_batched(att, static_cast<long long>(H_) * Rkv_, Rkv_, up_v_.ptr, static_cast<long long>(V_) * Rkv_, /*w_is_k_by_n=*/false, o,
                                static_cast<long long>(H_) * V_, V_, act, ctx.T, V_, Rkv_, H_, ctx.stream);
        ctx.give(att);
        return o;
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const DType act = ctx.act_dtype;
        KVView kv = ctx.kv();
        if (kv.owns != own_)
            throw ConfigError(own_ ? "a latent-attention layer with a down-projection of its own was scheduled onto another run's cache"
                                   : "a latent-attention layer without a down-projection must read another run's cache");
        const bool few = skinny(ctx);                      // (a choice by the step's capacity bucket)
        void* o = heads(ctx, x, nullptr, 0.f, kv, few);
        if (few) ops::skinny_linear(o, nullptr, 0.f, out_.weight, ctx.T, out, hidden_, false, nullptr, ctx.err, ctx.stream);
        else out_.apply(ctx, o, act, out, act, ctx.T, ctx.T_cap);
        ctx.give(o);
    }

private:
    int hidden_, H_, D_, V_, Rq_, Rkv_, R_, window_;
    bool own_, sink_, gate_;
    float scale_, eps_;
    std::shared_ptr<Position> position_;
    RotaryTable rotary_;
    Linear down_, up_q_, out_;
    DeviceTensor q_norm_, kv_norm_, up_k_, up_v_, sinks_;
};

namespace {
RegisterPart reg("mixer", "latent_attention", [](const json::Value& a) {
    const char* k = "latent_attention";
    LatentAttention::Options o;
    o.rot_dim = static_cast<int>(arg_int_or(a, "rot_dim", 0, k));
    o.window = static_cast<int>(arg_int_or(a, "window", 0, k));
    o.sink = arg_int_or(a, "sink", 0, k) != 0;
    o.gate = arg_int_or(a, "gate", 0, k) != 0;
    if (const json::Value* pos = a.find("position")) o.position = part_spec_from_json(*pos, "latent_attention.position");
    return std::make_shared<LatentAttention>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "heads", k)),
                                             static_cast<int>(arg_int(a, "dim", k)), static_cast<int>(arg_int(a, "vdim", k)),
                                             static_cast<int>(arg_int(a, "q_rank", k)), static_cast<int>(arg_int(a, "kv_rank", k)),
                                             arg_number_or(a, "scale", 0.0, k), arg_number(a, "eps", k), arg_int_or(a, "own_latent", 1, k) != 0, o);
});
}  // namespace

}  // namespace vmb
