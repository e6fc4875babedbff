// Grouped-query softmax attention whose variations are arguments, as a mixer.
//
//   q, k, v = W_q x, W_k x, W_v x      H query heads and G key heads of `dim`, G value heads of `vdim`; `bias`: with biases q.b, k.b, v.b
//   `taps` K >= 1: a short causal convolution over time on every channel of q | k | v directly behind the projection,
//       y_t = sum_j w[:, j] u_(t - K + 1 + j), zeros before the sequence's start (tensors q.conv, k.conv, v.conv, [channels, K]);
//       the K - 1 last projected rows of a sequence are part of its state
//   `values_are_keys`: there is no W_v; a token's value is its key as it leaves the convolution, before norm and rotation
//   `qk_norm`: RMS norm over the whole projection of q (and of k), all heads at once, with a weight per column (q.norm, k.norm)
//   `position`: rotary positions on the first rotary_dim values of every q and k head, either pairing
//   score(i, j) = scale q_i . k_j;  i sees j  iff  j <= i and (window == 0 or i - j < window or j < keep_first)
//   `sink`: exp(sink_h), a learned number per head, joins head h's softmax denominator without a key or a value
//   `gate`: "values": the heads' outputs times sigmoid(W_g x) value by value ([H vdim, hidden]); "heads": one gate per head ([H, hidden])
//   then W_o, with the bias o.b if `out_bias`
//
// The projections (gate included) are one stacked product with a float32 result; bias, convolution, norm and rotation work on it in
// float32 and only the query rows and the cache rows are rounded to the activation dtype.  The cache holds what attention reads:
// turned keys, and values.
#include <cmath>

#include "args.h"
#include "linear.h"

namespace vmb {

class GeneralAttention : public Mixer {
public:
    explicit GeneralAttention(const json::Value& a) {
        const char* k = "general_attention";
        hidden_ = static_cast<int>(arg_int(a, "hidden", k));
        H_ = static_cast<int>(arg_int(a, "heads", k));
        G_ = static_cast<int>(arg_int_or(a, "kv_heads", H_, k));
        Dk_ = static_cast<int>(arg_int(a, "dim", k));
        Dv_ = static_cast<int>(arg_int_or(a, "vdim", Dk_, k));
        scale_ = static_cast<float>(arg_number_or(a, "scale", 1.0 / std::sqrt(static_cast<double>(Dk_)), k));
        window_ = static_cast<int>(arg_int_or(a, "window", 0, k));
        keep_first_ = static_cast<int>(arg_int_or(a, "keep_first", 0, k));
        K_ = static_cast<int>(arg_int_or(a, "taps", 0, k));
        bias_ = arg_int_or(a, "bias", 0, k) != 0;
        out_bias_ = arg_int_or(a, "out_bias", 0, k) != 0;
        qk_norm_ = arg_int_or(a, "qk_norm", 0, k) != 0;
        sink_ = arg_int_or(a, "sink", 0, k) != 0;
        values_are_keys_ = arg_int_or(a, "values_are_keys", 0, k) != 0;
        eps_ = static_cast<float>(arg_number_or(a, "eps", 1e-6, k));
        const std::string gate = arg_string_or(a, "gate", "none", k);
        if (gate != "none" && gate != "values" && gate != "heads") throw ConfigError(format("part '%s': gate is \"none\", \"values\" or \"heads\"", k));
        gate_cols_ = gate == "values" ? H_ * Dv_ : (gate == "heads" ? H_ : 0);
        gate_per_ = gate == "heads" ? Dv_ : 1;
        if (H_ <= 0 || G_ <= 0 || H_ % G_) throw ConfigError(format("part '%s': heads (%d) must be a multiple of kv_heads (%d)", k, H_, G_));
        if (Dk_ <= 0 || Dv_ <= 0) throw ConfigError(format("part '%s': dim and vdim must be positive", k));
        if (values_are_keys_ && Dv_ != Dk_) throw ConfigError(format("part '%s': values that are the keys have the keys' size (vdim %d, dim %d)", k, Dv_, Dk_));
        if (window_ < 0 || keep_first_ < 0) throw ConfigError(format("part '%s': window and keep_first must not be negative", k));
        if (window_ == 0) keep_first_ = 0;
        if (K_ < 0 || K_ > 16) throw ConfigError(format("part '%s': taps (%d) must be within 0..16", k, K_));
        if (const json::Value* pos = a.find("position")) position_ = build_part_as<Position>("position", part_spec_from_json(*pos, "general_attention.position"));
    }

    long long row_cols() const { return static_cast<long long>(H_ + G_) * Dk_ + (values_are_keys_ ? 0 : static_cast<long long>(G_) * Dv_); }
    long long proj_cols() const { return row_cols() + gate_cols_; }

    WeightTable weight_specs() const override {
        WeightTable t;
        t["q"].shape = {static_cast<long long>(H_) * Dk_, hidden_};
        t["k"].shape = {static_cast<long long>(G_) * Dk_, hidden_};
        if (!values_are_keys_) t["v"].shape = {static_cast<long long>(G_) * Dv_, hidden_};
        t["o"].shape = {hidden_, static_cast<long long>(H_) * Dv_};
        if (bias_) {
            t["q.b"].shape = {static_cast<long long>(H_) * Dk_};
            t["k.b"].shape = {static_cast<long long>(G_) * Dk_};
            if (!values_are_keys_) t["v.b"].shape = {static_cast<long long>(G_) * Dv_};
        }
        if (out_bias_) t["o.b"].shape = {hidden_};
        if (K_ >= 1) {
            t["q.conv"].shape = {static_cast<long long>(H_) * Dk_, K_};
            t["k.conv"].shape = {static_cast<long long>(G_) * Dk_, K_};
            if (!values_are_keys_) t["v.conv"].shape = {static_cast<long long>(G_) * Dv_, K_};
        }
        if (qk_norm_) {
            t["q.norm"].shape = {static_cast<long long>(H_) * Dk_};
            t["k.norm"].shape = {static_cast<long long>(G_) * Dk_};
            t["q.norm"].init_ones = t["k.norm"].init_ones = true;
        }
        if (sink_) t["sink"].shape = {H_};
        if (gate_cols_) t["g"].shape = {gate_cols_, hidden_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        std::vector<const HostTensor*> stacked = {&w.at("q"), &w.at("k")}, biases, taps;
        if (!values_are_keys_) stacked.push_back(&w.at("v"));
        if (gate_cols_) stacked.push_back(&w.at("g"));
        proj_.bind(stacked, bc);
        out_.bind({&w.at("o")}, bc);
        const char* parts[3] = {"q", "k", "v"};
        for (int i = 0; i < (values_are_keys_ ? 2 : 3); ++i) {
            if (bias_) biases.push_back(&w.at(std::string(parts[i]) + ".b"));
            if (K_ >= 1) taps.push_back(&w.at(std::string(parts[i]) + ".conv"));
        }
        if (bias_) b_ = bc.upload_stacked(biases, DType::F32);
        if (K_ >= 1) taps_ = bc.upload_stacked(taps, DType::F32);
        if (out_bias_) ob_ = bc.upload(w.at("o.b"), DType::F32);
        if (qk_norm_) {
            wq_ = bc.upload(w.at("q.norm"), DType::F32);
            wk_ = bc.upload(w.at("k.norm"), DType::F32);
        }
        if (sink_) sinks_ = bc.upload(w.at("sink"), DType::F32);
        if (position_) rotary_ = position_->tables(bc);
        if (rotary_.inv_freq && rotary_.rotary_dim > Dk_) throw ConfigError("part 'general_attention': the rotation covers more values than a head has");
    }

    bool graph_safe() const override { return !position_ || position_->graph_safe(); }

    CacheNeed cache_need() const override {
        CacheNeed n;
        n.kind = window_ > 0 ? CacheNeed::Window : CacheNeed::All;
        n.kv_heads = G_;
        n.key_dim = Dk_;
        n.value_dim = Dv_;
        n.window = window_;
        n.keep_first = keep_first_;
        n.state_floats = K_ > 1 ? static_cast<int>((K_ - 1) * row_cols()) : 0;
        return n;
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const DType act = ctx.act_dtype;
        const int ld = static_cast<int>(proj_cols());
        float* proj = static_cast<float*>(ctx.take_tokens(ld, DType::F32));
        project_f32(ctx, proj_, x, proj);
        const KVView kv = ctx.kv();
        ops::PrepareArgs p;
        p.bias = bias_ ? static_cast<const float*>(b_.ptr) : nullptr;
        p.taps = K_ >= 1 ? static_cast<const float*>(taps_.ptr) : nullptr;
        p.K = K_;
        p.q_norm = qk_norm_ ? static_cast<const float*>(wq_.ptr) : nullptr;
        p.k_norm = qk_norm_ ? static_cast<const float*>(wk_.ptr) : nullptr;
        p.eps = eps_;
        p.rot = rotary_;
        p.H = H_;
        p.G = G_;
        p.Dk = Dk_;
        p.Dv = Dv_;
        p.values_are_keys = values_are_keys_;
        void* q = ctx.take_tokens(static_cast<long long>(H_) * Dk_, act);
        ops::mixer_prepare(proj, ld, p, ctx, kv, q);
        void* att = ctx.take_tokens(static_cast<long long>(H_) * Dv_, act);
        ops::BiasedMask mask;
        mask.window = window_;
        mask.keep_first = keep_first_;
        mask.sink = sink_ ? static_cast<const float*>(sinks_.ptr) : nullptr;
        ops::attention_biased(ctx, q, H_ * Dk_, kv, att, H_, G_, Dk_, Dv_, scale_, mask);
        ctx.give(q);
        if (gate_cols_ && gate_per_ == 1) ops::sigmoid_gate(att, proj + row_cols(), ld, ctx.T, H_ * Dv_, act, ctx.stream);
        else if (gate_cols_) ops::sigmoid_gate_heads(att, proj + row_cols(), ld, ctx.T, H_ * Dv_, gate_per_, act, ctx.stream);
        ctx.give(proj);
        project(ctx, out_, att, out);
        ctx.give(att);
        if (out_bias_) ops::join_rows(out, nullptr, static_cast<const float*>(ob_.ptr), 1.f, 0.f, nullptr, nullptr, 0.f, out, ctx.T, hidden_, act, ctx.stream);
    }

private:
    int hidden_ = 0, H_ = 0, G_ = 0, Dk_ = 0, Dv_ = 0, window_ = 0, keep_first_ = 0, K_ = 0, gate_cols_ = 0, gate_per_ = 1;
    float scale_ = 1.f, eps_ = 1e-6f;
    bool bias_ = false, out_bias_ = false, qk_norm_ = false, sink_ = false, values_are_keys_ = false;
    std::shared_ptr<Position> position_;
    RotaryTable rotary_;
    Linear proj_, out_;
    DeviceTensor b_, taps_, ob_, wq_, wk_, sinks_;
};

namespace {
RegisterPart reg("mixer", "general_attention", [](const json::Value& a) { return std::make_shared<GeneralAttention>(a); });
}  // namespace

}  // namespace vmb
