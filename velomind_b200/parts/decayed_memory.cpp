// Linear attention with a decaying matrix memory, as a mixer (retention, gated linear attention).
//
//   q, k = W_q x, W_k x  [heads, dim];  v = W_v x  [heads, vdim];  no biases
//   `position`: rotary positions on the first rotary_dim values of every q and k head;  then q *= q_scale, k *= k_scale
//   per head  S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t          S [dim, vdim], zero at the sequence's start
//     `decay` = "fixed":   a_t = decay_h, one number per head (argument `decays`, a list)
//     `decay` = "channel": a_t = sigmoid(z_t)^(1 / tau) per key channel, z = W_a2 (W_a1 x) + b  (tensors a1 [rank, hidden], a2 [heads dim, rank], a2.b)
//   every head's o is divided by its root mean square (eps inside the root), times the weight `norm` [vdim] if `norm_weight`;
//   the heads side by side are multiplied by silu(W_g x) and projected by W_o.
//
// The memory lives in the cache's float32 state area of the sequence.  q | k | v | g come out of one stacked product as float32, the
// decay's logits out of two small float32 products (their matrices are kept in float32); decays, their logarithms, the memory and
// every sum over it are float32; only the gated heads are rounded to the activation dtype.
#include <cmath>

#include "args.h"
#include "linear.h"

namespace vmb {

class DecayedMemory : public Mixer {
public:
    explicit DecayedMemory(const json::Value& a) {
        const char* k = "decayed_memory";
        hidden_ = static_cast<int>(arg_int(a, "hidden", k));
        H_ = static_cast<int>(arg_int(a, "heads", k));
        Dk_ = static_cast<int>(arg_int(a, "dim", k));
        Dv_ = static_cast<int>(arg_int_or(a, "vdim", Dk_, k));
        q_scale_ = static_cast<float>(arg_number_or(a, "q_scale", 1.0, k));
        k_scale_ = static_cast<float>(arg_number_or(a, "k_scale", 1.0, k));
        eps_ = static_cast<float>(arg_number_or(a, "eps", 1e-6, k));
        norm_weight_ = arg_int_or(a, "norm_weight", 0, k) != 0;
        const std::string decay = arg_string_or(a, "decay", "fixed", k);
        if (decay != "fixed" && decay != "channel") throw ConfigError(format("part '%s': decay is \"fixed\" or \"channel\"", k));
        channel_ = decay == "channel";
        if (H_ <= 0 || Dk_ <= 0 || Dv_ <= 0) throw ConfigError(format("part '%s': heads, dim and vdim must be positive", k));
        if (Dk_ > 512) throw ConfigError(format("part '%s': dim (%d) above 512 has no kernel", k, Dk_));
        if (channel_) {
            tau_ = static_cast<float>(arg_number(a, "tau", k));
            rank_ = static_cast<int>(arg_int(a, "decay_rank", k));
            if (!(tau_ > 0) || rank_ <= 0) throw ConfigError(format("part '%s': tau and decay_rank must be positive", k));
        } else {
            const json::Value* d = a.find("decays");
            if (!d || !d->is_array() || static_cast<int>(d->as_array().size()) != H_)
                throw ConfigError(format("part '%s': a fixed decay needs the list 'decays' with one number per head (%d)", k, H_));
            for (const auto& v : d->as_array()) {
                if (!v.is_number() || !(v.as_double() > 0.0) || v.as_double() > 1.0) throw ConfigError(format("part '%s': a decay lies in (0, 1]", k));
                log_decay_.push_back(static_cast<float>(std::log(v.as_double())));
            }
        }
        if (const json::Value* pos = a.find("position")) position_ = build_part_as<Position>("position", part_spec_from_json(*pos, "decayed_memory.position"));
    }

    long long proj_cols() const { return 2ll * H_ * Dk_ + 2ll * H_ * Dv_; }      // q | k | v | g

    WeightTable weight_specs() const override {
        WeightTable t;
        t["q"].shape = t["k"].shape = {static_cast<long long>(H_) * Dk_, hidden_};
        t["v"].shape = t["g"].shape = {static_cast<long long>(H_) * Dv_, hidden_};
        t["o"].shape = {hidden_, static_cast<long long>(H_) * Dv_};
        if (norm_weight_) {
            t["norm"].shape = {Dv_};
            t["norm"].init_ones = true;
        }
        if (channel_) {
            t["a1"].shape = {rank_, hidden_};
            t["a2"].shape = {static_cast<long long>(H_) * Dk_, rank_};
            t["a2.b"].shape = {static_cast<long long>(H_) * Dk_};
        }
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        proj_.bind({&w.at("q"), &w.at("k"), &w.at("v"), &w.at("g")}, bc);
        out_.bind({&w.at("o")}, bc);
        if (norm_weight_) norm_ = bc.upload(w.at("norm"), DType::F32);
        if (channel_) {
            // the decay's two small matrices stay float32: their result enters the recurrence
            a1_.weight = bc.upload(w.at("a1"), DType::F32);
            a1_.out_features = rank_;
            a1_.in_features = hidden_;
            a2_.weight = bc.upload(w.at("a2"), DType::F32);
            a2_.out_features = static_cast<long long>(H_) * Dk_;
            a2_.in_features = rank_;
            a2b_ = bc.upload(w.at("a2.b"), DType::F32);
        } else {
            log_decay_dev_ = bc.upload_floats(log_decay_);
        }
        if (position_) rotary_ = position_->tables(bc);
        if (rotary_.inv_freq && rotary_.rotary_dim > Dk_) throw ConfigError("part 'decayed_memory': the rotation covers more values than a head has");
    }

    bool graph_safe() const override { return !position_ || position_->graph_safe(); }

    CacheNeed cache_need() const override {
        CacheNeed n;
        n.state_floats = H_ * Dk_ * Dv_;
        return n;
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const DType act = ctx.act_dtype;
        const int ld = static_cast<int>(proj_cols());
        const long long nqk = static_cast<long long>(H_) * Dk_, nv = static_cast<long long>(H_) * Dv_;
        float* proj = static_cast<float*>(ctx.take_tokens(ld, DType::F32));
        project_f32(ctx, proj_, x, proj);
        float* z = nullptr;
        if (channel_) {
            float* low = static_cast<float*>(ctx.take_tokens(rank_, DType::F32));
            a1_.apply(ctx, x, act, low, DType::F32, ctx.T, ctx.T_cap);
            z = static_cast<float*>(ctx.take_tokens(nqk, DType::F32));
            a2_.apply(ctx, low, DType::F32, z, DType::F32, ctx.T, ctx.T_cap);
            ctx.give(low);
        }
        ops::MemoryArgs m;
        m.q_off = 0;
        m.k_off = static_cast<int>(nqk);
        m.v_off = static_cast<int>(2 * nqk);
        m.z = z;
        m.ldz = static_cast<int>(nqk);
        m.tau = tau_;
        m.z_bias = channel_ ? static_cast<const float*>(a2b_.ptr) : nullptr;      // (the second product's bias rides in the recurrence kernel)
        m.head_log_decay = channel_ ? nullptr : static_cast<const float*>(log_decay_dev_.ptr);
        m.rot = rotary_;
        m.q_scale = q_scale_;
        m.k_scale = k_scale_;
        m.H = H_;
        m.Dk = Dk_;
        m.Dv = Dv_;
        float* o = static_cast<float*>(ctx.take_tokens(nv, DType::F32));
        ops::decayed_memory(proj, ld, m, ctx, o);
        ctx.give(z);
        void* gated = ctx.take_tokens(nv, act);
        ops::memory_output(o, proj + 2 * nqk + nv, ld, norm_weight_ ? static_cast<const float*>(norm_.ptr) : nullptr, eps_, gated, ctx.T, H_, Dv_, act, ctx.stream);
        ctx.give(o);
        ctx.give(proj);
        project(ctx, out_, gated, out);
        ctx.give(gated);
    }

private:
    int hidden_ = 0, H_ = 0, Dk_ = 0, Dv_ = 0, rank_ = 0;
    float q_scale_ = 1.f, k_scale_ = 1.f, eps_ = 1e-6f, tau_ = 1.f;
    bool norm_weight_ = false, channel_ = false;
    std::vector<float> log_decay_;
    std::shared_ptr<Position> position_;
    RotaryTable rotary_;
    Linear proj_, out_, a1_, a2_;
    DeviceTensor norm_, a2b_, log_decay_dev_;
};

namespace {
RegisterPart reg("mixer", "decayed_memory", [](const json::Value& a) { return std::make_shared<DecayedMemory>(a); });
}  // namespace

}  // namespace vmb
