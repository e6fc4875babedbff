// Two mixers side by side, both reading the same input, joined into one result.
//
//   `join` = "weighted":     out = left_scale * left(x) + right_scale * right(x)
//   `join` = "normed_mean":  out = (rmsnorm(left(x)) * w_left + rmsnorm(right(x)) * w_right) / 2     RMS norm over the model width, eps inside
//                            the root, plain weights (tensors `left.out`, `right.out`)
//
// `left` and `right` are mixer parts of any kind ({"kind", "args"}); their tensors hang under `left.` and `right.`.  At most one of the
// two may keep keys and values in pages; the fixed-size state of both lies in the run's state area, the left one's first.
#include "args.h"
#include "../engine/ops.h"

namespace vmb {

class SideBySide : public Mixer {
public:
    explicit SideBySide(const json::Value& a) {
        const char* k = "side_by_side";
        hidden_ = static_cast<int>(arg_int(a, "hidden", k));
        const json::Value *l = a.find("left"), *r = a.find("right");
        if (!l || !r) throw ConfigError(format("part '%s': needs the mixers 'left' and 'right'", k));
        left_ = build_part_as<Mixer>("mixer", part_spec_from_json(*l, "side_by_side.left"));
        right_ = build_part_as<Mixer>("mixer", part_spec_from_json(*r, "side_by_side.right"));
        const std::string join = arg_string_or(a, "join", "weighted", k);
        if (join != "weighted" && join != "normed_mean") throw ConfigError(format("part '%s': join is \"weighted\" or \"normed_mean\"", k));
        normed_ = join == "normed_mean";
        left_scale_ = static_cast<float>(arg_number_or(a, "left_scale", normed_ ? 0.5 : 1.0, k));
        right_scale_ = static_cast<float>(arg_number_or(a, "right_scale", normed_ ? 0.5 : 1.0, k));
        eps_ = static_cast<float>(arg_number_or(a, "eps", 1e-6, k));
        const CacheNeed nl = left_->cache_need(), nr = right_->cache_need();
        if (nl.kind != CacheNeed::None && nr.kind != CacheNeed::None) throw ConfigError(format("part '%s': only one of the two mixers may keep keys and values", k));
    }

    WeightTable weight_specs() const override {
        WeightTable t;
        for (const auto& kv : left_->weight_specs()) t["left." + kv.first] = kv.second;
        for (const auto& kv : right_->weight_specs()) t["right." + kv.first] = kv.second;
        if (normed_) {
            t["left.out"].shape = t["right.out"].shape = {hidden_};
            t["left.out"].init_ones = t["right.out"].init_ones = true;
        }
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        auto under = [&](const std::string& prefix, Mixer& m) {
            Weights sub;
            for (const auto& kv : m.weight_specs()) sub[kv.first] = w.at(prefix + kv.first);
            m.bind(sub, bc);
        };
        under("left.", *left_);
        under("right.", *right_);
        if (normed_) {
            wl_ = bc.upload(w.at("left.out"), DType::F32);
            wr_ = bc.upload(w.at("right.out"), DType::F32);
        }
    }

    bool graph_safe() const override { return left_->graph_safe() && right_->graph_safe(); }

    CacheNeed cache_need() const override {
        const CacheNeed nl = left_->cache_need(), nr = right_->cache_need();
        CacheNeed n = nl.kind != CacheNeed::None ? nl : nr;
        n.state_floats = nl.state_floats + nr.state_floats;
        return n;
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const int base = ctx.state_offset;
        void* a = ctx.take_tokens(hidden_, ctx.act_dtype);
        left_->forward(ctx, x, a);
        ctx.state_offset = base + left_->cache_need().state_floats;
        void* b = ctx.take_tokens(hidden_, ctx.act_dtype);
        right_->forward(ctx, x, b);
        ctx.state_offset = base;
        ops::join_rows(a, b, nullptr, left_scale_, right_scale_, normed_ ? static_cast<const float*>(wl_.ptr) : nullptr,
                       normed_ ? static_cast<const float*>(wr_.ptr) : nullptr, eps_, out, ctx.T, hidden_, ctx.act_dtype, ctx.stream);
        ctx.give(b);
        ctx.give(a);
    }

private:
    int hidden_ = 0;
    bool normed_ = false;
    float left_scale_ = 1.f, right_scale_ = 1.f, eps_ = 1e-6f;
    std::shared_ptr<Mixer> left_, right_;
    DeviceTensor wl_, wr_;
};

namespace {
RegisterPart reg("mixer", "side_by_side", [](const json::Value& a) { return std::make_shared<SideBySide>(a); });
}  // namespace

}  // namespace vmb
