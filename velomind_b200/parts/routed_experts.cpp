// A routed feed-forward (mixture of experts) with an optional shared expert.
//
//   z = W_router x + b (float32)          the `top` experts with the largest logits are chosen
//   w = softmax over the chosen logits    y = sum_k w_k W_down[e_k] act(W_up[e_k] x)
//   shared expert (if any): runs for every token and is added, times sigmoid(w_sg . x) if it has a gate
//
// Experts are two-layer networks without biases; `activation` names theirs (the shared expert may have another).  The router,
// its bias and the shared gate stay float32 on the device whatever the compute dtype.
//
// A second form of routing (`routing` = "scored"): s = softmax(z) over ALL the router's outputs; the choice goes by s plus a
// stored correction (tensor `correction`), which steers the choice but not the weights, among the outputs of the `groups_keep`
// best of `groups` equal groups of neighbours (a group's score is its largest choice score); the weights are s * `scale`, not
// renormalised.  The last `identity` outputs of the router are identity experts without tensors: their result is the input.
// A second form of expert (`glu` = 1): gate and up matrices, min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, +-limit) + 1).
//
// A third form of routing (`routing` = "sigmoid"): s = sigmoid(z), every output scored alone; the `top` largest are chosen and their
// scores are the weights, not renormalised; there is no correction tensor unless `correction` = 1.  A third form of expert (`glu` = 2):
// W_down (silu(W_gate h) * (W_up h)) where the routing weight multiplies the expert's INPUT, h = w x, not its output; the shared expert
// (tensors shared.gate, shared.up, shared.down) has the same form and runs with w = 1, without a gate of its own.  `glu` = 3 is the same unit
// with the routing weight on the expert's OUTPUT.  `groups_top` = n makes a group's score the sum of its n largest scores (default 1).
#include "args.h"
#include "linear.h"

namespace vmb {

int activation_code(const std::string& name, const char* part) {
    if (name == "silu") return VM_ACT_SILU;
    if (name == "gelu_tanh") return VM_ACT_GELU_TANH;
    if (name == "relu_squared") return VM_ACT_RELU_SQUARED;
    throw ConfigError(format("part '%s': activation '%s' is not known (silu, gelu_tanh, relu_squared)", part, name.c_str()));
}

// how the router turns its outputs into chosen experts and weights
struct Routing {
    bool scored = false;                 // false: softmax over the chosen logits; true: the form described above
    int groups = 1, groups_keep = 1, groups_top = 1, identity = 0;      // groups_top: a group's score is the sum of that many of its largest scores
    float scale = 1.f;
    int glu = VM_GLU_NONE;               // VM_GLU_*
    float limit = 0.f, alpha = 1.702f;
    int score_kind = VM_SCORE_SOFTMAX;   // of the scored form
    bool correction = true;              // the scored form has a correction tensor
};

class RoutedExperts : public FeedForward {
public:
    RoutedExperts(int hidden, int experts, int top, int ff, int act, int shared_ff, int shared_act, bool shared_gate, const Routing& r = {})
        : hidden_(hidden), E_(experts), top_(top), ff_(ff), act_(act), sff_(shared_ff), sact_(shared_act), gate_(shared_gate && shared_ff > 0), r_(r) {
        const char* k = "routed_experts";
        if (experts < 1 || r.identity < 0) throw ConfigError(format("part '%s': experts must be positive and identity not negative", k));
        const int outputs = experts + r.identity;
        if (!r.scored && (r.identity > 0 || r.groups != 1)) throw ConfigError(format("part '%s': identity experts and groups belong to routing \"scored\"", k));
        if (r.groups < 1 || outputs % r.groups || r.groups_keep < 1 || r.groups_keep > r.groups)
            throw ConfigError(format("part '%s': %d groups (of which %d stay) must divide the router's %d outputs", k, r.groups, r.groups_keep, outputs));
        const int eligible = outputs / r.groups * r.groups_keep;
        if (top < 1 || top > eligible) throw ConfigError(format("part '%s': top (%d) must be within 1..%d, the outputs that can be chosen", k, top, eligible));
        if (r.glu == VM_GLU_CLAMPED && !(r.limit > 0)) throw ConfigError(format("part '%s': gated experts need a positive limit", k));
        if (r.glu >= VM_GLU_SILU_WEIGHTED_INPUT && (r.identity > 0 || gate_)) throw ConfigError(format("part '%s': SiLU-gated experts have neither identity experts nor a gate on the shared expert", k));
        if (r.groups_top < 1) throw ConfigError(format("part '%s': groups_top must be positive", k));
    }

    ops::ExpertKind kind() const {
        ops::ExpertKind k;
        k.E = E_;
        k.n_identity = r_.identity;
        k.act_kind = act_;
        k.glu = r_.glu;
        k.limit = r_.limit;
        k.alpha = r_.alpha;
        return k;
    }
    bool general() const { return r_.scored || r_.glu; }      // the steps that take the general kernels
    bool shared_glu() const { return r_.glu >= VM_GLU_SILU_WEIGHTED_INPUT; }      // the shared expert has a gate matrix too

    WeightTable weight_specs() const override {
        WeightTable t;
        t["router"].shape = {E_ + r_.identity, hidden_};
        if (r_.scored) {
            if (r_.correction) t["correction"].shape = {E_ + r_.identity};
        } else {
            t["router.b"].shape = {E_};
        }
        for (int e = 0; e < E_; ++e) {
            if (r_.glu) t[format("e%d.gate", e)].shape = {ff_, hidden_};
            t[format("e%d.up", e)].shape = {ff_, hidden_};
            t[format("e%d.down", e)].shape = {hidden_, ff_};
        }
        if (sff_ > 0) {
            if (shared_glu()) t["shared.gate"].shape = {sff_, hidden_};
            t["shared.up"].shape = {sff_, hidden_};
            t["shared.down"].shape = {hidden_, sff_};
            if (gate_) t["shared.sg"].shape = {1, hidden_};
        }
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        router_ = bc.upload(w.at("router"), DType::F32);
        if (!r_.scored || r_.correction) router_b_ = bc.upload(w.at(r_.scored ? "correction" : "router.b"), DType::F32);
        std::vector<const HostTensor*> ups, downs, all;
        for (int e = 0; e < E_; ++e) {
            if (r_.glu) ups.push_back(&w.at(format("e%d.gate", e)));      // an expert's gate rows lie before its up rows
            ups.push_back(&w.at(format("e%d.up", e)));
            downs.push_back(&w.at(format("e%d.down", e)));
        }
        all = ups;
        all.insert(all.end(), downs.begin(), downs.end());
        if (sff_ > 0) {
            if (shared_glu()) all.push_back(&w.at("shared.gate"));
            all.push_back(&w.at("shared.up"));
            all.push_back(&w.at("shared.down"));
        }
        const DType kept = bc.matrix_dtype(all);           // one dtype for every expert matrix
        up_ = bc.upload_stacked(ups, kept);
        down_ = bc.upload_stacked(downs, kept);
        if (sff_ > 0) {
            if (shared_glu()) s_up_ = bc.upload_stacked({&w.at("shared.gate"), &w.at("shared.up")}, kept);      // gate rows before up rows
            else s_up_ = bc.upload(w.at("shared.up"), kept);
            s_down_ = bc.upload(w.at("shared.down"), kept);
            if (gate_) s_gate_ = bc.upload(w.at("shared.sg"), DType::F32);
        }
    }

    bool graph_safe() const override { return true; }

    // whether a step of this capacity groups its pairs by expert (many tokens) or streams each token's experts (few)
    bool grouped(const StepContext& ctx) const {
        return ctx.act_dtype == DType::BF16 && up_.dtype == DType::BF16 && hidden_ % 32 == 0 && ff_ % 32 == 0 && ctx.T_cap > GROUPED_FROM_TOKENS &&
               !ctx.one_token_each;
    }

    // Few tokens in bfloat16: router and up-projections norm the residual stream's rows themselves, the down-projections add
    // into it: three launches for the layer half.
    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        return norm.as_rms(&nw, &eps) && ctx.act_dtype == DType::BF16 && !grouped(ctx);
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        run_few(ctx, h, nw, eps, nullptr, h);
    }

    // chosen experts and weights of every token (and the shared expert's gate), by the part's form of routing
    void route(StepContext& ctx, const void* x, const float* nw, float eps, int* chosen, float* weight, float* sgate) {
        if (r_.scored) {
            if (gate_) throw Error("routed_experts: the scored router has no gate for a shared expert");
            ops::expert_router_scored(x, nw, eps, static_cast<const float*>(router_.ptr), r_.correction ? static_cast<const float*>(router_b_.ptr) : nullptr,
                                      ctx.T, hidden_, E_ + r_.identity, top_, r_.groups, r_.groups_keep, r_.groups_top, r_.scale, r_.score_kind, chosen, weight,
                                      ctx.act_dtype, ctx.stream);
            return;
        }
        ops::expert_router(x, nw, eps, static_cast<const float*>(router_.ptr), static_cast<const float*>(router_b_.ptr),
                           gate_ ? static_cast<const float*>(s_gate_.ptr) : nullptr, ctx.T, hidden_, E_, top_, chosen, weight, sgate, ctx.act_dtype,
                           ctx.stream);
    }

    // the few-token path: x in the activation dtype, or (nw given) the float32 residual stream; `residual` given: added into
    void run_few(StepContext& ctx, const void* x, const float* nw, float eps, void* out, float* residual) {
        int* chosen = static_cast<int*>(ctx.take_tokens(top_, DType::I32));
        float* weight = static_cast<float*>(ctx.take_tokens(top_, DType::F32));
        float* sgate = gate_ ? static_cast<float*>(ctx.take_tokens(1, DType::F32)) : nullptr;
        route(ctx, x, nw, eps, chosen, weight, sgate);
        void* act = ctx.take_tokens(vm_experts_act_cols(hidden_, ff_, sff_, top_, r_.identity), ctx.act_dtype);
        if (general())
            ops::experts_few_tokens_glu(x, nw, eps, up_, down_, sff_ > 0 ? s_up_.ptr : nullptr, sff_ > 0 ? s_down_.ptr : nullptr, chosen, weight, sgate,
                                        ctx.T, hidden_, ff_, sff_, top_, sact_, kind(), act, out, residual, ctx.act_dtype, ctx.stream);
        else
            ops::experts_few_tokens(x, nw, eps, up_, down_, sff_ > 0 ? s_up_.ptr : nullptr, sff_ > 0 ? s_down_.ptr : nullptr, chosen, weight, sgate, ctx.T,
                                    hidden_, ff_, sff_, top_, act_, sact_, act, out, residual, ctx.act_dtype, ctx.stream);
        ctx.give(act);
        ctx.give(sgate);
        ctx.give(weight);
        ctx.give(chosen);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        if (!grouped(ctx)) {
            run_few(ctx, x, nullptr, 0.f, out, nullptr);
            return;
        }
        int* chosen = static_cast<int*>(ctx.take_tokens(top_, DType::I32));
        float* weight = static_cast<float*>(ctx.take_tokens(top_, DType::F32));
        float* sgate = gate_ ? static_cast<float*>(ctx.take_tokens(1, DType::F32)) : nullptr;
        route(ctx, x, nullptr, 0.f, chosen, weight, sgate);
        // Many tokens (by the step's capacity, so that a bucket's steps ask for the same scratch): pairs grouped by expert, tensor-core
        // tiles per expert, the shared expert as two library products.  Few tokens: every token streams the rows of its experts.
        {
            float* shared_y = nullptr;
            if (sff_ > 0) {
                void* u = ctx.take_tokens(sff_, DType::BF16);
                if (shared_glu()) {
                    void* gu = ctx.take_tokens(2ll * sff_, DType::BF16);
                    ops::linear(x, DType::BF16, hidden_, s_up_, gu, DType::BF16, ctx.T, ctx.stream);
                    ops::gated_activation(gu, u, ctx.T, sff_, VM_ACT_SILU, DType::BF16, ctx.stream);
                    ctx.give(gu);
                } else {
                    ops::linear(x, DType::BF16, hidden_, s_up_, u, DType::BF16, ctx.T, ctx.stream);
                    ops::activation(u, u, static_cast<long long>(ctx.T) * sff_, sact_, DType::BF16, ctx.stream);
                }
                shared_y = static_cast<float*>(ctx.take_tokens(hidden_, DType::F32));
                ops::linear(u, DType::BF16, sff_, s_down_, shared_y, DType::F32, ctx.T, ctx.stream);
                ctx.give(u);
            }
            // the experts' tiles on tcgen05 from TC_FROM_TOKENS on (tiles of 128 rows, rows gathered first), on mma.sync below
            const bool tc = ctx.T_cap >= TC_FROM_TOKENS && ctx.err != nullptr && (!general() || (ff_ % 64 == 0 && hidden_ % 64 == 0));
            const int row_cap = static_cast<int>(tc ? vm_experts_grouped_rows_tiled(ctx.T_cap, top_, E_, 128) : vm_experts_grouped_rows(ctx.T_cap, top_, E_));
            int* row_of_pair = static_cast<int*>(ctx.take_tokens(top_, DType::I32));
            int* token_of_row = static_cast<int*>(ctx.take(row_cap, DType::I32));
            int* expert_of_tile = static_cast<int*>(ctx.take(row_cap / 64, DType::I32));
            void* act = ctx.take(static_cast<long long>(row_cap) * ff_, DType::BF16);
            float* y = static_cast<float*>(ctx.take(static_cast<long long>(row_cap) * hidden_, DType::F32));
            if (general()) {
                void* gate_up = r_.glu ? ctx.take(2ll * row_cap * ff_, DType::BF16) : nullptr;
                void* x_sorted = tc ? ctx.take(static_cast<long long>(row_cap) * hidden_, DType::BF16) : nullptr;
                ops::experts_grouped_glu(x, up_, down_, chosen, weight, shared_y, sgate, ctx.T, hidden_, ff_, top_, kind(), row_cap, row_of_pair,
                                         token_of_row, expert_of_tile, x_sorted, act, gate_up, y, out, ctx.err, ctx.stream);
                ctx.give(x_sorted);
                ctx.give(gate_up);
            } else if (tc) {
                void* x_sorted = ctx.take(static_cast<long long>(row_cap) * hidden_, DType::BF16);
                ops::experts_grouped_tc(x, up_, down_, chosen, weight, shared_y, sgate, ctx.T, hidden_, ff_, top_, E_, act_, row_cap, row_of_pair,
                                        token_of_row, expert_of_tile, x_sorted, act, y, out, ctx.err, ctx.stream);
                ctx.give(x_sorted);
            } else {
                ops::experts_grouped(x, up_, down_, chosen, weight, shared_y, sgate, ctx.T, hidden_, ff_, top_, E_, act_, row_cap, row_of_pair,
                                     token_of_row, expert_of_tile, act, y, out, ctx.stream);
            }
            ctx.give(y);
            ctx.give(act);
            ctx.give(expert_of_tile);
            ctx.give(token_of_row);
            ctx.give(row_of_pair);
            ctx.give(shared_y);
            ctx.give(sgate);
            ctx.give(weight);
            ctx.give(chosen);
            return;
        }
    }

    static constexpr int GROUPED_FROM_TOKENS = 64;      // a step's capacity above which the pairs are grouped by expert
    static constexpr int TC_FROM_TOKENS = 256;          // ... and from which the experts' tiles run on tcgen05

private:
    int hidden_, E_, top_, ff_, act_, sff_, sact_;
    bool gate_;
    Routing r_;
    DeviceTensor router_, router_b_, up_, down_, s_up_, s_down_, s_gate_;
};

namespace {
RegisterPart reg("feed_forward", "routed_experts", [](const json::Value& a) {
    const char* k = "routed_experts";
    const std::string act = arg_string_or(a, "activation", "relu_squared", k);
    Routing r;
    const std::string routing = arg_string_or(a, "routing", "chosen_softmax", k);
    if (routing != "chosen_softmax" && routing != "scored" && routing != "sigmoid")
        throw ConfigError("part 'routed_experts': routing is \"chosen_softmax\", \"scored\" or \"sigmoid\"");
    r.scored = routing != "chosen_softmax";
    r.score_kind = routing == "sigmoid" ? VM_SCORE_SIGMOID : VM_SCORE_SOFTMAX;
    r.correction = arg_int_or(a, "correction", routing == "scored" ? 1 : 0, k) != 0;
    r.groups = static_cast<int>(arg_int_or(a, "groups", 1, k));
    r.groups_keep = static_cast<int>(arg_int_or(a, "groups_keep", r.groups, k));
    r.groups_top = static_cast<int>(arg_int_or(a, "groups_top", 1, k));
    r.identity = static_cast<int>(arg_int_or(a, "identity", 0, k));
    r.scale = static_cast<float>(arg_number_or(a, "scale", 1.0, k));
    r.glu = static_cast<int>(arg_int_or(a, "glu", 0, k));
    if (r.glu < VM_GLU_NONE || r.glu > VM_GLU_SILU) throw ConfigError("part 'routed_experts': glu is 0 (none), 1 (clamped), 2 (SiLU, weight on the input) or 3 (SiLU, weight on the output)");
    r.limit = static_cast<float>(arg_number_or(a, "limit", 0.0, k));
    r.alpha = static_cast<float>(arg_number_or(a, "alpha", 1.702, k));
    return std::make_shared<RoutedExperts>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "experts", k)),
                                           static_cast<int>(arg_int(a, "top", k)), static_cast<int>(arg_int(a, "ff", k)), activation_code(act, k),
                                           static_cast<int>(arg_int_or(a, "shared_ff", 0, k)),
                                           activation_code(arg_string_or(a, "shared_activation", act, k), k), arg_int_or(a, "shared_gate", 1, k) != 0, r);
});
}  // namespace

}  // namespace vmb
