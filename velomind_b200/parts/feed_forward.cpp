// Gated feed-forward: down(act(gate(x)) * up(x)); SwiGLU with act = SiLU.
#include "args.h"
#include "linear.h"

namespace vmb {

// down(silu(gate(x)) * up(x)), no biases (examples/common/llama/llama_graph.cpp:22-28,122-138).  gate and up are one
// stacked product; the activation kernel reads both halves.
//
// `activation` (VM_ACT_*) and the three tensors' names are arguments; the weight-streaming kernels take the activation as an
// argument, the tcgen05 epilogue knows SiLU (other activations take the library products there).
class SwiGLU : public FeedForward {
public:
    SwiGLU(int hidden, int intermediate, int activation = VM_ACT_SILU, std::string gate = "gate_proj.weight", std::string up = "up_proj.weight",
           std::string down = "down_proj.weight")
        : hidden_(hidden), I_(intermediate), act_(activation), gate_name_(std::move(gate)), up_name_(std::move(up)), down_name_(std::move(down)) {}

    WeightTable weight_specs() const override {
        WeightTable t;
        t[gate_name_].shape = {I_, hidden_};
        t[up_name_].shape = {I_, hidden_};
        t[down_name_].shape = {hidden_, I_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        gate_up_.bind({&w.at(gate_name_), &w.at(up_name_)}, bc);
        down_.bind({&w.at(down_name_)}, bc);
    }

    bool graph_safe() const override { return true; }

    // rows up to which the weight-streaming kernels take this part (fewer when its matrices are large)
    int max_rows() const {
        return ops::skinny_max_rows(2 * std::max(gate_up_.weight.rows() * gate_up_.weight.cols(), down_.weight.rows() * down_.weight.cols()));
    }

    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16) return false;
        if (gate_up_.weight.dtype != DType::BF16 || down_.weight.dtype != DType::BF16) return false;
        if (ctx.T_cap <= max_rows()) return hidden_ % 32 == 0 && I_ % 32 == 0;
        return hidden_ % 8 == 0 && I_ % 8 == 0;
    }

    // h += down(silu(gate(norm(h))) * up(norm(h))): two or three launches.
    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const bool skinny = ctx.T_cap <= max_rows();
        const bool tc = !skinny && act_ == VM_ACT_SILU && ops::tc_fused_rows(ctx) && I_ % 64 == 0;      // (that epilogue knows SiLU)
        if (!skinny && !tc) {
            // the library's products: norm, gate and up, SwiGLU, down added into h by the product itself
            void* x = ctx.take_tokens(hidden_, DType::BF16);
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            void* gu = ctx.take_tokens(2ll * I_, DType::BF16);
            ops::linear(x, DType::BF16, hidden_, gate_up_.weight, gu, DType::BF16, ctx.T, ctx.stream);
            ctx.give(x);
            void* a = ctx.take_tokens(I_, DType::BF16);
            ops::gated_activation(gu, a, ctx.T, I_, act_, DType::BF16, ctx.stream);
            ctx.give(gu);
            ops::linear_residual(a, I_, down_.weight, h, ctx.T, ctx.stream);
            ctx.give(a);
            return;
        }
        void* act = ctx.take_tokens(I_, DType::BF16);
        if (skinny && ctx.T_cap <= ops::SKINNY_NORM_ROWS) {
            ops::skinny_gated(h, nw, eps, gate_up_.weight, ctx.T, I_, act_, act, ctx.err, ctx.stream);
        } else {
            void* x = ctx.take_tokens(hidden_, DType::BF16);           // many rows: norm once, not once per CTA
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            if (skinny) ops::skinny_gated(x, nullptr, 0.f, gate_up_.weight, ctx.T, I_, act_, act, ctx.err, ctx.stream);
            else ops::tc_swiglu(x, hidden_, gate_up_.weight, ctx.T, I_, act, ctx.err, ctx.stream);
            ctx.give(x);
        }
        if (skinny) ops::skinny_linear(act, nullptr, 0.f, down_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        else ops::tc_linear(act, I_, down_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        ctx.give(act);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        // few rows in bfloat16 (a layer whose wiring adds the result itself): the weight-streaming kernels, without norm or sum
        if (ctx.act_dtype == DType::BF16 && gate_up_.weight.dtype == DType::BF16 && down_.weight.dtype == DType::BF16 && ctx.T_cap <= max_rows() &&
            hidden_ % 32 == 0 && I_ % 32 == 0 && ctx.T > 0) {
            void* act = ctx.take_tokens(I_, DType::BF16);
            ops::skinny_gated(x, nullptr, 0.f, gate_up_.weight, ctx.T, I_, act_, act, ctx.err, ctx.stream);
            ops::skinny_linear(act, nullptr, 0.f, down_.weight, ctx.T, out, hidden_, false, nullptr, ctx.err, ctx.stream);
            ctx.give(act);
            return;
        }
        void* gu = ctx.take_tokens(2ll * I_, ctx.act_dtype);
        gate_up_.apply(ctx, x, ctx.act_dtype, gu, ctx.act_dtype, ctx.T, ctx.T_cap);
        void* act = ctx.take_tokens(I_, ctx.act_dtype);
        ops::gated_activation(gu, act, ctx.T, I_, act_, ctx.act_dtype, ctx.stream);
        ctx.give(gu);
        down_.apply(ctx, act, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(act);
    }

private:
    int hidden_, I_, act_;
    std::string gate_name_, up_name_, down_name_;
    Linear gate_up_, down_;
};

int activation_code(const std::string& name, const char* part);     // parts/routed_experts.cpp

// The two-matrix unit without a gate: down(act(up(x))), no biases; `activation` and the tensors' names are arguments.
//
// The activation "polynorm" is not elementwise: a N(z) + b N(z^2) + c N(z^3) + e with the powers taken value by value, N the
// division of a token's row of `intermediate` values by its root mean square (`eps` inside the root), and a, b, c, e the four
// numbers of the tensor `coefficients`.  Its sums are float32.
class PlainMLP : public FeedForward {
public:
    PlainMLP(int hidden, int intermediate, int activation, std::string up, std::string down, std::string coefficients = "", float eps = 0.f)
        : hidden_(hidden), I_(intermediate), act_(activation), up_name_(std::move(up)), down_name_(std::move(down)), coef_name_(std::move(coefficients)),
          eps_(eps) {
        if (act_ == VM_ACT_POLYNORM && coef_name_.empty()) throw ConfigError("part 'mlp': the activation \"polynorm\" needs the name of its tensor of coefficients");
    }

    WeightTable weight_specs() const override {
        WeightTable t;
        t[up_name_].shape = {I_, hidden_};
        t[down_name_].shape = {hidden_, I_};
        if (act_ == VM_ACT_POLYNORM) t[coef_name_].shape = {4};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        up_.bind({&w.at(up_name_)}, bc);
        down_.bind({&w.at(down_name_)}, bc);
        if (act_ == VM_ACT_POLYNORM) coef_ = bc.upload(w.at(coef_name_), DType::F32);
    }

    bool graph_safe() const override { return true; }

    int max_rows() const { return ops::skinny_max_rows(2 * up_.weight.rows() * up_.weight.cols()); }

    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16 || act_ == VM_ACT_POLYNORM) return false;
        if (up_.weight.dtype != DType::BF16 || down_.weight.dtype != DType::BF16) return false;
        if (ctx.T_cap <= max_rows()) return hidden_ % 32 == 0 && I_ % 32 == 0;
        return hidden_ % 8 == 0 && I_ % 8 == 0;
    }

    // h += down(act(up(norm(h)))): the norm in the first product (few tokens), the sum in the second
    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const bool skinny = ctx.T_cap <= max_rows();
        void* u = ctx.take_tokens(I_, DType::BF16);
        // (few tokens: the activation rides in the first product's epilogue)
        if (skinny && ctx.T_cap <= ops::SKINNY_NORM_ROWS) {
            ops::skinny_linear_act(h, nw, eps, up_.weight, ctx.T, act_, u, I_, ctx.err, ctx.stream);
        } else {
            void* x = ctx.take_tokens(hidden_, DType::BF16);
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            if (skinny) {
                ops::skinny_linear_act(x, nullptr, 0.f, up_.weight, ctx.T, act_, u, I_, ctx.err, ctx.stream);
            } else {
                ops::linear(x, DType::BF16, hidden_, up_.weight, u, DType::BF16, ctx.T, ctx.stream);
                ops::activation(u, u, static_cast<long long>(ctx.T) * I_, act_, DType::BF16, ctx.stream);
            }
            ctx.give(x);
        }
        if (skinny) ops::skinny_linear(u, nullptr, 0.f, down_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        else ops::linear_residual(u, I_, down_.weight, h, ctx.T, ctx.stream);
        ctx.give(u);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        // few tokens in bfloat16: the weight-streaming products (the first one with a float32 result where the activation sums over the row)
        const bool few = ctx.act_dtype == DType::BF16 && ctx.T_cap <= max_rows() && up_.weight.dtype == DType::BF16 && down_.weight.dtype == DType::BF16 &&
                         hidden_ % 32 == 0 && I_ % 32 == 0;
        void* u = ctx.take_tokens(I_, ctx.act_dtype);
        if (act_ == VM_ACT_POLYNORM) {
            if (few) {
                float* z = static_cast<float*>(ctx.take_tokens(I_, DType::F32));
                ops::skinny_linear(x, nullptr, 0.f, up_.weight, ctx.T, z, I_, true, nullptr, ctx.err, ctx.stream);
                ops::polynorm(z, DType::F32, static_cast<const float*>(coef_.ptr), u, ctx.T, I_, eps_, ctx.act_dtype, ctx.stream);
                ctx.give(z);
            } else {
                up_.apply(ctx, x, ctx.act_dtype, u, ctx.act_dtype, ctx.T, ctx.T_cap);
                ops::polynorm(u, ctx.act_dtype, static_cast<const float*>(coef_.ptr), u, ctx.T, I_, eps_, ctx.act_dtype, ctx.stream);
            }
        } else if (few) {
            ops::skinny_linear_act(x, nullptr, 0.f, up_.weight, ctx.T, act_, u, I_, ctx.err, ctx.stream);
        } else {
            up_.apply(ctx, x, ctx.act_dtype, u, ctx.act_dtype, ctx.T, ctx.T_cap);
            ops::activation(u, u, static_cast<long long>(ctx.T) * I_, act_, ctx.act_dtype, ctx.stream);
        }
        if (few) ops::skinny_linear(u, nullptr, 0.f, down_.weight, ctx.T, out, hidden_, false, nullptr, ctx.err, ctx.stream);
        else down_.apply(ctx, u, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(u);
    }

private:
    int hidden_, I_, act_;
    std::string up_name_, down_name_, coef_name_;
    float eps_;
    Linear up_, down_;
    DeviceTensor coef_;
};

namespace {
RegisterPart reg("feed_forward", "swiglu", [](const json::Value& a) {
    return std::make_shared<SwiGLU>(static_cast<int>(arg_int(a, "hidden", "swiglu")), static_cast<int>(arg_int(a, "intermediate", "swiglu")));
});
// the same unit with the activation and the tensor names as arguments
RegisterPart reg_gated("feed_forward", "gated", [](const json::Value& a) {
    const char* k = "gated";
    return std::make_shared<SwiGLU>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "intermediate", k)),
                                    activation_code(arg_string_or(a, "activation", "silu", k), k), arg_string_or(a, "gate", "gate_proj.weight", k),
                                    arg_string_or(a, "up", "up_proj.weight", k), arg_string_or(a, "down", "down_proj.weight", k));
});
// the unit without a gate
RegisterPart reg_mlp("feed_forward", "mlp", [](const json::Value& a) {
    const char* k = "mlp";
    const std::string act = arg_string_or(a, "activation", "relu_squared", k);
    return std::make_shared<PlainMLP>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "intermediate", k)),
                                      act == "polynorm" ? static_cast<int>(VM_ACT_POLYNORM) : activation_code(act, k), arg_string_or(a, "up", "up", k),
                                      arg_string_or(a, "down", "down", k), arg_string_or(a, "coefficients", "", k),
                                      static_cast<float>(arg_number_or(a, "eps", 0.0, k)));
});
}  // namespace

}  // namespace vmb
