// Token embedding table and the output head.
#include "args.h"
#include "linear.h"

namespace vmb {

// h[t, :] = table[token[t], :] into the float32 residual stream (src/cpu/ops/embedding.cpp:27-32).
class TokenEmbedding : public Embedding {
public:
    // `tensor`: what the table is called behind the part's prefix ("weight" unless the checkpoint says otherwise; may be empty)
    // `scale`: every row is multiplied by it on the way into the stream (in float32)
    TokenEmbedding(int vocab, int hidden, std::string tensor = "weight", float scale = 1.0f)
        : vocab_(vocab), hidden_(hidden), tensor_(std::move(tensor)), scale_(scale) {}
    WeightTable weight_specs() const override {
        WeightTable t;
        t[tensor_].shape = {vocab_, hidden_};
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override { table_ = bc.upload(w.at(tensor_), bc.matrix_dtype({&w.at(tensor_)})); }
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, const int* tokens, float* h) override { ops::embed_gather(table_, tokens, h, ctx.T, hidden_, scale_, ctx.err, ctx.stream); }

private:
    int vocab_, hidden_;
    std::string tensor_;
    float scale_;
    DeviceTensor table_;
};

// h[t, :] = table[token[t], :] + pairs[row(previous token, token[t]), :]: a second table read by a hash of the token and the one before it,
//     row = (previous * mul_prev + token * mul_cur) mod buckets,     and row `buckets` (the table's last) for a sequence's first token.
// The token before a step's first one is part of a sequence's state: one word per sequence in the cache's state area, left there by
// the step that fed it, so a prompt may be cut anywhere and decode steps queued on the device find the token they follow.
class TokenPairsEmbedding : public Embedding {
public:
    TokenPairsEmbedding(int vocab, int hidden, std::string tensor, std::string pairs, long long buckets, long long mul_prev, long long mul_cur)
        : vocab_(vocab), hidden_(hidden), tensor_(std::move(tensor)), pairs_name_(std::move(pairs)), buckets_(buckets), mul_prev_(mul_prev), mul_cur_(mul_cur) {
        if (buckets_ < 1) throw ConfigError("part 'token_pairs_table': buckets must be positive");
    }
    WeightTable weight_specs() const override {
        WeightTable t;
        t[tensor_].shape = {vocab_, hidden_};
        t[pairs_name_].shape = {buckets_ + 1, hidden_};
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override {
        const DType kept = bc.matrix_dtype({&w.at(tensor_), &w.at(pairs_name_)});      // one dtype for both tables
        table_ = bc.upload(w.at(tensor_), kept);
        pairs_ = bc.upload(w.at(pairs_name_), kept);
    }
    bool graph_safe() const override { return true; }
    int state_floats() const override { return 1; }
    void forward(StepContext& ctx, const int*, float* h) override { ops::embed_pairs(table_, pairs_, buckets_, mul_prev_, mul_cur_, ctx, h); }

private:
    int vocab_, hidden_;
    std::string tensor_, pairs_name_;
    long long buckets_, mul_prev_, mul_cur_;
    DeviceTensor table_, pairs_;
};

// logits = x W^T in float32.  `tied_to` names the tensor that stands in when the checkpoint has no head of its own
// (examples/smollm2/model_loader.cpp:124-158: lm_head.weight if present, else the embedding when tied); the device tensor is
// then shared with the embedding, not copied.
class LinearHead : public Head {
public:
    LinearHead(int vocab, int hidden, std::string tied_to, std::string tensor = "weight")
        : vocab_(vocab), hidden_(hidden), tied_to_(std::move(tied_to)), tensor_(std::move(tensor)) {}
    WeightTable weight_specs() const override {
        WeightTable t;
        t[tensor_].shape = {vocab_, hidden_};
        t[tensor_].alias_of = tied_to_;
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override { proj_.bind({&w.at(tensor_)}, bc); }
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, const void* x, float* logits) override {
        if (ctx.act_dtype == DType::BF16 && ops::skinny_ok(ctx.R, hidden_, proj_.weight) && vocab_ % 8 == 0 && ctx.R_cap <= ops::SKINNY_HEAD_MAX_ROWS)
            ops::skinny_linear(x, nullptr, 0.f, proj_.weight, ctx.R, logits, vocab_, true, nullptr, ctx.err, ctx.stream);   // few rows: stream the table once
        else
            proj_.apply(ctx, x, ctx.act_dtype, logits, DType::F32, ctx.R, ctx.R_cap);
    }

private:
    int vocab_, hidden_;
    std::string tied_to_, tensor_;
    Linear proj_;
};

namespace {
RegisterPart reg_embed("embedding", "token_table", [](const json::Value& a) {
    return std::make_shared<TokenEmbedding>(static_cast<int>(arg_int(a, "vocab", "token_table")), static_cast<int>(arg_int(a, "hidden", "token_table")),
                                            arg_string_or(a, "tensor", "weight", "token_table"),
                                            static_cast<float>(arg_number_or(a, "scale", 1.0, "token_table")));
});
RegisterPart reg_pairs("embedding", "token_pairs_table", [](const json::Value& a) {
    const char* k = "token_pairs_table";
    return std::make_shared<TokenPairsEmbedding>(static_cast<int>(arg_int(a, "vocab", k)), static_cast<int>(arg_int(a, "hidden", k)),
                                                 arg_string_or(a, "tensor", "weight", k), arg_string_or(a, "pairs_tensor", "pairs", k), arg_int(a, "buckets", k),
                                                 arg_int(a, "mul_prev", k), arg_int(a, "mul_cur", k));
});
RegisterPart reg_head("head", "linear", [](const json::Value& a) {
    return std::make_shared<LinearHead>(static_cast<int>(arg_int(a, "vocab", "linear")), static_cast<int>(arg_int(a, "hidden", "linear")),
                                        arg_string_or(a, "tied_to", "", "linear"), arg_string_or(a, "tensor", "weight", "linear"));
});
}  // namespace

}  // namespace vmb
