// Arrangements: how a layer wires its norms, mixer, feed-forward and the residual stream.
#include "args.h"
#include "../engine/ops.h"

namespace vmb {

// Add a delta that is still pending to the residual stream: as it is, or through the norm its layer left with it.
static void settle_pending(StepContext& ctx, float* h, void* pending, long long hid) {
    if (!pending) return;
    if (ctx.pending_norm_weight)
        ops::norm_residual_add(h, pending, hid, ctx.act_dtype, ctx.pending_norm_weight, ctx.pending_norm_eps, ctx.T, static_cast<int>(hid), ctx.stream);
    else
        ops::residual_add(h, pending, static_cast<long long>(ctx.T) * hid, ctx.act_dtype, ctx.stream);
    ctx.pending_norm_weight = nullptr;
    ctx.give(pending);
}

// h += mixer(norm(h)); h += feed_forward(norm(h))  (examples/common/llama/llama_graph.cpp:203-229).
//
// The residual stream h is float32.  Each sum is carried out by the norm kernel that follows it, so `forward` takes the
// delta the previous layer left pending and returns its own last delta pending.  A part that can take the preceding norm
// into its first kernel and the residual sum into its last one (can_fuse / forward_fused) does so.
class PreNormBlock : public Arrangement {
public:
    explicit PreNormBlock(const BlockParts& p, bool feed_forward = true) : p_(p), feed_forward_(feed_forward) {}
    bool graph_safe() const override { return true; }

    void* forward(StepContext& ctx, float* h, void* pending) override {
        const long long hid = hidden(ctx);
        if (pending && ctx.pending_norm_weight) {   // a delta that joins the stream through its own layer's norm: added here, not by this layer's norm kernel
            settle(ctx, h, pending, hid);
            pending = nullptr;
        }
        if (p_.mixer->can_fuse(ctx, *p_.mixer_norm)) {
            settle(ctx, h, pending, hid);
            p_.mixer->forward_fused(ctx, h, *p_.mixer_norm);
            pending = nullptr;
        } else {
            void* x = ctx.take_tokens(hid, ctx.act_dtype);
            p_.mixer_norm->forward(ctx, h, pending, x, nullptr, 0);
            ctx.give(pending);
            pending = ctx.take_tokens(hid, ctx.act_dtype);
            p_.mixer->forward(ctx, x, pending);
            ctx.give(x);
        }
        if (!feed_forward_) return pending;        // a layer that is its mixer alone
        if (p_.feed_forward->can_fuse(ctx, *p_.feed_forward_norm)) {
            settle(ctx, h, pending, hid);
            p_.feed_forward->forward_fused(ctx, h, *p_.feed_forward_norm);
            return nullptr;
        }
        void* x = ctx.take_tokens(hid, ctx.act_dtype);
        p_.feed_forward_norm->forward(ctx, h, pending, x, nullptr, 0);
        ctx.give(pending);
        void* out = ctx.take_tokens(hid, ctx.act_dtype);
        p_.feed_forward->forward(ctx, x, out);
        ctx.give(x);
        return out;
    }

private:
    static long long hidden(const StepContext& ctx) { return ctx.hidden; }
    // add a delta that is still pending to the residual stream
    static void settle(StepContext& ctx, float* h, void* pending, long long hid) { settle_pending(ctx, h, pending, hid); }
    BlockParts p_;
    bool feed_forward_;
};

// h += norm(mixer(in(h))); h += norm(feed_forward(in(h))): the sublayers read the residual stream itself and the norm sits on
// each sublayer's OUTPUT.  in(h) = h + conv(h) when `taps` >= 1: a causal convolution over time on every channel,
//   conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j)     (tensors `mixer_conv` and `feed_forward_conv`, [hidden, taps], no bias),
// zeros before a sequence's start; with taps = 0 in(h) = h.  The last taps - 1 inputs of either
// convolution are part of a sequence's state: they live in the run's float32 state area behind the mixer's own state, and
// move on with every step.  Residual stream, convolution and norm are float32; what the sublayer reads is rounded to the
// activation dtype once.
class OutputNormBlock : public Arrangement {
public:
    OutputNormBlock(const BlockParts& p, int hidden, int taps, std::string mixer_conv, std::string ff_conv, bool feed_forward)
        : p_(p), hidden_(hidden), K_(taps < 0 ? 0 : taps), mixer_conv_(std::move(mixer_conv)), ff_conv_(std::move(ff_conv)), feed_forward_(feed_forward) {
        if (hidden <= 0) throw ConfigError("arrangement 'output_norm': argument 'hidden' must be positive");
        if (K_ > 64) throw ConfigError(format("arrangement 'output_norm': taps (%d) must be within 0..64", K_));
        if (K_ >= 1 && (mixer_conv_.empty() || (feed_forward_ && ff_conv_.empty())))
            throw ConfigError("arrangement 'output_norm': a convolution needs the names of its tensors");
    }
    bool graph_safe() const override { return true; }
    bool convolves() const { return K_ >= 1; }

    WeightTable weight_specs() const override {
        WeightTable t;
        if (!convolves()) return t;
        t[mixer_conv_].shape = {hidden_, K_};
        if (feed_forward_) t[ff_conv_].shape = {hidden_, K_};
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override {
        if (!convolves()) return;
        taps_mixer_ = bc.upload(w.at(mixer_conv_), DType::F32);
        if (feed_forward_) taps_ff_ = bc.upload(w.at(ff_conv_), DType::F32);
    }
    int state_floats() const override { return convolves() ? (feed_forward_ ? 2 : 1) * (K_ - 1) * hidden_ : 0; }

    void* forward(StepContext& ctx, float* h, void* pending) override {
        if (ctx.hidden != hidden_) throw ConfigError("arrangement 'output_norm': the stream's width is not the one it was built for");
        const int base = p_.mixer->cache_need().state_floats;
        const Rms n1 = rms_of(*p_.mixer_norm);
        const long long n = static_cast<long long>(ctx.T) * hidden_;
        const bool copies = convolves() || ctx.act_dtype != DType::F32;      // (a float32 sublayer without a convolution reads the stream in place)
        void* x = ctx.take_tokens(hidden_, ctx.act_dtype);
        if (pending && ctx.pending_norm_weight && joins_steps(ctx)) {
            // a decode step after a layer of this wiring: its last sum and this mixer's convolution on the row just made, one launch
            ops::norm_residual_conv_step(h, pending, ctx.act_dtype, ctx.pending_norm_weight, ctx.pending_norm_eps, static_cast<const float*>(taps_mixer_.ptr), K_,
                                         base, ctx, x);
            ctx.pending_norm_weight = nullptr;
            ctx.give(pending);
        } else {
            settle_pending(ctx, h, pending, hidden_);    // (a layer of another wiring left its last sum to its successor)
            read_stream(ctx, h, taps_mixer_, base, x, n);
        }
        void* y = ctx.take_tokens(hidden_, ctx.act_dtype);
        p_.mixer->forward(ctx, copies ? x : h, y);
        ctx.give(x);
        if (!feed_forward_) {
            if (joins_steps(ctx)) return leave(ctx, y, n1);
            ops::norm_residual_add(h, y, hidden_, ctx.act_dtype, n1.weight, n1.eps, ctx.T, hidden_, ctx.stream);
            ctx.give(y);
            return nullptr;
        }
        const Rms n2 = rms_of(*p_.feed_forward_norm);
        x = ctx.take_tokens(hidden_, ctx.act_dtype);
        if (joins_steps(ctx)) {
            // a decode step: the mixer's sum and the feed-forward's convolution on the row just made, one launch
            ops::norm_residual_conv_step(h, y, ctx.act_dtype, n1.weight, n1.eps, static_cast<const float*>(taps_ff_.ptr), K_, base + (K_ - 1) * hidden_, ctx, x);
        } else {
            ops::norm_residual_add(h, y, hidden_, ctx.act_dtype, n1.weight, n1.eps, ctx.T, hidden_, ctx.stream);
            read_stream(ctx, h, taps_ff_, base + (K_ - 1) * hidden_, x, n);
        }
        ctx.give(y);
        y = ctx.take_tokens(hidden_, ctx.act_dtype);
        p_.feed_forward->forward(ctx, copies ? x : h, y);
        ctx.give(x);
        if (joins_steps(ctx)) return leave(ctx, y, n2);
        ops::norm_residual_add(h, y, hidden_, ctx.act_dtype, n2.weight, n2.eps, ctx.T, hidden_, ctx.stream);
        ctx.give(y);
        return nullptr;
    }

private:
    struct Rms {
        const float* weight = nullptr;
        float eps = 0.f;
    };
    // a decode step of a convolving layer: a sum and the next convolution go into one launch
    bool joins_steps(const StepContext& ctx) const { return convolves() && ctx.one_token_each; }
    // the layer's last delta stays pending with its norm: the next layer adds it (with its own convolution, if it is of this wiring)
    static void* leave(StepContext& ctx, void* y, const Rms& norm) {
        ctx.pending_norm_weight = norm.weight;
        ctx.pending_norm_eps = norm.eps;
        return y;
    }
    static Rms rms_of(Norm& norm) {
        Rms r;
        if (!norm.as_rms(&r.weight, &r.eps)) throw ConfigError("arrangement 'output_norm': the norm on a sublayer's output must be a root-mean-square norm");
        return r;
    }
    // x = what a sublayer reads of the stream: h + conv(h), or h in the activation dtype
    void read_stream(StepContext& ctx, const float* h, const DeviceTensor& taps, int state_offset, void* x, long long n) {
        if (convolves()) ops::input_conv(h, static_cast<const float*>(taps.ptr), K_, state_offset, ctx, x);
        else if (ctx.act_dtype != DType::F32) ops::convert(h, DType::F32, x, ctx.act_dtype, n, ctx.stream);
    }
    BlockParts p_;
    int hidden_, K_;
    std::string mixer_conv_, ff_conv_;
    bool feed_forward_;
    DeviceTensor taps_mixer_, taps_ff_;
};

// Several copies x_1 .. x_S of the residual stream (hyper-connections): a sublayer reads the norm of a weighted sum of the copies,
// and its result y goes back into every copy while the copies are mixed:
//     u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] * y     (all copies at once from the old ones)
// with the tensors `<first>.in` [S], `<first>.out` [S], `<first>.mix` [S, S] (indexed [from, to]) for the mixer and `<second>.*` for the
// feed-forward.  Sums, mixing and norm are float32.  A sublayer's write and the next sublayer's read are one kernel: the layer leaves
// its last y pending with its `mix` and `out`, and whoever comes next (a layer of this wiring, or the model before its final norm)
// carries the write out.
class HyperConnections : public Arrangement {
public:
    HyperConnections(const BlockParts& p, int hidden, int streams, std::string first, std::string second, bool feed_forward)
        : p_(p), hidden_(hidden), S_(streams), first_(std::move(first)), second_(std::move(second)), feed_forward_(feed_forward) {
        if (hidden <= 0 || streams < 1 || streams > 16) throw ConfigError(format("arrangement 'hyper_connections': streams (%d) must be within 1..16", streams));
    }
    bool graph_safe() const override { return true; }
    bool mixes_streams() const override { return true; }

    WeightTable weight_specs() const override {
        WeightTable t;
        for (const std::string& n : names()) {
            t[n + ".in"].shape = t[n + ".out"].shape = {S_};
            t[n + ".mix"].shape = {S_, S_};
        }
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override {
        int i = 0;
        for (const std::string& n : names()) {
            in_[i] = bc.upload(w.at(n + ".in"), DType::F32);
            out_[i] = bc.upload(w.at(n + ".out"), DType::F32);
            mix_[i] = bc.upload(w.at(n + ".mix"), DType::F32);
            ++i;
        }
    }

    void* forward(StepContext& ctx, float* h, void* pending) override {
        if (ctx.hidden != hidden_ || ctx.streams != S_) throw ConfigError("arrangement 'hyper_connections': the model's stream is not the one this layer was built for");
        if (pending && !ctx.pending_mix) throw Error("arrangement 'hyper_connections': a layer of another wiring left a delta this layer cannot add");
        const Rms n1 = rms_of(*p_.mixer_norm);
        void* x = ctx.take_tokens(hidden_, ctx.act_dtype);
        ops::streams_step(h, ctx, pending, ctx.pending_mix, ctx.pending_out, fp(in_[0]), n1.weight, n1.eps, x);
        ctx.pending_mix = ctx.pending_out = nullptr;
        ctx.give(pending);
        void* y = ctx.take_tokens(hidden_, ctx.act_dtype);
        p_.mixer->forward(ctx, x, y);
        ctx.give(x);
        if (!feed_forward_) return leave(ctx, y, 0);
        const Rms n2 = rms_of(*p_.feed_forward_norm);
        x = ctx.take_tokens(hidden_, ctx.act_dtype);
        ops::streams_step(h, ctx, y, fp(mix_[0]), fp(out_[0]), fp(in_[1]), n2.weight, n2.eps, x);
        ctx.give(y);
        y = ctx.take_tokens(hidden_, ctx.act_dtype);
        p_.feed_forward->forward(ctx, x, y);
        ctx.give(x);
        return leave(ctx, y, 1);
    }

private:
    struct Rms {
        const float* weight = nullptr;
        float eps = 0.f;
    };
    static Rms rms_of(Norm& norm) {
        Rms r;
        if (!norm.as_rms(&r.weight, &r.eps)) throw ConfigError("arrangement 'hyper_connections': the norm in front of a sublayer must be a root-mean-square norm");
        return r;
    }
    static const float* fp(const DeviceTensor& t) { return static_cast<const float*>(t.ptr); }
    std::vector<std::string> names() const { return feed_forward_ ? std::vector<std::string>{first_, second_} : std::vector<std::string>{first_}; }
    void* leave(StepContext& ctx, void* y, int which) {
        ctx.pending_mix = fp(mix_[which]);
        ctx.pending_out = fp(out_[which]);
        return y;
    }
    BlockParts p_;
    int hidden_, S_;
    std::string first_, second_;
    bool feed_forward_;
    DeviceTensor in_[2], out_[2], mix_[2];
};

// The feed-forward of a layer that has none: no weights, never run.
class NoFeedForward : public FeedForward {
public:
    bool graph_safe() const override { return true; }
    void forward(StepContext&, const void*, void*) override { throw Error("a feed-forward of kind 'none' stands for a part that is not there; it cannot run"); }
};

namespace {
struct Reg {
    Reg() {
        register_arrangement("prenorm", [](const json::Value&, const BlockParts& parts) { return std::make_shared<PreNormBlock>(parts); });
        // h += mixer(norm(h)) and nothing else: the layer's feed-forward and its norm are parts of kind "none"
        register_arrangement("prenorm_mixer", [](const json::Value&, const BlockParts& parts) { return std::make_shared<PreNormBlock>(parts, false); });
        // the norm on each sublayer's output, the sublayers reading the stream through an optional short convolution over time
        register_arrangement("output_norm", [](const json::Value& a, const BlockParts& parts) {
            const char* k = "output_norm";
            return std::make_shared<OutputNormBlock>(parts, static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int_or(a, "taps", 0, k)),
                                                     arg_string_or(a, "mixer_conv", "", k), arg_string_or(a, "feed_forward_conv", "", k),
                                                     arg_int_or(a, "feed_forward", 1, k) != 0);
        });
        // several copies of the residual stream, read through weighted sums and mixed at every write
        register_arrangement("hyper_connections", [](const json::Value& a, const BlockParts& parts) {
            const char* k = "hyper_connections";
            return std::make_shared<HyperConnections>(parts, static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "streams", k)),
                                                      arg_string_or(a, "mixer_tensors", "hc1", k), arg_string_or(a, "feed_forward_tensors", "hc2", k),
                                                      arg_int_or(a, "feed_forward", 1, k) != 0);
        });
        register_part("feed_forward", "none", [](const json::Value&) { return std::make_shared<NoFeedForward>(); });
    }
} reg;
}  // namespace

}  // namespace vmb
