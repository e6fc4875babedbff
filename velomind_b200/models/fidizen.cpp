// Fidizen as a plan of parts: a decoder whose config.json lists its layers one by one.  Every layer's mixer is latent attention
// with a rotated key part shared by all heads, a sliding window, a sink in the softmax and a sigmoid gate on the heads' outputs;
// its optional feed-forward is a two-matrix unit with the polynomial unit-rms activation, or routed experts (sigmoid scores, the
// routing weight on the expert's input, SiLU-gated experts, an ungated shared expert).  The sublayers read the residual stream
// through a short causal convolution over time, and the RMS norm sits on each sublayer's OUTPUT (arrangement `output_norm`).
// The embedding is scaled; the head is untied.  A layer may run with another layer's weights and a cache and state of its own:
// the schedule then names that layer's block once more.
//
// config.json: "architecture": "Fidizen", "vocab", "width", "norm": {"eps"}, "embedding": {"scale"}, "canon": {"taps"},
//   "layers": [{"type": "latent_attention", "mixer": {...}, "mlp": {...} | null, "weights_of": j (optional)}].
//   mixer:            heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims}, mask: {size}
//   mlp kind "dense": ff
//   mlp kind "moe":   expert: {ff}, router: {experts, top}, shared: {ff} | null
// Tensors: embed, head, final.norm, and per layer l<i>.norm1, l<i>.norm2, l<i>.canon1, l<i>.canon2, l<i>.mix.*, l<i>.mlp.*.
#include "velomind_b200/velomind.h"

namespace vmb {

namespace {

const json::Value& need(const json::Value& o, const char* key, const std::string& where) {
    const json::Value* v = o.is_object() ? o.find(key) : nullptr;
    if (!v) throw ConfigError(where + ": missing required key '" + key + "'");
    return *v;
}

const json::Value& need_object(const json::Value& o, const char* key, const std::string& where) {
    const json::Value& v = need(o, key, where);
    if (!v.is_object()) throw ConfigError(where + ": key '" + key + "' must be an object");
    return v;
}

const json::Value* optional_object(const json::Value& o, const char* key, const std::string& where) {
    const json::Value* v = o.find(key);
    if (!v || v->is_null()) return nullptr;
    if (!v->is_object()) throw ConfigError(where + ": key '" + key + "' must be an object or null");
    return v;
}

ModelPlan fidizen_plan(const json::Value& config, const std::string& where) {
    KeyReader top(config, where);
    const int vocab = static_cast<int>(top.integer("vocab")), width = static_cast<int>(top.integer("width"));
    const double eps = KeyReader(need_object(config, "norm", where), where + ": norm").number("eps");
    double embed_scale = 1.0;
    if (const json::Value* e = optional_object(config, "embedding", where)) embed_scale = KeyReader(*e, where + ": embedding").number_or("scale", 1.0);
    int taps = 0;
    if (const json::Value* c = optional_object(config, "canon", where)) taps = static_cast<int>(KeyReader(*c, where + ": canon").integer_or("taps", 0, 0));
    const json::Value& layers = need(config, "layers", where);
    if (!layers.is_array() || layers.as_array().empty()) throw ConfigError(where + ": key 'layers' must be a list of layers");

    auto norm = [&]() {
        json::Value a;
        a.set("size", width);
        a.set("eps", eps);
        a.set("tensor", "");                    // the prefix is the tensor's whole name
        return PartSpec{"rmsnorm", a};
    };

    ModelPlan plan;
    plan.hidden_size = width;
    plan.vocab_size = vocab;
    const int n = static_cast<int>(layers.as_array().size());
    std::vector<int> block_of(static_cast<size_t>(n), -1);      // layer -> its block (a layer that borrows weights has none)
    int n_dense = 0, n_moe = 0, n_borrowed = 0;
    for (int l = 0; l < n; ++l) {
        const json::Value& L = layers.as_array()[l];
        const std::string lw = format("%s: layers[%d]", where.c_str(), l);
        if (!L.is_object()) throw ConfigError(lw + " must be an object");
        if (const json::Value* from = L.find("weights_of"); from && !from->is_null()) {
            // the layer runs another layer's tensors (mixer, feed-forward, norms, convolutions) over a cache and state of its own
            if (!from->is_integer() || from->as_int() < 0 || from->as_int() >= n || from->as_int() == l)
                throw ConfigError(lw + ": weights_of must name another layer");
            ++n_borrowed;
            continue;                                // (scheduled below, once every layer with tensors of its own has its block)
        }
        const json::Value& type = need(L, "type", lw);
        if (!type.is_string() || type.as_string() != "latent_attention")
            throw ConfigError(format("%s: type '%s' is not a mixer of this architecture (latent_attention)", lw.c_str(), type.is_string() ? type.as_string().c_str() : "?"));
        const json::Value& mx = need_object(L, "mixer", lw);
        KeyReader m(mx, lw + ".mixer");
        BlockSpec b;
        b.prefix = format("l%d.", l);
        b.names = {{"mixer", "mix."}, {"feed_forward", "mlp."}, {"mixer_norm", "norm1"}, {"feed_forward_norm", "norm2"}};
        json::Value a;
        a.set("hidden", width);
        a.set("heads", m.integer("heads"));
        a.set("dim", m.integer("dim"));
        a.set("vdim", m.integer("vdim"));
        a.set("q_rank", m.integer("q_rank"));
        a.set("kv_rank", m.integer("kv_rank"));
        a.set("scale", m.number("scale"));
        a.set("eps", eps);
        a.set("sink", 1);
        a.set("gate", 1);
        const long long rot_dim = m.integer_or("rot_dim", 0, 0);
        a.set("rot_dim", rot_dim);
        if (rot_dim > 0) {
            KeyReader rot(need_object(mx, "rot", lw + ".mixer"), lw + ".mixer.rot");
            json::Value pa;
            pa.set("head_dim", rot_dim);
            pa.set("theta", rot.number("base"));
            pa.set("rotary_dim", rot.integer_or("dims", rot_dim));
            json::Value pos;
            pos.set("kind", "rotary_interleaved");
            pos.set("args", pa);
            a.set("position", pos);
        }
        if (const json::Value* mask = optional_object(mx, "mask", lw + ".mixer")) a.set("window", KeyReader(*mask, lw + ".mixer.mask").integer_or("size", 0, 0));
        b.mixer = PartSpec{"latent_attention", a};
        b.mixer_norm = norm();
        json::Value wiring;
        wiring.set("hidden", width);
        wiring.set("taps", taps);
        wiring.set("mixer_conv", "canon1");
        wiring.set("feed_forward_conv", "canon2");
        b.arrangement = "output_norm";
        const json::Value* mlp = L.find("mlp");
        if (!mlp || mlp->is_null()) {
            wiring.set("feed_forward", 0);
            b.feed_forward = PartSpec{"none", json::Value()};
            b.feed_forward_norm = PartSpec{"none", json::Value()};
        } else {
            b.feed_forward_norm = norm();
            const std::string fw = lw + ".mlp";
            const json::Value& kind = need(*mlp, "kind", fw);
            json::Value f;
            f.set("hidden", width);
            if (kind.is_string() && kind.as_string() == "dense") {
                f.set("intermediate", KeyReader(*mlp, fw).integer("ff"));
                f.set("activation", "polynorm");
                f.set("coefficients", "act");
                f.set("eps", eps);
                f.set("up", "up");
                f.set("down", "down");
                b.feed_forward = PartSpec{"mlp", f};
                ++n_dense;
            } else if (kind.is_string() && kind.as_string() == "moe") {
                KeyReader router(need_object(*mlp, "router", fw), fw + ".router");
                f.set("experts", router.integer("experts"));
                f.set("top", router.integer("top"));
                f.set("ff", KeyReader(need_object(*mlp, "expert", fw), fw + ".expert").integer("ff"));
                f.set("routing", "sigmoid");
                f.set("glu", 2);                     // SiLU-gated experts, the routing weight on their input
                f.set("activation", "silu");
                if (const json::Value* shared = optional_object(*mlp, "shared", fw)) {
                    f.set("shared_ff", KeyReader(*shared, fw + ".shared").integer("ff"));
                    f.set("shared_gate", 0);
                }
                b.feed_forward = PartSpec{"routed_experts", f};
                ++n_moe;
            } else {
                throw ConfigError(fw + ": kind must be 'dense' or 'moe'");
            }
        }
        b.arrangement_args = wiring;
        block_of[l] = static_cast<int>(plan.blocks.size());
        plan.blocks.push_back(std::move(b));
    }
    for (int l = 0; l < n; ++l) {                    // the order of runs: every layer once, each with a cache and state of its own
        int j = l;
        for (int hops = 0; block_of[j] < 0; ++hops) {
            if (hops > n) throw ConfigError(format("%s: layers[%d]: weights_of leads in a circle", where.c_str(), l));
            j = static_cast<int>(layers.as_array()[j].find("weights_of")->as_int());
        }
        plan.schedule.push_back(ScheduleEntry{block_of[j], -1});
    }
    json::Value e;
    e.set("vocab", vocab);
    e.set("hidden", width);
    e.set("tensor", "");
    json::Value emb;
    emb.set("vocab", vocab);
    emb.set("hidden", width);
    emb.set("tensor", "");
    emb.set("scale", embed_scale);
    plan.embedding = PartSpec{"token_table", emb};
    plan.embedding_prefix = "embed";
    plan.final_norm = norm();
    plan.final_norm_prefix = "final.norm";
    plan.head = PartSpec{"linear", e};
    plan.head_prefix = "head";
    plan.max_positions = 0;                      // rotary angles are computed from the position itself: no table, no limit of its own
    json::Value d;
    d.set("Vocab", format("%d tokens", vocab));
    d.set("Hidden", width);
    d.set("Layers", format("%d latent attention (%d with another layer's weights)", n, n_borrowed));
    d.set("FeedForward", format("%d dense, %d routed", n_dense, n_moe));
    plan.describe = d;
    return plan;
}

struct RegisterFidizen {
    RegisterFidizen() { register_architecture("Fidizen", fidizen_plan); }
} register_fidizen;

}  // namespace

}  // namespace vmb
