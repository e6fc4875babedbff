// Vozetar as a plan of parts: a decoder whose config.json lists its layers one by one, over several copies of the residual stream.
//
// The embedding adds a second table read by a hash of (previous token, token).  Every layer is pre-norm (RMSNorm) around a mixer and an
// optional feed-forward; with the key `streams` the layers are wired by hyper-connections (arrangement `hyper_connections`), the
// copies start as the embedding's output and their sum goes to the final norm.  Mixers:
//   "attention":   grouped-query softmax attention with biases (also on the output), a short convolution over time on q, k and v, rotary
//                  positions (pairs i, i + dims/2), every earlier token visible, a sink in the softmax, a sigmoid gate per value
//   "parallel":    left: softmax attention with biases on q, k, v, rotary positions (pairs 2i, 2i + 1), a sliding window with kept first
//                  tokens and a sink; right: retention (rotary pairs i, i + dims/2, keys scaled by dim^(-1/2), one fixed decay per head,
//                  heads divided by their root mean square, SiLU gate); joined as left_scale * left + right_scale * right
//   "parallel_2":  left: softmax attention whose values are its keys (as they leave the convolution), a convolution on q and k, a norm over
//                  the whole q and the whole k projection, rotary pairs 2i, 2i + 1, window with kept first tokens, a sigmoid gate per head;
//                  right: gated linear attention (queries scaled by dim^(-1/2), a decay per key channel sigmoid(z)^(1 / tau) from a low-rank
//                  projection, heads RMS-normed with a shared weight, SiLU gate); joined as half the sum of the two RMS-normed results
// Feed-forward: a SiLU-gated unit, or routed experts (sigmoid scores, the `top` largest among the experts of the best groups, a group's
// score being the sum of its two largest scores; weights are the scores, not renormalised; SiLU-gated experts; a shared expert).
//
// config.json: "architecture": "Vozetar", "vocab", "width", "streams", "norm": {"eps"}, "embedding": {"bigram": {"buckets", "mul_prev",
//   "mul_cur"}}, "layers": [{"type", "mixer": {...}, "mlp": {...} | null}].
// Tensors: embed, bigram, head, final.norm, and per layer l<i>.norm1, l<i>.norm2, l<i>.hc1.*, l<i>.hc2.*, l<i>.mix.*, l<i>.mlp.*.
// The rank of a gated-linear-attention layer's decay projection is the first extent of its tensor `a1`, read from the checkpoint's
// header (where there is no checkpoint yet, the optional key `decay_rank`, 16 by default).
#include <cmath>

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

long long first_extent(const json::Value& config, const std::string& tensor, long long fallback) {
    const json::Value* shapes = config.find("tensor_shapes");
    const json::Value* s = shapes ? shapes->find(tensor) : nullptr;
    if (!s || !s->is_array() || s->as_array().empty() || !s->as_array()[0].is_integer()) return fallback;
    return s->as_array()[0].as_int();
}

json::Value part(const std::string& kind, const json::Value& args) {
    json::Value p;
    p.set("kind", kind);
    p.set("args", args);
    return p;
}

// {"kind": rotary_*, "args": {...}} from a mixer's "rot": {base, dims}
json::Value rotation(const json::Value& mixer, long long dim, bool interleaved, const std::string& where) {
    KeyReader rot(need_object(mixer, "rot", where), where + ".rot");
    if (rot.integer_or("dims", dim, 0) == 0) return part("none", json::Value());      // a rotation over no values
    json::Value a;
    a.set("head_dim", dim);
    a.set("theta", rot.number("base"));
    a.set("rotary_dim", rot.integer_or("dims", dim));
    a.set("exact_frequencies", 1);           // base^(-2i / dims) in double precision, rounded once
    return part(interleaved ? "rotary_interleaved" : "rotary_half_split", a);
}

// the arguments every softmax attention of this architecture shares
json::Value attention_args(const json::Value& mx, int width, double eps, bool interleaved, const std::string& where) {
    KeyReader m(mx, where);
    json::Value a;
    a.set("hidden", width);
    const long long heads = m.integer("heads"), dim = m.integer("dim");
    a.set("heads", heads);
    a.set("kv_heads", m.integer_or("kv_heads", heads));
    a.set("dim", dim);
    a.set("vdim", m.integer_or("vdim", dim));
    a.set("scale", m.number("scale"));
    a.set("eps", eps);
    if (mx.find("rot") && !mx.find("rot")->is_null()) a.set("position", rotation(mx, dim, interleaved, where));
    if (const json::Value* mask = optional_object(mx, "mask", where)) {
        KeyReader k(*mask, where + ".mask");
        a.set("window", k.integer("size"));
        a.set("keep_first", k.integer_or("keep_first", 0, 0));
    }
    a.set("taps", m.integer_or("conv", 0, 0));
    return a;
}

json::Value mixer_attention(const json::Value& mx, int width, double eps, const std::string& where) {
    json::Value a = attention_args(mx, width, eps, false, where);
    a.set("bias", 1);
    a.set("out_bias", 1);
    a.set("sink", 1);
    a.set("gate", "values");
    return part("general_attention", a);
}

json::Value mixer_parallel(const json::Value& mx, int width, double eps, const std::string& where) {
    const json::Value& lj = need_object(mx, "left", where);
    const json::Value& rj = need_object(mx, "right", where);
    json::Value left = attention_args(lj, width, eps, true, where + ".left");
    left.set("bias", 1);
    left.set("sink", 1);
    KeyReader r(rj, where + ".right");
    const long long dim = r.integer("dim");
    json::Value right;
    right.set("hidden", width);
    right.set("heads", r.integer("heads"));
    right.set("dim", dim);
    right.set("vdim", r.integer_or("vdim", dim));
    right.set("decay", "fixed");
    right.set("decays", need(rj, "decay", where + ".right"));
    right.set("k_scale", 1.0 / std::sqrt(static_cast<double>(dim)));
    right.set("eps", eps);
    if (rj.find("rot") && !rj.find("rot")->is_null()) right.set("position", rotation(rj, dim, false, where + ".right"));
    KeyReader m(mx, where);
    json::Value a;
    a.set("hidden", width);
    a.set("left", part("general_attention", left));
    a.set("right", part("decayed_memory", right));
    a.set("join", "weighted");
    a.set("left_scale", m.number("left_scale", false));
    a.set("right_scale", m.number("right_scale", false));
    return part("side_by_side", a);
}

json::Value mixer_parallel_2(const json::Value& config, const json::Value& mx, int width, double eps, const std::string& prefix, const std::string& where) {
    const json::Value& lj = need_object(mx, "left", where);
    const json::Value& rj = need_object(mx, "right", where);
    json::Value left = attention_args(lj, width, eps, true, where + ".left");
    left.set("values_are_keys", 1);
    left.set("qk_norm", 1);
    left.set("gate", "heads");
    KeyReader r(rj, where + ".right");
    const long long dim = r.integer("dim");
    json::Value right;
    right.set("hidden", width);
    right.set("heads", r.integer("heads"));
    right.set("dim", dim);
    right.set("vdim", r.integer_or("vdim", dim));
    right.set("decay", "channel");
    right.set("tau", r.number("tau"));
    right.set("decay_rank", first_extent(config, prefix + "mix.right.a1", r.integer_or("decay_rank", 16)));
    right.set("q_scale", 1.0 / std::sqrt(static_cast<double>(dim)));
    right.set("norm_weight", 1);
    right.set("eps", eps);
    json::Value a;
    a.set("hidden", width);
    a.set("left", part("general_attention", left));
    a.set("right", part("decayed_memory", right));
    a.set("join", "normed_mean");
    a.set("eps", eps);
    return part("side_by_side", a);
}

ModelPlan vozetar_plan(const json::Value& config, const std::string& where) {
    KeyReader top(config, where);
    const int vocab = static_cast<int>(top.integer("vocab")), width = static_cast<int>(top.integer("width"));
    const double eps = KeyReader(need_object(config, "norm", where), where + ": norm").number("eps");
    const bool hyper = top.has("streams");
    const int streams = hyper ? static_cast<int>(top.integer("streams")) : 1;
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
    plan.residual_streams = streams;
    const int n = static_cast<int>(layers.as_array().size());
    int n_att = 0, n_par = 0, n_par2 = 0, n_dense = 0, n_moe = 0;
    for (int l = 0; l < n; ++l) {
        const json::Value& L = layers.as_array()[l];
        const std::string lw = format("%s: layers[%d]", where.c_str(), l);
        if (!L.is_object()) throw ConfigError(lw + " must be an object");
        const json::Value& type = need(L, "type", lw);
        const json::Value& mx = need_object(L, "mixer", lw);
        BlockSpec b;
        b.prefix = format("l%d.", l);
        b.names = {{"mixer", "mix."}, {"feed_forward", "mlp."}, {"mixer_norm", "norm1"}, {"feed_forward_norm", "norm2"}};
        const std::string t = type.is_string() ? type.as_string() : "?";
        json::Value mixer;
        if (t == "attention") { mixer = mixer_attention(mx, width, eps, lw + ".mixer"); ++n_att; }
        else if (t == "parallel") { mixer = mixer_parallel(mx, width, eps, lw + ".mixer"); ++n_par; }
        else if (t == "parallel_2") { mixer = mixer_parallel_2(config, mx, width, eps, b.prefix, lw + ".mixer"); ++n_par2; }
        else throw ConfigError(format("%s: type '%s' is not a mixer of this architecture (attention, parallel, parallel_2)", lw.c_str(), t.c_str()));
        b.mixer = part_spec_from_json(mixer, lw + ".mixer");
        b.mixer_norm = norm();
        json::Value wiring;
        wiring.set("hidden", width);
        wiring.set("streams", streams);
        b.arrangement = hyper ? "hyper_connections" : "prenorm";
        const json::Value* mlp = L.find("mlp");
        if (!mlp || mlp->is_null()) {
            wiring.set("feed_forward", 0);
            if (!hyper) b.arrangement = "prenorm_mixer";
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
                f.set("activation", "silu");
                f.set("gate", "gate");
                f.set("up", "up");
                f.set("down", "down");
                b.feed_forward = PartSpec{"gated", f};
                ++n_dense;
            } else if (kind.is_string() && kind.as_string() == "moe") {
                const json::Value& rj = need_object(*mlp, "router", fw);
                KeyReader router(rj, fw + ".router");
                f.set("experts", router.integer("experts"));
                f.set("top", router.integer("top"));
                f.set("ff", KeyReader(need_object(*mlp, "expert", fw), fw + ".expert").integer("ff"));
                f.set("routing", "sigmoid");
                f.set("glu", 3);                     // SiLU-gated experts, the routing weight on their output
                f.set("activation", "silu");
                if (const json::Value* groups = optional_object(rj, "groups", fw + ".router")) {
                    KeyReader g(*groups, fw + ".router.groups");
                    const long long count = g.integer("count");
                    f.set("groups", count);
                    f.set("groups_keep", g.integer_or("keep", count));
                    f.set("groups_top", 2);          // a group's score: the sum of its two largest scores
                }
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
        if (hyper) b.arrangement_args = wiring;
        plan.blocks.push_back(std::move(b));
        plan.schedule.push_back(ScheduleEntry{l, -1});
    }
    json::Value emb;
    emb.set("vocab", vocab);
    emb.set("hidden", width);
    const json::Value* e = optional_object(config, "embedding", where);
    const json::Value* big = e ? optional_object(*e, "bigram", where + ": embedding") : nullptr;
    if (big) {
        KeyReader k(*big, where + ": embedding.bigram");
        emb.set("tensor", "embed");
        emb.set("pairs_tensor", "bigram");
        emb.set("buckets", k.integer("buckets"));
        emb.set("mul_prev", k.integer("mul_prev", 0));
        emb.set("mul_cur", k.integer("mul_cur", 0));
        plan.embedding = PartSpec{"token_pairs_table", emb};
        plan.embedding_prefix = "";
    } else {
        emb.set("tensor", "");
        plan.embedding = PartSpec{"token_table", emb};
        plan.embedding_prefix = "embed";
    }
    json::Value h;
    h.set("vocab", vocab);
    h.set("hidden", width);
    h.set("tensor", "");
    plan.final_norm = norm();
    plan.final_norm_prefix = "final.norm";
    plan.head = PartSpec{"linear", h};
    plan.head_prefix = "head";
    plan.max_positions = 0;                      // rotary angles are computed from the position itself: no table, no limit of its own
    json::Value d;
    d.set("Vocab", format("%d tokens", vocab));
    d.set("Hidden", width);
    d.set("Streams", streams);
    d.set("Layers", format("%d attention, %d parallel, %d parallel_2", n_att, n_par, n_par2));
    d.set("FeedForward", format("%d dense, %d routed", n_dense, n_moe));
    plan.describe = d;
    return plan;
}

struct RegisterVozetar {
    RegisterVozetar() { register_architecture("Vozetar", vozetar_plan); }
} register_vozetar;

}  // namespace

}  // namespace vmb
