// A decoder model built from a plan: embedding, layers run in the plan's order, final norm, head.
// Nothing here names an architecture; the plan says which parts and which order.
#include <cstdio>
#include <cstdlib>

#include "ops.h"

namespace vmb {

// ------------------------------------------------------------------------------------------------ StepContext
void* StepContext::take_tokens(long long cols, DType dtype) { return ws->take(static_cast<size_t>(T_cap) * cols * dtype_size(dtype)); }

void* StepContext::take(long long elements, DType dtype) { return ws->take(static_cast<size_t>(elements) * dtype_size(dtype)); }

void* StepContext::share(const std::string& name, long long cols, DType dtype) {
    if (shared_buffers.count(name)) throw Error("a step buffer named '" + name + "' is shared twice");
    Shared s{take_tokens(cols, dtype), cols, dtype};
    shared_buffers[name] = s;
    return s.ptr;
}

const StepContext::Shared* StepContext::shared(const std::string& name) const {
    auto it = shared_buffers.find(name);
    return it == shared_buffers.end() ? nullptr : &it->second;
}

KVView StepContext::kv() const {
    const std::pair<int, int> where = cache->book.where(run);
    if (where.first < 0) throw CacheError(format("schedule position %d has no key/value cache", run));
    KVView v;
    v.k_pages = cache->k_pages(where.first, where.second);
    v.v_pages = cache->v_pages(where.first, where.second);
    v.block_table = tables[where.first];
    v.table_width = table_widths[where.first];
    v.n_pages = cache->book.n_pages;
    v.owns = (*schedule)[run].cache_of < 0;
    return v;
}

float* StepContext::state() const {
    const auto& s = cache->state[run];
    return s ? static_cast<float*>(s->ptr) : nullptr;
}

int StepContext::state_floats() const { return cache->book.state_floats[run]; }

// ------------------------------------------------------------------------------------------------ Layer
Layer::Layer(const BlockSpec& s) : spec(s) {
    parts.mixer = build_part_as<Mixer>("mixer", s.mixer);
    parts.feed_forward = build_part_as<FeedForward>("feed_forward", s.feed_forward);
    parts.mixer_norm = build_part_as<Norm>("norm", s.mixer_norm);
    parts.feed_forward_norm = build_part_as<Norm>("norm", s.feed_forward_norm);
    block = build_arrangement(s.arrangement, s.arrangement_args, parts);
}

std::vector<std::pair<std::string, Part*>> Layer::named_parts() const {
    auto sub = [&](const char* role) {
        auto it = spec.names.find(role);
        return spec.prefix + (it != spec.names.end() ? it->second : std::string(role) + ".");
    };
    return {{sub("mixer"), parts.mixer.get()},
            {sub("feed_forward"), parts.feed_forward.get()},
            {sub("mixer_norm"), parts.mixer_norm.get()},
            {sub("feed_forward_norm"), parts.feed_forward_norm.get()},
            {spec.prefix, block.get()}};               // tensors of the wiring itself, if it has any
}

// ------------------------------------------------------------------------------------------------ DecoderModel
DecoderModel::DecoderModel(ModelPlan p) : plan(std::move(p)) {
    plan.validate();
    embedding = build_part_as<Embedding>("embedding", plan.embedding);
    for (const BlockSpec& b : plan.blocks) layers.emplace_back(b);
    for (const Layer& l : layers)
        if (plan.residual_streams > 1 && !l.block->mixes_streams())
            throw ConfigError("a model with several copies of the residual stream needs a wiring that mixes them in every layer ('" + l.spec.arrangement + "' does not)");
    final_norm = build_part_as<Norm>("norm", plan.final_norm);
    head = build_part_as<Head>("head", plan.head);
}

std::vector<std::pair<std::string, Part*>> DecoderModel::named_parts() const {
    std::vector<std::pair<std::string, Part*>> out;
    out.emplace_back(plan.embedding_prefix, embedding.get());
    for (const Layer& l : layers)
        for (auto& np : l.named_parts()) out.push_back(np);
    out.emplace_back(plan.final_norm_prefix, final_norm.get());
    out.emplace_back(plan.head_prefix, head.get());
    return out;
}

WeightTable DecoderModel::weight_table() const {
    WeightTable table;
    for (const auto& np : named_parts())
        for (const auto& kv : np.second->weight_specs()) table[np.first + kv.first] = kv.second;
    return table;
}

void DecoderModel::bind(const HostTensors& tensors, DType dt, int dev, cudaStream_t stream) {
    if (dt != DType::F32 && dt != DType::BF16) throw KernelError("a model computes in float32 or bfloat16");
    BindContext bc(dt, stream);
    for (const auto& np : named_parts()) {
        Weights w;
        for (const auto& kv : np.second->weight_specs()) w[kv.first] = tensors.at(np.first + kv.first);
        np.second->bind(w, bc);
    }
    dtype = dt;
    device = dev;
}

bool DecoderModel::graph_safe() const {
    for (const auto& np : named_parts())
        if (!np.second->graph_safe()) return false;
    for (const Layer& l : layers)
        if (!l.block->graph_safe()) return false;
    return true;
}

std::vector<CacheNeed> DecoderModel::cache_needs() const {
    std::vector<CacheNeed> out;
    for (const ScheduleEntry& e : plan.schedule) {
        const Layer& l = layers[e.layer];
        const int wiring = l.block->state_floats();      // what the wiring keeps per sequence lies behind the mixer's own state
        if (wiring > 0 && e.cache_of >= 0) throw ConfigError("a layer whose wiring keeps state of its own cannot read another run's cache");
        CacheNeed need = e.cache_of >= 0 ? CacheNeed{} : l.parts.mixer->cache_need();
        need.state_floats += wiring;
        out.push_back(need);
    }
    if (embedding->state_floats() > 0) {             // what the embedding keeps per sequence: one more state area behind the runs'
        CacheNeed need;
        need.state_floats = embedding->state_floats();
        out.push_back(need);
    }
    return out;
}

std::vector<int> DecoderModel::cache_shares() const {
    std::vector<int> out;
    for (const ScheduleEntry& e : plan.schedule) out.push_back(e.cache_of);
    if (embedding->state_floats() > 0) out.push_back(-1);
    return out;
}

// Debugging aid: VELOMIND_B200_DUMP_STREAM=<file> appends, after every run of a layer, the residual stream of the step's tokens (the
// sum of its copies) to that file as float32 [T, hidden].  It waits for the device after every layer, so it belongs with
// VELOMIND_B200_SYNC=1 (no recorded steps); a delta that a layer left pending is not in the rows it writes.
static const char* dump_stream_path() {
    static const char* path = std::getenv("VELOMIND_B200_DUMP_STREAM");
    return path && *path ? path : nullptr;
}

static void dump_stream(StepContext& ctx, const float* h, bool pending) {
    if (ctx.capturing) return;
    const size_t n = static_cast<size_t>(ctx.T) * ctx.hidden;
    std::vector<float> sum(n, 0.f), one(n);
    for (int s = 0; s < ctx.streams; ++s) {
        ops::cuda_check(cudaMemcpyAsync(one.data(), h + s * ctx.stream_stride, n * sizeof(float), cudaMemcpyDeviceToHost, ctx.stream), "reading the residual stream");
        ops::cuda_check(cudaStreamSynchronize(ctx.stream), "reading the residual stream");
        for (size_t i = 0; i < n; ++i) sum[i] += one[i];
    }
    if (FILE* f = std::fopen(dump_stream_path(), "ab")) {
        std::fwrite(sum.data(), sizeof(float), n, f);
        std::fclose(f);
    }
    if (pending) std::fprintf(stderr, "velomind_b200: a layer left a delta pending; the dumped rows are without it\n");
}

// Run the step's tokens through every layer of the schedule; float32 logits [R, vocab] at ctx.logit_rows.
void DecoderModel::forward(StepContext& ctx) {
    const long long hid = plan.hidden_size;
    ctx.hidden = plan.hidden_size;
    const int S = plan.residual_streams;
    ctx.streams = S;
    ctx.stream_stride = static_cast<long long>(ctx.T_cap) * hid;
    ctx.state_offset = 0;
    float* h = static_cast<float*>(ctx.take_tokens(hid * S, DType::F32));      // copy s of the stream: [T, hid] at h + s * stream_stride
    ctx.run = static_cast<int>(plan.schedule.size());                          // the embedding's own state area, if it keeps one
    embedding->forward(ctx, ctx.tokens, h);
    for (int s = 1; s < S; ++s)                                               // every copy starts as the embedding's output
        ops::cuda_check(cudaMemcpyAsync(h + s * ctx.stream_stride, h, static_cast<size_t>(ctx.T) * hid * sizeof(float), cudaMemcpyDeviceToDevice, ctx.stream),
                        "copying the residual stream");
    void* pending = nullptr;
    for (size_t run = 0; run < plan.schedule.size(); ++run) {
        ctx.run = static_cast<int>(run);
        ctx.state_offset = 0;
        pending = layers[plan.schedule[run].layer].block->forward(ctx, h, pending);
        if (dump_stream_path() && !ctx.capturing) {
            if (pending && ctx.pending_mix) {        // (written into the copies now, so that the dumped rows hold it)
                ops::streams_step(h, ctx, pending, ctx.pending_mix, ctx.pending_out, nullptr, nullptr, 0.f, nullptr);
                ctx.give(pending);
                pending = nullptr;
                ctx.pending_mix = ctx.pending_out = nullptr;
            }
            dump_stream(ctx, h, pending != nullptr);
        }
    }
    ctx.run = -1;
    if (pending && ctx.pending_mix) {                // the last layer's result still has to be written into the copies of the stream
        ops::streams_step(h, ctx, pending, ctx.pending_mix, ctx.pending_out, nullptr, nullptr, 0.f, nullptr);
        ctx.give(pending);
        pending = nullptr;
    }
    ctx.pending_mix = ctx.pending_out = nullptr;
    if (S > 1 && ctx.R > 0) ops::streams_sum_rows(h, ctx.stream_stride, S, ctx.logit_rows, ctx.R, static_cast<int>(hid), ctx.stream);   // copy 0 <- the sum, at the wanted rows
    if (pending && ctx.pending_norm_weight) {        // the last layer's norm sits on its output: add its normed delta first
        ops::norm_residual_add(h, pending, hid, ctx.act_dtype, ctx.pending_norm_weight, ctx.pending_norm_eps, ctx.T, static_cast<int>(hid), ctx.stream);
        ctx.give(pending);
        pending = nullptr;
    }
    ctx.pending_norm_weight = nullptr;
    // Final norm and head on the wanted rows (plus `pending`, a product not yet added to the residual stream).  A step that
    // wants no logits (a prompt cut into several steps) has a bucket of its own, so it asks for nothing here.
    if (ctx.R > 0) {
        void* rows = ctx.take(static_cast<long long>(ctx.R_cap) * hid, ctx.act_dtype);
        final_norm->forward(ctx, h, pending, rows, ctx.logit_rows, ctx.R);
        head->forward(ctx, rows, ctx.logits);
        ctx.give(rows);
    }
    ctx.give(pending);
    for (auto& kv : ctx.shared_buffers) ctx.give(kv.second.ptr);      // what runs left for later runs of this step
    ctx.shared_buffers.clear();
    ctx.give(h);
}

WeightTable weight_table(const ModelPlan& plan) { return DecoderModel(plan).weight_table(); }

json::Value read_model_config(const std::string& folder) {
    json::Value data = read_config_json(folder);
    const std::string path = folder + "/model.safetensors";
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return data;
    std::fclose(f);
    json::Value shapes;
    shapes.object();
    for (const auto& kv : load_safetensors(path)) {      // (a mapping of the file: nothing is copied)
        json::Array extents;
        for (long long d : kv.second.shape) extents.emplace_back(d);
        shapes.set(kv.first, json::Value(extents));
    }
    data.set("tensor_shapes", shapes);
    return data;
}

std::shared_ptr<DecoderModel> load_model(const std::string& folder, DType dtype, const std::string& device) {
    const json::Value data = read_config_json(folder);
    const std::string where = folder + "/config.json";
    const PlanFunction plan_of = resolve_architecture(data, where);
    auto model = std::make_shared<DecoderModel>(plan_of(read_model_config(folder), where));
    model->config = data;
    const HostTensors tensors = load_weights(folder, model->weight_table());
    const int dev = require_cuda(device);          // one clear refusal before the first tensor moves: there is no CPU fallback
    cudaStream_t stream = nullptr;
    ops::cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "creating a stream");
    try {
        model->bind(tensors, dtype, dev, stream);
    } catch (...) {
        cudaStreamDestroy(stream);
        throw;
    }
    cudaStreamDestroy(stream);
    return model;
}

}  // namespace vmb
