// Windowed attention with a learned bias by distance and a few first tokens that stay visible: the preparation of a step's
// queries, keys and values, and the plain kernel (float32 arithmetic, any sizes).
//
//   q_h <- q_h / rms(q_h) * wq,  k_g <- k_g / rms(k_g) * wk          per head, one weight vector for all heads
//   v   <- (1 - lambda) v + lambda v_first                            optional: the values of an earlier layer blended in
//   score(i, j) = scale q_i . k_j + rel[bucket(i - j), h]             bucket: a table from the distance to a row of `rel`
//   i sees j  iff  j <= i and (i - j < window  or  j < keep_first)    window 0: every earlier key
//   out_i = softmax_j(score) v_j
//
// Keys have `Dk` values per head and values `Dv`; the paged cache keeps them in pools of their own
// (k [n_pages, Hkv, VM_PAGE_TOKENS, Dk], v [n_pages, Hkv, VM_PAGE_TOKENS, Dv]).  The distance table `bucket_of` has
// `far + 1` entries; every distance beyond `far` reads the last one.
//
// In the plain kernel a warp owns a (token, query head); keys are walked in chunks of 32 that start at absolute multiples
// of 32, one key per lane, and every dot product is summed in index order by one lane: the result for a position does not
// depend on how the tokens were cut into steps or on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int PREP_WARPS = 4;

// One block per token; its warps take the token's H query heads, Hkv key heads and Hkv value heads in turn.
template <typename T>
__global__ void qkv_prepare_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                   const float* __restrict__ lambda, const T* __restrict__ v_first, T* __restrict__ v_keep,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                   int max_blocks, T* __restrict__ kpages, T* __restrict__ vpages, int H, int Hkv, int Dk, int Dv, int n_pages,
                                   int* __restrict__ err) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int pos = positions[t], seq = seq_of_token[t];
    const int blk = pos / VM_PAGE_TOKENS, in_page = pos % VM_PAGE_TOKENS;
    int page = -1;
    if (kpages) {
        page = blk < max_blocks ? block_table[(size_t)seq * max_blocks + blk] : -1;
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0 && err) atomicExch(err, VM_ERRWORD_CACHE_WRITE);
            page = -1;
        }
    }
    T* row = qkv + (size_t)t * ld;
    const float lam = lambda ? lambda[0] : 0.f;
    for (int item = warp; item < H + 2 * Hkv; item += PREP_WARPS) {
        if (item < H + Hkv) {
            const bool is_q = item < H;
            T* head = row + (size_t)item * Dk;                    // q heads, then k heads, lie side by side
            const float* w = is_q ? wq : wk;
            float ss = 0.f;
            for (int d = lane; d < Dk; d += 32) { const float x = vm_to_float(head[d]); ss += x * x; }
            ss = vm_warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)Dk + eps);
            T* dst = head;
            if (!is_q) {
                if (page < 0) continue;
                dst = kpages + (((size_t)page * Hkv + (item - H)) * VM_PAGE_TOKENS + in_page) * Dk;
            }
            for (int d = lane; d < Dk; d += 32) dst[d] = vm_from_float<T>(vm_to_float(head[d]) * inv * (w ? w[d] : 1.0f));
        } else {
            const int g = item - H - Hkv;
            const T* v = row + (size_t)(H + Hkv) * Dk + (size_t)g * Dv;
            T* dst = page >= 0 ? vpages + (((size_t)page * Hkv + g) * VM_PAGE_TOKENS + in_page) * Dv : nullptr;
            for (int d = lane; d < Dv; d += 32) {
                float x = vm_to_float(v[d]);
                if (v_keep) v_keep[((size_t)t * Hkv + g) * Dv + d] = v[d];
                if (v_first) x = (1.0f - lam) * x + lam * vm_to_float(v_first[((size_t)t * Hkv + g) * Dv + d]);
                if (dst) dst[d] = vm_from_float<T>(x);
            }
        }
    }
}

constexpr int ATT_WARPS = 4;

template <typename T, int EPL>
__global__ void attn_biased_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ kpages, const T* __restrict__ vpages,
                                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token, const float* __restrict__ rel, const int* __restrict__ bucket_of, int far,
                                   T* __restrict__ out, int n_tokens, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first,
                                   int n_pages, const float* __restrict__ sink, int v_stride, int* __restrict__ err) {
    extern __shared__ float qs_all[];                       // ATT_WARPS x Dk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * ATT_WARPS + warp;
    if (w >= (long long)n_tokens * H) return;
    const int t = (int)(w / H), h = (int)(w - (long long)t * H);
    const int hk = h / (H / Hkv);
    const int pos = positions[t], seq = seq_of_token[t];
    float* qs = qs_all + warp * Dk;
    const T* qrow = q + (size_t)t * q_row_stride + (size_t)h * Dk;
    for (int d = lane; d < Dk; d += 32) qs[d] = vm_to_float(qrow[d]) * scale;
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;      // the window is [lo, pos]
    const int kept = min(keep_first, lo);                                             // keys [0, kept) are seen although outside it
    const int first_window_chunk = (lo / 32) * 32;
    float m = -INFINITY, l = 0.f;
    float acc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[i] = 0.f;

    for (int base = 0; base <= pos; base += 32) {
        if (base >= kept && base < first_window_chunk) { base = first_window_chunk - 32; continue; }      // nothing to see in between
        const int blk = base / VM_PAGE_TOKENS;
        const int page = (blk < max_blocks) ? block_table[(size_t)seq * max_blocks + blk] : -1;
        if (page < 0 || page >= n_pages) {                 // a page the step needs is not there: report, skip
            if (lane == 0 && err) atomicExch(err, VM_ERRWORD_CACHE_READ);
            continue;
        }
        const size_t tok0 = ((size_t)page * Hkv + hk) * VM_PAGE_TOKENS + (base % VM_PAGE_TOKENS);
        const int j = base + lane;
        const bool valid = j <= pos && (j >= lo || j < kept);
        float s = -INFINITY;
        if (valid) {
            const T* krow = kpages + (tok0 + lane) * Dk;
            float a = 0.f;
            for (int d = 0; d < Dk; ++d) a = fmaf(qs[d], vm_to_float(krow[d]), a);
            if (rel) a += rel[(size_t)bucket_of[min(pos - j, far)] * H + h];
            s = a;
        }
        const float m_new = fmaxf(m, vm_warp_max(s));
        if (m_new == -INFINITY) continue;                  // a chunk of kept tokens may hold none this query sees
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);               // m == -inf on the first chunk: alpha = 0
        l = l * alpha + vm_warp_sum(p);
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] *= alpha;
        const int cnt = min(32, pos - base + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj == 0.f) continue;                       // (the same for every lane)
            const T* vrow = vpages + (tok0 + jj) * v_stride;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int d = lane + 32 * i;
                if (d < Dv) acc[i] = fmaf(pj, vm_to_float(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    float keep = 1.0f;
    if (sink) {                                            // one more term of the denominator: exp(sink), with no key and no value
        const float sk = sink[h], m_all = fmaxf(m, sk);
        keep = expf(m - m_all);
        l = l * keep + expf(sk - m_all);
    }
    const float inv = keep / l;
    T* orow = out + ((size_t)t * H + h) * Dv;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) orow[d] = vm_from_float<T>(acc[i] * inv);
    }
}

template <typename T>
int launch_biased(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                  const int* positions, const int* seq_of_token, const float* rel, const int* bucket_of, int far, void* out, int n_tokens, int H,
                  int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages, const float* sink, int v_stride, int* err,
                  cudaStream_t stream) {
    const long long warps = (long long)n_tokens * H;
    const int blocks = (int)((warps + ATT_WARPS - 1) / ATT_WARPS);
    const size_t smem = (size_t)ATT_WARPS * Dk * sizeof(float);
    int epl = (Dv + 31) / 32;                    // value columns a lane: 1 to 8, then 12, 16, 24 or 32 (values of up to 1,024)
    if (epl > 8) epl = epl <= 12 ? 12 : epl <= 16 ? 16 : epl <= 24 ? 24 : 32;
#define VM_ATT_CASE(E)                                                                                                                   \
    case E:                                                                                                                              \
        attn_biased_kernel<T, E><<<blocks, ATT_WARPS * 32, smem, stream>>>((const T*)q, q_row_stride, (const T*)kpages, (const T*)vpages, \
                                                                           block_table, max_blocks, positions, seq_of_token, rel,       \
                                                                           bucket_of, far, (T*)out, n_tokens, H, Hkv, Dk, Dv, scale,     \
                                                                           window, keep_first, n_pages, sink, v_stride, err);            \
        break;
    switch (epl) {
        VM_ATT_CASE(1) VM_ATT_CASE(2) VM_ATT_CASE(3) VM_ATT_CASE(4) VM_ATT_CASE(5) VM_ATT_CASE(6) VM_ATT_CASE(7) VM_ATT_CASE(8)
        VM_ATT_CASE(12) VM_ATT_CASE(16) VM_ATT_CASE(24) VM_ATT_CASE(32)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_ATT_CASE
    return vm_launch_status();
}

}  // namespace

// qkv [T, ld] in the activation dtype: H query heads of Dk, Hkv key heads of Dk, Hkv value heads of Dv, side by side.  Queries are
// normed in place; normed keys and (blended) values go to the cache pages (kpages null: nothing is written, the run reads another's
// cache).  wq / wk float32 [Dk] (null: no weight).  v_first [T, Hkv * Dv] with lambda (a device float): blended into the values;
// v_keep [T, Hkv * Dv]: receives this layer's values as they were projected.
VM_API int vm_qkv_prepare(void* qkv, int ld, const float* wq, const float* wk, float eps, const float* lambda, const void* v_first, void* v_keep,
                          const int* positions, const int* seq_of_token, const int* block_table, int max_blocks, void* kpages, void* vpages, int T,
                          int H, int Hkv, int Dk, int Dv, int n_pages, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || Dk <= 0 || Dv <= 0 || ld < (H + Hkv) * Dk + Hkv * Dv) return VM_ERR_BAD_ARG;
    if ((v_first != nullptr) != (lambda != nullptr)) return VM_ERR_BAD_ARG;
    if (act_dtype == VM_F32)
        vm_launch_pdl(qkv_prepare_kernel<float>, dim3(T), dim3(PREP_WARPS * 32), 0, stream, (float*)qkv, ld, wq, wk, eps, lambda, (const float*)v_first,
                      (float*)v_keep, positions, seq_of_token, block_table, max_blocks, (float*)kpages, (float*)vpages, H, Hkv, Dk, Dv, n_pages, err);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(qkv_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(PREP_WARPS * 32), 0, stream, (__nv_bfloat16*)qkv, ld, wq, wk, eps, lambda,
                      (const __nv_bfloat16*)v_first, (__nv_bfloat16*)v_keep, positions, seq_of_token, block_table, max_blocks, (__nv_bfloat16*)kpages,
                      (__nv_bfloat16*)vpages, H, Hkv, Dk, Dv, n_pages, err);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// q: [n_tokens, H, Dk] rows with stride q_row_stride elements; out: [n_tokens, H * Dv] contiguous.  rel float32 [rows, H] with
// bucket_of int32 [far + 1] (both null: no bias).
VM_API int vm_attention_biased_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                                       const int* positions, const int* seq_of_token, const float* rel, const int* bucket_of, int far, void* out,
                                       int n_tokens, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages,
                                       int act_dtype, int* err, cudaStream_t stream) {
    return vm_attention_sink_generic(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, seq_of_token, rel, bucket_of, far, nullptr, 0, out,
                                     n_tokens, H, Hkv, Dk, Dv, scale, window, keep_first, n_pages, act_dtype, err, stream);
}

// The same with a sink and values that may lie inside the key rows.  sink float32 [H] (null: none): exp(sink[h]) is one more term
// of head h's softmax denominator, without a key or a value, not scaled.  v_row_stride: elements from one token's value row to the
// next in `vpages` (0: Dv); with vpages == kpages and v_row_stride == Dk a token's value is the first Dv values of its key row.
VM_API int vm_attention_sink_generic(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                                     const int* positions, const int* seq_of_token, const float* rel, const int* bucket_of, int far, const float* sink,
                                     int v_row_stride, void* out, int n_tokens, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first,
                                     int n_pages, int act_dtype, int* err, cudaStream_t stream) {
    const int v_stride = v_row_stride > 0 ? v_row_stride : Dv;
    if (v_stride < Dv) return VM_ERR_BAD_ARG;
    if (n_tokens <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || Dk <= 0 || Dk > 2048 || Dv <= 0 || Dv > 1024 || window < 0 || keep_first < 0) return VM_ERR_UNSUPPORTED;
    if ((rel != nullptr) != (bucket_of != nullptr) || (rel && far < 0)) return VM_ERR_BAD_ARG;
    if (act_dtype == VM_F32)
        return launch_biased<float>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, seq_of_token, rel, bucket_of, far, out, n_tokens, H,
                                    Hkv, Dk, Dv, scale, window, keep_first, n_pages, sink, v_stride, err, stream);
    if (act_dtype == VM_BF16)
        return launch_biased<__nv_bfloat16>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, seq_of_token, rel, bucket_of, far, out,
                                            n_tokens, H, Hkv, Dk, Dv, scale, window, keep_first, n_pages, sink, v_stride, err, stream);
    return VM_ERR_UNSUPPORTED;
}
