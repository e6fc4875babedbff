// Several copies of the residual stream (hyper-connections), and an embedding with a second table read by pairs of tokens.
//
// A model with S copies x_1 .. x_S of the stream (each [T, hid] float32, copy s at h + s * stride) wires a sublayer so:
//     u   = sum_s in[s] x_s                         what the sublayer reads, through its RMS norm
//     x_t <- sum_s mix[s, t] x_s + out[t] * y       every copy at once from the old ones; y is the sublayer's result
// Both steps are float32.  One kernel does a pending write (y given) and the next read (out given) of a token's row in one pass.
#include "common.cuh"

constexpr int HC_MAX_STREAMS = 16;         // copies the plain kernel takes
constexpr int HC_VEC_STREAMS = 8;          // ... and the kernel with 16-byte loads, which keeps a run of every copy in registers

// One block per token.  y [T, hid] in the activation dtype or null; mix float32 [S, S] indexed [from, to]; w_out, w_in float32 [S];
// out [T, hid] (activation dtype) = rmsnorm(u) * norm_w, or null.
template <typename T>
__global__ void streams_step_kernel(float* __restrict__ h, long long stride, int S, const T* __restrict__ y, const float* __restrict__ mix,
                                    const float* __restrict__ w_out, const float* __restrict__ w_in, const float* __restrict__ norm_w, float eps,
                                    T* __restrict__ out, int hid) {
    extern __shared__ float urow[];          // hid floats
    __shared__ float red[32];
    __shared__ float cm[HC_MAX_STREAMS * HC_MAX_STREAMS], co[HC_MAX_STREAMS], ci[HC_MAX_STREAMS];
    if (threadIdx.x < S * S && y) cm[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (y) co[threadIdx.x] = w_out[threadIdx.x];
        if (out) ci[threadIdx.x] = w_in[threadIdx.x];
    }
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    __syncthreads();
    const size_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        float x[HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) x[s] = h[s * stride + t * hid + i];
        if (y) {
            const float yv = vm_to_float(y[t * hid + i]);
            float nx[HC_MAX_STREAMS];
#pragma unroll
            for (int to = 0; to < HC_MAX_STREAMS; ++to)
                if (to < S) {
                    float a = co[to] * yv;
#pragma unroll
                    for (int s = 0; s < HC_MAX_STREAMS; ++s)
                        if (s < S) a = fmaf(cm[s * S + to], x[s], a);
                    nx[to] = a;
                }
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) {
                    x[s] = nx[s];
                    h[s * stride + t * hid + i] = nx[s];
                }
        }
        if (out) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) u = fmaf(ci[s], x[s], u);
            urow[i] = u;
            ss += u * u;
        }
    }
    if (!out) return;
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    for (int i = threadIdx.x; i < hid; i += blockDim.x) out[t * hid + i] = vm_from_float<T>(urow[i] * inv * norm_w[i]);
}

// four neighbouring values of a row in the activation dtype, as float32 and back
__device__ __forceinline__ float4 hc_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 hc_load4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void hc_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void hc_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

// The same for widths that are multiples of 4 up to 4,096: a thread takes up to four runs of four neighbouring values, fetches every copy's
// run with one 16-byte load (all of them in flight before the first sum) and keeps what the norm needs in registers.
constexpr int HC_VEC_THREADS = 256, HC_VEC_RUNS = 4;
template <typename T>
__global__ void __launch_bounds__(HC_VEC_THREADS)
streams_step_vec_kernel(float* __restrict__ h, long long stride, int S, const T* __restrict__ y, const float* __restrict__ mix,
                        const float* __restrict__ w_out, const float* __restrict__ w_in, const float* __restrict__ norm_w, float eps,
                        T* __restrict__ out, int hid) {
    __shared__ float red[32];
    __shared__ float cm[HC_VEC_STREAMS * HC_VEC_STREAMS], co[HC_VEC_STREAMS], ci[HC_VEC_STREAMS];
    if (threadIdx.x < S * S && y) cm[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (y) co[threadIdx.x] = w_out[threadIdx.x];
        if (out) ci[threadIdx.x] = w_in[threadIdx.x];
    }
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    __syncthreads();
    const size_t t = blockIdx.x;
    float4 u[HC_VEC_RUNS];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < HC_VEC_RUNS; ++c) {
        const int i = (threadIdx.x + c * HC_VEC_THREADS) * 4;
        u[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i >= hid) continue;
        float4 x[HC_VEC_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_VEC_STREAMS; ++s)
            if (s < S) x[s] = *reinterpret_cast<const float4*>(h + s * stride + t * hid + i);
        if (y) {
            const float4 yv = hc_load4(y + t * hid + i);
            float4 nx[HC_VEC_STREAMS];
#pragma unroll
            for (int to = 0; to < HC_VEC_STREAMS; ++to)
                if (to < S) {
                    float4 a = make_float4(co[to] * yv.x, co[to] * yv.y, co[to] * yv.z, co[to] * yv.w);
#pragma unroll
                    for (int s = 0; s < HC_VEC_STREAMS; ++s)
                        if (s < S) {
                            const float m = cm[s * S + to];
                            a.x = fmaf(m, x[s].x, a.x); a.y = fmaf(m, x[s].y, a.y); a.z = fmaf(m, x[s].z, a.z); a.w = fmaf(m, x[s].w, a.w);
                        }
                    nx[to] = a;
                }
#pragma unroll
            for (int s = 0; s < HC_VEC_STREAMS; ++s)
                if (s < S) {
                    x[s] = nx[s];
                    *reinterpret_cast<float4*>(h + s * stride + t * hid + i) = nx[s];
                }
        }
        if (out) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < HC_VEC_STREAMS; ++s)
                if (s < S) { a.x = fmaf(ci[s], x[s].x, a.x); a.y = fmaf(ci[s], x[s].y, a.y); a.z = fmaf(ci[s], x[s].z, a.z); a.w = fmaf(ci[s], x[s].w, a.w); }
            u[c] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    if (!out) return;
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
#pragma unroll
    for (int c = 0; c < HC_VEC_RUNS; ++c) {
        const int i = (threadIdx.x + c * HC_VEC_THREADS) * 4;
        if (i >= hid) continue;
        const float4 w = *reinterpret_cast<const float4*>(norm_w + i);
        hc_store4(out + t * hid + i, make_float4(u[c].x * inv * w.x, u[c].y * inv * w.y, u[c].z * inv * w.z, u[c].w * inv * w.w));
    }
}

VM_API int vm_streams_step(float* h, long long stride, int S, const void* y, const float* mix, const float* w_out, const float* w_in,
                           const float* norm_w, float eps, void* out, int T, int hid, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (S < 1 || S > HC_MAX_STREAMS) return VM_ERR_UNSUPPORTED;
    if (hid <= 0 || (y && (!mix || !w_out)) || (out && (!w_in || !norm_w)) || (!y && !out)) return VM_ERR_BAD_ARG;
    if (act_dtype != VM_F32 && act_dtype != VM_BF16) return VM_ERR_UNSUPPORTED;
    if (S <= HC_VEC_STREAMS && hid % 4 == 0 && hid >= 128 && hid <= 4 * HC_VEC_THREADS * HC_VEC_RUNS && stride % 4 == 0) {
        if (act_dtype == VM_F32)
            vm_launch_pdl(streams_step_vec_kernel<float>, dim3(T), dim3(HC_VEC_THREADS), 0, stream, h, stride, S, (const float*)y, mix, w_out, w_in, norm_w,
                          eps, (float*)out, hid);
        else
            vm_launch_pdl(streams_step_vec_kernel<__nv_bfloat16>, dim3(T), dim3(HC_VEC_THREADS), 0, stream, h, stride, S, (const __nv_bfloat16*)y, mix, w_out,
                          w_in, norm_w, eps, (__nv_bfloat16*)out, hid);
        return vm_launch_status();
    }
    const size_t smem = (size_t)hid * sizeof(float);
    if (smem > 48 * 1024) return VM_ERR_UNSUPPORTED;
    const int threads = (hid >= 1024 || S > 8) ? 256 : 128;      // (the block's first S * S threads stage the mixing matrix)
    if (act_dtype == VM_F32)
        vm_launch_pdl(streams_step_kernel<float>, dim3(T), dim3(threads), smem, stream, h, stride, S, (const float*)y, mix, w_out, w_in, norm_w, eps,
                      (float*)out, hid);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(streams_step_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, h, stride, S, (const __nv_bfloat16*)y, mix, w_out, w_in,
                      norm_w, eps, (__nv_bfloat16*)out, hid);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// copy 0 <- the sum of all copies, at the rows named by `rows` (what the final norm reads)
__global__ void streams_sum_rows_kernel(float* __restrict__ h, long long stride, int S, const int* __restrict__ rows, int hid) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const size_t t = rows ? rows[blockIdx.x] : blockIdx.x;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        float a = h[t * hid + i];
        for (int s = 1; s < S; ++s) a += h[s * stride + t * hid + i];
        h[t * hid + i] = a;
    }
}

VM_API int vm_streams_sum_rows(float* h, long long stride, int S, const int* rows, int n_rows, int hid, cudaStream_t stream) {
    if (n_rows <= 0 || S <= 1) return 0;
    vm_launch_pdl(streams_sum_rows_kernel, dim3(n_rows), dim3(128), 0, stream, h, stride, S, rows, hid);
    return vm_launch_status();
}

// ------------------------------------------------------------------------------------------------ embedding with a table of pairs
// out[t] = table[token] + pairs[(previous * mul_prev + token * mul_cur) mod buckets], row `buckets` for a sequence's first token.
// The token before a step's first one is kept per sequence in `last` (an int per slot, at last + slot * last_stride words);
// the thread block of a sequence's last token of the step leaves that token there.  A block that needs the kept token reads it
// before any block can overwrite it only if the two are the same block (one token in the step); otherwise `last` is read here and
// written by vm_embed_pairs_keep, a second launch.
template <typename W>
__global__ void embed_pairs_kernel(const W* __restrict__ table, const W* __restrict__ pairs, const int* __restrict__ tokens,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ cu_tokens,
                                   const int* __restrict__ slots, int* __restrict__ last, long long last_stride, int keep_here, float* __restrict__ out,
                                   int hid, int vocab, long long buckets, long long mul_prev, long long mul_cur, int* __restrict__ err) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t], seq = seq_of_token[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && err) atomicExch(err, VM_ERRWORD_TOKEN_ID);
    long long row = buckets;
    if (positions[t] > 0) {
        const int prev = t > cu_tokens[seq] ? tokens[t - 1] : last[(size_t)slots[seq] * last_stride];
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const W* a = table + (size_t)(ok ? id : 0) * hid;
    const W* b = pairs + (size_t)row * hid;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) out[(size_t)t * hid + i] = ok ? vm_to_float(a[i]) + vm_to_float(b[i]) : 0.f;
    if (keep_here) {                         // one token per sequence: this block alone reads and writes the sequence's word
        __syncthreads();
        if (threadIdx.x == 0) last[(size_t)slots[seq] * last_stride] = id;
    }
}

__global__ void embed_pairs_keep_kernel(const int* __restrict__ tokens, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                                        int* __restrict__ last, long long last_stride, int B) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B && cu_tokens[b + 1] > cu_tokens[b]) last[(size_t)slots[b] * last_stride] = tokens[cu_tokens[b + 1] - 1];
}

// table [vocab, hid] and pairs [buckets + 1, hid] in one dtype; `last`: an int32 word per slot, last_stride words apart
VM_API int vm_embed_pairs(const void* table, const void* pairs, int table_dtype, const int* tokens, const int* positions, const int* seq_of_token,
                          const int* cu_tokens, const int* slots, int* last, long long last_stride, float* out, int T, int B, int hid, int vocab,
                          long long buckets, long long mul_prev, long long mul_cur, int one_token_each, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (buckets <= 0 || !last) return VM_ERR_BAD_ARG;
    const int threads = hid >= 512 ? 256 : 128;
    if (table_dtype == VM_F32)
        vm_launch_pdl(embed_pairs_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, (const float*)pairs, tokens, positions,
                      seq_of_token, cu_tokens, slots, last, last_stride, one_token_each, out, hid, vocab, buckets, mul_prev, mul_cur, err);
    else if (table_dtype == VM_BF16)
        vm_launch_pdl(embed_pairs_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs,
                      tokens, positions, seq_of_token, cu_tokens, slots, last, last_stride, one_token_each, out, hid, vocab, buckets, mul_prev, mul_cur,
                      err);
    else return VM_ERR_UNSUPPORTED;
    int st = vm_launch_status();
    if (st || one_token_each) return st;
    vm_launch_pdl(embed_pairs_keep_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, cu_tokens, slots, last, last_stride, B);
    return vm_launch_status();
}
