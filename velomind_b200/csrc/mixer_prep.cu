// What lies between the projections of an attention mixer and its attention kernel, and between that kernel and the output
// projection, for mixers whose options are arguments:
//
//   row = [q | k | v] projected (float32), plus an optional bias per column
//   row <- short causal convolution over time per channel (taps [C, K]; the K - 1 last projected rows of a sequence are kept)
//   values that are the keys: v = k as it leaves the convolution
//   q, k <- RMS norm over the WHOLE projection (all heads at once) with a weight per column
//   q, k <- rotary positions on the first rotary_dim values of every head, either pairing, angles in float32
//   q -> its own buffer (activation dtype); k, v -> the sequence's cache page
//
// and afterwards: a sigmoid gate per value or per head on the heads' outputs; a bias on rows; the joining of two mixers' results.
// Everything here is float32 arithmetic; only what is stored is rounded.
#include "common.cuh"

constexpr int PREP_MAX_TAPS = 16;

template <typename T>
__global__ void mixer_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias, const float* __restrict__ taps, int K,
                                     float* __restrict__ state, long long state_stride, int state_offset, const float* __restrict__ q_norm,
                                     const float* __restrict__ k_norm, float eps, const float* __restrict__ inv_freq, int rotary_dim, int pairing,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ slots, const int* __restrict__ block_table, int max_blocks, T* __restrict__ q_out,
                                     T* __restrict__ kpages, T* __restrict__ vpages, int n_pages, int H, int G, int Dk, int Dv, int values_are_keys,
                                     int keep_here, int* __restrict__ err) {
    extern __shared__ float row[];           // C floats: q heads, k heads, v heads
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t], seq = seq_of_token[t];
    const int nq = H * Dk, nk = G * Dk, nv = values_are_keys ? 0 : G * Dv;
    const int C = nq + nk + nv;
    const int first = cu_tokens[seq];                     // the step's first token of this sequence, at place pos - (t - first)
    float* kept = (K > 1 && state) ? state + (size_t)slots[seq] * state_stride + state_offset : nullptr;      // [K - 1, C]: the rows before the step
    // 1. bias and convolution
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float b = bias ? bias[c] : 0.f;
        float v;
        if (K >= 1 && taps) {
            v = 0.f;
            for (int j = 0; j < K; ++j) {
                const int back = K - 1 - j;               // tap j weighs the token `back` places before this one
                if (pos - back < 0) continue;             // nothing lies before a sequence's start
                float u;
                if (t - back >= first) u = proj[(size_t)(t - back) * ld + c];
                else u = kept[(size_t)((K - 1) - (back - (t - first))) * C + c];      // row K - 1 - d holds the token d places before the step
                v = fmaf(taps[(size_t)c * K + j], u + b, v);
            }
        } else {
            v = proj[(size_t)t * ld + c] + b;
        }
        row[c] = v;
    }
    __syncthreads();
    // where this token's key and value go
    int page = -1;
    const int blk = pos / VM_PAGE_TOKENS, in_page = pos % VM_PAGE_TOKENS;
    if (kpages) {
        page = blk < max_blocks ? block_table[(size_t)seq * max_blocks + blk] : -1;
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0 && err) atomicExch(err, VM_ERRWORD_CACHE_WRITE);
            page = -1;
        }
    }
    // 2. values: the keys as they left the convolution, or the row's own value columns
    if (page >= 0 && vpages) {
        const float* src = values_are_keys ? row + nq : row + nq + nk;
        for (int c = threadIdx.x; c < G * Dv; c += blockDim.x) {
            const int g = c / Dv, d = c - g * Dv;
            vpages[(((size_t)page * G + g) * VM_PAGE_TOKENS + in_page) * Dv + d] = vm_from_float<T>(src[c]);
        }
    }
    // the kept rows move on by this token (a step of one token per sequence: no other block reads or writes them)
    if (keep_here && kept) {
        float old[PREP_MAX_TAPS];
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            for (int j = 1; j < K - 1; ++j) old[j] = kept[(size_t)j * C + c];
            for (int j = 1; j < K - 1; ++j) kept[(size_t)(j - 1) * C + c] = old[j];
            kept[(size_t)(K - 2) * C + c] = proj[(size_t)t * ld + c];
        }
    }
    // 3. norm over the whole projection
    if (q_norm) {
        __syncthreads();
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < nq; c += blockDim.x) sq += row[c] * row[c];
        for (int c = threadIdx.x; c < nk; c += blockDim.x) sk += row[nq + c] * row[nq + c];
        sq = vm_block_sum(sq, red);
        sk = vm_block_sum(sk, red);
        const float iq = 1.0f / sqrtf(sq / (float)nq + eps), ik = 1.0f / sqrtf(sk / (float)nk + eps);
        __syncthreads();
        for (int c = threadIdx.x; c < nq + nk; c += blockDim.x) row[c] = c < nq ? row[c] * iq * q_norm[c] : row[c] * ik * k_norm[c - nq];
    }
    __syncthreads();
    // 4. rotary positions on q and k heads, in place (a thread per pair)
    if (inv_freq && rotary_dim > 0) {
        const int half = rotary_dim / 2;
        for (int p = threadIdx.x; p < (H + G) * half; p += blockDim.x) {
            const int head = p / half, i = p - head * half;
            float* x = row + (size_t)head * Dk;
            const int a = pairing == VM_PAIR_INTERLEAVED ? 2 * i : i, b = pairing == VM_PAIR_INTERLEAVED ? 2 * i + 1 : i + half;
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float u = x[a], v = x[b];
            x[a] = u * cs - v * sn;
            x[b] = v * cs + u * sn;
        }
        __syncthreads();
    }
    // 5. out
    for (int c = threadIdx.x; c < nq; c += blockDim.x) q_out[(size_t)t * nq + c] = vm_from_float<T>(row[c]);
    if (page >= 0)
        for (int c = threadIdx.x; c < nk; c += blockDim.x) {
            const int g = c / Dk, d = c - g * Dk;
            kpages[(((size_t)page * G + g) * VM_PAGE_TOKENS + in_page) * Dk + d] = vm_from_float<T>(row[nq + c]);
        }
}

// the kept rows of every sequence move on by the step's tokens: row K - 1 - d holds the projected row d places before the next step
__global__ void mixer_keep_rows_kernel(const float* __restrict__ proj, int ld, int C, int K, float* __restrict__ state, long long state_stride,
                                       int state_offset, const int* __restrict__ cu_tokens, const int* __restrict__ slots) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int seq = blockIdx.x;
    const int first = cu_tokens[seq], n = cu_tokens[seq + 1] - first;
    if (n <= 0) return;
    float* kept = state + (size_t)slots[seq] * state_stride + state_offset;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float nw[PREP_MAX_TAPS];
        for (int j = 0; j < K - 1; ++j) {                // new row j: the token K - 1 - j places before the next step
            const int d = K - 1 - j;                      // 1 .. K - 1
            nw[j] = d <= n ? proj[(size_t)(first + n - d) * ld + c] : kept[(size_t)(j + n) * C + c];
        }
        for (int j = 0; j < K - 1; ++j) kept[(size_t)j * C + c] = nw[j];
    }
}

// proj float32 [T, ld]: columns [0, H Dk) queries, then G Dk keys, then (unless the values are the keys) G Dv values; bias float32 [C]
// or null; taps float32 [C, K] or null (K taps; the K - 1 rows kept per sequence lie in state [slot, state_stride] at state_offset);
// q_norm [H Dk], k_norm [G Dk] or both null; inv_freq [rotary_dim / 2] or null.  q_out [T, H Dk] and the pages in the activation dtype.
VM_API int vm_mixer_prepare(const float* proj, int ld, const float* bias, const float* taps, int K, float* state, long long state_stride,
                            int state_offset, const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rotary_dim, int pairing,
                            const int* positions, const int* seq_of_token, const int* cu_tokens, const int* slots, const int* block_table,
                            int max_blocks, void* q_out, void* kpages, void* vpages, int n_pages, int T, int B, int H, int G, int Dk, int Dv,
                            int values_are_keys, int one_token_each, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || Dk <= 0 || Dv <= 0 || (values_are_keys && Dv != Dk)) return VM_ERR_BAD_ARG;
    if (taps && (K < 1 || K > PREP_MAX_TAPS || (K > 1 && !state))) return VM_ERR_BAD_ARG;
    if ((q_norm != nullptr) != (k_norm != nullptr)) return VM_ERR_BAD_ARG;
    if (inv_freq && (rotary_dim < 0 || rotary_dim > Dk || rotary_dim % 2)) return VM_ERR_BAD_ARG;
    if (!taps) K = 0;
    const int C = (H + G) * Dk + (values_are_keys ? 0 : G * Dv);
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 160 * 1024) return VM_ERR_UNSUPPORTED;
    const int threads = C >= 2048 ? 512 : 256;
    const int keep_here = (one_token_each && K > 1) ? 1 : 0;
    cudaError_t e = cudaSuccess;
    if (act_dtype == VM_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(mixer_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        vm_launch_pdl(mixer_prepare_kernel<float>, dim3(T), dim3(threads), smem, stream, proj, ld, bias, taps, K, state, state_stride, state_offset, q_norm,
                      k_norm, eps, inv_freq, rotary_dim, pairing, positions, seq_of_token, cu_tokens, slots, block_table, max_blocks, (float*)q_out,
                      (float*)kpages, (float*)vpages, n_pages, H, G, Dk, Dv, values_are_keys, keep_here, err);
    } else if (act_dtype == VM_BF16) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(mixer_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        vm_launch_pdl(mixer_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, proj, ld, bias, taps, K, state, state_stride, state_offset,
                      q_norm, k_norm, eps, inv_freq, rotary_dim, pairing, positions, seq_of_token, cu_tokens, slots, block_table, max_blocks,
                      (__nv_bfloat16*)q_out, (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, n_pages, H, G, Dk, Dv, values_are_keys, keep_here, err);
    } else return VM_ERR_UNSUPPORTED;
    int st = vm_launch_status();
    if (st || K <= 1 || keep_here) return st;
    vm_launch_pdl(mixer_keep_rows_kernel, dim3(B, (C + 255) / 256 > 8 ? 8 : (C + 255) / 256), dim3(256), 0, stream, proj, ld, C, K, state, state_stride,
                  state_offset, cu_tokens, slots);
    return vm_launch_status();
}

// ------------------------------------------------------------------------------------------------ gates, biases, joins
// x[t, c] *= sigmoid(g[t, c / per]) with g float32 rows of stride ldg: per = 1 gates every value alone, per = Dv a whole head
template <typename T>
__global__ void sigmoid_gate_heads_kernel(T* __restrict__ x, const float* __restrict__ g, int ldg, int cols, int per, long long n) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols;
        const int c = (int)(i - t * cols);
        const float z = g[t * ldg + c / per];
        x[i] = vm_from_float<T>(vm_to_float(x[i]) / (1.0f + expf(-z)));
    }
}

VM_API int vm_sigmoid_gate_heads(void* x, const float* g, int ldg, int T, int cols, int per, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (cols <= 0 || per <= 0) return VM_ERR_BAD_ARG;
    const long long n = (long long)T * cols, want = (n + 255) / 256;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    if (act_dtype == VM_F32) vm_launch_pdl(sigmoid_gate_heads_kernel<float>, dim3(grid), dim3(256), 0, stream, (float*)x, g, ldg, cols, per, n);
    else if (act_dtype == VM_BF16) vm_launch_pdl(sigmoid_gate_heads_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (__nv_bfloat16*)x, g, ldg, cols, per, n);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// out[t, :] = ca * f(a[t, :]) + cb * f(b[t, :]); f is the identity, or (wa, wb given) the RMS norm over the row with that weight.
// `bias_a` (float32 [cols] or null) is added to a's rows first.  One block per token.
template <typename T>
__global__ void join_rows_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ bias_a, float ca, float cb,
                                 const float* __restrict__ wa, const float* __restrict__ wb, float eps, T* __restrict__ out, int cols) {
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const size_t t = blockIdx.x;
    float ia = 1.f, ib = 1.f;
    if (wa) {
        float sa = 0.f, sb = 0.f;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float x = vm_to_float(a[t * cols + i]) + (bias_a ? bias_a[i] : 0.f), y = b ? vm_to_float(b[t * cols + i]) : 0.f;
            sa += x * x;
            sb += y * y;
        }
        sa = vm_block_sum(sa, red);
        sb = vm_block_sum(sb, red);
        ia = 1.0f / sqrtf(sa / (float)cols + eps);
        ib = 1.0f / sqrtf(sb / (float)cols + eps);
    }
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float x = (vm_to_float(a[t * cols + i]) + (bias_a ? bias_a[i] : 0.f)) * ia * ca;
        if (wa) x *= wa[i];
        if (b) {
            float y = vm_to_float(b[t * cols + i]) * ib * cb;
            if (wb) y *= wb[i];
            x += y;
        }
        out[t * cols + i] = vm_from_float<T>(x);
    }
}

__device__ __forceinline__ float4 jr_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 jr_load4(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void jr_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void jr_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

// the same for rows of 4 n values up to 4,096: every thread keeps up to four runs of four values of both rows in registers
constexpr int JR_THREADS = 256, JR_RUNS = 4;
template <typename T>
__global__ void __launch_bounds__(JR_THREADS)
join_rows_vec_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ bias_a, float ca, float cb,
                     const float* __restrict__ wa, const float* __restrict__ wb, float eps, T* __restrict__ out, int cols) {
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const size_t t = blockIdx.x;
    float4 x[JR_RUNS], y[JR_RUNS];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int c = 0; c < JR_RUNS; ++c) {
        const int i = (threadIdx.x + c * JR_THREADS) * 4;
        x[c] = y[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i >= cols) continue;
        x[c] = jr_load4(a + t * cols + i);
        if (bias_a) {
            const float4 bb = *reinterpret_cast<const float4*>(bias_a + i);
            x[c].x += bb.x; x[c].y += bb.y; x[c].z += bb.z; x[c].w += bb.w;
        }
        if (b) y[c] = jr_load4(b + t * cols + i);
        sa += x[c].x * x[c].x + x[c].y * x[c].y + x[c].z * x[c].z + x[c].w * x[c].w;
        sb += y[c].x * y[c].x + y[c].y * y[c].y + y[c].z * y[c].z + y[c].w * y[c].w;
    }
    float ia = ca, ib = cb;
    if (wa) {
        sa = vm_block_sum(sa, red);
        sb = vm_block_sum(sb, red);
        ia = ca / sqrtf(sa / (float)cols + eps);
        ib = cb / sqrtf(sb / (float)cols + eps);
    }
#pragma unroll
    for (int c = 0; c < JR_RUNS; ++c) {
        const int i = (threadIdx.x + c * JR_THREADS) * 4;
        if (i >= cols) continue;
        float4 r = make_float4(x[c].x * ia, x[c].y * ia, x[c].z * ia, x[c].w * ia);
        if (wa) {
            const float4 w = *reinterpret_cast<const float4*>(wa + i);
            r.x *= w.x; r.y *= w.y; r.z *= w.z; r.w *= w.w;
        }
        if (b) {
            float4 q = make_float4(y[c].x * ib, y[c].y * ib, y[c].z * ib, y[c].w * ib);
            if (wb) {
                const float4 w = *reinterpret_cast<const float4*>(wb + i);
                q.x *= w.x; q.y *= w.y; q.z *= w.z; q.w *= w.w;
            }
            r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
        }
        jr_store4(out + t * cols + i, r);
    }
}

// b null: out = ca * (a + bias_a) alone (a bias on rows, in place if out == a)
VM_API int vm_join_rows(const void* a, const void* b, const float* bias_a, float ca, float cb, const float* wa, const float* wb, float eps, void* out,
                        int T, int cols, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (cols <= 0 || (b && (wa != nullptr) != (wb != nullptr))) return VM_ERR_BAD_ARG;
    if (act_dtype != VM_F32 && act_dtype != VM_BF16) return VM_ERR_UNSUPPORTED;
    if (cols % 4 == 0 && cols >= 128 && cols <= 4 * JR_THREADS * JR_RUNS) {
        if (act_dtype == VM_F32)
            vm_launch_pdl(join_rows_vec_kernel<float>, dim3(T), dim3(JR_THREADS), 0, stream, (const float*)a, (const float*)b, bias_a, ca, cb, wa, wb, eps,
                          (float*)out, cols);
        else
            vm_launch_pdl(join_rows_vec_kernel<__nv_bfloat16>, dim3(T), dim3(JR_THREADS), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, bias_a, ca,
                          cb, wa, wb, eps, (__nv_bfloat16*)out, cols);
        return vm_launch_status();
    }
    const int threads = cols >= 1024 ? 256 : 128;
    if (act_dtype == VM_F32)
        vm_launch_pdl(join_rows_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)a, (const float*)b, bias_a, ca, cb, wa, wb, eps, (float*)out,
                      cols);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(join_rows_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, bias_a, ca, cb,
                      wa, wb, eps, (__nv_bfloat16*)out, cols);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
