// Kernels of a layer whose sublayers read the residual stream itself and whose norm sits on the sublayer's OUTPUT:
//
//   a short causal convolution over time on every channel of what a sublayer reads, added to it:
//       out_t = h_t + sum_j taps[:, j] * h_(t - K + 1 + j)        (zeros before the sequence's start)
//     with the last K - 1 inputs of every sequence kept in a float32 state area from step to step;
//   h += rmsnorm(y) * w, the residual sum of a normed sublayer output;
//   the polynomial activation  a N(z) + b N(z^2) + c N(z^3) + e, N = division of a token's row by its root mean square;
//   rotation of a slice of every head's row (rotary positions on a part of the head), copied to another layout;
//   multiplication by the sigmoid of a gate.
//
// The residual stream is float32; everything here computes in float32 and rounds once on the way out.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------ convolution on the input
// grid (T); a block walks the channels of one token.  state [max_slots, state_stride] float32; this convolution's K - 1 kept
// rows of `hid` channels start at state_offset: row i holds the input at position p0 - (K - 1) + i, p0 the step's first position
// of the sequence.
template <typename T>
__global__ void input_conv_kernel(const float* __restrict__ h, const float* __restrict__ taps, const float* __restrict__ state, long long state_stride,
                                  int state_offset, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                  const int* __restrict__ cu_tokens, const int* __restrict__ slots, T* __restrict__ out, int hid, int K) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = cu_tokens[seq];                    // the sequence's first token of this step
    const int in_step = t - first;                       // tokens of the sequence before this one in the step
    const float* kept = state + (size_t)slots[seq] * state_stride + state_offset;
    (void)positions;
    for (int c = threadIdx.x; c < hid; c += blockDim.x) {
        const float* w = taps + (size_t)c * K;
        float acc = h[(size_t)t * hid + c] * (1.0f + w[K - 1]);
        for (int j = 0; j < K - 1; ++j) {
            const int back = K - 1 - j;                  // how many tokens before t
            const float v = back <= in_step ? h[(size_t)(t - back) * hid + c] : kept[(size_t)(K - 1 - back + in_step) * hid + c];
            acc = fmaf(w[j], v, acc);
        }
        out[(size_t)t * hid + c] = vm_from_float<T>(acc);
    }
}

// grid (B, ceil(hid / threads)); a thread owns one channel of one sequence and moves its K - 1 kept inputs on by the step's tokens.
// Row i of the new state is the input n - (K - 1) + i tokens into the step, or, before the step, row i + n of the old state; rows are
// written in ascending order, so a row is read before it is overwritten.
__global__ void input_conv_keep_kernel(const float* __restrict__ h, float* __restrict__ state, long long state_stride, int state_offset,
                                       const int* __restrict__ cu_tokens, const int* __restrict__ slots, int hid, int K) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int seq = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= hid) return;
    const int first = cu_tokens[seq], n = cu_tokens[seq + 1] - first;
    float* kept = state + (size_t)slots[seq] * state_stride + state_offset;
    for (int i = 0; i < K - 1; ++i) {
        const int at = n - (K - 1) + i;
        float v;
        if (at >= 0) v = h[(size_t)(first + at) * hid + c];
        else v = kept[(size_t)(i + n) * hid + c];
        kept[(size_t)i * hid + c] = v;
    }
}

// one token per sequence: convolution and kept inputs in one pass (a thread owns its channel's kept inputs)
template <typename T>
__global__ void input_conv_step_kernel(const float* __restrict__ h, const float* __restrict__ taps, float* __restrict__ state, long long state_stride,
                                       int state_offset, const int* __restrict__ slots, T* __restrict__ out, int hid, int K) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int seq = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= hid) return;
    float* kept = state + (size_t)slots[seq] * state_stride + state_offset;
    const float* w = taps + (size_t)c * K;
    const float x = h[(size_t)seq * hid + c];
    float acc = x * (1.0f + w[K - 1]);
    for (int j = 0; j < K - 1; ++j) {
        const float v = kept[(size_t)j * hid + c];
        acc = fmaf(w[j], v, acc);
        if (j > 0) kept[(size_t)(j - 1) * hid + c] = v;
    }
    if (K > 1) kept[(size_t)(K - 2) * hid + c] = x;
    out[(size_t)seq * hid + c] = vm_from_float<T>(acc);
}

// ------------------------------------------------------------------------------------------------ h += rmsnorm(y) * w
// one block per token; y float32 or T, rows of ld elements
template <typename Y>
__global__ void norm_residual_kernel(float* __restrict__ h, const Y* __restrict__ y, long long ld, const float* __restrict__ w, int hid, float eps) {
    extern __shared__ float row[];
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const Y* yr = y + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        const float v = vm_to_float(yr[i]);
        row[i] = v;
        ss += v * v;
    }
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    for (int i = threadIdx.x; i < hid; i += blockDim.x) h[(size_t)t * hid + i] += row[i] * inv * w[i];
}

// The same sum for steps of one token per sequence, followed by the NEXT sublayer's input convolution on the row just made (a thread owns
// its channels through both): h += rmsnorm(y) * w ; out = h + conv(h) with the kept inputs moved on.  grid (B).
template <typename Y, typename T>
__global__ void norm_residual_conv_step_kernel(float* __restrict__ h, const Y* __restrict__ y, long long ld, const float* __restrict__ w, int hid, float eps,
                                               const float* __restrict__ taps, float* __restrict__ state, long long state_stride, int state_offset,
                                               const int* __restrict__ slots, T* __restrict__ out, int K) {
    extern __shared__ float row[];
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const Y* yr = y + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        const float v = vm_to_float(yr[i]);
        row[i] = v;
        ss += v * v;
    }
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    float* kept = state + (size_t)slots[t] * state_stride + state_offset;
    for (int c = threadIdx.x; c < hid; c += blockDim.x) {
        const float x = h[(size_t)t * hid + c] + row[c] * inv * w[c];
        h[(size_t)t * hid + c] = x;
        const float* tw = taps + (size_t)c * K;
        float acc = x * (1.0f + tw[K - 1]);
        for (int j = 0; j < K - 1; ++j) {
            const float v = kept[(size_t)j * hid + c];
            acc = fmaf(tw[j], v, acc);
            if (j > 0) kept[(size_t)(j - 1) * hid + c] = v;
        }
        if (K > 1) kept[(size_t)(K - 2) * hid + c] = x;
        out[(size_t)t * hid + c] = vm_from_float<T>(acc);
    }
}

// ------------------------------------------------------------------------------------------------ polynomial activation with unit-rms powers
// one block per token; z [T, n] in Z (float32 or the activation dtype), out in T
template <typename Z, typename T>
__global__ void polynorm_kernel(const Z* z, const float* __restrict__ coef, T* out, int n, float eps) {      // (z may be out)
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const Z* zr = z + (size_t)t * n;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = vm_to_float(zr[i]), v2 = v * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v2 * v2 * v2;
    }
    s2 = vm_block_sum(s2, red);
    s4 = vm_block_sum(s4, red);
    s6 = vm_block_sum(s6, red);
    const float a = coef[0] / sqrtf(s2 / (float)n + eps), b = coef[1] / sqrtf(s4 / (float)n + eps), c = coef[2] / sqrtf(s6 / (float)n + eps),
                e = coef[3];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = vm_to_float(zr[i]);
        out[(size_t)t * n + i] = vm_from_float<T>(fmaf(v, fmaf(v, fmaf(v, c, b), a), e));
    }
}

// ------------------------------------------------------------------------------------------------ rotation of a slice of every head
// dst[t, h, dst_off + i] = rotated src[t, h, src_off + i], i < width: the first rotary_dim values turn by the token's position (pairs by
// `pairing`), the rest pass.  One thread per (token, head, pair or passing value).
template <typename T>
__global__ void rotate_slice_kernel(const T* __restrict__ src, long long src_ld, int src_head, int src_off, T* __restrict__ dst, long long dst_ld,
                                    int dst_head, int dst_off, const int* __restrict__ positions, const float* __restrict__ inv_freq, int rotary_dim,
                                    int pairing, int width, int H, int n_tokens) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int half = rotary_dim / 2, per = half + (width - rotary_dim);
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * H * per) return;
    const int i = (int)(idx % per);
    const int hh = (int)((idx / per) % H);
    const int t = (int)(idx / ((long long)per * H));
    const T* s = src + (size_t)t * src_ld + (size_t)hh * src_head + src_off;
    T* d = dst + (size_t)t * dst_ld + (size_t)hh * dst_head + dst_off;
    if (i >= half) {
        const int k = rotary_dim + (i - half);
        d[k] = s[k];
        return;
    }
    const int ia = pairing == VM_PAIR_INTERLEAVED ? 2 * i : i, ib = pairing == VM_PAIR_INTERLEAVED ? 2 * i + 1 : i + half;
    const float ang = (float)positions[t] * inv_freq[i];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float u = vm_to_float(s[ia]), v = vm_to_float(s[ib]);
    d[ia] = vm_from_float<T>(u * cs - v * sn);
    d[ib] = vm_from_float<T>(v * cs + u * sn);
}

// ------------------------------------------------------------------------------------------------ x *= sigmoid(gate)
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const float* __restrict__ gate, long long gate_ld, int cols, long long n) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols;
        const int c = (int)(i - t * cols);
        const float g = gate[t * gate_ld + c];
        x[i] = vm_from_float<T>(vm_to_float(x[i]) / (1.0f + expf(-g)));
    }
}

}  // namespace

// h float32 [T, hid]; taps float32 [hid, K]; out [T, hid] in the activation dtype.  The kept inputs of every sequence of the step are moved on
// (after the convolution has read them): h must still hold the step's inputs.  one_token_each: token s is sequence s's only one.
VM_API int vm_input_conv(const float* h, const float* taps, float* state, long long state_stride, int state_offset, const int* positions,
                         const int* seq_of_token, const int* cu_tokens, const int* slots, void* out, int T, int B, int hid, int K, int one_token_each,
                         int act_dtype, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (hid <= 0 || K < 1 || K > 64 || (K > 1 && (!state || state_offset < 0 || state_offset + (long long)(K - 1) * hid > state_stride)))
        return VM_ERR_BAD_ARG;
    if (act_dtype != VM_F32 && act_dtype != VM_BF16) return VM_ERR_UNSUPPORTED;
    const int threads = hid >= 512 ? 256 : 128;
    if (one_token_each) {
        if (T != B) return VM_ERR_BAD_ARG;
        const dim3 grid(B, (hid + threads - 1) / threads);
        if (act_dtype == VM_F32)
            vm_launch_pdl(input_conv_step_kernel<float>, grid, dim3(threads), 0, stream, h, taps, state, state_stride, state_offset, slots, (float*)out, hid, K);
        else
            vm_launch_pdl(input_conv_step_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, h, taps, state, state_stride, state_offset, slots,
                          (__nv_bfloat16*)out, hid, K);
        return vm_launch_status();
    }
    if (act_dtype == VM_F32)
        vm_launch_pdl(input_conv_kernel<float>, dim3(T), dim3(threads), 0, stream, h, taps, (const float*)state, state_stride, state_offset, positions,
                      seq_of_token, cu_tokens, slots, (float*)out, hid, K);
    else
        vm_launch_pdl(input_conv_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, h, taps, (const float*)state, state_stride, state_offset,
                      positions, seq_of_token, cu_tokens, slots, (__nv_bfloat16*)out, hid, K);
    int st = vm_launch_status();
    if (st || K == 1) return st;
    vm_launch_pdl(input_conv_keep_kernel, dim3(B, (hid + threads - 1) / threads), dim3(threads), 0, stream, h, state, state_stride, state_offset, cu_tokens,
                  slots, hid, K);
    return vm_launch_status();
}

// h float32 [T, hid] += rmsnorm(y) * w; y [T, ld] float32 (y_dtype VM_F32) or bfloat16
VM_API int vm_norm_residual_add(float* h, const void* y, long long ld, int y_dtype, const float* w, int T, int hid, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hid <= 0 || ld < hid) return VM_ERR_BAD_ARG;
    const int threads = hid >= 512 ? 256 : 128;
    const size_t smem = (size_t)hid * sizeof(float);
    if (smem > 48 * 1024) return VM_ERR_UNSUPPORTED;
    if (y_dtype == VM_F32) vm_launch_pdl(norm_residual_kernel<float>, dim3(T), dim3(threads), smem, stream, h, (const float*)y, ld, w, hid, eps);
    else if (y_dtype == VM_BF16)
        vm_launch_pdl(norm_residual_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, h, (const __nv_bfloat16*)y, ld, w, hid, eps);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// One token per sequence (token s is sequence s's): h += rmsnorm(y) * w, then out = h + conv(h) as vm_input_conv does for such a step,
// the kept inputs at state_offset moved on.  y and out in act_dtype (y_dtype VM_F32: y float32).
VM_API int vm_norm_residual_conv_step(float* h, const void* y, long long ld, int y_dtype, const float* w, int B, int hid, float eps, const float* taps,
                                      float* state, long long state_stride, int state_offset, const int* slots, void* out, int K, int act_dtype,
                                      cudaStream_t stream) {
    if (B <= 0) return 0;
    if (hid <= 0 || ld < hid || K < 1 || K > 64 || (K > 1 && (!state || state_offset < 0 || state_offset + (long long)(K - 1) * hid > state_stride)))
        return VM_ERR_BAD_ARG;
    const int threads = hid >= 512 ? 256 : 128;
    const size_t smem = (size_t)hid * sizeof(float);
    if (smem > 48 * 1024) return VM_ERR_UNSUPPORTED;
    if (y_dtype == VM_F32 && act_dtype == VM_F32)
        vm_launch_pdl(norm_residual_conv_step_kernel<float, float>, dim3(B), dim3(threads), smem, stream, h, (const float*)y, ld, w, hid, eps, taps, state,
                      state_stride, state_offset, slots, (float*)out, K);
    else if (y_dtype == VM_F32 && act_dtype == VM_BF16)
        vm_launch_pdl(norm_residual_conv_step_kernel<float, __nv_bfloat16>, dim3(B), dim3(threads), smem, stream, h, (const float*)y, ld, w, hid, eps, taps,
                      state, state_stride, state_offset, slots, (__nv_bfloat16*)out, K);
    else if (y_dtype == VM_BF16 && act_dtype == VM_BF16)
        vm_launch_pdl(norm_residual_conv_step_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(B), dim3(threads), smem, stream, h, (const __nv_bfloat16*)y, ld, w,
                      hid, eps, taps, state, state_stride, state_offset, slots, (__nv_bfloat16*)out, K);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// out[t, :] = a N(z) + b N(z^2) + c N(z^3) + e over the n values of a token; coef float32 [4] = a, b, c, e; z in z_dtype, out in act_dtype
VM_API int vm_polynorm(const void* z, int z_dtype, const float* coef, void* out, int T, int n, float eps, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n <= 0) return VM_ERR_BAD_ARG;
    const int threads = n >= 1024 ? 512 : (n >= 512 ? 256 : 128);
    if (z_dtype == VM_F32 && act_dtype == VM_F32)
        vm_launch_pdl(polynorm_kernel<float, float>, dim3(T), dim3(threads), 0, stream, (const float*)z, coef, (float*)out, n, eps);
    else if (z_dtype == VM_F32 && act_dtype == VM_BF16)
        vm_launch_pdl(polynorm_kernel<float, __nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const float*)z, coef, (__nv_bfloat16*)out, n, eps);
    else if (z_dtype == VM_BF16 && act_dtype == VM_BF16)
        vm_launch_pdl(polynorm_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)z, coef, (__nv_bfloat16*)out, n,
                      eps);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// rows of H heads: src [T, src_ld] with a head every src_head elements, the slice at src_off; dst likewise (src == dst with equal
// layouts: in place).  The slice's first rotary_dim of `width` values are rotated.
VM_API int vm_rotate_slice(const void* src, long long src_ld, int src_head, int src_off, void* dst, long long dst_ld, int dst_head, int dst_off,
                           const int* positions, const float* inv_freq, int rotary_dim, int pairing, int width, int H, int T, int act_dtype,
                           cudaStream_t stream) {
    if (T <= 0 || width <= 0) return 0;
    if (H <= 0 || rotary_dim < 0 || rotary_dim % 2 || rotary_dim > width || (rotary_dim > 0 && !inv_freq)) return VM_ERR_BAD_ARG;
    const long long n = (long long)T * H * (rotary_dim / 2 + width - rotary_dim);
    const int blocks = (int)((n + 255) / 256);
    if (act_dtype == VM_F32)
        vm_launch_pdl(rotate_slice_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)src, src_ld, src_head, src_off, (float*)dst, dst_ld,
                      dst_head, dst_off, positions, inv_freq, rotary_dim, pairing, width, H, T);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(rotate_slice_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)src, src_ld, src_head, src_off,
                      (__nv_bfloat16*)dst, dst_ld, dst_head, dst_off, positions, inv_freq, rotary_dim, pairing, width, H, T);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// x [T, cols] (activation dtype) *= sigmoid(gate [T, gate_ld] float32, its first `cols` columns)
VM_API int vm_sigmoid_gate(void* x, const float* gate, long long gate_ld, int T, int cols, int act_dtype, cudaStream_t stream) {
    if (T <= 0 || cols <= 0) return 0;
    const long long n = (long long)T * cols;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (act_dtype == VM_F32) vm_launch_pdl(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, gate, gate_ld, cols, n);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, gate, gate_ld, cols, n);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
