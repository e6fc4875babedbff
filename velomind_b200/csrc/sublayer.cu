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
#include <cstdint>

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

// The same for bfloat16 outputs and hid % 4 == 0: a thread makes four neighbouring channels of one token with 16-byte loads (the rows of
// earlier tokens come out of L1 / L2: the step's rows are read from memory once).  KT: the number of taps when it is 2, 3 or 4 (their
// 4 x K weights are K 16-byte loads), 0: any number (scalar loads of the weights).
template <int KT>
__global__ void __launch_bounds__(256)
input_conv_vec_kernel(const float* __restrict__ h, const float* __restrict__ taps, const float* __restrict__ state, long long state_stride,
                      int state_offset, const int* __restrict__ seq_of_token, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                      __nv_bfloat16* __restrict__ out, int hid, int K_any, long long n_vec) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_vec) return;
    const int K = KT ? KT : K_any;
    const int per = hid >> 2;
    const int t = (int)(idx / per), c = (int)(idx - (long long)t * per) << 2;
    const int seq = seq_of_token[t];
    const int in_step = t - cu_tokens[seq];
    const float* kept = state + (size_t)slots[seq] * state_stride + state_offset;
    float tw[KT ? 4 * KT : 4];
    if (KT) {
        const float4* w4 = reinterpret_cast<const float4*>(taps + (size_t)c * K);
#pragma unroll
        for (int q = 0; q < (KT ? KT : 1); ++q) {
            const float4 v = w4[q];
            tw[4 * q] = v.x; tw[4 * q + 1] = v.y; tw[4 * q + 2] = v.z; tw[4 * q + 3] = v.w;
        }
    }
    const float4 x = *reinterpret_cast<const float4*>(h + (size_t)t * hid + c);
    float4 acc;
    if (KT) {
        acc.x = x.x * (1.0f + tw[0 * KT + KT - 1]); acc.y = x.y * (1.0f + tw[1 * KT + KT - 1]);
        acc.z = x.z * (1.0f + tw[2 * KT + KT - 1]); acc.w = x.w * (1.0f + tw[3 * KT + KT - 1]);
    } else {
        acc.x = x.x * (1.0f + taps[(size_t)c * K + K - 1]); acc.y = x.y * (1.0f + taps[(size_t)(c + 1) * K + K - 1]);
        acc.z = x.z * (1.0f + taps[(size_t)(c + 2) * K + K - 1]); acc.w = x.w * (1.0f + taps[(size_t)(c + 3) * K + K - 1]);
    }
#pragma unroll
    for (int j = 0; j < (KT ? KT - 1 : 64); ++j) {
        if (!KT && j >= K - 1) break;
        const int back = K - 1 - j;
        const float* src = back <= in_step ? h + (size_t)(t - back) * hid + c : kept + (size_t)(K - 1 - back + in_step) * hid + c;
        const float4 v = *reinterpret_cast<const float4*>(src);
        if (KT) {
            acc.x = fmaf(tw[0 * KT + j], v.x, acc.x); acc.y = fmaf(tw[1 * KT + j], v.y, acc.y);
            acc.z = fmaf(tw[2 * KT + j], v.z, acc.z); acc.w = fmaf(tw[3 * KT + j], v.w, acc.w);
        } else {
            acc.x = fmaf(taps[(size_t)c * K + j], v.x, acc.x); acc.y = fmaf(taps[(size_t)(c + 1) * K + j], v.y, acc.y);
            acc.z = fmaf(taps[(size_t)(c + 2) * K + j], v.z, acc.z); acc.w = fmaf(taps[(size_t)(c + 3) * K + j], v.w, acc.w);
        }
    }
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc.x, acc.y), o23 = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<const unsigned*>(&o01); o.y = *reinterpret_cast<const unsigned*>(&o23);
    *reinterpret_cast<uint2*>(out + (size_t)t * hid + c) = o;
}

// Many tokens, 2 to 4 taps: a thread makes four neighbouring channels of RUN consecutive tokens and carries the K - 1 earlier rows along in
// registers, so every row of the step is loaded once per thread that needs it as a halo and once as the token itself (K - 1 + RUN loads
// for RUN tokens).  Where the next token belongs to another sequence the carried rows are fetched anew (from the step or the kept rows).
template <int KT, int RUN>
__global__ void __launch_bounds__(256)
input_conv_run_kernel(const float* __restrict__ h, const float* __restrict__ taps, const float* __restrict__ state, long long state_stride,
                      int state_offset, const int* __restrict__ seq_of_token, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                      __nv_bfloat16* __restrict__ out, int hid, int T, long long n_vec) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_vec) return;
    const int per = hid >> 2;
    const int g = (int)(idx / per), c = (int)(idx - (long long)g * per) << 2;
    float tw[4 * KT];
    {
        const float4* w4 = reinterpret_cast<const float4*>(taps + (size_t)c * KT);
#pragma unroll
        for (int q = 0; q < KT; ++q) {
            const float4 v = w4[q];
            tw[4 * q] = v.x; tw[4 * q + 1] = v.y; tw[4 * q + 2] = v.z; tw[4 * q + 3] = v.w;
        }
    }
    float4 win[KT - 1];                      // win[j]: the input KT - 1 - j tokens back
    int seq_before = -1;
#pragma unroll
    for (int i = 0; i < RUN; ++i) {
        const int t = g * RUN + i;
        if (t >= T) break;
        const int seq = seq_of_token[t];
        if (seq != seq_before) {
            const int in_step = t - cu_tokens[seq];
            const float* kept = state + (size_t)slots[seq] * state_stride + state_offset;
#pragma unroll
            for (int j = 0; j < KT - 1; ++j) {
                const int back = KT - 1 - j;
                const float* src = back <= in_step ? h + (size_t)(t - back) * hid + c : kept + (size_t)(KT - 1 - back + in_step) * hid + c;
                win[j] = *reinterpret_cast<const float4*>(src);
            }
            seq_before = seq;
        }
        const float4 x = *reinterpret_cast<const float4*>(h + (size_t)t * hid + c);
        float4 acc;
        acc.x = x.x * (1.0f + tw[0 * KT + KT - 1]); acc.y = x.y * (1.0f + tw[1 * KT + KT - 1]);
        acc.z = x.z * (1.0f + tw[2 * KT + KT - 1]); acc.w = x.w * (1.0f + tw[3 * KT + KT - 1]);
#pragma unroll
        for (int j = 0; j < KT - 1; ++j) {
            acc.x = fmaf(tw[0 * KT + j], win[j].x, acc.x); acc.y = fmaf(tw[1 * KT + j], win[j].y, acc.y);
            acc.z = fmaf(tw[2 * KT + j], win[j].z, acc.z); acc.w = fmaf(tw[3 * KT + j], win[j].w, acc.w);
        }
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc.x, acc.y), o23 = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 o;
        o.x = *reinterpret_cast<const unsigned*>(&o01); o.y = *reinterpret_cast<const unsigned*>(&o23);
        *reinterpret_cast<uint2*>(out + (size_t)t * hid + c) = o;
#pragma unroll
        for (int j = 0; j + 1 < KT - 1; ++j) win[j] = win[j + 1];
        win[KT - 2] = x;
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
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const Y* yr = y + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        const float v = vm_to_float(yr[i]);
        ss += v * v;
    }
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    for (int i = threadIdx.x; i < hid; i += blockDim.x) h[(size_t)t * hid + i] += vm_to_float(yr[i]) * inv * w[i];      // (the row comes out of L1 again)
}

// The same for bfloat16 y with hid % 4 == 0 and ld % 4 == 0: a warp per token, 8-byte loads of y (its second pass finds the row in L1),
// 16-byte updates of h; no block-wide barrier.
constexpr int NR_WARPS = 4;
__global__ void __launch_bounds__(NR_WARPS * 32)
norm_residual_vec_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ y, long long ld, const float* __restrict__ w, int T, int hid, float eps) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x * NR_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const uint2* yr = reinterpret_cast<const uint2*>(y + (size_t)t * ld);
    const int n4 = hid >> 2;
    float ss = 0.f;
    for (int i = lane; i < n4; i += 32) {
        const uint2 d = yr[i];
        const __nv_bfloat162 d01 = *reinterpret_cast<const __nv_bfloat162*>(&d.x), d23 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
        const float a = __low2float(d01), b = __high2float(d01), c = __low2float(d23), e = __high2float(d23);
        ss += a * a + b * b + c * c + e * e;
    }
    ss = vm_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    float4* hr = reinterpret_cast<float4*>(h + (size_t)t * hid);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (int i = lane; i < n4; i += 32) {
        const uint2 d = yr[i];
        const __nv_bfloat162 d01 = *reinterpret_cast<const __nv_bfloat162*>(&d.x), d23 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
        const float4 ww = w4[i];
        float4 v = hr[i];
        v.x += __low2float(d01) * inv * ww.x; v.y += __high2float(d01) * inv * ww.y;
        v.z += __low2float(d23) * inv * ww.z; v.w += __high2float(d23) * inv * ww.w;
        hr[i] = v;
    }
}

// The same sum for steps of one token per sequence, followed by the NEXT sublayer's input convolution on the row just made (a thread owns
// its channel through both): h += rmsnorm(y) * w ; out = h + conv(h) with the kept inputs moved on.  grid (B, ceil(hid / blockDim)): every
// block sums the squares of the token's whole row (a few KB out of L2) and then makes its own blockDim channels, so that a wide row is
// spread over several SMs instead of walked by one block.
template <typename Y, typename T>
__global__ void norm_residual_conv_step_kernel(float* __restrict__ h, const Y* __restrict__ y, long long ld, const float* __restrict__ w, int hid, float eps,
                                               const float* __restrict__ taps, float* __restrict__ state, long long state_stride, int state_offset,
                                               const int* __restrict__ slots, T* __restrict__ out, int K) {
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const bool mine = c < hid;
    // weights are constants: they may be read before the wait on the kernel that makes y
    const float* tw = taps + (size_t)(mine ? c : 0) * K;
    const float wc = mine ? w[c] : 0.f, last = tw[K - 1];
    vm_pdl_wait();
    float* kept = state + (size_t)slots[t] * state_stride + state_offset;
    const Y* yr = y + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hid; i += blockDim.x) {
        const float v = vm_to_float(yr[i]);
        ss += v * v;
    }
    ss = vm_block_sum(ss, red);
    if (!mine) return;
    const float inv = 1.0f / sqrtf(ss / (float)hid + eps);
    const float x = h[(size_t)t * hid + c] + vm_to_float(yr[c]) * inv * wc;
    h[(size_t)t * hid + c] = x;
    float acc = x * (1.0f + last);
    for (int j = 0; j < K - 1; ++j) {
        const float v = kept[(size_t)j * hid + c];
        acc = fmaf(tw[j], v, acc);
        if (j > 0) kept[(size_t)(j - 1) * hid + c] = v;
    }
    if (K > 1) kept[(size_t)(K - 2) * hid + c] = x;
    out[(size_t)t * hid + c] = vm_from_float<T>(acc);
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

// The same in bfloat16 with n % 8 == 0: 16-byte loads and stores, the three sums reduced together.  (z may be out.)
__global__ void __launch_bounds__(256) polynorm_vec_kernel(const __nv_bfloat16* z, const float* __restrict__ coef, __nv_bfloat16* out, int n, float eps) {
    __shared__ float red[3][8];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* zr = reinterpret_cast<const uint4*>(z + (size_t)t * n);
    uint4* orow = reinterpret_cast<uint4*>(out + (size_t)t * n);
    const int n8 = n >> 3;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < n8; i += 256) {
        const uint4 d = zr[i];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a = __low2float(p[k]), b = __high2float(p[k]), a2 = a * a, b2 = b * b;
            s2 += a2 + b2;
            s4 += a2 * a2 + b2 * b2;
            s6 += a2 * a2 * a2 + b2 * b2 * b2;
        }
    }
    s2 = vm_warp_sum(s2); s4 = vm_warp_sum(s4); s6 = vm_warp_sum(s6);
    if (lane == 0) { red[0][warp] = s2; red[1][warp] = s4; red[2][warp] = s6; }
    __syncthreads();
    s2 = s4 = s6 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { s2 += red[0][k]; s4 += red[1][k]; s6 += red[2][k]; }
    const float a = coef[0] / sqrtf(s2 / (float)n + eps), b = coef[1] / sqrtf(s4 / (float)n + eps), c = coef[2] / sqrtf(s6 / (float)n + eps),
                e = coef[3];
    for (int i = threadIdx.x; i < n8; i += 256) {
        const uint4 d = zr[i];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&d);
        uint4 o;
        __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float u = __low2float(p[k]), v = __high2float(p[k]);
            q[k] = __floats2bfloat162_rn(fmaf(u, fmaf(u, fmaf(u, c, b), a), e), fmaf(v, fmaf(v, fmaf(v, c, b), a), e));
        }
        orow[i] = o;
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

// bfloat16, cols % 4 == 0, gate rows 16-byte aligned: four values per thread
__global__ void __launch_bounds__(256) sigmoid_gate_vec_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ gate, long long gate_ld, int cols,
                                                               long long n_vec) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int per = cols >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per;
        const int c = (int)(i - t * per) << 2;
        const float4 g = *reinterpret_cast<const float4*>(gate + t * gate_ld + c);
        uint2* px = reinterpret_cast<uint2*>(x + t * cols + c);
        const uint2 d = *px;
        const __nv_bfloat162 d01 = *reinterpret_cast<const __nv_bfloat162*>(&d.x), d23 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(__low2float(d01) / (1.0f + expf(-g.x)), __high2float(d01) / (1.0f + expf(-g.y)));
        const __nv_bfloat162 o23 = __floats2bfloat162_rn(__low2float(d23) / (1.0f + expf(-g.z)), __high2float(d23) / (1.0f + expf(-g.w)));
        uint2 o;
        o.x = *reinterpret_cast<const unsigned*>(&o01); o.y = *reinterpret_cast<const unsigned*>(&o23);
        *px = o;
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
    const bool aligned = hid % 4 == 0 && state_stride % 4 == 0 && state_offset % 4 == 0 && ((uintptr_t)h | (uintptr_t)taps | (uintptr_t)state) % 16 == 0 &&
                         (uintptr_t)out % 8 == 0;
    if (act_dtype == VM_BF16 && aligned && K >= 2 && K <= 4 && T >= 64) {
        constexpr int RUN = 4;
        const long long n_vec = (long long)((T + RUN - 1) / RUN) * (hid >> 2);
        const dim3 grid((unsigned)((n_vec + 255) / 256));
#define VM_CONV_RUN(KT)                                                                                                                                   \
    vm_launch_pdl(input_conv_run_kernel<KT, RUN>, grid, dim3(256), 0, stream, h, taps, (const float*)state, state_stride, state_offset, seq_of_token, cu_tokens, \
                  slots, (__nv_bfloat16*)out, hid, T, n_vec)
        if (K == 2) VM_CONV_RUN(2);
        else if (K == 3) VM_CONV_RUN(3);
        else VM_CONV_RUN(4);
#undef VM_CONV_RUN
    } else if (act_dtype == VM_BF16 && aligned) {
        const long long n_vec = (long long)T * (hid >> 2);
        const dim3 grid((unsigned)((n_vec + 255) / 256));
#define VM_CONV_VEC(KT)                                                                                                                              \
    vm_launch_pdl(input_conv_vec_kernel<KT>, grid, dim3(256), 0, stream, h, taps, (const float*)state, state_stride, state_offset, seq_of_token, cu_tokens, \
                  slots, (__nv_bfloat16*)out, hid, K, n_vec)
        if (K == 2) VM_CONV_VEC(2);
        else if (K == 3) VM_CONV_VEC(3);
        else if (K == 4) VM_CONV_VEC(4);
        else VM_CONV_VEC(0);
#undef VM_CONV_VEC
    } else if (act_dtype == VM_F32)
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
    const size_t smem = 0;
    if (y_dtype == VM_BF16 && T > 32 && hid % 4 == 0 && ld % 4 == 0 && ((uintptr_t)h | (uintptr_t)w) % 16 == 0 && (uintptr_t)y % 8 == 0) {
        vm_launch_pdl(norm_residual_vec_kernel, dim3((T + NR_WARPS - 1) / NR_WARPS), dim3(NR_WARPS * 32), 0, stream, h, (const __nv_bfloat16*)y, ld, w, T, hid,
                      eps);
        return vm_launch_status();
    }
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
    const size_t smem = 0;
    const dim3 grid(B, (hid + threads - 1) / threads);
    if (y_dtype == VM_F32 && act_dtype == VM_F32)
        vm_launch_pdl(norm_residual_conv_step_kernel<float, float>, grid, dim3(threads), smem, stream, h, (const float*)y, ld, w, hid, eps, taps, state,
                      state_stride, state_offset, slots, (float*)out, K);
    else if (y_dtype == VM_F32 && act_dtype == VM_BF16)
        vm_launch_pdl(norm_residual_conv_step_kernel<float, __nv_bfloat16>, grid, dim3(threads), smem, stream, h, (const float*)y, ld, w, hid, eps, taps,
                      state, state_stride, state_offset, slots, (__nv_bfloat16*)out, K);
    else if (y_dtype == VM_BF16 && act_dtype == VM_BF16)
        vm_launch_pdl(norm_residual_conv_step_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(threads), smem, stream, h, (const __nv_bfloat16*)y, ld, w,
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
    else if (z_dtype == VM_BF16 && act_dtype == VM_BF16 && n % 8 == 0 && ((uintptr_t)z | (uintptr_t)out) % 16 == 0)
        vm_launch_pdl(polynorm_vec_kernel, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)z, coef, (__nv_bfloat16*)out, n, eps);
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
    if (act_dtype == VM_BF16 && cols % 4 == 0 && gate_ld % 4 == 0 && (uintptr_t)gate % 16 == 0 && (uintptr_t)x % 8 == 0) {
        const long long n_vec = n >> 2, want_vec = (n_vec + 255) / 256;
        vm_launch_pdl(sigmoid_gate_vec_kernel, dim3((unsigned)(want_vec < 148 * 16 ? want_vec : 148 * 16)), dim3(256), 0, stream, (__nv_bfloat16*)x, gate,
                      gate_ld, cols, n_vec);
        return vm_launch_status();
    }
    if (act_dtype == VM_F32) vm_launch_pdl(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, gate, gate_ld, cols, n);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, gate, gate_ld, cols, n);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
