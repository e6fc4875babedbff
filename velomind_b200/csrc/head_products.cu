// Per-head matrix products of a step of few tokens (decode), bfloat16 with float32 sums:
//
//     out[t, h, 0:N] = W_h x[t, h, 0:K]          W_h = w + h * w_head, stored [N, K] (rows along the sum) or [K, N]
//
// with what follows such a product in a latent-attention layer taken into the same launch:
//   gate:  out[t, h, n] *= sigmoid(gate[t, h * N + n])                       (float32 gate rows)
//   tail:  out[t, h, N : N + tail] = x[t, h, K : K + tail], its first rotary_dim values turned by the token's position
//          (the rotated part of a query that passes the key up-projection by)
//
// The weights of a head are a few KB and every token of the step needs all of them: a block stages the rows of up to 8 tokens in
// shared memory and reads its share of the head's weights once.
#include <cstdint>

#include "common.cuh"

namespace {

constexpr int HP_TOKENS = 8;

// x rows of the block's tokens and head -> xs[HP_TOKENS][K] float32 (rows past the step's end: zeros)
__device__ __forceinline__ void stage_rows(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_head, int h, int t0, int T, int K, float* xs) {
    for (int i = threadIdx.x; i < HP_TOKENS * K; i += blockDim.x) {
        const int r = i / K, k = i - r * K;
        xs[i] = t0 + r < T ? __bfloat162float(x[(size_t)(t0 + r) * x_ld + (size_t)h * x_head + k]) : 0.f;
    }
}

// the values behind the K that were multiplied: turned in pairs (the first rotary_dim) or passed on
__device__ __forceinline__ void turn_tail(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_head, __nv_bfloat16* __restrict__ out, long long out_ld,
                                          int out_head, int h, int t0, int T, int N, int K, int tail, const int* __restrict__ positions,
                                          const float* __restrict__ inv_freq, int rotary_dim, int pairing) {
    const int half = rotary_dim / 2, per = half + (tail - rotary_dim);
    for (int i = threadIdx.x; i < HP_TOKENS * per; i += blockDim.x) {
        const int r = i / per, j = i - r * per, t = t0 + r;
        if (t >= T) continue;
        const __nv_bfloat16* s = x + (size_t)t * x_ld + (size_t)h * x_head + K;
        __nv_bfloat16* d = out + (size_t)t * out_ld + (size_t)h * out_head + N;
        if (j >= half) {
            d[rotary_dim + (j - half)] = s[rotary_dim + (j - half)];
            continue;
        }
        const int ia = pairing == VM_PAIR_INTERLEAVED ? 2 * j : j, ib = pairing == VM_PAIR_INTERLEAVED ? 2 * j + 1 : j + half;
        float sn, cs;
        sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
        const float u = __bfloat162float(s[ia]), v = __bfloat162float(s[ib]);
        d[ia] = __float2bfloat16_rn(u * cs - v * sn);
        d[ib] = __float2bfloat16_rn(v * cs + u * sn);
    }
}

// W_h stored [K, N]: a thread owns output column n, consecutive threads read consecutive weights.  grid (H, ceil(N / 128), ceil(T / 8)).
__global__ void __launch_bounds__(128)
head_product_kn_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_head, const __nv_bfloat16* __restrict__ w, long long w_head,
                       __nv_bfloat16* __restrict__ out, long long out_ld, int out_head, int T, int N, int K, int tail, const int* __restrict__ positions,
                       const float* __restrict__ inv_freq, int rotary_dim, int pairing) {
    extern __shared__ __align__(16) float xs[];          // [HP_TOKENS][K]
    const int h = blockIdx.x, n = blockIdx.y * 128 + threadIdx.x, t0 = blockIdx.z * HP_TOKENS;
    const __nv_bfloat16* wh = w + (size_t)h * w_head;
    // (weights are constants: they may be asked for before the wait on the kernel that makes x)
    float first = n < N ? __bfloat162float(wh[n]) : 0.f;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    stage_rows(x, x_ld, x_head, h, t0, T, K, xs);
    __syncthreads();
    if (n < N) {
        float acc[HP_TOKENS];
#pragma unroll
        for (int r = 0; r < HP_TOKENS; ++r) acc[r] = 0.f;
        float wk = first;
        for (int k = 0; k < K; ++k) {
            const float nxt = k + 1 < K ? __bfloat162float(wh[(size_t)(k + 1) * N + n]) : 0.f;
#pragma unroll
            for (int r = 0; r < HP_TOKENS; ++r) acc[r] = fmaf(xs[r * K + k], wk, acc[r]);
            wk = nxt;
        }
#pragma unroll
        for (int r = 0; r < HP_TOKENS; ++r)
            if (t0 + r < T) out[(size_t)(t0 + r) * out_ld + (size_t)h * out_head + n] = __float2bfloat16_rn(acc[r]);
    }
    if (tail > 0 && blockIdx.y == 0) turn_tail(x, x_ld, x_head, out, out_ld, out_head, h, t0, T, N, K, tail, positions, inv_freq, rotary_dim, pairing);
}

// The same product with paired columns and the sum split over the block's warps: warp g takes rows g, g + 8, ... of W_h, a lane two
// neighbouring columns (one 4-byte load per row, four rows asked for ahead of their use), and the warps' parts are added in shared
// memory.  Needs N even and 4-byte aligned head matrices.  grid (H, ceil(N / 64), ceil(T / 8)), 8 warps.
constexpr int KN_COLS = 64, KN_GROUPS = 8, KN_AHEAD = 4;
__global__ void __launch_bounds__(KN_GROUPS * 32)
head_product_kn_pairs_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_head, const __nv_bfloat16* __restrict__ w, long long w_head,
                             __nv_bfloat16* __restrict__ out, long long out_ld, int out_head, int T, int N, int K, int tail,
                             const int* __restrict__ positions, const float* __restrict__ inv_freq, int rotary_dim, int pairing) {
    extern __shared__ __align__(16) float xs[];          // [HP_TOKENS][K], then the warps' parts [KN_GROUPS][HP_TOKENS][KN_COLS]
    float* part = xs + HP_TOKENS * K;
    const int h = blockIdx.x, g = threadIdx.x >> 5, lane = threadIdx.x & 31, n0 = blockIdx.y * KN_COLS, n = n0 + 2 * lane, t0 = blockIdx.z * HP_TOKENS;
    const __nv_bfloat16* wh = w + (size_t)h * w_head;
    const bool col = n < N;                              // (N is even: the pair's second column exists with its first)
    // (weights are constants: the first rows may be asked for before the wait on the kernel that makes x)
    __nv_bfloat162 ahead[KN_AHEAD];
#pragma unroll
    for (int u = 0; u < KN_AHEAD; ++u) {
        const int k = g + KN_GROUPS * u;
        ahead[u] = col && k < K ? *reinterpret_cast<const __nv_bfloat162*>(wh + (size_t)k * N + n) : __floats2bfloat162_rn(0.f, 0.f);
    }
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    stage_rows(x, x_ld, x_head, h, t0, T, K, xs);
    __syncthreads();
    float acc[HP_TOKENS][2];
#pragma unroll
    for (int r = 0; r < HP_TOKENS; ++r) acc[r][0] = acc[r][1] = 0.f;
    for (int k0 = g; k0 < K; k0 += KN_GROUPS * KN_AHEAD) {
        float a[KN_AHEAD], b[KN_AHEAD];
#pragma unroll
        for (int u = 0; u < KN_AHEAD; ++u) {
            a[u] = __low2float(ahead[u]);
            b[u] = __high2float(ahead[u]);
            const int k = k0 + KN_GROUPS * (KN_AHEAD + u);
            ahead[u] = col && k < K ? *reinterpret_cast<const __nv_bfloat162*>(wh + (size_t)k * N + n) : __floats2bfloat162_rn(0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < KN_AHEAD; ++u) {
            const int k = k0 + KN_GROUPS * u;
            if (k < K) {
#pragma unroll
                for (int r = 0; r < HP_TOKENS; ++r) {
                    const float xv = xs[r * K + k];
                    acc[r][0] = fmaf(xv, a[u], acc[r][0]);
                    acc[r][1] = fmaf(xv, b[u], acc[r][1]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < HP_TOKENS; ++r)
        *reinterpret_cast<float2*>(part + ((size_t)g * HP_TOKENS + r) * KN_COLS + 2 * lane) = make_float2(acc[r][0], acc[r][1]);
    __syncthreads();
    {   // warp r adds the parts of token t0 + r
        const int r = g, t = t0 + r;
        if (t < T && col) {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int q = 0; q < KN_GROUPS; ++q) {
                const float2 v = *reinterpret_cast<const float2*>(part + ((size_t)q * HP_TOKENS + r) * KN_COLS + 2 * lane);
                s0 += v.x;
                s1 += v.y;
            }
            __nv_bfloat16* o = out + (size_t)t * out_ld + (size_t)h * out_head + n;
            o[0] = __float2bfloat16_rn(s0);
            o[1] = __float2bfloat16_rn(s1);
        }
    }
    if (tail > 0 && blockIdx.y == 0) turn_tail(x, x_ld, x_head, out, out_ld, out_head, h, t0, T, N, K, tail, positions, inv_freq, rotary_dim, pairing);
}

// W_h stored [N, K]: a warp owns output row n and its lanes share the sum.  grid (H, ceil(N / 8), ceil(T / 8)), 8 warps.
__global__ void __launch_bounds__(256)
head_product_nk_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_head, const __nv_bfloat16* __restrict__ w, long long w_head,
                       __nv_bfloat16* __restrict__ out, long long out_ld, int out_head, int T, int N, int K, const float* __restrict__ gate,
                       long long gate_ld) {
    extern __shared__ __align__(16) float xs[];          // [HP_TOKENS][K]
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = blockIdx.y * 8 + warp, t0 = blockIdx.z * HP_TOKENS;
    const __nv_bfloat16* row = w + (size_t)h * w_head + (size_t)min(n, N - 1) * K;
    const bool pairs = (K & 1) == 0 && (((size_t)h * w_head + (size_t)min(n, N - 1) * K) & 1) == 0 && (reinterpret_cast<size_t>(w) & 3) == 0;
    // a lane's first weights, asked for before the wait on the kernel that makes x
    __nv_bfloat162 w01 = __floats2bfloat162_rn(0.f, 0.f);
    if (pairs && 2 * lane < K) w01 = *reinterpret_cast<const __nv_bfloat162*>(row + 2 * lane);
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    stage_rows(x, x_ld, x_head, h, t0, T, K, xs);
    __syncthreads();
    if (n >= N) return;
    float acc[HP_TOKENS];
#pragma unroll
    for (int r = 0; r < HP_TOKENS; ++r) acc[r] = 0.f;
    if (pairs) {
        for (int k = 2 * lane; k < K; k += 64) {
            const float a = __low2float(w01), b = __high2float(w01);
            if (k + 64 < K) w01 = *reinterpret_cast<const __nv_bfloat162*>(row + k + 64);
#pragma unroll
            for (int r = 0; r < HP_TOKENS; ++r) acc[r] = fmaf(xs[r * K + k + 1], b, fmaf(xs[r * K + k], a, acc[r]));
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float a = __bfloat162float(row[k]);
#pragma unroll
            for (int r = 0; r < HP_TOKENS; ++r) acc[r] = fmaf(xs[r * K + k], a, acc[r]);
        }
    }
    float mine = 0.f;
#pragma unroll
    for (int r = 0; r < HP_TOKENS; ++r) {
        const float s = vm_warp_sum(acc[r]);
        if (lane == r) mine = s;
    }
    const int t = t0 + lane;
    if (lane < HP_TOKENS && t < T) {
        if (gate) mine = mine / (1.0f + expf(-gate[(size_t)t * gate_ld + (size_t)h * N + n]));
        out[(size_t)t * out_ld + (size_t)h * out_head + n] = __float2bfloat16_rn(mine);
    }
}

}  // namespace

// x [T, x_ld] with head h's K (+ tail) values at h * x_head; out [T, out_ld] with head h's N (+ tail) values at h * out_head; both
// bfloat16.  k_by_n: the heads' weights are stored [K, N] (else [N, K]); a gate goes with [N, K], a tail with [K, N].
VM_API int vm_head_products_few(const void* x, long long x_ld, int x_head, const void* w, long long w_head, int k_by_n, void* out, long long out_ld,
                                int out_head, int T, int N, int K, int H, const float* gate, long long gate_ld, int tail, const int* positions,
                                const float* inv_freq, int rotary_dim, int pairing, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return 0;
    if (N <= 0 || K <= 0 || tail < 0 || rotary_dim < 0 || rotary_dim % 2 || rotary_dim > tail || (rotary_dim > 0 && (!inv_freq || !positions)))
        return VM_ERR_BAD_ARG;
    if ((gate && k_by_n) || (tail && !k_by_n)) return VM_ERR_UNSUPPORTED;
    const size_t smem = (size_t)HP_TOKENS * K * sizeof(float);
    if (smem > 48 * 1024 || H > 65535) return VM_ERR_UNSUPPORTED;
    const unsigned tiles = (unsigned)((T + HP_TOKENS - 1) / HP_TOKENS);
    const size_t smem_pairs = smem + (size_t)KN_GROUPS * HP_TOKENS * KN_COLS * sizeof(float);
    if (k_by_n && N % 2 == 0 && w_head % 2 == 0 && reinterpret_cast<uintptr_t>(w) % 4 == 0 && smem_pairs <= 48 * 1024)
        vm_launch_pdl(head_product_kn_pairs_kernel, dim3(H, (N + KN_COLS - 1) / KN_COLS, tiles), dim3(KN_GROUPS * 32), smem_pairs, stream,
                      (const __nv_bfloat16*)x, x_ld, x_head, (const __nv_bfloat16*)w, w_head, (__nv_bfloat16*)out, out_ld, out_head, T, N, K, tail, positions,
                      inv_freq, rotary_dim, pairing);
    else if (k_by_n)
        vm_launch_pdl(head_product_kn_kernel, dim3(H, (N + 127) / 128, tiles), dim3(128), smem, stream, (const __nv_bfloat16*)x, x_ld, x_head,
                      (const __nv_bfloat16*)w, w_head, (__nv_bfloat16*)out, out_ld, out_head, T, N, K, tail, positions, inv_freq, rotary_dim, pairing);
    else
        vm_launch_pdl(head_product_nk_kernel, dim3(H, (N + 7) / 8, tiles), dim3(256), smem, stream, (const __nv_bfloat16*)x, x_ld, x_head,
                      (const __nv_bfloat16*)w, w_head, (__nv_bfloat16*)out, out_ld, out_head, T, N, K, gate, gate_ld);
    return vm_launch_status();
}
