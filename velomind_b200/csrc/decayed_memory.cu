// Linear attention with a decaying matrix memory, per sequence and head:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          S [Dk, Dv] float32, zero at a sequence's start, kept per sequence
//     o_t = S_t^T q_t
//
// a_t is one number per head for all tokens and key channels (a fixed decay: retention), or a number per token and key
// channel, a = sigmoid(z)^(1 / tau) from the logits z (gated linear attention).  Queries and keys may be turned by rotary
// positions first (either pairing, the first rotary_dim values of a head) and scaled afterwards.  No softmax, no denominator.
// The output stage divides every head's o by its root mean square (times an optional weight over Dv), multiplies by
// silu(g) and rounds to the activation dtype.  Everything up to that rounding is float32.
#include "common.cuh"

constexpr int DM_WARPS = 8;          // a warp owns a band of key channels, a lane a value column
constexpr int DM_COLS = 32;

// log(a) of key channel i of head h at token t
__device__ __forceinline__ float dm_log_decay(const float* __restrict__ head_log_decay, const float* __restrict__ z, int ldz, float inv_tau, size_t t,
                                              int h, int Dk, int i) {
    if (!z) return head_log_decay[h];
    const float x = z[t * ldz + (size_t)h * Dk + i];
    // log sigmoid(x) = -softplus(-x), stable on both sides
    const float ls = x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
    return ls * inv_tau;
}

// One value of a head's query or key at token t after rotation: x [Dk] float32 is the head's projected row.
__device__ __forceinline__ float dm_turned(const float* __restrict__ x, int i, int pos, const float* __restrict__ inv_freq, int rotary_dim, int pairing) {
    if (!inv_freq || i >= rotary_dim) return x[i];
    const int half = rotary_dim / 2;
    int pair, partner;
    bool first;
    if (pairing == VM_PAIR_INTERLEAVED) { pair = i >> 1; first = (i & 1) == 0; partner = first ? i + 1 : i - 1; }
    else { first = i < half; pair = first ? i : i - half; partner = first ? i + half : i - half; }
    float sn, cs;
    sincosf((float)pos * inv_freq[pair], &sn, &cs);
    return first ? x[i] * cs - x[partner] * sn : x[i] * cs + x[partner] * sn;
}

// grid (sequences, heads, slices of DM_COLS value columns); NR: key channels per warp (DM_WARPS * NR >= Dk).
// The block walks its sequence's tokens of the step in order; thread (warp w, lane l) keeps S[w NR .. w NR + NR, column l] in registers.
template <int NR>
__global__ void __launch_bounds__(DM_WARPS * 32)
decayed_memory_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ z, int ldz, float inv_tau,
                           const float* __restrict__ head_log_decay, const float* __restrict__ inv_freq, int rotary_dim, int pairing, float q_scale,
                           float k_scale, float* __restrict__ state, long long state_stride, int state_offset, const int* __restrict__ positions,
                           const int* __restrict__ cu_tokens, const int* __restrict__ slots, float* __restrict__ o, int H, int Dk, int Dv) {
    extern __shared__ float sm[];            // q [Dk], k [Dk], a [Dk], partial sums [DM_WARPS, DM_COLS]
    float* qs = sm;
    float* ks = sm + Dk;
    float* as = sm + 2 * Dk;
    float* part = sm + 3 * Dk;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, col = blockIdx.z * DM_COLS + (threadIdx.x & 31);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = cu_tokens[seq], n = cu_tokens[seq + 1] - first;
    if (n <= 0) return;
    const bool live = col < Dv;
    float* S = state + (size_t)slots[seq] * state_stride + state_offset + (size_t)h * Dk * Dv;
    float s[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int i = warp * NR + r;
        s[r] = (live && i < Dk) ? S[(size_t)i * Dv + col] : 0.f;
    }
    for (int n0 = 0; n0 < n; ++n0) {
        const size_t t = (size_t)first + n0;
        const int pos = positions[t];
        const float* row = proj + t * ld;
        __syncthreads();                     // the previous token's q, k, a and partial sums are no longer read
        for (int i = threadIdx.x; i < Dk; i += blockDim.x) {
            qs[i] = dm_turned(row + q_off + (size_t)h * Dk, i, pos, inv_freq, rotary_dim, pairing) * q_scale;
            ks[i] = dm_turned(row + k_off + (size_t)h * Dk, i, pos, inv_freq, rotary_dim, pairing) * k_scale;
            as[i] = expf(dm_log_decay(head_log_decay, z, ldz, inv_tau, t, h, Dk, i));
        }
        __syncthreads();
        const float v = live ? row[v_off + (size_t)h * Dv + col] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int i = warp * NR + r;
            if (i < Dk) {
                s[r] = fmaf(as[i], s[r], ks[i] * v);
                acc = fmaf(s[r], qs[i], acc);
            }
        }
        part[warp * DM_COLS + lane] = acc;
        __syncthreads();
        if (warp == 0 && live) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < DM_WARPS; ++w) sum += part[w * DM_COLS + lane];
            o[t * ((size_t)H * Dv) + (size_t)h * Dv + col] = sum;
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int i = warp * NR + r;
        if (live && i < Dk) S[(size_t)i * Dv + col] = s[r];
    }
}

// proj float32 [T, ld] with the queries at column q_off ([H, Dk]), the keys at k_off ([H, Dk]) and the values at v_off ([H, Dv]);
// z float32 [T, ldz] logits of the decay ([H, Dk]) with tau, or null and head_log_decay float32 [H] (log of the fixed decay);
// inv_freq [rotary_dim / 2] or null; state [slot, state_stride] float32 with this mixer's [H, Dk, Dv] at state_offset; o float32 [T, H Dv].
VM_API int vm_decayed_memory(const float* proj, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, float tau, const float* head_log_decay,
                             const float* inv_freq, int rotary_dim, int pairing, float q_scale, float k_scale, float* state, long long state_stride,
                             int state_offset, const int* positions, const int* cu_tokens, const int* slots, float* o, int T, int B, int H, int Dk, int Dv,
                             cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (H <= 0 || Dk <= 0 || Dv <= 0 || !state || (!z && !head_log_decay) || (z && !(tau > 0.f))) return VM_ERR_BAD_ARG;
    if (inv_freq && (rotary_dim < 0 || rotary_dim > Dk || rotary_dim % 2)) return VM_ERR_BAD_ARG;
    if (Dk > DM_WARPS * 64) return VM_ERR_UNSUPPORTED;
    const dim3 grid(B, H, (Dv + DM_COLS - 1) / DM_COLS), block(DM_WARPS * 32);
    const size_t smem = (size_t)(3 * Dk + DM_WARPS * DM_COLS) * sizeof(float);
    const float inv_tau = z ? 1.0f / tau : 0.f;
#define DM_LAUNCH(NR)                                                                                                                             \
    vm_launch_pdl(decayed_memory_scan_kernel<NR>, grid, block, smem, stream, proj, ld, q_off, k_off, v_off, z, ldz, inv_tau, head_log_decay, inv_freq, \
                  rotary_dim, pairing, q_scale, k_scale, state, state_stride, state_offset, positions, cu_tokens, slots, o, H, Dk, Dv)
    const int per = (Dk + DM_WARPS - 1) / DM_WARPS;
    if (per <= 4) DM_LAUNCH(4);
    else if (per <= 8) DM_LAUNCH(8);
    else if (per <= 16) DM_LAUNCH(16);
    else if (per <= 32) DM_LAUNCH(32);
    else DM_LAUNCH(64);
#undef DM_LAUNCH
    return vm_launch_status();
}

// ------------------------------------------------------------------------------------------------ the output stage
// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * silu(g[t, h, :]); a warp per (token, head); w float32 [Dv] or null; g float32 rows of stride ldg
template <typename T>
__global__ void memory_output_kernel(const float* __restrict__ o, const float* __restrict__ g, int ldg, const float* __restrict__ w, float eps,
                                     T* __restrict__ out, long long n_heads, int H, int Dv) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= n_heads) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / H;
    const int h = (int)(item - t * H);
    const float* x = o + (size_t)item * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) ss += x[d] * x[d];
    ss = vm_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int d = lane; d < Dv; d += 32) {
        const float gv = g[(size_t)t * ldg + (size_t)h * Dv + d];
        out[(size_t)item * Dv + d] = vm_from_float<T>(x[d] * inv * (w ? w[d] : 1.0f) * (gv / (1.0f + expf(-gv))));
    }
}

VM_API int vm_memory_output(const float* o, const float* g, int ldg, const float* w, float eps, void* out, int T, int H, int Dv, int act_dtype,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || Dv <= 0) return VM_ERR_BAD_ARG;
    const long long n = (long long)T * H;
    const int grid = (int)((n + 7) / 8);
    if (act_dtype == VM_F32) vm_launch_pdl(memory_output_kernel<float>, dim3(grid), dim3(256), 0, stream, o, g, ldg, w, eps, (float*)out, n, H, Dv);
    else if (act_dtype == VM_BF16) vm_launch_pdl(memory_output_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, o, g, ldg, w, eps, (__nv_bfloat16*)out, n, H, Dv);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
