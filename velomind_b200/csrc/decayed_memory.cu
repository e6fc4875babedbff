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
__device__ __forceinline__ float dm_log_decay(const float* __restrict__ head_log_decay, const float* __restrict__ z, int ldz, float inv_tau,
                                              const float* __restrict__ z_bias, size_t t, int h, int Dk, int i) {
    if (!z) return head_log_decay[h];
    const float x = z[t * ldz + (size_t)h * Dk + i] + (z_bias ? z_bias[(size_t)h * Dk + i] : 0.f);
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
decayed_memory_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ z, int ldz, float inv_tau, const float* __restrict__ z_bias,
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
            as[i] = expf(dm_log_decay(head_log_decay, z, ldz, inv_tau, z_bias, t, h, Dk, i));
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
VM_API int vm_decayed_memory(const float* proj, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, float tau, const float* z_bias,
                             const float* head_log_decay, const float* inv_freq, int rotary_dim, int pairing, float q_scale, float k_scale, float* state, long long state_stride,
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
    vm_launch_pdl(decayed_memory_scan_kernel<NR>, grid, block, smem, stream, proj, ld, q_off, k_off, v_off, z, ldz, inv_tau, z_bias, head_log_decay, inv_freq, \
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

// ------------------------------------------------------------------------------------------------ prompts, chunk by chunk
// Inside a chunk of C tokens the recurrence has a closed form.  With l_t = log a_t and b_t = l_(first) + .. + l_t (per key channel),
//     o_t   = sum_(s <= t) [ sum_i q_t[i] k_s[i] exp(b_t[i] - b_s[i]) ] v_s  +  (q_t * exp(b_t))^T S_start
//     S_end = diag(exp(b_last)) S_start + sum_s (k_s * exp(b_last - b_s)) v_s^T
// and every exponent is <= 0.  Three passes: `local` computes for all chunks of all sequences and heads at once the first sum, the
// chunk's own contribution to the memory, exp(b_last) and q * exp(b); `carry` walks each sequence's chunks elementwise and leaves the
// memory at every chunk's start in place of the chunk's contribution; `finish`, parallel again, adds the second term.
constexpr int DMC_THREADS = 256;

// the chunk's sequence, its first token among the step's tokens and its number of tokens
__device__ __forceinline__ bool dm_chunk_of(int chunk, const int* __restrict__ cu_tokens, int B, int C, int& seq, int& start, int& len) {
    int before = 0;
    for (int b = 0; b < B; ++b) {
        const int n = cu_tokens[b + 1] - cu_tokens[b], nc = (n + C - 1) / C;
        if (chunk < before + nc) {
            const int c = chunk - before;
            seq = b;
            start = cu_tokens[b] + c * C;
            len = min(C, n - c * C);
            return true;
        }
        before += nc;
    }
    return false;
}

// Rotary positions on the queries and keys of all heads, in place in the float32 projections: the angle of a (token, pair) is computed
// once and serves every head.  One block per token.
__global__ void dm_turn_rows_kernel(float* __restrict__ proj, int ld, int q_off, int k_off, const float* __restrict__ inv_freq, int rotary_dim, int pairing,
                                    const int* __restrict__ positions, int H, int Dk) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const size_t t = blockIdx.x;
    const int half = rotary_dim / 2;
    const float pos = (float)positions[t];
    float* row = proj + t * ld;
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[p], &sn, &cs);
        const int a = pairing == VM_PAIR_INTERLEAVED ? 2 * p : p, b = pairing == VM_PAIR_INTERLEAVED ? 2 * p + 1 : p + half;
        for (int h = 0; h < 2 * H; ++h) {
            float* x = row + (h < H ? q_off + (size_t)h * Dk : k_off + (size_t)(h - H) * Dk);
            const float u = x[a], v = x[b];
            x[a] = u * cs - v * sn;
            x[b] = v * cs + u * sn;
        }
    }
}

// grid (chunks, heads).  Shared: qT, kT, bT [Dk][C + 4] (channel-major, so that four neighbouring tokens are one 16-byte load),
// v [C][Dv], A [C][C].  Dk and Dv are multiples of 4, and so are ld and the three offsets; q and k come already turned (dm_turn_rows_kernel).
template <int C>
__global__ void __launch_bounds__(DMC_THREADS)
dm_chunk_local_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ z, int ldz, float inv_tau, const float* __restrict__ z_bias,
                      const float* __restrict__ head_log_decay, const float* __restrict__ inv_freq, int rotary_dim, int pairing, float q_scale,
                      float k_scale, const int* __restrict__ positions, const int* __restrict__ cu_tokens, int B, float* __restrict__ o,
                      float* __restrict__ dS, float* __restrict__ decay_all, float* __restrict__ q_decayed, int H, int Dk, int Dv) {
    constexpr int CP = C + 4;
    extern __shared__ __align__(16) float sm[];
    float* qT = sm;
    float* kT = qT + (size_t)Dk * CP;
    float* bT = kT + (size_t)Dk * CP;
    float* vs = bT + (size_t)Dk * CP;
    float* A = vs + (size_t)C * Dv;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    int seq, start, len;
    if (!dm_chunk_of(blockIdx.x, cu_tokens, B, C, seq, start, len)) return;
    const int h = blockIdx.y, tid = threadIdx.x;
    const bool per_channel = z != nullptr;
    // a. queries and keys (already turned; scaled here) and log decays, channel-major.  A thread takes four neighbouring channels of a
    // token with 16-byte loads; neighbouring lanes take neighbouring tokens, so the transposed stores meet no bank twice.
    (void)inv_freq; (void)rotary_dim; (void)pairing; (void)positions;
    for (int idx = tid; idx < C * (Dk / 4); idx += DMC_THREADS) {
        const int t = idx % C, i = (idx / C) * 4;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f), k = q, l = q;
        if (t < len) {
            const size_t tok = (size_t)start + t;
            const float* row = proj + tok * ld;
            q = *reinterpret_cast<const float4*>(row + q_off + (size_t)h * Dk + i);
            k = *reinterpret_cast<const float4*>(row + k_off + (size_t)h * Dk + i);
            l.x = dm_log_decay(head_log_decay, z, ldz, inv_tau, z_bias, tok, h, Dk, i);
            l.y = per_channel ? dm_log_decay(head_log_decay, z, ldz, inv_tau, z_bias, tok, h, Dk, i + 1) : l.x;
            l.z = per_channel ? dm_log_decay(head_log_decay, z, ldz, inv_tau, z_bias, tok, h, Dk, i + 2) : l.x;
            l.w = per_channel ? dm_log_decay(head_log_decay, z, ldz, inv_tau, z_bias, tok, h, Dk, i + 3) : l.x;
        }
        qT[(i + 0) * CP + t] = q.x * q_scale; qT[(i + 1) * CP + t] = q.y * q_scale; qT[(i + 2) * CP + t] = q.z * q_scale; qT[(i + 3) * CP + t] = q.w * q_scale;
        kT[(i + 0) * CP + t] = k.x * k_scale; kT[(i + 1) * CP + t] = k.y * k_scale; kT[(i + 2) * CP + t] = k.z * k_scale; kT[(i + 3) * CP + t] = k.w * k_scale;
        bT[(i + 0) * CP + t] = l.x; bT[(i + 1) * CP + t] = l.y; bT[(i + 2) * CP + t] = l.z; bT[(i + 3) * CP + t] = l.w;
    }
    for (int idx = tid; idx < C * Dv; idx += DMC_THREADS) {
        const int t = idx / Dv, j = idx - t * Dv;
        vs[idx] = t < len ? proj[((size_t)start + t) * ld + v_off + (size_t)h * Dv + j] : 0.f;
    }
    __syncthreads();
    // b. running sums of the log decays along the chunk
    for (int i = tid; i < Dk; i += DMC_THREADS) {
        float run = 0.f;
        for (int t = 0; t < C; ++t) {
            run += bT[i * CP + t];
            bT[i * CP + t] = run;
        }
    }
    __syncthreads();
    // c. A[t][s] = sum_i q_t[i] k_s[i] exp(b_t[i] - b_s[i]) for s <= t, in tiles of 4 x 4.  Only the tiles on and below the diagonal are
    // computed (the others are never read): the C / 4 diagonal ones first, so that they share a warp, then the rest row by row.  Below
    // the diagonal every key of a tile lies before every query of it, and the decay factors through the tile's last key m:
    // exp(b_t - b_s) = exp(b_t - b_m) exp(b_m - b_s), both exponents <= 0, eight exponentials per channel instead of sixteen.
    constexpr int NT = C / 4;
    for (int item = tid; item < NT * (NT + 1) / 2; item += DMC_THREADS) {
        int tt, st;
        if (item < NT) { tt = st = item; }
        else {
            int r = item - NT;                              // the r-th tile below the diagonal: row tt has tt of them
            tt = 1;
            while (r >= tt) { r -= tt; ++tt; }
            st = r;
        }
        const int t0 = tt * 4, s0 = st * 4;
        if (t0 >= len) continue;
        float acc[4][4] = {};
        if (per_channel && tt == st) {
            for (int i = 0; i < Dk; ++i) {
                const float4 q4 = *reinterpret_cast<const float4*>(qT + i * CP + t0), k4 = *reinterpret_cast<const float4*>(kT + i * CP + s0);
                const float4 bt = *reinterpret_cast<const float4*>(bT + i * CP + t0);
                const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w}, ba[4] = {bt.x, bt.y, bt.z, bt.w};
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        if (b <= a) acc[a][b] = fmaf(qa[a] * ka[b], __expf(ba[a] - ba[b]), acc[a][b]);
            }
        } else if (per_channel) {
            for (int i = 0; i < Dk; ++i) {
                const float4 q4 = *reinterpret_cast<const float4*>(qT + i * CP + t0), k4 = *reinterpret_cast<const float4*>(kT + i * CP + s0);
                const float4 bt = *reinterpret_cast<const float4*>(bT + i * CP + t0), bs = *reinterpret_cast<const float4*>(bT + i * CP + s0);
                const float m = bs.w;
                const float qa[4] = {q4.x * __expf(bt.x - m), q4.y * __expf(bt.y - m), q4.z * __expf(bt.z - m), q4.w * __expf(bt.w - m)};
                const float ka[4] = {k4.x * __expf(m - bs.x), k4.y * __expf(m - bs.y), k4.z * __expf(m - bs.z), k4.w};
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], ka[b], acc[a][b]);
            }
        } else {
            for (int i = 0; i < Dk; ++i) {
                const float4 q4 = *reinterpret_cast<const float4*>(qT + i * CP + t0), k4 = *reinterpret_cast<const float4*>(kT + i * CP + s0);
                const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], ka[b], acc[a][b]);
            }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] *= expf(fminf(bT[t0 + a] - bT[s0 + b], 0.f));      // (every channel has the same sums)
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) A[(t0 + a) * C + s0 + b] = (s0 + b <= t0 + a) ? acc[a][b] : 0.f;
    }
    __syncthreads();
    // d. what the finish pass and the carry pass need: q * exp(b), exp(b_last); keys scaled to the chunk's end, in place
    const size_t ch = (size_t)blockIdx.x * H + h;
    for (int idx = tid; idx < Dk * C; idx += DMC_THREADS) {
        const int i = idx / C, t = idx - i * C;
        const float b = bT[i * CP + t];
        q_decayed[ch * Dk * C + idx] = qT[i * CP + t] * expf(b);
        kT[i * CP + t] = t < len ? kT[i * CP + t] * expf(bT[i * CP + len - 1] - b) : 0.f;
    }
    for (int i = tid; i < Dk; i += DMC_THREADS) decay_all[ch * Dk + i] = expf(bT[i * CP + len - 1]);
    __syncthreads();
    // e. o_t = sum_(s <= t) A[t][s] v_s, tiles of 4 tokens x 4 values
    for (int tile = tid; tile < (C / 4) * (Dv / 4); tile += DMC_THREADS) {
        const int t0 = (tile / (Dv / 4)) * 4, j0 = (tile % (Dv / 4)) * 4;
        if (t0 >= len) continue;
        float acc[4][4] = {};
        const int s_end = min(t0 + 4, len);
        for (int s = 0; s < s_end; ++s) {
            const float4 v4 = *reinterpret_cast<const float4*>(vs + s * Dv + j0);
            const float va[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float w = A[(t0 + a) * C + s];
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(w, va[b], acc[a][b]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
            if (t0 + a < len)
                *reinterpret_cast<float4*>(o + ((size_t)start + t0 + a) * ((size_t)H * Dv) + (size_t)h * Dv + j0) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
    // f. the chunk's contribution to the memory: sum_s (k_s exp(b_last - b_s)) v_s^T, tiles of 4 channels x 4 values
    for (int tile = tid; tile < (Dk / 4) * (Dv / 4); tile += DMC_THREADS) {
        const int i0 = (tile / (Dv / 4)) * 4, j0 = (tile % (Dv / 4)) * 4;
        float acc[4][4] = {};
        for (int s = 0; s < len; ++s) {
            const float4 v4 = *reinterpret_cast<const float4*>(vs + s * Dv + j0);
            const float va[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float w = kT[(i0 + a) * CP + s];
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(w, va[b], acc[a][b]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
            *reinterpret_cast<float4*>(dS + (ch * Dk + i0 + a) * Dv + j0) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
}

// grid (sequences, heads, slices of the memory's values); a thread walks one value of the memory through its sequence's chunks
template <int C>
__global__ void dm_chunk_carry_kernel(float* __restrict__ dS, const float* __restrict__ decay_all, float* __restrict__ state, long long state_stride,
                                      int state_offset, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int H, int Dk, int Dv) {
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= Dk * Dv) return;
    int first = 0;
    for (int b = 0; b < seq; ++b) first += (cu_tokens[b + 1] - cu_tokens[b] + C - 1) / C;
    const int nc = (cu_tokens[seq + 1] - cu_tokens[seq] + C - 1) / C;
    if (nc <= 0) return;
    float* S = state + (size_t)slots[seq] * state_stride + state_offset + (size_t)h * Dk * Dv + e;
    float cur = *S;
    const int i = e / Dv;
    // eight chunks' values are fetched before the first store (the compiler cannot move a load over a store into the same array)
    for (int c0 = 0; c0 < nc; c0 += 8) {
        float add[8], dec[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const size_t ch = (size_t)(first + min(c0 + j, nc - 1)) * H + h;
            add[j] = dS[ch * Dk * Dv + e];
            dec[j] = decay_all[ch * Dk + i];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (c0 + j < nc) {
                const size_t ch = (size_t)(first + c0 + j) * H + h;
                dS[ch * Dk * Dv + e] = cur;               // the memory at this chunk's start, for the finish pass
                cur = fmaf(dec[j], cur, add[j]);
            }
    }
    *S = cur;
}

// grid (chunks, heads, slices of VS values): o_t += (q_t exp(b_t))^T S_start
template <int C>
__global__ void __launch_bounds__(DMC_THREADS)
dm_chunk_finish_kernel(const float* __restrict__ q_decayed, const float* __restrict__ S_start, const int* __restrict__ cu_tokens, int B,
                       float* __restrict__ o, int H, int Dk, int Dv, int VS) {
    extern __shared__ __align__(16) float sm[];
    float* qT = sm;                          // [Dk][C]
    float* S = sm + (size_t)Dk * C;          // [Dk][VS]
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    int seq, start, len;
    if (!dm_chunk_of(blockIdx.x, cu_tokens, B, C, seq, start, len)) return;
    const int h = blockIdx.y, j_base = blockIdx.z * VS, tid = threadIdx.x;
    const int width = min(VS, Dv - j_base);
    const size_t ch = (size_t)blockIdx.x * H + h;
    for (int idx = tid; idx < Dk * C; idx += DMC_THREADS) qT[idx] = q_decayed[ch * Dk * C + idx];
    for (int idx = tid; idx < Dk * width; idx += DMC_THREADS) {
        const int i = idx / width, j = idx - i * width;
        S[i * VS + j] = S_start[(ch * Dk + i) * Dv + j_base + j];
    }
    __syncthreads();
    for (int tile = tid; tile < (C / 4) * (width / 4); tile += DMC_THREADS) {
        const int t0 = (tile / (width / 4)) * 4, j0 = (tile % (width / 4)) * 4;
        if (t0 >= len) continue;
        float acc[4][4] = {};
        for (int i = 0; i < Dk; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(qT + i * C + t0), s4 = *reinterpret_cast<const float4*>(S + i * VS + j0);
            const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, sa[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], sa[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
            if (t0 + a < len) {
                float4* dst = reinterpret_cast<float4*>(o + ((size_t)start + t0 + a) * ((size_t)H * Dv) + (size_t)h * Dv + j_base + j0);
                float4 v = *dst;
                v.x += acc[a][0]; v.y += acc[a][1]; v.z += acc[a][2]; v.w += acc[a][3];
                *dst = v;
            }
    }
}

// tokens per chunk for these sizes (0: the chunked form does not take them), and the scratch it needs
static int dm_chunk_tokens(int Dk, int Dv) {
    if (Dk % 4 || Dv % 4) return 0;
    for (int C = 64; C >= 16; C /= 2) {
        const size_t local = ((size_t)3 * Dk * (C + 4) + (size_t)C * Dv + (size_t)C * C) * sizeof(float);
        const size_t finish = ((size_t)Dk * C + (size_t)Dk * (Dv < 128 ? Dv : 128)) * sizeof(float);
        if (local <= 200 * 1024 && finish <= 200 * 1024) return C;
    }
    return 0;
}

VM_API int vm_decayed_memory_chunk_tokens(int Dk, int Dv) { return dm_chunk_tokens(Dk, Dv); }

// float32 words of scratch for a step of up to T tokens in up to B sequences
VM_API long long vm_decayed_memory_scratch_floats(int T, int B, int H, int Dk, int Dv) {
    const int C = dm_chunk_tokens(Dk, Dv);
    if (C == 0) return 0;
    const long long chunks = T / C + B;
    return chunks * H * ((long long)Dk * Dv + Dk + (long long)Dk * C);
}

template <int C>
static int dm_launch_chunks(float* proj, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, float inv_tau, const float* z_bias,
                            const float* head_log_decay, const float* inv_freq, int rotary_dim, int pairing, float q_scale, float k_scale, float* state, long long state_stride,
                            int state_offset, const int* positions, const int* cu_tokens, const int* slots, float* o, float* scratch, int n_chunks, int T,
                            int B, int H, int Dk, int Dv, cudaStream_t stream) {
    float* dS = scratch;
    float* decay_all = dS + (size_t)n_chunks * H * Dk * Dv;
    float* q_decayed = decay_all + (size_t)n_chunks * H * Dk;
    const size_t local = ((size_t)3 * Dk * (C + 4) + (size_t)C * Dv + (size_t)C * C) * sizeof(float);
    const int VS = Dv < 128 ? Dv : 128;
    const size_t finish = ((size_t)Dk * C + (size_t)Dk * VS) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(dm_chunk_local_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)local);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dm_chunk_finish_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)finish);
    if (e != cudaSuccess) return (int)e;
    int st = 0;
    if (inv_freq && rotary_dim > 0) {              // turn q and k once for all heads; the chunk kernels then read them as they are
        vm_launch_pdl(dm_turn_rows_kernel, dim3(T), dim3(64), 0, stream, proj, ld, q_off, k_off, inv_freq, rotary_dim, pairing, positions, H, Dk);
        st = vm_launch_status();
        if (st) return st;
    }
    vm_launch_pdl(dm_chunk_local_kernel<C>, dim3(n_chunks, H), dim3(DMC_THREADS), local, stream, (const float*)proj, ld, q_off, k_off, v_off, z, ldz, inv_tau,
                  z_bias, head_log_decay, (const float*)nullptr, 0, pairing, q_scale, k_scale, positions, cu_tokens, B, o, dS, decay_all, q_decayed, H, Dk, Dv);
    st = vm_launch_status();
    if (st) return st;
    vm_launch_pdl(dm_chunk_carry_kernel<C>, dim3(B, H, (Dk * Dv + 255) / 256), dim3(256), 0, stream, dS, (const float*)decay_all, state, state_stride,
                  state_offset, cu_tokens, slots, H, Dk, Dv);
    st = vm_launch_status();
    if (st) return st;
    vm_launch_pdl(dm_chunk_finish_kernel<C>, dim3(n_chunks, H, (Dv + VS - 1) / VS), dim3(DMC_THREADS), finish, stream, (const float*)q_decayed, (const float*)dS,
                  cu_tokens, B, o, H, Dk, Dv, VS);
    return vm_launch_status();
}

// The same recurrence for prompts, chunk by chunk (three launches, and one before them that turns the queries and keys of `proj` in place).  n_chunks: the step's chunks, sum over its sequences of
// ceil(tokens / vm_decayed_memory_chunk_tokens(Dk, Dv)); scratch: vm_decayed_memory_scratch_floats(...) float32 words.
VM_API int vm_decayed_memory_chunked(float* proj, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, float tau, const float* z_bias,
                                     const float* head_log_decay, const float* inv_freq, int rotary_dim, int pairing, float q_scale, float k_scale,
                                     float* state, long long state_stride, int state_offset, const int* positions, const int* cu_tokens, const int* slots,
                                     float* o, float* scratch, int n_chunks, int T, int B, int H, int Dk, int Dv, cudaStream_t stream) {
    if (T <= 0 || B <= 0 || n_chunks <= 0) return 0;
    if (H <= 0 || Dk <= 0 || Dv <= 0 || !state || !scratch || (!z && !head_log_decay) || (z && !(tau > 0.f))) return VM_ERR_BAD_ARG;
    if (inv_freq && (rotary_dim < 0 || rotary_dim > Dk || rotary_dim % 2)) return VM_ERR_BAD_ARG;
    if (ld % 4 || q_off % 4 || k_off % 4 || (z && ldz % 4)) return VM_ERR_BAD_ARG;      // (16-byte loads of a token's queries and keys)
    const int C = dm_chunk_tokens(Dk, Dv);
    const float inv_tau = z ? 1.0f / tau : 0.f;
#define DMC(CC)                                                                                                                                        \
    return dm_launch_chunks<CC>(proj, ld, q_off, k_off, v_off, z, ldz, inv_tau, z_bias, head_log_decay, inv_freq, rotary_dim, pairing, q_scale, k_scale, state, \
                                state_stride, state_offset, positions, cu_tokens, slots, o, scratch, n_chunks, T, B, H, Dk, Dv, stream)
    if (C == 64) DMC(64);
    if (C == 32) DMC(32);
    if (C == 16) DMC(16);
#undef DMC
    return VM_ERR_UNSUPPORTED;
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
