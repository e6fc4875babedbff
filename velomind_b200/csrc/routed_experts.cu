// A routed feed-forward (mixture of experts) for few tokens: every token streams the weight rows of ITS experts.
//
//   z = W_router x + b                      float32 logits; the `top` largest are chosen (the lowest index wins a tie)
//   w = softmax over the chosen logits only
//   y = sum_k w_k  W_down[e_k] act(W_up[e_k] x)   (+ s * W_down_shared act(W_up_shared x),  s = sigmoid(w_sg . x))
//
// Three launches: the router (a block per token), the up-projections with their activation (a warp per four rows of the token's
// virtual matrix [top * ff + ff_shared, hidden]), the down-projections with the weighted sum (a warp per four output columns; the
// experts are added in the order of their rank, so a token's result does not depend on the batch it is in).
// Experts have no biases.  Weights are float32 or bfloat16 (template W), activations float32 or bfloat16 (template T);
// all sums are float32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float expert_act(float z, int kind) {
    if (kind == VM_ACT_RELU_SQUARED) { const float r = fmaxf(z, 0.f); return r * r; }
    if (kind == VM_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + expf(-z));
}

// the clamped gated unit: g <- min(g, limit), u <- clamp(u, -limit, limit), g sigmoid(alpha g) (u + 1)
__device__ __forceinline__ float glu_clamped(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

// dot product of a weight row with a float32 vector in shared memory, summed over a warp
template <typename W> __device__ __forceinline__ float warp_dot(const W* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.f;
    if ((n & 3) == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        const float4* w4 = reinterpret_cast<const float4*>(w);
        const float4* x4 = reinterpret_cast<const float4*>(x);
        float acc1 = 0.f;
        int i = lane;
        for (; i + 32 < n / 4; i += 64) {              // two independent loads in flight
            const float4 a = w4[i], b = w4[i + 32], xa = x4[i], xb = x4[i + 32];
            acc = fmaf(a.x, xa.x, fmaf(a.y, xa.y, fmaf(a.z, xa.z, fmaf(a.w, xa.w, acc))));
            acc1 = fmaf(b.x, xb.x, fmaf(b.y, xb.y, fmaf(b.z, xb.z, fmaf(b.w, xb.w, acc1))));
        }
        if (i < n / 4) {
            const float4 a = w4[i], xa = x4[i];
            acc = fmaf(a.x, xa.x, fmaf(a.y, xa.y, fmaf(a.z, xa.z, fmaf(a.w, xa.w, acc))));
        }
        return vm_warp_sum(acc + acc1);
    }
    for (int i = lane; i < n; i += 32) acc = fmaf(vm_to_float(w[i]), x[i], acc);
    return vm_warp_sum(acc);
}
template <> __device__ __forceinline__ float warp_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.f;
    if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        const uint4* w8 = reinterpret_cast<const uint4*>(w);
        uint4 p = make_uint4(0, 0, 0, 0), nxt = lane < n / 8 ? w8[lane] : p;
        for (int i = lane; i < n / 8; i += 32) {
            p = nxt;
            if (i + 32 < n / 8) nxt = w8[i + 32];       // the next piece is on its way while this one is summed
            const unsigned u[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u[k]);
                acc = fmaf(__low2float(b), x[i * 8 + 2 * k], acc);
                acc = fmaf(__high2float(b), x[i * 8 + 2 * k + 1], acc);
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(__bfloat162float(w[i]), x[i], acc);
    }
    return vm_warp_sum(acc);
}

// R rows at once against the same vector: the rows' loads are independent and in flight together
template <typename W, int R>
__device__ __forceinline__ void warp_dot_rows(const W* const (&w)[R], const float* __restrict__ x, int n, int lane, float (&out)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = 0.f;
    bool vec = (n & 7) == 0 && sizeof(W) == 2;
#pragma unroll
    for (int r = 0; r < R; ++r) vec = vec && (reinterpret_cast<uintptr_t>(w[r]) & 15) == 0;
    if (vec) {
        for (int i = lane; i < n / 8; i += 32) {
            uint4 p[R];
#pragma unroll
            for (int r = 0; r < R; ++r) p[r] = reinterpret_cast<const uint4*>(w[r])[i];
            float xv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) xv[k] = x[i * 8 + k];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const unsigned u[4] = {p[r].x, p[r].y, p[r].z, p[r].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u[k]);
                    out[r] = fmaf(__low2float(b), xv[2 * k], out[r]);
                    out[r] = fmaf(__high2float(b), xv[2 * k + 1], out[r]);
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            const float xi = x[i];
#pragma unroll
            for (int r = 0; r < R; ++r) out[r] = fmaf(vm_to_float(w[r][i]), xi, out[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = vm_warp_sum(out[r]);
}

constexpr int ROWS_PER_WARP = 4;

// A token's input row as float32 in shared memory.  norm_w == nullptr: x is the row in the activation dtype.  Otherwise x is the
// float32 residual stream and the row is rmsnorm(x) * norm_w, rounded as the activation dtype would hold it, so that a step
// gives the same numbers whether the norm ran here or in a kernel of its own.  `red`: 32 floats of shared memory.
template <typename T>
__device__ __forceinline__ void stage_row(const void* __restrict__ x, const float* __restrict__ norm_w, float eps, int t, int hidden, float* xs,
                                          float* red) {
    if (norm_w == nullptr) {
        const T* row = static_cast<const T*>(x) + (size_t)t * hidden;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = vm_to_float(row[i]);
        __syncthreads();
        return;
    }
    const float* row = static_cast<const float*>(x) + (size_t)t * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float v = row[i]; xs[i] = v; ss += v * v; }
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = vm_to_float(vm_from_float<T>(xs[i] * inv * norm_w[i]));
    __syncthreads();
}

// ------------------------------------------------------------------------------------------------ router
// Router weights, bias and the shared expert's gate row are float32 (exact copies of what the checkpoint stores).
template <typename T>
__global__ void router_kernel(const void* __restrict__ x, const float* __restrict__ norm_w, float eps, const float* __restrict__ w_router,
                              const float* __restrict__ b_router, const float* __restrict__ w_gate, int hidden, int E, int top,
                              int* __restrict__ chosen, float* __restrict__ weight, float* __restrict__ shared_gate) {
    __shared__ float red[32];
    extern __shared__ __align__(16) float sm[];          // [hidden] input, [E] logits
    float* xs = sm;
    float* z = sm + hidden;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    stage_row<T>(x, norm_w, eps, t, hidden, xs, red);
    for (int e = warp; e < E + (w_gate ? 1 : 0); e += nw) {
        if (e < E) {
            const float d = warp_dot<float>(w_router + (size_t)e * hidden, xs, hidden, lane);
            if (lane == 0) z[e] = d + (b_router ? b_router[e] : 0.f);
        } else {
            const float d = warp_dot<float>(w_gate, xs, hidden, lane);
            if (lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-d));
        }
    }
    __syncthreads();
    if (warp == 0) {
        // `top` rounds of arg-max over the logits not yet taken; the lowest index wins a tie
        float first = 0.f, sum = 0.f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = z[e];
                if (v > best) { best = v; at = e; }     // ascending e: the first maximum stays
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (k == 0) first = best;
            const float p = expf(best - first);          // the largest chosen logit is the softmax's reference
            sum += p;
            if (lane == 0) {
                chosen[(size_t)t * top + k] = at;
                weight[(size_t)t * top + k] = p;
                z[at] = -INFINITY;
            }
            __syncwarp();
        }
        const float inv = 1.0f / sum;
        for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= inv;
    }
}


// ------------------------------------------------------------------------------------------------ router with scores over all outputs
//   s = softmax(z) over all n_out outputs;  choice = s + correction (the correction steers the choice, not the weights)
//   outputs form `group_count` equal groups of neighbours; a group's score is its largest choice score; only outputs of the
//   `group_keep` best groups can be chosen (the lowest group index wins a tie, as the lowest output index does below)
//   the `top` largest choice scores are chosen; weight = s * scale, not renormalised
template <typename T>
__global__ void router_scored_kernel(const void* __restrict__ x, const float* __restrict__ norm_w, float eps, const float* __restrict__ w_router,
                                     const float* __restrict__ correction, int hidden, int n_out, int top, int group_count, int group_keep,
                                     int group_top, float scale, int score_kind, int* __restrict__ chosen, float* __restrict__ weight) {
    __shared__ float red[32];
    extern __shared__ __align__(16) float sm[];          // [hidden] input, [n_out] scores, [n_out] choice scores, [group_count] group scores
    float* xs = sm;
    float* sc = sm + hidden;
    float* ch = sc + n_out;
    float* gs = ch + n_out;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    stage_row<T>(x, norm_w, eps, t, hidden, xs, red);
    for (int e = warp; e < n_out; e += nw) {
        const float d = warp_dot<float>(w_router + (size_t)e * hidden, xs, hidden, lane);
        if (lane == 0) sc[e] = d;
    }
    __syncthreads();
    if (warp != 0) return;
    if (score_kind == VM_SCORE_SIGMOID) {                 // every output scored alone: s = 1 / (1 + exp(-z))
        // Without a correction the order of the scores is the order of the logits, and the logits still tell apart what the sigmoid
        // rounds to the same number (every z above 17 gives 1.0f): the choice is made on z.
        for (int e = lane; e < n_out; e += 32) {
            const float z = sc[e], p = 1.0f / (1.0f + expf(-z));
            sc[e] = p;
            ch[e] = correction ? p + correction[e] : z;
        }
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < n_out; e += 32) mx = fmaxf(mx, sc[e]);
        mx = vm_warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < n_out; e += 32) sum += expf(sc[e] - mx);
        sum = vm_warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < n_out; e += 32) {
            const float p = expf(sc[e] - mx) * inv;
            sc[e] = p;
            ch[e] = p + (correction ? correction[e] : 0.f);
        }
    }
    __syncwarp();
    if (group_count > 1 && group_keep < group_count) {
        const int per = n_out / group_count;
        // a group's score: the sum of its group_top largest scores (1: the largest).  Groups are scored on the scores themselves
        // (with the correction, if any), also where the choice inside them goes by the logits.
        const bool by_logit = score_kind == VM_SCORE_SIGMOID && !correction;
        for (int g = lane; g < group_count; g += 32) {
            float total = 0.f, last = INFINITY;
            int last_at = -1;
            for (int k = 0; k < group_top && k < per; ++k) {      // the k-th largest: the largest below (last, last_at) in the order (score descending, index ascending)
                float best = -INFINITY;
                int at = -1;
                for (int i = 0; i < per; ++i) {
                    const float v = by_logit ? sc[g * per + i] : ch[g * per + i];
                    const bool after = v < last || (v == last && i > last_at);
                    if (after && v > best) { best = v; at = i; }
                }
                total += best;
                last = best;
                last_at = at;
            }
            gs[g] = total;
        }
        __syncwarp();
        // a group stays if fewer than group_keep groups come before it in the order (score descending, index ascending)
        for (int g = lane; g < group_count; g += 32) {
            int before = 0;
            for (int o = 0; o < group_count; ++o) before += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
            if (before >= group_keep)
                for (int i = 0; i < per; ++i) ch[g * per + i] = -INFINITY;
        }
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_out; e += 32) {
            const float v = ch[e];
            if (v > best) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) at = 0;                      // fewer eligible outputs than `top` (a configuration the host refuses)
        if (lane == 0) {
            chosen[(size_t)t * top + k] = at;
            weight[(size_t)t * top + k] = sc[at] * scale;
            ch[at] = -INFINITY;
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------------ up-projections
// grid (row tiles, T); a warp per row r of the token's [top * ff + ff_shared] rows.  An act row has `act_cols` columns:
// those rows and, where identity experts exist (E_real < the router's outputs), the token's input row behind them.
// glu: an expert's up matrix is [2 * ff, hidden], gate rows first, and row r is glu_clamped(gate_r . x, up_r . x).
template <typename T, typename W>
__global__ void experts_up_kernel(const void* __restrict__ x, const float* __restrict__ norm_w, float eps, const W* __restrict__ w_up,
                                  const W* __restrict__ w_up_shared, const int* __restrict__ chosen, int hidden, int ff, int ff_shared, int top,
                                  int act_kind, int act_kind_shared, int E_real, int glu, float limit, float alpha, int act_cols,
                                  const float* __restrict__ weight, T* __restrict__ act) {
    extern __shared__ __align__(16) float xs[];          // [hidden]
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    stage_row<T>(x, norm_w, eps, t, hidden, xs, red);
    const int rows = top * ff + ff_shared;
    if (blockIdx.x == 0 && act_cols > rows)               // the input row, for the identity experts of the down kernel
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) act[(size_t)t * act_cols + rows + i] = vm_from_float<T>(xs[i]);
    const int r0 = (blockIdx.x * nw + warp) * ROWS_PER_WARP;
    if (r0 >= rows) return;
    const W* wrow[ROWS_PER_WARP];
    const W* urow[ROWS_PER_WARP];
    int kind[ROWS_PER_WARP];
    bool routed[ROWS_PER_WARP], skip[ROWS_PER_WARP];
    float wgt[ROWS_PER_WARP];                             // glu == VM_GLU_SILU_WEIGHTED_INPUT: the routing weight scales the expert's input
    const int per = glu ? 2 * ff : ff;                    // rows of one expert's up matrix
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        const int r = min(r0 + i, rows - 1);              // (a row past the end repeats the last one and is not stored)
        routed[i] = r < top * ff;
        skip[i] = false;
        wgt[i] = 1.0f;
        if (routed[i]) {
            int e = chosen[(size_t)t * top + r / ff];
            if (glu == VM_GLU_SILU_WEIGHTED_INPUT) wgt[i] = weight[(size_t)t * top + r / ff];
            if (e >= E_real) { skip[i] = true; e = 0; }   // an identity expert has no rows: zeros
            wrow[i] = w_up + ((size_t)e * per + r % ff) * hidden;
            urow[i] = wrow[i] + (size_t)ff * hidden;
            kind[i] = act_kind;
        } else {
            wrow[i] = urow[i] = w_up_shared + (size_t)(r - top * ff) * hidden;
            if (glu >= VM_GLU_SILU_WEIGHTED_INPUT) urow[i] = wrow[i] + (size_t)ff_shared * hidden;      // the shared expert is gated too
            kind[i] = act_kind_shared;
        }
    }
    float d[ROWS_PER_WARP], u[ROWS_PER_WARP];
    warp_dot_rows<W, ROWS_PER_WARP>(wrow, xs, hidden, lane, d);
    if (glu) warp_dot_rows<W, ROWS_PER_WARP>(urow, xs, hidden, lane, u);
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i)
            if (r0 + i < rows) {
                float v;
                if (skip[i]) v = 0.f;
                else if (glu >= VM_GLU_SILU_WEIGHTED_INPUT) {      // (VM_GLU_SILU: wgt stays 1, the weight is the down kernel's)
                    // W (w x) = w (W x): gate and up as the activation dtype holds them, the weight applied in float32
                    const float g = wgt[i] * vm_to_float(vm_from_float<T>(d[i])), uu = wgt[i] * vm_to_float(vm_from_float<T>(u[i]));
                    v = g / (1.0f + expf(-g)) * uu;
                } else if (glu && routed[i]) v = glu_clamped(vm_to_float(vm_from_float<T>(d[i])), vm_to_float(vm_from_float<T>(u[i])), limit, alpha);
                else v = expert_act(d[i], kind[i]);
                act[(size_t)t * act_cols + r0 + i] = vm_from_float<T>(v);
            }
    }
}

// ------------------------------------------------------------------------------------------------ down-projections
// grid (column tiles, T); a warp per output column
template <typename T, typename W>
__global__ void experts_down_kernel(const T* __restrict__ act, const W* __restrict__ w_down, const W* __restrict__ w_down_shared,
                                    const int* __restrict__ chosen, const float* __restrict__ weight, const float* __restrict__ shared_gate,
                                    int hidden, int ff, int ff_shared, int top, int E_real, int act_cols, int unit_weights, T* __restrict__ out,
                                    float* __restrict__ residual) {
    extern __shared__ __align__(16) float as[];          // [act_cols]: top * ff + ff_shared, then (identity experts) the input row
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int rows = top * ff + ff_shared;
    for (int i = threadIdx.x; i < act_cols; i += blockDim.x) as[i] = vm_to_float(act[(size_t)t * act_cols + i]);
    __syncthreads();
    const int c0 = (blockIdx.x * nw + warp) * ROWS_PER_WARP;
    if (c0 >= hidden) return;
    float y[ROWS_PER_WARP] = {};
    const W* wrow[ROWS_PER_WARP];
    float d[ROWS_PER_WARP];
    for (int k = 0; k < top; ++k) {
        const int e = chosen[(size_t)t * top + k];
        if (e >= E_real) {                                // an identity expert: the input itself, times the weight
            const float wk = weight[(size_t)t * top + k];
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) y[i] = fmaf(wk, as[rows + min(c0 + i, hidden - 1)], y[i]);
            continue;
        }
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) wrow[i] = w_down + ((size_t)e * hidden + min(c0 + i, hidden - 1)) * ff;
        warp_dot_rows<W, ROWS_PER_WARP>(wrow, as + k * ff, ff, lane, d);
        const float wk = unit_weights ? 1.0f : weight[(size_t)t * top + k];      // (the weight went into the expert's input)
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) y[i] = fmaf(wk, d[i], y[i]);
    }
    if (ff_shared > 0) {
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) wrow[i] = w_down_shared + (size_t)min(c0 + i, hidden - 1) * ff_shared;
        warp_dot_rows<W, ROWS_PER_WARP>(wrow, as + top * ff, ff_shared, lane, d);
        const float g = shared_gate ? shared_gate[t] : 1.0f;
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) y[i] = fmaf(g, d[i], y[i]);
    }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i)
            if (c0 + i < hidden) {
                // into the float32 residual stream if one is given (through the activation dtype's rounding, as the unfused step adds it)
                if (residual) residual[(size_t)t * hidden + c0 + i] += vm_to_float(vm_from_float<T>(y[i]));
                else out[(size_t)t * hidden + c0 + i] = vm_from_float<T>(y[i]);
            }
    }
}

template <typename T, typename W>
int launch_experts(const void* x, const float* norm_w, float eps, const void* w_up, const void* w_down, const void* w_up_shared,
                   const void* w_down_shared, const int* chosen, const float* weight, const float* shared_gate, int T_, int hidden, int ff,
                   int ff_shared, int top, int act_kind, int act_kind_shared, int E_real, int n_identity, int glu, float limit, float alpha, void* act,
                   void* out, float* residual, cudaStream_t stream) {
    const int rows = top * ff + ff_shared;
    const int act_cols = rows + (n_identity > 0 ? hidden : 0);
    const int warps = 8;
    const size_t up_smem = (size_t)hidden * sizeof(float), down_smem = (size_t)act_cols * sizeof(float);
    if (up_smem > 200 * 1024 || down_smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    static size_t up_raised = 48 * 1024, down_raised = 48 * 1024;       // per instantiation
    if (up_smem > up_raised) {
        if (cudaFuncSetAttribute(experts_up_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)up_smem) != cudaSuccess) return vm_launch_status();
        up_raised = up_smem;
    }
    if (down_smem > down_raised) {
        if (cudaFuncSetAttribute(experts_down_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)down_smem) != cudaSuccess) return vm_launch_status();
        down_raised = down_smem;
    }
    const int per_block = warps * ROWS_PER_WARP;
    vm_launch_pdl(experts_up_kernel<T, W>, dim3((rows + per_block - 1) / per_block, T_), dim3(warps * 32), (size_t)hidden * sizeof(float), stream, x, norm_w, eps,
                  (const W*)w_up, (const W*)w_up_shared, chosen, hidden, ff, ff_shared, top, act_kind, act_kind_shared, E_real, glu, limit, alpha, act_cols,
                  weight, (T*)act);
    int st = vm_launch_status();
    if (st) return st;
    vm_launch_pdl(experts_down_kernel<T, W>, dim3((hidden + per_block - 1) / per_block, T_), dim3(warps * 32), down_smem, stream, (const T*)act,
                  (const W*)w_down, (const W*)w_down_shared, chosen, weight, shared_gate, hidden, ff, ff_shared, top, E_real, act_cols,
                  glu == VM_GLU_SILU_WEIGHTED_INPUT ? 1 : 0, (T*)out, residual);
    return vm_launch_status();
}

}  // namespace

// chosen int32 [T, top], weight float32 [T, top], shared_gate float32 [T] (written only if w_gate is given)
// norm_w given: x is the float32 residual stream and the router (like the experts below) norms its rows itself
VM_API int vm_expert_router(const void* x, const float* norm_w, float eps, const float* w_router, const float* b_router, const float* w_gate, int T,
                            int hidden, int E, int top, int* chosen, float* weight, float* shared_gate, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || hidden <= 0) return VM_ERR_BAD_ARG;
    const size_t smem = (size_t)(hidden + E) * sizeof(float);
    if (smem > 48 * 1024) return VM_ERR_UNSUPPORTED;
    if (act_dtype == VM_F32)
        vm_launch_pdl(router_kernel<float>, dim3(T), dim3(256), smem, stream, x, norm_w, eps, w_router, b_router, w_gate, hidden, E, top, chosen, weight,
                      shared_gate);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(router_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, x, norm_w, eps, w_router, b_router, w_gate, hidden, E, top, chosen,
                      weight, shared_gate);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

// x, out [T, hidden] and the scratch `act` [T, vm_experts_act_cols(...)] in the activation dtype; expert weights stacked:
// w_up [E * ff, hidden] (glu: [E * 2 * ff, hidden], an expert's gate rows before its up rows), w_down [E * hidden, ff]; the shared expert's
// w_up_shared [ff_shared, hidden], w_down_shared [hidden, ff_shared] (ff_shared 0: none).  weight_dtype is the experts' storage.
// A chosen index >= E names an identity expert (n_identity of them): its result is the input row.  glu: act = glu_clamped(gate, up)
// with `limit` and `alpha`; else act_kind.
// norm_w given: x is the float32 residual stream, normed here.  residual given: the result is added into it and `out` is not written.
VM_API long long vm_experts_act_cols(int hidden, int ff, int ff_shared, int top, int n_identity) {
    return (long long)top * ff + ff_shared + (n_identity > 0 ? hidden : 0);
}

VM_API int vm_experts_few_tokens_glu(const void* x, const float* norm_w, float eps, const void* w_up, const void* w_down, const void* w_up_shared,
                                     const void* w_down_shared, int weight_dtype, const int* chosen, const float* weight, const float* shared_gate,
                                     int T, int hidden, int ff, int ff_shared, int top, int act_kind, int act_kind_shared, int E, int n_identity,
                                     int glu, float limit, float alpha, void* act, void* out, float* residual, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hidden <= 0 || ff <= 0 || ff_shared < 0 || top <= 0 || E <= 0 || n_identity < 0) return VM_ERR_BAD_ARG;
    if (act_dtype == VM_F32 && weight_dtype == VM_F32)
        return launch_experts<float, float>(x, norm_w, eps, w_up, w_down, w_up_shared, w_down_shared, chosen, weight, shared_gate, T, hidden, ff, ff_shared,
                                            top, act_kind, act_kind_shared, E, n_identity, glu, limit, alpha, act, out, residual, stream);
    if (act_dtype == VM_BF16 && weight_dtype == VM_BF16)
        return launch_experts<__nv_bfloat16, __nv_bfloat16>(x, norm_w, eps, w_up, w_down, w_up_shared, w_down_shared, chosen, weight, shared_gate, T,
                                                            hidden, ff, ff_shared, top, act_kind, act_kind_shared, E, n_identity, glu, limit, alpha, act,
                                                            out, residual, stream);
    if (act_dtype == VM_BF16 && weight_dtype == VM_F32)
        return launch_experts<__nv_bfloat16, float>(x, norm_w, eps, w_up, w_down, w_up_shared, w_down_shared, chosen, weight, shared_gate, T, hidden, ff,
                                                    ff_shared, top, act_kind, act_kind_shared, E, n_identity, glu, limit, alpha, act, out, residual,
                                                    stream);
    return VM_ERR_UNSUPPORTED;
}

// the same for experts of one up matrix and an activation, every chosen index a real expert
VM_API int vm_experts_few_tokens(const void* x, const float* norm_w, float eps, const void* w_up, const void* w_down, const void* w_up_shared,
                                 const void* w_down_shared, int weight_dtype, const int* chosen, const float* weight, const float* shared_gate, int T,
                                 int hidden, int ff, int ff_shared, int top, int act_kind, int act_kind_shared, void* act, void* out,
                                 float* residual, int act_dtype, cudaStream_t stream) {
    return vm_experts_few_tokens_glu(x, norm_w, eps, w_up, w_down, w_up_shared, w_down_shared, weight_dtype, chosen, weight, shared_gate, T, hidden, ff,
                                     ff_shared, top, act_kind, act_kind_shared, 0x7fffffff, 0, 0, 0.f, 0.f, act, out, residual, act_dtype, stream);
}

// chosen int32 [T, top] (an index >= the number of real experts names an identity expert), weight float32 [T, top]; w_router float32
// [n_out, hidden], correction float32 [n_out] or null; group_count must divide n_out
VM_API int vm_expert_router_scored(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                                   int n_out, int top, int group_count, int group_keep, float scale, int* chosen, float* weight, int act_dtype,
                                   cudaStream_t stream) {
    return vm_expert_router_scores(x, norm_w, eps, w_router, correction, T, hidden, n_out, top, group_count, group_keep, scale, VM_SCORE_SOFTMAX, chosen,
                                   weight, act_dtype, stream);
}

// the same with the kind of score as an argument: VM_SCORE_SOFTMAX over all outputs, or VM_SCORE_SIGMOID of each output alone
VM_API int vm_expert_router_scores(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                                   int n_out, int top, int group_count, int group_keep, float scale, int score_kind, int* chosen, float* weight,
                                   int act_dtype, cudaStream_t stream) {
    return vm_expert_router_groups(x, norm_w, eps, w_router, correction, T, hidden, n_out, top, group_count, group_keep, 1, scale, score_kind, chosen,
                                   weight, act_dtype, stream);
}

// the same with the number of a group's largest scores whose sum is the group's score
VM_API int vm_expert_router_groups(const void* x, const float* norm_w, float eps, const float* w_router, const float* correction, int T, int hidden,
                                   int n_out, int top, int group_count, int group_keep, int group_top, float scale, int score_kind, int* chosen,
                                   float* weight, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (group_top < 1) return VM_ERR_BAD_ARG;
    if (score_kind != VM_SCORE_SOFTMAX && score_kind != VM_SCORE_SIGMOID) return VM_ERR_BAD_ARG;
    if (n_out <= 0 || top <= 0 || hidden <= 0 || group_count <= 0 || n_out % group_count || group_keep <= 0 || group_keep > group_count) return VM_ERR_BAD_ARG;
    if (top > (n_out / group_count) * group_keep) return VM_ERR_BAD_ARG;
    const size_t smem = (size_t)(hidden + 2 * n_out + group_count) * sizeof(float);
    if (smem > 48 * 1024) return VM_ERR_UNSUPPORTED;
    if (act_dtype == VM_F32)
        vm_launch_pdl(router_scored_kernel<float>, dim3(T), dim3(256), smem, stream, x, norm_w, eps, w_router, correction, hidden, n_out, top, group_count,
                      group_keep, group_top, scale, score_kind, chosen, weight);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(router_scored_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, x, norm_w, eps, w_router, correction, hidden, n_out, top,
                      group_count, group_keep, group_top, scale, score_kind, chosen, weight);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
