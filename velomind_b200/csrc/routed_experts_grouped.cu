// A routed feed-forward (mixture of experts) for many tokens: the (token, expert) pairs are grouped by expert on the device
// and each expert multiplies only the rows that chose it.
//
//   group:    count the pairs of every expert, give each expert a run of rows padded to whole tiles of 64, and place every
//             pair in its expert's run.  Everything stays on the device: the launches that follow have a fixed shape
//             (the step's capacity), and tiles without an expert return at once.
//   up:       act[row, :] = activation(W_up[e] x[token(row)])          bf16 tensor-core tiles (mma.sync m16n8k16), rows gathered
//   down:     y[row, :] = W_down[e] act[row, :]                         float32 result
//   combine:  out[t] = sum_k w[t, k] y[row(t, k)] (+ gate[t] * shared[t])   in the order of the token's ranks: deterministic
//
// Which row of its run a pair gets depends on the order in which threads arrive, but no result depends on the row.
#include "mma.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 32, PAD = 8;       // tile of rows, of columns, of the summed dimension; padding of a shared-memory row
constexpr int GROUP_THREADS = 1024;

__device__ __forceinline__ float act_of(float z, int kind) {
    if (kind < 0) return z;                                  // no activation
    if (kind == VM_ACT_RELU_SQUARED) { const float r = fmaxf(z, 0.f); return r * r; }
    if (kind == VM_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + expf(-z));
}

// one block: counts, padded offsets, placement.  row_of_pair [T * top]; token_of_row [row_cap] (-1: padding); expert_of_tile [row_cap / TM] (-1: unused)
__global__ void group_pairs_kernel(const int* __restrict__ chosen, int n_pairs, int top, int E, int row_cap, int tile, int* __restrict__ row_of_pair,
                                   int* __restrict__ token_of_row, int* __restrict__ expert_of_tile) {
    extern __shared__ int sh[];            // [E] counts, [E] cursors
    int* count = sh;
    int* cursor = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < row_cap; i += blockDim.x) token_of_row[i] = -1;
    for (int i = threadIdx.x; i < row_cap / tile; i += blockDim.x) expert_of_tile[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            const int tiles = (count[e] + tile - 1) / tile;
            cursor[e] = at;
            for (int k = 0; k < tiles; ++k) expert_of_tile[at / tile + k] = e;
            at += tiles * tile;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e < 0 || e >= E) { row_of_pair[i] = -1; continue; }
        const int row = atomicAdd(&cursor[e], 1);
        row_of_pair[i] = row;
        token_of_row[row] = i / top;
    }
}

// C[TM, TN] tile of A[rows, K] B[e][N, K]^T; 4 warps, each 32 x 32.  A rows come from `a_row(r)` (a pointer or null for a zero row).
template <typename ARow, typename Epilogue>
__device__ __forceinline__ void tile_product(ARow a_row, const __nv_bfloat16* __restrict__ B, int N, int K, int n0, Epilogue epilogue) {
    __shared__ __align__(16) __nv_bfloat16 As[TM][TK + PAD];
    __shared__ __align__(16) __nv_bfloat16 Bs[TN][TK + PAD];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
    // each thread moves two 16-byte pieces of each operand per step: rows tid / 4 and tid / 4 + 32, piece tid % 4
    const int lr = tid >> 2, lp = (tid & 3) * 8;
    const __nv_bfloat16* a_src[2] = {a_row(lr), a_row(lr + 32)};
    const __nv_bfloat16* b_src[2] = {n0 + lr < N ? B + (size_t)(n0 + lr) * K : nullptr, n0 + lr + 32 < N ? B + (size_t)(n0 + lr + 32) * K : nullptr};
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 av[2], bv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        av[i] = a_src[i] ? *reinterpret_cast<const uint4*>(a_src[i] + lp) : zero;
        bv[i] = b_src[i] ? *reinterpret_cast<const uint4*>(b_src[i] + lp) : zero;
    }
    for (int k0 = 0; k0 < K; k0 += TK) {
        __syncthreads();                   // the previous step's fragments are read
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            *reinterpret_cast<uint4*>(&As[lr + 32 * i][lp]) = av[i];
            *reinterpret_cast<uint4*>(&Bs[lr + 32 * i][lp]) = bv[i];
        }
        __syncthreads();
        if (k0 + TK < K) {                 // the next step's pieces are on their way while this one is multiplied
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                av[i] = a_src[i] ? *reinterpret_cast<const uint4*>(a_src[i] + k0 + TK + lp) : zero;
                bv[i] = b_src[i] ? *reinterpret_cast<const uint4*>(b_src[i] + k0 + TK + lp) : zero;
            }
        }
#pragma unroll
        for (int kk = 0; kk < TK; kk += 16) {
            // fragments through ldmatrix: four 8 x 8 blocks per instruction.  A: rows r..r+15, the two halves of k; B (stored [n][k],
            // the "col" operand): two n-blocks of 8, the two halves of k each
            unsigned a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                vm_ldmatrix_x4(a[i][0], a[i][1], a[i][2], a[i][3], &As[wm + 16 * i + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj)
                vm_ldmatrix_x4(b[2 * jj][0], b[2 * jj][1], b[2 * jj + 1][0], b[2 * jj + 1][1],
                               &Bs[wn + 16 * jj + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) vm_mma_bf16_16816(acc[i][j], a[i][0], a[i][1], a[i][2], a[i][3], b[j][0], b[j][1]);
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = wm + 16 * i + g, n = n0 + wn + 8 * j + 2 * t;
            epilogue(r, n, acc[i][j][0], acc[i][j][1]);
            epilogue(r + 8, n, acc[i][j][2], acc[i][j][3]);
        }
}

__global__ void __launch_bounds__(128)
experts_up_grouped_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_up, const int* __restrict__ token_of_row,
                          const int* __restrict__ expert_of_tile, int hidden, int ff, int act_kind, __nv_bfloat16* __restrict__ act) {
    const int e = expert_of_tile[blockIdx.x];
    if (e < 0) return;
    const int row0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    auto a_row = [&](int r) -> const __nv_bfloat16* {
        const int tok = token_of_row[row0 + r];
        return tok >= 0 ? x + (size_t)tok * hidden : nullptr;
    };
    // (`ff` here is the number of rows of one expert's up matrix: twice the expert's size for gated experts)
    tile_product(a_row, w_up + (size_t)e * ff * hidden, ff, hidden, n0, [&](int r, int n, float c0, float c1) {
        __nv_bfloat16* dst = act + (size_t)(row0 + r) * ff + n;
        if (n + 1 < ff) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(act_of(c0, act_kind), act_of(c1, act_kind));
        else if (n < ff) dst[0] = __float2bfloat16_rn(act_of(c0, act_kind));
    });
}

__global__ void __launch_bounds__(128)
experts_down_grouped_kernel(const __nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ w_down, const int* __restrict__ expert_of_tile,
                            int hidden, int ff, float* __restrict__ y) {
    const int e = expert_of_tile[blockIdx.x];
    if (e < 0) return;
    const int row0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    auto a_row = [&](int r) -> const __nv_bfloat16* { return act + (size_t)(row0 + r) * ff; };
    tile_product(a_row, w_down + (size_t)e * hidden * ff, hidden, ff, n0, [&](int r, int n, float c0, float c1) {
        float* dst = y + (size_t)(row0 + r) * hidden + n;
        if (n + 1 < hidden) *reinterpret_cast<float2*>(dst) = make_float2(c0, c1);
        else if (n < hidden) dst[0] = c0;
    });
}

// act[row, i] = silu(w g) (w u) with g = gate_up[row, i], u = gate_up[row, ff + i] and w the routing weight of the row's (token, expert)
// pair: the weight scales the expert's INPUT, and W (w x) = w (W x).  Rows of padding give zeros.
__global__ void silu_weighted_rows_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ act, int rows, int ff,
                                          const int* __restrict__ token_of_row, const int* __restrict__ row_of_pair, const float* __restrict__ weight,
                                          int top) {
    if ((ff & 7) == 0) {                   // eight values a thread, 16-byte loads and stores; the row's weight is looked up once
        const unsigned per = (unsigned)ff >> 3;
        const size_t n8 = (size_t)rows * per;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
            const int row = (int)(i / per), c = (int)(i - (size_t)row * per) << 3;
            const int tok = token_of_row[row];
            unsigned o[4] = {0u, 0u, 0u, 0u};
            if (tok >= 0) {
                float w = weight ? 0.f : 1.0f;          // (no weights: the unit itself)
                for (int k = 0; weight && k < top; ++k)
                    if (row_of_pair[(size_t)tok * top + k] == row) w = weight[(size_t)tok * top + k];
                const __nv_bfloat16* src = gate_up + (size_t)row * 2 * ff + c;
                const uint4 gv = *reinterpret_cast<const uint4*>(src), uv = *reinterpret_cast<const uint4*>(src + ff);
                const unsigned gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
                    const float2 u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[k]));
                    const float g0 = w * g2.x, g1 = w * g2.y;
                    o[k] = vm_pack_bf16(g0 / (1.0f + expf(-g0)) * (w * u2.x), g1 / (1.0f + expf(-g1)) * (w * u2.y));
                }
            }
            *reinterpret_cast<uint4*>(act + (size_t)row * ff + c) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }
    const size_t n = (size_t)rows * ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / ff), c = (int)(i - (size_t)row * ff);
        const int tok = token_of_row[row];
        float v = 0.f;
        if (tok >= 0) {
            float w = weight ? 0.f : 1.0f;
            for (int k = 0; weight && k < top; ++k)
                if (row_of_pair[(size_t)tok * top + k] == row) w = weight[(size_t)tok * top + k];
            const float g = w * __bfloat162float(gate_up[(size_t)row * 2 * ff + c]), u = w * __bfloat162float(gate_up[(size_t)row * 2 * ff + ff + c]);
            v = g / (1.0f + expf(-g)) * u;
        }
        act[i] = __float2bfloat16_rn(v);
    }
}

// (x and chosen given: a pair whose index is E or more is an identity expert, its result the token's input row)
__global__ void experts_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair, const float* __restrict__ weight,
                                       const float* __restrict__ shared_y, const float* __restrict__ shared_gate, int T, int hidden, int top,
                                       const __nv_bfloat16* __restrict__ x, const int* __restrict__ chosen, int E, __nv_bfloat16* __restrict__ out) {
    const size_t n = (size_t)T * hidden;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / hidden), c = (int)(i - (size_t)t * hidden);
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = row_of_pair[(size_t)t * top + k];
            if (row >= 0) acc = fmaf(weight ? weight[(size_t)t * top + k] : 1.0f, y[(size_t)row * hidden + c], acc);
            else if (x && chosen[(size_t)t * top + k] >= E) acc = fmaf(weight[(size_t)t * top + k], __bfloat162float(x[i]), acc);
        }
        if (shared_y) acc = fmaf(shared_gate ? shared_gate[t] : 1.0f, shared_y[i], acc);
        out[i] = __float2bfloat16_rn(acc);
    }
}

// x_sorted[row] = x[token_of_row[row]], zeros for a row of padding; 16 bytes per thread
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ token_of_row, int rows, int hidden,
                                   __nv_bfloat16* __restrict__ x_sorted) {
    const int per_row = hidden / 8;
    const size_t n = (size_t)rows * per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / per_row), piece = (int)(i - (size_t)row * per_row);
        const int tok = token_of_row[row];
        reinterpret_cast<uint4*>(x_sorted)[i] = tok >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)tok * hidden)[piece] : make_uint4(0, 0, 0, 0);
    }
}

// act[row, i] = glu_clamped(gate_up[row, i], gate_up[row, ff + i]); rows of padding hold zeros and give zeros
__global__ void glu_rows_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ act, size_t n, int ff, float limit, float alpha) {
    if ((ff & 7) == 0) {                   // eight values a thread, 16-byte loads and stores
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8) {
            const size_t row = i / ff;
            const int c = (int)(i - row * ff);
            const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + row * 2 * ff + c), uv = *reinterpret_cast<const uint4*>(gate_up + row * 2 * ff + ff + c);
            const unsigned gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            unsigned o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
                const float2 u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[k]));
                const float g0 = fminf(g2.x, limit), g1 = fminf(g2.y, limit);
                const float u0 = fminf(fmaxf(u2.x, -limit), limit), u1 = fminf(fmaxf(u2.y, -limit), limit);
                o[k] = vm_pack_bf16(g0 / (1.0f + expf(-alpha * g0)) * (u0 + 1.0f), g1 / (1.0f + expf(-alpha * g1)) * (u1 + 1.0f));
            }
            *reinterpret_cast<uint4*>(act + i) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / ff;
        const int c = (int)(i - row * ff);
        float g = __bfloat162float(gate_up[row * 2 * ff + c]), u = __bfloat162float(gate_up[row * 2 * ff + ff + c]);
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        act[i] = __float2bfloat16_rn(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

template <typename T> __global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, size_t n, int kind) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = vm_from_float<T>(act_of(vm_to_float(in[i]), kind));
}

}  // namespace

// rows the grouped layout may need for T tokens: every pair, plus padding of each expert's run to whole tiles
VM_API long long vm_experts_grouped_rows(int T, int top, int E) { return ((long long)T * top + (long long)E * (TM - 1) + TM - 1) / TM * TM; }

VM_API long long vm_experts_grouped_rows_tiled(int T, int top, int E, int tile) {
    return ((long long)T * top + (long long)E * (tile - 1) + tile - 1) / tile * tile;
}

// x, out [T, hidden] bfloat16; w_up [E * ff, hidden] (glu: [E * 2 * ff, hidden], gate rows before up rows), w_down [E * hidden, ff] bfloat16;
// chosen / weight [T, top] (an index >= E: an identity expert, when n_identity > 0);
// scratch: row_of_pair int [T * top], token_of_row int [row_cap], expert_of_tile int [row_cap / tile], act bf16 [row_cap, ff],
// gate_up bf16 [row_cap, 2 * ff] (glu only), y float32 [row_cap, hidden]; shared_y float32 [T, hidden] (or null) is added times shared_gate [T] (or 1).
// x_sorted given (bf16 [row_cap, hidden]): the products run on tcgen05 in tiles of 128 rows (row_cap from vm_experts_grouped_rows_tiled(..., 128);
// hidden and ff multiples of 8); else on mma.sync in tiles of 64 (row_cap from vm_experts_grouped_rows; multiples of 32).
VM_API int vm_experts_grouped_glu(const void* x, const void* w_up, const void* w_down, const int* chosen, const float* weight, const float* shared_y,
                                  const float* shared_gate, int T, int hidden, int ff, int top, int E, int n_identity, int act_kind, int glu, float limit,
                                  float alpha, int row_cap, int* row_of_pair, int* token_of_row, int* expert_of_tile, void* x_sorted, void* act,
                                  void* gate_up, float* y, void* out, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    const bool tc = x_sorted != nullptr;
    const int tile = tc ? 128 : TM;
    if (top <= 0 || E <= 0 || n_identity < 0 || (glu && !gate_up)) return VM_ERR_BAD_ARG;
    if (tc ? (hidden % 8 || ff % 8) : (hidden % TK || ff % TK)) return VM_ERR_UNSUPPORTED;
    const long long need = tc ? vm_experts_grouped_rows_tiled(T, top, E, tile) : vm_experts_grouped_rows(T, top, E);
    if (row_cap % tile || row_cap < need) return VM_ERR_BAD_ARG;
    if ((size_t)2 * E * sizeof(int) > 48 * 1024) return VM_ERR_UNSUPPORTED;
    group_pairs_kernel<<<1, GROUP_THREADS, (size_t)2 * E * sizeof(int), stream>>>(chosen, T * top, top, E, row_cap, tile, row_of_pair, token_of_row,
                                                                                  expert_of_tile);
    int st = vm_launch_status();
    if (st) return st;
    const int rows = (int)need;                 // rows this step can need at most (the capacity may be larger)
    const int n_up = glu ? 2 * ff : ff;
    void* up_out = glu ? gate_up : act;
    const int up_act = glu ? -1 : act_kind;
    if (tc) {
        const size_t n = (size_t)rows * (hidden / 8), want = (n + 255) / 256;
        gather_rows_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>((const __nv_bfloat16*)x, token_of_row, rows, hidden,
                                                                                         (__nv_bfloat16*)x_sorted);
        st = vm_launch_status();
        if (st) return st;
        st = vm_tc_grouped_linear(x_sorted, hidden, w_up, rows, n_up, hidden, E, expert_of_tile, up_out, n_up, 0, up_act, err, stream);
        if (st) return st;
    } else {
        experts_up_grouped_kernel<<<dim3(rows / TM, (n_up + TN - 1) / TN), 128, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w_up,
                                                                                            token_of_row, expert_of_tile, hidden, n_up, up_act,
                                                                                            (__nv_bfloat16*)up_out);
        st = vm_launch_status();
        if (st) return st;
    }
    if (glu >= VM_GLU_SILU_WEIGHTED_INPUT) {      // (VM_GLU_SILU: unit weights here, the routing weight in the combine)
        const size_t n = (size_t)rows * ff, want = ((ff & 7) == 0 ? n / 8 : n) / 256 + 1;
        silu_weighted_rows_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, rows, ff,
                                                                                               token_of_row, row_of_pair, glu == VM_GLU_SILU ? nullptr : weight, top);
        st = vm_launch_status();
        if (st) return st;
    } else if (glu) {
        const size_t n = (size_t)rows * ff, want = ((ff & 7) == 0 ? n / 8 : n) / 256 + 1;
        glu_rows_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, n, ff, limit, alpha);
        st = vm_launch_status();
        if (st) return st;
    }
    if (tc) {
        st = vm_tc_grouped_linear(act, ff, w_down, rows, hidden, ff, E, expert_of_tile, y, hidden, 1, -1, err, stream);
        if (st) return st;
    } else {
        experts_down_grouped_kernel<<<dim3(rows / TM, (hidden + TN - 1) / TN), 128, 0, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down,
                                                                                                expert_of_tile, hidden, ff, y);
        st = vm_launch_status();
        if (st) return st;
    }
    const size_t n = (size_t)T * hidden;
    const size_t want = (n + 255) / 256;
    // (a weight that went into the expert's input is not applied again)
    experts_combine_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>(y, row_of_pair, glu == VM_GLU_SILU_WEIGHTED_INPUT ? nullptr : weight,
                                                                                         shared_y, shared_gate, T, hidden, top,
                                                                                         n_identity > 0 ? (const __nv_bfloat16*)x : nullptr, chosen, E,
                                                                                         (__nv_bfloat16*)out);
    return vm_launch_status();
}

// experts of one up matrix and an activation, every chosen index a real expert: on mma.sync tiles ...
VM_API int vm_experts_grouped(const void* x, const void* w_up, const void* w_down, const int* chosen, const float* weight, const float* shared_y,
                              const float* shared_gate, int T, int hidden, int ff, int top, int E, int act_kind, int row_cap, int* row_of_pair,
                              int* token_of_row, int* expert_of_tile, void* act, float* y, void* out, cudaStream_t stream) {
    return vm_experts_grouped_glu(x, w_up, w_down, chosen, weight, shared_y, shared_gate, T, hidden, ff, top, E, 0, act_kind, 0, 0.f, 0.f, row_cap,
                                  row_of_pair, token_of_row, expert_of_tile, nullptr, act, nullptr, y, out, nullptr, stream);
}

// ... and on tcgen05 (csrc/tc_gemm.cu, grouped): runs padded to tiles of 128 rows, the rows gathered into x_sorted [row_cap, hidden] first
VM_API int vm_experts_grouped_tc(const void* x, const void* w_up, const void* w_down, const int* chosen, const float* weight, const float* shared_y,
                                 const float* shared_gate, int T, int hidden, int ff, int top, int E, int act_kind, int row_cap, int* row_of_pair,
                                 int* token_of_row, int* expert_of_tile, void* x_sorted, void* act, float* y, void* out, int* err,
                                 cudaStream_t stream) {
    if (!x_sorted) return VM_ERR_BAD_ARG;
    return vm_experts_grouped_glu(x, w_up, w_down, chosen, weight, shared_y, shared_gate, T, hidden, ff, top, E, 0, act_kind, 0, 0.f, 0.f, row_cap,
                                  row_of_pair, token_of_row, expert_of_tile, x_sorted, act, nullptr, y, out, err, stream);
}

VM_API int vm_activation(const void* in, void* out, long long n, int kind, int act_dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t want = ((size_t)n + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (act_dtype == VM_F32) activation_kernel<float><<<blocks, 256, 0, stream>>>((const float*)in, (float*)out, (size_t)n, kind);
    else if (act_dtype == VM_BF16) activation_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, (size_t)n, kind);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}
