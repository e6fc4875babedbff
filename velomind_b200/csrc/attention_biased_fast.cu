// The bfloat16 kernels of the windowed attention with a distance bias and kept first tokens (arithmetic and arguments as in
// attention_biased.cu): prompts on the tensor cores, decode steps with the keys of one query dealt out to the warps of a CTA.
//
// Prompts.  One CTA owns 64 consecutive new tokens of one sequence and one query head; its four warps own 16 query rows
// each.  The key blocks a tile can see are the pages of the kept first tokens and the pages its rows' windows touch; they
// arrive one cache page (64 tokens of one kv head) at a time through cp.async into double-buffered shared memory, keys with
// DK values a row and values with DV.  Q K^T and P V run on mma.sync m16n8k16 (bf16 in, float32 accumulate); the bias is
// added to the float32 scores from a table by distance that the CTA builds in shared memory for its head (rel[bucket(d)],
// in the softmax's base-2 units), the mask is applied per score, the online softmax is float32.
//
// Decode steps.  One CTA per (sequence, query head); its warps take the visible keys in chunks of 32 (a key per lane,
// float32 dot products from 16-byte loads), keep a float32 online softmax each, and warp 0 joins the warps' results in warp
// order: the answer does not depend on the batch.
#include "mma.cuh"

namespace {

constexpr int BM = 64;      // query rows per CTA
constexpr int BN = 64;      // keys per block = one cache page
static_assert(BN == VM_PAGE_TOKENS, "a key block is one page");
constexpr int DIRECT_TABLE_MAX = 8192;       // distances up to which the bias is one look-up in shared memory

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool pred) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;                       // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
template <int N> __device__ __forceinline__ void cp_async_wait_n() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// VK: a token's value is the first DV values of its key row (one pool, one tile in shared memory: nothing else is fetched for the values)
template <int DK, int DV, bool VK>
__global__ void __launch_bounds__(128)
attn_biased_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                           const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ positions, const int* __restrict__ cu_tokens, int B, const float* __restrict__ rel,
                           const int* __restrict__ bucket_of, int far, int rel_rows, __nv_bfloat16* __restrict__ out, int H, int Hkv,
                           float scale_log2, int window, int keep_first, int n_pages, const float* __restrict__ sink, int* __restrict__ err) {
    constexpr int KP = DK + 8, VP = VK ? KP : DV + 8;     // padded rows: an odd number of 16-byte units -> no ldmatrix conflicts
    constexpr int KCH = DK / 8, VCH = DV / 8;   // 16-byte chunks per row
    constexpr float LOG2E = 1.4426950408889634f;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [BM][KP]
    __nv_bfloat16* sK = sQ + BM * KP;                                    // [2][BN][KP]
    __nv_bfloat16* sV = sK + 2 * BN * KP;                                // [2][BN][VP]
    float* sBias = reinterpret_cast<float*>(VK ? sV : sV + 2 * BN * VP);  // direct: [far + 1] by distance; else [rel_rows] by table row
    constexpr int THREADS = 128;
    const bool biased = rel != nullptr;
    const bool direct = biased && far + 1 <= DIRECT_TABLE_MAX;

    // ---- which 64 tokens of which sequence (the last tiles of a sequence see the most keys: they are started first)
    int tile = gridDim.x - 1 - blockIdx.x, seq = 0, t0 = 0, n_rows = 0;
    for (; seq < B; ++seq) {
        const int a = cu_tokens[seq], b = cu_tokens[seq + 1];
        const int nt = (b - a + BM - 1) / BM;
        if (tile < nt) { t0 = a + tile * BM; n_rows = min(BM, b - t0); break; }
        tile -= nt;
    }
    if (seq >= B) return;
    const int h = blockIdx.y, hk = h / (H / Hkv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos0 = positions[t0];
    const int hi = pos0 + n_rows - 1;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;      // the first row's window start: the tile's lowest
    const int blk_lo = lo / BN, blk_hi = hi / BN;
    // pages of kept first tokens that lie before the window's pages (keys below keep_first are seen by every row)
    const int kept_blocks = min((min(keep_first, lo) + BN - 1) / BN, blk_lo);
    const int n_steps = kept_blocks + (blk_hi - blk_lo + 1);
    const int* table = block_table + (size_t)seq * max_blocks;

    if (biased) {
        if (direct) for (int d = tid; d <= far; d += THREADS) sBias[d] = rel[(size_t)bucket_of[d] * H + h] * LOG2E;
        else for (int r = tid; r < rel_rows; r += THREADS) sBias[r] = rel[(size_t)r * H + h] * LOG2E;
    }
    // ---- Q tile -> shared (rows past the sequence's end are zero)
    for (int c = tid; c < BM * KCH; c += THREADS) {
        const int r = c / KCH, ch = c - r * KCH;
        cp_async16_zfill(sQ + r * KP + ch * 8, q + (size_t)(t0 + (r < n_rows ? r : 0)) * q_row_stride + (size_t)h * DK + ch * 8, r < n_rows);
    }
    auto block_of = [&](int step) { return step < kept_blocks ? step : blk_lo + (step - kept_blocks); };
    auto load_kv = [&](int step, int buf) {
        const int blk = block_of(step);
        int page = (blk < max_blocks) ? table[blk] : -1;
        const bool ok = (page >= 0 && page < n_pages);
        if (!ok) { if (tid == 0 && err) atomicExch(err, VM_ERRWORD_CACHE_READ); page = 0; }
        const __nv_bfloat16* kg = kpages + ((size_t)page * Hkv + hk) * BN * DK;
        const __nv_bfloat16* vg = vpages + ((size_t)page * Hkv + hk) * BN * DV;
        __nv_bfloat16* ks = sK + (size_t)buf * BN * KP;
        __nv_bfloat16* vs = sV + (size_t)buf * BN * VP;
        for (int c = tid; c < BN * KCH; c += THREADS) {
            const int r = c / KCH, ch = c - r * KCH;
            cp_async16_zfill(ks + r * KP + ch * 8, kg + r * DK + ch * 8, ok);
        }
        if (!VK)
            for (int c = tid; c < BN * VCH; c += THREADS) {
                const int r = c / VCH, ch = c - r * VCH;
                cp_async16_zfill(vs + r * VP + ch * 8, vg + r * DV + ch * 8, ok);
            }
    };
    load_kv(0, 0);
    vm_cp_async_commit();

    // ---- per-thread state: rows g and g+8 of the warp's 16 rows
    const int g = lane >> 2, t4 = lane & 3;
    const int row_a = warp * 16 + g, row_b = row_a + 8;
    const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;
    const int lo_a = (window > 0) ? pos_a - window + 1 : 0, lo_b = (window > 0) ? pos_b - window + 1 : 0;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    unsigned qa[DK / 16][4];
    bool q_loaded = false;
    const int warp_min_pos = pos0 + warp * 16, warp_max_pos = warp_min_pos + 15;

    for (int step = 0; step < n_steps; ++step) {
        const int buf = step & 1;
        const int blk = block_of(step);
        if (step + 1 < n_steps) load_kv(step + 1, buf ^ 1);
        vm_cp_async_commit();
        cp_async_wait_n<1>();
        __syncthreads();
        if (!q_loaded) {
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk)
                vm_ldmatrix_x4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3],
                               sQ + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * KP + kk * 16 + 8 * (lane >> 4));
            q_loaded = true;
        }
        const int key0 = blk * BN;
        // does any row of this warp see any key of this page?  (its window reaches down to warp_min_pos - window + 1)
        const bool in_reach = key0 <= warp_max_pos && (window <= 0 || key0 + BN - 1 >= warp_min_pos - window + 1 || key0 < keep_first);
        if (in_reach && warp * 16 < n_rows) {
            const __nv_bfloat16* ks = sK + (size_t)buf * BN * KP;
            const __nv_bfloat16* vs = VK ? ks : sV + (size_t)buf * BN * VP;
            float s[BN / 8][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < BN / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    vm_ldmatrix_x4(b0, b1, b2, b3, ks + (nb * 8 + (lane & 7) + 8 * (lane >> 4)) * KP + kk * 16 + 8 * ((lane >> 3) & 1));
                    vm_mma_bf16_16816(s[nb], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
                    vm_mma_bf16_16816(s[nb + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
                }
            }
            // ---- scale, bias and mask, in base-2 units: t = s * scale * log2(e) + bias * log2(e)
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + nb * 8 + 2 * t4 + e;
                    const bool see_a = key <= pos_a && (key >= lo_a || key < keep_first);
                    const bool see_b = key <= pos_b && (key >= lo_b || key < keep_first);
                    float ba = 0.f, bb = 0.f;
                    if (biased) {
                        const int da = min(max(pos_a - key, 0), far), db = min(max(pos_b - key, 0), far);
                        ba = direct ? sBias[da] : sBias[bucket_of[da]];
                        bb = direct ? sBias[db] : sBias[bucket_of[db]];
                    }
                    s[nb][e] = see_a ? fmaf(s[nb][e], scale_log2, ba) : -INFINITY;
                    s[nb][2 + e] = see_b ? fmaf(s[nb][2 + e], scale_log2, bb) : -INFINITY;
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                mx_a = fmaxf(mx_a, fmaxf(s[nb][0], s[nb][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[nb][2], s[nb][3]));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a, use_b = (mn_b == -INFINITY) ? 0.f : mn_b;   // row sees nothing yet
            const float al_a = fast_exp2(m_a - use_a), al_b = fast_exp2(m_b - use_b);
            float sum_a = 0.f, sum_b = 0.f;
            unsigned pa[BN / 16][4];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                const float p0 = fast_exp2(s[nb][0] - use_a), p1 = fast_exp2(s[nb][1] - use_a);
                const float p2 = fast_exp2(s[nb][2] - use_b), p3 = fast_exp2(s[nb][3] - use_b);
                sum_a += p0 + p1; sum_b += p2 + p3;
                pa[nb >> 1][(nb & 1) * 2 + 0] = vm_pack_bf16(p0, p1);
                pa[nb >> 1][(nb & 1) * 2 + 1] = vm_pack_bf16(p2, p3);
            }
            l_a = l_a * al_a + sum_a; l_b = l_b * al_b + sum_b;          // per-thread partial sums; quads are joined at the end
            m_a = mn_a; m_b = mn_b;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
                for (int nb = 0; nb < DV / 8; nb += 2) {
                    unsigned b0, b1, b2, b3;
                    vm_ldmatrix_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * VP + nb * 8 + 8 * (lane >> 4));
                    vm_mma_bf16_16816(o[nb], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    vm_mma_bf16_16816(o[nb + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        __syncthreads();          // everyone is done with `buf` before the next iteration's prefetch overwrites it
    }
    vm_cp_async_wait_all();

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
    if (sink) {                                            // exp(sink) joins the denominator (scores here are in base-2 units)
        const float sk = sink[h] * LOG2E;
        const float top_a = fmaxf(m_a, sk), top_b = fmaxf(m_b, sk);
        const float keep_a = fast_exp2(m_a - top_a), keep_b = fast_exp2(m_b - top_b);
        inv_a = keep_a / (l_a * keep_a + fast_exp2(sk - top_a));
        inv_b = keep_b / (l_b * keep_b + fast_exp2(sk - top_b));
    }
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
        const int d = i * 8 + 2 * t4;
        if (row_a < n_rows)
            *reinterpret_cast<unsigned*>(out + ((size_t)(t0 + row_a) * H + h) * DV + d) = vm_pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < n_rows)
            *reinterpret_cast<unsigned*>(out + ((size_t)(t0 + row_b) * H + h) * DV + d) = vm_pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

template <int DK, int DV, bool VK>
int launch_biased_prefill(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table, int max_blocks,
                          const int* positions, const int* cu_tokens, int B, int n_tiles, const float* rel, const int* bucket_of, int far,
                          int rel_rows, void* out, int H, int Hkv, float scale, int window, int keep_first, int n_pages, const float* sink, int* err,
                          cudaStream_t stream) {
    const int table = rel ? (far + 1 <= DIRECT_TABLE_MAX ? far + 1 : rel_rows) : 0;
    const size_t smem = (size_t)(BM + 2 * BN) * (DK + 8) * sizeof(__nv_bfloat16) + (VK ? 0 : (size_t)2 * BN * (DV + 8) * sizeof(__nv_bfloat16)) +
                        (size_t)table * sizeof(float);
    if (smem > 200 * 1024) return VM_ERR_UNSUPPORTED;
    static size_t raised = 48 * 1024;                       // per instantiation
    if (smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_biased_prefill_kernel<DK, DV, VK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = smem;
    }
    attn_biased_prefill_kernel<DK, DV, VK><<<dim3(n_tiles, H), 128, smem, stream>>>(
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)kpages, (const __nv_bfloat16*)vpages, block_table, max_blocks, positions,
        cu_tokens, B, rel, bucket_of, far, rel_rows, (__nv_bfloat16*)out, H, Hkv, scale * 1.4426950408889634f, window, keep_first, n_pages, sink, err);
    return vm_launch_status();
}

// ------------------------------------------------------------------------------------------------ decode steps
constexpr int DEC_WARPS = 16;

// token s of the step is sequence s's one new token
template <int VPL>      // pairs of values per lane: ceil(Dv / 64); lane owns columns 2 lane + 64 i and the next
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_biased_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ kpages,
                          const __nv_bfloat16* __restrict__ vpages, const int* __restrict__ block_table, int max_blocks,
                          const int* __restrict__ positions, const float* __restrict__ rel, const int* __restrict__ bucket_of, int far,
                          __nv_bfloat16* __restrict__ out, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages,
                          const float* __restrict__ sink, int v_stride, int* __restrict__ err) {
    extern __shared__ __align__(16) float dsm[];            // [Dk] the query; then per warp: m, l, acc[Dv]
    float* qs = dsm;
    float* part = dsm + ((Dk + 3) & ~3);
    const int seq = blockIdx.x, h = blockIdx.y, hk = h / (H / Hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int pos = positions[seq];
    const __nv_bfloat16* qrow = q + (size_t)seq * q_row_stride + (size_t)h * Dk;
    for (int d = threadIdx.x; d < Dk; d += blockDim.x) qs[d] = __bfloat162float(qrow[d]) * scale;
    __syncthreads();
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kept = min(keep_first, lo);
    // the chunks of 32 keys (at absolute multiples of 32) that hold a visible key: those of the kept tokens, then those of the window
    const int kept_chunks = min((kept + 31) / 32, lo / 32);
    const int first_window_chunk = lo / 32;
    const int n_chunks = kept_chunks + (pos / 32 - first_window_chunk + 1);
    float m = -INFINITY, l = 0.f;
    float acc[VPL][2];
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i][0] = acc[i][1] = 0.f;
    const bool vec = (Dk % 8) == 0, pairs = (Dv % 2) == 0;
    for (int c = warp; c < n_chunks; c += DEC_WARPS) {
        const int base = (c < kept_chunks ? c : first_window_chunk + (c - kept_chunks)) * 32;
        const int blk = base / VM_PAGE_TOKENS;
        const int page = (blk < max_blocks) ? block_table[(size_t)seq * max_blocks + blk] : -1;
        if (page < 0 || page >= n_pages) {
            if (lane == 0 && err) atomicExch(err, VM_ERRWORD_CACHE_READ);
            continue;
        }
        const size_t tok0 = ((size_t)page * Hkv + hk) * VM_PAGE_TOKENS + (base % VM_PAGE_TOKENS);
        const int j = base + lane;
        const bool valid = j <= pos && (j >= lo || j < kept);
        float s = -INFINITY;
        if (valid) {
            const __nv_bfloat16* krow = kpages + (tok0 + lane) * Dk;
            float a = 0.f;
            if (vec) {
#pragma unroll 4
                for (int d = 0; d < Dk; d += 8) {         // (unrolled: the row's 16-byte loads are in flight together)
                    const uint4 u = *reinterpret_cast<const uint4*>(krow + d);
                    const unsigned w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w4[k]);
                        a = fmaf(qs[d + 2 * k], __low2float(b), a);
                        a = fmaf(qs[d + 2 * k + 1], __high2float(b), a);
                    }
                }
            } else {
                for (int d = 0; d < Dk; ++d) a = fmaf(qs[d], __bfloat162float(krow[d]), a);
            }
            if (rel) a += rel[(size_t)bucket_of[min(pos - j, far)] * H + h];
            s = a;
        }
        const float m_new = fmaxf(m, vm_warp_max(s));
        if (m_new == -INFINITY) continue;
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);
        l = l * alpha + vm_warp_sum(p);
#pragma unroll
        for (int i = 0; i < VPL; ++i) { acc[i][0] *= alpha; acc[i][1] *= alpha; }
        const int cnt = min(32, pos - base + 1);
#pragma unroll 8
        for (int jj = 0; jj < cnt; ++jj) {                 // (no branch inside: the rows' loads overlap; a key that is not seen has p = 0)
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const __nv_bfloat16* vrow = vpages + (tok0 + jj) * v_stride;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int d = 2 * lane + 64 * i;
                if (pairs) {
                    if (d < Dv) {
                        const float2 v2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vrow + d));
                        acc[i][0] = fmaf(pj, v2.x, acc[i][0]);
                        acc[i][1] = fmaf(pj, v2.y, acc[i][1]);
                    }
                } else {
                    if (d < Dv) acc[i][0] = fmaf(pj, __bfloat162float(vrow[d]), acc[i][0]);
                    if (d + 1 < Dv) acc[i][1] = fmaf(pj, __bfloat162float(vrow[d + 1]), acc[i][1]);
                }
            }
        }
        m = m_new;
    }
    float* mine = part + (size_t)warp * (Dv + 2);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d < Dv) mine[2 + d] = acc[i][0];
        if (d + 1 < Dv) mine[2 + d + 1] = acc[i][1];
    }
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, part[(size_t)w * (Dv + 2)]);
    float L = 0.f;
    float res[2 * VPL];
#pragma unroll
    for (int i = 0; i < 2 * VPL; ++i) res[i] = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) {                   // in warp order: the same sum whatever else runs
        const float* pw = part + (size_t)w * (Dv + 2);
        if (pw[0] == -INFINITY) continue;
        const float f = expf(pw[0] - M);
        L = fmaf(pw[1], f, L);
#pragma unroll
        for (int i = 0; i < 2 * VPL; ++i) {
            const int d = lane + 32 * i;
            if (d < Dv) res[i] = fmaf(pw[2 + d], f, res[i]);
        }
    }
    float inv = 1.0f / L;
    if (sink) {                                            // exp(sink): one more term of the denominator, without a value
        const float sk = sink[h], top = fmaxf(M, sk), keep = expf(M - top);
        inv = keep / (L * keep + expf(sk - top));
    }
    __nv_bfloat16* orow = out + ((size_t)seq * H + h) * Dv;
#pragma unroll
    for (int i = 0; i < 2 * VPL; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) orow[d] = __float2bfloat16_rn(res[i] * inv);
    }
}

}  // namespace

// 1 if vm_attention_biased_prefill_bf16 takes keys of Dk and values of Dv
VM_API int vm_attention_biased_prefill_fits(int Dk, int Dv) {
    return (Dk == 32 || Dk == 64 || Dk == 96 || Dk == 128) && (Dv == 16 || Dv == 32 || Dv == 64 || Dv == 128) ? 1 : 0;
}

// 1 if vm_attention_sink_prefill_bf16 takes these sizes; values_in_keys: a token's value is the first Dv values of its key row
VM_API int vm_attention_sink_prefill_fits(int Dk, int Dv, int values_in_keys) {
    if (!values_in_keys) return vm_attention_biased_prefill_fits(Dk, Dv);
    const int extra = Dk - Dv;
    return (Dv == 16 || Dv == 32 || Dv == 64 || Dv == 128) && (extra == 16 || extra == 32 || extra == 64) ? 1 : 0;
}

// n_tiles = sum over the step's sequences of ceil(new tokens / 64), computed by the host.  rel float32 [rel_rows, H] with bucket_of
// int32 [far + 1], or both null.  q rows of stride q_row_stride (a multiple of 8), out [T, H * Dv].
VM_API int vm_attention_biased_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                            int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, const float* rel,
                                            const int* bucket_of, int far, int rel_rows, void* out, int H, int Hkv, int Dk, int Dv, float scale,
                                            int window, int keep_first, int n_pages, int* err, cudaStream_t stream) {
    return vm_attention_sink_prefill_bf16(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B, n_tiles, rel, bucket_of, far,
                                          rel_rows, nullptr, 0, out, H, Hkv, Dk, Dv, scale, window, keep_first, n_pages, err, stream);
}

// The same with a sink (float32 [H], null: none; exp(sink[h]) joins head h's denominator) and, with vpages == kpages and
// v_row_stride == Dk, values that are the first Dv values of the key rows (sizes: vm_attention_sink_prefill_fits).
VM_API int vm_attention_sink_prefill_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                          int max_blocks, const int* positions, const int* cu_tokens, int B, int n_tiles, const float* rel,
                                          const int* bucket_of, int far, int rel_rows, const float* sink, int v_row_stride, void* out, int H, int Hkv,
                                          int Dk, int Dv, float scale, int window, int keep_first, int n_pages, int* err, cudaStream_t stream) {
    if (n_tiles <= 0 || B <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || (q_row_stride % 8) != 0 || window < 0 || keep_first < 0) return VM_ERR_UNSUPPORTED;
    if ((rel != nullptr) != (bucket_of != nullptr) || (rel && (far < 0 || rel_rows <= 0))) return VM_ERR_BAD_ARG;
    const bool in_keys = vpages == kpages && v_row_stride == Dk && Dv < Dk;
    if (!in_keys && v_row_stride != 0 && v_row_stride != Dv) return VM_ERR_UNSUPPORTED;
#define VM_BP(K, V, IN)                                                                                                                        \
    if (Dk == K && Dv == V && in_keys == IN)                                                                                                   \
        return launch_biased_prefill<K, V, IN>(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, cu_tokens, B, n_tiles, rel, \
                                               bucket_of, far, rel_rows, out, H, Hkv, scale, window, keep_first, n_pages, sink, err, stream);
    VM_BP(32, 16, false) VM_BP(32, 32, false) VM_BP(32, 64, false) VM_BP(32, 128, false)
    VM_BP(64, 16, false) VM_BP(64, 32, false) VM_BP(64, 64, false) VM_BP(64, 128, false)
    VM_BP(96, 16, false) VM_BP(96, 32, false) VM_BP(96, 64, false) VM_BP(96, 128, false)
    VM_BP(128, 16, false) VM_BP(128, 32, false) VM_BP(128, 64, false) VM_BP(128, 128, false)
    VM_BP(32, 16, true) VM_BP(48, 16, true) VM_BP(80, 16, true)
    VM_BP(48, 32, true) VM_BP(64, 32, true) VM_BP(96, 32, true)
    VM_BP(80, 64, true) VM_BP(96, 64, true) VM_BP(128, 64, true)
    VM_BP(144, 128, true) VM_BP(160, 128, true) VM_BP(192, 128, true)
#undef VM_BP
    return VM_ERR_UNSUPPORTED;
}

// one new token per sequence (token s belongs to sequence s); any Dk up to 1,024, Dv up to 256
VM_API int vm_attention_biased_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                           int max_blocks, const int* positions, const float* rel, const int* bucket_of, int far, void* out, int B,
                                           int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first, int n_pages, int* err,
                                           cudaStream_t stream) {
    return vm_attention_sink_decode_bf16(q, q_row_stride, kpages, vpages, block_table, max_blocks, positions, rel, bucket_of, far, nullptr, 0, out, B, H, Hkv,
                                         Dk, Dv, scale, window, keep_first, n_pages, err, stream);
}

// the same with a sink and a stride between value rows (0: Dv), as vm_attention_sink_generic
VM_API int vm_attention_sink_decode_bf16(const void* q, int q_row_stride, const void* kpages, const void* vpages, const int* block_table,
                                         int max_blocks, const int* positions, const float* rel, const int* bucket_of, int far, const float* sink,
                                         int v_row_stride, void* out, int B, int H, int Hkv, int Dk, int Dv, float scale, int window, int keep_first,
                                         int n_pages, int* err, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || Dk <= 0 || Dk > 1024 || Dv <= 0 || Dv > 256 || window < 0 || keep_first < 0) return VM_ERR_UNSUPPORTED;
    if ((rel != nullptr) != (bucket_of != nullptr) || (rel && far < 0)) return VM_ERR_BAD_ARG;
    if (H > 65535) return VM_ERR_UNSUPPORTED;
    const int v_stride = v_row_stride > 0 ? v_row_stride : Dv;
    if (v_stride < Dv || ((Dv % 2) == 0 && (v_stride % 2) != 0)) return VM_ERR_BAD_ARG;
    const size_t smem = ((size_t)((Dk + 3) & ~3) + (size_t)DEC_WARPS * (Dv + 2)) * sizeof(float);
    const dim3 grid(B, H);
    cudaError_t e;
#define VM_BD(V)                                                                                                                              \
    case V:                                                                                                                                   \
        e = vm_launch_pdl(attn_biased_decode_kernel<V>, grid, dim3(DEC_WARPS * 32), smem, stream, (const __nv_bfloat16*)q, q_row_stride,      \
                          (const __nv_bfloat16*)kpages, (const __nv_bfloat16*)vpages, block_table, max_blocks, positions, rel, bucket_of, far, \
                          (__nv_bfloat16*)out, H, Hkv, Dk, Dv, scale, window, keep_first, n_pages, sink, v_stride, err);                       \
        break;
    switch ((Dv + 63) / 64) {
        VM_BD(1) VM_BD(2) VM_BD(3) VM_BD(4)
        default: return VM_ERR_UNSUPPORTED;
    }
#undef VM_BD
    (void)e;
    return vm_launch_status();
}
