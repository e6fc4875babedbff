// The two norms of a latent-attention layer and the cache write of its key/value latent, one launch.
//
// A latent-attention layer projects its input down twice: to a query latent and to a key/value latent.  Both are
// RMS-normed with a learned scale.  The query latent goes on to the query up-projection; the key/value latent is all the
// layer remembers of a token: one row per token in the paged cache (a group with one "head" of the latent's size and no
// second row), from which keys and values are made again, or, with the up-projections moved to the query's and the
// output's side, never made at all.
//
// Input: the down projections' float32 result [T, ld]: columns [0, q_rank) the query latent, [q_rank, q_rank + kv_rank) the
// key/value latent (absent for a layer that reads another layer's latents).  Statistics in float32.  One block per token.
//
// A layer with rotary positions keeps `rot_dim` more values per token behind the latent: columns [q_rank + kv_rank, q_rank +
// kv_rank + rot_dim) of the input, not normed, one key part that all heads share; its first `rotary_dim` values are turned by the
// token's position (angle and its sine and cosine in float32) before they are written.  A cache row then has kv_rank + rot_dim values.
#include "common.cuh"

template <typename T>
__global__ void latent_norm_write_kernel(const float* __restrict__ down, int ld, int q_rank, int kv_rank, const float* __restrict__ wq,
                                         const float* __restrict__ wkv, float eps, T* __restrict__ cq, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_blocks,
                                         T* __restrict__ pages, int n_pages, int rot_dim, int rotary_dim, const float* __restrict__ inv_freq,
                                         int pairing, int* __restrict__ err) {
    __shared__ float red[32];
    vm_pdl_launch_dependents();
    vm_pdl_wait();
    const int t = blockIdx.x;
    const float* row = down + (size_t)t * ld;
    {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss += row[i] * row[i];
        ss = vm_block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = vm_from_float<T>(row[i] * inv * wq[i]);
    }
    if (!pages) return;
    const float* lat = row + q_rank;
    float ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss += lat[i] * lat[i];
    ss = vm_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    const int pos = positions[t], seq = seq_of_token[t];
    const int blk = pos / VM_PAGE_TOKENS;
    const int page = blk < max_blocks ? block_table[(size_t)seq * max_blocks + blk] : -1;
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0 && err) atomicExch(err, VM_ERRWORD_CACHE_WRITE);
        return;
    }
    T* dst = pages + ((size_t)page * VM_PAGE_TOKENS + (pos % VM_PAGE_TOKENS)) * (kv_rank + rot_dim);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = vm_from_float<T>(lat[i] * inv * wkv[i]);
    const float* kr = lat + kv_rank;
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half + (rot_dim - rotary_dim); i += blockDim.x) {
        if (i >= half) {                                   // behind the rotated values: as projected
            const int k = rotary_dim + (i - half);
            dst[kv_rank + k] = vm_from_float<T>(kr[k]);
            continue;
        }
        const int ia = pairing == VM_PAIR_INTERLEAVED ? 2 * i : i, ib = pairing == VM_PAIR_INTERLEAVED ? 2 * i + 1 : i + half;
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float u = kr[ia], v = kr[ib];
        dst[kv_rank + ia] = vm_from_float<T>(u * cs - v * sn);
        dst[kv_rank + ib] = vm_from_float<T>(v * cs + u * sn);
    }
}

// pages [n_pages, VM_PAGE_TOKENS, kv_rank + rot_dim]; inv_freq float32 [rotary_dim / 2]
VM_API int vm_latent_rope_norm_write(const float* down, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps, void* cq,
                                     const int* positions, const int* seq_of_token, const int* block_table, int max_blocks, void* pages,
                                     int n_pages, int rot_dim, int rotary_dim, const float* inv_freq, int pairing, int T, int act_dtype, int* err,
                                     cudaStream_t stream) {
    if (T <= 0) return 0;
    if (q_rank <= 0 || kv_rank <= 0 || rot_dim < 0 || ld < q_rank + (pages ? kv_rank + rot_dim : 0)) return VM_ERR_BAD_ARG;
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > rot_dim || (rotary_dim > 0 && !inv_freq)) return VM_ERR_BAD_ARG;
    const int widest = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = widest >= 512 ? 256 : 128;
    if (act_dtype == VM_F32)
        vm_launch_pdl(latent_norm_write_kernel<float>, dim3(T), dim3(threads), 0, stream, down, ld, q_rank, kv_rank, wq, wkv, eps, (float*)cq, positions,
                      seq_of_token, block_table, max_blocks, (float*)pages, n_pages, rot_dim, rotary_dim, inv_freq, pairing, err);
    else if (act_dtype == VM_BF16)
        vm_launch_pdl(latent_norm_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, down, ld, q_rank, kv_rank, wq, wkv, eps,
                      (__nv_bfloat16*)cq, positions, seq_of_token, block_table, max_blocks, (__nv_bfloat16*)pages, n_pages, rot_dim, rotary_dim, inv_freq,
                      pairing, err);
    else return VM_ERR_UNSUPPORTED;
    return vm_launch_status();
}

VM_API int vm_latent_norm_write(const float* down, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps, void* cq,
                                const int* positions, const int* seq_of_token, const int* block_table, int max_blocks, void* pages,
                                int n_pages, int T, int act_dtype, int* err, cudaStream_t stream) {
    return vm_latent_rope_norm_write(down, ld, q_rank, kv_rank, wq, wkv, eps, cq, positions, seq_of_token, block_table, max_blocks, pages, n_pages, 0, 0,
                                     nullptr, VM_PAIR_HALF_SPLIT, T, act_dtype, err, stream);
}
