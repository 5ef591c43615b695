// Sliding-window attention that also sees one pooled key/value per block of old tokens.
//
// Position i of a sequence sees the tokens j with 0 <= i - j < window and, in the same softmax,
// for every block b of `pool` consecutive positions with b * pool + pool - 1 <= i - window the
// mean of the block's cached keys and the mean of its cached values.  Three kernels:
//
//   store_kv   a step's keys and values into the paged cache (as projected: no norm, no rotation)
//   pool_kv    for every row of the step whose position ends a block: the block's means, in float,
//              from the cache (the block may have begun in an earlier step) into the pooled cache
//   attention  the general kernel: one warp per (row, query head); a lane takes a key, forms the
//              whole dot product, the warp keeps a running maximum and sum, and the lanes then
//              share the value channels.  Pooled blocks come first, then the window's tokens, in
//              position order, 32 at a time from the start of each list: a row's result does not
//              depend on the batch or on how the sequence was cut.  Scores, softmax and the
//              output sum are float.
//
// Cache rows: row(p) = table[p / page_size] * page_size + p % page_size, as everywhere; a pooled
// cache holds row b of a sequence at the same formula over its own table.
#include "common.cuh"

template <typename AT>
__global__ void store_kv_kernel(const AT* __restrict__ k, long long k_ld, const AT* __restrict__ v, long long v_ld,
                                const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                const int* __restrict__ table, int table_width, AT* __restrict__ k_cache, AT* __restrict__ v_cache,
                                int kv_heads, int dim, int vdim, int page_size) {
    pdl_begin();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int page = table[(size_t)seq_of_token[t] * table_width + pos / page_size];
    if (page < 0) return;
    const size_t row = (size_t)page * page_size + pos % page_size;
    const int kw = kv_heads * dim, vw = kv_heads * vdim;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) k_cache[row * kw + c] = k[(size_t)t * k_ld + c];
    for (int c = threadIdx.x; c < vw; c += blockDim.x) v_cache[row * vw + c] = v[(size_t)t * v_ld + c];
}

SHISO_API int shiso_store_kv(const void* k, long long k_ld, const void* v, long long v_ld, int act_dtype, const int* positions,
                             const int* seq_of_token, const int* table, int table_width, void* k_cache, void* v_cache, int tokens,
                             int kv_heads, int dim, int vdim, int page_size, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (act_dtype == SHISO_F32)
        launch_kernel(store_kv_kernel<float>, tokens, 128, 0, stream, (const float*)k, k_ld, (const float*)v, v_ld, positions,
                      seq_of_token, table, table_width, (float*)k_cache, (float*)v_cache, kv_heads, dim, vdim, page_size);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(store_kv_kernel<__nv_bfloat16>, tokens, 128, 0, stream, (const __nv_bfloat16*)k, k_ld, (const __nv_bfloat16*)v,
                      v_ld, positions, seq_of_token, table, table_width, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, kv_heads,
                      dim, vdim, page_size);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

template <typename AT>
__global__ void pool_kv_kernel(const AT* __restrict__ k_cache, const AT* __restrict__ v_cache, const int* __restrict__ table,
                               float* __restrict__ pooled_k, float* __restrict__ pooled_v, const int* __restrict__ pooled_table,
                               int table_width, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                               int kw, int vw, int page_size, int pool) {
    pdl_begin();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if ((pos + 1) % pool) return;
    const int seq = seq_of_token[t];
    const int block = pos / pool;
    const int to_page = pooled_table[(size_t)seq * table_width + block / page_size];
    if (to_page < 0) return;
    const size_t to_row = (size_t)to_page * page_size + block % page_size;
    const int* pages = table + (size_t)seq * table_width;
    const int first = pos + 1 - pool;
    for (int c = threadIdx.x; c < kw + vw; c += blockDim.x) {
        const bool key = c < kw;
        const AT* cache = key ? k_cache : v_cache;
        const int width = key ? kw : vw, col = key ? c : c - kw;
        float sum = 0.0f;
        for (int p = first; p <= pos; ++p) {
            const int page = pages[p / page_size];
            sum += page < 0 ? 0.0f : to_f32(cache[((size_t)page * page_size + p % page_size) * width + col]);
        }
        (key ? pooled_k : pooled_v)[to_row * width + col] = sum / (float)pool;
    }
}

SHISO_API int shiso_pool_kv(const void* k_cache, const void* v_cache, int cache_dtype, const int* table, float* pooled_k,
                            float* pooled_v, const int* pooled_table, int table_width, const int* positions,
                            const int* seq_of_token, int tokens, int kv_heads, int dim, int vdim, int page_size, int pool,
                            cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (pool < 1) return SHISO_ERR_SHAPE;
    if (cache_dtype == SHISO_F32)
        launch_kernel(pool_kv_kernel<float>, tokens, 128, 0, stream, (const float*)k_cache, (const float*)v_cache, table, pooled_k,
                      pooled_v, pooled_table, table_width, positions, seq_of_token, kv_heads * dim, kv_heads * vdim, page_size, pool);
    else if (cache_dtype == SHISO_BF16)
        launch_kernel(pool_kv_kernel<__nv_bfloat16>, tokens, 128, 0, stream, (const __nv_bfloat16*)k_cache,
                      (const __nv_bfloat16*)v_cache, table, pooled_k, pooled_v, pooled_table, table_width, positions, seq_of_token,
                      kv_heads * dim, kv_heads * vdim, page_size, pool);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

constexpr int PWA_WARPS = 4;
constexpr int PWA_MAX_DIM = 256;

// One list of keys (pooled blocks or tokens) folded into a warp's running softmax.
template <typename CT>
__device__ __forceinline__ void fold_keys(const CT* __restrict__ k_cache, const CT* __restrict__ v_cache, const int* pages,
                                          int first, int count, int page_size, int kv_heads, int kv_head, int dim, int vdim,
                                          const float* q, float scale, float& running_max, float& running_sum,
                                          float (&acc)[PWA_MAX_DIM / 32], int lane) {
    for (int base = 0; base < count; base += 32) {
        const int n = min(32, count - base);
        long long row = -1;
        float score = -INFINITY;
        if (lane < n) {
            const int p = first + base + lane;
            const int page = pages[p / page_size];
            if (page >= 0) {
                row = (long long)page * page_size + p % page_size;
                const CT* key = k_cache + ((size_t)row * kv_heads + kv_head) * dim;
                float dot = 0.0f;
                for (int c = 0; c < dim; ++c) dot += q[c] * to_f32(key[c]);
                score = dot * scale;
            }
        }
        const float new_max = fmaxf(running_max, warp_max(score));
        if (new_max == -INFINITY) continue;
        const float keep = expf(running_max - new_max);  // 0 while nothing was seen
        const float weight = row >= 0 ? expf(score - new_max) : 0.0f;
        running_sum = running_sum * keep + warp_sum(weight);
        running_max = new_max;
#pragma unroll
        for (int e = 0; e < PWA_MAX_DIM / 32; ++e) acc[e] *= keep;
        for (int kk = 0; kk < n; ++kk) {
            const float w = __shfl_sync(0xffffffffu, weight, kk);
            const long long r = __shfl_sync(0xffffffffu, row, kk);
            if (r < 0) continue;
            const CT* value = v_cache + ((size_t)r * kv_heads + kv_head) * vdim;
#pragma unroll
            for (int e = 0; e < PWA_MAX_DIM / 32; ++e) {
                const int c = e * 32 + lane;
                if (c < vdim) acc[e] += w * to_f32(value[c]);
            }
        }
    }
}

template <typename AT>
__global__ void __launch_bounds__(PWA_WARPS * 32)
pooled_window_attention_kernel(const AT* __restrict__ q, long long q_ld, const AT* __restrict__ k_cache,
                               const AT* __restrict__ v_cache, const int* __restrict__ table, const float* __restrict__ pooled_k,
                               const float* __restrict__ pooled_v, const int* __restrict__ pooled_table, int table_width,
                               const int* __restrict__ positions, const int* __restrict__ seq_of_token, AT* __restrict__ out,
                               long long out_ld, int tokens, int heads, int kv_heads, int dim, int vdim, int page_size, float scale,
                               int window, int pool, float out_scale) {
    __shared__ float sq[PWA_WARPS][PWA_MAX_DIM];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * PWA_WARPS + warp;
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const int kv_head = head / (heads / kv_heads);
    for (int c = lane; c < dim; c += 32) sq[warp][c] = to_f32(q[(size_t)t * q_ld + (size_t)head * dim + c]);
    __syncwarp();
    const int pos = positions[t], seq = seq_of_token[t];
    const int first = max(0, pos - window + 1);
    const int behind = pos - window + 1;  // positions before this one lie behind the window
    const int blocks = behind > 0 ? behind / pool : 0;
    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[PWA_MAX_DIM / 32];
#pragma unroll
    for (int e = 0; e < PWA_MAX_DIM / 32; ++e) acc[e] = 0.0f;
    fold_keys<float>(pooled_k, pooled_v, pooled_table + (size_t)seq * table_width, 0, blocks, page_size, kv_heads, kv_head, dim, vdim,
                     sq[warp], scale, running_max, running_sum, acc, lane);
    fold_keys<AT>(k_cache, v_cache, table + (size_t)seq * table_width, first, pos - first + 1, page_size, kv_heads, kv_head, dim, vdim,
                  sq[warp], scale, running_max, running_sum, acc, lane);
    const float inv = running_sum > 0.0f ? out_scale / running_sum : 0.0f;
#pragma unroll
    for (int e = 0; e < PWA_MAX_DIM / 32; ++e) {
        const int c = e * 32 + lane;
        if (c < vdim) out[(size_t)t * out_ld + (size_t)head * vdim + c] = from_f32<AT>(acc[e] * inv);
    }
}

SHISO_API int shiso_pooled_window_attention(const void* q, long long q_ld, int act_dtype, const void* k_cache, const void* v_cache,
                                            const int* table, const float* pooled_k, const float* pooled_v,
                                            const int* pooled_table, int table_width, const int* positions,
                                            const int* seq_of_token, void* out, long long out_ld, int tokens, int heads,
                                            int kv_heads, int dim, int vdim, int page_size, float scale, int window, int pool,
                                            float out_scale, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (dim > PWA_MAX_DIM || vdim > PWA_MAX_DIM || kv_heads <= 0 || heads % kv_heads || window < 1 || pool < 1) return SHISO_ERR_SHAPE;
    const unsigned blocks = ceil_div_u((long long)tokens * heads, PWA_WARPS);
    if (act_dtype == SHISO_F32)
        launch_kernel(pooled_window_attention_kernel<float>, blocks, PWA_WARPS * 32, 0, stream, (const float*)q, q_ld,
                      (const float*)k_cache, (const float*)v_cache, table, pooled_k, pooled_v, pooled_table, table_width, positions,
                      seq_of_token, (float*)out, out_ld, tokens, heads, kv_heads, dim, vdim, page_size, scale, window, pool, out_scale);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(pooled_window_attention_kernel<__nv_bfloat16>, blocks, PWA_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_ld,
                      (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, table, pooled_k, pooled_v, pooled_table,
                      table_width, positions, seq_of_token, (__nv_bfloat16*)out, out_ld, tokens, heads, kv_heads, dim, vdim,
                      page_size, scale, window, pool, out_scale);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
