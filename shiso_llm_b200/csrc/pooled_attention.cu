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
    // (the row's columns are spread over blockIdx.y: few rows of a step end a block)
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < kw + vw; c += gridDim.y * blockDim.x) {
        const bool key = c < kw;
        const AT* cache = key ? k_cache : v_cache;
        const int width = key ? kw : vw, col = key ? c : c - kw;
        float sum = 0.0f;
#pragma unroll 4
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
    const dim3 grid(tokens, ceil_div_u((long long)kv_heads * (dim + vdim), 128) < 16 ? ceil_div_u((long long)kv_heads * (dim + vdim), 128) : 16);
    if (cache_dtype == SHISO_F32)
        launch_kernel(pool_kv_kernel<float>, grid, 128, 0, stream, (const float*)k_cache, (const float*)v_cache, table, pooled_k,
                      pooled_v, pooled_table, table_width, positions, seq_of_token, kv_heads * dim, kv_heads * vdim, page_size, pool);
    else if (cache_dtype == SHISO_BF16)
        launch_kernel(pool_kv_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)k_cache,
                      (const __nv_bfloat16*)v_cache, table, pooled_k, pooled_v, pooled_table, table_width, positions, seq_of_token,
                      kv_heads * dim, kv_heads * vdim, page_size, pool);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

constexpr int PWA_WARPS = 8;
constexpr int PWA_MAX_DIM = 256;
constexpr int PWA_PAIRS = PWA_MAX_DIM / 64;  // a lane holds the value channels 2 * lane + 64 * e and the one after

__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// q . key over `dim` channels; 16-byte loads of the key where its rows allow them.
__device__ __forceinline__ float dot_key(const float* __restrict__ q, const float* __restrict__ key, int dim, bool wide) {
    float dot = 0.0f;
    if (wide) {
#pragma unroll 4
        for (int c = 0; c < dim; c += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(key + c);
            dot += q[c] * k4.x + q[c + 1] * k4.y + q[c + 2] * k4.z + q[c + 3] * k4.w;
        }
    } else {
        for (int c = 0; c < dim; ++c) dot += q[c] * key[c];
    }
    return dot;
}
__device__ __forceinline__ float dot_key(const float* __restrict__ q, const __nv_bfloat16* __restrict__ key, int dim, bool wide) {
    float dot = 0.0f;
    if (wide) {
#pragma unroll 4
        for (int c = 0; c < dim; c += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(key + c);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                dot += q[c + 2 * i] * __uint_as_float(w[i] << 16);
                dot += q[c + 2 * i + 1] * __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    } else {
        for (int c = 0; c < dim; ++c) dot += q[c] * __bfloat162float(key[c]);
    }
    return dot;
}

// A warp folds 32 keys of one list (pooled blocks or tokens), starting at list index `base`, into
// its running softmax: a lane takes a key and forms the whole dot product; the lanes then share
// the value channels.
template <typename CT>
__device__ __forceinline__ void fold_chunk(const CT* __restrict__ k_cache, const CT* __restrict__ v_cache, const int* pages,
                                           int first, int count, int base, int page_size, int kv_heads, int kv_head, int dim,
                                           int vdim, const float* q, float scale, float& running_max, float& running_sum,
                                           float (&acc)[PWA_PAIRS][2], int lane, float* run_weight, long long* run_row) {
    const int n = min(32, count - base);
    long long row = -1;
    float score = -INFINITY;
    if (lane < n) {
        const int p = first + base + lane;
        const int page = pages[p / page_size];
        if (page >= 0) {
            row = (long long)page * page_size + p % page_size;
            const bool wide = (dim * (int)sizeof(CT)) % 16 == 0;
            score = dot_key(q, k_cache + ((size_t)row * kv_heads + kv_head) * dim, dim, wide) * scale;
        }
    }
    const float new_max = fmaxf(running_max, warp_max(score));
    if (new_max == -INFINITY) return;
    const float keep = expf(running_max - new_max);  // 0 while nothing was seen
    const float weight = row >= 0 ? expf(score - new_max) : 0.0f;
    running_sum = running_sum * keep + warp_sum(weight);
    running_max = new_max;
#pragma unroll
    for (int e = 0; e < PWA_PAIRS; ++e) {
        acc[e][0] *= keep;
        acc[e][1] *= keep;
    }
    const bool paired = vdim % 2 == 0;
    // the run's weights and rows go through the warp's shared memory: every lane reads them all
    __syncwarp();
    run_weight[lane] = weight;
    run_row[lane] = row >= 0 ? ((long long)row * kv_heads + kv_head) * vdim : -1;
    __syncwarp();
    // (unrolled and without a branch between two loads - a key the run does not have reads row 0 with
    // weight zero - so that the value rows of eight keys are asked for together)
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
        const long long r = run_row[kk];
        const bool live = r >= 0;
        const float w = live ? run_weight[kk] : 0.0f;
        const CT* value = v_cache + (live ? r : 0);
#pragma unroll
        for (int e = 0; e < PWA_PAIRS; ++e) {
            const int c = e * 64 + 2 * lane;
            if (paired) {
                if (c < vdim) {
                    const float2 v2 = load_pair(value + c);
                    acc[e][0] += live ? w * v2.x : 0.0f;
                    acc[e][1] += live ? w * v2.y : 0.0f;
                }
            } else {
                if (c < vdim) acc[e][0] += live ? w * to_f32(value[c]) : 0.0f;
                if (c + 1 < vdim) acc[e][1] += live ? w * to_f32(value[c + 1]) : 0.0f;
            }
        }
    }
}

// One CTA per (row, query head).  The two lists - pooled blocks, then the window's tokens - are cut
// into runs of 32 keys from each list's start; run c belongs to warp c % 8, and the warps' partial
// softmaxes are merged in warp order.  What a row adds up, and in which order, depends on its
// position only.
template <typename AT>
__global__ void __launch_bounds__(PWA_WARPS * 32)
pooled_window_attention_kernel(const AT* __restrict__ q, long long q_ld, const AT* __restrict__ k_cache,
                               const AT* __restrict__ v_cache, const int* __restrict__ table, const float* __restrict__ pooled_k,
                               const float* __restrict__ pooled_v, const int* __restrict__ pooled_table, int table_width,
                               const int* __restrict__ positions, const int* __restrict__ seq_of_token, AT* out,
                               long long out_ld, int heads, int kv_heads, int dim, int vdim,
                               int page_size, float scale, int window, int pool, float out_scale) {
    __shared__ float sq[PWA_MAX_DIM];
    __shared__ float run_weight[PWA_WARPS][32];
    __shared__ long long run_row[PWA_WARPS][32];
    __shared__ float part_max[PWA_WARPS], part_sum[PWA_WARPS];
    __shared__ float part_acc[PWA_WARPS][PWA_MAX_DIM];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x / heads, head = blockIdx.x % heads;
    const int kv_head = head / (heads / kv_heads);
    for (int c = threadIdx.x; c < dim; c += blockDim.x) sq[c] = to_f32(q[(size_t)t * q_ld + (size_t)head * dim + c]);
    __syncthreads();
    const int pos = positions[t], seq = seq_of_token[t];
    const int first = max(0, pos - window + 1);
    const int behind = pos - window + 1;  // positions before this one lie behind the window
    const int blocks = behind > 0 ? behind / pool : 0;
    const int tokens_seen = pos - first + 1;
    const int pooled_runs = (blocks + 31) / 32, token_runs = (tokens_seen + 31) / 32;
    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[PWA_PAIRS][2];
#pragma unroll
    for (int e = 0; e < PWA_PAIRS; ++e) acc[e][0] = acc[e][1] = 0.0f;
    for (int run = warp; run < pooled_runs + token_runs; run += PWA_WARPS) {
        if (run < pooled_runs)
            fold_chunk<float>(pooled_k, pooled_v, pooled_table + (size_t)seq * table_width, 0, blocks, run * 32, page_size, kv_heads,
                              kv_head, dim, vdim, sq, scale, running_max, running_sum, acc, lane, run_weight[warp], run_row[warp]);
        else
            fold_chunk<AT>(k_cache, v_cache, table + (size_t)seq * table_width, first, tokens_seen, (run - pooled_runs) * 32,
                           page_size, kv_heads, kv_head, dim, vdim, sq, scale, running_max, running_sum, acc, lane, run_weight[warp],
                           run_row[warp]);
    }
    if (lane == 0) {
        part_max[warp] = running_max;
        part_sum[warp] = running_sum;
    }
#pragma unroll
    for (int e = 0; e < PWA_PAIRS; ++e) {
        const int c = e * 64 + 2 * lane;
        if (c < PWA_MAX_DIM) {
            part_acc[warp][c] = acc[e][0];
            part_acc[warp][c + 1] = acc[e][1];
        }
    }
    __syncthreads();
    AT* dst = out + (size_t)t * out_ld + (size_t)head * vdim;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < PWA_WARPS; ++w) top = fmaxf(top, part_max[w]);
    if (top == -INFINITY) {
        for (int c = threadIdx.x; c < vdim; c += blockDim.x) dst[c] = from_f32<AT>(0.0f);
        return;
    }
    float factor[PWA_WARPS];
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < PWA_WARPS; ++w) {
        factor[w] = part_max[w] == -INFINITY ? 0.0f : expf(part_max[w] - top);
        total += part_sum[w] * factor[w];
    }
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < PWA_WARPS; ++w) sum += part_acc[w][c] * factor[w];
        dst[c] = from_f32<AT>(sum / total * out_scale);
    }
}

// The pooled blocks alone, folded into a softmax whose window part another kernel has taken:
// `out` holds that part's normalised result, already times out_scale, and `seen` the logarithm of
// its sum; a row that sees no block is finished as it stands.  A row sees few
// blocks (its position / pool at most), so a warp takes a (row, head) by itself, eight to a CTA.
template <typename AT>
__global__ void __launch_bounds__(PWA_WARPS * 32)
pooled_blocks_merge_kernel(const AT* __restrict__ q, long long q_ld, const float* __restrict__ pooled_k,
                           const float* __restrict__ pooled_v, const int* __restrict__ pooled_table, int table_width,
                           const int* __restrict__ positions, const int* __restrict__ seq_of_token, AT* out, long long out_ld,
                           const float* __restrict__ seen, int tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                           float scale, int window, int pool, float out_scale) {
    __shared__ float sq[PWA_WARPS][PWA_MAX_DIM];
    __shared__ float run_weight[PWA_WARPS][32];
    __shared__ long long run_row[PWA_WARPS][32];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * PWA_WARPS + warp;
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const int kv_head = head / (heads / kv_heads);
    const int pos = positions[t], seq = seq_of_token[t];
    const int behind = pos - window + 1;
    const int blocks = behind > 0 ? behind / pool : 0;
    if (blocks <= 0) return;
    AT* dst = out + (size_t)t * out_ld + (size_t)head * vdim;
    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[PWA_PAIRS][2];
#pragma unroll
    for (int e = 0; e < PWA_PAIRS; ++e) acc[e][0] = acc[e][1] = 0.0f;
    {
        for (int c = lane; c < dim; c += 32) sq[warp][c] = to_f32(q[(size_t)t * q_ld + (size_t)head * dim + c]);
        __syncwarp();
        for (int base = 0; base < blocks; base += 32)
            fold_chunk<float>(pooled_k, pooled_v, pooled_table + (size_t)seq * table_width, 0, blocks, base, page_size, kv_heads,
                              kv_head, dim, vdim, sq[warp], scale, running_max, running_sum, acc, lane, run_weight[warp], run_row[warp]);
    }
    const float before = seen[(size_t)t * heads + head];
    const float top = fmaxf(before, running_max);
    const float old = top == -INFINITY ? 0.0f : expf(before - top);
    const float fresh = running_max == -INFINITY ? 0.0f : expf(running_max - top);
    const float total = old + running_sum * fresh;
#pragma unroll
    for (int e = 0; e < PWA_PAIRS; ++e) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = e * 64 + 2 * lane + h;
            if (c < vdim) {
                const float sum = old * to_f32(dst[c]) + acc[e][h] * fresh * out_scale;
                dst[c] = from_f32<AT>(total > 0.0f ? sum / total : 0.0f);
            }
        }
    }
}

SHISO_API int shiso_pooled_window_attention(const void* q, long long q_ld, int act_dtype, const void* k_cache, const void* v_cache,
                                            const int* table, const float* pooled_k, const float* pooled_v,
                                            const int* pooled_table, int table_width, const int* positions,
                                            const int* seq_of_token, void* out, long long out_ld, const float* seen, int tokens,
                                            int heads, int kv_heads, int dim, int vdim, int page_size, float scale, int window,
                                            int pool, float out_scale, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (dim > PWA_MAX_DIM || vdim > PWA_MAX_DIM || kv_heads <= 0 || heads % kv_heads || window < 1 || pool < 1) return SHISO_ERR_SHAPE;
    if ((long long)tokens * heads > 0x7fffffffLL) return SHISO_ERR_SHAPE;
    const unsigned blocks = (unsigned)tokens * heads;
    if (seen) {
        const unsigned few = ceil_div_u((long long)tokens * heads, PWA_WARPS);
        if (act_dtype == SHISO_F32)
            launch_kernel(pooled_blocks_merge_kernel<float>, few, PWA_WARPS * 32, 0, stream, (const float*)q, q_ld, pooled_k, pooled_v,
                          pooled_table, table_width, positions, seq_of_token, (float*)out, out_ld, seen, tokens, heads, kv_heads, dim,
                          vdim, page_size, scale, window, pool, out_scale);
        else if (act_dtype == SHISO_BF16)
            launch_kernel(pooled_blocks_merge_kernel<__nv_bfloat16>, few, PWA_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_ld,
                          pooled_k, pooled_v, pooled_table, table_width, positions, seq_of_token, (__nv_bfloat16*)out, out_ld, seen,
                          tokens, heads, kv_heads, dim, vdim, page_size, scale, window, pool, out_scale);
        else
            return SHISO_ERR_DTYPE;
        return launch_status();
    }
    if (act_dtype == SHISO_F32)
        launch_kernel(pooled_window_attention_kernel<float>, blocks, PWA_WARPS * 32, 0, stream, (const float*)q, q_ld,
                      (const float*)k_cache, (const float*)v_cache, table, pooled_k, pooled_v, pooled_table, table_width, positions,
                      seq_of_token, (float*)out, out_ld, heads, kv_heads, dim, vdim, page_size, scale, window, pool, out_scale);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(pooled_window_attention_kernel<__nv_bfloat16>, blocks, PWA_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_ld,
                      (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, table, pooled_k, pooled_v, pooled_table,
                      table_width, positions, seq_of_token, (__nv_bfloat16*)out, out_ld, heads, kv_heads, dim, vdim,
                      page_size, scale, window, pool, out_scale);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
