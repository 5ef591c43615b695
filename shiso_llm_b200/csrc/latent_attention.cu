// Attention over a latent cache: every head of a row scores against the same cached row
// [latent (rank) | rotated shared key part] of each visible position, and the value it sums is
// the latent itself (the first `rank` entries of that row).  Queries arrive already carried into
// the latent space, [T, H, width] with width = rank + the shared part; the result is the
// softmax-weighted sum of latents, [T, H, rank], to be expanded per head by the caller.
//
// One CTA per (row, group of four heads, share of the keys), eight warps.  The row's visible
// positions are cut into runs of 32 from position 0; run c belongs to warp c % 8 of share
// (c / 8) % shares.  A lane scores its own key against the four queries (the cached row is read
// once for four heads, 16 bytes at a time where the width allows), the run's softmax is folded
// into the warp's running maximum and sum, and for the values the lanes change roles: lane l sums
// latent entries l, l + 32, ... over the run's keys.  Warps' results are merged in warp order,
// shares (decode steps at long contexts) through a scratch buffer by a second kernel, in share
// order.  What is added in which order depends on the row's position and the number of shares
// only.  Scores, softmax and sums are float.
#include "common.cuh"

#define LA_HEADS 4
#define LA_WARPS 8

template <typename AT> struct LaVec;
template <> struct LaVec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* f) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
    }
};
template <> struct LaVec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float* f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 v = __bfloat1622float2(h[e]);
            f[2 * e] = v.x, f[2 * e + 1] = v.y;
        }
    }
};

// RV: latent entries a lane sums (rank <= 32 RV).  VEC: the cached rows are read 16 bytes at a time.
template <typename AT, int RV, bool VEC>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(
    const AT* __restrict__ q, const AT* __restrict__ cache, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, AT* __restrict__ out, float* __restrict__ scratch,
    int heads, int rank, int width, int page_size, float scale, int shares) {
    extern __shared__ float sm[];
    float* sq = sm;                                  // [LA_HEADS][width], times scale
    float* sp = sq + LA_HEADS * width;               // [LA_WARPS][LA_HEADS][32] a run's softmax weights
    float* sml = sp + LA_WARPS * LA_HEADS * 32;      // [LA_WARPS][LA_HEADS][2] running maximum and sum
    float* sacc = sml + LA_WARPS * LA_HEADS * 2;     // [LA_WARPS][LA_HEADS][rank]
    const int t = blockIdx.x, h0 = blockIdx.y * LA_HEADS, share = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    const int pos = positions[t];
    const int* table = block_table + (size_t)seq_of_token[t] * table_width;
    for (int i = threadIdx.x; i < LA_HEADS * width; i += blockDim.x) {
        const int g = i / width, d = i - g * width;
        sq[i] = (h0 + g < heads) ? to_f32(q[((size_t)t * heads + h0 + g) * width + d]) * scale : 0.0f;
    }
    __syncthreads();
    float m[LA_HEADS], l[LA_HEADS], acc[LA_HEADS][RV];
#pragma unroll
    for (int g = 0; g < LA_HEADS; ++g) {
        m[g] = -INFINITY, l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < RV; ++i) acc[g][i] = 0.0f;
    }
    float* wp = sp + warp * LA_HEADS * 32;
    const int runs = pos / 32 + 1;
    for (int c = share * LA_WARPS + warp; c < runs; c += LA_WARPS * shares) {
        const int j = c * 32 + lane;
        const bool valid = j <= pos;
        const int jj = valid ? j : pos;
        const int page = table[jj / page_size];
        const size_t at = ((size_t)page * page_size + jj % page_size) * width;
        const AT* row = cache + at;
        float s[LA_HEADS] = {};
        if (VEC) {
            constexpr int N = LaVec<AT>::N;
            for (int d = 0; d < width; d += N) {
                float kv[N];
                LaVec<AT>::load(row + d, kv);
#pragma unroll
                for (int g = 0; g < LA_HEADS; ++g)
#pragma unroll
                    for (int e = 0; e < N; ++e) s[g] = fmaf(kv[e], sq[g * width + d + e], s[g]);
            }
        } else {
            for (int d = 0; d < width; ++d) {
                const float kv = to_f32(row[d]);
#pragma unroll
                for (int g = 0; g < LA_HEADS; ++g) s[g] = fmaf(kv, sq[g * width + d], s[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < LA_HEADS; ++g) {
            const float top = fmaxf(m[g], warp_max(valid ? s[g] : -INFINITY));
            const float keep = expf(m[g] - top);  // 0 at the first run
            const float p = valid ? expf(s[g] - top) : 0.0f;
            l[g] = l[g] * keep + warp_sum(p);
            m[g] = top;
#pragma unroll
            for (int i = 0; i < RV; ++i) acc[g][i] *= keep;
            wp[g * 32 + lane] = p;
        }
        __syncwarp();
        const int count = min(32, pos + 1 - c * 32);
        for (int key = 0; key < count; ++key) {
            const size_t kat = __shfl_sync(0xffffffffu, at, key);
            const AT* krow = cache + kat;
            float p[LA_HEADS];
#pragma unroll
            for (int g = 0; g < LA_HEADS; ++g) p[g] = wp[g * 32 + key];
#pragma unroll
            for (int i = 0; i < RV; ++i) {
                const int r = lane + 32 * i;
                if (r < rank) {
                    const float cv = to_f32(krow[r]);
#pragma unroll
                    for (int g = 0; g < LA_HEADS; ++g) acc[g][i] = fmaf(p[g], cv, acc[g][i]);
                }
            }
        }
        __syncwarp();
    }
    pdl_trigger();
#pragma unroll
    for (int g = 0; g < LA_HEADS; ++g) {
        if (lane == 0) sml[(warp * LA_HEADS + g) * 2] = m[g], sml[(warp * LA_HEADS + g) * 2 + 1] = l[g];
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const int r = lane + 32 * i;
            if (r < rank) sacc[((size_t)warp * LA_HEADS + g) * rank + r] = acc[g][i];
        }
    }
    __syncthreads();
    // the warps' results in warp order
    for (int i = threadIdx.x; i < LA_HEADS * rank; i += blockDim.x) {
        const int g = i / rank, r = i - g * rank;
        if (h0 + g >= heads) continue;
        float top = -INFINITY;
        for (int w = 0; w < LA_WARPS; ++w) top = fmaxf(top, sml[(w * LA_HEADS + g) * 2]);
        float total = 0.0f, sum = 0.0f;
        if (top > -INFINITY) {
            for (int w = 0; w < LA_WARPS; ++w) {
                const float f = expf(sml[(w * LA_HEADS + g) * 2] - top);
                total = fmaf(sml[(w * LA_HEADS + g) * 2 + 1], f, total);
                sum = fmaf(sacc[((size_t)w * LA_HEADS + g) * rank + r], f, sum);
            }
        }
        if (shares == 1) {
            out[((size_t)t * heads + h0 + g) * rank + r] = from_f32<AT>(sum / total);
        } else {
            float* part = scratch + (((size_t)t * heads + h0 + g) * shares + share) * (rank + 2);
            part[2 + r] = sum;
            if (r == 0) part[0] = top, part[1] = total;
        }
    }
}

// The shares of a (row, head) in share order: [maximum, sum, rank sums] each.
template <typename AT>
__global__ void latent_attention_merge_kernel(const float* __restrict__ scratch, AT* __restrict__ out, int rank, int shares) {
    pdl_begin();
    const float* parts = scratch + (size_t)blockIdx.x * shares * (rank + 2);
    float top = -INFINITY;
    for (int s = 0; s < shares; ++s) top = fmaxf(top, parts[(size_t)s * (rank + 2)]);
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        float total = 0.0f, sum = 0.0f;
        for (int s = 0; s < shares; ++s) {
            const float* p = parts + (size_t)s * (rank + 2);
            if (p[0] == -INFINITY) continue;
            const float f = expf(p[0] - top);
            total = fmaf(p[1], f, total);
            sum = fmaf(p[2 + r], f, sum);
        }
        out[(size_t)blockIdx.x * rank + r] = from_f32<AT>(sum / total);
    }
}

SHISO_API int shiso_latent_attention_smem(int rank, int width) {
    return (int)((LA_HEADS * width + LA_WARPS * LA_HEADS * 34 + (size_t)LA_WARPS * LA_HEADS * rank) * sizeof(float));
}

template <typename AT>
static int launch_latent_attention(const void* q, const void* cache, const int* block_table, int table_width, const int* positions,
                                   const int* seq_of_token, void* out, float* scratch, int tokens, int heads, int rank, int width,
                                   int page_size, float scale, int shares, cudaStream_t stream) {
    const size_t smem = (size_t)shiso_latent_attention_smem(rank, width);
    if (smem > 220 * 1024) return SHISO_ERR_SHAPE;
    const dim3 grid(tokens, (heads + LA_HEADS - 1) / LA_HEADS, shares), block(LA_WARPS * 32);
    constexpr int N = LaVec<AT>::N;
    const bool vec = width % N == 0 && ((uintptr_t)cache & 15) == 0;
    const int rv = (rank + 31) / 32;
#define LA_CASE(R)                                                                                                       \
    if (rv <= R) {                                                                                                       \
        auto kern = vec ? latent_attention_kernel<AT, R, true> : latent_attention_kernel<AT, R, false>;                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        launch_kernel(kern, grid, block, smem, stream, (const AT*)q, (const AT*)cache, block_table, table_width, positions, \
                      seq_of_token, (AT*)out, scratch, heads, rank, width, page_size, scale, shares);                    \
        if (shares > 1)                                                                                                  \
            launch_kernel(latent_attention_merge_kernel<AT>, tokens * heads, 128, 0, stream, (const float*)scratch, (AT*)out, rank, shares); \
        return launch_status();                                                                                          \
    }
    LA_CASE(1) LA_CASE(2) LA_CASE(4) LA_CASE(8) LA_CASE(16)
#undef LA_CASE
    return SHISO_ERR_SHAPE;
}

// q [T, H, width], cache [pages, page_size, width], out [T, H, rank]; scratch: floats
// [T, H, shares, rank + 2] when shares > 1.
SHISO_API int shiso_latent_attention(const void* q, int act_dtype, const void* cache, const int* block_table, int table_width,
                                     const int* positions, const int* seq_of_token, void* out, float* scratch, int tokens, int heads,
                                     int rank, int width, int page_size, float scale, int shares, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0) return SHISO_OK;
    if (rank <= 0 || rank > 512 || width < rank || page_size <= 0 || shares < 1 || (shares > 1 && !scratch)) return SHISO_ERR_SHAPE;
    if (act_dtype == SHISO_F32)
        return launch_latent_attention<float>(q, cache, block_table, table_width, positions, seq_of_token, out, scratch, tokens, heads,
                                              rank, width, page_size, scale, shares, stream);
    if (act_dtype == SHISO_BF16)
        return launch_latent_attention<__nv_bfloat16>(q, cache, block_table, table_width, positions, seq_of_token, out, scratch, tokens,
                                                      heads, rank, width, page_size, scale, shares, stream);
    return SHISO_ERR_DTYPE;
}
