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
// into the warp's running maximum and sum, and for the values the lanes change roles: a lane sums
// a few neighbouring latent entries (one load of up to 16 bytes a key) over the run's keys.  Warps' results are merged in warp order,
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

template <typename AT, int E> __device__ __forceinline__ void la_load(const AT* p, float* f) {
    if constexpr (E == 1) {
        f[0] = to_f32(p[0]);
    } else {
        struct alignas(sizeof(AT) * E) Pack {
            AT v[E];
        };
        const Pack pack = *reinterpret_cast<const Pack*>(p);
#pragma unroll
        for (int e = 0; e < E; ++e) f[e] = to_f32(pack.v[e]);
    }
}

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
    // Latent entries a lane reads at once in the value pass (VEC: as many as a 16-byte load or the
    // lane's share holds; the rank is then a multiple of it): entry i of a lane is latent entry
    // (i / E) * 32 E + lane * E + i % E.
    constexpr int E = VEC ? (RV < LaVec<AT>::N ? RV : LaVec<AT>::N) : 1;
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
            for (int c = 0; c < RV / E; ++c) {
                const int r0 = c * 32 * E + lane * E;  // this lane's E neighbouring latent entries of the chunk
                if (r0 < rank) {
                    float cv[E];
                    la_load<AT, E>(krow + r0, cv);
#pragma unroll
                    for (int e = 0; e < E; ++e)
#pragma unroll
                        for (int g = 0; g < LA_HEADS; ++g) acc[g][c * E + e] = fmaf(p[g], cv[e], acc[g][c * E + e]);
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
            const int r = (i / E) * 32 * E + lane * E + (i % E);
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
        const bool wide = vec && rank % (R < N ? R : N) == 0;                                                            \
        auto kern = wide ? latent_attention_kernel<AT, R, true> : latent_attention_kernel<AT, R, false>;                 \
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

// --------------------------------------------------------------------------- prompt portions on the tensor cores
//
// bfloat16 steps with prompt portions: a CTA takes 16 query rows of one sequence and up to eight
// heads, a warp a head.  All heads score against the same cached rows, so a tile of 32 keys is brought
// into shared memory once (16-byte cp.async through the block table, two stages) and read by every
// warp: S = Q K^T by mma.sync m16n8k16 over the whole row width, a base-2 online softmax in
// registers, P rounded to bfloat16 as the A operand of O += P V, where V is the first `rank`
// columns of the very same shared-memory tile, read transposed by ldmatrix.  Needs the row width
// and the rank to be multiples of 16 and a rank of at most 256 (a warp keeps 16 x rank sums).

struct LatentPrefillArgs {
    const __nv_bfloat16* q;
    const __nv_bfloat16* cache;
    const int* block_table;
    int table_width;
    const int *q_start, *start_pos;
    __nv_bfloat16* out;
    int num_seqs, heads, rank, width, page_size;
    float scale_log2;
};

__device__ __forceinline__ uint32_t lp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lp_cp16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(lp_smem(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lp_ldmatrix(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lp_ldmatrix_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lp_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lp_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

#define LP_BM 16
#define LP_BN 32

// RT: 8-column tiles of the result a warp keeps (rank <= 8 RT).  HG: heads (warps) per CTA.
template <int RT, int HG>
__global__ void __launch_bounds__(HG * 32) latent_prefill_mma_kernel(const LatentPrefillArgs a) {
    extern __shared__ __align__(16) uint8_t lp_sm[];
    const int WB = a.width * 2 + 16;  // bytes of a padded shared-memory row
    uint8_t* q_s = lp_sm;                       // [HG][LP_BM][WB]
    uint8_t* k_s = q_s + HG * LP_BM * WB;       // [2][LP_BN][WB]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    pdl_wait();
    int tile = blockIdx.y, s = 0, len = 0;
    for (; s < a.num_seqs; ++s) {
        len = a.q_start[s + 1] - a.q_start[s];
        const int nt = (len + LP_BM - 1) / LP_BM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (s == a.num_seqs) return;
    const int first_token = a.q_start[s] + tile * LP_BM;
    const int rows = min(LP_BM, len - tile * LP_BM);
    const int first_pos = a.start_pos[s] + tile * LP_BM, last_pos = first_pos + rows - 1;
    const int* table = a.block_table + (size_t)s * a.table_width;
    const int head0 = blockIdx.x * HG, head = head0 + warp;
    const bool active = head < a.heads;
    const int chunks = a.width / 8, rt = a.rank / 8;

    for (int c = tid; c < HG * LP_BM * chunks; c += HG * 32) {
        const int hh = c / (LP_BM * chunks), rem = c - hh * (LP_BM * chunks), r = rem / chunks, ch = rem - r * chunks;
        const bool valid = r < rows && head0 + hh < a.heads;
        const __nv_bfloat16* src = a.q + ((size_t)(first_token + r) * a.heads + head0 + hh) * a.width + ch * 8;
        lp_cp16(q_s + (hh * LP_BM + r) * WB + ch * 16, valid ? src : a.q, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    auto load_keys = [&](int kt, int stage) {
        for (int c = tid; c < LP_BN * chunks; c += HG * 32) {
            const int r = c / chunks, ch = c - r * chunks;
            const int key = kt * LP_BN + r;
            const bool valid = key <= last_pos;
            size_t row = 0;
            if (valid) row = (size_t)table[key / a.page_size] * a.page_size + key % a.page_size;
            lp_cp16(k_s + (stage * LP_BN + r) * WB + ch * 16, a.cache + row * a.width + ch * 8, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_keys(0, 0);

    float o_acc[RT][4];
#pragma unroll
    for (int i = 0; i < RT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    const int my_pos[2] = {first_pos + g, first_pos + g + 8};
    const int n_tiles = last_pos / LP_BN + 1;
    for (int kt = 0; kt < n_tiles; ++kt) {
        const int stage = kt & 1;
        if (kt + 1 < n_tiles) load_keys(kt + 1, stage ^ 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const uint8_t* ks = k_s + stage * LP_BN * WB;
        if (active && kt * LP_BN <= first_pos + LP_BM - 1) {
            float s_acc[LP_BN / 8][4];
#pragma unroll
            for (int j = 0; j < LP_BN / 8; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
#pragma unroll 4
            for (int kk = 0; kk < a.width / 16; ++kk) {  // (unrolled so that the next fragments are asked for under this step's products)
                uint32_t af[4];
                {
                    const int r = warp * LP_BM + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int col = kk * 16 + (lane >> 4) * 8;
                    lp_ldmatrix(lp_smem(q_s + r * WB + col * 2), af[0], af[1], af[2], af[3]);
                }
#pragma unroll
                for (int j = 0; j < LP_BN / 8; j += 2) {
                    const int r = j * 8 + (lane & 7) + (lane >> 4) * 8;
                    const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                    uint32_t b0, b1, b2, b3;
                    lp_ldmatrix(lp_smem(ks + r * WB + col * 2), b0, b1, b2, b3);
                    lp_mma(s_acc[j], af, b0, b1);
                    lp_mma(s_acc[j + 1], af, b2, b3);
                }
            }
            const int key0 = kt * LP_BN;
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < LP_BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                    const float v = key <= my_pos[e >> 1] ? s_acc[j][e] * a.scale_log2 : -INFINITY;
                    s_acc[j][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
            float correction[2], use_max[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float m = tile_max[r];
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                const float new_max = fmaxf(row_max[r], m);
                use_max[r] = new_max == -INFINITY ? 0.0f : new_max;
                correction[r] = exp2f(row_max[r] - use_max[r]);
                row_max[r] = new_max;
            }
            float tile_sum[2] = {0.0f, 0.0f};
            uint32_t p_frag[LP_BN / 16][4];
#pragma unroll
            for (int j = 0; j < LP_BN / 8; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[e] = exp2f(s_acc[j][e] - use_max[e >> 1]);
                    tile_sum[e >> 1] += p[e];
                }
                p_frag[j >> 1][(j & 1) * 2 + 0] = lp_pack(p[0], p[1]);
                p_frag[j >> 1][(j & 1) * 2 + 1] = lp_pack(p[2], p[3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * correction[r] + tile_sum[r];
#pragma unroll
            for (int i = 0; i < RT; ++i) {
                o_acc[i][0] *= correction[0];
                o_acc[i][1] *= correction[0];
                o_acc[i][2] *= correction[1];
                o_acc[i][3] *= correction[1];
            }
#pragma unroll
            for (int kb = 0; kb < LP_BN / 16; ++kb) {
#pragma unroll
                for (int dn = 0; dn < RT; dn += 2) {
                    if (dn < rt) {
                        const int r = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                        const int col = (dn + (lane >> 4)) * 8;
                        uint32_t b0, b1, b2, b3;
                        lp_ldmatrix_trans(lp_smem(ks + r * WB + col * 2), b0, b1, b2, b3);
                        lp_mma(o_acc[dn], p_frag[kb], b0, b1);
                        lp_mma(o_acc[dn + 1], p_frag[kb], b2, b3);
                    }
                }
            }
        }
        __syncthreads();  // the stage is refilled by the next iteration's copies
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    pdl_trigger();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        row_sum[r] = sum > 0.0f ? 1.0f / sum : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + r * 8;
        if (active && row < rows) {
            __nv_bfloat16* dst = a.out + ((size_t)(first_token + row) * a.heads + head) * a.rank;
#pragma unroll
            for (int i = 0; i < RT; ++i)
                if (i < rt) *reinterpret_cast<uint32_t*>(dst + i * 8 + t4 * 2) = lp_pack(o_acc[i][r * 2] * row_sum[r], o_acc[i][r * 2 + 1] * row_sum[r]);
        }
    }
}

template <int RT, int HG>
static int launch_latent_prefill(const LatentPrefillArgs& a, int tiles, cudaStream_t stream) {
    const size_t smem = (size_t)(HG * LP_BM + 2 * LP_BN) * (a.width * 2 + 16);
    if (smem > 200 * 1024) return SHISO_ERR_SHAPE;
    auto kern = latent_prefill_mma_kernel<RT, HG>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    launch_kernel(kern, dim3((a.heads + HG - 1) / HG, tiles), dim3(HG * 32), smem, stream, a);
    return launch_status();
}

SHISO_API int shiso_latent_prefill_supported(int rank, int width) {
    return rank > 0 && rank % 16 == 0 && rank <= 256 && width % 16 == 0 && width >= rank &&
           (size_t)(8 * LP_BM + 2 * LP_BN) * (width * 2 + 16) <= 200 * 1024;
}

// q [T, H, width], out [T, H, rank], both bfloat16; `tiles`: an upper bound of the 16-row tiles of all sequences.
SHISO_API int shiso_latent_prefill(const void* q, const void* cache, const int* block_table, int table_width, const int* q_start,
                                   const int* start_pos, void* out, int num_seqs, int tiles, int heads, int rank, int width,
                                   int page_size, float scale, cudaStream_t stream) {
    if (tiles <= 0 || heads <= 0 || num_seqs <= 0) return SHISO_OK;
    if (!shiso_latent_prefill_supported(rank, width) || page_size <= 0) return SHISO_ERR_SHAPE;
    if ((((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15) != 0) return SHISO_ERR_ALIGN;
    LatentPrefillArgs a = {(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_table, table_width, q_start, start_pos,
                           (__nv_bfloat16*)out, num_seqs, heads, rank, width, page_size, scale * 1.4426950408889634f};
    if (rank <= 128) return heads > 4 ? launch_latent_prefill<16, 8>(a, tiles, stream) : launch_latent_prefill<16, 4>(a, tiles, stream);
    return heads > 4 ? launch_latent_prefill<32, 8>(a, tiles, stream) : launch_latent_prefill<32, 4>(a, tiles, stream);
}
