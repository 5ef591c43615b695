// Matrix-state recurrences with one scalar decay per head and token:
//
//     S_t = a_t S_{t-1} + b_t k_t v_t^T,        o_t = S_t^T q_t + skip_h v_t,
//
// S[dim, vdim] per head, float, carried per request in its state slot.  Two ways to give a and b:
// a fixed decay per head (loss_h = 1 - decay_h; S - loss S is formed, so that a decay near one
// loses nothing to its own rounding; b = 1), or a step size per token and head, dt, with
// b = softplus(dt + dt_bias_h) and a = exp(-exp(a_log_h) b).  q and k may be shared by the heads of
// a group (head h reads group h / (heads / groups)); silu may be applied to q, k and v on load.
//
// One CTA walks the rows of one (head, sequence, range of value columns) in order.  A warp holds 8
// columns: a lane has two neighbouring columns and an eighth of the key rows, in runs of four (rows
// 32 j + 4 lane .. + 3, so that a lane reads its keys and queries as 16-byte words of shared memory,
// eight lanes a full 128-byte line, and uses each word for both of its columns); it keeps dim / 4
// state values in registers and an output is a sum over a lane's rows followed by three shuffles:
// what is added to what, and in which order, depends on dim only - never on how
// the sequence was cut into steps, on the batch, or on how many columns a CTA was given.  Rows are
// staged in shared memory sixteen at a time (activations and the two exponentials applied once, on
// the way in) by four warps that hold no state, into the stage the others are not reading: the
// warps that walk the rows never wait for global memory, and meet the others once per sixteen rows.  Outputs are float rows [T, heads * vdim]: the norm and gate that follow them are a
// row kernel's.
#include "common.cuh"

#define SR_TOKENS 16

struct StateRecurrenceArgs {
    const void *q, *k, *v, *dt;
    long long q_ld, k_ld, v_ld, dt_ld;
    const float *dt_bias, *a_log, *skip, *head_loss;
    float* state;
    long long slot_stride;
    const int *q_start, *state_slots;
    float* out;
    int heads, groups, dim, vdim, cols, silu;
    int bulk;  // rows may be fetched 16 bytes at a time (widths, strides and addresses allow it)
};

// silu of a projection's output on its way into shared memory.  float rows: the accurate expf and
// division.  bfloat16 rows: the special-function unit's exponential and reciprocal (relative error
// about 2^-21, far below the 2^-9 the input was rounded to) - the staging warps repeat this for
// every CTA of a head, and the accurate forms were most of their instructions.
template <typename AT> __device__ __forceinline__ float sr_silu(float z);
template <> __device__ __forceinline__ float sr_silu<float>(float z) { return z / (1.0f + expf(-z)); }
template <> __device__ __forceinline__ float sr_silu<__nv_bfloat16>(float z) { return __fdividef(z, 1.0f + __expf(-z)); }
__device__ __forceinline__ void sr_cp16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}

#define SR_PRODUCERS 128  // threads behind the ones that hold state: they stage the next rows

template <typename AT, int RPT>
__global__ void __launch_bounds__(256 + SR_PRODUCERS) state_recurrence_kernel(const StateRecurrenceArgs a) {
    const int h = blockIdx.x, s = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int workers = a.cols * 4;  // threads that hold state; the rest stage rows
    const bool producer = (int)threadIdx.x >= workers;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = lane & 7, local = warp * 8 + (lane >> 3) * 2, col = col0 + local;  // columns col and col + 1
    const bool live = !producer && col < a.vdim, live1 = !producer && col + 1 < a.vdim;
    const int dim = a.dim, vdim = a.vdim, g = h / (a.heads / a.groups);
    constexpr int DP = 8 * RPT;             // key rows with padding (zeros: their state stays zero)
    extern __shared__ __align__(16) float sm[];
    const int stage_floats = 2 * SR_TOKENS * DP + SR_TOKENS * a.cols + 2 * SR_TOKENS;  // q, k, v, decay, input scale
    const float skip = a.skip ? a.skip[h] : 0.0f;
    const float loss = a.head_loss ? a.head_loss[h] : 0.0f;
    const float rate = a.a_log ? expf(a.a_log[h]) : 0.0f;
    const float dt_bias = a.dt_bias ? a.dt_bias[h] : 0.0f;
    pdl_wait();
    const int first = a.q_start[s], n = a.q_start[s + 1] - first;
    if (n <= 0) return;
    float* slot = a.state + (size_t)a.state_slots[s] * a.slot_stride + (size_t)h * dim * vdim;
    float S[RPT], S1[RPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
        const int row = (r >> 2) * 32 + part * 4 + (r & 3);
        S[r] = (live && row < dim) ? slot[(size_t)row * vdim + col] : 0.0f;
        S1[r] = (live1 && row < dim) ? slot[(size_t)row * vdim + col + 1] : 0.0f;
    }
    const AT* qp = (const AT*)a.q + (size_t)g * dim;
    const AT* kp = (const AT*)a.k + (size_t)g * dim;
    const AT* vp = (const AT*)a.v + (size_t)h * vdim + col0;
    const AT* dtp = a.dt ? (const AT*)a.dt + h : nullptr;
    float* op = a.out + (size_t)h * vdim + col;

    // Rows base .. base + count - 1 into a stage, by `threads` threads of which this is number `me`.
    // Sixteen loads are asked for before the first is converted, at addresses that are valid whatever
    // the count (a place beyond it reads the chunk's first row and stores zero).
    auto stage_rows = [&](int base, float* st, int me, int threads) {
        const int count = min(SR_TOKENS, n - base);
        const size_t row0 = (size_t)(first + base);
        float* sq = st;
        float* sk = sq + SR_TOKENS * DP;
        float* sv = sk + SR_TOKENS * DP;
        float* sa = sv + SR_TOKENS * a.cols;
        float* sb = sa + SR_TOKENS;
        constexpr int U = 8;  // loads of q and of k a thread has in flight
        for (int i0 = me; i0 < SR_TOKENS * DP; i0 += threads * U) {
            float qv[U], kv[U];
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * threads, t = i / DP, c = i - t * DP;
                ok[u] = i < SR_TOKENS * DP && t < count && c < dim;
                const size_t at_t = ok[u] ? row0 + t : row0;
                const int at_c = ok[u] ? c : 0;
                qv[u] = to_f32(qp[at_t * a.q_ld + at_c]);
                kv[u] = to_f32(kp[at_t * a.k_ld + at_c]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * threads;
                if (i >= SR_TOKENS * DP) continue;
                if (a.silu) qv[u] = sr_silu<AT>(qv[u]), kv[u] = sr_silu<AT>(kv[u]);
                sq[i] = ok[u] ? qv[u] : 0.0f;
                sk[i] = ok[u] ? kv[u] : 0.0f;
            }
        }
        for (int i0 = me; i0 < SR_TOKENS * a.cols; i0 += threads * 4) {
            float vv[4];
            bool ok[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * threads, t = i / a.cols, c = i - t * a.cols;
                ok[u] = i < SR_TOKENS * a.cols && t < count && col0 + c < vdim;
                vv[u] = to_f32(vp[(ok[u] ? row0 + t : row0) * a.v_ld + (ok[u] ? c : 0)]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * threads;
                if (i >= SR_TOKENS * a.cols) continue;
                if (a.silu) vv[u] = sr_silu<AT>(vv[u]);
                sv[i] = ok[u] ? vv[u] : 0.0f;
            }
        }
        if (dtp) {
            for (int t = me; t < count; t += threads) {
                const float z = to_f32(dtp[(row0 + t) * a.dt_ld]) + dt_bias;
                const float step = z > 20.0f ? z : log1pf(expf(z));
                sb[t] = step;
                sa[t] = expf(-rate * step);
            }
        }
    };

    // The same by the staging warps alone, in two halves.  bulk_fetch asks for every byte of sixteen
    // rows at once (16-byte cp.async into one of two raw areas of their own); bulk_convert, an
    // iteration later, turns a raw area that has landed into a stage (conversion, activation, the
    // decays).  The copies of the rows after next are thus on their way while the next rows are
    // converted and the current ones walked: a row costs no visible trip to memory.
    const int raw_elems = SR_TOKENS * (2 * dim + a.cols);
    AT* raw_base = reinterpret_cast<AT*>(sm + 2 * stage_floats);  // two areas: [SR_TOKENS][dim] q, the same of k, [SR_TOKENS][cols] v
    float z_next = 0.0f, z_cur = 0.0f;  // the step size's logit of this thread's row, fetched with the copies
    auto bulk_fetch = [&](int base, AT* raw, int me, int threads) {
        constexpr int EPV = 16 / (int)sizeof(AT);  // elements a copy
        const int count = min(SR_TOKENS, n - base);
        const size_t row0 = (size_t)(first + base);
        AT* rq = raw;
        AT* rk = rq + SR_TOKENS * dim;
        AT* rv = rk + SR_TOKENS * dim;
        const int qpieces = dim / EPV, vpieces = a.cols / EPV;
        for (int i = me; i < SR_TOKENS * qpieces; i += threads) {
            const int t = i / qpieces, c = (i - t * qpieces) * EPV;
            const bool ok = t < count;
            sr_cp16(rq + t * dim + c, ok ? qp + (row0 + t) * a.q_ld + c : qp, ok);
            sr_cp16(rk + t * dim + c, ok ? kp + (row0 + t) * a.k_ld + c : kp, ok);
        }
        for (int i = me; i < SR_TOKENS * vpieces; i += threads) {
            const int t = i / vpieces, c = (i - t * vpieces) * EPV;
            const bool ok = t < count && col0 + c < vdim;
            sr_cp16(rv + t * a.cols + c, ok ? vp + (row0 + t) * a.v_ld + c : vp, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (dtp && me < count) z_next = to_f32(dtp[(row0 + me) * a.dt_ld]) + dt_bias;
    };
    auto bulk_convert = [&](int base, const AT* raw, float* st, int me, int threads, float z) {
        const int count = min(SR_TOKENS, n - base);
        float* sq = st;
        float* sk = sq + SR_TOKENS * DP;
        float* sv = sk + SR_TOKENS * DP;
        float* sa = sv + SR_TOKENS * a.cols;
        float* sb = sa + SR_TOKENS;
        const AT* rq = raw;
        const AT* rk = rq + SR_TOKENS * dim;
        const AT* rv = rk + SR_TOKENS * dim;
        for (int i = me; i < SR_TOKENS * DP; i += threads) {
            const int t = i / DP, c = i - t * DP;
            float qv = 0.0f, kv = 0.0f;
            if (c < dim && t < count) {
                qv = to_f32(rq[t * dim + c]), kv = to_f32(rk[t * dim + c]);
                if (a.silu) qv = sr_silu<AT>(qv), kv = sr_silu<AT>(kv);
            }
            sq[i] = qv;
            sk[i] = kv;
        }
        for (int i = me; i < SR_TOKENS * a.cols; i += threads) {
            float vv = to_f32(rv[i]);  // zeros where the copy was left out
            if (a.silu) vv = sr_silu<AT>(vv);
            sv[i] = vv;
        }
        if (dtp && me < count) {
            const float step = z > 20.0f ? z : log1pf(expf(z));
            sb[me] = step;
            sa[me] = expf(-rate * step);
        }
    };

    stage_rows(0, sm, threadIdx.x, blockDim.x);  // the first rows: everybody
    const int me = (int)threadIdx.x - workers, stagers = (int)blockDim.x - workers;
    if (producer && a.bulk && SR_TOKENS < n) bulk_fetch(SR_TOKENS, raw_base + raw_elems, me, stagers);  // rows 16 .. 31 into area 1
    __syncthreads();
    int buf = 0;
    for (int base = 0; base < n; base += SR_TOKENS, buf ^= 1) {
        const int count = min(SR_TOKENS, n - base);
        if (producer) {
            if (base + SR_TOKENS < n) {  // the rows after these: into the other stage
                float* next_stage = sm + (buf ^ 1) * stage_floats;
                if (a.bulk) {
                    // area (buf ^ 1) holds them once this thread's and the other staging threads' copies are done
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    asm volatile("bar.sync 1, %0;" ::"r"(stagers) : "memory");
                    z_cur = z_next;
                    // area buf was converted an iteration ago (the block's barrier lies between): the rows after next go there
                    if (base + 2 * SR_TOKENS < n) bulk_fetch(base + 2 * SR_TOKENS, raw_base + buf * raw_elems, me, stagers);
                    bulk_convert(base + SR_TOKENS, raw_base + (buf ^ 1) * raw_elems, next_stage, me, stagers, z_cur);
                } else {
                    stage_rows(base + SR_TOKENS, next_stage, me, stagers);
                }
            }
        } else {
            const float* st = sm + buf * stage_floats;
            const float* sq = st;
            const float* sk = sq + SR_TOKENS * DP;
            const float* sv = sk + SR_TOKENS * DP;
            const float* sa = sv + SR_TOKENS * a.cols;
            const float* sb = sa + SR_TOKENS;
            const size_t row0 = (size_t)(first + base);
            for (int t = 0; t < count; ++t) {
                const float4* qt = reinterpret_cast<const float4*>(sq + t * DP) + part;
                const float4* kt = reinterpret_cast<const float4*>(sk + t * DP) + part;
                const float2 vt = *reinterpret_cast<const float2*>(sv + t * a.cols + local);
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;  // four chains a column instead of one of dim / 8 links
                float b0 = 0.0f, b1 = 0.0f, b2 = 0.0f, b3 = 0.0f;
                if (dtp) {
                    const float decay = sa[t], bv0 = sb[t] * vt.x, bv1 = sb[t] * vt.y;
#pragma unroll
                    for (int j = 0; j < RPT / 4; ++j) {
                        const float4 k4 = kt[8 * j], q4 = qt[8 * j];
                        S[4 * j] = fmaf(decay, S[4 * j], k4.x * bv0);
                        S[4 * j + 1] = fmaf(decay, S[4 * j + 1], k4.y * bv0);
                        S[4 * j + 2] = fmaf(decay, S[4 * j + 2], k4.z * bv0);
                        S[4 * j + 3] = fmaf(decay, S[4 * j + 3], k4.w * bv0);
                        S1[4 * j] = fmaf(decay, S1[4 * j], k4.x * bv1);
                        S1[4 * j + 1] = fmaf(decay, S1[4 * j + 1], k4.y * bv1);
                        S1[4 * j + 2] = fmaf(decay, S1[4 * j + 2], k4.z * bv1);
                        S1[4 * j + 3] = fmaf(decay, S1[4 * j + 3], k4.w * bv1);
                        a0 = fmaf(S[4 * j], q4.x, a0);
                        a1 = fmaf(S[4 * j + 1], q4.y, a1);
                        a2 = fmaf(S[4 * j + 2], q4.z, a2);
                        a3 = fmaf(S[4 * j + 3], q4.w, a3);
                        b0 = fmaf(S1[4 * j], q4.x, b0);
                        b1 = fmaf(S1[4 * j + 1], q4.y, b1);
                        b2 = fmaf(S1[4 * j + 2], q4.z, b2);
                        b3 = fmaf(S1[4 * j + 3], q4.w, b3);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < RPT / 4; ++j) {
                        const float4 k4 = kt[8 * j], q4 = qt[8 * j];
                        S[4 * j] = fmaf(k4.x, vt.x, fmaf(-loss, S[4 * j], S[4 * j]));
                        S[4 * j + 1] = fmaf(k4.y, vt.x, fmaf(-loss, S[4 * j + 1], S[4 * j + 1]));
                        S[4 * j + 2] = fmaf(k4.z, vt.x, fmaf(-loss, S[4 * j + 2], S[4 * j + 2]));
                        S[4 * j + 3] = fmaf(k4.w, vt.x, fmaf(-loss, S[4 * j + 3], S[4 * j + 3]));
                        S1[4 * j] = fmaf(k4.x, vt.y, fmaf(-loss, S1[4 * j], S1[4 * j]));
                        S1[4 * j + 1] = fmaf(k4.y, vt.y, fmaf(-loss, S1[4 * j + 1], S1[4 * j + 1]));
                        S1[4 * j + 2] = fmaf(k4.z, vt.y, fmaf(-loss, S1[4 * j + 2], S1[4 * j + 2]));
                        S1[4 * j + 3] = fmaf(k4.w, vt.y, fmaf(-loss, S1[4 * j + 3], S1[4 * j + 3]));
                        a0 = fmaf(S[4 * j], q4.x, a0);
                        a1 = fmaf(S[4 * j + 1], q4.y, a1);
                        a2 = fmaf(S[4 * j + 2], q4.z, a2);
                        a3 = fmaf(S[4 * j + 3], q4.w, a3);
                        b0 = fmaf(S1[4 * j], q4.x, b0);
                        b1 = fmaf(S1[4 * j + 1], q4.y, b1);
                        b2 = fmaf(S1[4 * j + 2], q4.z, b2);
                        b3 = fmaf(S1[4 * j + 3], q4.w, b3);
                    }
                }
                float acc = (a0 + a1) + (a2 + a3), acc1 = (b0 + b1) + (b2 + b3);
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
                }
                if (part == 0) {
                    float* o_row = op + (row0 + t) * ((size_t)a.heads * vdim);
                    if (live) o_row[0] = fmaf(skip, vt.x, acc);
                    if (live1) o_row[1] = fmaf(skip, vt.y, acc1);
                }
            }
        }
        __syncthreads();
    }
    pdl_trigger();
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
        const int row = (r >> 2) * 32 + part * 4 + (r & 3);
        if (live && row < dim) slot[(size_t)row * vdim + col] = S[r];
        if (live1 && row < dim) slot[(size_t)row * vdim + col + 1] = S1[r];
    }
}

template <typename AT>
static int launch_state_recurrence(const StateRecurrenceArgs& a, int num_seqs, int sm_count, cudaStream_t stream) {
    // value columns per CTA: fewer while SMs would stay idle, but at least 16 (every CTA's staging
    // warps bring and activate its head's keys and queries themselves, so narrow CTAs repeat that
    // work), or what the head has
    int cols = 64;
    while (cols > 16 && (long long)a.heads * num_seqs * ((a.vdim + cols - 1) / cols) < sm_count) cols /= 2;
    while (cols > 8 && cols / 2 >= a.vdim) cols /= 2;
    StateRecurrenceArgs args = a;
    args.cols = cols;
    const int epv = 16 / (int)sizeof(AT);
    args.bulk = a.dim % epv == 0 && a.vdim % epv == 0 && a.q_ld % epv == 0 && a.k_ld % epv == 0 && a.v_ld % epv == 0 &&
                (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v) & 15) == 0;
    const dim3 grid(a.heads, num_seqs, (a.vdim + cols - 1) / cols), block(cols * 4 + SR_PRODUCERS);
    const int rpt = (a.dim + 31) / 32 * 4;  // key rows in runs of 32: four to each of a column pair's eight lanes
#define SR_CASE(R)                                                                                                   \
    if (rpt <= R) {                                                                                                  \
        const size_t smem = (size_t)2 * (2 * SR_TOKENS * 8 * R + SR_TOKENS * cols + 2 * SR_TOKENS) * sizeof(float) + \
                            (size_t)2 * SR_TOKENS * (2 * a.dim + cols) * sizeof(AT);                                  \
        auto kern = state_recurrence_kernel<AT, R>;                                                                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        launch_kernel(kern, grid, block, smem, stream, args);                                                        \
        return launch_status();                                                                                      \
    }
    SR_CASE(4) SR_CASE(8) SR_CASE(16) SR_CASE(32)
#undef SR_CASE
    return SHISO_ERR_SHAPE;
}

SHISO_API int shiso_state_recurrence(const void* q, const void* k, const void* v, const void* dt, long long q_ld, long long k_ld,
                                     long long v_ld, long long dt_ld, int act_dtype, const float* dt_bias, const float* a_log,
                                     const float* skip, const float* head_loss, float* state, long long slot_stride,
                                     const int* q_start, const int* state_slots, float* out, int tokens, int num_seqs, int heads,
                                     int groups, int dim, int vdim, int silu, int sm_count, cudaStream_t stream) {
    if (tokens <= 0 || num_seqs <= 0) return SHISO_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || dim <= 0 || dim > 256 || vdim <= 0) return SHISO_ERR_SHAPE;
    if ((dt != nullptr) == (head_loss != nullptr)) return SHISO_ERR_UNSUPPORTED;  // one of the two forms
    if (dt && (!dt_bias || !a_log)) return SHISO_ERR_UNSUPPORTED;
    StateRecurrenceArgs a = {q, k, v, dt, q_ld, k_ld, v_ld, dt_ld, dt_bias, a_log, skip, head_loss, state, slot_stride,
                             q_start, state_slots, out, heads, groups, dim, vdim, 0, silu, 0};
    if (act_dtype == SHISO_F32) return launch_state_recurrence<float>(a, num_seqs, sm_count, stream);
    if (act_dtype == SHISO_BF16) return launch_state_recurrence<__nv_bfloat16>(a, num_seqs, sm_count, stream);
    return SHISO_ERR_DTYPE;
}
