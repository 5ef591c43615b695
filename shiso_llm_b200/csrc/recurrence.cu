// Linear recurrences with a matrix state per head, walked token by token in float.
//
// One CTA per (head, sequence) holds the head's state S[key, value] in registers and walks the
// sequence's rows of this step in order, so a position's output does not depend on how the
// sequence was cut into steps or on what else is in the batch.  Two forms:
//
// A decay w multiplies the state as S - (1 - w) S with 1 - w formed directly (expm1f; the host
// hands over 1 - decay_h): a decay close to 1 rounded to float32 as such would be off by 2^-24 of
// itself per step, which a thousand steps multiply, while 1 - w keeps its own 24 bits.
//
//   channel decay (time mixing of the RWKV family)
//       w_t = exp(-exp(logit_t + bias))                       per key channel
//       o_t = (S_{t-1} + diag(bonus) k_t v_t^T)^T q_t
//       S_t = diag(w_t) S_{t-1} + k_t v_t^T
//   head decay (retention)
//       q_t, k_t rotated by the position (half-split pairs), k_t times key_scale
//       S_t = decay_h S_{t-1} + k_t v_t^T                 (head_loss = 1 - decay_h is what is handed over)
//       o_t = S_t^T q_t
//
// then, for both, o_t brought to unit RMS over the head's value channels, times an optional
// weight, times silu(gate), times a constant, rounded to the activation type.
//
// Thread layout: a value column j of the state belongs to SPLIT neighbouring lanes, each
// holding dim / SPLIT neighbouring rows in registers; the SPLIT partial sums of o_j meet in
// a few shuffles.  q, k and the decays of eight tokens at a time are staged in shared memory; a
// thread walks the eight tokens over its rows of the state without meeting the others, so a
// batch costs two barriers (the staged batch; the sums of squares of its eight outputs), and what
// the next batch brings is asked for from global memory while this one is walked.  The sums a
// token takes part in and their order are the same whatever the batch: cuts change no bit.
#include "common.cuh"

constexpr int REC_MAX_DIM = 256;
constexpr int REC_MAX_STATE = 32768;  // floats of one head's state: what a CTA keeps in registers

struct RecurrenceArgs {
    const void* q; const void* k; const void* v; const void* gate;
    long long q_ld, k_ld, v_ld, gate_ld, out_ld;
    void* out;
    float* state; long long state_stride;  // [slots][heads][dim][vdim], slots `state_stride` floats apart
    const int* q_start; const int* slots; const int* positions;
    const float* decay_logits; long long logits_ld; const float* decay_bias; const float* bonus;  // channel decay
    const float* head_loss; const float* inv_freq; int rotary_dim; float key_scale;               // head decay
    const float* out_weight;
    float eps, out_scale;
    int heads, dim, vdim;
    // With `raw` (float [T, heads * vdim]) a head's value columns are shared out over col_parts CTAs
    // (blockIdx.z), which leave the unnormalised outputs there; unit RMS, weight and gate follow in
    // a row kernel.  For long portions: more SMs walk the same tokens, each with fewer columns.
    float* raw; int col_parts;
};

// Threads a CTA may have so that RPT rows of the state (and what else a thread needs) stay in registers.
constexpr int rec_max_threads(int rpt) { return rpt <= 32 ? 512 : (rpt <= 128 ? 256 : 128); }

constexpr int REC_BATCH = 8;   // tokens staged and walked between two barriers
constexpr int REC_STAGED = 4;  // channels of q and k a thread stages per batch, at most

template <typename AT, int RPT, int SPLIT, bool CHANNEL>
__global__ void __launch_bounds__(rec_max_threads(RPT)) decay_recurrence_kernel(const RecurrenceArgs a) {
    __shared__ __align__(16) float sq[REC_BATCH][REC_MAX_DIM], sk[REC_BATCH][REC_MAX_DIM], sw[CHANNEL ? REC_BATCH : 1][REC_MAX_DIM];
    __shared__ __align__(16) float su[REC_MAX_DIM];
    __shared__ float red[REC_BATCH][32];
    const int head = blockIdx.x, seq = blockIdx.y;
    const int tid = threadIdx.x, threads = blockDim.x;
    const int part = tid % SPLIT;
    const int dim = a.dim, vdim = a.vdim;
    const int cols = vdim / a.col_parts;  // value columns of this CTA
    const int j = blockIdx.z * cols + tid / SPLIT;  // this thread's column
    const int rpt = dim / SPLIT;  // rows of the state per thread (dim is a multiple of SPLIT)
    const bool owns = tid / SPLIT < cols;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (threads + 31) >> 5;
    // tokens per batch: what the threads can stage with REC_STAGED channels each (at least two:
    // the CTA has half as many threads as there are key channels)
    const int batch = min(REC_BATCH, REC_STAGED * threads / dim);

    if (CHANNEL)
        for (int c = tid; c < dim; c += threads) su[c] = a.bonus[head * dim + c];
    const float head_loss = CHANNEL ? 0.0f : a.head_loss[head];  // 1 - decay
    const int half = a.rotary_dim / 2;
    // what a thread stages of every batch: element e = tid + l * threads is channel e % dim of token e / dim
    int st_token[REC_STAGED], st_chan[REC_STAGED];
    float st_const[REC_STAGED];  // the channel's decay bias, or its rotation frequency
#pragma unroll
    for (int l = 0; l < REC_STAGED; ++l) {
        const int e = tid + l * threads;
        st_token[l] = e / dim;
        st_chan[l] = e % dim;
        st_const[l] = 0.0f;
        if (st_token[l] < batch) {
            const int c = st_chan[l];
            if (CHANNEL) st_const[l] = a.decay_bias[head * dim + c];
            else if (c < a.rotary_dim) st_const[l] = a.inv_freq[c < half ? c : c - half];
        }
    }
    const float out_weight = (a.out_weight && owns) ? a.out_weight[head * vdim + j] : 1.0f;
    pdl_wait();
    const int first = a.q_start[seq], last = a.q_start[seq + 1];
    if (last <= first) return;
    __syncthreads();  // the bonus is staged
    // a thread's rows of the state are neighbours: row = part * rpt + ii
    const int row0 = part * rpt;
    const bool wide = rpt % 4 == 0;  // its slices of the staged vectors are read 16 bytes at a time
    float* state = a.state + (long long)a.slots[seq] * a.state_stride + (size_t)head * dim * vdim;
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
        S[ii] = (owns && ii < rpt) ? state[(size_t)(row0 + ii) * vdim + j] : 0.0f;
    }

    const AT* q = (const AT*)a.q + (size_t)head * dim;
    const AT* k = (const AT*)a.k + (size_t)head * dim;
    const AT* v = (const AT*)a.v + (size_t)head * vdim;
    const AT* gate = a.gate ? (const AT*)a.gate + (size_t)head * vdim : nullptr;
    AT* out = (AT*)a.out + (size_t)head * vdim;

    // What a batch of tokens brings is asked for one batch ahead: the loads are in flight while the
    // state walks the batch before.
    struct Raw { float q[REC_STAGED], k[REC_STAGED], q_other[REC_STAGED], k_other[REC_STAGED], v[REC_BATCH]; };
    // (Every load below has a valid address whatever n is - a token index beyond the batch is the
    // batch's last, an idle thread's column is the CTA's first - and nothing is converted before all
    // are asked for: a branch or a conversion between two loads would make each wait for the one before.)
    const int jc = owns ? j : blockIdx.z * cols;
    auto fetch = [&](int t0, int n, Raw& r) {
        AT raw_q[REC_STAGED], raw_k[REC_STAGED], raw_qo[REC_STAGED], raw_ko[REC_STAGED], raw_v[REC_BATCH];
        float raw_logit[REC_STAGED];
#pragma unroll
        for (int l = 0; l < REC_STAGED; ++l) {
            const int t = t0 + min(st_token[l], n - 1), c = st_chan[l];
            raw_q[l] = q[(size_t)t * a.q_ld + c];
            raw_k[l] = k[(size_t)t * a.k_ld + c];
            if (CHANNEL) {
                raw_logit[l] = a.decay_logits[(size_t)t * a.logits_ld + head * dim + c];
            } else {
                const int other = c < a.rotary_dim ? (c < half ? c + half : c - half) : c;
                raw_qo[l] = q[(size_t)t * a.q_ld + other];
                raw_ko[l] = k[(size_t)t * a.k_ld + other];
            }
        }
#pragma unroll
        for (int i = 0; i < REC_BATCH; ++i) raw_v[i] = v[(size_t)(t0 + min(i, n - 1)) * a.v_ld + jc];
#pragma unroll
        for (int l = 0; l < REC_STAGED; ++l) {
            r.q[l] = to_f32(raw_q[l]);
            r.k[l] = to_f32(raw_k[l]);
            r.q_other[l] = CHANNEL ? raw_logit[l] : to_f32(raw_qo[l]);
            r.k_other[l] = CHANNEL ? 0.0f : to_f32(raw_ko[l]);
        }
#pragma unroll
        for (int i = 0; i < REC_BATCH; ++i) r.v[i] = to_f32(raw_v[i]);
    };
    auto stage = [&](int t0, int n, const Raw& r) {
#pragma unroll
        for (int l = 0; l < REC_STAGED; ++l) {
            if (st_token[l] >= n) continue;
            const int i = st_token[l], c = st_chan[l];
            float qc = r.q[l], kc = r.k[l];
            if (!CHANNEL) {
                if (c < a.rotary_dim) {
                    float sn, cs;
                    sincosf((float)a.positions[t0 + i] * st_const[l], &sn, &cs);
                    qc = c < half ? qc * cs - r.q_other[l] * sn : qc * cs + r.q_other[l] * sn;
                    kc = c < half ? kc * cs - r.k_other[l] * sn : kc * cs + r.k_other[l] * sn;
                }
                kc *= a.key_scale;
            } else {
                sw[i][c] = -expm1f(-expf(r.q_other[l] + st_const[l]));  // 1 - w, exact to the last bit also where w is close to 1
            }
            sq[i][c] = qc;
            sk[i][c] = kc;
        }
    };
    // one row of the state takes one token
    auto take = [&](int ii, float qv, float kval, float wv, float uv, float vj, float& o) {
        const float kv = kval * vj;
        if (CHANNEL) {
            o += qv * (S[ii] + uv * kv);
            S[ii] = fmaf(-wv, S[ii], S[ii]) + kv;
        } else {
            S[ii] = fmaf(-head_loss, S[ii], S[ii]) + kv;
            o += qv * S[ii];
        }
    };
    Raw cur, next;
    fetch(first, min(batch, last - first), cur);
    stage(first, min(batch, last - first), cur);
    for (int t0 = first; t0 < last; t0 += batch) {
        const int n = min(batch, last - t0);
        const int n_next = min(batch, last - t0 - n);
        if (n_next > 0) fetch(t0 + n, n_next, next);
        float gates[REC_BATCH];  // asked for now, needed after the batch is walked
        if (gate && !a.raw) {
            AT raw_gate[REC_BATCH];
#pragma unroll
            for (int i = 0; i < REC_BATCH; ++i) raw_gate[i] = gate[(size_t)(t0 + min(i, n - 1)) * a.gate_ld + jc];
#pragma unroll
            for (int i = 0; i < REC_BATCH; ++i) gates[i] = to_f32(raw_gate[i]);
        } else {
#pragma unroll
            for (int i = 0; i < REC_BATCH; ++i) gates[i] = 0.0f;
        }
        __syncthreads();  // the batch is staged
        float o[REC_BATCH];
#pragma unroll
        for (int i = 0; i < REC_BATCH; ++i) {
            o[i] = 0.0f;
            if (i < n) {
                const float vj = cur.v[i];
                // (the sum over a thread's rows runs in row order, as four interleaved chains)
                float o4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (wide) {
#pragma unroll
                    for (int g4 = 0; g4 < RPT / 4; ++g4) {
                        if (4 * g4 < rpt) {
                            const float4 q4 = *reinterpret_cast<const float4*>(&sq[i][row0 + 4 * g4]);
                            const float4 k4 = *reinterpret_cast<const float4*>(&sk[i][row0 + 4 * g4]);
                            float4 w4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), u4 = w4;
                            if (CHANNEL) {
                                w4 = *reinterpret_cast<const float4*>(&sw[i][row0 + 4 * g4]);
                                u4 = *reinterpret_cast<const float4*>(&su[row0 + 4 * g4]);
                            }
                            take(4 * g4 + 0, q4.x, k4.x, w4.x, u4.x, vj, o4[0]);
                            take(4 * g4 + 1, q4.y, k4.y, w4.y, u4.y, vj, o4[1]);
                            take(4 * g4 + 2, q4.z, k4.z, w4.z, u4.z, vj, o4[2]);
                            take(4 * g4 + 3, q4.w, k4.w, w4.w, u4.w, vj, o4[3]);
                        }
                    }
                } else {
#pragma unroll
                    for (int ii = 0; ii < RPT; ++ii)
                        if (ii < rpt) take(ii, sq[i][row0 + ii], sk[i][row0 + ii], CHANNEL ? sw[i][row0 + ii] : 0.0f, CHANNEL ? su[row0 + ii] : 0.0f, vj, o4[ii & 3]);
                }
                o[i] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
            }
        }
#pragma unroll
        for (int i = 0; i < REC_BATCH; ++i) {
#pragma unroll
            for (int off = 1; off < SPLIT; off <<= 1) o[i] += __shfl_xor_sync(0xffffffffu, o[i], off);
            if (a.raw) {
                if (owns && i % SPLIT == part && i < n) a.raw[(size_t)(t0 + i) * a.heads * vdim + (size_t)head * vdim + j] = o[i];
            } else {
                const float partial = warp_sum((owns && part == 0) ? o[i] * o[i] : 0.0f);
                if (lane == 0) red[i][warp] = partial;
            }
        }
        __syncthreads();  // every thread has read the staged batch; the sums of squares are written
        if (owns && !a.raw) {
            // (every lane of a column holds the column's sums: the lanes share the batch's tokens)
#pragma unroll
            for (int i = 0; i < REC_BATCH; ++i) {
                if (i % SPLIT == part && i < n) {
                    float squares = 0.0f;
                    for (int w = 0; w < nwarps; ++w) squares += red[i][w];
                    float y = o[i] * rsqrtf(squares / (float)vdim + a.eps) * out_weight;
                    if (gate) y *= gates[i] / (1.0f + expf(-gates[i]));
                    out[(size_t)(t0 + i) * a.out_ld + j] = from_f32<AT>(y * a.out_scale);
                }
            }
        }
        if (n_next > 0) {
            stage(t0 + n, n_next, next);
            cur = next;
        }
        // (the next batch's first barrier orders these writes before its reads, and this batch's
        // reads of the sums before their next writes)
    }
    pdl_trigger();
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii)
        if (owns && ii < rpt) state[(size_t)(row0 + ii) * vdim + j] = S[ii];
}

template <typename AT, int SPLIT, bool CHANNEL>
static int launch_recurrence(const RecurrenceArgs& a, int num_seqs, cudaStream_t stream) {
    const int rpt = a.dim / SPLIT;
    // a thread per lane of a column, and at least half as many threads as key channels (they stage q and k)
    const int columns = (a.vdim / a.col_parts * SPLIT + 31) / 32 * 32, stagers = ((a.dim + 1) / 2 + 31) / 32 * 32;
    const unsigned threads = (unsigned)(columns > stagers ? columns : stagers);
    const dim3 grid(a.heads, num_seqs, a.col_parts);
#define SHISO_REC(R)                                                                                          \
    if constexpr (R * SPLIT <= REC_MAX_DIM) {                                                                 \
        if (rpt <= R) {                                                                                       \
            if (threads > (unsigned)rec_max_threads(R)) return SHISO_ERR_SHAPE;                               \
            launch_kernel(decay_recurrence_kernel<AT, R, SPLIT, CHANNEL>, grid, threads, 0, stream, a);       \
            return launch_status();                                                                           \
        }                                                                                                     \
    }
    SHISO_REC(8) SHISO_REC(16) SHISO_REC(32) SHISO_REC(64) SHISO_REC(128) SHISO_REC(256)
#undef SHISO_REC
    return SHISO_ERR_SHAPE;
}

static int rows_bucket(int rpt) {
    for (int r = 8; r <= REC_MAX_DIM; r *= 2)
        if (rpt <= r) return r;
    return REC_MAX_DIM;
}

// Into how many lanes a column of the state is split: as many (8, 4, 2, 1) as divide the key size
// and leave the CTA within the threads its rows per thread allow; 0 when nothing fits.
static int choose_split(int dim, int vdim) {
    for (int split = 8; split >= 1; split /= 2) {
        if (dim % split || dim / split < 1) continue;
        const int columns = (vdim * split + 31) / 32 * 32, stagers = ((dim + 1) / 2 + 31) / 32 * 32;
        if ((columns > stagers ? columns : stagers) <= rec_max_threads(rows_bucket(dim / split))) return split;
    }
    return 0;
}

SHISO_API int shiso_decay_recurrence_supported(int dim, int vdim) {
    return dim > 0 && vdim > 0 && dim <= REC_MAX_DIM && vdim <= REC_MAX_DIM && dim * vdim <= REC_MAX_STATE && choose_split(dim, vdim) > 0;
}

template <typename AT, bool CHANNEL>
static int pick_split(const RecurrenceArgs& a, int num_seqs, cudaStream_t stream) {
    switch (choose_split(a.dim, a.vdim / a.col_parts)) {
        case 8: return launch_recurrence<AT, 8, CHANNEL>(a, num_seqs, stream);
        case 4: return launch_recurrence<AT, 4, CHANNEL>(a, num_seqs, stream);
        case 2: return launch_recurrence<AT, 2, CHANNEL>(a, num_seqs, stream);
        case 1: return launch_recurrence<AT, 1, CHANNEL>(a, num_seqs, stream);
    }
    return SHISO_ERR_SHAPE;
}

// Unit RMS over a head's value channels, times weight, silu(gate) and a constant: what follows the
// recurrence when its outputs were left unnormalised.  A warp per (row, head).
template <typename AT>
__global__ void unit_rms_gate_kernel(const float* __restrict__ raw, const AT* __restrict__ gate, long long gate_ld,
                                     const float* __restrict__ out_weight, AT* __restrict__ out, long long out_ld, int tokens,
                                     int heads, int vdim, float eps, float out_scale) {
    pdl_begin();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const float* o = raw + ((size_t)t * heads + head) * vdim;
    float vals[REC_MAX_DIM / 32];
    float squares = 0.0f;
#pragma unroll
    for (int e = 0; e < REC_MAX_DIM / 32; ++e) {
        const int c = e * 32 + lane;
        vals[e] = c < vdim ? o[c] : 0.0f;
        squares += vals[e] * vals[e];
    }
    const float unit = rsqrtf(warp_sum(squares) / (float)vdim + eps);
#pragma unroll
    for (int e = 0; e < REC_MAX_DIM / 32; ++e) {
        const int c = e * 32 + lane;
        if (c < vdim) {
            float y = vals[e] * unit;
            if (out_weight) y *= out_weight[head * vdim + c];
            if (gate) {
                const float g = to_f32(gate[(size_t)t * gate_ld + (size_t)head * vdim + c]);
                y *= g / (1.0f + expf(-g));
            }
            out[(size_t)t * out_ld + (size_t)head * vdim + c] = from_f32<AT>(y * out_scale);
        }
    }
}

SHISO_API int shiso_decay_recurrence(const void* q, const void* k, const void* v, const void* gate, long long q_ld, long long k_ld,
                                     long long v_ld, long long gate_ld, void* out, long long out_ld, int act_dtype, float* state,
                                     long long state_stride, const int* q_start, const int* slots, const int* positions,
                                     const float* decay_logits, long long logits_ld, const float* decay_bias, const float* bonus,
                                     const float* head_loss, const float* inv_freq, int rotary_dim, float key_scale,
                                     const float* out_weight, float eps, float out_scale, float* raw, int col_parts, int tokens,
                                     int num_seqs, int heads, int dim, int vdim, cudaStream_t stream) {
    if (num_seqs <= 0 || heads <= 0) return SHISO_OK;
    if (dim <= 0 || vdim <= 0 || dim > REC_MAX_DIM || vdim > REC_MAX_DIM || dim * vdim > REC_MAX_STATE) return SHISO_ERR_SHAPE;
    const bool channel = decay_logits != nullptr;
    if (channel == (head_loss != nullptr)) return SHISO_ERR_UNSUPPORTED;
    if (channel && (!decay_bias || !bonus)) return SHISO_ERR_UNSUPPORTED;
    if (rotary_dim && (channel || !inv_freq || rotary_dim % 2 || rotary_dim > dim)) return SHISO_ERR_UNSUPPORTED;
    RecurrenceArgs a;
    a.q = q; a.k = k; a.v = v; a.gate = gate;
    a.q_ld = q_ld; a.k_ld = k_ld; a.v_ld = v_ld; a.gate_ld = gate_ld; a.out_ld = out_ld;
    a.out = out; a.state = state; a.state_stride = state_stride;
    a.q_start = q_start; a.slots = slots; a.positions = positions;
    a.decay_logits = decay_logits; a.logits_ld = logits_ld; a.decay_bias = decay_bias; a.bonus = bonus;
    a.head_loss = head_loss; a.inv_freq = inv_freq; a.rotary_dim = rotary_dim; a.key_scale = key_scale;
    a.out_weight = out_weight; a.eps = eps; a.out_scale = out_scale;
    a.heads = heads; a.dim = dim; a.vdim = vdim;
    a.raw = raw; a.col_parts = raw ? col_parts : 1;
    if (a.col_parts < 1 || vdim % a.col_parts || !shiso_decay_recurrence_supported(dim, vdim / a.col_parts)) return SHISO_ERR_SHAPE;
    int status;
    if (act_dtype == SHISO_F32) status = channel ? pick_split<float, true>(a, num_seqs, stream) : pick_split<float, false>(a, num_seqs, stream);
    else if (act_dtype == SHISO_BF16)
        status = channel ? pick_split<__nv_bfloat16, true>(a, num_seqs, stream) : pick_split<__nv_bfloat16, false>(a, num_seqs, stream);
    else return SHISO_ERR_DTYPE;
    if (status != SHISO_OK || !raw) return status;
    const unsigned blocks = ceil_div_u((long long)tokens * heads, 8);
    if (act_dtype == SHISO_F32)
        launch_kernel(unit_rms_gate_kernel<float>, blocks, 256, 0, stream, (const float*)raw, (const float*)gate, gate_ld, out_weight,
                      (float*)out, out_ld, tokens, heads, vdim, eps, out_scale);
    else
        launch_kernel(unit_rms_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const float*)raw, (const __nv_bfloat16*)gate, gate_ld,
                      out_weight, (__nv_bfloat16*)out, out_ld, tokens, heads, vdim, eps, out_scale);
    return launch_status();
}
