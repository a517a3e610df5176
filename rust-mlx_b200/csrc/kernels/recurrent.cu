// Layers that carry a state of fixed size from token to token: a short causal convolution over time, and the
// gated linear recurrence  S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  (S is K x V per head, float, kept transposed).
//
// Two ways of forming a_t, k_t, q_t, v_t from a layer's projections are built:
//   "ssd"  (a state-space layer with a scalar decay a head): a = exp(-exp(A_log) dt), dt = softplus(raw + bias),
//          k = dt * B, q = C (B and C shared by the heads of a group), v = x, and o += D x;
//   "gate" (linear attention whose forget gate also decides what is written): a = f, k = 1 - f,
//          f = low + (1 - low) sigmoid(raw + bias) per head and channel, q = silu(raw q).
// Everything after the projections (step sizes, decays, gates, the state, the sums) is float; results leave as float and
// are normed by group_rmsnorm_kernel, which rounds once.  A sequence's tokens are taken in order, one after another,
// with the same arithmetic for every token, so results do not depend on how a prompt is cut into steps.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------------------------------
// Causal convolution over time on each channel:  y_t = act(bias + sum_j w[j, c] x_(t - taps + 1 + j)) (+ x_t); the weight
// is held taps-major ([taps, channels]: neighbouring threads read neighbouring numbers).
// The last taps - 1 inputs of every sequence live in `ring` [slots, taps - 1, channels], input p at row p % (taps - 1).
// Inputs of the step's own tokens come from `x`, older ones from the ring, positions below 0 are zero.
// write_state: a thread whose token is among the last taps - 1 of its sequence's portion stores its input.  That is
// safe inside this kernel only when no other thread reads the row it overwrites, which holds when every sequence
// brings one token (the row it overwrites is the oldest one it read itself); otherwise the state is written by
// short_conv_state_kernel afterwards.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                                  T* __restrict__ out, int ld_out, T* __restrict__ ring, int channels, int taps,
                                  const int* __restrict__ positions, const int* __restrict__ seq_index,
                                  const int* __restrict__ slots, const int* __restrict__ q_start, size_t total, int act,
                                  int residual, int write_state) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx / channels), c = (int)(idx - (size_t)t * channels);
    const int seq = seq_index[t], pos = positions[t];
    const int i = t - q_start[seq];
    const int keep = taps - 1;
    T* rows = ring + (size_t)slots[seq] * (keep > 0 ? keep : 1) * channels;
    const float cur = to_float(x[(size_t)t * ld_x + c]);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j, p = pos - back;
        float v;
        if (back == 0) v = cur;
        else if (p < 0) v = 0.f;
        else if (back <= i) v = to_float(x[(size_t)(t - back) * ld_x + c]);
        else v = to_float(rows[(size_t)(p % keep) * channels + c]);
        acc = fmaf(w[(size_t)j * channels + c], v, acc);
    }
    if (act == 1) acc = siluf_(acc);
    if (residual) acc += cur;
    out[(size_t)t * ld_out + c] = from_float<T>(acc);
    if (write_state && keep > 0 && q_start[seq + 1] - 1 - t < keep) rows[(size_t)(pos % keep) * channels + c] = x[(size_t)t * ld_x + c];
}

// bfloat16, eight neighbouring channels a thread (16-byte accesses): channels, both row strides and every base address are
// multiples of eight numbers.  The same sums in the same order as above.
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__global__ void short_conv8_kernel(const __nv_bfloat16* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                                   __nv_bfloat16* __restrict__ out, int ld_out, __nv_bfloat16* __restrict__ ring, int channels, int taps,
                                   const int* __restrict__ positions, const int* __restrict__ seq_index, const int* __restrict__ slots,
                                   const int* __restrict__ q_start, size_t total8, int act, int residual, int write_state) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const int c8 = channels >> 3;
    const int t = (int)(idx / c8), c = (int)(idx - (size_t)t * c8) * 8;
    const int seq = seq_index[t], pos = positions[t];
    const int i = t - q_start[seq];
    const int keep = taps - 1;
    __nv_bfloat16* rows = ring + (size_t)slots[seq] * (keep > 0 ? keep : 1) * channels;
    const uint4 cur_raw = *reinterpret_cast<const uint4*>(x + (size_t)t * ld_x + c);
    float cur[8], acc[8];
    unpack8(cur_raw, cur);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j, p = pos - back;
        float v[8];
        if (back == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = cur[e];
        } else if (p < 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        } else if (back <= i) {
            unpack8(*reinterpret_cast<const uint4*>(x + (size_t)(t - back) * ld_x + c), v);
        } else {
            unpack8(*reinterpret_cast<const uint4*>(rows + (size_t)(p % keep) * channels + c), v);
        }
        const float4 w0 = *reinterpret_cast<const float4*>(w + (size_t)j * channels + c);
        const float4 w1 = *reinterpret_cast<const float4*>(w + (size_t)j * channels + c + 4);
        const float wj[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wj[e], v[e], acc[e]);
    }
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        float a = acc[e], b = acc[e + 1];
        if (act == 1) { a = siluf_(a); b = siluf_(b); }
        if (residual) { a += cur[e]; b += cur[e + 1]; }
        __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
        o[e >> 1] = *reinterpret_cast<uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * ld_out + c) = make_uint4(o[0], o[1], o[2], o[3]);
    if (write_state && keep > 0 && q_start[seq + 1] - 1 - t < keep)
        *reinterpret_cast<uint4*>(rows + (size_t)(pos % keep) * channels + c) = cur_raw;
}

// The inputs of the last taps - 1 tokens of every sequence's portion go into the ring (after the kernel above has read it).
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ x, int ld_x, T* __restrict__ ring, int channels, int keep,
                                        const int* __restrict__ positions, const int* __restrict__ slots,
                                        const int* __restrict__ q_start, int n_seqs) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_seqs * keep * channels) return;
    const int c = (int)(idx % channels);
    const int r = (int)((idx / channels) % keep);
    const int seq = (int)(idx / ((size_t)channels * keep));
    const int t = q_start[seq + 1] - 1 - r;
    if (t < q_start[seq]) return;
    T* rows = ring + (size_t)slots[seq] * keep * channels;
    rows[(size_t)(positions[t] % keep) * channels + c] = x[(size_t)t * ld_x + c];
}

// ---------------------------------------------------------------------------------------------------------------------
// The recurrence, in two kernels.
//
// First the step's a, k, q (and for "ssd" the step sizes) are formed in float for all tokens at once, by as many threads
// as there are numbers, into scratch rows laid out as the second kernel reads them: a head's K numbers in eight runs of
// KPT (one for each of the eight lanes that share a column of the state), some floats of padding after each run, zeros
// where K ends.  Then the scan: a warp owns 8 columns (v) of a head's state, the K numbers of a column are shared by 8
// lanes and a lane holds KPT consecutive ones of TWO neighbouring columns (what it reads of a, k, q from shared memory
// serves both: the loop is bound by those reads), the state is kept [V, K] so that a lane's numbers are neighbours in
// memory, and a token's outputs need three shuffles each.  A block has blockDim.x / 32 warps on neighbouring columns of one head
// of one sequence; grid (column tiles, heads, sequences).  The rows of STEPS tokens at a time are copied into shared
// memory (cp.async, two buffers: the next tokens' rows arrive while these are worked on), and the warps run those tokens
// without meeting.  Every token is the same arithmetic in the same order wherever a step's portions are cut.
constexpr int REC_COLS = 8, REC_PARTS = 8;   // a warp's columns (two a lane), lanes that share a column
__host__ __device__ constexpr int rec_pad(int kpt) { return kpt == 4 ? 0 : 4; }   // (keeps the lanes' 16-byte reads on different banks)
__host__ __device__ constexpr int rec_row(int kpt) { return REC_PARTS * (kpt + rec_pad(kpt)); }
__device__ __forceinline__ int rec_k_of(int j, int kpt) {   // which of the K numbers stands at place j of a row (-1: padding)
    const int run = kpt + rec_pad(kpt);
    const int part = j / run, i = j - part * run;
    return i < kpt ? part * kpt + i : -1;
}

// "ssd": conv rows [x (heads * V) | B (groups * K) | C (groups * K)], raw step sizes dt [tokens, heads].
//   kf[t, g, :] = B, qf[t, g, :] = C (as floats, padded rows), step[t, h] = softplus(dt + bias), decay[t, h] = exp(-exp(A_log) step)
template <typename T>
__global__ void recurrence_prepare_ssd_kernel(const T* __restrict__ conv, int ld_conv, const T* __restrict__ dt, int ld_dt,
                                              const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ kf,
                                              float* __restrict__ qf, float* __restrict__ step, float* __restrict__ decay, int heads,
                                              int groups, int K, int V, int kpt) {
    allow_dependents();
    wait_for_prior_kernels();
    const int row = rec_row(kpt), per_token = groups * row;
    const int t = blockIdx.x, r = blockIdx.y * blockDim.x + threadIdx.x;     // grid (tokens, pieces of a token's rows)
    if (r >= per_token) return;
    const size_t idx = (size_t)t * per_token + r;
    const int g = r / row, j = r - g * row;
    const int k = rec_k_of(j, kpt);
    const bool ok = k >= 0 && k < K;
    const T* src = conv + (size_t)t * ld_conv + heads * V + g * K;
    kf[idx] = ok ? to_float(src[k]) : 0.f;
    qf[idx] = ok ? to_float(src[groups * K + k]) : 0.f;
    for (int hh = r; hh < heads; hh += per_token) {     // (the token's threads share out its heads' scalars)
        const float d = softplusf_(to_float(dt[(size_t)t * ld_dt + hh]) + dt_bias[hh]);
        step[(size_t)t * heads + hh] = d;
        decay[(size_t)t * heads + hh] = expf(-expf(a_log[hh]) * d);
    }
}

// "gate": af = f = low + (1 - low) sigmoid(raw f + bias), kf = 1 - f, qf = silu(raw q), per head and channel, padded rows.
template <typename T>
__global__ void recurrence_prepare_gate_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ f, int ld_f,
                                               const float* __restrict__ f_bias, const float* __restrict__ lower, float* __restrict__ af,
                                               float* __restrict__ kf, float* __restrict__ qf, int heads, int K, int kpt) {
    allow_dependents();
    wait_for_prior_kernels();
    const int row = rec_row(kpt), per_token = heads * row;
    const int t = blockIdx.x, r = blockIdx.y * blockDim.x + threadIdx.x;     // grid (tokens, pieces of a token's rows)
    if (r >= per_token) return;
    const size_t idx = (size_t)t * per_token + r;
    const int h = r / row, j = r - h * row;
    const int k = rec_k_of(j, kpt);
    float fv = 0.f, wv = 0.f, qv = 0.f;
    if (k >= 0 && k < K) {
        const float low = lower[h * K + k];
        fv = low + (1.f - low) * sigmoidf_(to_float(f[(size_t)t * ld_f + h * K + k]) + f_bias[h * K + k]);
        wv = 1.f - fv;
        qv = siluf_(to_float(q[(size_t)t * ld_q + h * K + k]));
    }
    af[idx] = fv;
    kf[idx] = wv;
    qf[idx] = qv;
}

// "decay" (linear attention with a learned decay a head and channel and a bonus for the current token):
//   af = exp(-exp(raw w + w0)), kf = k, qf = r as floats in padded rows; bonus[t, h] = sum_c r_c u_c k_c (ascending c).
template <typename T>
__global__ void recurrence_prepare_decay_kernel(const T* __restrict__ r, int ld_r, const T* __restrict__ k, int ld_k,
                                                const T* __restrict__ w, int ld_w, const float* __restrict__ w0, const float* __restrict__ u,
                                                float* __restrict__ af, float* __restrict__ kf, float* __restrict__ qf,
                                                float* __restrict__ bonus, int heads, int K, int kpt) {
    allow_dependents();
    wait_for_prior_kernels();
    const int row = rec_row(kpt), per_token = heads * row;
    const int t = blockIdx.x, x = blockIdx.y * blockDim.x + threadIdx.x;     // grid (tokens, pieces of a token's rows)
    if (x >= per_token) return;
    const size_t idx = (size_t)t * per_token + x;
    const int h = x / row, j = x - h * row;
    const int c = rec_k_of(j, kpt);
    float av = 0.f, kv = 0.f, qv = 0.f;
    if (c >= 0 && c < K) {
        av = expf(-expf(to_float(w[(size_t)t * ld_w + h * K + c]) + w0[h * K + c]));
        kv = to_float(k[(size_t)t * ld_k + h * K + c]);
        qv = to_float(r[(size_t)t * ld_r + h * K + c]);
    }
    af[idx] = av;
    kf[idx] = kv;
    qf[idx] = qv;
    for (int hh = x; hh < heads; hh += per_token) {     // (the token's threads share out its heads' scalars)
        float b = 0.f;
        for (int i = 0; i < K; ++i)
            b = fmaf(to_float(r[(size_t)t * ld_r + hh * K + i]) * u[hh * K + i], to_float(k[(size_t)t * ld_k + hh * K + i]), b);
        bonus[(size_t)t * heads + hh] = b;
    }
}

struct ScanArgs {
    float* state;           // [slots, heads, V, K]
    float* out;             // [tokens, heads * V]
    const int* q_start;
    const int* slots;
    const float* af;        // a vector a head: [tokens, heads, row]; a scalar a head: [tokens, heads]
    const float* kf;        // [tokens, row_heads, row]
    const float* qf;
    const void* v;          // [tokens, ld_v] of T, head h at columns h * V
    const float* v_scale;   // [tokens, heads] or null: v is multiplied with it
    const float* skip;      // [heads] or null: out += skip * (unscaled) v
    const float* bonus;     // [tokens, heads] or null: out += bonus * (unscaled) v (the current token's own share, formed by the prepare kernel)
    int heads, row_heads, K, V, ld_v, steps;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void st_global(float* p, float v) { asm volatile("st.global.f32 [%0], %1;\n" ::"l"(p), "f"(v)); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// PRE: a token's output is read from the state as the token finds it, o_t = S_(t-1)^T q_t, before the state is stepped (the
// current token then enters through `bonus` alone).
template <typename T, int KPT, bool VEC, bool PRE = false>
__global__ void __launch_bounds__(256) recurrence_scan_kernel(const ScanArgs A) {
    extern __shared__ __align__(16) float rec_smem[];
    allow_dependents();
    wait_for_prior_kernels();
    constexpr int ROW = rec_row(KPT), RUN = KPT + rec_pad(KPT);
    constexpr int MAXV = 4;                         // values of v a thread fetches for a buffer: steps * cols / threads = steps / 4
    const int warps = blockDim.x >> 5, cols = warps * REC_COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int part = lane & 7, pair = lane >> 3;    // the lane's two columns are 2 * pair and 2 * pair + 1 of the warp's eight
    const int h = blockIdx.y, seq = blockIdx.z;
    const int v0 = blockIdx.x * cols;
    const int vcol = v0 + warp * REC_COLS + 2 * pair;
    const bool v_ok = vcol < A.V, v_ok1 = vcol + 1 < A.V;
    const int t0 = A.q_start[seq], t1 = A.q_start[seq + 1];
    const int K = A.K, V = A.V, H = A.heads, STEPS = A.steps;
    const int hk = h / (H / A.row_heads);           // the row that this head reads of kf and qf
    // one buffer: q rows, k rows, (a rows | a scalars), v (scaled), v (as it came)
    const int buf_floats = STEPS * ROW * 2 + (VEC ? STEPS * ROW : STEPS) + 2 * STEPS * cols + (PRE ? STEPS : 0);
    float* sbase = A.state + ((size_t)A.slots[seq] * H + h) * K * V;
    const T* vsrc = (const T*)A.v;

    float S[KPT], S1[KPT];
    const bool vec4 = (K & 3) == 0;     // a lane's run of a column starts on a 16-byte boundary: four numbers a load
    if (vec4) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) {
            const int k = part * KPT + i;
            const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 s0 = (v_ok && k < K) ? __ldcs(reinterpret_cast<const float4*>(sbase + (size_t)vcol * K + k)) : z;
            const float4 s1 = (v_ok1 && k < K) ? __ldcs(reinterpret_cast<const float4*>(sbase + (size_t)(vcol + 1) * K + k)) : z;
            S[i] = s0.x; S[i + 1] = s0.y; S[i + 2] = s0.z; S[i + 3] = s0.w;
            S1[i] = s1.x; S1[i + 1] = s1.y; S1[i + 2] = s1.z; S1[i + 3] = s1.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < KPT; ++i) {
            const int k = part * KPT + i;
            S[i] = (v_ok && k < K) ? sbase[(size_t)vcol * K + k] : 0.f;
            S1[i] = (v_ok1 && k < K) ? sbase[(size_t)(vcol + 1) * K + k] : 0.f;
        }
    }
    const float skip = A.skip ? A.skip[h] : 0.f;
    const int n_chunks = (t1 - t0 + STEPS - 1) / STEPS;
    T vreg[MAXV];
    float sreg[MAXV], areg = 0.f, breg = 0.f;

    // the copies of a chunk's rows into buffer b, and its v (and scalars) into registers
    auto fetch = [&](int c) {
        float* buf = rec_smem + (c & 1) * buf_floats;
        const int ts = t0 + c * STEPS, ns = min(STEPS, t1 - ts);
        const int pieces = ROW / 4;
        for (int e = threadIdx.x; e < ns * pieces; e += blockDim.x) {
            const int s = e / pieces, j = (e - s * pieces) * 4;
            const size_t at = ((size_t)(ts + s) * A.row_heads + hk) * ROW + j;
            cp_async16(buf + s * ROW + j, A.qf + at);
            cp_async16(buf + STEPS * ROW + s * ROW + j, A.kf + at);
            if (VEC) cp_async16(buf + 2 * STEPS * ROW + s * ROW + j, A.af + ((size_t)(ts + s) * H + h) * ROW + j);
        }
        cp_async_commit();
#pragma unroll
        for (int r = 0; r < MAXV; ++r) {
            const int e = threadIdx.x + r * blockDim.x;
            const int s = e / cols, j = e - s * cols;
            vreg[r] = from_float<T>(0.f);
            sreg[r] = 1.f;
            if (s < ns && v0 + j < V) {      // (kept as they come: a conversion here would wait for the load)
                vreg[r] = vsrc[(size_t)(ts + s) * A.ld_v + h * V + v0 + j];
                if (A.v_scale) sreg[r] = A.v_scale[(size_t)(ts + s) * H + h];
            }
        }
        if (!VEC && threadIdx.x < ns) areg = A.af[(size_t)(ts + threadIdx.x) * H + h];
        if (PRE && threadIdx.x < ns) breg = A.bonus[(size_t)(ts + threadIdx.x) * H + h];
    };
    // the registers of chunk c go into its buffer
    auto settle = [&](int c) {
        float* buf = rec_smem + (c & 1) * buf_floats;
        float* vs = buf + STEPS * ROW * 2 + (VEC ? STEPS * ROW : STEPS);
#pragma unroll
        for (int r = 0; r < MAXV; ++r) {
            const int e = threadIdx.x + r * blockDim.x;
            if (e < STEPS * cols) {
                vs[e] = to_float(vreg[r]) * sreg[r];
                vs[STEPS * cols + e] = to_float(vreg[r]);
            }
        }
        if (!VEC && threadIdx.x < STEPS) buf[2 * STEPS * ROW + threadIdx.x] = areg;
        if (PRE && threadIdx.x < STEPS) vs[2 * STEPS * cols + threadIdx.x] = breg;
    };

    if (n_chunks > 0) {
        fetch(0);
        settle(0);
    }
    for (int c = 0; c < n_chunks; ++c) {
        const bool more = c + 1 < n_chunks;
        if (more) fetch(c + 1);          // the next chunk's rows are on their way while this one is worked on
        if (more) cp_async_wait_group<1>(); else cp_async_wait_group<0>();
        __syncthreads();
        const float* buf = rec_smem + (c & 1) * buf_floats;
        const float* vs = buf + STEPS * ROW * 2 + (VEC ? STEPS * ROW : STEPS);
        const int ts = t0 + c * STEPS, ns = min(STEPS, t1 - ts);
#pragma unroll 4
        for (int s = 0; s < ns; ++s) {
            const float2 v = *reinterpret_cast<const float2*>(vs + s * cols + warp * REC_COLS + 2 * pair);
            const float* qrow = buf + s * ROW + part * RUN;
            const float* krow = buf + STEPS * ROW + s * ROW + part * RUN;
            const float* arow = buf + 2 * STEPS * ROW + (VEC ? s * ROW + part * RUN : s);
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
            const float a = VEC ? 0.f : arow[0];
#pragma unroll
            for (int i = 0; i < KPT; i += 4) {
                const float4 a4 = VEC ? *reinterpret_cast<const float4*>(arow + i) : make_float4(a, a, a, a);
                const float4 k4 = *reinterpret_cast<const float4*>(krow + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qrow + i);
                if (PRE) {
                    acc[0] = fmaf(S[i], q4.x, acc[0]);         acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                    acc[2] = fmaf(S[i + 2], q4.z, acc[2]);     acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
                    acc1[0] = fmaf(S1[i], q4.x, acc1[0]);      acc1[1] = fmaf(S1[i + 1], q4.y, acc1[1]);
                    acc1[2] = fmaf(S1[i + 2], q4.z, acc1[2]);  acc1[3] = fmaf(S1[i + 3], q4.w, acc1[3]);
                }
                S[i] = fmaf(a4.x, S[i], k4.x * v.x);           if (!PRE) acc[0] = fmaf(S[i], q4.x, acc[0]);
                S[i + 1] = fmaf(a4.y, S[i + 1], k4.y * v.x);   if (!PRE) acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                S[i + 2] = fmaf(a4.z, S[i + 2], k4.z * v.x);   if (!PRE) acc[2] = fmaf(S[i + 2], q4.z, acc[2]);
                S[i + 3] = fmaf(a4.w, S[i + 3], k4.w * v.x);   if (!PRE) acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
                S1[i] = fmaf(a4.x, S1[i], k4.x * v.y);         if (!PRE) acc1[0] = fmaf(S1[i], q4.x, acc1[0]);
                S1[i + 1] = fmaf(a4.y, S1[i + 1], k4.y * v.y); if (!PRE) acc1[1] = fmaf(S1[i + 1], q4.y, acc1[1]);
                S1[i + 2] = fmaf(a4.z, S1[i + 2], k4.z * v.y); if (!PRE) acc1[2] = fmaf(S1[i + 2], q4.z, acc1[2]);
                S1[i + 3] = fmaf(a4.w, S1[i + 3], k4.w * v.y); if (!PRE) acc1[3] = fmaf(S1[i + 3], q4.w, acc1[3]);
            }
            float o = (acc[0] + acc[1]) + (acc[2] + acc[3]), o1 = (acc1[0] + acc1[1]) + (acc1[2] + acc1[3]);
            o += __shfl_xor_sync(0xffffffffu, o, 1);   o1 += __shfl_xor_sync(0xffffffffu, o1, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);   o1 += __shfl_xor_sync(0xffffffffu, o1, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);   o1 += __shfl_xor_sync(0xffffffffu, o1, 4);
            const float2 raw = *reinterpret_cast<const float2*>(vs + STEPS * cols + s * cols + warp * REC_COLS + 2 * pair);
            // (stored as what it is, a store to global memory: through a generic pointer the compiler would have to assume
            // that it may change the rows in shared memory, and could not start the next token's reads before it)
            float* dst = A.out + ((size_t)(ts + s) * H + h) * V + vcol;
            const float own = PRE ? vs[2 * STEPS * cols + s] : skip;
            if (part == 0 && v_ok) st_global(dst, fmaf(own, raw.x, o));
            if (part == 1 && v_ok1) st_global(dst + 1, fmaf(own, raw.y, o1));
        }
        if (more) settle(c + 1);          // (the other buffer: nobody reads it before the next barrier)
        __syncthreads();
    }
    if (vec4) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) {
            const int k = part * KPT + i;
            if (v_ok && k < K) *reinterpret_cast<float4*>(sbase + (size_t)vcol * K + k) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
            if (v_ok1 && k < K) *reinterpret_cast<float4*>(sbase + (size_t)(vcol + 1) * K + k) = make_float4(S1[i], S1[i + 1], S1[i + 2], S1[i + 3]);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int k = part * KPT + i;
        if (v_ok && k < K) sbase[(size_t)vcol * K + k] = S[i];
        if (v_ok1 && k < K) sbase[(size_t)(vcol + 1) * K + k] = S1[i];
    }
}

// out[t, g, :] = u / sqrt(mean(u^2) + eps) * w,  u = y[t, g, :] (* act(gate[t, g, :])): an RMS norm on each of a row's
// groups, the optional gate applied BEFORE the norm.  y is float; the weight has `period` numbers and repeats (a weight
// of one group's size is shared by all groups).  One block a (token, group).  out_scale multiplies the result before it is
// rounded.
template <typename T>
__global__ void group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                                     int period, float eps, T* __restrict__ out, int ld_out, int groups, int size, float out_scale, int gate_after) {
    __shared__ float scratch[32];
    allow_dependents();
    wait_for_prior_kernels();
    const int t = blockIdx.x / groups, g = blockIdx.x - t * groups;
    const float* row = y + ((size_t)t * groups + g) * size;
    const T* grow = gate ? gate + (size_t)t * ld_gate + (size_t)g * size : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float u = row[i];
        if (grow && !gate_after) u *= siluf_(to_float(grow[i]));
        ss += u * u;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float u = row[i];
        if (grow && !gate_after) u *= siluf_(to_float(grow[i]));
        float r = u * inv * w[(g * size + i) % period] * out_scale;
        if (grow && gate_after) r *= siluf_(to_float(grow[i]));
        out[(size_t)t * ld_out + (size_t)g * size + i] = from_float<T>(r);
    }
}

// The same with a warp a (token, group) and four numbers a lane and pass (the group's size, the row strides and the
// weight's period are multiples of four): no barrier, 16-byte reads of y.  The order of a group's sum follows its size alone.
template <typename T>
__global__ void __launch_bounds__(128) group_rmsnorm4_kernel(const float* __restrict__ y, const T* __restrict__ gate, int ld_gate,
                                                             const float* __restrict__ w, int period, float eps, T* __restrict__ out,
                                                             int ld_out, int groups, int size, float out_scale, int total, int gate_after) {
    allow_dependents();
    wait_for_prior_kernels();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= total) return;
    const int t = item / groups, g = item - t * groups;
    const float* row = y + ((size_t)t * groups + g) * size;
    const T* grow = gate ? gate + (size_t)t * ld_gate + (size_t)g * size : nullptr;
    T* orow = out + (size_t)t * ld_out + (size_t)g * size;
    float ss = 0.f;
    for (int i = lane * 4; i < size; i += 128) {
        float4 u = *reinterpret_cast<const float4*>(row + i);
        if (grow && !gate_after) {
            u.x *= siluf_(to_float(grow[i])); u.y *= siluf_(to_float(grow[i + 1]));
            u.z *= siluf_(to_float(grow[i + 2])); u.w *= siluf_(to_float(grow[i + 3]));
        }
        ss += u.x * u.x;
        ss += u.y * u.y;
        ss += u.z * u.z;
        ss += u.w * u.w;
    }
    const float inv = rsqrtf(warp_sum(ss) / (float)size + eps) * out_scale;
    for (int i = lane * 4; i < size; i += 128) {
        float4 u = *reinterpret_cast<const float4*>(row + i);
        float4 gt = make_float4(1.f, 1.f, 1.f, 1.f);
        if (grow) gt = make_float4(siluf_(to_float(grow[i])), siluf_(to_float(grow[i + 1])), siluf_(to_float(grow[i + 2])), siluf_(to_float(grow[i + 3])));
        if (grow && !gate_after) {
            u.x *= gt.x; u.y *= gt.y; u.z *= gt.z; u.w *= gt.w;
            gt = make_float4(1.f, 1.f, 1.f, 1.f);
        }
        const float4 wv = *reinterpret_cast<const float4*>(w + (g * size + i) % period);
        orow[i] = from_float<T>(grow && gate_after ? u.x * inv * wv.x * gt.x : u.x * inv * wv.x);
        orow[i + 1] = from_float<T>(grow && gate_after ? u.y * inv * wv.y * gt.y : u.y * inv * wv.y);
        orow[i + 2] = from_float<T>(grow && gate_after ? u.z * inv * wv.z * gt.z : u.z * inv * wv.z);
        orow[i + 3] = from_float<T>(grow && gate_after ? u.w * inv * wv.w * gt.w : u.w * inv * wv.w);
    }
}

// out[t, h, 0:vdim] = o[t, h, 0:vdim] * sigmoid(gate[t, h * vdim + d]); o's heads are `o_head` numbers apart (heads
// padded to a wider size keep their first vdim numbers), out is dense.  out may be o when o_head == vdim.
template <typename T>
__global__ void sigmoid_gate_kernel(const T* o, int o_head, const T* __restrict__ gate, int ld_gate, T* out, int heads, int vdim,
                                    size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t per_row = (size_t)heads * vdim;
    const size_t t = idx / per_row;
    const int r = (int)(idx - t * per_row);
    const int h = r / vdim, d = r - h * vdim;
    const float v = to_float(o[(t * heads + h) * o_head + d]);
    out[idx] = from_float<T>(v * sigmoidf_(to_float(gate[t * ld_gate + r])));
}

// What the mixes of a token with the token before it read:  out[s][t, c] = x[t, c] + (prev[t, c] - x[t, c]) * mu[s, c] for
// s < n_mix, prev the row of the token before in the same sequence: of this step (t - 1), or `last` [slots, channels] (what
// the sequence's last step left), or zeros at position 0.  Float, one rounding.  write_state: the thread of a sequence's
// last token of the step stores its x into `last`; safe in this kernel only when every sequence brings one token (the
// thread that writes the row is the one that read it), otherwise token_shift_state_kernel stores afterwards.
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, T* __restrict__ out, T* __restrict__ last,
                                       int channels, int n_mix, const int* __restrict__ positions, const int* __restrict__ seq_index,
                                       const int* __restrict__ slots, const int* __restrict__ q_start, size_t total, int write_state) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx / channels), c = (int)(idx - (size_t)t * channels);
    const int seq = seq_index[t];
    const float cur = to_float(x[idx]);
    float prev = 0.f;
    if (t > q_start[seq]) prev = to_float(x[idx - channels]);
    else if (positions[t] > 0) prev = to_float(last[(size_t)slots[seq] * channels + c]);
    const float d = prev - cur;
    for (int s = 0; s < n_mix; ++s) out[(size_t)s * total + idx] = from_float<T>(fmaf(d, mu[(size_t)s * channels + c], cur));
    if (write_state && t == q_start[seq + 1] - 1) last[(size_t)slots[seq] * channels + c] = x[idx];
}

// bfloat16, eight channels a thread (16-byte accesses; channels a multiple of eight): the same numbers.
__global__ void token_shift_mix8_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ mu, __nv_bfloat16* __restrict__ out,
                                        __nv_bfloat16* __restrict__ last, int channels, int n_mix, const int* __restrict__ positions,
                                        const int* __restrict__ seq_index, const int* __restrict__ slots, const int* __restrict__ q_start,
                                        size_t total8, int write_state) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx8 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx8 >= total8) return;
    const int per_row = channels >> 3;
    const int t = (int)(idx8 / per_row), c = (int)(idx8 - (size_t)t * per_row) * 8;
    const size_t idx = (size_t)t * channels + c;
    const int seq = seq_index[t];
    const uint4 raw = *reinterpret_cast<const uint4*>(x + idx);
    uint4 before = make_uint4(0u, 0u, 0u, 0u);
    if (t > q_start[seq]) before = *reinterpret_cast<const uint4*>(x + idx - channels);
    else if (positions[t] > 0) before = *reinterpret_cast<const uint4*>(last + (size_t)slots[seq] * channels + c);
    const uint32_t cw[4] = {raw.x, raw.y, raw.z, raw.w}, pw[4] = {before.x, before.y, before.z, before.w};
    float cur[8], d[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cw[j]));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pw[j]));
        cur[2 * j] = a.x; cur[2 * j + 1] = a.y;
        d[2 * j] = b.x - a.x; d[2 * j + 1] = b.y - a.y;
    }
    const size_t total = total8 * 8;
    for (int s = 0; s < n_mix; ++s) {
        const float4 m0 = *reinterpret_cast<const float4*>(mu + (size_t)s * channels + c);
        const float4 m1 = *reinterpret_cast<const float4*>(mu + (size_t)s * channels + c + 4);
        const float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 r = __floats2bfloat162_rn(fmaf(d[2 * j], m[2 * j], cur[2 * j]), fmaf(d[2 * j + 1], m[2 * j + 1], cur[2 * j + 1]));
            packed[j] = *reinterpret_cast<uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(out + (size_t)s * total + idx) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    if (write_state && t == q_start[seq + 1] - 1) *reinterpret_cast<uint4*>(last + (size_t)slots[seq] * channels + c) = raw;
}

template <typename T>
__global__ void token_shift_state_kernel(const T* __restrict__ x, T* __restrict__ last, int channels, const int* __restrict__ slots,
                                         const int* __restrict__ q_start, int n_seqs) {
    allow_dependents();
    wait_for_prior_kernels();
    const int seq = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels || q_start[seq + 1] <= q_start[seq]) return;
    last[(size_t)slots[seq] * channels + c] = x[(size_t)(q_start[seq + 1] - 1) * channels + c];
}

static int rec_kpt(int K) { return K <= 32 ? 4 : (K <= 64 ? 8 : (K <= 128 ? 16 : 32)); }
static int rec_steps(int kpt) { return kpt == 4 ? 16 : (kpt <= 16 ? 8 : 4); }

template <typename T, bool VEC, bool PRE = false>
int launch_scan(const ScanArgs& a, int n_seqs, int warps, cudaStream_t s) {
    const int cols = warps * REC_COLS;
    dim3 grid((a.V + cols - 1) / cols, a.heads, n_seqs), block(warps * 32);
    ScanArgs args = a;
    const int kpt = rec_kpt(a.K);
    args.steps = rec_steps(kpt);
    const int row = rec_row(kpt);
    const size_t smem = 2 * (size_t)(args.steps * row * 2 + (VEC ? args.steps * row : args.steps) + 2 * args.steps * cols + (PRE ? args.steps : 0)) * sizeof(float);
    switch (kpt) {
        case 4: RMX_CHECK_LAUNCHED(launch_dependent(recurrence_scan_kernel<T, 4, VEC, PRE>, grid, block, smem, s, args), "recurrence_scan"); break;
        case 8: RMX_CHECK_LAUNCHED(launch_dependent(recurrence_scan_kernel<T, 8, VEC, PRE>, grid, block, smem, s, args), "recurrence_scan"); break;
        case 16: RMX_CHECK_LAUNCHED(launch_dependent(recurrence_scan_kernel<T, 16, VEC, PRE>, grid, block, smem, s, args), "recurrence_scan"); break;
        default: RMX_CHECK_LAUNCHED(launch_dependent(recurrence_scan_kernel<T, 32, VEC, PRE>, grid, block, smem, s, args), "recurrence_scan"); break;
    }
    return 0;
}
}  // namespace

RMX_API int rmx_short_conv(const void* x, int ld_x, const float* w, const float* bias, void* out, int ld_out, void* ring, int channels,
                           int taps, const int* positions, const int* seq_index, const int* slots, const int* q_start, int n_tokens,
                           int n_seqs, int act, int residual, int single_tokens, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && n_seqs > 0 && channels > 0 && taps >= 1 && ld_x >= channels && ld_out >= channels, "short_conv: bad sizes");
    RMX_REQUIRE(x && w && out && ring && positions && seq_index && slots && q_start, "short_conv: a null pointer");
    RMX_REQUIRE(act == 0 || act == 1, "short_conv: unknown activation %d", act);
    const size_t total = (size_t)n_tokens * channels;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    const int keep = taps - 1;
    const size_t state_items = (size_t)n_seqs * keep * channels;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32) {
        RMX_CHECK_LAUNCHED(launch_dependent(short_conv_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)x, ld_x, w, bias, (float*)out,
                                            ld_out, (float*)ring, channels, taps, positions, seq_index, slots, q_start, total, act, residual,
                                            single_tokens), "short_conv");
        if (!single_tokens && keep > 0)
            RMX_CHECK_LAUNCHED(launch_dependent(short_conv_state_kernel<float>, dim3((unsigned)((state_items + threads - 1) / threads)), dim3(threads),
                                                0, s, (const float*)x, ld_x, (float*)ring, channels, keep, positions, slots, q_start, n_seqs),
                               "short_conv_state");
    } else if (dtype == RMX_BF16) {
        if (channels % 8 == 0 && ld_x % 8 == 0 && ld_out % 8 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)ring) & 15) == 0)
            RMX_CHECK_LAUNCHED(launch_dependent(short_conv8_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, s,
                                                (const __nv_bfloat16*)x, ld_x, w, bias, (__nv_bfloat16*)out, ld_out, (__nv_bfloat16*)ring, channels,
                                                taps, positions, seq_index, slots, q_start, total / 8, act, residual, single_tokens), "short_conv");
        else
        RMX_CHECK_LAUNCHED(launch_dependent(short_conv_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x, ld_x, w,
                                            bias, (__nv_bfloat16*)out, ld_out, (__nv_bfloat16*)ring, channels, taps, positions, seq_index, slots,
                                            q_start, total, act, residual, single_tokens), "short_conv");
        if (!single_tokens && keep > 0)
            RMX_CHECK_LAUNCHED(launch_dependent(short_conv_state_kernel<__nv_bfloat16>, dim3((unsigned)((state_items + threads - 1) / threads)),
                                                dim3(threads), 0, s, (const __nv_bfloat16*)x, ld_x, (__nv_bfloat16*)ring, channels, keep, positions,
                                                slots, q_start, n_seqs), "short_conv_state");
    } else {
        RMX_FAIL("short_conv: unknown dtype %d", dtype);
    }
    return 0;
}

// How many floats of scratch the recurrence wants for n_tokens tokens: (floats of each padded array, padded row length).
RMX_API long long rmx_recurrence_row(int K) { return K > 0 && K <= 256 ? rec_row(rec_kpt(K)) : -1; }

// mode 0 ("ssd"): a0 = conv rows [x | B | C], a1 = dt columns, p0 = dt bias, p1 = A_log, p2 = D (or null), groups;
//   scratch: kf, qf [tokens, groups, row] and s0 = step, s1 = decay [tokens, heads].
// mode 1 ("gate"): a0 = q, a1 = f, a2 = v columns, p0 = f bias, p1 = lower bound; scratch: s0 = af, kf, qf [tokens, heads, row].
RMX_API int rmx_linear_recurrence(int mode, float* state, float* out, const int* q_start, const int* slots, int n_seqs, int n_tokens,
                                  int heads, int K, int V, const void* a0, int ld0, const void* a1, int ld1, const void* a2, int ld2,
                                  const float* p0, const float* p1, const float* p2, int groups, float* kf, float* qf, float* s0, float* s1,
                                  int warps, int dtype, void* stream) {
    if (n_seqs == 0 || n_tokens == 0) return 0;
    RMX_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && heads > 0 && heads <= 65535 && K > 0 && V > 0 && n_tokens > 0, "linear_recurrence: bad sizes");
    RMX_REQUIRE(K <= 256, "linear_recurrence: a state of %d rows a head is beyond 256", K);
    RMX_REQUIRE(state && out && q_start && slots && a0 && a1 && p0 && p1 && kf && qf && s0, "linear_recurrence: a null pointer");
    RMX_REQUIRE(warps >= 1 && warps <= 8, "linear_recurrence: 1 to 8 warps a block");
    RMX_REQUIRE(dtype == RMX_F32 || dtype == RMX_BF16, "linear_recurrence: unknown dtype %d", dtype);
    const int kpt = rec_kpt(K), row = rec_row(kpt), threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    ScanArgs a;
    a.state = state; a.out = out; a.q_start = q_start; a.slots = slots; a.kf = kf; a.qf = qf;
    a.heads = heads; a.K = K; a.V = V; a.steps = 0; a.bonus = nullptr;
    if (mode == 0) {
        RMX_REQUIRE(groups > 0 && heads % groups == 0 && s1, "linear_recurrence: %d heads in %d groups", heads, groups);
        const dim3 grid(n_tokens, (groups * row + threads - 1) / threads);
        if (dtype == RMX_F32)
            RMX_CHECK_LAUNCHED(launch_dependent(recurrence_prepare_ssd_kernel<float>, grid, dim3(threads), 0, s, (const float*)a0, ld0, (const float*)a1,
                                                ld1, p0, p1, kf, qf, s0, s1, heads, groups, K, V, kpt), "recurrence_prepare");
        else
            RMX_CHECK_LAUNCHED(launch_dependent(recurrence_prepare_ssd_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, (const __nv_bfloat16*)a0, ld0,
                                                (const __nv_bfloat16*)a1, ld1, p0, p1, kf, qf, s0, s1, heads, groups, K, V, kpt),
                               "recurrence_prepare");
        a.af = s1; a.v = a0; a.ld_v = ld0; a.v_scale = s0; a.skip = p2; a.row_heads = groups;
        return dtype == RMX_F32 ? launch_scan<float, false>(a, n_seqs, warps, s) : launch_scan<__nv_bfloat16, false>(a, n_seqs, warps, s);
    }
    RMX_REQUIRE(mode == 1, "linear_recurrence: unknown mode %d", mode);
    RMX_REQUIRE(a2 != nullptr, "linear_recurrence: the gated form needs values");
    RMX_REQUIRE((heads * row + threads - 1) / threads <= 65535, "linear_recurrence: too many heads");
    const dim3 grid(n_tokens, (heads * row + threads - 1) / threads);
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(recurrence_prepare_gate_kernel<float>, grid, dim3(threads), 0, s, (const float*)a0, ld0, (const float*)a1,
                                            ld1, p0, p1, s0, kf, qf, heads, K, kpt), "recurrence_prepare");
    else
        RMX_CHECK_LAUNCHED(launch_dependent(recurrence_prepare_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, (const __nv_bfloat16*)a0, ld0,
                                            (const __nv_bfloat16*)a1, ld1, p0, p1, s0, kf, qf, heads, K, kpt), "recurrence_prepare");
    a.af = s0; a.v = a2; a.ld_v = ld2; a.v_scale = nullptr; a.skip = nullptr; a.row_heads = heads;
    return dtype == RMX_F32 ? launch_scan<float, true>(a, n_seqs, warps, s) : launch_scan<__nv_bfloat16, true>(a, n_seqs, warps, s);
}

RMX_API int rmx_group_rmsnorm(const float* y, const void* gate, int ld_gate, const float* w, int period, float eps, void* out, int ld_out,
                              int n_tokens, int groups, int size, float out_scale, int gate_after, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && groups > 0 && size > 0 && period > 0 && y && w && out, "group_rmsnorm: bad sizes or a null pointer");
    RMX_REQUIRE((long long)n_tokens * groups < (1LL << 31), "group_rmsnorm: too many groups");
    int threads = (size + 31) / 32 * 32;
    threads = threads > 256 ? 256 : threads;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)(n_tokens * groups));
    // Which arrangement runs decides the order of a group's sum: in the 32-bit run the group's size alone may choose (the
    // same bits however a step is cut); in bfloat16 a warp a group also serves long groups once there are many of them.
    const bool many = dtype == RMX_BF16 && (long long)n_tokens * groups >= 1024;
    if (size % 4 == 0 && period % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)w & 15) == 0 && (size <= 256 || (many && size <= 4096))) {
        const int total = n_tokens * groups;
        const dim3 grid4((unsigned)((total + 3) / 4));
        if (dtype == RMX_F32)
            RMX_CHECK_LAUNCHED(launch_dependent(group_rmsnorm4_kernel<float>, grid4, dim3(128), 0, s, y, (const float*)gate, ld_gate, w, period, eps,
                                                (float*)out, ld_out, groups, size, out_scale, total, gate_after), "group_rmsnorm");
        else if (dtype == RMX_BF16)
            RMX_CHECK_LAUNCHED(launch_dependent(group_rmsnorm4_kernel<__nv_bfloat16>, grid4, dim3(128), 0, s, y, (const __nv_bfloat16*)gate, ld_gate,
                                                w, period, eps, (__nv_bfloat16*)out, ld_out, groups, size, out_scale, total, gate_after), "group_rmsnorm");
        else
            RMX_FAIL("group_rmsnorm: unknown dtype %d", dtype);
        return 0;
    }
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(group_rmsnorm_kernel<float>, grid, dim3(threads), 0, s, y, (const float*)gate, ld_gate, w, period, eps,
                                            (float*)out, ld_out, groups, size, out_scale, gate_after), "group_rmsnorm");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(group_rmsnorm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, y, (const __nv_bfloat16*)gate, ld_gate,
                                            w, period, eps, (__nv_bfloat16*)out, ld_out, groups, size, out_scale, gate_after), "group_rmsnorm");
    else
        RMX_FAIL("group_rmsnorm: unknown dtype %d", dtype);
    return 0;
}

RMX_API int rmx_sigmoid_gate(const void* o, int o_head, const void* gate, int ld_gate, void* out, int n_tokens, int heads, int vdim,
                             int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && heads > 0 && vdim > 0 && o_head >= vdim && ld_gate >= heads * vdim && o && gate && out,
                "sigmoid_gate: bad sizes or a null pointer");
    RMX_REQUIRE(o != out || o_head == vdim, "sigmoid_gate: in place only where heads are not padded");
    const size_t total = (size_t)n_tokens * heads * vdim;
    const int threads = 256;
    const dim3 grid((unsigned)((total + threads - 1) / threads));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(sigmoid_gate_kernel<float>, grid, dim3(threads), 0, s, (const float*)o, o_head, (const float*)gate,
                                            ld_gate, (float*)out, heads, vdim, total), "sigmoid_gate");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, (const __nv_bfloat16*)o, o_head,
                                            (const __nv_bfloat16*)gate, ld_gate, (__nv_bfloat16*)out, heads, vdim, total), "sigmoid_gate");
    else
        RMX_FAIL("sigmoid_gate: unknown dtype %d", dtype);
    return 0;
}

// The "decay" form: per head and channel a_t = exp(-exp(w_t + w0)); o_t = S_(t-1)^T r_t + (sum_c r_c u_c k_c) v_t, then
// S_t = diag(a_t) S_(t-1) + k_t v_t^T.  r, k, w: [tokens, heads * K] columns, v: [tokens, heads * V] columns, w0 and u float
// [heads * K]; scratch af, kf, qf [tokens, heads, row] and bonus [tokens, heads].
RMX_API int rmx_decay_recurrence(float* state, float* out, const int* q_start, const int* slots, int n_seqs, int n_tokens, int heads, int K,
                                 int V, const void* r, int ld_r, const void* k, int ld_k, const void* w, int ld_w, const void* v, int ld_v,
                                 const float* w0, const float* u, float* af, float* kf, float* qf, float* bonus, int warps, int dtype,
                                 void* stream) {
    if (n_seqs == 0 || n_tokens == 0) return 0;
    RMX_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && heads > 0 && heads <= 65535 && K > 0 && V > 0 && n_tokens > 0, "decay_recurrence: bad sizes");
    RMX_REQUIRE(K <= 256, "decay_recurrence: a state of %d rows a head is beyond 256", K);
    RMX_REQUIRE(state && out && q_start && slots && r && k && w && v && w0 && u && af && kf && qf && bonus, "decay_recurrence: a null pointer");
    RMX_REQUIRE(warps >= 1 && warps <= 8, "decay_recurrence: 1 to 8 warps a block");
    RMX_REQUIRE(dtype == RMX_F32 || dtype == RMX_BF16, "decay_recurrence: unknown dtype %d", dtype);
    const int kpt = rec_kpt(K), row = rec_row(kpt), threads = 256;
    RMX_REQUIRE((heads * row + threads - 1) / threads <= 65535, "decay_recurrence: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens, (heads * row + threads - 1) / threads);
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(recurrence_prepare_decay_kernel<float>, grid, dim3(threads), 0, s, (const float*)r, ld_r, (const float*)k,
                                            ld_k, (const float*)w, ld_w, w0, u, af, kf, qf, bonus, heads, K, kpt), "recurrence_prepare");
    else
        RMX_CHECK_LAUNCHED(launch_dependent(recurrence_prepare_decay_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, (const __nv_bfloat16*)r, ld_r,
                                            (const __nv_bfloat16*)k, ld_k, (const __nv_bfloat16*)w, ld_w, w0, u, af, kf, qf, bonus, heads, K, kpt),
                           "recurrence_prepare");
    ScanArgs a;
    a.state = state; a.out = out; a.q_start = q_start; a.slots = slots; a.kf = kf; a.qf = qf; a.af = af;
    a.heads = heads; a.K = K; a.V = V; a.steps = 0; a.bonus = bonus; a.v = v; a.ld_v = ld_v; a.v_scale = nullptr; a.skip = nullptr;
    a.row_heads = heads;
    return dtype == RMX_F32 ? launch_scan<float, true, true>(a, n_seqs, warps, s) : launch_scan<__nv_bfloat16, true, true>(a, n_seqs, warps, s);
}

// x [tokens, channels] dense, mu float [n_mix, channels], out [n_mix, tokens, channels], last [slots, channels] of x's type.
RMX_API int rmx_token_shift_mix(const void* x, const float* mu, void* out, void* last, int channels, int n_mix, const int* positions,
                                const int* seq_index, const int* slots, const int* q_start, int n_tokens, int n_seqs, int single_tokens,
                                int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(channels > 0 && n_mix > 0 && n_seqs > 0 && n_seqs <= 65535 && x && mu && out && last, "token_shift_mix: bad sizes or a null pointer");
    const size_t total = (size_t)n_tokens * channels;
    const dim3 grid((unsigned)((total + 255) / 256)), sgrid((channels + 255) / 256, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32) {
        RMX_CHECK_LAUNCHED(launch_dependent(token_shift_mix_kernel<float>, grid, dim3(256), 0, s, (const float*)x, mu, (float*)out, (float*)last,
                                            channels, n_mix, positions, seq_index, slots, q_start, total, single_tokens), "token_shift_mix");
        if (!single_tokens)
            RMX_CHECK_LAUNCHED(launch_dependent(token_shift_state_kernel<float>, sgrid, dim3(256), 0, s, (const float*)x, (float*)last, channels,
                                                slots, q_start, n_seqs), "token_shift_state");
    } else if (dtype == RMX_BF16) {
        if (channels % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)last & 15) == 0 && ((uintptr_t)mu & 15) == 0)
            RMX_CHECK_LAUNCHED(launch_dependent(token_shift_mix8_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, s,
                                                (const __nv_bfloat16*)x, mu, (__nv_bfloat16*)out, (__nv_bfloat16*)last, channels, n_mix, positions,
                                                seq_index, slots, q_start, total / 8, single_tokens), "token_shift_mix");
        else
            RMX_CHECK_LAUNCHED(launch_dependent(token_shift_mix_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x, mu,
                                                (__nv_bfloat16*)out, (__nv_bfloat16*)last, channels, n_mix, positions, seq_index, slots, q_start,
                                                total, single_tokens), "token_shift_mix");
        if (!single_tokens)
            RMX_CHECK_LAUNCHED(launch_dependent(token_shift_state_kernel<__nv_bfloat16>, sgrid, dim3(256), 0, s, (const __nv_bfloat16*)x,
                                                (__nv_bfloat16*)last, channels, slots, q_start, n_seqs), "token_shift_state");
    } else {
        RMX_FAIL("token_shift_mix: unknown dtype %d", dtype);
    }
    return 0;
}
