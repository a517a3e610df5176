// Per-head RMSNorm of q and k, rotation, and the write of keys and values into pages.
//
// Input is the fused projection row [q heads | k heads | v heads] of every token.  One
// warp takes one (token, head):
//   q head: q = RMSNorm(q; q_norm, eps) -> rotate -> q_out[token, head, :]
//   k head: k = RMSNorm(k; k_norm, eps) -> rotate -> k_pool[page, kv head, slot, :]
//   v head: copy                                   -> v_pool[page, kv head, slot, :]
// with page = block_table[seq, pos / page_size], slot = pos % page_size.
// Rotation (half-split): for j < rotary_dim / 2, angle = pos * inv_freq[j] in float,
//   out[j] = x[j] cos - x[j + half] sin, out[j + half] = x[j + half] cos + x[j] sin;
// numbers from rotary_dim on pass through.  Norm weights are float; either may be null
// (no norm).  With write_kv == 0 only q is produced (a layer that reads another layer's
// cache).  Everything is computed in float and rounded once to T.
//
// The cosines and sines of a step's positions are the same for every head and every layer:
// rope_table_kernel forms them once per step ([token][cos of j | sin of j], float, with the same
// float product and the same sincosf), and the kernels here read them when the table is given.
#include "common.cuh"
#include "rope128.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 512;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) qk_rope_cache_kernel(
    const T* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ inv_freq, int rotary_dim, const int* __restrict__ positions,
    const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, T* __restrict__ q_out, int n_tokens, int nq, int nkv, int hd,
    int row_stride, int write_kv, int* __restrict__ status, const float* __restrict__ cos_sin) {
    extern __shared__ float smem[];
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * heads_total) return;
    const int t = (int)(item / heads_total);
    const int head = (int)(item % heads_total);
    float* buf = smem + warp * hd;
    const T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;

    const int pos = positions[t];
    T* dst;
    const float* norm_w;
    bool rotate = true;
    if (head < nq) {
        dst = q_out + ((size_t)t * nq + head) * hd;
        norm_w = q_norm;
    } else {
        const int kvh = (head - nq) % nkv;
        const bool is_v = head >= nq + nkv;
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {  // the host reserves pages before the step; never write through a hole
            if (lane == 0) atomicExch(status, 1);
            return;
        }
        const size_t off = (((size_t)page * nkv + kvh) * page_size + pos % page_size) * hd;
        dst = (is_v ? v_pool : k_pool) + off;
        norm_w = is_v ? nullptr : k_norm;
        rotate = !is_v;
    }

    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) {
        const float v = to_float(src[d]);
        buf[d] = v;
        ss += v * v;
    }
    if (norm_w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)hd + eps);
        __syncwarp();
        for (int d = lane; d < hd; d += 32) buf[d] = buf[d] * inv * norm_w[d];
    }
    __syncwarp();
    const int half = rotary_dim >> 1;
    if (rotate && half > 0) {
        for (int j = lane; j < half; j += 32) {
            float sn, cs;
            if (cos_sin) {
                cs = cos_sin[(size_t)t * rotary_dim + j];
                sn = cos_sin[(size_t)t * rotary_dim + half + j];
            } else {
                sincosf((float)pos * inv_freq[j], &sn, &cs);
            }
            const float a = buf[j], b = buf[j + half];
            dst[j] = from_float<T>(a * cs - b * sn);
            dst[j + half] = from_float<T>(b * cs + a * sn);
        }
        for (int d = rotary_dim + lane; d < hd; d += 32) dst[d] = from_float<T>(buf[d]);
    } else {
        for (int d = lane; d < hd; d += 32) dst[d] = from_float<T>(buf[d]);
    }
}

// cos_sin[t][j] = magnitude * cos(pos_t * inv_freq[j]), cos_sin[t][half + j] = magnitude * sin(...): once per step.
// (magnitude: a factor that some scaled rotations put on the rotated numbers, and on them only; 1 otherwise.)
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_sin, int n_tokens, int half, float magnitude) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tokens * half) return;
    const int t = idx / half, j = idx - t * half;
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
    cos_sin[(size_t)t * 2 * half + j] = magnitude == 1.f ? cs : cs * magnitude;
    cos_sin[(size_t)t * 2 * half + half + j] = magnitude == 1.f ? sn : sn * magnitude;
}

// bfloat16, head size 128, all 128 numbers rotated, table given: a lane holds four neighbouring numbers of the
// head; the partner of number j is j + 64, sixteen lanes away.  A warp takes PER_WARP (token, head) items and
// issues all their loads before it works on the first, so that their latencies overlap.
constexpr int PER_WARP = 4;

__global__ void __launch_bounds__(WARPS * 32) qk_rope_cache_128_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ cos_sin, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int table_stride, int page_size, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ q_out, int n_tokens, int nq, int nkv, int row_stride,
    int write_kv, int* __restrict__ status) {
    constexpr int hd = 128;
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int total = n_tokens * heads_total;   // the launcher keeps this below 2^31
    const int first = (blockIdx.x * WARPS + warp) * PER_WARP;
    if (first >= total) return;
    uint2 raw[PER_WARP];
    __nv_bfloat16* dst[PER_WARP];
    const float* norm_w[PER_WARP];
    int tok[PER_WARP];
    bool rotate[PER_WARP], live[PER_WARP];
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
        const int item = first + u;
        live[u] = item < total;
        const int t = live[u] ? item / heads_total : 0;
        const int head = live[u] ? item - t * heads_total : 0;
        tok[u] = t;
        raw[u] = *reinterpret_cast<const uint2*>(qkv + (size_t)t * row_stride + (size_t)head * hd + lane * 4);
        rotate[u] = true;
        if (head < nq) {
            dst[u] = q_out + ((size_t)t * nq + head) * hd;
            norm_w[u] = q_norm;
        } else {
            const int pos = positions[t];
            const int kvh = (head - nq) % nkv;
            const bool is_v = head >= nq + nkv;
            const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
            if (page < 0) {  // the host reserves pages before the step; never write through a hole
                if (lane == 0 && live[u]) atomicExch(status, 1);
                live[u] = false;
            }
            dst[u] = (is_v ? v_pool : k_pool) + (((size_t)(page < 0 ? 0 : page) * nkv + kvh) * page_size + pos % page_size) * hd;
            norm_w[u] = is_v ? nullptr : k_norm;
            rotate[u] = !is_v;
        }
    }
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
        if (!live[u]) continue;
        if (!rotate[u]) {  // values pass through
            *reinterpret_cast<uint2*>(dst[u] + lane * 4) = raw[u];
            continue;
        }
        const uint2 packed = rope128_head(raw[u], norm_w[u], eps, cos_sin + (size_t)tok[u] * hd, lane);
        *reinterpret_cast<uint2*>(dst[u] + lane * 4) = packed;
    }
}
// The same for many tokens (prompt portions): a warp takes one token and HEADS_PER_WARP neighbouring heads of it,
// two heads a pass (sixteen lanes a head, eight neighbouring numbers a lane, 16-byte loads and stores; the partner
// of number j is j + 64, eight lanes away).  The token's position, page and its cosines and sines are read once a
// warp, and all loads of the warp's heads are under way before the first is worked on.
constexpr int HEADS_PER_WARP = 8;

__global__ void __launch_bounds__(WARPS * 32, 8) qk_rope_cache_128_wide_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ cos_sin, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int table_stride, int page_size, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ q_out, int n_tokens, int nq, int nkv, int row_stride,
    int write_kv, int* __restrict__ status) {
    constexpr int hd = 128, PASSES = HEADS_PER_WARP / 2;
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int groups = (heads_total + HEADS_PER_WARP - 1) / HEADS_PER_WARP;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * groups) return;
    const int t = (int)(item / groups), head0 = (int)(item - (long long)t * groups) * HEADS_PER_WARP;
    const int sub = lane >> 4, l16 = lane & 15;       // which of the pass's two heads, and where in it
    const __nv_bfloat16* src = qkv + (size_t)t * row_stride + l16 * 8;
    uint4 raw[PASSES];
#pragma unroll
    for (int u = 0; u < PASSES; ++u) {
        const int head = head0 + 2 * u + sub;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (head < heads_total) raw[u] = *reinterpret_cast<const uint4*>(src + (size_t)head * hd);
    }
    // cosines and sines of the pairs (j, j + 64) that this lane's eight numbers belong to
    const int j = (l16 & 7) * 8;
    float cs[8], sn[8];
    {
        const float4 c0 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + j);
        const float4 c1 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + j + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + 64 + j);
        const float4 s1 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + 64 + j + 4);
        cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    long long slot_row = -1;   // the row of the pools' [pages * nkv * page_size] rows that kv head 0 of this token has
    if (head0 + HEADS_PER_WARP > nq && write_kv) {
        const int pos = positions[t];
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {  // the host reserves pages before the step; never write through a hole
            if (lane == 0) atomicExch(status, 1);
        } else {
            slot_row = (long long)page * nkv * page_size + pos % page_size;
        }
    }
#pragma unroll
    for (int u = 0; u < PASSES; ++u) {
        const int head = head0 + 2 * u + sub;
        const bool live = head < heads_total;
        const bool is_q = head < nq, is_v = head >= nq + nkv;
        __nv_bfloat16* dst = nullptr;
        if (live) {
            if (is_q) dst = q_out + ((size_t)t * nq + head) * hd + l16 * 8;
            else if (slot_row >= 0)
                dst = (is_v ? v_pool : k_pool) + (size_t)(slot_row + (long long)((head - nq) % nkv) * page_size) * hd + l16 * 8;
        }
        const uint32_t rw[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
        // every lane takes part in the shuffles, whatever its head is
        const bool normed = live && !is_v && (is_q ? q_norm != nullptr : k_norm != nullptr);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (normed) {
            const float inv = rsqrtf(ss / (float)hd + eps);
            const float* w = (is_q ? q_norm : k_norm) + l16 * 8;   // (the same 512 bytes for every warp: they stay in L1)
            const float4 a = *reinterpret_cast<const float4*>(w), b = *reinterpret_cast<const float4*>(w + 4);
            v[0] = v[0] * inv * a.x; v[1] = v[1] * inv * a.y; v[2] = v[2] * inv * a.z; v[3] = v[3] * inv * a.w;
            v[4] = v[4] * inv * b.x; v[5] = v[5] * inv * b.y; v[6] = v[6] * inv * b.z; v[7] = v[7] * inv * b.w;
        }
        float out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
            // lanes 0..7 of a head hold x[j] (partner x[j + 64] eight lanes on): out = a cos - b sin
            // lanes 8..15 hold x[j + 64] (partner x[j]):                          out = b cos + a sin
            out[i] = is_v ? v[i] : (l16 < 8 ? v[i] * cs[i] - other * sn[i] : v[i] * cs[i] + other * sn[i]);
        }
        if (dst) {
            if (is_v) {
                *reinterpret_cast<uint4*>(dst) = raw[u];   // values pass through
            } else {
                uint32_t ow[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 r = __floats2bfloat162_rn(out[2 * i], out[2 * i + 1]);
                    ow[i] = *reinterpret_cast<uint32_t*>(&r);
                }
                *reinterpret_cast<uint4*>(dst) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
        }
    }
}
// The norm taken over the whole projection instead of a head at a time: q (all nq * dq numbers of a token at once) and k
// (all nkv * dq) are each divided by their root mean square and multiplied by a weight of the projection's size, then
// split into heads and rotated as above.  Query/key heads have dq numbers, value heads dv; the cache's heads have
// hd >= max(dq, dv) numbers, the rest of a head is written as zeros (a zero in q and k adds nothing to a score, and the
// zero columns of a value head come out as zeros).  Input rows are [q | k | v].  One block a token.
template <typename T>
__global__ void __launch_bounds__(1024) qk_whole_norm_rope_cache_kernel(
    const T* __restrict__ qkv, int row_stride, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ inv_freq, int rotary_dim, const float* __restrict__ cos_sin, const int* __restrict__ positions,
    const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, T* __restrict__ q_out, int nq, int nkv, int dq, int dv, int hd,
    int write_kv, int* __restrict__ status) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    allow_dependents();
    wait_for_prior_kernels();
    const int t = blockIdx.x;
    const int nqd = nq * dq, nkd = nkv * dq;
    const T* row = qkv + (size_t)t * row_stride;
    float* qb = smem;            // [nq * dq]
    float* kb = smem + nqd;      // [nkv * dq]
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nqd; i += blockDim.x) {
        const float v = to_float(row[i]);
        qb[i] = v;
        sq += v * v;
    }
    for (int i = threadIdx.x; i < nkd; i += blockDim.x) {
        const float v = to_float(row[nqd + i]);
        kb[i] = v;
        sk += v * v;
    }
    const float inv_q = q_norm ? rsqrtf(block_sum(sq, scratch) / (float)nqd + eps) : 1.f;
    const float inv_k = k_norm ? rsqrtf(block_sum(sk, scratch) / (float)nkd + eps) : 1.f;
    __syncthreads();
    for (int i = threadIdx.x; i < nqd; i += blockDim.x) qb[i] = q_norm ? qb[i] * inv_q * q_norm[i] : qb[i];
    for (int i = threadIdx.x; i < nkd; i += blockDim.x) kb[i] = k_norm ? kb[i] * inv_k * k_norm[i] : kb[i];
    __syncthreads();
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    size_t page_off = 0;
    if (write_kv) {
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {
            if (threadIdx.x == 0) atomicExch(status, 1);
            write_kv = 0;
        }
        page_off = (size_t)(page < 0 ? 0 : page) * nkv;
    }
    const int heads = nq + (write_kv ? nkv : 0);
    for (int e = threadIdx.x; e < heads * hd; e += blockDim.x) {
        const int head = e / hd, d = e - head * hd;
        const float* src = head < nq ? qb + head * dq : kb + (head - nq) * dq;
        float v = 0.f;
        if (d < dq) {
            v = src[d];
            if (d < rotary_dim) {
                const int j = d < half ? d : d - half;
                float sn, cs;
                if (cos_sin) {
                    cs = cos_sin[(size_t)t * rotary_dim + j];
                    sn = cos_sin[(size_t)t * rotary_dim + half + j];
                } else {
                    sincosf((float)pos * inv_freq[j], &sn, &cs);
                }
                v = d < half ? src[d] * cs - src[d + half] * sn : src[d] * cs + src[d - half] * sn;
            }
        }
        if (head < nq) q_out[((size_t)t * nq + head) * hd + d] = from_float<T>(v);
        else k_pool[((page_off + (head - nq)) * page_size + pos % page_size) * hd + d] = from_float<T>(v);
    }
    if (write_kv) {
        const T* vrow = row + nqd + nkd;
        for (int e = threadIdx.x; e < nkv * hd; e += blockDim.x) {
            const int head = e / hd, d = e - head * hd;
            v_pool[((page_off + head) * page_size + pos % page_size) * hd + d] = d < dv ? vrow[head * dv + d] : from_float<T>(0.f);
        }
    }
}

// The same split, rotation and page write where nothing is normed, for bfloat16 rows whose sizes are all multiples of
// eight: no staging and no sums.  A thread takes eight neighbouring numbers of a head; in the rotated part it takes the
// eight they pair with as well (d and d + rotary_dim / 2) and writes both.  Cosines and sines come from the step's table
// [token, rotary_dim] (cosines, then sines), in float.
__global__ void __launch_bounds__(256) qk_part_rope_cache_bf16_kernel(
    const __nv_bfloat16* __restrict__ qkv, int row_stride, int rotary_dim, const float* __restrict__ cos_sin,
    const int* __restrict__ positions, const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride,
    int page_size, __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ q_out,
    int n_tokens, int nq, int nkv, int dq, int dv, int hd, int write_kv, int* __restrict__ status) {
    allow_dependents();
    wait_for_prior_kernels();
    const int half = rotary_dim >> 1;
    const int rotated = half >> 3;                              // units of a head that hold a rotated pair of eights
    const int per_head = rotated + ((hd - rotary_dim) >> 3);    // then the numbers that pass unchanged, then zeros up to hd
    const int qk_units = (nq + nkv) * per_head;
    const int per_token = qk_units + nkv * (hd >> 3);
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * per_token) return;
    const int t = (int)(idx / per_token);
    int u = (int)(idx - (long long)t * per_token);
    const __nv_bfloat16* row = qkv + (size_t)t * row_stride;
    const int pos = positions[t];
    size_t slot = 0;                                            // the token's place in its page, in heads' rows
    if (u >= nq * per_head) {
        if (!write_kv) return;
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {
            atomicExch(status, 1);
            return;
        }
        slot = (size_t)page * nkv;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    if (u < qk_units) {
        const int head = u / per_head, w = u - head * per_head;
        const __nv_bfloat16* src = row + (size_t)head * dq;     // (key heads follow the query heads in the row)
        __nv_bfloat16* dst = head < nq ? q_out + ((size_t)t * nq + head) * hd
                                       : k_pool + ((slot + (head - nq)) * page_size + pos % page_size) * hd;
        if (w < rotated) {
            const int d0 = w << 3;
            const uint4 ra = *reinterpret_cast<const uint4*>(src + d0), rb = *reinterpret_cast<const uint4*>(src + d0 + half);
            const float* cs = cos_sin + (size_t)t * rotary_dim + d0;
            const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(cs + half), s1 = *reinterpret_cast<const float4*>(cs + half + 4);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(&ra);
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&rb);
            uint4 oa, ob;
            __nv_bfloat16* pa = reinterpret_cast<__nv_bfloat16*>(&oa);
            __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(&ob);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float x = __bfloat162float(a[i]), y = __bfloat162float(b[i]);
                pa[i] = __float2bfloat16_rn(x * c[i] - y * sn[i]);
                pb[i] = __float2bfloat16_rn(y * c[i] + x * sn[i]);
            }
            *reinterpret_cast<uint4*>(dst + d0) = oa;
            *reinterpret_cast<uint4*>(dst + d0 + half) = ob;
        } else {
            const int d0 = rotary_dim + ((w - rotated) << 3);
            *reinterpret_cast<uint4*>(dst + d0) = d0 < dq ? *reinterpret_cast<const uint4*>(src + d0) : zero;
        }
    } else if (v_pool != nullptr) {
        u -= qk_units;
        const int head = u / (hd >> 3), d0 = (u - head * (hd >> 3)) << 3;
        __nv_bfloat16* dst = v_pool + ((slot + head) * page_size + pos % page_size) * hd + d0;
        *reinterpret_cast<uint4*>(dst) = d0 < dv ? *reinterpret_cast<const uint4*>(row + (size_t)(nq + nkv) * dq + (size_t)head * dv + d0) : zero;
    }
}
}  // namespace

RMX_API int rmx_qk_whole_norm_rope_cache(const void* qkv, int row_stride, const float* q_norm, const float* k_norm, float eps,
                                         const float* inv_freq, int rotary_dim, const float* cos_sin, const int* positions,
                                         const int* seq_index, const int* block_table, int table_stride, int page_size, void* k_pool,
                                         void* v_pool, void* q_out, int n_tokens, int nq, int nkv, int dq, int dv, int hd, int write_kv,
                                         int* status, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && dq > 0 && dv > 0 && hd >= dq && hd >= dv, "qk_whole_norm_rope_cache: bad head sizes");
    RMX_REQUIRE(rotary_dim >= 0 && rotary_dim <= dq && rotary_dim % 2 == 0, "qk_whole_norm_rope_cache: rotary_dim %d must be even and at most %d", rotary_dim, dq);
    RMX_REQUIRE(rotary_dim == 0 || inv_freq != nullptr || cos_sin != nullptr, "qk_whole_norm_rope_cache: rotation without a table");
    RMX_REQUIRE(page_size > 0 && table_stride > 0, "qk_whole_norm_rope_cache: bad page geometry");
    RMX_REQUIRE(row_stride >= (nq + nkv) * dq + nkv * dv, "qk_whole_norm_rope_cache: row stride %d too small", row_stride);
    const size_t smem = (size_t)(nq + nkv) * dq * sizeof(float);
    RMX_REQUIRE(smem <= 200 * 1024, "qk_whole_norm_rope_cache: a projection of %d numbers is beyond 51200", (nq + nkv) * dq);
    cudaStream_t s = (cudaStream_t)stream;
    const bool eights = dq % 8 == 0 && dv % 8 == 0 && hd % 8 == 0 && rotary_dim % 16 == 0 && row_stride % 8 == 0 &&
                        ((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)q_out | (uintptr_t)cos_sin) % 16 == 0;
    if (dtype == RMX_BF16 && q_norm == nullptr && k_norm == nullptr && eights && (rotary_dim == 0 || cos_sin != nullptr)) {
        const long long units = (long long)n_tokens * ((nq + nkv) * (rotary_dim / 16 + (hd - rotary_dim) / 8) + nkv * (hd / 8));
        RMX_CHECK_LAUNCHED(launch_dependent(qk_part_rope_cache_bf16_kernel, dim3((unsigned)((units + 255) / 256)), dim3(256), 0, s,
            (const __nv_bfloat16*)qkv, row_stride, rotary_dim, cos_sin, positions, seq_index, block_table, table_stride, page_size,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens, nq, nkv, dq, dv, hd, write_kv, status),
            "qk_part_rope_cache");
        return 0;
    }
    if (dtype == RMX_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(qk_whole_norm_rope_cache_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        RMX_CHECK_LAUNCHED(launch_dependent(qk_whole_norm_rope_cache_kernel<float>, dim3(n_tokens), dim3(256), smem, s, (const float*)qkv, row_stride,
            q_norm, k_norm, eps, inv_freq, rotary_dim, cos_sin, positions, seq_index, block_table, table_stride, page_size, (float*)k_pool,
            (float*)v_pool, (float*)q_out, nq, nkv, dq, dv, hd, write_kv, status), "qk_whole_norm_rope_cache");
    } else if (dtype == RMX_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(qk_whole_norm_rope_cache_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // (few tokens, decoding: a block a token is all the parallelism there is, so the block is as large as it can be; the
        // 32-bit run keeps one block size, because the size decides the order in which the squares are added)
        RMX_CHECK_LAUNCHED(launch_dependent(qk_whole_norm_rope_cache_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(n_tokens <= 64 ? 1024 : 256), smem, s,
            (const __nv_bfloat16*)qkv, row_stride, q_norm, k_norm, eps, inv_freq, rotary_dim, cos_sin, positions, seq_index, block_table,
            table_stride, page_size, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, nq, nkv, dq, dv, hd, write_kv,
            status), "qk_whole_norm_rope_cache");
    } else {
        RMX_FAIL("qk_whole_norm_rope_cache: unknown dtype %d", dtype);
    }
    return 0;
}

RMX_API int rmx_rope_table(const int* positions, const float* inv_freq, float* cos_sin, int n_tokens, int rotary_dim,
                           float magnitude, void* stream) {
    if (n_tokens == 0 || rotary_dim == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && rotary_dim > 0 && rotary_dim % 2 == 0, "rope_table: bad sizes");
    const int half = rotary_dim / 2, total = n_tokens * half;
    RMX_CHECK_LAUNCHED(launch_dependent(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, positions,
                                        inv_freq, cos_sin, n_tokens, half, magnitude), "rope_table");
    return 0;
}

RMX_API int rmx_qk_rope_cache(const void* qkv, const float* q_norm, const float* k_norm, float eps,
                              const float* inv_freq, int rotary_dim, const int* positions, const int* seq_index,
                              const int* block_table, int table_stride, int page_size, void* k_pool, void* v_pool,
                              void* q_out, int n_tokens, int nq, int nkv, int hd, int row_stride, int write_kv,
                              int* status, const float* cos_sin, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && hd > 0 && hd <= MAX_HD, "qk_rope_cache: head_dim %d must be in 1..%d", hd, MAX_HD);
    RMX_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "qk_rope_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    RMX_REQUIRE(page_size > 0 && table_stride > 0, "qk_rope_cache: bad page geometry");
    RMX_REQUIRE(row_stride >= (nq + (write_kv ? 2 * nkv : 0)) * hd, "qk_rope_cache: row stride %d too small", row_stride);
    RMX_REQUIRE(rotary_dim == 0 || inv_freq != nullptr || cos_sin != nullptr, "qk_rope_cache: rotation without a table");
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long items = (long long)n_tokens * heads_total;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_BF16 && hd == 128 && rotary_dim == 128 && cos_sin != nullptr && row_stride % 4 == 0 &&
        ((uintptr_t)qkv & 7) == 0 && items < (1LL << 30)) {
        if (n_tokens >= 256 && row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0) {   // prompt portions
            const long long warps = (long long)n_tokens * ((heads_total + HEADS_PER_WARP - 1) / HEADS_PER_WARP);
            RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_128_wide_kernel, dim3((unsigned)((warps + WARPS - 1) / WARPS)), dim3(WARPS * 32), 0, s,
                (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, cos_sin, positions, seq_index, block_table, table_stride, page_size,
                (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens, nq, nkv, row_stride, write_kv, status),
                "qk_rope_cache_128_wide");
            return 0;
        }
        const unsigned blocks128 = (unsigned)((items + (long long)WARPS * PER_WARP - 1) / (WARPS * PER_WARP));
        RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_128_kernel, dim3(blocks128), dim3(WARPS * 32), 0, s,
            (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, cos_sin, positions, seq_index, block_table, table_stride, page_size,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens, nq, nkv, row_stride, write_kv, status),
            "qk_rope_cache_128");
        return 0;
    }
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_kernel<float>, dim3(blocks), dim3(WARPS * 32), smem, s,
            (const float*)qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table,
            table_stride, page_size, (float*)k_pool, (float*)v_pool, (float*)q_out, n_tokens, nq, nkv, hd, row_stride, write_kv, status, cos_sin), "qk_rope_cache");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), smem, s,
            (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table,
            table_stride, page_size, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens,
            nq, nkv, hd, row_stride, write_kv, status, cos_sin), "qk_rope_cache");
    else
        RMX_FAIL("qk_rope_cache: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("qk_rope_cache");
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// The general split of a projection row [q (nq * dq) | k (nkv * dq) | v (nkv * dv)] into heads, for mixers whose options
// the kernels above do not take together.  One warp a (token, head), everything in float, one rounding:
//   + bias (float, as long as the row; or null)
//   q, k: RMS norm over the head's dq numbers with a weight of dq numbers that all heads share (null: no norm)
//   q, k: rotation of the first `rot` numbers by the step's table `cos_sin` [tokens][cos of pair j | sin of pair j];
//         pairs are (j, j + rot / 2), or with `interleaved` neighbours (2j, 2j + 1)
//   v:    with `v_cos_sin` (a table over dv numbers) the value is rotated too, over all its dv numbers, pairs as
//         `v_interleaved` says: a value is then cached turned by its own position
//   q goes to q_out [tokens, nq, hd], k and v into their pages; heads narrower than hd are padded with zeros.
namespace {
template <typename T>
__global__ void __launch_bounds__(WARPS * 32) heads_rope_cache_kernel(
    const T* __restrict__ qkv, int row_stride, const float* __restrict__ bias, const float* __restrict__ q_norm,
    const float* __restrict__ k_norm, float eps, const float* __restrict__ cos_sin, int rot, int interleaved,
    const float* __restrict__ v_cos_sin, int v_interleaved, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int table_stride, int page_size, T* __restrict__ k_pool, T* __restrict__ v_pool,
    T* __restrict__ q_out, int n_tokens, int nq, int nkv, int dq, int dv, int hd, int write_kv, int* __restrict__ status) {
    extern __shared__ float smem[];
    allow_dependents();
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * heads_total) return;
    const int t = (int)(item / heads_total);
    const int head = (int)(item % heads_total);
    float* buf = smem + warp * hd;
    const int pos = positions[t];
    int col, n, turn = rot, neighbours = interleaved;
    const float* table = cos_sin;
    const float* norm_w;
    T* dst;
    if (head < nq) {
        col = head * dq; n = dq; norm_w = q_norm;
        dst = q_out + ((size_t)t * nq + head) * hd;
    } else {
        const int kvh = (head - nq) % nkv;
        const bool is_v = head >= nq + nkv;
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {
            if (lane == 0) atomicExch(status, 1);
            return;
        }
        const size_t off = (((size_t)page * nkv + kvh) * page_size + pos % page_size) * hd;
        dst = (is_v ? v_pool : k_pool) + off;
        if (is_v) {
            col = (nq + nkv) * dq + kvh * dv; n = dv; norm_w = nullptr;
            table = v_cos_sin; turn = v_cos_sin ? dv : 0; neighbours = v_interleaved;
        } else {
            col = nq * dq + kvh * dq; n = dq; norm_w = k_norm;
        }
    }
    const T* src = qkv + (size_t)t * row_stride + col;
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) {
        float v = to_float(src[d]);
        if (bias) v += bias[col + d];
        buf[d] = v;
        ss = fmaf(v, v, ss);
    }
    if (norm_w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)n + eps);
        __syncwarp();
        for (int d = lane; d < n; d += 32) buf[d] = buf[d] * inv * norm_w[d];
    }
    __syncwarp();
    const int half = (table ? turn : 0) >> 1;
    for (int j = lane; j < half; j += 32) {
        const float cs = table[(size_t)t * turn + j], sn = table[(size_t)t * turn + half + j];
        const int ia = neighbours ? 2 * j : j, ib = neighbours ? 2 * j + 1 : j + half;
        const float a = buf[ia], b = buf[ib];
        dst[ia] = from_float<T>(a * cs - b * sn);
        dst[ib] = from_float<T>(b * cs + a * sn);
    }
    for (int d = 2 * half + lane; d < n; d += 32) dst[d] = from_float<T>(buf[d]);
    for (int d = n + lane; d < hd; d += 32) dst[d] = from_float<T>(0.f);
}

// out[t, h, 0:dv] = o[t, h, 0:dv] turned by MINUS the token's angles (table [tokens][cos | sin] over dv numbers): what a
// head gives when its values were cached turned by their own positions.  o's heads are hd numbers apart, out is dense.
template <typename T>
__global__ void unrotate_heads_kernel(const T* __restrict__ o, const float* __restrict__ cos_sin, int interleaved, T* __restrict__ out,
                                      int heads, int dv, int hd, size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int half = dv >> 1;
    const size_t th = idx / half;
    const int j = (int)(idx - th * half);
    const size_t t = th / heads;
    const float cs = cos_sin[t * dv + j], sn = cos_sin[t * dv + half + j];
    const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
    const float a = to_float(o[th * hd + ia]), b = to_float(o[th * hd + ib]);
    out[th * dv + ia] = from_float<T>(a * cs + b * sn);
    out[th * dv + ib] = from_float<T>(b * cs - a * sn);
}
}  // namespace

RMX_API int rmx_heads_rope_cache(const void* qkv, int row_stride, const float* bias, const float* q_norm, const float* k_norm, float eps,
                                 const float* cos_sin, int rot, int interleaved, const float* v_cos_sin, int v_interleaved,
                                 const int* positions, const int* seq_index, const int* block_table, int table_stride, int page_size,
                                 void* k_pool, void* v_pool, void* q_out, int n_tokens, int nq, int nkv, int dq, int dv, int hd,
                                 int write_kv, int* status, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && dq > 0 && dv > 0 && hd >= dq && hd >= dv && hd <= MAX_HD, "heads_rope_cache: bad head sizes %d %d %d", dq, dv, hd);
    RMX_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dq && (rot == 0 || cos_sin), "heads_rope_cache: %d rotated numbers of %d", rot, dq);
    RMX_REQUIRE(v_cos_sin == nullptr || dv % 2 == 0, "heads_rope_cache: rotated values need an even size");
    RMX_REQUIRE(page_size > 0 && table_stride > 0, "heads_rope_cache: bad page geometry");
    const long long items = (long long)n_tokens * (nq + (write_kv ? 2 * nkv : 0));
    const dim3 grid((unsigned)((items + WARPS - 1) / WARPS));
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(heads_rope_cache_kernel<float>, grid, dim3(WARPS * 32), smem, s, (const float*)qkv, row_stride, bias,
                                            q_norm, k_norm, eps, cos_sin, rot, interleaved, v_cos_sin, v_interleaved, positions, seq_index,
                                            block_table, table_stride, page_size, (float*)k_pool, (float*)v_pool, (float*)q_out, n_tokens, nq,
                                            nkv, dq, dv, hd, write_kv, status), "heads_rope_cache");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(heads_rope_cache_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), smem, s, (const __nv_bfloat16*)qkv,
                                            row_stride, bias, q_norm, k_norm, eps, cos_sin, rot, interleaved, v_cos_sin, v_interleaved,
                                            positions, seq_index, block_table, table_stride, page_size, (__nv_bfloat16*)k_pool,
                                            (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens, nq, nkv, dq, dv, hd, write_kv, status),
                           "heads_rope_cache");
    else
        RMX_FAIL("heads_rope_cache: unknown dtype %d", dtype);
    return 0;
}

RMX_API int rmx_unrotate_heads(const void* o, const float* cos_sin, int interleaved, void* out, int n_tokens, int heads, int dv, int hd,
                               int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(heads > 0 && dv > 0 && dv % 2 == 0 && hd >= dv && o && out && cos_sin && o != out, "unrotate_heads: bad sizes or pointers");
    const size_t total = (size_t)n_tokens * heads * (dv / 2);
    const dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(unrotate_heads_kernel<float>, grid, dim3(256), 0, s, (const float*)o, cos_sin, interleaved,
                                            (float*)out, heads, dv, hd, total), "unrotate_heads");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(unrotate_heads_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)o, cos_sin,
                                            interleaved, (__nv_bfloat16*)out, heads, dv, hd, total), "unrotate_heads");
    else
        RMX_FAIL("unrotate_heads: unknown dtype %d", dtype);
    return 0;
}
