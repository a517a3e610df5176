// Attention whose scores are mixed over the heads before the softmax ("talking heads"), over the paged cache:
//
//   s_g[i, j] = scale * q_g[i] . k_kv(g)[j]                   every query head g against its key head
//   s'_h[i, j] = sum_g talk[h, g] * s_g[i, j]                 a learned H x H matrix mixes the heads' scores
//   p_h = softmax_j (s'_h[i, j]) over the keys that i reads;  o_h[i] = sum_j p_h[j] v_kv(h)[j]
//
// A query's row of scores therefore needs ALL heads' scores of the same (query, key) pair: a block takes a token with all
// its heads, one warp a head.  Keys are visited in blocks of 32 aligned to absolute positions in ascending order with an
// online softmax in float; a raw score is summed in ascending d, a mixed score in ascending g.  The order in which numbers
// are added depends on the token's position (and the window) only: not on how a prompt was cut, on the batch, the page
// size or which pages hold the keys.
//
// attention_talk_kernel is the arrangement on the FMA units (both dtypes; the 32-bit path).
#include "common.cuh"

namespace {
constexpr int TKB = 32;   // keys per block

template <typename T>
__global__ void attention_talk_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                      const float* __restrict__ talk, const int* __restrict__ positions,
                                      const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride,
                                      int page_size, T* __restrict__ out, int nq, int nkv, int hd, int dq, int dv, int window,
                                      float scale, int* __restrict__ status) {
    extern __shared__ float smem[];
    const int group = nq / nkv;
    const int t = blockIdx.x;
    const int head = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = head / group;
    const int kstride = dq + 1;
    float* Ks = smem;                               // [TKB][nkv][dq + 1]
    float* Ss = Ks + (size_t)TKB * nkv * kstride;   // [nq][TKB] raw scores
    float* Qs = Ss + nq * TKB;                      // [nq][dq]
    float* Ts = Qs + nq * dq;                       // [nq][nq]
    const int pos = positions[t];
    const int* table = block_table + (size_t)seq_index[t] * table_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    for (int d = lane; d < dq; d += 32) Qs[head * dq + d] = to_float(q[((size_t)t * nq + head) * hd + d]) * scale;
    for (int g = lane; g < nq; g += 32) Ts[head * nq + g] = talk[head * nq + g];

    const int per_lane = (dv + 31) / 32;
    float acc[16];  // value heads of up to 512 numbers
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int row = nkv * dq;

    for (int b = lo / TKB; b <= pos / TKB; ++b) {
        const int base = b * TKB;
        __syncthreads();
        for (int idx = threadIdx.x; idx < TKB * row; idx += blockDim.x) {
            const int j = idx / row, r = idx - j * row;
            const int kh = r / dq, d = r - kh * dq;
            const int kp = base + j;
            float kv = 0.f;
            if (kp >= lo && kp <= pos) {
                const int page = table[kp / page_size];
                if (page >= 0)
                    kv = to_float(k_pool[(((size_t)page * nkv + kh) * page_size + kp % page_size) * hd + d]);
                else if (r == 0)
                    atomicExch(status, 2);  // a key that should be there has no page
            }
            Ks[((size_t)j * nkv + kh) * kstride + d] = kv;
        }
        __syncthreads();
        const int kp = base + lane;
        const bool valid = kp >= lo && kp <= pos;
        {
            float s = 0.f;
            const float* qrow = Qs + head * dq;
            const float* krow = Ks + ((size_t)lane * nkv + kvh) * kstride;
            for (int d = 0; d < dq; ++d) s = fmaf(qrow[d], krow[d], s);
            Ss[head * TKB + lane] = s;
        }
        __syncthreads();
        float s = 0.f;
        for (int g = 0; g < nq; ++g) s = fmaf(Ts[head * nq + g], Ss[g * TKB + lane], s);
        s = valid ? s : -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);  // first block: exp(-inf) = 0
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= corr;
        // where this lane's key has its value (of this warp's value head); -1: nothing to read
        long long voff = -1;
        if (valid) {
            const int page = table[kp / page_size];
            if (page >= 0) voff = (long long)((((size_t)page * nkv + kvh) * page_size + kp % page_size) * hd);
        }
        for (int j = 0; j < TKB; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long off = __shfl_sync(0xffffffffu, voff, j);
            if (off < 0) continue;
            const T* vrow = v_pool + off;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int d = lane + 32 * i;
                if (i < per_lane && d < dv) acc[i] = fmaf(pj, to_float(vrow[d]), acc[i]);
            }
        }
    }
    const float inv_l = 1.f / l;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int d = lane + 32 * i;
        if (i < per_lane && d < dv) out[((size_t)t * nq + head) * dv + d] = from_float<T>(acc[i] * inv_l);
    }
}
}  // namespace

// q [tokens, nq, hd] (the first dq numbers of a head count), pools with heads of hd numbers (keys: the first dq, values: the
// first dv), talk float [nq, nq], out [tokens, nq, dv] dense.
RMX_API int rmx_attention_talk(const void* q, const void* k_pool, const void* v_pool, const float* talk, const int* positions,
                               const int* seq_index, const int* block_table, int table_stride, int page_size, void* out,
                               int n_tokens, int nq, int nkv, int hd, int dq, int dv, int window, float scale, int* status,
                               int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && nq <= 32, "attention_talk: %d query heads over %d kv heads (at most 32)", nq, nkv);
    RMX_REQUIRE(dq > 0 && dv > 0 && dq <= hd && dv <= hd && hd <= 512, "attention_talk: head sizes %d %d in %d", dq, dv, hd);
    RMX_REQUIRE(page_size > 0 && table_stride > 0 && window >= 0 && talk, "attention_talk: bad page geometry or no mixing matrix");
    const size_t smem = ((size_t)TKB * nkv * (dq + 1) + (size_t)nq * TKB + (size_t)nq * dq + (size_t)nq * nq) * sizeof(float);
    RMX_REQUIRE(smem <= 200 * 1024, "attention_talk: %d key heads of %d numbers need too much shared memory", nkv, dq);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_talk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_talk_kernel<float><<<n_tokens, nq * 32, smem, s>>>((const float*)q, (const float*)k_pool, (const float*)v_pool, talk,
                                                                     positions, seq_index, block_table, table_stride, page_size,
                                                                     (float*)out, nq, nkv, hd, dq, dv, window, scale, status);
    } else if (dtype == RMX_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_talk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_talk_kernel<__nv_bfloat16><<<n_tokens, nq * 32, smem, s>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, talk, positions, seq_index,
            block_table, table_stride, page_size, (__nv_bfloat16*)out, nq, nkv, hd, dq, dv, window, scale, status);
    } else {
        RMX_FAIL("attention_talk: unknown dtype %d", dtype);
    }
    RMX_CHECK_LAUNCH("attention_talk");
    return 0;
}
