// Pieces of attention through a cached latent: the two RMS norms after the down projections (the key/value
// latent goes straight into its page), and the per-head output gate.
//
// A mixer of this kind projects its input to a query latent and a key/value latent, both much narrower than
// heads * head size, norms each, and keeps only the key/value latent per token; keys and values are products
// of that latent with per-head weights.  Norms are formed in float whatever the activations' type.
#include "common.cuh"

namespace {
constexpr int THREADS = 128;

// One block per token.  row = proj[t] holds [query latent (q_rank) | key/value latent (kv_rank) | ...].
//   cq[t]   = row[0 : q_rank]            / sqrt(mean(.^2) + eps) * wq
//   page[t] = row[q_rank : q_rank + kv]  / sqrt(mean(.^2) + eps) * wkv     (kv_rank 0: the layer reads another's latents)
// The order of every sum depends on the sizes only.
template <typename T>
__global__ void __launch_bounds__(THREADS) latent_norms_kernel(
    const T* __restrict__ proj, int ld, int q_rank, int kv_rank, const float* __restrict__ wq,
    const float* __restrict__ wkv, float eps, T* __restrict__ cq, T* __restrict__ pool,
    const int* __restrict__ positions, const int* __restrict__ seq_index, const int* __restrict__ block_table,
    int table_stride, int page_size, int* __restrict__ status) {
    __shared__ float scratch[32];
    allow_dependents();
    wait_for_prior_kernels();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += THREADS) {
        const float v = to_float(row[i]);
        ss += v * v;
    }
    const float inv_q = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += THREADS)
        cq[(size_t)t * q_rank + i] = from_float<T>(to_float(row[i]) * inv_q * wq[i]);
    if (kv_rank == 0 || pool == nullptr) return;
    const T* kv = row + q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) {
        const float v = to_float(kv[i]);
        ss += v * v;
    }
    const float inv_kv = rsqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(status, 1);  // a latent was to be written to a position without a page
        return;
    }
    T* dst = pool + ((size_t)page * page_size + pos % page_size) * kv_rank;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) dst[i] = from_float<T>(to_float(kv[i]) * inv_kv * wkv[i]);
}

// A latent with a rotated part.  One block per token.  kv = kvrow[t] holds [latent (kv_rank) | key part (rot)]:
//   page[t] = [ kv[0 : kv_rank] / sqrt(mean(.^2) + eps) * wkv  |  rotate(kv[kv_rank : kv_rank + rot])  |  zeros up to `row` ]
// (the key part is not normed and is shared by all heads), and of every query head h the part that is rotated,
//   q_out[t, h, kv_rank : kv_rank + rot] = rotate(q[t, h, q_rot_at : q_rot_at + rot]),  zeros up to `row`,
// so that a query row [its part carried into the latent's space | its rotated part] meets a page row as one dot product.
// rotate: the pair (u, v) turns by the token's angle j into (u cos - v sin, v cos + u sin); pairs are numbers (2j, 2j + 1)
// (`interleaved`) or (j, j + rot / 2).  cos_sin[t] = [cos of the rot / 2 angles | their sines], float.  Rotation and norm in float.
template <typename T>
__global__ void __launch_bounds__(THREADS) latent_rope_kernel(
    const T* __restrict__ kvrow, int ld_kv, int kv_rank, int rot, int interleaved, const float* __restrict__ wkv, float eps,
    const T* __restrict__ q, int ld_q, int q_head_stride, int q_rot_at, int heads, T* __restrict__ q_out, int row,
    const float* __restrict__ cos_sin, T* __restrict__ pool, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int table_stride, int page_size, int* __restrict__ status) {
    __shared__ float scratch[32];
    allow_dependents();
    wait_for_prior_kernels();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const float* cs = cos_sin + (size_t)t * rot;
    // the queries' rotated parts
    const int tail = row - kv_rank;          // numbers of a row after the latent's: the rotated part, then zeros
    for (int e = threadIdx.x; e < heads * tail; e += THREADS) {
        const int h = e / tail, d = e - h * tail;
        float v = 0.f;
        if (d < rot) {
            const T* src = q + (size_t)t * ld_q + (size_t)h * q_head_stride + q_rot_at;
            const int j = interleaved ? d >> 1 : (d < half ? d : d - half);
            const bool first = interleaved ? (d & 1) == 0 : d < half;
            const int other = interleaved ? d ^ 1 : (d < half ? d + half : d - half);
            const float a = to_float(src[d]), b = to_float(src[other]);
            v = first ? a * cs[j] - b * cs[half + j] : a * cs[j] + b * cs[half + j];
        }
        q_out[((size_t)t * heads + h) * row + kv_rank + d] = from_float<T>(v);
    }
    if (pool == nullptr) return;
    const T* kv = kvrow + (size_t)t * ld_kv;
    float ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) {
        const float v = to_float(kv[i]);
        ss += v * v;
    }
    const float inv_kv = rsqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(status, 1);  // a latent was to be written to a position without a page
        return;
    }
    T* dst = pool + ((size_t)page * page_size + pos % page_size) * row;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) dst[i] = from_float<T>(to_float(kv[i]) * inv_kv * wkv[i]);
    for (int d = threadIdx.x; d < tail; d += THREADS) {
        float v = 0.f;
        if (d < rot) {
            const T* src = kv + kv_rank;
            const int j = interleaved ? d >> 1 : (d < half ? d : d - half);
            const bool first = interleaved ? (d & 1) == 0 : d < half;
            const int other = interleaved ? d ^ 1 : (d < half ? d + half : d - half);
            const float a = to_float(src[d]), b = to_float(src[other]);
            v = first ? a * cs[j] - b * cs[half + j] : a * cs[j] + b * cs[half + j];
        }
        dst[kv_rank + d] = from_float<T>(v);
    }
}

// o[t, h, :] *= sigmoid(gate[t, h]), gate rows ld_gate apart (columns of the down projection's output).
template <typename T>
__global__ void gate_heads_kernel(T* __restrict__ o, const T* __restrict__ gate, int ld_gate, int heads, int vdim,
                                  size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t per_row = (size_t)heads * vdim;
    const size_t t = idx / per_row;
    const int h = (int)((idx - t * per_row) / vdim);
    const float g = to_float(gate[t * ld_gate + h]);
    o[idx] = from_float<T>(to_float(o[idx]) / (1.f + expf(-g)));
}

// bfloat16, eight numbers a thread (16-byte accesses); vdim is a multiple of 8.
__global__ void gate_heads8_kernel(__nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ gate, int ld_gate, int heads,
                                   int vdim, size_t total8) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const size_t per_row = (size_t)heads * vdim / 8;
    const size_t t = idx / per_row;
    const int h = (int)((idx - t * per_row) * 8 / vdim);
    const float g = __bfloat162float(gate[t * ld_gate + h]);
    const float f = 1.f / (1.f + expf(-g));
    uint4 raw = *reinterpret_cast<const uint4*>(o + idx * 8);
    uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
        __nv_bfloat162 r = __floats2bfloat162_rn(v.x * f, v.y * f);
        words[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(o + idx * 8) = make_uint4(words[0], words[1], words[2], words[3]);
}
}  // namespace

RMX_API int rmx_latent_norms(const void* proj, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv,
                             float eps, void* cq, void* pool, const int* positions, const int* seq_index,
                             const int* block_table, int table_stride, int page_size, int n_tokens, int* status,
                             int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && q_rank > 0 && kv_rank >= 0 && ld >= q_rank + kv_rank, "latent_norms: bad sizes");
    RMX_REQUIRE(proj && wq && cq, "latent_norms: a null pointer");
    RMX_REQUIRE(kv_rank == 0 || pool == nullptr || (wkv && positions && seq_index && block_table && table_stride > 0 && page_size > 0 && status),
                "latent_norms: writing latents needs their norm's weight, positions, the block table and a status word");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(latent_norms_kernel<float>, dim3(n_tokens), dim3(THREADS), 0, s, (const float*)proj, ld, q_rank,
                                            kv_rank, wq, wkv, eps, (float*)cq, (float*)pool, positions, seq_index, block_table,
                                            table_stride, page_size, status), "latent_norms");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(latent_norms_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(THREADS), 0, s,
                                            (const __nv_bfloat16*)proj, ld, q_rank, kv_rank, wq, wkv, eps, (__nv_bfloat16*)cq,
                                            (__nv_bfloat16*)pool, positions, seq_index, block_table, table_stride, page_size, status),
                           "latent_norms");
    else
        RMX_FAIL("latent_norms: unknown dtype %d", dtype);
    return 0;
}

// kvrow [tokens] rows ld_kv apart: [latent (kv_rank) | key part (rot)]; q [tokens] rows ld_q apart, head h's rotated part at
// h * q_head_stride + q_rot_at; q_out [tokens, heads, row]; pool [pages, 1, page_size, row] or null (a layer that reads another's
// latents); cos_sin [tokens, rot].  row >= kv_rank + rot.
RMX_API int rmx_latent_rope(const void* kvrow, int ld_kv, int kv_rank, int rot, int interleaved, const float* wkv, float eps,
                            const void* q, int ld_q, int q_head_stride, int q_rot_at, int heads, void* q_out, int row,
                            const float* cos_sin, void* pool, const int* positions, const int* seq_index, const int* block_table,
                            int table_stride, int page_size, int n_tokens, int* status, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && kv_rank > 0 && rot >= 0 && rot % 2 == 0 && row >= kv_rank + rot && heads > 0, "latent_rope: bad sizes");
    RMX_REQUIRE(q && q_out && (rot == 0 || cos_sin), "latent_rope: a null pointer");
    RMX_REQUIRE(pool == nullptr || (kvrow && wkv && positions && seq_index && block_table && table_stride > 0 && page_size > 0 && status),
                "latent_rope: writing latents needs their rows, their norm's weight, positions, the block table and a status word");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(latent_rope_kernel<float>, dim3(n_tokens), dim3(THREADS), 0, s, (const float*)kvrow, ld_kv, kv_rank,
                                            rot, interleaved, wkv, eps, (const float*)q, ld_q, q_head_stride, q_rot_at, heads, (float*)q_out, row,
                                            cos_sin, (float*)pool, positions, seq_index, block_table, table_stride, page_size, status),
                           "latent_rope");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(latent_rope_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(THREADS), 0, s, (const __nv_bfloat16*)kvrow,
                                            ld_kv, kv_rank, rot, interleaved, wkv, eps, (const __nv_bfloat16*)q, ld_q, q_head_stride, q_rot_at,
                                            heads, (__nv_bfloat16*)q_out, row, cos_sin, (__nv_bfloat16*)pool, positions, seq_index, block_table,
                                            table_stride, page_size, status), "latent_rope");
    else
        RMX_FAIL("latent_rope: unknown dtype %d", dtype);
    return 0;
}

RMX_API int rmx_gate_heads(void* o, const void* gate, int ld_gate, int n_tokens, int heads, int vdim, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && heads > 0 && vdim > 0 && ld_gate >= heads && o && gate, "gate_heads: bad sizes or a null pointer");
    const size_t total = (size_t)n_tokens * heads * vdim;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(gate_heads_kernel<float>, dim3(blocks), dim3(threads), 0, s, (float*)o, (const float*)gate,
                                            ld_gate, heads, vdim, total), "gate_heads");
    else if (dtype == RMX_BF16 && (vdim & 7) == 0 && ((uintptr_t)o & 15) == 0)
        RMX_CHECK_LAUNCHED(launch_dependent(gate_heads8_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, s,
                                            (__nv_bfloat16*)o, (const __nv_bfloat16*)gate, ld_gate, heads, vdim, total / 8), "gate_heads");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(gate_heads_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (__nv_bfloat16*)o,
                                            (const __nv_bfloat16*)gate, ld_gate, heads, vdim, total), "gate_heads");
    else
        RMX_FAIL("gate_heads: unknown dtype %d", dtype);
    return 0;
}
