// Embedding gather, residual add + RMSNorm, and SwiGLU.
//
// The residual stream is float32 in every run; activations that kernels hand to one
// another are in the compute type T (float or bfloat16).  Sums of squares, rsqrt and the
// scaling are done in float and rounded once.
#include <type_traits>

#include "activation.cuh"
#include "common.cuh"

// Four consecutive numbers as floats (the address is 16-byte aligned for float, 8 for bfloat16).
__device__ __forceinline__ void load4(const float* p, float4& v) { v = *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float4& v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v = make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4& v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
// Threads of a block that takes one row: four numbers per thread, a whole number of warps.
static inline int block_threads(int width) {
    int t = ((width + 3) / 4 + 31) / 32 * 32;
    return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

// h[t, :] = table[ids[t], :] as float.  An id outside the table writes zeros (the host
// rejects such ids before the step; the kernel never reads outside the table).
// from_last (or null): where from_last[t] != 0 the token's id is not ids[t] but the one the last step's sampling
// left for the token's sequence, last_tokens[slots[seq_index[t]]] (the host launched this step before it read it).
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ h, int width, int vocab, const int* __restrict__ from_last,
                                 const int* __restrict__ seq_index, const int* __restrict__ slots,
                                 const int* __restrict__ last_tokens, const T* __restrict__ pos_table,
                                 const int* __restrict__ positions, int max_positions, float scale, T* __restrict__ rows_out) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int t = blockIdx.x;
    const int id = (from_last && from_last[t]) ? last_tokens[slots[seq_index[t]]] : ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * width;
    // a learned vector of the token's position, added in float (a position outside the table adds nothing: the
    // host refuses such a step before it runs)
    const int pos = pos_table ? positions[t] : -1;
    const T* prow = (pos >= 0 && pos < max_positions) ? pos_table + (size_t)pos * width : nullptr;
    float* out = h + (size_t)t * width;
    // rows_out (or null): the same rows once more, in the table's type, for a model whose later layers read the
    // embedding's output again (the stream itself is overwritten as the layers add to it)
    T* copy = rows_out ? rows_out + (size_t)t * width : nullptr;
    if ((width & 3) == 0) {  // four numbers per thread and pass
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ok) load4(row + i, v);
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;   // (1 unless the model scales its embeddings: exact then)
            if (prow) {
                float4 a;
                load4(prow + i, a);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            *reinterpret_cast<float4*>(out + i) = v;
            if (copy) store4(copy + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = (ok ? to_float(row[i]) : 0.f) * scale + (prow ? to_float(prow[i]) : 0.f);
            out[i] = v;
            if (copy) copy[i] = from_float<T>(v);
        }
    }
}

RMX_API int rmx_embedding(const int* ids, const void* table, float* h, int n_tokens, int width, int vocab,
                          const int* from_last, const int* seq_index, const int* slots, const int* last_tokens,
                          const void* pos_table, const int* positions, int max_positions, float scale, void* rows_out, int dtype,
                          void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embedding: bad sizes");
    RMX_REQUIRE(pos_table == nullptr || (positions && max_positions > 0), "embedding: a position table needs positions and its row count");
    RMX_REQUIRE(from_last == nullptr || (seq_index && slots && last_tokens), "embedding: from_last needs seq_index, slots and last_tokens");
    const int threads = block_threads(width);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, ids, (const float*)table, h, width,
                                            vocab, from_last, seq_index, slots, last_tokens, (const float*)pos_table, positions,
                                            max_positions, scale, (float*)rows_out), "embedding");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(embedding_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, ids,
                                            (const __nv_bfloat16*)table, h, width, vocab, from_last, seq_index, slots, last_tokens,
                                            (const __nv_bfloat16*)pos_table, positions, max_positions, scale, (__nv_bfloat16*)rows_out), "embedding");
    else
        RMX_FAIL("embedding: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("embedding");
    return 0;
}

// One block per output row.  src_row = rows ? rows[r] : r.
//   v = h[src_row] + mult * (delta[src_row] + mult2 * delta2[src_row])   (float; either delta may be null; factors of 1 change nothing)
//   if (write_h) h[src_row] = v
//   x[r] = v * rsqrt(mean(v^2) + eps) * w     (rounded once to T)
//   x2[r] = v * rsqrt(mean(v^2) + eps) * w2   (w2 and x2 given: a layer with two norms of the same stream, one for each of
//                                              two sublayers that run side by side; the mean is formed once)
// The reduction order depends on the width and the block size only.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta, const T* __restrict__ delta2, float mult, float mult2,
                                   const int* __restrict__ rows, const float* __restrict__ w, float eps,
                                   T* __restrict__ x, int width, int write_h, const float* __restrict__ w2, T* __restrict__ x2) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float vals[];
    // what follows (a product) may take its place and fetch its weights now: it waits for this kernel, and so for the
    // one before it, before it touches what they write
    allow_dependents();
    wait_for_prior_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * width;
    const T* drow = delta ? delta + (size_t)src * width : nullptr;
    const T* drow2 = delta2 ? delta2 + (size_t)src * width : nullptr;
    T* xrow = x + (size_t)r * width;
    T* xrow2 = w2 ? x2 + (size_t)r * width : nullptr;
    float ss = 0.f;
    if ((width & 3) == 0) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(hrow + i);
            if (drow) {
                float4 d;
                load4(drow + i, d);
                if (drow2) {
                    float4 e;
                    load4(drow2 + i, e);
                    d.x += mult2 * e.x; d.y += mult2 * e.y; d.z += mult2 * e.z; d.w += mult2 * e.w;
                }
                v.x += mult * d.x; v.y += mult * d.y; v.z += mult * d.z; v.w += mult * d.w;
            }
            *reinterpret_cast<float4*>(vals + i) = v;
            if (write_h) *reinterpret_cast<float4*>(hrow + i) = v;
            ss += v.x * v.x;
            ss += v.y * v.y;
            ss += v.z * v.z;
            ss += v.w * v.w;
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(vals + i);
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            store4(xrow + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
            if (xrow2) {
                const float4 g2 = *reinterpret_cast<const float4*>(w2 + i);
                store4(xrow2 + i, make_float4(v.x * inv * g2.x, v.y * inv * g2.y, v.z * inv * g2.z, v.w * inv * g2.w));
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = hrow[i];
            if (drow) v += mult * (to_float(drow[i]) + (drow2 ? mult2 * to_float(drow2[i]) : 0.f));
            vals[i] = v;
            if (write_h) hrow[i] = v;
            ss += v * v;
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            xrow[i] = from_float<T>(vals[i] * inv * w[i]);
            if (xrow2) xrow2[i] = from_float<T>(vals[i] * inv * w2[i]);
        }
    }
}

// The same for rows of up to CHUNKS * 4 * blockDim numbers (a multiple of 4): every thread keeps its CHUNKS groups
// of four in registers, all their loads under way at once, and the blocks are small enough for several to share an
// SM.  The reduction order depends on the width and the block size only, as above.
template <typename T, int CHUNKS>
__global__ void add_rmsnorm_rows_kernel(float* __restrict__ h, const T* __restrict__ delta, const T* __restrict__ delta2, float mult, float mult2,
                                        const int* __restrict__ rows, const float* __restrict__ w, float eps,
                                        T* __restrict__ x, int width, int write_h, const float* __restrict__ w2, T* __restrict__ x2) {
    __shared__ float scratch[32];
    // the norm's weight does not come from the kernel before this one: it is fetched before the wait for it
    float4 g[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        g[c] = i < width ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // what follows (a product) may take its place and fetch its weights now: it waits for this kernel, and so for the
    // one before it, before it touches what they write
    allow_dependents();
    wait_for_prior_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * width;
    const T* drow = delta ? delta + (size_t)src * width : nullptr;
    const T* drow2 = (delta && delta2) ? delta2 + (size_t)src * width : nullptr;
    T* xrow = x + (size_t)r * width;
    float4 v[CHUNKS], d[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        v[c] = d[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < width) {
            v[c] = *reinterpret_cast<const float4*>(hrow + i);
            if (drow) load4(drow + i, d[c]);
            if (drow2) {
                float4 e;
                load4(drow2 + i, e);
                d[c].x += mult2 * e.x; d[c].y += mult2 * e.y; d[c].z += mult2 * e.z; d[c].w += mult2 * e.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        // (mult is 1 unless the layer scales what it adds to the stream: the product is then exact)
        v[c].x += mult * d[c].x; v[c].y += mult * d[c].y; v[c].z += mult * d[c].z; v[c].w += mult * d[c].w;
        if (write_h && i < width) *reinterpret_cast<float4*>(hrow + i) = v[c];
        ss += v[c].x * v[c].x;
        ss += v[c].y * v[c].y;
        ss += v[c].z * v[c].z;
        ss += v[c].w * v[c].w;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < width)
            store4(xrow + i, make_float4(v[c].x * inv * g[c].x, v[c].y * inv * g[c].y, v[c].z * inv * g[c].z, v[c].w * inv * g[c].w));
    }
    if (w2) {   // the second norm of the same rows: the same mean, its own weight
        T* xrow2 = x2 + (size_t)r * width;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int i = (c * blockDim.x + threadIdx.x) * 4;
            if (i < width) {
                const float4 g2 = *reinterpret_cast<const float4*>(w2 + i);
                store4(xrow2 + i, make_float4(v[c].x * inv * g2.x, v[c].y * inv * g2.y, v[c].z * inv * g2.z, v[c].w * inv * g2.w));
            }
        }
    }
}

template <typename T>
int launch_add_rmsnorm(float* h, const T* delta, const T* delta2, float mult, float mult2, const int* rows, const float* w, float eps, T* x,
                       int n_rows, int width, int write_h, const float* w2, T* x2, cudaStream_t s) {
    const int groups = width / 4;
    // Which arrangement runs decides the order in which a row's squares are added.  In the 32-bit path that order
    // may depend on the width only (the same bits however a step is cut), so the number of rows chooses between
    // the arrangements for bfloat16 alone.
    const bool by_rows = !std::is_same<T, float>::value;
    if ((width & 3) == 0 && groups <= 1024 && (n_rows <= 256 || !by_rows)) {
        // few rows (decoding): as many threads as the row has groups of four, so that a row's latency is one load
        const int threads = (groups + 31) / 32 * 32;
        RMX_CHECK_LAUNCHED(launch_dependent(add_rmsnorm_rows_kernel<T, 1>, dim3(n_rows), dim3(threads), 0, s, h, delta, delta2, mult, mult2, rows, w, eps,
                                            x, width, write_h, w2, x2), "add_rmsnorm");
        return 0;
    }
    constexpr int CHUNKS = 4;
    if ((width & 3) == 0 && groups <= CHUNKS * 1024) {
        // many rows: as few threads as hold the row in CHUNKS groups each (at least a warp), several blocks an SM
        int threads = ((groups + CHUNKS - 1) / CHUNKS + 31) / 32 * 32;
        threads = threads < 32 ? 32 : threads;
        RMX_CHECK_LAUNCHED(launch_dependent(add_rmsnorm_rows_kernel<T, CHUNKS>, dim3(n_rows), dim3(threads), 0, s, h, delta, delta2, mult, mult2, rows, w, eps,
                                            x, width, write_h, w2, x2), "add_rmsnorm");
        return 0;
    }
    const int threads = block_threads(width);
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    RMX_CHECK_LAUNCHED(launch_dependent(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, s, h, delta, delta2, mult, mult2, rows, w, eps, x, width,
                                        write_h, w2, x2), "add_rmsnorm");
    return 0;
}

// delta2 (or null), mult and mult2: what is added to the stream is mult * (delta + mult2 * delta2), formed in float (a layer whose
// mixer and feed-forward read the same norm adds both at once, scaled by the model's factor).
// w2 and x2 (or null): a second norm of the same rows with its own weight, written to x2.
RMX_API int rmx_add_rmsnorm(float* h, const void* delta, const void* delta2, float mult, float mult2, const int* rows, const float* w, float eps,
                            void* x, int n_rows, int width, int write_h, const float* w2, void* x2, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(delta != nullptr || delta2 == nullptr, "add_rmsnorm: a second delta without a first");
    RMX_REQUIRE(n_rows > 0 && width > 0, "add_rmsnorm: bad sizes");
    RMX_REQUIRE((size_t)width * 4 <= 160 * 1024, "add_rmsnorm: width %d is beyond 40960", width);
    RMX_REQUIRE(!(rows && write_h), "add_rmsnorm: rows and write_h do not go together");
    RMX_REQUIRE((w2 == nullptr) == (x2 == nullptr), "add_rmsnorm: a second weight goes with a second output");
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (dtype == RMX_F32) rc = launch_add_rmsnorm<float>(h, (const float*)delta, (const float*)delta2, mult, mult2, rows, w, eps, (float*)x, n_rows, width, write_h, w2, (float*)x2, s);
    else if (dtype == RMX_BF16)
        rc = launch_add_rmsnorm<__nv_bfloat16>(h, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)delta2, mult, mult2, rows, w, eps,
                                               (__nv_bfloat16*)x, n_rows, width, write_h, w2, (__nv_bfloat16*)x2, s);
    else RMX_FAIL("add_rmsnorm: unknown dtype %d", dtype);
    if (rc != 0) return rc;
    RMX_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// out[t, j] = act(gate_up[t, gate j], gate_up[t, up j]) (see activation.cuh), in float with one rounding.
// Where gate j and up j lie in a row of 2 * inter numbers: concatenated [gate | up] (block == 0), or in blocks of
// `block` gate numbers followed by their `block` up numbers.
__device__ __forceinline__ void gate_up_at(int j, int inter, int block, int& gi, int& ui) {
    if (block == 0) {
        gi = j;
        ui = inter + j;
    } else {
        gi = (j / block) * 2 * block + j % block;
        ui = gi + block;
    }
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block, size_t total, int act, float limit, float alpha) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    int gi, ui;
    gate_up_at(j, inter, block, gi, ui);
    const float g = to_float(gate_up[t * 2 * inter + gi]);
    const float u = to_float(gate_up[t * 2 * inter + ui]);
    out[idx] = from_float<T>(gated_act(g, u, act, limit, alpha));
}

// four outputs per thread; inter is a multiple of 4
template <typename T>
__global__ void swiglu_kernel4(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block, size_t total4, int act, float limit, float alpha) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int per_row = inter >> 2;
    const size_t t = idx / per_row;
    const int j = (int)(idx - t * per_row) * 4;
    int gi, ui;
    gate_up_at(j, inter, block, gi, ui);   // four neighbours stay together: block is a multiple of 4
    float4 g, u;
    load4(gate_up + t * 2 * inter + gi, g);
    load4(gate_up + t * 2 * inter + ui, u);
    store4(out + t * inter + j, make_float4(gated_act(g.x, u.x, act, limit, alpha), gated_act(g.y, u.y, act, limit, alpha), gated_act(g.z, u.z, act, limit, alpha), gated_act(g.w, u.w, act, limit, alpha)));
}

// bfloat16, sixteen outputs per thread as two groups of eight (16-byte loads and stores); inter and block are
// multiples of 8.  blockIdx.x is the token, blockIdx.y the part of its row.  The exponential and the division are
// the fast ones (about two units in the last place of a float): the result is rounded to bfloat16, eight bits.

__global__ void swiglu_kernel8(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter,
                               int block, int act, float limit, float alpha) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int per_row = inter >> 3;
    const __nv_bfloat16* src = gate_up + (size_t)blockIdx.x * 2 * inter;
    __nv_bfloat16* dst = out + (size_t)blockIdx.x * inter;
    uint4 g[2], u[2];
    int j[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int item = (blockIdx.y * 2 + c) * blockDim.x + threadIdx.x;
        j[c] = item < per_row ? item * 8 : -1;
        if (j[c] >= 0) {
            int gi, ui;
            gate_up_at(j[c], inter, block, gi, ui);
            g[c] = *reinterpret_cast<const uint4*>(src + gi);
            u[c] = *reinterpret_cast<const uint4*>(src + ui);
        }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        if (j[c] < 0) continue;
        const uint32_t gw[4] = {g[c].x, g[c].y, g[c].z, g[c].w}, uw[4] = {u[c].x, u[c].y, u[c].z, u[c].w};
        uint32_t ow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
            __nv_bfloat162 r = __floats2bfloat162_rn(gated_act_fast(a.x, b.x, act, limit, alpha), gated_act_fast(a.y, b.y, act, limit, alpha));
            ow[i] = *reinterpret_cast<uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(dst + j[c]) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// act: which function forms an output from its gate and up numbers (activation.cuh): 0 silu, 1 the tanh form of GELU,
// 2 the clamped swish, which reads `limit` and `alpha`.
RMX_API int rmx_swiglu(const void* gate_up, void* out, int n_tokens, int inter, int block, int act, float limit, float alpha, int dtype,
                       void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && inter > 0, "swiglu: bad sizes");
    RMX_REQUIRE(act >= 0 && act <= 2, "swiglu: unknown activation %d", act);
    RMX_REQUIRE(block == 0 || (block > 0 && inter % block == 0), "swiglu: blocks of %d do not divide %d", block, inter);
    const bool vec = (inter & 3) == 0 && (block & 3) == 0;
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_BF16 && (inter & 7) == 0 && (block & 7) == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const int per_row = inter / 8;
        const int t8 = per_row >= 512 ? 256 : 128;
        RMX_CHECK_LAUNCHED(launch_dependent(swiglu_kernel8, dim3(n_tokens, (per_row + 2 * t8 - 1) / (2 * t8)), dim3(t8), 0, s,
                                            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, act, limit, alpha), "swiglu");
        return 0;
    }
    const size_t total = (size_t)n_tokens * inter / (vec ? 4 : 1);
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RMX_F32) {
        if (vec) RMX_CHECK_LAUNCHED(launch_dependent(swiglu_kernel4<float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, inter, block, total, act, limit, alpha), "swiglu");
        else swiglu_kernel<float><<<blocks, threads, 0, s>>>((const float*)gate_up, (float*)out, inter, block, total, act, limit, alpha);
    } else if (dtype == RMX_BF16) {
        if (vec) RMX_CHECK_LAUNCHED(launch_dependent(swiglu_kernel4<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total, act, limit, alpha), "swiglu");
        else swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total, act, limit, alpha);
    } else {
        RMX_FAIL("swiglu: unknown dtype %d", dtype);
    }
    RMX_CHECK_LAUNCH("swiglu");
    return 0;
}

// h[t, :] += delta[t, :] (float add, delta in T): closes the residual stream when no norm follows.
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ h, const T* __restrict__ delta, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) h[idx] += to_float(delta[idx]);
}

RMX_API int rmx_add_residual(float* h, const void* delta, int n_rows, int width, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    const size_t total = (size_t)n_rows * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        add_residual_kernel<float><<<blocks, threads, 0, s>>>(h, (const float*)delta, total);
    else if (dtype == RMX_BF16)
        add_residual_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>(h, (const __nv_bfloat16*)delta, total);
    else
        RMX_FAIL("add_residual: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("add_residual");
    return 0;
}

// x[t, j] = x[t, j] + bias[j] (float add, one rounding): the bias of a projection, added to the product as the
// reference does (src/weights.rs:198-200).  `ld` is the distance between rows of x.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int width, int ld, size_t total) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / width;
    const int col = (int)(idx - row * width);
    T* at = x + row * ld + col;
    *at = from_float<T>(to_float(*at) + bias[col]);
}

RMX_API int rmx_add_bias(void* x, const float* bias, int n_rows, int width, int ld, int dtype, void* stream) {
    if (n_rows == 0 || width == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && width > 0 && ld >= width && x && bias, "add_bias: bad sizes or a null pointer");
    const size_t total = (size_t)n_rows * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(add_bias_kernel<float>, dim3(blocks), dim3(threads), 0, s, (float*)x, bias, width, ld, total), "add_bias");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(add_bias_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (__nv_bfloat16*)x, bias, width, ld, total), "add_bias");
    else
        RMX_FAIL("add_bias: unknown dtype %d", dtype);
    return 0;
}

// out[t] = [ round(h[t] + mult * (delta[t] + mult2 * delta2[t])) | extra[t] ]: the stream, with what the layer before left to be
// added to it, beside `extra` rows of the same width (in T), as ONE row of 2 * width numbers in T for a product
// that reads both (a model that mixes the embedding's output back into the stream before a group of layers).  The sum
// is formed in float and, with write_h, stored back into the stream.
template <typename T>
__global__ void stream_concat_kernel(float* __restrict__ h, const T* __restrict__ delta, const T* __restrict__ delta2, float mult,
                                     float mult2, const T* __restrict__ extra, T* __restrict__ out, int width, int write_h) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t t = blockIdx.x;
    float* hrow = h + t * width;
    const T* drow = delta ? delta + t * width : nullptr;
    const T* drow2 = (delta && delta2) ? delta2 + t * width : nullptr;
    const T* erow = extra + t * width;
    T* orow = out + t * 2 * width;
    if ((width & 3) == 0) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(hrow + i);
            if (drow) {
                float4 d;
                load4(drow + i, d);
                if (drow2) {
                    float4 e;
                    load4(drow2 + i, e);
                    d.x += mult2 * e.x; d.y += mult2 * e.y; d.z += mult2 * e.z; d.w += mult2 * e.w;
                }
                v.x += mult * d.x; v.y += mult * d.y; v.z += mult * d.z; v.w += mult * d.w;
                if (write_h) *reinterpret_cast<float4*>(hrow + i) = v;
            }
            store4(orow + i, v);
            float4 x;
            load4(erow + i, x);
            store4(orow + width + i, x);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = hrow[i];
            if (drow) {
                v += mult * (to_float(drow[i]) + (drow2 ? mult2 * to_float(drow2[i]) : 0.f));
                if (write_h) hrow[i] = v;
            }
            orow[i] = from_float<T>(v);
            orow[width + i] = erow[i];
        }
    }
}

RMX_API int rmx_stream_concat(float* h, const void* delta, const void* delta2, float mult, float mult2, const void* extra, void* out,
                              int n_rows, int width, int write_h, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && width > 0 && h && extra && out, "stream_concat: bad sizes or a null pointer");
    RMX_REQUIRE(delta != nullptr || delta2 == nullptr, "stream_concat: a second delta without a first");
    const int threads = block_threads(width);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(stream_concat_kernel<float>, dim3(n_rows), dim3(threads), 0, s, h, (const float*)delta,
                                            (const float*)delta2, mult, mult2, (const float*)extra, (float*)out, width, write_h), "stream_concat");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(stream_concat_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, h, (const __nv_bfloat16*)delta,
                                            (const __nv_bfloat16*)delta2, mult, mult2, (const __nv_bfloat16*)extra, (__nv_bfloat16*)out, width,
                                            write_h), "stream_concat");
    else
        RMX_FAIL("stream_concat: unknown dtype %d", dtype);
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// The stream's add and norm for layers that scale what they add number by number and norm the row in parts:
//   v = h + va * (m1 * d1 + m2 * d2) + vb * d3        (float; any of d1, d2, d3, va, vb may be null: a null vector is ones)
//   if (write_h) h = v
//   the row is `groups` equal consecutive parts; part g is divided by sqrt(mean(part^2) + eps)
//   x = that * w  (and x2 = that * w2 when a second weight is given), rounded once
// One block a row (src = rows ? rows[r] : r), the row held in shared memory.  A part's squares are added by the warps
// that the part falls to (warp i of the part takes numbers i*32 + lane, stepping by 32 * warps-a-part), each warp by the
// butterfly, the warps in their order: the order follows the width, the number of parts and the block size, which the
// width decides.
template <typename T>
__global__ void add_group_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ d1, const T* __restrict__ d2, const T* __restrict__ d3,
                                         float m1, float m2, const float* __restrict__ va, const float* __restrict__ vb,
                                         const int* __restrict__ rows, const float* __restrict__ w, float eps, T* __restrict__ x, int width,
                                         int groups, int write_h, const float* __restrict__ w2, T* __restrict__ x2) {
    extern __shared__ __align__(16) float gvals[];     // [width] the row, then [groups * warps_a_part] partial sums, then [groups]
    allow_dependents();
    wait_for_prior_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const size_t at = (size_t)src * width;
    float* hrow = h + at;
    const int size = width / groups;
    // four numbers a thread and pass where the row and its parts allow it (16-byte accesses; a part's sum is then formed
    // over groups of four neighbours: the order still follows the sizes alone)
    const bool vec = (width & 3) == 0 && (size & 3) == 0;
    if (vec) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(hrow + i);
            if (d1) {
                float4 a;
                load4(d1 + at + i, a);
                a.x *= m1; a.y *= m1; a.z *= m1; a.w *= m1;
                if (d2) {
                    float4 e;
                    load4(d2 + at + i, e);
                    a.x = fmaf(m2, e.x, a.x); a.y = fmaf(m2, e.y, a.y); a.z = fmaf(m2, e.z, a.z); a.w = fmaf(m2, e.w, a.w);
                }
                if (va) {
                    const float4 s = *reinterpret_cast<const float4*>(va + i);
                    a.x *= s.x; a.y *= s.y; a.z *= s.z; a.w *= s.w;
                }
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (d3) {
                float4 b;
                load4(d3 + at + i, b);
                if (vb) {
                    const float4 s = *reinterpret_cast<const float4*>(vb + i);
                    b.x *= s.x; b.y *= s.y; b.z *= s.z; b.w *= s.w;
                }
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            *reinterpret_cast<float4*>(gvals + i) = v;
            if (write_h) *reinterpret_cast<float4*>(hrow + i) = v;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = hrow[i];
            if (d1) {
                float a = m1 * to_float(d1[at + i]);
                if (d2) a = fmaf(m2, to_float(d2[at + i]), a);
                v += va ? va[i] * a : a;
            }
            if (d3) {
                const float b = to_float(d3[at + i]);
                v += vb ? vb[i] * b : b;
            }
            gvals[i] = v;
            if (write_h) hrow[i] = v;
        }
    }
    __syncthreads();
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpp = warps >= groups ? warps / groups : 1;     // warps a part
    float* part = gvals + width;
    float* inv = part + groups * wpp;
    for (int item = warp; item < groups * wpp; item += warps) {
        const int g = item / wpp, sub = item - g * wpp;
        const float* p = gvals + g * size;
        float ss = 0.f;
        if (vec) {
            for (int i = (sub * 32 + lane) * 4; i < size; i += 128 * wpp) {
                const float4 v = *reinterpret_cast<const float4*>(p + i);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
        } else {
            for (int i = sub * 32 + lane; i < size; i += 32 * wpp) ss = fmaf(p[i], p[i], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) part[item] = ss;
    }
    __syncthreads();
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float total = 0.f;
        for (int sub = 0; sub < wpp; ++sub) total += part[g * wpp + sub];
        inv[g] = rsqrtf(total / (float)size + eps);
    }
    __syncthreads();
    T* xrow = x + (size_t)r * width;
    T* xrow2 = w2 ? x2 + (size_t)r * width : nullptr;
    if (vec) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(gvals + i);
            const float n = inv[i / size];
            v.x *= n; v.y *= n; v.z *= n; v.w *= n;
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            store4(xrow + i, make_float4(v.x * g.x, v.y * g.y, v.z * g.z, v.w * g.w));
            if (xrow2) {
                const float4 g2 = *reinterpret_cast<const float4*>(w2 + i);
                store4(xrow2 + i, make_float4(v.x * g2.x, v.y * g2.y, v.z * g2.z, v.w * g2.w));
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float n = gvals[i] * inv[i / size];
        xrow[i] = from_float<T>(n * w[i]);
        if (xrow2) xrow2[i] = from_float<T>(n * w2[i]);
    }
}

RMX_API int rmx_add_group_rmsnorm(float* h, const void* d1, const void* d2, const void* d3, float m1, float m2, const float* va,
                                  const float* vb, const int* rows, const float* w, float eps, void* x, int n_rows, int width, int groups,
                                  int write_h, const float* w2, void* x2, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && width > 0 && groups > 0 && width % groups == 0, "add_group_rmsnorm: %d numbers in %d parts", width, groups);
    RMX_REQUIRE(d1 != nullptr || d2 == nullptr, "add_group_rmsnorm: a second term without a first");
    RMX_REQUIRE(!(rows && write_h), "add_group_rmsnorm: rows and write_h do not go together");
    RMX_REQUIRE((w2 == nullptr) == (x2 == nullptr), "add_group_rmsnorm: a second weight goes with a second output");
    const int threads = block_threads(width);
    const int warps = threads / 32, wpp = warps >= groups ? warps / groups : 1;
    const size_t smem = ((size_t)width + (size_t)groups * wpp + groups) * sizeof(float);
    RMX_REQUIRE(smem <= 200 * 1024, "add_group_rmsnorm: a row of %d numbers in %d parts needs too much shared memory", width, groups);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32) {
        static bool raised[64] = {};
        if (smem > 48 * 1024 && rmx_first_on_device(raised))
            cudaFuncSetAttribute(add_group_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        RMX_CHECK_LAUNCHED(launch_dependent(add_group_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), smem, s, h, (const float*)d1,
                                            (const float*)d2, (const float*)d3, m1, m2, va, vb, rows, w, eps, (float*)x, width, groups,
                                            write_h, w2, (float*)x2), "add_group_rmsnorm");
    } else if (dtype == RMX_BF16) {
        static bool raised[64] = {};
        if (smem > 48 * 1024 && rmx_first_on_device(raised))
            cudaFuncSetAttribute(add_group_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        RMX_CHECK_LAUNCHED(launch_dependent(add_group_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, s, h,
                                            (const __nv_bfloat16*)d1, (const __nv_bfloat16*)d2, (const __nv_bfloat16*)d3, m1, m2, va, vb, rows,
                                            w, eps, (__nv_bfloat16*)x, width, groups, write_h, w2, (__nv_bfloat16*)x2), "add_group_rmsnorm");
    } else {
        RMX_FAIL("add_group_rmsnorm: unknown dtype %d", dtype);
    }
    return 0;
}

// out = f(x) number by number, in float with one rounding (activation.cuh: squared relu, tanh); out may be x.
template <typename T>
__global__ void unary_act_kernel(const T* x, T* out, size_t total, int act) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    out[idx] = from_float<T>(unary_act(to_float(x[idx]), act));
}

RMX_API int rmx_unary_act(const void* x, void* out, long long total, int act, int dtype, void* stream) {
    if (total == 0) return 0;
    RMX_REQUIRE(total > 0 && (act == RMX_ACT_RELU2 || act == RMX_ACT_TANH), "unary_act: bad size or unknown activation %d", act);
    const dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(unary_act_kernel<float>, grid, dim3(256), 0, s, (const float*)x, (float*)out, (size_t)total, act), "unary_act");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(unary_act_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                            (size_t)total, act), "unary_act");
    else
        RMX_FAIL("unary_act: unknown dtype %d", dtype);
    return 0;
}
