// A routed feed-forward (mixture of experts): router, grouping of rows by expert, the experts' products over
// their groups, and the weighted sum.
//
//   z = W_router x (float)            the `top` largest z choose a row's experts; their weights are
//                                     softmax over the chosen z alone
//   (row, choice) pairs are sorted by expert, so that every expert's rows are neighbours: `offsets[e]` is where
//   expert e's run starts, `sorted[p]` is the pair (row * top + choice) at place p, `where[pair]` the place of a pair
//   the experts' products run over those runs, each tile of rows with its expert's weights
//   out[row] = sum over choices of weight * y[where[row * top + choice]]  (+ what a shared expert gave)
//
// Nothing here waits for the host: counts and offsets stay on the device, grids are sized for the worst case and
// blocks without work leave at once, so a step can be captured in a graph.  A row's result does not depend on
// which other rows are in the batch: its router sum, its products (ascending k in one thread) and its weighted
// sum (ascending choice) have fixed orders.
#include "common.cuh"

namespace {

// ---- router ---------------------------------------------------------------------------------------------------
// Logits in float from the rows (in T) and the router's weight (float).  A warp takes one expert and up to ROWS rows,
// so that a weight row is read once for all of them; a (row, expert) sum is formed lane by lane over groups of four
// neighbouring numbers and then across the lanes, in an order that the width alone decides.
__device__ __forceinline__ void route_load4(const float* p, float4& v) { v = *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void route_load4(const __nv_bfloat16* p, float4& v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v = make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, int ROWS, int EXP>
__global__ void __launch_bounds__(128) moe_logits_kernel(const T* __restrict__ x, const float* __restrict__ w, int width, int n_experts,
                                                         int n_rows, float* __restrict__ logits) {
    // a block of four warps takes EXP experts and up to ROWS rows, so that a row is fetched once for EXP experts and a
    // weight row once for ROWS rows; its 128 threads walk the width together (groups of four neighbouring numbers), each
    // warp's lanes are added by the butterfly and the warps in their order: the order of a (row, expert) sum follows the
    // width alone
    __shared__ float part[4][ROWS][EXP];
    allow_dependents();
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = blockIdx.y * EXP;
    const int row0 = blockIdx.x * ROWS;
    float acc[ROWS][EXP];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int j = 0; j < EXP; ++j) acc[r][j] = 0.f;
    if ((width & 3) == 0) {
#pragma unroll 2
        for (int i = threadIdx.x * 4; i < width; i += 512) {
            float4 wv[EXP];
#pragma unroll
            for (int j = 0; j < EXP; ++j) {
                wv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e0 + j < n_experts) route_load4(w + (size_t)(e0 + j) * width + i, wv[j]);
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (row0 + r < n_rows) {
                    float4 xv;
                    route_load4(x + (size_t)(row0 + r) * width + i, xv);
#pragma unroll
                    for (int j = 0; j < EXP; ++j) {
                        acc[r][j] = fmaf(xv.x, wv[j].x, acc[r][j]);
                        acc[r][j] = fmaf(xv.y, wv[j].y, acc[r][j]);
                        acc[r][j] = fmaf(xv.z, wv[j].z, acc[r][j]);
                        acc[r][j] = fmaf(xv.w, wv[j].w, acc[r][j]);
                    }
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += 128) {
            float wv[EXP];
#pragma unroll
            for (int j = 0; j < EXP; ++j) wv[j] = e0 + j < n_experts ? w[(size_t)(e0 + j) * width + i] : 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (row0 + r < n_rows) {
                    const float xv = to_float(x[(size_t)(row0 + r) * width + i]);
#pragma unroll
                    for (int j = 0; j < EXP; ++j) acc[r][j] = fmaf(xv, wv[j], acc[r][j]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int j = 0; j < EXP; ++j) {
            const float s = warp_sum(acc[r][j]);
            if (lane == 0) part[warp][r][j] = s;
        }
    __syncthreads();
    if (threadIdx.x < ROWS * EXP) {
        const int r = threadIdx.x / EXP, j = threadIdx.x % EXP;
        if (row0 + r < n_rows && e0 + j < n_experts)
            logits[(size_t)(row0 + r) * n_experts + e0 + j] = ((part[0][r][j] + part[1][r][j]) + part[2][r][j]) + part[3][r][j];
    }
}

// One warp per row: the `top` largest logits choose the experts (ties go to the lower expert); their weights are the
// softmax over the chosen logits alone.  ids [rows, top], weights [rows, top].
__global__ void moe_topk_kernel(const float* __restrict__ logits_in, int n_experts, int top, int* __restrict__ ids,
                                float* __restrict__ weights, int n_rows) {
    extern __shared__ float logits_all[];
    allow_dependents();
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= n_rows) return;
    float* logits = logits_all + warp * n_experts;
    for (int e = lane; e < n_experts; e += 32) logits[e] = logits_in[(size_t)row * n_experts + e];
    __syncwarp();
    float first = 0.f, total = 0.f, mine = 0.f;   // lane k keeps the k-th chosen logit (top <= 32)
    int mine_id = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = n_experts;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = logits[e];
            if (v > best) { best = v; best_e = e; }      // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e >= n_experts) best_e = 0;             // (all values NaN: still a valid expert)
        if (k == 0) first = best;
        if (lane == k) { mine = best; mine_id = best_e; }
        if (lane == 0) logits[best_e] = -INFINITY;
        __syncwarp();
    }
    const float p = lane < top ? expf(mine - first) : 0.f;
    total = warp_sum(p);
    if (lane < top) {
        ids[(size_t)row * top + lane] = mine_id;
        weights[(size_t)row * top + lane] = p / total;
    }
}

// The other way of choosing, one warp per row:
//   s_e = sigmoid(z_e)                              what an expert's weight is made of
//   c_e = s_e + correction_e                        what the choice goes by (correction may be null)
//   the experts form `groups` equal groups of neighbours; a group's score is the sum of its two largest c (its one c if it
//   has one expert); only experts of the `keep` groups with the largest scores can be chosen (the others' c counts as
//   minus infinity: c itself may be negative)
//   the `top` largest c among those choose the experts (ties go to the lower expert, or group)
//   weight_e = s_e / (sum of the chosen s + 1e-20) * scale, or with normalize == 0 the score as it is: s_e * scale
// Everything in float.  Shared memory: per warp n_experts floats of c, n_experts of s, `groups` of group scores.
__global__ void moe_group_topk_kernel(const float* __restrict__ logits_in, const float* __restrict__ correction, int n_experts, int top,
                                      int groups, int keep, float scale, int normalize, int* __restrict__ ids, float* __restrict__ weights,
                                      int n_rows) {
    extern __shared__ float route_all[];
    allow_dependents();
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= n_rows) return;
    float* choice = route_all + (size_t)warp * (2 * n_experts + groups);
    float* score = choice + n_experts;
    float* group_score = score + n_experts;
    for (int e = lane; e < n_experts; e += 32) {
        const float z = logits_in[(size_t)row * n_experts + e];
        const float sg = 1.f / (1.f + expf(-z));
        score[e] = sg;
        choice[e] = sg + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = n_experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;      // the largest and the second largest of the group
            for (int i = 0; i < per; ++i) {
                const float v = choice[g * per + i];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            group_score[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups, one after the other; a group that is kept gets +inf as its mark
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int best_g = groups;
            for (int g = lane; g < groups; g += 32) {
                const float v = group_score[g];
                if (v != INFINITY && (v > best || best_g == groups)) { best = v; best_g = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (og < groups && (best_g == groups || ob > best || (ob == best && og < best_g))) { best = ob; best_g = og; }
            }
            if (lane == 0 && best_g < groups) group_score[best_g] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < n_experts; e += 32)
            if (group_score[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    float mine = 0.f;      // lane k keeps the score s of the k-th chosen expert (top <= 32)
    int mine_id = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = n_experts;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = choice[e];
            if (v > best) { best = v; best_e = e; }      // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e >= n_experts) best_e = 0;             // (nothing left to choose from, or all values NaN: still a valid expert)
        if (lane == k) { mine = score[best_e]; mine_id = best_e; }
        __syncwarp();
        if (lane == 0) choice[best_e] = -INFINITY;
        __syncwarp();
    }
    // the chosen scores are added in the order in which they were chosen, by every lane alike
    float total = 0.f;
    for (int k = 0; k < top; ++k) total += __shfl_sync(0xffffffffu, mine, k);
    if (lane < top) {
        ids[(size_t)row * top + lane] = mine_id;
        weights[(size_t)row * top + lane] = normalize ? mine / (total + 1e-20f) * scale : mine * scale;
    }
}

// ---- grouping -------------------------------------------------------------------------------------------------
// One block.  Counting sort of the pairs by expert.
__global__ void moe_sort_kernel(const int* __restrict__ ids, int total, int n_experts, int* __restrict__ offsets,
                                int* __restrict__ sorted, int* __restrict__ where) {
    extern __shared__ int counts[];          // [n_experts] counts, then [n_experts] cursors
    int* cursor = counts + n_experts;
    allow_dependents();
    wait_for_prior_kernels();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            at += counts[e];
        }
        offsets[n_experts] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int p = atomicAdd(&cursor[ids[i]], 1);
        sorted[p] = i;
        where[i] = p;
    }
}

// ---- the experts' products ------------------------------------------------------------------------------------
// C[p, :] = A[row(p), :] . W[e]^T for every place p of expert e's run; row(p) = sorted[p] / divisor when the rows
// are gathered from the layer's input (divisor = top), p itself when A is already in sorted order (divisor 0).
// blockIdx.y counts row tiles across all experts; a block finds its expert by walking the offsets.
// Every output is accumulated by one thread over k in ascending order.
constexpr int BN = 64, BK = 16;

template <typename TA, typename TC, int BM>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ sorted,
                                                       int divisor, const TA* __restrict__ W, TC* __restrict__ C, int ldc,
                                                       const int* __restrict__ offsets, int n_experts, int N, int K) {
    constexpr int RM = BM / 16;            // rows per thread
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int rows[BM];
    allow_dependents();
    wait_for_prior_kernels();
    int tile = blockIdx.y, e = 0, begin = 0, end = 0;
    for (; e < n_experts; ++e) {
        begin = offsets[e];
        end = offsets[e + 1];
        const int tiles = (end - begin + BM - 1) / BM;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (e >= n_experts) return;
    const int m0 = begin + tile * BM;
    const int n0 = blockIdx.x * BN;
    const TA* We = W + (size_t)e * N * K;
    for (int i = threadIdx.x; i < BM; i += 256) {
        const int p = m0 + i;
        rows[i] = p < end ? (divisor > 0 ? sorted[p] / divisor : p) : -1;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[RM][4];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
            const int r = idx / BK, k = k0 + idx % BK;
            const int src = rows[r];
            As[idx % BK][r] = (src >= 0 && k < K) ? to_float(A[(size_t)src * lda + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
            const int r = idx / BK, k = k0 + idx % BK;
            Ws[idx % BK][r] = (n0 + r < N && k < K) ? to_float(We[(size_t)(n0 + r) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[RM], b[4];
#pragma unroll
            for (int i = 0; i < RM; ++i) a[i] = As[kk][ty * RM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < RM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int p = m0 + ty * RM + i;
        if (p >= end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)p * ldc + n] = from_float<TC>(acc[i][j]);
        }
    }
}

// ---- rows into the experts' order, each times its weight ---------------------------------------------------------
// out[p, :] = weights[pair] * x[pair / top, :] with pair = sorted[p]: for experts that are given the weighted row
// instead of having their result weighted.  Float product, one rounding.
template <typename T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ x, const int* __restrict__ sorted, const float* __restrict__ weights, int top,
                                         T* __restrict__ out, int width, size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t p = idx / width;
    const int c = (int)(idx - p * width);
    const int pair = sorted[p];
    out[idx] = from_float<T>(weights[pair] * to_float(x[(size_t)(pair / top) * width + c]));
}

// bfloat16, eight numbers a thread (16-byte accesses; rows of a multiple of eight numbers): the same products.
__global__ void moe_gather_scaled8_kernel(const uint4* __restrict__ x, const int* __restrict__ sorted, const float* __restrict__ weights,
                                          int top, uint4* __restrict__ out, int chunks, size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t p = idx / chunks;
    const int c = (int)(idx - p * chunks);
    const int pair = sorted[p];
    const float w = weights[pair];
    const uint4 raw = x[(size_t)(pair / top) * chunks + c];
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
        __nv_bfloat162 r = __floats2bfloat162_rn(w * v.x, w * v.y);
        packed[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    out[idx] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// ---- the weighted sum -----------------------------------------------------------------------------------------
// (weights may be null: every choice counts once)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ where, const float* __restrict__ weights,
                                   const T* __restrict__ shared_out, T* __restrict__ out, int top, int width, size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / width;
    const int col = (int)(idx - row * width);
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
        acc = fmaf(weights ? weights[row * top + k] : 1.f, to_float(y[(size_t)where[row * top + k] * width + col]), acc);
    if (shared_out) acc += to_float(shared_out[idx]);
    out[idx] = from_float<T>(acc);
}

// bfloat16, eight columns a thread (16-byte accesses); width is a multiple of 8.  The same sums in the same order.
__global__ void moe_combine8_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ where, const float* __restrict__ weights,
                                    const __nv_bfloat16* __restrict__ shared_out, __nv_bfloat16* __restrict__ out, int top, int width,
                                    size_t total8) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const int per_row = width >> 3;
    const size_t row = idx / per_row;
    const int col = (int)(idx - row * per_row) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < top; ++k) {
        const float wk = weights ? weights[row * top + k] : 1.f;
        const uint4 raw = *reinterpret_cast<const uint4*>(y + (size_t)where[row * top + k] * width + col);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
            acc[2 * j] = fmaf(wk, v.x, acc[2 * j]);
            acc[2 * j + 1] = fmaf(wk, v.y, acc[2 * j + 1]);
        }
    }
    if (shared_out) {
        const uint4 raw = *reinterpret_cast<const uint4*>(shared_out + row * width + col);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
            acc[2 * j] += v.x;
            acc[2 * j + 1] += v.y;
        }
    }
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 r = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        packed[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + row * width + col) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}
}  // namespace

// logits: [n_rows, n_experts] floats of scratch.
// scoring 0: the `top` largest logits, weights = softmax over them.  scoring 1: sigmoid scores, chosen by score + correction among
// the experts of the `keep` best of `groups` groups, weights = the chosen scores over their sum, times route_scale (see
// moe_group_topk_kernel); correction may be null, groups 1 means no groups.
RMX_API int rmx_moe_route(const void* x, const float* w_router, int n_rows, int width, int n_experts, int top, int* ids,
                          float* weights, float* logits, int scoring, const float* correction, int groups, int keep,
                          float route_scale, int normalize, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts && top <= 32,
                "moe_route: %d of %d experts (at most 32 a row)", top, n_experts);
    RMX_REQUIRE(n_experts <= 2048, "moe_route: more than 2048 experts");
    RMX_REQUIRE(logits != nullptr, "moe_route: no room for the logits");
    RMX_REQUIRE(scoring == 0 || (scoring == 1 && groups >= 1 && n_experts % groups == 0 && keep >= 1 && keep <= groups &&
                                 (long long)keep * (n_experts / groups) >= top),
                "moe_route: %d groups of which %d are kept do not fit %d experts of which %d are chosen", groups, keep, n_experts, top);
    cudaStream_t s = (cudaStream_t)stream;
    constexpr int ROWS = 8;
    constexpr int EXP = 1;    // (four experts a block were measured and slower: 120 us against 98 for 2,048 rows, 24 against 14 for 8)
    const int warps = 4;
    dim3 grid((n_rows + ROWS - 1) / ROWS, (n_experts + EXP - 1) / EXP);
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_logits_kernel<float, ROWS, EXP>, grid, dim3(warps * 32), 0, s, (const float*)x, w_router, width,
                                            n_experts, n_rows, logits), "moe_route");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_logits_kernel<__nv_bfloat16, ROWS, EXP>, grid, dim3(warps * 32), 0, s, (const __nv_bfloat16*)x,
                                            w_router, width, n_experts, n_rows, logits), "moe_route");
    else
        RMX_FAIL("moe_route: unknown dtype %d", dtype);
    const int tw = 4;
    if (scoring == 1)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_group_topk_kernel, dim3((n_rows + tw - 1) / tw), dim3(tw * 32),
                                            (size_t)tw * (2 * n_experts + groups) * sizeof(float), s, (const float*)logits, correction, n_experts,
                                            top, groups, keep, route_scale, normalize, ids, weights, n_rows), "moe_route");
    else
        RMX_CHECK_LAUNCHED(launch_dependent(moe_topk_kernel, dim3((n_rows + tw - 1) / tw), dim3(tw * 32), (size_t)tw * n_experts * sizeof(float), s,
                                            (const float*)logits, n_experts, top, ids, weights, n_rows), "moe_route");
    return 0;
}

RMX_API int rmx_moe_sort(const int* ids, int total, int n_experts, int* offsets, int* sorted, int* where, void* stream) {
    if (total == 0) return 0;
    RMX_REQUIRE(total > 0 && n_experts > 0 && n_experts <= 2048 && ids && offsets && sorted && where, "moe_sort: bad arguments");
    RMX_CHECK_LAUNCHED(launch_dependent(moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * n_experts * sizeof(int), (cudaStream_t)stream,
                                        ids, total, n_experts, offsets, sorted, where), "moe_sort");
    return 0;
}

// total: places in all (rows * top).  W: [n_experts, N, K].  C: [total, N], rows ldc apart.
RMX_API int rmx_moe_gemm(const void* A, int lda, const int* sorted, int divisor, const void* W, void* C, int ldc,
                         const int* offsets, int n_experts, int total, int N, int K, int dtype, void* stream) {
    if (total == 0 || N == 0) return 0;
    RMX_REQUIRE(total > 0 && N > 0 && K > 0 && n_experts > 0 && lda >= K && ldc >= N, "moe_gemm: bad sizes");
    RMX_REQUIRE(divisor == 0 || sorted != nullptr, "moe_gemm: gathered rows need the sorted pairs");
    cudaStream_t s = (cudaStream_t)stream;
    // few rows an expert (decoding): tiles of 16 rows, so that a tile's work follows the weights it reads
    const bool small = total <= 16 * n_experts;
    const int bm = small ? 16 : 64;
    const int tiles = (total + bm - 1) / bm + n_experts;
    RMX_REQUIRE(tiles <= 65535, "moe_gemm: too many row tiles (%d)", tiles);
    dim3 grid((N + BN - 1) / BN, tiles);
#define RMX_MOE_GEMM(TA, BM_)                                                                                              \
    RMX_CHECK_LAUNCHED(launch_dependent(moe_gemm_kernel<TA, TA, BM_>, grid, dim3(256), 0, s, (const TA*)A, lda, sorted, divisor, \
                                        (const TA*)W, (TA*)C, ldc, offsets, n_experts, N, K), "moe_gemm")
    if (dtype == RMX_F32) {
        if (small) RMX_MOE_GEMM(float, 16); else RMX_MOE_GEMM(float, 64);
    } else if (dtype == RMX_BF16) {
        if (small) RMX_MOE_GEMM(__nv_bfloat16, 16); else RMX_MOE_GEMM(__nv_bfloat16, 64);
    } else {
        RMX_FAIL("moe_gemm: unknown dtype %d", dtype);
    }
#undef RMX_MOE_GEMM
    return 0;
}

RMX_API int rmx_moe_combine(const void* y, const int* where, const float* weights, const void* shared_out, void* out,
                            int n_rows, int top, int width, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && top > 0 && width > 0 && y && where && out, "moe_combine: bad arguments");
    const size_t total = (size_t)n_rows * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_combine_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)y, where, weights,
                                            (const float*)shared_out, (float*)out, top, width, total), "moe_combine");
    else if (dtype == RMX_BF16 && (width & 7) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)shared_out & 15) == 0) {
        const size_t total8 = total / 8;
        RMX_CHECK_LAUNCHED(launch_dependent(moe_combine8_kernel, dim3((unsigned)((total8 + threads - 1) / threads)), dim3(threads), 0, s,
                                            (const __nv_bfloat16*)y, where, weights, (const __nv_bfloat16*)shared_out, (__nv_bfloat16*)out,
                                            top, width, total8), "moe_combine");
    } else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)y,
                                            where, weights, (const __nv_bfloat16*)shared_out, (__nv_bfloat16*)out, top, width, total),
                           "moe_combine");
    else
        RMX_FAIL("moe_combine: unknown dtype %d", dtype);
    return 0;
}

RMX_API int rmx_moe_gather_scaled(const void* x, const int* sorted, const float* weights, int top, void* out, int total, int width,
                                  int dtype, void* stream) {
    if (total == 0) return 0;
    RMX_REQUIRE(total > 0 && top > 0 && width > 0 && x && sorted && weights && out, "moe_gather_scaled: bad sizes or a null pointer");
    const size_t n = (size_t)total * width;
    const dim3 grid((unsigned)((n + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_gather_scaled_kernel<float>, grid, dim3(256), 0, s, (const float*)x, sorted, weights, top,
                                            (float*)out, width, n), "moe_gather_scaled");
    else if (dtype == RMX_BF16 && width % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const size_t n8 = n / 8;
        RMX_CHECK_LAUNCHED(launch_dependent(moe_gather_scaled8_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, s, (const uint4*)x, sorted,
                                            weights, top, (uint4*)out, width / 8, n8), "moe_gather_scaled");
    } else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(moe_gather_scaled_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x, sorted,
                                            weights, top, (__nv_bfloat16*)out, width, n), "moe_gather_scaled");
    else
        RMX_FAIL("moe_gather_scaled: unknown dtype %d", dtype);
    return 0;
}
