// The experts' products of a routed feed-forward on the Blackwell tensor cores (bfloat16):
//   C[p, :] = W[e] . A[p, :]   for every place p of expert e's run of rows,
// rows sorted by expert (see moe.cu), W [experts, N, K] stacked.
//
// The arrangement is the one of the few-rows product (gemm_tcgen05.cu): the weight fills the 128-row side of the
// instruction, D[128 weight rows, MPAD rows of activations] += Wtile[128, 64] . Atile[MPAD, 64]^T with the
// accumulator in tensor memory, tiles by TMA (128-byte swizzle) through a ring of stages, one thread issuing copies
// and one the MMAs.  A block owns 128 weight rows of ONE expert and one tile of MPAD of that expert's rows; which
// expert and which rows it finds by walking the offsets on the device, so nothing waits for the host and blocks
// beyond the step's tiles leave at once.  An A tile may reach past its expert's run (into the next expert's rows,
// or past the last row, which reads as zeros): those columns of the accumulator are never stored.
// MPAD 16 (decoding: a row or two an expert, the time is the weights' bytes), 64, 128 or 256 (prompts).  WT = 2: a block
// takes two neighbouring tiles of 128 weight rows against the same rows of activations, an accumulator each, so that
// every byte of an A tile in flight feeds twice the products.
// epilogue 1: an expert's weight rows come in blocks of 64 gate rows and their 64 up rows, and the block stores
// act(gate) * up, [rows, N / 2], formed in float and rounded once: no round trip of the gate/up rows.
//
// Every wait on a barrier gives up after a bounded number of polls, records status 3 and lets the block run to its
// end (tensor memory is always freed).
#include <cuda.h>

#include "activation.cuh"
#include "tcgen05.cuh"

namespace {
constexpr int TILE_N = 128, TILE_K = 64, UMMA_K = 16, THREADS = 128;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

struct GroupedParams {
    __nv_bfloat16* c;
    const int* offsets;      // [n_experts + 1]
    int* status;
    int n_experts, N, K, ldc, k_blocks, epilogue, act;
    float limit, alpha;      // of the gated epilogue's activation (activation.cuh), where it has such constants
};

template <int MPAD, int STAGES, int WT>
__global__ void __launch_bounds__(THREADS) moe_grouped_kernel(const __grid_constant__ CUtensorMap map_w,
                                                              const __grid_constant__ CUtensorMap map_a,
                                                              const GroupedParams p) {
    constexpr int W_BYTES = TILE_N * TILE_K * 2, A_BYTES = MPAD * TILE_K * 2;
    constexpr int STAGE_BYTES = WT * W_BYTES + A_BYTES;
    constexpr int TMEM_COLS = WT * MPAD < 32 ? 32 : WT * MPAD;      // (16, 64, 128, 256 or 512: a power of two)
    constexpr int CH = MPAD < 128 ? MPAD : 128;                      // columns of an accumulator a thread holds at a time
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int s_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    allow_dependents();
    wait_for_prior_kernels();          // the offsets and the rows come from the kernels before this one
    // which expert, which of its rows
    int tile_m = blockIdx.y, e = 0, begin = 0, end = 0;
    for (; e < p.n_experts; ++e) {
        begin = p.offsets[e];
        end = p.offsets[e + 1];
        const int tiles_e = (end - begin + MPAD - 1) / MPAD;
        if (tile_m < tiles_e) break;
        tile_m -= tiles_e;
    }
    if (e >= p.n_experts) return;      // (the whole block alike: nothing is allocated yet)
    const int m0 = begin + tile_m * MPAD;
    const int rows = min(MPAD, end - m0);
    const int w_row0 = e * p.N + blockIdx.x * (WT * TILE_N);
    const int n_kb = p.k_blocks;

    if (tid == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_smem)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_acc = tmem_base_smem;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % STAGES, round = i / STAGES;
            if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, SPIN_LIMIT)) { atomicExch(&s_failed, 1); break; }
            unsigned char* dst = tiles + s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
#pragma unroll
            for (int wt = 0; wt < WT; ++wt) tma_load_2d(dst + wt * W_BYTES, &map_w, &full_bar[s], i * TILE_K, w_row0 + wt * TILE_N);
            tma_load_2d(dst + WT * W_BYTES, &map_a, &full_bar[s], i * TILE_K, m0);
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = umma_idesc(MPAD);
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % STAGES, round = i / STAGES;
            if (!mbar_wait(&full_bar[s], round & 1, SPIN_LIMIT)) { atomicExch(&s_failed, 1); break; }
            tcgen05_fence_after();
            const uint32_t w_addr = smem_addr(tiles + s * STAGE_BYTES), a_addr = w_addr + WT * W_BYTES;
#pragma unroll
            for (int wt = 0; wt < WT; ++wt)
#pragma unroll
                for (int k = 0; k < TILE_K / UMMA_K; ++k)
                    umma_mma(tmem_acc + wt * MPAD, umma_desc(w_addr + wt * W_BYTES + k * UMMA_K * 2), umma_desc(a_addr + k * UMMA_K * 2),
                             idesc, i > 0 || k > 0);
            umma_commit(&empty_bar[s]);
        }
        umma_commit(&acc_bar);
    }
    __syncwarp();

    // ---- epilogue: every thread owns one weight row of each tile, CH rows of activations at a time
    const bool ok = mbar_wait(&acc_bar, 0, SPIN_LIMIT);
    if (!ok) atomicExch(&s_failed, 1);
    tcgen05_fence_after();
    __syncthreads();                   // every MMA has completed: the stages are free (the gated epilogue uses them)
    const bool failed = s_failed != 0;
    if (!failed) {
        float* ex = reinterpret_cast<float*>(tiles);   // [CH][64]: the gated epilogue's exchange between the halves of the block
#pragma unroll 1
        for (int wt = 0; wt < WT; ++wt) {
#pragma unroll 1
            for (int c0 = 0; c0 < MPAD; c0 += CH) {
                if (c0 >= rows) break;             // (the whole block alike)
                float acc[CH];
#pragma unroll
                for (int c = 0; c < CH; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem_acc + ((uint32_t)(warp * 32) << 16) + wt * MPAD + c0 + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[c + j] = __uint_as_float(r[j]);
                }
                const int tile_x = blockIdx.x * WT + wt;
                if (p.epilogue == 1) {
                    // the upper half of the block (up rows) hands its sums to the lower half (gate rows)
                    __syncthreads();               // (whoever still reads the exchange of the chunk before)
                    if (tid >= 64) {
#pragma unroll
                        for (int t = 0; t < CH; ++t) ex[t * 64 + tid - 64] = acc[t];
                    }
                    __syncthreads();
                    const int col = tile_x * 64 + tid;
                    if (tid < 64 && col < p.N / 2) {
#pragma unroll
                        for (int t = 0; t < CH; ++t)
                            if (c0 + t < rows)
                                p.c[(size_t)(m0 + c0 + t) * p.ldc + col] = __float2bfloat16_rn(gated_act(acc[t], ex[t * 64 + tid], p.act, p.limit, p.alpha));
                    }
                } else {
                    const int n = tile_x * TILE_N + tid;
                    if (n < p.N) {
#pragma unroll
                        for (int t = 0; t < CH; ++t)
                            if (c0 + t < rows)
                                p.c[(size_t)(m0 + c0 + t) * p.ldc + n] = __float2bfloat16_rn(p.epilogue == 2 ? unary_act(acc[t], p.act) : acc[t]);
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_acc), "r"(TMEM_COLS));
    if (failed && tid == 0) atomicExch(p.status, 3);
}

template <int MPAD, int STAGES, int WT>
int launch_grouped(const CUtensorMap& mw, const CUtensorMap& ma, const GroupedParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t smem = (size_t)STAGES * (WT * TILE_N * TILE_K * 2 + MPAD * TILE_K * 2) + 1024;
    grid.x = (grid.x + WT - 1) / WT;
    static bool raised[64] = {};
    if (rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<MPAD, STAGES, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RMX_FAIL("moe_gemm_tcgen05: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    }
    RMX_CHECK_LAUNCHED(launch_dependent(moe_grouped_kernel<MPAD, STAGES, WT>, grid, dim3(THREADS), smem, s, mw, ma, p), "moe_gemm_tcgen05");
    return 0;
}

// out[p, :] = x[pairs[p] / top, :]: the layer's rows in the order of the experts' runs (16-byte copies).
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ pairs, int top, uint4* __restrict__ out,
                                  int chunks, size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t p = idx / chunks;
    const int c = (int)(idx - p * chunks);
    out[idx] = x[(size_t)(pairs[p] / top) * chunks + c];
}
}  // namespace

static int g_tile_variant = 0;

// What the kernel takes: K a multiple of 8 (rows of 16-byte multiples for TMA).
RMX_API int rmx_moe_gemm_tcgen05_supports(int N, int K) { return N >= 1 && K >= 8 && K % 8 == 0; }

// A [total, K] (rows lda apart) in sorted order, W [n_experts, N, K], C [total, N] or, with epilogue 1, [total, N / 2];
// all bfloat16.  act, limit, alpha: the gated epilogue's activation (activation.cuh; epilogue 1).  Epilogue 2: C = f(A W^T) number by
// number with a one-argument activation (act 3: squared relu).
RMX_API int rmx_moe_gemm_tcgen05(const void* A, int lda, const void* W, void* C, int ldc, const int* offsets, int n_experts,
                                 int total, int N, int K, int epilogue, int act, float limit, float alpha, int* status, void* stream) {
    if (total == 0 || N == 0) return 0;
    RMX_REQUIRE(total > 0 && n_experts > 0 && rmx_moe_gemm_tcgen05_supports(N, K), "moe_gemm_tcgen05: bad sizes total=%d N=%d K=%d", total, N, K);
    RMX_REQUIRE(lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "moe_gemm_tcgen05: operands must be 16-byte aligned");
    RMX_REQUIRE(epilogue == 0 || epilogue == 2 || (epilogue == 1 && N % 128 == 0), "moe_gemm_tcgen05: the gated epilogue needs N to be a multiple of 128, got %d", N);
    RMX_REQUIRE(epilogue == 2 ? act == RMX_ACT_RELU2 : (act >= 0 && act <= 2), "moe_gemm_tcgen05: unknown activation %d for epilogue %d", act, epilogue);
    RMX_REQUIRE((long long)n_experts * N < (1ll << 31), "moe_gemm_tcgen05: too many weight rows");
    RMX_REQUIRE(offsets && status && C, "moe_gemm_tcgen05: a null pointer");
    // tiles of rows: 16 while experts have a row or two (decoding), 64, then 128
    int mpad = total <= 16 * n_experts ? 16 : (total < 96 * n_experts ? 64 : 128);
    const int variant = mpad == 128 ? g_tile_variant : 0;
    if (variant == 2) mpad = 256;
    const int tiles_m = (total + mpad - 1) / mpad + n_experts;
    RMX_REQUIRE(tiles_m <= 65535, "moe_gemm_tcgen05: too many row tiles (%d)", tiles_m);
    CUtensorMap mw, ma;
    if (rmx_make_tensor_map(&mw, W, n_experts * N, K, K, TILE_N) != 0) return -1;
    if (rmx_encode_tensor_map(&ma, A, total, K, lda, mpad) != 0) return -1;
    GroupedParams p;
    p.c = (__nv_bfloat16*)C; p.offsets = offsets; p.status = status; p.n_experts = n_experts; p.N = N; p.K = K; p.ldc = ldc;
    p.k_blocks = (K + TILE_K - 1) / TILE_K; p.epilogue = epilogue; p.act = act; p.limit = limit; p.alpha = alpha;
    dim3 grid((N + TILE_N - 1) / TILE_N, tiles_m);
    cudaStream_t s = (cudaStream_t)stream;
    if (mpad == 16) return launch_grouped<16, 6, 1>(mw, ma, p, grid, s);
    if (mpad == 64) return launch_grouped<64, 4, 1>(mw, ma, p, grid, s);
    if (variant == 1) return launch_grouped<128, 2, 2>(mw, ma, p, grid, s);
    if (variant == 2) return launch_grouped<256, 2, 1>(mw, ma, p, grid, s);
    // Two stages: three blocks fit an SM, and while one waits for a tile or stores its sums the others multiply.  Measured at
    // 64 experts of [2816, 4096], 192 rows each (us): 4 stages, a block an SM 1,575; 3 stages, two blocks 893; 2 stages, three
    // blocks 660; two weight tiles a block (two blocks an SM) 715; tiles of 256 rows (two blocks an SM) 579, but 198 against
    // 170 where experts have 256 rows each.  An MMA of 128 x 128 x 16 with both operands in shared memory reads 8 KB in its
    // 64 cycles, which is all an SM's shared memory gives, and the copies that fill the stages want as much again: one CTA
    // a tile cannot keep the tensor cores more than half busy, whatever the arrangement.
    return launch_grouped<128, 2, 1>(mw, ma, p, grid, s);
}

// Which arrangement tiles of 128 rows take, for comparisons: 0 the one above; 1 two weight tiles a block against the same
// rows; 2 tiles of 256 rows.
RMX_API void rmx_moe_set_tile_variant(int v) { g_tile_variant = v; }

RMX_API int rmx_moe_gather(const void* x, const int* pairs, int top, void* out, int total, int width, void* stream) {
    if (total == 0) return 0;
    RMX_REQUIRE(total > 0 && top > 0 && width > 0 && width % 8 == 0, "moe_gather: rows of %d bfloat16 are no multiple of 16 bytes", width);
    RMX_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0, "moe_gather: operands must be 16-byte aligned");
    const int chunks = width / 8;
    const size_t n = (size_t)total * chunks;
    RMX_CHECK_LAUNCHED(launch_dependent(moe_gather_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                                        (const uint4*)x, pairs, top, (uint4*)out, chunks, n), "moe_gather");
    return 0;
}
