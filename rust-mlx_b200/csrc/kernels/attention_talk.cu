// Attention whose scores are mixed over the heads before the softmax ("talking heads"), over the paged cache:
//
//   s_g[i, j] = scale * q_g[i] . k_kv(g)[j]                   every query head g against its key head
//   s'_h[i, j] = sum_g talk[h, g] * s_g[i, j]                 a learned H x H matrix mixes the heads' scores
//   p_h = softmax_j (s'_h[i, j]) over the keys that i reads;  o_h[i] = sum_j p_h[j] v_kv(h)[j]
//
// A query's row of scores therefore needs ALL heads' scores of the same (query, key) pair: a block takes a token with all
// its heads, one warp a head.  Keys are visited in blocks of 32 (fewer for very wide key rows) aligned to absolute positions in ascending order with an
// online softmax in float; a raw score is summed in ascending d, a mixed score in ascending g.  The order in which numbers
// are added depends on the token's position (and the window) only: not on how a prompt was cut, on the batch, the page
// size or which pages hold the keys.
//
// attention_talk_kernel is the arrangement on the FMA units (both dtypes; the 32-bit path, and in bfloat16 the decoded tokens,
// whose keys may be split over several blocks that a second kernel merges).  attention_talk_mma_kernel is the arrangement
// on the tensor cores for bfloat16 steps with prompt portions.
#include "common.cuh"

namespace {
constexpr int TKB_MOST = 32;   // keys per block, at most (fewer where shared memory has no room for 32 keys of all key heads)

__device__ __forceinline__ void talk_load4(const float* p, float4& v) { v = *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void talk_load4(const __nv_bfloat16* p, float4& v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v = make_float4(a.x, a.y, b.x, b.y);
}

// (a block has up to 32 warps, one a head: the registers of a thread are bounded for the largest block)
template <typename T>
__global__ void __launch_bounds__(1024) attention_talk_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                      const float* __restrict__ talk, const int* __restrict__ positions,
                                      const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride,
                                      int page_size, T* __restrict__ out, int nq, int nkv, int hd, int dq, int dv, int window,
                                      float scale, int* __restrict__ status, int splits, float* __restrict__ partial, int TKB) {
    extern __shared__ float smem[];
    const int group = nq / nkv;
    const int t = blockIdx.x, split = blockIdx.y;
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

    // with splits, this block takes a run of the token's key blocks and leaves (m, l, unnormalised sums) for the merge
    int b_first = lo / TKB, b_last = pos / TKB;
    if (splits > 1) {
        const int per = (b_last - b_first + splits) / splits;
        b_first += split * per;
        b_last = min(b_last, b_first + per - 1);
    }
    for (int b = b_first; b <= b_last; ++b) {
        const int base = b * TKB;
        __syncthreads();
        if (((dq | hd) & 3) == 0) {        // four numbers a load
            const int row4 = row >> 2, dq4 = dq >> 2;
            for (int idx = threadIdx.x; idx < TKB * row4; idx += blockDim.x) {
                const int j = idx / row4, r = idx - j * row4;
                const int kh = r / dq4, d = (r - kh * dq4) * 4;
                const int kp = base + j;
                float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (kp >= lo && kp <= pos) {
                    const int page = table[kp / page_size];
                    if (page >= 0)
                        talk_load4(k_pool + (((size_t)page * nkv + kh) * page_size + kp % page_size) * hd + d, kv);
                    else if (r == 0)
                        atomicExch(status, 2);  // a key that should be there has no page
                }
                float* dst = Ks + ((size_t)j * nkv + kh) * kstride + d;
                dst[0] = kv.x; dst[1] = kv.y; dst[2] = kv.z; dst[3] = kv.w;
            }
        } else {
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
        }
        __syncthreads();
        const int kp = base + lane;
        const bool valid = lane < TKB && kp >= lo && kp <= pos;
        if (lane < TKB) {
            float s = 0.f;
            const float* qrow = Qs + head * dq;
            const float* krow = Ks + ((size_t)lane * nkv + kvh) * kstride;
            for (int d = 0; d < dq; ++d) s = fmaf(qrow[d], krow[d], s);
            Ss[head * TKB + lane] = s;
        }
        __syncthreads();
        float s = 0.f;
        if (lane < TKB)
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
        // eight keys' values are asked for before the first is used (the sums keep the keys' order).  Every lane takes part
        // in the shuffles; only what follows them depends on the lane's column.
        for (int j0 = 0; j0 < TKB; j0 += 8) {
            float pj[8];
            long long off[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                pj[j] = __shfl_sync(0xffffffffu, p, j0 + j);
                off[j] = __shfl_sync(0xffffffffu, voff, j0 + j);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int d = lane + 32 * i;
                if (i < per_lane && d < dv) {
                    float vv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) vv[j] = off[j] >= 0 ? to_float(v_pool[off[j] + d]) : 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i] = fmaf(pj[j], vv[j], acc[i]);
                }
            }
        }
    }
    if (splits > 1) {
        float* dst = partial + (((size_t)t * splits + split) * nq + head) * (dv + 2);
        if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int d = lane + 32 * i;
            if (i < per_lane && d < dv) dst[2 + d] = acc[i];
        }
        return;
    }
    const float inv_l = 1.f / l;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int d = lane + 32 * i;
        if (i < per_lane && d < dv) out[((size_t)t * nq + head) * dv + d] = from_float<T>(acc[i] * inv_l);
    }
}

// The shares of a token's key splits added up: one warp a (token, head); partial [tokens, splits, heads, 2 + dv] holds each
// split's maximum, sum of weights and unnormalised sums (a split without keys left m = -inf, l = 0).
template <typename T>
__global__ void attention_talk_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, int n_items, int nq, int dv, int splits) {
    allow_dependents();
    wait_for_prior_kernels();
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= n_items) return;
    const int t = item / nq, head = item - t * nq;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, partial[(((size_t)t * splits + s) * nq + head) * (dv + 2)]);
    float l = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float* p = partial + (((size_t)t * splits + s) * nq + head) * (dv + 2);
        if (p[1] > 0.f) l += p[1] * expf(p[0] - m);
    }
    const float inv_l = 1.f / l;
    for (int d = lane; d < dv; d += 32) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float* p = partial + (((size_t)t * splits + s) * nq + head) * (dv + 2);
            if (p[1] > 0.f) acc = fmaf(p[2 + d], expf(p[0] - m), acc);
        }
        out[((size_t)t * nq + head) * dv + d] = from_float<T>(acc * inv_l);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The arrangement on the tensor cores (bfloat16): a block takes 16 neighbouring tokens of one sequence with all heads, one
// warp a head, and walks the keys in tiles of 32 aligned to absolute positions.  For a tile every warp forms its head's raw
// scores S_g = Q_g K^T by mma.sync (m16n8k16, float accumulators) and leaves them, scaled, in shared memory; after a
// barrier the block's threads mix them in place, a thread a (token, key) pair with all its heads (a float multiply-add a
// pair of heads and score: the scores stay 32-bit; a raw score is read once, not once a head); after another barrier
// every warp takes its head's mixed scores back as its accumulator fragment, runs the online softmax on it and adds P V by
// mma.sync, V fetched by ldmatrix.trans.  K and V of
// all key heads of the tile are fetched once a block, 16 bytes a thread and piece, through the block table.
constexpr int MT = 16, MB = 32;    // tokens a block, keys a tile

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void talk_cp_async16(void* smem, const void* gmem, int bytes) {     // bytes 16, or 0: zeros are stored
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void talk_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void talk_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// NW: the most warps (heads) a block of this instance has; it bounds the registers a thread may take (16 heads: 128).
// stages 2: the next tile's keys and values are copied (cp.async) while this tile is worked on; 1 where shared memory has
// no room for two tiles.
template <int HD, int NW>
__global__ void __launch_bounds__(NW * 32) attention_talk_mma_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
    const float* __restrict__ talk, const int* __restrict__ positions, const int* __restrict__ q_start, int n_seqs,
    const int* __restrict__ block_table, int table_stride, int page_size, __nv_bfloat16* __restrict__ out, int nq, int nkv, int dv,
    int window, float scale, int* __restrict__ status, int stages, int splits, float* __restrict__ partial) {
    extern __shared__ __align__(16) unsigned char talk_smem[];
    constexpr int KS = HD + 8;                  // a key row in shared memory (16 bytes of padding: rows fall on different banks)
    constexpr int SB = MB + 4;                  // a row of scores
    allow_dependents();
    wait_for_prior_kernels();
    // which (sequence, tile of 16 tokens) this block takes: tiles are counted through the sequences in their order
    int tile = blockIdx.x, seq = 0, r0 = 0, r1 = 0;
    for (; seq < n_seqs; ++seq) {
        r0 = q_start[seq];
        r1 = q_start[seq + 1];
        const int tiles = (r1 - r0 + MT - 1) / MT;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (seq >= n_seqs) return;
    r0 += tile * MT;
    const int rows = min(MT, r1 - r0);
    const int head = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int kvh = head / (nq / nkv);
    const size_t tile_elems = (size_t)MB * nkv * KS;
    __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(talk_smem);                 // [stages][K, V][nkv][MB][KS]
    float* Ss = reinterpret_cast<float*>(KV + 2 * tile_elems * stages);              // [nq][MT][SB]
    float* Ts = Ss + (size_t)nq * MT * SB;                                           // [nq][nq]
    const int* table = block_table + (size_t)seq * table_stride;
    const int pos0 = positions[r0], pos_last = pos0 + rows - 1;
    const int lo0 = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int TS = (nq + 3) & ~3;               // a row of the mixing matrix in shared memory, padded with zeros
    for (int g = lane; g < TS; g += 32) Ts[head * TS + g] = g < nq ? talk[head * nq + g] : 0.f;

    // this head's queries as A fragments: rows gid and gid + 8 of the tile, all of a head's numbers
    uint32_t qa[HD / 16][4];
    {
        const __nv_bfloat16* qrow0 = q + ((size_t)(r0 + gid) * nq + head) * HD;
        const __nv_bfloat16* qrow1 = q + ((size_t)(r0 + gid + 8) * nq + head) * HD;
        const bool ok0 = gid < rows, ok1 = gid + 8 < rows;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            const int c = ks * 16 + 2 * tig;
            qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(qrow0 + c) : 0u;
            qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(qrow1 + c) : 0u;
            qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(qrow0 + c + 8) : 0u;
            qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(qrow1 + c + 8) : 0u;
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // of rows gid and gid + 8 (sums: this thread's share)
    const int prow0 = pos0 + gid, prow1 = pos0 + gid + 8;
    const int lrow0 = window > 0 ? max(0, prow0 - window + 1) : 0, lrow1 = window > 0 ? max(0, prow1 - window + 1) : 0;
    constexpr int PIECES = HD / 8;              // 16-byte pieces of a key row

    // the copies of key tile b into buffer `stage`: keys outside what the block's rows read, and holes, become zeros
    auto fetch = [&](int b, int stage) {
        __nv_bfloat16* kd = KV + 2 * tile_elems * stage;
        __nv_bfloat16* vd = kd + tile_elems;
        for (int idx = threadIdx.x; idx < MB * nkv * PIECES; idx += blockDim.x) {
            const int piece = idx % PIECES, kh = (idx / PIECES) % nkv, j = idx / (PIECES * nkv);
            const int kp = b * MB + j;
            size_t off = 0;
            int bytes = 0;
            if (kp >= lo0 && kp <= pos_last) {
                const int page = table[kp / page_size];
                if (page >= 0) {
                    off = (((size_t)page * nkv + kh) * page_size + kp % page_size) * HD + piece * 8;
                    bytes = 16;
                } else if (piece == 0 && kh == 0) {
                    atomicExch(status, 2);      // a key that should be there has no page
                }
            }
            const size_t at = ((size_t)kh * MB + j) * KS + piece * 8;      // (a key head's rows are neighbours: rows fall on different banks)
            talk_cp_async16(kd + at, k_pool + off, bytes);
            talk_cp_async16(vd + at, v_pool + off, bytes);
        }
        talk_cp_async_commit();
    };
    // with splits (grid.y), this block takes a run of the tile's key tiles and leaves (m, l, unnormalised sums) for the merge
    int b_first = lo0 / MB, b_last = pos_last / MB;
    if (splits > 1) {
        const int per = (b_last - b_first + splits) / splits;
        b_first += blockIdx.y * per;
        b_last = min(b_last, b_first + per - 1);
    }
    if (b_first <= b_last) fetch(b_first, 0);
    for (int b = b_first; b <= b_last; ++b) {
        const int base = b * MB;
        const int stage = stages == 2 ? (b - b_first) & 1 : 0;
        if (stages == 2 && b < b_last) {
            fetch(b + 1, stage ^ 1);            // (its buffer was last read a tile ago: everyone has passed that tile's last barrier)
            talk_cp_async_wait<1>();
        } else {
            talk_cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* Ks = KV + 2 * tile_elems * stage;
        const __nv_bfloat16* Vs = Ks + tile_elems;
        // raw scores of this head, scaled, into shared memory
#pragma unroll
        for (int nt = 0; nt < MB / 8; ++nt) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const __nv_bfloat16* krow = Ks + ((size_t)kvh * MB + nt * 8 + gid) * KS + 2 * tig;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                mma_bf16(c, qa[ks], *reinterpret_cast<const uint32_t*>(krow + ks * 16), *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8));
            float* srow = Ss + ((size_t)head * MT + gid) * SB + nt * 8 + 2 * tig;
            *reinterpret_cast<float2*>(srow) = make_float2(c[0] * scale, c[1] * scale);
            *reinterpret_cast<float2*>(srow + 8 * SB) = make_float2(c[2] * scale, c[3] * scale);
        }
        __syncthreads();
        // the scores are mixed in place, a thread a (token, key) pair of the tile: it takes the pair's raw scores of all heads
        // (what every head's row needs is read once, not once a head), forms every head's mixed score in float, ascending g,
        // and puts them back; nobody else touches the pair
        for (int pair = threadIdx.x; pair < MT * MB; pair += blockDim.x) {
            float* at = Ss + (size_t)(pair / MB) * SB + pair % MB;
            float raw[NW];
#pragma unroll
            for (int g = 0; g < NW; ++g) raw[g] = g < nq ? at[(size_t)g * MT * SB] : 0.f;
            for (int h = 0; h < nq; ++h) {
                const float4* w4 = reinterpret_cast<const float4*>(Ts + h * TS);
                float acc = 0.f;
#pragma unroll
                for (int g4 = 0; g4 < NW / 4; ++g4) {
                    if (g4 * 4 < nq) {
                        const float4 w = w4[g4];
                        acc = fmaf(w.x, raw[4 * g4], acc);
                        acc = fmaf(w.y, raw[4 * g4 + 1], acc);
                        acc = fmaf(w.z, raw[4 * g4 + 2], acc);
                        acc = fmaf(w.w, raw[4 * g4 + 3], acc);
                    }
                }
                at[(size_t)h * MT * SB] = acc;
            }
        }
        __syncthreads();
        // this head's mixed scores, at its own fragment's places
        float s[MB / 8][4];
        {
            const float* srow = Ss + ((size_t)head * MT + gid) * SB + 2 * tig;
#pragma unroll
            for (int nt = 0; nt < MB / 8; ++nt) {
                const float2 a = *reinterpret_cast<const float2*>(srow + nt * 8);
                const float2 c = *reinterpret_cast<const float2*>(srow + 8 * SB + nt * 8);
                s[nt][0] = a.x; s[nt][1] = a.y; s[nt][2] = c.x; s[nt][3] = c.y;
            }
        }
        // which keys each row reads, the rows' maxima, the weights
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < MB / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kp = base + nt * 8 + 2 * tig + e;
                if (!(kp >= lrow0 && kp <= prow0)) s[nt][e] = -INFINITY;
                if (!(kp >= lrow1 && kp <= prow1)) s[nt][2 + e] = -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        // (a row that has seen no key yet keeps zeros: nothing to rescale, no weights)
        const float corr0 = n0 == -INFINITY ? 1.f : __expf(m0 - n0), corr1 = n1 == -INFINITY ? 1.f : __expf(m1 - n1);
        const float ref0 = n0 == -INFINITY ? 0.f : n0, ref1 = n1 == -INFINITY ? 0.f : n1;
        m0 = n0;
        m1 = n1;
        l0 *= corr0;
        l1 *= corr1;
#pragma unroll
        for (int nt = 0; nt < MB / 8; ++nt) {
            s[nt][0] = __expf(s[nt][0] - ref0);
            s[nt][1] = __expf(s[nt][1] - ref0);
            s[nt][2] = __expf(s[nt][2] - ref1);
            s[nt][3] = __expf(s[nt][3] - ref1);
            l0 += s[nt][0] + s[nt][1];
            l1 += s[nt][2] + s[nt][3];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= corr0; o[i][1] *= corr0;
            o[i][2] *= corr1; o[i][3] *= corr1;
        }
        // O += P V: the weights are the A fragments as they stand, V comes transposed out of shared memory
#pragma unroll
        for (int kt = 0; kt < MB / 16; ++kt) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            pa[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            pa[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            pa[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
            const __nv_bfloat16* vrow = Vs + ((size_t)kvh * MB + kt * 16 + (lane & 15)) * KS;
#pragma unroll
            for (int dt = 0; dt < HD / 8; ++dt) {
                uint32_t b0, b1;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow + dt * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma_bf16(o[dt], pa, b0, b1);
            }
        }
        __syncthreads();                        // (the scores and this tile's buffer are free again)
        if (stages == 1 && b < b_last) fetch(b + 1, 0);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (splits > 1) {
        float* dst0 = partial + (((size_t)(r0 + gid) * splits + blockIdx.y) * nq + head) * (dv + 2);
        float* dst1 = partial + (((size_t)(r0 + gid + 8) * splits + blockIdx.y) * nq + head) * (dv + 2);
        if (tig == 0 && gid < rows) { dst0[0] = m0; dst0[1] = l0; }
        if (tig == 0 && gid + 8 < rows) { dst1[0] = m1; dst1[1] = l1; }
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
            const int d = dt * 8 + 2 * tig;
            if (gid < rows) {
                if (d < dv) dst0[2 + d] = o[dt][0];
                if (d + 1 < dv) dst0[3 + d] = o[dt][1];
            }
            if (gid + 8 < rows) {
                if (d < dv) dst1[2 + d] = o[dt][2];
                if (d + 1 < dv) dst1[3 + d] = o[dt][3];
            }
        }
        return;
    }
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
        const int d = dt * 8 + 2 * tig;
        if (d < dv) {       // (dv is even whenever it is below HD's padding: a pair is written whole or not at all, except the last odd one)
            __nv_bfloat16* dst0 = out + ((size_t)(r0 + gid) * nq + head) * dv + d;
            __nv_bfloat16* dst1 = out + ((size_t)(r0 + gid + 8) * nq + head) * dv + d;
            if (gid < rows) {
                dst0[0] = __float2bfloat16_rn(o[dt][0] * inv0);
                if (d + 1 < dv) dst0[1] = __float2bfloat16_rn(o[dt][1] * inv0);
            }
            if (gid + 8 < rows) {
                dst1[0] = __float2bfloat16_rn(o[dt][2] * inv1);
                if (d + 1 < dv) dst1[1] = __float2bfloat16_rn(o[dt][3] * inv1);
            }
        }
    }
}

template <int HD, int NW>
int launch_talk_mma_n(const void* q, const void* k_pool, const void* v_pool, const float* talk, const int* positions, const int* q_start,
                      int n_seqs, int n_tokens, const int* block_table, int table_stride, int page_size, void* out, int nq, int nkv, int dv,
                      int window, float scale, int* status, size_t smem, int stages, int splits, float* partial, cudaStream_t s) {
    static bool raised[64] = {};
    if (rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(attention_talk_mma_kernel<HD, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) RMX_FAIL("attention_talk_mma: shared memory refused: %s", cudaGetErrorString(e));
    }
    const int tiles = (n_tokens + MT - 1) / MT + n_seqs;      // (an upper bound: blocks beyond the step's tiles leave at once)
    RMX_CHECK_LAUNCHED(launch_dependent(attention_talk_mma_kernel<HD, NW>, dim3(tiles, splits), dim3(nq * 32), smem, s, (const __nv_bfloat16*)q,
                                        (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, talk, positions, q_start, n_seqs,
                                        block_table, table_stride, page_size, (__nv_bfloat16*)out, nq, nkv, dv, window, scale, status, stages, splits,
                                        partial),
                       "attention_talk_mma");
    return 0;
}

template <int HD>
int launch_talk_mma(const void* q, const void* k_pool, const void* v_pool, const float* talk, const int* positions, const int* q_start,
                    int n_seqs, int n_tokens, const int* block_table, int table_stride, int page_size, void* out, int nq, int nkv, int dv,
                    int window, float scale, int* status, size_t smem, int stages, int splits, float* partial, cudaStream_t s) {
    if (nq <= 8)
        return launch_talk_mma_n<HD, 8>(q, k_pool, v_pool, talk, positions, q_start, n_seqs, n_tokens, block_table, table_stride, page_size, out,
                                        nq, nkv, dv, window, scale, status, smem, stages, splits, partial, s);
    if (nq <= 16)
        return launch_talk_mma_n<HD, 16>(q, k_pool, v_pool, talk, positions, q_start, n_seqs, n_tokens, block_table, table_stride, page_size, out,
                                         nq, nkv, dv, window, scale, status, smem, stages, splits, partial, s);
    return launch_talk_mma_n<HD, 32>(q, k_pool, v_pool, talk, positions, q_start, n_seqs, n_tokens, block_table, table_stride, page_size, out,
                                     nq, nkv, dv, window, scale, status, smem, stages, splits, partial, s);
}
}  // namespace

static size_t talk_mma_smem(int nq, int nkv, int hd, int stages) {
    return 2 * (size_t)stages * MB * nkv * (hd + 8) * 2 + ((size_t)nq * MT * (MB + 4) + (size_t)nq * ((nq + 3) & ~3)) * 4;
}

// Whether the tensor-core arrangement takes these sizes (bfloat16 only): heads of a multiple of 16 numbers up to 128, and room
// in shared memory for a tile's keys and values of all key heads and all heads' scores.
RMX_API int rmx_attention_talk_mma_supports(int nq, int nkv, int hd) {
    return nq > 0 && nq <= 32 && nkv > 0 && nq % nkv == 0 && hd >= 16 && hd <= 128 && hd % 16 == 0 && talk_mma_smem(nq, nkv, hd, 1) <= 220 * 1024;
}

// q [tokens, nq, hd], pools with heads of hd numbers, talk float [nq, nq], out [tokens, nq, dv] dense; q_start [n_seqs + 1].
RMX_API int rmx_attention_talk_mma(const void* q, const void* k_pool, const void* v_pool, const float* talk, const int* positions,
                                   const int* q_start, int n_seqs, int n_tokens, const int* block_table, int table_stride, int page_size,
                                   void* out, int nq, int nkv, int hd, int dv, int window, float scale, int* status, int splits,
                                   float* partial, void* stream) {
    if (n_tokens == 0 || n_seqs == 0) return 0;
    RMX_REQUIRE(rmx_attention_talk_mma_supports(nq, nkv, hd), "attention_talk_mma: %d heads over %d key heads of %d numbers are not taken", nq, nkv, hd);
    RMX_REQUIRE(dv > 0 && dv <= hd && page_size > 0 && table_stride > 0 && window >= 0 && talk && q_start, "attention_talk_mma: bad arguments");
    RMX_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0, "attention_talk_mma: operands must be 16-byte aligned");
    RMX_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || partial), "attention_talk_mma: %d splits need room for their shares", splits);
    const int stages = talk_mma_smem(nq, nkv, hd, 2) <= 220 * 1024 ? 2 : 1;
    const size_t smem = talk_mma_smem(nq, nkv, hd, stages);
    cudaStream_t s = (cudaStream_t)stream;
    int rc = -2;
#define TALK_CASE(HD_)                                                                                                                     \
    case HD_: rc = launch_talk_mma<HD_>(q, k_pool, v_pool, talk, positions, q_start, n_seqs, n_tokens, block_table, table_stride, page_size, \
                                        out, nq, nkv, dv, window, scale, status, smem, stages, splits, partial, s); break;
    switch (hd) {
        TALK_CASE(16) TALK_CASE(32) TALK_CASE(48) TALK_CASE(64) TALK_CASE(80) TALK_CASE(96) TALK_CASE(112) TALK_CASE(128)
    }
#undef TALK_CASE
    if (rc == -2) RMX_FAIL("attention_talk_mma: head size %d", hd);
    if (rc != 0) return rc;
    if (splits > 1) {
        attention_talk_merge_kernel<__nv_bfloat16><<<(n_tokens * nq + 3) / 4, 128, 0, s>>>(partial, (__nv_bfloat16*)out, n_tokens * nq, nq, dv, splits);
        RMX_CHECK_LAUNCH("attention_talk_merge");
    }
    return 0;
}

// q [tokens, nq, hd] (the first dq numbers of a head count), pools with heads of hd numbers (keys: the first dq, values: the
// first dv), talk float [nq, nq], out [tokens, nq, dv] dense.
RMX_API int rmx_attention_talk(const void* q, const void* k_pool, const void* v_pool, const float* talk, const int* positions,
                               const int* seq_index, const int* block_table, int table_stride, int page_size, void* out,
                               int n_tokens, int nq, int nkv, int hd, int dq, int dv, int window, float scale, int* status,
                               int splits, float* partial, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && nq <= 32, "attention_talk: %d query heads over %d kv heads (at most 32)", nq, nkv);
    RMX_REQUIRE(dq > 0 && dv > 0 && dq <= hd && dv <= hd && hd <= 512, "attention_talk: head sizes %d %d in %d", dq, dv, hd);
    RMX_REQUIRE(page_size > 0 && table_stride > 0 && window >= 0 && talk, "attention_talk: bad page geometry or no mixing matrix");
    // keys a block: 32, or fewer where 32 keys of all key heads have no room (what the sizes alone decide: the order of a
    // row's sums follows them)
    int TKB = TKB_MOST;
    auto need = [&](int kb) { return ((size_t)kb * nkv * (dq + 1) + (size_t)nq * kb + (size_t)nq * dq + (size_t)nq * nq) * sizeof(float); };
    while (TKB > 8 && need(TKB) > 200 * 1024) TKB /= 2;
    const size_t smem = need(TKB);
    RMX_REQUIRE(smem <= 200 * 1024, "attention_talk: %d key heads of %d numbers need too much shared memory", nkv, dq);
    RMX_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || partial), "attention_talk: %d splits need room for their shares", splits);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens, splits);
    const int merge_blocks = (n_tokens * nq + 3) / 4;
    if (dtype == RMX_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_talk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_talk_kernel<float><<<grid, nq * 32, smem, s>>>((const float*)q, (const float*)k_pool, (const float*)v_pool, talk,
                                                                 positions, seq_index, block_table, table_stride, page_size,
                                                                 (float*)out, nq, nkv, hd, dq, dv, window, scale, status, splits, partial, TKB);
        if (splits > 1) attention_talk_merge_kernel<float><<<merge_blocks, 128, 0, s>>>(partial, (float*)out, n_tokens * nq, nq, dv, splits);
    } else if (dtype == RMX_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_talk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_talk_kernel<__nv_bfloat16><<<grid, nq * 32, smem, s>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, talk, positions, seq_index,
            block_table, table_stride, page_size, (__nv_bfloat16*)out, nq, nkv, hd, dq, dv, window, scale, status, splits, partial, TKB);
        if (splits > 1)
            attention_talk_merge_kernel<__nv_bfloat16><<<merge_blocks, 128, 0, s>>>(partial, (__nv_bfloat16*)out, n_tokens * nq, nq, dv, splits);
    } else {
        RMX_FAIL("attention_talk: unknown dtype %d", dtype);
    }
    RMX_CHECK_LAUNCH("attention_talk");
    return 0;
}
