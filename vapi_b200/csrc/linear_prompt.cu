// Matrix product for prompt-sized steps (from 33 rows up to a whole prompt portion):
//   y[m][n] = sum_k a[m][k] * W[n][k],  bfloat16 in, float accumulate,
// as a persistent kernel on the fifth-generation tensor cores: one block per multiprocessor walks
// over output tiles; operands come into a ring of shared-memory stages by TMA (128-byte swizzle),
// tcgen05.mma accumulates a tile in tensor memory, and while the next tile accumulates in a second
// buffer of tensor memory the epilogue warps read the finished one back with tcgen05.ld and apply
// the fused epilogue.
//
// Orientation.  The tokens are the 128-row operand (tensor-memory lanes), the weight rows are the
// columns (BN = 128 or 256 features a tile), so that one epilogue thread owns one token of the
// tile: what belongs to a token (the factor of a deferred RMSNorm, the sum of squares the next norm
// needs) never crosses threads.
//
// Pairs.  With PAIR = 2 two blocks on neighbouring multiprocessors form a cluster and work on
// one tile of 256 tokens x BN features with tcgen05.mma.cta_group::2: each block loads its own
// 128 tokens and its own half of the weight rows, the even block issues the MMAs for both, and
// each block holds (and finishes) the accumulator of its own 128 tokens.  Every operand byte then
// crosses from L2 into a multiprocessor half as often.
//
// Roles (64 threads and the epilogue warps).  Warp 0, one lane: TMA producer.  Warp 1: tensor-memory
// allocation, and one lane of the even block: the MMA issue loop; tcgen05.commit hands a stage back
// to the producers of both blocks and a finished accumulator to the epilogue warps of both.
// Warps 2..: epilogue, a warp for 32 tokens of the tile, one token per thread while the sums come
// out of tensor memory: bfloat16 out | float out | SwiGLU (a tile's columns are BN/2 gate features
// followed by the BN/2 matching up features) | add into the float residual stream with what the
// next norm needs (bfloat16(stream * next norm weight), one partial sum of squares per token and
// tile column).  The token operand may be the residual stream seen through a deferred RMSNorm (see
// gemv.cu): then the epilogue scales every token's row by rsqrt(mean x^2 + eps).
//
// Every mbarrier wait is bounded: after the limit a role records that it gave up, every role of the
// block leaves its loop at its next wait, status 16 is recorded and the block drains to its end
// (tensor memory is released on every path; the cluster barriers at both ends are hardware barriers
// that every thread reaches on every path).
#include "tcgen05.cuh"

#include <unordered_map>

using namespace vapi;

constexpr int PL_BM = 128;
constexpr int PL_BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
#ifndef PL_EPI_WARPS
#define PL_EPI_WARPS 4                    // 4: one epilogue warp for each 32 tokens of a tile; 8: two, each with half of the features
#endif
constexpr int PL_HALVES = PL_EPI_WARPS / 4;
constexpr int PL_EPI_THREADS = 32 * PL_EPI_WARPS;
constexpr int PL_THREADS = 64 + PL_EPI_THREADS;
constexpr int PL_A_BYTES = PL_BM * PL_BK * 2;
#ifndef PL_RING_KB
#define PL_RING_KB 192
#endif

enum { PL_PRO_ACT = 0, PL_PRO_NORM = 1 };
enum { PL_EPI_BF16 = 0, PL_EPI_SWIGLU = 1, PL_EPI_RESID = 2, PL_EPI_F32 = 3 };

struct PlParams {
    int N, K, M, epi, pro, ff;
    int num_kb, num_m, num_n, num_tiles;
    const float* ss_in; int ss_parts; float eps;
    __nv_bfloat16* out_bf16; float* out_f32; long long out_stride;
    const float* bias; float* resid; float* ss_out; const float* next_w; __nv_bfloat16* xw_out;
    int* status;
};

template <int BN, int PAIR> struct PlCfg {
    static constexpr int B_BYTES = (BN / PAIR) * PL_BK * 2;                  // this block's share of the weight rows
    static constexpr int STAGE_BYTES = PL_A_BYTES + B_BYTES;
    static constexpr int STAGES_RAW = (PL_RING_KB * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS = 2 * BN;                                 // two accumulators
    static constexpr int TAIL_BYTES = 256 /*barriers, slot, flag*/ + 2 * 256 * 4 /*bias, next norm weight*/ +
                                      PL_EPI_WARPS * 32 * 32 * 4 /*a 32 x 32 float patch for each epilogue warp*/;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment*/ + TAIL_BYTES;
};

__device__ __forceinline__ void pl_epi_bar() { asm volatile("bar.sync 1, %0;" ::"n"(PL_EPI_THREADS) : "memory"); }
__device__ __forceinline__ void pl_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned pl_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's window, of the same shared-memory location in the block of `rank`
__device__ __forceinline__ unsigned pl_map_rank(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void pl_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of one block of a pair; the bytes are counted on the barrier of the even block
__device__ __forceinline__ void pl_tma_load_pair(unsigned dst, const CUtensorMap* map, unsigned bar_cluster, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void pl_umma_pair(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrive, once the MMAs issued so far are complete, on the barrier at this offset in both blocks of the pair
__device__ __forceinline__ void pl_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void pl_tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
// bounded wait that also ends when another role of the block has given up
__device__ __forceinline__ bool pl_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < TC5_WAIT_LIMIT; ++i) {
        unsigned done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 0xFFF) == 0xFFF && *abort_flag) break;
    }
    *abort_flag = 1;
    return false;
}
// barrier of the four epilogue warps that also tells whether every thread brought `ok`
__device__ __forceinline__ bool pl_epi_all(bool ok) {
    unsigned r;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 q, %1, 0;\nbar.red.and.pred p, 1, %2, q;\nselp.b32 %0, 1, 0, p;\n}"
                 : "=r"(r) : "r"((unsigned)ok), "n"(PL_EPI_THREADS) : "memory");
    return r != 0;
}
__device__ __forceinline__ unsigned pl_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int BN, int PAIR>
__global__ void __launch_bounds__(PL_THREADS, 1)
prompt_linear_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const PlParams p) {
    using Cfg = PlCfg<BN, PAIR>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ unsigned char pl_smem_raw[];
    // (the same offset in both blocks of a pair: descriptors and barrier offsets are shared)
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pl_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_mem = base;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(base + (size_t)STAGES * Cfg::STAGE_BYTES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* colv = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 256);   // [2][256]: bias, next norm weight

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = PAIR == 2 ? pl_cluster_rank() : 0u;
    const bool leader = rank == 0;
    const int cluster_id = (int)blockIdx.x / PAIR, num_clusters = (int)gridDim.x / PAIR;
    const bool glu = p.epi == PL_EPI_SWIGLU;
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const unsigned accfull0 = smem_u32(bars + 2 * STAGES), accempty0 = smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(accfull0 + 8 * i, 1); mbar_init(accempty0 + 8 * i, PL_EPI_WARPS * PAIR); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc5_fence_before();
    __syncthreads();
    __syncwarp();
    if (PAIR == 2) pl_cluster_sync();          // the other block's barriers exist before anything arrives on them
    tc5_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_trigger();
    pdl_wait();                                // tokens, residual stream and partial sums are the predecessors' output

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer: this block's tokens and its share of the weight rows ----
            const unsigned full_leader0 = PAIR == 2 ? pl_map_rank(full0, 0) : full0;
            int it = 0;
            bool ok = true;
            for (int t = cluster_id; t < p.num_tiles && ok; t += num_clusters) {
                const int m_blk = t % p.num_m, n_blk = t / p.num_m;
                const int m0 = (m_blk * PAIR + (int)rank) * PL_BM;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!pl_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const unsigned a = smem_u32(stage_mem + (size_t)s * Cfg::STAGE_BYTES), b = a + PL_A_BYTES;
                    if (PAIR == 2) {
                        if (leader) mbar_expect_tx(full0 + 8 * s, 2 * Cfg::STAGE_BYTES);
                        const unsigned bar = full_leader0 + 8 * s;
                        pl_tma_load_pair(a, &tm_a, bar, kb * PL_BK, m0);
                        // columns [0, BN/2) are this pair's first half of the weight rows (SwiGLU: the gate rows),
                        // columns [BN/2, BN) the second half (the up rows): one half per block
                        const int wrow = glu ? (int)rank * p.ff + n_blk * (BN / 2) : n_blk * BN + (int)rank * (BN / 2);
                        pl_tma_load_pair(b, &tm_w, bar, kb * PL_BK, wrow);
                    } else {
                        mbar_expect_tx(full0 + 8 * s, Cfg::STAGE_BYTES);
                        tma_load_2d(a, &tm_a, full0 + 8 * s, kb * PL_BK, m0);
                        if (glu) {         // boxes of BN/2 rows: gate rows, then the matching up rows
                            tma_load_2d(b, &tm_w, full0 + 8 * s, kb * PL_BK, n_blk * (BN / 2));
                            tma_load_2d(b + Cfg::B_BYTES / 2, &tm_w, full0 + 8 * s, kb * PL_BK, p.ff + n_blk * (BN / 2));
                        } else {
                            tma_load_2d(b, &tm_w, full0 + 8 * s, kb * PL_BK, n_blk * BN);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---- MMA issue ----
            // instruction descriptor: float accumulate, bf16 x bf16, both K-major, N = BN, M = 128 a block
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)((PL_BM * PAIR) >> 4) << 24);
            int it = 0, tl = 0;
            bool ok = true;
            for (int t = cluster_id; t < p.num_tiles && ok; t += num_clusters, ++tl) {
                const int buf = tl & 1;
                if (!pl_wait(accempty0 + 8 * buf, ((tl >> 1) & 1) ^ 1, abort_flag)) break;     // the epilogues have read this buffer
                tc5_fence_after();
                const unsigned d = tmem_base + (unsigned)(buf * BN);
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!pl_wait(full0 + 8 * s, (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc5_fence_after();
                    const unsigned a = smem_u32(stage_mem + (size_t)s * Cfg::STAGE_BYTES), b = a + PL_A_BYTES;
#pragma unroll
                    for (int k = 0; k < PL_BK / 16; ++k) {
                        if (PAIR == 2) pl_umma_pair(d, umma_desc(a + k * 32), umma_desc(b + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else umma_f16(d, umma_desc(a + k * 32), umma_desc(b + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    if (PAIR == 2) pl_commit_pair(empty0 + 8 * s);      // the stage is free, in both blocks, once these MMAs have read it
                    else umma_commit(empty0 + 8 * s);
                }
                if (!ok) break;
                if (PAIR == 2) pl_commit_pair(accfull0 + 8 * buf);      // the accumulator is complete
                else umma_commit(accfull0 + 8 * buf);
            }
        }
    } else {
        // ---- epilogue: warps 2.., a warp for 32 tokens (and, with eight warps, one half of the tile's features) ----
        // A thread reads 32 columns of its token's row from tensor memory and finishes them (scale of a
        // deferred norm, bias, SwiGLU); the warp then turns the 32 x 32 patch round through shared memory
        // so that global memory is read and written in whole rows of the patch: 128 contiguous bytes of
        // float, 64 of bfloat16, by 8 or 4 neighbouring lanes.
        const int et = (int)threadIdx.x - 64;                           // 0..PL_EPI_THREADS-1
        const int quarter = warp & 3;                                   // the 32 tensor-memory lanes this warp may read
        const int half = (warp - 2) >> 2;                               // which part of the features
        const unsigned accempty_leader0 = PAIR == 2 ? pl_map_rank(accempty0, 0) : accempty0;
        float* patch = colv + 512 + (warp - 2) * 1024;                 // [32 tokens][32 columns], 16-byte pieces swizzled by the token
        const bool vec_out = (p.out_stride & 7) == 0;                   // 16-byte pieces of output rows are aligned
        const bool vec_res = (p.N & 7) == 0;
        constexpr int COLS = BN / PL_HALVES;                            // accumulator columns of this warp
        constexpr int GCOLS = BN / 2 / PL_HALVES;                       // SwiGLU: features of this warp
        auto put = [&](const float (&v)[32]) {                         // this thread's token, 32 columns
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(patch + lane * 32 + ((j ^ (lane & 7)) << 2)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        };
        auto get = [&](int r, int piece) {                             // columns 4 piece .. 4 piece + 3 of token r
            return *reinterpret_cast<const float4*>(patch + r * 32 + ((piece ^ (r & 7)) << 2));
        };
        const int r4 = lane >> 3, p4 = lane & 7;                        // float rows: 4 tokens an instruction, 8 lanes a token
        const int r8 = lane >> 2, p8 = lane & 3;                        // bfloat16 rows: 8 tokens an instruction, 4 lanes a token
        int tl = 0;
        for (int t = cluster_id; t < p.num_tiles; t += num_clusters, ++tl) {
            const int buf = tl & 1;
            const int m_blk = t % p.num_m, n_blk = t / p.num_m;
            const long long mw = (long long)(m_blk * PAIR + (int)rank) * PL_BM + quarter * 32;      // first token of this warp
            const long long m = mw + lane;
            const bool m_ok = m < p.M;
            const long long n0 = glu ? (long long)n_blk * (BN / 2) : (long long)n_blk * BN;      // first feature of the tile
            float scale = 1.f;
            if (p.pro == PL_PRO_NORM && m_ok) {
                float s = 0.f;
                for (int i = 0; i < p.ss_parts; ++i) s += p.ss_in[(size_t)i * p.M + m];
                scale = rsqrtf(s / (float)p.K + p.eps);
            }
            pl_epi_bar();                                               // the previous tile's column vectors are no longer read
            for (int j = et; j < BN; j += PL_EPI_THREADS) {
                const long long n = n0 + j;
                colv[j] = (p.bias && !glu && n < p.N) ? p.bias[n] : 0.f;
                colv[256 + j] = (p.next_w && n < p.N) ? p.next_w[n] : 0.f;
            }
            // (the warps leave together or not at all: they meet at barriers in every tile)
            if (!pl_epi_all(pl_wait(accfull0 + 8 * buf, (tl >> 1) & 1, abort_flag))) break;
            tc5_fence_after();
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN);
            // 32 finished columns of bfloat16 output, from the patch, as rows of 64 bytes
            auto store_bf16_rows = [&](__nv_bfloat16* out, long long stride, long long f0, long long limit) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = i * 8 + r8;
                    const long long f = f0 + p8 * 8;
                    if (mw + r < p.M && f + 7 < limit) {
                        const float4 a = get(r, 2 * p8), b = get(r, 2 * p8 + 1);
                        *reinterpret_cast<uint4*>(out + (size_t)(mw + r) * stride + f) =
                            make_uint4(pl_pack(a.x, a.y), pl_pack(a.z, a.w), pl_pack(b.x, b.y), pl_pack(b.z, b.w));
                    }
                }
            };

            if (glu) {
#pragma unroll 1
                for (int c = half * GCOLS; c < (half + 1) * GCOLS; c += 32) {
                    const long long f0 = n0 + c;
                    if (f0 >= p.ff) break;
                    unsigned g[32], u[32];
                    pl_tmem_ld32(taddr + c, g);
                    pl_tmem_ld32(taddr + BN / 2 + c, u);
                    tmem_ld_wait();
                    float sv[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float gv = __uint_as_float(g[j]) * scale, uv = __uint_as_float(u[j]) * scale;
                        // (fast exponential and division: their error is far below the bfloat16 rounding of the result)
                        sv[j] = __fdividef(gv, 1.f + __expf(-gv)) * uv;
                    }
                    if (vec_out && f0 + 31 < p.ff) {
                        put(sv);
                        __syncwarp();
                        store_bf16_rows(p.out_bf16, p.out_stride, f0, p.ff);
                        __syncwarp();
                    } else if (m_ok) {
                        __nv_bfloat16* orow = p.out_bf16 + (size_t)m * p.out_stride;
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (f0 + j < p.ff) orow[f0 + j] = __float2bfloat16_rn(sv[j]);
                    }
                }
            } else {
                float ssq[8];                                           // residual epilogue: tokens 4 i + r4 of this warp
#pragma unroll
                for (int i = 0; i < 8; ++i) ssq[i] = 0.f;
                float ssq_row = 0.f;                                    // the same for rows that are not 16-byte aligned: this thread's token
#pragma unroll 1
                for (int c = half * COLS; c < (half + 1) * COLS; c += 32) {
                    const long long f0 = n0 + c;
                    if (f0 >= p.N) break;
                    unsigned r[32];
                    pl_tmem_ld32(taddr + c, r);
                    const bool full = f0 + 31 < p.N;
                    const bool fast = full && (p.epi == PL_EPI_RESID ? vec_res : vec_out);
                    // the stream's old values, on their way while the sums are finished and turned round
                    float4 old[8];
                    if (p.epi == PL_EPI_RESID && fast) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const long long mr = mw + i * 4 + r4;
                            old[i] = mr < p.M ? *reinterpret_cast<const float4*>(p.resid + (size_t)mr * p.N + f0 + p4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * scale + colv[c + j];
                    if (fast) {
                        put(v);
                        __syncwarp();
                        if (p.epi == PL_EPI_BF16) {
                            store_bf16_rows(p.out_bf16, p.out_stride, f0, p.N);
                        } else if (p.epi == PL_EPI_F32) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const long long mr = mw + i * 4 + r4;
                                if (mr < p.M) *reinterpret_cast<float4*>(p.out_f32 + (size_t)mr * p.out_stride + f0 + p4 * 4) = get(i * 4 + r4, p4);
                            }
                        } else {
                            const float4 nw = *reinterpret_cast<const float4*>(colv + 256 + c + p4 * 4);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const long long mr = mw + i * 4 + r4;
                                if (mr < p.M) {
                                    float4 a = get(i * 4 + r4, p4);
                                    a.x += old[i].x; a.y += old[i].y; a.z += old[i].z; a.w += old[i].w;
                                    const size_t at = (size_t)mr * p.N + f0 + p4 * 4;
                                    *reinterpret_cast<float4*>(p.resid + at) = a;
                                    ssq[i] += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                                    if (p.xw_out)
                                        *reinterpret_cast<uint2*>(p.xw_out + at) = make_uint2(pl_pack(a.x * nw.x, a.y * nw.y), pl_pack(a.z * nw.z, a.w * nw.w));
                                }
                            }
                        }
                        __syncwarp();
                    } else if (m_ok) {                                  // a ragged edge or unaligned rows: this thread's token, value by value
                        if (p.epi == PL_EPI_BF16) {
                            __nv_bfloat16* o = p.out_bf16 + (size_t)m * p.out_stride + f0;
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (f0 + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
                        } else if (p.epi == PL_EPI_F32) {
                            float* o = p.out_f32 + (size_t)m * p.out_stride + f0;
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (f0 + j < p.N) o[j] = v[j];
                        } else {
                            float* x = p.resid + (size_t)m * p.N + f0;
                            __nv_bfloat16* o = p.xw_out ? p.xw_out + (size_t)m * p.N + f0 : nullptr;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (f0 + j < p.N) {
                                    const float nv = v[j] + x[j];
                                    x[j] = nv;
                                    ssq_row += nv * nv;
                                    if (o) o[j] = __float2bfloat16_rn(nv * colv[256 + c + j]);
                                }
                            }
                        }
                    }
                }
                if (p.epi == PL_EPI_RESID && p.ss_out) {
                    // a token's sum lies in the 8 lanes that shared its rows, and (ragged edges) in the token's own thread
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float q = ssq[i];
                        q += __shfl_xor_sync(0xffffffffu, q, 1);
                        q += __shfl_xor_sync(0xffffffffu, q, 2);
                        q += __shfl_xor_sync(0xffffffffu, q, 4);
                        ssq[i] = q;
                    }
                    // token `lane` = 4 i + r4 with i = lane / 4, r4 = lane % 4: its sum is ssq[lane / 4] of the lanes 8 (lane % 4) ..
                    float mine = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float q = __shfl_sync(0xffffffffu, ssq[i], (lane & 3) * 8);
                        if ((lane >> 2) == i) mine = q;
                    }
                    if (m_ok) p.ss_out[((size_t)n_blk * PL_HALVES + half) * p.M + m] = mine + ssq_row;
                }
            }
            // this warp has read its part of the accumulator: hand the buffer back to the MMA issuer
            tc5_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR == 2) pl_arrive_cluster(accempty_leader0 + 8 * buf);
                else mbar_arrive(accempty0 + 8 * buf);
            }
        }
    }

    tc5_fence_before();
    __syncthreads();
    __syncwarp();
    if (PAIR == 2) pl_cluster_sync();          // nothing of the other block touches this block's memory any more
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 16);
    if (warp == 1) {
        __syncwarp();
        tc5_fence_after();
        if (PAIR == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------
// a [rows][K] bfloat16 matrix, K contiguous, tiled in boxes of 64 k x box_rows rows, 128-byte swizzle;
// encoded once per (address, shape, box) and thread
static int pl_map(const CUtensorMap** out, const void* ptr, long long rows, long long K, int box_rows) {
    struct Key {
        const void* p; long long r, k; int b;
        bool operator==(const Key& o) const { return p == o.p && r == o.r && k == o.k && b == o.b; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.r) * 31) ^ (std::hash<long long>()(k.k) * 131) ^ (size_t)k.b;
        }
    };
    static thread_local std::unordered_map<Key, CUtensorMap, Hash> cache;
    const Key key{ptr, rows, K, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = &it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(-102, "prompt_linear: cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)ptr & 15) != 0 || (K * 2) % 16 != 0)
        return fail(-1, "prompt_linear: operand address or row pitch is not 16-byte aligned (K=%lld)", K);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)PL_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(-103, "prompt_linear: cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    *out = &cache.emplace(key, map).first->second;
    return 0;
}

template <int BN, int PAIR>
static int launch_pl(const CUtensorMap& ta, const CUtensorMap& tw, const PlParams& p, cudaStream_t stream) {
    using Cfg = PlCfg<BN, PAIR>;
    auto kern = prompt_linear_kernel<BN, PAIR>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return fail(-101, "prompt_linear: cannot reserve %zu bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
        attr_done = true;
    }
    int clusters = sm_count() / PAIR;
    if (clusters > p.num_tiles) clusters = p.num_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * PAIR);
    cfg.blockDim = dim3(PL_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (PAIR == 2) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 2;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return check_launch("prompt_linear", cudaLaunchKernelEx(&cfg, kern, ta, tw, p));
}

static int pl_env(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

// How a call is cut: features a tile, blocks a tile (1 or 2), tiles along the features (= partial
// sums of squares per token that a residual epilogue leaves).
static int pl_force_bn = -1, pl_force_pair = -1;       // -1: read VAPI_PL_BN / VAPI_PL_PAIR at the first call; 0: choose

// Fix the tile's features (128 | 256) and the blocks a tile (1 | 2) for the calls that follow; 0 lets the plan choose.
VAPI_EXPORT int vapi_prompt_linear_force(int bn, int pair) {
    if ((bn != 0 && bn != 128 && bn != 256) || pair < 0 || pair > 2) return fail(-1, "prompt_linear: no tiles of %d features on %d blocks", bn, pair);
    pl_force_bn = bn; pl_force_pair = pair;
    return 0;
}

// How a call is cut: features a tile, blocks a tile (1 or 2), tiles along the features (= partial
// sums of squares per token that a residual epilogue leaves).
VAPI_EXPORT int vapi_prompt_linear_plan(int N, int K, int M, int epi, int* bn, int* pair, int* parts) {
    if (pl_force_bn < 0) { pl_force_bn = pl_env("VAPI_PL_BN", 0); pl_force_pair = pl_env("VAPI_PL_PAIR", 0); }
    const int cols = epi == PL_EPI_SWIGLU ? N / 2 : N;            // output features
    const int pr = pl_force_pair ? pl_force_pair : (M > PL_BM ? 2 : 1);
    // 256 features a tile: tiles of 128 keep more multiprocessors busy in a last round, but every operand byte then
    // crosses from L2 twice as often for the same arithmetic, which costs more than the idle blocks (measured)
    const int b = pl_force_bn ? pl_force_bn : 256;
    const int per = epi == PL_EPI_SWIGLU ? b / 2 : b;
    *bn = b; *pair = pr; *parts = ((cols + per - 1) / per) * (epi == PL_EPI_RESID ? PL_HALVES : 1);
    return 0;
}

VAPI_EXPORT int vapi_prompt_linear(const void* W, int N, int K, int M, int pro, const void* tokens,
                                   const float* ss_in, int ss_parts, float eps, int epi, void* out_bf16,
                                   float* out_f32, long long out_stride, const float* bias, float* resid,
                                   float* ss_out, const float* next_w, void* xw_out, int* status,
                                   cudaStream_t stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0 || K % 8 != 0) return fail(-1, "prompt_linear: K=%d must be a positive multiple of 8 (N=%d)", K, N);
    if (epi == PL_EPI_SWIGLU && N % 2 != 0) return fail(-1, "prompt_linear: SwiGLU needs an even N");
    if (!tokens) return fail(-1, "prompt_linear: no token operand");
    if (pro == PL_PRO_NORM && (!ss_in || ss_parts <= 0)) return fail(-1, "prompt_linear: the deferred norm needs partial sums");
    if ((epi == PL_EPI_BF16 || epi == PL_EPI_SWIGLU) && !out_bf16) return fail(-1, "prompt_linear: no output");
    if (epi == PL_EPI_F32 && !out_f32) return fail(-1, "prompt_linear: no output");
    if (epi == PL_EPI_RESID && !resid) return fail(-1, "prompt_linear: no residual stream");
    if (xw_out && !next_w) return fail(-1, "prompt_linear: a weighted copy of the stream needs the next norm's weight");
    if (((uintptr_t)out_bf16 & 15) || ((uintptr_t)out_f32 & 15) || ((uintptr_t)resid & 15) || ((uintptr_t)xw_out & 15))
        return fail(-1, "prompt_linear: outputs must be 16-byte aligned");
    int bn, pair, parts;
    vapi_prompt_linear_plan(N, K, M, epi, &bn, &pair, &parts);
    PlParams p;
    p.N = N; p.K = K; p.M = M; p.epi = epi; p.pro = pro; p.ff = N / 2;
    p.num_kb = (K + PL_BK - 1) / PL_BK;
    p.num_m = (M + PL_BM * pair - 1) / (PL_BM * pair);
    p.num_n = epi == PL_EPI_RESID ? parts / PL_HALVES : parts;
    p.num_tiles = p.num_m * p.num_n;
    p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps;
    p.out_bf16 = (__nv_bfloat16*)out_bf16; p.out_f32 = out_f32; p.out_stride = out_stride; p.bias = bias;
    p.resid = resid; p.ss_out = ss_out; p.next_w = next_w; p.xw_out = (__nv_bfloat16*)xw_out;
    p.status = status;
    const bool half_rows = epi == PL_EPI_SWIGLU || pair == 2;      // boxes of BN/2 weight rows
    const CUtensorMap *ta, *tw;
    int rc = pl_map(&ta, tokens, M, K, PL_BM);
    if (rc) return rc;
    rc = pl_map(&tw, W, N, K, half_rows ? bn / 2 : bn);
    if (rc) return rc;
    if (bn == 256 && pair == 2) return launch_pl<256, 2>(*ta, *tw, p, stream);
    if (bn == 128 && pair == 2) return launch_pl<128, 2>(*ta, *tw, p, stream);
    if (bn == 256 && pair == 1) return launch_pl<256, 1>(*ta, *tw, p, stream);
    if (bn == 128 && pair == 1) return launch_pl<128, 1>(*ta, *tw, p, stream);
    return fail(-2, "prompt_linear: no kernel for tiles of %d features and %d blocks", bn, pair);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
