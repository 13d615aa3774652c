// Matrix product for steps of 17 .. 256 rows (decode at batch 32 / 64, short prompt portions):
//   y[m][n] = sum_k a[m][k] * W[n][k],  bfloat16 in, float accumulate,
// on the fifth-generation tensor cores: tcgen05.mma issued by one thread, operands brought into
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), accumulators in tensor memory,
// read back with tcgen05.ld for a fused epilogue.
//
// Orientation.  The weight is the 128-row operand (MMA M = 128 weight rows of a tile), the tokens
// are the narrow operand (MMA N = BN = 32 .. 256 tokens, rows beyond M zero-filled by TMA), so
// a small batch does not waste the tensor core's fixed M and every weight byte is read once.
// A block owns one tile of 128 weight rows (for SwiGLU: 64 gate rows and the 64 matching up
// rows) and a slice of K.  When N is small there are too few tiles for the device's multiprocessors, so K is cut
// into up to 8 slices whose blocks form a thread-block cluster: each block leaves its partial
// tile in its own shared memory, and after a cluster barrier every block sums, for its share
// of the tokens, the partials of all blocks through distributed shared memory in rank order
// (no scratch in global memory, no atomics, a sum that does not depend on timing).
//
// Roles.  Warp 0 (one lane): TMA producer over a ring of shared-memory stages; weights of the
// first stages are requested before griddepcontrol.wait, activations after it.  Warp 1: tensor
// memory allocation, and (one lane) the MMA issue loop; tcgen05.commit hands a stage back to
// the producer and, at the end, the accumulator to the epilogue.  Warps 2-5: epilogue, one
// weight row per thread: bfloat16 out | float out | SwiGLU | add into the float residual stream
// with what the next norm needs (partial sums of squares, bfloat16(stream * next norm weight)).
// The token operand may be the residual stream seen through a deferred RMSNorm (see gemv.cu):
// then the epilogue scales every token's column by rsqrt(mean x^2 + eps).
//
// Every mbarrier wait is bounded: after TC_WAIT_LIMIT polls a role gives up, records status
// 16 and the block drains to its end (tensor memory is released on every path; the cluster
// barriers are hardware barriers that every thread reaches on every path).
#include "tcgen05.cuh"

using namespace vapi;

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int TC_THREADS = 192;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;

enum { TC_PRO_ACT = 0, TC_PRO_NORM = 1 };
enum { TC_EPI_BF16 = 0, TC_EPI_SWIGLU = 1, TC_EPI_RESID = 2, TC_EPI_F32 = 3 };

struct TcParams {
    int N, K, M, epi, pro, ff;
    int num_kb, kb_per_split, splits;
    const float* ss_in; int ss_parts; float eps;
    __nv_bfloat16* out_bf16; float* out_f32; long long out_stride;
    const float* bias; float* resid; float* ss_out; const float* next_w; __nv_bfloat16* xw_out;
    int* status;
};

template <int BN> struct TcCfg {
    static constexpr int STAGE_BYTES = TC_A_BYTES + BN * TC_BK * 2;
    static constexpr int STAGES_RAW = (96 * 1024) / STAGE_BYTES;             // two blocks fit on an SM
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + 4 * 256 * 4 /*sums*/ + 256 * 4;
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(unsigned local_smem_addr, unsigned rank) {
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 2)
linear_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a, const TcParams p) {
    using Cfg = TcCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_mem = base;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(base + (size_t)STAGES * Cfg::STAGE_BYTES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 1);
    int* flags = reinterpret_cast<int*>(tmem_slot + 1);           // [0] a bounded wait ran out
    float* sums = reinterpret_cast<float*>(bars) + 64;            // [4][256] partial sums of squares
    float* inv_s = sums + 4 * 256;                                 // [256]
    float* part_s = reinterpret_cast<float*>(stage_mem);          // after the main loop: [BN][128] partial tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, sp = blockIdx.y;                  // sp is also the rank in the cluster
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), accbar = smem_u32(bars + 2 * STAGES);
    const int kb0 = sp * p.kb_per_split;
    const int nkb = max(0, min(p.num_kb, kb0 + p.kb_per_split) - kb0);
    const bool glu = p.epi == TC_EPI_SWIGLU;
    // rows of the tile: 128 weight rows, or 64 gate rows (MMA rows 0..63) + the 64 up rows (64..127)
    const int n0 = glu ? tile * 64 : tile * TC_BM;

    auto load_weights = [&](unsigned a, unsigned bar, int kb) {
        if (glu) {      // tm_w has boxes of 64 rows here
            tma_load_2d(a, &tm_w, bar, kb * TC_BK, n0);
            tma_load_2d(a + TC_A_BYTES / 2, &tm_w, bar, kb * TC_BK, p.ff + n0);
        } else {
            tma_load_2d(a, &tm_w, bar, kb * TC_BK, n0);
        }
    };

    pdl_trigger();
    const int pre = min(STAGES, nkb);
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
        mbar_init(accbar, 1);
        flags[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The weights depend on nothing that runs before this kernel: request the first stages
        // right away, before tensor memory is even allocated (this thread is the producer).
        for (int i = 0; i < pre; ++i) {
            mbar_expect_tx(full0 + 8 * i, Cfg::STAGE_BYTES);
            load_weights(smem_u32(stage_mem + (size_t)i * Cfg::STAGE_BYTES), full0 + 8 * i, kb0 + i);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            pdl_wait();                                             // the activations are the predecessor's output
            for (int i = 0; i < pre; ++i)
                tma_load_2d(smem_u32(stage_mem + (size_t)i * Cfg::STAGE_BYTES) + TC_A_BYTES, &tm_a, full0 + 8 * i, (kb0 + i) * TC_BK, 0);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(empty0 + 8 * s, ((i / STAGES) & 1) ^ 1)) { flags[0] = 1; break; }
                const unsigned a = smem_u32(stage_mem + (size_t)s * Cfg::STAGE_BYTES);
                mbar_expect_tx(full0 + 8 * s, Cfg::STAGE_BYTES);
                load_weights(a, full0 + 8 * s, kb0 + i);
                tma_load_2d(a + TC_A_BYTES, &tm_a, full0 + 8 * s, (kb0 + i) * TC_BK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issue ----
            // instruction descriptor: float accumulate, bf16 x bf16, both K-major, N = BN, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(full0 + 8 * s, (i / STAGES) & 1)) { flags[0] = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned a = smem_u32(stage_mem + (size_t)s * Cfg::STAGE_BYTES);
                const unsigned b = a + TC_A_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    umma_f16(tmem_base, umma_desc(a + k * 32), umma_desc(b + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);                        // the stage is free once these MMAs have read it
            }
            umma_commit(accbar);                                    // the accumulator is complete
        }
    }

    // ---- epilogue: warps 2..5, one weight row per thread ----
    const bool epi_warp = warp >= 2;
    const int et = threadIdx.x - 64;                                // 0..127 in epilogue warps
    const int quarter = warp & 3;                                   // the 32 tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;                            // MMA row
    const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
    // the output feature of this row: for SwiGLU rows 0..63 are gate rows of feature n0 + row,
    // rows 64..127 the up rows of feature n0 + row - 64
    const long long n = glu ? (long long)n0 + (row & 63) : (long long)n0 + row;
    const bool row_ok = glu ? n < p.ff : n < p.N;
    bool ok = true;

    // Phase A (one weight row per thread): the finished sums over K, scaled for a deferred norm
    // and with the bias, go to shared memory as [token][128 rows].  Phase B (one warp per token,
    // lanes across the features): coalesced 16-byte traffic to global memory with the epilogue's
    // arithmetic.  `fin` aliases the stages, which are idle once the accumulator is complete.
    float* fin = part_s;
    auto finish = [&](int slot, float v, int m) {                  // phase A for token m, kept in `slot`
        if (p.pro == TC_PRO_NORM) v *= inv_s[m];
        if (!glu && p.bias && row_ok) v += p.bias[n];
        fin[slot * TC_BM + row] = v;
    };
    auto store_token = [&](int slot, int m) {                      // phase B for token m, whole warp
        const float* f = fin + slot * TC_BM;
        if (glu) {
            // 64 features: gate in rows 0..63, up in rows 64..127; two features per lane
            const long long f0 = (long long)n0 + 2 * lane;
            const float g0 = f[2 * lane], g1 = f[2 * lane + 1], u0 = f[64 + 2 * lane], u1 = f[64 + 2 * lane + 1];
            // (fast exponential and division: their error is far below the bfloat16 rounding of the result)
            const float s0 = __fdividef(g0, 1.f + __expf(-g0)) * u0, s1 = __fdividef(g1, 1.f + __expf(-g1)) * u1;
            __nv_bfloat16* o = p.out_bf16 + (size_t)m * p.out_stride + f0;
            if (f0 + 1 < p.ff && (p.out_stride & 1) == 0) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(s0, s1);
            else {
                if (f0 < p.ff) o[0] = __float2bfloat16_rn(s0);
                if (f0 + 1 < p.ff) o[1] = __float2bfloat16_rn(s1);
            }
            return;
        }
        const long long f0 = (long long)n0 + 4 * lane;             // four features per lane
        const float4 v = *reinterpret_cast<const float4*>(f + 4 * lane);
        const float vv[4] = {v.x, v.y, v.z, v.w};
        const bool full = f0 + 3 < p.N;
        if (p.epi == TC_EPI_BF16) {
            __nv_bfloat16* o = p.out_bf16 + (size_t)m * p.out_stride + f0;
            if (full && (p.out_stride & 3) == 0) {
                uint2 pk;
                __nv_bfloat162 a = __floats2bfloat162_rn(vv[0], vv[1]), b = __floats2bfloat162_rn(vv[2], vv[3]);
                pk.x = *reinterpret_cast<unsigned*>(&a); pk.y = *reinterpret_cast<unsigned*>(&b);
                *reinterpret_cast<uint2*>(o) = pk;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (f0 + i < p.N) o[i] = __float2bfloat16_rn(vv[i]);
            }
        } else if (p.epi == TC_EPI_F32) {
            float* o = p.out_f32 + (size_t)m * p.out_stride + f0;
            if (full && (p.out_stride & 3) == 0) *reinterpret_cast<float4*>(o) = v;
            else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (f0 + i < p.N) o[i] = vv[i];
            }
        } else {                                                   // add into the residual stream
            float* x = p.resid + (size_t)m * p.N + f0;
            float nv[4] = {0.f, 0.f, 0.f, 0.f};
            if (full && (p.N & 3) == 0) {
                const float4 old = *reinterpret_cast<const float4*>(x);
                nv[0] = old.x + vv[0]; nv[1] = old.y + vv[1]; nv[2] = old.z + vv[2]; nv[3] = old.w + vv[3];
                *reinterpret_cast<float4*>(x) = make_float4(nv[0], nv[1], nv[2], nv[3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (f0 + i < p.N) { nv[i] = x[i] + vv[i]; x[i] = nv[i]; }
            }
            if (p.xw_out) {
                __nv_bfloat16* o = p.xw_out + (size_t)m * p.N + f0;
#pragma unroll
                for (int i = 0; i < 4; ++i) if (f0 + i < p.N) o[i] = __float2bfloat16_rn(nv[i] * p.next_w[f0 + i]);
            }
            if (p.ss_out) {
                const float sq = warp_sum(nv[0] * nv[0] + nv[1] * nv[1] + nv[2] * nv[2] + nv[3] * nv[3]);
                if (lane == 0) p.ss_out[(size_t)tile * p.M + m] = sq;
            }
        }
    };

    if (epi_warp) {
        pdl_wait();
        if (p.pro == TC_PRO_NORM) {
            for (int m = et; m < p.M; m += 128) {
                float s = 0.f;
                for (int i = 0; i < p.ss_parts; ++i) s += p.ss_in[(size_t)i * p.M + m];
                inv_s[m] = rsqrtf(s / (float)p.K + p.eps);
            }
        }
        epi_bar();
        ok = mbar_wait(accbar, 0);
        if (!ok) flags[0] = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // the accumulator (this block's sum over its slice of K) into shared memory: [token][row].
        // Without slices of K the tokens are finished right here, at most 128 at a time (what
        // the idle stages hold), each group followed by its phase B.
        constexpr int GROUP = BN < 128 ? BN : 128;
        for (int g0 = 0; g0 < BN; g0 += GROUP) {
            if (g0 >= p.M) break;
            for (int c0 = g0; c0 < g0 + GROUP; c0 += 16) {
                if (c0 >= p.M) break;                                // uniform: tokens beyond M are padding
                float y[16];
                tmem_ld16(taddr + c0, y);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (p.splits == 1) { if (c0 + j < p.M) finish(c0 + j - g0, y[j], c0 + j); }
                    else part_s[(c0 + j) * TC_BM + row] = y[j];
                }
            }
            if (p.splits == 1) {
                epi_bar();
#pragma unroll 4
                for (int m = g0 + warp - 2; m < min(p.M, g0 + GROUP); m += 4) store_token(m - g0, m);
                epi_bar();
            }
        }
    }
    if (p.splits > 1) {
        cluster_sync_all();                                          // every block's partial tile is in place
        if (epi_warp) {
            // token m belongs to the block of rank m % splits; partials are added in rank order.
            // Remote shared memory is far away: fetch the partials of eight tokens from every
            // rank first, then add them.  The sums replace this block's own partials of its tokens
            // (which no other block reads).
            for (int m0 = sp; m0 < p.M; m0 += 8 * p.splits) {
                float part[8][8];
#pragma unroll
                for (int t8 = 0; t8 < 8; ++t8) {
                    const int m = m0 + t8 * p.splits;
                    const unsigned a = smem_u32(part_s + (m < p.M ? m : 0) * TC_BM + row);
#pragma unroll
                    for (int r = 0; r < 8; ++r) part[t8][r] = (m < p.M && r < p.splits) ? ld_cluster_f32(a, (unsigned)r) : 0.f;
                }
#pragma unroll
                for (int t8 = 0; t8 < 8; ++t8) {
                    const int m = m0 + t8 * p.splits;
                    if (m < p.M) {
                        float v = 0.f;
#pragma unroll
                        for (int r = 0; r < 8; ++r) v += part[t8][r];
                        finish(m, v, m);
                    }
                }
            }
        }
    }
    if (epi_warp && p.splits > 1) {
        epi_bar();                                                   // phase A is complete for this block's tokens
        for (int i = warp - 2; sp + i * p.splits < p.M; i += 4) store_token(sp + i * p.splits, sp + i * p.splits);
    }
    if (p.splits > 1) cluster_sync_all();                            // nobody reads this block's memory any more

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && flags[0] && p.status) atomicExch(p.status, 16);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------
// a [rows][K] bfloat16 matrix, K contiguous, tiled in boxes of 64 k x box_rows rows, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(-102, "linear_tc: cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)ptr & 15) != 0 || (K * 2) % 16 != 0)
        return fail(-1, "linear_tc: operand address or row pitch is not 16-byte aligned (K=%lld)", K);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(-103, "linear_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

template <int BN>
static int launch_tc(const CUtensorMap& tw, const CUtensorMap& ta, const TcParams& p, int tiles, cudaStream_t stream) {
    using Cfg = TcCfg<BN>;
    auto kern = linear_tc_kernel<BN>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return fail(-101, "linear_tc: cannot reserve %zu bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, p.splits);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.splits > 1) {                      // the slices of K of one tile form a cluster
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = p.splits;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return check_launch("linear_tc", cudaLaunchKernelEx(&cfg, kern, tw, ta, p));
}

// How a call is cut: tiles of weight rows, slices of K (= cluster size), tokens per tile.
VAPI_EXPORT int vapi_linear_tc_plan(int N, int K, int M, int epi, int* tiles, int* splits, int* bn) {
    const int t = epi == TC_EPI_SWIGLU ? (N / 2 + 63) / 64 : (N + TC_BM - 1) / TC_BM;
    int b = 32;
    while (b < M) b *= 2;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    int s = 1;
    const int sms = sm_count();
    if (3 * t <= 2 * sms && b <= 128) {               // too few tiles for the multiprocessors: cut K (partials must fit the stages)
        s = sms / t;
        if (s > 8) s = 8;                            // portable cluster size
        const int max_s = num_kb / 2 > 0 ? num_kb / 2 : 1;      // at least 2 k-blocks a slice
        if (s > max_s) s = max_s;
        if (s < 1) s = 1;
        const int per = (num_kb + s - 1) / s;
        s = (num_kb + per - 1) / per;                // no empty slice
    }
    *tiles = t; *splits = s; *bn = b;
    return 0;
}

VAPI_EXPORT int vapi_linear_tc(const void* W, int N, int K, int M, int pro, const void* tokens,
                               const float* ss_in, int ss_parts, float eps, int epi, void* out_bf16,
                               float* out_f32, long long out_stride, const float* bias, float* resid,
                               float* ss_out, const float* next_w, void* xw_out, int* status,
                               cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 256) return fail(-1, "linear_tc: %d rows are more than 256", M);
    if (N <= 0 || K <= 0 || K % 8 != 0) return fail(-1, "linear_tc: K=%d must be a positive multiple of 8 (N=%d)", K, N);
    if (epi == TC_EPI_SWIGLU && N % 2 != 0) return fail(-1, "linear_tc: SwiGLU needs an even N");
    if (!tokens) return fail(-1, "linear_tc: no token operand");
    if (pro == TC_PRO_NORM && (!ss_in || ss_parts <= 0)) return fail(-1, "linear_tc: the deferred norm needs partial sums");
    if ((epi == TC_EPI_BF16 || epi == TC_EPI_SWIGLU) && !out_bf16) return fail(-1, "linear_tc: no output");
    if (epi == TC_EPI_F32 && !out_f32) return fail(-1, "linear_tc: no output");
    if (epi == TC_EPI_RESID && !resid) return fail(-1, "linear_tc: no residual stream");
    if (xw_out && !next_w) return fail(-1, "linear_tc: a weighted copy of the stream needs the next norm's weight");
    int tiles, splits, bn;
    vapi_linear_tc_plan(N, K, M, epi, &tiles, &splits, &bn);
    TcParams p;
    p.N = N; p.K = K; p.M = M; p.epi = epi; p.pro = pro; p.ff = N / 2;
    p.num_kb = (K + TC_BK - 1) / TC_BK; p.splits = splits; p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps;
    p.out_bf16 = (__nv_bfloat16*)out_bf16; p.out_f32 = out_f32; p.out_stride = out_stride; p.bias = bias;
    p.resid = resid; p.ss_out = ss_out; p.next_w = next_w; p.xw_out = (__nv_bfloat16*)xw_out;
    p.status = status;
    CUtensorMap tw, ta;
    int rc = make_map(&tw, W, N, K, epi == TC_EPI_SWIGLU ? 64 : TC_BM);
    if (rc) return rc;
    rc = make_map(&ta, tokens, M, K, bn);
    if (rc) return rc;
    switch (bn) {
        case 32: return launch_tc<32>(tw, ta, p, tiles, stream);
        case 64: return launch_tc<64>(tw, ta, p, tiles, stream);
        case 128: return launch_tc<128>(tw, ta, p, tiles, stream);
        case 256: return launch_tc<256>(tw, ta, p, tiles, stream);
    }
    return fail(-2, "linear_tc: no kernel for %d tokens", bn);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
