// Matrix product for steps of 17 .. 256 rows (decode at batch 32 / 64, short prompt portions):
//   y[m][n] = sum_k a[m][k] * W[n][k],  bfloat16 in, float accumulate,
// on the fifth-generation tensor cores: tcgen05.mma issued by one thread, operands brought into
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), accumulators in tensor memory,
// read back with tcgen05.ld for a fused epilogue.
//
// Orientation.  The weight is the 128-row operand (MMA M = 128 weight rows of a tile), the tokens
// are the narrow operand (MMA N = BN = 32 .. 256 tokens, rows beyond M zero-filled by TMA), so
// a small batch does not waste the tensor core's fixed M and every weight byte is read once.
// A block owns one tile of 128 weight rows (for SwiGLU: 128 gate rows and the 128 matching up
// rows, two accumulators) and a slice of K; slices of K of one tile (split-K, to give all SMs
// work when N is small) meet in scratch memory, and the block that arrives last adds them in
// slice order, so the sum does not depend on which block that is.
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
// 16 and the block drains to its end (tensor memory is released on every path).
#include "common.cuh"
#include <cuda.h>

using namespace vapi;

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int TC_THREADS = 192;
constexpr unsigned TC_WAIT_LIMIT = 1u << 24;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;

enum { TC_PRO_ACT = 0, TC_PRO_NORM = 1 };
enum { TC_EPI_BF16 = 0, TC_EPI_SWIGLU = 1, TC_EPI_RESID = 2, TC_EPI_F32 = 3 };

struct TcParams {
    int N, K, M, epi, pro, ff;
    int num_kb, kb_per_split, splits;
    const float* ss_in; int ss_parts; float eps;
    __nv_bfloat16* out_bf16; float* out_f32; long long out_stride;
    const float* bias; float* resid; float* ss_out; const float* next_w; __nv_bfloat16* xw_out;
    float* scratch; unsigned* counters;
    int* status;
};

template <int BN, int NACC> struct TcCfg {
    static constexpr int STAGE_BYTES = NACC * TC_A_BYTES + BN * TC_BK * 2;
    static constexpr int STAGES_RAW = (180 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);
    static constexpr int TMEM_COLS = NACC * BN < 32 ? 32 : NACC * BN;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + 4 * 256 * 4 /*sums*/ + 256 * 4;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait on a phase parity; false when the limit ran out
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned i = 0; i < TC_WAIT_LIMIT; ++i) {
        unsigned done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// shared-memory matrix descriptor: K-major tile of rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr >> 4) & 0x3FFF);        // start address
    d |= (unsigned long long)1 << 16;                             // leading byte offset (unused with swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                   // stride byte offset: 8 rows * 128 B
    d |= (unsigned long long)1 << 46;                             // descriptor version of this architecture
    d |= (unsigned long long)2 << 61;                             // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_f16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN, int NACC>
__global__ void __launch_bounds__(TC_THREADS, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a, const TcParams p) {
    using Cfg = TcCfg<BN, NACC>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_mem = base;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(base + (size_t)STAGES * Cfg::STAGE_BYTES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 1);
    int* flags = reinterpret_cast<int*>(tmem_slot + 1);           // [0] abort, [1] last arriver
    float* sums = reinterpret_cast<float*>(bars) + 64;            // [4][256] partial sums of squares
    float* inv_s = sums + 4 * 256;                                 // [256]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, sp = blockIdx.y;
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), accbar = smem_u32(bars + 2 * STAGES);
    const int kb0 = sp * p.kb_per_split;
    const int nkb = max(0, min(p.num_kb, kb0 + p.kb_per_split) - kb0);
    const int n0 = tile * TC_BM;                                   // first weight row (gate row for SwiGLU)

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
        mbar_init(accbar, 1);
        flags[0] = 0; flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
            const int pre = min(STAGES, nkb);
            for (int i = 0; i < pre; ++i) {                         // weights first: they depend on nothing
                const unsigned a = smem_u32(stage_mem + (size_t)i * Cfg::STAGE_BYTES);
                mbar_expect_tx(full0 + 8 * i, Cfg::STAGE_BYTES);
                tma_load_2d(a, &tm_w, full0 + 8 * i, (kb0 + i) * TC_BK, n0);
                if (NACC == 2) tma_load_2d(a + TC_A_BYTES, &tm_w, full0 + 8 * i, (kb0 + i) * TC_BK, p.ff + n0);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                const unsigned b = smem_u32(stage_mem + (size_t)i * Cfg::STAGE_BYTES) + NACC * TC_A_BYTES;
                tma_load_2d(b, &tm_a, full0 + 8 * i, (kb0 + i) * TC_BK, 0);
            }
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(empty0 + 8 * s, ((i / STAGES) & 1) ^ 1)) { flags[0] = 1; break; }
                const unsigned a = smem_u32(stage_mem + (size_t)s * Cfg::STAGE_BYTES);
                mbar_expect_tx(full0 + 8 * s, Cfg::STAGE_BYTES);
                tma_load_2d(a, &tm_w, full0 + 8 * s, (kb0 + i) * TC_BK, n0);
                if (NACC == 2) tma_load_2d(a + TC_A_BYTES, &tm_w, full0 + 8 * s, (kb0 + i) * TC_BK, p.ff + n0);
                tma_load_2d(a + NACC * TC_A_BYTES, &tm_a, full0 + 8 * s, (kb0 + i) * TC_BK, 0);
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
                const unsigned b = a + NACC * TC_A_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k) {
                    const unsigned acc = (i > 0 || k > 0) ? 1u : 0u;
                    umma_f16(tmem_base, umma_desc(a + k * 32), umma_desc(b + k * 32), idesc, acc);
                    if (NACC == 2) umma_f16(tmem_base + BN, umma_desc(a + TC_A_BYTES + k * 32), umma_desc(b + k * 32), idesc, acc);
                }
                umma_commit(empty0 + 8 * s);                        // the stage is free once these MMAs have read it
            }
            umma_commit(accbar);                                    // the accumulator is complete
        }
    } else {
        // ---- epilogue: warps 2..5, one weight row per thread ----
        const int et = threadIdx.x - 64;                            // 0..127
        const int quarter = warp & 3;                               // the 32 tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;                        // MMA row = weight row within the tile
        pdl_wait();
        if (p.pro == TC_PRO_NORM) {
            for (int m = et; m < p.M; m += 128) {
                float s = 0.f;
                for (int i = 0; i < p.ss_parts; ++i) s += p.ss_in[(size_t)i * p.M + m];
                inv_s[m] = rsqrtf(s / (float)p.K + p.eps);
            }
        }
        for (int i = et; i < 4 * 256; i += 128) sums[i] = 0.f;
        epi_bar();
        bool ok = mbar_wait(accbar, 0);
        if (!ok) flags[0] = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
        const long long n = p.epi == TC_EPI_SWIGLU ? (long long)n0 + row : (long long)n0 + row;
        const bool row_ok = p.epi == TC_EPI_SWIGLU ? n < p.ff : n < p.N;

        auto emit16 = [&](int c0, float (&y)[16], float (&y2)[16]) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int m = c0 + j;
                float v = y[j], v2 = y2[j];
                if (p.pro == TC_PRO_NORM && m < p.M) { v *= inv_s[m]; v2 *= inv_s[m]; }
                const bool valid = row_ok && m < p.M;
                if (p.epi == TC_EPI_SWIGLU) {
                    if (valid) p.out_bf16[(size_t)m * p.out_stride + n] = __float2bfloat16_rn(v / (1.f + expf(-v)) * v2);
                    continue;
                }
                if (valid && p.bias) v += p.bias[n];
                if (p.epi == TC_EPI_BF16) {
                    if (valid) p.out_bf16[(size_t)m * p.out_stride + n] = __float2bfloat16_rn(v);
                } else if (p.epi == TC_EPI_F32) {
                    if (valid) p.out_f32[(size_t)m * p.out_stride + n] = v;
                } else {
                    float nv = 0.f;
                    if (valid) {
                        nv = p.resid[(size_t)m * p.N + n] + v;
                        p.resid[(size_t)m * p.N + n] = nv;
                        if (p.xw_out) p.xw_out[(size_t)m * p.N + n] = __float2bfloat16_rn(nv * p.next_w[n]);
                    }
                    if (p.ss_out) {
                        const float sq = warp_sum(nv * nv);          // over this warp's 32 weight rows
                        if (lane == 0) sums[quarter * 256 + m] = sq;
                    }
                }
            }
        };

        if (ok && p.splits == 1) {
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= p.M) break;                                // uniform: tokens beyond M are padding
                float y[16], y2[16];
                tmem_ld16(taddr + c0, y);
                if (NACC == 2) tmem_ld16(taddr + BN + c0, y2);
                else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) y2[j] = 0.f;
                }
                emit16(c0, y, y2);
            }
        } else if (ok) {
            // partial tile to scratch: [tile][split][acc][token][128 rows], rows fastest
            float* mine = p.scratch + ((size_t)(tile * p.splits + sp) * NACC) * BN * TC_BM;
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= p.M) break;
                float y[16];
#pragma unroll
                for (int a = 0; a < NACC; ++a) {
                    tmem_ld16(taddr + a * BN + c0, y);
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[((size_t)a * BN + c0 + j) * TC_BM + row] = y[j];
                }
            }
            __threadfence();
            epi_bar();
            if (et == 0) flags[1] = atomicAdd(&p.counters[tile], 1u) == (unsigned)p.splits - 1 ? 1 : 0;
            epi_bar();
            if (flags[1]) {
                __threadfence();
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (c0 >= p.M) break;
                    float y[16], y2[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) { y[j] = 0.f; y2[j] = 0.f; }
                    for (int s2 = 0; s2 < p.splits; ++s2) {          // slice order, whoever arrived last
                        const float* part = p.scratch + ((size_t)(tile * p.splits + s2) * NACC) * BN * TC_BM;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            y[j] += part[((size_t)c0 + j) * TC_BM + row];
                            if (NACC == 2) y2[j] += part[((size_t)BN + c0 + j) * TC_BM + row];
                        }
                    }
                    emit16(c0, y, y2);
                }
                if (et == 0) p.counters[tile] = 0;                  // ready for the next call
            }
        }
        if (p.epi == TC_EPI_RESID && p.ss_out && (p.splits == 1 || flags[1])) {
            epi_bar();
            for (int m = et; m < p.M; m += 128)
                p.ss_out[(size_t)tile * p.M + m] = sums[m] + sums[256 + m] + sums[512 + m] + sums[768 + m];
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && flags[0] && p.status) atomicExch(p.status, 16);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)Cfg::TMEM_COLS) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

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

template <int BN, int NACC>
static int launch_tc(const CUtensorMap& tw, const CUtensorMap& ta, const TcParams& p, int tiles, cudaStream_t stream) {
    using Cfg = TcCfg<BN, NACC>;
    auto kern = linear_tc_kernel<BN, NACC>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return fail(-101, "linear_tc: cannot reserve %zu bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
        attr_done = true;
    }
    return check_launch("linear_tc", launch(kern, dim3(tiles, p.splits), TC_THREADS, Cfg::SMEM, stream, tw, ta, p));
}

// How many slices of K a call will use, and the scratch it needs: floats = tiles*splits*nacc*BN*128.
VAPI_EXPORT int vapi_linear_tc_plan(int N, int K, int M, int epi, int* tiles, int* splits, int* bn, long long* scratch_floats) {
    const int nacc = epi == TC_EPI_SWIGLU ? 2 : 1;
    const int rows = epi == TC_EPI_SWIGLU ? N / 2 : N;
    const int t = (rows + TC_BM - 1) / TC_BM;
    int b = 32;
    while (b < M) b *= 2;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    int s = 1;
    if (t < 120) {                                   // too few tiles for 148 SMs: cut K
        s = (148 + t - 1) / t;
        const int max_s = num_kb / 4 > 0 ? num_kb / 4 : 1;      // at least 4 k-blocks a slice
        if (s > max_s) s = max_s;
        if (s > 16) s = 16;
        const int per = (num_kb + s - 1) / s;
        s = (num_kb + per - 1) / per;                // no empty slice
    }
    *tiles = t; *splits = s; *bn = b;
    *scratch_floats = s > 1 ? (long long)t * s * nacc * b * TC_BM : 0;
    return 0;
}

VAPI_EXPORT int vapi_linear_tc(const void* W, int N, int K, int M, int pro, const void* tokens,
                               const float* ss_in, int ss_parts, float eps, int epi, void* out_bf16,
                               float* out_f32, long long out_stride, const float* bias, float* resid,
                               float* ss_out, const float* next_w, void* xw_out, float* scratch,
                               unsigned* counters, int* status, cudaStream_t stream) {
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
    long long need;
    vapi_linear_tc_plan(N, K, M, epi, &tiles, &splits, &bn, &need);
    if (splits > 1 && (!scratch || !counters)) return fail(-1, "linear_tc: %d slices of K need scratch memory and counters", splits);
    TcParams p;
    p.N = N; p.K = K; p.M = M; p.epi = epi; p.pro = pro; p.ff = N / 2;
    p.num_kb = (K + TC_BK - 1) / TC_BK; p.splits = splits; p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps;
    p.out_bf16 = (__nv_bfloat16*)out_bf16; p.out_f32 = out_f32; p.out_stride = out_stride; p.bias = bias;
    p.resid = resid; p.ss_out = ss_out; p.next_w = next_w; p.xw_out = (__nv_bfloat16*)xw_out;
    p.scratch = scratch; p.counters = counters; p.status = status;
    CUtensorMap tw, ta;
    int rc = make_map(&tw, W, N, K, TC_BM);
    if (rc) return rc;
    rc = make_map(&ta, tokens, M, K, bn);
    if (rc) return rc;
    const bool two = epi == TC_EPI_SWIGLU;
#define TC_GO(BN) return two ? launch_tc<BN, 2>(tw, ta, p, tiles, stream) : launch_tc<BN, 1>(tw, ta, p, tiles, stream)
    switch (bn) {
        case 32: TC_GO(32);
        case 64: TC_GO(64);
        case 128: TC_GO(128);
        case 256: TC_GO(256);
    }
#undef TC_GO
    return fail(-2, "linear_tc: no kernel for %d tokens", bn);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
