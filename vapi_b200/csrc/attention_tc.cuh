// Paged GQA attention for prompt portions on the fifth-generation tensor cores (tcgen05):
// bfloat16, head_dim 64, pages whose size is a multiple of 64.  Same semantics and the same rows
// as the other kernels of attention.cu (rows = (query token, q head of the group) pairs of one
// (sequence, kv head), bottom-right causal over the cached prefix, optional window), for
// sequences that bring at least `min_q` tokens to the step; shorter ones (decode tokens) are left
// to flash_paged_kernel, which the dispatcher launches beside this one.
//
// A block owns 128 rows and walks the key tiles (64 keys = one page's worth, one contiguous
// [64][64] block of K and of V) that any of its rows can see:
//   warp 0 (one lane)  TMA producer: K and V tiles through a ring of shared-memory stages;
//   warp 1 (one lane)  issues S = Q.K^T (128 x 64, K-major operands) into one of two
//                      tensor-memory buffers and O += P.V (V as an operand whose contiguous
//                      dimension is N) into a third; owns the tensor-memory allocation;
//   warps 2..5         softmax, one row per thread: S comes out of tensor memory with
//                      tcgen05.ld, so a row's maximum and sum need no shuffles; P goes to shared
//                      memory as bfloat16 in the operand layout; at the end O is scaled by 1/l
//                      and stored.
// The running maximum is only raised when a tile exceeds it by more than 2^8 (the exponentials
// stay below 256, which float accumulation and bfloat16 P carry without loss of accuracy), so
// the accumulator in tensor memory is rescaled a few times per row, not once per tile.
// S and P are double-buffered and S(i+1) is issued before P.V(i), so the softmax warps wait
// for the tensor core only when they must rescale the accumulator; two blocks per SM overlap
// the rest.
//
// Keys beyond the sequence's end in its last page may hold anything (memory is never cleared):
// their scores are replaced by -inf by selection, and their V rows are zeroed in shared memory
// before P.V, so that 0 * garbage cannot produce a NaN.
//
// Every mbarrier wait is bounded; a role that gives up records status 16 and the block drains
// (tensor memory is released on every path).
#pragma once
#include "tcgen05.cuh"

namespace vapi {

constexpr int FT_ROWS = 128;
constexpr int FT_BK = 64;
constexpr int FT_HD = 64;
constexpr int FT_STAGES = 3;
constexpr int FT_THREADS = 192;
constexpr int FT_TMEM_COLS = 256;                  // S0 | S1 | O, 64 columns each (a power of two is allocated)
constexpr int FT_TILE_BYTES = FT_BK * FT_HD * 2;   // one K or V tile
constexpr size_t FT_SMEM = 1024 + 3 * FT_ROWS * FT_HD * 2 + (size_t)FT_STAGES * 2 * FT_TILE_BYTES + 256;
constexpr int FT_MIN_Q = 32;                       // in a mixed step, sequences with fewer tokens go to the flash kernel
constexpr int FT_AUTO_MAX_Q = 64;                  // the dispatcher picks this kernel from this longest portion on
constexpr float FT_RAISE = 8.f;                    // log2 units by which a tile must exceed the running maximum to raise it

struct FaTcParams {
    const __nv_bfloat16* q; long long q_row_stride;
    const int* block_table; int table_stride;
    const int* cu_q; const int* seqlens_k;
    __nv_bfloat16* out;
    int nh, nkv, page_size, num_pages;
    float scale_log2e;
    int window, min_q;
    int* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(FT_THREADS, 2)
flash_tc_kernel(const __grid_constant__ CUtensorMap tm_kv, const FaTcParams p) {
    extern __shared__ unsigned char ft_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ft_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;                                   // [128 rows][128 B], 128-byte swizzle
    unsigned char* sP = base + FT_ROWS * FT_HD * 2;             // two buffers of the same shape: P of tile i in buffer i & 1
    unsigned char* sKV = sP + 2 * FT_ROWS * FT_BK * 2;          // [stage][K tile | V tile]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sKV + (size_t)FT_STAGES * 2 * FT_TILE_BYTES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 16);
    int* flags = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.z, g = blockIdx.y;
    pdl_trigger();
    // index data was copied from the host before the step's first kernel: safe before the wait
    const int q0 = p.cu_q[s], qlen = p.cu_q[s + 1] - q0, klen = p.seqlens_k[s];
    const int n_rep = p.nh / p.nkv;
    const int rows_total = qlen * n_rep;
    const int tile_start = ((int)gridDim.x - 1 - (int)blockIdx.x) * FT_ROWS;     // longest tiles first
    if (qlen < p.min_q || tile_start >= rows_total) {
        pdl_wait();
        return;
    }
    const int last_row = min(rows_total, tile_start + FT_ROWS) - 1;
    const int base_pos = klen - qlen;
    const int p_min = base_pos + tile_start / n_rep;
    const int p_max = base_pos + last_row / n_rep;
    const int key_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt_lo = key_lo / FT_BK, kt_hi = p_max / FT_BK;
    const int nt = kt_hi - kt_lo + 1;

    const unsigned kv_full = smem_u32(bars), kv_empty = smem_u32(bars + FT_STAGES);
    const unsigned s_full = smem_u32(bars + 2 * FT_STAGES), s_free = smem_u32(bars + 2 * FT_STAGES + 2);
    const unsigned p_ready = smem_u32(bars + 2 * FT_STAGES + 4), pv_done = smem_u32(bars + 2 * FT_STAGES + 6);   // one per P buffer
    const unsigned q_ready = smem_u32(bars + 2 * FT_STAGES + 8);

    if (threadIdx.x == 0) {
        for (int i = 0; i < FT_STAGES; ++i) { mbar_init(kv_full + 8 * i, 1); mbar_init(kv_empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + 8 * i, 1);
            mbar_init(s_free + 8 * i, 128);
            mbar_init(p_ready + 8 * i, 128);
            mbar_init(pv_done + 8 * i, 1);
        }
        mbar_init(q_ready, 128);
        flags[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)FT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const unsigned tmem_base = *tmem_slot;
    const unsigned tS0 = tmem_base, tO = tmem_base + 128;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            const int* bt = p.block_table + (size_t)s * p.table_stride;
            bool waited = false;
            for (int i = 0; i < nt; ++i) {
                const int stage = i % FT_STAGES;
                const int k0 = (kt_lo + i) * FT_BK;
                if (i >= FT_STAGES && !mbar_wait(kv_empty + 8 * stage, ((i / FT_STAGES) - 1) & 1)) { flags[0] = 1; break; }
                // a tile that reaches into this step's keys was written by the kernel before this one
                if (!waited && k0 + FT_BK > base_pos) { pdl_wait(); waited = true; }
                int page = bt[k0 / p.page_size];
                if (page < 0 || page >= p.num_pages) {
                    if (p.status) atomicExch(p.status, 4);
                    page = 0;
                }
                const int row = (page * 2 * p.nkv + g) * p.page_size + k0 % p.page_size;
                const unsigned dst = smem_u32(sKV + (size_t)stage * 2 * FT_TILE_BYTES);
                mbar_expect_tx(kv_full + 8 * stage, 2 * FT_TILE_BYTES);
                tma_load_2d(dst, &tm_kv, kv_full + 8 * stage, 0, row);
                tma_load_2d(dst + FT_TILE_BYTES, &tm_kv, kv_full + 8 * stage, 0, row + p.nkv * p.page_size);
            }
            if (!waited) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issue ----
            // instruction descriptor: float accumulate, bf16 x bf16, N = 64, M = 128; bit 16: B's
            // contiguous dimension is N (V tiles), else both operands are K-major
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FT_BK >> 3) << 17) | ((unsigned)(FT_ROWS >> 4) << 24);
            const unsigned idesc_o = idesc_s | (1u << 16);
            bool ok = true;
            auto pv = [&](int j) {          // O += P(j) . V(j)
                if (!ok) return;
                if (!mbar_wait(p_ready + 8 * (j & 1), (j >> 1) & 1)) { ok = false; return; }
                tc5_fence_after();
                const int stage = j % FT_STAGES;
                const unsigned pa = smem_u32(sP + (j & 1) * FT_ROWS * FT_BK * 2);
                const unsigned vb = smem_u32(sKV + (size_t)stage * 2 * FT_TILE_BYTES) + FT_TILE_BYTES;
#pragma unroll
                for (int k = 0; k < FT_BK / 16; ++k)
                    umma_f16(tO, umma_desc(pa + k * 32), umma_desc_mn(vb + k * 16 * 128), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(pv_done + 8 * (j & 1));
                umma_commit(kv_empty + 8 * stage);
            };
            for (int i = 0; i < nt && ok; ++i) {
                const int stage = i % FT_STAGES, sb = i & 1;
                if (!mbar_wait(kv_full + 8 * stage, (i / FT_STAGES) & 1)) { ok = false; break; }
                if (i >= 2 && !mbar_wait(s_free + 8 * sb, ((i >> 1) - 1) & 1)) { ok = false; break; }
                if (i == 0 && !mbar_wait(q_ready, 0)) { ok = false; break; }
                tc5_fence_after();
                const unsigned qa = smem_u32(sQ);
                const unsigned kb = smem_u32(sKV + (size_t)stage * 2 * FT_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < FT_HD / 16; ++k)
                    umma_f16(tS0 + sb * 64, umma_desc(qa + k * 32), umma_desc(kb + k * 32), idesc_s, k > 0 ? 1u : 0u);
                umma_commit(s_full + 8 * sb);
                if (i >= 1) pv(i - 1);
            }
            pv(nt - 1);
            if (!ok) flags[0] = 1;
        }
    } else {
        // ---- softmax and epilogue: one row per thread ----
        const int quarter = warp & 3;                               // the tensor-memory lanes this warp may touch
        const int row = quarter * 32 + lane;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const int rr = tile_start + row;
        const bool row_ok = rr < rows_total;
        const int tok = row_ok ? rr / n_rep : 0;
        const int head = g * n_rep + (row_ok ? rr - tok * n_rep : 0);
        const int pos = row_ok ? base_pos + tok : -1;               // -1: sees nothing
        const bool partial = tile_start + FT_ROWS > rows_total;
        pdl_wait();                                                 // q was rotated by the kernel before this one
        {
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + tok) * p.q_row_stride + (size_t)head * FT_HD);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 v = row_ok ? src[c] : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(sQ + row * 128 + ((c ^ (row & 7)) << 4)) = v;
            }
            fence_proxy_async();
            mbar_arrive(q_ready);
        }
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int i = 0; i < nt && ok; ++i) {
            const int sb = i & 1, stage = i % FT_STAGES;
            const int k0 = (kt_lo + i) * FT_BK;
            // (a wait's outcome is made uniform over the warp: the tensor-memory accesses below are
            // warp-wide instructions)
            if (!__all_sync(0xffffffffu, mbar_wait(s_full + 8 * sb, (i >> 1) & 1))) { ok = false; break; }
            tc5_fence_after();
            float sv[FT_BK];
            {
                unsigned raw[FT_BK / 16][16];                           // all four loads in flight, one wait
#pragma unroll
                for (int j = 0; j < FT_BK / 16; ++j) tmem_ld16_nowait(tS0 + sb * 64 + lane_addr + j * 16, raw[j]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < FT_BK / 16; ++j)
#pragma unroll
                    for (int e = 0; e < 16; ++e) sv[j * 16 + e] = __uint_as_float(raw[j][e]);
            }
            tc5_fence_before();
            mbar_arrive(s_free + 8 * sb);                           // the scores are in registers

            const bool need_mask = partial || (k0 + FT_BK - 1 > p_min) || (k0 + FT_BK > klen) ||
                                   (p.window > 0 && k0 <= p_max - p.window);
            // (four running maxima and, below, four running sums: a single chain of 64 dependent
            // operations would leave the few warps of an SM waiting on latency)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < FT_BK; ++e) {
                    const int kj = k0 + e;
                    const bool vis = kj <= pos && kj < klen && (p.window <= 0 || kj > pos - p.window);
                    sv[e] = vis ? sv[e] : -INFINITY;
                    mx4[e & 3] = fmaxf(mx4[e & 3], sv[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < FT_BK; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], sv[e]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float mx_s = mx * p.scale_log2e;                  // (the scale is positive)
            const bool grow = mx_s > m_run + FT_RAISE;              // also the first tile with a visible key
            const float m_new = grow ? mx_s : m_run;
            const float alpha = grow ? ex2_approx(m_run - m_new) : 1.f;     // m_run = -inf: 0
            if (i >= 1 && __any_sync(0xffffffffu, grow)) {
                // the accumulator must be at rest: P.V of the tile before this one has completed
                if (!__all_sync(0xffffffffu, mbar_wait(pv_done + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1))) { ok = false; break; }
                tc5_fence_after();
#pragma unroll
                for (int j = 0; j < FT_HD / 16; ++j) {
                    float o16[16];
                    tmem_ld16(tO + lane_addr + j * 16, o16);
#pragma unroll
                    for (int e = 0; e < 16; ++e) o16[e] *= alpha;
                    tmem_st16(tO + lane_addr + j * 16, o16);
                }
                tmem_st_wait();
            }
            // this tile's P buffer was last read by P.V of the tile two before
            if (i >= 2 && !__all_sync(0xffffffffu, mbar_wait(pv_done + 8 * sb, ((i >> 1) - 1) & 1))) { ok = false; break; }
            l_run *= alpha;
            m_run = m_new;
            const float m_use = m_run == -INFINITY ? 0.f : m_run;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                unsigned w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float a = ex2_approx(fmaf(sv[c * 8 + 2 * e], p.scale_log2e, -m_use));
                    const float b = ex2_approx(fmaf(sv[c * 8 + 2 * e + 1], p.scale_log2e, -m_use));
                    rs4[e] += a + b;
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
                    w[e] = *reinterpret_cast<unsigned*>(&h2);
                }
                *reinterpret_cast<uint4*>(sP + sb * FT_ROWS * FT_BK * 2 + row * 128 + ((c ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            if (k0 + FT_BK > klen) {
                // V rows of keys beyond the sequence: zero them (a row is 128 bytes whatever the swizzle)
                if (!__all_sync(0xffffffffu, mbar_wait(kv_full + 8 * stage, (i / FT_STAGES) & 1))) { ok = false; break; }   // complete already: makes the tile visible here
                if (row < FT_BK && k0 + row >= klen) {
                    uint4* vr = reinterpret_cast<uint4*>(sKV + (size_t)stage * 2 * FT_TILE_BYTES + FT_TILE_BYTES + row * 128);
#pragma unroll
                    for (int c = 0; c < 8; ++c) vr[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            fence_proxy_async();
            tc5_fence_before();
            mbar_arrive(p_ready + 8 * sb);
        }
        if (ok && !__all_sync(0xffffffffu, mbar_wait(pv_done + 8 * ((nt - 1) & 1), ((nt - 1) >> 1) & 1))) ok = false;
        tc5_fence_after();
        if (ok) {                                                   // (uniform over the warp)
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* o = p.out + ((size_t)(q0 + tok) * p.nh + head) * FT_HD;
#pragma unroll
            for (int j = 0; j < FT_HD / 16; ++j) {
                float o16[16];
                tmem_ld16(tO + lane_addr + j * 16, o16);
                unsigned w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(o16[2 * e] * inv, o16[2 * e + 1] * inv);
                    w[e] = *reinterpret_cast<unsigned*>(&h2);
                }
                if (row_ok) {
                    *reinterpret_cast<uint4*>(o + j * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(o + j * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
        if (!ok) flags[0] = 1;
    }

    tc5_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && flags[0] && p.status) atomicExch(p.status, 16);
    if (warp == 1) {
        tc5_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)FT_TMEM_COLS) : "memory");
    }
}

// the cache layer [pages][2][nkv][page_size][64] as rows of 64 bfloat16, tiled in boxes of 64 rows
static int make_kv_map(CUtensorMap* map, const void* cache, long long rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(-102, "paged_attention: cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)cache & 15) != 0) return fail(-1, "paged_attention: the cache is not 16-byte aligned");
    if (rows > 0x7fffffffLL) return fail(-1, "paged_attention: %lld cache rows exceed a TMA coordinate", rows);
    cuuint64_t dims[2] = {(cuuint64_t)FT_HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)FT_HD * 2};
    cuuint32_t box[2] = {(cuuint32_t)FT_HD, (cuuint32_t)FT_BK};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(-103, "paged_attention: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

static int launch_flash_tc(const void* q, long long q_row_stride, const void* cache, const int* block_table,
                           int table_stride, const int* cu_q, const int* seqlens_k, void* out, int num_seqs,
                           int max_q, int nh, int nkv, int page_size, int num_pages, float scale, int window,
                           int min_q, int* status, cudaStream_t stream) {
    const int n_rep = nh / nkv;
    const long long tiles = ((long long)max_q * n_rep + FT_ROWS - 1) / FT_ROWS;
    if (tiles > 0x7fffffffLL || nkv > 65535 || num_seqs > 65535)
        return fail(-1, "paged_attention: the step exceeds the grid (%lld row tiles, %d kv heads, %d sequences)", tiles, nkv, num_seqs);
    if (!(scale > 0.f)) return fail(-1, "paged_attention: the tcgen05 kernel needs a positive scale");
    if (q_row_stride % 8 != 0 || ((uintptr_t)q & 15) != 0 || ((uintptr_t)out & 15) != 0)
        return fail(-1, "paged_attention: the tcgen05 kernel needs 16-byte aligned query and output rows");
    CUtensorMap map;
    int rc = make_kv_map(&map, cache, (long long)num_pages * 2 * nkv * page_size);
    if (rc != 0) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM);
        if (e != cudaSuccess) return fail(-101, "paged_attention: cannot reserve %zu bytes of shared memory: %s", FT_SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    FaTcParams p;
    p.q = (const __nv_bfloat16*)q; p.q_row_stride = q_row_stride; p.block_table = block_table; p.table_stride = table_stride;
    p.cu_q = cu_q; p.seqlens_k = seqlens_k; p.out = (__nv_bfloat16*)out; p.nh = nh; p.nkv = nkv; p.page_size = page_size;
    p.num_pages = num_pages; p.scale_log2e = scale * 1.4426950408889634f; p.window = window; p.min_q = min_q; p.status = status;
    dim3 grid((unsigned)tiles, nkv, num_seqs);
    return check_launch("paged_attention (tcgen05)", launch(flash_tc_kernel, grid, FT_THREADS, FT_SMEM, stream, map, p));
}

}  // namespace vapi
