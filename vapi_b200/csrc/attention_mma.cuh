// Tensor-core paged GQA attention for the serving path: bfloat16, head_dim 64 or 128, pages
// whose size is a multiple of 64.  Same semantics and the same work decomposition as the
// general kernel in attention.cu (rows = (query token, q head of the group) pairs of one
// (sequence, kv head); keys walked in tiles that all rows of the block share; optional
// split over the keys with a fixed-order combine), but
//   * a warp owns 16 rows and computes Q.K^T and P.V with mma.sync m16n8k16 (bf16 in, float
//     accumulate); softmax statistics stay in float registers, P is rounded to bfloat16 only
//     as the operand of P.V;
//   * a key tile is 64 keys, which always lie in one page, so a tile of K (or V) of one kv
//     head is one contiguous run of 64*head_dim elements; it is brought in with 16-byte
//     cp.async copies through a ring of shared-memory stages and stored with an XOR swizzle
//     of the 16-byte chunks so that ldmatrix reads without bank conflicts;
//   * keys no row can see (beyond the sequence, behind the window) are zero-filled by the
//     copy itself, so uninitialised cache memory never reaches the arithmetic.
// One block is NWARPS warps (4 for prompt portions: 64 rows; 1 for decode steps, where a
// (sequence, kv head) has only n_rep rows and many small blocks keep more loads in flight).
#pragma once
#include "common.cuh"

namespace vapi {

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, int src_bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

constexpr int FA_BK = 64;

template <int HD, int NWARPS, int STAGES>
__global__ void __launch_bounds__(NWARPS * 32, (HD <= 64 && NWARPS == 4) ? 4 : 1)
flash_paged_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride,
                   const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table,
                   int table_stride, const int* __restrict__ cu_q, const int* __restrict__ seqlens_k,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int nh, int nkv, int page_size, int num_pages,
                   float scale_log2e, int window, int splits, int q_below, int rows_above,
                   int* __restrict__ status) {
    // q_below > 0: sequences that bring q_below tokens or more belong to another kernel, and so do
    // sequences of at most rows_above rows (rows_above > 0)
    constexpr int ROWS = NWARPS * 16;
    constexpr int CPR = HD / 8;            // 16-byte chunks in a row
    constexpr int TILE = FA_BK * HD;       // elements of one K (or V) tile
    constexpr int KSTEPS = HD / 16;
    extern __shared__ __align__(128) unsigned char fa_smem[];
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(fa_smem);   // [STAGES][64][HD]
    __nv_bfloat16* sV = sK + STAGES * TILE;                           // [STAGES][64][HD]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;                          // row / column-pair of the fragment
    const int s = blockIdx.z / splits, sp = blockIdx.z - s * splits;
    const int g = blockIdx.y;
    pdl_trigger();
    // index data was copied from the host before the step's first kernel: safe before the wait
    const int q0 = cu_q[s], qlen = cu_q[s + 1] - q0, klen = seqlens_k[s];
    const int n_rep = nh / nkv;
    const int rows_total = qlen * n_rep;
    // row tiles late in a sequence see the most keys: hand them out first, so that the last
    // blocks to start are the short ones
    const int tile_start = ((int)gridDim.x - 1 - (int)blockIdx.x) * ROWS;
    if (tile_start >= rows_total || (q_below > 0 && qlen >= q_below) || rows_total <= rows_above) {
        pdl_wait();
        return;
    }
    const int last_row = min(rows_total, tile_start + ROWS) - 1;
    const int base_pos = klen - qlen;
    const int p_min = base_pos + tile_start / n_rep;
    const int p_max = base_pos + last_row / n_rep;
    const int key_lo = window > 0 ? max(0, p_min - window + 1) : 0;
    const int kt_lo = key_lo / FA_BK, kt_hi = p_max / FA_BK;
    const int ntiles_all = kt_hi - kt_lo + 1;
    const int chunk = (ntiles_all + splits - 1) / splits;
    const int kt_begin = kt_lo + sp * chunk;
    const int kt_end = min(kt_hi + 1, kt_begin + chunk);
    const int nt = max(0, kt_end - kt_begin);

    // this thread's two rows: (gq) and (gq + 8) of the warp's 16
    int row_id[2], row_pos[2], row_tok[2], row_head[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int rr = tile_start + warp * 16 + gq + 8 * h;
        row_ok[h] = rr < rows_total;
        row_id[h] = rr;
        row_tok[h] = row_ok[h] ? rr / n_rep : 0;
        row_head[h] = g * n_rep + (row_ok[h] ? rr - row_tok[h] * n_rep : 0);
        row_pos[h] = row_ok[h] ? base_pos + row_tok[h] : -1;       // -1: sees nothing
    }
    // lowest / highest position among the warp's 16 rows (for skipping and for mask decisions)
    const int w_first = tile_start + warp * 16;
    const bool warp_has_rows = w_first < rows_total;
    const int w_pos_min = base_pos + w_first / n_rep;
    const int w_pos_max = base_pos + (min(rows_total, w_first + 16) - 1) / n_rep;

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }

    const int* bt = block_table + (size_t)s * table_stride;
    const int key_hi = min(klen - 1, p_max);

    auto load_tile = [&](int kt, int stage) {
        const int k0 = kt * FA_BK;
        int page = bt[k0 / page_size];
        bool page_ok = page >= 0 && page < num_pages;
        if (!page_ok) {
            if (threadIdx.x == 0 && status && k0 <= key_hi && k0 + FA_BK > key_lo) atomicExch(status, 4);
            page = 0;
        }
        const __nv_bfloat16* kbase = cache + ((((size_t)page * 2) * nkv + g) * page_size + (k0 % page_size)) * HD;
        const __nv_bfloat16* vbase = kbase + (size_t)nkv * page_size * HD;
        __nv_bfloat16* dk = sK + stage * TILE;
        __nv_bfloat16* dv = sV + stage * TILE;
        for (int i = threadIdx.x; i < FA_BK * CPR; i += NWARPS * 32) {
            const int r = i / CPR, c = i - r * CPR;
            const int kj = k0 + r;
            const int bytes = (page_ok && kj >= key_lo && kj <= key_hi) ? 16 : 0;   // 0: zero-fill
            const int doff = r * HD + ((c ^ (r & 7)) << 3);
            cp_async_16(dk + doff, kbase + r * HD + c * 8, bytes);
            cp_async_16(dv + doff, vbase + r * HD + c * 8, bytes);
        }
    };

    // Tiles that hold only keys of earlier steps do not depend on the kernel before this one
    // (which wrote this step's keys and rotated this step's queries): bring them in first.
    const int kt_old_end = base_pos / FA_BK;
    const int pre = max(0, min(min(STAGES - 1, nt), kt_old_end - kt_begin));
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < pre) {
            load_tile(kt_begin + st, st);
            cp_async_commit();
        }
    }
    pdl_wait();
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st >= pre) {
            if (st < nt) load_tile(kt_begin + st, st);
            cp_async_commit();
        }
    }

    // Q fragments, kept for the whole kernel
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            unsigned lo = 0u, hi = 0u;
            if (row_ok[h]) {
                const __nv_bfloat16* p = q + (size_t)(q0 + row_tok[h]) * q_row_stride + (size_t)row_head[h] * HD + kk * 16 + 2 * tq;
                lo = *reinterpret_cast<const unsigned*>(p);
                hi = *reinterpret_cast<const unsigned*>(p + 8);
            }
            qf[kk][h] = lo;          // a0 (row g) / a1 (row g+8): columns 2t, 2t+1
            qf[kk][2 + h] = hi;      // a2 / a3: columns 2t+8, 2t+9
        }
    }


    for (int it = 0; it < nt; ++it) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (it + STAGES - 1 < nt) load_tile(kt_begin + it + STAGES - 1, (it + STAGES - 1) % STAGES);
        cp_async_commit();

        const int kt = kt_begin + it;
        const int k0 = kt * FA_BK;
        // a warp none of whose rows reaches this tile (causal) or whose window has passed it skips it
        if (!warp_has_rows || k0 > w_pos_max || (window > 0 && k0 + FA_BK - 1 <= w_pos_min - window)) continue;
        const __nv_bfloat16* ks = sK + (it % STAGES) * TILE;
        const __nv_bfloat16* vs = sV + (it % STAGES) * TILE;

        float sc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
            for (int nj = 0; nj < 4; ++nj) {
                const int mat = lane >> 3, rin = lane & 7;
                const int key = nj * 16 + (mat >> 1) * 8 + rin;
                const int ch = kk * 2 + (mat & 1);
                unsigned r0, r1, r2, r3;
                ldmatrix_x4(r0, r1, r2, r3, ks + key * HD + ((ch ^ (key & 7)) << 3));
                mma_bf16_16816(sc[2 * nj], qf[kk], r0, r1);
                mma_bf16_16816(sc[2 * nj + 1], qf[kk], r2, r3);
            }
        }
        // scale, mask, online softmax (base 2)
        const bool need_mask = (k0 + FA_BK - 1 > w_pos_min) || (k0 + FA_BK > klen) ||
                               (window > 0 && k0 <= w_pos_max - window);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float v = sc[i][2 * h + e] * scale_log2e;
                    if (need_mask) {
                        const int kj = k0 + i * 8 + 2 * tq + e;
                        const bool vis = kj <= row_pos[h] && kj < klen && (window <= 0 || kj > row_pos[h] - window);
                        v = vis ? v : -INFINITY;
                    }
                    sc[i][2 * h + e] = v;
                    mx = fmaxf(mx, v);
                }
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = exp2f(m_run[h] - m_use);
            float rs = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float p = exp2f(sc[i][2 * h + e] - m_use);
                    sc[i][2 * h + e] = p;
                    rs += p;
                }
            }
            l_run[h] = l_run[h] * alpha + rs;       // per-thread part of the row sum; quad-reduced at the end
            m_run[h] = m_new;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o_acc[i][2 * h] *= alpha; o_acc[i][2 * h + 1] *= alpha; }
        }
        // O += P.V
#pragma unroll
        for (int kk2 = 0; kk2 < 4; ++kk2) {
            unsigned pa[4];
            pa[0] = pack_bf16(sc[2 * kk2][0], sc[2 * kk2][1]);
            pa[1] = pack_bf16(sc[2 * kk2][2], sc[2 * kk2][3]);
            pa[2] = pack_bf16(sc[2 * kk2 + 1][0], sc[2 * kk2 + 1][1]);
            pa[3] = pack_bf16(sc[2 * kk2 + 1][2], sc[2 * kk2 + 1][3]);
#pragma unroll
            for (int nd = 0; nd < HD / 16; ++nd) {
                const int mat = lane >> 3, rin = lane & 7;
                const int key = kk2 * 16 + (mat & 1) * 8 + rin;
                const int ch = nd * 2 + (mat >> 1);
                unsigned r0, r1, r2, r3;
                ldmatrix_x4_trans(r0, r1, r2, r3, vs + key * HD + ((ch ^ (key & 7)) << 3));
                mma_bf16_16816(o_acc[2 * nd], pa, r0, r1);
                mma_bf16_16816(o_acc[2 * nd + 1], pa, r2, r3);
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!row_ok[h]) continue;
        const size_t grow = (size_t)(q0 + row_tok[h]) * nh + row_head[h];
        if (splits == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* o = out + grow * HD;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[i][2 * h] * inv, o_acc[i][2 * h + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + 2 * tq) = v;
            }
        } else {
            float* po = part_o + (grow * splits + sp) * (size_t)HD;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                *reinterpret_cast<float2*>(po + i * 8 + 2 * tq) = make_float2(o_acc[i][2 * h], o_acc[i][2 * h + 1]);
            }
            if (tq == 0) {
                // the combine step works with natural-log maxima
                part_ml[(grow * splits + sp) * 2] = m_run[h] == -INFINITY ? -INFINITY : m_run[h] * 0.6931471805599453f;
                part_ml[(grow * splits + sp) * 2 + 1] = l;
            }
        }
    }
}

template <int HD, int NWARPS, int STAGES>
static int launch_flash(const void* q, long long q_row_stride, const void* cache,
                        const int* block_table, int table_stride, const int* cu_q,
                        const int* seqlens_k, void* out, float* part_o, float* part_ml, int num_seqs,
                        int max_q, int nh, int nkv, int page_size, int num_pages, float scale,
                        int window, int splits, int* status, cudaStream_t stream, int q_below = 0, int rows_above = 0) {
    const int n_rep = nh / nkv;
    const long long max_rows = (long long)max_q * n_rep;
    const long long tiles = (max_rows + NWARPS * 16 - 1) / (NWARPS * 16);
    if (tiles > 0x7fffffffLL) return fail(-1, "paged_attention: too many query rows");
    if (nkv > 65535 || (long long)num_seqs * splits > 65535)
        return fail(-1, "paged_attention: %d kv heads or %d sequences x %d splits exceed the grid", nkv, num_seqs, splits);
    const size_t smem = (size_t)2 * STAGES * FA_BK * HD * sizeof(__nv_bfloat16);
    auto kern = flash_paged_kernel<HD, NWARPS, STAGES>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-101, "paged_attention: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid((unsigned)tiles, nkv, num_seqs * splits);
    return check_launch("paged_attention (tensor-core)", launch(kern, grid, NWARPS * 32, smem, stream,
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)cache, block_table, table_stride, cu_q,
        seqlens_k, (__nv_bfloat16*)out, part_o, part_ml, nh, nkv, page_size, num_pages,
        scale * 1.4426950408889634f, window, splits, q_below, rows_above, status));
}

}  // namespace vapi
