// Paged grouped-query attention over the block table, for prompt portions and decode
// tokens in one launch.  This is the general kernel: any head_dim that is a multiple of
// 16 up to 256, any number of heads and groups, an optional sliding window, float or
// bfloat16 storage, all arithmetic in float.  It is the attention of the true 32-bit
// path, and of the serving path wherever no faster specialisation applies.
//
// Semantics of the reference's paged attention
// (crates/vapi-backend-candle/src/attention.rs:90-163): a sequence brings len_q queries
// over len_k keys; query j sits at position p = len_k - len_q + j and sees keys i <= p
// (and i > p - window when a window is set); scores are scale * q.k in float, softmax in
// float, q head h reads kv head h / (nh / nkv).
//
// Work decomposition.  For one (sequence, kv head) the rows are the pairs (query token,
// q head of the group), row = token * n_rep + rep, cut into tiles of 16; a block of four
// warps takes one tile and walks the keys in tiles of 32 that all its rows share.  Warp w
// owns rows w, w+4, w+8, w+12 of the tile entirely (scores, running max and sum, output),
// so the only block-wide synchronisation is around the key/value tile in shared memory.
// With `splits` > 1 the key tiles of a row tile are divided among `splits` blocks that
// write unnormalised partial results to scratch memory, and a second kernel combines them
// in a fixed order.
#include "common.cuh"
#include "attention_mma.cuh"
#include "attention_tc.cuh"
#include "attention_decode.cuh"

using namespace vapi;

constexpr int ATT_ROWS = 16;
constexpr int ATT_BK = 32;
constexpr int ATT_WARPS = 4;
constexpr int ATT_RPW = ATT_ROWS / ATT_WARPS;  // rows per warp

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    using type = float4;
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Vec4<__nv_bfloat16> {
    using type = uint2;
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
};

template <typename T, int DMAX>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_kernel(const T* __restrict__ q, long long q_row_stride,
                       const T* __restrict__ cache, const int* __restrict__ block_table,
                       int table_stride, const int* __restrict__ cu_q,
                       const int* __restrict__ seqlens_k, T* __restrict__ out,
                       float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
                       int d, int page_size, int num_pages, float scale, int window, int splits,
                       int* __restrict__ status) {
    constexpr int DPL = DMAX / 32;
    extern __shared__ __align__(16) float smem[];
    const int ld = d + 4;  // row pitch in floats: keeps float4 alignment, spreads banks
    float* Qs = smem;                     // [ATT_ROWS][ld]
    float* Ks = Qs + ATT_ROWS * ld;       // [ATT_BK][ld]
    float* Vs = Ks + ATT_BK * ld;         // [ATT_BK][ld]
    float* Ps = Vs + ATT_BK * ld;         // [ATT_WARPS][ATT_RPW][ATT_BK]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.z / splits, sp = blockIdx.z - s * splits;
    const int g = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    const int q0 = cu_q[s], qlen = cu_q[s + 1] - q0, klen = seqlens_k[s];
    const int n_rep = nh / nkv;
    const int rows_total = qlen * n_rep;
    const int tile_start = blockIdx.x * ATT_ROWS;
    if (tile_start >= rows_total) return;
    const int last_row = min(rows_total, tile_start + ATT_ROWS) - 1;
    const int base_pos = klen - qlen;
    const int p_min = base_pos + tile_start / n_rep;
    const int p_max = base_pos + last_row / n_rep;
    const int key_lo = window > 0 ? max(0, p_min - window + 1) : 0;
    const int kt_lo = key_lo / ATT_BK, kt_hi = p_max / ATT_BK;
    const int nt = kt_hi - kt_lo + 1;
    const int chunk = (nt + splits - 1) / splits;
    const int kt_begin = kt_lo + sp * chunk;
    const int kt_end = min(kt_hi + 1, kt_begin + chunk);

    // queries of the tile, scaled, as float
    for (int idx = threadIdx.x; idx < ATT_ROWS * (d / 4); idx += blockDim.x) {
        const int lr = idx / (d / 4), c4 = idx - lr * (d / 4);
        const int rr = tile_start + lr;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rr < rows_total) {
            const int tok = rr / n_rep, h = g * n_rep + (rr - tok * n_rep);
            v = Vec4<T>::load(q + (size_t)(q0 + tok) * q_row_stride + (size_t)h * d + c4 * 4);
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
        }
        *reinterpret_cast<float4*>(Qs + lr * ld + c4 * 4) = v;
    }

    int row_pos[ATT_RPW];
    bool row_ok[ATT_RPW];
    float m[ATT_RPW], l[ATT_RPW], acc[ATT_RPW][DPL];
#pragma unroll
    for (int a = 0; a < ATT_RPW; ++a) {
        const int rr = tile_start + warp + ATT_WARPS * a;
        row_ok[a] = rr < rows_total;
        row_pos[a] = base_pos + (row_ok[a] ? rr / n_rep : 0);
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[a][c] = 0.f;
    }

    const int* bt = block_table + (size_t)s * table_stride;
    for (int kt = kt_begin; kt < kt_end; ++kt) {
        __syncthreads();  // the previous tile is no longer read (and Qs is written)
        for (int idx = threadIdx.x; idx < ATT_BK * (d / 4); idx += blockDim.x) {
            const int jj = idx / (d / 4), c4 = idx - jj * (d / 4);
            const int j = kt * ATT_BK + jj;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (j >= key_lo && j <= p_max && j < klen) {  // keys no row of the tile can see stay zero
                const int page = bt[j / page_size];
                if (page < 0 || page >= num_pages) {
                    if (status) atomicExch(status, 4);
                } else {
                    const size_t base = (((size_t)page * 2) * nkv + g) * page_size * (size_t)d +
                                        (size_t)(j % page_size) * d + c4 * 4;
                    kv = Vec4<T>::load(cache + base);
                    vv = Vec4<T>::load(cache + base + (size_t)nkv * page_size * d);
                }
            }
            *reinterpret_cast<float4*>(Ks + jj * ld + c4 * 4) = kv;
            *reinterpret_cast<float4*>(Vs + jj * ld + c4 * 4) = vv;
        }
        __syncthreads();

        // scores of this warp's rows against key `lane` of the tile
        float sc[ATT_RPW];
#pragma unroll
        for (int a = 0; a < ATT_RPW; ++a) sc[a] = 0.f;
        const float4* k4 = reinterpret_cast<const float4*>(Ks + lane * ld);
        for (int c4 = 0; c4 < d / 4; ++c4) {
            const float4 kv = k4[c4];
#pragma unroll
            for (int a = 0; a < ATT_RPW; ++a) {
                if (!row_ok[a]) continue;
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp + ATT_WARPS * a) * ld + c4 * 4);
                sc[a] = fmaf(qv.x, kv.x, sc[a]);
                sc[a] = fmaf(qv.y, kv.y, sc[a]);
                sc[a] = fmaf(qv.z, kv.z, sc[a]);
                sc[a] = fmaf(qv.w, kv.w, sc[a]);
            }
        }
        const int j = kt * ATT_BK + lane;
        float* pw = Ps + (warp * ATT_RPW) * ATT_BK;
#pragma unroll
        for (int a = 0; a < ATT_RPW; ++a) {
            if (!row_ok[a]) continue;  // uniform across the warp
            const bool vis = j <= row_pos[a] && j < klen && (window <= 0 || j > row_pos[a] - window);
            const float sv = vis ? sc[a] : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max(sv));
            float p = 0.f, alpha = 1.f;
            if (m_new != -INFINITY) {
                alpha = expf(m[a] - m_new);  // m[a] = -inf gives 0
                p = vis ? expf(sv - m_new) : 0.f;
            }
            l[a] = l[a] * alpha + warp_sum(p);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[a][c] *= alpha;
            pw[a * ATT_BK + lane] = p;
        }
        __syncwarp();
        for (int jj = 0; jj < ATT_BK; ++jj) {
            float vcol[DPL];
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int col = lane + 32 * c;
                vcol[c] = col < d ? Vs[jj * ld + col] : 0.f;
            }
#pragma unroll
            for (int a = 0; a < ATT_RPW; ++a) {
                if (!row_ok[a]) continue;
                const float p = pw[a * ATT_BK + jj];
#pragma unroll
                for (int c = 0; c < DPL; ++c) acc[a][c] = fmaf(p, vcol[c], acc[a][c]);
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int a = 0; a < ATT_RPW; ++a) {
        if (!row_ok[a]) continue;
        const int rr = tile_start + warp + ATT_WARPS * a;
        const int tok = rr / n_rep, h = g * n_rep + (rr - tok * n_rep);
        const size_t grow = (size_t)(q0 + tok) * nh + h;
        if (splits == 1) {
            const float inv = l[a] > 0.f ? 1.f / l[a] : 0.f;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int col = lane + 32 * c;
                if (col < d) out[grow * d + col] = from_f32<T>(acc[a][c] * inv);
            }
        } else {
            float* po = part_o + (grow * splits + sp) * (size_t)d;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int col = lane + 32 * c;
                if (col < d) po[col] = acc[a][c];
            }
            if (lane == 0) {
                part_ml[(grow * splits + sp) * 2] = m[a];
                part_ml[(grow * splits + sp) * 2 + 1] = l[a];
            }
        }
    }
}

// Combine the partial results of `splits` (at most 32) blocks: one warp per (token, head).
// Lane sp holds the weight exp(m_sp - max) of split sp; the sums over the splits run in
// split order whatever finished first.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, T* __restrict__ out,
                                         long long rows, int d, int splits) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    if (row >= rows) return;
    float ms = -INFINITY, ls = 0.f;
    if (lane < splits) {
        ms = part_ml[(row * splits + lane) * 2];
        ls = part_ml[(row * splits + lane) * 2 + 1];
    }
    const float mx = warp_max(ms);
    const float w = ms == -INFINITY ? 0.f : expf(ms - mx);
    float lsum = 0.f;
    for (int sp = 0; sp < splits; ++sp) lsum += __shfl_sync(0xffffffffu, ls * w, sp);
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    for (int c0 = 0; c0 < d; c0 += 32) {
        const int col = c0 + lane;
        float o = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < splits; ++sp) {
            const float ws = __shfl_sync(0xffffffffu, w, sp);
            const float v = col < d ? part_o[(row * splits + sp) * (size_t)d + col] : 0.f;
            o += v * ws;
        }
        if (col < d) out[row * d + col] = from_f32<T>(o * inv);
    }
}

template <typename T, int DMAX>
static int launch_attention(const void* q, long long q_row_stride, const void* cache,
                            const int* block_table, int table_stride, const int* cu_q,
                            const int* seqlens_k, void* out, float* part_o, float* part_ml,
                            int num_seqs, int max_q, int nh, int nkv, int d, int page_size,
                            int num_pages, float scale, int window, int splits, int* status,
                            cudaStream_t stream) {
    const int n_rep = nh / nkv;
    const long long max_rows = (long long)max_q * n_rep;
    const long long tiles = (max_rows + ATT_ROWS - 1) / ATT_ROWS;
    if (tiles > 0x7fffffffLL) return fail(-1, "paged_attention: too many query rows");
    if (nkv > 65535 || (long long)num_seqs * splits > 65535)
        return fail(-1, "paged_attention: %d kv heads or %d sequences x %d splits exceed the grid",
                    nkv, num_seqs, splits);
    const size_t smem = ((size_t)(ATT_ROWS + 2 * ATT_BK) * (d + 4) + ATT_WARPS * ATT_RPW * ATT_BK) * sizeof(float);
    auto kern = paged_attention_kernel<T, DMAX>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-101, "paged_attention: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid((unsigned)tiles, nkv, num_seqs * splits);
    return check_launch("paged_attention", launch(kern, grid, ATT_WARPS * 32, smem, stream,
        (const T*)q, q_row_stride, (const T*)cache, block_table, table_stride, cu_q, seqlens_k,
        (T*)out, part_o, part_ml, nh, nkv, d, page_size, num_pages, scale, window, splits, status));
}

// q: [n, *] with `q_row_stride` elements between tokens, head h at h*d.
// cache: one layer, [num_pages, 2, nkv, page_size, d].  out: [n, nh*d].
// splits > 1 needs part_o [n*nh*splits*d] and part_ml [n*nh*splits*2] floats of scratch.
// impl: 0 = the fastest kernel that applies: for bfloat16, head_dim 64 or 128 and a page size
// that is a multiple of 64 the mma.sync flash kernel; at head_dim 64 the TMA-fed decode kernel for
// steps whose sequences bring at most 16 rows per kv head, and for steps with prompt portions (no
// split) the tcgen05 kernel for every sequence of at least FT_MIN_Q tokens beside the flash
// kernel and the decode kernel for the shorter ones; else the general kernel.  1 = the general kernel; 2 = the mma.sync
// flash kernel or an error; 3 = the tcgen05 kernel for every sequence, or an error; 4 = the
// decode kernel, or an error.
// whether impl 0 may pick the decode kernel (a switch for comparisons; on unless turned off)
static int g_decode_kernel = 1;
VAPI_EXPORT void vapi_attention_use_decode_kernel(int on) { g_decode_kernel = on != 0; }

VAPI_EXPORT int vapi_paged_attention(const void* q, long long q_row_stride, const void* cache,
                                     int dtype, const int* block_table, int table_stride,
                                     const int* cu_q, const int* seqlens_k, void* out,
                                     float* part_o, float* part_ml, int n, int num_seqs,
                                     int max_q, int nh, int nkv, int d, int page_size,
                                     int num_pages, float scale, int window, int splits,
                                     int impl, int* status, cudaStream_t stream) {
    if (n <= 0 || num_seqs <= 0 || max_q <= 0) return 0;
    if (d < 16 || d > 256 || d % 16 != 0)
        return fail(-1, "paged_attention: head_dim %d is not a multiple of 16 in 16..256", d);
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0)
        return fail(-1, "paged_attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    if (page_size <= 0 || num_pages <= 0) return fail(-1, "paged_attention: no pages");
    if (q_row_stride % 4 != 0) return fail(-1, "paged_attention: q row stride %lld is not a multiple of 4", q_row_stride);
    if (splits < 1) splits = 1;
    if (splits > 32) return fail(-1, "paged_attention: %d splits are more than 32", splits);
    if (splits > 1 && (!part_o || !part_ml))
        return fail(-1, "paged_attention: %d splits need scratch buffers", splits);
    int rc;
    const bool fast_ok = dtype == VAPI_BF16 && (d == 64 || d == 128) && page_size % FA_BK == 0 &&
                         q_row_stride % 2 == 0;
    if (impl == 2 && !fast_ok)
        return fail(-3, "paged_attention: the tensor-core kernel needs bfloat16, head_dim 64 or 128 and a page "
                        "size that is a multiple of 64 (got dtype %d, head_dim %d, page size %d)", dtype, d, page_size);
    const bool fast = fast_ok && impl != 1;
    const bool tc_ok = fast_ok && d == FT_HD && splits == 1 && q_row_stride % 8 == 0 && scale > 0.f;
    if (impl == 3 && !tc_ok)
        return fail(-3, "paged_attention: the tcgen05 kernel needs bfloat16, head_dim 64, a page size that is a multiple "
                        "of 64, no split and a positive scale (got dtype %d, head_dim %d, page size %d, %d splits)",
                    dtype, d, page_size, splits);
    if (impl == 3 || (impl == 0 && tc_ok && max_q >= FT_AUTO_MAX_Q)) {
        // prompt portions on tcgen05; in a mixed step the short sequences (decode tokens) go to the
        // flash kernel, whose small blocks suit them: each kernel skips the other's sequences
        const int min_q = (impl == 3 || num_seqs == 1) ? 1 : FT_MIN_Q;
        rc = launch_flash_tc(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, num_seqs, max_q,
                             nh, nkv, page_size, num_pages, scale, window, min_q, status, stream);
        if (rc != 0 || min_q == 1) return rc;
        // (of the shorter ones, those of at most 16 rows - decode tokens, whose contexts can be long -
        // go to the decode kernel, which puts four warps on their keys where the flash kernel has one)
        const bool dec_too = g_decode_kernel && nh / nkv <= FD_MAX_ROWS && ((uintptr_t)out & 15) == 0;
        rc = launch_flash<64, 4, 3>(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o,
                                    part_ml, num_seqs, FT_MIN_Q - 1, nh, nkv, page_size, num_pages, scale, window, 1,
                                    status, stream, FT_MIN_Q, dec_too ? FD_MAX_ROWS : 0);
        if (rc != 0 || !dec_too) return rc;
        return launch_flash_decode(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,
                                   num_seqs, nh, nkv, page_size, num_pages, scale, window, 1, status, stream);
    }
#define VAPI_FLASH(HD, NW, ST)                                                                   \
    rc = launch_flash<HD, NW, ST>(q, q_row_stride, cache, block_table, table_stride, cu_q,       \
                                  seqlens_k, out, part_o, part_ml, num_seqs, max_q, nh, nkv,     \
                                  page_size, num_pages, scale, window, splits, status, stream)
#define VAPI_ATT(T, DM)                                                                         \
    rc = launch_attention<T, DM>(q, q_row_stride, cache, block_table, table_stride, cu_q,       \
                                 seqlens_k, out, part_o, part_ml, num_seqs, max_q, nh, nkv, d,  \
                                 page_size, num_pages, scale, window, splits, status, stream)
    const bool few_rows = (long long)max_q * (nh / nkv) <= FD_MAX_ROWS;
    const bool dec_ok = fast_ok && d == FD_HD && few_rows && ((uintptr_t)out & 15) == 0 && (g_decode_kernel || impl == 4);
    if (impl == 4 && !dec_ok)
        return fail(-3, "paged_attention: the decode kernel needs bfloat16, head_dim 64, a page size that is a multiple of 64 "
                        "and at most 16 rows per sequence and kv head (got dtype %d, head_dim %d, page size %d, %lld rows)",
                    dtype, d, page_size, (long long)max_q * (nh / nkv));
    if (impl == 4 || (impl == 0 && dec_ok)) {
        rc = launch_flash_decode(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,
                                 num_seqs, nh, nkv, page_size, num_pages, scale, window, splits, status, stream);
    } else if (fast && impl == 0 && g_decode_kernel && d == FD_HD && nh / nkv <= FD_MAX_ROWS && ((uintptr_t)out & 15) == 0) {
        // a step with portions of more than 16 rows: those on the four-warp flash kernel, the decode
        // tokens beside them on the decode kernel (its slices, if any, go to the combine kernel with the rest)
        rc = launch_flash<64, 4, 3>(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o,
                                    part_ml, num_seqs, max_q, nh, nkv, page_size, num_pages, scale, window, splits,
                                    status, stream, 0, FD_MAX_ROWS);
        if (rc == 0)
            rc = launch_flash_decode(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,
                                     num_seqs, nh, nkv, page_size, num_pages, scale, window, splits, status, stream, false);
    } else if (fast) {
        if (d == 64) { if (few_rows) VAPI_FLASH(64, 1, 3); else VAPI_FLASH(64, 4, 3); }
        else         { if (few_rows) VAPI_FLASH(128, 1, 3); else VAPI_FLASH(128, 4, 3); }
    } else if (dtype == VAPI_F32) {
        if (d <= 64) VAPI_ATT(float, 64); else if (d <= 128) VAPI_ATT(float, 128); else VAPI_ATT(float, 256);
    } else if (dtype == VAPI_BF16) {
        if (d <= 64) VAPI_ATT(__nv_bfloat16, 64); else if (d <= 128) VAPI_ATT(__nv_bfloat16, 128); else VAPI_ATT(__nv_bfloat16, 256);
    } else {
        return fail(-2, "paged_attention: unsupported dtype %d", dtype);
    }
#undef VAPI_ATT
#undef VAPI_FLASH
    if (rc != 0) return rc;
    const bool combined = (impl == 4 || (impl == 0 && dec_ok)) && flash_decode_combines(num_seqs, nkv, splits);   // the decode kernel's clusters did it
    if (splits > 1 && !combined) {
        const long long rows = (long long)n * nh;
        const int wpb = 4;
        const long long blocks = (rows + wpb - 1) / wpb;
        cudaError_t e;
        if (dtype == VAPI_F32)
            e = launch(attention_combine_kernel<float>, (unsigned)blocks, wpb * 32, 0, stream, (const float*)part_o, (const float*)part_ml, (float*)out, rows, d, splits);
        else
            e = launch(attention_combine_kernel<__nv_bfloat16>, (unsigned)blocks, wpb * 32, 0, stream, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, rows, d, splits);
        return check_launch("attention_combine", e);
    }
    return 0;
}

// How many blocks of the decode kernel the device holds at once (0: unknown), and the largest
// number of key slices that it combines inside the kernel.
VAPI_EXPORT int vapi_decode_attention_slots() { return flash_decode_slots(); }
VAPI_EXPORT int vapi_decode_attention_cluster() { return FD_MAX_CLUSTER; }
// whether the decode kernel would combine the slices of such a step itself (1) or leave them to the combine kernel (0)
VAPI_EXPORT int vapi_decode_attention_combines(int num_seqs, int nkv, int splits) { return flash_decode_combines(num_seqs, nkv, splits) ? 1 : 0; }

// A decode step's attention with what precedes it: qkv [n][(nh + 2 nkv) * 64] is the fused product as
// it was left; the kernel applies the per-head RMSNorm (qw, kw: [64] or null) and rotate-half RoPE
// (cosr, sinr: [n][32] or null) to q and to the new keys, writes the new keys and values into the
// cache (write_kv; 0 for a layer that reads another layer's cache) and attends.  bfloat16, head_dim
// 64, a page size that is a multiple of 64, at most 16 rows per sequence and kv head.  qkv is left
// as it was.  splits > 1: scratch as for vapi_paged_attention.
VAPI_EXPORT int vapi_decode_attention_fused(const void* qkv, const float* qw, const float* kw, float eps,
                                            const float* cosr, const float* sinr, void* cache, int write_kv,
                                            const int* block_table, int table_stride, const int* cu_q,
                                            const int* seqlens_k, void* out, float* part_o, float* part_ml,
                                            int n, int num_seqs, int max_q, int nh, int nkv, int d,
                                            int page_size, int num_pages, float scale, int window, int splits,
                                            int* status, cudaStream_t stream) {
    if (n <= 0 || num_seqs <= 0 || max_q <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0)
        return fail(-1, "decode_attention_fused: %d heads are not a multiple of %d kv heads", nh, nkv);
    if (d != FD_HD || page_size <= 0 || page_size % FD_BK != 0 || num_pages <= 0 || (long long)max_q * (nh / nkv) > FD_MAX_ROWS)
        return fail(-3, "decode_attention_fused: needs head_dim 64, a page size that is a multiple of 64 and at most 16 rows "
                        "per sequence and kv head (got head_dim %d, page size %d, %lld rows)", d, page_size,
                    (long long)max_q * (nh / nkv));
    if ((cosr == nullptr) != (sinr == nullptr)) return fail(-1, "decode_attention_fused: cos and sin come together");
    if (splits < 1) splits = 1;
    if (splits > 32) return fail(-1, "decode_attention_fused: %d splits are more than 32", splits);
    if (splits > 1 && (!part_o || !part_ml)) return fail(-1, "decode_attention_fused: %d splits need scratch buffers", splits);
    if (((uintptr_t)out & 15) != 0) return fail(-1, "decode_attention_fused: the output is not 16-byte aligned");
    FdParams f = {};
    f.write_kv = write_kv ? 1 : 0; f.qw = qw; f.kw = kw; f.eps = eps; f.cosr = cosr; f.sinr = sinr;
    const long long stride = (long long)(nh + 2 * nkv) * d;
    int rc = launch_flash_decode(qkv, stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,
                                 num_seqs, nh, nkv, page_size, num_pages, scale, window, splits, status, stream, true, &f);
    if (rc != 0) return rc;
    if (splits > 1 && !flash_decode_combines(num_seqs, nkv, splits)) {
        const long long rows = (long long)n * nh;
        const int wpb = 4;
        const long long blocks = (rows + wpb - 1) / wpb;
        return check_launch("attention_combine", launch(attention_combine_kernel<__nv_bfloat16>, (unsigned)blocks, wpb * 32, 0, stream,
                                                        (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, rows, d, splits));
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The same attention with its scratch inside the library (see attention_noalloc.h for who needs
// this and what it costs).  In host code the name of a __device__ array is only a handle: the
// address a kernel can use has to be asked for, once per device, with that device current.
#include "attention_noalloc.h"

static __device__ __align__(256) float vapi_attn_noalloc_scratch[VAPI_ATTN_NOALLOC_MAX_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* noalloc_scratch_addr[NOALLOC_MAX_DEVICES] = {nullptr};

VAPI_EXPORT int vapi_paged_attention_noalloc(const void* q, long long q_row_stride, const void* cache,
                                             int dtype, const int* block_table, int table_stride,
                                             const int* cu_q, const int* seqlens_k, void* out, int n,
                                             int num_seqs, int max_q, int nh, int nkv, int d,
                                             int page_size, int num_pages, float scale, int window,
                                             int splits, int impl, int* status, cudaStream_t stream) {
    if (splits < 1) splits = 1;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (splits > 1 && n > 0) {
        const long long rows = (long long)n * nh * splits;
        const long long need = rows * ((long long)d + 2);
        if (nh <= 0 || d <= 0 || need > VAPI_ATTN_NOALLOC_MAX_FLOATS)
            return fail(-4, "paged_attention_noalloc: %d tokens x %d heads x %d splits x (head size %d + 2) = %lld floats "
                            "of scratch, the built-in array holds %d", n, nh, splits, d, need, VAPI_ATTN_NOALLOC_MAX_FLOATS);
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES)
            return fail(-5, "paged_attention_noalloc: cannot tell the current device: %s", cudaGetErrorString(e));
        if (!noalloc_scratch_addr[dev]) {                  // set-up: once per device, before any capture
            float* addr = nullptr;
            e = cudaGetSymbolAddress((void**)&addr, vapi_attn_noalloc_scratch);
            if (e != cudaSuccess || !addr)
                return fail(-6, "paged_attention_noalloc: the scratch array has no address on device %d: %s", dev, cudaGetErrorString(e));
            noalloc_scratch_addr[dev] = addr;
        }
        part_o = noalloc_scratch_addr[dev];
        part_ml = part_o + rows * d;                       // rows * d is a multiple of 16 floats: stays aligned
    }
    return vapi_paged_attention(q, q_row_stride, cache, dtype, block_table, table_stride, cu_q, seqlens_k, out,
                                part_o, part_ml, n, num_seqs, max_q, nh, nkv, d, page_size, num_pages, scale,
                                window, splits, impl, status, stream);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
