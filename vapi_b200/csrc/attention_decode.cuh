// Paged GQA attention for decode steps: bfloat16, head_dim 64, pages whose size is a multiple of
// 64, sequences that bring at most 16 rows (query tokens x q heads of one kv head).  The step reads
// every key and value of every live request once, so the kernel is built around that stream:
//
//   * a block owns one (sequence, kv head, slice of the keys) and has five warps.  One is the
//     producer: it looks the pages up in the block table (32 entries at a time, one per lane)
//     and brings each 64-key tile of K and of V in with one TMA copy each (a tensor map over the
//     cache layer as rows of 64 bfloat16, 128-byte swizzle), into a ring of stages guarded by
//     full/empty mbarriers.  Tiles that hold only keys of earlier steps are requested before the
//     wait for the kernel that wrote this step's keys.
//   * the four consumer warps share every tile: warp w takes keys 16w..16w+15 of it, computes
//     S = Q.K^T for them (mma.sync m16n8k16, the up-to-16 rows as M), keeps an online softmax of
//     its own over its keys (float registers, base 2) and adds P.V into its own accumulator.  Four
//     warps on one tile mean four times the warps for the same bytes in flight, which is what a
//     stream of this kind needs: one warp per tile spends its time on dependent instructions.
//   * at the end the four partial results are merged through shared memory, in warp order, and
//     written as the final bfloat16 output, or as this slice's partial result for the combine
//     kernel.
//
// Keys beyond the sequence's end are masked, and their V rows (memory that was never written)
// are zeroed in shared memory before they are multiplied by a zero weight.  Every mbarrier wait
// is bounded; when one runs out the block records status 16 and writes nothing.
#pragma once
#include "attention_mma.cuh"
#include "tcgen05.cuh"

namespace vapi {

constexpr int FD_BK = 64;
constexpr int FD_HD = 64;
constexpr int FD_CWARPS = 4;                               // consumer warps: 16 keys of every tile each
constexpr int FD_THREADS = (FD_CWARPS + 1) * 32;
constexpr int FD_MAX_ROWS = 16;
#ifndef FD_MAX_CLUSTER_N
#define FD_MAX_CLUSTER_N 16
#endif
constexpr int FD_MAX_CLUSTER = FD_MAX_CLUSTER_N;           // slices of the keys that combine inside the kernel (above 8: a cluster size the device must allow)
constexpr int FD_TILE_BYTES = FD_BK * FD_HD * 2;           // one K (or V) tile
#ifndef FD_STAGES_N
#define FD_STAGES_N 4
#endif
constexpr int FD_STAGES = FD_STAGES_N;
#ifndef FD_MIN_BLOCKS_N
#define FD_MIN_BLOCKS_N 3
#endif
constexpr size_t FD_SMEM = (size_t)FD_STAGES * 2 * FD_TILE_BYTES + 1024;     // + room to align to the swizzle's 1024 bytes
static_assert(FD_STAGES * 2 * FD_TILE_BYTES >= (FD_CWARPS + 1) * FD_MAX_ROWS * FD_HD * 4, "the merge reuses the stages");

struct FdParams {
    const __nv_bfloat16* q; long long q_row_stride;
    const int* block_table; int table_stride;
    const int* cu_q; const int* seqlens_k;
    __nv_bfloat16* out; float* part_o; float* part_ml;
    int nh, nkv, page_size, num_pages;
    float scale_log2e; int window, splits;
    int* status;
    // fused mode (fused != 0): q points at this step's fused qkv rows [n][(nh + 2 nkv) * 64] as the product
    // left them; the kernel norms and rotates q itself and, with write_kv, norms and rotates the new keys,
    // writes them and the new values into the cache and into the tiles it has in shared memory
    int fused, write_kv;
    const float* qw; const float* kw; float eps;       // per-head RMSNorm weights [64] or null
    const float* cosr; const float* sinr;              // [n][32] or null
    __nv_bfloat16* cache;
};

// eight bfloat16 (16 bytes) to floats and back
__device__ __forceinline__ void fd_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 fd_pack8(const float (&v)[8]) {
    return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

__device__ __forceinline__ void fd_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned fd_peer(const void* local, unsigned rank) {     // this address in the shared memory of block `rank`
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ float fd_peer_f32(unsigned addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float4 fd_peer_f32x4(unsigned addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// CLUSTER: the blocks of one (sequence, kv head) - its slices of the keys, at most 16 (above 8 a cluster size that the device has to allow; asked once) - form a
// thread-block cluster; each leaves its partial result in its own shared memory and, after a
// cluster barrier, they share out the rows' final sums among themselves (slice sp is rank sp).
// FUSED: q/k norm, RoPE and the cache write of the new tokens happen here too (FdParams::fused).
template <bool CLUSTER, bool FUSED>
__global__ void __launch_bounds__(FD_THREADS, FD_MIN_BLOCKS_N)
flash_decode_kernel(const __grid_constant__ CUtensorMap tm_kv, const FdParams p) {
    extern __shared__ unsigned char fd_smem_raw[];
    unsigned char* sKV = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fd_smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bars[2 * FD_STAGES];
    __shared__ float sM[FD_CWARPS][FD_MAX_ROWS], sL[FD_CWARPS][FD_MAX_ROWS];
    __shared__ float xM[FD_MAX_ROWS], xL[FD_MAX_ROWS];          // CLUSTER: this slice's result, read by its peers
    // fused mode: the rows' queries and the new tokens' keys and values, normed and rotated
    constexpr int FR = FUSED ? FD_MAX_ROWS : 1;
    __shared__ __align__(16) __nv_bfloat16 sQ[FR][FD_HD], sKn[FR][FD_HD], sVn[FR][FD_HD];
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.z / p.splits, sp = blockIdx.z - s * p.splits;
    const int g = blockIdx.y;
    pdl_trigger();
    // index data was copied from the host before the step's first kernel: safe before the wait
    const int q0 = p.cu_q[s], qlen = p.cu_q[s + 1] - q0, klen = p.seqlens_k[s];
    const int n_rep = p.nh / p.nkv;
    const int rows_total = qlen * n_rep;
    if (rows_total <= 0 || rows_total > FD_MAX_ROWS) {         // longer portions belong to another kernel
        pdl_wait();
        return;
    }
    const int base_pos = klen - qlen;
    const int p_min = base_pos, p_max = klen - 1;
    const int key_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt_lo = key_lo / FD_BK, kt_hi = p_max / FD_BK;
    const int ntiles_all = kt_hi - kt_lo + 1;
    const int chunk = (ntiles_all + p.splits - 1) / p.splits;
    const int kt_begin = kt_lo + sp * chunk;
    const int kt_end = min(kt_hi + 1, kt_begin + chunk);
    const int nt = max(0, kt_end - kt_begin);

    const unsigned full = smem_u32(bars), empty = smem_u32(bars + FD_STAGES);
    if (threadIdx.x == 0) {
        for (int i = 0; i < FD_STAGES; ++i) { mbar_init(full + 8 * i, 1); mbar_init(empty + 8 * i, FD_CWARPS); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o_acc[FD_HD / 8][4];
#pragma unroll
    for (int i = 0; i < FD_HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    const int gq = lane >> 2, tq = lane & 3;                          // row / column pair of the fragments
    int row_tok[2], row_head[2], row_pos[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int rr = gq + 8 * h;
        row_ok[h] = rr < rows_total;
        row_tok[h] = row_ok[h] ? rr / n_rep : 0;
        row_head[h] = g * n_rep + (row_ok[h] ? rr - row_tok[h] * n_rep : 0);
        row_pos[h] = row_ok[h] ? base_pos + row_tok[h] : -1;          // -1: sees nothing
    }
    bool ok = true;

    if (warp == FD_CWARPS) {
        // ---- producer ----
        const int* bt = p.block_table + (size_t)s * p.table_stride;
        const int kt_old_end = base_pos / FD_BK;                      // tiles before this one hold keys of earlier steps only
        bool waited = false;
        int pg_base = -(1 << 30), entry = 0;
        for (int it = 0; it < nt; ++it) {
            const int kt = kt_begin + it, k0 = kt * FD_BK, stage = it % FD_STAGES;
            if (!waited && kt >= kt_old_end && !(FUSED && p.write_kv)) {
                pdl_wait();                                           // this step's keys are in the cache now
                waited = true;                                        // (fused and writing: the consumers put them into the tile)
            }
            const int pg = k0 / p.page_size;
            if (pg - pg_base >= 32) {
                pg_base = pg;
                const int last_pg = p_max / p.page_size;
                entry = pg + lane <= last_pg ? bt[pg + lane] : 0;
            }
            int page = __shfl_sync(0xffffffffu, entry, pg - pg_base);
            if (page < 0 || page >= p.num_pages) {
                if (lane == 0 && p.status) atomicExch(p.status, 4);
                page = 0;
            }
            int good = 1;
            if (lane == 0) {
                if (it >= FD_STAGES && !mbar_wait(empty + 8 * stage, ((it / FD_STAGES) - 1) & 1)) good = 0;
                if (good) {
                    const int row = ((page * 2) * p.nkv + g) * p.page_size + (k0 % p.page_size);
                    const unsigned dst = smem_u32(sKV + (size_t)stage * 2 * FD_TILE_BYTES);
                    mbar_expect_tx(full + 8 * stage, 2 * FD_TILE_BYTES);
                    tma_load_2d(dst, &tm_kv, full + 8 * stage, 0, row);
                    tma_load_2d(dst + FD_TILE_BYTES, &tm_kv, full + 8 * stage, 0, row + p.nkv * p.page_size);
                }
            }
            if (!__shfl_sync(0xffffffffu, good, 0)) { ok = false; break; }
        }
        if (!waited) pdl_wait();
    } else {
        // ---- consumers ----
        pdl_wait();                                                   // q (or qkv) comes from the kernel before this one
        if (FUSED) {
            // Four lanes per item, eight low and eight high elements each, as in the stand-alone kernel
            // for this (rope.cu), sums in the same order: the rows' queries, then the keys and the values
            // of the new tokens whose tile belongs to this block.
            const int sub = threadIdx.x & 3, e = sub * 8;
            for (int item = threadIdx.x >> 2; item < 3 * FD_MAX_ROWS; item += FD_CWARPS * 8) {
                const int kind = item / FD_MAX_ROWS, idx = item - kind * FD_MAX_ROWS;     // 0 q, 1 k, 2 v
                bool active;
                int tok, col;
                if (kind == 0) {
                    active = idx < rows_total;
                    tok = active ? idx / n_rep : 0;
                    col = g * n_rep + (active ? idx - tok * n_rep : 0);
                } else {
                    const int kt_own = (base_pos + idx) / FD_BK;
                    active = p.write_kv && idx < qlen && kt_own >= kt_begin && kt_own < kt_end;
                    tok = active ? idx : 0;
                    col = kind == 1 ? p.nh + g : p.nh + p.nkv + g;
                }
                const __nv_bfloat16* src = p.q + (size_t)(q0 + tok) * p.q_row_stride + (size_t)col * FD_HD;
                float lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) lo[i] = hi[i] = 0.f;
                if (active) {
                    fd_load8(src + e, lo);
                    fd_load8(src + FD_HD / 2 + e, hi);
                }
                const float* w = kind == 0 ? p.qw : (kind == 1 ? p.kw : nullptr);
                float inv = 1.f;
                if (p.qw || p.kw) {                                   // (uniform: every lane takes part in the shuffles)
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
                    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                    inv = rsqrtf(ss / (float)FD_HD + p.eps);
                }
                if (!active) continue;
                if (w) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        lo[i] = lo[i] * inv * w[e + i];
                        hi[i] = hi[i] * inv * w[FD_HD / 2 + e + i];
                    }
                }
                if (kind != 2 && p.cosr) {
                    const float* c = p.cosr + (size_t)(q0 + tok) * (FD_HD / 2) + e;
                    const float* sn = p.sinr + (size_t)(q0 + tok) * (FD_HD / 2) + e;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a = lo[i], b = hi[i];
                        lo[i] = a * c[i] - b * sn[i];
                        hi[i] = b * c[i] + a * sn[i];
                    }
                }
                const uint4 plo = fd_pack8(lo), phi = fd_pack8(hi);
                __nv_bfloat16* dst = kind == 0 ? sQ[FUSED ? idx : 0] : (kind == 1 ? sKn[FUSED ? idx : 0] : sVn[FUSED ? idx : 0]);
                *reinterpret_cast<uint4*>(dst + e) = plo;
                *reinterpret_cast<uint4*>(dst + FD_HD / 2 + e) = phi;
                if (kind != 0) {
                    // the cache gets the new token too (later steps read it from there)
                    const int pos = base_pos + idx;
                    const int page = p.block_table[(size_t)s * p.table_stride + pos / p.page_size];
                    if (page < 0 || page >= p.num_pages) {
                        if (sub == 0 && p.status) atomicExch(p.status, 2);
                    } else {
                        __nv_bfloat16* cd = p.cache + ((((size_t)page * 2 + (kind == 1 ? 0 : 1)) * p.nkv + g) * p.page_size + pos % p.page_size) * FD_HD;
                        *reinterpret_cast<uint4*>(cd + e) = plo;
                        *reinterpret_cast<uint4*>(cd + FD_HD / 2 + e) = phi;
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(FD_CWARPS * 32) : "memory");       // the consumers only
        }
        unsigned qf[FD_HD / 16][4];
#pragma unroll
        for (int kk = 0; kk < FD_HD / 16; ++kk) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                unsigned lo = 0u, hi = 0u;
                if (row_ok[h]) {
                    const __nv_bfloat16* src = FUSED ? &sQ[FUSED ? gq + 8 * h : 0][kk * 16 + 2 * tq]
                                                       : p.q + (size_t)(q0 + row_tok[h]) * p.q_row_stride + (size_t)row_head[h] * FD_HD + kk * 16 + 2 * tq;
                    lo = *reinterpret_cast<const unsigned*>(src);
                    hi = *reinterpret_cast<const unsigned*>(src + 8);
                }
                qf[kk][h] = lo;
                qf[kk][2 + h] = hi;
            }
        }
        const int mat = lane >> 3, rin = lane & 7;
        for (int it = 0; it < nt; ++it) {
            const int k0 = (kt_begin + it) * FD_BK, stage = it % FD_STAGES;
            const int kw = k0 + warp * 16;                            // this warp's first key of the tile
            if (!__all_sync(0xffffffffu, mbar_wait(full + 8 * stage, (it / FD_STAGES) & 1))) { ok = false; break; }
            // a warp whose keys no row can see (beyond the newest position, behind every window) skips them
            const bool skip = kw > p_max || (p.window > 0 && kw + 15 <= p_min - p.window);
            if (!skip) {
                const __nv_bfloat16* ks = reinterpret_cast<const __nv_bfloat16*>(sKV + (size_t)stage * 2 * FD_TILE_BYTES);
                __nv_bfloat16* vs = reinterpret_cast<__nv_bfloat16*>(sKV + (size_t)stage * 2 * FD_TILE_BYTES + FD_TILE_BYTES);
                if (FUSED && p.write_kv && k0 + FD_BK > base_pos) {
                    // new tokens of this tile: their rows in the cache may be older than the copy, so the
                    // warp that owns a row puts the key and the value in by hand (lanes 0..7 the key's
                    // eight 16-byte pieces, lanes 8..15 the value's)
                    const int j_end = min(qlen, k0 + FD_BK - base_pos);
                    for (int j = max(0, k0 - base_pos); j < j_end; ++j) {
                        const int r = base_pos + j - k0;
                        if ((r >> 4) == warp && lane < 16) {
                            const int c = lane & 7;
                            const __nv_bfloat16* from = (lane < 8 ? sKn[FUSED ? j : 0] : sVn[FUSED ? j : 0]) + c * 8;
                            __nv_bfloat16* to = (lane < 8 ? const_cast<__nv_bfloat16*>(ks) : vs) + r * FD_HD + ((c ^ (r & 7)) << 3);
                            *reinterpret_cast<uint4*>(to) = *reinterpret_cast<const uint4*>(from);
                        }
                    }
                    fence_proxy_async();                              // the stage's next writer is a TMA copy
                    __syncwarp();
                }
                float sc[2][4];
#pragma unroll
                for (int i = 0; i < 2; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < FD_HD / 16; ++kk) {
                    const int key = warp * 16 + (mat >> 1) * 8 + rin;
                    const int ch = kk * 2 + (mat & 1);
                    unsigned r0, r1, r2, r3;
                    ldmatrix_x4(r0, r1, r2, r3, ks + key * FD_HD + ((ch ^ (key & 7)) << 3));
                    mma_bf16_16816(sc[0], qf[kk], r0, r1);
                    mma_bf16_16816(sc[1], qf[kk], r2, r3);
                }
                if (kw + 16 > klen) {
                    // V rows of keys beyond the sequence: zero them (two lanes per row of 128 bytes)
                    const int r = warp * 16 + (lane >> 1);
                    if (k0 + r >= klen) {
                        uint4* vr = reinterpret_cast<uint4*>(vs + r * FD_HD) + (lane & 1) * 4;
#pragma unroll
                        for (int c = 0; c < 4; ++c) vr[c] = make_uint4(0u, 0u, 0u, 0u);
                        fence_proxy_async();                          // the stage's next writer is a TMA copy
                    }
                    __syncwarp();
                }
                const bool need_mask = (kw + 15 > p_min) || (kw + 16 > klen) || (p.window > 0 && kw <= p_max - p.window);
                float alpha[2];
                bool grew = false;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float mx = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            float v = sc[i][2 * h + e] * p.scale_log2e;
                            if (need_mask) {
                                const int kj = kw + i * 8 + 2 * tq + e;
                                const bool vis = kj <= row_pos[h] && kj < klen && (p.window <= 0 || kj > row_pos[h] - p.window);
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
                    alpha[h] = exp2f(m_run[h] - m_use);
                    grew = grew || m_new > m_run[h];
                    float rs = 0.f;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float pe = exp2f(sc[i][2 * h + e] - m_use);
                            sc[i][2 * h + e] = pe;
                            rs += pe;
                        }
                    }
                    l_run[h] = l_run[h] * alpha[h] + rs;        // per-thread part of the row sum; quad-reduced at the end
                    m_run[h] = m_new;
                }
                if (__any_sync(0xffffffffu, grew)) {            // the maximum moves in the first tiles and rarely later
#pragma unroll
                    for (int i = 0; i < FD_HD / 8; ++i) {
                        o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
                        o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
                    }
                }
                unsigned pa[4];
                pa[0] = pack_bf16(sc[0][0], sc[0][1]);
                pa[1] = pack_bf16(sc[0][2], sc[0][3]);
                pa[2] = pack_bf16(sc[1][0], sc[1][1]);
                pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
                for (int nd = 0; nd < FD_HD / 16; ++nd) {
                    const int key = warp * 16 + (mat & 1) * 8 + rin;
                    const int ch = nd * 2 + (mat >> 1);
                    unsigned r0, r1, r2, r3;
                    ldmatrix_x4_trans(r0, r1, r2, r3, vs + key * FD_HD + ((ch ^ (key & 7)) << 3));
                    mma_bf16_16816(o_acc[2 * nd], pa, r0, r1);
                    mma_bf16_16816(o_acc[2 * nd + 1], pa, r2, r3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + 8 * stage);
        }
    }

    if (!ok) failed = 1;
    __syncthreads();                                                  // every tile that was requested has arrived and been used
    if (failed) {
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, 16);
        if (CLUSTER) {                                                // the peers wait for this block at both barriers
            fd_cluster_sync();
            fd_cluster_sync();
        }
        return;
    }
    // ---- merge the four warps' partial results ----
    float* sO = reinterpret_cast<float*>(sKV);                        // [warp][16 rows][64]
    float* xO = sO + FD_CWARPS * FD_MAX_ROWS * FD_HD;                 // CLUSTER: [16 rows][64], behind it
    if (warp < FD_CWARPS) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float l = l_run[h];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const int r = gq + 8 * h;
            if (tq == 0) { sM[warp][r] = m_run[h]; sL[warp][r] = l; }
#pragma unroll
            for (int i = 0; i < FD_HD / 8; ++i)
                *reinterpret_cast<float2*>(sO + ((size_t)warp * FD_MAX_ROWS + r) * FD_HD + i * 8 + 2 * tq) =
                    make_float2(o_acc[i][2 * h], o_acc[i][2 * h + 1]);
        }
    }
    __syncthreads();
    const int r = threadIdx.x >> 3, c0 = (threadIdx.x & 7) * 8;      // a row and 8 of its 64 columns
    const bool mine = warp < FD_CWARPS && r < rows_total;
    const int tok = mine ? r / n_rep : 0, head = g * n_rep + (mine ? r - tok * n_rep : 0);
    const size_t grow = (size_t)(q0 + tok) * p.nh + head;
    if (mine) {
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < FD_CWARPS; ++w) m = fmaxf(m, sM[w][r]);
        const float m_use = m == -INFINITY ? 0.f : m;
        float l = 0.f, o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) o[c] = 0.f;
#pragma unroll
        for (int w = 0; w < FD_CWARPS; ++w) {
            const float a = exp2f(sM[w][r] - m_use);              // -inf: 0
            l += sL[w][r] * a;
            const float4 x0 = *reinterpret_cast<const float4*>(sO + ((size_t)w * FD_MAX_ROWS + r) * FD_HD + c0);
            const float4 x1 = *reinterpret_cast<const float4*>(sO + ((size_t)w * FD_MAX_ROWS + r) * FD_HD + c0 + 4);
            o[0] += x0.x * a; o[1] += x0.y * a; o[2] += x0.z * a; o[3] += x0.w * a;
            o[4] += x1.x * a; o[5] += x1.y * a; o[6] += x1.z * a; o[7] += x1.w * a;
        }
        if (p.splits == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            uint4 w4;
            w4.x = pack_bf16(o[0] * inv, o[1] * inv); w4.y = pack_bf16(o[2] * inv, o[3] * inv);
            w4.z = pack_bf16(o[4] * inv, o[5] * inv); w4.w = pack_bf16(o[6] * inv, o[7] * inv);
            *reinterpret_cast<uint4*>(p.out + grow * FD_HD + c0) = w4;
        } else if (CLUSTER) {
            *reinterpret_cast<float4*>(xO + r * FD_HD + c0) = make_float4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<float4*>(xO + r * FD_HD + c0 + 4) = make_float4(o[4], o[5], o[6], o[7]);
            if ((threadIdx.x & 7) == 0) { xM[r] = m; xL[r] = l; }
        } else {
            float* po = p.part_o + (grow * p.splits + sp) * (size_t)FD_HD + c0;
            *reinterpret_cast<float4*>(po) = make_float4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<float4*>(po + 4) = make_float4(o[4], o[5], o[6], o[7]);
            if ((threadIdx.x & 7) == 0) {
                // the combine step works with natural-log maxima
                p.part_ml[(grow * p.splits + sp) * 2] = m == -INFINITY ? -INFINITY : m * 0.6931471805599453f;
                p.part_ml[(grow * p.splits + sp) * 2 + 1] = l;
            }
        }
    }
    if (CLUSTER && p.splits > 1) {
        fd_cluster_sync();                                            // every slice's result is in place
        // the (row, 8 columns) pieces go round the slices; each sums its pieces over all slices, in slice order
        if (mine && (int)(threadIdx.x % (unsigned)p.splits) == sp) {
            float m = -INFINITY;
            for (int j = 0; j < p.splits; ++j) m = fmaxf(m, fd_peer_f32(fd_peer(&xM[r], (unsigned)j)));
            const float m_use = m == -INFINITY ? 0.f : m;
            float l = 0.f, o[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) o[c] = 0.f;
            for (int j = 0; j < p.splits; ++j) {
                const float a = exp2f(fd_peer_f32(fd_peer(&xM[r], (unsigned)j)) - m_use);
                l += fd_peer_f32(fd_peer(&xL[r], (unsigned)j)) * a;
                const unsigned src = fd_peer(xO + r * FD_HD + c0, (unsigned)j);
                const float4 x0 = fd_peer_f32x4(src), x1 = fd_peer_f32x4(src + 16);
                o[0] += x0.x * a; o[1] += x0.y * a; o[2] += x0.z * a; o[3] += x0.w * a;
                o[4] += x1.x * a; o[5] += x1.y * a; o[6] += x1.z * a; o[7] += x1.w * a;
            }
            const float inv = l > 0.f ? 1.f / l : 0.f;
            uint4 w4;
            w4.x = pack_bf16(o[0] * inv, o[1] * inv); w4.y = pack_bf16(o[2] * inv, o[3] * inv);
            w4.z = pack_bf16(o[4] * inv, o[5] * inv); w4.w = pack_bf16(o[6] * inv, o[7] * inv);
            *reinterpret_cast<uint4*>(p.out + grow * FD_HD + c0) = w4;
        }
        fd_cluster_sync();                                            // nobody reads this block's memory any more
    }
}

static int make_kv_map(CUtensorMap* map, const void* cache, long long rows);

// blocks of the decode kernel that one device holds at a time
static int flash_decode_slots() {
    static int slots = 0;
    if (slots == 0) {
        int dev = 0, sms = 0, per_sm = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cudaFuncSetAttribute(flash_decode_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, flash_decode_kernel<false, false>, FD_THREADS, FD_SMEM) != cudaSuccess) return 0;
        slots = sms * per_sm;
    }
    return slots;
}
// Whether the slices of the keys combine inside the kernel, as clusters: only while the whole grid
// is resident at once.  With more blocks than that, clusters (which start together and leave
// together) keep places occupied that single blocks would give up as they finish.
static bool flash_decode_combines(int num_seqs, int nkv, int splits) {
    if (splits <= 1 || splits > FD_MAX_CLUSTER || (long long)num_seqs * nkv * splits > flash_decode_slots()) return false;
    // a cluster of this size must fit the device at all (asked once per size)
    static int fits[FD_MAX_CLUSTER + 1] = {};              // 0 unknown, 1 yes, -1 no
    if (fits[splits] == 0) {
        cudaFuncSetAttribute(flash_decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM);
        if (FD_MAX_CLUSTER > 8) {
            cudaFuncSetAttribute(flash_decode_kernel<true, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(flash_decode_kernel<true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, (unsigned)splits);
        cfg.blockDim = dim3(FD_THREADS);
        cfg.dynamicSmemBytes = FD_SMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = (unsigned)splits;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, flash_decode_kernel<true, false>, &cfg);
        if (e != cudaSuccess) cudaGetLastError();
        fits[splits] = (e == cudaSuccess && clusters > 0) ? 1 : -1;
    }
    return fits[splits] == 1;
}

static int launch_flash_decode(const void* q, long long q_row_stride, const void* cache, const int* block_table,
                               int table_stride, const int* cu_q, const int* seqlens_k, void* out, float* part_o,
                               float* part_ml, int num_seqs, int nh, int nkv, int page_size, int num_pages,
                               float scale, int window, int splits, int* status, cudaStream_t stream,
                               bool may_combine = true, const FdParams* fused = nullptr) {
    if (nkv > 65535 || (long long)num_seqs * splits > 65535)
        return fail(-1, "paged_attention: %d kv heads or %d sequences x %d splits exceed the grid", nkv, num_seqs, splits);
    if (q_row_stride % 2 != 0 || ((uintptr_t)q & 3) != 0 || ((uintptr_t)out & 15) != 0)
        return fail(-1, "paged_attention: the decode kernel needs 4-byte aligned query rows and a 16-byte aligned output");
    CUtensorMap map;
    int rc = make_kv_map(&map, cache, (long long)num_pages * 2 * nkv * page_size);
    if (rc != 0) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_decode_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_decode_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM);
        if (e != cudaSuccess) return fail(-101, "paged_attention: cannot reserve %zu bytes of shared memory: %s", FD_SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    FdParams p;
    p.q = (const __nv_bfloat16*)q; p.q_row_stride = q_row_stride; p.block_table = block_table; p.table_stride = table_stride;
    p.cu_q = cu_q; p.seqlens_k = seqlens_k; p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_ml = part_ml;
    p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.num_pages = num_pages; p.scale_log2e = scale * 1.4426950408889634f;
    p.window = window; p.splits = splits; p.status = status;
    p.fused = 0; p.write_kv = 0; p.qw = p.kw = nullptr; p.eps = 0.f; p.cosr = p.sinr = nullptr; p.cache = nullptr;
    if (fused) {
        if (q_row_stride % 8 != 0 || ((uintptr_t)q & 15) != 0)
            return fail(-1, "paged_attention: the fused decode kernel needs 16-byte aligned qkv rows");
        p.fused = 1; p.write_kv = fused->write_kv; p.qw = fused->qw; p.kw = fused->kw; p.eps = fused->eps;
        p.cosr = fused->cosr; p.sinr = fused->sinr; p.cache = (__nv_bfloat16*)const_cast<void*>(cache);
    }
    dim3 grid(1, nkv, num_seqs * splits);
    if (may_combine && flash_decode_combines(num_seqs, nkv, splits)) {
        // the slices of one (sequence, kv head) are a cluster along z and combine among themselves
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(FD_THREADS);
        cfg.dynamicSmemBytes = FD_SMEM;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = (unsigned)splits;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        return check_launch("paged_attention (decode, cluster)",
                            fused ? cudaLaunchKernelEx(&cfg, flash_decode_kernel<true, true>, map, p)
                                  : cudaLaunchKernelEx(&cfg, flash_decode_kernel<true, false>, map, p));
    }
    return check_launch("paged_attention (decode)",
                        fused ? launch(flash_decode_kernel<false, true>, grid, FD_THREADS, FD_SMEM, stream, map, p)
                              : launch(flash_decode_kernel<false, false>, grid, FD_THREADS, FD_SMEM, stream, map, p));
}

}  // namespace vapi
