// Weight-streaming matrix product for decode steps: y[m][n] = sum_k a[m][k] * W[n][k] with
// few rows m (up to 16 tokens) against a large bfloat16 weight.  At these sizes the product is
// bound by reading W once from HBM, so the kernel is organised around that stream:
//
//  * W is the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the tokens are the n
//    dimension (8 per tile).  Each lane reads 16 contiguous bytes of a weight row straight from
//    global memory into its fragment registers.  That is legal because a dot product does not
//    care about the order of k: lane (g, t) takes physical k = 32c + 8t .. 8t+7 of rows g and
//    g+8, uses elements 0..3 for one MMA and 4..7 for the next, and the activation fragment is
//    read with exactly the same mapping.  The 16-byte pieces travel by cp.async through a
//    small per-lane queue in shared memory (a lane reads back only what it queued itself), so
//    several chunks are always in flight whatever the arithmetic is doing, and there is no
//    barrier in the loop.
//  * the 8 warps of a block split K and add their partial tiles in a fixed order through shared
//    memory (deterministic: no atomics), then one thread per output applies the epilogue.  (For
//    9..16 tokens a block has 16 warps, as one group or as two groups of 8: see GV_WIDE_WARPS.)
//  * prologue (what the token operand is): bfloat16 activations, or the residual stream seen
//    through an RMSNorm that was not applied yet.  RMSNorm is x * w * rsqrt(mean x^2 + eps): the
//    last factor is one number per token, so the product runs on bfloat16(x * w), which the
//    producer of x left beside it, and the epilogue multiplies each token's column by its factor,
//    taken from the partial sums of squares the producer left (summed here in a fixed order).
//  * epilogue: bfloat16 out (+bias) | float out (logits) | SwiGLU (a block owns 8 gate rows and
//    the 8 matching up rows, so silu(gate)*up happens before anything is stored) | add into the
//    float residual stream (+bias), leaving for the norm that follows the partial sums of squares
//    of the new stream values and bfloat16(new value * that norm's weight) | the whole gated
//    short convolution of a decode step (W is the mixer's in_proj; a block owns the B, C and x
//    rows of 8 channels, so gate, taps over the request's state, C * conv and the state update
//    happen before anything is stored; every token must be a sequence of its own).
//
// The reference does these products with cuBLAS and separate norm / SwiGLU / add kernels
// (crates/vapi-backend-candle/src/models/lfm2.rs:519-534, 591-593, 645-647).
#include "tcgen05.cuh"
#include <unordered_map>

using namespace vapi;

constexpr int GV_WARPS = 8;
// For 9..16 tokens the tokens' rows take 66 KB of a block's shared memory at K = 2048, so that two blocks
// of eight warps have room for four stages each: too few bytes in flight.  One block of sixteen warps
// shares one copy of the rows and has the room for a full queue per warp; it is used where it fits.
constexpr int GV_WIDE_WARPS = 16;
#ifndef GV_STAGES_N
#define GV_STAGES_N 8
#endif
#ifndef GV_DEEP_STAGES_N
#define GV_DEEP_STAGES_N 16
#endif
constexpr int GV_DEEP_STAGES = GV_DEEP_STAGES_N;
#ifndef GV_NT2_STAGES_N
#define GV_NT2_STAGES_N 4
#endif
constexpr int GV_NT2_STAGES = GV_NT2_STAGES_N;      // queue depth for 9..16 tokens: with 16 staged rows, two blocks fit on an SM only at 4
constexpr int GV_STAGES_DEFAULT = GV_STAGES_N;   // depth of the per-lane copy queue (chunks of 32 k)
// the conv epilogue streams three weight rows per lane: six stages keep two blocks on an SM
// (DEEP: a product with a long K and no more tiles than SMs has one block per SM anyway and takes
// a deeper queue instead of a second block)
// (16 stages of 3 slots for up to 8 tokens, 12 of 4 slots for up to 16: 196 KB either way)
#ifndef GV_REGB_STAGES_N
#define GV_REGB_STAGES_N 12
#endif
// REGB: the tokens' operand is kept in registers (see the kernel), so the queue holds weights only and the
// room that the staged rows took goes to more stages: 12 of two weight rows (96 KB a block, two blocks on
// an SM), 8 of three for the conv epilogue; one block of sixteen warps: 11 and 7.
template <int EPI, bool DEEP = false, int NT = 1, int PRO = 1, int WARPS = GV_WARPS, bool REGB = false> __host__ __device__ constexpr int gv_stages() {
    if (REGB)
        return WARPS == GV_WIDE_WARPS ? (EPI == 4 ? 7 : 11) : (EPI == 4 ? (GV_REGB_STAGES_N * 2) / 3 : GV_REGB_STAGES_N);
    if (WARPS == GV_WIDE_WARPS)      // one block per SM: 8 stages beside the staged rows, 6 when the rows travel in the queue, 5 with three weight rows
        return EPI == 4 ? 5 : (PRO == 0 ? 6 : 8);
    return DEEP ? (NT == 1 ? GV_DEEP_STAGES : (GV_DEEP_STAGES * 3) / 4)
                : (NT == 2 ? GV_NT2_STAGES : (EPI == 4 ? (GV_STAGES_DEFAULT < 6 ? GV_STAGES_DEFAULT : 6) : GV_STAGES_DEFAULT));
}

enum { GV_PRO_ACT = 0, GV_PRO_NORM = 1 };
enum { GV_EPI_BF16 = 0, GV_EPI_SWIGLU = 1, GV_EPI_RESID = 2, GV_EPI_F32 = 3, GV_EPI_CONV = 4 };
constexpr int GV_CONV_LMAX = 8;

struct GvParams {
    const __nv_bfloat16* W; int N, K, M;
    const __nv_bfloat16* act;                      // PRO_ACT: [M][K]
    const __nv_bfloat16* xw; const float* ss_in; int ss_parts; float eps;   // PRO_NORM: [M][K] stream * norm weight
    __nv_bfloat16* out_bf16; float* out_f32; long long out_stride;
    const float* bias;
    float* resid; float* ss_out;                   // EPI_RESID
    const float* next_w; __nv_bfloat16* xw_out;    // EPI_RESID: weight of the norm that follows, [M][N] out
    int ff;                                        // EPI_SWIGLU: N == 2*ff
    int rows_per_cta;                              // 16 or 8 (always 8 gate + 8 up for SwiGLU)
    int num_tiles;                                 // tiles of rows_per_cta weight rows (8 gate/up pairs)
    // EPI_CONV (W is a short-conv in_proj [3*ff][K], rows B | C | x; every token is a sequence of its own)
    const float* taps; const float* conv_bias;     // [L][ff] oldest tap first, [ff] or null
    __nv_bfloat16* state; long long slot_stride;   // [slots][L-1][ff]
    const int* state_slots; const int* positions;  // [M]
    int L, num_slots; int* status;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ void gv_cp16(void* smem_dst, const void* gsrc, int bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(bytes));
}
__device__ __forceinline__ void gv_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void gv_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int NT, int PRO, int EPI, bool REGB = false>
__host__ __device__ constexpr int gv_slots() { return (EPI == GV_EPI_CONV ? 3 : 2) + ((PRO == GV_PRO_ACT && !REGB) ? NT : 0); }

// chunks of 32 k that a warp keeps of every token's row in registers (REGB): K up to 8 * 32 * 8 = 2048
constexpr int GV_REGB_CHUNKS = 8;

template <int NT, int PRO, int EPI, bool DEEP, int WARPS = GV_WARPS, bool REGB = false>
static size_t gv_smem_bytes(int K) {
    size_t b = (size_t)WARPS * gv_stages<EPI, DEEP, NT, PRO, WARPS, REGB>() * gv_slots<NT, PRO, EPI, REGB>() * 32 * sizeof(uint4);
    if (PRO == GV_PRO_NORM && !REGB) b += (size_t)8 * NT * (K + 32) * sizeof(__nv_bfloat16);
    return b;
}

// What a tile's epilogue needs beside the sums and does not depend on them: asked for at the top
// of the tile, so that it is here when the sums are.  The residual epilogue: the stream's old
// value and the next norm's weight.  The conv epilogue: the request's state, the taps and the
// biases (none of them is written by a kernel of this step before this one).
template <int EPI> struct GvTilePre {
    float r_old = 0.f, r_nw = 0.f;
    float hist[EPI == GV_EPI_CONV ? GV_CONV_LMAX : 1], tapv[EPI == GV_EPI_CONV ? GV_CONV_LMAX : 1];
    float cbias = 0.f, bB = 0.f, bC = 0.f, bX = 0.f;
    bool slot_ok = true;
    __nv_bfloat16* st_ptr = nullptr;
};

template <int EPI>
__device__ __forceinline__ GvTilePre<EPI> gv_tile_prefetch(const GvParams& p, int tile, int R, int ei, int em) {
    GvTilePre<EPI> q;
    q.hist[0] = q.tapv[0] = 0.f;
    if (EPI == GV_EPI_RESID) {
        const long long n = (long long)tile * R + ei;
        if (ei < R && n < p.N && em < p.M) {
            q.r_old = __ldcg(&p.resid[(size_t)em * p.N + n]);
            if (p.xw_out) q.r_nw = p.next_w[n];
        }
    }
    if (EPI == GV_EPI_CONV) {
        const long long c = (long long)tile * 8 + ei;
        const int L = p.L;
#pragma unroll
        for (int j = 0; j < (EPI == GV_EPI_CONV ? GV_CONV_LMAX : 1); ++j) q.hist[j] = q.tapv[j] = 0.f;
        if (ei < 8 && em < p.M && c < p.ff) {
#pragma unroll
            for (int j = 0; j < (EPI == GV_EPI_CONV ? GV_CONV_LMAX : 1); ++j)
                if (j < L) q.tapv[j] = p.taps[(size_t)j * p.ff + c];
            if (p.conv_bias) q.cbias = p.conv_bias[c];
            if (p.bias) { q.bB = p.bias[c]; q.bC = p.bias[p.ff + c]; q.bX = p.bias[2 * (long long)p.ff + c]; }
            if (L > 1) {
                const int slot = p.state_slots[em], p0 = p.positions[em];
                q.slot_ok = slot >= 0 && slot < p.num_slots;
                if (q.slot_ok) {
                    q.st_ptr = p.state + (size_t)slot * p.slot_stride + c;
#pragma unroll
                    for (int j = 0; j < (EPI == GV_EPI_CONV ? GV_CONV_LMAX : 1); ++j)      // rows for positions before 0 count as zero
                        if (j < L - 1 && p0 - (L - 1) + j >= 0) q.hist[j] = __bfloat162float(q.st_ptr[(size_t)j * p.ff]);
                }
            }
        }
    }
    return q;
}

// The end of a tile: the warps' partial sums are added in warp order through shared memory, then
// one thread per output applies the epilogue.  `sync` is the barrier of the warps that share the
// tile (`gw` warps from warp `w0` on).
template <int NT, int PRO, int EPI, int WARPS, typename Sync>
__device__ __forceinline__ void gv_tile_finish(const GvParams& p, int tile, int R, float (&acc)[NT][4],
                                               float (&acc_x)[EPI == GV_EPI_CONV ? NT : 1][4], const GvTilePre<EPI>& pre,
                                               float (&red)[WARPS][16][8 * NT + 1],
                                               float (&red_x)[EPI == GV_EPI_CONV ? WARPS : 1][8][8 * NT + 1],
                                               const float* inv_s, int warp, int g, int t, int tig, int ei, int em,
                                               int w0, int gw, Sync sync) {
    constexpr int COLS = 8 * NT;
    // partial tiles of the group's warps, added in warp order
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][g][nt * 8 + 2 * t] = acc[nt][0];
        red[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
        red[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
        red[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
        if (EPI == GV_EPI_CONV) {
            red_x[warp][g][nt * 8 + 2 * t] = acc_x[nt][0];
            red_x[warp][g][nt * 8 + 2 * t + 1] = acc_x[nt][1];
        }
    }
    sync();
    const int i = ei, m = em;
    float y = 0.f, y2 = 0.f;
    if (i < 16) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) if (w < gw) y += red[w0 + w][i][m];
        if ((EPI == GV_EPI_SWIGLU || EPI == GV_EPI_CONV) && i < 8) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) if (w < gw) y2 += red[w0 + w][i + 8][m];
        }
    }
    float y3 = 0.f;
    if (EPI == GV_EPI_CONV && i < 8) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) if (w < gw) y3 += red_x[w0 + w][i][m];
    }
    if (PRO == GV_PRO_NORM && m < p.M) {
        y *= inv_s[m];
        y2 *= inv_s[m];
        y3 *= inv_s[m];
    }
    if (EPI == GV_EPI_CONV) {
        // y, y2, y3 = B, C, x of channel c for token m, which is a sequence of its own.  The
        // values are rounded where the unfused path stores them (in_proj's output, then g).
        const long long c = (long long)tile * 8 + i;
        if (i < 8 && m < p.M && c < p.ff) {
            float B = __bfloat162float(__float2bfloat16_rn(y));
            float C = __bfloat162float(__float2bfloat16_rn(y2));
            float X = __bfloat162float(__float2bfloat16_rn(y3));
            if (p.bias) { B += pre.bB; C += pre.bC; X += pre.bX; }
            const float gate = __bfloat162float(__float2bfloat16_rn(B * X));
            const int L = p.L;
            float conv = 0.f;
#pragma unroll
            for (int j = 0; j < GV_CONV_LMAX; ++j)
                if (j == L - 1) conv = pre.tapv[j] * gate;
            if (L > 1) {
                if (!pre.slot_ok) {
                    if (p.status) atomicExch(p.status, 3);
                } else {
                    float acc_c = 0.f;
#pragma unroll
                    for (int j = 0; j < GV_CONV_LMAX; ++j)
                        if (j < L - 1) acc_c += pre.tapv[j] * pre.hist[j];
                    conv += acc_c;
#pragma unroll
                    for (int j = 0; j < GV_CONV_LMAX; ++j)
                        if (j < L - 1) pre.st_ptr[(size_t)j * p.ff] = __float2bfloat16_rn(j + 1 < L - 1 ? pre.hist[j + 1 < GV_CONV_LMAX ? j + 1 : 0] : gate);
                }
            }
            conv += pre.cbias;
            p.out_bf16[(size_t)m * p.out_stride + c] = __float2bfloat16_rn(C * conv);
        }
    } else if (EPI == GV_EPI_SWIGLU) {
        const long long col = (long long)tile * 8 + i;
        if (i < 8 && m < p.M && col < p.ff) {
            const float sg = y / (1.f + expf(-y));
            p.out_bf16[(size_t)m * p.out_stride + col] = __float2bfloat16_rn(sg * y2);
        }
    } else {
        const long long n = (long long)tile * R + i;
        const bool valid = i < R && n < p.N && m < p.M;
        if (valid && p.bias) y += p.bias[n];
        if (EPI == GV_EPI_BF16) {
            if (valid) p.out_bf16[(size_t)m * p.out_stride + n] = __float2bfloat16_rn(y);
        } else if (EPI == GV_EPI_F32) {
            if (valid) p.out_f32[(size_t)m * p.out_stride + n] = y;
        } else {   // GV_EPI_RESID
            float v = 0.f;
            if (valid) {
                v = pre.r_old + y;
                p.resid[(size_t)m * p.N + n] = v;
                if (p.xw_out) p.xw_out[(size_t)m * p.N + n] = __float2bfloat16_rn(v * pre.r_nw);
            }
            if (p.ss_out) {
                sync();                        // everyone has read its sums out of red[]
                if (i < 16) red[w0][i][m] = v * v;
                sync();
                if (tig < COLS && tig < p.M) {
                    float sq = 0.f;
#pragma unroll
                    for (int r = 0; r < 16; ++r) sq += red[w0][r][tig];
                    p.ss_out[(size_t)tile * p.M + tig] = sq;
                }
            }
        }
    }
}

// REGB (products with K of at most 2048): a warp owns the same slice of K in every tile, so it reads
// its slice of the tokens' rows once, straight from global memory into the registers that the MMAs take
// them from, as soon as the dependency wait has returned: no staging in shared memory, no barrier
// between the wait and the first MMA, and the queue's room all goes to weights.
template <int NT, int PRO, int EPI, bool DEEP = false, int WARPS = GV_WARPS, bool REGB = false>
__global__ void __launch_bounds__(WARPS * 32)
skinny_linear_kernel(const GvParams p) {
    constexpr int SLOTS = gv_slots<NT, PRO, EPI, REGB>();
    constexpr int GV_STAGES = gv_stages<EPI, DEEP, NT, PRO, WARPS, REGB>();
    constexpr int WS = EPI == GV_EPI_CONV ? 3 : 2;     // weight rows a lane streams per chunk
    constexpr int COLS = 8 * NT;
    extern __shared__ __align__(16) unsigned char gv_smem[];
    __shared__ float red[WARPS][16][COLS + 1];
    __shared__ float red_x[EPI == GV_EPI_CONV ? WARPS : 1][8][COLS + 1];
    __shared__ float inv_s[COLS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Sixteen warps are two groups of eight that walk tiles of their own (their epilogues then fall at
    // different times, so that one group streams while the other adds up) when the product has more
    // tiles than blocks, and one group that splits K sixteen ways when it has not.
    const int groups = (WARPS == GV_WIDE_WARPS && p.num_tiles > (int)gridDim.x) ? 2 : 1;
    const int gw = WARPS / groups;                                 // warps of a group
    const int grp = warp / gw, wig = warp - grp * gw;              // group, warp in the group
    const int tig = (int)threadIdx.x - grp * gw * 32;              // thread in the group
    const int vblock = (int)blockIdx.x * groups + grp, vgrid = (int)gridDim.x * groups;
    auto group_sync = [&]() {
        if (WARPS == GV_WIDE_WARPS && groups == 2) asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(gw * 32) : "memory");
        else __syncthreads();
    };
    const int g = lane >> 2, t = lane & 3;
    const int R = p.rows_per_cta;
    uint4* fifo = reinterpret_cast<uint4*>(gv_smem) + (size_t)warp * (GV_STAGES * SLOTS * 32);
    __nv_bfloat16* act_s = reinterpret_cast<__nv_bfloat16*>(
        reinterpret_cast<uint4*>(gv_smem) + (size_t)WARPS * GV_STAGES * SLOTS * 32);   // PRO_NORM only
    const int pitch = p.K + 32;

    // A block works through tiles blockIdx.x, blockIdx.x + gridDim.x, ...; a warp owns the
    // same slice of K in every tile, so its copy queue runs on across tile boundaries.
    const int my_tiles = vblock < p.num_tiles ? (p.num_tiles - vblock + vgrid - 1) / vgrid : 0;
    const int nchunks = p.K >> 5;
    const int cpw = (nchunks + gw - 1) / gw;
    const int c_begin = min(nchunks, wig * cpw), c_end = min(nchunks, c_begin + cpw);
    const int len = c_end - c_begin;

    // the two weight rows (MMA rows g and g + 8) this lane streams in a given tile
    auto rows_of = [&](int tile, long long& row_lo, long long& row_hi, bool& ok_lo, bool& ok_hi) {
        if (EPI == GV_EPI_SWIGLU || EPI == GV_EPI_CONV) {
            row_lo = (long long)tile * 8 + g;               // gate | B
            row_hi = (long long)p.ff + row_lo;              // up | C  (x: 2 ff + row_lo)
            ok_lo = ok_hi = row_lo < p.ff;
        } else {
            row_lo = (long long)tile * R + g;
            row_hi = row_lo + 8;
            ok_lo = row_lo < p.N;
            ok_hi = R == 16 && row_hi < p.N;
        }
    };
    // the copy queue's own position: tile ordinal and chunk of the next piece to request
    int q_tile = 0, q_c = c_begin;
    const __nv_bfloat16 *q_lo = p.W, *q_hi = p.W, *q_x = p.W;
    int q_lo_bytes = 0, q_hi_bytes = 0;
    auto queue_enter_tile = [&]() {
        if (q_tile < my_tiles) {
            long long row_lo, row_hi;
            bool ok_lo, ok_hi;
            rows_of(vblock + q_tile * vgrid, row_lo, row_hi, ok_lo, ok_hi);
            q_lo = p.W + (size_t)(ok_lo ? row_lo : 0) * p.K + 8 * t;
            q_hi = p.W + (size_t)(ok_hi ? row_hi : 0) * p.K + 8 * t;
            if (EPI == GV_EPI_CONV) q_x = p.W + (size_t)(ok_lo ? 2 * (long long)p.ff + row_lo : 0) * p.K + 8 * t;
            q_lo_bytes = ok_lo ? 16 : 0;
            q_hi_bytes = ok_hi ? 16 : 0;
        }
    };
    auto queue_act_chunk = [&](int c, int stage) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = nt * 8 + g;
            const bool ok = m < p.M;
            gv_cp16(&fifo[(stage * SLOTS + WS + nt) * 32 + lane],
                    p.act + (size_t)(ok ? m : 0) * p.K + ((size_t)c << 5) + 8 * t, ok ? 16 : 0);
        }
    };
    // request the next chunk's weights (and, in the loop, its activations) into `stage`
    auto queue_next = [&](int stage, bool with_acts) {
        if (len > 0 && q_tile < my_tiles) {
            const size_t k = (size_t)q_c << 5;
            gv_cp16(&fifo[(stage * SLOTS + 0) * 32 + lane], q_lo + k, q_lo_bytes);
            gv_cp16(&fifo[(stage * SLOTS + 1) * 32 + lane], q_hi + k, q_hi_bytes);
            if (EPI == GV_EPI_CONV) gv_cp16(&fifo[(stage * SLOTS + 2) * 32 + lane], q_x + k, q_lo_bytes);
            if (PRO == GV_PRO_ACT && with_acts) queue_act_chunk(q_c, stage);
            if (++q_c == c_end) {
                q_c = c_begin;
                ++q_tile;
                queue_enter_tile();
            }
        }
    };

    pdl_trigger();
    queue_enter_tile();
    // the weights do not depend on the kernel before this one: start streaming them, then wait
#pragma unroll
    for (int st = 0; st < GV_STAGES - 1; ++st) {
        queue_next(st, false);
        gv_commit();
    }
    pdl_wait();

    uint4 breg[REGB ? NT : 1][REGB ? GV_REGB_CHUNKS : 1];
    if (REGB) {
        const __nv_bfloat16* tok = PRO == GV_PRO_NORM ? p.xw : p.act;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = nt * 8 + g;
#pragma unroll
            for (int j = 0; j < GV_REGB_CHUNKS; ++j)
                breg[nt][j] = (j < len && m < p.M)
                    ? __ldcg(reinterpret_cast<const uint4*>(tok + (size_t)m * p.K + ((size_t)(c_begin + j) << 5) + 8 * t))
                    : make_uint4(0u, 0u, 0u, 0u);
        }
        if (PRO == GV_PRO_NORM) {
            for (int m = warp; m < p.M; m += WARPS) {
                float s = 0.f;
                for (int i = lane; i < p.ss_parts; i += 32) s += p.ss_in[(size_t)i * p.M + m];
                s = warp_sum(s);
                if (lane == 0) inv_s[m] = rsqrtf(s / (float)p.K + p.eps);
            }
            __syncthreads();
        }
    } else if (PRO == GV_PRO_NORM) {
        // every token's row (already multiplied by the norm's weight) into shared memory, by
        // asynchronous copies that overlap the weights already on their way
        const int k8 = p.K >> 3;
        for (int idx = threadIdx.x; idx < COLS * k8; idx += WARPS * 32) {
            const int m = idx / k8, k = (idx - m * k8) << 3;
            const bool ok = m < p.M;
            gv_cp16(act_s + (size_t)m * pitch + k, p.xw + (size_t)(ok ? m : 0) * p.K + k, ok ? 16 : 0);
        }
        gv_commit();
        // the token's factor rsqrt(mean x^2 + eps) from the producer's partial sums, in a fixed order
        for (int m = warp; m < p.M; m += WARPS) {
            float s = 0.f;
            for (int i = lane; i < p.ss_parts; i += 32) s += p.ss_in[(size_t)i * p.M + m];
            s = warp_sum(s);
            if (lane == 0) inv_s[m] = rsqrtf(s / (float)p.K + p.eps);
        }
        gv_wait<0>();
        __syncthreads();
    } else {
        // activations of the chunks whose weights are already on their way
        if (len > 0 && my_tiles > 0) {
            int c = c_begin, tl = 0;
#pragma unroll
            for (int st = 0; st < GV_STAGES - 1; ++st) {
                if (tl < my_tiles) queue_act_chunk(c, st);
                if (++c == c_end) { c = c_begin; ++tl; }
            }
        }
        gv_commit();
    }

    bool first = true;
    int stage = 0;
    for (int ti = 0; ti < my_tiles; ++ti) {
        const int tile = vblock + ti * vgrid;
        float acc[NT][4];
        float acc_x[EPI == GV_EPI_CONV ? NT : 1][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
        for (int i = 0; i < (EPI == GV_EPI_CONV ? NT : 1); ++i) acc_x[i][0] = acc_x[i][1] = acc_x[i][2] = acc_x[i][3] = 0.f;

        const int ei = tig / COLS, em = tig - ei * COLS;                   // MMA row, token of this thread's output
        const GvTilePre<EPI> pre = gv_tile_prefetch<EPI>(p, tile, R, ei, em);
        if (REGB) {
#pragma unroll
            for (int j = 0; j < GV_REGB_CHUNKS; ++j) {
                if (j < len) {
                    const int nstage = stage == 0 ? GV_STAGES - 1 : stage - 1;
                    queue_next(nstage, false);
                    gv_commit();
                    gv_wait<GV_STAGES - 1>();
                    const uint4 wl = fifo[(stage * SLOTS + 0) * 32 + lane];
                    const uint4 wh = fifo[(stage * SLOTS + 1) * 32 + lane];
                    uint4 wx = make_uint4(0u, 0u, 0u, 0u);
                    if (EPI == GV_EPI_CONV) wx = fifo[(stage * SLOTS + 2) * 32 + lane];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint4 av = breg[nt][j];
                        mma16816(acc[nt], wl.x, wh.x, wl.y, wh.y, av.x, av.y);
                        mma16816(acc[nt], wl.z, wh.z, wl.w, wh.w, av.z, av.w);
                        if (EPI == GV_EPI_CONV) {
                            mma16816(acc_x[nt], wx.x, 0u, wx.y, 0u, av.x, av.y);
                            mma16816(acc_x[nt], wx.z, 0u, wx.w, 0u, av.z, av.w);
                        }
                    }
                    stage = stage == GV_STAGES - 1 ? 0 : stage + 1;
                }
            }
        } else
        for (int c = c_begin; c < c_end; ++c) {
            const int nstage = stage == 0 ? GV_STAGES - 1 : stage - 1;      // (stage + STAGES - 1) % STAGES
            queue_next(nstage, true);
            gv_commit();
            if (PRO == GV_PRO_ACT && first) gv_wait<1>();                   // every group queued before the loop
            else gv_wait<GV_STAGES - 1>();
            first = false;
            const uint4 wl = fifo[(stage * SLOTS + 0) * 32 + lane];
            const uint4 wh = fifo[(stage * SLOTS + 1) * 32 + lane];
            uint4 wx = make_uint4(0u, 0u, 0u, 0u);
            if (EPI == GV_EPI_CONV) wx = fifo[(stage * SLOTS + 2) * 32 + lane];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                uint4 av;
                if (PRO == GV_PRO_ACT) av = fifo[(stage * SLOTS + WS + nt) * 32 + lane];
                else av = *reinterpret_cast<const uint4*>(act_s + (size_t)(nt * 8 + g) * pitch + ((size_t)c << 5) + 8 * t);
                mma16816(acc[nt], wl.x, wh.x, wl.y, wh.y, av.x, av.y);
                mma16816(acc[nt], wl.z, wh.z, wl.w, wh.w, av.z, av.w);
                if (EPI == GV_EPI_CONV) {                        // the x rows: the MMA's upper eight rows stay empty
                    mma16816(acc_x[nt], wx.x, 0u, wx.y, 0u, av.x, av.y);
                    mma16816(acc_x[nt], wx.z, 0u, wx.w, 0u, av.z, av.w);
                }
            }
            stage = stage == GV_STAGES - 1 ? 0 : stage + 1;
        }

        gv_tile_finish<NT, PRO, EPI, WARPS>(p, tile, R, acc, acc_x, pre, red, red_x, inv_s, warp, g, t, tig, ei, em,
                                            grp * gw, gw, group_sync);
        group_sync();                                    // red[] is free for the next tile
    }
    gv_wait<0>();
}

static int gv_sm_count() { return sm_count(); }

// ---------------------------------------------------------------------------------------------
// The same product with the weight stream moved by the tensor memory accelerator: a second form of
// the kernel above for steps of at most 8 tokens and K of at most 2048 (the tokens' rows in
// registers), chosen with VAPI_GV_TMA.  A ninth warp's first lane is the producer: it brings the
// weights in with cp.async.bulk.tensor, one box per half-tile of 8 rows and GT_SUB chunks of 32 k,
// into per-warp rings of shared-memory stages guarded by full / empty mbarriers (the tensor map
// sees the weight as [K/32 chunks][rows][32 k], so a box lands as [chunk][8 rows][64 bytes]: the
// layout in which a quarter-warp's 16-byte reads touch every bank once).  The eight consumer
// warps do what they do above: each owns a slice of K, multiplies with mma.sync out of shared
// memory and hands its stage back; the tiles' ends are the same code.  Nothing is requested by the
// consumers' lanes, so their issue slots are free and a block holds its whole ring in flight from
// its first cycle, before the dependency wait.  Every mbarrier wait is bounded; when one runs out
// the block records status 16, stops waiting and runs to its end (its output is then not valid).
constexpr int GT_SUB = 4;                                   // chunks of 32 k in a stage
template <int EPI> __host__ __device__ constexpr int gt_halves() { return EPI == GV_EPI_CONV ? 3 : 2; }
template <int EPI> __host__ __device__ constexpr int gt_stage_bytes() { return gt_halves<EPI>() * GT_SUB * 512; }
#ifndef GT_RING_KB
#define GT_RING_KB 96
#endif
template <int EPI> __host__ __device__ constexpr int gt_depth() { return (GT_RING_KB * 1024) / (GV_WARPS * gt_stage_bytes<EPI>()); }

__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

template <int PRO, int EPI>
__global__ void __launch_bounds__((GV_WARPS + 1) * 32, 2)
skinny_linear_tma_kernel(const __grid_constant__ CUtensorMap tm_w, const GvParams p) {
    constexpr int NT = 1, COLS = 8, WARPS = GV_WARPS;
    constexpr int HALVES = gt_halves<EPI>(), SB = gt_stage_bytes<EPI>(), DW = gt_depth<EPI>();
    extern __shared__ __align__(128) unsigned char gt_smem[];      // [warp][DW][HALVES][GT_SUB][8 rows][32 k]
    __shared__ float red[WARPS][16][COLS + 1];
    __shared__ float red_x[EPI == GV_EPI_CONV ? WARPS : 1][8][COLS + 1];
    __shared__ float inv_s[COLS];
    __shared__ unsigned long long bars[2 * WARPS * DW];             // full[warp][slot], then empty[warp][slot]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int R = p.rows_per_cta;
    const int vblock = (int)blockIdx.x, vgrid = (int)gridDim.x;
    const int my_tiles = vblock < p.num_tiles ? (p.num_tiles - vblock + vgrid - 1) / vgrid : 0;
    const int nchunks = p.K >> 5;
    const int cpw = (nchunks + WARPS - 1) / WARPS;
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + WARPS * DW);
    auto consumer_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"r"(WARPS * 32) : "memory"); };

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * WARPS * DW; ++i) mbar_init(full0 + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---- producer: nothing it moves depends on the kernel before this one ----
        if (lane == 0) {
            bool ok = true;
            const int nsub_max = (cpw + GT_SUB - 1) / GT_SUB;
            for (int ti = 0; ti < my_tiles && ok; ++ti) {
                const int tile = vblock + ti * vgrid;
                int row[3];
                if (EPI == GV_EPI_SWIGLU || EPI == GV_EPI_CONV) { row[0] = tile * 8; row[1] = p.ff + tile * 8; row[2] = 2 * p.ff + tile * 8; }
                else { row[0] = tile * 16; row[1] = tile * 16 + 8; row[2] = 0; }
                for (int sub = 0; sub < nsub_max && ok; ++sub) {
                    for (int w = 0; w < WARPS; ++w) {
                        const int cb = min(nchunks, w * cpw), len = min(nchunks, cb + cpw) - cb;
                        if (sub * GT_SUB >= len) continue;
                        const int nsub = (len + GT_SUB - 1) / GT_SUB;
                        const int q = ti * nsub + sub, slot = q % DW;
                        if (q >= DW && !mbar_wait(empty0 + 8 * (w * DW + slot), ((q / DW) - 1) & 1)) { ok = false; break; }
                        const unsigned bar = full0 + 8 * (w * DW + slot);
                        const unsigned dst = smem_u32(gt_smem + (size_t)(w * DW + slot) * SB);
                        mbar_expect_tx(bar, SB);
#pragma unroll
                        for (int h = 0; h < HALVES; ++h)
                            tma_load_3d(dst + h * GT_SUB * 512, &tm_w, bar, 0, row[h], cb + sub * GT_SUB);
                    }
                }
            }
            if (!ok && p.status) atomicExch(p.status, 16);
        }
        return;
    }

    // ---- consumers ----
    const int c_begin = min(nchunks, warp * cpw), c_end = min(nchunks, c_begin + cpw);
    const int len = c_end - c_begin;
    const int nsub = (len + GT_SUB - 1) / GT_SUB;
    pdl_wait();
    uint4 breg[GV_REGB_CHUNKS];
    {
        const __nv_bfloat16* tok = PRO == GV_PRO_NORM ? p.xw : p.act;
#pragma unroll
        for (int j = 0; j < GV_REGB_CHUNKS; ++j)
            breg[j] = (j < len && g < p.M)
                ? __ldcg(reinterpret_cast<const uint4*>(tok + (size_t)g * p.K + ((size_t)(c_begin + j) << 5) + 8 * t))
                : make_uint4(0u, 0u, 0u, 0u);
    }
    if (PRO == GV_PRO_NORM) {
        for (int m = warp; m < p.M; m += WARPS) {
            float s = 0.f;
            for (int i = lane; i < p.ss_parts; i += 32) s += p.ss_in[(size_t)i * p.M + m];
            s = warp_sum(s);
            if (lane == 0) inv_s[m] = rsqrtf(s / (float)p.K + p.eps);
        }
        consumer_sync();
    }
    const int tig = (int)threadIdx.x;
    bool ok = true;
    int q = 0;
    for (int ti = 0; ti < my_tiles; ++ti) {
        const int tile = vblock + ti * vgrid;
        float acc[NT][4] = {{0.f, 0.f, 0.f, 0.f}};
        float acc_x[EPI == GV_EPI_CONV ? NT : 1][4] = {{0.f, 0.f, 0.f, 0.f}};
        const int ei = tig / COLS, em = tig - ei * COLS;
        const GvTilePre<EPI> pre = gv_tile_prefetch<EPI>(p, tile, R, ei, em);
#pragma unroll
        for (int sub = 0; sub < GV_REGB_CHUNKS / GT_SUB; ++sub) {
            if (sub < nsub) {
                const int slot = q % DW;
                ok = ok && mbar_wait(full0 + 8 * (warp * DW + slot), (q / DW) & 1);
                const unsigned char* base = gt_smem + (size_t)(warp * DW + slot) * SB + g * 64 + t * 16;
#pragma unroll
                for (int j = 0; j < GT_SUB; ++j) {
                    if (sub * GT_SUB + j < len) {
                        const uint4 wl = *reinterpret_cast<const uint4*>(base + (0 * GT_SUB + j) * 512);
                        const uint4 wh = *reinterpret_cast<const uint4*>(base + (1 * GT_SUB + j) * 512);
                        const uint4 av = breg[sub * GT_SUB + j];
                        mma16816(acc[0], wl.x, wh.x, wl.y, wh.y, av.x, av.y);
                        mma16816(acc[0], wl.z, wh.z, wl.w, wh.w, av.z, av.w);
                        if (EPI == GV_EPI_CONV) {
                            const uint4 wx = *reinterpret_cast<const uint4*>(base + (2 * GT_SUB + j) * 512);
                            mma16816(acc_x[0], wx.x, 0u, wx.y, 0u, av.x, av.y);
                            mma16816(acc_x[0], wx.z, 0u, wx.w, 0u, av.z, av.w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * (warp * DW + slot));
                ++q;
            }
        }
        gv_tile_finish<NT, PRO, EPI, WARPS>(p, tile, R, acc, acc_x, pre, red, red_x, inv_s, warp, g, t, tig, ei, em,
                                            0, WARPS, consumer_sync);
        consumer_sync();                                    // red[] is free for the next tile
    }
    if (!ok && lane == 0 && p.status) atomicExch(p.status, 16);
}

// the weight [rows][K] seen as [K/32 chunks][rows][32 k], in boxes of GT_SUB chunks x 8 rows; one map
// per weight is kept (a map holds nothing but the address and the shape)
static int gt_weight_map(CUtensorMap* out, const void* W, long long rows, long long K) {
    struct Key { const void* w; long long rows, K; bool operator==(const Key& o) const { return w == o.w && rows == o.rows && K == o.K; } };
    struct Hash { size_t operator()(const Key& k) const { return (size_t)k.w ^ ((size_t)k.rows << 20) ^ (size_t)k.K; } };
    static thread_local std::unordered_map<Key, CUtensorMap, Hash> cache;
    const Key key{W, rows, K};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(-102, "skinny_linear: cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)W & 15) != 0 || K % 32 != 0) return fail(-1, "skinny_linear: the weight is not 16-byte aligned or K=%lld is no multiple of 32", K);
    cuuint64_t dims[3] = {32, (cuuint64_t)rows, (cuuint64_t)(K / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, 64};
    cuuint32_t box[3] = {32, 8, (cuuint32_t)GT_SUB};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(W), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(-103, "skinny_linear: cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

static int g_gt_enabled = -1;          // -1: not asked yet (then VAPI_GV_TMA decides)
static bool gt_enabled() {
    if (g_gt_enabled < 0) {
        const char* e = getenv("VAPI_GV_TMA");
        g_gt_enabled = (e && e[0] == '1') ? 1 : 0;
    }
    return g_gt_enabled == 1;
}
// 1: steps of at most 8 tokens take the form whose weights come by TMA where it applies; 0: never
VAPI_EXPORT int vapi_skinny_linear_use_tma(int on) {
    const int was = gt_enabled() ? 1 : 0;
    g_gt_enabled = on ? 1 : 0;
    return was;
}
// whether the form above takes a call: at most 8 tokens, tiles of 16 rows, a warp's slice of K in registers
static bool gt_applies(const GvParams& p) {
    return gt_enabled() && p.M <= 8 && p.rows_per_cta == 16 && (p.K >> 5) <= GV_REGB_CHUNKS * GV_WARPS && p.K % 32 == 0 &&
           ((uintptr_t)p.W & 15) == 0;
}

template <int PRO, int EPI>
static int launch_gt(const GvParams& p, int blocks, cudaStream_t stream) {
    CUtensorMap map;
    int rc = gt_weight_map(&map, p.W, p.N, p.K);
    if (rc) return rc;
    constexpr size_t smem = (size_t)GV_WARPS * gt_depth<EPI>() * gt_stage_bytes<EPI>();
    auto kern = skinny_linear_tma_kernel<PRO, EPI>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-101, "skinny_linear: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        attr_done = true;
    }
    const int cap = gv_sm_count() * 2;
    return check_launch("skinny_linear (tma)", launch(kern, blocks < cap ? blocks : cap, (GV_WARPS + 1) * 32, smem, stream, map, p));
}



template <int NT, int PRO, int EPI, bool DEEP, int WARPS, bool REGB = false>
static int launch_gv_as(const GvParams& p, int blocks, int blocks_per_sm, cudaStream_t stream) {
    const size_t smem = gv_smem_bytes<NT, PRO, EPI, DEEP, WARPS, REGB>(p.K);
    auto kern = skinny_linear_kernel<NT, PRO, EPI, DEEP, WARPS, REGB>;
    if (smem > 200 * 1024) return fail(-1, "skinny_linear: K=%d needs %zu bytes of shared memory", p.K, smem);
    if (smem + 28 * 1024 > 48 * 1024) {      // (static shared memory, up to about 26 KB, counts toward the default limit)
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-101, "skinny_linear: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    // a fixed number of blocks per SM, each walking its share of the tiles
    const int cap = blocks_per_sm > 0 ? gv_sm_count() * blocks_per_sm : blocks;
    return check_launch("skinny_linear", launch(kern, blocks < cap ? blocks : cap, WARPS * 32, smem, stream, p));
}

template <int NT, int PRO, int EPI, bool DEEP = false>
static int launch_gv(const GvParams& p, int blocks, cudaStream_t stream) {
    static int per_sm = -1, wide = -1, regb = -1;
    if (per_sm < 0) {
        const char* e = getenv("VAPI_GV_BLOCKS_PER_SM");
        per_sm = e ? atoi(e) : 2;
        const char* w = getenv("VAPI_GV_WIDE");
        wide = (w && w[0] == '0') ? 0 : 1;
        const char* r = getenv("VAPI_GV_REGB");     // bits: 1 norm prologue, 2 plain activations, 4 nine to sixteen tokens
        regb = r ? atoi(r) : 1;
    }
    // the tokens' rows in registers where a warp's slice of K is at most GV_REGB_CHUNKS chunks
    const bool in_regs = (regb & (PRO == GV_PRO_NORM ? 1 : 2)) && (NT == 1 || (regb & 4)) && !DEEP &&
                         (p.K >> 5) <= GV_REGB_CHUNKS * GV_WARPS;
    if (NT == 2 && wide) {
        // sixteen warps, one block per SM, where the queue and the tokens' rows fit (with the static arrays beside them)
        constexpr int W = NT == 2 ? GV_WIDE_WARPS : GV_WARPS;
        if (in_regs) return launch_gv_as<NT, PRO, EPI, false, W, !DEEP>(p, blocks, 1, stream);
        if (gv_smem_bytes<NT, PRO, EPI, false, W>(p.K) <= 198 * 1024)
            return launch_gv_as<NT, PRO, EPI, false, W>(p, blocks, 1, stream);
    }
    if (in_regs) return launch_gv_as<NT, PRO, EPI, false, GV_WARPS, !DEEP>(p, blocks, per_sm, stream);
    return launch_gv_as<NT, PRO, EPI, DEEP, GV_WARPS>(p, blocks, per_sm, stream);
}

// Number of blocks (and so of partial sums a residual epilogue leaves) for a given shape.
VAPI_EXPORT int vapi_skinny_linear_blocks(int N, int epi, int rows_per_cta) {
    if (epi == GV_EPI_SWIGLU) return (N / 2 + 7) / 8;
    return (N + rows_per_cta - 1) / rows_per_cta;
}

VAPI_EXPORT int vapi_skinny_linear(const void* W, int N, int K, int M, int pro, const void* act,
                                   const void* xw, const float* ss_in, int ss_parts, float eps,
                                   int epi, void* out_bf16, float* out_f32, long long out_stride,
                                   const float* bias, float* resid, float* ss_out,
                                   const float* next_w, void* xw_out, int rows_per_cta,
                                   cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16) return fail(-1, "skinny_linear: %d rows are more than 16", M);
    if (N <= 0 || K <= 0 || K % 32 != 0) return fail(-1, "skinny_linear: K=%d must be a positive multiple of 32 (N=%d)", K, N);
    if (rows_per_cta != 8 && rows_per_cta != 16) return fail(-1, "skinny_linear: rows per block must be 8 or 16");
    if (epi == GV_EPI_SWIGLU && N % 2 != 0) return fail(-1, "skinny_linear: SwiGLU needs an even N");
    if (pro == GV_PRO_ACT && !act) return fail(-1, "skinny_linear: no activations");
    if (pro == GV_PRO_NORM && (!xw || !ss_in || ss_parts <= 0)) return fail(-1, "skinny_linear: norm prologue needs the weighted stream and its partial sums");
    if (xw_out && !next_w) return fail(-1, "skinny_linear: a weighted copy of the stream needs the next norm's weight");
    if ((epi == GV_EPI_BF16 || epi == GV_EPI_SWIGLU) && !out_bf16) return fail(-1, "skinny_linear: no output");
    if (epi == GV_EPI_F32 && !out_f32) return fail(-1, "skinny_linear: no output");
    if (epi == GV_EPI_RESID && !resid) return fail(-1, "skinny_linear: no residual stream");
    GvParams p = {};
    p.W = (const __nv_bfloat16*)W; p.N = N; p.K = K; p.M = M;
    p.act = (const __nv_bfloat16*)act; p.xw = (const __nv_bfloat16*)xw; p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps;
    p.next_w = next_w; p.xw_out = (__nv_bfloat16*)xw_out;
    p.out_bf16 = (__nv_bfloat16*)out_bf16; p.out_f32 = out_f32; p.out_stride = out_stride; p.bias = bias;
    p.resid = resid; p.ss_out = ss_out; p.ff = N / 2; p.rows_per_cta = epi == GV_EPI_SWIGLU ? 16 : rows_per_cta;
    const int blocks = vapi_skinny_linear_blocks(N, epi, rows_per_cta);
    p.num_tiles = blocks;
#define GV_GO(NT, PRO, EPI) return launch_gv<NT, PRO, EPI>(p, blocks, stream)
#define GV_EPIS(NT, PRO)                                      \
    switch (epi) {                                            \
        case GV_EPI_BF16: GV_GO(NT, PRO, GV_EPI_BF16);        \
        case GV_EPI_SWIGLU: GV_GO(NT, PRO, GV_EPI_SWIGLU);    \
        case GV_EPI_RESID: GV_GO(NT, PRO, GV_EPI_RESID);      \
        case GV_EPI_F32: GV_GO(NT, PRO, GV_EPI_F32);          \
        default: return fail(-2, "skinny_linear: unknown epilogue %d", epi); \
    }
    if (gt_applies(p)) {
        if (pro == GV_PRO_ACT) {
            switch (epi) {
                case GV_EPI_BF16: return launch_gt<GV_PRO_ACT, GV_EPI_BF16>(p, blocks, stream);
                case GV_EPI_SWIGLU: return launch_gt<GV_PRO_ACT, GV_EPI_SWIGLU>(p, blocks, stream);
                case GV_EPI_RESID: return launch_gt<GV_PRO_ACT, GV_EPI_RESID>(p, blocks, stream);
                case GV_EPI_F32: return launch_gt<GV_PRO_ACT, GV_EPI_F32>(p, blocks, stream);
            }
        } else if (pro == GV_PRO_NORM) {
            switch (epi) {
                case GV_EPI_BF16: return launch_gt<GV_PRO_NORM, GV_EPI_BF16>(p, blocks, stream);
                case GV_EPI_SWIGLU: return launch_gt<GV_PRO_NORM, GV_EPI_SWIGLU>(p, blocks, stream);
                case GV_EPI_RESID: return launch_gt<GV_PRO_NORM, GV_EPI_RESID>(p, blocks, stream);
                case GV_EPI_F32: return launch_gt<GV_PRO_NORM, GV_EPI_F32>(p, blocks, stream);
            }
        }
    }
    static int deep_k = -1;
    if (deep_k < 0) {
        const char* e = getenv("VAPI_GV_DEEP_K");
        deep_k = e ? atoi(e) : 4096;
    }
    if (pro == GV_PRO_ACT && epi == GV_EPI_RESID && deep_k > 0 && K >= deep_k && blocks <= gv_sm_count()) {
        if (M <= 8) return launch_gv<1, GV_PRO_ACT, GV_EPI_RESID, true>(p, blocks, stream);
        return launch_gv<2, GV_PRO_ACT, GV_EPI_RESID, true>(p, blocks, stream);
    }
    if (pro == GV_PRO_ACT) {
        if (M <= 8) { GV_EPIS(1, GV_PRO_ACT) } else { GV_EPIS(2, GV_PRO_ACT) }
    } else if (pro == GV_PRO_NORM) {
        if (M <= 8) { GV_EPIS(1, GV_PRO_NORM) } else { GV_EPIS(2, GV_PRO_NORM) }
    }
    return fail(-2, "skinny_linear: unknown prologue %d", pro);
#undef GV_EPIS
#undef GV_GO
}

// The short-conv mixer's in_proj with the whole gated convolution of a decode step as its
// epilogue: W [3H][K] (rows B | C | x), token operand the residual stream seen through a deferred
// norm, out [M][H] = C * conv(B * x over the request's state), state updated in place.  Every one
// of the M tokens must be a sequence of its own (one state slot and one position per token).
VAPI_EXPORT int vapi_skinny_linear_conv(const void* W, int H, int K, int M, const void* xw, const float* ss_in,
                                        int ss_parts, float eps, const float* in_bias, const float* taps,
                                        const float* conv_bias, int L, void* state, long long slot_stride,
                                        int num_slots, const int* state_slots, const int* positions, void* out,
                                        int* status, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16) return fail(-1, "skinny_linear_conv: %d rows are more than 16", M);
    if (H <= 0 || K <= 0 || K % 32 != 0) return fail(-1, "skinny_linear_conv: K=%d must be a positive multiple of 32 (H=%d)", K, H);
    if (L < 1 || L > GV_CONV_LMAX) return fail(-1, "skinny_linear_conv: kernel length %d is outside 1..%d", L, GV_CONV_LMAX);
    if (!xw || !ss_in || ss_parts <= 0) return fail(-1, "skinny_linear_conv: the norm prologue needs the weighted stream and its partial sums");
    if (!taps || !out || !state_slots || !positions) return fail(-1, "skinny_linear_conv: missing array");
    if (L > 1 && (!state || num_slots <= 0)) return fail(-1, "skinny_linear_conv: no state buffer");
    GvParams p = {};
    p.W = (const __nv_bfloat16*)W; p.N = 3 * H; p.K = K; p.M = M;
    p.xw = (const __nv_bfloat16*)xw; p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps;
    p.out_bf16 = (__nv_bfloat16*)out; p.out_stride = H; p.bias = in_bias; p.ff = H; p.rows_per_cta = 16;
    p.taps = taps; p.conv_bias = conv_bias; p.state = (__nv_bfloat16*)state; p.slot_stride = slot_stride;
    p.state_slots = state_slots; p.positions = positions; p.L = L; p.num_slots = num_slots; p.status = status;
    const int blocks = (H + 7) / 8;
    p.num_tiles = blocks;
    if (gt_applies(p)) return launch_gt<GV_PRO_NORM, GV_EPI_CONV>(p, blocks, stream);
    if (M <= 8) return launch_gv<1, GV_PRO_NORM, GV_EPI_CONV>(p, blocks, stream);
    return launch_gv<2, GV_PRO_NORM, GV_EPI_CONV>(p, blocks, stream);
}

// ---------------------------------------------------------------------------------------------
// The same product on the true 32-bit path: float weights, float tokens, float FMA and nothing
// else (no tensor cores, no reduced-precision mode), for the decode steps of that path.  A warp
// owns a few weight rows and walks K in 16-byte pieces, a chunk of K at a time; the tokens' pieces
// of a chunk are used for all rows of all warps of the block.  The sum over K is formed per (token, row) in an order that depends on K alone:
// lane-strided partial sums, then a butterfly over the lanes, so a token's result does not
// depend on what else is in the batch.
constexpr int F32_WARPS = 8;
// rows of the weight a warp owns, and 16-byte pieces of each row that a lane asks for together
// (fewer of both for nine to sixteen tokens, whose sums take the registers)
__host__ __device__ constexpr int f32_rows(int mt) { return mt <= 8 ? 4 : 2; }
__host__ __device__ constexpr int f32_depth(int mt) { return mt <= 8 ? 4 : 2; }

// The tokens' rows travel through shared memory, a chunk of K at a time (two buffers, filled by
// asynchronous copies one chunk ahead), so that they are read from L2 once per block, not once per warp.
template <int MT>
__global__ void __launch_bounds__(F32_WARPS * 32)
skinny_linear_f32_kernel(const float* __restrict__ W, const float* __restrict__ act, const float* __restrict__ bias,
                         float* __restrict__ out, int N, int K, int M, long long out_stride) {
    constexpr int F32_ROWS = f32_rows(MT), F32_DEPTH = f32_depth(MT);
    constexpr int F32_CHUNK = 32 * F32_DEPTH;             // pieces of K in a chunk
    __shared__ float4 abuf[2][MT][F32_CHUNK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long n0 = ((long long)blockIdx.x * F32_WARPS + warp) * F32_ROWS;
    pdl_trigger();
    float acc[F32_ROWS][MT];
#pragma unroll
    for (int r = 0; r < F32_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
    const int k4 = K >> 2;
    const int chunks = (k4 + F32_CHUNK - 1) / F32_CHUNK;
    const float4* wrow[F32_ROWS];
#pragma unroll
    for (int r = 0; r < F32_ROWS; ++r) wrow[r] = reinterpret_cast<const float4*>(W + (size_t)(n0 + r < N ? n0 + r : 0) * K);
    float4 w[F32_DEPTH][F32_ROWS];
    auto fetch = [&](int c0) {          // this lane's pieces of a chunk of its rows
#pragma unroll
        for (int u = 0; u < F32_DEPTH; ++u)
#pragma unroll
            for (int r = 0; r < F32_ROWS; ++r)
                w[u][r] = (c0 + 32 * u < k4 && n0 < N) ? __ldcs(wrow[r] + c0 + 32 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto stage = [&](int chunk, int buf) {     // the tokens' pieces of a chunk, by the whole block
        for (int idx = threadIdx.x; idx < MT * F32_CHUNK; idx += F32_WARPS * 32) {
            const int m = idx / F32_CHUNK, c = idx - m * F32_CHUNK, cg = chunk * F32_CHUNK + c;
            const bool ok = m < M && cg < k4;
            gv_cp16(&abuf[buf][m][c], reinterpret_cast<const float4*>(act + (size_t)(ok ? m : 0) * K) + (ok ? cg : 0), ok ? 16 : 0);
        }
        gv_commit();
    };
    fetch(lane);                         // the weights do not depend on the kernel before this one
    pdl_wait();
    stage(0, 0);
    for (int ch = 0; ch < chunks; ++ch) {
        if (ch + 1 < chunks) stage(ch + 1, (ch + 1) & 1);
        else gv_commit();
        gv_wait<1>();
        __syncthreads();                 // chunk ch of the tokens is in place for every warp
        if (ch > 0) fetch(ch * F32_CHUNK + lane);
#pragma unroll
        for (int u = 0; u < F32_DEPTH; ++u) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float4 a = abuf[ch & 1][m][lane + 32 * u];
#pragma unroll
                for (int r = 0; r < F32_ROWS; ++r) {
                    acc[r][m] = fmaf(w[u][r].x, a.x, acc[r][m]);
                    acc[r][m] = fmaf(w[u][r].y, a.y, acc[r][m]);
                    acc[r][m] = fmaf(w[u][r].z, a.z, acc[r][m]);
                    acc[r][m] = fmaf(w[u][r].w, a.w, acc[r][m]);
                }
            }
        }
        __syncthreads();                 // everyone is done with this buffer before it is filled again
    }
    gv_wait<0>();
    if (n0 >= N) return;
#pragma unroll
    for (int r = 0; r < F32_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = warp_sum(acc[r][m]);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < F32_ROWS; ++r) {
            if (n0 + r < N) {
                const float b = bias ? bias[n0 + r] : 0.f;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < M) out[(size_t)m * out_stride + n0 + r] = acc[r][m] + b;
            }
        }
    }
}

// y[m][n] = sum_k act[m][k] * W[n][k] (+ bias[n]) in float, M <= 16, K a multiple of 4.
VAPI_EXPORT int vapi_skinny_linear_f32(const float* W, int N, int K, int M, const float* act, const float* bias,
                                       float* out, long long out_stride, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16) return fail(-1, "skinny_linear_f32: %d rows are more than 16", M);
    if (N <= 0 || K <= 0 || K % 4 != 0) return fail(-1, "skinny_linear_f32: K=%d must be a positive multiple of 4 (N=%d)", K, N);
    if (!W || !act || !out) return fail(-1, "skinny_linear_f32: missing array");
    if ((((uintptr_t)W | (uintptr_t)act) & 15) != 0) return fail(-1, "skinny_linear_f32: operands must be 16-byte aligned");
    const int mt = M <= 1 ? 1 : (M <= 4 ? 4 : (M <= 8 ? 8 : 16));
    const int blocks = (N + F32_WARPS * f32_rows(mt) - 1) / (F32_WARPS * f32_rows(mt));
    cudaError_t e;
    if (M <= 1) e = launch(skinny_linear_f32_kernel<1>, blocks, F32_WARPS * 32, 0, stream, W, act, bias, out, N, K, M, out_stride);
    else if (M <= 4) e = launch(skinny_linear_f32_kernel<4>, blocks, F32_WARPS * 32, 0, stream, W, act, bias, out, N, K, M, out_stride);
    else if (M <= 8) e = launch(skinny_linear_f32_kernel<8>, blocks, F32_WARPS * 32, 0, stream, W, act, bias, out, N, K, M, out_stride);
    else e = launch(skinny_linear_f32_kernel<16>, blocks, F32_WARPS * 32, 0, stream, W, act, bias, out, N, K, M, out_stride);
    return check_launch("skinny_linear_f32", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
