// Token selection on the device: greedy argmax, temperature sampling by the Gumbel-max
// trick, and the repetition / frequency / presence penalties.
//
// Same definitions as the reference's device sampler
// (crates/vapi-backend-candle/src/fused.rs:236-293): ties go to the lowest token id; the
// noise of draw number `draw` of a request seeded `seed` is
//   key = mix64(seed ^ mix64(draw + 0x9E3779B97F4A7C15)),
//   u_v = ((mix64(key + v * 0xBF58476D1CE4E5B9) >> 40) + 0.5) / 2^24,  g_v = -ln(-ln u_v),
// and the token is argmax_v(logit_v / T + g_v): deterministic in (seed, draw), independent
// of what else is in the batch.
#include "common.cuh"

using namespace vapi;

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}

__device__ __forceinline__ void arg_better(float& bv, unsigned& bi, float v, unsigned i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

// Block-wide (value, index) argmax with lowest-index tie-break; result valid in thread 0.
__device__ __forceinline__ void block_argmax(float& bv, unsigned& bi, float* sv, unsigned* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
        arg_better(bv, bi, ov, oi);
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
            arg_better(bv, bi, ov, oi);
        }
    }
}

// mode[row]: 0 = skip (out untouched), 1 = greedy, 2 = Gumbel-max; mode == nullptr: all greedy.
// A row of logits is cut into gridDim.y slices; each block finds the best (value, id) of its
// slice; the block that finishes a row last (a counter per row) reduces the slices in slice
// order, so the result does not depend on which block that is.
constexpr int SAMPLE_MAX_SLICES = 32;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                   const int* __restrict__ mode, const float* __restrict__ inv_t,
                   const unsigned long long* __restrict__ seeds,
                   const unsigned long long* __restrict__ draws, int* __restrict__ out,
                   float* __restrict__ part_v, unsigned* __restrict__ part_i,
                   unsigned* __restrict__ counters) {
    __shared__ float sv[32];
    __shared__ unsigned si[32];
    __shared__ bool last;
    const int row = blockIdx.x, slice = blockIdx.y, slices = gridDim.y;
    pdl_trigger();
    pdl_wait();
    const int md = mode ? mode[row] : 1;
    if (md == 0) return;
    const float* l = logits + (size_t)row * row_stride;
    // a slice is a multiple of 4 entries, so that an aligned row is read in 16-byte pieces
    const unsigned per = ((((unsigned)vocab + slices - 1) / slices) + 3u) & ~3u;
    const unsigned lo = min((unsigned)vocab, slice * per), hi = min((unsigned)vocab, lo + per);
    float bv = -INFINITY;
    unsigned bi = 0xffffffffu;
    const bool vec = (reinterpret_cast<uintptr_t>(l) & 15) == 0;
    const unsigned hi4 = vec ? lo + ((hi - lo) & ~3u) : lo;      // [lo, hi4) in pieces of 4, [hi4, hi) one by one
    if (md == 1) {
#pragma unroll 4
        for (unsigned i = lo + 4 * threadIdx.x; i < hi4; i += 4 * blockDim.x) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(l + i));
            arg_better(bv, bi, v.x, i);
            arg_better(bv, bi, v.y, i + 1);
            arg_better(bv, bi, v.z, i + 2);
            arg_better(bv, bi, v.w, i + 3);
        }
        for (unsigned i = hi4 + threadIdx.x; i < hi; i += blockDim.x) arg_better(bv, bi, l[i], i);
    } else {
        const float it = inv_t[row];
        const unsigned long long key = mix64(seeds[row] ^ mix64(draws[row] + 0x9E3779B97F4A7C15ULL));
        auto noisy = [&](float x, unsigned i) {
            const unsigned long long h = mix64(key + (unsigned long long)i * 0xBF58476D1CE4E5B9ULL);
            const float u = ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
            const float g = -logf(-logf(u));
            arg_better(bv, bi, x * it + g, i);
        };
#pragma unroll 2
        for (unsigned i = lo + 4 * threadIdx.x; i < hi4; i += 4 * blockDim.x) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(l + i));
            noisy(v.x, i);
            noisy(v.y, i + 1);
            noisy(v.z, i + 2);
            noisy(v.w, i + 3);
        }
        for (unsigned i = hi4 + threadIdx.x; i < hi; i += blockDim.x) noisy(l[i], i);
    }
    block_argmax(bv, bi, sv, si);
    if (slices == 1) {
        if (threadIdx.x == 0) out[row] = bi == 0xffffffffu ? 0 : (int)bi;
        return;
    }
    if (threadIdx.x == 0) {
        part_v[(size_t)row * slices + slice] = bv;
        part_i[(size_t)row * slices + slice] = bi;
        __threadfence();
        last = atomicAdd(&counters[row], 1u) == (unsigned)slices - 1;
    }
    __syncthreads();
    if (!last) return;
    if (threadIdx.x == 0) {
        __threadfence();
        float fv = -INFINITY;
        unsigned fi = 0xffffffffu;
        for (int sidx = 0; sidx < slices; ++sidx)
            arg_better(fv, fi, part_v[(size_t)row * slices + sidx], part_i[(size_t)row * slices + sidx]);
        out[row] = fi == 0xffffffffu ? 0 : (int)fi;
        counters[row] = 0;                      // ready for the next call
    }
}

// scratch: rows * slices floats + rows * slices + rows unsigned (the counters must be zero at
// the first call; every call leaves them zero)
VAPI_EXPORT int vapi_sample_rows(const float* logits, int rows, int vocab, long long row_stride,
                                 const int* mode, const float* inv_t,
                                 const unsigned long long* seeds,
                                 const unsigned long long* draws, int* out, int slices,
                                 float* part_v, unsigned* part_i, unsigned* counters,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fail(-1, "sample_rows: vocab=%d", vocab);
    if (mode && (!inv_t || !seeds || !draws))
        return fail(-1, "sample_rows: per-row modes need temperatures, seeds and draw counters");
    if (slices < 1 || slices > SAMPLE_MAX_SLICES) return fail(-1, "sample_rows: %d slices are outside 1..%d", slices, SAMPLE_MAX_SLICES);
    if (slices > 1 && (!part_v || !part_i || !counters)) return fail(-1, "sample_rows: slices need scratch");
    return check_launch("sample_rows", launch(sample_rows_kernel, dim3(rows, slices), SAMPLE_THREADS, 0, stream,
                                                logits, vocab, row_stride, mode, inv_t, seeds, draws, out,
                                                part_v, part_i, counters));
}

// ---------------------------------------------------------------------------------------------
// Temperature sampling from a truncated distribution (top-k, min-p, top-p) on the device.
//
// The truncations are those of the host sampler (crates/vapi-engine/src/sampler.rs:302-376), in
// its order: scaled logits s = l / T; only tokens within 30 nats of the maximum count; top-k keeps
// the k most likely; min-p keeps those whose probability is at least min_p times the largest;
// top-p keeps the smallest set of the most likely tokens whose probability (over the 30-nat
// window, not renormalised after the other cuts) reaches top_p.  Each cut is a threshold on s, so
// the survivors are {s >= tau}; tokens that tie with the last survivor are all kept.  The token is
// then drawn by the Gumbel-max trick over the survivors, with the same keyed noise as
// sample_rows_kernel: an exact draw from the renormalised truncated distribution, deterministic
// in (seed, draw), independent of the batch, and needing no sort.
//
// One block per row.  Thresholds are found by radix descent over an order-preserving 32-bit key of
// s, eight bits a pass: the k-th largest with counts, the top-p cut with probability mass held as
// 64-bit fixed point, so that the sums are integers and do not depend on the order of addition.
constexpr int TR_THREADS = 1024;
constexpr int TR_WARPS = TR_THREADS / 32;
constexpr float TR_WINDOW = 30.f;
constexpr float TR_FIX = 1099511627776.f;      // 2^40: exp(s - max) in (0, 1] as fixed point

__device__ __forceinline__ unsigned tr_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float tr_unkey(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Radix descent: the largest key K with weight({key >= K, s >= tau}) >= target, where the weight
// of an element is 1 (MASS false) or its fixed-point probability (MASS true).  hist is
// [TR_WARPS][256] of 64-bit bins.  Returns false when even all survivors weigh less than target.
template <bool MASS>
__device__ bool tr_descend(const float* __restrict__ l, int vocab, float it, float m, float tau,
                           unsigned long long target, unsigned long long* hist, unsigned long long* bins,
                           unsigned* sh_u, unsigned& key_out) {
    const int warp = threadIdx.x >> 5;
    unsigned prefix = 0;
    for (int level = 0; level < 4; ++level) {
        const int shift = 24 - 8 * level;
        for (int i = threadIdx.x; i < TR_WARPS * 256; i += TR_THREADS) hist[i] = 0ull;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += TR_THREADS) {
            const float sc = l[i] * it;
            if (!(sc >= tau)) continue;
            const unsigned key = tr_key(sc);
            if (level > 0 && (key >> (shift + 8)) != prefix) continue;
            const unsigned long long w = MASS ? (unsigned long long)(expf(sc - m) * TR_FIX) : 1ull;
            atomicAdd(&hist[warp * 256 + ((key >> shift) & 255u)], w);
        }
        __syncthreads();
        if (threadIdx.x < 256) {
            unsigned long long t = 0ull;
            for (int w = 0; w < TR_WARPS; ++w) t += hist[w * 256 + threadIdx.x];
            bins[threadIdx.x] = t;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long above = 0ull;
            int pick = -1;
            for (int b = 255; b >= 0; --b) {
                if (above + bins[b] >= target) { pick = b; break; }
                above += bins[b];
            }
            sh_u[0] = (unsigned)pick;
            if (pick >= 0) bins[256] = target - above;       // what this bin still has to supply
        }
        __syncthreads();
        const int pick = (int)sh_u[0];
        if (pick < 0) return false;                            // (uniform over the block)
        target = bins[256];
        prefix = (prefix << 8) | (unsigned)pick;
        __syncthreads();
    }
    key_out = prefix;
    return true;
}

__global__ void __launch_bounds__(TR_THREADS)
sample_truncated_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                        const float* __restrict__ inv_t, const int* __restrict__ top_k,
                        const float* __restrict__ top_p, const float* __restrict__ min_p,
                        const unsigned long long* __restrict__ seeds,
                        const unsigned long long* __restrict__ draws, int* __restrict__ out,
                        float* __restrict__ tau_out, int* __restrict__ count_out) {
    extern __shared__ __align__(16) unsigned char tr_smem[];
    unsigned long long* hist = reinterpret_cast<unsigned long long*>(tr_smem);         // [TR_WARPS][256]
    unsigned long long* bins = hist + TR_WARPS * 256;                                   // [257]
    __shared__ float sv[32];
    __shared__ unsigned si[32];
    __shared__ unsigned sh_u[2];
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_trigger();
    pdl_wait();
    const int k = top_k ? top_k[row] : 0;
    if (k < 0) return;                                  // not a row of this kernel (uniform over the block)
    const float* l = logits + (size_t)row * row_stride;
    const float it = inv_t[row];

    // the maximum of the scaled logits
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += TR_THREADS) m = fmaxf(m, l[i] * it);
    m = warp_max(m);
    if (lane == 0) sv[warp] = m;
    __syncthreads();
    m = sv[0];
    for (int w = 1; w < TR_WARPS; ++w) m = fmaxf(m, sv[w]);
    __syncthreads();
    float tau = m - TR_WINDOW;

    if (k > 0 && k < vocab) {
        unsigned key;
        if (tr_descend<false>(l, vocab, it, m, tau, (unsigned long long)k, hist, bins, sh_u, key))
            tau = fmaxf(tau, tr_unkey(key));
    }
    const float mp = min_p ? min_p[row] : 0.f;
    if (mp > 0.f) tau = fmaxf(tau, m + logf(mp));
    const float tp = top_p ? top_p[row] : 1.f;
    if (tp < 1.f) {
        // the mass of the whole 30-nat window, in fixed point (integer sums: any order)
        unsigned long long z = 0ull;
        for (int i = threadIdx.x; i < vocab; i += TR_THREADS) {
            const float sc = l[i] * it;
            if (sc >= m - TR_WINDOW) z += (unsigned long long)(expf(sc - m) * TR_FIX);
        }
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        if (lane == 0) bins[warp] = z;
        __syncthreads();
        z = 0ull;
        for (int w = 0; w < TR_WARPS; ++w) z += bins[w];
        __syncthreads();
        const unsigned long long target = (unsigned long long)((double)z * (double)tp);
        unsigned key;
        if (target > 0ull && tr_descend<true>(l, vocab, it, m, tau, target, hist, bins, sh_u, key))
            tau = fmaxf(tau, tr_unkey(key));
    }

    // Gumbel-max over the survivors
    const unsigned long long gkey = mix64(seeds[row] ^ mix64(draws[row] + 0x9E3779B97F4A7C15ULL));
    float bv = -INFINITY;
    unsigned bi = 0xffffffffu;
    int cnt = 0;
    for (unsigned i = threadIdx.x; i < (unsigned)vocab; i += TR_THREADS) {
        const float sc = l[i] * it;
        if (!(sc >= tau)) continue;
        ++cnt;
        const unsigned long long h = mix64(gkey + (unsigned long long)i * 0xBF58476D1CE4E5B9ULL);
        const float u = ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
        arg_better(bv, bi, sc - logf(-logf(u)), i);
    }
    block_argmax(bv, bi, sv, si);
    if (threadIdx.x == 0) out[row] = bi == 0xffffffffu ? 0 : (int)bi;
    if (count_out) {
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        __syncthreads();
        if (lane == 0) si[warp] = (unsigned)cnt;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned t = 0;
            for (int w = 0; w < TR_WARPS; ++w) t += si[w];
            count_out[row] = (int)t;
        }
    }
    if (tau_out && threadIdx.x == 0) tau_out[row] = tau;
}

// One token per row of float32 logits from the truncated distribution; top_k (0: none; negative:
// the row is left alone), top_p (1: none) and min_p (0: none) may each be null.  tau_out / count_out (optional): the threshold on
// the scaled logits and how many tokens survived, for checking.
VAPI_EXPORT int vapi_sample_truncated(const float* logits, int rows, int vocab, long long row_stride,
                                      const float* inv_t, const int* top_k, const float* top_p,
                                      const float* min_p, const unsigned long long* seeds,
                                      const unsigned long long* draws, int* out, float* tau_out,
                                      int* count_out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fail(-1, "sample_truncated: vocab=%d", vocab);
    if (!inv_t || !seeds || !draws || !out) return fail(-1, "sample_truncated: temperatures, seeds, draw counters and an output are needed");
    const size_t smem = (size_t)(TR_WARPS * 256 + 264) * sizeof(unsigned long long);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(sample_truncated_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-101, "sample_truncated: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        attr_set = true;
    }
    return check_launch("sample_truncated", launch(sample_truncated_kernel, rows, TR_THREADS, smem, stream, logits, vocab,
                                                     row_stride, inv_t, top_k, top_p, min_p, seeds, draws, out, tau_out, count_out));
}

// Penalties on (row, token) pairs, in place
// (crates/vapi-engine/src/sampler.rs:262-283, crates/vapi-backend-candle/src/fused.rs:236-250):
// repetition divides a positive logit and multiplies a negative one; frequency subtracts
// freq * count; presence subtracts once when count > 0.  A pair must appear once only.
__global__ void apply_penalties_kernel(float* __restrict__ logits, int vocab, long long row_stride,
                                       const int* __restrict__ rows, const int* __restrict__ toks,
                                       const float* __restrict__ counts,
                                       const float* __restrict__ rep, const float* __restrict__ freq,
                                       const float* __restrict__ pres, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= n) return;
    const int r = rows[i], t = toks[i];
    if (t < 0 || t >= vocab) return;
    float* l = logits + (size_t)r * row_stride + t;
    float v = *l;
    const float p = rep[r];
    if (p != 1.0f) v = v > 0.0f ? v / p : v * p;
    v -= freq[r] * counts[i];
    if (counts[i] > 0.0f) v -= pres[r];
    *l = v;
}

VAPI_EXPORT int vapi_apply_penalties(float* logits, int vocab, long long row_stride,
                                     const int* rows, const int* toks, const float* counts,
                                     const float* rep, const float* freq, const float* pres,
                                     int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return check_launch("apply_penalties", launch(apply_penalties_kernel, (n + 255) / 256, 256, 0, stream,
                                                    logits, vocab, row_stride, rows, toks, counts, rep, freq, pres, n));
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
