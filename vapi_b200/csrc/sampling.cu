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
    const unsigned per = ((unsigned)vocab + slices - 1) / slices;
    const unsigned lo = slice * per, hi = min((unsigned)vocab, lo + per);
    float bv = -INFINITY;
    unsigned bi = 0xffffffffu;
    if (md == 1) {
        for (unsigned i = lo + threadIdx.x; i < hi; i += blockDim.x) arg_better(bv, bi, l[i], i);
    } else {
        const float it = inv_t[row];
        const unsigned long long key = mix64(seeds[row] ^ mix64(draws[row] + 0x9E3779B97F4A7C15ULL));
        for (unsigned i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const unsigned long long h = mix64(key + (unsigned long long)i * 0xBF58476D1CE4E5B9ULL);
            const float u = ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
            const float g = -logf(-logf(u));
            arg_better(bv, bi, l[i] * it + g, i);
        }
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
