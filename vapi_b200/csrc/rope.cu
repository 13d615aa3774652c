// Rotary position tables for a step, and the fused per-head q/k RMSNorm + RoPE +
// paged K/V write that follows the q/k/v projection.
//
// Reference behaviour: inv_freq_i = 1 / theta^(2i/d) and angle = p * inv_freq_i in
// float (crates/vapi-backend-candle/src/models/lfm2.rs:163-183); per-head RMSNorm of
// q and k, then rotate-half RoPE (pairs (i, i + d/2)), then the roped-normed k and
// the raw v go to the token's cache slot (lfm2.rs:343-375).  Here the angles, the
// norm and the rotation are float end to end with one rounding at the store.
#include "common.cuh"

using namespace vapi;

// cos/sin rows for the step's tokens: [n, half] each, float.
__global__ void rope_cos_sin_kernel(const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq,
                                    float* __restrict__ cosr, float* __restrict__ sinr,
                                    int n, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= n * half) return;
    const int t = i / half, j = i - t * half;
    const float a = (float)positions[t] * inv_freq[j];
    cosr[i] = cosf(a);
    sinr[i] = sinf(a);
}

VAPI_EXPORT int vapi_rope_cos_sin(const int* positions, const float* inv_freq, float* cosr,
                                  float* sinr, int n, int half, cudaStream_t stream) {
    if (n <= 0 || half <= 0) return 0;
    const int total = n * half;
    return check_launch("rope_cos_sin", launch(rope_cos_sin_kernel, (total + 255) / 256, 256, 0, stream,
                                                 positions, inv_freq, cosr, sinr, n, half));
}

// One warp per (token, head).  Heads are laid out in a qkv row as
// [q heads | k heads | v heads], each head_dim wide.
//   q: norm (if qw) -> rope (if cosr) -> written back in place
//   k: norm (if kw) -> rope (if cosr) -> written to the cache slot (if cache)
//   v: copied to the cache slot (if cache)
// Cache layer layout: [num_pages, 2 (k,v), n_kv, page_size, head_dim].
constexpr int QK_WARPS = 4;
constexpr int QK_MAX_D = 256;

template <typename T>
__global__ void qk_norm_rope_write_kernel(T* __restrict__ qkv, const float* __restrict__ qw,
                                          const float* __restrict__ kw, float eps,
                                          const float* __restrict__ cosr,
                                          const float* __restrict__ sinr, int rot,
                                          T* __restrict__ cache,
                                          const int* __restrict__ slot_mapping, int n, int nh,
                                          int nkv, int d, int page_size, int num_pages,
                                          int* __restrict__ status) {
    __shared__ float sh[QK_WARPS][QK_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = nh + 2 * nkv;
    const long long item = (long long)blockIdx.x * QK_WARPS + warp;
    pdl_trigger();
    if (item >= (long long)n * heads) {
        pdl_wait();
        return;
    }
    const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
    const int slot_pre = (cache && h >= nh) ? slot_mapping[t] : 0;     // host-copied index data: safe before the wait
    pdl_wait();
    T* src = qkv + (size_t)t * heads * d + (size_t)h * d;
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
    const bool rope = (is_q || is_k) && cosr != nullptr;
    float* s = sh[warp];

    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = to_f32(src[i]);
        s[i] = v;
        ss += v * v;
    }
    float inv = 1.f;
    if (w) {
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)d + eps);
    }
    __syncwarp();

    T* dst = nullptr;
    if (is_q) {
        dst = src;
    } else if (cache) {
        const int slot = slot_pre;
        const int page = slot / page_size, off = slot - page * page_size;
        if (slot < 0 || page >= num_pages) {
            if (lane == 0 && status) atomicExch(status, 2);
            return;
        }
        const int g = is_k ? h - nh : h - nh - nkv;
        dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + g) * page_size + off) * d;
    }
    if (!dst) return;

    const int half = rot >> 1;
    for (int i = lane; i < d; i += 32) {
        float v = w ? s[i] * inv * w[i] : s[i];
        if (rope && i < rot) {
            const int j = i < half ? i : i - half;
            const int pi = i < half ? i + half : i - half;
            const float pv = w ? s[pi] * inv * w[pi] : s[pi];
            const float c = cosr[(size_t)t * half + j], sn = sinr[(size_t)t * half + j];
            v = i < half ? v * c - pv * sn : v * c + pv * sn;
        }
        dst[i] = from_f32<T>(v);
    }
}

// The same work with 16-byte accesses, for a rotation over the whole head (rot == d) and a
// half head that 16-byte groups tile evenly: a group of G = (d/2) / VEC lanes (a power of two)
// takes one (token, head); each lane holds VEC elements of the first half and their rotation
// partners in the second half, so no shared memory is needed.
template <typename T> struct Pack16;
template <> struct Pack16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Pack16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 a = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<unsigned*>(&a);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <typename T>
__global__ void qk_norm_rope_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ qw,
                                              const float* __restrict__ kw, float eps,
                                              const float* __restrict__ cosr,
                                              const float* __restrict__ sinr, T* __restrict__ cache,
                                              const int* __restrict__ slot_mapping, int n, int nh,
                                              int nkv, int d, int page_size, int num_pages, int G,
                                              int* __restrict__ status) {
    constexpr int VEC = Pack16<T>::N;
    const int heads = nh + 2 * nkv, half = d >> 1;
    const long long gl = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long item = gl / G;
    const int sub = (int)(gl - item * G);
    const bool active = item < (long long)n * heads;     // whole groups are active or not
    const int t = active ? (int)(item / heads) : 0, h = active ? (int)(item - (long long)t * heads) : 0;
    pdl_trigger();
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    const int slot = (active && cache && !is_q) ? slot_mapping[t] : 0;     // host-copied index data
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
    const bool rope = (is_q || is_k) && cosr != nullptr;
    const int e = sub * VEC;                               // this lane's elements: e.. and half+e..
    float wl[VEC], wh[VEC];
    if (w) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float4 a = *reinterpret_cast<const float4*>(w + e + i);
            const float4 b = *reinterpret_cast<const float4*>(w + half + e + i);
            wl[i] = a.x; wl[i + 1] = a.y; wl[i + 2] = a.z; wl[i + 3] = a.w;
            wh[i] = b.x; wh[i + 1] = b.y; wh[i + 2] = b.z; wh[i + 3] = b.w;
        }
    }
    pdl_wait();         // the row and the cos/sin tables come from kernels of this step
    float c[VEC], sn[VEC];
    if (rope && active) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float4 a = *reinterpret_cast<const float4*>(cosr + (size_t)t * half + e + i);
            const float4 b = *reinterpret_cast<const float4*>(sinr + (size_t)t * half + e + i);
            c[i] = a.x; c[i + 1] = a.y; c[i + 2] = a.z; c[i + 3] = a.w;
            sn[i] = b.x; sn[i + 1] = b.y; sn[i + 2] = b.z; sn[i + 3] = b.w;
        }
    }
    T* src = qkv + (size_t)t * heads * d + (size_t)h * d;
    float lo[VEC], hi[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) lo[i] = hi[i] = 0.f;
    if (active) {
        Pack16<T>::load(src + e, lo);
        Pack16<T>::load(src + half + e, hi);
    }
    float inv = 1.f;
    if (qw || kw) {     // (uniform over the warp: every lane takes part in the shuffles)
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
        for (int o = G >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        inv = rsqrtf(ss / (float)d + eps);
    }
    if (!active) return;
    T* dst = nullptr;
    if (is_q) {
        dst = src;
    } else if (cache) {
        const int page = slot / page_size, off = slot - page * page_size;
        if (slot < 0 || page >= num_pages) {
            if (sub == 0 && status) atomicExch(status, 2);
            return;
        }
        const int g = is_k ? h - nh : h - nh - nkv;
        dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + g) * page_size + off) * d;
    }
    if (!dst) return;
    if (w) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            lo[i] = lo[i] * inv * wl[i];
            hi[i] = hi[i] * inv * wh[i];
        }
    }
    if (rope) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float a = lo[i], b = hi[i];
            lo[i] = a * c[i] - b * sn[i];
            hi[i] = b * c[i] + a * sn[i];
        }
    }
    Pack16<T>::store(dst + e, lo);
    Pack16<T>::store(dst + half + e, hi);
}

VAPI_EXPORT int vapi_qk_norm_rope_write(void* qkv, int dtype, const float* qw, const float* kw,
                                        float eps, const float* cosr, const float* sinr, int rot,
                                        void* cache, const int* slot_mapping, int n, int nh,
                                        int nkv, int d, int page_size, int num_pages,
                                        int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || d > QK_MAX_D || (d % 2) != 0)
        return fail(-1, "qk_norm_rope_write: head_dim %d is not an even size up to %d", d, QK_MAX_D);
    if (cosr && (rot <= 0 || rot > d || (rot % 2) != 0))
        return fail(-1, "qk_norm_rope_write: rotary width %d does not fit head_dim %d", rot, d);
    if (nh <= 0 || nkv < 0) return fail(-1, "qk_norm_rope_write: bad head counts %d/%d", nh, nkv);
    if (cache && (page_size <= 0 || num_pages <= 0 || !slot_mapping))
        return fail(-1, "qk_norm_rope_write: cache given without pages or slot mapping");
    const long long items = (long long)n * (nh + 2 * nkv);
    const int blocks = (int)((items + QK_WARPS - 1) / QK_WARPS);
    cudaError_t e;
    {
        // 16-byte form: whole-head rotation (or none) and half a head tiled by 16-byte groups
        const int vec = dtype == VAPI_BF16 ? 8 : 4;
        const int half = d / 2;
        const int G = half % vec == 0 ? half / vec : 0;
        if ((dtype == VAPI_BF16 || dtype == VAPI_F32) && (!cosr || rot == d) && G >= 1 && G <= 32 && (G & (G - 1)) == 0) {
            const long long lanes = items * G;
            const int vblocks = (int)((lanes + 127) / 128);
            if (dtype == VAPI_F32)
                e = launch(qk_norm_rope_write_vec_kernel<float>, vblocks, 128, 0, stream, (float*)qkv, qw, kw, eps,
                           cosr, sinr, (float*)cache, slot_mapping, n, nh, nkv, d, page_size, num_pages, G, status);
            else
                e = launch(qk_norm_rope_write_vec_kernel<__nv_bfloat16>, vblocks, 128, 0, stream,
                           (__nv_bfloat16*)qkv, qw, kw, eps, cosr, sinr, (__nv_bfloat16*)cache, slot_mapping, n,
                           nh, nkv, d, page_size, num_pages, G, status);
            return check_launch("qk_norm_rope_write", e);
        }
    }
    if (dtype == VAPI_F32)
        e = launch(qk_norm_rope_write_kernel<float>, blocks, QK_WARPS * 32, 0, stream,
                   (float*)qkv, qw, kw, eps, cosr, sinr, rot, (float*)cache, slot_mapping, n, nh, nkv, d,
                   page_size, num_pages, status);
    else if (dtype == VAPI_BF16)
        e = launch(qk_norm_rope_write_kernel<__nv_bfloat16>, blocks, QK_WARPS * 32, 0, stream,
                   (__nv_bfloat16*)qkv, qw, kw, eps, cosr, sinr, rot, (__nv_bfloat16*)cache,
                   slot_mapping, n, nh, nkv, d, page_size, num_pages, status);
    else
        return fail(-2, "qk_norm_rope_write: unsupported dtype %d", dtype);
    return check_launch("qk_norm_rope_write", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
