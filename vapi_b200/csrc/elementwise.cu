// Embedding gather, fused residual-add + RMSNorm, and SwiGLU.
//
// What the reference does with library calls (candle RmsNorm, residual adds,
// crates/vapi-backend-candle/src/models/lfm2.rs:633-648, 808-817) and one small
// kernel (swiglu, crates/vapi-backend-candle/src/fused.rs:157-165) is done here
// with the residual stream kept in float: the add of a layer's output into the
// stream and the norm that follows are one pass over the row.
#include "common.cuh"

using namespace vapi;

// ---------------------------------------------------------------------------
// embedding: out[r, :] = float(table[tokens[r], :])
// For a norm that follows (optional): ss = the sum of squares of each produced row, [1][n];
// xw = bfloat16(row * next_w), [n][hidden].
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, float* __restrict__ ss,
                             const float* __restrict__ next_w, __nv_bfloat16* __restrict__ xw,
                             int n, int hidden, int vocab, int* __restrict__ status) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (r >= n) return;
    int tok = tokens[r];
    if (tok < 0 || tok >= vocab) {  // never read outside the table
        if (threadIdx.x == 0 && status) atomicExch(status, 1);
        tok = 0;
    }
    const TW* src = table + (size_t)tok * hidden;
    float* dst = out + (size_t)r * hidden;
    float acc = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f32(src[c]);
        dst[c] = v;
        if (xw) xw[(size_t)r * hidden + c] = __float2bfloat16_rn(v * next_w[c]);
        acc += v * v;
    }
    if (ss) {
        acc = block_sum(acc, red);
        if (threadIdx.x == 0) ss[r] = acc;
    }
}

VAPI_EXPORT int vapi_embed(const void* table, int table_dtype, const int* tokens, float* out,
                           float* ss, const float* next_w, void* xw, int n, int hidden, int vocab,
                           int* status, cudaStream_t stream) {
    if (xw && !next_w) return fail(-1, "embed: a weighted copy needs the next norm's weight");
    if (n <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return fail(-1, "embed: bad sizes hidden=%d vocab=%d", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dtype == VAPI_F32)
        e = launch(embed_kernel<float>, n, threads, 0, stream, (const float*)table, tokens, out, ss, next_w, (__nv_bfloat16*)xw, n, hidden, vocab, status);
    else if (table_dtype == VAPI_BF16)
        e = launch(embed_kernel<__nv_bfloat16>, n, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, ss, next_w, (__nv_bfloat16*)xw, n, hidden, vocab, status);
    else
        return fail(-2, "embed: unsupported table dtype %d", table_dtype);
    return check_launch("embed", e);
}

// ---------------------------------------------------------------------------
// tokens the host does not know yet: tokens[i] = prev[src[i]] where src[i] >= 0.
// An engine that runs one step ahead enqueues a step before it has read what the step before
// sampled; `prev` is that step's sampled output on the device.  Rows outside `prev` are refused.
__global__ void resolve_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                      const int* __restrict__ prev, int n, int prev_rows,
                                      int* __restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i < n) {
        const int r = src[i];
        if (r >= 0) {
            if (r < prev_rows) tokens[i] = prev[r];
            else if (status) atomicExch(status, 1);
        }
    }
}

VAPI_EXPORT int vapi_resolve_tokens(int* tokens, const int* src, const int* prev, int n, int prev_rows,
                                    int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!tokens || !src || !prev || prev_rows <= 0) return fail(-1, "resolve_tokens: missing array");
    cudaError_t e = launch(resolve_tokens_kernel, (n + 127) / 128, 128, 0, stream, tokens, src, prev, n, prev_rows, status);
    return check_launch("resolve_tokens", e);
}

// ---------------------------------------------------------------------------
// fused residual add + RMSNorm.
//   if delta: x[row] += float(delta[row])           (x is the float residual stream)
//   out[j]   = T( x[row] * rsqrt(mean(x[row]^2) + eps) * w )
// rows == nullptr: row = j for j in [0, n_out), and x is updated in place.
// rows != nullptr: row = rows[j]; x is NOT written (several j may name one row),
//                  the sum x+delta is formed on the fly.
// Mean and rsqrt in float; the sum of squares is reduced in an order that depends
// only on the block size.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                   const float* __restrict__ w, float eps,
                                   const int* __restrict__ rows, T* __restrict__ out,
                                   int n_out, int hidden, int write_x) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (dr) {
            v += to_f32(dr[c]);
            if (write_x) xr[c] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    T* orow = out + (size_t)j * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (dr && !write_x) v += to_f32(dr[c]);
        orow[c] = from_f32<T>(v * inv * w[c]);
    }
}

// The same with 16-byte accesses and the row held in registers between the two passes
// (hidden a multiple of 4, at most 4 * 4 * blockDim elements): one read of x and delta, one
// write of x, one write of the output.
template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&a);
        u.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

constexpr int NORM_KMAX = 4;

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                       const float* __restrict__ w, float eps,
                                       const int* __restrict__ rows, T* __restrict__ out,
                                       int n_out, int hidden, int write_x) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
    const int h4 = hidden >> 2;
    float4 v[NORM_KMAX];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < h4) {
            v[k] = Pack4<float>::load(xr + 4 * c);
            if (dr) {
                const float4 d = Pack4<T>::load(dr + 4 * c);
                v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
                if (write_x) Pack4<float>::store(xr + 4 * c, v[k]);
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    T* orow = out + (size_t)j * hidden;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < h4) {
            const float4 wv = Pack4<float>::load(w + 4 * c);
            Pack4<T>::store(orow + 4 * c, make_float4(v[k].x * inv * wv.x, v[k].y * inv * wv.y, v[k].z * inv * wv.z, v[k].w * inv * wv.w));
        }
    }
}

VAPI_EXPORT int vapi_add_rmsnorm(float* x, const void* delta, const float* w, float eps,
                                 const int* rows, void* out, int out_dtype, int n_out,
                                 int hidden, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (hidden <= 0) return fail(-1, "add_rmsnorm: hidden=%d", hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int write_x = rows ? 0 : 1;
    cudaError_t e;
    if (hidden % 4 == 0 && hidden <= 4 * NORM_KMAX * 256 && (out_dtype == VAPI_F32 || out_dtype == VAPI_BF16)) {
        const int vt = hidden >= 1024 ? 256 : 128;
        if (hidden / 4 <= NORM_KMAX * vt) {
            if (out_dtype == VAPI_F32)
                e = launch(add_rmsnorm_vec_kernel<float>, n_out, vt, 0, stream, x, (const float*)delta, w, eps, rows, (float*)out, n_out, hidden, write_x);
            else
                e = launch(add_rmsnorm_vec_kernel<__nv_bfloat16>, n_out, vt, 0, stream, x, (const __nv_bfloat16*)delta, w, eps, rows, (__nv_bfloat16*)out, n_out, hidden, write_x);
            return check_launch("add_rmsnorm", e);
        }
    }
    if (out_dtype == VAPI_F32)
        e = launch(add_rmsnorm_kernel<float>, n_out, threads, 0, stream, x, (const float*)delta, w, eps, rows, (float*)out, n_out, hidden, write_x);
    else if (out_dtype == VAPI_BF16)
        e = launch(add_rmsnorm_kernel<__nv_bfloat16>, n_out, threads, 0, stream, x, (const __nv_bfloat16*)delta, w, eps, rows, (__nv_bfloat16*)out, n_out, hidden, write_x);
    else
        return fail(-2, "add_rmsnorm: unsupported dtype %d", out_dtype);
    return check_launch("add_rmsnorm", e);
}

// residual add alone (used at the very end of a step when nothing follows the
// last layer but the stream itself is wanted): x += delta
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) x[i] += to_f32(delta[i]);
}

// x[row] += delta[row]; ss[row] = sum of squares of the new row; xw = bfloat16(new row * next_w)
// (one block per row)
template <typename T>
__global__ void add_residual_ss_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                       float* __restrict__ ss, const float* __restrict__ next_w,
                                       __nv_bfloat16* __restrict__ xw, int n, int hidden) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (r >= n) return;
    float acc = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = x[(size_t)r * hidden + c] + to_f32(delta[(size_t)r * hidden + c]);
        x[(size_t)r * hidden + c] = v;
        if (xw) xw[(size_t)r * hidden + c] = __float2bfloat16_rn(v * next_w[c]);
        acc += v * v;
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) ss[r] = acc;
}

VAPI_EXPORT int vapi_add_residual_ss(float* x, const void* delta, int dtype, float* ss,
                                     const float* next_w, void* xw, int n, int hidden,
                                     cudaStream_t stream) {
    if (n <= 0) return 0;
    if (xw && !next_w) return fail(-1, "add_residual_ss: a weighted copy needs the next norm's weight");
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(add_residual_ss_kernel<float>, n, 256, 0, stream, x, (const float*)delta, ss, next_w, (__nv_bfloat16*)xw, n, hidden);
    else if (dtype == VAPI_BF16)
        e = launch(add_residual_ss_kernel<__nv_bfloat16>, n, 256, 0, stream, x, (const __nv_bfloat16*)delta, ss, next_w, (__nv_bfloat16*)xw, n, hidden);
    else
        return fail(-2, "add_residual_ss: unsupported dtype %d", dtype);
    return check_launch("add_residual_ss", e);
}

VAPI_EXPORT int vapi_add_residual(float* x, const void* delta, int dtype, long long total,
                                  cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(add_residual_kernel<float>, (int)blocks, threads, 0, stream, x, (const float*)delta, (size_t)total);
    else if (dtype == VAPI_BF16)
        e = launch(add_residual_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, x, (const __nv_bfloat16*)delta, (size_t)total);
    else
        return fail(-2, "add_residual: unsupported dtype %d", dtype);
    return check_launch("add_residual", e);
}

// ---------------------------------------------------------------------------
// SwiGLU on a stacked gate/up product: out[r, c] = silu(g[r, c]) * g[r, F + c],
// silu(v) = v / (1 + exp(-v)); float math, one rounding
// (crates/vapi-backend-candle/src/fused.rs:16-25, 157-165).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ g, T* __restrict__ out, int rows, int ff) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rows * ff;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) {
        const size_t r = i / ff, c = i - r * ff;
        const float a = to_f32(g[r * 2 * ff + c]);
        const float b = to_f32(g[r * 2 * ff + ff + c]);
        const float s = a / (1.f + expf(-a));
        out[i] = from_f32<T>(s * b);
    }
}

// four outputs per thread with 16-byte (float) / 8-byte (bfloat16) accesses; ff a multiple of 4
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ g, T* __restrict__ out, int rows, int ff) {
    const int f4 = ff >> 2;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rows * f4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) {
        const size_t r = i / f4, c = (i - r * f4) << 2;
        const float4 a = Pack4<T>::load(g + r * 2 * ff + c);
        const float4 b = Pack4<T>::load(g + r * 2 * ff + ff + c);
        Pack4<T>::store(out + r * ff + c, make_float4(a.x / (1.f + expf(-a.x)) * b.x, a.y / (1.f + expf(-a.y)) * b.y,
                                                      a.z / (1.f + expf(-a.z)) * b.z, a.w / (1.f + expf(-a.w)) * b.w));
    }
}

// bfloat16, ff a multiple of 8: one thread per eight outputs of one row, 16-byte accesses, no
// loop and no index division (the row is the block's y index)
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ out, int ff) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) << 3;
    const size_t r = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    if (c >= ff) return;
    const uint4 a = *reinterpret_cast<const uint4*>(g + r * 2 * ff + c);
    const uint4 b = *reinterpret_cast<const uint4*>(g + r * 2 * ff + ff + c);
    const unsigned aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    unsigned o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
        const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
        __nv_bfloat162 y = __floats2bfloat162_rn(x.x / (1.f + expf(-x.x)) * u.x, x.y / (1.f + expf(-x.y)) * u.y);
        o[i] = *reinterpret_cast<unsigned*>(&y);
    }
    *reinterpret_cast<uint4*>(out + r * ff + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

VAPI_EXPORT int vapi_swiglu(const void* g, void* out, int dtype, int rows, int ff,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (ff <= 0) return fail(-1, "swiglu: ff=%d", ff);
    const int threads = 256;
    long long total = (long long)rows * ff;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > sm_count() * 32) blocks = sm_count() * 32;
    cudaError_t e;
    if (dtype == VAPI_BF16 && ff % 8 == 0 && rows <= 65535) {
        const int th = 128;
        dim3 grid((ff / 8 + th - 1) / th, rows);
        e = launch(swiglu_bf16x8_kernel, grid, th, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, ff);
        return check_launch("swiglu", e);
    }
    if (ff % 4 == 0 && (dtype == VAPI_F32 || dtype == VAPI_BF16)) {
        long long vb = (total / 4 + threads - 1) / threads;
        if (vb > sm_count() * 16) vb = sm_count() * 16;
        if (dtype == VAPI_F32) e = launch(swiglu_vec_kernel<float>, (int)vb, threads, 0, stream, (const float*)g, (float*)out, rows, ff);
        else e = launch(swiglu_vec_kernel<__nv_bfloat16>, (int)vb, threads, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, rows, ff);
        return check_launch("swiglu", e);
    }
    if (dtype == VAPI_F32)
        e = launch(swiglu_kernel<float>, (int)blocks, threads, 0, stream, (const float*)g, (float*)out, rows, ff);
    else if (dtype == VAPI_BF16)
        e = launch(swiglu_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, rows, ff);
    else
        return fail(-2, "swiglu: unsupported dtype %d", dtype);
    return check_launch("swiglu", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
