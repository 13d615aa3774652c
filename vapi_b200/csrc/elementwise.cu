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

VAPI_EXPORT int vapi_add_rmsnorm(float* x, const void* delta, const float* w, float eps,
                                 const int* rows, void* out, int out_dtype, int n_out,
                                 int hidden, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (hidden <= 0) return fail(-1, "add_rmsnorm: hidden=%d", hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int write_x = rows ? 0 : 1;
    cudaError_t e;
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
    if (blocks > 148 * 16) blocks = 148 * 16;
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

VAPI_EXPORT int vapi_swiglu(const void* g, void* out, int dtype, int rows, int ff,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (ff <= 0) return fail(-1, "swiglu: ff=%d", ff);
    const int threads = 256;
    long long total = (long long)rows * ff;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(swiglu_kernel<float>, (int)blocks, threads, 0, stream, (const float*)g, (float*)out, rows, ff);
    else if (dtype == VAPI_BF16)
        e = launch(swiglu_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, rows, ff);
    else
        return fail(-2, "swiglu: unsupported dtype %d", dtype);
    return check_launch("swiglu", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
