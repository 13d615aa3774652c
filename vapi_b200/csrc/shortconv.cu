// The gated short convolution between in_proj and out_proj, with its rolling state.
//
// Math of the reference (crates/vapi-backend-candle/src/models/lfm2.rs:509-565 and the
// conv_write / conv_apply kernels, crates/vapi-backend-candle/src/fused.rs:167-233):
//   h3 = [B | C | x] (+ in_proj bias);  g[t] = B[t] * x[t], rounded to the storage type;
//   conv[t][c] = sum_k w[k][c] * g[t - (L-1-k)][c] (+ conv bias), g before the start of
//   the sequence = 0;  y[t] = C[t] * conv[t], one rounding.
//
// The reference keeps g per token in paged rows and gathers L-1 predecessors through the
// block table.  Here each request owns one fixed-size state per conv layer, the last L-1
// rows of g, [L-1, H] in the storage type.  One kernel serves prompt portions of any
// length (down to one token, shorter than the state) and decode tokens:
//   * a token at index i >= L-1 of its portion needs only rows of this step;
//   * the tokens i < L-1 need the old state.  They are all handled, one after the other,
//     by the thread of token i == 0, which reads the old state into registers before it
//     writes the new one: no other thread reads or writes that request's state, so there
//     is no ordering to arrange between blocks;
//   * rows of the state that stand for positions before 0 are never read (taken as zero),
//     so a slot needs no clearing when another request takes it over.
#include "common.cuh"

using namespace vapi;

constexpr int CONV_LMAX = 8;
#ifndef SC_TT_N
#define SC_TT_N 4
#endif
constexpr int SC_TT = SC_TT_N;          // tokens of a tile in the prompt-sized form

// V consecutive channels of one row as floats (V = 1, or 4 with one 16-byte / 8-byte access)
template <typename T, int V> struct Chan;
template <typename T> struct Chan<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = to_f32(p[0]); }
    static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { p[0] = from_f32<T>(v[0]); }
};
template <> struct Chan<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Chan<__nv_bfloat16, 4> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&a);
        u.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <> struct Chan<__nv_bfloat16, 8> {
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

// g = (B + bias_B) * (x + bias_x) of one row, rounded to the storage type
template <typename T, int V>
__device__ __forceinline__ void gate_row(const T* __restrict__ h3, const float* __restrict__ in_bias,
                                         size_t row, int c, int hidden, float (&g)[V]) {
    const T* r = h3 + row * 3 * (size_t)hidden;
    float b[V], x[V];
    Chan<T, V>::load(r + c, b);
    Chan<T, V>::load(r + 2 * hidden + c, x);
#pragma unroll
    for (int v = 0; v < V; ++v) {
        if (in_bias) {
            b[v] += in_bias[c + v];
            x[v] += in_bias[2 * hidden + c + v];
        }
        g[v] = round_to<T>(b[v] * x[v]);
    }
}

template <typename T, int V>
__device__ __forceinline__ void emit(const T* __restrict__ h3, const float* __restrict__ in_bias,
                                     const float* __restrict__ conv_bias, T* __restrict__ out,
                                     size_t row, int c, int hidden, const float (&acc)[V]) {
    float cc[V], y[V];
    Chan<T, V>::load(h3 + row * 3 * (size_t)hidden + hidden + c, cc);
#pragma unroll
    for (int v = 0; v < V; ++v) {
        if (in_bias) cc[v] += in_bias[hidden + c + v];
        y[v] = cc[v] * (acc[v] + (conv_bias ? conv_bias[c + v] : 0.f));
    }
    Chan<T, V>::store(out + row * (size_t)hidden + c, y);
}

// One block row (index bx) of the per-token form.  heads_only: bx is a sequence, and the work is
// its first L-1 tokens and its state (the other tokens belong to the tiled form); else bx is a token.
template <typename T, int V>
__device__ __forceinline__ void shortconv_token_body(
        const T* __restrict__ h3, const float* __restrict__ in_bias,
        const float* __restrict__ taps,  // [L, H], k = 0 oldest
        const float* __restrict__ conv_bias, T* __restrict__ state, long long slot_stride,
        const int* __restrict__ state_slots, const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
        const int* __restrict__ positions, T* __restrict__ out, int n, int hidden, int L, int num_slots,
        int heads_only, int* __restrict__ status, int bx) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int r = heads_only ? cu_q[bx] : bx;
    pdl_trigger();
    if (c >= hidden || r >= n) {
        pdl_wait();
        return;
    }
    // Everything read up to pdl_wait() was written before this step's first kernel began
    // (index data copied from the host, weights, the state the previous step left), so it can
    // be fetched while the kernel before this one is still finishing.
    const int s = heads_only ? bx : tok_seq[r];
    const int r0 = cu_q[s], q = cu_q[s + 1] - r0;
    const int i = r - r0;
    if (q <= 0) {       // (a sequence without tokens in this step)
        pdl_wait();
        return;
    }
    float w[CONV_LMAX][V];
#pragma unroll
    for (int k = 0; k < CONV_LMAX; ++k)
#pragma unroll
        for (int v = 0; v < V; ++v) w[k][v] = k < L ? taps[(size_t)k * hidden + c + v] : 0.f;
    int slot = -1, p0 = 0;
    float hist[CONV_LMAX][V];
#pragma unroll
    for (int j = 0; j < CONV_LMAX; ++j)
#pragma unroll
        for (int v = 0; v < V; ++v) hist[j][v] = 0.f;
    if (i == 0 && L > 1) {
        slot = state_slots[s];
        p0 = positions[r];
        if (slot >= 0 && slot < num_slots) {
            const T* st0 = state + (size_t)slot * slot_stride;
            // hist[0 .. L-2] = g at positions p0-(L-1) .. p0-1; hist[L-1] = the current token
#pragma unroll
            for (int j = 0; j < CONV_LMAX; ++j)
                if (j < L - 1 && p0 - (L - 1) + j >= 0) Chan<T, V>::load(st0 + (size_t)j * hidden + c, hist[j]);
        }
    }
    pdl_wait();

    if (i >= L - 1 && !heads_only) {
        // every tap lies inside this step's rows
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
        for (int k = 0; k < CONV_LMAX; ++k)
            if (k < L) {
                float g[V];
                gate_row<T, V>(h3, in_bias, (size_t)(r - (L - 1 - k)), c, hidden, g);
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] += w[k][v] * g[v];
            }
        emit<T, V>(h3, in_bias, conv_bias, out, (size_t)r, c, hidden, acc);
        return;
    }
    if (i != 0) return;  // tokens 1 .. L-2 of a portion belong to the thread of token 0

    if (slot < 0 || slot >= num_slots) {
        if (status) atomicExch(status, 3);
        return;
    }
    T* st = state + (size_t)slot * slot_stride;
    const int m = q < L - 1 ? q : L - 1;
    for (int ii = 0; ii < m; ++ii) {
        float g[V], acc[V];
        gate_row<T, V>(h3, in_bias, (size_t)(r + ii), c, hidden, g);
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
        for (int k = 0; k < CONV_LMAX; ++k)
#pragma unroll
            for (int v = 0; v < V; ++v) {
                if (k < L - 1) acc[v] += w[k][v] * hist[k][v];
                if (k == L - 1) acc[v] += w[k][v] * g[v];
            }
        emit<T, V>(h3, in_bias, conv_bias, out, (size_t)(r + ii), c, hidden, acc);
        // slide: drop the oldest row, the current one becomes the newest of the history
#pragma unroll
        for (int k = 0; k < CONV_LMAX - 1; ++k)
#pragma unroll
            for (int v = 0; v < V; ++v)
                if (k < L - 2) hist[k][v] = hist[k + 1][v];
#pragma unroll
        for (int k = 0; k < CONV_LMAX; ++k)
#pragma unroll
            for (int v = 0; v < V; ++v)
                if (k == L - 2) hist[k][v] = g[v];
    }
    // the new state: the last L-1 rows of g up to position p0 + q - 1
    if (q <= L - 1) {
#pragma unroll
        for (int j = 0; j < CONV_LMAX; ++j)
            if (j < L - 1) Chan<T, V>::store(st + (size_t)j * hidden + c, hist[j]);
    } else {
        for (int j = 0; j < L - 1; ++j) {
            float g[V];
            gate_row<T, V>(h3, in_bias, (size_t)(r + q - (L - 1) + j), c, hidden, g);
            Chan<T, V>::store(st + (size_t)j * hidden + c, g);
        }
    }
}

template <typename T, int V>
__global__ void shortconv_kernel(const T* __restrict__ h3, const float* __restrict__ in_bias,
                                 const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                 T* __restrict__ state, long long slot_stride,
                                 const int* __restrict__ state_slots, const int* __restrict__ tok_seq,
                                 const int* __restrict__ cu_q, const int* __restrict__ positions,
                                 T* __restrict__ out, int n, int hidden, int L, int num_slots,
                                 int* __restrict__ status) {
    shortconv_token_body<T, V>(h3, in_bias, taps, conv_bias, state, slot_stride, state_slots, tok_seq, cu_q, positions,
                               out, n, hidden, L, num_slots, 0, status, (int)blockIdx.x);
}

// Prompt portions: the tokens at index >= L-1 of their portion need nothing but rows of this
// step.  One thread takes TT consecutive tokens of V channels, so the L-1 predecessor rows are
// computed once per tile instead of once per token and all of a thread's loads are in flight
// together.  Tokens nearer to the start of their portion (and the state) are left to
// shortconv_kernel in its heads_only form.
template <typename T, int V, int LT, int TT>
__device__ __forceinline__ void shortconv_tile_body(const T* __restrict__ h3, const float* __restrict__ in_bias,
                                                    const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                                    const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                                                    T* __restrict__ out, int n, int hidden, int tile) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int r0 = tile * TT;
    pdl_trigger();
    if (c >= hidden) {
        pdl_wait();
        return;
    }
    bool mine[TT], any = false;
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        const int r = r0 + t;
        mine[t] = r < n && (r - cu_q[tok_seq[r < n ? r : n - 1]]) >= LT - 1;
        any = any || mine[t];
    }
    float w[LT][V];
#pragma unroll
    for (int k = 0; k < LT; ++k)
#pragma unroll
        for (int v = 0; v < V; ++v) w[k][v] = taps[(size_t)k * hidden + c + v];
    pdl_wait();
    if (!any) return;
    float g[TT + LT - 1][V];
#pragma unroll
    for (int j = 0; j < TT + LT - 1; ++j) {
        const int row = r0 - (LT - 1) + j;
        if (row >= 0 && row < n) {
            gate_row<T, V>(h3, in_bias, (size_t)row, c, hidden, g[j]);
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v) g[j][v] = 0.f;
        }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        if (!mine[t]) continue;
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
        for (int k = 0; k < LT; ++k)
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] += w[k][v] * g[t + k][v];
        emit<T, V>(h3, in_bias, conv_bias, out, (size_t)(r0 + t), c, hidden, acc);
    }
}

// A prompt-sized step in one launch: the first num_seqs block rows do the heads of the sequences
// (their first L-1 tokens and the state), the others one tile of TT tokens each, side by side.
template <typename T, int V, int LT, int TT>
__global__ void shortconv_prompt_kernel(const T* __restrict__ h3, const float* __restrict__ in_bias,
                                        const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                        T* __restrict__ state, long long slot_stride,
                                        const int* __restrict__ state_slots, const int* __restrict__ tok_seq,
                                        const int* __restrict__ cu_q, const int* __restrict__ positions,
                                        T* __restrict__ out, int n, int num_seqs, int hidden, int num_slots,
                                        int* __restrict__ status) {
    if ((int)blockIdx.x < num_seqs)
        shortconv_token_body<T, V>(h3, in_bias, taps, conv_bias, state, slot_stride, state_slots, tok_seq, cu_q,
                                   positions, out, n, hidden, LT, num_slots, 1, status, (int)blockIdx.x);
    else
        shortconv_tile_body<T, V, LT, TT>(h3, in_bias, taps, conv_bias, tok_seq, cu_q, out, n, hidden,
                                          (int)blockIdx.x - num_seqs);
}

template <typename T, int V>
static cudaError_t launch_prompt(int L, dim3 grid, int threads, cudaStream_t stream, const void* h3,
                                 const float* in_bias, const float* taps, const float* conv_bias, void* state,
                                 long long slot_stride, const int* state_slots, const int* tok_seq,
                                 const int* cu_q, const int* positions, void* out, int n, int num_seqs,
                                 int hidden, int num_slots, int* status) {
#define SC_PROMPT(LT)                                                                                     \
    return launch(shortconv_prompt_kernel<T, V, LT, SC_TT>, grid, threads, 0, stream, (const T*)h3, in_bias, taps, \
                  conv_bias, (T*)state, slot_stride, state_slots, tok_seq, cu_q, positions, (T*)out, n, num_seqs, \
                  hidden, num_slots, status)
    switch (L) {
        case 2: SC_PROMPT(2);
        case 3: SC_PROMPT(3);
        case 4: SC_PROMPT(4);
        case 5: SC_PROMPT(5);
    }
#undef SC_PROMPT
    return cudaErrorInvalidValue;
}

VAPI_EXPORT int vapi_shortconv(const void* h3, int dtype, const float* in_bias, const float* taps,
                               const float* conv_bias, void* state, long long slot_stride,
                               const int* state_slots, const int* tok_seq, const int* cu_q,
                               const int* positions, void* out, int n, int num_seqs, int hidden, int L,
                               int num_slots, int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (L < 1 || L > CONV_LMAX)
        return fail(-1, "shortconv: kernel length %d is outside 1..%d", L, CONV_LMAX);
    if (hidden <= 0) return fail(-1, "shortconv: hidden=%d", hidden);
    if (L > 1 && (!state || num_slots <= 0)) return fail(-1, "shortconv: no state buffer");
    const int threads = 128;
    // four channels a thread when rows and state rows stay 16-byte (float) / 8-byte (bfloat16) aligned
    const bool vec = hidden % 4 == 0 && slot_stride % 4 == 0;
    const int per = vec ? 4 : 1;
    const int cblocks = (hidden / per + threads - 1) / threads;
    if (cblocks > 65535) return fail(-1, "shortconv: hidden=%d is too wide for the grid", hidden);
    // prompt-sized steps: tiles of tokens for everything past the first L-1 tokens of a portion,
    // the per-token form only for those first tokens and the state, in one launch
    const int tile_v = dtype == VAPI_BF16 ? 8 : 4;
    const bool tiled = n >= 256 && num_seqs > 0 && num_seqs * 8 <= n && L >= 2 && L <= 5 && hidden % tile_v == 0 &&
                       slot_stride % tile_v == 0 && (dtype == VAPI_BF16 || dtype == VAPI_F32);
    cudaError_t e;
    if (tiled) {
        const int tcb = (hidden / tile_v + threads - 1) / threads;
        dim3 grid(num_seqs + (n + SC_TT - 1) / SC_TT, tcb);
        if (dtype == VAPI_F32)
            e = launch_prompt<float, 4>(L, grid, threads, stream, h3, in_bias, taps, conv_bias, state, slot_stride,
                                        state_slots, tok_seq, cu_q, positions, out, n, num_seqs, hidden, num_slots, status);
        else
            e = launch_prompt<__nv_bfloat16, 8>(L, grid, threads, stream, h3, in_bias, taps, conv_bias, state, slot_stride,
                                                state_slots, tok_seq, cu_q, positions, out, n, num_seqs, hidden, num_slots, status);
        return check_launch("shortconv", e);
    }
    dim3 grid(n, cblocks);
#define SC_LAUNCH(T, V)                                                                            \
    e = launch(shortconv_kernel<T, V>, grid, threads, 0, stream, (const T*)h3, in_bias, taps, conv_bias, \
               (T*)state, slot_stride, state_slots, tok_seq, cu_q, positions, (T*)out, n, hidden, L,      \
               num_slots, status)
    if (dtype == VAPI_F32) { if (vec) SC_LAUNCH(float, 4); else SC_LAUNCH(float, 1); }
    else if (dtype == VAPI_BF16) { if (vec) SC_LAUNCH(__nv_bfloat16, 4); else SC_LAUNCH(__nv_bfloat16, 1); }
    else return fail(-2, "shortconv: unsupported dtype %d", dtype);
#undef SC_LAUNCH
    return check_launch("shortconv", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
