// A recurrent mixer with a real-gated linear recurrent unit: a diagonal recurrence per channel whose
// decay and input gate are made from the recurrence's own input by block-diagonal products.
//
// The mixer projects its input to two branches of `C` channels in ONE fused product with columns
// [ y | x ] (plus the product's bias):
//
//     y = gelu_tanh(.)                                              the gate branch
//     u = conv(.)                                                   a short causal convolution per channel over time, with bias
//     r = sigmoid(Wa_b u_b + ba),  i = sigmoid(Wi_b u_b + bi)       per block b of channels (the products are head-wise products)
//     a = exp(-c * r * softplus(lam)),   S <- a S + sqrt(1 - a^2) (i u)   per channel; S starts at zero, also for the first token
//     out = S * y                                                   in the storage type, for the output projection
//
// The state slot of a request is [S: C | the convolution's last taps - 1 inputs: (taps - 1) C], float32.
//
// Kernels, in the order of a step:
//   branches   y and u of every token as float32, u also in the storage type (the operand of the gates' products);
//              inputs before this step's first token of a request come from the slot's tail (zeros for a new request)
//   tail       writes the last taps - 1 inputs back to the slot
//   scan       gates, decay and the recurrence, a thread a (request, channel), sequential over the request's tokens
//              of this step with the loads of eight tokens in flight; 1 - a^2 is taken as -expm1(2 ln a), which keeps
//              its digits where a is close to 1.  A token's result depends on the tokens before it alone: the same bits
//              however the request is cut into steps and whatever else is in the batch.
//   scan in chunks (steps that bring a request many tokens): the recurrence is linear in S, so a stretch of tokens acts
//              on the state as S -> A S + s.  A first kernel makes (A, s) of every chunk of `chunk` tokens, a thread a
//              (request, chunk, channel), the first chunk starting from the slot's state; a second kernel folds the
//              chunks before its own in ascending order, then runs its own chunk from there and writes the outputs (the last
//              chunk also the new state).  2 x T x C thread-steps instead of T sequential ones; the sums are grouped by
//              chunk, so the result differs from the sequential kernel's by rounding.
#include "common.cuh"
#include <math.h>

#define RG_MAX_TAPS 9
#define RG_CHUNK 8

__device__ __forceinline__ float rg_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float rg_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(256)
rglru_branches_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, const float *__restrict__ bias,
                      const float *__restrict__ conv_w, const float *__restrict__ conv_b, int taps, const float *__restrict__ state,
                      size_t state_stride, size_t tail_off, const int *__restrict__ seq_of_token, const int *__restrict__ cu_seqlens,
                      const int *__restrict__ slots, float *__restrict__ y_out, float *__restrict__ u_out, T *__restrict__ u_st, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = cu_seqlens[seq];
    const int i = t - first;
    const float *tail = state + (size_t)slots[seq] * state_stride + tail_off;     // [taps - 1][C], oldest first
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float yb = bias ? bias[c] : 0.f, xb = bias ? bias[C + c] : 0.f;
        y_out[(size_t)t * C + c] = rg_gelu_tanh(sum_slices(partial, S, slice_stride, (size_t)t * ld + c) + yb);
        float u = conv_b ? conv_b[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int n = i - (taps - 1) + j;          // input index among this step's tokens of the request
            const float x = n >= 0 ? sum_slices(partial, S, slice_stride, (size_t)(first + n) * ld + C + c) + xb
                                   : tail[(size_t)(taps - 1 + n) * C + c];
            u = fmaf(conv_w[(size_t)c * taps + j], x, u);
        }
        u_out[(size_t)t * C + c] = u;
        u_st[(size_t)t * C + c] = from_f32<T>(u);
    }
}

__global__ void __launch_bounds__(256)
rglru_tail_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, const float *__restrict__ bias, int taps,
                  float *__restrict__ state, size_t state_stride, size_t tail_off, const int *__restrict__ cu_seqlens,
                  const int *__restrict__ slots, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x;
    const int first = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - first;
    if (n_tok <= 0) return;
    float *tail = state + (size_t)slots[seq] * state_stride + tail_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float xb = bias ? bias[C + c] : 0.f;
        float keep[RG_MAX_TAPS - 1];
#pragma unroll
        for (int r = 0; r < RG_MAX_TAPS - 1; ++r) {
            if (r < taps - 1) {
                const int n = n_tok - (taps - 1) + r;
                keep[r] = n >= 0 ? sum_slices(partial, S, slice_stride, (size_t)(first + n) * ld + C + c) + xb
                                 : tail[(size_t)(taps - 1 + n) * C + c];
            }
        }
#pragma unroll
        for (int r = 0; r < RG_MAX_TAPS - 1; ++r)
            if (r < taps - 1) tail[(size_t)r * C + c] = keep[r];
    }
}

// y, u: float32 [T, C]; gr, gi: the gates' products, float32 [T, C]; out in the storage type
template <typename T>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const float *__restrict__ y, const float *__restrict__ u, const float *__restrict__ gr, const float *__restrict__ gi,
                  const float *__restrict__ r_bias, const float *__restrict__ i_bias, const float *__restrict__ lam, float rate,
                  float *__restrict__ state, size_t state_stride, const int *__restrict__ cu_seqlens, const int *__restrict__ slots,
                  T *__restrict__ out, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - first;
    if (n_tok <= 0) return;
    float *sp_ = state + (size_t)slots[seq] * state_stride + c;
    float s = *sp_;
    const float l = lam[c];
    const float neg = -rate * (l > 20.f ? l : log1pf(expf(l)));         // -rate * softplus(lam)
    const float rb = r_bias ? r_bias[c] : 0.f, ib = i_bias ? i_bias[c] : 0.f;
    for (int t0 = 0; t0 < n_tok; t0 += RG_CHUNK) {
        float a[RG_CHUNK], b[RG_CHUNK], yy[RG_CHUNK];
#pragma unroll
        for (int k = 0; k < RG_CHUNK; ++k) {
            const bool ok = t0 + k < n_tok;
            const size_t at = (size_t)(first + min(t0 + k, n_tok - 1)) * C + c;
            const float zr = gr[at] + rb, zi = gi[at] + ib, uu = u[at];
            yy[k] = y[at];
            const float log_a = neg * rg_sigmoid(zr);
            a[k] = ok ? expf(log_a) : 1.f;
            b[k] = ok ? sqrtf(-expm1f(2.0f * log_a)) * (rg_sigmoid(zi) * uu) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < RG_CHUNK; ++k) {
            s = fmaf(a[k], s, b[k]);
            if (t0 + k < n_tok) out[(size_t)(first + t0 + k) * C + c] = from_f32<T>(s * yy[k]);
        }
    }
    *sp_ = s;
}

// one token's decay and drive
__device__ __forceinline__ void rg_token(float zr, float zi, float uu, float neg, float &a, float &b) {
    const float log_a = neg * rg_sigmoid(zr);
    a = expf(log_a);
    b = sqrtf(-expm1f(2.0f * log_a)) * (rg_sigmoid(zi) * uu);
}

// sums [nseq, chunks, 2, C]: a chunk's action on the state, S -> A S + s (the first chunk's s starts from the slot's state)
__global__ void __launch_bounds__(128)
rglru_chunk_sums_kernel(const float *__restrict__ u, const float *__restrict__ gr, const float *__restrict__ gi, const float *__restrict__ r_bias,
                        const float *__restrict__ i_bias, const float *__restrict__ lam, float rate, const float *__restrict__ state,
                        size_t state_stride, const int *__restrict__ cu_seqlens, const int *__restrict__ slots, float *__restrict__ sums,
                        int chunk, int chunks, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, k = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - first;
    const int t0 = k * chunk, t1 = min(t0 + chunk, n_tok);
    if (t0 >= n_tok) return;
    const float l = lam[c];
    const float neg = -rate * (l > 20.f ? l : log1pf(expf(l)));
    const float rb = r_bias ? r_bias[c] : 0.f, ib = i_bias ? i_bias[c] : 0.f;
    float A = 1.f, s = k == 0 ? state[(size_t)slots[seq] * state_stride + c] : 0.f;
    for (int t = t0; t < t1; t += RG_CHUNK) {
        float a[RG_CHUNK], b[RG_CHUNK];
#pragma unroll
        for (int j = 0; j < RG_CHUNK; ++j) {
            const size_t at = (size_t)(first + min(t + j, t1 - 1)) * C + c;
            rg_token(gr[at] + rb, gi[at] + ib, u[at], neg, a[j], b[j]);
            if (t + j >= t1) { a[j] = 1.f; b[j] = 0.f; }
        }
#pragma unroll
        for (int j = 0; j < RG_CHUNK; ++j) {
            s = fmaf(a[j], s, b[j]);
            A *= a[j];
        }
    }
    float *o = sums + ((size_t)seq * chunks + k) * 2 * C;
    o[c] = k == 0 ? state[(size_t)slots[seq] * state_stride + c] : A;      // the first chunk's A is never used (it acts on nothing): the state it started from
    o[C + c] = s;
}

template <typename T>
__global__ void __launch_bounds__(128)
rglru_chunk_apply_kernel(const float *__restrict__ y, const float *__restrict__ u, const float *__restrict__ gr, const float *__restrict__ gi,
                         const float *__restrict__ r_bias, const float *__restrict__ i_bias, const float *__restrict__ lam, float rate,
                         float *__restrict__ state, size_t state_stride, const int *__restrict__ cu_seqlens, const int *__restrict__ slots,
                         const float *__restrict__ sums, T *__restrict__ out, int chunk, int chunks, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, k = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - first;
    const int t0 = k * chunk, t1 = min(t0 + chunk, n_tok);
    if (t0 >= n_tok) return;
    const float l = lam[c];
    const float neg = -rate * (l > 20.f ? l : log1pf(expf(l)));
    const float rb = r_bias ? r_bias[c] : 0.f, ib = i_bias ? i_bias[c] : 0.f;
    // The state at this chunk's start.  Chunk 0's s carries the slot's state and its A slot holds that state itself: the slot is
    // not read here, since the last chunk's thread writes it.
    const float *p = sums + (size_t)seq * chunks * 2 * C + c;
    float s = k == 0 ? p[0] : p[C];
    for (int j = 1; j < k; ++j) s = fmaf(p[(size_t)j * 2 * C], s, p[(size_t)j * 2 * C + C]);
    for (int t = t0; t < t1; t += RG_CHUNK) {
        float a[RG_CHUNK], b[RG_CHUNK], yy[RG_CHUNK];
#pragma unroll
        for (int j = 0; j < RG_CHUNK; ++j) {
            const size_t at = (size_t)(first + min(t + j, t1 - 1)) * C + c;
            rg_token(gr[at] + rb, gi[at] + ib, u[at], neg, a[j], b[j]);
            yy[j] = y[at];
        }
#pragma unroll
        for (int j = 0; j < RG_CHUNK; ++j) {
            if (t + j < t1) {
                s = fmaf(a[j], s, b[j]);
                out[(size_t)(first + t + j) * C + c] = from_f32<T>(s * yy[j]);
            }
        }
    }
    if (t1 == n_tok) state[(size_t)slots[seq] * state_stride + c] = s;
}

// The scan in chunks of `chunk` tokens (a multiple of 8), for steps in which a request brings many tokens; max_count: the most tokens
// of one request in this step; scratch: float32 [nseq * ceil(max_count / chunk) * 2 * C]
KESTREL_API int kestrel_rglru_scan_chunked(const float *y, const float *u, const float *gr, const float *gi, const float *r_bias, const float *i_bias,
                                           const float *lam, float rate, float *state, long long state_stride, const int *cu_seqlens,
                                           const int *slots, void *out, int dtype, int nseq, int max_count, int chunk, float *scratch, int C,
                                           cudaStream_t stream) {
    if (nseq == 0 || max_count == 0) return 0;
    KESTREL_REQUIRE(nseq > 0 && nseq <= 65535 && C > 0 && rate > 0.f && chunk >= 8 && chunk % 8 == 0 && max_count > 0 && scratch, "rglru_scan_chunked: bad sizes");
    const int chunks = (max_count + chunk - 1) / chunk;
    KESTREL_REQUIRE(chunks <= 65535, "rglru_scan_chunked: %d chunks exceed the grid", chunks);
    dim3 grid((C + 127) / 128, chunks, nseq);
    kestrel_launch(rglru_chunk_sums_kernel, grid, dim3(128), 0, stream, u, gr, gi, r_bias, i_bias, lam, rate, (const float *)state, (size_t)state_stride,
                   cu_seqlens, slots, scratch, chunk, chunks, C);
    int rc = kestrel_check_launch("rglru_chunk_sums");
    if (rc != 0) return rc;
    if (dtype == KESTREL_F32)
        kestrel_launch(rglru_chunk_apply_kernel<float>, grid, dim3(128), 0, stream, y, u, gr, gi, r_bias, i_bias, lam, rate, state, (size_t)state_stride,
                       cu_seqlens, slots, (const float *)scratch, (float *)out, chunk, chunks, C);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(rglru_chunk_apply_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, y, u, gr, gi, r_bias, i_bias, lam, rate, state, (size_t)state_stride,
                       cu_seqlens, slots, (const float *)scratch, (__nv_bfloat16 *)out, chunk, chunks, C);
    else
        return kestrel_fail(-2, "rglru_scan_chunked: unknown dtype %d", dtype);
    return kestrel_check_launch("rglru_chunk_apply");
}

// partial: the fused product [y | x] as float32 slices, bias [2 C] or NULL; conv_w [C, taps] (last column the current token's),
// conv_b [C] or NULL; state: the requests' slots, the tail [taps - 1, C] at tail_off; y_out, u_out float32 [T, C]; u_st [T, C] in the storage type
KESTREL_API int kestrel_rglru_branches(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *conv_w,
                                       const float *conv_b, int taps, float *state, long long state_stride, long long tail_off,
                                       const int *seq_of_token, const int *cu_seqlens, const int *slots, float *y_out, float *u_out, void *u_st,
                                       int dtype, int T, int nseq, int C, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && nseq > 0 && C > 0 && S > 0 && ld >= 2 * C && taps >= 1 && taps <= RG_MAX_TAPS, "rglru_branches: bad sizes (taps %d)", taps);
    const int by = T >= 256 ? 1 : min((C + 255) / 256, 32);
    if (dtype == KESTREL_F32)
        kestrel_launch(rglru_branches_kernel<float>, dim3(T, by), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, bias, conv_w, conv_b, taps,
                       (const float *)state, (size_t)state_stride, (size_t)tail_off, seq_of_token, cu_seqlens, slots, y_out, u_out, (float *)u_st, C);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(rglru_branches_kernel<__nv_bfloat16>, dim3(T, by), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, bias, conv_w, conv_b, taps,
                       (const float *)state, (size_t)state_stride, (size_t)tail_off, seq_of_token, cu_seqlens, slots, y_out, u_out, (__nv_bfloat16 *)u_st, C);
    else
        return kestrel_fail(-2, "rglru_branches: unknown dtype %d", dtype);
    int rc = kestrel_check_launch("rglru_branches");
    if (rc != 0 || taps == 1) return rc;
    kestrel_launch(rglru_tail_kernel, dim3(nseq, min((C + 255) / 256, 64)), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, bias, taps, state,
                   (size_t)state_stride, (size_t)tail_off, cu_seqlens, slots, C);
    return kestrel_check_launch("rglru_tail");
}

// gr, gi: float32 [T, C] products of the gates, r_bias / i_bias [C] or NULL; lam [C]; rate: the c of a = exp(-c r softplus(lam));
// state: S [C] at the start of every slot; out [T, C] in the storage type
KESTREL_API int kestrel_rglru_scan(const float *y, const float *u, const float *gr, const float *gi, const float *r_bias, const float *i_bias,
                                   const float *lam, float rate, float *state, long long state_stride, const int *cu_seqlens, const int *slots,
                                   void *out, int dtype, int nseq, int C, cudaStream_t stream) {
    if (nseq == 0) return 0;
    KESTREL_REQUIRE(nseq > 0 && nseq <= 65535 && C > 0 && rate > 0.f, "rglru_scan: bad sizes");
    dim3 grid((C + 127) / 128, nseq);
    if (dtype == KESTREL_F32)
        kestrel_launch(rglru_scan_kernel<float>, grid, dim3(128), 0, stream, y, u, gr, gi, r_bias, i_bias, lam, rate, state, (size_t)state_stride, cu_seqlens, slots,
                       (float *)out, C);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(rglru_scan_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, y, u, gr, gi, r_bias, i_bias, lam, rate, state, (size_t)state_stride, cu_seqlens,
                       slots, (__nv_bfloat16 *)out, C);
    else
        return kestrel_fail(-2, "rglru_scan: unknown dtype %d", dtype);
    return kestrel_check_launch("rglru_scan");
}
