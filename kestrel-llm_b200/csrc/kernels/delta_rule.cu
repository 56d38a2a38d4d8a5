// A recurrent mixer: the gated delta rule with one decay per key channel, and the short causal
// convolutions in front of it.  Per head, with a state S [d, dv] that starts at zero and is
// carried from token to token of a request (float32, in the request's state slot):
//
//     S <- diag(a_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// The read-out sees the token's own write.  Everything that enters the recurrence is float32.
//
// Kernels, in the order of a step:
//   conv_silu     y[t, c] = silu(sum_j w[c, j] x[t - (taps-1) + j, c]) per channel of the fused
//                 q|k|v product; inputs before this step's first token of a request come from the
//                 request's state slot (the last taps-1 inputs; zeros for a new request)
//   conv_tail     writes the last taps-1 inputs back to the slot
//   gates         q, k made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q scaled by d^-1/2;
//                 beta = sigmoid(.); a = exp(-exp(A_log[h]) softplus(. + dt_bias))
//   scan          the recurrence; a value column of S stays in the registers of eight lanes (an
//                 eighth of the key channels each), so S^T k and S^T q are sums inside a thread
//                 and one fixed shuffle tree - a token's result does not depend on how the
//                 request was cut into steps or on the batch
//   out_norm_gate o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) per head, in the storage type
#include "common.cuh"
#include <math.h>

#define DR_MAX_TAPS 8

// sum of a product's slices at (token, column)
__device__ __forceinline__ float slices_at(const float *p, int S, size_t slice_stride, size_t off) {
    return sum_slices(p, S, slice_stride, off);
}

__global__ void delta_conv_silu_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, const float *__restrict__ w,
                                       int taps, const float *__restrict__ state, size_t state_stride, size_t tail_off,
                                       const int *__restrict__ seq_of_token, const int *__restrict__ cu_seqlens,
                                       const int *__restrict__ slots, float *__restrict__ out, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = cu_seqlens[seq];
    const int i = t - first;
    const float *tail = state + (size_t)slots[seq] * state_stride + tail_off;     // [taps - 1][C], oldest first
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float y = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int n = i - (taps - 1) + j;          // input index among this step's tokens of the request
            const float x = n >= 0 ? slices_at(partial, S, slice_stride, (size_t)(first + n) * ld + c)
                                   : tail[(size_t)(taps - 1 + n) * C + c];
            y = fmaf(w[(size_t)c * taps + j], x, y);
        }
        out[(size_t)t * C + c] = y / (1.0f + expf(-y));
    }
}

__global__ void delta_conv_tail_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, int taps,
                                       float *__restrict__ state, size_t state_stride, size_t tail_off,
                                       const int *__restrict__ cu_seqlens, const int *__restrict__ slots, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x;
    const int first = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - first;
    float *tail = state + (size_t)slots[seq] * state_stride + tail_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float keep[DR_MAX_TAPS];
#pragma unroll
        for (int r = 0; r < DR_MAX_TAPS; ++r) {
            if (r < taps - 1) {
                const int n = n_tok - (taps - 1) + r;
                keep[r] = n >= 0 ? slices_at(partial, S, slice_stride, (size_t)(first + n) * ld + c)
                                 : tail[(size_t)(taps - 1 + n) * C + c];
            }
        }
#pragma unroll
        for (int r = 0; r < DR_MAX_TAPS; ++r)
            if (r < taps - 1) tail[(size_t)r * C + c] = keep[r];
    }
}

// act [T, C] = q (G*d) | k (G*d) | v (H*dv) after convolution and silu
__global__ void __launch_bounds__(128)
delta_gates_kernel(const float *__restrict__ act, int C, const float *__restrict__ partial, int S, size_t slice_stride, int ld, int col_beta,
                   const float *__restrict__ a_part, int Sa, size_t a_stride, const float *__restrict__ A_log,
                   const float *__restrict__ dt_bias, float *__restrict__ qn, float *__restrict__ kn, float *__restrict__ decay,
                   float *__restrict__ beta, int H, int G, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float q_scale = 1.0f / sqrtf((float)d);
    for (int r = warp; r < 2 * G; r += 4) {                // q heads, then k heads
        const float *x = act + (size_t)t * C + (size_t)r * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float mul = (1.0f / sqrtf(ss + 1e-6f)) * (r < G ? q_scale : 1.0f);
        float *dst = r < G ? qn + ((size_t)t * G + r) * d : kn + ((size_t)t * G + (r - G)) * d;
        for (int i = lane; i < d; i += 32) dst[i] = x[i] * mul;
    }
    for (int idx = threadIdx.x; idx < H * d; idx += 128) {
        const int h = idx / d;
        const float a = slices_at(a_part, Sa, a_stride, (size_t)t * H * d + idx) + dt_bias[idx];
        const float sp = a > 20.f ? a : log1pf(expf(a));
        decay[(size_t)t * H * d + idx] = expf(-expf(A_log[h]) * sp);
    }
    for (int h = threadIdx.x; h < H; h += 128) {
        const float z = slices_at(partial, S, slice_stride, (size_t)t * ld + col_beta + h);
        beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-z));
    }
}

#define DR_TC 8        // tokens staged in shared memory at a time
#define DR_LPC 8       // lanes that share a value column's key channels
#define DR_COLS (128 / DR_LPC)      // value columns of a CTA of four warps

__device__ __forceinline__ void dr_cp_async(float *dst, const float *src, bool vec4) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    if (vec4) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// A CTA of four warps takes DR_COLS value columns of one (request, head); the DR_LPC lanes of a
// column hold interleaved parts of its D (padded) key channels: lane part s owns channels
// 4 (DR_LPC m + s) + {0..3}.  Per token a thread does D / DR_LPC decays and multiply-adds twice
// (S^T k, then the write and S^T q) on four partial sums each, and the lanes of a column add their
// parts in a fixed shuffle tree.  The time of a token is the latency of this chain, so the parts
// are short: with four lanes a column a token took 0.41 us, with eight it takes less.  k, q, the decays, v and beta of DR_TC tokens are staged in
// shared memory with cp.async, the next stage in flight while the current one is used.
template <int D>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float *__restrict__ qn, const float *__restrict__ kn, const float *__restrict__ decay,
                  const float *__restrict__ act, int C, int col_v, const float *__restrict__ beta, float *__restrict__ state,
                  size_t state_stride, const int *__restrict__ cu_seqlens, const int *__restrict__ slots,
                  float *__restrict__ out, int H, int G, int d, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int STAGE = DR_TC * (3 * D + 32) + DR_TC;      // floats: k, q, a [TC][D]; v [TC][32, DR_COLS used]; beta [TC]
    constexpr int M = D / (4 * DR_LPC);                      // float4s of a thread's part
    extern __shared__ float4 dr_smem4[];
    float *sm = reinterpret_cast<float *>(dr_smem4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = lane % DR_LPC, cj = lane / DR_LPC;
    const int jl = warp * (32 / DR_LPC) + cj, j = blockIdx.x * DR_COLS + jl, h = blockIdx.y, seq = blockIdx.z;
    const int g = h / (H / G);
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    const bool live = j < dv;
    const bool vec4 = d % 4 == 0;
    float *Sg = state + (size_t)slots[seq] * state_stride + (size_t)h * d * dv;     // [d][dv]
    float Sc[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int i = 4 * (DR_LPC * m + part) + c;
            Sc[m][c] = (i < d && live) ? Sg[(size_t)i * dv + j] : 0.f;
        }
    for (int idx = tid; idx < 2 * STAGE; idx += 128) sm[idx] = 0.f;       // the padded channels stay zero
    __syncthreads();

    auto issue = [&](int tb, int stage) {
        float *sk = sm + (size_t)stage * STAGE, *sq = sk + DR_TC * D, *sa = sq + DR_TC * D, *sv = sa + DR_TC * D, *sb = sv + DR_TC * 32;
        const int per = vec4 ? d / 4 : d, w = vec4 ? 4 : 1;
        for (int idx = tid; idx < DR_TC * per; idx += 128) {
            const int c = idx / per, e = (idx % per) * w, t = tb + c;
            if (t < t1) {
                dr_cp_async(sk + c * D + e, kn + ((size_t)t * G + g) * d + e, vec4);
                dr_cp_async(sq + c * D + e, qn + ((size_t)t * G + g) * d + e, vec4);
                dr_cp_async(sa + c * D + e, decay + ((size_t)t * H + h) * d + e, vec4);
            }
        }
        for (int idx = tid; idx < DR_TC * 32; idx += 128) {
            const int c = idx / 32, jj = idx % 32, t = tb + c, col = blockIdx.x * DR_COLS + jj;
            if (t < t1 && jj < DR_COLS && col < dv) dr_cp_async(sv + c * 32 + jj, act + (size_t)t * C + col_v + (size_t)h * dv + col, false);
        }
        if (tid < DR_TC && tb + tid < t1) dr_cp_async(sb + tid, beta + (size_t)(tb + tid) * H + h, false);
    };
    if (t0 < t1) issue(t0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int stage = 0;
    for (int tb = t0; tb < t1; tb += DR_TC, stage ^= 1) {
        if (tb + DR_TC < t1) issue(tb + DR_TC, stage ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const float *sk = sm + (size_t)stage * STAGE, *sq = sk + DR_TC * D, *sa = sq + DR_TC * D, *sv = sa + DR_TC * D, *sb = sv + DR_TC * 32;
        const int n = min(DR_TC, t1 - tb);
#pragma unroll
        for (int c = 0; c < DR_TC; ++c) {             // unrolled: the next token's operands are fetched under this token's chain
            if (c >= n) break;
            const float4 *k4 = reinterpret_cast<const float4 *>(sk + c * D), *q4 = reinterpret_cast<const float4 *>(sq + c * D),
                         *a4 = reinterpret_cast<const float4 *>(sa + c * D);
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float4 kk = k4[DR_LPC * m + part], aa = a4[DR_LPC * m + part];
                Sc[m][0] *= aa.x; s0 = fmaf(Sc[m][0], kk.x, s0);
                Sc[m][1] *= aa.y; s1 = fmaf(Sc[m][1], kk.y, s1);
                Sc[m][2] *= aa.z; s2 = fmaf(Sc[m][2], kk.z, s2);
                Sc[m][3] *= aa.w; s3 = fmaf(Sc[m][3], kk.w, s3);
            }
            float acc = (s0 + s1) + (s2 + s3);
#pragma unroll
            for (int sh = 1; sh < DR_LPC; sh <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
            const float u = sb[c] * (sv[c * 32 + jl] - acc);
            s0 = s1 = s2 = s3 = 0.f;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float4 kk = k4[DR_LPC * m + part], qq = q4[DR_LPC * m + part];
                Sc[m][0] = fmaf(kk.x, u, Sc[m][0]); s0 = fmaf(Sc[m][0], qq.x, s0);
                Sc[m][1] = fmaf(kk.y, u, Sc[m][1]); s1 = fmaf(Sc[m][1], qq.y, s1);
                Sc[m][2] = fmaf(kk.z, u, Sc[m][2]); s2 = fmaf(Sc[m][2], qq.z, s2);
                Sc[m][3] = fmaf(kk.w, u, Sc[m][3]); s3 = fmaf(Sc[m][3], qq.w, s3);
            }
            float o = (s0 + s1) + (s2 + s3);
#pragma unroll
            for (int sh = 1; sh < DR_LPC; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
            if (live && part == 0) out[((size_t)(tb + c) * H + h) * dv + j] = o;
        }
        __syncthreads();                              // the stage may be filled again
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (live) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = 4 * (DR_LPC * m + part) + c;
                if (i < d) Sg[(size_t)i * dv + j] = Sc[m][c];
            }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
delta_out_kernel(const float *__restrict__ o, const float *__restrict__ w, float eps, const float *__restrict__ g_part, int Sg,
                 size_t g_stride, T *__restrict__ out, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < H; h += 4) {
        const size_t base = ((size_t)t * H + h) * dv;
        float ss = 0.f;
        for (int i = lane; i < dv; i += 32) ss = fmaf(o[base + i], o[base + i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int i = lane; i < dv; i += 32) {
            const float z = slices_at(g_part, Sg, g_stride, base + i);
            out[base + i] = from_f32<T>(o[base + i] * r * w[i] * (1.0f / (1.0f + expf(-z))));
        }
    }
}

KESTREL_API int kestrel_delta_conv_silu(const float *partial, int S, long long slice_stride, int ld, const float *w, int taps, float *state,
                                        long long state_stride, long long tail_off, const int *seq_of_token, const int *cu_seqlens,
                                        const int *slots, float *out, int T, int nseq, int C, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && nseq > 0 && C > 0 && S > 0 && taps >= 1 && taps <= DR_MAX_TAPS + 1, "delta_conv_silu: bad sizes (taps %d)", taps);
    kestrel_launch(delta_conv_silu_kernel, dim3(T), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, w, taps, (const float *)state,
                   (size_t)state_stride, (size_t)tail_off, seq_of_token, cu_seqlens, slots, out, C);
    int rc = kestrel_check_launch("delta_conv_silu");
    if (rc != 0 || taps == 1) return rc;
    kestrel_launch(delta_conv_tail_kernel, dim3(nseq, (C + 255) / 256), dim3(256), 0, stream, partial, S, (size_t)slice_stride, ld, taps, state,
                   (size_t)state_stride, (size_t)tail_off, cu_seqlens, slots, C);
    return kestrel_check_launch("delta_conv_tail");
}

KESTREL_API int kestrel_delta_gates(const float *act, int C, const float *partial, int S, long long slice_stride, int ld, int col_beta,
                                    const float *a_part, int Sa, long long a_stride, const float *A_log, const float *dt_bias, float *qn,
                                    float *kn, float *decay, float *beta, int T, int H, int G, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && d > 0, "delta_gates: bad sizes");
    kestrel_launch(delta_gates_kernel, dim3(T), dim3(128), 0, stream, act, C, partial, S, (size_t)slice_stride, ld, col_beta, a_part, Sa,
                   (size_t)a_stride, A_log, dt_bias, qn, kn, decay, beta, H, G, d);
    return kestrel_check_launch("delta_gates");
}

KESTREL_API int kestrel_delta_scan(const float *qn, const float *kn, const float *decay, const float *act, int C, int col_v, const float *beta,
                                   float *state, long long state_stride, const int *cu_seqlens, const int *slots, float *out, int nseq,
                                   int H, int G, int d, int dv, cudaStream_t stream) {
    if (nseq == 0) return 0;
    KESTREL_REQUIRE(nseq > 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "delta_scan: bad sizes");
    KESTREL_REQUIRE(d <= 256, "delta_scan: key size %d exceeds 256", d);
    KESTREL_REQUIRE(H <= 65535 && nseq <= 65535, "delta_scan: grid too large");
    dim3 grid((dv + DR_COLS - 1) / DR_COLS, H, nseq);
#define DR_LAUNCH(D)                                                                                                                  \
    {                                                                                                                                 \
        static bool attr_set = false;                                                                                                 \
        if (!attr_set && cudaFuncSetAttribute(delta_scan_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,                      \
                                              KESTREL_SMEM_MAX_DYNAMIC) != cudaSuccess)                                               \
            return kestrel_fail(-3, "delta_scan: cannot set the shared memory size");                                                 \
        attr_set = true;                                                                                                              \
    }                                                                                                                                 \
    kestrel_launch(delta_scan_kernel<D>, grid, dim3(128),                                                                             \
                   kestrel_spread_smem((long)grid.x * grid.y * grid.z, (size_t)2 * (DR_TC * (3 * D + 32) + DR_TC) * sizeof(float)),   \
                   stream, qn, kn, decay, act, C, col_v, beta, state, (size_t)state_stride, cu_seqlens, slots, out, H, G, d, dv)
    if (d <= 32) { DR_LAUNCH(32); }
    else if (d <= 64) { DR_LAUNCH(64); }
    else if (d <= 128) { DR_LAUNCH(128); }
    else { DR_LAUNCH(256); }
#undef DR_LAUNCH
    return kestrel_check_launch("delta_scan");
}

KESTREL_API int kestrel_delta_out(const float *o, const float *w, float eps, const float *g_part, int Sg, long long g_stride, void *out,
                                  int dtype, int T, int H, int dv, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && dv > 0 && Sg > 0, "delta_out: bad sizes");
    if (dtype == KESTREL_F32)
        kestrel_launch(delta_out_kernel<float>, dim3(T), dim3(128), 0, stream, o, w, eps, g_part, Sg, (size_t)g_stride, (float *)out, H, dv);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(delta_out_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, o, w, eps, g_part, Sg, (size_t)g_stride, (__nv_bfloat16 *)out, H, dv);
    else
        return kestrel_fail(-2, "delta_out: unknown dtype %d", dtype);
    return kestrel_check_launch("delta_out");
}
