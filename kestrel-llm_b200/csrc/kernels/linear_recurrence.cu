// Linear recurrences with a matrix of state per head: S [d, dv], float32, in the request's state
// slot, from zero at admission, carried from token to token.  One scan serves the mixers whose
// step is a diagonal decay, optionally a rank-one correction that reads the OLD state, and a
// rank-one write:
//
//     S_t = diag(w_t) S_{t-1} + a_t (b_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T r_t
//
// w, a, b, k, r are vectors over the d key channels of a head, v over its dv value channels.
//   * a gated linear recurrence whose forget gate also sets what is written (HGRN2 style):
//       w = f, k = 1 - f, no correction, r = silu(query);  f = lower + (1 - lower) sigmoid(z)
//   * a generalised delta rule: with u the unit key k / sqrt(sum k^2 + 1e-6),
//       a = -(rate * u), b = u: what the state holds along u is taken out at `rate` per channel
//       before the write; w = exp(-c sigmoid(z)) with c a constant of the design.
// Everything that enters the scan is float32 and is made by the `gates` kernels from the
// float32 slices of the mixer's input product.
//
// The scan is the kernel of delta_rule.cu in another order of operations: a CTA of four warps
// takes 16 value columns of one (request, head); the eight lanes of a column hold interleaved
// parts of its key channels; per token a thread makes its part of b^T S, the lanes add in a
// fixed shuffle tree, then each channel is updated and read out.  The order of every sum is
// fixed, so a token's result does not depend on how the request was cut into steps or batched.
#include "common.cuh"
#include <math.h>

#define LR_TC 8        // tokens staged in shared memory at a time
#define LR_LPC 8       // lanes that share a value column's key channels
#define LR_COLS (128 / LR_LPC)

__device__ __forceinline__ float lr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---- gates of the forget-gate recurrence -------------------------------------------------------
// product columns: q at col_q, f at col_f (n = H d each), v at col_v (nv = H dv)
__global__ void __launch_bounds__(1024)
forget_gates_kernel(const float *__restrict__ p, int S, size_t slice_stride, int ld, int col_q, int col_f, int col_v,
                    const float *__restrict__ f_bias, const float *__restrict__ lower, float *__restrict__ r_out,
                    float *__restrict__ w_out, float *__restrict__ k_out, float *__restrict__ v_out, int n, int nv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const size_t row = (size_t)t * ld;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float q = sum_slices(p, S, slice_stride, row + col_q + i);
        const float z = sum_slices(p, S, slice_stride, row + col_f + i) + (f_bias ? f_bias[i] : 0.f);
        const float lo = lower ? lower[i] : 0.f;
        const float f = lo + (1.0f - lo) * lr_sigmoid(z);
        r_out[(size_t)t * n + i] = q * lr_sigmoid(q);
        w_out[(size_t)t * n + i] = f;
        k_out[(size_t)t * n + i] = 1.0f - f;
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) v_out[(size_t)t * nv + i] = sum_slices(p, S, slice_stride, row + col_v + i);
}

// ---- gates of the generalised delta rule -------------------------------------------------------
// product columns: r, k, v, rate logits at col_r, col_k, col_v, col_a (H d each); the decay's logits are a second
// product `wz` [T, H d]; a warp a head, J = ceil(d / 32) channels a lane
template <int J>
__global__ void __launch_bounds__(128)
removal_gates_kernel(const float *__restrict__ p, int S, size_t slice_stride, int ld, int col_r, int col_k, int col_v, int col_a,
                     const float *__restrict__ a_bias, const float *__restrict__ wz, int Sw, size_t w_stride,
                     const float *__restrict__ w_bias, float decay_rate, float *__restrict__ r_out, float *__restrict__ k_out,
                     float *__restrict__ v_out, float *__restrict__ w_out, float *__restrict__ a_out, float *__restrict__ b_out,
                     int H, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = (size_t)t * ld, n = (size_t)H * d;
    for (int h = blockIdx.y * 4 + warp; h < H; h += gridDim.y * 4) {
        // Slice by slice, all of a lane's loads of a slice in flight at once: a step of few tokens is bound by their
        // latency.  Every element's sum runs over the slices in ascending order from 0, as sum_slices does: same bits.
        float k[J], ar[J], z[J], r[J], v[J];
        int cc[J];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int i = lane + 32 * j;
            cc[j] = h * d + (i < d ? i : d - 1);              // lanes past the head's end load its last channel and drop it
            k[j] = ar[j] = z[j] = r[j] = v[j] = 0.f;
        }
        for (int s = 0; s < S; ++s) {
            const float *ps = p + (size_t)s * slice_stride + row;
#pragma unroll
            for (int j = 0; j < J; ++j) {
                k[j] += ps[col_k + cc[j]];
                ar[j] += ps[col_a + cc[j]];
                r[j] += ps[col_r + cc[j]];
                v[j] += ps[col_v + cc[j]];
            }
        }
        for (int s = 0; s < Sw; ++s) {
            const float *ps = wz + (size_t)s * w_stride + (size_t)t * n;
#pragma unroll
            for (int j = 0; j < J; ++j) z[j] += ps[cc[j]];
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < J; ++j)
            if (lane + 32 * j < d) ss = fmaf(k[j], k[j], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int i = lane + 32 * j, c = h * d + i;
            if (i >= d) continue;
            const size_t o = (size_t)t * n + c;
            const float u = k[j] * inv;
            const float rate = lr_sigmoid(ar[j] + (a_bias ? a_bias[c] : 0.f));
            r_out[o] = r[j];
            k_out[o] = k[j];
            v_out[o] = v[j];
            w_out[o] = expf(-decay_rate * lr_sigmoid(z[j] + (w_bias ? w_bias[c] : 0.f)));
            a_out[o] = -(rate * u);
            b_out[o] = u;
        }
    }
}

// the same gates for a step of many tokens: blocks enough to hide the loads, an element at a time (same sums, same bits)
__global__ void __launch_bounds__(128)
removal_gates_stream_kernel(const float *__restrict__ p, int S, size_t slice_stride, int ld, int col_r, int col_k, int col_v, int col_a,
                     const float *__restrict__ a_bias, const float *__restrict__ wz, int Sw, size_t w_stride,
                     const float *__restrict__ w_bias, float decay_rate, float *__restrict__ r_out, float *__restrict__ k_out,
                     float *__restrict__ v_out, float *__restrict__ w_out, float *__restrict__ a_out, float *__restrict__ b_out,
                     int H, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = (size_t)t * ld, n = (size_t)H * d;
    for (int h = blockIdx.y * 4 + warp; h < H; h += gridDim.y * 4) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float k = sum_slices(p, S, slice_stride, row + col_k + h * d + i);
            ss = fmaf(k, k, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + 1e-6f);
        for (int i = lane; i < d; i += 32) {
            const int c = h * d + i;
            const size_t o = (size_t)t * n + c;
            const float k = sum_slices(p, S, slice_stride, row + col_k + c);
            const float u = k * inv;
            const float rate = lr_sigmoid(sum_slices(p, S, slice_stride, row + col_a + c) + (a_bias ? a_bias[c] : 0.f));
            const float z = sum_slices(wz, Sw, w_stride, o) + (w_bias ? w_bias[c] : 0.f);
            r_out[o] = sum_slices(p, S, slice_stride, row + col_r + c);
            k_out[o] = k;
            v_out[o] = sum_slices(p, S, slice_stride, row + col_v + c);
            w_out[o] = expf(-decay_rate * lr_sigmoid(z));
            a_out[o] = -(rate * u);
            b_out[o] = u;
        }
    }
}

__device__ __forceinline__ void lr_cp_async(float *dst, const float *src, bool vec4) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    if (vec4) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// D: key channels padded to 32, 64, 128 or 256; RANK1: the correction a (b^T S) is present
template <int D, bool RANK1>
__global__ void __launch_bounds__(128)
recurrence_scan_kernel(const float *__restrict__ r, const float *__restrict__ w, const float *__restrict__ k, const float *__restrict__ v,
                       const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ state, size_t state_stride,
                       size_t state_off, const int *__restrict__ cu_seqlens, const int *__restrict__ slots, float *__restrict__ out,
                       int H, int d, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int NV = RANK1 ? 5 : 3;                        // vectors over key channels per token: k, r, w (, a, b)
    constexpr int STAGE = LR_TC * (NV * D + 32);             // floats; v [TC][32, LR_COLS used]
    constexpr int M = D / (4 * LR_LPC);                      // float4s of a thread's part
    extern __shared__ float4 lr_smem4[];
    float *sm = reinterpret_cast<float *>(lr_smem4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = lane % LR_LPC, cj = lane / LR_LPC;
    const int jl = warp * (32 / LR_LPC) + cj, j = blockIdx.x * LR_COLS + jl, h = blockIdx.y, seq = blockIdx.z;
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    const bool live = j < dv;
    const bool vec4 = d % 4 == 0;
    float *Sg = state + (size_t)slots[seq] * state_stride + state_off + (size_t)h * d * dv;     // [d][dv]
    float Sc[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int i = 4 * (LR_LPC * m + part) + c;
            Sc[m][c] = (i < d && live) ? Sg[(size_t)i * dv + j] : 0.f;
        }
    for (int idx = tid; idx < 2 * STAGE; idx += 128) sm[idx] = 0.f;       // the padded channels stay zero
    __syncthreads();

    auto issue = [&](int tb, int stage) {
        float *sk = sm + (size_t)stage * STAGE, *sr = sk + LR_TC * D, *sw = sr + LR_TC * D;
        float *sa = sw + LR_TC * D, *sb = sa + (RANK1 ? LR_TC * D : 0), *sv = sb + (RANK1 ? LR_TC * D : 0);
        const int per = vec4 ? d / 4 : d, wd = vec4 ? 4 : 1;
        for (int idx = tid; idx < LR_TC * per; idx += 128) {
            const int c = idx / per, e = (idx % per) * wd, t = tb + c;
            if (t < t1) {
                const size_t o = ((size_t)t * H + h) * d + e;
                lr_cp_async(sk + c * D + e, k + o, vec4);
                lr_cp_async(sr + c * D + e, r + o, vec4);
                lr_cp_async(sw + c * D + e, w + o, vec4);
                if (RANK1) {
                    lr_cp_async(sa + c * D + e, a + o, vec4);
                    lr_cp_async(sb + c * D + e, b + o, vec4);
                }
            }
        }
        for (int idx = tid; idx < LR_TC * 32; idx += 128) {
            const int c = idx / 32, jj = idx % 32, t = tb + c, col = blockIdx.x * LR_COLS + jj;
            if (t < t1 && jj < LR_COLS && col < dv) lr_cp_async(sv + c * 32 + jj, v + ((size_t)t * H + h) * dv + col, false);
        }
    };
    if (t0 < t1) issue(t0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int stage = 0;
    for (int tb = t0; tb < t1; tb += LR_TC, stage ^= 1) {
        if (tb + LR_TC < t1) issue(tb + LR_TC, stage ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const float *sk = sm + (size_t)stage * STAGE, *sr = sk + LR_TC * D, *sw = sr + LR_TC * D;
        const float *sa = sw + LR_TC * D, *sb = sa + (RANK1 ? LR_TC * D : 0), *sv = sb + (RANK1 ? LR_TC * D : 0);
        const int n = min(LR_TC, t1 - tb);
        auto token = [&](int c) -> float {
            const float4 *k4 = reinterpret_cast<const float4 *>(sk + c * D), *r4 = reinterpret_cast<const float4 *>(sr + c * D),
                         *w4 = reinterpret_cast<const float4 *>(sw + c * D), *a4 = reinterpret_cast<const float4 *>(sa + c * D),
                         *b4 = reinterpret_cast<const float4 *>(sb + c * D);
            float held = 0.f;
            if (RANK1) {
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float4 bb = b4[LR_LPC * m + part];
                    s0 = fmaf(Sc[m][0], bb.x, s0);
                    s1 = fmaf(Sc[m][1], bb.y, s1);
                    s2 = fmaf(Sc[m][2], bb.z, s2);
                    s3 = fmaf(Sc[m][3], bb.w, s3);
                }
                held = (s0 + s1) + (s2 + s3);
#pragma unroll
                for (int sh = 1; sh < LR_LPC; sh <<= 1) held += __shfl_xor_sync(0xffffffffu, held, sh);
            }
            const float vj = sv[c * 32 + jl];
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float4 kk = k4[LR_LPC * m + part], rr = r4[LR_LPC * m + part], ww = w4[LR_LPC * m + part];
                float e0 = kk.x * vj, e1 = kk.y * vj, e2 = kk.z * vj, e3 = kk.w * vj;
                if (RANK1) {
                    const float4 aa = a4[LR_LPC * m + part];
                    e0 = fmaf(aa.x, held, e0); e1 = fmaf(aa.y, held, e1); e2 = fmaf(aa.z, held, e2); e3 = fmaf(aa.w, held, e3);
                }
                Sc[m][0] = fmaf(ww.x, Sc[m][0], e0); s0 = fmaf(Sc[m][0], rr.x, s0);
                Sc[m][1] = fmaf(ww.y, Sc[m][1], e1); s1 = fmaf(Sc[m][1], rr.y, s1);
                Sc[m][2] = fmaf(ww.z, Sc[m][2], e2); s2 = fmaf(Sc[m][2], rr.z, s2);
                Sc[m][3] = fmaf(ww.w, Sc[m][3], e3); s3 = fmaf(Sc[m][3], rr.w, s3);
            }
            return (s0 + s1) + (s2 + s3);             // this thread's part of the read-out; the lanes' parts are summed below
        };
        auto reduce_store = [&](int c, float o) {
#pragma unroll
            for (int sh = 1; sh < LR_LPC; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
            if (live && part == 0) out[((size_t)(tb + c) * H + h) * dv + j] = o;
        };
        // A full stage is one block of code, so that the next token's operands are fetched under this token's chain.
        if (n == LR_TC && !RANK1) {
            // No sum over lanes lies on the way from state to state.  The next token's operands are in registers before
            // this token's update starts, and the read-outs of the stage's tokens go through the shuffle tree together at
            // its end: eight independent chains instead of one after every token (2,048 tokens of 16 heads of 64 x 128:
            // 436 -> 290 us).  The tree is the same one either way: same bits.
            float o[LR_TC];
            float4 K[M], R[M], W[M];
            float vj = sv[jl];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                K[m] = reinterpret_cast<const float4 *>(sk)[LR_LPC * m + part]; R[m] = reinterpret_cast<const float4 *>(sr)[LR_LPC * m + part];
                W[m] = reinterpret_cast<const float4 *>(sw)[LR_LPC * m + part];
            }
#pragma unroll
            for (int c = 0; c < LR_TC; ++c) {
                float4 K2[M], R2[M], W2[M];
                float v2 = 0.f;
                if (c + 1 < LR_TC) {
                    v2 = sv[(c + 1) * 32 + jl];
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const int e = (c + 1) * (D / 4) + LR_LPC * m + part;
                        K2[m] = reinterpret_cast<const float4 *>(sk)[e]; R2[m] = reinterpret_cast<const float4 *>(sr)[e];
                        W2[m] = reinterpret_cast<const float4 *>(sw)[e];
                    }
                }
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    Sc[m][0] = fmaf(W[m].x, Sc[m][0], K[m].x * vj); s0 = fmaf(Sc[m][0], R[m].x, s0);
                    Sc[m][1] = fmaf(W[m].y, Sc[m][1], K[m].y * vj); s1 = fmaf(Sc[m][1], R[m].y, s1);
                    Sc[m][2] = fmaf(W[m].z, Sc[m][2], K[m].z * vj); s2 = fmaf(Sc[m][2], R[m].z, s2);
                    Sc[m][3] = fmaf(W[m].w, Sc[m][3], K[m].w * vj); s3 = fmaf(Sc[m][3], R[m].w, s3);
                }
                o[c] = (s0 + s1) + (s2 + s3);
                if (c + 1 < LR_TC) {
                    vj = v2;
#pragma unroll
                    for (int m = 0; m < M; ++m) { K[m] = K2[m]; R[m] = R2[m]; W[m] = W2[m]; }
                }
            }
#pragma unroll
            for (int sh = 1; sh < LR_LPC; sh <<= 1)
#pragma unroll
                for (int c = 0; c < LR_TC; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], sh);
            if (live && part == 0) {
#pragma unroll
                for (int c = 0; c < LR_TC; ++c) out[((size_t)(tb + c) * H + h) * dv + j] = o[c];
            }
        } else if (n == LR_TC && D <= 32) {
            // few channels with the correction: the read-outs of the stage together as above (471 -> 354 us for 2,048 tokens)
            float o[LR_TC];
#pragma unroll
            for (int c = 0; c < LR_TC; ++c) o[c] = token(c);
#pragma unroll
            for (int sh = 1; sh < LR_LPC; sh <<= 1)
#pragma unroll
                for (int c = 0; c < LR_TC; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], sh);
            if (live && part == 0) {
#pragma unroll
                for (int c = 0; c < LR_TC; ++c) out[((size_t)(tb + c) * H + h) * dv + j] = o[c];
            }
        } else if (n == LR_TC && D <= 128) {
            // With the correction the sum b^T S over a column's lanes lies on the way from state to state.  Two things keep
            // the rest off that way: the next token's operands are in registers before this token's chain starts, and the
            // previous token's read-out goes through the shuffle tree level by level beside this token's b^T S (the same
            // tree as alone: same bits).
            float4 K[M], R[M], W[M], A[M], B[M];
            float vj = sv[jl];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                K[m] = reinterpret_cast<const float4 *>(sk)[LR_LPC * m + part]; R[m] = reinterpret_cast<const float4 *>(sr)[LR_LPC * m + part];
                W[m] = reinterpret_cast<const float4 *>(sw)[LR_LPC * m + part]; A[m] = reinterpret_cast<const float4 *>(sa)[LR_LPC * m + part];
                B[m] = reinterpret_cast<const float4 *>(sb)[LR_LPC * m + part];
            }
            float o_prev = 0.f;
#pragma unroll
            for (int c = 0; c < LR_TC; ++c) {
                float4 K2[M], R2[M], W2[M], A2[M], B2[M];
                float v2 = 0.f;
                if (c + 1 < LR_TC) {
                    v2 = sv[(c + 1) * 32 + jl];
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const int e = (c + 1) * (D / 4) + LR_LPC * m + part;
                        K2[m] = reinterpret_cast<const float4 *>(sk)[e]; R2[m] = reinterpret_cast<const float4 *>(sr)[e];
                        W2[m] = reinterpret_cast<const float4 *>(sw)[e]; A2[m] = reinterpret_cast<const float4 *>(sa)[e];
                        B2[m] = reinterpret_cast<const float4 *>(sb)[e];
                    }
                }
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    s0 = fmaf(Sc[m][0], B[m].x, s0);
                    s1 = fmaf(Sc[m][1], B[m].y, s1);
                    s2 = fmaf(Sc[m][2], B[m].z, s2);
                    s3 = fmaf(Sc[m][3], B[m].w, s3);
                }
                float held = (s0 + s1) + (s2 + s3);
#pragma unroll
                for (int sh = 1; sh < LR_LPC; sh <<= 1) {
                    const float hx = __shfl_xor_sync(0xffffffffu, held, sh);
                    const float ox = c > 0 ? __shfl_xor_sync(0xffffffffu, o_prev, sh) : 0.f;
                    held += hx;
                    if (c > 0) o_prev += ox;
                }
                if (c > 0 && live && part == 0) out[((size_t)(tb + c - 1) * H + h) * dv + j] = o_prev;
                s0 = s1 = s2 = s3 = 0.f;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float e0 = fmaf(A[m].x, held, K[m].x * vj), e1 = fmaf(A[m].y, held, K[m].y * vj);
                    const float e2 = fmaf(A[m].z, held, K[m].z * vj), e3 = fmaf(A[m].w, held, K[m].w * vj);
                    Sc[m][0] = fmaf(W[m].x, Sc[m][0], e0); s0 = fmaf(Sc[m][0], R[m].x, s0);
                    Sc[m][1] = fmaf(W[m].y, Sc[m][1], e1); s1 = fmaf(Sc[m][1], R[m].y, s1);
                    Sc[m][2] = fmaf(W[m].z, Sc[m][2], e2); s2 = fmaf(Sc[m][2], R[m].z, s2);
                    Sc[m][3] = fmaf(W[m].w, Sc[m][3], e3); s3 = fmaf(Sc[m][3], R[m].w, s3);
                }
                o_prev = (s0 + s1) + (s2 + s3);
                if (c + 1 < LR_TC) {
                    vj = v2;
#pragma unroll
                    for (int m = 0; m < M; ++m) { K[m] = K2[m]; R[m] = R2[m]; W[m] = W2[m]; A[m] = A2[m]; B[m] = B2[m]; }
                }
            }
            reduce_store(LR_TC - 1, o_prev);
        } else if (n == LR_TC) {
#pragma unroll
            for (int c = 0; c < LR_TC; ++c) reduce_store(c, token(c));
        } else {
            for (int c = 0; c < n; ++c) reduce_store(c, token(c));
        }
        __syncthreads();                              // the stage may be filled again
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (live) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = 4 * (LR_LPC * m + part) + c;
                if (i < d) Sg[(size_t)i * dv + j] = Sc[m][c];
            }
    }
}

// ---- per-head norm of the read-out, weight, optional sigmoid gate ---------------------------------
// out = o / sqrt(mean(o^2) + eps) * w[h * w_stride + i] (* sigmoid(gate column g_col0 + h dv + i)) in the storage type
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float *__restrict__ o, const float *__restrict__ w, int w_stride, float eps, const float *__restrict__ g_part,
                      int Sg, size_t g_stride, int g_ld, int g_col0, T *__restrict__ out, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = blockIdx.y * 4 + warp; h < H; h += gridDim.y * 4) {
        const size_t base = ((size_t)t * H + h) * dv;
        float ss = 0.f;
        for (int i = lane; i < dv; i += 32) ss = fmaf(o[base + i], o[base + i], ss);
        ss = warp_sum(ss);
        const float rn = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int i = lane; i < dv; i += 32) {
            float y = o[base + i] * rn * w[(size_t)h * w_stride + i];
            if (g_part) y *= lr_sigmoid(sum_slices(g_part, Sg, g_stride, (size_t)t * g_ld + g_col0 + (size_t)h * dv + i));
            out[base + i] = from_f32<T>(y);
        }
    }
}

KESTREL_API int kestrel_forget_gates(const float *partial, int S, long long slice_stride, int ld, int col_q, int col_f, int col_v,
                                     const float *f_bias, const float *lower, float *r_out, float *w_out, float *k_out, float *v_out,
                                     int T, int n, int nv, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && S > 0 && n > 0 && nv > 0 && col_q >= 0 && col_f >= 0 && col_v >= 0 && col_q + n <= ld && col_f + n <= ld && col_v + nv <= ld,
                    "forget_gates: bad sizes");
    // elementwise: any block size gives the same bits; a step of few tokens has few blocks, so each gets more threads
    kestrel_launch(forget_gates_kernel, dim3(T), dim3(T >= 512 ? 256 : 1024), 0, stream, partial, S, (size_t)slice_stride, ld, col_q, col_f, col_v, f_bias, lower,
                   r_out, w_out, k_out, v_out, n, nv);
    return kestrel_check_launch("forget_gates");
}

KESTREL_API int kestrel_removal_gates(const float *partial, int S, long long slice_stride, int ld, int col_r, int col_k, int col_v, int col_a,
                                      const float *a_bias, const float *wz, int Sw, long long w_stride, const float *w_bias, float decay_rate,
                                      float *r_out, float *k_out, float *v_out, float *w_out, float *a_out, float *b_out, int T, int H, int d,
                                      cudaStream_t stream) {
    if (T == 0) return 0;
    const int n = H * d;
    KESTREL_REQUIRE(T > 0 && S > 0 && Sw > 0 && H > 0 && d > 0 && col_r >= 0 && col_k >= 0 && col_v >= 0 && col_a >= 0 && col_r + n <= ld &&
                    col_k + n <= ld && col_v + n <= ld && col_a + n <= ld && d <= 256, "removal_gates: bad sizes");
    const int by = T >= 512 ? 1 : (H + 3) / 4;
    if (T >= 512) {
        kestrel_launch(removal_gates_stream_kernel, dim3(T, by), dim3(128), 0, stream, partial, S, (size_t)slice_stride, ld, col_r, col_k, col_v, col_a, a_bias,
                   wz, Sw, (size_t)w_stride, w_bias, decay_rate, r_out, k_out, v_out, w_out, a_out, b_out, H, d);
        return kestrel_check_launch("removal_gates");
    }
#define RG_LAUNCH(J) kestrel_launch(removal_gates_kernel<J>, dim3(T, by), dim3(128), 0, stream, partial, S, (size_t)slice_stride, ld, col_r, col_k, col_v, col_a, a_bias, \
                   wz, Sw, (size_t)w_stride, w_bias, decay_rate, r_out, k_out, v_out, w_out, a_out, b_out, H, d)
    if (d <= 64) RG_LAUNCH(2);
    else if (d <= 128) RG_LAUNCH(4);
    else RG_LAUNCH(8);
#undef RG_LAUNCH
    return kestrel_check_launch("removal_gates");
}

template <int D, bool RANK1>
static int lr_launch(dim3 grid, cudaStream_t stream, const float *r, const float *w, const float *k, const float *v, const float *a,
                     const float *b, float *state, size_t state_stride, size_t state_off, const int *cu_seqlens, const int *slots, float *out,
                     int H, int d, int dv) {
    constexpr size_t smem_need = (size_t)2 * LR_TC * ((RANK1 ? 5 : 3) * D + 32) * sizeof(float);
    static bool attr_set = false;
    if (!attr_set && cudaFuncSetAttribute(recurrence_scan_kernel<D, RANK1>, cudaFuncAttributeMaxDynamicSharedMemorySize, KESTREL_SMEM_MAX_DYNAMIC) != cudaSuccess)
        return kestrel_fail(-3, "recurrence_scan: cannot set the shared memory size");
    attr_set = true;
    // a prompt's scan is few CTAs that run for hundreds of microseconds: one SM each (kestrel_spread_smem)
    const size_t smem = kestrel_spread_smem((long)grid.x * grid.y * grid.z, smem_need);
    kestrel_launch(recurrence_scan_kernel<D, RANK1>, grid, dim3(128), smem, stream, r, w, k, v, a, b, state, state_stride, state_off, cu_seqlens,
                   slots, out, H, d, dv);
    return kestrel_check_launch("recurrence_scan");
}

KESTREL_API int kestrel_recurrence_scan(const float *r, const float *w, const float *k, const float *v, const float *a, const float *b,
                                        float *state, long long state_stride, long long state_off, const int *cu_seqlens, const int *slots,
                                        float *out, int nseq, int H, int d, int dv, cudaStream_t stream) {
    if (nseq == 0) return 0;
    KESTREL_REQUIRE(nseq > 0 && H > 0 && d > 0 && dv > 0 && state_off >= 0, "recurrence_scan: bad sizes");
    KESTREL_REQUIRE((a == nullptr) == (b == nullptr), "recurrence_scan: the correction needs both of its vectors");
    KESTREL_REQUIRE(d <= 256, "recurrence_scan: key size %d exceeds 256", d);
    KESTREL_REQUIRE(H <= 65535 && nseq <= 65535, "recurrence_scan: grid too large");
    dim3 grid((dv + LR_COLS - 1) / LR_COLS, H, nseq);
#define LR_CASE(D)                                                                                                                            \
    return a ? lr_launch<D, true>(grid, stream, r, w, k, v, a, b, state, (size_t)state_stride, (size_t)state_off, cu_seqlens, slots, out, H, d, dv) \
             : lr_launch<D, false>(grid, stream, r, w, k, v, a, b, state, (size_t)state_stride, (size_t)state_off, cu_seqlens, slots, out, H, d, dv)
    if (d <= 32) { LR_CASE(32); }
    if (d <= 64) { LR_CASE(64); }
    if (d <= 128) { LR_CASE(128); }
    LR_CASE(256);
#undef LR_CASE
}

KESTREL_API int kestrel_head_norm_gate(const float *o, const float *w, int w_stride, float eps, const float *g_part, int Sg, long long g_stride,
                                       int g_ld, int g_col0, void *out, int dtype, int T, int H, int dv, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && dv > 0 && (w_stride == 0 || w_stride == dv) && (!g_part || (Sg > 0 && g_col0 >= 0 && g_col0 + H * dv <= g_ld)),
                    "head_norm_gate: bad sizes");
    const int by = T >= 512 ? 1 : (H + 3) / 4;
    if (dtype == KESTREL_F32)
        kestrel_launch(head_norm_gate_kernel<float>, dim3(T, by), dim3(128), 0, stream, o, w, w_stride, eps, g_part, Sg, (size_t)g_stride, g_ld, g_col0,
                       (float *)out, H, dv);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(T, by), dim3(128), 0, stream, o, w, w_stride, eps, g_part, Sg, (size_t)g_stride, g_ld,
                       g_col0, (__nv_bfloat16 *)out, H, dv);
    else
        return kestrel_fail(-2, "head_norm_gate: unknown dtype %d", dtype);
    return kestrel_check_launch("head_norm_gate");
}
