// Row-wise kernels around the residual stream that arrangements other than the pre-norm block
// need: an absolute sinusoidal position vector added to the embedded tokens, the add of two
// sublayers' outputs at once (a block whose mixer and feed-forward read the same norm), a
// gated look-up of a per-token table, and the add of a normalised product.
//
// A product reaches these kernels as float32 slices [S, T, N] that are summed in ascending s, as
// everywhere in the library; all sums and norms are float32.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// x[t, 2i] += sin(pos[t] * f[i]), x[t, 2i + 1] += cos(pos[t] * f[i]); angles in float32
// ------------------------------------------------------------------------------------------
__global__ void add_sinusoid_kernel(float *__restrict__ x, const int *__restrict__ positions,
                                    const float *__restrict__ freq, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    float *row = x + (size_t)t * d;
    for (int i = threadIdx.x; 2 * i < d; i += blockDim.x) {
        float s, c;
        sincosf(p * freq[i], &s, &c);
        row[2 * i] += s;
        if (2 * i + 1 < d) row[2 * i + 1] += c;
    }
}

KESTREL_API int kestrel_add_sinusoid(float *x, const int *positions, const float *freq, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0, "add_sinusoid: bad sizes T=%d d=%d", T, d);
    kestrel_launch(add_sinusoid_kernel, dim3(T), dim3(128), 0, stream, x, positions, freq, d);
    return kestrel_check_launch("add_sinusoid");
}

// ------------------------------------------------------------------------------------------
// residual[t] += sum_s a[s, t] + sum_s b[s, t]  (b may be null); cast[t] = residual[t] in the
// storage type (cast may be null).  The order of the sum is fixed: a's slices, then b's.
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void add_two_kernel(float *__restrict__ residual, const float *__restrict__ a, int Sa, size_t stride_a,
                               const float *__restrict__ b, int Sb, size_t stride_b, TOut *__restrict__ cast, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float va = sum_slices(a, Sa, stride_a, idx), vb = Sb > 0 ? sum_slices(b, Sb, stride_b, idx) : 0.f;
    float v = residual[idx] + (va + vb);
    residual[idx] = v;
    if (cast) cast[idx] = from_f32<TOut>(v);
}

KESTREL_API int kestrel_add_two(float *residual, const float *a, int Sa, long long stride_a, const float *b, int Sb, long long stride_b,
                                void *cast, int cast_dtype, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && a && Sa > 0 && (b || Sb == 0), "add_two: bad arguments");
    size_t n = (size_t)T * d;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (cast_dtype == KESTREL_F32)
        kestrel_launch(add_two_kernel<float>, dim3(blocks), dim3(256), 0, stream, residual, a, Sa, (size_t)stride_a, b, Sb, (size_t)stride_b, (float *)cast, n);
    else if (cast_dtype == KESTREL_BF16)
        kestrel_launch(add_two_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, residual, a, Sa, (size_t)stride_a, b, Sb, (size_t)stride_b, (__nv_bfloat16 *)cast, n);
    else
        return kestrel_fail(-2, "add_two: unknown dtype %d", cast_dtype);
    return kestrel_check_launch("add_two");
}

// ------------------------------------------------------------------------------------------
// out[t, i] = gelu_tanh(sum_s g[s, t, i]) * table[ids[t], col0 + i], i < n
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TW, typename TOut>
__global__ void gelu_table_mul_kernel(const float *__restrict__ g, int S, size_t slice_stride, int ld, const TW *__restrict__ table,
                                      int table_ld, int col0, const int *__restrict__ ids, TOut *__restrict__ out, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const TW *row = table + (size_t)ids[t] * table_ld + col0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float z = sum_slices(g, S, slice_stride, (size_t)t * ld + i);
        out[(size_t)t * n + i] = from_f32<TOut>(gelu_tanh_f(z) * to_f32<TW>(row[i]));
    }
}

KESTREL_API int kestrel_gelu_table_mul(const float *g, int S, long long slice_stride, int ld, const void *table, int table_ld, int col0,
                                       const int *ids, void *out, int dtype, int T, int n, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && n > 0 && S > 0, "gelu_table_mul: bad sizes");
    if (dtype == KESTREL_F32)
        kestrel_launch(gelu_table_mul_kernel<float, float>, dim3(T), dim3(128), 0, stream, g, S, (size_t)slice_stride, ld, (const float *)table, table_ld, col0, ids, (float *)out, n);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(gelu_table_mul_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(128), 0, stream, g, S, (size_t)slice_stride, ld, (const __nv_bfloat16 *)table, table_ld, col0, ids,
                       (__nv_bfloat16 *)out, n);
    else
        return kestrel_fail(-2, "gelu_table_mul: unknown dtype %d", dtype);
    return kestrel_check_launch("gelu_table_mul");
}

// ------------------------------------------------------------------------------------------
// y = sum_s p[s, t]; residual[t] += y / sqrt(mean(y^2) + eps) * w.  One block a row, the sum of
// squares in a fixed tree.
// ------------------------------------------------------------------------------------------
#define AN_THREADS 256
__global__ void __launch_bounds__(AN_THREADS)
add_normed_kernel(float *__restrict__ residual, const float *__restrict__ p, int S, size_t slice_stride,
                  const float *__restrict__ w, float eps, int d) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float ys[];
    __shared__ float red[AN_THREADS / 32];
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += AN_THREADS) {
        const float y = sum_slices(p, S, slice_stride, (size_t)t * d + i);
        ys[i] = y;
        ss = fmaf(y, y, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < AN_THREADS / 32; ++k) tot += red[k];
    const float r = 1.0f / sqrtf(tot / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += AN_THREADS) residual[(size_t)t * d + i] += ys[i] * r * w[i];
}

KESTREL_API int kestrel_add_normed(float *residual, const float *p, int S, long long slice_stride, const float *w, float eps, int T, int d,
                                   cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && S > 0 && d <= 12000, "add_normed: bad sizes T=%d d=%d", T, d);
    kestrel_launch(add_normed_kernel, dim3(T), dim3(AN_THREADS), (size_t)d * sizeof(float), stream, residual, p, S, (size_t)slice_stride, w, eps, d);
    return kestrel_check_launch("add_normed");
}

// ------------------------------------------------------------------------------------------
// out[t, i] = sum_s p[s, t, col0 + i] in the storage type, i < n: some columns of a fused
// product, as the input of a second product
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void partial_columns_kernel(const float *__restrict__ p, int S, size_t slice_stride, int ld, int col0,
                                       TOut *__restrict__ out, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t t = idx / n;
    int i = (int)(idx % n);
    out[idx] = from_f32<TOut>(sum_slices(p, S, slice_stride, t * ld + col0 + i));
}

KESTREL_API int kestrel_partial_columns(const float *p, int S, long long slice_stride, int ld, int col0, void *out, int dtype, int T, int n,
                                        cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && n > 0 && S > 0 && col0 >= 0 && col0 + n <= ld, "partial_columns: bad sizes");
    size_t total = (size_t)T * n;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KESTREL_F32)
        kestrel_launch(partial_columns_kernel<float>, dim3(blocks), dim3(256), 0, stream, p, S, (size_t)slice_stride, ld, col0, (float *)out, n, total);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(partial_columns_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, p, S, (size_t)slice_stride, ld, col0, (__nv_bfloat16 *)out, n, total);
    else
        return kestrel_fail(-2, "partial_columns: unknown dtype %d", dtype);
    return kestrel_check_launch("partial_columns");
}

// ------------------------------------------------------------------------------------------
// The same with an activation on the summed columns: 0 none, 1 the square of relu, 2 tanh, 3 silu, 4 gelu (erf), 5 gelu (tanh form).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float column_act(float z, int act) {
    if (act == 4) return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));                                   // the exact gelu
    if (act == 5) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));       // its tanh form
    if (act == 1) { const float r = fmaxf(z, 0.f); return r * r; }
    if (act == 2) return tanhf(z);
    if (act == 3) return z / (1.0f + expf(-z));
    return z;
}

template <typename TOut>
__global__ void partial_columns_act_kernel(const float *__restrict__ p, int S, size_t slice_stride, int ld, int col0,
                                           const float *__restrict__ bias, int act, TOut *__restrict__ out, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t t = idx / n;
    int i = (int)(idx % n);
    float z = sum_slices(p, S, slice_stride, t * ld + col0 + i);
    if (bias) z += bias[col0 + i];
    out[idx] = from_f32<TOut>(column_act(z, act));
}

KESTREL_API int kestrel_partial_columns_act(const float *p, int S, long long slice_stride, int ld, int col0, const float *bias, int act, void *out,
                                            int dtype, int T, int n, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && n > 0 && S > 0 && col0 >= 0 && col0 + n <= ld && act >= 0 && act <= 5, "partial_columns_act: bad sizes or activation %d", act);
    size_t total = (size_t)T * n;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KESTREL_F32)
        kestrel_launch(partial_columns_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, p, S, (size_t)slice_stride, ld, col0, bias, act, (float *)out, n, total);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(partial_columns_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, p, S, (size_t)slice_stride, ld, col0, bias, act, (__nv_bfloat16 *)out, n, total);
    else
        return kestrel_fail(-2, "partial_columns_act: unknown dtype %d", dtype);
    return kestrel_check_launch("partial_columns_act");
}

// ------------------------------------------------------------------------------------------
// Block-wide sum in a fixed tree: lanes by shuffle, warps in ascending order.  Every thread gets it.
// ------------------------------------------------------------------------------------------
// A block takes one row of width d and sums over it as VT = gn_threads(d) "virtual threads" would: virtual
// thread u owns the elements u, u + VT, u + 2 VT, ... in ascending order, 32 consecutive ones add in a
// shuffle tree, and the VT / 32 sums are added in ascending order.  VT depends on d alone, so every bit
// of a row is the same whether the step has one token or thousands.  How many REAL threads play them is
// free: a step of few tokens has few blocks, each bound by the latency of its loads, and gets VT threads
// (Q = 1: all of a row's loads in flight at once); a step of many tokens gets VT / Q threads that each
// keep Q partial sums, which loads the SMs more evenly.
#define GN_VT_MAX 1024
static inline int gn_threads(int d) { return d >= 1024 ? 1024 : d >= 512 ? 512 : 256; }
static inline int gn_fold(int T, int d) { return T >= 256 ? gn_threads(d) / 256 : 1; }        // Q: 1, 2 or 4
template <int Q>
__device__ __forceinline__ float gn_block_sum(const float (&part)[Q], float *red) {
    const int warps = blockDim.x >> 5;
    __syncthreads();                                  // red may still be read from the sum before
#pragma unroll
    for (int q = 0; q < Q; ++q) {
        const float v = warp_sum(part[q]);
        if ((threadIdx.x & 31) == 0) red[q * warps + (threadIdx.x >> 5)] = v;
    }
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < Q * warps; ++k) tot += red[k];
    return tot;
}

// ------------------------------------------------------------------------------------------
// Two products side by side, each normalised over the row with a weight of its own, then mixed:
// out[t] = mix * (a / sqrt(mean(a^2) + eps) * wa + b / sqrt(mean(b^2) + eps) * wb), float32.
// ------------------------------------------------------------------------------------------
template <int Q>
__global__ void __launch_bounds__(GN_VT_MAX / Q, 2 * Q)          // 2,048 threads an SM in every form
combine_normed_kernel(const float *__restrict__ a, int Sa, size_t stride_a, const float *__restrict__ wa, const float *__restrict__ b, int Sb,
                      size_t stride_b, const float *__restrict__ wb, float eps, float mix, float *__restrict__ out, int d) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float cn_rows[];               // a's row, then b's
    __shared__ float red[GN_VT_MAX / 32];
    const int t = blockIdx.x, nt = blockDim.x;
    float *ra = cn_rows, *rb = cn_rows + d;
    float sa[Q], sb[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) sa[q] = sb[q] = 0.f;
#pragma unroll
    for (int q = 0; q < Q; ++q) {                    // one partial sum live at a time: few registers, many warps an SM
        for (int i = q * nt + threadIdx.x; i < d; i += Q * nt) {
            {
                const float x = sum_slices(a, Sa, stride_a, (size_t)t * d + i), y = sum_slices(b, Sb, stride_b, (size_t)t * d + i);
                ra[i] = x;
                rb[i] = y;
                sa[q] = fmaf(x, x, sa[q]);
                sb[q] = fmaf(y, y, sb[q]);
            }
        }
    }
    const float na = 1.0f / sqrtf(gn_block_sum<Q>(sa, red) / (float)d + eps);
    const float nb = 1.0f / sqrtf(gn_block_sum<Q>(sb, red) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += nt) out[(size_t)t * d + i] = mix * (ra[i] * na * wa[i] + rb[i] * nb * wb[i]);
}

KESTREL_API int kestrel_combine_normed(const float *a, int Sa, long long stride_a, const float *wa, const float *b, int Sb, long long stride_b,
                                       const float *wb, float eps, float mix, float *out, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && Sa > 0 && Sb > 0 && d <= 12000, "combine_normed: bad sizes T=%d d=%d", T, d);
    if ((size_t)2 * d * sizeof(float) > 48 * 1024) {          // both rows of a wide model: more shared memory than a kernel gets unasked
        static bool attr_set = false;
        if (!attr_set && (cudaFuncSetAttribute(combine_normed_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 12000 * 2 * (int)sizeof(float)) != cudaSuccess ||
                          cudaFuncSetAttribute(combine_normed_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 12000 * 2 * (int)sizeof(float)) != cudaSuccess ||
                          cudaFuncSetAttribute(combine_normed_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 12000 * 2 * (int)sizeof(float)) != cudaSuccess))
            return kestrel_fail(-3, "combine_normed: cannot set the shared memory size");
        attr_set = true;
    }
    const int Q = gn_fold(T, d);
#define CN_LAUNCH(QQ) kestrel_launch(combine_normed_kernel<QQ>, dim3(T), dim3(gn_threads(d) / QQ), (size_t)2 * d * sizeof(float), stream, a, Sa, (size_t)stride_a, wa, b, Sb, \
                   (size_t)stride_b, wb, eps, mix, out, d)
    if (Q == 4) CN_LAUNCH(4);
    else if (Q == 2) CN_LAUNCH(2);
    else CN_LAUNCH(1);
#undef CN_LAUNCH
    return kestrel_check_launch("combine_normed");
}

// ------------------------------------------------------------------------------------------
// A sublayer's result y (slices, optional bias) is gated by sigmoid(g + g_bias) where a gate product g is
// given, normalised over the row with the weight w, and added to the residual stream:
//     residual[t] += (y * sigmoid(g)) / sqrt(mean((y * sigmoid(g))^2) + eps) * w
// and, where `next_w` is given, the next norm of the stream is made in the same pass:
//     next_out[t] = residual[t] / sqrt(mean(residual[t]^2) + eps_next) * next_w       (storage type)
// ------------------------------------------------------------------------------------------
template <typename TOut, int Q>
__global__ void __launch_bounds__(GN_VT_MAX / Q, 2 * Q)          // 2,048 threads an SM in every form
add_gated_normed_kernel(float *__restrict__ residual, const float *__restrict__ y, int Sy, size_t stride_y, const float *__restrict__ y_bias,
                        const float *__restrict__ g, int Sg, size_t stride_g, const float *__restrict__ g_bias, const float *__restrict__ w,
                        float eps, const float *__restrict__ next_w, float eps_next, TOut *__restrict__ next_out, int d) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float gn_row[];
    __shared__ float red[GN_VT_MAX / 32];
    const int t = blockIdx.x, nt = blockDim.x;
    float ss[Q], s2[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) ss[q] = s2[q] = 0.f;
#pragma unroll
    for (int q = 0; q < Q; ++q) {                    // one partial sum live at a time: few registers, many warps an SM
        for (int i = q * nt + threadIdx.x; i < d; i += Q * nt) {
            {
                float v = sum_slices(y, Sy, stride_y, (size_t)t * d + i);
                if (y_bias) v += y_bias[i];
                if (g) {
                    float z = sum_slices(g, Sg, stride_g, (size_t)t * d + i);
                    if (g_bias) z += g_bias[i];
                    v *= 1.0f / (1.0f + expf(-z));
                }
                gn_row[i] = v;
                ss[q] = fmaf(v, v, ss[q]);
            }
        }
    }
    const float rn = 1.0f / sqrtf(gn_block_sum<Q>(ss, red) / (float)d + eps);
#pragma unroll
    for (int q = 0; q < Q; ++q) {                    // one partial sum live at a time: few registers, many warps an SM
        for (int i = q * nt + threadIdx.x; i < d; i += Q * nt) {
            {
                const float x = residual[(size_t)t * d + i] + gn_row[i] * rn * w[i];
                residual[(size_t)t * d + i] = x;
                gn_row[i] = x;
                s2[q] = fmaf(x, x, s2[q]);
            }
        }
    }
    if (!next_w) return;
    const float r2 = 1.0f / sqrtf(gn_block_sum<Q>(s2, red) / (float)d + eps_next);
    for (int i = threadIdx.x; i < d; i += nt) next_out[(size_t)t * d + i] = from_f32<TOut>(gn_row[i] * r2 * next_w[i]);
}

KESTREL_API int kestrel_add_gated_normed(float *residual, const float *y, int Sy, long long stride_y, const float *y_bias, const float *g, int Sg,
                                         long long stride_g, const float *g_bias, const float *w, float eps, const float *next_w, float eps_next,
                                         void *next_out, int next_dtype, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && Sy > 0 && (!g || Sg > 0) && d <= 12000 && ((next_w == nullptr) == (next_out == nullptr)),
                    "add_gated_normed: bad arguments T=%d d=%d", T, d);
    const int Q = gn_fold(T, d);
#define GN_LAUNCH(TT, QQ) kestrel_launch(add_gated_normed_kernel<TT, QQ>, dim3(T), dim3(gn_threads(d) / QQ), (size_t)d * sizeof(float), stream, residual, y, Sy, \
                   (size_t)stride_y, y_bias, g, Sg, (size_t)stride_g, g_bias, w, eps, next_w, eps_next, (TT *)next_out, d)
#define GN_LAUNCH_Q(TT) do { if (Q == 4) GN_LAUNCH(TT, 4); else if (Q == 2) GN_LAUNCH(TT, 2); else GN_LAUNCH(TT, 1); } while (0)
    if (next_dtype == KESTREL_F32 || !next_w) GN_LAUNCH_Q(float);
    else if (next_dtype == KESTREL_BF16) GN_LAUNCH_Q(__nv_bfloat16);
    else return kestrel_fail(-2, "add_gated_normed: unknown dtype %d", next_dtype);
#undef GN_LAUNCH_Q
#undef GN_LAUNCH
    return kestrel_check_launch("add_gated_normed");
}

// ------------------------------------------------------------------------------------------
// x[t] += table[ids[t]]: the embedded tokens added to the stream again (a model that runs some
// of its layers several times feeds them in before each further pass)
// ------------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_add_kernel(const TW *__restrict__ table, const int *__restrict__ ids, float *__restrict__ x, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const TW *row = table + (size_t)ids[t] * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) x[(size_t)t * d + i] += to_f32<TW>(row[i]);
}

KESTREL_API int kestrel_embed_add(const void *table, int dtype, const int *ids, float *x, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0, "embed_add: bad sizes");
    if (dtype == KESTREL_F32) kestrel_launch(embed_add_kernel<float>, dim3(T), dim3(256), 0, stream, (const float *)table, ids, x, d);
    else if (dtype == KESTREL_BF16) kestrel_launch(embed_add_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16 *)table, ids, x, d);
    else return kestrel_fail(-2, "embed_add: unknown dtype %d", dtype);
    return kestrel_check_launch("embed_add");
}

// ------------------------------------------------------------------------------------------
// logits <- logits * scale, then cap * tanh(logits / cap) where cap > 0; in place, float32
// ------------------------------------------------------------------------------------------
__global__ void logit_scale_cap_kernel(float *__restrict__ logits, size_t ld, int R, int V, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= V) return;
    for (int r = blockIdx.y; r < R; r += gridDim.y) {
        float *row = logits + (size_t)r * ld;
        float z = row[i] * scale;
        if (cap > 0.f) z = cap * tanhf(z / cap);
        row[i] = z;
    }
}

KESTREL_API int kestrel_logit_scale_cap(float *logits, long long ld, int R, int V, float scale, float cap, cudaStream_t stream) {
    if (R == 0) return 0;
    KESTREL_REQUIRE(R > 0 && V > 0 && cap >= 0.f, "logit_scale_cap: bad sizes R=%d V=%d", R, V);
    kestrel_launch(logit_scale_cap_kernel, dim3((V + 255) / 256, R < 32768 ? R : 32768), dim3(256), 0, stream, logits, (size_t)ld, R, V, scale, cap);
    return kestrel_check_launch("logit_scale_cap");
}

// ------------------------------------------------------------------------------------------
// residual[t] += sum_s a[s, t] + sum_s b[s, t] + sum_s c[s, t]  (b and c may be null): `add_two` with one more
// product, for a layer whose feed-forward is two (routed experts and one that every token takes).  The order of
// the sum is fixed: (a + b) + c, each its slices in ascending order; without c the bits of `add_two`.
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void add_three_kernel(float *__restrict__ residual, const float *__restrict__ a, int Sa, size_t stride_a,
                                 const float *__restrict__ b, int Sb, size_t stride_b, const float *__restrict__ c, int Sc, size_t stride_c,
                                 TOut *__restrict__ cast, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float va = sum_slices(a, Sa, stride_a, idx), vb = Sb > 0 ? sum_slices(b, Sb, stride_b, idx) : 0.f;
    float add = va + vb;
    if (Sc > 0) add += sum_slices(c, Sc, stride_c, idx);
    float v = residual[idx] + add;
    residual[idx] = v;
    if (cast) cast[idx] = from_f32<TOut>(v);
}

KESTREL_API int kestrel_add_three(float *residual, const float *a, int Sa, long long stride_a, const float *b, int Sb, long long stride_b,
                                  const float *c, int Sc, long long stride_c, void *cast, int cast_dtype, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0 && a && Sa > 0 && (b || Sb == 0) && (c || Sc == 0), "add_three: bad arguments");
    size_t n = (size_t)T * d;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (cast_dtype == KESTREL_F32)
        kestrel_launch(add_three_kernel<float>, dim3(blocks), dim3(256), 0, stream, residual, a, Sa, (size_t)stride_a, b, Sb, (size_t)stride_b, c, Sc, (size_t)stride_c, (float *)cast, n);
    else if (cast_dtype == KESTREL_BF16)
        kestrel_launch(add_three_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, residual, a, Sa, (size_t)stride_a, b, Sb, (size_t)stride_b, c, Sc, (size_t)stride_c, (__nv_bfloat16 *)cast, n);
    else
        return kestrel_fail(-2, "add_three: unknown dtype %d", cast_dtype);
    return kestrel_check_launch("add_three");
}

// ------------------------------------------------------------------------------------------
// x[t, i] *= sigmoid(sum_s g[s, t, col0 + i] + bias[col0 + i]), i < n, in place in the storage type: a gate per element of a
// mixer's output, its logits columns of a product of the mixer's input.  The sigmoid is float32.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void gate_columns_mul_kernel(T *__restrict__ x, const float *__restrict__ g, int S, size_t slice_stride, int ld, int col0,
                                        const float *__restrict__ bias, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t t = idx / n;
    int i = (int)(idx % n);
    float z = sum_slices(g, S, slice_stride, t * ld + col0 + i);
    if (bias) z += bias[col0 + i];
    x[idx] = from_f32<T>(to_f32<T>(x[idx]) * (1.0f / (1.0f + expf(-z))));
}

KESTREL_API int kestrel_gate_columns_mul(void *x, int dtype, const float *g, int S, long long slice_stride, int ld, int col0, const float *bias,
                                         int T, int n, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && n > 0 && S > 0 && col0 >= 0 && col0 + n <= ld, "gate_columns_mul: bad sizes");
    size_t total = (size_t)T * n;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == KESTREL_F32)
        kestrel_launch(gate_columns_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float *)x, g, S, (size_t)slice_stride, ld, col0, bias, n, total);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(gate_columns_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16 *)x, g, S, (size_t)slice_stride, ld, col0, bias, n, total);
    else
        return kestrel_fail(-2, "gate_columns_mul: unknown dtype %d", dtype);
    return kestrel_check_launch("gate_columns_mul");
}

// ------------------------------------------------------------------------------------------
// x[t, :] += row[:] for every token: a learned vector fed into the stream (in front of a pass over a stretch of layers)
// ------------------------------------------------------------------------------------------
__global__ void add_row_kernel(float *__restrict__ x, const float *__restrict__ row, int d, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) x[idx] += row[idx % d];
}

KESTREL_API int kestrel_add_row(float *x, const float *row, int T, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0, "add_row: bad sizes");
    size_t n = (size_t)T * d;
    kestrel_launch(add_row_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, row, d, n);
    return kestrel_check_launch("add_row");
}

// ------------------------------------------------------------------------------------------
// out[t, :] = table[ids[t], :] * scale, float32: an embedding with a constant factor
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_scaled_kernel(const T *__restrict__ table, const int *__restrict__ ids, float *__restrict__ out, int d, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T *row = table + (size_t)ids[t] * d;
    float *o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<T>(row[i]) * scale;
}

KESTREL_API int kestrel_embed_scaled(const void *table, int dtype, const int *ids, float *out, int T, int d, float scale, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0, "embed_scaled: bad sizes T=%d d=%d", T, d);
    if (dtype == KESTREL_F32)
        kestrel_launch(embed_scaled_kernel<float>, dim3(T), dim3(256), 0, stream, (const float *)table, ids, out, d, scale);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(embed_scaled_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16 *)table, ids, out, d, scale);
    else
        return kestrel_fail(-2, "embed_scaled: unknown dtype %d", dtype);
    return kestrel_check_launch("embed_scaled");
}
