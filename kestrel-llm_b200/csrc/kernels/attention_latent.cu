// Kernels of attention whose keys and values are expanded from one cached latent vector a token.
//
// Such a layer projects its input to a query latent (q_rank numbers), a key/value latent (kv_rank
// numbers) and a gate logit per head in ONE fused product; both latents are RMS-normed with a weight;
// only the key/value latent c is cached.  With per-head expansions k_h = Uk_h c and v_h = Uv_h c,
//
//   q_h . k_h = (Uk_h^T q_h) . c          sum_j p_j v_hj = Uv_h (sum_j p_j c_j)
//
// so attention runs over the cached latents themselves, as one shared key/value head of size
// kv_rank for all query heads, between two head-wise products: queries into the latent space before
// it, the mixed latents out of it afterwards.
//
//   latent_prepare   columns [q latent | kv latent | gate] of the fused product -> normed query latent
//                    in the storage type, normed kv latent into the token's cache slot, sigmoid of the
//                    gate columns as float32.  One block a token; sums of squares in float32, lanes
//                    strided over the columns, a fixed tree over lanes and warps.
//   head_gemm        out[t, h, :] = x[t, h, :] times head h's own matrix, for all heads in one launch.
//                    The matrices are slices of one checkpoint tensor in either orientation:
//                    `w_kn` = 0: rows [h N, (h + 1) N) of w [H N, K]  (out = x w_h^T, as a projection is stored);
//                    `w_kn` = 1: rows [h K, (h + 1) K) of w [H K, N]  (out = x w_h: the transposed use of an
//                    expansion, without a transposed copy of the weights).
//                    float32 accumulation in ascending k per output element: a token's result does not
//                    depend on the batch.  bfloat16 operands of enough tokens take mma.sync tiles.
#include "common.cuh"
#include "mma_sync.cuh"
#include <math.h>

#define LP_THREADS 128          // threads a token of steps with many tokens; few tokens take LP_THREADS_FEW
#define LP_THREADS_FEW 512

// sum over the block in a fixed order: lanes by the shuffle tree, warps in ascending order
template <int THREADS>
__device__ __forceinline__ float lp_block_sum(float v, float *scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                       // the scratch may still be read from the call before
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) t += scratch[w];
    return t;
}

// The order of a sum of squares depends on THREADS.  float32 always runs LP_THREADS (a token's bits do not depend on
// the step it is in); bfloat16 steps of few tokens take more threads a token, and differ by the rounding of that sum.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
latent_prepare_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld, const float *__restrict__ q_w,
                      const float *__restrict__ kv_w, float eps, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
                      const int *__restrict__ block_table, int table_stride, int page_size, T *__restrict__ latent_cache,
                      T *__restrict__ q_out, float *__restrict__ gate_out, int q_rank, int kv_rank, int n_gate, T *__restrict__ kv_out,
                      int rot_cols, const float *__restrict__ inv_freq, int rot, int rot_mode, float rot_scale) {
    __shared__ float scratch[THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const float *row = partial + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < q_rank; i += THREADS) {
        const float v = sum_slices(row, S, slice_stride, i);
        sq = fmaf(v, v, sq);
    }
    for (int i = tid; i < kv_rank; i += THREADS) {
        const float v = sum_slices(row, S, slice_stride, q_rank + i);
        sk = fmaf(v, v, sk);
    }
    const float mul_q = 1.0f / sqrtf(lp_block_sum<THREADS>(sq, scratch) / (float)q_rank + eps);
    const float mul_k = 1.0f / sqrtf(lp_block_sum<THREADS>(sk, scratch) / (float)kv_rank + eps);
    T *qrow = q_out + (size_t)t * q_rank;
    for (int i = tid; i < q_rank; i += THREADS) qrow[i] = from_f32<T>(sum_slices(row, S, slice_stride, i) * mul_q * q_w[i]);
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
    T *crow = latent_cache + ((size_t)page * page_size + (pos % page_size)) * (kv_rank + rot_cols);
    T *orow = kv_out ? kv_out + (size_t)t * kv_rank : nullptr;      // the step's latents as rows too, for callers that expand them
    for (int i = tid; i < kv_rank; i += THREADS) {
        const T c = from_f32<T>(sum_slices(row, S, slice_stride, q_rank + i) * mul_k * kv_w[i]);
        crow[i] = c;
        if (orow) orow[i] = c;
    }
    // the key part that all heads share: columns behind the latent, not normed, turned by position, cached behind the latent
    const int c0 = q_rank + kv_rank, half = rot / 2;
    for (int j = tid; j < half; j += THREADS) {
        const int ia = rot_mode == 0 ? j : 2 * j, ib = rot_mode == 0 ? j + half : 2 * j + 1;
        const float a = sum_slices(row, S, slice_stride, c0 + ia), b = sum_slices(row, S, slice_stride, c0 + ib);
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        sn *= rot_scale;
        cs *= rot_scale;
        crow[kv_rank + ia] = from_f32<T>(a * cs - b * sn);
        crow[kv_rank + ib] = from_f32<T>(b * cs + a * sn);
    }
    for (int i = rot + tid; i < rot_cols; i += THREADS) crow[kv_rank + i] = from_f32<T>(sum_slices(row, S, slice_stride, c0 + i));
    for (int h = tid; h < n_gate; h += THREADS)
        gate_out[(size_t)t * n_gate + h] = 1.0f / (1.0f + expf(-sum_slices(row, S, slice_stride, c0 + rot_cols + h)));
}

// q_lat[t, h, col0 + i] = the rotated part of head h's query: columns [d, d + rot_cols) of q[t, h, :], the first `rot` of
// them turned by position (pairing, frequencies and scale as in the prepare kernels), the rest as they are
template <typename T>
__global__ void __launch_bounds__(128)
latent_rotate_queries_kernel(const T *__restrict__ q, int ldq, int head_stride, int d, T *__restrict__ q_lat, int ldo, int out_head_stride, int col0,
                             const int *__restrict__ positions, int H, int rot_cols, const float *__restrict__ inv_freq, int rot, int rot_mode,
                             float rot_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, half = rot / 2;
    const float pos = (float)positions[t];
    for (int idx = threadIdx.x; idx < H * half; idx += 128) {
        const int h = idx / half, j = idx % half;
        const int ia = rot_mode == 0 ? j : 2 * j, ib = rot_mode == 0 ? j + half : 2 * j + 1;
        const T *src = q + (size_t)t * ldq + (size_t)h * head_stride + d;
        T *dst = q_lat + (size_t)t * ldo + (size_t)h * out_head_stride + col0;
        const float a = to_f32<T>(src[ia]), b = to_f32<T>(src[ib]);
        float sn, cs;
        sincosf(pos * inv_freq[j], &sn, &cs);
        sn *= rot_scale;
        cs *= rot_scale;
        dst[ia] = from_f32<T>(a * cs - b * sn);
        dst[ib] = from_f32<T>(b * cs + a * sn);
    }
    const int rest = rot_cols - rot;
    for (int idx = threadIdx.x; idx < H * rest; idx += 128) {
        const int h = idx / rest, i = rot + idx % rest;
        q_lat[(size_t)t * ldo + (size_t)h * out_head_stride + col0 + i] = q[(size_t)t * ldq + (size_t)h * head_stride + d + i];
    }
}

KESTREL_API int kestrel_latent_rotate_queries(const void *q, int ldq, int head_stride, int d, void *q_lat, int ldo, int out_head_stride, int col0,
                                              const int *positions, int dtype, int T, int H, int rot_cols, const float *inv_freq, int rot,
                                              int rot_mode, float rot_scale, cudaStream_t stream) {
    if (T == 0 || rot_cols == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && rot_cols > 0 && rot >= 0 && rot % 2 == 0 && rot <= rot_cols && (rot == 0 || inv_freq) && (rot_mode == 0 || rot_mode == 1) &&
                    head_stride >= d + rot_cols && out_head_stride >= col0 + rot_cols, "latent_rotate_queries: bad sizes");
    if (dtype == KESTREL_F32)
        kestrel_launch(latent_rotate_queries_kernel<float>, dim3(T), dim3(128), 0, stream, (const float *)q, ldq, head_stride, d, (float *)q_lat, ldo, out_head_stride,
                       col0, positions, H, rot_cols, inv_freq, rot, rot_mode, rot_scale);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(latent_rotate_queries_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16 *)q, ldq, head_stride, d, (__nv_bfloat16 *)q_lat,
                       ldo, out_head_stride, col0, positions, H, rot_cols, inv_freq, rot, rot_mode, rot_scale);
    else
        return kestrel_fail(-2, "latent_rotate_queries: unknown dtype %d", dtype);
    return kestrel_check_launch("latent_rotate_queries");
}

KESTREL_API int kestrel_latent_prepare(const float *partial, int S, long long slice_stride, int ld, const float *q_norm_w, const float *kv_norm_w,
                                       float norm_eps, const int *positions, const int *seq_of_token, const int *block_table, int table_stride,
                                       int page_size, void *latent_cache, void *q_out, float *gate_out, void *kv_out, int dtype, int T, int q_rank,
                                       int kv_rank, int n_gate, cudaStream_t stream) {
    return kestrel_latent_prepare_rotated(partial, S, slice_stride, ld, q_norm_w, kv_norm_w, norm_eps, positions, seq_of_token, block_table, table_stride,
                                          page_size, latent_cache, q_out, gate_out, kv_out, dtype, T, q_rank, kv_rank, n_gate, 0, nullptr, 0, 0, 1.f, stream);
}

// the same with `rot_cols` more columns between the kv latent and the gates: a key part that all heads share, not normed,
// its first `rot` dimensions turned by position; a cache row is then [latent: kv_rank | key part: rot_cols]
KESTREL_API int kestrel_latent_prepare_rotated(const float *partial, int S, long long slice_stride, int ld, const float *q_norm_w, const float *kv_norm_w,
                                               float norm_eps, const int *positions, const int *seq_of_token, const int *block_table, int table_stride,
                                               int page_size, void *latent_cache, void *q_out, float *gate_out, void *kv_out, int dtype, int T, int q_rank,
                                               int kv_rank, int n_gate, int rot_cols, const float *inv_freq, int rot, int rot_mode, float rot_scale,
                                               cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(rot_cols >= 0 && rot >= 0 && rot % 2 == 0 && rot <= rot_cols && (rot == 0 || inv_freq) && (rot_mode == 0 || rot_mode == 1),
                    "latent_prepare: %d rotated dimensions of a key part of %d", rot, rot_cols);
    KESTREL_REQUIRE(T > 0 && S > 0 && q_rank > 0 && kv_rank > 0 && n_gate >= 0 && (n_gate == 0 || gate_out), "latent_prepare: bad sizes");
    KESTREL_REQUIRE(ld >= q_rank + kv_rank + rot_cols + n_gate, "latent_prepare: the product has %d columns, the latents and gates need %d", ld, q_rank + kv_rank + rot_cols + n_gate);
    if (dtype == KESTREL_F32)
        kestrel_launch(latent_prepare_kernel<float, LP_THREADS>, dim3(T), dim3(LP_THREADS), 0, stream, partial, S, (size_t)slice_stride, ld, q_norm_w, kv_norm_w, norm_eps,
                       positions, seq_of_token, block_table, table_stride, page_size, (float *)latent_cache, (float *)q_out, gate_out, q_rank, kv_rank, n_gate, (float *)kv_out, rot_cols, inv_freq, rot, rot_mode, rot_scale);
    else if (dtype == KESTREL_BF16 && T <= 64)
        kestrel_launch(latent_prepare_kernel<__nv_bfloat16, LP_THREADS_FEW>, dim3(T), dim3(LP_THREADS_FEW), 0, stream, partial, S, (size_t)slice_stride, ld, q_norm_w, kv_norm_w, norm_eps,
                       positions, seq_of_token, block_table, table_stride, page_size, (__nv_bfloat16 *)latent_cache, (__nv_bfloat16 *)q_out, gate_out, q_rank, kv_rank,
                       n_gate, (__nv_bfloat16 *)kv_out, rot_cols, inv_freq, rot, rot_mode, rot_scale);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(latent_prepare_kernel<__nv_bfloat16, LP_THREADS>, dim3(T), dim3(LP_THREADS), 0, stream, partial, S, (size_t)slice_stride, ld, q_norm_w, kv_norm_w, norm_eps,
                       positions, seq_of_token, block_table, table_stride, page_size, (__nv_bfloat16 *)latent_cache, (__nv_bfloat16 *)q_out, gate_out, q_rank, kv_rank,
                       n_gate, (__nv_bfloat16 *)kv_out, rot_cols, inv_freq, rot, rot_mode, rot_scale);
    else
        return kestrel_fail(-2, "latent_prepare: unknown dtype %d", dtype);
    return kestrel_check_launch("latent_prepare");
}

// x[t, h, :] *= gate[t, h]: a gate per head on rows of heads, in place
template <typename T>
__global__ void __launch_bounds__(256)
head_scale_kernel(T *__restrict__ x, const float *__restrict__ gate, int heads, int d, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256)
        x[i] = from_f32<T>(to_f32<T>(x[i]) * gate[i / d]);          // i / d = t * heads + h
}

KESTREL_API int kestrel_head_scale(void *x, const float *gate, int dtype, int T, int heads, int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && heads > 0 && d > 0, "head_scale: bad sizes");
    const size_t n = (size_t)T * heads * d;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (dtype == KESTREL_F32) kestrel_launch(head_scale_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float *)x, gate, heads, d, n);
    else if (dtype == KESTREL_BF16) kestrel_launch(head_scale_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16 *)x, gate, heads, d, n);
    else return kestrel_fail(-2, "head_scale: unknown dtype %d", dtype);
    return kestrel_check_launch("head_scale");
}

// ---- head-wise products ------------------------------------------------------------------------

#define HG_TOK 8            // tokens of a block of the plain kernel
#define HG_THREADS 128      // output columns of a block of the plain kernel

template <typename T>
__global__ void __launch_bounds__(HG_THREADS)
head_gemm_plain_kernel(const T *__restrict__ x, int ldx, int hsx, const T *__restrict__ w, int ldw, int w_kn, void *__restrict__ out_, int ldo, int hso,
                       int out_f32, int Tn, int N, int K) {
    extern __shared__ float hg_x[];          // [HG_TOK][K]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * HG_TOK, h = blockIdx.y, n = blockIdx.z * HG_THREADS + threadIdx.x;
    const int rows = min(HG_TOK, Tn - t0);
    for (int idx = threadIdx.x; idx < rows * K; idx += HG_THREADS) {
        const int r = idx / K, k = idx % K;
        hg_x[idx] = to_f32<T>(x[(size_t)(t0 + r) * ldx + (size_t)h * hsx + k]);
    }
    __syncthreads();
    if (n >= N) return;
    float acc[HG_TOK];
#pragma unroll
    for (int r = 0; r < HG_TOK; ++r) acc[r] = 0.f;
    const T *wp = w_kn ? w + (size_t)h * K * ldw + n : w + ((size_t)h * N + n) * ldw;
    const size_t step = w_kn ? ldw : 1;
    for (int k = 0; k < K; ++k) {
        const float wv = to_f32<T>(wp[(size_t)k * step]);
#pragma unroll
        for (int r = 0; r < HG_TOK; ++r) acc[r] = fmaf(hg_x[r * K + k], wv, acc[r]);
    }
    for (int r = 0; r < rows; ++r) {
        const size_t at = (size_t)(t0 + r) * ldo + (size_t)h * hso + n;
        if (out_f32) ((float *)out_)[at] = acc[r];
        else ((T *)out_)[at] = from_f32<T>(acc[r]);
    }
}

// bfloat16 on the tensor cores: a CTA of four warps takes 64 tokens x 64 output columns of one head;
// K goes by in chunks of 32 through two cp.async stages.  The weight tile is kept as the checkpoint
// has it - [n][k] rows for `w_kn` = 0, [k][n] rows for `w_kn` = 1 - and ldmatrix (transposing for the
// second) makes the B fragments of either.
#define HM_BM 64
#define HM_BN 64
#define HM_BK 32

__device__ __forceinline__ void hm_cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}

template <int W_KN, typename TO>
__global__ void __launch_bounds__(128)
head_gemm_mma_kernel(const __nv_bfloat16 *__restrict__ x, int ldx, int hsx, const __nv_bfloat16 *__restrict__ w, int ldw,
                     TO *__restrict__ out, int ldo, int hso, int Tn, int N, int K) {
    constexpr int LDA = HM_BK + 8, LDB = W_KN ? HM_BN + 8 : HM_BK + 8;
    constexpr int B_ROWS = W_KN ? HM_BK : HM_BN;
    __shared__ __align__(16) __nv_bfloat16 As[2][HM_BM * LDA];
    __shared__ __align__(16) __nv_bfloat16 Bs[2][B_ROWS * LDB];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = blockIdx.x * HM_BM, h = blockIdx.y, n0 = blockIdx.z * HM_BN;
    const __nv_bfloat16 *xh = x + (size_t)h * hsx;
    const __nv_bfloat16 *wh = W_KN ? w + (size_t)h * K * ldw : w + (size_t)h * N * ldw;

    auto load = [&](int kc, int st) {
        const int k0 = kc * HM_BK;
        for (int idx = tid; idx < HM_BM * (HM_BK / 8); idx += 128) {
            const int r = idx / (HM_BK / 8), c = idx % (HM_BK / 8);
            const bool ok = t0 + r < Tn && k0 + c * 8 < K;
            hm_cp_async16((uint32_t)__cvta_generic_to_shared(&As[st][r * LDA + c * 8]), ok ? xh + (size_t)(t0 + r) * ldx + k0 + c * 8 : xh, ok);
        }
        if (W_KN) {
            for (int idx = tid; idx < HM_BK * (HM_BN / 8); idx += 128) {
                const int r = idx / (HM_BN / 8), c = idx % (HM_BN / 8);
                const bool ok = k0 + r < K && n0 + c * 8 < N;
                hm_cp_async16((uint32_t)__cvta_generic_to_shared(&Bs[st][r * LDB + c * 8]), ok ? wh + (size_t)(k0 + r) * ldw + n0 + c * 8 : wh, ok);
            }
        } else {
            for (int idx = tid; idx < HM_BN * (HM_BK / 8); idx += 128) {
                const int r = idx / (HM_BK / 8), c = idx % (HM_BK / 8);
                const bool ok = n0 + r < N && k0 + c * 8 < K;
                hm_cp_async16((uint32_t)__cvta_generic_to_shared(&Bs[st][r * LDB + c * 8]), ok ? wh + (size_t)(n0 + r) * ldw + k0 + c * 8 : wh, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[HM_BN / 8][4];
#pragma unroll
    for (int j = 0; j < HM_BN / 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
    const int a_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_k = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_k = ((lane >> 3) & 1) * 8;           // [n][k] tiles
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;         // [k][n] tiles, transposed on load
    const int chunks = (K + HM_BK - 1) / HM_BK;
    load(0, 0);
    for (int kc = 0; kc < chunks; ++kc) {
        const int st = kc & 1;
        if (kc + 1 < chunks) {
            load(kc + 1, st ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HM_BK / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4((uint32_t)__cvta_generic_to_shared(&As[st][a_row * LDA + kk * 16 + a_k]), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int jp = 0; jp < HM_BN / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                if (W_KN) {
                    ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(&Bs[st][(kk * 16 + v_row) * LDB + jp * 16 + v_col]), b0, b1, b2, b3);
                } else {
                    ldmatrix_x4((uint32_t)__cvta_generic_to_shared(&Bs[st][(jp * 16 + b_row) * LDB + kk * 16 + b_k]), b0, b1, b2, b3);
                }
                mma_bf16(acc[2 * jp], a, b0, b1);
                mma_bf16(acc[2 * jp + 1], a, b2, b3);
            }
        }
        __syncthreads();                   // the stage is refilled by the load after next
    }
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int t = t0 + warp * 16 + g + 8 * h2;
        if (t >= Tn) continue;
        TO *dst = out + (size_t)t * ldo + (size_t)h * hso + n0;
#pragma unroll
        for (int j = 0; j < HM_BN / 8; ++j) {
            const int col = j * 8 + 2 * tq;
            if (n0 + col < N) {
                if (sizeof(TO) == 4) *reinterpret_cast<float2 *>(dst + col) = make_float2(acc[j][2 * h2], acc[j][2 * h2 + 1]);
                else *reinterpret_cast<uint32_t *>(dst + col) = pack_bf16(acc[j][2 * h2], acc[j][2 * h2 + 1]);
            }
        }
    }
}

static int g_head_gemm_plain = 0;
KESTREL_API void kestrel_head_gemm_set_plain(int on) { g_head_gemm_plain = on; }

KESTREL_API int kestrel_head_gemm(const void *x, int ldx, const void *w, int ldw, int w_kn,
                                  void *out, int ldo, int dtype, int T, int H, int N, int K, cudaStream_t stream) {
    return kestrel_head_gemm_strided(x, ldx, K, w, ldw, w_kn, out, ldo, N, 0, dtype, T, H, N, K, stream);
}

// the same with head h's input at x[t, h hsx ..] and its output at out[t, h hso ..] (a head's columns may lie among others),
// and the output as float32 if `out_f32`
KESTREL_API int kestrel_head_gemm_strided(const void *x, int ldx, int hsx, const void *w, int ldw, int w_kn, void *out, int ldo, int hso, int out_f32,
                                          int dtype, int T, int H, int N, int K, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && H > 0 && N > 0 && K > 0 && H <= 65535 && hsx >= K && hso >= N, "head_gemm: bad sizes");
    KESTREL_REQUIRE(ldx >= (H - 1) * hsx + K && ldo >= (H - 1) * hso + N && ldw >= (w_kn ? N : K), "head_gemm: a row stride is shorter than its row");
    if (dtype == KESTREL_BF16 && !g_head_gemm_plain && K % 8 == 0 && N % 8 == 0 && ldx % 8 == 0 && hsx % 8 == 0 && ldw % 8 == 0 && ldo % 2 == 0 && hso % 2 == 0 &&
        ((uintptr_t)x | (uintptr_t)w) % 16 == 0 && (uintptr_t)out % 8 == 0) {
        dim3 grid((T + HM_BM - 1) / HM_BM, H, (N + HM_BN - 1) / HM_BN);
        KESTREL_REQUIRE(grid.z <= 65535, "head_gemm: %d output columns exceed the grid", N);
#define HG_LAUNCH(KN, TO) kestrel_launch(head_gemm_mma_kernel<KN, TO>, grid, dim3(128), 0, stream, (const __nv_bfloat16 *)x, ldx, hsx, (const __nv_bfloat16 *)w, ldw, (TO *)out, ldo, hso, T, N, K)
        if (w_kn) { if (out_f32) HG_LAUNCH(1, float); else HG_LAUNCH(1, __nv_bfloat16); }
        else { if (out_f32) HG_LAUNCH(0, float); else HG_LAUNCH(0, __nv_bfloat16); }
#undef HG_LAUNCH
        return kestrel_check_launch("head_gemm_mma");
    }
    const size_t smem = (size_t)HG_TOK * K * sizeof(float);
    KESTREL_REQUIRE(smem <= 48 * 1024, "head_gemm: an inner size of %d exceeds the plain kernel's shared memory", K);
    dim3 grid((T + HG_TOK - 1) / HG_TOK, H, (N + HG_THREADS - 1) / HG_THREADS);
    KESTREL_REQUIRE(grid.z <= 65535, "head_gemm: %d output columns exceed the grid", N);
    if (dtype == KESTREL_F32)
        kestrel_launch(head_gemm_plain_kernel<float>, grid, dim3(HG_THREADS), smem, stream, (const float *)x, ldx, hsx, (const float *)w, ldw, w_kn,
                       out, ldo, hso, 1, T, N, K);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(head_gemm_plain_kernel<__nv_bfloat16>, grid, dim3(HG_THREADS), smem, stream, (const __nv_bfloat16 *)x, ldx, hsx,
                       (const __nv_bfloat16 *)w, ldw, w_kn, out, ldo, hso, out_f32, T, N, K);
    else
        return kestrel_fail(-2, "head_gemm: unknown dtype %d", dtype);
    return kestrel_check_launch("head_gemm");
}
