// The step between a fused query/key/value product and attention, for mixers whose heads are
// not rotated and whose values may have a size of their own.
//
// The product's columns are [ q: nq*hd | k: nkv*hd | v: nkv*vd | gate: nq ]; the k and v parts are
// absent (`has_kv` = 0) in a layer that attends over another layer's cache, the gate part where
// `gate_out` is null, the q part where `nq` = 0 (keys and values alone, into pages).  Per token:
//   every column gets its entry of `bias` (float32, indexed like the product's columns) if one is given;
//   `qk_norm` = 1: q, k <- x / sqrt(mean(x^2) + eps) per head, times a weight [hd] where one is given;
//   `qk_norm` = 2: the same over the whole q projection (all nq * hd columns at once) and the whole k
//            projection, with weights [nq * hd] and [nkv * hd]; `qk_norm` = 0 leaves them as they are;
//   `v_norm`: v <- v / sqrt(mean(v^2) + eps) per head, no weight (it is cached so);
//   `inv_freq` given: q and k (after their norm) are turned by position - pair j of a head's first `rot` dimensions
//            by the angle position * inv_freq[j] (float32), `rot_mode` 0 pairing dimension j with j + rot / 2, 1 pairing
//            2j with 2j + 1; `rot_scale` multiplies cos and sin; the rest of a head passes unchanged;
//   `q_temp_every` > 0: q (after norm and rotation) times 1 + q_temp_coef * ln(floor((position + 1) / q_temp_every) + 1),
//            a query temperature that grows with the position, in float32;
//   q -> q_out in the storage type; k, v -> the token's slot in its request's pages;
//   gate_out[t, h] = sigmoid(gate column h), float32.
// One warp a head row (the blocks of a token share its head rows out), lanes over the head's
// entries, sums of squares in float32 in a fixed shuffle tree: a token's result does not depend on
// the batch.  For the norm over a whole projection every block first sums the squares of each q and
// k head (a warp a head, as above) into shared memory and adds the heads' sums in ascending order; the
// columns it has summed over the product's slices stay in shared memory for the second pass where they fit.
#include "common.cuh"
#include <math.h>

#define APX_WARPS 4
#define APX_PER_LANE 8          // head sizes up to 256

// A head's columns summed over the product's slices (ascending, from zero: the bits of `sum_slices`), plus the bias;
// the loads of a slice's columns are all in flight at once, so a head costs one round trip a slice.
__device__ __forceinline__ void apx_load_head(float (&x)[APX_PER_LANE], const float *__restrict__ row, int S, size_t slice_stride, int col0,
                                              int n, int lane, const float *__restrict__ bias) {
#pragma unroll
    for (int c = 0; c < APX_PER_LANE; ++c) x[c] = 0.f;
#pragma unroll 4
    for (int s = 0; s < S; ++s) {
        float v[APX_PER_LANE];
#pragma unroll
        for (int c = 0; c < APX_PER_LANE; ++c) {
            const int i = lane + 32 * c;
            v[c] = i < n ? row[(size_t)s * slice_stride + col0 + i] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < APX_PER_LANE; ++c) x[c] += v[c];
    }
    if (bias) {
#pragma unroll
        for (int c = 0; c < APX_PER_LANE; ++c) {
            const int i = lane + 32 * c;
            if (i < n) x[c] += bias[col0 + i];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(APX_WARPS * 32)
attn_prepare_ex_kernel(const float *__restrict__ partial, int S, size_t slice_stride, int ld,
                       const float *__restrict__ q_w, const float *__restrict__ k_w, int qk_norm, float eps,
                       const int *__restrict__ positions, const int *__restrict__ seq_of_token,
                       const int *__restrict__ block_table, int table_stride, int page_size,
                       T *__restrict__ k_cache, T *__restrict__ v_cache, T *__restrict__ q_out, float *__restrict__ gate_out,
                       int nq, int nkv, int hd, int vd, int has_kv, const float *__restrict__ bias, int v_norm, int keep_x,
                       const float *__restrict__ inv_freq, int rot, int rot_mode, float rot_scale, float q_temp_coef, int q_temp_every) {
    extern __shared__ float apx_ss[];              // qk_norm = 2: sum of squares of every q and k head, then (keep_x) their columns
    __shared__ float apx_rot[APX_WARPS][32 * APX_PER_LANE];   // rotate-half pairing: a warp's head, so that a lane reaches its partner
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *row = partial + (size_t)t * ld;
    const int n_heads = nq + (has_kv ? 2 * nkv : 0);
    float mul_q = 1.f, mul_k = 1.f;
    if (qk_norm == 2) {
        const int n_qk = nq + (has_kv ? nkv : 0);
        float *apx_x = apx_ss + nq + nkv;
        for (int r = warp; r < n_qk; r += APX_WARPS) {
            float ss = 0.f, xa[APX_PER_LANE];
            apx_load_head(xa, row, S, slice_stride, r * hd, hd, lane, bias);
#pragma unroll
            for (int c = 0; c < APX_PER_LANE; ++c) {
                const int i = lane + 32 * c;
                if (i < hd) {
                    if (keep_x) apx_x[r * hd + i] = xa[c];
                    ss = fmaf(xa[c], xa[c], ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) apx_ss[r] = ss;
        }
        __syncthreads();
        float tq = 0.f, tk = 0.f;
        for (int r = 0; r < nq; ++r) tq += apx_ss[r];
        for (int r = nq; r < n_qk; ++r) tk += apx_ss[r];
        mul_q = 1.0f / sqrtf(tq / (float)(nq * hd) + eps);
        mul_k = 1.0f / sqrtf(tk / (float)(nkv * hd) + eps);
    }
    size_t slot_row = 0;
    const int pos = positions[t];
    const float q_temp = q_temp_every > 0 ? 1.0f + q_temp_coef * logf((float)((pos + 1) / q_temp_every) + 1.0f) : 1.0f;
    if (has_kv) {
        const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
        slot_row = (size_t)page * nkv * page_size + (pos % page_size);      // + kv head * page_size
    }
    for (int r = blockIdx.y * APX_WARPS + warp; r < n_heads; r += gridDim.y * APX_WARPS) {
        // which part: 0 = q head r, 1 = k head, 2 = v head
        const int kind = r < nq ? 0 : (r < nq + nkv ? 1 : 2);
        const int head = kind == 0 ? r : (kind == 1 ? r - nq : r - nq - nkv);
        const int n = kind == 2 ? vd : hd;
        const int col0 = kind == 0 ? head * hd : (kind == 1 ? nq * hd + head * hd : nq * hd + nkv * hd + head * vd);
        float x[APX_PER_LANE];
        float ss = 0.f;
        if (keep_x && qk_norm == 2 && kind != 2) {                 // summed in the first pass
#pragma unroll
            for (int c = 0; c < APX_PER_LANE; ++c) {
                const int i = lane + 32 * c;
                x[c] = i < n ? apx_ss[nq + nkv + r * hd + i] : 0.f;
            }
        } else {
            apx_load_head(x, row, S, slice_stride, col0, n, lane, bias);
        }
#pragma unroll
        for (int c = 0; c < APX_PER_LANE; ++c) ss = fmaf(x[c], x[c], ss);
        float mul = 1.f;
        const float *w = nullptr;
        const float after = kind == 0 ? q_temp : 1.0f;
        if (kind != 2 && qk_norm == 1) {
            ss = warp_sum(ss);
            mul = 1.0f / sqrtf(ss / (float)n + eps);
            w = kind == 0 ? q_w : k_w;
        } else if (kind != 2 && qk_norm == 2) {
            mul = kind == 0 ? mul_q : mul_k;
            w = (kind == 0 ? q_w : k_w) + (size_t)head * hd;       // a weight per column of the projection
        } else if (kind == 2 && v_norm) {
            ss = warp_sum(ss);
            mul = 1.0f / sqrtf(ss / (float)n + eps);
        }
        T *dst = kind == 0 ? q_out + ((size_t)t * nq + head) * hd
                           : (kind == 1 ? k_cache + (slot_row + (size_t)head * page_size) * hd
                                        : v_cache + (slot_row + (size_t)head * page_size) * vd);
#pragma unroll
        for (int c = 0; c < APX_PER_LANE; ++c) {
            const int i = lane + 32 * c;
            x[c] = i < n ? (w ? x[c] * mul * w[i] : x[c] * mul) : 0.f;
        }
        if (inv_freq && kind != 2) {                // the branch is the same for the whole warp
            const int half = rot / 2;
            if (rot_mode == 0) {
#pragma unroll
                for (int c = 0; c < APX_PER_LANE; ++c) apx_rot[warp][lane + 32 * c] = x[c];
                __syncwarp();
            }
#pragma unroll
            for (int c = 0; c < APX_PER_LANE; ++c) {
                const int i = lane + 32 * c;
                // interleaved pairs sit in neighbouring lanes; every lane takes part in the exchange
                const float other = rot_mode == 0 ? apx_rot[warp][i < half ? min(i + half, 32 * APX_PER_LANE - 1) : max(i - half, 0)]
                                                  : __shfl_xor_sync(0xffffffffu, x[c], 1);
                if (i < rot) {
                    const bool first = rot_mode == 0 ? i < half : (i & 1) == 0;
                    const int j = rot_mode == 0 ? (i < half ? i : i - half) : i >> 1;
                    float sn, cs;
                    sincosf((float)pos * inv_freq[j], &sn, &cs);
                    sn *= rot_scale;
                    cs *= rot_scale;
                    x[c] = first ? x[c] * cs - other * sn : x[c] * cs + other * sn;
                }
            }
            if (rot_mode == 0) __syncwarp();        // the next head of this warp writes the same rows
        }
#pragma unroll
        for (int c = 0; c < APX_PER_LANE; ++c) {
            const int i = lane + 32 * c;
            if (i < n) dst[i] = from_f32<T>(q_temp_every > 0 ? x[c] * after : x[c]);
        }
    }
    if (gate_out && blockIdx.y == 0) {
        const int col0 = nq * hd + (has_kv ? nkv * (hd + vd) : 0);
        for (int h = threadIdx.x; h < nq; h += APX_WARPS * 32) {
            float z = sum_slices(row, S, slice_stride, col0 + h);
            if (bias) z += bias[col0 + h];
            gate_out[(size_t)t * nq + h] = 1.0f / (1.0f + expf(-z));
        }
    }
}

KESTREL_API int kestrel_attn_prepare_normed(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *q_norm_w,
                                            const float *k_norm_w, int qk_norm, int v_norm, float norm_eps, const int *positions,
                                            const int *seq_of_token, const int *block_table, int table_stride, int page_size,
                                            void *k_cache, void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq,
                                            int nkv, int hd, int vd, int has_kv, cudaStream_t stream) {
    return kestrel_attn_prepare_rotated(partial, S, slice_stride, ld, bias, q_norm_w, k_norm_w, qk_norm, v_norm, norm_eps, nullptr, 0, 0, 1.f,
                                        positions, seq_of_token, block_table, table_stride, page_size, k_cache, v_cache, q_out, gate_out, dtype,
                                        T, nq, nkv, hd, vd, has_kv, stream);
}

KESTREL_API int kestrel_attn_prepare_rotated(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *q_norm_w,
                                             const float *k_norm_w, int qk_norm, int v_norm, float norm_eps, const float *inv_freq, int rot,
                                             int rot_mode, float rot_scale, const int *positions, const int *seq_of_token,
                                             const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache,
                                             void *q_out, float *gate_out, int dtype, int T, int nq, int nkv, int hd, int vd, int has_kv,
                                             cudaStream_t stream) {
    return kestrel_attn_prepare_tempered(partial, S, slice_stride, ld, bias, q_norm_w, k_norm_w, qk_norm, v_norm, norm_eps, inv_freq, rot, rot_mode,
                                         rot_scale, 0.f, 0, positions, seq_of_token, block_table, table_stride, page_size, k_cache, v_cache, q_out,
                                         gate_out, dtype, T, nq, nkv, hd, vd, has_kv, stream);
}

// the same with a query temperature: q times 1 + q_temp_coef * ln(floor((position + 1) / q_temp_every) + 1); q_temp_every = 0: none
KESTREL_API int kestrel_attn_prepare_tempered(const float *partial, int S, long long slice_stride, int ld, const float *bias, const float *q_norm_w,
                                              const float *k_norm_w, int qk_norm, int v_norm, float norm_eps, const float *inv_freq, int rot,
                                              int rot_mode, float rot_scale, float q_temp_coef, int q_temp_every, const int *positions,
                                              const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache,
                                              void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq, int nkv, int hd, int vd,
                                              int has_kv, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(q_temp_every >= 0, "attn_prepare_ex: a query temperature every %d positions", q_temp_every);
    KESTREL_REQUIRE(!inv_freq || (rot > 0 && rot % 2 == 0 && rot <= hd && (rot_mode == 0 || rot_mode == 1)),
                    "attn_prepare_ex: %d rotated dimensions of a head of %d (mode %d)", rot, hd, rot_mode);
    KESTREL_REQUIRE(qk_norm >= 0 && qk_norm <= 2, "attn_prepare_ex: qk_norm %d is none of 0, 1, 2", qk_norm);
    KESTREL_REQUIRE(qk_norm != 2 || (q_norm_w && (k_norm_w || !has_kv)), "attn_prepare_ex: the norm over a whole projection needs its weights");
    size_t smem = qk_norm == 2 ? (size_t)(nq + nkv) * sizeof(float) : 0;
    KESTREL_REQUIRE(smem <= 40000, "attn_prepare_ex: %d heads exceed the shared memory of the norm over a whole projection", nq + nkv);
    const int keep_x = qk_norm == 2 && smem + (size_t)(nq + nkv) * hd * sizeof(float) <= 44 * 1024;
    if (keep_x) smem += (size_t)(nq + nkv) * hd * sizeof(float);
    KESTREL_REQUIRE(T > 0 && nq >= 0 && nkv > 0 && hd > 0 && vd > 0 && S > 0 && (nq > 0 || has_kv), "attn_prepare_ex: bad sizes");
    KESTREL_REQUIRE(hd <= 32 * APX_PER_LANE && vd <= 32 * APX_PER_LANE, "attn_prepare_ex: head size %d / %d exceeds %d", hd, vd, 32 * APX_PER_LANE);
    const int need = nq * hd + (has_kv ? nkv * (hd + vd) : 0) + (gate_out ? nq : 0);
    KESTREL_REQUIRE(ld >= need, "attn_prepare_ex: the product has %d columns, the heads need %d", ld, need);
    // few tokens: a block per four head rows, so that the step's few tokens still fill the device
    const int n_heads = nq + (has_kv ? 2 * nkv : 0);
    const int by = T >= 512 ? 1 : (n_heads + APX_WARPS - 1) / APX_WARPS;
    if (dtype == KESTREL_F32)
        kestrel_launch(attn_prepare_ex_kernel<float>, dim3(T, by), dim3(APX_WARPS * 32), smem, stream, partial, S, (size_t)slice_stride, ld, q_norm_w, k_norm_w, qk_norm, norm_eps,
                       positions, seq_of_token, block_table, table_stride, page_size, (float *)k_cache, (float *)v_cache, (float *)q_out, gate_out, nq, nkv, hd, vd, has_kv, bias, v_norm, keep_x, inv_freq, rot, rot_mode, rot_scale, q_temp_coef, q_temp_every);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(attn_prepare_ex_kernel<__nv_bfloat16>, dim3(T, by), dim3(APX_WARPS * 32), smem, stream, partial, S, (size_t)slice_stride, ld, q_norm_w, k_norm_w, qk_norm, norm_eps,
                       positions, seq_of_token, block_table, table_stride, page_size, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, (__nv_bfloat16 *)q_out, gate_out, nq, nkv,
                       hd, vd, has_kv, bias, v_norm, keep_x, inv_freq, rot, rot_mode, rot_scale, q_temp_coef, q_temp_every);
    else
        return kestrel_fail(-2, "attn_prepare_ex: unknown dtype %d", dtype);
    return kestrel_check_launch("attn_prepare_ex");
}

KESTREL_API int kestrel_attn_prepare_ex(const float *partial, int S, long long slice_stride, int ld, const float *q_norm_w,
                                        const float *k_norm_w, int qk_norm, float norm_eps, const int *positions,
                                        const int *seq_of_token, const int *block_table, int table_stride, int page_size,
                                        void *k_cache, void *v_cache, void *q_out, float *gate_out, int dtype, int T, int nq,
                                        int nkv, int hd, int vd, int has_kv, cudaStream_t stream) {
    return kestrel_attn_prepare_normed(partial, S, slice_stride, ld, nullptr, q_norm_w, k_norm_w, qk_norm ? 1 : 0, 0, norm_eps, positions,
                                       seq_of_token, block_table, table_stride, page_size, k_cache, v_cache, q_out, gate_out, dtype, T,
                                       nq, nkv, hd, vd, has_kv, stream);
}
