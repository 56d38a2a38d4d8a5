// Routed feed-forward: a router picks `top` of E experts per token, the tokens are grouped by
// expert on the device (no value of the step is read on the host), two grouped products run the
// chosen experts, and the results are summed per token in the order of the router's choice.
//
//   route      z = sum of the router product's slices + bias (float32); the `top` largest
//              (lowest index first among equals), weights = softmax over the chosen logits
//   group      pairs (token, choice) sorted by expert: offsets per expert, row <-> pair maps and
//              a list of row tiles that never span two experts
//   gate_up    per tile: g = Wg[e] x, u = Wu[e] x for the rows' tokens (gathered), then the
//              expert's activation  y = min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)
//   down       per tile: W_down[e] y, times the pair's routing weight, float32
//   combine    out[t] = sum over the token's choices, in the order of choice
//
// The plain products (float32, and bfloat16 sizes the tensor-core kernel refuses) accumulate by
// FMA in ascending k per output element; the bfloat16 products run on the tensor cores
// (mma.sync.m16n8k16, float32 accumulators), where an output element is a sum over k in the
// hardware's fixed order.  Either way a pair's result depends neither on the tile it falls into
// nor on the other rows: the feed-forward of a token is the same bits however the step is
// batched or cut.
#include "common.cuh"
#include "mma_sync.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
moe_route_kernel(const float *__restrict__ z_part, int S, size_t slice_stride, const float *__restrict__ bias, int E, int top,
                 int *__restrict__ ids, float *__restrict__ weights) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float z[];
    const int t = blockIdx.x, lane = threadIdx.x;
    for (int e = lane; e < E; e += 32) {
        z[e] = sum_slices(z_part, S, slice_stride, (size_t)t * E + e) + (bias ? bias[e] : 0.f);
    }
    __syncwarp();
    float zmax = 0.f, denom = 0.f, mine = 0.f;       // lane k keeps the k-th chosen logit
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (z[e] > best) { best = z[e]; arg = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (k == 0) zmax = best;
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            z[arg] = -INFINITY;
        }
        if (lane == k % 32) mine = best;              // top <= 32
        __syncwarp();
    }
    const float p = lane < top ? expf(mine - zmax) : 0.f;
    denom = p;
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    if (lane < top) weights[(size_t)t * top + lane] = p / denom;
}

KESTREL_API int kestrel_moe_route(const float *z_part, int S, long long slice_stride, const float *bias, int *ids, float *weights, int T,
                                  int E, int top, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && E > 0 && top > 0 && top <= E && top <= 32 && S > 0, "moe_route: bad sizes E=%d top=%d", E, top);
    KESTREL_REQUIRE(E <= 8192, "moe_route: %d experts exceed 8192", E);
    kestrel_launch(moe_route_kernel, dim3(T), dim3(32), (size_t)E * sizeof(float), stream, z_part, S, (size_t)slice_stride, bias, E, top, ids, weights);
    return kestrel_check_launch("moe_route");
}

// A router of another kind: scores s = sigmoid(z); the experts are CHOSEN by s + correction[e] (a number per expert that
// steers the load), but weighted by s alone.  The experts form `n_groups` equal groups of neighbours; a group's score is
// the sum of its two largest choice scores (its only one where a group is one expert), and only experts of the `keep`
// best groups can be chosen.  Weights: the chosen experts' s divided by their sum (+ 1e-20), times `scale`.  Among equal
// scores the lowest index wins.  A warp a token; all float32.
__device__ __forceinline__ void warp_argmax(float &best, int &arg) {
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
}

__global__ void __launch_bounds__(32)
moe_route_sigmoid_kernel(const float *__restrict__ z_part, int S, size_t slice_stride, const float *__restrict__ correction, int E, int top,
                         int n_groups, int keep, float scale, int *__restrict__ ids, float *__restrict__ weights) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float rs[];
    float *s = rs, *choice = rs + E, *gs = rs + 2 * E;          // s [E], choice [E], gs [n_groups]
    const int t = blockIdx.x, lane = threadIdx.x;
    for (int e = lane; e < E; e += 32) {
        const float z = sum_slices(z_part, S, slice_stride, (size_t)t * E + e);
        s[e] = 1.0f / (1.0f + expf(-z));
        choice[e] = s[e] + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;                   // the two largest, a >= b
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = choice[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the groups that stay are marked by +inf; then every expert of another group is closed
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32)
                if (gs[g] != INFINITY && (gs[g] > best || arg == 0x7fffffff)) { best = gs[g]; arg = g; }
            warp_argmax(best, arg);
            if (lane == 0 && arg != 0x7fffffff) gs[arg] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    float mine = 0.f;                                  // lane k keeps the k-th chosen expert's score s
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (choice[e] > best) { best = choice[e]; arg = e; }
        warp_argmax(best, arg);
        if (arg == 0x7fffffff) arg = 0;               // fewer open experts than `top`: never with keep * (E / n_groups) >= top
        if (lane == 0) ids[(size_t)t * top + k] = arg;
        if (lane == k % 32) mine = s[arg];
        __syncwarp();
        if (lane == 0) choice[arg] = -INFINITY;
        __syncwarp();
    }
    float denom = lane < top ? mine : 0.f;
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    if (lane < top) weights[(size_t)t * top + lane] = mine / (denom + 1e-20f) * scale;
}

KESTREL_API int kestrel_moe_route_sigmoid(const float *z_part, int S, long long slice_stride, const float *correction, int n_groups, int keep,
                                          float scale, int *ids, float *weights, int T, int E, int top, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && E > 0 && top > 0 && top <= E && top <= 32 && S > 0, "moe_route_sigmoid: bad sizes E=%d top=%d", E, top);
    KESTREL_REQUIRE(E <= 4096, "moe_route_sigmoid: %d experts exceed 4096", E);
    KESTREL_REQUIRE(n_groups >= 1 && E % n_groups == 0 && keep >= 1 && keep <= n_groups && (long long)keep * (E / n_groups) >= top,
                    "moe_route_sigmoid: %d groups of %d experts, %d kept, %d chosen", n_groups, E, keep, top);
    kestrel_launch(moe_route_sigmoid_kernel, dim3(T), dim3(32), (size_t)(2 * E + n_groups) * sizeof(float), stream, z_part, S, (size_t)slice_stride,
                   correction, E, top, n_groups, keep, scale, ids, weights);
    return kestrel_check_launch("moe_route_sigmoid");
}

// ------------------------------------------------------------------------------------------
// One block groups the P = T * top pairs by expert.
//   offsets [E + 1]; row_pair [P]: pair of sorted row r; pair_row [P]: sorted row of a pair;
//   tile_expert / tile_row0 [ceil(P / rows) + E]; n_tiles [1]
// ------------------------------------------------------------------------------------------
#define MG_THREADS 1024
__global__ void __launch_bounds__(MG_THREADS)
moe_group_kernel(const int *__restrict__ ids, int P, int E, int rows_per_tile, int *__restrict__ offsets, int *__restrict__ row_pair,
                 int *__restrict__ pair_row, int *__restrict__ tile_expert, int *__restrict__ tile_row0, int *__restrict__ n_tiles) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int sh[];
    int *cnt = sh, *off = sh + E;                     // cnt [E], off [E + 1]
    for (int e = threadIdx.x; e < E; e += MG_THREADS) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += MG_THREADS) atomicAdd(&cnt[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = acc;
            for (int r = 0; r < cnt[e]; r += rows_per_tile) {
                tile_expert[nt] = e;
                tile_row0[nt] = acc + r;
                ++nt;
            }
            acc += cnt[e];
        }
        off[E] = acc;
        *n_tiles = nt;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += MG_THREADS) offsets[e] = off[e];
    // a pair's row among its expert's rows: handed out by a counter per expert.  The order of the
    // rows inside an expert is then not fixed, which no result depends on: every row of a grouped
    // product is computed by itself.
    for (int e = threadIdx.x; e < E; e += MG_THREADS) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += MG_THREADS) {
        const int e = ids[p];
        const int r = off[e] + atomicAdd(&cnt[e], 1);
        row_pair[r] = p;
        pair_row[p] = r;
    }
}

KESTREL_API int kestrel_moe_group(const int *ids, int P, int E, int rows_per_tile, int *offsets, int *row_pair, int *pair_row, int *tile_expert,
                                  int *tile_row0, int *n_tiles, cudaStream_t stream) {
    if (P == 0) return 0;
    KESTREL_REQUIRE(P > 0 && E > 0 && E <= 8192 && rows_per_tile > 0, "moe_group: bad sizes");
    kestrel_launch(moe_group_kernel, dim3(1), dim3(MG_THREADS), (size_t)(2 * E + 1) * sizeof(int), stream, ids, P, E, rows_per_tile, offsets, row_pair,
                   pair_row, tile_expert, tile_row0, n_tiles);
    return kestrel_check_launch("moe_group");
}

KESTREL_API int kestrel_moe_max_tiles(int P, int E, int rows_per_tile) { return (P + rows_per_tile - 1) / rows_per_tile + E; }

// ------------------------------------------------------------------------------------------
// Grouped products on the CUDA cores: tile of 64 rows x 64 features, 256 threads, 4 x 4 outputs a
// thread, K in steps of 16 through shared memory (the plain product's scheme with an expert per
// row tile).  GATE_UP: two accumulators (rows n and ff + n of the expert's stacked gate/up
// matrix) and the activation as epilogue; else one accumulator times the pair's weight.
// ------------------------------------------------------------------------------------------
#define MP_BM 64
#define MP_BN 64
#define MP_BK 16

// activations of an expert without a gate, y = W_down act(W_up x): 1 the exact gelu (erf), 2 its tanh form, 3 silu, 4 relu squared
__device__ __forceinline__ float expert_up_act(float z, int kind) {
    if (kind == 1) return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
    if (kind == 2) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    if (kind == 3) return z / (1.0f + expf(-z));
    const float r = fmaxf(z, 0.f);
    return r * r;
}

__device__ __forceinline__ float expert_act(float g, float u, float limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * (1.0f / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
}

template <typename T, bool GATE_UP>
__global__ void __launch_bounds__(256)
moe_gemm_plain_kernel(const T *__restrict__ x, long long ldx, const T *__restrict__ w, long long expert_stride, long long ldw,
                      const int *__restrict__ offsets, const int *__restrict__ row_pair, const int *__restrict__ tile_expert,
                      const int *__restrict__ tile_row0, const int *__restrict__ n_tiles, int top, const float *__restrict__ pair_weight,
                      float limit, void *__restrict__ out, long long ldo, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.y >= *n_tiles) return;
    __shared__ float xs[MP_BK][MP_BM + 4];
    __shared__ float ws[GATE_UP ? 2 : 1][MP_BK][MP_BN + 4];
    __shared__ int src_row[MP_BM];
    const int tid = threadIdx.x;
    const int e = tile_expert[blockIdx.y], r0 = tile_row0[blockIdx.y];
    const int rows = min(MP_BM, offsets[e + 1] - r0);
    const int n0 = blockIdx.x * MP_BN;
    const T *we = w + (size_t)e * expert_stride;
    if (tid < MP_BM) src_row[tid] = tid < rows ? (GATE_UP ? row_pair[r0 + tid] / top : r0 + tid) : -1;
    __syncthreads();
    const int ty = tid / 16, tx = tid % 16;
    float acc[GATE_UP ? 2 : 1][4][4];
#pragma unroll
    for (int a = 0; a < (GATE_UP ? 2 : 1); ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[a][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MP_BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = tid + 256 * q;
            const int r = idx / MP_BK, kk = idx % MP_BK;
            const int gk = k0 + kk;
            float xv = 0.f, wv = 0.f, wv2 = 0.f;
            if (gk < K) {
                if (src_row[r] >= 0) xv = to_f32<T>(x[(size_t)src_row[r] * ldx + gk]);
                if (n0 + r < N) {
                    wv = to_f32<T>(we[(size_t)(n0 + r) * ldw + gk]);
                    if (GATE_UP) wv2 = to_f32<T>(we[(size_t)(N + n0 + r) * ldw + gk]);
                }
            }
            xs[kk][r] = xv;
            ws[0][kk][r] = wv;
            if (GATE_UP) ws[GATE_UP ? 1 : 0][kk][r] = wv2;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MP_BK; ++kk) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[j] = ws[0][kk][tx * 4 + j];
                if (GATE_UP) b2[j] = ws[GATE_UP ? 1 : 0][kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[0][i][j] = fmaf(a[i], b[j], acc[0][i][j]);
                    if (GATE_UP) acc[GATE_UP ? 1 : 0][i][j] = fmaf(a[i], b2[j], acc[GATE_UP ? 1 : 0][i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
        const float pw = (GATE_UP || !pair_weight) ? 0.f : pair_weight[row_pair[r0 + r]];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GATE_UP)
                ((T *)out)[(size_t)(r0 + r) * ldo + n] = from_f32<T>(expert_act(acc[0][i][j], acc[GATE_UP ? 1 : 0][i][j], limit));
            else if (!pair_weight)          // an up product: the activation `limit` names, in the storage type
                ((T *)out)[(size_t)(r0 + r) * ldo + n] = from_f32<T>(expert_up_act(acc[0][i][j], (int)limit));
            else
                ((float *)out)[(size_t)(r0 + r) * ldo + n] = acc[0][i][j] * pw;
        }
    }
}

// ------------------------------------------------------------------------------------------
// Grouped products on the tensor cores, bfloat16: a CTA of four warps takes a tile of 64 rows of
// one expert (warp w rows 16 w ..) against 128 weight rows - 128 features of W_down, or 64 gate
// rows and the 64 up rows of the same features, so that the activation is the epilogue and the
// gate/up product never reaches memory.  K in steps of 32 through a three-stage cp.async ring;
// rows of 40 elements in shared memory keep ldmatrix free of bank conflicts.  Needs K and the row
// strides in multiples of 8 elements and 16-byte aligned bases (cp.async of 16 bytes).
// ------------------------------------------------------------------------------------------
#define MM_BM 64
#define MM_BN 128
#define MM_BK 32
#define MM_LDS 40
#define MM_STAGES 3
#define MM_SMEM (MM_STAGES * (MM_BM + MM_BN) * MM_LDS * 2)

__device__ __forceinline__ void moe_cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}

template <bool GATE_UP>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const __nv_bfloat16 *__restrict__ x, long long ldx, const __nv_bfloat16 *__restrict__ w, long long expert_stride,
                    long long ldw, const int *__restrict__ offsets, const int *__restrict__ row_pair, const int *__restrict__ tile_expert,
                    const int *__restrict__ tile_row0, const int *__restrict__ n_tiles, int top, const float *__restrict__ pair_weight,
                    float limit, void *__restrict__ out, long long ldo, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.y >= *n_tiles) return;
    extern __shared__ __align__(16) uint8_t moe_smem[];
    __nv_bfloat16 *As = reinterpret_cast<__nv_bfloat16 *>(moe_smem);              // [stage][64][40]
    __nv_bfloat16 *Bs = As + MM_STAGES * MM_BM * MM_LDS;                          // [stage][128][40]
    __shared__ int src_row[MM_BM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int e = tile_expert[blockIdx.y], r0 = tile_row0[blockIdx.y];
    const int rows = min(MM_BM, offsets[e + 1] - r0);
    const int n0 = blockIdx.x * (GATE_UP ? MM_BN / 2 : MM_BN);
    const __nv_bfloat16 *we = w + (size_t)e * expert_stride;
    if (tid < MM_BM) src_row[tid] = tid < rows ? (GATE_UP ? row_pair[r0 + tid] / top : r0 + tid) : -1;
    __syncthreads();

    // what this thread copies of every k-block: 2 chunks of 16 bytes of the rows' tile, 4 of the weights'
    const int kc = tid & 3;
    const __nv_bfloat16 *a_src[2], *b_src[4];
    bool a_ok[2], b_ok[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = (tid >> 2) + 32 * i;
        a_ok[i] = src_row[r] >= 0;
        a_src[i] = x + (size_t)(a_ok[i] ? src_row[r] : 0) * ldx + kc * 8;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = (tid >> 2) + 32 * i;
        const int f = GATE_UP ? n0 + (r & 63) : n0 + r;                           // feature of this weight row
        b_ok[i] = f < N;
        const int wrow = GATE_UP ? (r < 64 ? f : N + f) : f;
        b_src[i] = we + (size_t)(b_ok[i] ? wrow : 0) * ldw + kc * 8;
    }
    auto load = [&](int kt, int stage) {
        const int k = kt * MM_BK + kc * 8;
        const bool k_ok = k < K;                                                   // K is a multiple of 8: a chunk is whole or absent
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = (tid >> 2) + 32 * i;
            moe_cp_async16((uint32_t)__cvta_generic_to_shared(As + ((size_t)stage * MM_BM + r) * MM_LDS + kc * 8),
                           a_src[i] + (k_ok ? kt * MM_BK : 0), a_ok[i] && k_ok);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = (tid >> 2) + 32 * i;
            moe_cp_async16((uint32_t)__cvta_generic_to_shared(Bs + ((size_t)stage * MM_BN + r) * MM_LDS + kc * 8),
                           b_src[i] + (k_ok ? kt * MM_BK : 0), b_ok[i] && k_ok);
        }
    };
    const int KT = (K + MM_BK - 1) / MM_BK;
#pragma unroll
    for (int s = 0; s < MM_STAGES - 1; ++s) {
        if (s < KT) load(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;

    const int a_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_k = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_k = ((lane >> 3) & 1) * 8;
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(MM_STAGES - 2) : "memory");
        __syncthreads();                              // block kt has landed, and everyone has left the stage that is filled next
        const int nk = kt + MM_STAGES - 1;
        if (nk < KT) load(nk, nk % MM_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int stage = kt % MM_STAGES;
        const __nv_bfloat16 *Asg = As + (size_t)stage * MM_BM * MM_LDS, *Bsg = Bs + (size_t)stage * MM_BN * MM_LDS;
#pragma unroll
        for (int ks = 0; ks < MM_BK / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Asg + a_row * MM_LDS + ks * 16 + a_k), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int jp = 0; jp < 8; ++jp) {
                uint32_t b00, b01, b10, b11;
                ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Bsg + (jp * 16 + b_row) * MM_LDS + ks * 16 + b_k), b00, b01, b10, b11);
                mma_bf16(acc[2 * jp], a, b00, b01);
                mma_bf16(acc[2 * jp + 1], a, b10, b11);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + 8 * half;
        if (r >= rows) continue;
        if (GATE_UP) {
            __nv_bfloat16 *o = (__nv_bfloat16 *)out + (size_t)(r0 + r) * ldo;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int f = n0 + j * 8 + 2 * tq + c;
                    if (f < N) o[f] = __float2bfloat16_rn(expert_act(acc[j][2 * half + c], acc[j + 8][2 * half + c], limit));
                }
        } else if (!pair_weight) {          // an up product: the activation `limit` names, in the storage type
            __nv_bfloat16 *o = (__nv_bfloat16 *)out + (size_t)(r0 + r) * ldo;
#pragma unroll
            for (int j = 0; j < 16; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int f = n0 + j * 8 + 2 * tq + c;
                    if (f < N) o[f] = __float2bfloat16_rn(expert_up_act(acc[j][2 * half + c], (int)limit));
                }
        } else {
            const float pw = pair_weight[row_pair[r0 + r]];
            float *o = (float *)out + (size_t)(r0 + r) * ldo;
#pragma unroll
            for (int j = 0; j < 16; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int f = n0 + j * 8 + 2 * tq + c;
                    if (f < N) o[f] = acc[j][2 * half + c] * pw;
                }
        }
    }
}

static int g_moe_plain = 0;
// 1: the bfloat16 grouped products take the CUDA-core kernel too (for tests of both)
KESTREL_API void kestrel_moe_set_plain(int on) { g_moe_plain = on ? 1 : 0; }

static bool moe_mma_takes(const void *x, long long ldx, const void *w, int K) {
    return !g_moe_plain && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
}

template <bool GATE_UP>
static cudaError_t moe_mma_attr() {
    static bool done = false;
    if (done) return cudaSuccess;
    done = true;
    return cudaFuncSetAttribute(moe_gemm_mma_kernel<GATE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM);
}

// x [T, K] tokens; w [E, 2 ff, K] (gate rows, then up rows); act [P, ff] in the storage type, rows sorted by expert
KESTREL_API int kestrel_moe_gate_up(const void *x, long long ldx, const void *w, const int *offsets, const int *row_pair, const int *tile_expert,
                                    const int *tile_row0, const int *n_tiles, int max_tiles, int top, float limit, void *act, int dtype,
                                    int ff, int K, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    KESTREL_REQUIRE(max_tiles > 0 && max_tiles <= 65535 && ff > 0 && K > 0 && top > 0, "moe_gate_up: bad sizes");
    dim3 grid((ff + MP_BN - 1) / MP_BN, max_tiles);
    if (dtype == KESTREL_F32)
        kestrel_launch(moe_gemm_plain_kernel<float, true>, grid, dim3(256), 0, stream, (const float *)x, ldx, (const float *)w, (long long)2 * ff * K, (long long)K, offsets,
                       row_pair, tile_expert, tile_row0, n_tiles, top, (const float *)nullptr, limit, act, (long long)ff, ff, K);
    else if (dtype == KESTREL_BF16 && moe_mma_takes(x, ldx, w, K)) {
        moe_mma_attr<true>();
        kestrel_launch(moe_gemm_mma_kernel<true>, dim3((ff + MM_BN / 2 - 1) / (MM_BN / 2), max_tiles), dim3(128), MM_SMEM, stream, (const __nv_bfloat16 *)x, ldx,
                       (const __nv_bfloat16 *)w, (long long)2 * ff * K, (long long)K, offsets, row_pair, tile_expert, tile_row0, n_tiles, top, (const float *)nullptr, limit, act,
                       (long long)ff, ff, K);
    } else if (dtype == KESTREL_BF16)
        kestrel_launch(moe_gemm_plain_kernel<__nv_bfloat16, true>, grid, dim3(256), 0, stream, (const __nv_bfloat16 *)x, ldx, (const __nv_bfloat16 *)w, (long long)2 * ff * K,
                       (long long)K, offsets, row_pair, tile_expert, tile_row0, n_tiles, top, (const float *)nullptr, limit, act, (long long)ff, ff, K);
    else
        return kestrel_fail(-2, "moe_gate_up: unknown dtype %d", dtype);
    return kestrel_check_launch("moe_gate_up");
}

// act [P, ff]; w [E, N, ff]; y [P, N] float32 = (W_down[e] act) * weight of the pair
KESTREL_API int kestrel_moe_down(const void *act, const void *w, const int *offsets, const int *row_pair, const int *tile_expert,
                                 const int *tile_row0, const int *n_tiles, int max_tiles, const float *pair_weight, float *y, int dtype, int N,
                                 int ff, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    KESTREL_REQUIRE(max_tiles > 0 && max_tiles <= 65535 && ff > 0 && N > 0, "moe_down: bad sizes");
    dim3 grid((N + MP_BN - 1) / MP_BN, max_tiles);
    if (dtype == KESTREL_F32)
        kestrel_launch(moe_gemm_plain_kernel<float, false>, grid, dim3(256), 0, stream, (const float *)act, (long long)ff, (const float *)w, (long long)N * ff, (long long)ff,
                       offsets, row_pair, tile_expert, tile_row0, n_tiles, 1, pair_weight, 0.f, (void *)y, (long long)N, N, ff);
    else if (dtype == KESTREL_BF16 && moe_mma_takes(act, (long long)ff, w, ff)) {
        moe_mma_attr<false>();
        kestrel_launch(moe_gemm_mma_kernel<false>, dim3((N + MM_BN - 1) / MM_BN, max_tiles), dim3(128), MM_SMEM, stream, (const __nv_bfloat16 *)act, (long long)ff,
                       (const __nv_bfloat16 *)w, (long long)N * ff, (long long)ff, offsets, row_pair, tile_expert, tile_row0, n_tiles, 1, pair_weight, 0.f, (void *)y,
                       (long long)N, N, ff);
    } else if (dtype == KESTREL_BF16)
        kestrel_launch(moe_gemm_plain_kernel<__nv_bfloat16, false>, grid, dim3(256), 0, stream, (const __nv_bfloat16 *)act, (long long)ff, (const __nv_bfloat16 *)w,
                       (long long)N * ff, (long long)ff, offsets, row_pair, tile_expert, tile_row0, n_tiles, 1, pair_weight, 0.f, (void *)y, (long long)N, N, ff);
    else
        return kestrel_fail(-2, "moe_down: unknown dtype %d", dtype);
    return kestrel_check_launch("moe_down");
}

// Experts without a gate: act [P, ff] = activation(W_up[e] xs) in the storage type, xs [P, K] the pairs' input rows gathered in
// sorted order, w [E, ff, K]; `act_kind` 1 exact gelu (erf), 2 gelu in its tanh form, 3 silu, 4 relu squared
KESTREL_API int kestrel_moe_up_act(const void *xs, const void *w, const int *offsets, const int *row_pair, const int *tile_expert,
                                   const int *tile_row0, const int *n_tiles, int max_tiles, int act_kind, void *act, int dtype, int ff, int K,
                                   cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    KESTREL_REQUIRE(max_tiles > 0 && max_tiles <= 65535 && ff > 0 && K > 0 && act_kind >= 1 && act_kind <= 4, "moe_up_act: bad sizes or activation %d", act_kind);
    dim3 grid((ff + MP_BN - 1) / MP_BN, max_tiles);
    const float kind = (float)act_kind;
    if (dtype == KESTREL_F32)
        kestrel_launch(moe_gemm_plain_kernel<float, false>, grid, dim3(256), 0, stream, (const float *)xs, (long long)K, (const float *)w, (long long)ff * K, (long long)K,
                       offsets, row_pair, tile_expert, tile_row0, n_tiles, 1, (const float *)nullptr, kind, act, (long long)ff, ff, K);
    else if (dtype == KESTREL_BF16 && moe_mma_takes(xs, (long long)K, w, K)) {
        moe_mma_attr<false>();
        kestrel_launch(moe_gemm_mma_kernel<false>, dim3((ff + MM_BN - 1) / MM_BN, max_tiles), dim3(128), MM_SMEM, stream, (const __nv_bfloat16 *)xs, (long long)K,
                       (const __nv_bfloat16 *)w, (long long)ff * K, (long long)K, offsets, row_pair, tile_expert, tile_row0, n_tiles, 1, (const float *)nullptr, kind, act,
                       (long long)ff, ff, K);
    } else if (dtype == KESTREL_BF16)
        kestrel_launch(moe_gemm_plain_kernel<__nv_bfloat16, false>, grid, dim3(256), 0, stream, (const __nv_bfloat16 *)xs, (long long)K, (const __nv_bfloat16 *)w,
                       (long long)ff * K, (long long)K, offsets, row_pair, tile_expert, tile_row0, n_tiles, 1, (const float *)nullptr, kind, act, (long long)ff, ff, K);
    else
        return kestrel_fail(-2, "moe_up_act: unknown dtype %d", dtype);
    return kestrel_check_launch("moe_up_act");
}

// xs[r, :] = x[row_pair[r] / top, :] in any storage type
template <typename T>
__global__ void moe_gather_rows_any_kernel(const T *__restrict__ x, long long ldx, const int *__restrict__ row_pair, int top, T *__restrict__ xs, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const T *src = x + (size_t)(row_pair[r] / top) * ldx;
    for (int i = threadIdx.x; i < K; i += blockDim.x) xs[(size_t)r * K + i] = src[i];
}

KESTREL_API int kestrel_moe_gather_rows_any(const void *x, long long ldx, const int *row_pair, int top, void *xs, int dtype, int P, int K, cudaStream_t stream) {
    if (P == 0) return 0;
    KESTREL_REQUIRE(P > 0 && K > 0 && top > 0, "moe_gather_rows: bad sizes");
    if (dtype == KESTREL_F32)
        kestrel_launch(moe_gather_rows_any_kernel<float>, dim3(P), dim3(128), 0, stream, (const float *)x, ldx, row_pair, top, (float *)xs, K);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(moe_gather_rows_any_kernel<__nv_bfloat16>, dim3(P), dim3(128), 0, stream, (const __nv_bfloat16 *)x, ldx, row_pair, top, (__nv_bfloat16 *)xs, K);
    else
        return kestrel_fail(-2, "moe_gather_rows: unknown dtype %d", dtype);
    return kestrel_check_launch("moe_gather_rows");
}

// out[t, n] = sum_k y[pair_row[t * top + k], n], k ascending
__global__ void moe_combine_kernel(const float *__restrict__ y, const int *__restrict__ pair_row, int top, float *__restrict__ out, int N) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) v += y[(size_t)pair_row[(size_t)t * top + k] * N + n];
        out[(size_t)t * N + n] = v;
    }
}

KESTREL_API int kestrel_moe_combine(const float *y, const int *pair_row, int top, float *out, int T, int N, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && N > 0 && top > 0, "moe_combine: bad sizes");
    kestrel_launch(moe_combine_kernel, dim3(T), dim3(256), 0, stream, y, pair_row, top, out, N);
    return kestrel_check_launch("moe_combine");
}
