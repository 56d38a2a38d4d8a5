// Grouped expert products of many tokens on the 5th-generation tensor cores: the scheme of the
// one-tile-a-CTA product of gemm_tcgen05.cu (TMA with 128-byte swizzle into a ring of stages,
// one thread issuing tcgen05.mma M = 128 weight rows x N = 128 tokens x K = 16 into TMEM, four
// epilogue warps reading it back with tcgen05.ld) with a tile list in place of a regular grid.
//
// The step's (token, choice) pairs are sorted by expert (moe.cu: group) and their input rows
// gathered into one matrix xs [P, K], so that a tile of 128 rows of one expert is a TMA box of
// xs; the experts' stacked weights [E, rows, K] are ONE 2-D tensor [E * rows, K] whose box starts
// at row e * rows + n0.  A tile may reach into the next expert's rows of xs and a feature block
// into the next expert's weight rows: what they compute is never stored.
//   GATE_UP  two weight tiles a CTA (gate rows n0.. and up rows ff + n0..) into two accumulators;
//            epilogue y = min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1) as bfloat16
//   DOWN     one weight tile; epilogue times the pair's routing weight, float32
// The tile list lives on the device; the grid covers its upper bound and surplus CTAs leave
// before they touch a barrier or TMEM.  All mbarrier waits are bounded (error word
// kestrel_moe_tc_error).
#include "tcgen05.cuh"
#include <math.h>

#define MT_BM 128          // weight rows of a tile (the MMA's M)
#define MT_BN 128          // tokens of a tile (the MMA's N)
#define MT_BK 64
#define MT_THREADS 192     // loader warp, MMA warp, four epilogue warps

__device__ int g_moe_tc_error = 0;

template <bool GATE_UP>
__global__ void __launch_bounds__(MT_THREADS)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, void *__restrict__ out,
              const int *__restrict__ offsets, const int *__restrict__ row_pair, const int *__restrict__ tile_expert,
              const int *__restrict__ tile_row0, const int *__restrict__ n_tiles, const float *__restrict__ pair_weight, float limit,
              int w_rows_per_expert, int up_row_offset, int N, int K, long long ldo, int stages) {
    pdl_launch_dependents();
    pdl_wait();                                       // the tile list is the predecessors' work
    if ((int)blockIdx.y >= *n_tiles) return;
    constexpr int A_TILES = GATE_UP ? 2 : 1;
    constexpr uint32_t A_BYTES = MT_BM * MT_BK * 2;
    constexpr uint32_t B_BYTES = MT_BN * MT_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = A_TILES * MT_BN;
    // M = 128, N = 128, bf16 x bf16 -> f32, both operands K-major
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT_BN >> 3) << 17) | ((uint32_t)(MT_BM >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + (uint32_t)stages * STAGE_BYTES;      // full[stages], empty[stages], accum, tmem slot
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
    const uint32_t accum_bar = bars + 16u * stages;
    const uint32_t tmem_slot = accum_bar + 8;
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = tile_expert[blockIdx.y], t0 = tile_row0[blockIdx.y];
    const int valid = min(MT_BN, offsets[e + 1] - t0);
    const int n0 = blockIdx.x * MT_BM;
    const int w_row = e * w_rows_per_expert + n0;
    const int num_kb = (K + MT_BK - 1) / MT_BK;

    if (warp == 0) {
        if (lane < stages) { mbar_init(full_bar(lane), 1); mbar_init(empty_bar(lane), 1); }
        if (lane == 31) mbar_init(accum_bar, 1);
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t tmem = 0;
    if (warp != 0) {
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(MT_THREADS - 32) : "memory");
        tc_fence_after();
        tmem = *tmem_slot_ptr;
    }
    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (kb >= stages && !mbar_wait(empty_bar(stage), phase ^ 1)) { atomicExch(&g_moe_tc_error, 1); break; }
                mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                const uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                const int kc = kb * MT_BK;
                tma_load_2d(sa, &map_w, full_bar(stage), kc, w_row);
                if (GATE_UP) tma_load_2d(sa + A_BYTES, &map_w, full_bar(stage), kc, w_row + up_row_offset);
                tma_load_2d(sa + A_TILES * A_BYTES, &map_x, full_bar(stage), kc, t0);
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait(full_bar(stage), phase)) { atomicExch(&g_moe_tc_error, 2); break; }
                tc_fence_after();
                const uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                const uint64_t da = smem_desc(sa), db = smem_desc(sa + A_TILES * A_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < MT_BK / 16; ++k4) {
                    const uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;
                    tc_mma(tmem, da + 2 * k4, db + 2 * k4, IDESC, acc);
                    if (GATE_UP) tc_mma(tmem + MT_BN, smem_desc(sa + A_BYTES) + 2 * k4, db + 2 * k4, IDESC, acc);
                }
                tc_commit(empty_bar(stage));
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
            tc_commit(accum_bar);
        }
    } else {
        const int q = warp & 3;                       // TMEM lanes 32q .. 32q+31 belong to this warp
        const int n = n0 + 32 * q + lane;
        const bool waited = mbar_wait(accum_bar, 0);
        if (!waited && lane == 0) atomicExch(&g_moe_tc_error, 3);
        tc_fence_after();
        if (waited) {
#pragma unroll 1
            for (int c = 0; c < MT_BN; c += 16) {
                if (c >= valid) break;
                float g[16];
                tc_ld16(tmem + ((uint32_t)(32 * q) << 16) + c, g);
                if (GATE_UP) {
                    float u[16];
                    tc_ld16(tmem + ((uint32_t)(32 * q) << 16) + MT_BN + c, u);
                    __nv_bfloat16 *o = (__nv_bfloat16 *)out;
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + j < valid) {
                                const float gg = fminf(g[j], limit), uu = fminf(fmaxf(u[j], -limit), limit);
                                o[(size_t)(t0 + c + j) * ldo + n] = __float2bfloat16_rn(gg * (1.0f / (1.0f + expf(-1.702f * gg))) * (uu + 1.0f));
                            }
                    }
                } else if (!pair_weight) {          // an up product of experts without a gate: the activation `limit` names
                    __nv_bfloat16 *o = (__nv_bfloat16 *)out;
                    const int kind = (int)limit;
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + j < valid) {
                                const float z = g[j];
                                float a;
                                if (kind == 1) a = 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
                                else if (kind == 2) a = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
                                else if (kind == 3) a = z / (1.0f + expf(-z));
                                else a = fmaxf(z, 0.f) * fmaxf(z, 0.f);
                                o[(size_t)(t0 + c + j) * ldo + n] = __float2bfloat16_rn(a);
                            }
                    }
                } else {
                    float *o = (float *)out;
                    // the 16 rows' routing weights: lane j fetches row j's, the others get it by shuffle
                    const float pw_mine = (lane < 16 && c + lane < valid) ? pair_weight[row_pair[t0 + c + lane]] : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float pw = __shfl_sync(0xffffffffu, pw_mine, j);
                        if (n < N && c + j < valid) o[(size_t)(t0 + c + j) * ldo + n] = g[j] * pw;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

static int g_moe_tc_smem_kb = 104;
// shared memory of a CTA's ring of stages in KB (104: two CTAs an SM; 200: one); for measurements
KESTREL_API void kestrel_moe_tc_set_ring_kb(int kb) { g_moe_tc_smem_kb = kb < 64 ? 64 : (kb > 200 ? 200 : kb); }

template <bool GATE_UP>
static int moe_tc_launch(const CUtensorMap &mw, const CUtensorMap &mx, void *out, const int *offsets, const int *row_pair,
                         const int *tile_expert, const int *tile_row0, const int *n_tiles, int max_tiles, const float *pair_weight,
                         float limit, int w_rows_per_expert, int up_off, int N, int K, long long ldo, cudaStream_t stream) {
    constexpr int STAGE_BYTES = (GATE_UP ? 2 : 1) * MT_BM * MT_BK * 2 + MT_BN * MT_BK * 2;
    const int num_kb = (K + MT_BK - 1) / MT_BK;
    // two CTAs share an SM (half of its shared memory and at most half of TMEM each): the epilogue of
    // one runs under the main loop of the other
    int stages = (g_moe_tc_smem_kb * 1024) / STAGE_BYTES;
    if (stages < 2) stages = 2;
    if (stages > num_kb) stages = num_kb < 2 ? 2 : num_kb;
    if (stages > 12) stages = 12;
    const size_t smem = (size_t)stages * STAGE_BYTES + 16 * stages + 16 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(moe_tc_kernel<GATE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return kestrel_fail(-3, "moe_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid((N + MT_BM - 1) / MT_BM, max_tiles);
    kestrel_launch(moe_tc_kernel<GATE_UP>, grid, dim3(MT_THREADS), smem, stream, mw, mx, out, offsets, row_pair, tile_expert, tile_row0, n_tiles,
                   pair_weight, limit, w_rows_per_expert, up_off, N, K, ldo, stages);
    return kestrel_check_launch("moe_tc");
}

// rows of a tile list these kernels take
KESTREL_API int kestrel_moe_tc_tile_rows(void) { return MT_BN; }

// whether the tensor-core grouped products take these operands (the TMA rules: 16-byte aligned bases and row strides)
KESTREL_API int kestrel_moe_tc_supported(const void *xs, const void *act, const void *w_gate_up, const void *w_down, int ff, int K) {
    auto aligned = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    return K % 8 == 0 && ff % 8 == 0 && aligned(xs) && aligned(act) && aligned(w_gate_up) && aligned(w_down);
}

// xs [P, K] rows sorted by expert; w [E, 2 ff, K]; act [P, ff] bfloat16
KESTREL_API int kestrel_moe_gate_up_tc(const void *xs, const void *w, const int *offsets, const int *tile_expert, const int *tile_row0,
                                       const int *n_tiles, int max_tiles, float limit, void *act, int P, int E, int ff, int K,
                                       cudaStream_t stream) {
    if (P == 0) return 0;
    KESTREL_REQUIRE(P > 0 && E > 0 && ff > 0 && K > 0 && max_tiles > 0 && max_tiles <= 65535, "moe_gate_up_tc: bad sizes");
    CUtensorMap mw, mx;
    int rc = kestrel_tensor_map_bf16(&mw, w, (long long)E * 2 * ff, K, K, MT_BM);
    if (rc == 0) rc = kestrel_tensor_map_bf16(&mx, xs, P, K, K, MT_BN);
    if (rc != 0) return rc;
    return moe_tc_launch<true>(mw, mx, act, offsets, nullptr, tile_expert, tile_row0, n_tiles, max_tiles, nullptr, limit, 2 * ff, ff, ff, K, ff, stream);
}

// act [P, ff]; w [E, N, ff]; y [P, N] float32 = (W_down[e] act) * weight of the pair
KESTREL_API int kestrel_moe_down_tc(const void *act, const void *w, const int *offsets, const int *row_pair, const int *tile_expert,
                                    const int *tile_row0, const int *n_tiles, int max_tiles, const float *pair_weight, float *y, int P,
                                    int E, int N, int ff, cudaStream_t stream) {
    if (P == 0) return 0;
    KESTREL_REQUIRE(P > 0 && E > 0 && ff > 0 && N > 0 && max_tiles > 0 && max_tiles <= 65535, "moe_down_tc: bad sizes");
    CUtensorMap mw, mx;
    int rc = kestrel_tensor_map_bf16(&mw, w, (long long)E * N, ff, ff, MT_BM);
    if (rc == 0) rc = kestrel_tensor_map_bf16(&mx, act, P, ff, ff, MT_BN);
    if (rc != 0) return rc;
    return moe_tc_launch<false>(mw, mx, (void *)y, offsets, row_pair, tile_expert, tile_row0, n_tiles, max_tiles, pair_weight, 0.f, N, 0, N, ff, N, stream);
}

// xs [P, K] rows sorted by expert; w [E, ff, K]; act [P, ff] bfloat16 = activation(W_up[e] xs) of experts without a gate
KESTREL_API int kestrel_moe_up_act_tc(const void *xs, const void *w, const int *offsets, const int *tile_expert, const int *tile_row0,
                                      const int *n_tiles, int max_tiles, int act_kind, void *act, int P, int E, int ff, int K, cudaStream_t stream) {
    if (P == 0) return 0;
    KESTREL_REQUIRE(P > 0 && E > 0 && ff > 0 && K > 0 && max_tiles > 0 && max_tiles <= 65535 && act_kind >= 1 && act_kind <= 4, "moe_up_act_tc: bad sizes");
    CUtensorMap mw, mx;
    int rc = kestrel_tensor_map_bf16(&mw, w, (long long)E * ff, K, K, MT_BM);
    if (rc == 0) rc = kestrel_tensor_map_bf16(&mx, xs, P, K, K, MT_BN);
    if (rc != 0) return rc;
    return moe_tc_launch<false>(mw, mx, act, offsets, nullptr, tile_expert, tile_row0, n_tiles, max_tiles, nullptr, (float)act_kind, ff, 0, ff, K, ff, stream);
}

// xs[r, :] = x[row_pair[r] / top, :], 16 bytes a thread and step
__global__ void moe_gather_rows_kernel(const __nv_bfloat16 *__restrict__ x, long long ldx, const int *__restrict__ row_pair, int top,
                                       __nv_bfloat16 *__restrict__ xs, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)(row_pair[r] / top) * ldx);
    uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)r * K);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
}

KESTREL_API int kestrel_moe_gather_rows(const void *x, long long ldx, const int *row_pair, int top, void *xs, int P, int K, cudaStream_t stream) {
    if (P == 0) return 0;
    KESTREL_REQUIRE(P > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0 && top > 0, "moe_gather_rows: bad sizes");
    kestrel_launch(moe_gather_rows_kernel, dim3(P), dim3(128), 0, stream, (const __nv_bfloat16 *)x, ldx, row_pair, top, (__nv_bfloat16 *)xs, K);
    return kestrel_check_launch("moe_gather_rows");
}

// error word of these kernels' bounded waits (0 = none); synchronises the device and clears it
KESTREL_API int kestrel_moe_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_moe_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_moe_tc_error, &zero, sizeof(int));
    return v;
}
