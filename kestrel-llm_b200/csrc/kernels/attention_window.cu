// Softmax attention of bfloat16 queries over the paged cache on the tensor cores
// (mma.sync.m16n8k16, float32 scores, statistics and accumulators) for layers whose mask is a
// window that keeps a request's first tokens, whose values have a size of their own, and whose
// head outputs are gated:
//
//   query at position i sees key j <= i  if  i - j < window  or  j < keep_first   (window 0: all)
//   out[i, head] = gate[i, head] * softmax_j(q_i . k_j * scale) V
//
// Rows of work are (token, query head of one kv group) pairs of one request's tokens in this
// step, token-major, so the heads that share a kv head read its keys and values once.  A CTA of
// four warps takes one (request, kv head, row tile):
//   KW = 1  tile of 64 rows, 16 a warp; every warp walks all key tiles (prompt portions);
//   KW = 4  tile of 16 rows shared by the warps; key tiles of 32 go round by round, four a round,
//           one a warp, all four computed at once; the four running (max, sum, out) states are
//           merged in warp order at the end (decode tokens).  The rounds may be shared out over
//           several CTAs (`ksplit`, the grid's x), each of which leaves its merged state (maximum, sum,
//           unnormalised out) in scratch; a second kernel merges the CTAs' states in ascending order
//           and writes the output: a step of few requests then fills the device.  Requests of up to 64
//           rows (two tokens of 32 heads on one key head, say) go this way as row tiles of 16.
// The keys a tile can see are two ranges: the kept first tokens [0, ka) and the window
// [kb, last position]; positions between them are never read (their pages may be gone).  Key
// tiles go from the pages to shared memory with cp.async, the next round of tiles in flight
// while the current one is used, rows beyond a range zero-filled; Q K^T and P V take their fragments with ldmatrix (V transposed), P goes
// from the score accumulators to the second product's A operand in registers.  The grid covers
// the longest request's row tiles for every request; CTAs beyond a request's rows leave at once,
// so nothing of the step is read on the host and a launch can be recorded for replay.
//
// A layer may change the scores and the weighing of keys (`ScoreOpts`, attention_score.cuh): a cap and a
// logarithmic distance term on the float32 scores; a softmax whose denominator has a valueless extra
// term exp(sink[head]) (exp(0) without learned numbers), added where a row's states are closed; or sigmoid weights that are not normalised,
// which need no running maximum - P is the weights themselves.  Without options the scores keep the
// short path (one multiply into the exponent's base-2 scale).
//
// Head sizes in multiples of 8 up to 256; the kernel is instantiated for 32, 64, 128 and 256 and
// smaller heads are padded with zero columns in shared memory.
#include "common.cuh"
#include "mma_sync.cuh"
#include "attention_score.cuh"
#include <math.h>

#define AW_THREADS 128
#define AW_BN_ROWS 64        // keys of a tile, KW = 1
#define AW_BN_KEYS 32        // keys of a tile, KW = 4

struct AwParams {
    const __nv_bfloat16 *q;         // [T, nq * hd]
    const __nv_bfloat16 *k_cache;   // [pages, nkv, page_size, hd]
    const __nv_bfloat16 *v_cache;   // [pages, nkv, page_size, v_ld]: a value is the first vd numbers of its row (v_ld = vd unless the rows hold more)
    int v_ld;
    __nv_bfloat16 *out;             // [T, nq * vd]
    const float *gate;              // [T, nq] or null
    const int *cu_seqlens, *kv_lens, *block_table;
    int table_stride, page_size, nq, nkv, hd, vd, window, keep_first;
    float scale_log2, scale;
    ScoreOpts opts;
    int scored;                     // any of the options is on
    float *part_o, *part_ml;        // KW = 4 with several CTAs a row tile: [seq, kv head, row tile, split, 16, D] and [.., 16, 2]
    int ksplit, row_tiles;          // KW = 4: shares of the key rounds a row tile, and row tiles of 16 a request (the grid's x is their product)
};

__device__ __forceinline__ void aw_cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}

template <int D, int KW>
__global__ void __launch_bounds__(AW_THREADS)
attention_window_kernel(const AwParams p) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int RW = 4 / KW, BM = 16 * RW, LDS = D + 8, CH = D / 8;
    constexpr int AW_BN = KW == 1 ? (D > 128 ? AW_BN_ROWS / 2 : AW_BN_ROWS) : (D > 128 ? AW_BN_KEYS / 2 : AW_BN_KEYS);   // head size 256: shorter tiles, two CTAs an SM
    constexpr int SLOTS = 2 * KW;                     // two rounds of KW tiles
    extern __shared__ __align__(16) uint8_t aw_smem[];
    __nv_bfloat16 *Qs = reinterpret_cast<__nv_bfloat16 *>(aw_smem);      // [BM][LDS]
    __nv_bfloat16 *Ks = Qs + BM * LDS;                                   // [SLOTS][AW_BN][LDS]
    __nv_bfloat16 *Vs = Ks + SLOTS * AW_BN * LDS;                        // [SLOTS][AW_BN][LDS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rt = warp % RW, ks = warp / RW;
    const int kvh = blockIdx.y, seq = blockIdx.z;
    const int G = p.nq / p.nkv, hd = p.hd, vd = p.vd;
    const int tok_begin = p.cu_seqlens[seq], n_tok = p.cu_seqlens[seq + 1] - tok_begin;
    // KW = 4: the grid's x counts (row tile, share of the key rounds) pairs
    const int ksplit = KW == 4 ? p.ksplit : 1, split = KW == 4 ? blockIdx.x % ksplit : 0;
    const int rt_idx = KW == 4 ? blockIdx.x / ksplit : blockIdx.x;
    const int n_rows = n_tok * G, row0 = rt_idx * BM;
    if (row0 >= n_rows) return;
    const int rows_here = min(BM, n_rows - row0);
    const int pos_begin = p.kv_lens[seq] - n_tok;
    const int p_lo = pos_begin + row0 / G, hi = pos_begin + (row0 + rows_here - 1) / G + 1;
    int kb = p.window > 0 ? max(0, p_lo - p.window + 1) : 0;
    int ka = p.window > 0 ? min(p.keep_first, kb) : 0;
    if (ka == kb) ka = kb = 0;                        // the kept tokens reach the window: one range
    const int nA = (ka + AW_BN - 1) / AW_BN, anchorB = (kb / AW_BN) * AW_BN;
    const int n_tiles = nA + (hi - anchorB + AW_BN - 1) / AW_BN;
    const int *table = p.block_table + (size_t)seq * p.table_stride;

    auto tile_range = [&](int ti, int &s0, int &lo, int &up) {
        if (ti < nA) { s0 = ti * AW_BN; lo = 0; up = ka; }
        else { s0 = anchorB + (ti - nA) * AW_BN; lo = kb; up = hi; }
    };
    auto load_tile = [&](int ti, int slot) {
        int s0, lo, up;
        tile_range(ti, s0, lo, up);
        for (int idx = tid; idx < AW_BN * CH; idx += AW_THREADS) {
            const int r = idx / CH, c = idx % CH, s = s0 + r;
            const bool in = s >= lo && s < up;
            size_t row = 0;
            if (in) row = ((size_t)table[s / p.page_size] * p.nkv + kvh) * p.page_size + (s % p.page_size);
            const bool k_ok = in && c * 8 < hd, v_ok = in && c * 8 < vd;
            aw_cp_async16((uint32_t)__cvta_generic_to_shared(Ks + ((size_t)slot * AW_BN + r) * LDS + c * 8), p.k_cache + (k_ok ? row * hd + c * 8 : 0), k_ok);
            aw_cp_async16((uint32_t)__cvta_generic_to_shared(Vs + ((size_t)slot * AW_BN + r) * LDS + c * 8), p.v_cache + (v_ok ? row * p.v_ld + c * 8 : 0), v_ok);
        }
    };
    auto load_round = [&](int rd) {                   // the KW tiles of round rd, into the slots of its parity
#pragma unroll
        for (int w = 0; w < KW; ++w)
            if (rd * KW + w < n_tiles) load_tile(rd * KW + w, (rd & 1) * KW + w);
    };
    for (int idx = tid; idx < BM * CH; idx += AW_THREADS) {
        const int r = idx / CH, c = idx % CH;
        const bool ok = r < rows_here && c * 8 < hd;
        size_t off = 0;
        if (ok) {
            const int row = row0 + r;
            off = ((size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G) * hd + c * 8;
        }
        aw_cp_async16((uint32_t)__cvta_generic_to_shared(Qs + r * LDS + c * 8), p.q + off, ok);
    }
    const int n_rounds = (n_tiles + KW - 1) / KW;
    const int per_split = (n_rounds + ksplit - 1) / ksplit;
    const int rd0 = split * per_split, rd1 = min(n_rounds, rd0 + per_split);
    if (rd0 < rd1) load_round(rd0);                   // Q travels with the first group
    asm volatile("cp.async.commit_group;" ::: "memory");

    // the two rows of this thread in its warp's 16-row tile: g and g + 8
    const int g = lane >> 2, tq = lane & 3;
    int pos_r[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int r = rt * 16 + g + 8 * h2;
        pos_r[h2] = r < rows_here ? pos_begin + (row0 + r) / G : -1;
    }
    const bool sigmoid = p.opts.weighting == KESTREL_WEIGH_SIGMOID, sink = p.opts.weighting == KESTREL_WEIGH_SOFTMAX_SINK;
    ScoreOpts no_opts = {0.f, nullptr, nullptr, nullptr, 0};
    const HeadScore hs[2] = {HeadScore(p.scored ? p.opts : no_opts, kvh * G + (row0 + min(rt * 16 + g, rows_here - 1)) % G),
                             HeadScore(p.scored ? p.opts : no_opts, kvh * G + (row0 + min(rt * 16 + g + 8, rows_here - 1)) % G)};
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
    const int a_row = rt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, a_k = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_k = ((lane >> 3) & 1) * 8;
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;
    const int k_steps = (hd + 15) / 16, v_pairs = (vd + 15) / 16;

    for (int rd = rd0; rd < rd1; ++rd) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                              // round rd has landed, and everyone has left the slots that are filled next
        if (rd + 1 < rd1) load_round(rd + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int ti = rd * KW + ks, stage = (rd & 1) * KW + ks;
        if (ti < n_tiles) {
            int s0, lo, up;
            tile_range(ti, s0, lo, up);
            const __nv_bfloat16 *Kg = Ks + (size_t)stage * AW_BN * LDS, *Vg = Vs + (size_t)stage * AW_BN * LDS;
            float sc[AW_BN / 8][4];
#pragma unroll
            for (int j = 0; j < AW_BN / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[j][c] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                if (kk < k_steps) {
                    uint32_t a[4];
                    ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Qs + a_row * LDS + kk * 16 + a_k), a[0], a[1], a[2], a[3]);
#pragma unroll
                    for (int jp = 0; jp < AW_BN / 16; ++jp) {
                        uint32_t b00, b01, b10, b11;
                        ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Kg + (jp * 16 + b_row) * LDS + kk * 16 + b_k), b00, b01, b10, b11);
                        mma_bf16(sc[2 * jp], a, b00, b01);
                        mma_bf16(sc[2 * jp + 1], a, b10, b11);
                    }
                }
            }
            // mask, scale, running maximum
            float mx[2] = {-INFINITY, -INFINITY};
            if (!p.scored) {
#pragma unroll
                for (int j = 0; j < AW_BN / 8; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int s = s0 + j * 8 + 2 * tq + (c & 1), pr = pos_r[c >> 1];
                        const bool ok = s >= lo && s < up && s <= pr && (p.window <= 0 || pr - s < p.window || s < p.keep_first);
                        sc[j][c] = ok ? sc[j][c] * p.scale_log2 : -INFINITY;
                        mx[c >> 1] = fmaxf(mx[c >> 1], sc[j][c]);
                    }
            } else {
#pragma unroll
                for (int j = 0; j < AW_BN / 8; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int s = s0 + j * 8 + 2 * tq + (c & 1), pr = pos_r[c >> 1];
                        const bool ok = s >= lo && s < up && s <= pr && (p.window <= 0 || pr - s < p.window || s < p.keep_first);
                        const float z = hs[c >> 1].fast(sc[j][c] * p.scale, max(pr - s, 0));
                        if (sigmoid) sc[j][c] = ok ? sigmoid_fast(z) : 0.f;          // the weight itself
                        else sc[j][c] = ok ? z * 1.4426950408889634f : -INFINITY;
                        mx[c >> 1] = fmaxf(mx[c >> 1], sc[j][c]);
                    }
            }
            if (sigmoid) {
#pragma unroll
                for (int k2 = 0; k2 < AW_BN / 16; ++k2) {
                    uint32_t a[4] = {pack_bf16(sc[2 * k2][0], sc[2 * k2][1]), pack_bf16(sc[2 * k2][2], sc[2 * k2][3]),
                                     pack_bf16(sc[2 * k2 + 1][0], sc[2 * k2 + 1][1]), pack_bf16(sc[2 * k2 + 1][2], sc[2 * k2 + 1][3])};
#pragma unroll
                    for (int np = 0; np < D / 16; ++np) {
                        if (np < v_pairs) {
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(Vg + (k2 * 16 + v_row) * LDS + np * 16 + v_col), b0, b1, b2, b3);
                            mma_bf16(o[2 * np], a, b0, b1);
                            mma_bf16(o[2 * np + 1], a, b2, b3);
                        }
                    }
                }
                continue;
            }
            float corr[2], ms[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
                const float mn = fmaxf(m_r[h2], mx[h2]);
                ms[h2] = mn == -INFINITY ? 0.f : mn;           // a row that has seen no key yet
                corr[h2] = fast_exp2(m_r[h2] - ms[h2]);
                m_r[h2] = mn;
                l_r[h2] *= corr[h2];
            }
#pragma unroll
            for (int j = 0; j < AW_BN / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    sc[j][c] = fast_exp2(sc[j][c] - ms[c >> 1]);
                    l_r[c >> 1] += sc[j][c];
                }
#pragma unroll
            for (int j = 0; j < D / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[j][c] *= corr[c >> 1];
#pragma unroll
            for (int k2 = 0; k2 < AW_BN / 16; ++k2) {
                uint32_t a[4] = {pack_bf16(sc[2 * k2][0], sc[2 * k2][1]), pack_bf16(sc[2 * k2][2], sc[2 * k2][3]),
                                 pack_bf16(sc[2 * k2 + 1][0], sc[2 * k2 + 1][1]), pack_bf16(sc[2 * k2 + 1][2], sc[2 * k2 + 1][3])};
#pragma unroll
                for (int np = 0; np < D / 16; ++np) {
                    if (np < v_pairs) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(Vg + (k2 * 16 + v_row) * LDS + np * 16 + v_col), b0, b1, b2, b3);
                        mma_bf16(o[2 * np], a, b0, b1);
                        mma_bf16(o[2 * np + 1], a, b2, b3);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                  // every warp is done with the tiles: their memory is free
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_r[h2] += __shfl_xor_sync(0xffffffffu, l_r[h2], 1);
        l_r[h2] += __shfl_xor_sync(0xffffffffu, l_r[h2], 2);
    }

    if (KW == 1) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int r = rt * 16 + g + 8 * h2;
            if (r >= rows_here) continue;
            const int row = row0 + r, tok = tok_begin + row / G, head = kvh * G + row % G;
            float inv = 1.0f / l_r[h2];
            if (sigmoid) inv = 1.0f;
            if (sink) {                                   // one more state in front: maximum sink, sum 1, no value
                const float s2 = (p.opts.sink ? p.opts.sink[head] : 0.f) * 1.4426950408889634f;
                const float M = fmaxf(m_r[h2], s2), f = fast_exp2(m_r[h2] - M);
                inv = f / (fast_exp2(s2 - M) + l_r[h2] * f);
            }
            if (p.gate) inv *= p.gate[(size_t)tok * p.nq + head];
            __nv_bfloat16 *dst = p.out + ((size_t)tok * p.nq + head) * vd;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                const int col = j * 8 + 2 * tq;
                if (col < vd) *reinterpret_cast<uint32_t *>(dst + col) = pack_bf16(o[j][2 * h2] * inv, o[j][2 * h2 + 1] * inv);
            }
        }
    } else {
        // the warps' states of the same 16 rows, merged in warp order
        float *sm_m = reinterpret_cast<float *>(Ks);          // [KW][16]
        float *sm_l = sm_m + KW * 16;                          // [KW][16]
        float *sm_o = sm_l + KW * 16;                          // [KW][16][D]
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int r = g + 8 * h2;
            if (tq == 0) { sm_m[ks * 16 + r] = m_r[h2]; sm_l[ks * 16 + r] = l_r[h2]; }
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                sm_o[((size_t)ks * 16 + r) * D + j * 8 + 2 * tq] = o[j][2 * h2];
                sm_o[((size_t)ks * 16 + r) * D + j * 8 + 2 * tq + 1] = o[j][2 * h2 + 1];
            }
        }
        __syncthreads();
        if (ksplit > 1) {
            // this CTA's share of the keys as one state: the warps' states merged in warp order, not normalised
            const size_t base = ((((size_t)seq * p.nkv + kvh) * p.row_tiles + rt_idx) * ksplit + split) * 16;
            for (int idx = tid; idx < rows_here * (vd + 1); idx += AW_THREADS) {
                const int r = idx / (vd + 1), col = idx % (vd + 1);
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < KW; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
                float L = 0.f, acc = 0.f;
#pragma unroll
                for (int w = 0; w < KW; ++w) {
                    if (col == vd) {
                        if (sm_m[w * 16 + r] != -INFINITY) L += sm_l[w * 16 + r] * fast_exp2(sm_m[w * 16 + r] - M);
                    } else if (sigmoid) {
                        acc += sm_o[((size_t)w * 16 + r) * D + col];
                    } else if (sm_m[w * 16 + r] != -INFINITY) {
                        acc += sm_o[((size_t)w * 16 + r) * D + col] * fast_exp2(sm_m[w * 16 + r] - M);
                    }
                }
                if (col == vd) { p.part_ml[(base + r) * 2] = M; p.part_ml[(base + r) * 2 + 1] = L; }
                else p.part_o[(base + r) * D + col] = acc;
            }
            return;
        }
        for (int idx = tid; idx < rows_here * vd; idx += AW_THREADS) {
            const int r = idx / vd, col = idx % vd;
            const float s2 = (sink && p.opts.sink) ? p.opts.sink[kvh * G + (row0 + r) % G] * 1.4426950408889634f : 0.f;
            float M = sink ? s2 : -INFINITY;
#pragma unroll
            for (int w = 0; w < KW; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
            float L = sink ? fast_exp2(s2 - M) : 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < KW; ++w) {
                if (sigmoid) { acc += sm_o[((size_t)w * 16 + r) * D + col]; continue; }
                if (sm_m[w * 16 + r] == -INFINITY) continue;
                const float f = fast_exp2(sm_m[w * 16 + r] - M);
                L += sm_l[w * 16 + r] * f;
                acc += sm_o[((size_t)w * 16 + r) * D + col] * f;
            }
            const int row = row0 + r, tok = tok_begin + row / G, head = kvh * G + row % G;
            float v = sigmoid ? acc : acc / L;
            if (p.gate) v *= p.gate[(size_t)tok * p.nq + head];
            p.out[((size_t)tok * p.nq + head) * vd + col] = __float2bfloat16_rn(v);
        }
    }
}

// KW = 4 with several CTAs a row tile: their states in ascending order of the keys, then the layer's
// way of closing a row (the softmax's extra term, no normalisation for sigmoid weights) and the gate.
__global__ void __launch_bounds__(AW_THREADS)
attention_window_merge_kernel(const AwParams p, int ksplit, int D) {
    __shared__ float f_s[64];                         // each share's factor 2^(m_s - M); then 1 / sum at [ksplit]
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, seq = blockIdx.y, row = blockIdx.z, G = p.nq / p.nkv, vd = p.vd;   // row among the request's rows
    const int tok_begin = p.cu_seqlens[seq];
    if (row >= (p.cu_seqlens[seq + 1] - tok_begin) * G) return;
    const int r = row % 16;
    const bool sigmoid = p.opts.weighting == KESTREL_WEIGH_SIGMOID, sink = p.opts.weighting == KESTREL_WEIGH_SOFTMAX_SINK;
    const size_t base = (((size_t)seq * p.nkv + kvh) * p.row_tiles + row / 16) * ksplit * 16 + r;      // + s * 16
    if (threadIdx.x < 32) {
        // lane s holds share s (ksplit <= 32); the sum goes over the shares in ascending order
        const int s = threadIdx.x;
        const float m = s < ksplit ? p.part_ml[(base + (size_t)s * 16) * 2] : -INFINITY;
        const float l = s < ksplit ? p.part_ml[(base + (size_t)s * 16) * 2 + 1] : 0.f;
        const float s2 = (sink && p.opts.sink) ? p.opts.sink[kvh * G + row % G] * 1.4426950408889634f : 0.f;
        float M = warp_max(m);
        if (sink) M = fmaxf(M, s2);
        const float f = m == -INFINITY ? 0.f : fast_exp2(m - M);
        if (s < ksplit) f_s[s] = sigmoid ? 1.f : f;
        float L = sink ? fast_exp2(s2 - M) : 0.f;
        for (int k = 0; k < ksplit; ++k) L += __shfl_sync(0xffffffffu, l * f, k);
        if (s == 0) f_s[ksplit] = sigmoid ? 1.f : 1.0f / L;
    }
    __syncthreads();
    const int tok = tok_begin + row / G, head = kvh * G + row % G;
    float inv = f_s[ksplit];
    if (p.gate) inv *= p.gate[(size_t)tok * p.nq + head];
    for (int col = threadIdx.x; col < vd; col += AW_THREADS) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < ksplit; ++s) acc = fmaf(p.part_o[(base + (size_t)s * 16) * D + col], f_s[s], acc);
        p.out[((size_t)tok * p.nq + head) * vd + col] = __float2bfloat16_rn(acc * inv);
    }
}

template <int D, int KW>
static int aw_launch(const AwParams &p, int nseq, int max_count, int ksplit, cudaStream_t stream) {
    constexpr int BM = 16 * (4 / KW), AW_BN = KW == 1 ? (D > 128 ? AW_BN_ROWS / 2 : AW_BN_ROWS) : (D > 128 ? AW_BN_KEYS / 2 : AW_BN_KEYS);
    const size_t smem = (size_t)(BM + 2 * 2 * KW * AW_BN) * (D + 8) * sizeof(__nv_bfloat16);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(attention_window_kernel<D, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return kestrel_fail(-3, "attention_window: cannot set the shared memory size %zu", smem);
        attr_set = true;
    }
    const int G = p.nq / p.nkv;
    dim3 grid(KW == 4 ? ksplit * p.row_tiles : ((size_t)max_count * G + BM - 1) / BM, p.nkv, nseq);
    kestrel_launch(attention_window_kernel<D, KW>, grid, dim3(AW_THREADS), smem, stream, p);
    int rc = kestrel_check_launch("attention_window");
    if (rc || KW != 4 || ksplit == 1) return rc;
    kestrel_launch(attention_window_merge_kernel, dim3(p.nkv, nseq, 16 * p.row_tiles), dim3(AW_THREADS), 0, stream, p, ksplit, D);
    return kestrel_check_launch("attention_window_merge");
}

#define AW_KEYS_MODE_ROWS 64     // steps whose requests bring at most this many rows (tokens x heads of a group) walk the keys in rounds

// Floats of scratch a launch with `ksplit` CTAs a row tile needs: 16 rows of D + 2 (D = the head sizes rounded up to
// 32, 64, 128 or 256) per request, kv head, row tile and share.
KESTREL_API long long kestrel_attention_window_scratch_floats(int nseq, int max_count, int nq, int nkv, int hd, int vd, int ksplit) {
    const int m = hd > vd ? hd : vd, D = m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256));
    const long long row_tiles = ((long long)max_count * (nq / nkv) + 15) / 16;
    return (long long)nseq * nkv * row_tiles * ksplit * 16 * (D + 2);
}

// Into how many shares the key rounds of a step of single tokens are cut: as many as fill the device once, each of at
// least one round; 1 for steps with portions (their row tiles fill it) and whenever the caller has no scratch.
KESTREL_API int kestrel_attention_window_splits(int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int max_kv_len) {
    if (nkv <= 0 || nseq <= 0 || (long long)max_count * (nq / nkv) > AW_KEYS_MODE_ROWS) return 1;
    const int row_tiles = (max_count * (nq / nkv) + 15) / 16;
    const int keys = window > 0 && window < max_kv_len ? window : max_kv_len;
    const int tile = (hd > 128 || vd > 128) ? AW_BN_KEYS / 2 : AW_BN_KEYS;
    const int rounds = (keys + 4 * tile - 1) / (4 * tile) + 1;
    int k = kestrel_sms() / (nseq * nkv * row_tiles);
    if (k > rounds) k = rounds;
    if (k > 32) k = 32;
    return k < 1 ? 1 : k;
}

// 1 if the kernel takes these sizes (the caller then need not fall back to the plain kernel)
KESTREL_API int kestrel_attention_window_supported(int hd, int vd, int nq, int nkv) {
    return hd > 0 && vd > 0 && hd % 8 == 0 && vd % 8 == 0 && hd <= 256 && vd <= 256 && nkv > 0 && nq % nkv == 0;
}

// max_count: the most tokens one request brings in this step (sizes the grid; a host constant of a recorded step)
KESTREL_API int kestrel_attention_window(const void *q, const void *k_cache, const void *v_cache, void *out, const float *gate,
                                         const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size,
                                         int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int keep_first, float scale,
                                         cudaStream_t stream) {
    return kestrel_attention_window_scored(q, k_cache, v_cache, out, gate, cu_seqlens, kv_lens, block_table, table_stride, page_size, nseq, max_count,
                                           nq, nkv, hd, vd, window, keep_first, scale, 0.f, nullptr, nullptr, nullptr, KESTREL_WEIGH_SOFTMAX, nullptr, 1, nullptr, stream);
}

KESTREL_API int kestrel_attention_window_scored(const void *q, const void *k_cache, const void *v_cache, void *out, const float *gate,
                                                const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size,
                                                int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int keep_first, float scale,
                                                float softcap, const float *r1, const float *r2, const float *head_bias, int weighting,
                                                const float *sink, int ksplit, float *scratch, cudaStream_t stream) {
    return kestrel_attention_window_biased(q, k_cache, v_cache, out, gate, cu_seqlens, kv_lens, block_table, table_stride, page_size, nseq, max_count,
                                           nq, nkv, hd, vd, window, keep_first, scale, softcap, r1, r2, head_bias, weighting, sink, nullptr, nullptr, 0, 0,
                                           ksplit, scratch, stream);
}

// the same with a learned number per head and bucket of distances added to the scores (ScoreOpts.rel), and with value rows of
// `v_ld` numbers of which the first vd are the value (0: vd) - a V plane that is the K plane of longer rows
KESTREL_API int kestrel_attention_window_biased(const void *q, const void *k_cache, const void *v_cache, void *out, const float *gate,
                                                const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size,
                                                int nseq, int max_count, int nq, int nkv, int hd, int vd, int window, int keep_first, float scale,
                                                float softcap, const float *r1, const float *r2, const float *head_bias, int weighting,
                                                const float *sink, const float *rel, const int *rel_bucket, int rel_far, int v_ld,
                                                int ksplit, float *scratch, cudaStream_t stream) {
    if (nseq == 0 || max_count == 0) return 0;
    KESTREL_REQUIRE(ksplit >= 1 && ksplit <= 65535 && (ksplit == 1 || scratch), "attention_window: %d shares of the keys without scratch", ksplit);
    KESTREL_REQUIRE(weighting >= 0 && weighting <= 2 && softcap >= 0.f && (r1 == nullptr) == (r2 == nullptr), "attention_window: bad score options");
    KESTREL_REQUIRE(kestrel_attention_window_supported(hd, vd, nq, nkv), "attention_window: head sizes %d / %d, heads %d / %d are not taken", hd, vd, nq, nkv);
    KESTREL_REQUIRE(nseq > 0 && nseq <= 65535 && nkv <= 65535 && max_count > 0 && window >= 0 && keep_first >= 0, "attention_window: bad sizes");
    AwParams p;
    p.q = (const __nv_bfloat16 *)q;
    p.k_cache = (const __nv_bfloat16 *)k_cache;
    p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out;
    p.gate = gate;
    p.cu_seqlens = cu_seqlens;
    p.kv_lens = kv_lens;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.page_size = page_size;
    p.nq = nq;
    p.nkv = nkv;
    p.hd = hd;
    p.vd = vd;
    p.v_ld = v_ld > 0 ? v_ld : vd;
    p.window = window;
    p.keep_first = window > 0 ? keep_first : 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.scale = scale;
    KESTREL_REQUIRE(!rel || (rel_bucket && rel_far >= 0), "attention_window: a distance table without its buckets");
    KESTREL_REQUIRE(v_ld == 0 || (v_ld >= vd && v_ld % 8 == 0), "attention_window: value rows of %d numbers for values of %d", v_ld, vd);
    p.opts = {softcap, r1, r2, head_bias, weighting, sink, rel, rel_bucket, rel_far, nq};
    p.scored = softcap > 0.f || r1 != nullptr || rel != nullptr || weighting != KESTREL_WEIGH_SOFTMAX;
    const int D = max(hd, vd), G = nq / nkv;
    const bool keys_mode = (long long)max_count * G <= AW_KEYS_MODE_ROWS;
    if (!keys_mode) ksplit = 1;
    const int Dt = D <= 32 ? 32 : (D <= 64 ? 64 : (D <= 128 ? 128 : 256));
    p.ksplit = ksplit;
    p.row_tiles = keys_mode ? (max_count * G + 15) / 16 : 1;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)nseq * nkv * p.row_tiles * ksplit * 16 * Dt : nullptr;
#define AW_CASE(DD)                                                                   \
    return keys_mode ? aw_launch<DD, 4>(p, nseq, max_count, ksplit, stream) : aw_launch<DD, 1>(p, nseq, max_count, 1, stream)
    if (D <= 32) { AW_CASE(32); }
    if (D <= 64) { AW_CASE(64); }
    if (D <= 128) { AW_CASE(128); }
    AW_CASE(256);
#undef AW_CASE
}
