// What a layer does to a raw score q . k * scale before it weighs a key, and how the weights of a
// query's keys are formed.  All of it is float32.
//
//   s <- cap * tanh(s / cap)                      if cap > 0
//   s <- s - r1[head] * ln(1 + r2[head] * (i - j))   if r1 is given (i the query's position, j the key's)
//   s <- s + rel[bucket[min(i - j, far)], head]   if rel is given: a learned number per head and bucket of distances;
//                the buckets of the distances 0 .. far come as a table (every distance beyond far shares far's)
//   weighting 0: softmax over the visible keys
//             1: softmax with one more term in the denominator that carries no value: exp(sink[head]) where a
//                layer has learned numbers for it, exp(0) otherwise
//             2: each visible key weighs sigmoid(s + head_bias[head]); nothing is normalised over keys
#pragma once
#include <math.h>

#define KESTREL_WEIGH_SOFTMAX 0
#define KESTREL_WEIGH_SOFTMAX_SINK 1
#define KESTREL_WEIGH_SIGMOID 2

struct ScoreOpts {
    float softcap;             // 0: none
    const float *r1, *r2;      // [nq] each, or both null
    const float *head_bias;    // [nq] or null; read by weighting 2 only
    int weighting;
    const float *sink;         // [nq] or null (= zeros); read by weighting 1 only
    const float *rel;          // [buckets, rel_heads] or null
    const int *rel_bucket;     // [rel_far + 1]: bucket of a distance
    int rel_far, rel_heads;
};

// the options of one head, fetched once
struct HeadScore {
    float cap, inv_cap, r1, r2, bias;
    float sink;                // the extra term's exponent (weighting 1), as the scores are: not in base-2 units
    bool dist;
    const float *rel;          // this head's column of the distance table, or null
    const int *rel_bucket;
    int rel_far, rel_heads;
    __device__ __forceinline__ float rel_of(int distance) const { return rel[(size_t)rel_bucket[min(distance, rel_far)] * rel_heads]; }
    __device__ __forceinline__ HeadScore(const ScoreOpts &o, int head) {
        rel = o.rel ? o.rel + head : nullptr;
        rel_bucket = o.rel_bucket;
        rel_far = o.rel_far;
        rel_heads = o.rel_heads;
        cap = o.softcap;
        inv_cap = o.softcap > 0.f ? 1.0f / o.softcap : 0.f;
        dist = o.r1 != nullptr;
        r1 = dist ? o.r1[head] : 0.f;
        r2 = dist ? o.r2[head] : 0.f;
        bias = (o.weighting == KESTREL_WEIGH_SIGMOID && o.head_bias) ? o.head_bias[head] : 0.f;
        sink = (o.weighting == KESTREL_WEIGH_SOFTMAX_SINK && o.sink) ? o.sink[head] : 0.f;
    }
    // s = q . k * scale of a key `distance` positions behind the query
    __device__ __forceinline__ float operator()(float s, int distance) const {
        if (cap > 0.f) s = cap * tanhf(s * inv_cap);
        if (dist) s -= r1 * logf(1.0f + r2 * (float)distance);
        if (rel) s += rel_of(distance);
        return s + bias;
    }
    // The same on the special-function unit, for the tensor-core kernels (their P is rounded to bfloat16
    // anyway): tanh(x) = 1 - 2 / (1 + e^2x) from one ex2 and one rcp - an absolute error of a few 2^-23,
    // so of cap * 1e-6 in the score, also where x is small - and the logarithm from lg2.
    __device__ __forceinline__ float fast(float s, int distance) const {
        if (cap > 0.f) s = fmaf(-2.0f * cap, score_rcp(1.0f + score_exp2(s * (inv_cap * 2.8853900817779268f))), cap);
        if (dist) s -= r1 * __logf(fmaf(r2, (float)distance, 1.0f));
        if (rel) s += rel_of(distance);
        return s + bias;
    }
    // The same with the layer's options as compile-time facts, for loops over many scores: nothing of an option that
    // is off is issued.  Returns the score in base-2 units (times log2 e) unless SIGMOID, which returns the weight.
    template <bool CAP, bool DIST, bool SIGMOID>
    __device__ __forceinline__ float fast_as(float s, int distance) const {
        constexpr float LOG2E = 1.4426950408889634f;
        if (SIGMOID) {
            if (CAP) s = fmaf(-2.0f * cap, score_rcp(1.0f + score_exp2(s * (inv_cap * 2.8853900817779268f))), cap);
            if (DIST) s -= r1 * __logf(fmaf(r2, (float)distance, 1.0f));
            return score_rcp(1.0f + score_exp2((s + bias) * -LOG2E));
        }
        if (CAP) s = fmaf(-2.0f * LOG2E * cap, score_rcp(1.0f + score_exp2(s * (inv_cap * 2.8853900817779268f))), LOG2E * cap);
        else s *= LOG2E;
        if (DIST) s -= (LOG2E * r1) * __logf(fmaf(r2, (float)distance, 1.0f));
        return s;
    }
    static __device__ __forceinline__ float score_exp2(float x) {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }
    static __device__ __forceinline__ float score_rcp(float x) {
        float y;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }
};

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_fast(float z) { return HeadScore::score_rcp(1.0f + HeadScore::score_exp2(z * -1.4426950408889634f)); }
