// Quantising a layer's PReLU output for the next layer, read off the raw accumulator.
//
// A producing layer's epilogue that writes the next layer's quantised activations would compute, per
// output, f = PReLU(a) (src/tnns/mm_p2_final_tnn_avx2.c:90-93: a > 0 ? a : a * alpha) and then the next
// layer's rule on f (src/tnns/ternarize2row_avx2.c:438-452: sign = f < -t, non-zero = |f| > t;
// src/tnns/binarize2row_avx2.c:19-21: sign = f < t).  For 0 < alpha <= 1 the PReLU as the kernels
// evaluate it, f(a) = max(a, fl(a * alpha)), never decreases in a (fl is monotone, and so is the max of
// two monotone functions), and the accumulator a is an integer below 2^22 in magnitude.  Each rule is
// therefore a threshold on a itself:
//     f(a) <  c   <=>  a <  L(c)    with L(c) = the smallest integer a for which f(a) >= c
//     f(a) >  c   <=>  a >  U(c)    with U(c) = the largest  integer a for which f(a) <= c
// and the epilogue spends two instructions per output and plane (a subtraction whose sign bit is the
// answer, a funnel shift) instead of evaluating f first.
//
// L and U are found exactly: on the side where f(a) = a they are ceil(c) / floor(c); on the other side
// an estimate c / alpha is off by less than one (|a| < 2^22, relative error of one rounding 2^-24), and
// the integers around it are tried with the very expression the epilogue would use.  Thresholds outside
// +-2^23 are clamped there: every reachable accumulator lies on the same side of them, and the
// subtraction stays exact.  A NaN threshold makes every comparison false, as it does in the reference.
//
// An accumulator offset `bias` (BNN: a = v + bias, an integer) is folded into the thresholds.
#pragma once
#include <cmath>

#if defined(__CUDACC__)
#define TNNS_HD __host__ __device__ __forceinline__
#else
#define TNNS_HD inline
#endif

namespace tnns_thr {

constexpr float kLimit = 8388608.0f;  // 2^23

TNNS_HD float prelu_unit(float a, float alpha) { return fmaxf(a, fmaf(a, alpha, 0.0f)); }

// smallest integer a with f(a) >= c (as a float; +-kLimit when out of reach)
TNNS_HD float lower_threshold(float c, float alpha) {
    if (!(c == c)) return -kLimit;                       // NaN: "f < c" is false for every a
    if (c > 0.0f) return fminf(ceilf(c), kLimit);        // f(a) = a there; a <= 0 gives f <= 0 < c
    float a = fmaxf(ceilf(c / alpha), -kLimit) - 2.0f;   // c <= 0: every a >= 0 has f(a) >= 0 >= c
#pragma unroll 1
    for (int i = 0; i < 5 && prelu_unit(a, alpha) < c; i++) a += 1.0f;
    return a;
}

// largest integer a with f(a) <= c
TNNS_HD float upper_threshold(float c, float alpha) {
    if (!(c == c)) return kLimit;                        // NaN: "f > c" is false for every a
    if (c >= 0.0f) return fminf(floorf(c), kLimit);      // f(a) = a for a > 0; a <= 0 gives f <= 0 <= c
    float a = fmaxf(floorf(c / alpha), -kLimit) - 2.0f;  // c < 0: every a >= 0 has f(a) >= 0 > c
#pragma unroll 1
    for (int i = 0; i < 5 && !(prelu_unit(a, alpha) > c); i++) a += 1.0f;
    return a - 1.0f;                                     // a is the first integer with f(a) > c
}

// What the epilogue keeps per image: for the raw accumulator v (a = v + bias)
//     sign      = signbit(v + n1)         n1 = bias - L   (ternary: L(-t); binary: L(t))
//     above     = signbit(t2 - v)         t2 = U(t) - bias        (ternary only; non-zero = sign | above)
// Both constants are +0 when they vanish, so that a -0 accumulator (a sum of -0 products) reads as 0.
struct Pair {
    float n1, t2;
};

TNNS_HD Pair make(float t, float alpha, float bias, bool ternary) {
    Pair r;
    r.n1 = bias - lower_threshold(ternary ? -t : t, alpha);  // x - x is +0 in round-to-nearest
    r.t2 = ternary ? upper_threshold(t, alpha) - bias : 0.0f;
    r.n1 += 0.0f;
    r.t2 += 0.0f;
    return r;
}

}  // namespace tnns_thr
