// Order-fixed float64 helpers: log2 / exp2 built from IEEE basic operations only, so that the side information
// derived from them (scale bins, column classes) is the same on every machine.  Restates dm_rint / dm_log2v /
// dm_exp2v of the reference (seedpack/detmath.py:19-65); compiled without FMA contraction like the rest of the
// library, every product and sum below is a separately rounded operation.
#pragma once
#include "common.cuh"

namespace sg {
namespace dm {

SG_DEVINL double rint_even(double x) {          // round half to even by letting an addition round
    if (!(fabs(x) < 4503599627370496.0)) return x;
    double y = fabs(x) + 4503599627370496.0;
    y = y - 4503599627370496.0;
    return copysign(y, x);
}

// log2 x = e + 2 atanh(s) / ln 2 with m in (1/sqrt 2, sqrt 2], s = (m - 1) / (m + 1); the atanh series to s^25
SG_DEVINL double log2v(double x) {
    if (isnan(x)) return x;
    if (x < 0.0) return __longlong_as_double(0x7ff8000000000000LL);
    if (x == 0.0) return __longlong_as_double((long long)0xfff0000000000000ULL);
    if (isinf(x)) return x;
    long long u = __double_as_longlong(x);
    int e = (int)((u >> 52) & 0x7ff);
    if (e == 0) {                                // subnormal: scale by 2^54 first
        x = x * 18014398509481984.0;
        u = __double_as_longlong(x);
        e = (int)((u >> 52) & 0x7ff) - 54;
    }
    e -= 1023;
    double m = __longlong_as_double((u & 0x000fffffffffffffLL) | 0x3ff0000000000000LL);
    if (m > 1.4142135623730951) { m = m * 0.5; e += 1; }
    const double s = (m - 1.0) / (m + 1.0), z = s * s;
    double p = 1.0 / 25.0;
#pragma unroll
    for (int k = 23; k >= 1; k -= 2) p = p * z + 1.0 / (double)k;
    return (double)e + (2.0 * s * p) * 1.4426950408889634;
}

// 2^y = 2^n e^t with n = rint(y), t = (y - n) ln 2; e^t by its Taylor polynomial to t^17, Horner form
SG_DEVINL double exp2v(double y) {
    if (isnan(y)) return y;
    if (y >= 1024.0) return __longlong_as_double(0x7ff0000000000000LL);
    if (y < -1075.0) return 0.0;
    const double n = rint_even(y), t = (y - n) * 0.6931471805599453;
    // reciprocal factorials; the reference's coefficients for 9! and 10! sit one ulp off the rounded quotient and
    // are kept bit for bit (seedpack/detmath.py:55-56), since the rounded results become stored side information
    const double inv_fact[18] = {1.0, 1.0, 1.0 / 2.0, 1.0 / 6.0, 1.0 / 24.0, 1.0 / 120.0, 1.0 / 720.0, 1.0 / 5040.0, 1.0 / 40320.0,
                                 0x1.71de3a556c733p-19, 0x1.27e4fb7789f5dp-22, 1.0 / 39916800.0, 1.0 / 479001600.0, 1.0 / 6227020800.0,
                                 1.0 / 87178291200.0, 1.0 / 1307674368000.0, 1.0 / 20922789888000.0, 1.0 / 355687428096000.0};
    double p = inv_fact[17];
#pragma unroll
    for (int k = 16; k >= 0; --k) p = p * t + inv_fact[k];
    const int k = (int)n, k1 = k / 2, k2 = k - k1;             // 2^k as two normal factors
    return p * __longlong_as_double((long long)(k1 + 1023) << 52) * __longlong_as_double((long long)(k2 + 1023) << 52);
}

}  // namespace dm
}  // namespace sg
