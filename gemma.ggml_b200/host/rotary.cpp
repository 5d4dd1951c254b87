// rotary.cpp — see rotary.h
#include "rotary.h"

#include <algorithm>
#include <cmath>
#include <cstdio>

std::string rot_spec::key() const {
    char b[256];
    snprintf(b, sizeof b, "%d|%.17g|%d%d%d|%.17g|%.17g|%.17g|%.17g|%.17g|%.17g", dims, base, (int)scaled, (int)linear, (int)banded, factor, original,
             fast, slow, low, high);
    return b;
}

std::vector<float> rot_table(const rot_spec &r, int64_t n_pos) {
    const int half = r.dims / 2;
    std::vector<double> f((size_t)half);
    double mag = 1.0;
    for (int i = 0; i < half; i++) f[(size_t)i] = std::pow(r.base, -2.0 * i / r.dims);
    if (r.scaled) {
        const double two_pi = 6.283185307179586476925286766559;
        auto corr = [&](double t) { return r.dims * std::log(r.original / (two_pi * t)) / (2.0 * std::log(r.base)); };
        const double lo = std::max(std::floor(corr(r.fast)), 0.0), hi = std::min(std::ceil(corr(r.slow)), (double)r.dims - 1.0);
        for (int i = 0; i < half; i++) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            f[(size_t)i] = f[(size_t)i] / r.factor * ramp + f[(size_t)i] * (1.0 - ramp);
        }
        mag = 0.1 * std::log(r.factor) + 1.0;
    } else if (r.linear) {
        for (int i = 0; i < half; i++) f[(size_t)i] /= r.factor;
    } else if (r.banded) {
        const double two_pi = 6.283185307179586476925286766559;
        for (int i = 0; i < half; i++) {
            const double fi = f[(size_t)i], wave = two_pi / fi;
            if (wave < r.original / r.high) continue;
            if (wave > r.original / r.low) {
                f[(size_t)i] = fi / r.factor;
            } else {
                const double s = (r.original / wave - r.low) / (r.high - r.low);
                f[(size_t)i] = (1.0 - s) * fi / r.factor + s * fi;
            }
        }
    }
    std::vector<float> t((size_t)n_pos * (size_t)half * 2);
    for (int64_t p = 0; p < n_pos; p++)
        for (int i = 0; i < half; i++) {
            const double a = (double)p * f[(size_t)i];
            t[((size_t)p * half + i) * 2] = (float)(std::cos(a) * mag);
            t[((size_t)p * half + i) * 2 + 1] = (float)(std::sin(a) * mag);
        }
    return t;
}
