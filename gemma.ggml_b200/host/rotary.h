// rotary.h — rotary positions as the models configure them: how many coordinates turn, the base of the frequencies
// f_i = base^(-2i / dims), and how a long context rescales them: not at all, every frequency divided by a factor
// (linear), the blend between divided and plain frequencies with a magnitude factor in the table (scaled), or by
// wavelength (banded): short waves stay, long ones are divided, and those between are blended.
// Tables are built on the host with angles in double: [positions][dims / 2][2] = (cos, sin) of position * f_i.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

struct rot_spec {
    int dims = 0;
    double base = 10000.0;
    bool scaled = false; // frequency blend over [fast, slow] turns of the original context, magnitude 0.1 ln(factor) + 1
    bool linear = false; // every frequency divided by factor
    // by wavelength l = 2 pi / f against the original context: l < original / high keeps f, l > original / low takes
    // f / factor, between them (1 - s) f / factor + s f with s = (original / l - low) / (high - low)
    bool banded = false;
    double low = 1.0, high = 1.0;
    double factor = 1.0, original = 0.0, fast = 0.0, slow = 0.0;
    std::string key() const; // two specs with the same key share a table
};

std::vector<float> rot_table(const rot_spec &r, int64_t n_pos);
