// Seeded input generators of the CPU oracle (test infrastructure only, never linked into the product).
//
// The reference's suites draw their inputs from std::mt19937 (seed 42 for A and C, 123 for B, 7 for
// bias) through the C++ standard library's distributions (test/common/data_generator.h:47-66,
// data_generator.cpp:14-19: one draw per element, row-major, narrowed with static_cast).  These
// entry points do the same with the standard library of the box they are built on, so that the
// full-size configuration tests and the benchmark can generate the reference's input streams
// where the reference checkout does not exist.  The uniform ones are pinned against the
// reference's own generator by tests/test_oracle_pins.py; the normal ones (the configurations'
// N(0, sigma) tensors; the reference has no normal generator) use std::normal_distribution<float>
// on the same engine.
#include <cstddef>
#include <cstdint>
#include <random>

extern "C" {

void tqo_fill_uniform_f32(float *dst, size_t count, float lo, float hi, uint32_t seed)
{
    std::mt19937 eng(seed);
    std::uniform_real_distribution<float> d(lo, hi);
    for (size_t i = 0; i < count; ++i) dst[i] = d(eng);
}

void tqo_fill_uniform_i8(int8_t *dst, size_t count, int lo, int hi, uint32_t seed)
{
    std::mt19937 eng(seed);
    std::uniform_int_distribution<int8_t> d(static_cast<int8_t>(lo), static_cast<int8_t>(hi));   // the reference's trait: the element type itself
    for (size_t i = 0; i < count; ++i) dst[i] = static_cast<int8_t>(d(eng));
}

void tqo_fill_uniform_i32(int32_t *dst, size_t count, int32_t lo, int32_t hi, uint32_t seed)
{
    std::mt19937 eng(seed);
    std::uniform_int_distribution<int32_t> d(lo, hi);
    for (size_t i = 0; i < count; ++i) dst[i] = d(eng);
}

void tqo_fill_normal_f32(float *dst, size_t count, float mean, float sigma, uint32_t seed)
{
    std::mt19937 eng(seed);
    std::normal_distribution<float> d(mean, sigma);
    for (size_t i = 0; i < count; ++i) dst[i] = d(eng);
}

}  // extern "C"
