// Counter-based generator shared by host and device code: element `index` of (seed, stream)
// is the index-th output of a splitmix64 sequence whose state is derived from seed and stream.
// Every synthetic input of the library is a pure function of these three numbers, so the host
// generators, the device generators and the tests produce identical bits.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define DLSPM_HD __host__ __device__ __forceinline__
#else
#define DLSPM_HD inline
#endif

DLSPM_HD uint64_t dlspm_mix64(uint64_t z)
{
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Key of one (seed, stream) pair.
DLSPM_HD uint64_t dlspm_rng_key(uint64_t seed, uint64_t stream)
{
    return dlspm_mix64(seed + 0x9E3779B97F4A7C15ull) ^ dlspm_mix64(stream * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull);
}

DLSPM_HD uint64_t dlspm_rng_at(uint64_t key, uint64_t index)
{
    return dlspm_mix64(key + (index + 1) * 0x9E3779B97F4A7C15ull);
}

// 24 uniform bits -> fp32 in [-1, 1): exact in fp32, no rounding anywhere.
DLSPM_HD float dlspm_u24_to_pm1(uint32_t u24) { return (float)u24 * (1.0f / 8388608.0f) - 1.0f; }
// 24 uniform bits -> fp32 in [0, 1).
DLSPM_HD float dlspm_u24_to_01(uint32_t u24) { return (float)u24 * (1.0f / 16777216.0f); }
DLSPM_HD uint32_t dlspm_u24(uint64_t h) { return (uint32_t)(h >> 40); }

// Integer threshold of a Bernoulli(density) test on 24 uniform bits.
inline uint32_t dlspm_density_threshold(double density)
{
    if (density <= 0.0) return 0u;
    if (density >= 1.0) return 1u << 24;
    return (uint32_t)(density * 16777216.0);
}

// Streams used by the generators (kept in one place so tests can address them).
enum {
    DLSPM_STREAM_PATTERN = 1, // pattern bits / column-sample keys: index = row*K + col
    DLSPM_STREAM_VALUES = 2,  // nonzero values: index = position in CSR order
    DLSPM_STREAM_ROWLEN = 3   // row lengths: two uniforms per row
};
