// Host twin of the device Philox4x32-7 mask stream (csrc/common.cuh: philox_uniform8).
//
// An element of a mask is the same function of (seed, stream, row, column) on the CPU path (the eager oracle, the
// toy models, every CPU test) as in the fused GEMM epilogues on the GPU. The counter of a group of eight columns
// is (group, row, stream, 0x5044), the key is the 64-bit seed; four output words give eight 16-bit uniforms
// (low half first). The pure-torch statement of the same stream (ops/philox_ref.py) stays the definition this
// file is tested against; this one exists because that form costs a dozen tensor ops per round.
//
// This file has no counterpart in the reference, whose random streams come from its array library.
#include <cstdint>

namespace {

constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u;
constexpr uint32_t kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
constexpr int kRounds = 7;

inline void philox4x32(uint32_t c[4], uint32_t k0, uint32_t k1) {
    for (int r = 0; r < kRounds; ++r) {
        const uint64_t p0 = static_cast<uint64_t>(kM0) * c[0];
        const uint64_t p1 = static_cast<uint64_t>(kM1) * c[2];
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
        const uint32_t n1 = static_cast<uint32_t>(p1);
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
        const uint32_t n3 = static_cast<uint32_t>(p0);
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += kW0;
        k1 += kW1;
    }
}

}  // namespace

extern "C" {

// out[rows, cols] fp32 (row pitch `pitch` floats), cols a multiple of 8, uniforms in (0, 1) with 16 random bits.
// Returns 0, or 1 when the arguments are refused.
int pd_host_philox_uniform(uint64_t seed, uint32_t stream, int64_t rows, int64_t cols, int64_t row_offset,
                           float* out, int64_t pitch) {
    if (rows < 0 || cols < 0 || (cols & 7) != 0 || out == nullptr || pitch < cols) return 1;
    const uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
    const int64_t groups = cols / 8;
    constexpr float kScale = 1.0f / 65536.0f;
    for (int64_t r = 0; r < rows; ++r) {
        float* row = out + r * pitch;
        const uint32_t row_word = static_cast<uint32_t>(row_offset + r);
        for (int64_t g = 0; g < groups; ++g) {
            uint32_t c[4] = {static_cast<uint32_t>(g), row_word, stream, 0x5044u};
            philox4x32(c, k0, k1);
            float* o = row + g * 8;
            for (int w = 0; w < 4; ++w) {
                o[2 * w] = (static_cast<float>(c[w] & 0xFFFFu) + 0.5f) * kScale;
                o[2 * w + 1] = (static_cast<float>(c[w] >> 16) + 0.5f) * kScale;
            }
        }
    }
    return 0;
}

}  // extern "C"
