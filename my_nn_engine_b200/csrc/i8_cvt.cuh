// Exact int8 -> bf16 / fp16 conversion of four packed bytes with byte-permute and one packed subtraction per pair.
#pragma once
#include <stdint.h>

namespace mynn {

// 4 int8 (one 32-bit word) -> 4 x 16-bit floats as two packed pairs {b0,b1} and {b2,b3}.
template <bool F16>
__device__ __forceinline__ void cvt_s8x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    if constexpr (F16) {
        // 0x6400 | (b ^ 0x80) is fp16(1024 + b + 128); subtracting 1152 gives b exactly.
        uint32_t p0 = __byte_perm(w, 0x64646464u, 0x4140) ^ 0x00800080u;
        uint32_t p1 = __byte_perm(w, 0x64646464u, 0x4342) ^ 0x00800080u;
        const uint32_t bias = 0x64806480u;
        asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(p0), "r"(bias));
        asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(p1), "r"(bias));
    } else {
        // 0x4300 | (b & 0x7f) is bf16(128 + (b & 0x7f)); the subtrahend 0x4300 | (b & 0x80) is 128 for b >= 0
        // and 256 for b < 0, so the difference is the signed byte exactly.
        uint32_t p0 = __byte_perm(w, 0x43434343u, 0x4140);
        uint32_t p1 = __byte_perm(w, 0x43434343u, 0x4342);
        uint32_t y0 = p0 & 0xFF7FFF7Fu, c0 = p0 & 0xFF80FF80u;
        uint32_t y1 = p1 & 0xFF7FFF7Fu, c1 = p1 & 0xFF80FF80u;
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(y0), "r"(c0));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(y1), "r"(c1));
    }
}

}  // namespace mynn
