// One row of a K-quant matrix expanded to floats on the host: the embedding lookup of a model with tied embeddings.
// Block layouts as GGUF defines them: Q4_K = d, dmin (fp16) | 12 bytes of 6-bit scales and mins | 128 bytes of
// nibbles; Q6_K = 128 bytes of low nibbles | 64 bytes of high bit pairs | 16 int8 scales | d (fp16).
#include "llm_host.hpp"

#include <cstring>

namespace llm::host {
namespace {

float halfToFloat(const uint8_t* p) {
    const uint32_t h = uint32_t(p[0]) | uint32_t(p[1]) << 8;
    const uint32_t sign = (h >> 15) << 31, exponent = (h >> 10) & 31u, fraction = h & 1023u;
    uint32_t bits = sign;
    if (exponent == 31) bits |= 0x7F800000u | fraction << 13;
    else if (exponent != 0) bits |= (exponent + 112u) << 23 | fraction << 13;
    else if (fraction != 0) {  // subnormal half: renormalise
        int shift = 0;
        uint32_t f = fraction;
        while ((f & 0x400u) == 0) f <<= 1, ++shift;
        bits |= uint32_t(113 - shift) << 23 | (f & 1023u) << 13;
    }
    float out;
    std::memcpy(&out, &bits, sizeof out);
    return out;
}

void expandQ4K(const uint8_t* block, float* y) {
    const float d = halfToFloat(block), dmin = halfToFloat(block + 2);
    const uint8_t* packed = block + 4;   // sub-blocks 0..3: six low bits of bytes 0..3 (scales) and 4..7 (mins);
    const uint8_t* nibbles = block + 16;  // sub-blocks 4..7: nibbles of bytes 8..11 plus the two high bits of the first eight
    for (int sub = 0; sub < 8; ++sub) {
        int scale, minimum;
        if (sub < 4) {
            scale = packed[sub] & 63;
            minimum = packed[sub + 4] & 63;
        } else {
            scale = (packed[sub + 4] & 15) | (packed[sub - 4] >> 6) << 4;
            minimum = (packed[sub + 4] >> 4) | (packed[sub] >> 6) << 4;
        }
        const float step = d * float(scale), offset = dmin * float(minimum);
        const uint8_t* src = nibbles + 32 * (sub / 2);
        const int shift = 4 * (sub & 1);
        for (int i = 0; i < 32; ++i) y[32 * sub + i] = step * float((src[i] >> shift) & 15) - offset;
    }
}

void expandQ6K(const uint8_t* block, float* y) {
    const uint8_t *low = block, *high = block + 128;
    const int8_t* scales = reinterpret_cast<const int8_t*>(block + 192);
    const float d = halfToFloat(block + 208);
    for (int half = 0; half < 2; ++half)       // 128 values each
        for (int quarter = 0; quarter < 4; ++quarter)
            for (int i = 0; i < 32; ++i) {
                const int byte = low[64 * half + 32 * (quarter & 1) + i];
                const int nibble = quarter < 2 ? byte & 15 : byte >> 4;
                const int top = (high[32 * half + i] >> (2 * quarter)) & 3;
                const int q = (nibble | top << 4) - 32;
                y[128 * half + 32 * quarter + i] = d * float(scales[8 * half + 2 * quarter + i / 16]) * float(q);
            }
}

}  // namespace

void expandRow(const uint8_t* blocks, bool q6, int row, int width, float* out) {
    const size_t per_row = size_t(width / 256), bytes = q6 ? 210 : 144;
    const uint8_t* first = blocks + size_t(row) * per_row * bytes;
    for (size_t b = 0; b < per_row; ++b) (q6 ? expandQ6K : expandQ4K)(first + b * bytes, out + 256 * b);
}

}  // namespace llm::host
