// Software bfloat16 for host-side code: storage type only, arithmetic happens in float.
// Conversion rule = the reference's (xstar_cpp/src/bfloat16.cpp:5-25): round to nearest, ties to even,
// on the upper 16 bits of the IEEE-754 single.
#pragma once
#include <cstdint>
#include <cstring>

struct bfloat16 {
    std::uint16_t bits;

    bfloat16() = default;
    explicit bfloat16(float value) : bits(round_from(value)) {}
    static bfloat16 from_bits(std::uint16_t b)
    {
        bfloat16 r;
        r.bits = b;
        return r;
    }
    operator float() const
    {
        const std::uint32_t wide = static_cast<std::uint32_t>(bits) << 16;
        float out;
        std::memcpy(&out, &wide, sizeof out);
        return out;
    }

private:
    static std::uint16_t round_from(float value)
    {
        std::uint32_t u;
        std::memcpy(&u, &value, sizeof u);
        u += 0x7FFFu + ((u >> 16) & 1u);
        return static_cast<std::uint16_t>(u >> 16);
    }
};
static_assert(sizeof(bfloat16) == 2, "bfloat16 must be two bytes");
