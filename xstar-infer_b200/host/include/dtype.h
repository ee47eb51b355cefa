// Element kinds the MoE path stores.  The engine's dense ops know two (f32, bf16: reference
// xstar_cpp/include/dtype.h:8-12); the MoE layer adds byte-wide storage kinds for quantised experts,
// their scales, and 32-bit indices.
#pragma once
#include <cstddef>
#include <stdexcept>

enum class DType {
    Float32,
    BFloat16,
    Float8E4M3,   // one e4m3 code per byte
    Float4E2M1x2, // two e2m1 codes per byte (low nibble = even index); shapes count BYTES in the last dim
    UE8M0,        // power-of-two scale, biased exponent
    Int32,
    UInt8, // raw bytes: how a checkpoint file stores packed FP4 codes and e8m0 scales before the loader tags them
};

inline std::size_t dtype_size(DType d)
{
    switch (d) {
    case DType::Float32:
    case DType::Int32:
        return 4;
    case DType::BFloat16:
        return 2;
    case DType::Float8E4M3:
    case DType::Float4E2M1x2:
    case DType::UE8M0:
    case DType::UInt8:
        return 1;
    }
    throw std::runtime_error("unknown DType");
}

inline const char *dtype_name(DType d)
{
    switch (d) {
    case DType::Float32: return "Float32";
    case DType::BFloat16: return "BFloat16";
    case DType::Float8E4M3: return "Float8E4M3";
    case DType::Float4E2M1x2: return "Float4E2M1x2";
    case DType::UE8M0: return "UE8M0";
    case DType::Int32: return "Int32";
    case DType::UInt8: return "UInt8";
    }
    return "?";
}
