// Where a Tensor's bytes live (same two places as the reference engine, xstar_cpp/include/device.h).
#pragma once

enum class Device {
    CPU,
    CUDA,
};
