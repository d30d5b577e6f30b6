// Handle layouts shared by the translation units that implement the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "launchers.h"

struct MlpDevice {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    uint64_t launches = 0;
    float* seq_scratch = nullptr;  // per-sample vectors of the sequential-sum mode
    size_t seq_scratch_floats = 0;
    mlpb200::TcWorkspace* tc = nullptr;
};

namespace mlpb200 {
// Sets the text mlp_last_error_string() returns on this thread (abi.cu).
void set_last_error(const char* text);
// Validity of a problem description: ranges of every enumerated field, widths, encoding consistency.
bool config_ok(const MlpConfig* c, std::string* why);
}  // namespace mlpb200
