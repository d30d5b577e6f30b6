// The example's host program written against include/slang_b200_mlp.h instead of slang-rhi.
//
// It follows the steps of ExampleProgram::execute in the reference
// (examples/mlp-training/mlp-training.cpp:92-214): create the device, look the two compute kernels up by
// name, lay the parameters of the 4 -> 16 -> 4 network out in one buffer of two congruent segments
// (parameters, gradients) with 64-byte sub-allocations, fill segment 1 from srand(1072) / rand(), create the
// optimiser-state, network-constant, input and loss buffers, then for 1000 iterations clear the loss,
// dispatch learnGradient over one group and adjustParameters over the parameter segment, and every tenth
// iteration wait and read the loss word back.  Every rhi call of that program maps to one call below.
//
// Built and run by tests/test_host_loop.py: g++ sees the public header exactly as a client would.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "slang_b200_mlp.h"

namespace {

#define CHECK(call)                                                                        \
    do {                                                                                   \
        int32_t rc_ = (call);                                                              \
        if (rc_ != MLP_OK) {                                                               \
            std::fprintf(stderr, "%s failed (%d): %s\n", #call, rc_, mlp_last_error_string()); \
            return 1;                                                                      \
        }                                                                                  \
    } while (0)

// float -> half bits the way the example's host does it: truncate to eleven mantissa bits and add the
// dropped bit back (round half up), no IEEE ties-to-even (examples/mlp-training/mlp-training.cpp:314-339).
// Enough for the values this program converts (finite, magnitude at most 1).
uint16_t to_half_bits(float v)
{
    uint32_t u;
    std::memcpy(&u, &v, 4);
    const uint16_t sign = uint16_t((u >> 16) & 0x8000u);
    const int exp = int((u >> 23) & 0xffu);
    const uint32_t man12 = (u >> 12) & 0x7ffu;  // eleven kept bits and the first dropped one
    if (exp < 103) return sign;                  // below half of the smallest subnormal
    if (exp < 113) {                             // subnormal half
        const uint32_t m = man12 | 0x800u;
        return uint16_t(sign | ((m >> (114 - exp)) + ((m >> (113 - exp)) & 1u)));
    }
    return uint16_t((sign | uint16_t((exp - 112) << 10) | uint16_t(man12 >> 1)) + (man12 & 1u));
}

struct SubAllocation { size_t offset, bytes; };

// allocateNetworkParameterStorage: one running offset, every sub-allocation rounded up to 64 bytes.
struct Arena {
    size_t size = 0;
    SubAllocation take(size_t bytes)
    {
        SubAllocation s{size, bytes};
        size += (bytes + 63) / 64 * 64;
        return s;
    }
};

}  // namespace

int main(int argc, char** argv)
{
    const int iterations = argc > 1 ? std::atoi(argv[1]) : 1000;
    const int layer_sizes[] = {4, 16, 4};
    const int n_layers = 2;

    MlpDevice* device = nullptr;
    CHECK(mlp_device_create(0, &device));
    MlpKernel *learn = nullptr, *adjust = nullptr;
    CHECK(mlp_kernel_get(device, "learnGradient", &learn));
    CHECK(mlp_kernel_get(device, "adjustParameters", &adjust));

    // Segment 1: weights and biases of every layer; segment 2: their gradients at the same offsets.
    Arena arena;
    SubAllocation weights[2], biases[2];
    for (int l = 0; l < n_layers; ++l) {
        weights[l] = arena.take(size_t(layer_sizes[l]) * layer_sizes[l + 1] * sizeof(uint16_t));
        biases[l] = arena.take(size_t(layer_sizes[l + 1]) * sizeof(uint16_t));
    }
    const size_t segment_bytes = arena.size;
    const size_t param_count = segment_bytes / sizeof(uint16_t);
    std::vector<uint16_t> init(2 * param_count, 0);
    std::srand(1072);
    for (size_t i = 0; i < param_count; ++i)
        init[i] = to_half_bits(float(std::rand()) / float(RAND_MAX) * 2.0f - 1.0f);

    MlpBuffer *params = nullptr, *states = nullptr, *network = nullptr, *inputs = nullptr, *loss = nullptr;
    CHECK(mlp_buffer_create(device, 2 * segment_bytes, init.data(), &params));
    CHECK(mlp_buffer_create(device, param_count * sizeof(MlpExampleAdamState), nullptr, &states));
    CHECK(mlp_buffer_clear(device, states, 0, param_count * sizeof(MlpExampleAdamState)));

    const uint64_t base = mlp_buffer_address(params);
    MlpLayerPointers net[2];
    for (int l = 0; l < n_layers; ++l) {
        net[l].weights = base + weights[l].offset;
        net[l].weightsGrad = base + segment_bytes + weights[l].offset;
        net[l].biases = base + biases[l].offset;
        net[l].biasesGrad = base + segment_bytes + biases[l].offset;
    }
    CHECK(mlp_buffer_create(device, sizeof net, net, &network));

    float input_values[32];
    for (float& v : input_values) v = float(std::rand()) / float(RAND_MAX);
    CHECK(mlp_buffer_create(device, sizeof input_values, input_values, &inputs));
    CHECK(mlp_buffer_create(device, 8, nullptr, &loss));

    const uint32_t sample_count = 16;
    for (int k = 0; k < iterations; ++k) {
        CHECK(mlp_buffer_clear(device, loss, 0, 8));
        MlpLearnGradParams lg{};
        lg.networkBuffer = mlp_buffer_address(network);
        lg.lossBuffer = mlp_buffer_address(loss);
        lg.inputs = mlp_buffer_address(inputs);
        lg.count = sample_count;
        CHECK(mlp_dispatch(device, learn, &lg, sizeof lg, (sample_count + 255) / 256, 1, 1));
        MlpAdjustParamsParams ap{};
        ap.adamStates = mlp_buffer_address(states);
        ap.params = base;
        ap.gradients = base + segment_bytes;
        ap.count = uint32_t(param_count);
        CHECK(mlp_dispatch(device, adjust, &ap, sizeof ap, (uint32_t(param_count) + 255) / 256, 1, 1));
        if (k % 10 == 0) {
            CHECK(mlp_wait(device));
            uint32_t word = 0;
            CHECK(mlp_buffer_read(device, loss, 0, 4, &word));
            float value;
            std::memcpy(&value, &word, 4);
            std::printf("Loss after %d iterations: %f [0x%08x]\n", k, value, word);
        }
    }
    CHECK(mlp_wait(device));
    std::vector<uint16_t> final_params(param_count);
    CHECK(mlp_buffer_read(device, params, 0, segment_bytes, final_params.data()));
    std::printf("launches: %llu\n", (unsigned long long)mlp_device_launch_count(device));

    mlp_kernel_destroy(learn);
    mlp_kernel_destroy(adjust);
    for (MlpBuffer* b : {params, states, network, inputs, loss}) mlp_buffer_destroy(b);
    mlp_device_destroy(device);
    return 0;
}
