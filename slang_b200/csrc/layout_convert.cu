// Network parameter layout conversion: portable (row-major per layer, bias right behind its weights,
// no padding) <-> the neural module's CUDA-optimal layout (every layer padded to multiples of 16,
// weights cut into 16x16 tiles ordered input-tile-major, each tile stored in the register order of a
// tensor-core B fragment, then a padded bias slot that is reserved even for layers without a bias).
// Restates NetworkParameterLayoutConverter.toOptimalLayout / toPortableLayout
// (source/standard-modules/neural/network-parameter-layout-converter.slang:469-555, CUDA tile order
// :54-68, 176-181) as grid-stride permutation kernels; the golden model it is tested against is the
// reference's own (tools/gfx-unit-test/neural-slang-network-converter.cpp:76-126).
#include <cuda_runtime.h>

#include <string>

#include "launchers.h"

namespace mlpb200 {

struct ShapeDev {
    int n_layers;
    int in[MLP_MAX_LAYERS], out[MLP_MAX_LAYERS], has_bias[MLP_MAX_LAYERS];
    long long logical_off[MLP_MAX_LAYERS + 1], physical_off[MLP_MAX_LAYERS + 1];
};

__host__ __device__ inline int align16(int v) { return (v + 15) / 16 * 16; }

// Position of (row = input within the tile, col = output within the tile) in the 256-element tile.
__host__ __device__ inline int native_tile_pos(int row, int col)
{
    const int row_group = row >> 3, row_in_group = row & 7;
    const int tid_local = row_in_group >> 1, pair = row_in_group & 1;
    const int sub = col >> 3, gid = col & 7;
    return (gid * 4 + tid_local) * 8 + sub * 4 + row_group * 2 + pair;
}

__host__ __device__ inline long long physical_weight_offset(const ShapeDev& s, int l, int output, int input)
{
    const int tile_cols = align16(s.out[l]) / 16;
    const long long tile_base = (long long)((input / 16) * tile_cols + output / 16) * 256;
    return tile_base + native_tile_pos(input % 16, output % 16);
}

template <typename T>
__global__ void to_optimal_kernel(ShapeDev s, const T* __restrict__ portable, T* __restrict__ optimal)
{
    const long long total = s.physical_off[s.n_layers];
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        int l = 0;
        while (e >= s.physical_off[l + 1]) ++l;
        const long long r = e - s.physical_off[l];
        const int pin = align16(s.in[l]), pout = align16(s.out[l]);
        const long long nw = (long long)pin * pout;
        T v = T(0);
        if (r < nw) {
            // invert the tile order and the in-tile fragment order
            const int tile = (int)(r / 256), pos = (int)(r % 256);
            const int tile_cols = pout / 16;
            const int lane = pos / 8, local = pos % 8;
            const int sub = local / 4, row_group = (local % 4) / 2, pair = local % 2;
            const int col = (lane / 4) + 8 * sub, row = (lane % 4) * 2 + pair + 8 * row_group;
            const int input = (tile / tile_cols) * 16 + row, output = (tile % tile_cols) * 16 + col;
            if (input < s.in[l] && output < s.out[l]) v = portable[s.logical_off[l] + (long long)output * s.in[l] + input];
        } else {
            const int j = (int)(r - nw);
            if (s.has_bias[l] && j < s.out[l]) v = portable[s.logical_off[l] + (long long)s.in[l] * s.out[l] + j];
        }
        optimal[e] = v;
    }
}

template <typename T>
__global__ void to_portable_kernel(ShapeDev s, const T* __restrict__ optimal, T* __restrict__ portable)
{
    const long long total = s.logical_off[s.n_layers];
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        int l = 0;
        while (e >= s.logical_off[l + 1]) ++l;
        const long long r = e - s.logical_off[l];
        const long long nw = (long long)s.in[l] * s.out[l];
        long long src;
        if (r < nw) src = s.physical_off[l] + physical_weight_offset(s, l, (int)(r / s.in[l]), (int)(r % s.in[l]));
        else src = s.physical_off[l] + (long long)align16(s.in[l]) * align16(s.out[l]) + (r - nw);
        portable[e] = optimal[src];
    }
}

static bool make_shape(const MlpNetworkShape& n, ShapeDev* s, std::string* err)
{
    if (n.n_layers < 1 || n.n_layers > MLP_MAX_LAYERS) { if (err) *err = "n_layers out of range"; return false; }
    if (n.elem_bytes != 2 && n.elem_bytes != 4) { if (err) *err = "element size must be 2 or 4 bytes"; return false; }
    s->n_layers = n.n_layers;
    long long lo = 0, po = 0;
    for (int l = 0; l < n.n_layers; ++l) {
        if (n.dims[l] < 1 || n.dims[l + 1] < 1) { if (err) *err = "layer width out of range"; return false; }
        s->in[l] = n.dims[l];
        s->out[l] = n.dims[l + 1];
        s->has_bias[l] = (int)((n.bias_mask >> l) & 1u);
        s->logical_off[l] = lo;
        s->physical_off[l] = po;
        lo += (long long)n.dims[l] * n.dims[l + 1] + (s->has_bias[l] ? n.dims[l + 1] : 0);
        po += (long long)align16(n.dims[l]) * align16(n.dims[l + 1]) + align16(n.dims[l + 1]);
    }
    s->logical_off[n.n_layers] = lo;
    s->physical_off[n.n_layers] = po;
    return true;
}

bool layout_sizes(const MlpNetworkShape& n, long long* logical, long long* physical, std::string* err)
{
    ShapeDev s;
    if (!make_shape(n, &s, err)) return false;
    *logical = s.logical_off[n.n_layers];
    *physical = s.physical_off[n.n_layers];
    return true;
}

cudaError_t launch_layout_convert(cudaStream_t st, const MlpNetworkShape& n, bool to_optimal, const void* src, void* dst,
                                  int* launches, std::string* err)
{
    ShapeDev s;
    if (!make_shape(n, &s, err)) return cudaErrorInvalidValue;
    const long long total = to_optimal ? s.physical_off[n.n_layers] : s.logical_off[n.n_layers];
    const int grid = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    if (n.elem_bytes == 4) {
        if (to_optimal) to_optimal_kernel<float><<<grid, 256, 0, st>>>(s, (const float*)src, (float*)dst);
        else to_portable_kernel<float><<<grid, 256, 0, st>>>(s, (const float*)src, (float*)dst);
    } else {
        if (to_optimal) to_optimal_kernel<unsigned short><<<grid, 256, 0, st>>>(s, (const unsigned short*)src, (unsigned short*)dst);
        else to_portable_kernel<unsigned short><<<grid, 256, 0, st>>>(s, (const unsigned short*)src, (unsigned short*)dst);
    }
    *launches += 1;
    return cudaGetLastError();
}

}  // namespace mlpb200
