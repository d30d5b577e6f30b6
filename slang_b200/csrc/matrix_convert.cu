// Matrix layout queries and conversion: the two host calls the cooperative-vector example makes besides
// the common ones, getCooperativeVectorMatrixSize and convertCooperativeVectorMatrix
// (examples/mlp-training-coopvec/mlp-training-coopvec.cpp:201-236, 305-311).
//
// Layouts (numbered like CoopVecMatrixLayout, source/slang/hlsl.meta.slang:32547-32553): row-major and
// column-major with a byte stride between rows / columns (0 = tightly packed), and the two "optimal"
// layouts, which the reference leaves to the driver.  Here both optimal layouts are the same documented
// format: rows and columns padded with zeros to multiples of 16, stored as 16x16 tiles, tiles in
// row-major order of the tile grid, elements row-major inside a tile.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "launchers.h"
#include "mlp_common.cuh"

namespace mlpb200 {

namespace {

__host__ __device__ inline uint32_t pad16(uint32_t v) { return (v + 15u) & ~15u; }
__host__ __device__ inline int elem_size(int32_t t) { return t == MLP_F32 ? 4 : 2; }

// Byte offset of element (r, c) inside a matrix of the given description (without desc.offset).
__host__ __device__ inline size_t elem_offset(const MlpMatrixDesc& d, uint32_t r, uint32_t c)
{
    const size_t es = (size_t)elem_size(d.component_type);
    switch (d.layout) {
    case MLP_MATRIX_ROW_MAJOR: return size_t(r) * (d.row_col_stride ? d.row_col_stride : d.cols * es) + c * es;
    case MLP_MATRIX_COLUMN_MAJOR: return size_t(c) * (d.row_col_stride ? d.row_col_stride : d.rows * es) + r * es;
    default: {
        const uint32_t tiles_c = pad16(d.cols) / 16;
        return ((size_t(r / 16) * tiles_c + c / 16) * 256 + (r % 16) * 16 + (c % 16)) * es;
    }
    }
}

__device__ inline float load_elem(const uint8_t* p, int32_t t)
{
    if (t == MLP_F32) return *(const float*)p;
    if (t == MLP_F16) return __half2float(*(const __half*)p);
    return __bfloat162float(*(const __nv_bfloat16*)p);
}
__device__ inline void store_elem(uint8_t* p, int32_t t, float v)
{
    if (t == MLP_F32) *(float*)p = v;
    else if (t == MLP_F16) *(__half*)p = __float2half_rn(v);
    else *(__nv_bfloat16*)p = __float2bfloat16_rn(v);
}

struct ConvertJob { MlpMatrixDesc dst, src; uint64_t dst_base, src_base; };

// One thread per element of the destination's padded extent: padding elements of an optimal layout are
// written as zeros; a row-/column-major destination has no padding elements.
__global__ void matrix_convert_kernel(ConvertJob job)
{
    const bool dst_opt = job.dst.layout >= MLP_MATRIX_INFERENCING_OPTIMAL;
    const uint32_t R = dst_opt ? pad16(job.dst.rows) : job.dst.rows, Cc = dst_opt ? pad16(job.dst.cols) : job.dst.cols;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= size_t(R) * Cc) return;
    const uint32_t r = uint32_t(idx / Cc), c = uint32_t(idx % Cc);
    float v = 0.0f;
    if (r < job.src.rows && c < job.src.cols)
        v = load_elem((const uint8_t*)job.src_base + job.src.offset + elem_offset(job.src, r, c), job.src.component_type);
    store_elem((uint8_t*)job.dst_base + job.dst.offset + elem_offset(job.dst, r, c), job.dst.component_type, v);
}

bool desc_ok(const MlpMatrixDesc& d, std::string* err)
{
    if (d.rows == 0 || d.cols == 0 || d.rows > (1u << 20) || d.cols > (1u << 20)) { *err = "matrix extent out of range"; return false; }
    if (d.component_type < MLP_F32 || d.component_type > MLP_BF16) { *err = "unknown component type"; return false; }
    if (d.layout < MLP_MATRIX_ROW_MAJOR || d.layout > MLP_MATRIX_TRAINING_OPTIMAL) { *err = "unknown matrix layout"; return false; }
    const size_t es = (size_t)elem_size(d.component_type);
    if (d.layout == MLP_MATRIX_ROW_MAJOR && d.row_col_stride && d.row_col_stride < d.cols * es) { *err = "row stride smaller than a row"; return false; }
    if (d.layout == MLP_MATRIX_COLUMN_MAJOR && d.row_col_stride && d.row_col_stride < d.rows * es) { *err = "column stride smaller than a column"; return false; }
    if ((d.row_col_stride % es) || (d.offset % es)) { *err = "stride and offset must be multiples of the element size"; return false; }
    size_t need = 0;
    if (!matrix_size(d.rows, d.cols, d.component_type, d.layout, d.row_col_stride, &need, err)) return false;
    if (d.size < need) { *err = "matrix description's size is smaller than its layout needs"; return false; }
    return true;
}

}  // namespace

bool matrix_size(uint32_t rows, uint32_t cols, int32_t component_type, int32_t layout, size_t stride, size_t* size,
                 std::string* err)
{
    if (rows == 0 || cols == 0 || rows > (1u << 20) || cols > (1u << 20)) { *err = "matrix extent out of range"; return false; }
    if (component_type < MLP_F32 || component_type > MLP_BF16) { *err = "unknown component type"; return false; }
    const size_t es = (size_t)elem_size(component_type);
    switch (layout) {
    case MLP_MATRIX_ROW_MAJOR: *size = stride ? size_t(rows - 1) * stride + cols * es : size_t(rows) * cols * es; return true;
    case MLP_MATRIX_COLUMN_MAJOR: *size = stride ? size_t(cols - 1) * stride + rows * es : size_t(rows) * cols * es; return true;
    case MLP_MATRIX_INFERENCING_OPTIMAL:
    case MLP_MATRIX_TRAINING_OPTIMAL: *size = size_t(pad16(rows)) * pad16(cols) * es; return true;
    default: *err = "unknown matrix layout"; return false;
    }
}

cudaError_t launch_matrix_convert(cudaStream_t st, uint64_t dst_base, const MlpMatrixDesc* dst, uint64_t src_base,
                                  const MlpMatrixDesc* src, uint32_t n, int* launches, std::string* err)
{
    *launches = 0;
    for (uint32_t i = 0; i < n; ++i) {
        if (!desc_ok(dst[i], err) || !desc_ok(src[i], err)) return cudaErrorInvalidValue;
        if (dst[i].rows != src[i].rows || dst[i].cols != src[i].cols) { *err = "source and destination extents differ"; return cudaErrorInvalidValue; }
        const uint64_t d0 = dst_base + dst[i].offset, d1 = d0 + dst[i].size, s0 = src_base + src[i].offset, s1 = s0 + src[i].size;
        if (d0 < s1 && s0 < d1) { *err = "source and destination ranges overlap"; return cudaErrorInvalidValue; }
    }
    for (uint32_t i = 0; i < n; ++i) {
        ConvertJob job{dst[i], src[i], dst_base, src_base};
        const bool dst_opt = dst[i].layout >= MLP_MATRIX_INFERENCING_OPTIMAL;
        const size_t total = size_t(dst_opt ? pad16(dst[i].rows) : dst[i].rows) * (dst_opt ? pad16(dst[i].cols) : dst[i].cols);
        matrix_convert_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(job);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ++*launches;
    }
    return cudaSuccess;
}

}  // namespace mlpb200
