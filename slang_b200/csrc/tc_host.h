// Host-side state shared by the tensor-core translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

namespace mlpb200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TcWorkspace {
    int ordinal = 0;
    int sm_count = 0;
    uint32_t* status = nullptr;            // device word, set by kernels that give up on a wait
    uint32_t* status_host = nullptr;       // pinned copy
    unsigned long long* timing = nullptr;  // device; allocated by developer trace builds only
    EncodeTiledFn encode = nullptr;        // cuTensorMapEncodeTiled, fetched through the runtime
    void* input_rows = nullptr;            // device; 16-bit copy of fp32 input rows for the kernels that take them by TMA
    size_t input_rows_bytes = 0;
};

// A [rows][cols] row-major matrix viewed in boxes of box_rows x box_cols elements.
bool make_tile_map(TcWorkspace* ws, CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, uint64_t base, uint64_t rows,
                   uint32_t cols, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle, std::string* err);

}  // namespace mlpb200
