// Host-side launch functions implemented by the kernel translation units and called by the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <string>

#include "../../include/slang_b200_mlp.h"

namespace mlpb200 {

// One-thread-per-sample kernels (simt_kernels.cu).
cudaError_t launch_example_learn_gradient(cudaStream_t st, const MlpLearnGradParams& a, uint32_t grid);
cudaError_t launch_example_learn_gradient_coopvec(cudaStream_t st, const MlpLearnGradParams& a, uint32_t grid);
cudaError_t launch_example_adjust_parameters(cudaStream_t st, const MlpAdjustParamsParams& a, uint32_t grid);
cudaError_t launch_forward_simt(cudaStream_t st, const MlpConfig& c, const MlpForwardParams& a, int* launches,
                                std::string* err);
cudaError_t launch_learn_gradient_simt(cudaStream_t st, const MlpConfig& c, const MlpLearnGradParamsEx& a,
                                       float* seq_scratch, int* launches, std::string* err,
                                       float* input_grads = nullptr);
size_t sequential_scratch_floats_per_sample(const MlpConfig& c);
cudaError_t launch_adjust_parameters(cudaStream_t st, const MlpConfig& c, const MlpAdjustParamsParams& a, int* launches);

// Parameter layout conversion (layout_convert.cu).
bool layout_sizes(const MlpNetworkShape& n, long long* logical, long long* physical, std::string* err);
cudaError_t launch_layout_convert(cudaStream_t st, const MlpNetworkShape& n, bool to_optimal, const void* src, void* dst,
                                  int* launches, std::string* err);

// Matrix layout conversion of the cooperative-vector host calls (matrix_convert.cu).
bool matrix_size(uint32_t rows, uint32_t cols, int32_t component_type, int32_t layout, size_t stride, size_t* size,
                 std::string* err);
cudaError_t launch_matrix_convert(cudaStream_t st, uint64_t dst_base, const MlpMatrixDesc* dst, uint64_t src_base,
                                  const MlpMatrixDesc* src, uint32_t n, int* launches, std::string* err);

// Tensor-core kernels (tc_kernels.cu).  tc_supported() says whether the shape is one they are built for.
bool tc_forward_supported(const MlpConfig& c);
bool tc_train_supported(const MlpConfig& c);
bool tc_train_narrow_supported(const MlpConfig& c);
struct TcWorkspace;  // per-device state: status word, SM count, tensor maps cache
TcWorkspace* tc_workspace_create(int device_ordinal, std::string* err);
void tc_workspace_destroy(TcWorkspace* ws);
cudaError_t launch_forward_tc(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a,
                              int* launches, std::string* err);
// input_grads (optional): [count][dims[0]] fp32 gradient with respect to the inputs (no input encoding).
cudaError_t launch_learn_gradient_tc(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c,
                                     const MlpLearnGradParamsEx& a, int* launches, std::string* err,
                                     float* input_grads = nullptr);
// Forward pass of the wide (zero-padded 64-128-...-64) kernel's shapes; fp32 outputs.
bool tc_forward_wide_supported(const MlpConfig& c);
cudaError_t launch_forward_wide(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a,
                                int* launches, std::string* err);
// input_grads (optional): [count][dims[0]] fp32 gradient with respect to the inputs (no input encoding).
cudaError_t launch_learn_gradient_narrow(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c,
                                         const MlpLearnGradParamsEx& a, int* launches, std::string* err,
                                         float* input_grads = nullptr);
// Forward pass of the same padded kernel (any widths up to 64, any activation, input conversion or the
// frequency encoding); fp32 outputs.
cudaError_t launch_forward_narrow(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a,
                                  int* launches, std::string* err);
// Developer builds (-DMLPB200_TRACE) only: time stamps CTA 0 of the last wide learnGradient recorded.
cudaError_t tc_read_timing(cudaStream_t st, TcWorkspace* ws, unsigned long long* out256);
// Reads and clears the device status word (0 = no kernel gave up on a bounded wait).
cudaError_t tc_read_status(cudaStream_t st, TcWorkspace* ws, uint32_t* status);

}  // namespace mlpb200
