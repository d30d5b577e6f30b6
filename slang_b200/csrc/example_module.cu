// Stand-alone device module with the two literal example entry points.
//
// Built with `nvcc -cubin` into slang_b200/mlp_training_kernels.cubin: a CUDA module a host can hand
// to cuModuleLoadData in place of the module slang-rhi's CUDA backend builds from
// examples/mlp-training/kernels.slang, and launch as tools/gfx/cuda/cuda-command-queue.cpp:122-147
// does (one packed parameter buffer, block (256,1,1)).
#include "example_kernels.cuh"
