/*
 * C ABI of the B200 small-MLP training step.
 *
 * The reference's example host loop (examples/mlp-training/mlp-training.cpp:92-214) talks to the GPU
 * through slang-rhi: create a device, load two compute kernels by name, create buffers, clear them,
 * dispatch a kernel with one packed argument struct and a grid size, wait, read a buffer back.  Each
 * function below stands in for one of those calls, so a copy of that loop can be compiled against
 * this header instead of slang-rhi.  Kernels are prebuilt for sm_100a; nothing is compiled at run time.
 *
 * Conventions (include/slang.h:1377-1426 of the reference): every function returns an int32 result,
 * 0 on success and negative on failure; no exceptions cross the boundary; the text of the last failure
 * on the calling thread is available from mlp_last_error_string().  Handles are opaque and are
 * destroyed explicitly.  A device handle owns one in-order CUDA stream (or borrows the caller's);
 * calls on one device handle are not thread-safe, which matches the example's single host thread and
 * single queue (mlp-training.cpp:174).
 */
#ifndef SLANG_B200_MLP_H
#define SLANG_B200_MLP_H

#include <stddef.h>
#include <stdint.h>

#include "slang_b200_mlp_config.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MLP_OK 0
#define MLP_FAIL (-1)             /* SLANG_FAIL */
#define MLP_E_INVALID_ARG (-2)    /* SLANG_E_INVALID_ARG */
#define MLP_E_NOT_AVAILABLE (-3)  /* SLANG_E_NOT_AVAILABLE: no kernel of that name / unsupported shape */
#define MLP_E_CUDA (-4)           /* a CUDA call failed; see mlp_last_error_string() */
#define MLP_E_DEVICE_STATUS (-5)  /* a kernel gave up on a bounded wait and set its status word */
#define MLP_E_COMM (-6)           /* a collective failed asynchronously or ran past its time limit; communicator aborted */

typedef struct MlpDevice MlpDevice;
typedef struct MlpBuffer MlpBuffer;
typedef struct MlpKernel MlpKernel;

/* ---- argument structs packed by the host, one per entry point ------------------------------- */

/* learnGradient of the literal example: LearnGradParams (mlp-training.cpp:55-61), 28 bytes used. */
typedef struct MlpLearnGradParams {
    uint64_t networkBuffer; /* device address of MlpLayerPointers[n_layers] */
    uint64_t lossBuffer;    /* device address of two 32-bit words, cleared by the host every step */
    uint64_t inputs;        /* device address of the inputs */
    uint32_t count;         /* samples */
} MlpLearnGradParams;

/* adjustParameters: AdjustParamsParams (mlp-training.cpp:63-69), 28 bytes used. */
typedef struct MlpAdjustParamsParams {
    uint64_t adamStates;
    uint64_t params;
    uint64_t gradients;
    uint32_t count; /* elements of the padded parameter segment */
} MlpAdjustParamsParams;

/* learnGradient of the configurable path: the example's struct plus a targets address, because the
 * benchmark configurations read their targets from a buffer instead of computing a closed form
 * inside the kernel (examples/mlp-training/network.slang:49-58 is the closed form of the example). */
typedef struct MlpLearnGradParamsEx {
    uint64_t networkBuffer;
    uint64_t lossBuffer; /* word 0: float bits of the largest per-sample loss (unsigned max);
                            word 1: float sum of the per-sample losses (atomic add) */
    uint64_t inputs;
    uint64_t targets;
    uint32_t count;
    uint32_t flags; /* MLP_FLAG_* */
} MlpLearnGradParamsEx;

/* MlpLearnGradParamsEx plus a destination for the gradient with respect to the inputs (fp32
 * [count][dims[0]], values rounded to the network's storage type), written when flags has
 * MLP_FLAG_INPUT_GRADIENT.  The example marks its inputs no_diff (examples/mlp-training/network.slang:36-43),
 * so this has no counterpart there; the neural module's layers do return it (FFLayer's reverse pass,
 * source/standard-modules/neural/layers.slang:34-110) and a trainable input encoder needs it. */
typedef struct MlpLearnGradParamsEx2 {
    MlpLearnGradParamsEx base;
    uint64_t inputGradients;
} MlpLearnGradParamsEx2;

/* forward only: outputs are fp32 [count][dims[n_layers]], or the network's storage type with
 * MLP_FLAG_OUTPUT_STORAGE_TYPE (for feeding another network's targets). */
typedef struct MlpForwardParams {
    uint64_t networkBuffer;
    uint64_t inputs;
    uint64_t outputs;
    uint32_t count;
    uint32_t flags;
} MlpForwardParams;

/* Gradient sums in ascending sample order, one add at a time, as the reference's CPU target runs
 * them (source/slang/slang-emit-cpp.cpp:2210-2284): bit-identical to a sequential machine, slow. */
#define MLP_FLAG_SEQUENTIAL_SUM 1u
/* forward: write the outputs rounded to the network's storage type (tensor-core path only). */
#define MLP_FLAG_OUTPUT_STORAGE_TYPE 2u
/* learnGradient with MlpLearnGradParamsEx2: also write the input gradients (networks without an input
 * encoding; on the tensor cores wherever learnGradient itself runs there, else one thread per sample). */
#define MLP_FLAG_INPUT_GRADIENT 4u

/* ---- device ------------------------------------------------------------------------------- */

/* rhi::getRHI()->createDevice (mlp-training.cpp:96-100).  `ordinal` is the CUDA device index. */
int32_t mlp_device_create(int32_t ordinal, MlpDevice** out_device);
/* Same, but work is issued on an existing CUDA stream (a cudaStream_t passed as a pointer) so that
 * the caller's own stream-ordered work (copies, collectives) interleaves with the kernels.  A null
 * handle means the legacy default stream. */
int32_t mlp_device_create_on_stream(int32_t ordinal, void* cuda_stream, MlpDevice** out_device);
int32_t mlp_device_destroy(MlpDevice* device);
/* queue->waitOnHost() (mlp-training.cpp:207).  Also reports a pending device status word. */
int32_t mlp_wait(MlpDevice* device);

/* ---- buffers ------------------------------------------------------------------------------ */

/* createBuffer(size, initData) (mlp-training.cpp:271-280): device-local, optional initial contents. */
int32_t mlp_buffer_create(MlpDevice* device, size_t size, const void* init_data, MlpBuffer** out_buffer);
/* Adopts device memory owned by the caller (for example a tensor of a host framework). */
int32_t mlp_buffer_wrap(MlpDevice* device, uint64_t device_address, size_t size, MlpBuffer** out_buffer);
int32_t mlp_buffer_destroy(MlpBuffer* buffer);
/* IBuffer::getDeviceAddress() (mlp-training.cpp:148).  Stable for the buffer's lifetime. */
uint64_t mlp_buffer_address(const MlpBuffer* buffer);
/* clearBuffer(buffer[, range]) (mlp-training.cpp:282-289): zero fill, stream ordered. */
int32_t mlp_buffer_clear(MlpDevice* device, MlpBuffer* buffer, size_t offset, size_t size);
/* gDevice->readBuffer(buffer, offset, size, blob) (mlp-training.cpp:208): waits for prior work. */
int32_t mlp_buffer_read(MlpDevice* device, const MlpBuffer* buffer, size_t offset, size_t size, void* dst);
int32_t mlp_buffer_write(MlpDevice* device, MlpBuffer* buffer, size_t offset, size_t size, const void* src);

/* ---- cooperative-vector matrices ------------------------------------------------------------ */

/* Layouts, numbered like CoopVecMatrixLayout (source/slang/hlsl.meta.slang:32547-32553).  The two optimal
 * layouts are one documented format here: rows and columns zero-padded to multiples of 16, 16x16 tiles in
 * row-major tile order, row-major inside a tile. */
enum MlpMatrixLayout {
    MLP_MATRIX_ROW_MAJOR = 0,
    MLP_MATRIX_COLUMN_MAJOR = 1,
    MLP_MATRIX_INFERENCING_OPTIMAL = 2,
    MLP_MATRIX_TRAINING_OPTIMAL = 3,
};
/* rhi::CooperativeVectorMatrixDesc (mlp-training-coopvec.cpp:205-225); component_type is an MlpDType;
 * offset is relative to the buffer address given to mlp_matrix_convert; row_col_stride in bytes, 0 = packed. */
typedef struct MlpMatrixDesc {
    uint32_t rows, cols;
    int32_t component_type, layout;
    uint64_t size, offset, row_col_stride;
} MlpMatrixDesc;
/* getCooperativeVectorMatrixSize(rows, cols, type, layout, stride, &size) (mlp-training-coopvec.cpp:305-311).
 * Needs no device. */
int32_t mlp_matrix_size(uint32_t rows, uint32_t cols, int32_t component_type, int32_t layout, uint64_t row_col_stride,
                        uint64_t* out_size);
/* encoder->convertCooperativeVectorMatrix(dstBuffer, dstDescs, srcBuffer, srcDescs, n)
 * (mlp-training-coopvec.cpp:226-235): layout and component-type conversion, stream ordered.  Ranges must
 * not overlap. */
int32_t mlp_matrix_convert(MlpDevice* device, uint64_t dst_address, const MlpMatrixDesc* dst_descs, uint64_t src_address,
                           const MlpMatrixDesc* src_descs, uint32_t count);

/* ---- gradient exchange between GPUs ------------------------------------------------------- */

/* The reference example runs on one device; a data-parallel run of the same step (one process per
 * GPU, each taking a contiguous block of every batch) needs exactly one exchange: the sum of the flat
 * fp32 gradient segment after learnGradient, before every rank runs the same adjustParameters
 * (examples/mlp-training/mlp-training.cpp:176-212 is the loop this slots into, between the two
 * dispatches).  These calls bind NCCL (resolved at run time; MLP_E_NOT_AVAILABLE without it). */
#define MLP_COMM_ID_BYTES 128
typedef struct MlpComm MlpComm;
/* Rank 0 creates the id and hands its bytes to the other ranks by any channel of the host's. */
int32_t mlp_comm_unique_id(void* id_out, size_t id_bytes);
/* Collective over the nranks processes; device is the rank's own GPU. */
int32_t mlp_comm_init(MlpDevice* device, int32_t nranks, int32_t rank, const void* id, size_t id_bytes,
                      MlpComm** out_comm);
int32_t mlp_comm_destroy(MlpComm* comm);
/* Add the ranks' terms in ascending rank order on every rank (all-gather plus a local ordered sum)
 * instead of an all-reduce: the same bits whatever algorithm the collective library picks. */
#define MLP_COMM_RANK_ORDERED_SUM 1u
/* In place, stream ordered on the device's stream: gradients (count floats) become the sum over the
 * ranks; loss_words (0 to skip) is two floats that combine as (max, sum). */
int32_t mlp_allreduce_grads(MlpDevice* device, MlpComm* comm, uint64_t gradients, size_t count, uint64_t loss_words,
                            uint32_t flags);

/* Waits on the host, with a limit, for everything queued on the device's stream so far (the
 * collectives of mlp_allreduce_grads included), asking the collective library for asynchronous errors
 * while it waits.  MLP_OK: the stream drained.  MLP_E_COMM: the library reported an error (a peer
 * process died, a link failed) or timeout_ms passed; the communicator has been aborted so that nothing
 * stays queued behind a peer that will never arrive, and the handle is good for mlp_comm_destroy only.
 * A data-parallel host calls this where it would otherwise synchronise (before reading the loss).
 * The environment variable SLANG_B200_NCCL_LIBRARY names the collective library file to bind in place
 * of the default search for libnccl.so.2. */
int32_t mlp_comm_wait(MlpDevice* device, MlpComm* comm, uint32_t timeout_ms);

/* ---- kernels ------------------------------------------------------------------------------ */

/* loadComputeProgram / findEntryPointByName (mlp-training.cpp:291-312): the literal example's entry
 * points "learnGradient" and "adjustParameters" (examples/mlp-training/kernels.slang:8-41), and
 * "learnGradient_coopvec", the learnGradient of examples/mlp-training-coopvec/kernels.slang:7-27 (its
 * adjustParameters is the same kernel). */
int32_t mlp_kernel_get(MlpDevice* device, const char* entry_point, MlpKernel** out_kernel);
/* createShaderProgram / createComputePipeline for precompiled device code (mlp-training.cpp:341-377;
 * the CUDA backend loads the module it gets with cuModuleLoadData and looks the entry point up by
 * name).  image is a cubin or PTX module, for example this library's own mlp_training_kernels.cubin
 * or a module built by nvcc from the CUDA source the reference compiler emits for kernels.slang.
 * mlp_dispatch on such a kernel passes the argument bytes unchanged as the kernel's packed parameter
 * buffer and launches block (256,1,1), grid (gx,gy,gz), as tools/gfx/cuda/cuda-command-queue.cpp:122-147
 * does; trailing struct padding beyond the entry point's last parameter is dropped (the pitfall
 * tests/cuda/cuda-kernel-param-layout.slang:1-8 describes).  mlp_kernel_implementation reports "module". */
int32_t mlp_kernel_load(MlpDevice* device, const void* image, size_t image_size, const char* entry_point,
                        MlpKernel** out_kernel);
/* The same entry points specialised for a problem description, the way the reference specialises
 * FeedForwardLayer<In, Out> at compile time.  entry_point is one of
 *   "learnGradient"      args MlpLearnGradParamsEx   (fastest implementation for the shape)
 *   "learnGradient_simt" args MlpLearnGradParamsEx   (one thread per sample, any shape)
 *   "adjustParameters"   args MlpAdjustParamsParams  (MlpAdamState per element, fp32 gradients)
 *   "forward"            args MlpForwardParams
 *   "forward_simt"       args MlpForwardParams */
int32_t mlp_kernel_get_for_config(MlpDevice* device, const MlpConfig* config, const char* entry_point,
                                  MlpKernel** out_kernel);
int32_t mlp_kernel_destroy(MlpKernel* kernel);
/* Name of the implementation a kernel handle resolved to ("simt", "tcgen05", ...). */
const char* mlp_kernel_implementation(const MlpKernel* kernel);

/* dispatchKernel (mlp-training.cpp:252-268): bind, setData(offset 0, &args, size), dispatchCompute.
 * The host passes the grid it would give a [numthreads(256,1,1)] kernel, ceil(count / 256); kernels
 * that are persistent size their own grid and treat the argument as a hint. */
int32_t mlp_dispatch(MlpDevice* device, MlpKernel* kernel, const void* args, size_t args_size,
                     uint32_t grid_x, uint32_t grid_y, uint32_t grid_z);
/* Number of CUDA kernels launched through this device handle since it was created. */
uint64_t mlp_device_launch_count(const MlpDevice* device);

/* ---- parameter layout conversion --------------------------------------------------------------- */

/* A network as the neural module's NetworkParameterLayoutConverter<T, BiasMask, In, Out, Rest...> sees
 * it (source/standard-modules/neural/network-parameter-layout-converter.slang:469-478): layer widths
 * and one bias bit per layer. */
typedef struct MlpNetworkShape {
    int32_t n_layers;
    int32_t dims[MLP_MAX_LAYERS + 1];
    uint64_t bias_mask;  /* bit l set: layer l has a bias */
    int32_t elem_bytes;  /* 4 (float) or 2 (half / bfloat16: a pure permutation of 16-bit patterns) */
    int32_t reserved;
} MlpNetworkShape;

/* ElementCountLogical / ElementCountPhysical of the converter (:480-483). */
int32_t mlp_layout_sizes(const MlpNetworkShape* shape, int64_t* logical_elements, int64_t* physical_elements);
/* toOptimalLayout (:492-520): portable row-major -> 16x16 tiles in tensor-core B-fragment order, padded
 * with zeros, bias slot reserved for every layer.  Device addresses; stream ordered. */
int32_t mlp_layout_to_optimal(MlpDevice* device, const MlpNetworkShape* shape, uint64_t portable, uint64_t optimal);
/* toPortableLayout (:529-554): the inverse. */
int32_t mlp_layout_to_portable(MlpDevice* device, const MlpNetworkShape* shape, uint64_t optimal, uint64_t portable);

/* ---- learnGradient without any allocation ------------------------------------------------- */

/* No counterpart in the reference.  For hosts that must not touch the CUDA allocator while they
 * train: an engine that claimed its whole device-memory budget at start-up and sub-allocates from its
 * own arena, or a frame loop that fits a small network between draws and cannot afford the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree.  This is learnGradient with ordered sums
 * (the same two kernels and the same results as entry point "learnGradient_simt" with
 * MLP_FLAG_SEQUENTIAL_SUM), but the per-sample vectors it parks between its two passes live in a
 * fixed 4 MiB area inside the library image rather than in a buffer the library would allocate.
 *   - Needs no MlpDevice: pass the device index and a cudaStream_t (null = legacy default stream).
 *     The network, loss, input and target addresses in `args` are the caller's own memory.
 *   - Limit: count * (sum over layers of in + out widths) floats must fit in 1 048 576 floats
 *     (e.g. 10 591 samples of the 2-16-16-16-1 network); larger batches get MLP_E_INVALID_ARG with
 *     the limit in the message.  Split them: gradients and loss words accumulate across calls.
 *   - The first call on each device resolves the area's device address.  That query allocates
 *     nothing through the allocator API, but with lazy module loading it is the moment the driver
 *     places this library's device image, the 4 MiB area included, on that GPU: make one call per
 *     device (count 0 is enough) at start-up, before the memory budget is claimed and before any
 *     stream capture begins.
 *   - The call makes device_ordinal current while it works and puts the caller's current device
 *     back before it returns.
 *   - The config goes through the same validity check as every other entry point; flag bits other
 *     than MLP_FLAG_SEQUENTIAL_SUM are refused (MLP_FLAG_INPUT_GRADIENT with MLP_E_NOT_AVAILABLE:
 *     the argument struct has no place for the result), all before any CUDA call.
 *   - Every call on a device uses the same area and leaves its contents behind; each call
 *     overwrites all the slots it later reads, so nothing has to be cleared.  Two calls whose
 *     kernels overlap on the GPU (different streams, no ordering between them) race on the area.
 *   - The 4 MiB are resident on every GPU that loads the library until the process exits. */
int32_t mlp_learn_gradient_ordered_noalloc(int32_t device_ordinal, void* cuda_stream, const MlpConfig* config,
                                           const MlpLearnGradParamsEx* args);

/* ---- self-test of the failure-reporting path ------------------------------------------------- */

/* No counterpart in the reference (its device code has no bounded waits; a hung kernel there ends in
 * the driver's watchdog, examples/nv-aftermath-example being the post-mortem tool).  Every wait inside
 * this library's tensor-core kernels gives up after a fixed number of polls, records a code in a device
 * status word and lets the kernel exit; mlp_wait() then returns MLP_E_DEVICE_STATUS once.  This call
 * launches a one-CTA kernel that makes such a wait run out on purpose (an mbarrier nobody arrives on,
 * max_polls polls, 1..100000) so that an integrator can see the whole path work: the launch returns
 * MLP_OK, the next mlp_wait() returns MLP_E_DEVICE_STATUS with status bit 0x40000000, the one after
 * that MLP_OK.  Nothing faults or hangs; bit 0x20000000 would mean the path itself is defective. */
int32_t mlp_selftest_bounded_wait(MlpDevice* device, uint32_t max_polls);

/* ---- host-side layout helpers ------------------------------------------------------------- */

/* allocateNetworkParameterStorage (mlp-training.cpp:217-250) in elements of the storage type:
 * w_off / b_off receive n_layers entries, total the padded element count of one segment. */
int32_t mlp_param_layout(const MlpConfig* config, int64_t* w_off, int64_t* b_off, int64_t* total);

const char* mlp_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif
