/*
 * Shapes, number formats and optimiser constants of one small-MLP training problem.
 *
 * The reference fixes these at compile time: the network shape is a generic argument of
 * FeedForwardLayer<In, Out> (examples/mlp-training/network.slang:8-9, kLayerSizes in
 * examples/mlp-training/mlp-training.cpp:24), the storage type is `typealias NFloat = half`
 * (examples/mlp-training/common.slang:1) and the Adam constants are static members of
 * AdamOptimizer (examples/mlp-training/adam.slang:15-19).  This library ships prebuilt sm_100a
 * kernels instead of compiling Slang at run time, so the same facts travel in this plain struct.
 *
 * Plain C, fixed-width fields only, no padding holes: the struct is passed across the C ABI and is
 * mirrored field by field by ctypes on the Python side.
 */
#ifndef SLANG_B200_MLP_CONFIG_H
#define SLANG_B200_MLP_CONFIG_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLP_MAX_LAYERS 8

/* Storage type of parameters and of the vectors passed between layers (the reference's NFloat). */
enum MlpDType { MLP_F32 = 0, MLP_F16 = 1, MLP_BF16 = 2 };

/* Activations.  IDENTITY..QUICK_GELU restate source/standard-modules/neural/activations.slang:8-228;
 * GELU_TANH is not in the reference and is written in the same style;
 * LEAKY_MAX is `max(o, o * alpha)` of examples/mlp-training-coopvec/fflayer.slang:61-66, whose
 * derivative at 0 follows the max tie rule (source/slang/diff.meta.slang:2268-2273). */
enum MlpActivation {
    MLP_ACT_IDENTITY = 0,
    MLP_ACT_RELU = 1,       /* max(x, 0); derivative 1/2 at exactly 0 (max tie rule) */
    MLP_ACT_LEAKY_RELU = 2, /* x < 0 ? alpha * x : x; derivative 1 at exactly 0 */
    MLP_ACT_SIGMOID = 3,
    MLP_ACT_TANH = 4,
    MLP_ACT_EXP = 5,
    MLP_ACT_SINE = 6,
    MLP_ACT_SILU = 7,
    MLP_ACT_QUICK_GELU = 8,
    MLP_ACT_GELU_TANH = 9,
    MLP_ACT_LEAKY_MAX = 10
};

/* Per-sample loss.  The reference example uses dot(diff, diff) (network.slang:40-47) = L2_SUM. */
enum MlpLoss { MLP_LOSS_MSE_MEAN = 0, MLP_LOSS_L2_SUM = 1 };

/* Input encoding in front of layer 0.  FREQ2D: a 2-D coordinate (u0, u1) becomes
 * [sin(2^k pi u), cos(2^k pi u)] for k = 0..7 and u in {u0, u1}: 32 features ordered
 * u-major, then k, then (sin, cos). */
enum MlpEncoding { MLP_ENC_NONE = 0, MLP_ENC_FREQ2D = 1 };

/* Order and rounding of a layer's scalar sums where one thread (or the CPU) adds the terms one at a
 * time.  NEURAL is what the neural module's InlineVector and the cooperative-vector software fallback
 * do: the sum starts at zero, every product is rounded before it is added, the bias is added after the
 * last term (source/standard-modules/neural/inline-vector.slang:101-110, 131-132;
 * source/slang/hlsl.meta.slang:32866, 33266-33274).  BIAS_FIRST_FUSED is the example's order, the sum
 * starting from the bias (examples/mlp-training/mlvec_sw.slang:31-34), with each term a fused
 * multiply-add.  The tensor-core kernels accumulate in fp32 in the hardware's own order and ignore it. */
enum MlpSumOrder { MLP_SUM_NEURAL = 0, MLP_SUM_BIAS_FIRST_FUSED = 1 };

/* How a layer's weights lie behind MlpLayerPointers.weights.  ROW_MAJOR is the example's layout, [out][in]
 * (examples/mlp-training/mlp-training.cpp:217-250).  OPTIMAL is the neural module's OptimalLayout on CUDA
 * (source/standard-modules/neural/layers.slang:53-71, network-parameter-layout-converter.slang:54-68,
 * 176-181): rows and columns padded to multiples of 16, 16x16 tiles ordered input-tile-major, inside a tile
 * the register order of a tensor-core B fragment; a layer's biases follow its weights in a padded slot
 * (MlpLayerPointers.biases points at that slot).  Every entry point built for an MlpConfig reads either:
 * weights a shader holds in OptimalLayout are used, and trained, in place, with no conversion pass.
 * learnGradient adds the gradient of a weight at the weight's own element offset behind
 * MlpLayerPointers.weightsGrad (an fp32 buffer of the same shape; the reference's own OptimalLayout gradient
 * buffers are in the target's accumulator-fragment order instead, a format no caller of this library sees),
 * and adjustParameters runs over all mlp_param_layout() elements, padding included (zero gradients leave
 * the zero padding as it is).  mlp_learn_gradient_ordered_noalloc takes ROW_MAJOR only. */
enum MlpParamLayout { MLP_PARAMS_ROW_MAJOR = 0, MLP_PARAMS_OPTIMAL = 1 };

typedef struct MlpConfig {
    int32_t n_layers;                  /* number of linear layers, 1..MLP_MAX_LAYERS */
    int32_t dims[MLP_MAX_LAYERS + 1];  /* dims[0] = width entering layer 0 (after encoding), dims[n_layers] = outputs */
    int32_t dtype;                     /* MlpDType of parameters and inter-layer vectors */
    int32_t input_dtype;               /* MlpDType of the inputs buffer */
    int32_t target_dtype;              /* MlpDType of the targets buffer */
    int32_t hidden_act;                /* MlpActivation after every layer but the last */
    int32_t output_act;                /* MlpActivation after the last layer */
    float act_alpha;                   /* slope of the leaky activations */
    int32_t loss;                      /* MlpLoss */
    int32_t encoding;                  /* MlpEncoding */
    int32_t input_width;               /* values per sample in the inputs buffer (2 for FREQ2D, else dims[0]) */
    float lr, beta1, beta2, eps;       /* Adam constants (adam.slang:15-19) */
    int32_t adam_master;               /* 1: Adam keeps an fp32 copy of each parameter in its state */
    int32_t sum_order;                 /* MlpSumOrder of the one-thread-per-sample kernels */
    int32_t param_layout;              /* MlpParamLayout of the weights and of their gradients */
    int32_t operand_dtype;             /* 0: products read the storage type.  MLP_F16 / MLP_BF16 with dtype = MLP_F32:
                                          the neural module's T = float on its tensor-core path, whose matrix
                                          operands are half whatever T is (source/standard-modules/neural/
                                          mma-tiled-cuda.slang:104-118, WaveMatrix.slang:62-64): weights and the
                                          vectors passed between layers are converted to that type where a product
                                          reads them; biases, sums, pre-activations, outputs, gradients and the
                                          optimiser stay fp32 */
} MlpConfig;

/* Optimiser state per parameter for the configurable path: the fp32 widening of the reference's
 * AdamState {half mean; half variance; int iteration} (examples/mlp-training/adam.slang:6-11). */
typedef struct MlpAdamState {
    float mean;
    float variance;
    int32_t iteration;
    float master; /* fp32 copy of the parameter, read only when MlpConfig.adam_master != 0 */
} MlpAdamState;

/* Optimiser state of the literal example kernels: 8 bytes (mlp-training.cpp:143). */
typedef struct MlpExampleAdamState {
    uint16_t mean;     /* half bits */
    uint16_t variance; /* half bits */
    int32_t iteration;
} MlpExampleAdamState;

/* One layer of the network constant buffer: four device addresses, in the order of
 * FeedForwardLayer's fields (examples/mlp-training/mlp_sw.slang:9-12) as the host writes them
 * (mlp-training.cpp:147-158). */
typedef struct MlpLayerPointers {
    uint64_t weights;      /* row-major [out][in], storage type */
    uint64_t weightsGrad;  /* row-major [out][in]; fp32 on the configurable path, half in the example */
    uint64_t biases;       /* [out] */
    uint64_t biasesGrad;   /* [out] */
} MlpLayerPointers;

#ifdef __cplusplus
}
#endif
#endif
