/* Cooperative-matrix multiply-add, D = A . B + C, on the tcgen05 tensor cores: the stand-alone tile product the
 * reference exposes as linalg::coopMatMulAdd and implements on CUDA as Slang_CUDA_WMMA::coopMatMulAdd over
 * mma.sync fragments (prelude/slang-cuda-prelude.h:8145-8340 f16/bf16, :8342-8463 s8/u8 with and without
 * saturation, :8465-8590 e4m3/e5m2 with f32 or f16 accumulators, :8599-8642 the dispatch).
 *
 * The reference's unit is a 16 x 16 x 16 tile held by one warp.  Here one call runs `count` independent
 * problems of any size M x N x K (N <= 256, N a multiple of 8, K a multiple of 16 elements for 16-bit and
 * of 32 for 8-bit inputs); every 128 rows of a problem are one tcgen05.mma accumulator in tensor memory,
 * preloaded with C, so the sum starts from C as in the reference.  Known answers:
 * tests/cooperative-matrix/{mat-mul-add,int8,uint8,int8-saturating,uint8-saturating,fp8-cuda,fp8-cuda-half-acc}.slang. */
#ifndef SLANG_B200_TILE_MMA_H
#define SLANG_B200_TILE_MMA_H

#include "slang_b200_mlp.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of A and B (both the same type, as in the reference's fragments). */
enum MlpTileInput {
    MLP_TILE_F16 = 1,  /* numbered like MlpDType */
    MLP_TILE_BF16 = 2,
    MLP_TILE_S8 = 3,
    MLP_TILE_U8 = 4,
    MLP_TILE_E4M3 = 5,
    MLP_TILE_E5M2 = 6,
};
/* Element types of C and D.  F32 for every floating input; F16 for f16 and fp8 inputs (the sum itself is kept
 * in fp32 and rounded to half once at the end, which is at least as accurate as a half accumulator); S32 for
 * the integer inputs. */
enum MlpTileAccumulator { MLP_TILE_ACC_F32 = 0, MLP_TILE_ACC_F16 = 1, MLP_TILE_ACC_S32 = 2 };

/* One batch of products.  Leading dimensions and batch strides are in elements of the matrix they belong to;
 * a layout is MLP_MATRIX_ROW_MAJOR or MLP_MATRIX_COLUMN_MAJOR (CoopMatMatrixLayout of Load / Store).  c may be
 * 0 (a zero accumulator); d may equal c. */
typedef struct MlpTileMmaDesc {
    int32_t input_type;   /* MlpTileInput */
    int32_t acc_type;     /* MlpTileAccumulator */
    int32_t m, n, k;
    int32_t a_layout, b_layout, cd_layout;
    int64_t lda, ldb, ldcd;
    int64_t stride_a, stride_b, stride_cd;
    int32_t saturate;     /* integer inputs only: clamp to the int32 range instead of wrapping (coopMatMulAdd<int, true>) */
    int32_t count;        /* independent problems, >= 1 */
} MlpTileMmaDesc;

/* Stream ordered.  MLP_E_INVALID_ARG for a combination of types the reference does not have either (for example
 * an S32 accumulator with floating inputs), sizes outside the limits above, or a null operand. */
int32_t mlp_tile_mma(MlpDevice* device, const MlpTileMmaDesc* desc, uint64_t a, uint64_t b, uint64_t c, uint64_t d);

#ifdef __cplusplus
}
#endif

#endif
