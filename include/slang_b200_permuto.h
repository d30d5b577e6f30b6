/* Permutohedral-lattice hash encoder: the trainable input encoder of the reference's neural module
 * (source/standard-modules/neural/permuto-encoder.slang, hash-function.slang), as C-ABI entry points.
 *
 * A position of `dims` floats is encoded, per level, by the barycentric blend of the `dims + 1` vertices of
 * the lattice simplex that contains it; each vertex owns `features_per_entry` values in a hash table of
 * 2^log2_hashmap_size entries per level.  Output row of one position: n_levels * features_per_entry values,
 * level-major (PermutoEncoder.encode, permuto-encoder.slang:312-330).  The backward pass adds
 * weight * upstream gradient into a gradient table of the same shape (readFeatureValueBwd,
 * permuto-encoder.slang:213-229) and optionally returns the gradient with respect to the positions. */
#ifndef SLANG_B200_PERMUTO_H
#define SLANG_B200_PERMUTO_H

#include "slang_b200_mlp.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MLP_PERMUTO_MAX_DIMS 4
#define MLP_PERMUTO_MAX_LEVELS 32

/* PermutoEncoder.PerLevelInfo (permuto-encoder.slang:21-29). */
typedef struct MlpPermutoLevelInfo {
    uint32_t level_index;
    uint32_t table_offset; /* in entries, not values */
    uint32_t table_size;   /* entries of this level's hash table */
    float scale;
    float scales_per_dim[MLP_PERMUTO_MAX_DIMS];
    float shifts_per_dim[MLP_PERMUTO_MAX_DIMS];
} MlpPermutoLevelInfo;

/* PermutoEncoder.HyperParameters (permuto-encoder.slang:37-41) plus the compile-time arguments of the
 * reference's generic type.  dtype (MlpDType: MLP_F32 or MLP_F16) is the type of the table, of the
 * output and of the gradient table; positions and their gradients are fp32. */
typedef struct MlpPermutoConfig {
    int32_t dims;               /* 1..MLP_PERMUTO_MAX_DIMS */
    int32_t features_per_entry; /* 1, 2, 4 or 8 */
    int32_t log2_hashmap_size;
    int32_t n_levels;           /* 1..MLP_PERMUTO_MAX_LEVELS */
    int32_t dtype;
    float max_level;            /* levels with index >= max_level + 1e-3 output zeros */
    MlpPermutoLevelInfo levels[MLP_PERMUTO_MAX_LEVELS];
} MlpPermutoConfig;

/* prepareLevelInfo for every level (permuto-encoder.slang:342-368): table size 2^log2_hashmap_size and
 * offset level * size; scale = base_scale * 2^(level * log2_per_level_scale); per-dimension scale
 * scale / sqrt((d+1)(d+2)); shifts drawn from PCG32(seed) advanced by level * dims, mapped to [-5, 5).
 * max_level = max_level_ratio * n_levels.  Host only, needs no device. */
int32_t mlp_permuto_prepare(int32_t dims, int32_t features_per_entry, int32_t log2_hashmap_size, int32_t n_levels,
                            float base_scale, float log2_per_level_scale, float max_level_ratio, uint32_t seed,
                            int32_t dtype, MlpPermutoConfig* out_config);

/* The grid hashes of hash-function.slang:66-145 (type: 0 Prime, 1 CoherentPrime, 2 ReversedPrime, 3 Rng,
 * 4 BaseConvert), on the host; the encoder itself uses BaseConvert.  Returns 0 for an unknown type. */
uint32_t mlp_grid_hash(int32_t type, int32_t dims, const uint32_t* position_grid);

/* encode (permuto-encoder.slang:312-330) for `count` positions: positions count x dims fp32,
 * table n_levels * 2^log2 * features values, out count x (n_levels * features) values. */
int32_t mlp_permuto_encode(MlpDevice* device, const MlpPermutoConfig* config, uint64_t positions, uint64_t table,
                           uint64_t out, uint32_t count);

/* Reverse pass for upstream gradients d_out (same shape and type as out): adds into d_table (same shape
 * and type as table; the caller clears it) and, when d_positions is not 0, writes count x dims fp32. */
int32_t mlp_permuto_backward(MlpDevice* device, const MlpPermutoConfig* config, uint64_t positions, uint64_t table,
                             uint64_t d_out, uint64_t d_table, uint64_t d_positions, uint32_t count);

#ifdef __cplusplus
}
#endif
#endif
