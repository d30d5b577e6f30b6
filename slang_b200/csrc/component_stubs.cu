// Entry points of the optional components, for builds that leave a component out
// (python -m slang_b200.build --without comm,permuto,tile_mma --out <file>): every declared symbol stays
// present, so a host that binds the whole header still loads the library, and answers MLP_E_NOT_AVAILABLE.
// Nothing here is compiled into the full library.
#include "../../include/slang_b200_mlp.h"
#include "../../include/slang_b200_permuto.h"
#include "../../include/slang_b200_tile_mma.h"
#include "abi_internal.h"

using namespace mlpb200;

static int32_t left_out(const char* what)
{
    set_last_error((std::string(what) + " was left out of this build").c_str());
    return MLP_E_NOT_AVAILABLE;
}

extern "C" {

#ifdef MLPB200_WITHOUT_COMM
int32_t mlp_comm_unique_id(void*, size_t) { return left_out("the gradient exchange"); }
int32_t mlp_comm_init(MlpDevice*, int32_t, int32_t, const void*, size_t, MlpComm**) { return left_out("the gradient exchange"); }
int32_t mlp_comm_destroy(MlpComm*) { return left_out("the gradient exchange"); }
int32_t mlp_allreduce_grads(MlpDevice*, MlpComm*, uint64_t, size_t, uint64_t, uint32_t) { return left_out("the gradient exchange"); }
int32_t mlp_comm_wait(MlpDevice*, MlpComm*, uint32_t) { return left_out("the gradient exchange"); }
#endif

#ifdef MLPB200_WITHOUT_PERMUTO
int32_t mlp_permuto_prepare(int32_t, int32_t, int32_t, int32_t, float, float, float, uint32_t, int32_t, MlpPermutoConfig*) { return left_out("the permutohedral encoder"); }
uint32_t mlp_grid_hash(int32_t, int32_t, const uint32_t*) { return 0u; }
int32_t mlp_permuto_encode(MlpDevice*, const MlpPermutoConfig*, uint64_t, uint64_t, uint64_t, uint32_t) { return left_out("the permutohedral encoder"); }
int32_t mlp_permuto_backward(MlpDevice*, const MlpPermutoConfig*, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint32_t) { return left_out("the permutohedral encoder"); }
#endif

#ifdef MLPB200_WITHOUT_TILE_MMA
int32_t mlp_tile_mma(MlpDevice*, const MlpTileMmaDesc*, uint64_t, uint64_t, uint64_t, uint64_t) { return left_out("the stand-alone tile product"); }
#endif

}  // extern "C"
