// placeholder, replaced below
#include "launchers.h"
namespace mlpb200 {
struct TcWorkspace { int dummy; };
bool tc_forward_supported(const MlpConfig&) { return false; }
bool tc_train_supported(const MlpConfig&) { return false; }
TcWorkspace* tc_workspace_create(int, std::string*) { return new TcWorkspace(); }
void tc_workspace_destroy(TcWorkspace* ws) { delete ws; }
cudaError_t launch_forward_tc(cudaStream_t, TcWorkspace*, const MlpConfig&, const MlpForwardParams&, int*, std::string*) { return cudaErrorInvalidValue; }
cudaError_t launch_learn_gradient_tc(cudaStream_t, TcWorkspace*, const MlpConfig&, const MlpLearnGradParamsEx&, int*, std::string*) { return cudaErrorInvalidValue; }
cudaError_t tc_read_status(cudaStream_t, TcWorkspace*, uint32_t* s) { *s = 0; return cudaSuccess; }
}
