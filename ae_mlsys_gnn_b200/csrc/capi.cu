// Error reporting shared by every entry point of the library.
#include <string.h>
#include <stdio.h>
#include "../../include/gnn_b200.h"
#include "common.cuh"

namespace gnn {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* msg) {
  strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

// Reports launch-configuration errors of the launches just issued.  Does not
// synchronise: execution errors surface at the caller's next synchronisation.
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return GNN_OK;
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  return GNN_ERR_CUDA;
}

}  // namespace gnn

extern "C" const char* gnn_last_error_string(void) { return gnn::g_last_error; }

extern "C" int gnn_abi_version(void) { return GNN_B200_ABI_VERSION; }
