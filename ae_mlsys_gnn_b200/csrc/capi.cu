// Error reporting shared by every entry point of the library.
#include <string.h>
#include <stdio.h>
#include "../../include/gnn_b200.h"
#include "common.cuh"

namespace gnn {

static thread_local char g_last_error[512] = "";

int g_chunk_override = 0;

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

extern "C" int gnn_debug_set_chunk(int chunk) {
  if (chunk != 0 && (chunk < 32 || chunk > 4096 || chunk % 32 != 0)) {
    gnn::set_last_error("gnn_debug_set_chunk: chunk must be 0 or a multiple of 32 in [32, 4096]");
    return GNN_ERR_INVALID_ARG;
  }
  gnn::g_chunk_override = chunk;
  return GNN_OK;
}
