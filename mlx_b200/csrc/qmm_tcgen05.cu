#include "common.cuh"
#include "kernels.h"
namespace b200q {
bool qmm_tc_supported(const QmmArgs&) { return false; }
size_t qmm_tc_workspace_bytes(const QmmArgs&) { return 0; }
int qmm_tc(const QmmArgs&, cudaStream_t) { return fail(B200Q_ERR_UNSUPPORTED, "qmm_tcgen05 not built"); }
}  // namespace b200q
