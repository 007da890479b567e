// placeholder until the tensor-core kernel lands
#include "linear.cuh"
namespace fb {
bool linear_tcgen05_supports(const LinearArgs&) { return false; }
size_t linear_tcgen05_workspace(int64_t, int64_t, int64_t) { return 0; }
int linear_tcgen05(const LinearArgs&, cudaStream_t) { set_error("tcgen05 path not built"); return FB_ERR_LAUNCH; }
}
