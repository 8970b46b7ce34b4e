#include "lp_internal.cuh"
namespace ge2 {
int lp_scores_tf32(const LpKernelArgs& a, cudaStream_t stream) { (void)a; (void)stream; return GE2_ERR_UNSUPPORTED; }
}
