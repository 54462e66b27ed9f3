// Placeholder until the tcgen05 kernel lands: no shape is supported yet.
#include "cfx_common.cuh"
#include "cfx_fused.h"
namespace cfx {
struct FusedPlan {};
bool fused_supported(int, int, int, int) { return false; }
int fused_create(FusedPlan**, int, int, int, int, int, int, float*) { return CFX_ERR_UNSUPPORTED; }
int fused_refresh(FusedPlan*, const float*, cudaStream_t) { return CFX_ERR_UNSUPPORTED; }
int fused_forward(FusedPlan*, const FusedArgs&, cudaStream_t, int*) { return CFX_ERR_UNSUPPORTED; }
int fused_check_status(FusedPlan*, cudaStream_t, unsigned* s) { if (s) *s = 0; return CFX_OK; }
void fused_destroy(FusedPlan*) {}
}
