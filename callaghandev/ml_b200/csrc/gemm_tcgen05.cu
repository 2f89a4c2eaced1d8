// Placeholder until the tensor-core engine lands: nothing is eligible, so every GEMM takes the FP32 SIMT kernel.
#include "common.h"
namespace b200 {
bool gemm_tcgen05_eligible(b200_ctx*, const Gemm&) { return false; }
int gemm_tcgen05(b200_ctx* ctx, const Gemm&) { return fail(ctx, B200_ERR_UNSUPPORTED, "tcgen05 GEMM not built"); }
}  // namespace b200
