// placeholder until the tcgen05 kernel lands
#include "common.h"
bool int4_gemm_tc_supported(const Int4Weight &, int) { return false; }
int launch_int4_gemm_tc(b200nn_ctx *ctx, const Int4Weight &, const __half *, int, const Epilogue &) {
    return set_error(ctx, B200NN_ERR_UNSUPPORTED, "tensor-core GEMM not built");
}
