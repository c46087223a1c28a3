// Tensor-core (tcgen05) GEMM for the Linear convention; filled in by gemm_tc kernels.
#include "common.cuh"

bool rcu_gemm_tc_eligible(int, int, uint64_t, uint64_t, uint64_t) { return false; }

rcu_status rcu_gemm_tc_dispatch(rcu_device* dev, int, const void*, int, const void*, const void*, void*, uint64_t, uint64_t,
                                uint64_t) {
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemm_tc: not available");
}
