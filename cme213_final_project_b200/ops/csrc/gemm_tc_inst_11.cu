// Instantiations of the tcgen05 GEMM launcher, group 11 of gemm_tc_inst_list.h (one translation unit per group so
// that the groups compile in parallel).
#include "gemm_tcgen05_kernel.cuh"

using namespace gemm_tc;

#define CME_GEMM_TC_GROUP 11
#define CME_GEMM_TC_EXTERN(BN, SIMPLE, PAIR, SPEC)                                                                   \
    template int gemm_tc::launch_bn<BN, SIMPLE, PAIR, SPEC>(bool, bool, const CUtensorMap&, const CUtensorMap&,      \
                                                            const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, \
                                                            const EpiParams&, int, cudaStream_t);
#include "gemm_tc_inst_list.h"
