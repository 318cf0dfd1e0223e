// Every instantiated launcher of the tcgen05 GEMM:  CME_GEMM_TC_EXTERN(tile width, plain epilogue, CTA pair, epilogue set).
// Included (several times, hence no include guard) by gemm_tcgen05.cu, which sees all groups, and by the
// gemm_tc_inst_*.cu translation units, which each define CME_GEMM_TC_GROUP and instantiate that group only.
#ifndef CME_GEMM_TC_GROUP
#define CME_GEMM_TC_GROUP (-1)
#define CME_GEMM_TC_GROUP_DEFAULTED 1
#endif

#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 0      // plain bf16 epilogue
CME_GEMM_TC_EXTERN(64, true, false, -1)
CME_GEMM_TC_EXTERN(128, true, false, -1)
CME_GEMM_TC_EXTERN(256, true, false, -1)
CME_GEMM_TC_EXTERN(256, true, true, -1)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 1      // run-time epilogue (any combination)
CME_GEMM_TC_EXTERN(64, false, false, -1)
CME_GEMM_TC_EXTERN(128, false, false, -1)
CME_GEMM_TC_EXTERN(256, false, false, -1)
CME_GEMM_TC_EXTERN(256, false, true, -1)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 2      // CTA pair, compile-time epilogues (a)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_BIAS)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_BIAS_RES)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_BIAS_GELU_AUX)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_DGELU)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_ACC)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 3      // CTA pair, compile-time epilogues (b)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_BIAS_RELU)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_DRELU)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_RES)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_F32)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 4      // 64-wide tiles, compile-time epilogues
CME_GEMM_TC_EXTERN(64, false, false, SPEC_BIAS_RELU)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_DRELU)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_RES)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_BIAS_RES)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_ACC)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_F32)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 5      // 128-wide tiles, compile-time epilogues (a)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_BIAS_RELU)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_DRELU)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_RES)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_BIAS_RES)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 6      // 128-wide tiles, compile-time epilogues (b)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_BIAS_GELU_AUX)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_DGELU)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_ACC)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_F32)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 7      // 64-wide tiles, GELU epilogues
CME_GEMM_TC_EXTERN(64, false, false, SPEC_BIAS_GELU_AUX)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_DGELU)
#endif

#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 8      // MLP pair with the derivative kept by forward: forward side
CME_GEMM_TC_EXTERN(256, false, true, SPEC_BIAS_GELU_AUXD)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_BIAS_GELU_AUXD)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_BIAS_GELU_AUXD)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 9      // ... backward side, with the bias gradient's column sums
CME_GEMM_TC_EXTERN(256, false, true, SPEC_DMUL_COLSUM)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_DMUL_COLSUM)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_DMUL_COLSUM)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_DMUL)            // same without the column sums (caller sums C itself)
#endif
#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 10     // ReLU derivative with column sums
CME_GEMM_TC_EXTERN(256, false, true, SPEC_DRELU_COLSUM)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_DRELU_COLSUM)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_DRELU_COLSUM)
#endif

#if CME_GEMM_TC_GROUP == -1 || CME_GEMM_TC_GROUP == 11     // fp32 storage multiplied as tf32 (plain fp32 output)
CME_GEMM_TC_EXTERN(64, false, false, SPEC_TF32)
CME_GEMM_TC_EXTERN(128, false, false, SPEC_TF32)
CME_GEMM_TC_EXTERN(256, false, false, SPEC_TF32)
CME_GEMM_TC_EXTERN(256, false, true, SPEC_TF32)
#endif

#ifdef CME_GEMM_TC_GROUP_DEFAULTED
#undef CME_GEMM_TC_GROUP
#undef CME_GEMM_TC_GROUP_DEFAULTED
#endif
