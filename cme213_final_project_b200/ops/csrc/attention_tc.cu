// Tensor-core (tcgen05) attention entry points.
#include "attention.h"

int attention_tc_supported(const CmeAttn* a) { (void)a; return 0; }
int attention_tc_fwd(const CmeAttn* a, cudaStream_t st) { (void)a; (void)st; return CME_ERR_UNSUPPORTED; }
int attention_tc_bwd(const CmeAttn* a, cudaStream_t st) { (void)a; (void)st; return CME_ERR_UNSUPPORTED; }
