// Allocation-free entry point of the native library.
//
// This has no counterpart in the reference project, whose kernels all take caller-allocated buffers and
// whose scratch (loss rows, norm scalar) is cudaMalloc'ed by the model at build time.
//
// Who needs it: code that must produce a bias gradient but is not allowed to obtain device memory at the
// point of the call -- a routine running inside a region where the process has handed every free byte of
// the GPU to another allocator (a serving framework's memory pool, a second library's arena), a plugin
// whose host contract forbids cudaMalloc / cudaFree because those calls synchronise the whole device and
// would stall the host's other streams, or a small C program that links this library without PyTorch and
// has no caching allocator of its own.  For those callers `cme_dact_colsum` is awkward: it wants a scratch
// buffer of `cme_colsum_splits(rows, cols) * cols` floats from the caller.
//
// `cme_dact_colsum_noalloc` computes the same thing -- g = dout * act'(pre) (optional) and
// dbias (+)= column sums of g -- and takes its scratch from a fixed array that is part of the loaded
// library image (CME_NOALLOC_SCRATCH_FLOATS floats = 1 MiB per GPU that loads the library, held until the
// process exits).  It calls no cudaMalloc, cudaFree or other allocating routine.
//
// Rules for callers:
//   * Sizes: cme_colsum_splits(rows, cols) * cols must not exceed CME_NOALLOC_SCRATCH_FLOATS; larger
//     problems are refused with CME_ERR_LIMIT and a message naming both numbers (use cme_dact_colsum).
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress) and
//     caches it.  Make that first call outside any stream capture.
//   * All calls on one device share the one array.  Two calls whose kernels can run at the same time (different
//     streams without an ordering between them) race on it; order them on one stream or with events.
//   * The array keeps whatever the previous call left.  Nothing here relies on it starting at zero: every
//     partial sum that the second stage reads is written by the first stage of the same call.
#pragma once
#include "common.h"

#define CME_NOALLOC_SCRATCH_FLOATS (1 << 18)

// dtype: CME_F32 or CME_BF16 (dout, pre, g, dbias all of that type).  pre / g may be null (plain column sum);
// act: 0 none, 1 relu, 2 gelu.  accumulate != 0 adds into dbias.  Returns CME_OK or an error status;
// cme_last_error() has the text.
CME_API int cme_dact_colsum_noalloc(int dtype, const void* dout, const void* pre, void* g, void* dbias, int rows,
                                    int cols, int act, int accumulate, void* stream);
