// Host-side helpers behind the C ABI: last-error text, FNV-1a hashing of float bit patterns
// (trajectory tracing, FINAL_CLEAN_CODE_/src/main.cu:40-65), library identification.
#include "common.h"

#include <cstdarg>
#include <cstring>

static thread_local char g_err[1024] = "";
long long g_cme_launches = 0;

void cme_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

CME_API const char* cme_last_error() { return g_err; }

CME_API int cme_abi_version() { return 1; }

// FNV-1a over 32-bit words with 64-bit state: h ^= word; h *= prime.
CME_API unsigned long long fnv1a_u32(const uint32_t* words, long long n, unsigned long long h) {
    for (long long i = 0; i < n; ++i) {
        h ^= (unsigned long long)words[i];
        h *= 1099511628211ull;
    }
    return h;
}

CME_API int cme_device_info(int* sms, int* cc_major, int* cc_minor, long long* smem_optin) {
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp prop;
    CME_CUDA(cudaGetDeviceProperties(&prop, dev));
    *sms = prop.multiProcessorCount;
    *cc_major = prop.major;
    *cc_minor = prop.minor;
    *smem_optin = (long long)prop.sharedMemPerBlockOptin;
    return CME_OK;
}

// Device-to-device copy on a stream (used to read engine-owned buffers into caller-owned tensors).
CME_API int cme_copy_d2d(void* dst, const void* src, long long bytes, void* stream) {
    CME_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return CME_OK;
}

// Number of kernels this library has launched (or captured into a graph) in this process.
CME_API long long cme_launch_count() { return g_cme_launches; }
