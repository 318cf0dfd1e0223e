// Host-side helpers behind the C ABI: last-error text, FNV-1a hashing of float bit patterns
// (trajectory tracing, FINAL_CLEAN_CODE_/src/main.cu:40-65), library identification.
#include "common.h"

#include <cstdarg>
#include <cstring>
#include <mutex>

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

static CmeDeviceState g_dev[CME_MAX_DEVICES];
static bool g_dev_ready[CME_MAX_DEVICES];
static std::mutex g_dev_mu;

// State of the current device; the first call on a device queries it and allocates its status words.
int cme_device_state(CmeDeviceState** out) {
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    CME_REQUIRE(dev >= 0 && dev < CME_MAX_DEVICES, CME_ERR_LIMIT, "device index %d beyond %d", dev, CME_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_dev_mu);
    if (!g_dev_ready[dev]) {
        CmeDeviceState st{};
        CME_CUDA(cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev));
        CME_CUDA(cudaMalloc(&st.status, CME_STATUS_WORDS * sizeof(int)));
        CME_CUDA(cudaMemset(st.status, 0, CME_STATUS_WORDS * sizeof(int)));
        st.max_pairs = -1;
        g_dev[dev] = st;
        g_dev_ready[dev] = true;
    }
    *out = &g_dev[dev];
    return CME_OK;
}

// Sets up the current device (SM count, status words).  Call once per device before the first stream capture;
// every launcher calls it too, so eager use needs no explicit call.
CME_API int cme_init_device() {
    CmeDeviceState* st;
    return cme_device_state(&st);
}

// Reads and clears one status word of the current device (0 = every bounded wait completed).
int cme_check_status_word(int which, int* host_out) {
    *host_out = 0;
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_dev_mu);
        if (dev >= 0 && dev < CME_MAX_DEVICES && g_dev_ready[dev]) word = g_dev[dev].status + which;
    }
    if (!word) return CME_OK;
    CME_CUDA(cudaMemcpy(host_out, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*host_out) CME_CUDA(cudaMemset(word, 0, sizeof(int)));
    return CME_OK;
}
