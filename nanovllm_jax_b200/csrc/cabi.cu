// Library-wide host helpers: version, thread-local error text, device queries,
// and the driver entry point used to encode TMA descriptors.
#include "common.cuh"

#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace nvllm {

char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

EncodeTiledFn encode_tiled_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
        (void)cudaGetLastError();
    });
    return fn;
}

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("NVLLM_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

}  // namespace nvllm

extern "C" int nvllm_b200_version(void) { return 200; }

extern "C" const char* nvllm_b200_last_error_string(void) { return nvllm::last_error_buffer(); }

extern "C" int nvllm_b200_device_status(int* flags_host) {
    using namespace nvllm;
    if (!flags_host) return fail(NVLLM_B200_EINVAL, "device_status: null pointer");
    int a = 0, b = 0, c = 0, rc;
    if ((rc = read_decode_flags(&a))) return rc;
    if ((rc = read_prefill_flags(&b))) return rc;
    if ((rc = read_comm_flags(&c))) return rc;
    *flags_host = a | b | c;
    return NVLLM_B200_OK;
}

extern "C" int nvllm_b200_device_status_reset(void) {
    using namespace nvllm;
    int rc;
    if ((rc = clear_decode_flags())) return rc;
    if ((rc = clear_prefill_flags())) return rc;
    return clear_comm_flags();
}
