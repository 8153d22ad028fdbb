// Version, status text and host helpers of the C ABI.

#include "hxq_common.cuh"

extern "C" int hxq_version(void) { return HXQ_VERSION_NUMBER; }

namespace hxq {
thread_local int g_weights_on_stream = 0;
}  // namespace hxq

extern "C" void hxq_set_weights_on_stream(int on) { hxq::g_weights_on_stream = on ? 1 : 0; }

extern "C" const char* hxq_strerror(int status) {
    switch (status) {
        case HXQ_OK: return "ok";
        case HXQ_E_ARG: return "bad argument (null pointer, enum or token count out of range)";
        case HXQ_E_SHAPE: return "shape not covered (sizes, strides or group size)";
        case HXQ_E_ALIGN: return "pointer or leading dimension not aligned as required";
        case HXQ_E_DTYPE: return "unsupported element type";
        case HXQ_E_DEVICE: return "CUDA runtime error before launch";
        case HXQ_E_LAUNCH: return "kernel launch failed";
        case HXQ_E_TIMEOUT: return "a bounded device-side wait gave up";
        case HXQ_E_WORKSPACE: return "workspace missing or too small";
        default: return "unknown status";
    }
}

extern "C" int hxq_csr_from_positions(const int64_t* positions, int64_t nnz, int32_t out_features,
                                      int32_t in_features, int32_t* rowptr, int32_t* cols) {
    if (!rowptr || out_features <= 0 || in_features <= 0 || nnz < 0) return HXQ_E_ARG;
    if (nnz > 0 && (!positions || !cols)) return HXQ_E_ARG;
    if (nnz > 0x7fffffffLL) return HXQ_E_SHAPE;
    const int64_t total = (int64_t)out_features * in_features;
    int64_t prev = -1;
    int32_t row = 0;
    rowptr[0] = 0;
    for (int64_t e = 0; e < nnz; ++e) {
        const int64_t p = positions[e];
        if (p <= prev || p >= total) return HXQ_E_ARG;
        prev = p;
        const int32_t r = (int32_t)(p / in_features);
        while (row < r) rowptr[++row] = (int32_t)e;
        cols[e] = (int32_t)(p - (int64_t)r * in_features);
    }
    while (row < out_features) rowptr[++row] = (int32_t)nnz;
    return HXQ_OK;
}
