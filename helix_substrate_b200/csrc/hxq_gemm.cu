// hxq_gemm: prefill-time product (placeholder body; see the tensor-core kernel below once built).
#include "hxq_common.cuh"

namespace hxq {
int gemv_any_m(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y, int y_dtype,
               int64_t ldy, void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t gemv_workspace_bytes(const hxq_desc* d, int32_t M);
}

extern "C" size_t hxq_gemm_workspace_bytes(const hxq_desc* d, int32_t M) {
    if (hxq::validate_desc(d) != HXQ_OK || M <= 0) return 0;
    return hxq::gemv_workspace_bytes(d, 4);
}

extern "C" int hxq_gemm(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y,
                        int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes,
                        int32_t* status_word, hxq_stream_t stream) {
    using namespace hxq;
    (void)status_word;
    int st = validate_desc(d);
    if (st != HXQ_OK) return st;
    if (!x || !y) return HXQ_E_ARG;
    if (M <= 0) return HXQ_E_ARG;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return HXQ_E_DTYPE;
    if (ldx < d->in_features || ldy < d->out_features) return HXQ_E_SHAPE;
    if (d->rowptr && !d->deltas) return HXQ_E_ARG;
    return gemv_any_m(d, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}
