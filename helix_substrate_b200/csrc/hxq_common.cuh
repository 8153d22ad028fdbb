// Shared device/host helpers for the HXQ sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hxq_b200.h"

#define HXQ_VERSION_NUMBER 100  // 0.1.0

namespace hxq {

// Set by hxq_set_weights_on_stream (per host thread): the decode kernels then launch without the
// programmatic-dependent-launch attribute, i.e. only after everything before them in the stream is done.
extern thread_local int g_weights_on_stream;

// ---- element conversion ----------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<HXQ_F32> {
    using type = float;
    static __device__ __forceinline__ float load(const void* p, int64_t i) {
        return reinterpret_cast<const float*>(p)[i];
    }
    static __device__ __forceinline__ void store(void* p, int64_t i, float v) {
        reinterpret_cast<float*>(p)[i] = v;
    }
};
template <> struct Elem<HXQ_F16> {
    using type = __half;
    static __device__ __forceinline__ float load(const void* p, int64_t i) {
        return __half2float(reinterpret_cast<const __half*>(p)[i]);
    }
    static __device__ __forceinline__ void store(void* p, int64_t i, float v) {
        reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
    }
};
template <> struct Elem<HXQ_BF16> {
    using type = __nv_bfloat16;
    static __device__ __forceinline__ float load(const void* p, int64_t i) {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    }
    static __device__ __forceinline__ void store(void* p, int64_t i, float v) {
        reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    }
};

// Runtime-typed scalar access (cold paths only).
__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dt) {
    if (dt == HXQ_F32) return Elem<HXQ_F32>::load(p, i);
    if (dt == HXQ_F16) return Elem<HXQ_F16>::load(p, i);
    return Elem<HXQ_BF16>::load(p, i);
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, float v, int dt) {
    if (dt == HXQ_F32) Elem<HXQ_F32>::store(p, i, v);
    else if (dt == HXQ_F16) Elem<HXQ_F16>::store(p, i, v);
    else Elem<HXQ_BF16>::store(p, i, v);
}

__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == HXQ_F32 ? 4 : 2; }
__host__ __forceinline__ bool dtype_ok(int dt) { return dt == HXQ_F32 || dt == HXQ_F16 || dt == HXQ_BF16; }

// 16-byte streaming load of index bytes: read-only path, do not keep in L1.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Weight value with the affine applied exactly as the CPU oracle does it:
// product rounded to fp32, then sum rounded to fp32 (no contraction to an FMA).
__device__ __forceinline__ float affine_2round(float c, float s, float t) {
    return __fadd_rn(__fmul_rn(c, s), t);
}

__host__ __forceinline__ bool aligned_to(const void* p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

// Host-side validation shared by the entry points.
inline int validate_desc(const hxq_desc* d) {
    if (!d || !d->indices || !d->codebook) return HXQ_E_ARG;
    if (d->out_features <= 0 || d->in_features <= 0) return HXQ_E_SHAPE;
    if (d->ld_idx < d->in_features || d->col0 < 0) return HXQ_E_SHAPE;
    if (d->group_size < 0) return HXQ_E_SHAPE;
    if (d->group_size > 0) {
        if (!d->scales || !d->offsets) return HXQ_E_ARG;
        if (d->st_dtype != HXQ_F32 && d->st_dtype != HXQ_F16) return HXQ_E_DTYPE;
        int64_t ng = (int64_t)(d->col0 + d->in_features - 1) / d->group_size - d->col0 / d->group_size + 1;
        if (d->ld_st < ng) return HXQ_E_SHAPE;
    }
    if (d->rowptr && (!d->cols)) return HXQ_E_ARG;
    return HXQ_OK;
}

}  // namespace hxq
