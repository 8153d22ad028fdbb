// hxq_gemv_packed6: decode-time product over 6-bit packed indices (four codes in three bytes),
//   y[m, o] = sum_i x[m, i] * (code[o, i] * s[o, i / G] + t[o, i / G]) + bias,   M <= 16,
// unpacked inside the kernel, so the weight stream is 0.75 byte per weight.
//
// There is no codebook in this format (the code is the value), hence no table: a code becomes a float
// by dropping it into the mantissa of 2^23 and subtracting 2^23 (exact), two plain ALU operations.
// One warp per output row; a lane takes 16 consecutive codes (12 bytes, three aligned 32-bit loads)
// per step, the warp 512 codes (384 contiguous bytes).  16 divides the group size, so a lane's codes
// share one scale and offset: s * sum(x c) + t * sum(x) per lane and step, fp32 accumulation, one
// warp reduction at the end of the row.

#include "hxq_common.cuh"

namespace hxq {

struct Packed6Args {
    const uint8_t* packed;     // [out, in * 3 / 4] bytes, row-major
    const void* scales;
    const void* offsets;
    const float* bias;
    const void* x;
    void* y;
    int64_t ldx, ldy;
    int32_t out_features, in_features, group_size, ld_st, st_dtype, x_dtype, y_dtype, M, x_vec;
};

__device__ __forceinline__ float code_to_float(uint32_t c) {   // c < 2^23
    return __uint_as_float(0x4B000000u | c) - 8388608.0f;
}

template <int XDT>
__global__ void __launch_bounds__(128) gemv_packed6_kernel(const Packed6Args a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= a.out_features) return;
    const int n_in = a.in_features;
    const uint32_t* prow = reinterpret_cast<const uint32_t*>(a.packed + (int64_t)row * (n_in / 4 * 3));
    const int steps = (n_in + 511) / 512;
    for (int m0 = 0; m0 < a.M; m0 += 4) {       // tokens in groups of four: the codes are unpacked once per group
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int st = 0; st < steps; ++st) {
            const int col = st * 512 + lane * 16;
            if (col >= n_in) break;
            const uint32_t w0 = __ldg(prow + (col / 16) * 3);
            const uint32_t w1 = __ldg(prow + (col / 16) * 3 + 1);
            const uint32_t w2 = __ldg(prow + (col / 16) * 3 + 2);
            float c[16];
            // 96 bits, code k at bits [6k, 6k + 6)
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int bit = 6 * k;
                uint32_t v;
                if (bit + 6 <= 32) v = w0 >> bit;
                else if (bit < 32) v = __funnelshift_r(w0, w1, bit);
                else if (bit + 6 <= 64) v = w1 >> (bit - 32);
                else if (bit < 64) v = __funnelshift_r(w1, w2, bit - 32);
                else v = w2 >> (bit - 64);
                c[k] = code_to_float(v & 63u);
            }
            const int64_t so = (int64_t)row * a.ld_st + col / a.group_size;
            float s, t;
            if (a.st_dtype == HXQ_F32) {
                s = reinterpret_cast<const float*>(a.scales)[so];
                t = reinterpret_cast<const float*>(a.offsets)[so];
            } else {
                s = __half2float(reinterpret_cast<const __half*>(a.scales)[so]);
                t = __half2float(reinterpret_cast<const __half*>(a.offsets)[so]);
            }
#pragma unroll
            for (int mm = 0; mm < 4; ++mm) {
                if (m0 + mm < a.M) {
                    float xv[16];
                    const int64_t xo = (int64_t)(m0 + mm) * a.ldx + col;
                    if (a.x_vec) {     // 16-byte aligned rows: two (four for fp32) vector loads
                        if (XDT == HXQ_F32) {
                            const float4* p4 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) + xo);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float4 v = p4[j];
                                xv[4 * j] = v.x; xv[4 * j + 1] = v.y; xv[4 * j + 2] = v.z; xv[4 * j + 3] = v.w;
                            }
                        } else {
                            const uint4* p4 = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.x) + xo);
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const uint4 v = p4[j];
                                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    if (XDT == HXQ_BF16) {
                                        xv[8 * j + 2 * q] = __uint_as_float(w[q] << 16);
                                        xv[8 * j + 2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
                                    } else {
                                        const __half2 h = *reinterpret_cast<const __half2*>(&w[q]);
                                        xv[8 * j + 2 * q] = __low2float(h);
                                        xv[8 * j + 2 * q + 1] = __high2float(h);
                                    }
                                }
                            }
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 16; ++k) xv[k] = Elem<XDT>::load(a.x, xo + k);
                    }
                    float p = 0.f, xs = 0.f;
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        p = fmaf(c[k], xv[k], p);
                        xs += xv[k];
                    }
                    acc[mm] += fmaf(s, p, t * xs);
                }
            }
        }
#pragma unroll
        for (int mm = 0; mm < 4; ++mm) {
            float v = acc[mm];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && m0 + mm < a.M) {
                if (a.bias != nullptr) v += a.bias[row];
                store_from_f32(a.y, (int64_t)(m0 + mm) * a.ldy + row, v, a.y_dtype);
            }
        }
    }
}

}  // namespace hxq

extern "C" int hxq_gemv_packed6(const uint8_t* packed, int32_t out_features, int32_t in_features,
                                const void* scales, const void* offsets, int st_dtype, int32_t ld_st,
                                int32_t group_size, const float* bias, const void* x, int x_dtype, int32_t M,
                                int64_t ldx, void* y, int y_dtype, int64_t ldy, hxq_stream_t stream_) {
    using namespace hxq;
    if (!packed || !scales || !offsets || !x || !y) return HXQ_E_ARG;
    if (out_features <= 0 || in_features <= 0 || M <= 0 || M > 16) return HXQ_E_ARG;
    if (in_features % 16 != 0 || group_size <= 0 || group_size % 16 != 0) return HXQ_E_SHAPE;
    if (ld_st < (in_features + group_size - 1) / group_size || ldx < in_features || ldy < out_features) return HXQ_E_SHAPE;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype) || (st_dtype != HXQ_F32 && st_dtype != HXQ_F16)) return HXQ_E_DTYPE;
    if (!aligned_to(packed, 4)) return HXQ_E_ALIGN;      // rows are in * 3 / 4 bytes: a multiple of 12
    Packed6Args a;
    a.packed = packed; a.scales = scales; a.offsets = offsets; a.bias = bias; a.x = x; a.y = y;
    a.ldx = ldx; a.ldy = ldy; a.out_features = out_features; a.in_features = in_features;
    a.group_size = group_size; a.ld_st = ld_st; a.st_dtype = st_dtype; a.x_dtype = x_dtype; a.y_dtype = y_dtype; a.M = M;
    a.x_vec = (aligned_to(x, 16) && (ldx * dtype_size(x_dtype)) % 16 == 0) ? 1 : 0;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int blocks = (out_features + 3) / 4;
    if (x_dtype == HXQ_F32) gemv_packed6_kernel<HXQ_F32><<<blocks, 128, 0, stream>>>(a);
    else if (x_dtype == HXQ_F16) gemv_packed6_kernel<HXQ_F16><<<blocks, 128, 0, stream>>>(a);
    else gemv_packed6_kernel<HXQ_BF16><<<blocks, 128, 0, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}
