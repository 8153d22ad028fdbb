// hxq_dequant: compressed rows -> dense fp32 / bf16 / fp16 rows.
//
// Bound by HBM writes (4 B or 2 B out per 1 B of index in).  fp32 output is
// bit-exact with the reference reader: codebook gather, optional affine with
// two roundings, then the sidecar VALUE overwrites the entry.

#include "hxq_common.cuh"

namespace hxq {

struct DequantArgs {
    const uint8_t* idx;
    const float* cb;
    const void* scales;
    const void* offsets;
    const int32_t* rowptr;
    const int32_t* cols;
    const float* values;
    void* out;
    int64_t ld_idx;
    int64_t ld_out;
    int32_t row0, row1, in_features, col0, group_size, ld_st, st_dtype;
};

__device__ __forceinline__ float weight_at(const DequantArgs& a, const float* cb_s, int row, int col,
                                           uint32_t code) {
    float w = cb_s[code];
    if (a.group_size > 0) {
        int g = (a.col0 + col) / a.group_size - a.col0 / a.group_size;
        int64_t o = (int64_t)row * a.ld_st + g;
        float s = load_as_f32(a.scales, o, a.st_dtype);
        float t = load_as_f32(a.offsets, o, a.st_dtype);
        w = affine_2round(w, s, t);
    }
    return w;
}

// Vector path: one thread = 16 consecutive columns of one row.
template <int OUT_DT>
__global__ void __launch_bounds__(256) dequant_vec_kernel(DequantArgs a) {
    __shared__ float cb_s[256];
    cb_s[threadIdx.x] = a.cb[threadIdx.x];
    __syncthreads();
    const int vec_per_row = a.in_features >> 4;
    const int64_t total = (int64_t)(a.row1 - a.row0) * vec_per_row;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total;
         v += (int64_t)gridDim.x * blockDim.x) {
        const int lr = (int)(v / vec_per_row);
        const int col = (int)(v - (int64_t)lr * vec_per_row) << 4;
        const int row = a.row0 + lr;
        const uint4 q = ld_stream_u4(a.idx + (int64_t)row * a.ld_idx + col);
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        float w[16];
        float s = 1.f, t = 0.f;
        if (a.group_size > 0) {  // group_size % 16 == 0 and col0 % 16 == 0 on this path
            int g = (a.col0 + col) / a.group_size - a.col0 / a.group_size;
            int64_t o = (int64_t)row * a.ld_st + g;
            s = load_as_f32(a.scales, o, a.st_dtype);
            t = load_as_f32(a.offsets, o, a.st_dtype);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float c = cb_s[(words[j >> 2] >> ((j & 3) * 8)) & 0xffu];
            w[j] = (a.group_size > 0) ? affine_2round(c, s, t) : c;
        }
        const int64_t o = (int64_t)lr * a.ld_out + col;
        if (OUT_DT == HXQ_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + o);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_float4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        } else {
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (OUT_DT == HXQ_BF16) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(w[2 * j], w[2 * j + 1]);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                    __half2 h = __floats2half2_rn(w[2 * j], w[2 * j + 1]);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.out) + o);
            dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
    }
}

// Scalar path for ragged / unaligned shapes.
__global__ void __launch_bounds__(256) dequant_scalar_kernel(DequantArgs a, int out_dt) {
    __shared__ float cb_s[256];
    cb_s[threadIdx.x] = a.cb[threadIdx.x];
    __syncthreads();
    const int64_t total = (int64_t)(a.row1 - a.row0) * a.in_features;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int lr = (int)(e / a.in_features);
        const int col = (int)(e - (int64_t)lr * a.in_features);
        const int row = a.row0 + lr;
        float w = weight_at(a, cb_s, row, col, a.idx[(int64_t)row * a.ld_idx + col]);
        store_from_f32(a.out, (int64_t)lr * a.ld_out + col, w, out_dt);
    }
}

// Sidecar overwrite: one warp per row, lanes stride over the row's entries.
__global__ void __launch_bounds__(256) dequant_sidecar_kernel(DequantArgs a, int out_dt) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int row = a.row0 + warp;
    if (row >= a.row1) return;
    const int e0 = a.rowptr[row], e1 = a.rowptr[row + 1];
    for (int e = e0 + lane; e < e1; e += 32) {
        store_from_f32(a.out, (int64_t)(row - a.row0) * a.ld_out + a.cols[e], a.values[e], out_dt);
    }
}

}  // namespace hxq

extern "C" int hxq_dequant(const hxq_desc* d, int32_t row0, int32_t row1, void* out, int out_dtype,
                           int64_t ld_out, hxq_stream_t stream_) {
    using namespace hxq;
    int st = validate_desc(d);
    if (st != HXQ_OK) return st;
    if (!out) return HXQ_E_ARG;
    if (!dtype_ok(out_dtype)) return HXQ_E_DTYPE;
    if (row0 < 0 || row1 > d->out_features || row0 > row1) return HXQ_E_SHAPE;
    if (ld_out < d->in_features) return HXQ_E_SHAPE;
    if (d->rowptr && !d->values) return HXQ_E_ARG;
    if (row0 == row1) return HXQ_OK;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);

    DequantArgs a;
    a.idx = d->indices; a.cb = d->codebook; a.scales = d->scales; a.offsets = d->offsets;
    a.rowptr = d->rowptr; a.cols = d->cols; a.values = d->values; a.out = out;
    a.ld_idx = d->ld_idx; a.ld_out = ld_out; a.row0 = row0; a.row1 = row1;
    a.in_features = d->in_features; a.col0 = d->col0; a.group_size = d->group_size;
    a.ld_st = d->ld_st; a.st_dtype = d->st_dtype;

    const int esz = dtype_size(out_dtype);
    const bool vec = (d->in_features % 16 == 0) && (d->ld_idx % 16 == 0) && aligned_to(d->indices, 16) &&
                     aligned_to(out, 16) && ((ld_out * esz) % 16 == 0) &&
                     (d->group_size == 0 || (d->group_size % 16 == 0 && d->col0 % 16 == 0));
    const int64_t rows = row1 - row0;
    if (vec) {
        int64_t total = rows * (d->in_features / 16);
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 16) blocks = 148 * 16;
        if (out_dtype == HXQ_F32) dequant_vec_kernel<HXQ_F32><<<blocks, 256, 0, stream>>>(a);
        else if (out_dtype == HXQ_BF16) dequant_vec_kernel<HXQ_BF16><<<blocks, 256, 0, stream>>>(a);
        else dequant_vec_kernel<HXQ_F16><<<blocks, 256, 0, stream>>>(a);
    } else {
        int64_t total = rows * d->in_features;
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 16) blocks = 148 * 16;
        dequant_scalar_kernel<<<blocks, 256, 0, stream>>>(a, out_dtype);
    }
    if (cudaGetLastError() != cudaSuccess) return HXQ_E_LAUNCH;
    if (d->rowptr) {
        int blocks = (int)((rows * 32 + 255) / 256);
        dequant_sidecar_kernel<<<blocks, 256, 0, stream>>>(a, out_dtype);
        if (cudaGetLastError() != cudaSuccess) return HXQ_E_LAUNCH;
    }
    return HXQ_OK;
}
