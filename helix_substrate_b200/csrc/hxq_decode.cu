// hxq_decode: the small kernels between the compressed linears of one decode step
// (one new token per sequence): residual add + RMSNorm, rotary embedding + KV-cache
// append, single-query grouped attention over the cache, SwiGLU.  The reference runs
// these as dozens of framework element-wise launches per layer around its linears
// (helix_substrate/basin_runtime.py:358-445 drives a stock HF Qwen2 forward per token);
// here each is one launch, bf16 in / bf16 out with fp32 arithmetic inside, rounded at
// the same places as the framework ops they replace.
//
// All kernels read the decode position from device memory, so a captured CUDA graph of
// the step can be replayed for every token.  They are launched with programmatic stream
// serialisation and open with griddepcontrol.launch_dependents / griddepcontrol.wait: the
// launch itself overlaps the tail of whatever precedes them in the stream (the compressed
// linears do the same), and nothing is read before the predecessor has completed.

#include <cuda_bf16.h>

#include <utility>

#include "hxq_common.cuh"

namespace hxq {
namespace dec {

__device__ __forceinline__ float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 to_bf(float v) { return __float2bfloat16_rn(v); }

// Let the next kernel in the stream be scheduled, then wait until everything before this one is done.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ float block_sum(float v, float* red) {   // blockDim.x <= 1024, all threads call
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    __syncthreads();
    return t;
}

// h[b,:] += delta[b,:] (bf16 add, skipped when delta == nullptr); out[b,:] = bf16(bf16(h * rsqrt(mean(h^2) + eps)) * w).
// One CTA per row.  Vector form: H % 8 == 0, 16-byte aligned rows, H <= 8 * 256 * kRmsVec: every thread
// issues all its loads (h, delta, w) before it touches any of them, so the row costs one memory round trip.
constexpr int kRmsVec = 6;

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        f[2 * e] = __uint_as_float(w[e] << 16);
        f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        w[e] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                                                              const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                              int H, int64_t ld_h, int64_t ld_delta, int64_t ld_out, float eps) {
    __shared__ float red[32];
    pdl_enter();
    const int nvec = H >> 3;
    uint4* hp = reinterpret_cast<uint4*>(h + (int64_t)blockIdx.x * ld_h);
    const uint4* dp = delta ? reinterpret_cast<const uint4*>(delta + (int64_t)blockIdx.x * ld_delta) : nullptr;
    const uint4* wp = reinterpret_cast<const uint4*>(w);
    uint4 hv[kRmsVec], dv[kRmsVec], wv[kRmsVec];
#pragma unroll
    for (int j = 0; j < kRmsVec; ++j) {
        const int i = threadIdx.x + j * 256;
        hv[j] = dv[j] = wv[j] = make_uint4(0, 0, 0, 0);
        if (i < nvec) {
            hv[j] = hp[i];
            if (dp) dv[j] = dp[i];
            wv[j] = wp[i];
        }
    }
    float x[kRmsVec][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kRmsVec; ++j) {
        const int i = threadIdx.x + j * 256;
        float d[8];
        unpack8(hv[j], x[j]);
        unpack8(dv[j], d);
        if (dp) {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[j][e] = bf(to_bf(x[j][e] + d[e]));
            if (i < nvec) hp[i] = pack8(x[j]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[j][e] * x[j][e];
    }
    const float tot = block_sum(ss, red);
    const float rs = rsqrtf(tot / (float)H + eps);
    uint4* op = reinterpret_cast<uint4*>(out + (int64_t)blockIdx.x * ld_out);
#pragma unroll
    for (int j = 0; j < kRmsVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < nvec) {
            float wf[8], o[8];
            unpack8(wv[j], wf);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = bf(to_bf(x[j][e] * rs)) * wf[e];
            op[i] = pack8(o);
        }
    }
}

// Any H (<= 12000) and alignment: element-wise, the row kept in shared memory.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                                                          const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                          int H, int64_t ld_h, int64_t ld_delta, int64_t ld_out, float eps) {
    __shared__ float red[32];
    extern __shared__ float row[];   // the updated row in fp32
    pdl_enter();
    __nv_bfloat16* hp = h + (int64_t)blockIdx.x * ld_h;
    const __nv_bfloat16* dp = delta ? delta + (int64_t)blockIdx.x * ld_delta : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = bf(hp[i]);
        if (dp) {
            v = bf(to_bf(v + bf(dp[i])));
            hp[i] = to_bf(v);
        }
        row[i] = v;
        ss += v * v;
    }
    const float tot = block_sum(ss, red);
    const float rs = rsqrtf(tot / (float)H + eps);
    __nv_bfloat16* op = out + (int64_t)blockIdx.x * ld_out;
    for (int i = threadIdx.x; i < H; i += blockDim.x) op[i] = to_bf(bf(to_bf(row[i] * rs)) * bf(w[i]));
}

// Rotary embedding (rotate-half convention) of the new token's q and k heads, k and v appended to the
// cache at row `pos`.  Grid (nq + 2 nkv, B), D/2 threads: thread i owns the pair (i, i + D/2).
__global__ void rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld_qkv, const int64_t* __restrict__ pos_p,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   __nv_bfloat16* __restrict__ q_out, int64_t ld_q,
                                   __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                   int nq, int nkv, int D, int max_len) {
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, half = D >> 1;
    pdl_enter();
    const int64_t pos = *pos_p;
    if (pos < 0 || pos >= max_len) return;
    const __nv_bfloat16* src = qkv + (int64_t)b * ld_qkv + (int64_t)head * D;
    if (head >= nq + nkv) {   // v: plain copy
        __nv_bfloat16* dst = v_cache + (((int64_t)b * nkv + (head - nq - nkv)) * max_len + pos) * D;
        dst[i] = src[i];
        dst[i + half] = src[i + half];
        return;
    }
    const float c0 = cos_t[pos * D + i], s0 = sin_t[pos * D + i];
    const float c1 = cos_t[pos * D + i + half], s1 = sin_t[pos * D + i + half];
    const float x0 = bf(src[i]), x1 = bf(src[i + half]);
    // x * cos + rotate_half(x) * sin, with rotate_half(x) = [-x1, x0], each product rounded as the framework's fp32 ops are
    const __nv_bfloat16 o0 = to_bf(x0 * c0 + (-x1) * s0);
    const __nv_bfloat16 o1 = to_bf(x1 * c1 + x0 * s1);
    __nv_bfloat16* dst = (head < nq) ? q_out + (int64_t)b * ld_q + (int64_t)head * D
                                     : k_cache + (((int64_t)b * nkv + (head - nq)) * max_len + pos) * D;
    dst[i] = o0;
    dst[i + half] = o1;
}

constexpr int kAttnChunk = 64;     // cache positions per CTA
constexpr int kAttnThreads = 128;
constexpr int kAttnMaxGroup = 8;   // query heads per KV head
constexpr int kAttnMaxD = 128;

// One CTA: positions [c*64, c*64+64) of one (sequence, KV head), all query heads of the group.
// Writes per (b, query head, chunk): running max m, sum l and the un-normalised output o[D] (fp32).
__global__ void __launch_bounds__(kAttnThreads) attn_partial_kernel(const __nv_bfloat16* __restrict__ q, int64_t ld_q,
                                                                    const __nv_bfloat16* __restrict__ k_cache,
                                                                    const __nv_bfloat16* __restrict__ v_cache,
                                                                    const int64_t* __restrict__ pos_p, float* __restrict__ part,
                                                                    int nq, int nkv, int D, int max_len, int n_chunks, float scale) {
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, t = threadIdx.x;
    pdl_enter();
    const int64_t pos = *pos_p;
    const int p0 = c * kAttnChunk;
    if (p0 > pos || pos >= max_len) return;
    const int G = nq / nkv;
    const int n_valid = (int)((pos - p0 + 1 < kAttnChunk) ? pos - p0 + 1 : kAttnChunk);

    __shared__ __align__(16) float q_s[kAttnMaxGroup][kAttnMaxD];
    __shared__ __align__(16) __nv_bfloat16 k_s[kAttnChunk][kAttnMaxD + 8];   // +16 B per row: rows start in different banks
    __shared__ __align__(16) __nv_bfloat16 v_s[kAttnChunk][kAttnMaxD + 8];
    __shared__ float s_s[kAttnMaxGroup][kAttnChunk];
    __shared__ float m_s[kAttnMaxGroup], l_s[kAttnMaxGroup];

    // K tile, then V tile, as two asynchronous copy groups: V lands while the scores are computed
    const int64_t base = (((int64_t)b * nkv + kvh) * max_len + p0) * D;
    const int vec_per_row = D / 8;    // 16-byte pieces per row
    for (int i = t; i < n_valid * vec_per_row; i += kAttnThreads) {
        const int r = i / vec_per_row, v = i - r * vec_per_row;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(&k_s[r][v * 8])),
                     "l"(k_cache + base + (int64_t)r * D + v * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = t; i < n_valid * vec_per_row; i += kAttnThreads) {
        const int r = i / vec_per_row, v = i - r * vec_per_row;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(&v_s[r][v * 8])),
                     "l"(v_cache + base + (int64_t)r * D + v * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (t < G * vec_per_row) {   // G * D / 8 <= 128 vectors of q
        const int g = t / vec_per_row, d = (t - g * vec_per_row) * 8;
        const uint4 qv = *reinterpret_cast<const uint4*>(q + (int64_t)b * ld_q + (int64_t)(kvh * G + g) * D + d);
        float f[8];
        unpack8(qv, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) q_s[g][d + e] = f[e] * scale;
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();

    // scores: thread (p = t % 64, hg = t / 64) takes query heads hg, hg + 2, ... of position p
    {
        const int p = t & (kAttnChunk - 1), hg = t / kAttnChunk;
        float acc[kAttnMaxGroup / 2];
#pragma unroll
        for (int j = 0; j < kAttnMaxGroup / 2; ++j) acc[j] = 0.f;
        if (p < n_valid) {
            for (int d = 0; d < D; d += 8) {
                const uint4 kk = *reinterpret_cast<const uint4*>(&k_s[p][d]);
                const uint32_t w[4] = {kk.x, kk.y, kk.z, kk.w};
                float kf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    kf[2 * e] = __uint_as_float(w[e] << 16);
                    kf[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                }
#pragma unroll
                for (int j = 0; j < kAttnMaxGroup / 2; ++j) {
                    const int g = hg + 2 * j;
                    if (g < G) {
                        const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][d]);
                        const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][d + 4]);
                        acc[j] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w
                                + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kAttnMaxGroup / 2; ++j) {
            const int g = hg + 2 * j;
            if (g < G) s_s[g][p] = (p < n_valid) ? acc[j] : -INFINITY;
        }
    }
    __syncthreads();

    // softmax pieces per head
    {
        const int warp = t >> 5, lane = t & 31;
        for (int g = warp; g < G; g += kAttnThreads / 32) {
            const float a0 = s_s[g][lane], a1 = s_s[g][lane + 32];
            float m = fmaxf(a0, a1);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float e0 = __expf(a0 - m), e1 = __expf(a1 - m);   // exp(-inf) = 0 for the masked tail
            float l = e0 + e1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            s_s[g][lane] = e0;
            s_s[g][lane + 32] = e1;
            if (lane == 0) { m_s[g] = m; l_s[g] = l; }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // o[g][d] = sum_p prob[g][p] * V[p][d]; thread t owns dimension d = t (and d + 128 ... if D > 128: not supported)
    if (t < D) {
        float o[kAttnMaxGroup];
#pragma unroll
        for (int g = 0; g < kAttnMaxGroup; ++g) o[g] = 0.f;
        for (int p = 0; p < n_valid; ++p) {
            const float v = bf(v_s[p][t]);
#pragma unroll
            for (int g = 0; g < kAttnMaxGroup; ++g)
                if (g < G) o[g] += s_s[g][p] * v;
        }
#pragma unroll
        for (int g = 0; g < kAttnMaxGroup; ++g)
            if (g < G) {
                float* dst = part + (((int64_t)b * nq + kvh * G + g) * n_chunks + c) * (D + 2);
                dst[2 + t] = o[g];
                if (t == 0) { dst[0] = m_s[g]; dst[1] = l_s[g]; }
            }
    }
}

// out[b, head, :] = sum_c exp(m_c - M) o_c / sum_c exp(m_c - M) l_c over the chunks up to the position.
// 4 x 128 threads: the chunk weights are computed by the block together (dynamic shared memory:
// n_chunks floats); thread (d, j) then adds up dimension d over chunks j, j + 4, ... eight
// independent loads at a time, and the four partial sums meet in shared memory.
constexpr int kCombineGroups = 4;
constexpr int kCombineThreads = kCombineGroups * kAttnMaxD;

__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    __syncthreads();
    return t;
}

__global__ void __launch_bounds__(kCombineThreads) attn_combine_kernel(const float* __restrict__ part, const int64_t* __restrict__ pos_p,
                                                                      __nv_bfloat16* __restrict__ out, int64_t ld_out,
                                                                      int nq, int D, int max_len, int n_chunks) {
    extern __shared__ float w_s[];   // [n_chunks]
    __shared__ float red[32];
    __shared__ float o_s[kCombineGroups][kAttnMaxD];
    const int head = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int d = tid & (kAttnMaxD - 1), j = tid / kAttnMaxD;
    pdl_enter();
    const int64_t pos = *pos_p;
    if (pos < 0 || pos >= max_len) return;
    const int nc = (int)(pos / kAttnChunk) + 1;
    const float* src = part + ((int64_t)b * nq + head) * n_chunks * (D + 2);
    float mx = -INFINITY;
    for (int c = tid; c < nc; c += kCombineThreads) {
        const float m = src[c * (D + 2)];
        w_s[c] = m;
        mx = fmaxf(mx, m);
    }
    mx = block_max(mx, red);
    float ls = 0.f;
    for (int c = tid; c < nc; c += kCombineThreads) {
        const float wgt = __expf(w_s[c] - mx);
        w_s[c] = wgt;
        ls += wgt * src[c * (D + 2) + 1];
    }
    const float L = block_sum(ls, red);   // also makes w_s visible to everyone
    float o = 0.f;
    if (d < D) {
        for (int c0 = j; c0 < nc; c0 += kCombineGroups * 8) {
            float a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c = c0 + k * kCombineGroups;
                a[k] = (c < nc) ? src[c * (D + 2) + 2 + d] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c = c0 + k * kCombineGroups;
                if (c < nc) o += w_s[c] * a[k];
            }
        }
    }
    o_s[j][d] = o;
    __syncthreads();
    if (j == 0 && d < D)
        out[(int64_t)b * ld_out + (int64_t)head * D + d] = to_bf((o_s[0][d] + o_s[1][d] + o_s[2][d] + o_s[3][d]) / L);
}

// out = bf16(bf16(silu(gate)) * up), element-wise over [B, n].
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                              __nv_bfloat16* __restrict__ out, int n, int64_t ld_g, int64_t ld_u, int64_t ld_o) {
    const int b = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    pdl_enter();
    if (i >= n) return;
    const __nv_bfloat16* g = gate + (int64_t)b * ld_g;
    const __nv_bfloat16* u = up + (int64_t)b * ld_u;
    __nv_bfloat16* o = out + (int64_t)b * ld_o;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        if (i + k < n) {
            const float x = bf(g[i + k]);
            const float s = bf(to_bf(x / (1.f + __expf(-x))));
            o[i + k] = to_bf(s * bf(u[i + k]));
        }
    }
}


// ---- dense bf16 weight x up to four tokens (the decoder's lm_head at decode time) -------------------
// y[m, o] = sum_i x[m, i] * W[o, i].  HBM-bound on W (2 bytes per weight, each read once): a warp
// owns FOUR rows at a time, a lane 16 bytes (8 weights) of every 512-byte piece of each, two pieces
// of the four rows (eight loads) in flight per lane; the activations sit in shared memory as fp32 and
// a lane's eight values per token are read once per piece for all four rows (one row per read made
// the shared-memory pipe, not HBM, the limit from two tokens on); fp32 accumulation, one warp
// reduction per row.  W is long-lived (see the weight precondition of the compressed products): its
// first loads are issued before the wait for the previous kernel.
template <int MP>
__global__ void __launch_bounds__(256) dense_gemv_kernel(const __nv_bfloat16* __restrict__ W, int64_t ldw, int n_out, int n_in,
                                                         const __nv_bfloat16* __restrict__ x, int64_t ldx, void* y, int y_dtype,
                                                         int64_t ldy, int M) {
    extern __shared__ __align__(16) float xs[];          // [MP][n_in]
    constexpr int R = 4, U = 2;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_chunk = n_in >> 3;
    const int groups_total = gridDim.x * (blockDim.x >> 5);
    const int n_groups = (n_out + R - 1) / R;
    int grp = blockIdx.x * (blockDim.x >> 5) + warp;
    uint4 w[R][U];
    auto load_w = [&](int g, int c0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = g * R + r;
            const uint4* p = reinterpret_cast<const uint4*>(W + (int64_t)(row < n_out ? row : 0) * ldw);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = c0 + u * 32 + lane;
                w[r][u] = (c < n_chunk && row < n_out) ? __ldcs(p + c) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (grp < n_groups) load_w(grp, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = threadIdx.x; i < MP * n_in; i += blockDim.x) {
        const int m = i / n_in, k = i - m * n_in;
        xs[i] = m < M ? __bfloat162float(x[(int64_t)m * ldx + k]) : 0.f;
    }
    __syncthreads();
    for (; grp < n_groups; grp += groups_total) {
        float acc[R][MP];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[r][m] = 0.f;
        for (int c0 = 0; c0 < n_chunk; c0 += U * 32) {
            if (c0 > 0) load_w(grp, c0);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < n_chunk) {
                    float xf[MP][8];
#pragma unroll
                    for (int m = 0; m < MP; ++m) {
                        const float4 x0 = *reinterpret_cast<const float4*>(xs + m * n_in + c * 8);
                        const float4 x1 = *reinterpret_cast<const float4*>(xs + m * n_in + c * 8 + 4);
                        xf[m][0] = x0.x; xf[m][1] = x0.y; xf[m][2] = x0.z; xf[m][3] = x0.w;
                        xf[m][4] = x1.x; xf[m][5] = x1.y; xf[m][6] = x1.z; xf[m][7] = x1.w;
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t q[4] = {w[r][u].x, w[r][u].y, w[r][u].z, w[r][u].w};
                        float wf[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            wf[2 * j] = __uint_as_float(q[j] << 16);
                            wf[2 * j + 1] = __uint_as_float(q[j] & 0xffff0000u);
                        }
#pragma unroll
                        for (int m = 0; m < MP; ++m) {
                            float a = acc[r][m];
#pragma unroll
                            for (int j = 0; j < 8; ++j) a = fmaf(wf[j], xf[m][j], a);
                            acc[r][m] = a;
                        }
                    }
                }
            }
        }
        // the next rows' first pieces are on their way while these rows are reduced and stored
        const int next = grp + groups_total;
        if (next < n_groups) load_w(next, 0);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = grp * R + r;
#pragma unroll
            for (int m = 0; m < MP; ++m) {
                float v = acc[r][m];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (lane == 0 && m < M && row < n_out) store_from_f32(y, (int64_t)m * ldy + row, v, y_dtype);
            }
        }
    }
}

}  // namespace dec
}  // namespace hxq

using namespace hxq::dec;

extern "C" int hxq_add_rmsnorm(void* h, const void* delta, const void* weight, void* out, int32_t B, int32_t H,
                               int64_t ld_h, int64_t ld_delta, int64_t ld_out, float eps, hxq_stream_t stream) {
    if (!h || !weight || !out || B <= 0 || H <= 0) return HXQ_E_ARG;
    if (H > 12000) return HXQ_E_SHAPE;   // the row is kept in registers / shared memory
    const bool vec = (H % 8 == 0) && H <= 8 * 256 * kRmsVec && hxq::aligned_to(h, 16) && hxq::aligned_to(out, 16) &&
                     hxq::aligned_to(weight, 16) && (!delta || hxq::aligned_to(delta, 16)) && ld_h % 8 == 0 &&
                     ld_out % 8 == 0 && (!delta || ld_delta % 8 == 0);
    const cudaError_t e = launch_pdl(vec ? add_rmsnorm_vec_kernel : add_rmsnorm_kernel, dim3(B), dim3(256),
                                     vec ? 0 : H * sizeof(float), reinterpret_cast<cudaStream_t>(stream),
        reinterpret_cast<__nv_bfloat16*>(h), reinterpret_cast<const __nv_bfloat16*>(delta),
        reinterpret_cast<const __nv_bfloat16*>(weight), reinterpret_cast<__nv_bfloat16*>(out), (int)H, ld_h, ld_delta, ld_out, eps);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

extern "C" int hxq_rope_append(const void* qkv, int64_t ld_qkv, const int64_t* pos, const float* cos_table,
                               const float* sin_table, void* q_out, int64_t ld_q, void* k_cache, void* v_cache,
                               int32_t B, int32_t nq, int32_t nkv, int32_t D, int32_t max_len, hxq_stream_t stream) {
    if (!qkv || !pos || !cos_table || !sin_table || !q_out || !k_cache || !v_cache) return HXQ_E_ARG;
    if (B <= 0 || nq <= 0 || nkv <= 0 || D <= 0 || (D & 1) || D > 2048 || max_len <= 0) return HXQ_E_SHAPE;
    const cudaError_t e = launch_pdl(rope_append_kernel, dim3(nq + 2 * nkv, B), dim3(D / 2), 0, reinterpret_cast<cudaStream_t>(stream),
        reinterpret_cast<const __nv_bfloat16*>(qkv), ld_qkv, pos, cos_table, sin_table,
        reinterpret_cast<__nv_bfloat16*>(q_out), ld_q, reinterpret_cast<__nv_bfloat16*>(k_cache),
        reinterpret_cast<__nv_bfloat16*>(v_cache), (int)nq, (int)nkv, (int)D, (int)max_len);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

extern "C" size_t hxq_attn_decode_workspace_bytes(int32_t B, int32_t nq, int32_t D, int32_t max_len) {
    if (B <= 0 || nq <= 0 || D <= 0 || max_len <= 0) return 0;
    const size_t n_chunks = ((size_t)max_len + kAttnChunk - 1) / kAttnChunk;
    return (size_t)B * nq * n_chunks * (D + 2) * sizeof(float);
}

extern "C" int hxq_attn_decode(const void* q, int64_t ld_q, const void* k_cache, const void* v_cache, const int64_t* pos,
                               void* out, int64_t ld_out, void* workspace, size_t workspace_bytes, int32_t B, int32_t nq,
                               int32_t nkv, int32_t D, int32_t max_len, float scale, hxq_stream_t stream) {
    if (!q || !k_cache || !v_cache || !pos || !out) return HXQ_E_ARG;
    if (B <= 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > kAttnMaxGroup) return HXQ_E_SHAPE;
    if (D <= 0 || D > kAttnMaxD || D % 8 != 0 || max_len <= 0 || max_len > 64 * 8192) return HXQ_E_SHAPE;
    if (!hxq::aligned_to(q, 16) || ld_q % 8 != 0) return HXQ_E_ALIGN;
    if (!hxq::aligned_to(k_cache, 16) || !hxq::aligned_to(v_cache, 16)) return HXQ_E_ALIGN;
    if (!workspace || workspace_bytes < hxq_attn_decode_workspace_bytes(B, nq, D, max_len)) return HXQ_E_WORKSPACE;
    const int n_chunks = (max_len + kAttnChunk - 1) / kAttnChunk;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (launch_pdl(attn_partial_kernel, dim3(n_chunks, nkv, B), dim3(kAttnThreads), 0, s,
                   reinterpret_cast<const __nv_bfloat16*>(q), ld_q, reinterpret_cast<const __nv_bfloat16*>(k_cache),
                   reinterpret_cast<const __nv_bfloat16*>(v_cache), pos, reinterpret_cast<float*>(workspace), (int)nq, (int)nkv,
                   (int)D, (int)max_len, n_chunks, scale) != cudaSuccess)
        return HXQ_E_LAUNCH;
    const cudaError_t e = launch_pdl(attn_combine_kernel, dim3(nq, B), dim3(kCombineThreads), n_chunks * sizeof(float), s,
                                     reinterpret_cast<const float*>(workspace), pos, reinterpret_cast<__nv_bfloat16*>(out), ld_out,
                                     (int)nq, (int)D, (int)max_len, n_chunks);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

extern "C" int hxq_swiglu(const void* gate, const void* up, void* out, int32_t B, int32_t n, int64_t ld_gate,
                          int64_t ld_up, int64_t ld_out, hxq_stream_t stream) {
    if (!gate || !up || !out || B <= 0 || n <= 0) return HXQ_E_ARG;
    const int threads = 256, per_block = threads * 2;
    const cudaError_t e = launch_pdl(swiglu_kernel, dim3((n + per_block - 1) / per_block, B), dim3(threads), 0,
        reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(gate),
        reinterpret_cast<const __nv_bfloat16*>(up), reinterpret_cast<__nv_bfloat16*>(out), (int)n, ld_gate, ld_up, ld_out);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

template <int MP>
static int launch_dense_gemv(const __nv_bfloat16* W, int64_t ldw, int n_out, int n_in, const __nv_bfloat16* x, int64_t ldx,
                             void* y, int y_dtype, int64_t ldy, int M, cudaStream_t stream) {
    const size_t smem = (size_t)MP * n_in * sizeof(float);
    static size_t smem_set[64] = {0};
    int dev = 0, n_sm = 148, occ = 1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HXQ_E_DEVICE;
    if (smem > 48 * 1024 && smem_set[dev] < smem) {
        if (cudaFuncSetAttribute(dense_gemv_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return HXQ_E_SHAPE;
        smem_set[dev] = smem;
    }
    // SM count and resident CTAs per SM, asked once per device and shared-memory size
    static int sm_cached[64] = {0}, occ_cached[64] = {0};
    static size_t occ_smem[64] = {0};
    if (sm_cached[dev] == 0) {
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
        sm_cached[dev] = n_sm;
    }
    if (occ_cached[dev] == 0 || occ_smem[dev] != smem) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, dense_gemv_kernel<MP>, 256, smem) != cudaSuccess || occ < 1) occ = 1;
        occ_cached[dev] = occ;
        occ_smem[dev] = smem;
    }
    int grid = sm_cached[dev] * occ_cached[dev];
    const int need = (n_out + 31) / 32;      // eight warps of four rows per CTA
    if (grid > need) grid = need;
    const cudaError_t e = launch_pdl(dense_gemv_kernel<MP>, dim3(grid), dim3(256), smem, stream, W, ldw, n_out, n_in, x, ldx, y,
                                     y_dtype, ldy, M);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

extern "C" int hxq_dense_gemv(const void* weight, int32_t out_features, int32_t in_features, int64_t ldw, const void* x,
                              int32_t M, int64_t ldx, void* y, int y_dtype, int64_t ldy, hxq_stream_t stream_) {
    if (!weight || !x || !y || out_features <= 0 || in_features <= 0 || M <= 0 || M > 4) return HXQ_E_ARG;
    if (in_features % 8 != 0 || in_features > 12288 || ldw < in_features || ldw % 8 != 0 || ldx < in_features || ldy < out_features)
        return HXQ_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(weight) & 15) != 0) return HXQ_E_ALIGN;
    if (y_dtype != HXQ_F32 && y_dtype != HXQ_F16 && y_dtype != HXQ_BF16) return HXQ_E_DTYPE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(weight);
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
    if (M == 1) return launch_dense_gemv<1>(W, ldw, out_features, in_features, xb, ldx, y, y_dtype, ldy, M, stream);
    if (M == 2) return launch_dense_gemv<2>(W, ldw, out_features, in_features, xb, ldx, y, y_dtype, ldy, M, stream);
    return launch_dense_gemv<4>(W, ldw, out_features, in_features, xb, ldx, y, y_dtype, ldy, M, stream);
}
