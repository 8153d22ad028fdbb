// hxq_allreduce_oneshot: the sum over tensor-parallel ranks after a row-parallel product
// (o_proj, down_proj) for decode-sized messages, as ONE kernel per rank over peer memory.
//
// Every rank owns a receive buffer that all ranks of the node can write (symmetric memory:
// the same allocation made on every GPU and mapped into every process).  A call PUSHES this
// rank's fp32 partial sums into slot [rank] of every rank's buffer with plain peer stores,
// raises a flag beside it, waits until the flags of all ranks are up in its own buffer, and
// adds the world's partials from LOCAL memory in rank order (the same order on every rank:
// results are bit-identical across ranks and from run to run), rounding once to bf16.
//
//  * no collective library, no multicast of any kind: ordinary stores to peer pointers, a
//    system-scope fence, ordinary loads of local memory that bypass L1;
//  * two slots alternate by call, so a rank that races ahead into call e+1 cannot overwrite
//    what a slower rank is still reading for call e (it cannot get to e+2 before every rank
//    has raised its e+1 flag, i.e. has finished e);
//  * flags carry the call number, read from a per-CTA counter in device memory that the
//    kernel itself advances: nothing has to be reset, and a captured CUDA graph replays
//    correctly because the call number is not a launch argument;
//  * each CTA handles its own 4096-element slice with its own flags and counter: no
//    grid-wide synchronisation; at most 32 CTAs, all resident at once;
//  * the wait is bounded (clock64): on expiry the CTA records HXQ_E_TIMEOUT in the status
//    word and returns without touching the output.
//
// The reference has no multi-GPU path at all; this replaces what torch.distributed.all_reduce
// (NCCL) does for the two row-parallel projections of a layer.

#include <cuda_bf16.h>

#include "hxq_common.cuh"

namespace hxq {
namespace ar {

constexpr int kThreads = 512;
constexpr int kPerCta = kThreads * 8;   // elements per CTA
constexpr int kMaxCtas = 32;
constexpr int kMaxWorld = 8;

struct Peers {
    float* buf[kMaxWorld];          // rank p's receive buffer: [2 slots][world][n_max] fp32
    uint32_t* flag[kMaxWorld];      // rank p's flags: [2 slots][world][kMaxCtas]
};

__global__ void __launch_bounds__(kThreads) allreduce_oneshot_kernel(const Peers peers, int rank, int world, int64_t n_max,
                                                                     const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                                     int64_t n, uint32_t* __restrict__ counters,
                                                                     long long wait_cycles, int32_t* __restrict__ status) {
    __shared__ uint32_t epoch_s;
    __shared__ int ok_s;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // src is the previous kernel's output
    const int cta = blockIdx.x, t = threadIdx.x;
    if (t == 0) {
        epoch_s = counters[cta] + 1u;
        counters[cta] = epoch_s;
        ok_s = 1;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int slot = (int)(epoch & 1u);
    const int64_t i0 = (int64_t)cta * kPerCta + (int64_t)t * 8;

    // push this rank's slice into slot [rank] of every rank's buffer (its own included)
    if (i0 < n) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (i0 + e < n) ? src[i0 + e] : 0.f;
        for (int p = 0; p < world; ++p) {
            float* d = peers.buf[p] + ((int64_t)slot * world + rank) * n_max + i0;
            *reinterpret_cast<float4*>(d) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(d + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (t < world) {   // one flag per destination rank, written after every thread's stores are fenced
        volatile uint32_t* f = peers.flag[t] + ((int64_t)slot * world + rank) * kMaxCtas + cta;
        *f = epoch;
    }
    // wait for the flags of all ranks in this rank's own memory
    if (t < world) {
        volatile uint32_t* f = peers.flag[rank] + ((int64_t)slot * world + t) * kMaxCtas + cta;
        const long long t0 = clock64();
        while (*f != epoch) {
            if (clock64() - t0 > wait_cycles) { ok_s = 0; break; }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (!ok_s) {
        if (t == 0 && status != nullptr) atomicExch(status, HXQ_E_TIMEOUT);
        return;
    }
    if (i0 < n) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const float* base = peers.buf[rank] + (int64_t)slot * world * n_max + i0;
        for (int p = 0; p < world; ++p) {   // fixed order: the same sum on every rank
            const float4 a = __ldcg(reinterpret_cast<const float4*>(base + (int64_t)p * n_max));
            const float4 b = __ldcg(reinterpret_cast<const float4*>(base + (int64_t)p * n_max + 4));
            acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
            acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (i0 + e < n) dst[i0 + e] = __float2bfloat16_rn(acc[e]);
    }
}


// The same exchange with what follows it in a decoder layer folded in: after the sum over ranks the
// row is added to the residual stream and RMS-normalised for the next projection,
//     delta = bf16(sum_p partial_p);  h = bf16(h + delta);  out = bf16(bf16(h * rsqrt(mean(h^2) + eps)) * w),
// rounded exactly where the separate kernels (hxq_allreduce_oneshot, then hxq_add_rmsnorm) round, so
// the fused step is bit-identical to the unfused one.  One CTA owns whole rows (row r goes to CTA
// r mod gridDim.x; H <= 8192) because the norm needs the whole row; flags, slots and call numbers
// work as above, one flag per CTA covering all of its rows.
constexpr int kRowMaxH = kThreads * 8 * 2;

__global__ void __launch_bounds__(kThreads) allreduce_add_rmsnorm_kernel(
    const Peers peers, int rank, int world, int64_t n_max, const float* __restrict__ src, int M, int H,
    __nv_bfloat16* __restrict__ h, int64_t ld_h, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
    int64_t ld_out, float eps, uint32_t* __restrict__ counters, long long wait_cycles, int32_t* __restrict__ status) {
    __shared__ uint32_t epoch_s;
    __shared__ int ok_s;
    __shared__ float red[kThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // src and h are earlier kernels' outputs
    const int cta = blockIdx.x, t = threadIdx.x, G = gridDim.x;
    if (t == 0) {
        epoch_s = counters[cta] + 1u;
        counters[cta] = epoch_s;
        ok_s = 1;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int slot = (int)(epoch & 1u);

    // push this rank's partial rows into slot [rank] of every rank's buffer (its own included)
    for (int r = cta; r < M; r += G) {
        for (int c0 = t * 8; c0 < H; c0 += kThreads * 8) {
            const int64_t i0 = (int64_t)r * H + c0;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (c0 + e < H) ? src[i0 + e] : 0.f;
            for (int p = 0; p < world; ++p) {
                float* d = peers.buf[p] + ((int64_t)slot * world + rank) * n_max + i0;
                if (c0 + 8 <= H && (i0 & 3) == 0) {
                    *reinterpret_cast<float4*>(d) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(d + 4) = make_float4(v[4], v[5], v[6], v[7]);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (c0 + e < H) d[e] = v[e];
                }
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (t < world) {
        volatile uint32_t* f = peers.flag[t] + ((int64_t)slot * world + rank) * kMaxCtas + cta;
        *f = epoch;
    }
    if (t < world) {
        volatile uint32_t* f = peers.flag[rank] + ((int64_t)slot * world + t) * kMaxCtas + cta;
        const long long t0 = clock64();
        while (*f != epoch) {
            if (clock64() - t0 > wait_cycles) { ok_s = 0; break; }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (!ok_s) {
        if (t == 0 && status != nullptr) atomicExch(status, HXQ_E_TIMEOUT);
        return;
    }
    for (int r = cta; r < M; r += G) {
        float hv[2][8];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c0 = t * 8 + j * kThreads * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) hv[j][e] = 0.f;
            if (c0 < H) {
                const float* base = peers.buf[rank] + (int64_t)slot * world * n_max + (int64_t)r * H + c0;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int p = 0; p < world; ++p) {   // fixed order: the same sum on every rank
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (c0 + e < H) acc[e] += __ldcg(base + (int64_t)p * n_max + e);
                }
                __nv_bfloat16* hp = h + (int64_t)r * ld_h + c0;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    if (c0 + e < H) {
                        const float delta = __bfloat162float(__float2bfloat16_rn(acc[e]));
                        const __nv_bfloat16 hn = __float2bfloat16_rn(__bfloat162float(hp[e]) + delta);
                        hp[e] = hn;
                        hv[j][e] = __bfloat162float(hn);
                        ss += hv[j][e] * hv[j][e];
                    }
                }
            }
        }
        // block sum of squares
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        __syncthreads();                      // red[] from the previous row has been read by everyone
        if ((t & 31) == 0) red[t >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int q = 0; q < kThreads / 32; ++q) tot += red[q];
        const float rs = rsqrtf(tot / (float)H + eps);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c0 = t * 8 + j * kThreads * 8;
            if (c0 < H) {
                __nv_bfloat16* op = out + (int64_t)r * ld_out + c0;
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (c0 + e < H)
                        op[e] = __float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(hv[j][e] * rs)) * __bfloat162float(w[c0 + e]));
            }
        }
    }
}

}  // namespace ar
}  // namespace hxq

extern "C" size_t hxq_allreduce_buffer_bytes(int32_t world, int64_t n_max) {
    if (world <= 0 || world > hxq::ar::kMaxWorld || n_max <= 0) return 0;
    return (size_t)2 * world * (size_t)n_max * sizeof(float);
}

extern "C" size_t hxq_allreduce_flag_bytes(int32_t world) {
    if (world <= 0 || world > hxq::ar::kMaxWorld) return 0;
    return (size_t)2 * world * hxq::ar::kMaxCtas * sizeof(uint32_t);
}

extern "C" int hxq_allreduce_oneshot(void* const* peer_buffers, void* const* peer_flags, int32_t rank, int32_t world,
                                     int64_t n_max, const void* src, void* dst, int64_t n, void* counters,
                                     int64_t wait_cycles, int32_t* status, hxq_stream_t stream) {
    using namespace hxq::ar;
    if (!peer_buffers || !peer_flags || !src || !dst || !counters) return HXQ_E_ARG;
    if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world) return HXQ_E_ARG;
    if (n <= 0 || n > n_max || n_max % 8 != 0 || n > (int64_t)kPerCta * kMaxCtas) return HXQ_E_SHAPE;
    if (!hxq::aligned_to(src, 16)) return HXQ_E_ALIGN;
    Peers peers;
    for (int p = 0; p < kMaxWorld; ++p) {
        peers.buf[p] = p < world ? reinterpret_cast<float*>(peer_buffers[p]) : nullptr;
        peers.flag[p] = p < world ? reinterpret_cast<uint32_t*>(peer_flags[p]) : nullptr;
        if (p < world && (!peers.buf[p] || !peers.flag[p] || !hxq::aligned_to(peers.buf[p], 16))) return HXQ_E_ARG;
    }
    const int grid = (int)((n + kPerCta - 1) / kPerCta);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long limit = wait_cycles > 0 ? (long long)wait_cycles : 2000000000LL;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel, peers, (int)rank, (int)world, n_max,
                                             reinterpret_cast<const float*>(src), reinterpret_cast<__nv_bfloat16*>(dst), n,
                                             reinterpret_cast<uint32_t*>(counters), limit, status);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

extern "C" int hxq_allreduce_add_rmsnorm(void* const* peer_buffers, void* const* peer_flags, int32_t rank, int32_t world,
                                         int64_t n_max, const void* src, int32_t M, int32_t H, void* h, int64_t ld_h,
                                         const void* weight, void* out, int64_t ld_out, float eps, void* counters,
                                         int64_t wait_cycles, int32_t* status, hxq_stream_t stream) {
    using namespace hxq::ar;
    if (!peer_buffers || !peer_flags || !src || !h || !weight || !out || !counters) return HXQ_E_ARG;
    if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world) return HXQ_E_ARG;
    if (M <= 0 || H <= 0 || H > kRowMaxH || (int64_t)M * H > n_max || n_max % 8 != 0) return HXQ_E_SHAPE;
    if (ld_h < H || ld_out < H) return HXQ_E_SHAPE;
    Peers peers;
    for (int p = 0; p < kMaxWorld; ++p) {
        peers.buf[p] = p < world ? reinterpret_cast<float*>(peer_buffers[p]) : nullptr;
        peers.flag[p] = p < world ? reinterpret_cast<uint32_t*>(peer_flags[p]) : nullptr;
        if (p < world && (!peers.buf[p] || !peers.flag[p] || !hxq::aligned_to(peers.buf[p], 16))) return HXQ_E_ARG;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M < kMaxCtas ? M : kMaxCtas);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long limit = wait_cycles > 0 ? (long long)wait_cycles : 2000000000LL;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, allreduce_add_rmsnorm_kernel, peers, (int)rank, (int)world, n_max,
                                             reinterpret_cast<const float*>(src), (int)M, (int)H,
                                             reinterpret_cast<__nv_bfloat16*>(h), ld_h,
                                             reinterpret_cast<const __nv_bfloat16*>(weight),
                                             reinterpret_cast<__nv_bfloat16*>(out), ld_out, eps,
                                             reinterpret_cast<uint32_t*>(counters), limit, status);
    return e == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}
