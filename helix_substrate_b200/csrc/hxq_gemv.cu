// hxq_gemv: decode-time product y[m,o] = sum_i x[m,i] * W^[o,i] + sidecar + bias, M <= 16.
//
// HBM-bound: 1 index byte per weight is the traffic, and every index byte is one
// codebook lookup, so the second wall is the shared-memory lookup rate (32 words
// per clock per SM).  Design, all of it in service of those two walls:
//
//  * Work unit = 8 rows x 512 columns of indices (4 KB).  A warp reads a unit as
//    8 coalesced 512-byte row segments, one 16-byte streaming load per lane per
//    row, straight into registers (no shared-memory staging: the lookup traffic
//    already needs most of the shared-memory bandwidth).  The next unit's loads
//    are issued before the current unit is consumed (register double buffer).
//  * Units are numbered chunk-major (all row blocks of column chunk 0, then chunk
//    1, ...) and dealt to the warps of a persistent grid (one CTA per SM) as equal
//    contiguous ranges, so every SM streams the same number of bytes whatever the
//    shape, and a warp keeps its 16 activations per token in registers for many
//    consecutive units.
//  * The 256-entry codebook is replicated per lane in shared memory at a 256-byte
//    stride (entry c, lane l at byte c*256 + l*4): every lookup hits bank == lane,
//    conflict free, and the address (c << 8) | (l << 2) is ONE byte-permute of the
//    index word with a per-lane constant.  Inner loop per weight: PRMT, LDS, FFMA.
//  * The group affine is applied to per-(row, group) partial sums, not to weights:
//    sum_i x_i (c_i s + t) = s * sum_i x_i c_i + t * sum_i x_i.  Eight lanes span one
//    128-column group, so after three exchange steps of the warp butterfly each
//    lane holds the partial of one (row, group) and needs one s and one t.
//  * Column chunks of one row block are summed deterministically: every unit
//    writes its 8 x M partials to scratch, bumps an arrival counter, and the last
//    arriver adds the partials in chunk order, adds the bias and stores y.  No
//    float atomics, so results are bit-identical from run to run.
//  * The sidecar (row-sorted CSR of deltas) of a row block is added by the unit
//    whose chunk equals rowblock % nchunks, which spreads that work evenly.

#include "hxq_common.cuh"

namespace hxq {

constexpr int kRows = 8;          // rows per unit
constexpr int kChunk = 512;       // columns per unit (32 lanes x 16)
constexpr int kLutBytes = 256 * 256;
constexpr int kGemvSmemBytes = 2 * kLutBytes;  // the table sits on a 64 KB boundary inside this window

struct GemvArgs {
    const uint8_t* idx;
    const float* cb;
    const void* scales;
    const void* offsets;
    const int32_t* rowptr;
    const int32_t* cols;
    const float* deltas;
    const float* bias;
    const void* x;
    void* y;
    float* partial;
    unsigned int* counters;
    int64_t ld_idx, ldx, ldy;
    int64_t units;
    int32_t out_features, in_features, col0, group_size, ld_st, st_dtype;
    int32_t x_dtype, y_dtype, x_vec;
    int32_t M;       // tokens in this launch (<= MP)
    int32_t kbase;   // local column of chunk 0, lane 0: -(col0 % 128)
    int32_t nch;     // column chunks
    int32_t nrb;     // row blocks
    int32_t total_warps;
};

struct GemvPlan {
    int nch, nrb, kbase, grid, warps_per_cta;
    int64_t units;
    size_t counter_bytes, partial_bytes;
};

template <int MP>
__device__ __forceinline__ void load_x_chunk(const GemvArgs& a, int col, bool col_ok, float (&xr)[MP][16]) {
#pragma unroll
    for (int m = 0; m < MP; ++m) {
        if (!col_ok || m >= a.M) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xr[m][j] = 0.f;
            continue;
        }
        const int64_t o = (int64_t)m * a.ldx + col;
        if (a.x_vec) {
            if (a.x_dtype == HXQ_F32) {
                const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) + o);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float4 v = p[j];
                    xr[m][4 * j] = v.x; xr[m][4 * j + 1] = v.y; xr[m][4 * j + 2] = v.z; xr[m][4 * j + 3] = v.w;
                }
            } else {
                const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.x) + o);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint4 v = p[j];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float lo, hi;
                        if (a.x_dtype == HXQ_BF16) {
                            lo = __uint_as_float(w[k] << 16);
                            hi = __uint_as_float(w[k] & 0xffff0000u);
                        } else {
                            __half2 h = *reinterpret_cast<const __half2*>(&w[k]);
                            lo = __low2float(h); hi = __high2float(h);
                        }
                        xr[m][8 * j + 2 * k] = lo; xr[m][8 * j + 2 * k + 1] = hi;
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) xr[m][j] = load_as_f32(a.x, o + j, a.x_dtype);
        }
    }
}

// One exchange step of the warp butterfly: n values -> n/2, summed across lane^off.
template <int N>
__device__ __forceinline__ void halve(float* v, int lane, int off) {
    constexpr int H = N / 2;
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < H; ++i) {
        const float keep = up ? v[H + i] : v[i];
        const float send = up ? v[i] : v[H + i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
}

template <int MP>
struct GemvCfg {
    static constexpr int kMaxThreads = (MP == 1) ? 512 : (MP == 2 ? 384 : 256);
};

// What a warp fetches one unit ahead of consuming it.
struct UnitPrefetch {
    uint4 q[kRows];   // 16 index bytes per row for this lane
    float s, t;       // group scale / offset of (row lane&7, 128-column span lane>>3)
    int e0, e1;       // sidecar entries of row lane&7 when this unit carries the row block's sidecar
};

// One codebook lookup: the byte permute builds the ABSOLUTE shared address
// lut_base | code << 8 | lane << 2 (lut_base is a multiple of 64 KB), so the
// inner loop per weight is exactly PRMT, LDS, FFMA.
__device__ __forceinline__ float lut_at(uint32_t word, uint32_t lane_key, int k) {
    const uint32_t addr = __byte_perm(word, lane_key, 0x7604u | (uint32_t)(k << 4));
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

template <int MP>
__global__ void __launch_bounds__(GemvCfg<MP>::kMaxThreads, 1) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(1024) char dyn_smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int gw = blockIdx.x * (blockDim.x >> 5) + warp;
    // table at the next 64 KB boundary of the shared window (the launch reserves 128 KB)
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(dyn_smem));
    const uint32_t lut_base = (smem_base + 0xFFFFu) & ~0xFFFFu;
    char* lut = dyn_smem + (lut_base - smem_base);
    const uint32_t lane_key = lut_base | ((uint32_t)lane << 2);

    const int n_units = (int)a.units;
    const int u_begin = (int)((int64_t)n_units * gw / a.total_warps);
    const int u_end = (int)((int64_t)n_units * (gw + 1) / a.total_warps);
    const int r_l = lane & 7;    // row this lane ends up holding after the butterfly
    const int h_l = lane >> 3;   // 128-column span of the chunk this lane belongs to
    const bool affine = a.group_size > 0;
    const int g_base = affine ? a.col0 / a.group_size : 0;

    auto fetch = [&](int ch, int rb, int own, UnitPrefetch& f) {
        const int col = a.kbase + ch * kChunk + lane * 16;
        const bool ok = (col >= 0) && (col < a.in_features);
        const int row0 = rb * kRows;
        const int rmax = a.out_features - 1 - row0;
        const uint8_t* p = a.idx + (int64_t)row0 * a.ld_idx + col;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int rr = r < rmax ? r : rmax;   // rows past the end re-read the last row (never stored)
            f.q[r] = ok ? ld_stream_u4(p + (int64_t)rr * a.ld_idx) : make_uint4(0, 0, 0, 0);
        }
        const int row_l = row0 + r_l;
        const bool row_ok = row_l < a.out_features;
        f.s = 1.f; f.t = 0.f;
        if (affine) {
            const int span_col = a.kbase + ch * kChunk + h_l * 128;
            if (span_col < a.in_features && row_ok) {
                const int64_t o = (int64_t)row_l * a.ld_st + ((a.col0 + span_col) / a.group_size - g_base);
                if (a.st_dtype == HXQ_F32) {
                    f.s = reinterpret_cast<const float*>(a.scales)[o];
                    f.t = reinterpret_cast<const float*>(a.offsets)[o];
                } else {
                    f.s = __half2float(reinterpret_cast<const __half*>(a.scales)[o]);
                    f.t = __half2float(reinterpret_cast<const __half*>(a.offsets)[o]);
                }
            }
        }
        f.e0 = 0; f.e1 = 0;
        if (a.rowptr != nullptr && ch == own && row_ok) {
            f.e0 = a.rowptr[row_l];
            f.e1 = a.rowptr[row_l + 1];
        }
    };

    // unit u = ch * nrb + rb; `own` = rb % nch is the chunk that carries the sidecar of row block rb
    int ch = 0, rb = 0, own = 0;
    if (u_begin < u_end) {
        ch = u_begin / a.nrb;
        rb = u_begin - ch * a.nrb;
        own = rb % a.nch;
    }
    auto advance = [&]() {
        ++rb; ++own;
        if (own == a.nch) own = 0;
        if (rb == a.nrb) { rb = 0; own = 0; ++ch; }
    };

    // First unit's loads go out before the table is built: the first HBM round
    // trip overlaps the set-up.
    UnitPrefetch fa, fb;
    if (u_begin < u_end) fetch(ch, rb, own, fa);

    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x)
        *reinterpret_cast<float*>(lut + (i >> 5) * 256 + (i & 31) * 4) = a.cb[i >> 5];
    __syncthreads();

    float xr[MP][16];
    float xsum[MP];
#pragma unroll
    for (int m = 0; m < MP; ++m) xsum[m] = 0.f;
    int cur_ch = -1;

    auto process = [&](int pch, int prb, const UnitPrefetch& f) {
        const int col = a.kbase + pch * kChunk + lane * 16;
        const bool col_ok = (col >= 0) && (col < a.in_features);
        if (pch != cur_ch) {  // warp-uniform
            cur_ch = pch;
            load_x_chunk<MP>(a, col, col_ok, xr);
            if (affine) {
#pragma unroll
                for (int m = 0; m < MP; ++m) {
                    float sx = 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) sx += xr[m][j];
                    sx += __shfl_xor_sync(0xffffffffu, sx, 4);
                    sx += __shfl_xor_sync(0xffffffffu, sx, 2);
                    sx += __shfl_xor_sync(0xffffffffu, sx, 1);
                    xsum[m] = sx;  // sum of x over this lane's 128-column span
                }
            }
        }

        // ---- lookups + FMAs: acc[r*MP + m] = this lane's 16-column partial ----
        float acc[kRows * MP];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const uint32_t w[4] = {f.q[r].x, f.q[r].y, f.q[r].z, f.q[r].w};
            float p0[MP], p1[MP];
#pragma unroll
            for (int m = 0; m < MP; ++m) { p0[m] = 0.f; p1[m] = 0.f; }
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const float w0 = lut_at(w[j >> 2], lane_key, j & 3);
                const float w1 = lut_at(w[(j + 1) >> 2], lane_key, (j + 1) & 3);
#pragma unroll
                for (int m = 0; m < MP; ++m) {
                    p0[m] = fmaf(w0, xr[m][j], p0[m]);
                    p1[m] = fmaf(w1, xr[m][j + 1], p1[m]);
                }
            }
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[r * MP + m] = col_ok ? (p0[m] + p1[m]) : 0.f;
        }

        // ---- butterfly over the 8 lanes of a group span: rows are dealt out ----
        halve<kRows * MP>(acc, lane, 4);
        halve<kRows * MP / 2>(acc, lane, 2);
        halve<kRows * MP / 4>(acc, lane, 1);
        // now acc[0..MP) = partial of row (lane & 7) over span (lane >> 3), per token
        const int row_l = prb * kRows + r_l;
        const bool row_ok = row_l < a.out_features;
        if (affine) {
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[m] = fmaf(f.s, acc[m], f.t * xsum[m]);
        }

        // ---- sidecar: the four lanes holding row r each take every 4th entry ----
        for (int e = f.e0 + h_l; e < f.e1; e += 4) {
            const int c = a.cols[e];
            const float dl = a.deltas[e];
#pragma unroll
            for (int m = 0; m < MP; ++m)
                if (m < a.M) acc[m] = fmaf(dl, load_as_f32(a.x, (int64_t)m * a.ldx + c, a.x_dtype), acc[m]);
        }

        // ---- finish across the four spans; tokens are dealt out for MP > 1 ----
        int m_l = 0;
        if (MP == 4) {
            halve<4>(acc, lane, 8);
            halve<2>(acc, lane, 16);
            m_l = ((lane >> 3) & 1) * 2 + ((lane >> 4) & 1);
        } else if (MP == 2) {
            halve<2>(acc, lane, 8);
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 16);
            m_l = (lane >> 3) & 1;
        } else {
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 8);
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 16);
        }
        float v = acc[0];
        const bool writer = (MP == 4) ? true : (MP == 2 ? (lane < 16) : (lane < 8));
        if (a.nch > 1) {
            // partial of this (row block, chunk); summed by whoever arrives last (after the loop)
            if (writer)
                __stcg(a.partial + ((int64_t)prb * a.nch + pch) * (kRows * MP) + r_l * MP + m_l, v);
        } else if (writer && row_ok && m_l < a.M) {
            if (a.bias != nullptr) v += a.bias[row_l];
            store_from_f32(a.y, (int64_t)m_l * a.ldy + row_l, v, a.y_dtype);
        }
    };

    for (int u = u_begin; u < u_end; u += 2) {
        const int cha = ch, rba = rb;
        advance();
        const bool has_b = (u + 1 < u_end);
        if (has_b) fetch(ch, rb, own, fb);
        process(cha, rba, fa);
        if (has_b) {
            const int chb = ch, rbb = rb;
            advance();
            if (u + 2 < u_end) fetch(ch, rb, own, fa);
            process(chb, rbb, fb);
        }
    }

    // ---- arrival + reduction, once per warp and off the streaming loop ----
    // (a fence or an atomic per unit would wait for the prefetched index loads
    // and serialise the pipeline).  Each lane announces one unit; the warp then
    // finishes every row block for which it was the last chunk to arrive:
    // partials are added in chunk order, so the result does not depend on timing.
    if (a.nch > 1 && u_begin < u_end) {
        __threadfence();
        __syncwarp();
        for (int base = u_begin; base < u_end; base += 32) {
            const int u = base + lane;
            bool last = false;
            int rbu = 0;
            if (u < u_end) {
                rbu = u % a.nrb;
                last = atomicAdd(a.counters + rbu, 1u) == (unsigned int)(a.nch - 1);
            }
            unsigned int todo = __ballot_sync(0xffffffffu, last);
            if (todo != 0u) __threadfence();
            while (todo != 0u) {
                const int src = __ffs(todo) - 1;
                todo &= todo - 1u;
                const int rbf = __shfl_sync(0xffffffffu, rbu, src);
                if (lane < kRows * MP) {
                    const float* p = a.partial + (int64_t)rbf * a.nch * (kRows * MP) + lane;
                    float v = 0.f;
                    for (int c = 0; c < a.nch; ++c) v += __ldcg(p + (int64_t)c * (kRows * MP));
                    const int row = rbf * kRows + lane / MP;
                    const int m = lane % MP;
                    if (row < a.out_features && m < a.M) {
                        if (a.bias != nullptr) v += a.bias[row];
                        store_from_f32(a.y, (int64_t)m * a.ldy + row, v, a.y_dtype);
                    }
                }
                if (lane == src) a.counters[rbf] = 0u;  // leave the workspace clean for the next call
            }
        }
    }
}

// Any-shape fallback (ragged IN, unaligned pointers, group sizes that are not a
// multiple of 128): one warp per output row, byte loads.  Correct, not fast.
__global__ void __launch_bounds__(256) gemv_generic_kernel(const GemvArgs a) {
    __shared__ float cb_s[256];
    cb_s[threadIdx.x] = a.cb[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= a.out_features) return;
    const int gbase = a.group_size > 0 ? a.col0 / a.group_size : 0;
    for (int m0 = 0; m0 < a.M; m0 += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int col = lane; col < a.in_features; col += 32) {
            float w = cb_s[a.idx[(int64_t)row * a.ld_idx + col]];
            if (a.group_size > 0) {
                const int64_t o = (int64_t)row * a.ld_st + ((a.col0 + col) / a.group_size - gbase);
                w = fmaf(w, load_as_f32(a.scales, o, a.st_dtype), load_as_f32(a.offsets, o, a.st_dtype));
            }
#pragma unroll
            for (int mm = 0; mm < 4; ++mm)
                if (m0 + mm < a.M) acc[mm] = fmaf(w, load_as_f32(a.x, (int64_t)(m0 + mm) * a.ldx + col, a.x_dtype), acc[mm]);
        }
        if (a.rowptr != nullptr) {
            const int e1 = a.rowptr[row + 1];
            for (int e = a.rowptr[row] + lane; e < e1; e += 32) {
                const int c = a.cols[e];
                const float dl = a.deltas[e];
#pragma unroll
                for (int mm = 0; mm < 4; ++mm)
                    if (m0 + mm < a.M) acc[mm] = fmaf(dl, load_as_f32(a.x, (int64_t)(m0 + mm) * a.ldx + c, a.x_dtype), acc[mm]);
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

// ---- host side ---------------------------------------------------------------

static int g_sm_count[64] = {0};

static int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

bool gemv_fast_ok(const hxq_desc* d) {
    return (d->in_features % 16 == 0) && (d->ld_idx % 16 == 0) && aligned_to(d->indices, 16) &&
           (d->col0 % 16 == 0) && (d->group_size == 0 || d->group_size % 128 == 0);
}

static int mp_for(int M) { return M >= 3 ? 4 : (M == 2 ? 2 : 1); }

GemvPlan gemv_plan(const hxq_desc* d, int MP, int n_sm) {
    GemvPlan p;
    p.kbase = -(d->col0 % 128);
    p.nch = (d->in_features - p.kbase + kChunk - 1) / kChunk;
    p.nrb = (d->out_features + kRows - 1) / kRows;
    p.units = (int64_t)p.nch * p.nrb;
    const int wmax = (MP == 1) ? 16 : (MP == 2 ? 12 : 8);
    const int wmin = wmax / 2;
    // warps per CTA: the count whose equal split of the units wastes least
    int best_w = wmax;
    double best_eff = -1.0;
    for (int w = wmax; w >= wmin; --w) {
        const int64_t tw = (int64_t)n_sm * w;
        const int64_t per = (p.units + tw - 1) / tw;
        const double eff = (double)p.units / (double)(per * tw);
        if (eff > best_eff + 1e-9) { best_eff = eff; best_w = w; }
    }
    p.warps_per_cta = best_w;
    int64_t ctas = (p.units + best_w - 1) / best_w;
    p.grid = (int)(ctas < n_sm ? ctas : n_sm);
    p.counter_bytes = (((size_t)p.nrb * sizeof(unsigned int)) + 255) & ~(size_t)255;
    p.partial_bytes = (p.nch > 1) ? (size_t)p.units * kRows * MP * sizeof(float) : 0;
    return p;
}

template <int MP>
static int launch_fast(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gemv_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes) != cudaSuccess)
            return HXQ_E_DEVICE;
        attr_set[dev] = true;
    }
    gemv_kernel<MP><<<p.grid, p.warps_per_cta * 32, kGemvSmemBytes, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

// Shared by hxq_gemv and (until M is large enough for the tensor-core kernel)
// hxq_gemm: tokens are processed in groups of at most four per launch.
int gemv_any_m(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y, int y_dtype,
               int64_t ldy, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    GemvArgs a;
    a.idx = d->indices; a.cb = d->codebook; a.scales = d->scales; a.offsets = d->offsets;
    a.rowptr = d->rowptr; a.cols = d->cols; a.deltas = d->deltas; a.bias = d->bias;
    a.ld_idx = d->ld_idx; a.ldx = ldx; a.ldy = ldy;
    a.out_features = d->out_features; a.in_features = d->in_features; a.col0 = d->col0;
    a.group_size = d->group_size; a.ld_st = d->ld_st; a.st_dtype = d->st_dtype;
    a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    a.partial = nullptr; a.counters = nullptr;
    a.units = 0; a.kbase = 0; a.nch = 1; a.nrb = 0; a.total_warps = 1; a.x_vec = 0;
    const int xs = dtype_size(x_dtype), ys = dtype_size(y_dtype);

    if (!gemv_fast_ok(d)) {
        a.x = x; a.y = y; a.M = M;
        const int blocks = (d->out_features * 32 + 255) / 256;
        gemv_generic_kernel<<<blocks, 256, 0, stream>>>(a);
        return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
    }

    const int n_sm = sm_count();
    for (int m0 = 0; m0 < M;) {
        const int rem = M - m0;
        const int MP = mp_for(rem);
        const int mm = rem < MP ? rem : MP;
        const GemvPlan p = gemv_plan(d, MP, n_sm);
        if (p.nch > 1) {
            if (!workspace || workspace_bytes < p.counter_bytes + p.partial_bytes) return HXQ_E_WORKSPACE;
            if (!aligned_to(workspace, 16)) return HXQ_E_ALIGN;
            a.counters = reinterpret_cast<unsigned int*>(workspace);
            a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + p.counter_bytes);
        }
        a.x = reinterpret_cast<const char*>(x) + (int64_t)m0 * ldx * xs;
        a.y = reinterpret_cast<char*>(y) + (int64_t)m0 * ldy * ys;
        a.M = mm;
        a.kbase = p.kbase; a.nch = p.nch; a.nrb = p.nrb; a.units = p.units;
        a.total_warps = p.grid * p.warps_per_cta;
        a.x_vec = (aligned_to(a.x, 16) && ((ldx * xs) % 16 == 0)) ? 1 : 0;
        int st;
        if (MP == 1) st = launch_fast<1>(a, p, stream);
        else if (MP == 2) st = launch_fast<2>(a, p, stream);
        else st = launch_fast<4>(a, p, stream);
        if (st != HXQ_OK) return st;
        m0 += mm;
    }
    return HXQ_OK;
}

size_t gemv_workspace_bytes(const hxq_desc* d, int32_t M) {
    if (!gemv_fast_ok(d)) return 0;
    const GemvPlan p = gemv_plan(d, M >= 3 ? 4 : (M == 2 ? 2 : 1), sm_count());
    // a call with M >= 3 may end with a 1- or 2-token launch: those need less
    return p.nch > 1 ? p.counter_bytes + p.partial_bytes : 0;
}

}  // namespace hxq

extern "C" size_t hxq_gemv_workspace_bytes(const hxq_desc* d, int32_t M) {
    if (hxq::validate_desc(d) != HXQ_OK || M <= 0) return 0;
    return hxq::gemv_workspace_bytes(d, M);
}

extern "C" int hxq_gemv(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y,
                        int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes,
                        hxq_stream_t stream) {
    using namespace hxq;
    int st = validate_desc(d);
    if (st != HXQ_OK) return st;
    if (!x || !y) return HXQ_E_ARG;
    if (M <= 0 || M > 16) return HXQ_E_ARG;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return HXQ_E_DTYPE;
    if (ldx < d->in_features || ldy < d->out_features) return HXQ_E_SHAPE;
    if (d->rowptr && !d->deltas) return HXQ_E_ARG;
    return gemv_any_m(d, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}
