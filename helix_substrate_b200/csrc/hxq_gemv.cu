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
//  * Units are numbered row-block-major (unit = rowblock * nchunks + chunk) and
//    cut into equal contiguous ranges, one per CTA of a one-CTA-per-SM grid, so
//    every SM streams the same number of bytes whatever the shape.  Inside a CTA
//    warp w takes units w, w + W, w + 2W, ...: at any moment the W warps read W
//    neighbouring chunks of the same rows, i.e. one long contiguous piece of the
//    row-major index matrix (DRAM page locality), and when W is a multiple of
//    the chunk count a warp keeps its 16 activations per token in registers for
//    the whole launch.
//  * The 256-entry codebook is replicated per lane in shared memory at a 256-byte
//    stride on a 64 KB boundary: every lookup hits bank == lane, conflict free,
//    and the absolute address base | code << 8 | lane << 2 is ONE byte-permute of
//    the index word with a per-lane constant.  Per weight: PRMT, LDS, FFMA.
//  * The group affine is applied to per-(row, group) partial sums, not to weights:
//    sum_i x_i (c_i s + t) = s * sum_i x_i c_i + t * sum_i x_i.  Eight lanes span one
//    128-column group, so after three exchange steps of the warp butterfly each
//    lane holds the partial of one (row, group) and needs one s and one t.
//  * Chunks of one row block are summed inside the CTA through shared memory:
//    each unit drops its 8 x M partials into a slot, bumps a shared counter, and
//    the last warp to arrive adds the slots in chunk order.  Only a row block
//    that straddles two CTAs' ranges (at most two per CTA) goes through global
//    scratch and one global atomic; there too the last arriver sums the parts in
//    fixed order.  No float atomics anywhere: results are bit-identical from run
//    to run.
//  * The sidecar (row-sorted CSR of deltas) of a row block is added by the unit
//    whose chunk equals rowblock % nchunks, which spreads that work evenly.

#include <cuda.h>

#include "hxq_common.cuh"

namespace hxq {

constexpr int kRows = 8;          // rows per unit
constexpr int kChunk = 512;       // columns per unit (32 lanes x 16)
constexpr int kLutBytes = 256 * 256;
constexpr int kSlotBudgetBytes = 56 * 1024;    // in-CTA reduction slots, right after the table
constexpr int kGemvSmemBytes = 2 * kLutBytes + kSlotBudgetBytes;  // the table sits on a 64 KB boundary inside this window

#ifndef HXQ_GEMV_W1
#define HXQ_GEMV_W1 16      // max warps per CTA at one token per launch
#endif

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
    float* scratch;           // [nrb][max_parts][8*MP] partials of row blocks shared by several CTAs
    unsigned int* counters;   // [nrb] arrivals of those row blocks (zero between calls)
    int64_t ld_idx, ldx, ldy;
    int32_t out_features, in_features, col0, group_size, ld_st, st_dtype;
    int32_t x_dtype, y_dtype, x_vec;
    int32_t M;          // tokens in this launch (<= MP)
    int32_t kbase;      // local column of chunk 0, lane 0: -(col0 % 128)
    int32_t nch;        // column chunks per row block
    int32_t nrb;        // row blocks
    int32_t units;      // nrb * nch
    int32_t max_parts;  // CTAs that can share one row block
    int32_t rbl_max;    // row blocks a CTA can touch (slots in shared memory)
    int32_t slot_bytes; // lean kernel: bytes of reduction slots after the table (multiple of 128)
    int32_t tail_lanes; // lean kernel: lanes of the last chunk that hold columns (32 when it is whole)
};

struct GemvPlan {
    int nch, nrb, kbase, grid, warps_per_cta, units, max_parts, rbl_max;
    size_t counter_bytes, scratch_bytes;
};

template <int MP>
struct GemvCfg {
    static constexpr int kMaxWarps = (MP == 1) ? HXQ_GEMV_W1 : 12;   // (four tokens: 168 registers at 12 warps, 4 % faster than 8 warps at 255)
    static constexpr int kMaxThreads = 32 * kMaxWarps;
    // the edge-tolerant kernel holds more state per lane: at four tokens it spills above 8 warps
    static constexpr int kEdgeMaxWarps = (MP == 4) ? 8 : kMaxWarps;
    static constexpr int kEdgeMaxThreads = 32 * kEdgeMaxWarps;
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

// Two neighbouring lookups of one index word as a packed pair: the two loads write the
// halves of one 64-bit register directly (no moves before the packed FMA).
__device__ __forceinline__ uint64_t lut_pair(uint32_t word, uint32_t lane_key, int k0) {
    const uint32_t a0 = __byte_perm(word, lane_key, 0x7604u | (uint32_t)(k0 << 4));
    const uint32_t a1 = __byte_perm(word, lane_key, 0x7604u | (uint32_t)((k0 + 1) << 4));
    uint64_t r;
    asm volatile("{\n\t.reg .f32 lo, hi;\n\tld.shared.f32 lo, [%1];\n\tld.shared.f32 hi, [%2];\n\t"
                 "mov.b64 %0, {lo, hi};\n\t}" : "=l"(r) : "r"(a0), "r"(a1));
    return r;
}

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

// First unit of CTA c when `units` are cut into `grid` equal contiguous ranges.
__host__ __device__ __forceinline__ int cta_first_unit(int units, int grid, int c) {
    return (int)((int64_t)units * c / grid);
}
// CTA that owns unit u under that cut.
__device__ __forceinline__ int cta_of_unit(int units, int grid, int u) {
    return (int)((((int64_t)u + 1) * grid + units - 1) / units) - 1;
}

// two fp32 lanes in one 64-bit register (operands of the packed fp32 FMA of sm_100)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void ffma2(uint64_t& acc, uint64_t w, uint64_t x) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(w), "l"(x));
}
__device__ __forceinline__ float sum2(uint64_t v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo + hi;
}

template <int MP>
__global__ void __launch_bounds__(GemvCfg<MP>::kEdgeMaxThreads, 1) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(1024) char dyn_smem[];
    constexpr int RM = kRows * MP;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int W = blockDim.x >> 5;
    // codebook table at the next 64 KB boundary of the shared window, reduction slots right after it
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(dyn_smem));
    const uint32_t lut_base = (smem_base + 0xFFFFu) & ~0xFFFFu;
    char* lut = dyn_smem + (lut_base - smem_base);
    const uint32_t lane_key = lut_base | ((uint32_t)lane << 2);
    unsigned int* cnt_s = reinterpret_cast<unsigned int*>(lut + kLutBytes);               // [rbl_max]
    float* part_s = reinterpret_cast<float*>(lut + kLutBytes + ((a.rbl_max * 4 + 15) & ~15));  // [rbl_max][nch][RM]

    const int nch = a.nch;
    const int U0 = cta_first_unit(a.units, gridDim.x, blockIdx.x);
    const int U1 = cta_first_unit(a.units, gridDim.x, blockIdx.x + 1);
    const int rb_first = U0 / nch;
    const bool cta_whole = (U0 - rb_first * nch == 0) && (U1 % nch == 0);   // no row block is shared with a neighbour
    const int r_l = lane & 7;    // row this lane ends up holding after the butterfly
    const int h_l = lane >> 3;   // 128-column span of the chunk this lane belongs to
    const bool affine = a.group_size > 0;
    const bool g128 = a.group_size == 128;
    const int g_base = affine ? a.col0 / a.group_size : 0;
    const int span0 = a.kbase + h_l * 128;                       // local column of this lane's span in chunk 0
    const int gq0 = (a.col0 + span0) / 128 - g_base;             // its group index when groups are 128 wide
    const int lane_col = a.kbase + lane * 16;
    const uint32_t ld = (uint32_t)a.ld_idx;
    // per-step advance of (row block, chunk) when the unit index grows by W
    const int d_rb = W / nch, d_ch = W - d_rb * nch;

    auto fetch = [&](int rb, int ch, int own, UnitPrefetch& f) {
        const int row0 = rb * kRows;
        const int c0 = a.kbase + ch * kChunk;                    // local column of the chunk
        const uint8_t* p = a.idx + (uint64_t)row0 * ld + (c0 + lane * 16);
        const bool interior = (row0 + kRows <= a.out_features) && (c0 >= 0) && (c0 + kChunk <= a.in_features);
        if (interior) {   // warp-uniform: no clamps, no predicates
#pragma unroll
            for (int r = 0; r < kRows; ++r) f.q[r] = ld_stream_u4(p + (uint64_t)(r * ld));
        } else {
            const int col = c0 + lane * 16;
            const bool ok = (col >= 0) && (col < a.in_features);
            const int rmax = a.out_features - 1 - row0;
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int rr = r < rmax ? r : rmax;   // rows past the end re-read the last row (never stored)
                f.q[r] = ok ? ld_stream_u4(p + (uint64_t)(rr * ld)) : make_uint4(0, 0, 0, 0);
            }
        }
        const int row_l = row0 + r_l;
        const bool row_ok = row_l < a.out_features;
        f.s = 1.f; f.t = 0.f;
        if (affine) {
            const int span_col = span0 + ch * kChunk;
            if (span_col < a.in_features && row_ok) {
                const int g = g128 ? gq0 + ch * 4 : (a.col0 + span_col) / a.group_size - g_base;
                const int64_t o = (int64_t)row_l * a.ld_st + g;
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
        if (a.rowptr != nullptr && ch == own && row_ok) {   // this unit carries the row block's sidecar
            f.e0 = a.rowptr[row_l];
            f.e1 = a.rowptr[row_l + 1];
        }
    };

    // this warp's units: U0 + warp, + W, + 2W, ...   (unit = rb * nch + ch, own = rb % nch)
    int ua = U0 + warp;
    int rb_a = ua / nch, ch_a = ua - rb_a * nch, own_a = rb_a % nch;
    auto step = [&](int& rb, int& ch, int& own) {
        ch += d_ch; rb += d_rb; own += d_rb;
        if (ch >= nch) { ch -= nch; ++rb; ++own; }
        while (own >= nch) own -= nch;
    };

    // The first unit's index rows and activations go out before the table is
    // built: the first HBM round trip overlaps the set-up.
    UnitPrefetch fa, fb;
    uint64_t xp[MP][8];      // activations of the current chunk, packed in pairs
    float xsum[MP];
    int cur_ch = -1;
    auto load_x = [&](int ch) {
        const int col = lane_col + ch * kChunk;
        const bool col_ok = (col >= 0) && (col < a.in_features);
        float xr[MP][16];
        load_x_chunk<MP>(a, col, col_ok, xr);
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            float sx = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xp[m][j] = pack2(xr[m][2 * j], xr[m][2 * j + 1]);
                sx += xr[m][2 * j] + xr[m][2 * j + 1];
            }
            if (affine) {   // sum of x over this lane's 128-column span
                sx += __shfl_xor_sync(0xffffffffu, sx, 4);
                sx += __shfl_xor_sync(0xffffffffu, sx, 2);
                sx += __shfl_xor_sync(0xffffffffu, sx, 1);
            }
            xsum[m] = sx;
        }
        cur_ch = ch;
    };
    // Programmatic dependent launch: the next kernel in the stream may start its own
    // set-up as soon as every CTA of this one has got here ...
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (ua < U1) fetch(rb_a, ch_a, own_a, fa);   // weights only: nothing an earlier kernel could still be writing
    {   // lane-replicated table: warp w fills entries [w*per, (w+1)*per): coalesced loads, then broadcasts
        const int per = (256 + W - 1) / W;
        const int c_end = (warp + 1) * per < 256 ? (warp + 1) * per : 256;
        for (int c0 = warp * per; c0 < c_end; c0 += 32) {
            const float mine = (c0 + lane < c_end) ? a.cb[c0 + lane] : 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) {     // fixed trip count: the 32 broadcasts pipeline instead of one shuffle -> store at a time
                const float v = __shfl_sync(0xffffffffu, mine, k);
                if (c0 + k < c_end) *reinterpret_cast<float*>(lut + (c0 + k) * 256 + lane * 4) = v;
            }
        }
    }
    for (int i = threadIdx.x; i < a.rbl_max; i += blockDim.x) cnt_s[i] = 0u;
    // ... and this one reads activations / touches y and the workspace only after everything
    // before it in the stream has finished (the table and the first index rows above did
    // not have to wait).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (ua < U1) {
        load_x(ch_a);
    } else {
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            xsum[m] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) xp[m][j] = 0ull;
        }
    }
    __syncthreads();

    auto process = [&](int prb, int pch, const UnitPrefetch& f) {
        if (pch != cur_ch) load_x(pch);   // warp-uniform; never taken again when W is a multiple of nch
        const int c0 = a.kbase + pch * kChunk;
        const bool interior = (prb * kRows + kRows <= a.out_features) && (c0 >= 0) && (c0 + kChunk <= a.in_features);
        const int col = c0 + lane * 16;
        const bool col_ok = interior || ((col >= 0) && (col < a.in_features));

        // ---- lookups + packed FMAs: acc[r*MP + m] = this lane's 16-column partial ----
        // Four rows at a time, column pairs outermost, lookups of the next pair issued before the
        // FMAs of the current one: every FMA finds its table value already landed.
        float acc[kRows * MP];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint64_t p2[4][MP];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int m = 0; m < MP; ++m) p2[r][m] = 0ull;
            uint64_t wa[4], wb[4];
            auto look = [&](int j, uint64_t (&wv)[4]) {
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const uint4 q = f.q[4 * half + r];
                    const uint32_t word = (j >> 1) == 0 ? q.x : ((j >> 1) == 1 ? q.y : ((j >> 1) == 2 ? q.z : q.w));
                    wv[r] = lut_pair(word, lane_key, (2 * j) & 3);
                }
            };
            look(0, wa);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                look(j + 1, wb);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int m = 0; m < MP; ++m) ffma2(p2[r][m], wa[r], xp[m][j]);
                if (j + 2 < 8) look(j + 2, wa);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int m = 0; m < MP; ++m) ffma2(p2[r][m], wb[r], xp[m][j + 1]);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int m = 0; m < MP; ++m) acc[(4 * half + r) * MP + m] = col_ok ? sum2(p2[r][m]) : 0.f;
        }

        // ---- butterfly over the 8 lanes of a group span: rows are dealt out ----
        halve<kRows * MP>(acc, lane, 4);
        halve<kRows * MP / 2>(acc, lane, 2);
        halve<kRows * MP / 4>(acc, lane, 1);
        // now acc[0..MP) = partial of row (lane & 7) over span (lane >> 3), per token
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
        int m_i = 0;
        if (MP == 4) {
            halve<4>(acc, lane, 8);
            halve<2>(acc, lane, 16);
            m_i = ((lane >> 3) & 1) * 2 + ((lane >> 4) & 1);
        } else if (MP == 2) {
            halve<2>(acc, lane, 8);
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 16);
            m_i = (lane >> 3) & 1;
        } else {
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 8);
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 16);
        }
        float v = acc[0];
        int row_i = r_l;                                            // (row, token) this lane holds
        bool has = (MP == 4) ? true : (MP == 2 ? (lane < 16) : (lane < 8));

        // ---- sum the chunks of the row block: inside the CTA through shared memory ----
        int lo = 0, hi = nch;                                       // this CTA's chunks of the row block: [lo, hi)
        if (!cta_whole) {
            const int rb_u0 = prb * nch;
            lo = (U0 > rb_u0 ? U0 : rb_u0) - rb_u0;
            hi = (U1 < rb_u0 + nch ? U1 : rb_u0 + nch) - rb_u0;
        }
        bool fin = true;                                            // warp-uniform: we finish the CTA's share
        if (hi - lo > 1) {
            const int rbl = prb - rb_first;
            float* slot = part_s + rbl * (nch * RM);
            if (has) slot[pch * RM + row_i * MP + m_i] = v;
            __threadfence_block();
            __syncwarp();
            unsigned int old = 0;
            if (lane == 0) old = atomicAdd(&cnt_s[rbl], 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            fin = (old == (unsigned int)(hi - lo - 1));
            if (fin) {      // last chunk to arrive: add the slots in chunk order, lane j owns value j
                __threadfence_block();
                has = lane < RM;
                row_i = lane / MP;
                m_i = lane % MP;
                v = 0.f;
                if (has)
                    for (int c = lo; c < hi; ++c) v += slot[c * RM + lane];
            }
        }
        if (!fin) return;

        // ---- a row block cut by the CTA boundary: parts meet in global scratch ----
        if (hi - lo < nch) {
            const int rb_u0 = prb * nch;
            const int c_first = cta_of_unit(a.units, gridDim.x, rb_u0);
            const int n_parts = cta_of_unit(a.units, gridDim.x, rb_u0 + nch - 1) - c_first + 1;
            float* sp = a.scratch + (int64_t)prb * a.max_parts * RM;
            if (has) __stcg(sp + ((int)blockIdx.x - c_first) * RM + row_i * MP + m_i, v);
            __threadfence();
            __syncwarp();
            unsigned int g = 0;
            if (lane == 0) g = atomicAdd(a.counters + prb, 1u);
            g = __shfl_sync(0xffffffffu, g, 0);
            if (g != (unsigned int)(n_parts - 1)) return;
            __threadfence();
            v = 0.f;
            if (has)
                for (int p = 0; p < n_parts; ++p) {
                    v += __ldcg(sp + p * RM + row_i * MP + m_i);
                    __stcg(sp + p * RM + row_i * MP + m_i, 0.f);   // the whole workspace goes back to zero:
                }                                                  // another shape lays it out differently
            if (lane == 0) a.counters[prb] = 0u;
        }
        const int row = prb * kRows + row_i;
        if (has && row < a.out_features && m_i < a.M) {
            if (a.bias != nullptr) v += a.bias[row];
            store_from_f32(a.y, (int64_t)m_i * a.ldy + row, v, a.y_dtype);
        }
    };

    while (ua < U1) {
        int rb_b = rb_a, ch_b = ch_a, own_b = own_a;
        step(rb_b, ch_b, own_b);
        const int ub = ua + W;
        if (ub < U1) fetch(rb_b, ch_b, own_b, fb);
        process(rb_a, ch_a, fa);
        if (ub >= U1) break;
        rb_a = rb_b; ch_a = ch_b; own_a = own_b;
        step(rb_a, ch_a, own_a);
        ua = ub + W;
        if (ua < U1) fetch(rb_a, ch_a, own_a, fa);
        process(rb_b, ch_b, fb);
    }
}

// ---- lean kernel: shapes where every unit is whole ---------------------------------------
//
// OUT % 8 == 0, IN % 128 == 0, no column offset inside a group, group size 0 or 128, 16-byte
// aligned activations: no unit touches a row edge, so the per-unit code carries no bounds logic
// at all.  Template parameters: MP tokens per launch, XDT activation type, STM scale/offset
// (0 none, 1 fp32, 2 fp16), SIDE "the matrix has a sidecar", TAIL "the last chunk of a row is
// shorter than 512 columns" (whole 128-column groups; its lanes past the end fetch lane 0's
// addresses and hold zero activations) - as run-time switches they cost 2-6 % per launch.
// Same unit, table and butterfly as gemv_kernel; what differs is the bookkeeping:
//  * index bytes travel global -> shared with 16-byte asynchronous copies (each lane copies, and
//    later reads back, its own 16 bytes of each of the 8 rows: a per-warp double buffer of two
//    4 KB units that needs no synchronisation beyond the copy-group wait).  Register loads for
//    the same bytes measured 5 us slower per launch: outstanding register loads and the table
//    lookups then wait on one another, while asynchronous copies leave the lookups alone.
//    Half as many registers hold index bytes, which is what lets 16 warps run unspilled,
//  * the activations of the next unit's chunk ride along in the same copy group whenever the
//    chunk changes, and a row block's sidecar is dealt out one entry per lane over up to eight
//    of its units, each fetching its entry's column and delta before the lookups start and the
//    activation it meets half-way through: no load is waited for right after it is issued,
//  * the walk over a warp's units is incremental (one 64-bit pointer, one scale offset, one
//    slot offset, each advanced by a warp-uniform delta),
//  * a unit ends with ONE store of its 8 x M partial sums into its own shared-memory slot;
//    there are no arrival counters inside the CTA.  After the last unit the CTA meets at one
//    barrier and the warps add the slots of each row block in a fixed order (deterministic; the
//    lane groups of a warp each take every n-th chunk and meet by shuffles), then store y - or,
//    for a row block cut by the CTA boundary, go through global scratch + an arrival counter
//    (one release/acquire atomic per warp; the last arriver adds the parts in CTA order).
constexpr int kLeanSmemBytes = 232448;          // all of the SM's shared memory: table + slots + index rings
constexpr int kLeanCarriers = 8;                // units of a row block that share its sidecar

#ifndef HXQ_GEMV_TMA
#define HXQ_GEMV_TMA 0     // 0: 16-byte asynchronous copies per lane; 1: one bulk tensor copy per unit, issued by one lane
#endif                     // (same results; measured 1.4-2 us slower per launch than the per-lane copies)
constexpr int kLeanBarBytes = 256;              // two mbarriers per warp, up to 16 warps
__device__ int g_gemv_status = 0;               // set to HXQ_E_TIMEOUT if a bounded wait on a copy gave up

struct LeanFetch {
    float s, t;       // group scale / offset of (row lane&7, 128-column span lane>>3)
    int e, e1;        // this lane's sidecar entry of row lane&7 (none if e >= e1) and the row's end
    bool last;        // this unit also walks the entries beyond kLeanCarriers * 4 per row
};

__device__ __forceinline__ uint64_t fmul2(uint64_t w, uint64_t x) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(w), "l"(x));
    return r;
}

// 16 activations of this lane (columns col .. col+15 of the token row at xrow) as 8 packed fp32 pairs
template <int XDT>
__device__ __forceinline__ void x_lane16(const void* xrow, int col, uint64_t (&xp)[8]) {
    if (XDT == HXQ_F32) {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(xrow) + col);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 v = p[j];
            xp[2 * j] = pack2(v.x, v.y);
            xp[2 * j + 1] = pack2(v.z, v.w);
        }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(xrow) + col);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint4 v = p[j];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float lo, hi;
                if (XDT == HXQ_BF16) {
                    lo = __uint_as_float(w[q] << 16);
                    hi = __uint_as_float(w[q] & 0xffff0000u);
                } else {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[q]);
                    lo = __low2float(h); hi = __high2float(h);
                }
                xp[4 * j + q] = pack2(lo, hi);
            }
        }
    }
}

template <int MP, int XDT, int STM, bool SIDE, bool TAIL>
__global__ void __launch_bounds__(GemvCfg<MP>::kMaxThreads, 1)
gemv_lean_kernel(const __grid_constant__ CUtensorMap tmap, const GemvArgs a) {
    extern __shared__ __align__(1024) char dyn_smem[];
    constexpr int RM = kRows * MP;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int W = blockDim.x >> 5;
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(dyn_smem));
    const uint32_t lut_base = (smem_base + 0xFFFFu) & ~0xFFFFu;
    char* lut = dyn_smem + (lut_base - smem_base);
    const uint32_t lane_key = lut_base | ((uint32_t)lane << 2);
    float* part_s = reinterpret_cast<float*>(lut + kLutBytes);   // [unit - S0][RM]
    // staging: 2 W unit buffers of 4 KB (warp w owns 2w and 2w+1), as many as fit below the table and
    // the rest above the slots, then one activation chunk per warp
    constexpr int xs_lane = (XDT == HXQ_F32) ? 64 : 32;          // bytes of one token's 16 activations
    uint32_t ring_q0, ring_q1, ring_x;
    {
        constexpr uint32_t kUnitBytes = kRows * kChunk;
        const uint32_t lo0 = (smem_base + 127u) & ~127u;
        const uint32_t hi0 = lut_base + kLutBytes + (uint32_t)a.slot_bytes;
        const uint32_t n_lo = (lut_base - lo0) / kUnitBytes;
        const uint32_t i0 = 2 * warp, i1 = 2 * warp + 1, n_q = 2 * W;
        ring_q0 = (i0 < n_lo ? lo0 + i0 * kUnitBytes : hi0 + (i0 - n_lo) * kUnitBytes) + lane * 16;
        ring_q1 = (i1 < n_lo ? lo0 + i1 * kUnitBytes : hi0 + (i1 - n_lo) * kUnitBytes) + lane * 16;
        const uint32_t n_hi = n_q > n_lo ? n_q - n_lo : 0u;
        // token m at + m * 32 * xs_lane; a lane's 32 or 64 bytes are contiguous (spreading its 16-byte pieces
        // 512 bytes apart removes the 2-way bank conflict of the read-back and measured 2.8 us SLOWER on down_proj)
        ring_x = hi0 + n_hi * kUnitBytes + warp * (MP * 32 * xs_lane) + lane * xs_lane;
    }
    constexpr int kXPiece = 16;   // distance between a lane's consecutive 16-byte pieces
#if HXQ_GEMV_TMA
    // one mbarrier per unit buffer, at the end of the slot area; only this warp ever touches its two
    const uint32_t bar0 = lut_base + kLutBytes + (uint32_t)a.slot_bytes - kLeanBarBytes + warp * 16;
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar0));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar0 + 8));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t phase = 0;
    bool alive = true;      // false once a wait on a copy has given up: the warp stops issuing and computing
#endif
    const int nch = a.nch;
    const int U0 = cta_first_unit(a.units, gridDim.x, blockIdx.x);
    const int U1 = cta_first_unit(a.units, gridDim.x, blockIdx.x + 1);
    const int rb_first = U0 / nch;
    const int S0 = rb_first * nch;           // first unit of the first row block this CTA touches
    const int r_l = lane & 7;
    const int h_l = lane >> 3;
    constexpr bool affine = STM != 0;
    constexpr bool st_f32 = STM == 1;
    const int M = a.M;
    const int64_t ldx = a.ldx;
    const char* const xbase = reinterpret_cast<const char*>(a.x);
    const uint32_t ld = (uint32_t)a.ld_idx;
    const int d_rb = W / nch, d_ch = W - d_rb * nch;
    // a last chunk with fewer than 512 columns (whole 128-column groups): lanes past its end fetch from lane 0's
    // addresses and hold zero activations, so they add nothing
    const bool tail_lane = TAIL && lane >= a.tail_lanes;
    // sidecar carriers of row block rb: the units with (chunk - rb) mod nch < n_car
    const int n_car = nch < kLeanCarriers ? nch : kLeanCarriers;
    const int own_step = d_rb % nch;

    // walking state: the unit about to be fetched
    int u = U0 + warp;
    int rb = u / nch, ch = u - rb * nch;
    int own = rb % nch;
    const uint8_t* p = a.idx + (uint64_t)rb * (8ull * ld) + (uint32_t)(ch * kChunk + lane * 16);
    int so = (rb * kRows + r_l) * a.ld_st + ch * 4 + h_l;
    const uint64_t dp_main = (uint64_t)d_rb * (8ull * ld) + (uint64_t)(d_ch * kChunk);
    const uint64_t dp_wrap = 8ull * ld - (uint64_t)(nch * kChunk);
    const int ds_main = d_rb * kRows * a.ld_st + d_ch * 4;
    const int ds_wrap = kRows * a.ld_st - nch * 4;
    const int n_my = (u < U1) ? (U1 - u + W - 1) / W : 0;

    auto fetch = [&](LeanFetch& f, int buf, bool with_x) {
#if HXQ_GEMV_TMA
        // the buffer was last read with ordinary loads: order them before the bulk copy's writes
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && alive) {
            const uint32_t bar = bar0 + buf * 8;
            const uint32_t xbytes = with_x ? (uint32_t)(M * 32 * xs_lane) : 0u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"((uint32_t)(kRows * kChunk) + xbytes) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                         :: "r"(buf ? ring_q1 : ring_q0), "l"(reinterpret_cast<uint64_t>(&tmap)), "r"(bar), "r"(ch * (kChunk / 4)), "r"(rb * kRows) : "memory");
            if (with_x) {
                const char* xg = xbase + (size_t)(ch * kChunk) * (xs_lane >> 4);
                for (int m = 0; m < M; ++m)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 :: "r"(ring_x + m * 32 * xs_lane), "l"(xg + (size_t)m * ldx * (xs_lane >> 4)), "r"(32 * xs_lane), "r"(bar) : "memory");
            }
        }
#else
        const bool cut = tail_lane && ch == nch - 1;
        const uint8_t* pq = cut ? p - lane * 16 : p;
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                         :: "r"((buf ? ring_q1 : ring_q0) + r * kChunk), "l"(pq + (uint64_t)ld * (uint32_t)r) : "memory");
        if (with_x) {   // warp-uniform: the unit's chunk differs from the one whose activations are in registers
            const char* xg = xbase + (size_t)(ch * kChunk + (cut ? 0 : lane * 16)) * (xs_lane >> 4);
#pragma unroll
            for (int m = 0; m < MP; ++m) {
                if (m < M) {
                    const char* xm = xg + (size_t)m * ldx * (xs_lane >> 4);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(ring_x + m * 32 * xs_lane), "l"(xm) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(ring_x + m * 32 * xs_lane + kXPiece), "l"(xm + 16) : "memory");
                    if (xs_lane == 64) {
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(ring_x + m * 32 * xs_lane + 2 * kXPiece), "l"(xm + 32) : "memory");
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(ring_x + m * 32 * xs_lane + 3 * kXPiece), "l"(xm + 48) : "memory");
                    }
                }
            }
        }
#endif
        f.s = 1.f; f.t = 0.f;
        if (affine) {
#if HXQ_GEMV_TMA
            const bool cut = tail_lane && ch == nch - 1;
#endif
            const int sq = cut ? so - h_l : so;
            if (st_f32) {
                f.s = reinterpret_cast<const float*>(a.scales)[sq];
                f.t = reinterpret_cast<const float*>(a.offsets)[sq];
            } else {
                f.s = __half2float(reinterpret_cast<const __half*>(a.scales)[sq]);
                f.t = __half2float(reinterpret_cast<const __half*>(a.offsets)[sq]);
            }
        }
        f.e = 0; f.e1 = 0; f.last = false;
        if (SIDE) {
            int i = ch - own;
            if (i < 0) i += nch;
            if (i < n_car) {   // entry 4 i + (lane >> 3) of row lane & 7
                f.e = a.rowptr[rb * kRows + r_l] + i * 4 + h_l;
                f.e1 = a.rowptr[rb * kRows + r_l + 1];
                f.last = (i == n_car - 1);
            }
        }
    };
    auto advance = [&]() {
        u += W; ch += d_ch; rb += d_rb; p += dp_main; so += ds_main; own += own_step;
        if (ch >= nch) { ch -= nch; ++rb; p += dp_wrap; so += ds_wrap; ++own; }
        if (own >= nch) own -= nch;
    };

    uint64_t xp[MP][8];
    float xsum[MP];
    int cur_ch = -1;
    auto set_x = [&](float (&xr)[MP][16], int c) {
        const bool cut = tail_lane && c == nch - 1;
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            if (cut) {
#pragma unroll
                for (int j = 0; j < 16; ++j) xr[m][j] = 0.f;
            }
            float sx = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xp[m][j] = pack2(xr[m][2 * j], xr[m][2 * j + 1]);
                sx += xr[m][2 * j] + xr[m][2 * j + 1];
            }
            if (affine) {
                sx += __shfl_xor_sync(0xffffffffu, sx, 4);
                sx += __shfl_xor_sync(0xffffffffu, sx, 2);
                sx += __shfl_xor_sync(0xffffffffu, sx, 1);
            }
            xsum[m] = sx;
        }
        cur_ch = c;
    };
    auto load_x = [&](int c) {          // straight from global: the first unit only
        float xr[MP][16];
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            uint64_t t8[8];
            if (m < M) x_lane16<XDT>(xbase + (size_t)m * ldx * (XDT == HXQ_F32 ? 4 : 2),
                                     c * kChunk + ((tail_lane && c == nch - 1) ? 0 : lane * 16), t8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float lo = 0.f, hi = 0.f;
                if (m < M) asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(t8[j]));
                xr[m][2 * j] = lo; xr[m][2 * j + 1] = hi;
            }
        }
        set_x(xr, c);
    };
    auto read_x = [&](int c) {          // from the copy a fetch left in shared memory
        float xr[MP][16];
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            if (m >= M) {
#pragma unroll
                for (int j = 0; j < 16; ++j) xr[m][j] = 0.f;
                continue;
            }
            uint32_t w[16];
            const int nq = xs_lane >> 4;
            for (int k = 0; k < 4; ++k) {
                if (k < nq)
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w[4 * k]), "=r"(w[4 * k + 1]), "=r"(w[4 * k + 2]), "=r"(w[4 * k + 3])
                                 : "r"(ring_x + m * 32 * xs_lane + kXPiece * k));
            }
            if (XDT == HXQ_F32) {
#pragma unroll
                for (int j = 0; j < 16; ++j) xr[m][j] = __uint_as_float(w[j]);
            } else if (XDT == HXQ_BF16) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { xr[m][2 * j] = __uint_as_float(w[j] << 16); xr[m][2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                    xr[m][2 * j] = __low2float(h); xr[m][2 * j + 1] = __high2float(h);
                }
            }
        }
        set_x(xr, c);
    };

    LeanFetch fa, fb;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int u_a = u, ch_a = ch;
    if (n_my > 0) fetch(fa, 0, false);   // no activations yet: an earlier kernel may still be writing them
#if !HXQ_GEMV_TMA
    asm volatile("cp.async.commit_group;" ::: "memory");
#endif
    {
        const int per = (256 + W - 1) / W;
        const int c_end = (warp + 1) * per < 256 ? (warp + 1) * per : 256;
        for (int c0 = warp * per; c0 < c_end; c0 += 32) {
            const float mine = (c0 + lane < c_end) ? a.cb[c0 + lane] : 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) {     // fixed trip count: the 32 broadcasts pipeline instead of one shuffle -> store at a time
                const float v = __shfl_sync(0xffffffffu, mine, k);
                if (c0 + k < c_end) *reinterpret_cast<float*>(lut + (c0 + k) * 256 + lane * 4) = v;
            }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (n_my > 0) {
        load_x(ch_a);
    } else {
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            xsum[m] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) xp[m][j] = 0ull;
        }
    }
    __syncthreads();

    auto compute = [&](const LeanFetch& f, int buf, int pu) {
        // this lane's sidecar entry: column and delta go out now, the activation it meets after the
        // first half of the lookups, the product at the end
        bool sc = false;
        int sc_c = 0;
        float sc_d = 0.f, sc_x[MP];
        if (SIDE) { sc = f.e < f.e1; if (sc) { sc_c = a.cols[f.e]; sc_d = a.deltas[f.e]; } }
#pragma unroll
        for (int m = 0; m < MP; ++m) sc_x[m] = 0.f;
        float acc[kRows * MP];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint4 qh[4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(qh[r].x), "=r"(qh[r].y), "=r"(qh[r].z), "=r"(qh[r].w)
                             : "r"((buf ? ring_q1 : ring_q0) + (4 * half + r) * kChunk));
            uint64_t p2[4][MP];
            uint64_t wa[4], wb[4];
            auto look = [&](int j, uint64_t (&wv)[4]) {
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const uint4 q = qh[r];
                    const uint32_t word = (j >> 1) == 0 ? q.x : ((j >> 1) == 1 ? q.y : ((j >> 1) == 2 ? q.z : q.w));
                    wv[r] = lut_pair(word, lane_key, (2 * j) & 3);
                }
            };
            look(0, wa);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                look(j + 1, wb);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int m = 0; m < MP; ++m) {
                        if (j == 0) p2[r][m] = fmul2(wa[r], xp[m][0]);
                        else ffma2(p2[r][m], wa[r], xp[m][j]);
                    }
                if (j + 2 < 8) look(j + 2, wa);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int m = 0; m < MP; ++m) ffma2(p2[r][m], wb[r], xp[m][j + 1]);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int m = 0; m < MP; ++m) acc[(4 * half + r) * MP + m] = sum2(p2[r][m]);
            if (SIDE && half == 0) {
#pragma unroll
                for (int m = 0; m < MP; ++m)
                    sc_x[m] = (sc && m < M) ? Elem<XDT>::load(xbase, (int64_t)m * ldx + sc_c) : 0.f;
            }
        }
        halve<kRows * MP>(acc, lane, 4);
        halve<kRows * MP / 2>(acc, lane, 2);
        halve<kRows * MP / 4>(acc, lane, 1);
        if (affine) {
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[m] = fmaf(f.s, acc[m], f.t * xsum[m]);
        }
        if (SIDE) {
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[m] = fmaf(sc_d, sc_x[m], acc[m]);
        }
        if (SIDE && f.last) {   // rows with more entries than the carriers take in one go
            for (int e = f.e + 4; e < f.e1; e += 4) {
                const int c = a.cols[e];
                const float dl = a.deltas[e];
#pragma unroll
                for (int m = 0; m < MP; ++m)
                    if (m < M) acc[m] = fmaf(dl, Elem<XDT>::load(xbase, (int64_t)m * ldx + c), acc[m]);
            }
        }
        int m_i = 0;
        if (MP == 4) {
            halve<4>(acc, lane, 8);
            halve<2>(acc, lane, 16);
            m_i = ((lane >> 3) & 1) * 2 + ((lane >> 4) & 1);
        } else if (MP == 2) {
            halve<2>(acc, lane, 8);
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 16);
            m_i = (lane >> 3) & 1;
        } else {
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 8);
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 16);
        }
        const bool has = (MP == 4) ? true : (MP == 2 ? (lane < 16) : (lane < 8));
        if (has) part_s[(pu - S0) * RM + r_l * MP + m_i] = acc[0];
    };

#if HXQ_GEMV_TMA
    // Bounded wait for the copies of one buffer; a warp that gives up raises the status word, lets
    // what it has in flight land (second, shorter wait) and does no more work.
    auto landed = [&](int buf) {
        if (!alive) return;
        const uint32_t bar = bar0 + buf * 8;
        uint32_t ok = 0;
        const long long t0 = clock64();
        for (;;) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar), "r"(phase) : "memory");
            if (ok) return;
            if (clock64() - t0 > 2000000000LL) break;
        }
        alive = false;
        if (lane == 0) atomicExch(&g_gemv_status, HXQ_E_TIMEOUT);
    };
#define HXQ_LEAN_COMMIT()
#define HXQ_LEAN_LANDED(buf) landed(buf)
#else
#define HXQ_LEAN_COMMIT() asm volatile("cp.async.commit_group;" ::: "memory")   /* one group per unit, empty past the end */
#define HXQ_LEAN_LANDED(buf) asm volatile("cp.async.wait_group 0;" ::: "memory")
    const bool alive = true;
#endif
    for (int k = 0; k < n_my; k += 2) {
        // unit k: index bytes in buffer 0; one unit's copies in flight at most, and they have to be in
        HXQ_LEAN_LANDED(0);
        if (alive && ch_a != cur_ch) read_x(ch_a);
        advance();
        const int u_b = u, ch_b = ch;
        if (k + 1 < n_my) fetch(fb, 1, ch_b != ch_a);
        HXQ_LEAN_COMMIT();
        if (alive) compute(fa, 0, u_a);
        if (k + 1 >= n_my) break;
        HXQ_LEAN_LANDED(1);
        if (alive && ch_b != cur_ch) read_x(ch_b);
        advance();
        u_a = u; ch_a = ch;
        if (k + 2 < n_my) fetch(fa, 0, ch_a != ch_b);
        HXQ_LEAN_COMMIT();
        if (alive) compute(fb, 1, u_b);
#if HXQ_GEMV_TMA
        phase ^= 1u;
#endif
    }
#if HXQ_GEMV_TMA
    if (!alive) {   // let the copy that never reported finish before the CTA's memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 200000000LL) { }
    }
#else
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#endif
#undef HXQ_LEAN_COMMIT
#undef HXQ_LEAN_LANDED
    __syncthreads();

    // ---- add the chunks of each row block; lane j < RM owns value j = row * MP + token.  The 32 / RM
    // lane groups each add every (32 / RM)-th chunk, then the groups' sums meet by shuffles: a fixed
    // order (results stay bit-identical from run to run) at a quarter of the dependent additions for
    // one token (37 chunks per row block in down_proj).
    const int rb_last = (U1 - 1) / nch;
    const bool has = lane < RM;
    constexpr int NG = 32 / RM;                 // lane groups
    const int lg = lane / RM, lj = lane % RM;
    const int row_i = lj / MP, m_i = lj % MP;
    for (int rbx = rb_first + warp; rbx <= rb_last; rbx += W) {
        const int rb_u0 = rbx * nch;
        const int lo = (U0 > rb_u0 ? U0 : rb_u0) - rb_u0;
        const int hi = (U1 < rb_u0 + nch ? U1 : rb_u0 + nch) - rb_u0;
        float v = 0.f;
        for (int c = lo + lg; c < hi; c += NG) v += part_s[(rb_u0 + c - S0) * RM + lj];
#pragma unroll
        for (int off = RM; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (hi - lo < nch) {   // cut by the CTA boundary: parts meet in global scratch
            const int c_first = cta_of_unit(a.units, gridDim.x, rb_u0);
            const int n_parts = cta_of_unit(a.units, gridDim.x, rb_u0 + nch - 1) - c_first + 1;
            float* sp = a.scratch + (int64_t)rbx * a.max_parts * RM;
            if (has) __stcg(sp + ((int)blockIdx.x - c_first) * RM + lane, v);
            // One release/acquire arrival per warp instead of fence + atomic + fence: the warp barrier orders
            // the lanes' stores before lane 0's release, and lane 0's acquire before the lanes' loads below.
            __syncwarp();
            unsigned int g = 0;
            if (lane == 0)
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(g) : "l"(a.counters + rbx) : "memory");
            g = __shfl_sync(0xffffffffu, g, 0);
            if (g != (unsigned int)(n_parts - 1)) continue;
            v = 0.f;
            if (has)
                for (int q = 0; q < n_parts; ++q) {
                    v += __ldcg(sp + q * RM + lane);
                    __stcg(sp + q * RM + lane, 0.f);
                }
            if (lane == 0) a.counters[rbx] = 0u;
        }
        const int row = rbx * kRows + row_i;
        if (has && m_i < a.M) {
            if (a.bias != nullptr) v += a.bias[row];
            store_from_f32(a.y, (int64_t)m_i * a.ldy + row, v, a.y_dtype);
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

// grid == 0 means the streaming kernel does not cover the shape (use the fallback).
GemvPlan gemv_plan(const hxq_desc* d, int MP, int n_sm) {
    GemvPlan p;
    const int RM = kRows * MP;
    p.kbase = -(d->col0 % 128);
    p.nch = (d->in_features - p.kbase + kChunk - 1) / kChunk;
    p.nrb = (d->out_features + kRows - 1) / kRows;
    p.grid = 0; p.units = 0; p.max_parts = 1; p.rbl_max = 1; p.warps_per_cta = 1;
    p.counter_bytes = p.scratch_bytes = 0;
    const int64_t units64 = (int64_t)p.nch * p.nrb;
    if (units64 > 0x3fffffffLL) return p;
    p.units = (int)units64;
    // one CTA per SM; more (whole multiples) only when a CTA's reduction slots would not fit
    int grid = p.units < n_sm ? p.units : n_sm;
    for (;;) {
        const int upc_max = (p.units + grid - 1) / grid;
        p.rbl_max = (upc_max - 1) / p.nch + 2;
        const int64_t bytes = (((int64_t)p.rbl_max * 4 + 15) & ~15LL) + (int64_t)p.rbl_max * p.nch * RM * 4;
        if (bytes <= kSlotBudgetBytes) break;
        if (grid >= p.units) return p;
        grid = grid + n_sm < p.units ? grid + n_sm : p.units;
    }
    p.grid = grid;
    const int upc_max = (p.units + grid - 1) / grid;
    const int upc_min = p.units / grid;
    p.max_parts = (p.nch - 1) / (upc_min > 0 ? upc_min : 1) + 2;
    // warps per CTA: least idle slots in the CTA's last round; prefer a count that keeps each
    // warp on one chunk (activations stay in registers), then the larger count
    const int wmax = (MP == 1) ? GemvCfg<1>::kMaxWarps : (MP == 2 ? GemvCfg<2>::kMaxWarps : GemvCfg<4>::kMaxWarps);
    const int wmin = wmax / 2 > 0 ? wmax / 2 : 1;
    double best = -1.0;
    p.warps_per_cta = wmax;
    for (int w = wmax; w >= wmin; --w) {
        const int rounds = (upc_max + w - 1) / w;
        double score = (double)upc_max / ((double)rounds * w) * ((double)w / wmax > 0.8 ? 1.0 : 0.9);
        if (w % p.nch != 0) score *= 0.97;
        if (score > best + 1e-9) { best = score; p.warps_per_cta = w; }
    }
    p.counter_bytes = (((size_t)p.nrb * sizeof(unsigned int)) + 255) & ~(size_t)255;
    p.scratch_bytes = (p.nch > 1) ? (size_t)p.nrb * p.max_parts * RM * sizeof(float) : 0;
    return p;
}

// Shapes the lean kernel takes: every unit whole; the slots of a CTA's units and two units of
// index bytes per warp fit beside the table.
static int lean_slot_bytes(const GemvPlan& p, int MP) {
    const int64_t slots = (p.units + p.grid - 1) / p.grid + p.nch - 1;
    const int64_t b = ((slots * kRows * MP * 4 + 127) & ~127LL) + kLeanBarBytes;
    return b > (1 << 20) ? (1 << 20) : (int)b;
}
// Most warps whose staging (two 4 KB unit buffers + one chunk of activations each) fits beside the
// table and the slots, wherever the table's 64 KB boundary falls in the window.
static int lean_max_warps(const GemvPlan& p, int MP, int x_dtype) {
    const int64_t per_warp = 2 * kRows * kChunk + (int64_t)MP * kChunk * (x_dtype == HXQ_F32 ? 4 : 2);
    const int64_t room = (int64_t)kLeanSmemBytes - kLutBytes - lean_slot_bytes(p, MP) - 256 - kRows * kChunk;
    return room > 0 ? (int)(room / per_warp) : 0;
}
// The index matrix as a 2-D tensor of 32-bit words for the bulk tensor copies (a box is at most
// 256 elements wide: 128 words are the 512 index bytes of one chunk), 8 rows per box.  The
// encoder is a driver entry point, looked up once.
#if HXQ_GEMV_TMA
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn gemv_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess &&
            r == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(q);
    }
    return fn;
}
#endif
static bool gemv_index_map(CUtensorMap* map, const hxq_desc* d) {
#if HXQ_GEMV_TMA
    EncodeTiledFn fn = gemv_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)(d->in_features / 4), (cuuint64_t)d->out_features};
    const cuuint64_t strides[1] = {(cuuint64_t)d->ld_idx};
    const cuuint32_t box[2] = {kChunk / 4, kRows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(d->indices), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
#else
    memset(map, 0, sizeof(*map));
    return true;
#endif
}

static bool gemv_lean_shape(const hxq_desc* d, const GemvPlan& p, bool x_vec) {
#ifdef HXQ_GEMV_NO_LEAN
    return false;
#endif
    if (p.grid <= 0 || p.kbase != 0 || !x_vec) return false;
    // whole 8-row blocks; whole 128-column groups (a short last chunk is masked by lane)
    if (d->in_features % 128 != 0 || d->out_features % kRows != 0) return false;
#if HXQ_GEMV_TMA
    if (d->in_features % kChunk != 0) return false;   // the bulk-copy variant reads whole chunks of activations
#endif
    if (d->group_size != 0 && d->group_size != 128) return false;
    return (int64_t)d->out_features * (d->group_size ? d->ld_st : 0) <= 0x7fffffffLL;
}

static cudaLaunchConfig_t gemv_launch_config(const GemvPlan& p, int smem_bytes, cudaStream_t stream, cudaLaunchAttribute* attr) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(p.warps_per_cta * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // set-up may overlap the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_weights_on_stream ? 0 : 1;   // weights still being written on this stream: no early start
    return cfg;
}

template <int MP>
static int launch_edge(const GemvArgs& a, const GemvPlan& p, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gemv_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes) != cudaSuccess)
            return HXQ_E_DEVICE;
        attr_set[dev] = true;
    }
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = gemv_launch_config(p, kGemvSmemBytes, stream, attr);
    return cudaLaunchKernelEx(&cfg, gemv_kernel<MP>, a) == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

// The lean kernel is compiled once per (tokens per launch, activation type, scale/offset type, sidecar, short last chunk):
// none of those is looked at inside the unit loop.
template <int MP, int XDT, int STM, bool SIDE, bool TAIL>
static int launch_lean_tail(const GemvArgs& a, const GemvPlan& p, const CUtensorMap& tmap, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = gemv_lean_kernel<MP, XDT, STM, SIDE, TAIL>;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kLeanSmemBytes) != cudaSuccess)
            return HXQ_E_DEVICE;
        attr_set[dev] = true;
    }
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = gemv_launch_config(p, kLeanSmemBytes, stream, attr);
    return cudaLaunchKernelEx(&cfg, kern, tmap, a) == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}
template <int MP, int XDT, int STM, bool SIDE>
static int launch_lean_one(const GemvArgs& a, const GemvPlan& p, const CUtensorMap& tmap, cudaStream_t stream) {
    return a.tail_lanes < 32 ? launch_lean_tail<MP, XDT, STM, SIDE, true>(a, p, tmap, stream)
                             : launch_lean_tail<MP, XDT, STM, SIDE, false>(a, p, tmap, stream);
}
template <int MP, int XDT>
static int launch_lean_st(const GemvArgs& a, const GemvPlan& p, const CUtensorMap& tmap, cudaStream_t stream) {
    const int stm = a.group_size > 0 ? (a.st_dtype == HXQ_F32 ? 1 : 2) : 0;
    const bool side = a.rowptr != nullptr;
    if (stm == 0) return side ? launch_lean_one<MP, XDT, 0, true>(a, p, tmap, stream) : launch_lean_one<MP, XDT, 0, false>(a, p, tmap, stream);
    if (stm == 1) return side ? launch_lean_one<MP, XDT, 1, true>(a, p, tmap, stream) : launch_lean_one<MP, XDT, 1, false>(a, p, tmap, stream);
    return side ? launch_lean_one<MP, XDT, 2, true>(a, p, tmap, stream) : launch_lean_one<MP, XDT, 2, false>(a, p, tmap, stream);
}
template <int MP>
static int launch_lean(const GemvArgs& a, const GemvPlan& p, const CUtensorMap& tmap, cudaStream_t stream) {
    if (a.x_dtype == HXQ_F32) return launch_lean_st<MP, HXQ_F32>(a, p, tmap, stream);
    if (a.x_dtype == HXQ_F16) return launch_lean_st<MP, HXQ_F16>(a, p, tmap, stream);
    return launch_lean_st<MP, HXQ_BF16>(a, p, tmap, stream);
}

template <int MP>
static int launch_fast(const GemvArgs& a, const GemvPlan& p, const CUtensorMap* tmap, cudaStream_t stream) {
    return tmap != nullptr ? launch_lean<MP>(a, p, *tmap, stream) : launch_edge<MP>(a, p, stream);
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
    a.scratch = nullptr; a.counters = nullptr;
    a.units = 0; a.kbase = 0; a.nch = 1; a.nrb = 0; a.max_parts = 1; a.rbl_max = 1; a.x_vec = 0; a.slot_bytes = 0; a.tail_lanes = 32;
    const int xs = dtype_size(x_dtype), ys = dtype_size(y_dtype);

    const int n_sm = sm_count();
    if (!gemv_fast_ok(d) || gemv_plan(d, 4, n_sm).grid == 0) {
        a.x = x; a.y = y; a.M = M;
        const int blocks = (d->out_features * 32 + 255) / 256;
        gemv_generic_kernel<<<blocks, 256, 0, stream>>>(a);
        return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
    }

    for (int m0 = 0; m0 < M;) {
        const int rem = M - m0;
        const int MP = mp_for(rem);
        const int mm = rem < MP ? rem : MP;
        const GemvPlan p = gemv_plan(d, MP, n_sm);
        if (p.nch > 1) {
            if (!workspace || workspace_bytes < p.counter_bytes + p.scratch_bytes) return HXQ_E_WORKSPACE;
            if (!aligned_to(workspace, 16)) return HXQ_E_ALIGN;
            a.counters = reinterpret_cast<unsigned int*>(workspace);
            a.scratch = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + p.counter_bytes);
        }
        a.x = reinterpret_cast<const char*>(x) + (int64_t)m0 * ldx * xs;
        a.y = reinterpret_cast<char*>(y) + (int64_t)m0 * ldy * ys;
        a.M = mm;
        a.kbase = p.kbase; a.nch = p.nch; a.nrb = p.nrb; a.units = p.units;
        a.max_parts = p.max_parts; a.rbl_max = p.rbl_max;
        a.x_vec = (aligned_to(a.x, 16) && ((ldx * xs) % 16 == 0)) ? 1 : 0;
        GemvPlan pl = p;
        bool lean = gemv_lean_shape(d, p, a.x_vec != 0);
        if (lean) {
            const int wfit = lean_max_warps(p, MP, x_dtype);
            if (pl.warps_per_cta > wfit) pl.warps_per_cta = wfit;
            lean = pl.warps_per_cta >= 4;
        }
        CUtensorMap tmap;
        if (lean) lean = gemv_index_map(&tmap, d);
        a.slot_bytes = lean ? lean_slot_bytes(p, MP) : 0;
        a.tail_lanes = (lean && d->in_features % kChunk) ? (d->in_features % kChunk) / 16 : 32;
        if (!lean) {     // the other kernel's warp limit
            pl = p;
            const int wedge = (MP == 4) ? GemvCfg<4>::kEdgeMaxWarps : (MP == 2 ? GemvCfg<2>::kEdgeMaxWarps : GemvCfg<1>::kEdgeMaxWarps);
            if (pl.warps_per_cta > wedge) pl.warps_per_cta = wedge;
        }
        int st;
        if (MP == 1) st = launch_fast<1>(a, pl, lean ? &tmap : nullptr, stream);
        else if (MP == 2) st = launch_fast<2>(a, pl, lean ? &tmap : nullptr, stream);
        else st = launch_fast<4>(a, pl, lean ? &tmap : nullptr, stream);
        if (st != HXQ_OK) return st;
        m0 += mm;
    }
    return HXQ_OK;
}

size_t gemv_workspace_bytes(const hxq_desc* d, int32_t M) {
    if (!gemv_fast_ok(d)) return 0;
    // a call with M >= 3 may end with a 1- or 2-token launch: those need less
    const GemvPlan p = gemv_plan(d, mp_for(M), sm_count());
    return (p.grid > 0 && p.nch > 1) ? p.counter_bytes + p.scratch_bytes : 0;
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

// ---- hxq_gemv_static: the decode product for callers that must not allocate -------------
//
// Some hosts hand every byte of device memory to their own pool at start-up, or sit inside
// a region where the CUDA allocator may not be called at all (a serving loop with a frozen
// memory plan, a plug-in that is only ever given input and output buffers).  They cannot
// provide the scratch buffer hxq_gemv asks for.  This entry point keeps that scratch inside
// the library instead: a fixed array in device memory that exists once per GPU from the
// moment the library is loaded until the process exits.
//
// The array's name is only a host-side handle; the device address comes from
// cudaGetSymbolAddress, looked up once per device (with that device current) on the first
// call and cached.  All calls on a GPU share the one array and it keeps whatever the last
// call left there, so the part this call needs is cleared on the stream first; two calls
// that can run at the same time on one GPU would trample each other's partial sums.
namespace hxq {

static __device__ __align__(256) unsigned char g_gemv_static_scratch[HXQ_GEMV_STATIC_SCRATCH_BYTES];
static void* g_gemv_static_ptr[64] = {nullptr};

}  // namespace hxq

extern "C" int hxq_gemv_static(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y,
                               int y_dtype, int64_t ldy, hxq_stream_t stream_) {
    using namespace hxq;
    int st = validate_desc(d);
    if (st != HXQ_OK) return st;
    if (!x || !y) return HXQ_E_ARG;
    if (M <= 0 || M > 16) return HXQ_E_ARG;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return HXQ_E_DTYPE;
    if (ldx < d->in_features || ldy < d->out_features) return HXQ_E_SHAPE;
    if (d->rowptr && !d->deltas) return HXQ_E_ARG;
    // size check first: nothing is touched or launched for a shape the fixed array cannot serve
    const size_t need = gemv_workspace_bytes(d, M);
    if (need > (size_t)HXQ_GEMV_STATIC_SCRATCH_BYTES) return HXQ_E_WORKSPACE;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HXQ_E_DEVICE;
    if (g_gemv_static_ptr[dev] == nullptr) {   // first call on this device (not inside a stream capture)
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_gemv_static_scratch) != cudaSuccess || p == nullptr) return HXQ_E_DEVICE;
        g_gemv_static_ptr[dev] = p;
    }
    void* scratch = g_gemv_static_ptr[dev];
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (need > 0 && cudaMemsetAsync(scratch, 0, need, stream) != cudaSuccess) return HXQ_E_LAUNCH;
    return gemv_any_m(d, x, x_dtype, M, ldx, y, y_dtype, ldy, scratch, (size_t)HXQ_GEMV_STATIC_SCRATCH_BYTES, stream);
}
