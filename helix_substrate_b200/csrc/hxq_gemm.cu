// hxq_gemm: prefill-time product on the tcgen05 tensor cores.
//
//   D[o, m] = sum_k W^[o, k] * x[m, k]      (o: 128 output rows per CTA, m: BN tokens; BN = 512 is two
//                                            256-token accumulators fed by ONE dequantised weight tile)
//
// Only here is the path a dense contraction, so only here tensor cores are used.
// One CTA owns a 128 x BN output tile; per 64-column K step
//
//   warp 0   (1 lane)  TMA: BN x 64 bf16 activations (128-byte swizzle) -> the activation ring
//   warp 18  (1 lane)  TMA: 128 x 64 index bytes -> the index ring (a warp of its own: its only
//                      condition, "the box was read", must not queue behind the activation ring's)
//   warps 2-17         dequantise the index box to bf16 in the UMMA K-major 128B-swizzled layout
//                      into the weight-tile ring: lane-replicated codebook lookup, group affine
//                      in fp32, sidecar deltas folded in (each row's CSR cursor walks forward as
//                      K advances), proxy fence, arrive
//   warp 1   (1 lane)  4 x tcgen05.mma (K = 16 each) per accumulator, fp32 in TMEM; two
//                      tcgen05.commit free the stage's activation tiles and its weight tile
//
// and after the last step the dequantising warps read TMEM (tcgen05.ld), add the bias and store
// y[m, o].  Three rings (activation tiles, weight tiles, index boxes: see Smem); every mbarrier wait
// is bounded and raises a status word.  The dequantising warps pace the kernel (a warp's chain per
// step - two waits, index load, 16 dependent lookups, stores, fence, arrival - takes about twice
// as long as the step's MMAs), so the token tile is made as wide as TMEM allows: at BN = 512 every
// dequantised tile feeds twice the tensor work.
// No cluster launch and no multicast anywhere.

#include <cuda.h>

#include "hxq_common.cuh"
#include "hxq_sm100.cuh"

namespace hxq {

int gemv_any_m(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y, int y_dtype,
               int64_t ldy, void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t gemv_workspace_bytes(const hxq_desc* d, int32_t M);

namespace gemmts {   // 17 .. 128 tokens: A operand through tensor memory (hxq_gemm_ts.cu)
bool covers(const hxq_desc* d, int32_t M);
size_t split_bytes(const hxq_desc* d, int32_t M);
int run(const hxq_desc* d, const __nv_bfloat16* xb, int64_t ldxb, int32_t M, void* y, int y_dtype, int64_t ldy,
        void* split_ws, size_t split_ws_bytes, int32_t* status_word, cudaStream_t stream);
}  // namespace gemmts

namespace gemm {

constexpr int BM = 128;        // output rows per CTA = UMMA M
constexpr int BK = 64;         // K per stage: 64 bf16 = one 128-byte swizzled row
constexpr int LUT_BYTES = 256 * 128;   // entry c, lane l at byte c*128 + l*4
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int IDX_BYTES = BM * BK;     // 8 KB
#ifndef HXQ_GEMM_DEQ_WARPS
#define HXQ_GEMM_DEQ_WARPS 16
#endif
constexpr int NUM_DEQ_WARPS = HXQ_GEMM_DEQ_WARPS;          // 8 or 16
constexpr int ROWS_PER_WARP = BM / NUM_DEQ_WARPS;           // 16 or 8
constexpr int PASSES = ROWS_PER_WARP / 8;                   // a warp covers 8 rows x 64 columns per pass
constexpr int NUM_THREADS = 32 * (3 + NUM_DEQ_WARPS);   // activation producer, MMA issuer, dequantisers, index producer
static_assert(NUM_DEQ_WARPS == 8 || NUM_DEQ_WARPS == 16, "dequantising warps: 8 or 16");

template <int BN> struct Smem {
    static constexpr int NSUB = BN > 256 ? 2 : 1;     // accumulators (UMMA N <= 256)
    static constexpr int BNS = BN / NSUB;             // tokens per accumulator
    static constexpr int STAGES = BN > 256 ? 2 : (BN == 256 ? 3 : (BN == 128 ? 4 : 6));   // activation-tile ring, as deep as shared memory allows
    // The dequantised weight tiles have a ring of their own.  With 512-token tiles it is one deeper than the
    // activation ring: with two slots only ONE stage can be dequantised at a time (the other slot belongs to
    // the running MMAs), and a stage's dequantisation - latency-bound bursts on all sixteen warps - takes
    // twice as long as its MMAs; with three, two stages are in dequantisation while the third is multiplied.
    static constexpr int ASTAGES = BN > 256 ? 3 : STAGES;
    static constexpr int B_BYTES = BN * BK * 2;
    // The index boxes have a ring too: they come from HBM and are consumed by the dequantising warps
    // long before the stage's MMAs retire.  (With the box inside the stage, a two-stage kernel had the HBM
    // round trip of the indices in series with dequantisation and the MMAs of every stage.)
    static constexpr int NIDX = BN > 256 ? 2 : (BN == 256 ? 6 : (BN == 128 ? 8 : 6));
    static constexpr int A_OFFSET = LUT_BYTES;
    static constexpr int B_OFFSET = A_OFFSET + ASTAGES * A_BYTES;
    static constexpr int IDX_OFFSET = B_OFFSET + STAGES * B_BYTES;
    static constexpr int BAR_OFFSET = IDX_OFFSET + NIDX * IDX_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;  // barriers + slack for 1024-byte alignment
    static_assert(TOTAL <= 232448, "stages + index ring must fit one SM's shared memory");
};

struct GemmArgs {
    const float* cb;
    const void* scales;
    const void* offsets;
    const int32_t* rowptr;
    const int32_t* cols;
    const float* deltas;
    const float* bias;
    void* y;
    int32_t* status;
    int64_t ldy;
    int32_t out_features, in_features, col0, group_size, ld_st, st_dtype, n_groups;
    int32_t M, y_dtype, k_steps;
    int32_t k_per_split;   // K steps per CTA along gridDim.z (== k_steps when the K range is not split)
    float* partial;        // [splits][M][out_features] fp32 partial products when split, else nullptr
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_idx, const __grid_constant__ CUtensorMap map_x,
            const GemmArgs a) {
    using S = Smem<BN>;
    constexpr int STAGES = S::STAGES;      // activation tiles
    constexpr int ASTAGES = S::ASTAGES;    // dequantised weight tiles
    extern __shared__ char smem_raw[];
    char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    char* lut = smem;
    char* a0 = smem + S::A_OFFSET;
    char* b0 = smem + S::B_OFFSET;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
    constexpr int NIDX = S::NIDX;
    char* idx0 = smem + S::IDX_OFFSET;
    uint64_t* b_full = bars;                    // [STAGES] activation tiles landed
    uint64_t* empty = bars + STAGES;            // [STAGES] UMMAs of the stage retired: its activation tiles are free
    uint64_t* a_full = bars + 2 * STAGES;       // [ASTAGES] bf16 weight tile written
    uint64_t* a_free = a_full + ASTAGES;        // [ASTAGES] UMMAs that read the weight tile retired
    uint64_t* idx_full = a_free + ASTAGES;      // [NIDX] index box landed
    uint64_t* idx_free = idx_full + NIDX;       // [NIDX] index box read by every dequantising warp
    uint64_t* acc_full = idx_free + NIDX;       // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    static_assert((4 * 6 + 2 * 8 + 2) * 8 <= 512, "barrier area");
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BN;     // token tile (fastest: neighbours share the weight tile in L2)
    const int o0 = blockIdx.y * BM;     // output-row tile
    // this CTA's K steps: [KS0, KS0 + KS) of the whole range
    const int KS0 = blockIdx.z * a.k_per_split;
    const int KS = (a.k_steps - KS0 < a.k_per_split) ? a.k_steps - KS0 : a.k_per_split;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            sm100::mbar_init(&b_full[s], 1);
            sm100::mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < ASTAGES; ++s) {
            sm100::mbar_init(&a_full[s], NUM_DEQ_WARPS);
            sm100::mbar_init(&a_free[s], 1);
        }
        for (int s = 0; s < NIDX; ++s) {
            sm100::mbar_init(&idx_full[s], 1);
            sm100::mbar_init(&idx_free[s], NUM_DEQ_WARPS);
        }
        sm100::mbar_init(acc_full, 1);
        *abort_flag = 0;
        sm100::fence_barrier_init();
        sm100::prefetch_tensormap(&map_idx);
        sm100::prefetch_tensormap(&map_x);
    }
    if (warp == 1) {
        sm100::tmem_alloc(tmem_slot, BN);
        sm100::tmem_relinquish();
    }
    // codebook table for the dequantising warps: entry c, lane l at c*128 + l*4
    for (int i = threadIdx.x; i < 256 * 32; i += NUM_THREADS)
        *reinterpret_cast<float*>(lut + (i >> 5) * 128 + (i & 31) * 4) = a.cb[i >> 5];
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int armed = 0;
            for (int ks = 0; ks < KS; ++ks) {
                const int s = ks % STAGES;
                const uint32_t ph = (uint32_t)(ks / STAGES) & 1u;
                if (!sm100::mbar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
                char* bt = b0 + s * S::B_BYTES;
                sm100::mbar_arrive_expect_tx(&b_full[s], (uint32_t)S::B_BYTES);
#pragma unroll
                for (int n = 0; n < S::NSUB; ++n)
                    sm100::tma_load_2d(bt + n * (S::BNS * BK * 2), &map_x, &b_full[s], (KS0 + ks) * BK, m0 + n * S::BNS);
                armed = ks + 1;
            }
            if (*abort_flag != 0) {
                // gave up: let copies already in flight land before the CTA retires
                for (int ks = (armed > STAGES ? armed - STAGES : 0); ks < armed; ++ks)
                    sm100::mbar_wait(&b_full[ks % STAGES], (uint32_t)(ks / STAGES) & 1u, abort_flag, 200000000LL);
            }
        }
    } else if (warp == 2 + NUM_DEQ_WARPS) {
        // ------------------------------------------------------------ index producer (TMA), a warp of its own:
        // its only condition is "the box was read", which must not queue behind the activation ring's
        if (lane == 0) {
            int armed_idx = 0;
            for (int ki = 0; ki < KS; ++ki) {
                const int si = ki % NIDX;
                if (ki >= NIDX && !sm100::mbar_wait(&idx_free[si], (uint32_t)(ki / NIDX - 1) & 1u, abort_flag)) break;
                sm100::mbar_arrive_expect_tx(&idx_full[si], (uint32_t)IDX_BYTES);
                sm100::tma_load_2d(idx0 + si * IDX_BYTES, &map_idx, &idx_full[si], (KS0 + ki) * BK, o0);
                armed_idx = ki + 1;
            }
            if (*abort_flag != 0) {
                for (int ki = (armed_idx > NIDX ? armed_idx - NIDX : 0); ki < armed_idx; ++ki)
                    sm100::mbar_wait(&idx_full[ki % NIDX], (uint32_t)(ki / NIDX) & 1u, abort_flag, 200000000LL);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = sm100::make_idesc_bf16(BM, S::BNS);
            bool ok = true;
            for (int ks = 0; ks < KS && ok; ++ks) {
                const int s = ks % STAGES, sa = ks % ASTAGES;
                const uint32_t ph = (uint32_t)(ks / STAGES) & 1u, pha = (uint32_t)(ks / ASTAGES) & 1u;
                ok = sm100::mbar_wait(&b_full[s], ph, abort_flag) && sm100::mbar_wait(&a_full[sa], pha, abort_flag);
                if (!ok) break;
                sm100::tc_fence_after_sync();
                char* bt = b0 + s * S::B_BYTES;
                const uint64_t da = sm100::make_desc_k_sw128(sm100::smem_u32(a0 + sa * A_BYTES));
#pragma unroll
                for (int n = 0; n < S::NSUB; ++n) {    // accumulator n: TMEM columns [n * BNS, +BNS)
                    const uint64_t db = sm100::make_desc_k_sw128(sm100::smem_u32(bt + n * (S::BNS * BK * 2)));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)   // +32 bytes (>> 4 = 2) per 16-element K slice
                        sm100::umma_bf16(tmem_base + (uint32_t)(n * S::BNS), da + 2 * kk, db + 2 * kk, idesc,
                                         (ks > 0 || kk > 0) ? 1u : 0u);
                }
                sm100::umma_commit(&empty[s]);      // the activation tiles of the stage ...
                sm100::umma_commit(&a_free[sa]);    // ... and its weight tile are free when these MMAs have retired
            }
            if (ok) sm100::umma_commit(acc_full);
        }
    } else {
        // ------------------------------------------------------------ dequantising warps
        const int dw = warp - 2;                     // rows [ROWS_PER_WARP * dw, + ROWS_PER_WARP)
        const int r_a = ROWS_PER_WARP * dw + (lane >> 2);   // first pass row (local); pass p is r_a + 8 p
        const int jc = lane & 3;                     // 16-column chunk of the 64-column step
        const uint32_t lane4x2 = (uint32_t)lane << 3;
        const bool affine = a.group_size > 0;

        auto load_st = [&](int ks, int row, float& s, float& t) {
            s = 1.f; t = 0.f;
            if (affine && row < a.out_features) {
                int g = (a.col0 + (KS0 + ks) * BK) / a.group_size - a.col0 / a.group_size;
                g = g < a.n_groups ? g : a.n_groups - 1;
                const int64_t o = (int64_t)row * a.ld_st + g;
                if (a.st_dtype == HXQ_F32) {
                    s = reinterpret_cast<const float*>(a.scales)[o];
                    t = reinterpret_cast<const float*>(a.offsets)[o];
                } else {
                    s = __half2float(reinterpret_cast<const __half*>(a.scales)[o]);
                    t = __half2float(reinterpret_cast<const __half*>(a.offsets)[o]);
                }
            }
        };
        float sc_c[PASSES], of_c[PASSES], sc_n[PASSES], of_n[PASSES];
        // Block case (128-column groups = two K steps each, fp32 tables with 16-byte aligned rows, shard
        // starting on a group - every Qwen2.5 shape): a row's scale and offset for FOUR groups (eight K steps)
        // come as one 16-byte load each, a block ahead.  One 4-byte load of each per row and K step is a
        // cache-line look-up per row and instruction on the pipe the table lookups use: the affine then cost
        // 14 % of the kernel (1036 -> 909 TFLOP/s on the gate projection at 2048 tokens).
        const bool st_block = affine && a.group_size == 2 * BK && a.col0 % (2 * BK) == 0 && a.st_dtype == HXQ_F32 &&
                              a.ld_st % 4 == 0 && (KS0 & 7) == 0 &&
                              ((reinterpret_cast<uintptr_t>(a.scales) | reinterpret_cast<uintptr_t>(a.offsets)) & 15) == 0;
        float4 s4c[PASSES], t4c[PASSES], s4n[PASSES], t4n[PASSES];
        auto load_block = [&](int blk, int p, float4& s4, float4& t4) {    // groups 4 blk .. 4 blk + 3 of pass p's row
            const int row = o0 + r_a + 8 * p;
            s4 = make_float4(1.f, 1.f, 1.f, 1.f); t4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < a.out_features && 4 * blk < a.n_groups) {
                const float* ps = reinterpret_cast<const float*>(a.scales) + (int64_t)row * a.ld_st + 4 * blk;
                const float* pt = reinterpret_cast<const float*>(a.offsets) + (int64_t)row * a.ld_st + 4 * blk;
                if (4 * blk + 4 <= a.n_groups) {
                    s4 = *reinterpret_cast<const float4*>(ps);
                    t4 = *reinterpret_cast<const float4*>(pt);
                } else {     // last, short block of the row: element by element, never past the row's groups
                    const int n = a.n_groups - 4 * blk;
                    s4.x = ps[0]; t4.x = pt[0];
                    if (n > 1) { s4.y = ps[1]; t4.y = pt[1]; }
                    if (n > 2) { s4.z = ps[2]; t4.z = pt[2]; }
                }
            }
        };
        if (st_block) {
#pragma unroll
            for (int p = 0; p < PASSES; ++p) load_block(KS0 >> 3, p, s4n[p], t4n[p]);
        } else {
#pragma unroll
            for (int p = 0; p < PASSES; ++p) load_st(0, o0 + r_a + 8 * p, sc_n[p], of_n[p]);
        }

        // sidecar cursor: lanes 0..ROWS_PER_WARP-1 each follow one of this warp's rows
        const int row_c = o0 + ROWS_PER_WARP * dw + lane;
        // (two entries are held ahead: the loads that refill them are not waited for inside the step)
        int e_cur = 0, e_end = 0, nc = 0x7fffffff, nc1 = 0x7fffffff;
        float nd = 0.f, nd1 = 0.f;
        if (a.rowptr != nullptr && lane < ROWS_PER_WARP && row_c < a.out_features) {
            e_cur = a.rowptr[row_c];
            e_end = a.rowptr[row_c + 1];
            if (KS0 > 0) {   // a later slice of the K range: skip the row's entries in front of it
                int lo = e_cur, hi = e_end;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (a.cols[mid] < KS0 * BK) lo = mid + 1; else hi = mid;
                }
                e_cur = lo;
            }
            if (e_cur < e_end) { nc = a.cols[e_cur]; nd = a.deltas[e_cur]; }
            if (e_cur + 1 < e_end) { nc1 = a.cols[e_cur + 1]; nd1 = a.deltas[e_cur + 1]; }
        }

        for (int ks = 0; ks < KS; ++ks) {
            const int sa = ks % ASTAGES;
            const uint32_t pha = (uint32_t)(ks / ASTAGES) & 1u;
            if (st_block) {
                const int ak = KS0 + ks;          // absolute K step; group ak >> 1, block ak >> 3
                if ((ak & 7) == 0) {              // a new block: take the prefetched one, ask for the next
#pragma unroll
                    for (int p = 0; p < PASSES; ++p) { s4c[p] = s4n[p]; t4c[p] = t4n[p]; }
                    if (ks + 8 < KS) {
#pragma unroll
                        for (int p = 0; p < PASSES; ++p) load_block((ak >> 3) + 1, p, s4n[p], t4n[p]);
                    }
                }
                const int q = (ak >> 1) & 3;
#pragma unroll
                for (int p = 0; p < PASSES; ++p) {
                    sc_c[p] = q == 0 ? s4c[p].x : (q == 1 ? s4c[p].y : (q == 2 ? s4c[p].z : s4c[p].w));
                    of_c[p] = q == 0 ? t4c[p].x : (q == 1 ? t4c[p].y : (q == 2 ? t4c[p].z : t4c[p].w));
                }
            } else {
#pragma unroll
                for (int p = 0; p < PASSES; ++p) { sc_c[p] = sc_n[p]; of_c[p] = of_n[p]; }
                if (ks + 1 < KS) {  // next step's scale/offset go out before we block
#pragma unroll
                    for (int p = 0; p < PASSES; ++p) load_st(ks + 1, o0 + r_a + 8 * p, sc_n[p], of_n[p]);
                }
            }
            const int si = ks % NIDX;
            // the stage's index box has landed, and the weight-tile slot is free (the MMAs that read it
            // ASTAGES steps ago have retired; parity 1 on a fresh barrier passes at once)
            if (!sm100::mbar_wait(&idx_full[si], (uint32_t)(ks / NIDX) & 1u, abort_flag)) break;
            if (!sm100::mbar_wait(&a_free[sa], pha ^ 1u, abort_flag)) break;
            char* st = a0 + sa * A_BYTES;
            const char* idx_s = idx0 + si * IDX_BYTES;

#pragma unroll
            for (int pass = 0; pass < PASSES; ++pass) {
                const int r = r_a + 8 * pass;
                const float sc = sc_c[pass], of = of_c[pass];
                const uint4 q = *reinterpret_cast<const uint4*>(idx_s + r * BK + jc * 16);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    // ((code << 8) | lane*8) >> 1 = code*128 + lane*4
                    const uint32_t off = __byte_perm(w[j >> 2], lane4x2, 0x5504u | (uint32_t)((j & 3) << 4)) >> 1;
                    v[j] = fmaf(*reinterpret_cast<const float*>(lut + off), sc, of);
                }
                uint4 lo, hi;
                lo.x = pack_bf16x2(v[0], v[1]);   lo.y = pack_bf16x2(v[2], v[3]);
                lo.z = pack_bf16x2(v[4], v[5]);   lo.w = pack_bf16x2(v[6], v[7]);
                hi.x = pack_bf16x2(v[8], v[9]);   hi.y = pack_bf16x2(v[10], v[11]);
                hi.z = pack_bf16x2(v[12], v[13]); hi.w = pack_bf16x2(v[14], v[15]);
                char* arow = st + r * 128;
                *reinterpret_cast<uint4*>(arow + (((2 * jc) ^ (r & 7)) << 4)) = lo;
                *reinterpret_cast<uint4*>(arow + (((2 * jc + 1) ^ (r & 7)) << 4)) = hi;
            }
            __syncwarp();

            // sidecar entries of this warp's rows that fall into this K step
            {
                const int rr = lane & (ROWS_PER_WARP - 1);      // row (within the warp's) this lane follows
                const int src = 4 * (rr & 7);                   // lane that holds that row's scale/offset
                float sc = __shfl_sync(0xffffffffu, sc_c[0], src), of = __shfl_sync(0xffffffffu, of_c[0], src);
                if (PASSES > 1) {
                    const float s1 = __shfl_sync(0xffffffffu, sc_c[PASSES - 1], src);
                    const float t1 = __shfl_sync(0xffffffffu, of_c[PASSES - 1], src);
                    if (rr & 8) { sc = s1; of = t1; }
                }
                const int k_hi = (KS0 + ks + 1) * BK;
                while (nc < k_hi) {                              // nc >= ks*BK: the cursor only moves forward
                    const int r = ROWS_PER_WARP * dw + rr;
                    const int c = nc - (KS0 + ks) * BK;
                    const uint32_t code = (uint8_t)idx_s[r * BK + c];
                    const float wv = fmaf(*reinterpret_cast<const float*>(lut + code * 128 + lane * 4), sc, of) + nd;
                    *reinterpret_cast<__nv_bfloat16*>(st + r * 128 + ((((c >> 3) ^ (r & 7)) << 4) | ((c & 7) << 1))) =
                        __float2bfloat16_rn(wv);
                    ++e_cur;
                    nc = nc1; nd = nd1;
                    if (e_cur + 1 < e_end) { nc1 = a.cols[e_cur + 1]; nd1 = a.deltas[e_cur + 1]; } else { nc1 = 0x7fffffff; }
                }
            }
            sm100::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                sm100::mbar_arrive(&idx_free[si]);     // the box has been read (sidecar patch included)
                sm100::mbar_arrive(&a_full[sa]);
            }
        }

        // ------------------------------------------------------------ epilogue (all dequantising warps)
        // A warp may read the 32 TMEM lanes of its quarter (warp % 4) only: the warps of one quarter share
        // its 32 output rows and split the token columns between them.
        {
            constexpr int COL_GROUPS = (BN / 32 < NUM_DEQ_WARPS / 4) ? BN / 32 : NUM_DEQ_WARPS / 4;
            constexpr int COLS_PER_GROUP = BN / COL_GROUPS;
            const int quarter = warp & 3;
            const int cg = dw >> 2;
            const int row = o0 + 32 * quarter + lane;
            const bool row_ok = row < a.out_features;
            if (cg < COL_GROUPS && sm100::mbar_wait(acc_full, 0u, abort_flag)) {
                sm100::tc_fence_after_sync();
                float* part = a.partial ? a.partial + (int64_t)blockIdx.z * a.M * a.out_features : nullptr;
                const float bias = (a.bias != nullptr && row_ok && part == nullptr) ? a.bias[row] : 0.f;
#pragma unroll 1
                for (int c0 = cg * COLS_PER_GROUP; c0 < (cg + 1) * COLS_PER_GROUP; c0 += 32) {
                    if (m0 + c0 >= a.M) break;       // warp-uniform
                    uint32_t r[32];
                    sm100::tmem_ld_32x32(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c0, r);
                    sm100::tmem_ld_wait();
                    if (part != nullptr) {           // warp-uniform: fp32 partial of this K slice
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int m = m0 + c0 + j;
                            if (row_ok && m < a.M) part[(int64_t)m * a.out_features + row] = __uint_as_float(r[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int m = m0 + c0 + j;
                            if (row_ok && m < a.M)
                                store_from_f32(a.y, (int64_t)m * a.ldy + row, __uint_as_float(r[j]) + bias, a.y_dtype);
                        }
                    }
                }
            }
        }
    }

    sm100::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        sm100::tc_fence_after_sync();
        sm100::tmem_dealloc(tmem_base, BN);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && a.status != nullptr) atomicExch(a.status, HXQ_E_TIMEOUT);
}

}  // namespace gemm
}  // namespace hxq

// ---- host side ---------------------------------------------------------------------
namespace hxq {
namespace gemm {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fp32 / fp16 activations -> contiguous bf16 [M, ld_out] (tensor-core operand type)
__global__ void __launch_bounds__(256) to_bf16_kernel(const void* x, int x_dtype, int64_t ldx, int M, int K,
                                                       __nv_bfloat16* out, int64_t ld_out) {
    const int64_t total = (int64_t)M * ld_out;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / ld_out), k = (int)(i - (int64_t)m * ld_out);
        out[i] = __float2bfloat16_rn(k < K ? load_as_f32(x, (int64_t)m * ldx + k, x_dtype) : 0.f);
    }
}

// y[m, o] = sum over the K slices of partial[z][m][o], + bias, rounded once (fixed order: deterministic).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int out_features,
                                                            const float* __restrict__ bias, void* y, int y_dtype, int64_t ldy) {
    const int64_t total = (int64_t)M * out_features;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / out_features), o = (int)(i - (int64_t)m * out_features);
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v += partial[(int64_t)z * total + i];
        if (bias != nullptr) v += bias[o];
        store_from_f32(y, (int64_t)m * ldy + o, v, y_dtype);
    }
}

void launch_splitk_reduce(const float* partial, int splits, int M, int out_features, const float* bias, void* y,
                          int y_dtype, int64_t ldy, cudaStream_t stream) {
    const int64_t total = (int64_t)M * out_features;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(partial, splits, M, out_features, bias, y, y_dtype, ldy);
}

// K slices per output tile: enough CTAs to fill the GPU when the tile grid alone does not
// (one token tile x few row tiles, e.g. down_proj at M <= 64), at least four K steps each.
static int pick_bn(int M) { return M > 256 ? 512 : (M > 128 ? 256 : (M > 64 ? 128 : 64)); }
static int sm_count() {
    int n_sm = 148, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n_sm <= 0)
        n_sm = 148;
    return n_sm;
}
static int pick_splits(int grid_m, int grid_o, int k_steps, int n_sm) {
    // only with a single token tile: with more, the fp32 partials (splits x M x OUT) cost more traffic than
    // the idle SMs are worth (measured: k/v at M = 2048 / 8192 split 8 / 2 ways lost 5-10 % of the whole pass)
    const int tiles = grid_m * grid_o;
    if (grid_m > 1 || tiles * 2 > n_sm) return 1;
    int s = n_sm / tiles;
    if (s > 8) s = 8;
    if (s > k_steps / 4) s = k_steps / 4;
    return s < 1 ? 1 : s;
}

bool fast_ok(const hxq_desc* d) {
    return (d->in_features % 16 == 0) && (d->ld_idx % 16 == 0) && aligned_to(d->indices, 16) &&
           (d->col0 % 64 == 0) && (d->group_size == 0 || d->group_size % 64 == 0) && encode_fn() != nullptr;
}

static int64_t x_pad(const hxq_desc* d) { return ((int64_t)d->in_features + 7) / 8 * 8; }

static size_t xcopy_bytes(const hxq_desc* d, int32_t M) { return (((size_t)M * x_pad(d) * 2 + 255) & ~(size_t)255) + 256; }

size_t workspace_bytes(const hxq_desc* d, int32_t M) {
    if (!fast_ok(d)) return gemv_workspace_bytes(d, 4);
    // room for a bf16 copy of x when it is not usable in place, then the fp32 partials of the K slices
    // when the output tile grid is too small to fill the GPU
    size_t split = 0;
    const int BN = pick_bn(M);
    const int s = pick_splits((M + BN - 1) / BN, (d->out_features + BM - 1) / BM, (d->in_features + BK - 1) / BK, sm_count());
    if (s > 1) split = (size_t)s * M * d->out_features * sizeof(float);
    if (gemmts::covers(d, M)) {
        const size_t ts = gemmts::split_bytes(d, M);
        split = ts > split ? ts : split;
    }
    return xcopy_bytes(d, M) + split;
}

template <int BN>
static int launch(const CUtensorMap& mi, const CUtensorMap& mx, const GemmArgs& a, int grid_m, int grid_o, int splits,
                  cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BN>::TOTAL) !=
            cudaSuccess)
            return HXQ_E_DEVICE;
        attr_set[dev] = true;
    }
    gemm_kernel<BN><<<dim3(grid_m, grid_o, splits), NUM_THREADS, Smem<BN>::TOTAL, stream>>>(mi, mx, a);
    return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

int run(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y, int y_dtype, int64_t ldy,
        void* workspace, size_t ws_bytes, int32_t* status_word, cudaStream_t stream) {
    const void* xb = x;
    int64_t ldxb = ldx;
    const bool x_in_place = (x_dtype == HXQ_BF16) && aligned_to(x, 16) && ((ldx * 2) % 16 == 0);
    if (!x_in_place) {
        const int64_t ld = x_pad(d);
        if (!workspace || ws_bytes < (size_t)M * ld * 2) return HXQ_E_WORKSPACE;   // (the first xcopy_bytes of the workspace)
        if (!aligned_to(workspace, 16)) return HXQ_E_ALIGN;
        int64_t total = (int64_t)M * ld;
        int blocks = (int)((total + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        to_bf16_kernel<<<blocks, 256, 0, stream>>>(x, x_dtype, ldx, M, d->in_features,
                                                   reinterpret_cast<__nv_bfloat16*>(workspace), ld);
        if (cudaGetLastError() != cudaSuccess) return HXQ_E_LAUNCH;
        xb = workspace;
        ldxb = ld;
    }
    if (gemmts::covers(d, M)) {   // up to 128 tokens: the index-stream-bound kernel
        const size_t off = xcopy_bytes(d, M);
        void* sws = (workspace && ws_bytes > off) ? reinterpret_cast<char*>(workspace) + off : nullptr;
        return gemmts::run(d, reinterpret_cast<const __nv_bfloat16*>(xb), ldxb, M, y, y_dtype, ldy, sws,
                           sws ? ws_bytes - off : 0, status_word, stream);
    }
    const int BN = pick_bn(M);
    CUtensorMap mi, mx;
    if (!make_map_2d(&mi, CU_TENSOR_MAP_DATA_TYPE_UINT8, d->indices, (uint64_t)d->in_features,
                     (uint64_t)d->out_features, (uint64_t)d->ld_idx, BK, BM, CU_TENSOR_MAP_SWIZZLE_NONE))
        return HXQ_E_DEVICE;
    if (!make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, xb, (uint64_t)d->in_features, (uint64_t)M,
                     (uint64_t)ldxb * 2, BK, (uint32_t)(BN > 256 ? 256 : BN), CU_TENSOR_MAP_SWIZZLE_128B))
        return HXQ_E_DEVICE;
    GemmArgs a;
    a.cb = d->codebook; a.scales = d->scales; a.offsets = d->offsets;
    a.rowptr = d->rowptr; a.cols = d->cols; a.deltas = d->deltas; a.bias = d->bias;
    a.y = y; a.status = status_word; a.ldy = ldy;
    a.out_features = d->out_features; a.in_features = d->in_features; a.col0 = d->col0;
    a.group_size = d->group_size; a.ld_st = d->ld_st; a.st_dtype = d->st_dtype;
    a.n_groups = d->group_size > 0
                     ? (d->col0 + d->in_features - 1) / d->group_size - d->col0 / d->group_size + 1 : 0;
    a.M = M; a.y_dtype = y_dtype;
    a.k_steps = (d->in_features + BK - 1) / BK;
    const int grid_o = (d->out_features + BM - 1) / BM;
    const int grid_m = (M + BN - 1) / BN;
    int splits = 1;
    a.k_per_split = a.k_steps;
    a.partial = nullptr;
    {
        splits = pick_splits(grid_m, grid_o, a.k_steps, sm_count());
        const size_t off = xcopy_bytes(d, M);
        if (splits > 1 && workspace && aligned_to(workspace, 16) &&
            ws_bytes >= off + (size_t)splits * M * d->out_features * sizeof(float)) {
            a.k_per_split = ((a.k_steps + splits - 1) / splits + 7) & ~7;   // whole blocks of eight K steps (scale/offset block loads)
            splits = (a.k_steps + a.k_per_split - 1) / a.k_per_split;   // no empty slice
            if (splits > 1) {
                a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + off);
            } else {        // a K range of one block: nothing to split
                a.k_per_split = a.k_steps;
            }
        } else {
            splits = 1;
        }
    }
    int st;
    if (BN == 512) st = launch<512>(mi, mx, a, grid_m, grid_o, splits, stream);
    else if (BN == 256) st = launch<256>(mi, mx, a, grid_m, grid_o, splits, stream);
    else if (BN == 128) st = launch<128>(mi, mx, a, grid_m, grid_o, splits, stream);
    else st = launch<64>(mi, mx, a, grid_m, grid_o, splits, stream);
    if (st != HXQ_OK || splits == 1) return st;
    launch_splitk_reduce(a.partial, splits, M, d->out_features, d->bias, y, y_dtype, ldy, stream);
    return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

}  // namespace gemm
}  // namespace hxq

extern "C" size_t hxq_gemm_workspace_bytes(const hxq_desc* d, int32_t M) {
    if (hxq::validate_desc(d) != HXQ_OK || M <= 0) return 0;
    return hxq::gemm::workspace_bytes(d, M);
}

extern "C" int hxq_gemm(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx, void* y,
                        int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes,
                        int32_t* status_word, hxq_stream_t stream_) {
    using namespace hxq;
    int st = validate_desc(d);
    if (st != HXQ_OK) return st;
    if (!x || !y) return HXQ_E_ARG;
    if (M <= 0) return HXQ_E_ARG;
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return HXQ_E_DTYPE;
    if (ldx < d->in_features || ldy < d->out_features) return HXQ_E_SHAPE;
    if (d->rowptr && !d->deltas) return HXQ_E_ARG;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!gemm::fast_ok(d)) {
        // ragged or unaligned shapes: token groups through the decode kernels, which need
        // zeroed arrival counters while this entry point's workspace may be dirty
        const size_t need = gemv_workspace_bytes(d, 4);
        if (need > 0) {
            if (!workspace || workspace_bytes < need) return HXQ_E_WORKSPACE;
            if (cudaMemsetAsync(workspace, 0, need, stream) != cudaSuccess) return HXQ_E_LAUNCH;
        }
        return gemv_any_m(d, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes, stream);
    }
    return gemm::run(d, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes, status_word, stream);
}
