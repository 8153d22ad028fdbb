// hxq_gemm, 5 .. 128 tokens: y[m, o] = sum_i x[m, i] * W^[o, i] + sidecar + bias on the tensor cores
// with the dequantised weights handed to the MMA through TENSOR MEMORY, never through shared memory.
//
// At these token counts the product is still bound by the index stream (one byte and one table lookup
// per weight, each weight used for at most 128 tokens), so the kernel is built like the decode kernel,
// not like a GEMM: everything that is not a lookup is kept off the instruction stream of the warps
// that do the lookups.
//
//   * CTA tile: 128 output rows x BN tokens (BN = 16, 32, 64, 128), K walked in stages of one or two
//     128-column boxes (two up to 64 tokens), one CTA per SM; small row-tile grids split K over
//     gridDim.z (fp32 partials + a fixed-order sum).
//   * index bytes: the 512 dequantising threads copy each stage's 128 x 128 box themselves with two
//     16-byte asynchronous copies per thread (eight lanes per 128-byte line: whole lines per request)
//     into a ring of up to eight 16 KB boxes laid out in the 128-byte swizzle, up to seven stages
//     (112 KB per SM) ahead: that much in flight is what this access pattern needs to run near the
//     DRAM rate.  Each thread's copies report to the box's mbarrier (cp.async.mbarrier.arrive); a
//     second barrier per box, one arrival per warp, says the codes are in registers and the box may
//     be refilled.  The warps are not otherwise synchronised: one named barrier per stage over all
//     512 threads instead was 15 % slower (every stage then takes as long as its slowest warp).
//   * scale and offset: the 128 rows' values for four stages at a time ride with the index copies
//     (one 16-byte copy per row and table) into the unused halves of the codebook table's rows.
//   * warp 0, one lane: TMA producer of the activation tiles (two 64-column boxes of bf16 per stage,
//     128-byte swizzled, ring of three to six).  No multicast, no cluster.
//   * warps 2..17: dequantisers, ONE THREAD PER OUTPUT ROW and 32-column quarter of the stage.  A
//     thread reads its row's 32 codes with two conflict-free 16-byte loads (the swizzle spreads eight
//     rows over all banks), looks each up in the lane-replicated codebook (one byte-permute + one
//     load per weight, bank == lane), applies its (row, group) scale and offset in fp32, adds the
//     row's sidecar deltas that fall into its columns, packs pairs to bf16 and stores its 16
//     registers straight into the A operand's columns of tensor memory (tcgen05.st 32x32b: TMEM
//     lane == output row).  The store of a stage is waited for after the lookups of the next one.
//     The sidecar cursor is thread-local: no cross-lane step anywhere.  (Adding the sidecar term in
//     the epilogue instead - delta times the activation at its column, per token - was tried: every
//     such load is a cache-line look-up per lane, 13 us per tile at 32 tokens and 44 us at 128.)
//   * warp 1, one lane: issues tcgen05.mma kind::f16 with A from tensor memory and B (activations,
//     K-major, 128-byte swizzle) from shared memory into the fp32 accumulator in tensor memory, and
//     commits the stage, which frees its activation tile and its A columns.
//   * epilogue (the dequantising warps): accumulator -> registers, + bias, store.
//
// Every mbarrier wait is clock-bounded; a wait that gives up raises a CTA-wide abort flag and the
// global status word (HXQ_E_TIMEOUT); every other wait of the CTA then returns at its next poll,
// in-flight copies are waited for and tensor memory is freed before the CTA returns.

#include <cuda.h>
#include <stdlib.h>

#include "hxq_common.cuh"
#include "hxq_sm100.cuh"

namespace hxq {
namespace gemm {   // helpers shared with the large-token kernel (hxq_gemm.cu)
bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw);
void launch_splitk_reduce(const float* partial, int splits, int M, int out_features, const float* bias, void* y,
                          int y_dtype, int64_t ldy, cudaStream_t stream);
}  // namespace gemm

namespace gemmts {

constexpr int BM = 128;             // output rows per CTA = UMMA M = TMEM lanes
constexpr int KS = 128;             // K columns per index box (a stage is one or two boxes, see Rings)
constexpr int DEQ_WARPS = 16;       // four warps per TMEM lane quarter, each takes 32 of a stage's 128 columns
constexpr int DEQ_THREADS = 32 * DEQ_WARPS;
constexpr int NUM_THREADS = 32 * (2 + DEQ_WARPS);   // activation producer, MMA issuer, 16 dequantisers
constexpr int LUT_BYTES = 256 * 256;            // entry c, lane l at c * 256 + l * 4, base on a 64 KB boundary
constexpr int IDX_BYTES = BM * KS;              // 16 KB per box
constexpr int SMEM_TOTAL = 232448;
constexpr int TMEM_COLS = 512;
constexpr int A_COLS = KS / 2;                  // 64 columns of packed bf16 pairs per box

struct Args {
    const float* cb;
    const void* scales;
    const void* offsets;
    const int32_t* rowptr;
    const int32_t* cols;
    const float* deltas;
    const float* bias;
    const uint8_t* idx;        // index matrix [out_features, ld_idx]
    int64_t ld_idx;
    void* y;
    int32_t* status;
    float* partial;            // [splits][M][out_features] when the K range is split, else nullptr
    int64_t ldy;
    int32_t out_features, in_features, col0, group_size, ld_st, st_dtype, n_groups;
    int32_t M, y_dtype, k_steps, k_per_split;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));   // first source -> upper half
    return r;
}

// D[tmem] (+)= A[tmem] * B[smem], bf16 x bf16 -> fp32, issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 16 registers per thread -> 16 consecutive columns of this thread's TMEM lane (whole warp).
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// One bf16 half of a packed pair += delta (the value is re-rounded to bf16).
__device__ __forceinline__ uint32_t add_to_half(uint32_t pair, int hi, float delta) {
    const float v = __uint_as_float(hi ? (pair & 0xffff0000u) : (pair << 16)) + delta;
    const uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
    return hi ? ((pair & 0x0000ffffu) | (b << 16)) : ((pair & 0xffff0000u) | b);
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Per token tile: H index boxes (128 columns each) per stage, NB activation tiles / A-operand column
// blocks, NI index boxes-of-a-stage.  Up to 64 tokens a stage is two boxes: what a thread does once
// per stage (barrier polls, the hand-over to the MMA warp, ring bookkeeping) is then paid once per
// 64 instead of 32 weights, and the two boxes' lookups overlap each other's tails (at 64 tokens
// even with rings of two: 76 vs 89 us); at 128 tokens the activation tiles leave no room for that.
// The table sits on a 64 KB boundary of the shared window, which leaves ~63 KB below and ~100 KB above it.
template <int BN> struct Rings;
template <> struct Rings<16> { static constexpr int NB = 3, NI = 4, H = 2; };
template <> struct Rings<32> { static constexpr int NB = 3, NI = 3, H = 2; };
template <> struct Rings<64> { static constexpr int NB = 2, NI = 2, H = 2; };
template <> struct Rings<128> { static constexpr int NB = 3, NI = 3, H = 1; };
static int halves_of(int BN) { return BN <= 64 ? 2 : 1; }

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_ts_kernel(const __grid_constant__ CUtensorMap map_x, const Args a) {
    constexpr int H = Rings<BN>::H;                      // index boxes per stage
    constexpr int KST = KS * H;                          // K columns per stage
    constexpr int B_BYTES = BN * KST * 2;                // 2 H [BN x 64] bf16 sub-tiles
    constexpr int IDXB = IDX_BYTES * H;                  // index bytes per stage
    constexpr int ACOLS = A_COLS * H;                    // A-operand columns per stage
    constexpr int NB = Rings<BN>::NB;
    constexpr int NI = Rings<BN>::NI;
    // stages the index copies run ahead: one box of slack where the ring is deep enough, so that a warp
    // can start the next stage while the slowest warp is still reading the previous one
    constexpr int PD = NI >= 5 ? NI - 2 : NI - 1;
    static_assert((BN < 32 ? 32 : BN) + NB * ACOLS <= TMEM_COLS, "accumulator + A ring must fit tensor memory");
    static_assert(NI >= 2 && NI <= 8 && NB >= 2 && NB <= 6, "barrier and slot-table layout");
    extern __shared__ __align__(1024) char smem_raw[];
    const uint32_t smem_base = sm100::smem_u32(smem_raw);
    const uint32_t lut_base = (smem_base + 0xFFFFu) & ~0xFFFFu;
    char* lut = smem_raw + (lut_base - smem_base);
    // Two rings share what is left of shared memory around the table: the larger items first, below
    // the table while they fit there, then the smaller ones in what is left below, the rest above.
    const uint32_t lo0 = (smem_base + 1023u) & ~1023u;
    const uint32_t hi0 = lut_base + LUT_BYTES;
    constexpr bool B_FIRST = B_BYTES > IDXB;
    constexpr uint32_t SZ1 = B_FIRST ? B_BYTES : IDXB, SZ2 = B_FIRST ? IDXB : B_BYTES;
    constexpr int N1 = B_FIRST ? NB : NI, N2 = B_FIRST ? NI : NB;
    const int room_lo = (int)(lut_base - lo0);
    const int n1_lo = room_lo / (int)SZ1 < N1 ? room_lo / (int)SZ1 : N1;
    const int n2_lo = (room_lo - n1_lo * (int)SZ1) / (int)SZ2 < N2 ? (room_lo - n1_lo * (int)SZ1) / (int)SZ2 : N2;
    const uint32_t lo2 = lo0 + (uint32_t)n1_lo * SZ1, hi2 = hi0 + (uint32_t)(N1 - n1_lo) * SZ1;
    const bool layout_ok = hi2 + (uint32_t)(N2 - n2_lo) * SZ2 <= smem_base + SMEM_TOTAL;
    auto slot1 = [&](int i) -> uint32_t { return i < n1_lo ? lo0 + (uint32_t)i * SZ1 : hi0 + (uint32_t)(i - n1_lo) * SZ1; };
    auto slot2 = [&](int i) -> uint32_t { return i < n2_lo ? lo2 + (uint32_t)i * SZ2 : hi2 + (uint32_t)(i - n2_lo) * SZ2; };
    auto b_slot = [&](int i) -> uint32_t { return B_FIRST ? slot1(i) : slot2(i); };       // activation tile i
    auto idx_slot = [&](int i) -> uint32_t { return B_FIRST ? slot2(i) : slot1(i); };     // index box i
    // barriers live in the unused upper halves of the table's first rows
    uint64_t* b_full = reinterpret_cast<uint64_t*>(lut + 128);       // [NB] activation tile landed
    uint64_t* a_full = b_full + 6;                                   // [NB] A columns of the stage written
    uint64_t* st_free = reinterpret_cast<uint64_t*>(lut + 256 + 128);// [NB] MMAs of the stage retired
    uint64_t* acc_full = st_free + 6;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(st_free + 7);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint64_t* idx_full = reinterpret_cast<uint64_t*>(lut + 512 + 128);   // [NI] index box landed (every copying thread reports)
    uint64_t* idx_free = idx_full + 8;                                   // [NI] codes read by all dequantising warps

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BN;
    const int o0 = blockIdx.y * BM;
    const int KS0 = blockIdx.z * a.k_per_split;
    const int NK = (a.k_steps - KS0 < a.k_per_split) ? a.k_steps - KS0 : a.k_per_split;

    // ---- the dequantising threads (warps 2..17; the definitions below are only used by them)
    const int dw = warp - 2;
    const int dt = threadIdx.x - 64;              // 0 .. 511
    const int quarter = warp & 3;                 // TMEM lanes this warp may touch: [32 * quarter, +32)
    const int kq = dw >> 2;                       // which 32 columns of each stage (warps 2..17: every quarter gets kq = 0..3 once)
    const int r = 32 * quarter + lane;            // row inside the CTA tile == TMEM lane
    const int row = o0 + r;
    const bool row_ok = row < a.out_features;
    const bool affine = a.group_size > 0;

    // ---- scale / offset of (row, this thread's 32 columns of a box)
    // Staged case (one group per box, fp32 tables with 16-byte aligned rows - every Qwen2.5 shape):
    // the 128 rows' values for FOUR boxes at a time ride with the index copies as one 16-byte
    // asynchronous copy per row and table into the unused halves of the codebook table's rows
    // (two buffers), and a thread picks its row's four values up with one 16-byte shared load.
    // A per-thread global load instead costs 32 cache-line look-ups per warp instruction, twice per
    // stage, on the same load/store pipe as the table lookups: it doubled the stage time.
    // Other layouts (fp16 tables, odd group sizes, shards starting mid-row-of-four) load per thread.
    // (a K slice must start on a block of four boxes: with two buffers, the third block's copy would
    // otherwise be issued in the prologue, before the first block has been read)
    const bool st_staged = affine && a.group_size == KS && a.col0 % KS == 0 && a.st_dtype == HXQ_F32 &&
                           a.ld_st % 4 == 0 && ((KS0 * H) & 3) == 0 &&
                           ((reinterpret_cast<uintptr_t>(a.scales) | reinterpret_cast<uintptr_t>(a.offsets)) & 15) == 0;
    const int g_base = affine ? a.col0 / a.group_size : 0;
    // hole h (16 bytes) of buffer b: entries [b][table][row], eight per table row, from table row 8 on
    auto st_hole = [&](int b, int which, int rr) -> uint32_t {
        const int h = b * 256 + which * 128 + rr;
        return lut_base + (uint32_t)((8 + (h >> 3)) * 256 + 128 + (h & 7) * 16);
    };
    const int sf_row = dt & 127, sf_which = (dt >> 7) & 1;       // fetch mapping (threads 0..255)
    const bool sf_ok = st_staged && dt < 256 && o0 + sf_row < a.out_features;
    const float* sf_src = reinterpret_cast<const float*>(sf_which ? a.offsets : a.scales) +
                          (int64_t)(sf_ok ? o0 + sf_row : 0) * a.ld_st;
    auto fetch_st4 = [&](int kj) {     // groups 4 B .. 4 B + 3 of the block B that stage kj's first box belongs to
        if (st_staged && dt < 256) {
            const int blk = ((KS0 + kj) * H) >> 2;
            int n = a.n_groups - 4 * blk;
            n = n > 4 ? 4 : (n < 0 ? 0 : n);
            const uint32_t bytes = sf_ok ? (uint32_t)(4 * n) : 0u;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;"
                         :: "r"(st_hole(blk & 1, sf_which, sf_row)), "l"(bytes ? sf_src + 4 * blk : reinterpret_cast<const float*>(a.scales)), "r"(bytes) : "memory");
        }
    };
    auto load_st = [&](int bx, float& s, float& t) {     // the per-thread path; bx: box number inside this K slice
        s = 1.f; t = 0.f;
        if (affine && row_ok) {
            int g = (a.col0 + (KS0 * H + bx) * KS + kq * 32) / a.group_size - g_base;
            g = g < a.n_groups ? g : a.n_groups - 1;      // K tail: those activations are zero
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

    // ---- index copies.  Copy mapping (not the row this thread dequantises), per box: chunk q = dt + 512 c,
    // c = 0, 1: box row q / 8, 16-byte piece q % 8 -> eight consecutive lanes fetch one 128-byte line.
    const int c_row = dt >> 3, c_piece = dt & 7;                 // second copy: row + 64, same piece
    const bool c_ok0 = o0 + c_row < a.out_features, c_ok1 = o0 + c_row + 64 < a.out_features;
    const uint8_t* c_src0 = a.idx + (int64_t)(c_ok0 ? o0 + c_row : 0) * a.ld_idx + (int64_t)KS0 * KST + c_piece * 16;
    const uint8_t* c_src1 = a.idx + (int64_t)(c_ok1 ? o0 + c_row + 64 : 0) * a.ld_idx + (int64_t)KS0 * KST + c_piece * 16;
    const uint32_t c_dst0 = (uint32_t)(c_row * 128) + ((uint32_t)(c_piece ^ (c_row & 7)) << 4);
    const uint32_t c_dst1 = c_dst0 + 64u * 128u;                 // (row + 64) & 7 == row & 7
    // stages whose columns all lie inside the matrix; the copies of later ones are cut at the edge
    const int full_stages = a.in_features / KST - KS0;
    auto copy_stage = [&](int kj) {     // this thread's 2 H pieces of stage kj into ring slot kj % NI
        if (kj < NK) {
            if (kj == 0 || (((KS0 + kj) * H) & 3) == 0) fetch_st4(kj);
            const uint32_t slot = idx_slot(kj % NI);
#pragma unroll
            for (int h = 0; h < H; ++h) {
                const int64_t off = (int64_t)kj * KST + h * KS;
                const bool in_k = kj < full_stages || (int64_t)KS0 * KST + off + c_piece * 16 + 16 <= a.in_features;
                // rows past the matrix and columns past its end are filled with zeros (source size 0)
                const uint32_t n0 = (c_ok0 && in_k) ? 16u : 0u, n1 = (c_ok1 && in_k) ? 16u : 0u;
                const uint32_t box = slot + (uint32_t)(h * IDX_BYTES);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(box + c_dst0), "l"(n0 ? c_src0 + off : a.idx), "r"(n0) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(box + c_dst1), "l"(n1 ? c_src1 + off : a.idx), "r"(n1) : "memory");
            }
            // one of the stage barrier's 512 expected arrivals, made when this thread's copies so far have landed
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(sm100::smem_u32(&idx_full[kj % NI])) : "memory");
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NB; ++s) {
            sm100::mbar_init(&b_full[s], 1);
            sm100::mbar_init(&a_full[s], DEQ_WARPS);
            sm100::mbar_init(&st_free[s], 1);
        }
        for (int s = 0; s < NI; ++s) {
            sm100::mbar_init(&idx_full[s], DEQ_THREADS);
            sm100::mbar_init(&idx_free[s], DEQ_WARPS);
        }
        sm100::mbar_init(acc_full, 1);
        *abort_flag = 0;
        sm100::fence_barrier_init();
        sm100::prefetch_tensormap(&map_x);
    }
    // ---- sidecar of this row tile: the CSR entries of rows o0 .. o0 + 127 are one contiguous run of
    // cols[] / deltas[]; up to SC_MAX of them are copied into the table's unused halves (rows 72 ..),
    // so that the per-thread cursors below read shared memory.  (Cursors on global memory made every
    // warp wait, once per stage, for the DRAM miss of the previous stage's cursor refill: that wait,
    // not the lookups, set the stage time.)  A tile with more entries keeps its cursors on global memory.
    constexpr int SC_MAX = 2944, SC_ROW_C = 72, SC_ROW_D = SC_ROW_C + SC_MAX / 32;   // (0.1 % of 128 x 18944 weights is 2425)
    static_assert(SC_ROW_D + SC_MAX / 32 <= 256, "sidecar staging must fit the table's rows");
    int sc_e0 = 0, sc_n = 0;
    if (a.rowptr != nullptr) {
        const int o1 = o0 + BM < a.out_features ? o0 + BM : a.out_features;
        sc_e0 = a.rowptr[o0];
        sc_n = a.rowptr[o1] - sc_e0;
    }
    const bool sc_staged = sc_n <= SC_MAX;
    auto sc_addr = [&](int base_row, int e) -> uint32_t {     // entry e (relative to the tile's first)
        return lut_base + ((uint32_t)(base_row + (e >> 5)) << 8) + 128u + ((uint32_t)(e & 31) << 2);
    };
    __syncthreads();          // barriers initialised
    // The first index boxes are asked for before the rest is set up: the table build and the
    // tensor-memory allocation below overlap their flight (they touch neither the ring slots nor the
    // table's holes the scale/offset values go to).
    if (layout_ok && warp >= 2) {
        if (sc_staged) {     // (these copies are covered by the first box's barrier arrival below)
            for (int e = dt; e < sc_n; e += DEQ_THREADS) {
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(sc_addr(SC_ROW_C, e)), "l"(a.cols + sc_e0 + e) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(sc_addr(SC_ROW_D, e)), "l"(a.deltas + sc_e0 + e) : "memory");
            }
        }
#pragma unroll
        for (int kj = 0; kj < PD; ++kj) copy_stage(kj);
    }
    if (warp == 1) {
        sm100::tmem_alloc(tmem_slot, TMEM_COLS);
        sm100::tmem_relinquish();
    }
    // lane-replicated codebook (the lower 128 bytes of each 256-byte row)
    for (int i = threadIdx.x; i < 256 * 32; i += NUM_THREADS)
        *reinterpret_cast<float*>(lut + (i >> 5) * 256 + (i & 31) * 4) = a.cb[i >> 5];
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a0 = tmem_base + (uint32_t)(BN < 32 ? 32 : BN);   // the A ring follows the accumulator's columns

    if (!layout_ok) {
        if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, HXQ_E_SHAPE);
    } else if (warp == 0) {
        // ------------------------------------------------------------ activation producer (TMA)
        if (lane == 0) {
            int armed = 0;
            for (int ks = 0; ks < NK; ++ks) {
                const int s = ks % NB;
                const uint32_t ph = (uint32_t)(ks / NB) & 1u;
                if (!sm100::mbar_wait(&st_free[s], ph ^ 1u, abort_flag, 2000000000LL, 200u)) break;
                char* bt = smem_raw + (b_slot(s) - smem_base);
                sm100::mbar_arrive_expect_tx(&b_full[s], (uint32_t)B_BYTES);
#pragma unroll
                for (int j = 0; j < 2 * H; ++j)       // 64-column sub-tiles
                    sm100::tma_load_2d(bt + j * (BN * 128), &map_x, &b_full[s], (KS0 + ks) * KST + 64 * j, m0);
                armed = ks + 1;
            }
            if (*abort_flag != 0) {
                for (int ks = (armed > NB ? armed - NB : 0); ks < armed; ++ks)
                    sm100::mbar_wait(&b_full[ks % NB], (uint32_t)(ks / NB) & 1u, abort_flag, 200000000LL);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = sm100::make_idesc_bf16(BM, BN);
            bool ok = true;
            for (int ks = 0; ks < NK && ok; ++ks) {
                const int s = ks % NB;
                const uint32_t ph = (uint32_t)(ks / NB) & 1u;
                ok = sm100::mbar_wait(&b_full[s], ph, abort_flag, 2000000000LL, 50u) && sm100::mbar_wait(&a_full[s], ph, abort_flag, 2000000000LL, 50u);
                if (!ok) break;
                sm100::tc_fence_after_sync();
                // B: sub-tile kk / 4 (64 K columns each), + 32 bytes (2 in descriptor units) per 16-column slice
                const uint64_t db0 = sm100::make_desc_k_sw128(b_slot(s));
                const uint32_t ta = tmem_a0 + (uint32_t)(s * ACOLS);
#pragma unroll
                for (int kk = 0; kk < KST / 16; ++kk) {
                    const uint64_t db = db0 + (uint64_t)((kk >> 2) * (BN * 128 / 16) + 2 * (kk & 3));
                    umma_bf16_ts(tmem_base, ta + (uint32_t)(kk * 8), db, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                }
                sm100::umma_commit(&st_free[s]);
            }
            if (ok) sm100::umma_commit(acc_full);
        }
    } else {
        // ------------------------------------------------------------ dequantising warps
        const uint32_t lane_key = lut_base | ((uint32_t)lane << 2);
        const uint32_t t_row = tmem_a0 + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(kq * 16);

        // sidecar cursor of this row: entries are sorted by column; this thread takes those inside its
        // 32 columns of every stage and steps over the others.  e_cur / e_end count from the tile's first
        // entry; nc is the column of entry e_cur (read when the cursor moves).
        int e_cur = 0, e_end = 0, nc = 0x7fffffff;
        if (a.rowptr != nullptr && row_ok) {
            e_cur = a.rowptr[row] - sc_e0;
            e_end = a.rowptr[row + 1] - sc_e0;
        }
        auto sc_col = [&](int e) -> int {
            if (sc_staged) {
                int v;
                asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(sc_addr(SC_ROW_C, e)));
                return v;
            }
            return a.cols[sc_e0 + e];
        };
        auto sc_delta = [&](int e) -> float {
            if (sc_staged) {
                float v;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(sc_addr(SC_ROW_D, e)));
                return v;
            }
            return a.deltas[sc_e0 + e];
        };
        float st_s_n = 1.f, st_t_n = 0.f;
        if (!st_staged) load_st(0, st_s_n, st_t_n);      // box 0
        float4 s4 = make_float4(1.f, 1.f, 1.f, 1.f), t4 = make_float4(0.f, 0.f, 0.f, 0.f);
        bool failed = false;          // one of this thread's bounded waits gave up (or saw the abort flag)
        int stored = -1;              // last stage whose tcgen05.st was issued and not yet handed over
        auto hand_over = [&]() {      // the pending store has completed: let the MMA warp have the stage
            tmem_st_wait();
            sm100::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) sm100::mbar_arrive(&a_full[stored % NB]);
            stored = -1;
        };
        for (int ks = 0; ks < NK; ++ks) {
            if (ks + PD < NK) {
                // the box of stage ks + PD held stage ks + PD - NI: wait until every warp has those codes in registers
                if (ks + PD >= NI && !__all_sync(0xffffffffu, sm100::mbar_wait(&idx_free[(ks + PD) % NI], (uint32_t)((ks + PD) / NI - 1) & 1u, abort_flag))) {
                    failed = true;
                    break;
                }
                copy_stage(ks + PD);
            }
            if (!__all_sync(0xffffffffu, sm100::mbar_wait(&idx_full[ks % NI], (uint32_t)(ks / NI) & 1u, abort_flag))) {
                failed = true;
                break;
            }
            if (ks == 0) {     // the staged sidecar has landed with the first box: position the cursor
                const int k_first = KS0 * KST;
                while (e_cur < e_end && sc_col(e_cur) < k_first) ++e_cur;
                nc = e_cur < e_end ? sc_col(e_cur) : 0x7fffffff;
            }
            const uint32_t slot = idx_slot(ks % NI);
            const int sb = ks % NB;
#pragma unroll
            for (int h = 0; h < H; ++h) {     // the stage's boxes; unrolled, so that the second box's code loads and lookups
                                              // are scheduled into the first one's patching and store (7 % at 32 tokens)
                const int bx = ks * H + h;            // box number inside this K slice
                float sc, of;
                if (st_staged) {
                    const int ag = KS0 * H + bx;      // == the box's group number
                    if (bx == 0 || (ag & 3) == 0) {
                        const uint32_t hs = st_hole((ag >> 2) & 1, 0, r), ht = st_hole((ag >> 2) & 1, 1, r);
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(s4.x), "=f"(s4.y), "=f"(s4.z), "=f"(s4.w) : "r"(hs));
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(t4.x), "=f"(t4.y), "=f"(t4.z), "=f"(t4.w) : "r"(ht));
                    }
                    const int q = ag & 3;
                    sc = q == 0 ? s4.x : (q == 1 ? s4.y : (q == 2 ? s4.z : s4.w));
                    of = q == 0 ? t4.x : (q == 1 ? t4.y : (q == 2 ? t4.z : t4.w));
                } else {
                    sc = st_s_n; of = st_t_n;
                    if (bx + 1 < NK * H) load_st(bx + 1, st_s_n, st_t_n);
                }
                uint32_t w[8];
                {
                    const uint32_t idx_row = slot + (uint32_t)(h * IDX_BYTES + r * 128);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {     // 16 codes per load: chunk 2 * kq + c of the row, swizzled by the row
                        const uint32_t addr = idx_row + ((uint32_t)((2 * kq + c) ^ (r & 7)) << 4);
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(w[4 * c]), "=r"(w[4 * c + 1]), "=r"(w[4 * c + 2]), "=r"(w[4 * c + 3]) : "r"(addr));
                    }
                }
                if (h == H - 1) {     // the stage's codes are (on their way) in registers: its boxes can be refilled
                    __syncwarp();
                    if (lane == 0) sm100::mbar_arrive(&idx_free[ks % NI]);
                }
                uint32_t out[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const uint32_t a0 = __byte_perm(w[j >> 2], lane_key, 0x7604u | (uint32_t)((j & 3) << 4));
                    const uint32_t a1 = __byte_perm(w[j >> 2], lane_key, 0x7604u | (uint32_t)(((j + 1) & 3) << 4));
                    float v0, v1;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v0) : "r"(a0));
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v1) : "r"(a1));
                    out[j >> 1] = pack_bf16x2(fmaf(v0, sc, of), fmaf(v1, sc, of));
                }
                // sidecar entries of this row inside this box: mine are patched into the packed registers
                // (a jump per entry instead of a dynamically indexed register array), the others skipped
                {
                    const int k_lo = (KS0 * H + bx) * KS + kq * 32;
                    const int k_st = (KS0 * H + bx + 1) * KS;
                    while (nc < k_st) {
                        const int j = nc - k_lo;
                        if (j >= 0 && j < 32) {
                            const int hi = j & 1;
                            const float nd = sc_delta(e_cur);
                            switch (j >> 1) {
                                case 0: out[0] = add_to_half(out[0], hi, nd); break;
                                case 1: out[1] = add_to_half(out[1], hi, nd); break;
                                case 2: out[2] = add_to_half(out[2], hi, nd); break;
                                case 3: out[3] = add_to_half(out[3], hi, nd); break;
                                case 4: out[4] = add_to_half(out[4], hi, nd); break;
                                case 5: out[5] = add_to_half(out[5], hi, nd); break;
                                case 6: out[6] = add_to_half(out[6], hi, nd); break;
                                case 7: out[7] = add_to_half(out[7], hi, nd); break;
                                case 8: out[8] = add_to_half(out[8], hi, nd); break;
                                case 9: out[9] = add_to_half(out[9], hi, nd); break;
                                case 10: out[10] = add_to_half(out[10], hi, nd); break;
                                case 11: out[11] = add_to_half(out[11], hi, nd); break;
                                case 12: out[12] = add_to_half(out[12], hi, nd); break;
                                case 13: out[13] = add_to_half(out[13], hi, nd); break;
                                case 14: out[14] = add_to_half(out[14], hi, nd); break;
                                default: out[15] = add_to_half(out[15], hi, nd); break;
                            }
                        }
                        ++e_cur;
                        nc = e_cur < e_end ? sc_col(e_cur) : 0x7fffffff;
                    }
                }
                __syncwarp();
                if (h == 0) {
                    // the previous stage's stores have had these lookups to complete
                    if (stored >= 0) hand_over();
                    // the A columns of this ring slot are free once the MMAs that read them NB stages ago have retired
                    // (warp-uniform outcome: the store below is a whole-warp instruction)
                    if (ks >= NB && !__all_sync(0xffffffffu, sm100::mbar_wait(&st_free[sb], (uint32_t)(ks / NB - 1) & 1u, abort_flag))) {
                        failed = true;
                        break;
                    }
                    sm100::tc_fence_after_sync();
                }
                tmem_st_32x16(t_row + (uint32_t)(sb * ACOLS + h * A_COLS), out);
            }
            if (failed) break;
            stored = ks;
        }
        if (stored >= 0) hand_over();
        asm volatile("cp.async.wait_all;" ::: "memory");   // (a loop left early must not retire with copies in flight)

        // ------------------------------------------------------------ epilogue
        // the four warps of a quarter split the token columns
        {
            constexpr int COLS_PER_WARP = BN / 4 < 8 ? 8 : BN / 4;   // 8, 16 or 32 (16 tokens: two of the four warps)
            const int c_lo = kq * COLS_PER_WARP;
            if (!failed && c_lo < BN && sm100::mbar_wait(acc_full, 0u, abort_flag)) {
                sm100::tc_fence_after_sync();
                float* part = a.partial ? a.partial + (int64_t)blockIdx.z * a.M * a.out_features : nullptr;
                const float bias = (a.bias != nullptr && row_ok && part == nullptr) ? a.bias[row] : 0.f;
#pragma unroll 1
                for (int c0 = c_lo; c0 < c_lo + COLS_PER_WARP; c0 += 8) {
                    if (m0 + c0 >= a.M) break;           // warp-uniform
                    uint32_t v[8];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                        : "r"(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c0)
                        : "memory");
                    sm100::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int m = m0 + c0 + j;
                        if (row_ok && m < a.M) {
                            const float acc = __uint_as_float(v[j]);
                            if (part != nullptr) part[(int64_t)m * a.out_features + row] = acc;
                            else store_from_f32(a.y, (int64_t)m * a.ldy + row, acc + bias, a.y_dtype);
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
        sm100::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag == 1 && a.status != nullptr) atomicExch(a.status, HXQ_E_TIMEOUT);
}

}  // namespace gemmts
}  // namespace hxq

namespace hxq {
namespace gemmts {

// ---- host side ---------------------------------------------------------------------

static int sm_count() {
    int n_sm = 148, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n_sm <= 0)
        n_sm = 148;
    return n_sm;
}

static int pick_bn(int M) { return M > 64 ? 128 : (M > 32 ? 64 : (M > 16 ? 32 : 16)); }

// K slices per output tile: enough CTAs to fill the GPU when the row-tile grid alone does not, at
// least four boxes (512 columns) each.  k_boxes: 128-column boxes of the K range.
static int pick_splits(int grid_m, int grid_o, int k_boxes, int n_sm) {
    const int tiles = grid_m * grid_o;
    if (tiles * 2 > n_sm) return 1;
    int s = n_sm / tiles;
    if (s > 8) s = 8;
    if (s > k_boxes / 4) s = k_boxes / 4;
    return s < 1 ? 1 : s;
}

// Largest token count this kernel takes (128); HXQ_GEMM_TS_MAX_M lowers it (0 = never) for A/B timing.
static int max_tokens() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("HXQ_GEMM_TS_MAX_M");
        int n = e ? atoi(e) : 128;
        v = n < 0 ? 0 : (n > 128 ? 128 : n);
    }
    return v;
}

bool covers(const hxq_desc* d, int32_t M) {
    return M >= 1 && M <= max_tokens() && (d->in_features % 16 == 0) && (d->ld_idx % 16 == 0) && aligned_to(d->indices, 16) &&
           (d->col0 % 64 == 0) && (d->group_size == 0 || d->group_size % 64 == 0);
}

size_t split_bytes(const hxq_desc* d, int32_t M) {
    const int BN = pick_bn(M);
    const int s = pick_splits((M + BN - 1) / BN, (d->out_features + BM - 1) / BM, (d->in_features + KS - 1) / KS, sm_count());
    return s > 1 ? (size_t)s * M * d->out_features * sizeof(float) : 0;
}

template <int BN>
static int launch(const CUtensorMap& mx, const Args& a, int grid_m, int grid_o, int splits, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gemm_ts_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) != cudaSuccess)
            return HXQ_E_DEVICE;
        attr_set[dev] = true;
    }
    gemm_ts_kernel<BN><<<dim3(grid_m, grid_o, splits), NUM_THREADS, SMEM_TOTAL, stream>>>(mx, a);
    return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

// xb: the activations as bf16 with a 16-byte aligned row stride (the caller converted them if needed);
// split_ws: room for the fp32 partials (split_bytes) or nullptr.
int run(const hxq_desc* d, const __nv_bfloat16* xb, int64_t ldxb, int32_t M, void* y, int y_dtype, int64_t ldy,
        void* split_ws, size_t split_ws_bytes, int32_t* status_word, cudaStream_t stream) {
    const int BN = pick_bn(M);
    CUtensorMap mx;
    if (!gemm::make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, xb, (uint64_t)d->in_features, (uint64_t)M,
                           (uint64_t)ldxb * 2, 64, (uint32_t)BN, CU_TENSOR_MAP_SWIZZLE_128B))
        return HXQ_E_DEVICE;
    Args a;
    a.cb = d->codebook; a.scales = d->scales; a.offsets = d->offsets;
    a.rowptr = d->rowptr; a.cols = d->cols; a.deltas = d->deltas; a.bias = d->bias;
    a.idx = d->indices; a.ld_idx = d->ld_idx;
    a.y = y; a.status = status_word; a.ldy = ldy;
    a.out_features = d->out_features; a.in_features = d->in_features; a.col0 = d->col0;
    a.group_size = d->group_size; a.ld_st = d->ld_st; a.st_dtype = d->st_dtype;
    a.n_groups = d->group_size > 0 ? (d->col0 + d->in_features - 1) / d->group_size - d->col0 / d->group_size + 1 : 0;
    a.M = M; a.y_dtype = y_dtype;
    const int H = halves_of(BN), k_boxes = (d->in_features + KS - 1) / KS;
    a.k_steps = (k_boxes + H - 1) / H;
    const int grid_o = (d->out_features + BM - 1) / BM;
    const int grid_m = (M + BN - 1) / BN;
    int splits = pick_splits(grid_m, grid_o, k_boxes, sm_count());
    a.k_per_split = a.k_steps;
    a.partial = nullptr;
    if (splits > 1 && split_ws && aligned_to(split_ws, 16) &&
        split_ws_bytes >= (size_t)splits * M * d->out_features * sizeof(float)) {
        const int per_block = 4 / H;      // stages per block of four boxes (scale/offset staging works in such blocks)
        a.k_per_split = ((a.k_steps + splits - 1) / splits + per_block - 1) / per_block * per_block;
        splits = (a.k_steps + a.k_per_split - 1) / a.k_per_split;   // no empty slice
        if (splits > 1) a.partial = reinterpret_cast<float*>(split_ws);
        else a.k_per_split = a.k_steps;                             // one slice after rounding: nothing to split
    } else {
        splits = 1;
    }
    int st;
    if (BN == 128) st = launch<128>(mx, a, grid_m, grid_o, splits, stream);
    else if (BN == 64) st = launch<64>(mx, a, grid_m, grid_o, splits, stream);
    else if (BN == 32) st = launch<32>(mx, a, grid_m, grid_o, splits, stream);
    else st = launch<16>(mx, a, grid_m, grid_o, splits, stream);
    if (st != HXQ_OK || splits == 1) return st;
    gemm::launch_splitk_reduce(a.partial, splits, M, d->out_features, d->bias, y, y_dtype, ldy, stream);
    return cudaGetLastError() == cudaSuccess ? HXQ_OK : HXQ_E_LAUNCH;
}

}  // namespace gemmts
}  // namespace hxq
