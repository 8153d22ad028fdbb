/*
 * hxq_b200.h - C ABI of libhxq_b200.so: the HXQ compressed-linear forward path
 * (uint8 indices into a 256-entry fp32 codebook, optional per-group affine
 * scale/offset, sparse outlier sidecar) as hand-written sm_100a CUDA kernels.
 *
 * Weight definition shared by every entry point (o = output row, i = local
 * input column of this shard):
 *
 *     W^[o, i] = cb[idx[o, i]] * s[o, g(i)] + t[o, g(i)],
 *     g(i)     = (col0 + i) / group_size - col0 / group_size
 *
 * with s == 1, t == 0 when group_size == 0.  Matrix products add the sidecar
 * as deltas (value - W^ at that position); hxq_dequant overwrites with values.
 *
 * Conventions: every pointer in hxq_desc and every x / y / out / workspace
 * pointer is a DEVICE pointer borrowed for the duration of the call; nothing
 * is allocated, freed or synchronised inside the library (except where an
 * entry point says otherwise); kernels are enqueued on the caller's stream.
 * All entry points return 0 on success or a negative HXQ_E_* code and never
 * throw, trap or abort.
 */
#ifndef HXQ_B200_H_
#define HXQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define HXQ_OK            0
#define HXQ_E_ARG        -1  /* null pointer / bad enum / bad M                    */
#define HXQ_E_SHAPE      -2  /* shape the kernels do not cover                     */
#define HXQ_E_ALIGN      -3  /* pointer or leading dimension not aligned as stated  */
#define HXQ_E_DTYPE      -4  /* unsupported element type                           */
#define HXQ_E_DEVICE     -5  /* CUDA runtime error before launch (device, attrs)   */
#define HXQ_E_LAUNCH     -6  /* kernel launch failed                               */
#define HXQ_E_TIMEOUT    -7  /* a bounded device-side wait gave up                 */
#define HXQ_E_WORKSPACE  -8  /* workspace missing or too small                     */

/* element types of x, y, out, scales/offsets */
#define HXQ_F32   0
#define HXQ_F16   1
#define HXQ_BF16  2

typedef void* hxq_stream_t; /* a cudaStream_t */

/*
 * One compressed weight matrix (or a tensor-parallel shard of one).
 * Replaces the buffer set of the reference module HelixLinear
 * (helix_substrate/helix_linear.py:166-239: codebook, indices,
 * _sidecar_rows/_cols/_deltas, bias) and the scales/offsets arguments of
 * fused_affine_group_matmul (helix_substrate/triton_affine_group_matmul.py:301-308).
 */
typedef struct hxq_desc {
    int32_t out_features;  /* rows of this shard                                          */
    int32_t in_features;   /* columns of this shard                                       */
    int32_t col0;          /* global column of local column 0 (row-parallel shards), else 0 */
    int32_t group_size;    /* affine group length along the input dim, 0 = no affine      */
    int64_t ld_idx;        /* row stride of indices in bytes (>= in_features)             */
    const uint8_t* indices;/* [out_features, ld_idx] uint8                                */
    const float* codebook; /* [256] fp32                                                  */
    const void* scales;    /* [out_features, ld_st] of st_dtype, NULL when group_size==0  */
    const void* offsets;   /* same layout as scales                                       */
    int32_t st_dtype;      /* HXQ_F32 or HXQ_F16                                          */
    int32_t ld_st;         /* row stride of scales/offsets in elements                    */
    const int32_t* rowptr; /* [out_features+1] CSR row pointer of the sidecar, NULL = none */
    const int32_t* cols;   /* [nnz] local column of each sidecar entry, row-sorted        */
    const float* deltas;   /* [nnz] value - W^ at the position (used by gemv / gemm)      */
    const float* values;   /* [nnz] exact value at the position (used by dequant)         */
    const float* bias;     /* [out_features] fp32 or NULL                                 */
} hxq_desc;

/* Library version as major*10000 + minor*100 + patch. */
int hxq_version(void);

/*
 * hxq_gemv / hxq_gemv_static start their set-up (codebook table, first index rows, scale / offset /
 * row-pointer reads) BEFORE the kernels in front of them on the stream have finished (programmatic
 * dependent launch) and only wait for those kernels before they touch x, y and the workspace.
 * PRECONDITION: every buffer named in the hxq_desc is complete before the call is enqueued - which
 * is the case for weights loaded once.  A caller that produces a descriptor's buffers with kernels
 * on the SAME stream right before the product (a codebook computed per call, indices unpacked per
 * call) brackets the call with hxq_set_weights_on_stream(1) ... (0): while set (per host thread),
 * the products launch as ordinary stream-ordered kernels.  No counterpart in the reference.
 */
void hxq_set_weights_on_stream(int on);

/* Static, human-readable text for a status code. */
const char* hxq_strerror(int status);

/*
 * Dequantise rows [row0, row1) to out[(row - row0) * ld_out + i].
 * out_dtype HXQ_F32 is bit-exact with CDNAv3Reader.reconstruct() /
 * reconstruct_block() (helix_substrate/hxq_reader_v3.py:102-187): codebook
 * gather, then the sidecar VALUE overwrites the entry.  HXQ_BF16 / HXQ_F16
 * round that fp32 result once.  Also serves HelixLinear.decode_weight /
 * _dequant_tile (helix_substrate/helix_linear.py:735-781,881-888) and the
 * "buffered" materialisation (helix_linear.py:556-634).
 */
int hxq_dequant(const hxq_desc* d, int32_t row0, int32_t row1,
                void* out, int out_dtype, int64_t ld_out, hxq_stream_t stream);

/*
 * Bytes of zero-initialised device workspace hxq_gemv needs for this shape
 * (split-K partial sums and arrival counters).  The workspace must be zero
 * before its first use; hxq_gemv leaves the counters zero again on return, so
 * one workspace can be reused by successive calls on the same stream.  Calls
 * that may overlap on the GPU need separate workspaces.
 */
size_t hxq_gemv_workspace_bytes(const hxq_desc* d, int32_t M);

/*
 * Decode-time product for M <= 16 tokens:  y[m, o] = sum_i x[m, i] * W^[o, i]
 * + sidecar + bias, fp32 accumulation, result rounded once to y_dtype.
 * Replaces fused_vq_matmul at N <= 16 (helix_substrate/triton_vq_matmul.py:521-727:
 * _vq_decode_dotprod_kernel + _sidecar_fused_kernel + bias) and
 * fused_affine_group_matmul's decode kernel
 * (helix_substrate/triton_affine_group_matmul.py:112-177,301-363).
 * x is [M, ldx] of x_dtype, y is [M, ldy] of y_dtype (strides in elements).
 */
int hxq_gemv(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx,
             void* y, int y_dtype, int64_t ldy,
             void* workspace, size_t workspace_bytes, hxq_stream_t stream);

/*
 * hxq_gemv without a caller-provided workspace (no counterpart in the reference:
 * its operators allocate freely through torch).  For hosts that may not call
 * the CUDA allocator where they run the product - a serving process that gave
 * all device memory to its own pool at start-up, a plug-in that only ever
 * receives input and output buffers.  The scratch is an array of
 * HXQ_GEMV_STATIC_SCRATCH_BYTES inside the library, present once on every GPU
 * that loads it, for as long as the process lives.
 *   - Shapes whose scratch need (hxq_gemv_workspace_bytes) exceeds that size are
 *     refused with HXQ_E_WORKSPACE before anything is launched.  2 MiB covers
 *     every Qwen2.5-7B/14B projection at M <= 16.
 *   - The first call on a device looks the array's device address up
 *     (cudaGetSymbolAddress); make that call once outside any stream capture.
 *   - All calls on one GPU share the array; it is cleared on the stream as far
 *     as the call needs it, so calls that can overlap on the GPU must not both
 *     use this entry point (use hxq_gemv with separate workspaces there).
 *   - Nothing is allocated or freed, by this library or by anything it calls.
 * Same arguments and result as hxq_gemv otherwise.
 */
#define HXQ_GEMV_STATIC_SCRATCH_BYTES (2u << 20)
int hxq_gemv_static(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx,
                    void* y, int y_dtype, int64_t ldy, hxq_stream_t stream);

/*
 * Decode-time product over 6-bit packed indices, M <= 16: four codes in three bytes
 * (b0 | b1 << 8 | b2 << 16 holds v0..v3 from the low bits up), unpacked inside the kernel, the
 * code itself being the value:  y[m, o] = sum_i x[m, i] * (code[o, i] * s[o, i / G] + t[o, i / G])
 * + bias.  Replaces fused_affine_group_matmul_packed6 / _affine_group_packed6_kernel
 * (helix_substrate/triton_affine_group_matmul.py:180-298; the reference serves one token only).
 * packed: [out_features, in_features * 3 / 4] bytes, 4-byte aligned; in_features and group_size
 * multiples of 16; scales / offsets [out_features, ld_st] of st_dtype (HXQ_F32 or HXQ_F16).
 */
int hxq_gemv_packed6(const uint8_t* packed, int32_t out_features, int32_t in_features,
                     const void* scales, const void* offsets, int st_dtype, int32_t ld_st,
                     int32_t group_size, const float* bias, const void* x, int x_dtype, int32_t M,
                     int64_t ldx, void* y, int y_dtype, int64_t ldy, hxq_stream_t stream);

/*
 * Prefill-time product for any M (meant for M >= 17):  same contract as
 * hxq_gemv but weights are dequantised to bf16 and contracted on the tcgen05
 * tensor cores with fp32 TMEM accumulators: up to 128 tokens the dequantised
 * tile goes to the MMA through tensor memory (one thread per output row), above
 * that through 128-byte swizzled shared-memory tiles.
 * Replaces fused_vq_matmul at N > 16 (_vq_gather_matmul_tiled_kernel,
 * helix_substrate/triton_vq_matmul.py:249-334,634-661, + scatter_add sidecar
 * :693-698) and _affine_group_tiled_kernel
 * (helix_substrate/triton_affine_group_matmul.py:32-109).
 * status_word: device int32 the kernel sets non-zero if a bounded wait gave
 * up (the host reads it after synchronising); may be NULL.
 * The workspace of hxq_gemm is plain scratch (a bf16 copy of x when x is not
 * bf16 or not 16-byte aligned): it need not be zeroed and is left dirty, so it
 * must not double as an hxq_gemv workspace.  When the output tile grid alone cannot fill
 * the GPU (one token tile and few row tiles, e.g. down_proj at M = 32) the K range is split over
 * CTAs and their fp32 partial products, also in the workspace, are added in fixed order by
 * a second launch; with a workspace too small for them the call runs unsplit.  Shapes the tensor-core kernel does
 * not cover (ragged or unaligned) run through the decode kernels; the call
 * clears the part of the workspace they need first.
 */
size_t hxq_gemm_workspace_bytes(const hxq_desc* d, int32_t M);
int hxq_gemm(const hxq_desc* d, const void* x, int x_dtype, int32_t M, int64_t ldx,
             void* y, int y_dtype, int64_t ldy,
             void* workspace, size_t workspace_bytes, int32_t* status_word,
             hxq_stream_t stream);

/*
 * ---- decode-step glue (bf16): the small operators between the compressed linears ----
 * The reference decodes with a stock HF Qwen2 forward per token
 * (helix_substrate/basin_runtime.py:358-445: model(...) inside a Python greedy loop), i.e.
 * dozens of framework element-wise launches per layer around the linears.  These four
 * entry points are those operators as one launch each, so that a decode step is
 * 13 launches per layer.  All tensors bf16 unless noted, strides in elements, the
 * decode position read from DEVICE memory (int64) so a captured step can be replayed.
 */

/* h[b,:] += delta[b,:] (skipped if delta is NULL), then out[b,:] = rmsnorm(h[b,:]) * weight,
 * fp32 statistics, rounded to bf16 before and after the weight product like
 * Qwen2RMSNorm (reference models: transformers' modeling_qwen2, driven by
 * helix_substrate/basin_runtime.py:281-330).  H <= 12000. */
int hxq_add_rmsnorm(void* h, const void* delta, const void* weight, void* out, int32_t B, int32_t H,
                    int64_t ld_h, int64_t ld_delta, int64_t ld_out, float eps, hxq_stream_t stream);

/* qkv[b, :] holds the new token's nq query heads, then nkv key heads, then nkv value heads
 * (D each).  Applies the rotary embedding (rotate-half convention, cos/sin fp32 tables
 * [max_len, D]) to q and k at row *pos, writes q to q_out[b, nq*D] and appends k, v to the
 * caches [B, nkv, max_len, D] at row *pos. */
int hxq_rope_append(const void* qkv, int64_t ld_qkv, const int64_t* pos, const float* cos_table,
                    const float* sin_table, void* q_out, int64_t ld_q, void* k_cache, void* v_cache,
                    int32_t B, int32_t nq, int32_t nkv, int32_t D, int32_t max_len, hxq_stream_t stream);

/* Single-query grouped attention over cache rows 0..*pos: out[b, h*D + d] =
 * softmax_p(scale * q[b,h,:] . K[b, h / (nq/nkv), p, :]) V[...].  D <= 128, D % 8 == 0,
 * nq / nkv <= 8.  workspace: hxq_attn_decode_workspace_bytes() of plain scratch. */
size_t hxq_attn_decode_workspace_bytes(int32_t B, int32_t nq, int32_t D, int32_t max_len);
int hxq_attn_decode(const void* q, int64_t ld_q, const void* k_cache, const void* v_cache, const int64_t* pos,
                    void* out, int64_t ld_out, void* workspace, size_t workspace_bytes, int32_t B, int32_t nq,
                    int32_t nkv, int32_t D, int32_t max_len, float scale, hxq_stream_t stream);

/* out[b, i] = silu(gate[b, i]) * up[b, i], i < n (the MLP between gate/up and down). */
int hxq_swiglu(const void* gate, const void* up, void* out, int32_t B, int32_t n, int64_t ld_gate,
               int64_t ld_up, int64_t ld_out, hxq_stream_t stream);

/* y[m, o] = sum_i x[m, i] * weight[o, i] for a DENSE bf16 weight [out_features, ldw] and up to four
 * tokens of bf16 activations: the decoder's lm_head at decode time, which the reference keeps dense
 * (helix_substrate/tensor_policy.py:199-208) and runs as its _BF16Linear
 * (helix_substrate/basin_runtime.py:181-205).  in_features % 8 == 0 and <= 12288, ldw % 8 == 0,
 * weight 16-byte aligned; y fp32, fp16 or bf16; fp32 accumulation.  The weight must be complete
 * before the previous kernel on the stream started (it is fetched while that kernel drains). */
int hxq_dense_gemv(const void* weight, int32_t out_features, int32_t in_features, int64_t ldw, const void* x,
                   int32_t M, int64_t ldx, void* y, int y_dtype, int64_t ldy, hxq_stream_t stream);

/*
 * ---- tensor-parallel sum after a row-parallel product, decode-sized messages ----
 * No counterpart in the reference (it has no multi-GPU path); replaces what
 * torch.distributed.all_reduce (NCCL) would do after o_proj / down_proj.  One kernel per
 * rank over peer memory: every rank pushes its fp32 partial sums into every rank's receive
 * buffer with plain peer stores, raises a flag, waits (bounded) for all ranks' flags in its
 * own buffer and adds the partials from local memory in rank order, rounding once to bf16:
 * the result is bit-identical on every rank and from run to run.
 *   peer_buffers[p], peer_flags[p]: HOST arrays of `world` DEVICE pointers, rank p's receive
 *     buffer (hxq_allreduce_buffer_bytes, 16-byte aligned) and flag array
 *     (hxq_allreduce_flag_bytes), both zero before the first call and mapped into this
 *     process (symmetric / IPC memory); the same n_max on every rank, n_max % 8 == 0.
 *   src: this rank's partial sums, fp32 [n], n <= n_max, n <= 131072; dst: bf16 [n].
 *   counters: 32 x uint32 of this rank's own device memory, zero before the first call;
 *     the kernel advances them, so a captured graph can be replayed.
 *   wait_cycles: limit of the flag wait in SM clock cycles (0 = about one second); on
 *     expiry *status (device int32, may be NULL) is set to HXQ_E_TIMEOUT and dst is left
 *     untouched.  Every rank must make the same sequence of calls.
 */
size_t hxq_allreduce_buffer_bytes(int32_t world, int64_t n_max);
size_t hxq_allreduce_flag_bytes(int32_t world);
int hxq_allreduce_oneshot(void* const* peer_buffers, void* const* peer_flags, int32_t rank, int32_t world,
                          int64_t n_max, const void* src, void* dst, int64_t n, void* counters,
                          int64_t wait_cycles, int32_t* status, hxq_stream_t stream);

/*
 * hxq_allreduce_oneshot with the next two steps of a decoder layer folded in (same buffers, flags,
 * counters, bounded wait and status word; no counterpart in the reference): after the sum over
 * ranks of src [M, H] (fp32 partials of a row-parallel o_proj / down_proj),
 *     delta = bf16(sum);   h[m, :] = bf16(h + delta);   out[m, :] = rmsnorm(h[m, :], eps) * weight
 * rounded exactly where hxq_allreduce_oneshot followed by hxq_add_rmsnorm round.  h, out: bf16
 * [M, ld]; weight: bf16 [H]; H <= 8192; M * H <= n_max.  One CTA owns whole rows, so calls of this
 * entry point and of hxq_allreduce_oneshot must not share one set of buffers / flags / counters.
 */
int hxq_allreduce_add_rmsnorm(void* const* peer_buffers, void* const* peer_flags, int32_t rank, int32_t world,
                              int64_t n_max, const void* src, int32_t M, int32_t H, void* h, int64_t ld_h,
                              const void* weight, void* out, int64_t ld_out, float eps, void* counters,
                              int64_t wait_cycles, int32_t* status, hxq_stream_t stream);

/*
 * Host helper: CSR row pointer from ascending flat positions
 * (rows = pos / in_features), the derivation HelixLinear does at load
 * (helix_substrate/helix_linear.py:196-203,960-997).  positions, rowptr and
 * cols are HOST pointers; rowptr has out_features+1 entries, cols nnz entries.
 * Fails with HXQ_E_ARG if positions are not strictly ascending or out of range.
 */
int hxq_csr_from_positions(const int64_t* positions, int64_t nnz,
                           int32_t out_features, int32_t in_features,
                           int32_t* rowptr, int32_t* cols);

#ifdef __cplusplus
}
#endif
#endif /* HXQ_B200_H_ */
