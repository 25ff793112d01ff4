/* libmosaicist_sm100a — C ABI of the B200 (sm_100a) block-scaled grouped-GEMM / MoE
 * hot path.
 *
 * The reference project has no native interface for this path: its kernels are Pallas /
 * CuTeDSL programs called from Python capture modules (experiments/loop/*.py).  Each
 * entry point below therefore cites the reference *function* whose arithmetic and
 * argument meaning it replaces.
 *
 * Conventions
 *   - every function returns 0 (MSC_OK) or a negative MSC_ERR_* code and never throws or
 *     exits; msc_last_error() gives a thread-local one-line message for the last failure;
 *   - the caller owns every buffer; all pointers are DEVICE pointers unless a comment
 *     says "host"; the library allocates nothing on the device unless a comment says so;
 *   - `stream` is a cudaStream_t passed as void*; every call that takes one only enqueues
 *     work and never synchronises (msc_status_word_read, which takes none, does);
 *   - device-side waits are bounded: a kernel that gives up records a code in the
 *     library's status word (msc_status_word_read) and leaves the context usable.
 */
#ifndef MOSAICIST_SM100A_H
#define MOSAICIST_SM100A_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSC_OK 0
#define MSC_ERR_BAD_ARG (-1)
#define MSC_ERR_UNSUPPORTED (-2)
#define MSC_ERR_SMEM (-3)
#define MSC_ERR_CUDA (-4)
#define MSC_ERR_TIMEOUT (-5)

/* Epilogue selection for the grouped GEMMs. */
#define MSC_EPI_PLAIN 0       /* out = bf16(alpha[g] * acc)                               */
#define MSC_EPI_ROW_SCALE 1   /* out = bf16(alpha[g] * row_scale[row] * acc)  (routing weight) */

/* Tuning knobs; zero-initialise for library defaults.  The fields mirror the KNOBS the
 * reference's candidate modules expose (experiments/loop/cand_pallas_gemm.py:24-38:
 * block_k / stages / persistent ...), restated for a persistent one-CTA-per-SM kernel. */
typedef struct msc_gemm_cfg {
  int tile_n;    /* CTA tile width: 128 or 256; 0 = default                             */
  int stages;    /* operand ring depth; 0 = as many as shared memory holds              */
  int raster;    /* 0: n-tile fastest inside a group, 1: m-tile fastest                 */
  int max_ctas;  /* persistent grid size; 0 = one CTA per SM                            */
  int epilogue;  /* MSC_EPI_*                                                            */
  int cta_pair;  /* 1: two CTAs share one 256x256 tile (tcgen05 cta_group::2; needs n % 256 == 0,
                    ignores tile_n); 2: one CTA per tile; 3 (row-concatenated groups only): CTA
                    pairs with the weights on the MMA's M side and the tokens on N, so that one
                    tile takes up to 320 rows of a group - the form for groups of a few hundred
                    rows (a routed MoE layer); 0: the library chooses (3 for row-concatenated
                    groups averaging <= 640 rows with n % 256 == 0 and >= 1 KB of K per row, else
                    pairs when n % 256 == 0 and groups have >= 256 rows).  The counterpart
                    of the reference's `collective` knob (cand_pallas_gemm.py:31)          */
  int sf_warps;  /* CTA-pair kernel only. 1: four extra warps write the scale factors into tensor
                    memory (tcgen05.st) instead of the MMA warp copying them (tcgen05.cp);
                    0: the default, copies                                              */
  int reserved;
} msc_gemm_cfg;

int msc_version(void);
const char* msc_last_error(void);

/* Releases what the library caches on the host: the encoded tensor maps, keyed by (address,
 * shape, box).  The library owns no device memory besides two small static arrays (the status
 * word and the planning scratch of msc_moe_plan_noalloc); every buffer belongs to the caller.
 * Call it when no launch is being issued; later calls encode their maps again. */
int msc_shutdown(void);

/* Path of the PTX text of this library's kernels (written next to the .so at build time),
 * so a capture module can drop it where the reference's collect_artifacts looks
 * (src/mosaicist/capture.py:81-116).  Host string, owned by the library. */
const char* msc_ptx_path(void);

/* Reads and clears the device status word of the current device (0 = no kernel gave up).
 * Synchronises the device.  `out` is a host pointer. */
int msc_status_word_read(int* out);

/* NVFP4 masked grouped GEMM:
 *   out[g, r, :] = bf16( alpha[g] * sum_k (a_q*a_sf)[g, r, k] * (b_q*b_sf)[g, :, k] ),  r < masked_m[g]
 * Replaces masked_grouped_gemm / masked_grouped_gemm_w1p
 * (experiments/flashinfer-megamoe-sm100a/masked_gemm.py:104, masked_gemm_ws.py:359) and the
 * FlashInfer call it stands in for (experiments/loop/ref_flashinfer_gemm.py:25-31).
 *   a_q  (l, m, k/2) bytes, two e2m1 per byte, element 2i in the low nibble, K-minor
 *   a_sf (l, m/128, k/64, 32, 16) e4m3, the tiling of nvfp4.py:121-131
 *   b_q  (l, n, k/2), b_sf (l, n/128, k/64, 32, 16)
 *   alpha (l) fp32 or NULL (= 1); masked_m (l) int32 or NULL (= m)
 *   out  (l, m, n) bf16; rows >= masked_m[g] are not written
 * Requires m % 128 == 0, n % tile_n == 0, k % 64 == 0. */
int msc_grouped_gemm_nvfp4(const void* a_q, const void* a_sf, const void* b_q, const void* b_sf,
                           const float* alpha, const int32_t* masked_m, void* out,
                           int l, int m, int n, int k, const msc_gemm_cfg* cfg, void* stream);

/* Same arithmetic over a row-concatenated ("ragged") activation tensor: group g owns rows
 * [group_offsets[g], group_offsets[g] + group_rows[g]) of a_q / out; offsets must be
 * multiples of 128 (the scale tiling is per 128 rows).  row_scale (rows_total) fp32 is read
 * when cfg->epilogue == MSC_EPI_ROW_SCALE.  The reference has no ragged form; this is the
 * layout the skewed-group MXFP8 benchmark (32 groups, Zipf row counts) and the MoE layer
 * use, with per-group semantics as above.
 *   a_q (rows_total, k/2), a_sf (ceil(rows_total/128), k/64, 32, 16), out (rows_total, n) */
int msc_grouped_gemm_nvfp4_ragged(const void* a_q, const void* a_sf, const void* b_q,
                                  const void* b_sf, const float* alpha,
                                  const int32_t* group_offsets, const int32_t* group_rows,
                                  const float* row_scale, void* out, int l, int rows_total,
                                  int n, int k, const msc_gemm_cfg* cfg, void* stream);

/* First expert GEMM with the SwiGLU activation and the requantisation fused into its epilogue:
 *   gateup = bf16(alpha[g] * A w1[g]^T);  act = silu(gate) * up in fp32;  (d_q, d_sf) = NVFP4(act)
 * w1_q (l, n2, k/2) holds the n2/2 gate rows first, then the n2/2 up rows (nvfp4.py:81-88);
 * d_q (rows_total, n2/4) bytes, d_sf tiled (ceil(rows_total/128), n2/128, 32, 16), quantised
 * with out_global_scale[g].  Replaces gemm1_silu_quantize
 * (experiments/flashinfer-megamoe-sm100a/gemm1_silu_quantize.py:94-241) and produces exactly
 * the bytes of msc_grouped_gemm_nvfp4_ragged followed by msc_nvfp4_quantize_ragged(silu=1),
 * without the (rows_total, n2) bf16 round trip.  CTA-pair kernel; n2 % 256 == 0, k % 64 == 0.
 * With cfg->cta_pair == 3 (tokens on N) w1_q / w1_sf must be the interleaved copy made by
 * msc_swiglu_interleave_w1; the result is the same bytes. */
int msc_grouped_gemm_nvfp4_swiglu_ragged(const void* a_q, const void* a_sf, const void* w1_q,
                                         const void* w1_sf, const float* alpha,
                                         const int32_t* group_offsets, const int32_t* group_rows,
                                         const float* out_global_scale, void* d_q, void* d_sf, int l,
                                         int rows_total, int n2, int k, const msc_gemm_cfg* cfg,
                                         void* stream);

/* MXFP8 grouped GEMM (e4m3 values, one ue8m0 scale per 32 K-elements), ragged rows as
 * above.  The nearest reference arithmetic is the Hopper analog's block-scaled FP8 GEMM
 * (experiments/flashinfer-megamoe-sm90a/quant.py:47-75) with the scale format and block
 * size of the MX formats (OCP Microscaling: one power-of-two scale per 32 elements).
 *   a_q (rows_total, k) e4m3, a_sf (ceil(rows_total/128), k/128, 32, 16) ue8m0 (same
 *   128-row tiling, 4 scale columns per chunk), b_q (l, n, k), b_sf (l, n/128, k/128, 32, 16)
 * Requires k % 128 == 0. */
int msc_grouped_gemm_mxfp8_ragged(const void* a_q, const void* a_sf, const void* b_q,
                                  const void* b_sf, const float* alpha,
                                  const int32_t* group_offsets, const int32_t* group_rows,
                                  const float* row_scale, void* out, int l, int rows_total,
                                  int n, int k, const msc_gemm_cfg* cfg, void* stream);

/* NVFP4 quantisation of activations: q = e2m1, one e4m3 scale per 16 K-elements,
 *   sf = e4m3(clip(amax/6 * gs, 0, 448)),  q = e2m1_rne(clip(x / (f32(sf)/gs), -6, 6)).
 * Replaces quantize_nvfp4 (experiments/flashinfer-megamoe-sm100a/nvfp4.py:39-57) and its
 * kernel quantize_nvfp4_pallas (quantize_kernels.py:119-159).
 *   x (l, m, k) bf16 (x_dtype 0) or fp32 (x_dtype 1); global_scale (l) fp32;
 *   masked_m (l) int32 or NULL: rows >= masked_m[g] are skipped;
 *   q (l, m, k/2) bytes; sf either row-major (l, m, k/16) (sf_layout 0, what the reference
 *   kernel writes) or already in the MMA tiling (l, m/128, k/64, 32, 16) (sf_layout 1, which
 *   removes the reference's separate re-tiling pass, moe.py:44).  Requires k % 64 == 0. */
int msc_nvfp4_quantize(const void* x, int x_dtype, const float* global_scale,
                       const int32_t* masked_m, void* q, void* sf, int sf_layout, int l, int m,
                       int k, void* stream);

/* SiLU(gate) * up in fp32 followed by the same quantiser; gate is the first n columns of
 * gateup (l, m, 2n) bf16.  Replaces silu_mul + quantize_nvfp4 (nvfp4.py:81-88, 39-57) and the
 * kernel silu_mul_quantize_nvfp4_pallas (quantize_kernels.py:162-213).  q (l, m, n/2). */
int msc_nvfp4_silu_mul_quantize(const void* gateup, const float* global_scale,
                                const int32_t* masked_m, void* q, void* sf, int sf_layout, int l,
                                int m, int n, void* stream);

/* The same two quantisers over row-concatenated groups (see msc_grouped_gemm_nvfp4_ragged):
 * x (rows_total, k) or, with silu != 0, (rows_total, 2k) bf16; scales always in the MMA tiling
 * (ceil(rows_total/128), k/64, 32, 16).  Rows outside every group are skipped. */
int msc_nvfp4_quantize_ragged(const void* x, int x_dtype, const float* global_scale,
                              const int32_t* group_offsets, const int32_t* group_rows, void* q,
                              void* sf, int l, int rows_total, int k, int silu, void* stream);

/* Per-group global scale of the NVFP4 quantiser: global_scale[g] = numerator / max|x[g]| over the
 * elems_per_group contiguous elements of group g, a maximum of 0 counted as 1.  Replaces
 * global_scale_for (experiments/flashinfer-megamoe-sm100a/nvfp4.py:29-36; numerator = 6 * 448 =
 * 2688 there).  x bf16 (x_dtype 0) or fp32 (1), (l, elems_per_group); elems_per_group % 8 == 0.
 * global_scale (l) fp32 doubles as the reduction's working array: it is cleared, receives the
 * maxima and is then overwritten with the quotients, all on `stream`. */
int msc_amax_global_scale(const void* x, int x_dtype, int l, long long elems_per_group, float numerator,
                          float* global_scale, void* stream);

/* MXFP8 quantisation (OCP Microscaling): q = e4m3, one ue8m0 scale byte per 32 K-elements,
 *   scale = 2^e, e = the smallest integer with blockmax <= 448 * 2^e, clamped to [-127, 127]
 *           (byte e + 127; a block of zeros gets byte 0),
 *   q     = e4m3_rne(clip(x / scale, -448, 448)).
 * The reference has no MXFP8 code; the structure is that of its block-scaled FP8 quantiser
 * (experiments/flashinfer-megamoe-sm90a/quant.py:47-75: scale from the block maximum, q = x /
 * scale clipped to the e4m3 range) with the MX scale rule and block size, and the kernel
 * parallels the NVFP4 one (experiments/flashinfer-megamoe-sm100a/quantize_kernels.py:119-159).
 *   x (rows, k) bf16 (x_dtype 0) or fp32 (1); q (rows, k) bytes; sf row-major (rows, k/32)
 *   (sf_layout 0) or in the MMA tiling (ceil(rows/128), k/128, 32, 16) (sf_layout 1), the form
 *   msc_grouped_gemm_mxfp8_ragged reads.  k % 128 == 0.
 * The ragged form quantises only rows inside a group (group_offsets ascending, multiples of 128)
 * and always writes tiled scales. */
int msc_mxfp8_quantize(const void* x, int x_dtype, void* q, void* sf, int sf_layout, int rows, int k,
                       void* stream);
int msc_mxfp8_quantize_ragged(const void* x, int x_dtype, const int32_t* group_offsets,
                              const int32_t* group_rows, void* q, void* sf, int l, int rows_total, int k,
                              void* stream);

/* Scale-factor re-tiling: (groups, mn, k_scales) row-major bytes -> (groups, ceil(mn/128),
 * k_scales/4, 32, 16) with zero padding rows; element (row = 128t + 32a + b, col = 4c + d)
 * lands at [t, c, b, 4a + d].  Replaces to_mma_scale_layout (nvfp4.py:121-131).  Works for
 * e4m3 and ue8m0 scale bytes alike.  Requires k_scales % 4 == 0. */
int msc_sf_swizzle(const void* sf_rowmajor, void* sf_tiled, int groups, int mn, int k_scales,
                   void* stream);

/* Dense 16-bit GEMM: C(m, n) = A(m, k) * B(k, n), all row-major, fp16 (dtype 0) or bf16
 * (dtype 1) in and out, fp32 accumulation.  The reference's dense benchmark problem
 * (experiments/hopper_gemm/gen_inputs.py:26-27, ref_cutedsl.py:50-74; its kernels are
 * third-party Hopper wgmma code, this is a tcgen05 CTA-pair kernel with 256x256 tiles).
 * lda / ldb / ldc are row pitches in elements, so a column shard of B and C (the N-sharded
 * multi-GPU form) is the shard's base pointer with the parent's pitch.  k, n and the pitches
 * must be multiples of 8; m, n, k need not be tile multiples.  max_ctas 0 = one CTA per SM.
 * Problems with enough columns run 256 x 512 tiles (two MMAs per K step share the A stage, so
 * the kernel is bounded by the tensor pipe rather than by L2 -> SM traffic); a negative max_ctas
 * forces the 256 x 256 form on |max_ctas| CTAs. */
int msc_gemm_f16(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb,
                 int ldc, int dtype, int max_ctas, void* stream);

/* Mixed-dtype grouped GEMM (bf16 activations x int4 weights with bf16 group scales), as two
 * launches.  Semantics of the reference's port of CUTLASS example 69
 * (ports/hopper_mixed_dtype_grouped_gemm/problems.py:1-16, 75-87): dequant(B)[n, k] =
 * bf16(bf16(Bq[n, k]) * scale[n, k / group_size]) with the multiply in bf16, then
 * D_g = alpha_g * A_g dequant(B_g)^T accumulated in fp32.  (The reference never ported the int4
 * variants, ports/.../README.md:95; its kernel is Hopper wgmma code.)
 *   msc_int4_dequant_bf16: q (groups, n, k/2) bytes, two int4 per byte, element 2i in the low
 *     nibble, two's complement [-8, 7]; scales (groups, n, k/group_size) bf16 -> out (groups, n, k) bf16.
 *   msc_grouped_gemm_bf16_ragged: a (rows_total, k) bf16, row-concatenated groups as in
 *     msc_grouped_gemm_nvfp4_ragged; b (l, n, k) bf16 K-contiguous; alpha (l) f32 or NULL;
 *     out (rows_total, n) bf16.  n % 256 == 0, k % 8 == 0. */
int msc_int4_dequant_bf16(const void* q, const void* scales, void* out, int groups, int n, int k,
                          int group_size, void* stream);
int msc_grouped_gemm_bf16_ragged(const void* a, const void* b, const float* alpha,
                                 const int32_t* group_offsets, const int32_t* group_rows, void* out,
                                 int l, int rows_total, int n, int k, int max_ctas, void* stream);
/* The two calls above as one kernel (the reference's problem statement dequantises inside the
 * GEMM, problems.py:84-87): b_q (l, n, k/2) packed int4 and scales (l, n, k/group_size) bf16 are
 * read once; converter warps expand each 64-element K stage to bf16(q) * scale in shared memory
 * for the tensor core.  Same bits as the two-call path.  n % 256 == 0, k % 64 == 0,
 * group_size % 64 == 0 and dividing k (MSC_ERR_UNSUPPORTED otherwise). */
int msc_grouped_gemm_bf16_int4_ragged(const void* a, const void* b_q, const void* scales,
                                      const float* alpha, const int32_t* group_offsets,
                                      const int32_t* group_rows, void* out, int l, int rows_total,
                                      int n, int k, int group_size, int max_ctas, void* stream);

/* ---- MoE routing and token movement ---------------------------------------------------
 * The reference's MoE takes per-expert padded batches and has no routing, permutation or
 * exchange code (experiments/flashinfer-megamoe-sm100a/moe.py:47-79; the only hint is that
 * the per-expert alphas "are the routing weights", flashinfer-megamoe-sm90a/moe.py:69).
 * These entry points build, from router logits, the row-concatenated 128-aligned group
 * layout the *_ragged GEMMs consume, and fold the expert outputs back per token. */

/* softmax over `experts` (multiple of 32, <= 1024), the `topk` (<= 32) largest, weights
 * renormalised to sum to 1; ties go to the lower expert index.
 * logits (tokens, experts) f32 -> ids (tokens, topk) i32, weights (tokens, topk) f32. */
int msc_moe_route_topk(const float* logits, int32_t* ids, float* weights, int tokens, int experts,
                       int topk, void* stream);

/* For the experts [expert_first, expert_first + experts_local): rows per expert, the rank of
 * every (token, k) pair inside its expert (token order), and 128-aligned group offsets.
 * ids (entries) i32 with entries = tokens * topk; rank (entries) i32 is written only where the
 * pair is routed to a local expert; group_rows, group_offsets (experts_local); total_rows (1):
 * the padded row count.  scratch: one int32 of device memory, zero before the first call,
 * left zero by every call (a ticket counter; calls sharing it must not overlap). */
int msc_moe_plan(const int32_t* ids, int entries, int expert_first, int experts_local,
                 int32_t* rank, int32_t* group_rows, int32_t* group_offsets, int32_t* total_rows,
                 int32_t* scratch, void* stream);

/* msc_moe_plan for callers that cannot allocate device memory (a serving loop whose pool is
 * frozen, a plugin inside a framework that owns all allocations): the ticket counter lives
 * in a 4352-byte array built into the library, and so do the row counts / total when
 * group_rows / total_rows are NULL.  No counterpart in the reference.  Limits and rules:
 *   - experts_local <= 1024, larger values are rejected with MSC_ERR_BAD_ARG;
 *   - the library never calls an allocator here; the first call on a device looks up the
 *     array's device address (cudaGetSymbolAddress), so make that first call outside any
 *     stream capture;
 *   - all calls on a device share the one array (it keeps the last call's counts): two calls
 *     that overlap on the GPU race, even on different streams. */
int msc_moe_plan_noalloc(const int32_t* ids, int entries, int expert_first, int experts_local,
                         int32_t* rank, int32_t* group_rows, int32_t* group_offsets,
                         int32_t* total_rows, void* stream);

/* Gathers each locally routed token row (tokens (tokens, hidden) bf16), quantises it to NVFP4
 * with its expert's global scale (arithmetic of quantize_nvfp4, nvfp4.py:39-57) and writes it
 * at row group_offsets[e] + rank: a_q (rows_cap, hidden/2), a_sf tiled
 * (rows_cap/128, hidden/64, 32, 16), plus row_weight (rows_cap) f32 = the pair's routing weight
 * and row_token (rows_cap) i32.  rows_cap is a multiple of 128 >= total_rows.  hidden % 64 == 0,
 * topk <= 64, a_q 16-byte aligned (rows leave shared memory as bulk copies).
 * sf_rows (rows_cap, hidden/16) u8 or NULL: staging for the scales.  With it (hidden % 256 == 0,
 * rows_cap a multiple of 128, both scale buffers 16-byte aligned) every row's scale bytes leave
 * as one bulk copy into sf_rows and a second kernel re-tiles them into a_sf - about 40 % less
 * time at top-8 than writing the tiling word by word; total_rows (device, i32, or NULL) is
 * the row count msc_moe_plan produced and bounds that pass, padding rows inside it receive
 * whatever sf_rows held.  Without it rows_cap and total_rows are ignored. */
int msc_moe_permute_quantize(const void* tokens_bf16, const int32_t* ids, const float* weights,
                             const int32_t* rank, const int32_t* group_offsets,
                             const float* input_gs, int tokens, int hidden, int topk,
                             int expert_first, int experts_local, void* a_q, void* a_sf,
                             float* row_weight, int32_t* row_token, void* sf_rows, int rows_cap,
                             const int32_t* total_rows, void* stream);

/* out[token] = bf16( sum over k (ascending, fp32) of y[group_offsets[e] + rank] ) over the
 * pairs routed to local experts; y (rows_cap, hidden) bf16, out (tokens, hidden) bf16;
 * topk <= 64. */
int msc_moe_unpermute(const void* y, const int32_t* ids, const int32_t* rank,
                      const int32_t* group_offsets, void* out, int tokens, int hidden, int topk,
                      int expert_first, int experts_local, void* stream);

/* w1 for the tokens-on-N form of msc_grouped_gemm_nvfp4_swiglu_ragged: gate and up rows
 * interleaved in blocks of 64, so that every 128 consecutive rows hold both halves of 64 output
 * columns - out row 128 i + j is gate row 64 i + j for j < 64, up row n2/2 + 64 i + j - 64
 * otherwise - and the tiled scales permuted alike.  Done once when the weights are loaded; not
 * in place.  w1_q / out_q (l, n2, k/2), w1_sf / out_sf (l, n2/128, k/64, 32, 16). */
int msc_swiglu_interleave_w1(const void* w1_q, const void* w1_sf, void* out_q, void* out_sf, int l,
                             int n2, int k, void* stream);

/* msc_grouped_gemm_nvfp4_ragged whose result rows are scattered instead of stored in place:
 * row r (times alpha and, if given, row_scale[r]) goes to
 * dest_bases[code >> 26] + (code & 0x3ffffff) * n bf16 with code = row_dest[r] (rows_total) i32;
 * rows with a negative code are skipped.  dest_bases is a host array of dest_count (<= 16)
 * device pointers to dest_rows rows of n bf16 each; a code that names a destination >= dest_count
 * or a row >= dest_rows is not stored and raises bit 0x00C00000 in the status word (the codes
 * are written by other ranks: reset row_dest to -1 between steps so a row nobody wrote in this
 * step is skipped).  The destinations may be other GPUs' mapped memory: each row leaves as untiled 256-byte
 * bulk copies (cp.async.bulk shared -> global), never as a tiled or multicast operation.  The
 * MoE's second GEMM uses it to deliver every result row to the token's home rank while the
 * GEMM is still running.  No counterpart in the reference.  n % 256 == 0, k % 64 == 0. */
int msc_grouped_gemm_nvfp4_scatter_ragged(const void* a_q, const void* a_sf, const void* b_q,
                                          const void* b_sf, const float* alpha,
                                          const int32_t* group_offsets, const int32_t* group_rows,
                                          const float* row_scale, const int32_t* row_dest,
                                          void* const* dest_bases, int dest_count, int dest_rows,
                                          int l, int rows_total, int n, int k,
                                          const msc_gemm_cfg* cfg, void* stream);

/* ---- expert-parallel exchange over peer memory --------------------------------------------
 * No counterpart in the reference, which runs on one GPU; the partitioning is the one its
 * benchmark configuration names (experts split over the GPUs of one box, token dispatch and
 * combine between them).  Rank r owns the experts [r * E / world, (r + 1) * E / world) and the
 * buffers a_q / sf_rows / row_weight / y of `rows_cap` rows (a multiple of 128): packed
 * values and result rows as its grouped GEMMs read and write them, scale bytes row-major
 * (rows_cap, hidden/16).  Every rank maps every other rank's buffers (msc_peer_*).  Per layer:
 * msc_moe_plan over all E experts (counts + position of each pair), an all-gather of the
 * counts, msc_ep_offsets, msc_ep_dispatch_quantize, a barrier, msc_sf_swizzle of the received
 * scale rows into the MMA tiling, the local GEMMs, a barrier, msc_ep_combine.  The barriers and
 * the all-gather are either the caller's collectives (NCCL, stream-ordered) or this library's
 * flags (msc_ep_signal / msc_ep_wait below).  A destination row at or beyond rows_cap is
 * never stored: the pair is dropped, its pair_row set to -1 and bit 0x00E00000 raised in the
 * status word (msc_status_word_read). */

/* cudaMalloc + cudaIpcGetMemHandle: *ptr is this process's pointer, handle64 receives the 64
 * bytes another process of the same box passes to msc_peer_open.  msc_peer_close unmaps an
 * opened pointer, msc_peer_free releases an allocated one (after every peer closed it). */
int msc_peer_alloc(size_t bytes, void** ptr, void* handle64);
int msc_peer_open(const void* handle64, void** ptr);
int msc_peer_close(void* ptr);
int msc_peer_free(void* ptr);

/* counts_all (world, experts_total) i32: pairs each rank routes to each expert.  Writes
 * send_base (experts_total): the first row of this rank's pairs of expert e in the owner's
 * buffers (owner's 128-aligned group offset + the pairs of lower ranks), and this rank's own
 * group table group_rows / group_offsets (experts_total / world), total_rows (1).  With
 * wait_flags (or NULL) the kernel first waits for the peers' flags of wait_slot to reach
 * wait_epoch (see msc_ep_wait): the counts were written by the peers' msc_ep_signal. */
int msc_ep_offsets(const int32_t* counts_all, int world, int rank, int experts_total, int rows_cap,
                   int32_t* send_base, int32_t* group_rows, int32_t* group_offsets,
                   int32_t* total_rows, const int32_t* wait_flags, int wait_slot, int wait_epoch,
                   void* stream);

/* Signalling between ranks without a collective.  Every rank owns a flag table of 4 slots x 16
 * ints (zero at start) in memory its peers have mapped.  msc_ep_signal raises this rank's flag
 * of `slot` to `epoch` on every peer (peer_flags: host array of `world` table pointers) after a
 * system-scope fence; launched after the kernels whose peer-memory writes it announces, it
 * makes them visible to a peer that then sees the flag.  With `counts` (experts_total) i32 it
 * first copies them into row `rank` of every peer's counts table (peer_counts_all: host array
 * of pointers to (world, experts_total) i32) - the all-gather of the per-expert counts.
 * msc_ep_wait (or msc_ep_offsets with wait_flags) waits until all `world` flags of `slot` in
 * this rank's own table have reached `epoch`: a bounded spin on local memory (one second), after
 * which bit 0x00D00000 is raised in the status word and the kernel returns.  Epochs must
 * increase from call to call.  Never run a wait before the matching signals when several
 * ranks share one GPU: launches of one device do not overlap reliably. */
int msc_ep_signal(int32_t* const* peer_flags, int world, int rank, int slot, int epoch,
                  const int32_t* counts, int32_t* const* peer_counts_all, int experts_total,
                  void* stream);
int msc_ep_wait(const int32_t* flags, int world, int slot, int epoch, void* stream);

/* msc_moe_permute_quantize across ranks: pair (token, k) with global expert e is quantised with
 * input_gs[e] (experts_total) and stored at row send_base[e] + rank_in_group[pair] of rank
 * e / (experts_total / world)'s a_q / sf_rows / row_weight, given as host arrays of `world`
 * device pointers.  pair_row (tokens, topk) i32 receives that row for msc_ep_combine.  With
 * peer_row_dest (host array of `world` pointers to (rows_cap) i32, or NULL) the owner also
 * learns where the row's result belongs: code (rank << 26) | (token * topk + k), the form
 * msc_grouped_gemm_nvfp4_scatter_ragged takes.  With peer_row_next as well (same shape, or
 * NULL; needs peer_row_dest, hidden % 256 == 0, topk <= 32) a token's rows on one owner are
 * chained in pair order for msc_ep_presum_push: row_next holds the next row of the chain or -1,
 * only the chain's first row keeps its code, the others get -2 there and in pair_row. */
int msc_ep_dispatch_quantize(const void* tokens_bf16, const int32_t* ids, const float* weights,
                             const int32_t* rank_in_group, const int32_t* send_base,
                             const float* input_gs, int tokens, int hidden, int topk,
                             int experts_total, int world, void* const* peer_a_q,
                             void* const* peer_sf_rows, float* const* peer_row_weight,
                             int32_t* const* peer_row_dest, int32_t* const* peer_row_next, int rank,
                             int rows_cap, int32_t* pair_row, void* stream);

/* The combine with a token's results pre-summed on every rank they were computed on: for each
 * local row r whose row_dest[r] >= 0 (the first row of a chain), bf16( sum in fp32, in chain
 * order, of y[r], y[row_next[r]], ... ) is written to dest_bases[code >> 26] at row
 * code & 0x3ffffff (codes outside dest_count / dest_rows are refused with status bit
 * 0x00C00000).  y (rows, hidden) bf16 is what the second GEMM stored locally (routing weights
 * applied); msc_ep_sum_pairs on the home rank then adds one row per rank the token visited.
 * About a third fewer rows cross NVLink than with msc_grouped_gemm_nvfp4_scatter_ragged under
 * uniform top-8 routing over 8 ranks; the transfer does not overlap the GEMM, and the result
 * differs from the single-GPU layer by one extra bf16 rounding per rank. */
int msc_ep_presum_push(const void* y, const int32_t* row_dest, const int32_t* row_next,
                       void* const* dest_bases, int dest_count, int dest_rows, int rows, int hidden,
                       void* stream);

/* out[token] = bf16( sum over k (ascending, fp32) of y_owner[pair_row] ), reading each owner's
 * y (rows_cap, hidden) bf16 through `peer_y` (host array of `world` device pointers). */
int msc_ep_combine(const void* const* peer_y, const int32_t* ids, const int32_t* pair_row, void* out,
                   int tokens, int hidden, int topk, int experts_total, int world, int rows_cap,
                   void* stream);

/* out[token] = bf16( sum over k (ascending, fp32) of y_pairs[token * topk + k] ): the last step
 * when the second GEMM scattered every pair's result row to the token's home rank.
 * y_pairs (tokens * topk, hidden) bf16, out (tokens, hidden) bf16.  pair_row (tokens, topk) i32
 * or NULL: pairs marked negative by msc_ep_dispatch_quantize (dropped because the owner's
 * buffers were full) are left out of the sum; their row of y_pairs holds stale data.
 * topk <= 64. */
int msc_ep_sum_pairs(const void* y_pairs, const int32_t* pair_row, void* out, int tokens, int hidden,
                     int topk, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOSAICIST_SM100A_H */
