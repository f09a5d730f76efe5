/* C-ABI of the B200 (sm_100a) low-precision DINOv3 ViT + EoMT inference hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), launches on that stream and
 * returns without synchronising: 0 = ok, negative = bad argument (see kf_last_error_string), positive = the
 * cudaError_t of a failed launch.  The caller owns every buffer and nothing here allocates device memory.  One thread
 * per device may call concurrently.
 *
 * Each declaration cites the reference interface it replaces (paths relative to the reference checkout).
 */
#ifndef KF_B200_H
#define KF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KF_API __attribute__((visibility("default")))
#else
#define KF_API
#endif

/* status codes */
#define KF_OK 0
#define KF_ERR_BAD_ARGUMENT (-1)
#define KF_ERR_UNSUPPORTED (-2)
#define KF_ERR_DEVICE_WAIT (-3) /* a bounded device-side wait ran out (reported by kf_check_device_error) */

/* block-scaled formats: element type, scale type, elements per scale along K */
#define KF_FMT_MX8 0 /* e4m3, ue8m0 per 32            */
#define KF_FMT_NV4 1 /* e2m1, e4m3 per 16 + fp32 per-tensor scale */
#define KF_FMT_MX4 2 /* e2m1, ue8m0 per 32            */
#define KF_FMT_BF16 3 /* plain bf16 operands (GEMM only; no scales) */

/* element types of float tensors */
#define KF_F32 0
#define KF_BF16 1
#define KF_F16 2

/* quantiser flags */
#define KF_Q_GELU 1        /* x <- gelu_erf(x + bias[col]) before quantising                         */
#define KF_Q_ROUND_BF16 2  /* round the (LN / GELU) value to bf16 before quantising                  */
#define KF_Q_RECIP_DIV 4   /* amax/448, amax/6 as multiply by the fp32 reciprocal (torch-on-CUDA rule) */
#define KF_Q_FAST_NV4 64   /* QUANT epilogue to nv4 only: block scale and element division through approximate
                              reciprocals instead of the IEEE divisions of the bit specification (opt-in; a code moves
                              only where the exact quotient lies within an ulp of a rounding boundary) */

/* GEMM epilogues */
#define KF_EPI_PLAIN 0 /* C = act(acc*ts + bias)                      f32 | bf16 | f16 [M,N]         */
#define KF_EPI_RES 1   /* C = R + gamma * (acc*ts + bias)             f32 [M,N]                      */
#define KF_EPI_ROPE 2  /* bias + RoPE on q,k + relayout               bf16 | f16 [3,B,Ntok,H,64]     */
#define KF_EPI_QUANT 3 /* gelu(acc*ts + bias) quantised to out_fmt    codes [M,N] + blocked scales   */

/* GEMM flags (share the flag word with KF_Q_ROUND_BF16 / KF_Q_RECIP_DIV / KF_Q_FAST_NV4, which act on the QUANT epilogue) */
#define KF_G_GELU 8        /* PLAIN: apply gelu_erf after the bias */
#define KF_G_ROUND_BF16 16 /* PLAIN: round the value to bf16 before storing (matters for an f32 output) */
#define KF_G_PRE_ROUND_BF16 32 /* PLAIN: round acc*ts to bf16 BEFORE the bias is added (a bf16 GEMM followed by bias + GELU) */
#define KF_G_ROPE_HALF 128 /* ROPE: the caller guarantees that columns 32..63 of sin / cos repeat columns 0..31 (the axial
                              tables of DINOv3 are the angle vector concatenated with itself); lets the kernel keep the table
                              rows of a tile in shared memory.  Without the flag both halves are read as given. */

/* Library version and the SM architecture the kernels were built for ("sm_100a"). */
KF_API const char* kf_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
KF_API const char* kf_last_error_string(void);

/* Bytes of the blocked scale tensor [ceil(R/128), K/(4*vec), 32, 4, 4] of an [R, K] operand.
 * Replaces the size arithmetic of ActBuf / MXW: infer-opt/round13_mxfp8_full/impl/mx13.py:53-61,74-84 and
 * infer-opt/round14_fp4_full/impl/stack14b.py:92-93. */
KF_API int64_t kf_sf_bytes(int64_t R, int64_t K, int fmt);

/* Row quantiser: x [M, K] (row stride ldx elements; f32 | bf16 | f16) -> codes q (mx8: [M, K] bytes; nv4 / mx4:
 * [M, K/2] bytes, even element in the low nibble) + blocked scales sf (rows M..pad128(M) written as zero).
 * ts: device fp32 per-tensor scale, nv4 only.  bias: fp32 [K], only with KF_Q_GELU.
 * Replaces quant_rows / gelu_quant (infer-opt/round13_mxfp8_full/impl/mx13.cu:191-217,329-330) and
 * quantx (infer-opt/round14_fp4_full/impl/lnq14.cu:133-154,171). */
KF_API int kf_quant_rows(int fmt, int in_dtype, const void* x, int64_t ldx, int M, int K, const float* ts,
                  const float* bias, int flags, void* q, void* sf, void* stream);

/* LayerNorm fused with quantisation: x fp32 [M, d] (the residual stream), w, b fp32 [d] -> codes + blocked scales
 * as in kf_quant_rows.  d must be a multiple of 256, at most 2048.  y_dbg (optional, fp32 [M, d]) receives the
 * normalised values that were quantised.
 * Replaces ln_mx8 (infer-opt/round13_mxfp8_full/impl/mx13.cu:95-136,299-310) and
 * lnq (infer-opt/round14_fp4_full/impl/lnq14.cu:85-130,158). */
KF_API int kf_ln_quant(int fmt, const float* x, const float* w, const float* b, float eps, int M, int d,
                const float* ts, int flags, void* q, void* sf, float* y_dbg, void* stream);

/* LayerNorm to a 16-bit tensor: x fp32 [M, d] -> y bf16 | f16 [M, d].
 * Replaces ln_bf16 (infer-opt/round14_fp4_full/impl/ln14.cu:23-58,67) and ln16
 * (infer-opt/round12_lowp_stack/impl/ln16.cu). */
KF_API int kf_ln_rows(const float* x, const float* w, const float* b, float eps, int M, int d, int out_dtype, void* y,
               void* stream);

/* Parameter block of kf_gemm_bs.  All pointers are device pointers; unused ones are NULL.
 * Replaces the by-value Params blobs of the reference GEMMs: "=12Q8i" (infer-opt/round13_mxfp8_full/impl/mgx.py:24,96-102;
 * mgx_core.cu:43-48) and "=14Q10i" (infer-opt/round14_fp4_full/impl/fp4gb.py:15,74-82; fp4g_core.cu:36-42). */
typedef struct kf_gemm_params {
  int fmt;       /* operand format of A and W: KF_FMT_MX8 | NV4 | MX4 | BF16                                 */
  int epi;       /* KF_EPI_*                                                                                   */
  int M, N, K;   /* C[M,N] = A[M,K] * W[N,K]^T; N % 128 == 0; K % 128 (mx8) | 256 (nv4, mx4) | 64 (bf16) == 0 */
  int out_dtype; /* KF_F32 | KF_BF16 | KF_F16 for PLAIN; KF_BF16 | KF_F16 for ROPE                             */
  int flags;     /* KF_G_GELU, KF_Q_ROUND_BF16, KF_Q_RECIP_DIV                                                 */
  int Ntok, prefix, H; /* ROPE: tokens per image, tokens that are not rotated (queries, cls, registers), heads */
  int out_fmt;   /* QUANT: KF_FMT_MX8 | NV4 | MX4                                                              */
  const void* A;   /* codes [M, K] (mx8), [M, K/2] (nv4, mx4) or bf16 [M, K], rows contiguous                  */
  const void* SFA; /* blocked scales of A (NULL for bf16)                                                      */
  const void* W;   /* codes / bf16 [N, K]                                                                      */
  const void* SFW; /* blocked scales of W                                                                      */
  const float* ts_a; /* nv4 per-tensor scale of A (NULL = 1)                                                   */
  const float* ts_w; /* nv4 per-tensor scale of W (NULL = 1); the accumulator is multiplied by ts_a*ts_w       */
  const float* bias;  /* fp32 [N] or NULL                                                                      */
  const float* gamma; /* RES: fp32 [N] LayerScale                                                              */
  const float* R;     /* RES: fp32 [M, N] residual stream (may alias C)                                        */
  const float* sin;   /* ROPE: fp32 [Ntok - prefix, 64]                                                        */
  const float* cos;   /* ROPE: fp32 [Ntok - prefix, 64]                                                        */
  void* C;            /* PLAIN / RES / ROPE output                                                             */
  void* Qo;           /* QUANT: output codes [M, N] (mx8) or [M, N/2]                                          */
  void* SFo;          /* QUANT: output blocked scales of an [M, N] operand                                     */
  const float* tso;   /* QUANT to nv4: static per-tensor scale of the output                                   */
  /* PLAIN and RES: output row of GEMM row m is (m / group) * stride + offset + m % group; group 0 = identity.
   * Lets the patch-embed GEMM write straight into the token stream behind each image's cls / register rows, and the last
   * fc2 before the queries join write the stream (read from R, row m) into the longer stream behind each image's query rows. */
  int out_row_group, out_row_stride, out_row_offset;
  /* QUANT only, optional (NULL = off): fp32 [M, N] that receives the values the epilogue quantised, i.e.
   * gelu(acc*ts + bias) after the optional bf16 rounding.  For parity tests: the written codes and scales are the bit
   * specification's quantisation of exactly these values (mirrors y_dbg of kf_ln_quant). */
  float* y_dbg;
  /* PLAIN with bf16 operands only, batch > 0: `batch` independent products in one launch, C_b = A_b * W_b^T with
   * A_b = rows b*a_rows_per_batch .. of A (M = batch * a_rows_per_batch), W_b = rows b*w_rows_per_batch .. of W
   * (w_rows_per_batch >= N) and C the flat [M, N] matrix (= [batch, a_rows_per_batch, N]).  One launch fills the SMs
   * where one product alone leaves a partial round of tiles.  Replaces the torch.bmm of the mask product
   * (infer-opt/round11_attn_tier0/impl/head11.py:95).  batch = 0: off. */
  int batch, a_rows_per_batch, w_rows_per_batch;
} kf_gemm_params;

/* Block-scaled GEMM on tcgen05 with a fused epilogue.
 * Replaces gemm_kernel + qkv_rope / gemm_res / gemm_gelu_q / gemm_plain
 * (infer-opt/round13_mxfp8_full/impl/mgx_core.cu:118-444, mgx.py:130-167), the FP4 gemm_kernel
 * (infer-opt/round14_fp4_full/impl/fp4g_core.cu:153-470, fp4gb.py:74-82), torch._scaled_mm at
 * infer-opt/round13_mxfp8_full/impl/mx13.py:87-88 and the QuACK GEMMs behind FP4Linear.fwd_*
 * (infer-opt/round14_fp4_full/impl/fp4util.py:137-159). */
KF_API int kf_gemm_bs(const kf_gemm_params* p, void* stream);

/* Final LayerNorm of the fp32 token stream x [B, Ntok, d] with the row gather of the EoMT head: query rows
 * (t < Q) -> qb bf16 [B*Q, d], patch rows (t >= Q + npre) -> xb bf16 [B*(Ntok-Q-npre), d].  With wcls (bf16 [ncls1, d],
 * optional) the class head runs on the query rows in the same pass: cl bf16 [B*Q, ncls1] = bf16(qb * wcls^T + bcls),
 * fp32 accumulation, bcls fp32 [ncls1].
 * Replaces tail_ln = LN + gather + class head in one kernel (infer-opt/round11_attn_tier0/impl/head_ext11.cu:252-320). */
KF_API int kf_ln_tail(const float* x, const float* w, const float* b, float eps, int B, int Ntok, int Q, int npre, int d, void* qb,
                      void* xb, const void* wcls, const float* bcls, int ncls1, void* cl, void* stream);

/* Writes the same R fp32 rows into every image of a token stream: dst[b][row_offset + r][:] = src[r][:], b < B, with
 * img_stride values between images.  The query rows joining the stream before the last blocks and the cls / register rows
 * in front of the patch tokens.
 * Replaces the torch.cat calls of the reference's token assembly (infer-opt/round13_mxfp8_full/impl/stack13.py:169-172;
 * src/lightly_train/_models/dinov3/dinov3_src/models/vision_transformer.py:244-251). */
KF_API int kf_broadcast_rows(const float* src, float* dst, int R, int d, int B, int64_t img_stride, int64_t row_offset, void* stream);

/* Patch gathering for the patch-embed GEMM: x bf16 [B, 3, S, S] -> bf16 [B*(S/16)^2, 768], k = c*256 + py*16 + px.
 * Replaces the implicit im2col of patch_gemm_kernel (infer-opt/round11_attn_tier0/impl/patch_embed.cu:76-194). */
KF_API int kf_im2col_patch16(const void* x, void* out, int B, int S, void* stream);

/* Patch embedding that allocates nothing: x bf16 [B, 3, S, S] -> tokens fp32 [B, tokens_per_image, d], rows
 * row_offset .. row_offset + (S/16)^2 - 1 of every image = patches * w^T + bias (w bf16 [d, 768], k = c*256 + py*16 + px;
 * bias fp32 [d] or NULL; flags: 0 or KF_G_ROUND_BF16).  The same result, bit for bit, as kf_im2col_patch16 into a
 * caller buffer followed by kf_gemm_bs with the output row mapping, but the gathered patch rows go to a fixed array inside
 * the library instead of a buffer the caller allocates.
 * For callers that cannot allocate: a plug-in inside another program's frame loop that receives inputs and outputs but no
 * allocator, or a latency-critical path where cudaMalloc's device-wide synchronisation is not acceptable.
 * Limits and rules:
 *   - at most KF_PATCH_STATIC_MAX_ROWS = B * (S/16)^2 patch rows per call (one 1024 x 1024 image, two 640 x 640 images);
 *     more is refused with KF_ERR_BAD_ARGUMENT and a message.  The array (6 MiB) is part of the library image: every GPU
 *     that loads the library holds it until the process exits.
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device current) and
 *     keeps it; make that first call before any stream capture.
 *   - every call uses the same array, which keeps the previous call's rows: nothing in it needs clearing (a call overwrites
 *     every row it reads), but two calls that overlap on the GPU (different streams, no ordering) race on it.
 *   - no cudaMalloc, cudaFree or other allocating routine is called.
 * No counterpart in the reference (its patch embed, infer-opt/round11_attn_tier0/impl/patch_embed.py:34-53, returns freshly
 * allocated torch tensors). */
#define KF_PATCH_STATIC_MAX_ROWS 4096
KF_API int kf_patch_embed_static(const void* x, const void* w, const float* bias, float* tokens, int B, int S, int d, int tokens_per_image,
                                 int row_offset, int flags, void* stream);

/* ScaleBlock tail: g bf16 [B*Hs*Ws, 4C] (ConvTranspose2d k2 s2 as a GEMM, column (dy*2+dx)*C + c) -> bias + GELU +
 * pixel shuffle + depthwise 3x3 (dww fp32 [9, C], tap-major, zero padding) + LayerNorm2D -> out bf16 [B, 2Hs, 2Ws, C].
 * pre_act != 0: g already holds bf16(gelu(conv + bias)) (applied by the GEMM epilogue: KF_G_PRE_ROUND_BF16 | KF_G_GELU
 * with the bias repeated 4x), so bias + GELU are skipped here.  C is a multiple of 128 up to 1024 (a CTA has C/4 threads,
 * each owning 4 channels); any Hs, Ws.
 * Replaces dw_ln (infer-opt/round11_attn_tier0/impl/head_ext11.cu:72-250) = ScaleBlock.forward after conv1
 * (src/lightly_train/_task_models/dinov3_eomt_semantic_segmentation/scale_block.py:39-44). */
KF_API int kf_dw_ln(const void* g, const float* bias, const float* dww, const float* lnw, const float* lnb, void* out, int B,
                    int Hs, int Ws, int C, float eps, int pre_act, void* stream);

/* Per-pixel semantic scores: scores[b,c,p] = sum_q sigmoid(mask_logits[b,q,p]) * softmax(class_logits[b,q,:])[c]
 * (fp32 [B, ncls+1, HW], optional) and labels[b,p] = argmax over the ncls real classes (uint8, optional).
 * mask_logits bf16 [B, Q, HW], class_logits bf16 [B, Q, ncls+1].
 * Replaces to_per_pixel_logits_semantic + argmax (src/lightly_train/_task_models/dinov3_eomt_semantic_segmentation/
 * task_model.py:583-594; scripts/infer_dinov3_eomt_head_video.py:90-94). */
KF_API int kf_semantic(const void* mask_logits, const void* class_logits, int B, int Q, int ncls, int HW, float* scores,
                       uint8_t* labels, void* stream);

/* Frame pre-processing: uint8 [B, Hi, Wi, 3] -> bf16 [B, 3, So, So], bilinear with antialiasing, then
 * (v/255 - mean[c]) / std[c]; mean3 / std3 are HOST arrays of three floats.
 * Replaces prep_kernel (infer-opt/round7_head_postprocess/impl/postfuse_ext.cu:30-72) / base_prep
 * (infer-opt/common/model_factory.py:99). */
KF_API int kf_resize_norm(const uint8_t* frames, void* out, int B, int Hi, int Wi, int So, const float* mean3,
                          const float* std3, void* stream);

/* FlashAttention-style forward, head dimension 64, no mask: qkv [3, B, N, H, 64] (bf16 | f16, RoPE already applied,
 * the layout KF_EPI_ROPE writes) -> O [B, N, H*64] of the same type; softmax scale 1/8, fp32 statistics and
 * accumulators.  `pre` is the reference's power-of-two Q pre-scale for fp16 accumulation; it is neutral here.
 * Replaces attn16_fwd / a16::fwd_kernel (infer-opt/round12_lowp_stack/impl/attn16o.cu:126-404). */
KF_API int kf_attn_fwd(int dtype, const void* qkv, void* O, int B, int N, int H, float pre, void* stream);

/* Tensor-core instruction-rate probe: every SM issues `iters` x 4 tcgen05.mma (M=128, N=n in {64,128,256}, 32 K-bytes each) of the
 * given operand format on shared-memory-resident operands; *flops_per_launch receives the FLOPs one launch performs.
 * sf_copies (0..8) scale-factor atoms are re-copied smem -> TMEM (tcgen05.cp) before every group of 4 MMAs, as a real
 * block-scaled main loop must (mx8: 2, mx4: 4, nv4: 8 at a 128 x 128 tile); 0 copies them once; 8 + c issues the c copies
 * per stage from a second warp with no ordering against the MMA stream (do the two overlap in the hardware?).
 * The caller times the launch to obtain the FP8 / FP4 / bf16 instruction-rate ceiling of the part.
 * Counterpart: the mma.sync probe infer-opt/round10_lowp_probe/peak_extra.cu. */
KF_API int kf_tensor_peak_probe(int fmt, int n, int iters, int sf_copies, double* flops_per_launch, void* stream);

/* The same attention forward with the quantisation of its output fused into the epilogue: the O row of every head is
 * rounded to the 16-bit input type and written as codes + blocked scales of the [B*N, H*64] operand the proj GEMM
 * reads (format out_fmt, nv4 with the static per-tensor scale tso).  Scale rows B*N..pad128(B*N) are not touched.
 * Replaces attn16_fwd followed by quant_rows / quantx (infer-opt/round13_mxfp8_full/impl/stack13.py:105-106,
 * infer-opt/round14_fp4_full/impl/stack14b.py:104-110); the reference lists this fusion as estimated but not built
 * (infer-opt/round14_fp4_full/NOTES.md:142-143). */
KF_API int kf_attn_fwd_quant(int dtype, const void* qkv, int B, int N, int H, float pre, int out_fmt, void* Qo, void* SFo,
                             const float* tso, int flags, void* stream);

/* Programmatic dependent launch for the kernels of the transformer block (LN + quant, GEMM, attention): on lets a
 * kernel's CTAs start on the SMs its predecessor has already left (partial last wave, teardown) and overlap their set-up with
 * it; every kernel waits for its predecessors' completion before touching global memory, so results do not change.
 * Off by default: every kernel of the block needs its predecessor's whole output, so only the set-up overlaps, and inside a
 * captured graph that measured slightly slower than plain stream order.
 * Counterpart: set_pdl(bool) (infer-opt/round13_mxfp8_full/impl/mx13.cu:282). */
KF_API int kf_set_pdl(int on);

/* Reads (and clears) the device error word that kernels with bounded waits write when a wait runs out.
 * Synchronises the device.  Returns KF_OK, or KF_ERR_DEVICE_WAIT with where/block in the error string.
 * While the word is set, the GEMM and attention kernels return at once without touching their outputs (a failed launch must not
 * make every later launch wait out its limits too), so the outputs of launches after a failure are undefined until this call.
 * No counterpart in the reference (its mbarrier waits spin without a bound: infer-opt/round12_lowp_stack/impl/attn16o.cu:77-79). */
KF_API int kf_check_device_error(void);

#ifdef __cplusplus
}
#endif
#endif /* KF_B200_H */
