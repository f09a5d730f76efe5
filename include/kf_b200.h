/* C-ABI of the B200 (sm_100a) low-precision DINOv3 ViT + EoMT inference hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), launches on that stream and
 * returns without synchronising: 0 = ok, negative = bad argument (see kf_last_error_string), positive = the
 * cudaError_t of a failed launch.  The caller owns every buffer; nothing here allocates (the one exception is
 * documented on the entry point).  One thread per device may call concurrently.
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

#ifdef __cplusplus
}
#endif
#endif /* KF_B200_H */
