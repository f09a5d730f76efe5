/* Development probes of the B200 library: measurement helpers that the micro-benchmarks use and a user of the operators
 * never needs.  Same conventions as kf_b200.h (plain pointers, a CUDA stream as void*, 0 / negative / cudaError_t). */
#ifndef KF_B200_DEV_H
#define KF_B200_DEV_H

#include "kf_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Shared-memory fill-rate probe: every SM streams `iters` stages of `stage_bytes` (a multiple of 1024, <= 65536) from the
 * `span` bytes at `src` into a three-stage shared-memory ring with bulk copies and consumes nothing; *bytes_per_launch
 * receives the bytes one launch moves.  With a span that fits L2 this is the L2 -> shared-memory rate that feeds a GEMM main
 * loop whose operands are re-read from L2 (the CTAs' walks over the span overlap, so a larger span is not an HBM figure).
 * The caller times the launch.  No reference counterpart. */
KF_API int kf_fill_rate_probe(const void* src, long long span, int stage_bytes, int iters, double* bytes_per_launch, void* stream);

/* Self-test of the three-instruction correctly rounded reciprocal the NVFP4 quantisers use for their block divisors:
 * sweeps all 2^23 - 1 significands (all ones excluded: outside the routine's contract) of the binade 2^exponent, both
 * signs, against __frcp_rn and adds the number of differing results to *mismatches (a zero-initialised device counter).
 * No reference counterpart. */
KF_API int kf_selftest_rcp(int exponent, unsigned int* mismatches, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KF_B200_DEV_H */
