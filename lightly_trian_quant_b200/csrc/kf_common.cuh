// Shared device/host helpers of the B200 (sm_100a) low-precision ViT path: format conversions, the 128x4 blocked
// scale-factor addressing, status codes and the last-error string of the C-ABI.
#pragma once
#include <utility>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/kf_b200.h"

namespace kf {

// ---------------------------------------------------------------------------------------------- host side status
void set_error(const char* fmt, ...);
int cuda_status(cudaError_t e, const char* what);
int device_sm_count(int* sms);   // multiprocessor count of the current device (cached)
bool pdl_enabled();              // kf_set_pdl: launch the block kernels with programmatic dependent launch

// Programmatic dependent launch: a kernel lets its successor's CTAs start on SMs it no longer occupies (its partial last
// wave, its teardown) and the successor runs its prologue (barrier set-up, TMEM allocation, descriptor prefetch) there; the
// successor must not touch global memory before pdl_wait(), which returns when every predecessor grid has completed
// and its writes are visible.  Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// <<<grid, block, smem, stream>>> with the programmatic-stream-serialization attribute when PDL is enabled
template <typename... KArgs, typename... Args>
inline cudaError_t launch_maybe_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

#define KF_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      kf::set_error(__VA_ARGS__);        \
      return KF_ERR_BAD_ARGUMENT;        \
    }                                    \
  } while (0)

// ---------------------------------------------------------------------------------------------- scale layout
// Byte offset of the scale of (row, kb) in the 128x4 blocked layout [ceil(R/128), nkb/4, 32, 4, 4]:
// one 512-byte atom holds 128 rows x 4 consecutive k-blocks, a 32-bit word the 4 k-block scales of one row.
__host__ __device__ __forceinline__ size_t sf_offset(int row, int kb, int nkb4 /* k-blocks / 4 */) {
  return ((size_t)(row >> 7) * nkb4 + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

__host__ __device__ __forceinline__ int fmt_vec(int fmt) { return fmt == KF_FMT_NV4 ? 16 : 32; }

// ---------------------------------------------------------------------------------------------- conversions
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {      // returns (hi << 8) | lo, RN-even, saturating
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  return cvt_e4m3x2(a, b) | (cvt_e4m3x2(c, d) << 16);
}

// 8 floats -> 8 e2m1 nibbles packed into 32 bits, element 0 in the lowest nibble (RN-even, saturating at 6).
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float* v) {
  uint32_t r;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}

// 4 floats -> 4 e2m1 nibbles in the low 16 bits, element 0 in the lowest nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x4(const float* v) {
  uint16_t r;
  asm("{\n\t"
      ".reg .b8 b0, b1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "mov.b16 %0, {b0, b1};\n\t"
      "}"
      : "=h"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]));
  return r;
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  uint32_t h2;
  uint16_t b = (uint16_t)byte;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(b));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF)));
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Packed fp32 pairs (the two-wide FFMA2 / FADD2 / FMUL2 of sm_100): each component is the IEEE round-to-nearest result of
// the scalar operation, at one issue slot per pair.  The CUDA-core-bound kernels here are short of issue slots, not of
// FMA lanes.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 splat2(float x) { return make_float2(x, x); }
// both values rounded to bf16 and widened again: one packed conversion and two bit operations
__device__ __forceinline__ float2 bf16_round2(float2 v) {
  const __nv_bfloat162 h = __float22bfloat162_rn(v);
  const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

// GELU with the exact (erf) definition 0.5*x*(1 + erf(x/sqrt(2))).  erfc(t) for t >= 0 is evaluated as
// poly5(k) * exp(-t^2), k = 1/(1 + p*t) (Abramowitz & Stegun 7.1.26, |error| <= 1.5e-7, the same class as fp32 erff)
// and the two signs are assembled without cancellation as relu(x) - 0.5*|x|*erfc(t).
// About 15 instructions (two of them MUFU) instead of the ~30 of erff: the fused GEMM epilogues are bound by
// CUDA-core issue.
__device__ __forceinline__ float gelu_erf(float x) {
  const float ax = fabsf(x);
  const float u = ax * 0.84932180028801904272f;          // exp(-x^2/2) = 2^(-u^2), u = |x| * sqrt(log2(e)/2)
  float k;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(k) : "f"(fmaf(0.23164189388980933f, ax, 1.0f)));   // 1 / (1 + p*|x|/sqrt2)
  float p = fmaf(k, 1.061405429f, -1.453152027f);
  p = fmaf(p, k, 1.421413741f);
  p = fmaf(p, k, -0.284496736f);
  p = fmaf(p, k, 0.254829592f);
  p *= k;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-u * u));
  return fmaxf(x, 0.f) - (0.5f * ax) * (p * e);         // relu(x) - 0.5*|x|*erfc(|x|/sqrt2), both signs without cancellation
}

// GELU (exact-erf definition) of two values for the fused GEMM epilogues, which are short of XU (MUFU) throughput: one
// exponential per value and no reciprocal.  gelu(x) = relu(x) - |x| * Phi(-|x|) with the normal tail written as
// Phi(-a) = 2^(-a^2 * log2(e)/2 + Q(a)); Q is smooth and logarithm-like (Q(0) = -1) and a degree-7 least-squares fit on
// Chebyshev nodes of [0, 6] keeps the exponent within 5.7e-6, |gelu error| <= 6.1e-7 (the class of fp32 erff); past 6 the
// quadratic term has pushed the product below 1e-8 and soon to an exact 0.  Evaluated on n = -|x| (odd coefficients
// negated) as packed pairs: 12 packed + 6 scalar instructions per pair.
__device__ __forceinline__ float2 gelu_erf2(float2 x) {
  const float2 n = make_float2(-fabsf(x.x), -fabsf(x.y));
  float2 q = fma2(n, splat2(1.8896262190537527e-06f), splat2(6.268139986786991e-05f));
  q = fma2(q, n, splat2(0.0009388679172843695f));
  q = fma2(q, n, splat2(0.00853946153074503f));
  q = fma2(q, n, splat2(0.05402068793773651f));
  q = fma2(q, n, splat2(0.2629377543926239f));
  q = fma2(q, n, splat2(1.1512691974639893f));
  q = fma2(q, n, splat2(-0.9999943375587463f));
  const float2 p = fma2(mul2(n, n), splat2(-0.72134752044448170368f), q);
  float2 e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(p.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(p.y));
  const float2 relu = make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f));
  return fma2(n, e, relu);
}

// max(a, b, c) in one instruction.  NaN-propagating (as are amax_nan / min_nan below): the block maxima of the quantisers
// must carry a NaN to the scale byte the way torch's amax does in the reference quantiser (a NaN activation gives scale byte
// 255 / 0x7f and is not silently quantised as a finite value); fmaxf would drop it.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float amax_nan(float a, float b) {
  float y;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(y) : "f"(a), "f"(b));
  return y;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float y;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(y) : "f"(a), "f"(b));
  return y;
}

// Correctly rounded x / d from a correctly rounded reciprocal r = RN(1/d) (one per block): q = RN(x*r), the exact
// remainder by FMA, one correction step.  Valid while no intermediate over- or underflows; callers check the block
// maximum once and fall back to __fdiv_rn otherwise.
__device__ __forceinline__ float div_by_rcp(float x, float d, float r) {
  const float q = x * r;
  const float rem = fmaf(-d, q, x);
  return fmaf(rem, r, q);
}

// 2^k for k in [-128, 127] including the two subnormal powers below 2^-126.
__device__ __forceinline__ float pow2_int(int k) {
  int eb = k + 127;
  return eb > 0 ? __uint_as_float((uint32_t)eb << 23) : __uint_as_float(0x00400000u >> (-eb));
}

// ue8m0 byte of a block: biased exponent of fl32(amax/denom) plus one when the mantissa is non-zero (round up to a
// power of two), clamped.  The division is a true IEEE division unless div_true == 0, in which case amax is
// multiplied by the fp32 reciprocal (what torch does for tensor / python-scalar on a CUDA device).
template <int DENOM>
__device__ __forceinline__ int rceil_byte(float amax, int max_byte, bool div_true) {
  float r = div_true ? __fdiv_rn(amax, (float)DENOM) : amax * (1.0f / (float)DENOM);
  uint32_t b = __float_as_uint(r);
  int e = (b >> 23) & 0xFF;
  e += (b & 0x7FFFFFu) != 0;
  return e < max_byte ? e : max_byte;
}

// ---------------------------------------------------------------------------------------------- block quantisers
// Each takes NL values held by one lane (NL = 8 or 16) whose block maximum `amax` has already been reduced over the
// lanes that share the block, and returns the packed codes.  `sf_byte` receives the block's scale byte.

template <int NL>
__device__ __forceinline__ void quant_mx8(const float (&v)[NL], float amax, bool div_true, uint32_t* out /* NL/4 words */, int& sf_byte) {
  int byte = rceil_byte<448>(amax, 255, div_true);
  float inv = pow2_int(127 - (byte < 1 ? 1 : byte));
#pragma unroll
  for (int i = 0; i < NL; i += 4) {
    // the clamp to +-448 of the reference is what cvt.rn.satfinite does
    const float2 a = mul2(make_float2(v[i], v[i + 1]), splat2(inv)), b = mul2(make_float2(v[i + 2], v[i + 3]), splat2(inv));
    out[i / 4] = cvt_e4m3x4(a.x, a.y, b.x, b.y);
  }
  sf_byte = byte;
}

template <int NL>
__device__ __forceinline__ void quant_mx4(const float (&v)[NL], float amax, bool div_true, uint32_t* out /* NL/8 words */, int& sf_byte) {
  int byte = rceil_byte<6>(amax, 254, div_true);
  float inv = pow2_int(127 - byte);
  const bool has_nan = amax != amax;            // the conversion instruction would turn a NaN into 6; the reference's comparisons give 0
  if constexpr (NL == 4) {
    float t[4] = {v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv};
    if (has_nan) {
#pragma unroll
      for (int j = 0; j < 4; ++j) t[j] = t[j] != t[j] ? 0.f : t[j];
    }
    out[0] = cvt_e2m1x4(t);                     // 16 bits
  } else {
    float t[8];
#pragma unroll
    for (int i = 0; i < NL; i += 8) {
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] = v[i + j] * inv;
      if (has_nan) {
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = t[j] != t[j] ? 0.f : t[j];
      }
      out[i / 8] = cvt_e2m1x8(t);
    }
  }
  sf_byte = byte;
}

// Correctly rounded x / d through a correctly rounded reciprocal r = RN(1/d) (Markstein: q = RN(x*r), exact remainder by
// FMA, one correction), valid while nothing over- or underflows and the significand of d is not all ones; anything else
// goes to __fdiv_rn.  `safe_d` says that d itself is in the safe range (checked once per tensor by the caller).
__device__ __forceinline__ float div_exact(float x, float d, float r, bool safe_d) {
  if (safe_d && (x == 0.f || (x > 1e-30f && x < 1e30f))) return div_by_rcp(x, d, r);
  return __fdiv_rn(x, d);
}
__device__ __forceinline__ bool div_safe_divisor(float d) {
  return d > 1e-30f && d < 1e30f && (__float_as_uint(d) & 0x7FFFFFu) != 0x7FFFFFu;
}

// Per-tensor constants of the NVFP4 quantiser, worked out once per thread: the per-tensor scale, its correctly rounded
// reciprocal and whether the reciprocal route is exact for it.
struct Nv4Scale {
  float ts, rcp_ts;
  bool safe;
};
__device__ __forceinline__ Nv4Scale nv4_scale(float t) {
  Nv4Scale s;
  s.ts = t;
  s.rcp_ts = __frcp_rn(t);
  s.safe = div_safe_divisor(t);
  return s;
}

// The scalars of one NVFP4 block, worked out from its maximum alone: the e4m3 scale byte, the element divisor
// dd = e4m3(scale) * ts, its correctly rounded reciprocal and how the elements are to be divided (0: the block is all
// zeros, 1: through the reciprocal, 2: by __fdiv_rn).  Lanes that share a block, or a lane that owns several, can work
// these out once and pass them on.
struct Nv4Block {
  float dd, rcp;
  uint32_t sb;
  int mode;
};
__device__ __forceinline__ Nv4Block nv4_block(float amax, const Nv4Scale& sc, bool div_true) {
  const float ts = sc.ts;
  // amax / 6 and (amax / 6) / ts are IEEE divisions; 1/6 as a constant reciprocal (RN(1/6) = 0x3E2AAAAB)
  float a6 = div_true ? div_exact(amax, 6.0f, 0.16666667163372040f, true) : amax * (1.0f / 6.0f);
  float t = min_nan(div_exact(a6, ts, sc.rcp_ts, sc.safe), 448.f);
  Nv4Block b;
  b.sb = cvt_e4m3x2(t, 0.f) & 0xFF;
  float denom = e4m3_to_float(b.sb) * ts;
  bool ok = denom > 0.f;
  b.dd = ok ? denom : 1.0f;
  // IEEE division of every element by the block's denominator: through one correctly rounded reciprocal when the
  // whole block stays in the normal range (|quotient| <= amax/dd), else by __fdiv_rn.
  b.rcp = __frcp_rn(b.dd);
  const float qmax = amax * b.rcp;
  const bool fast = div_safe_divisor(b.dd) && qmax < 1e30f;
  b.mode = !ok ? 0 : fast ? 1 : 2;
  return b;
}
template <int NL>
__device__ __forceinline__ void nv4_codes(const float (&v)[NL], const Nv4Block& b, uint32_t* out /* NL/8 words */) {
  const float dd = b.dd, rcp = b.rcp;
  constexpr int G = NL < 8 ? NL : 8;            // quotients are converted group by group so that few of them are live at once
#pragma unroll
  for (int i = 0; i < NL; i += G) {
    float q[G];
    if (b.mode == 1) {
      const float2 r2 = splat2(rcp), nd2 = splat2(-dd);
#pragma unroll
      for (int j = 0; j < G; j += 2) {          // div_by_rcp on packed pairs
        const float2 x = make_float2(v[i + j], v[i + j + 1]);
        const float2 q0 = mul2(x, r2);
        const float2 q1 = fma2(fma2(nd2, q0, x), r2, q0);
        q[j] = q1.x;
        q[j + 1] = q1.y;
      }
    } else if (b.mode == 0) {
#pragma unroll
      for (int j = 0; j < G; ++j) q[j] = 0.f;
    } else {
#pragma unroll
      for (int j = 0; j < G; ++j) q[j] = __fdiv_rn(v[i + j], dd);
    }
    if constexpr (NL == 4) out[0] = cvt_e2m1x4(q);   // 16 bits
    else out[i / 8] = cvt_e2m1x8(q);
  }
}
template <int NL>
__device__ __forceinline__ void quant_nv4(const float (&v)[NL], float amax, const Nv4Scale& sc, bool div_true, uint32_t* out /* NL/8 words */, int& sf_byte) {
  const Nv4Block b = nv4_block(amax, sc, div_true);
  nv4_codes<NL>(v, b, out);
  sf_byte = (int)b.sb;
}
template <int NL>
__device__ __forceinline__ void quant_nv4(const float (&v)[NL], float amax, float ts, bool div_true, uint32_t* out, int& sf_byte) {
  quant_nv4<NL>(v, amax, nv4_scale(ts), div_true, out, sf_byte);
}

// Correctly rounded 1/d from the approximate reciprocal and one Newton step (Markstein): r0 = rcp.approx(d) is within one
// ulp of 1/d, e = RN(1 - d*r0) is exact enough and RN(r0 + r0*e) is RN(1/d) unless the significand of d is all ones;
// valid for normal d whose reciprocal is normal (callers guarantee 1e-18 < d < 1e18).  Three instructions instead of the
// ten of __frcp_rn; kf_selftest_rcp sweeps every significand against __frcp_rn.
__device__ __forceinline__ float2 rcp_rn_pair(float2 d) {
  float2 r0;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0.x) : "f"(d.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0.y) : "f"(d.y));
  const float2 e = fma2(make_float2(-d.x, -d.y), r0, splat2(1.0f));
  return fma2(r0, e, r0);
}
__device__ __forceinline__ bool mant_all_ones(float d) { return (__float_as_uint(d) & 0x7FFFFFu) == 0x7FFFFFu; }

// Two NVFP4 blocks of 16 values at once (a thread of a GEMM epilogue owns both): the block scalars (amax/6, /ts, the e4m3
// scale, the element divisor and its reciprocal) are worked out on packed pairs, one conversion instruction serves both
// scale bytes.  Bit-identical to quant_nv4 on each block: inside the range where every step of the reciprocal route is an
// exact IEEE division (1e-15 < amax, ts < 1e15, hence no intermediate under- or overflow; divisor significands not all
// ones; non-zero scale) the packed route is taken, anything else goes through quant_nv4 itself.
// The scalars of two NVFP4 blocks at once, on packed pairs (see nv4_block for the single-block form and quant_nv4_pair16
// for the range argument): both results are bit-identical to nv4_block on each maximum.
__device__ __forceinline__ void nv4_block_pair(float am0, float am1, const Nv4Scale& sc, bool div_true, Nv4Block& b0, Nv4Block& b1) {
  const float lo = min_nan(am0, am1), hi = amax_nan(am0, am1);       // a NaN maximum fails both range tests and takes the scalar route
  if (sc.safe && sc.ts > 1e-15f && sc.ts < 1e15f && lo > 1e-15f && hi < 1e15f) {
    const float2 am = make_float2(am0, am1);
    float2 a6;
    if (div_true) {                              // amax / 6 through RN(1/6) = 0x3E2AAAAB with one correction
      const float2 r6 = splat2(0.16666667163372040f);
      const float2 q = mul2(am, r6);
      a6 = fma2(fma2(splat2(-6.0f), q, am), r6, q);
    } else {
      a6 = mul2(am, splat2(1.0f / 6.0f));
    }
    const float2 rts = splat2(sc.rcp_ts);
    const float2 q = mul2(a6, rts);
    const float2 t = fma2(fma2(splat2(-sc.ts), q, a6), rts, q);
    const uint32_t sb2 = cvt_e4m3x2(fminf(t.x, 448.f), fminf(t.y, 448.f));   // byte 0: block 0, byte 1: block 1
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)sb2));
    const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    const float2 dd = mul2(sf, splat2(sc.ts));
    if (fminf(dd.x, dd.y) > 0.f && !mant_all_ones(dd.x) && !mant_all_ones(dd.y)) {
      const float2 rcp = rcp_rn_pair(dd);
      b0.mode = b1.mode = 1;
      b0.dd = dd.x;
      b0.rcp = rcp.x;
      b0.sb = sb2 & 0xFF;
      b1.dd = dd.y;
      b1.rcp = rcp.y;
      b1.sb = (sb2 >> 8) & 0xFF;
      return;
    }
  }
  b0 = nv4_block(am0, sc, div_true);
  b1 = nv4_block(am1, sc, div_true);
}

// Two NVFP4 blocks of 16 values at once (a thread of a GEMM epilogue owns both): the block scalars (amax/6, /ts, the e4m3
// scale, the element divisor and its reciprocal) are worked out on packed pairs, one conversion instruction serves both
// scale bytes.  Bit-identical to quant_nv4 on each block: inside the range where every step of the reciprocal route is an
// exact IEEE division (1e-15 < amax, ts < 1e15, hence no intermediate under- or overflow; divisor significands not all
// ones; non-zero scale) the packed route is taken, anything else goes through quant_nv4 itself.
__device__ __forceinline__ void quant_nv4_pair16(const float (&v0)[16], float am0, const float (&v1)[16], float am1, const Nv4Scale& sc, bool div_true,
                                                 uint32_t* out /* 4 words */, int& by0, int& by1) {
  // the arithmetic of nv4_block_pair, written out here so that the common route carries no per-block mode (measured in the
  // fc1 epilogue: 94 us against 100 us when the scalars travel through Nv4Block)
  const float lo = min_nan(am0, am1), hi = amax_nan(am0, am1);
  if (sc.safe && sc.ts > 1e-15f && sc.ts < 1e15f && lo > 1e-15f && hi < 1e15f) {
    const float2 am = make_float2(am0, am1);
    float2 a6;
    if (div_true) {
      const float2 r6 = splat2(0.16666667163372040f);
      const float2 q = mul2(am, r6);
      a6 = fma2(fma2(splat2(-6.0f), q, am), r6, q);
    } else {
      a6 = mul2(am, splat2(1.0f / 6.0f));
    }
    const float2 rts = splat2(sc.rcp_ts);
    const float2 q = mul2(a6, rts);
    const float2 t = fma2(fma2(splat2(-sc.ts), q, a6), rts, q);
    const uint32_t sb2 = cvt_e4m3x2(fminf(t.x, 448.f), fminf(t.y, 448.f));
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)sb2));
    const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    const float2 dd = mul2(sf, splat2(sc.ts));
    if (fminf(dd.x, dd.y) > 0.f && !mant_all_ones(dd.x) && !mant_all_ones(dd.y)) {
      const float2 rcp = rcp_rn_pair(dd);
      Nv4Block b;
      b.mode = 1;
      b.sb = 0;
      b.dd = dd.x;
      b.rcp = rcp.x;
      nv4_codes<16>(v0, b, out);
      b.dd = dd.y;
      b.rcp = rcp.y;
      nv4_codes<16>(v1, b, out + 2);
      by0 = (int)(sb2 & 0xFF);
      by1 = (int)((sb2 >> 8) & 0xFF);
      return;
    }
  }
  quant_nv4<16>(v0, am0, sc, div_true, out, by0);
  quant_nv4<16>(v1, am1, sc, div_true, out + 2, by1);
}

// NVFP4 block quantiser for epilogues whose input is a fresh accumulator (no bit-exact counterpart exists: the
// accumulation order already differs from any other implementation in the last bits): the divisions become
// multiplications by reciprocals (rcp_ts = 1/ts is passed in; the element divisor uses rcp.approx), which changes a code
// only when the exact quotient lies within an ulp of a rounding boundary.  A third of the instructions of quant_nv4.
template <int NL>
__device__ __forceinline__ void quant_nv4_fast(const float (&v)[NL], float amax, float ts, float rcp_ts, uint32_t* out /* NL/8 words */, int& sf_byte) {
  const float t = fminf(amax * (1.0f / 6.0f) * rcp_ts, 448.f);
  const uint32_t sb = cvt_e4m3x2(t, 0.f) & 0xFF;
  const float denom = e4m3_to_float(sb) * ts;
  float rcp;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(denom));
  rcp = denom > 0.f ? rcp : 0.f;
  float q[NL];
  const float2 r2 = splat2(rcp);
#pragma unroll
  for (int j = 0; j < NL; j += 2) {
    const float2 t = mul2(make_float2(v[j], v[j + 1]), r2);
    q[j] = t.x;
    q[j + 1] = t.y;
  }
#pragma unroll
  for (int i = 0; i < NL; i += 8) out[i / 8] = cvt_e2m1x8(q + i);
  sf_byte = (int)sb;
}

}  // namespace kf
