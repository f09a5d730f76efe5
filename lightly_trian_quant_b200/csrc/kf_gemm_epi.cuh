// Shared pieces of the block-scaled GEMM kernels (one-CTA tiles in kf_gemm.cu, CTA-pair tiles in kf_gemm2.cu): argument
// block, per-format traits, and the fused epilogues (PLAIN / RES / ROPE / QUANT) as one device function that works on a
// 32-row x 64-column piece of the accumulator held in registers.  Epilogue math per
// infer-opt/round13_mxfp8_full/impl/mgx_core.cu:308-426 and infer-opt/round14_fp4_full/impl/fp4g_core.cu:309-382.
#pragma once
#include "kf_sm100.cuh"

namespace kf {

constexpr int KIND_MX8 = KF_FMT_MX8, KIND_NV4 = KF_FMT_NV4, KIND_MX4 = KF_FMT_MX4, KIND_BF16 = KF_FMT_BF16;
constexpr int BM = 128, BN = 256, BKB = 128;          // tile rows, tile columns, K bytes per stage
constexpr int A_BYTES = BM * BKB, TILE_BYTES = (BM + BN) * BKB;   // 16 KB of A, then 32 KB of W per stage
constexpr int SF_STAGE_BYTES = 6144;                   // up to 4 atoms for A, then up to 4 + 4 for the two 128-row halves of W
constexpr int STG_WARP_BYTES = 32 * 32 * 4;            // per epilogue warp: one 32 x 32 fp32 staging tile
constexpr int EPI_WARPS = 16;
constexpr int SF_WARP = 2 + EPI_WARPS;                 // warp index of the scale-factor copier
constexpr int GEMM_THREADS = 32 * (3 + EPI_WARPS);
constexpr int SF_BUFS = 4;                             // scale-factor buffers in TMEM, 48 columns each (A at +0, W at +16)
constexpr int SF_BUF_COLS = 48;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_SF_COL = 256;                       // accumulator: columns [0,256); scale factors from 256
// Only the epilogues that restage through shared memory (RES, ROPE) reserve the 64 KB of staging tiles.  A fourth
// pipeline stage in the space the others save was measured: no gain for the block-scaled kinds (NVFP4 plain 111 vs 104 us),
// 5 % for bf16, so all kernels run 3 stages.
template <int EPI>
struct Pipe {
  static constexpr bool STAGING = EPI == KF_EPI_RES || EPI == KF_EPI_ROPE;
  // per epilogue warp: a 32 x 32 fp32 staging tile (RES / ROPE), else the 64 bias values of the warp's columns (the
  // kernel's shared memory leaves little L1, so bias loads inside the chunk loops would each wait on L2)
  static constexpr int STG_STRIDE = STAGING ? STG_WARP_BYTES : 256;
  static constexpr int STG_BYTES = EPI_WARPS * STG_STRIDE;
  static constexpr int STAGES = 3;
  static constexpr size_t SMEM = (size_t)STAGES * (TILE_BYTES + SF_STAGE_BYTES) + STG_BYTES + 256;
};
static_assert(TMEM_SF_COL + SF_BUFS * SF_BUF_COLS <= TMEM_COLS, "TMEM budget");

struct GemmArgs {
  const uint8_t *sfa, *sfw;
  const float *ts_a, *ts_w, *bias, *gamma, *R, *sin, *cos, *tso;
  void* C;
  uint8_t *Qo, *SFo;
  int M, N, K;
  int Ntok, prefix, H, d;
  int out_dtype, flags, out_fmt;
  int m_tiles, n_tiles, k_tiles, nkb4;
  int row_group, row_stride, row_offset;   // PLAIN: output row = (m / group) * stride + offset + m % group (group 0: identity)
  float* y_dbg;                            // QUANT: optional export of the values that were quantised (fp32 [M, N])
  unsigned int* err;
};

template <int KIND>
struct KindTraits;
template <>
struct KindTraits<KIND_MX8> { static constexpr int ATOMS = 1; };   // 128 elements per stage = 4 k-blocks of 32
template <>
struct KindTraits<KIND_NV4> { static constexpr int ATOMS = 4; };   // 256 elements per stage = 16 k-blocks of 16
template <>
struct KindTraits<KIND_MX4> { static constexpr int ATOMS = 2; };   // 256 elements per stage = 8 k-blocks of 32
template <>
struct KindTraits<KIND_BF16> { static constexpr int ATOMS = 0; };

// ------------------------------------------------------------------------------------------------ epilogue pieces
// tcgen05.ld hands every thread one accumulator ROW (32 consecutive columns per load).  Where global memory wants a
// warp to touch consecutive addresses (the fp32 residual stream, the rotary tables), the warp restages a 32 x 32
// chunk through a private shared-memory tile (128 bytes per row, 16-byte pieces XOR-swizzled by the row so both
// directions are bank-conflict free) and continues in the "coalesced" layout: in pass i (0..7) lane l owns the 4
// columns 4*(l&7).. of row 4*i + (l>>3), so a warp instruction covers 4 rows x 128 contiguous bytes.
__device__ __forceinline__ void stg_put(float* stg, int lane, const uint32_t (&r)[32]) {
  uint4* row = reinterpret_cast<uint4*>(stg + lane * 32);
#pragma unroll
  for (int c = 0; c < 8; ++c) row[c ^ (lane & 7)] = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
}
__device__ __forceinline__ float4 stg_get(const float* stg, int lane, int i) {
  const int row = 4 * i + (lane >> 3);
  return reinterpret_cast<const float4*>(stg + row * 32)[(lane & 7) ^ (row & 7)];
}
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ld4_stream(const float* p) {   // read once: do not keep the line in L1
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
// four-wide helpers on packed pairs (two issue slots per float4)
__device__ __forceinline__ float4 join4(float2 a, float2 b) { return make_float4(a.x, a.y, b.x, b.y); }
__device__ __forceinline__ float4 fma4(float4 a, float s, float4 b) {
  const float2 s2 = splat2(s);
  return join4(fma2(make_float2(a.x, a.y), s2, make_float2(b.x, b.y)), fma2(make_float2(a.z, a.w), s2, make_float2(b.z, b.w)));
}
__device__ __forceinline__ float4 fma4v(float4 a, float4 b, float4 c) {      // a * b + c
  return join4(fma2(make_float2(a.x, a.y), make_float2(b.x, b.y), make_float2(c.x, c.y)),
               fma2(make_float2(a.z, a.w), make_float2(b.z, b.w), make_float2(c.z, c.w)));
}
__device__ __forceinline__ float4 mul4v(float4 a, float4 b) {
  return join4(mul2(make_float2(a.x, a.y), make_float2(b.x, b.y)), mul2(make_float2(a.z, a.w), make_float2(b.z, b.w)));
}
__device__ __forceinline__ uint2 pack4(float4 v, int out_dtype) {
  uint2 o;
  if (out_dtype == KF_BF16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
  } else {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
  }
  return o;
}

// QUANT epilogue of one 32-column chunk in the row layout: the thread owns columns n0..n0+31 of row m = two nv4 blocks
// or one mx block, so block maxima need no shuffles and the per-block scale arithmetic is paid once per 16 / 32 values.
// The codes and scale bytes are the bit specification's quantisation (IEEE divisions, as in the row quantiser) of the
// values gelu(acc*ts + bias), optionally rounded to bf16, which y_dbg exports for the parity tests.

// values 16*h .. 16*h+15 of the chunk: bias + GELU (+ bf16 rounding), exported when asked; returns their maximum magnitude
__device__ __forceinline__ float quant_values16(const GemmArgs& g, const uint32_t (&r)[32], int h, float ts, const float* bsm, float* dbg, float (&v)[16]) {
  const float2 ts2 = splat2(ts);
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) {
    const int k = 16 * h + 4 * q4;
    const float4 bb = g.bias ? *reinterpret_cast<const float4*>(bsm + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    float2 a = gelu_erf2(fma2(make_float2(__uint_as_float(r[k]), __uint_as_float(r[k + 1])), ts2, make_float2(bb.x, bb.y)));
    float2 b = gelu_erf2(fma2(make_float2(__uint_as_float(r[k + 2]), __uint_as_float(r[k + 3])), ts2, make_float2(bb.z, bb.w)));
    if (g.flags & KF_Q_ROUND_BF16) {
      a = bf16_round2(a);
      b = bf16_round2(b);
    }
    v[4 * q4] = a.x;
    v[4 * q4 + 1] = a.y;
    v[4 * q4 + 2] = b.x;
    v[4 * q4 + 3] = b.y;
    if (dbg) *reinterpret_cast<float4*>(dbg + k) = make_float4(a.x, a.y, b.x, b.y);
  }
  float am = 0.f;
#pragma unroll
  for (int k = 0; k < 16; k += 2) am = max3(am, fabsf(v[k]), fabsf(v[k + 1]));
  return am;
}

__device__ __forceinline__ void quant_chunk(const GemmArgs& g, const uint32_t (&r)[32], float ts, const Nv4Scale& sco /* per-tensor scale of an nv4 output */, int m, int n0,
                                            const float* bsm /* the chunk's 32 bias values in shared memory */) {
  const bool div_true = !(g.flags & KF_Q_RECIP_DIV);
  const bool ok = m < g.M;
  float* dbg = (g.y_dbg != nullptr && ok) ? g.y_dbg + (size_t)m * g.N + n0 : nullptr;
  int by0, by1;
  if (g.out_fmt == KF_FMT_NV4) {
    // one 16-value block at a time: the exact division keeps a quotient per value live
    uint32_t o[4];
    {
      float v[16];
      const float am = quant_values16(g, r, 0, ts, bsm, dbg, v);
      if (g.flags & KF_Q_FAST_NV4) quant_nv4_fast<16>(v, am, sco.ts, sco.rcp_ts, o, by0);
      else quant_nv4<16>(v, am, sco, div_true, o, by0);
    }
    {
      float v[16];
      const float am = quant_values16(g, r, 1, ts, bsm, dbg, v);
      if (g.flags & KF_Q_FAST_NV4) quant_nv4_fast<16>(v, am, sco.ts, sco.rcp_ts, o + 2, by1);
      else quant_nv4<16>(v, am, sco, div_true, o + 2, by1);
    }
    if (ok) *reinterpret_cast<uint4*>(g.Qo + (size_t)m * (g.N >> 1) + (n0 >> 1)) = make_uint4(o[0], o[1], o[2], o[3]);
    // two scale bytes of this row for the chunk (rows beyond M inside the last tile get zeros)
    *reinterpret_cast<uint16_t*>(g.SFo + sf_offset(m, n0 >> 4, g.N >> 6)) = ok ? (uint16_t)(by0 | (by1 << 8)) : (uint16_t)0;
    return;
  }
  float va[16], vb[16];
  const float am = fmaxf(quant_values16(g, r, 0, ts, bsm, dbg, va), quant_values16(g, r, 1, ts, bsm, dbg, vb));
  if (g.out_fmt == KF_FMT_MX8) {
    uint32_t o[8];
    quant_mx8<16>(va, am, div_true, o, by0);
    quant_mx8<16>(vb, am, div_true, o + 4, by0);
    if (ok) {
      uint4* p = reinterpret_cast<uint4*>(g.Qo + (size_t)m * g.N + n0);
      p[0] = make_uint4(o[0], o[1], o[2], o[3]);
      p[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
    g.SFo[sf_offset(m, n0 >> 5, g.N >> 7)] = ok ? (uint8_t)by0 : (uint8_t)0;
  } else {
    uint32_t o[4];
    quant_mx4<16>(va, am, div_true, o, by0);
    quant_mx4<16>(vb, am, div_true, o + 2, by0);
    if (ok) *reinterpret_cast<uint4*>(g.Qo + (size_t)m * (g.N >> 1) + (n0 >> 1)) = make_uint4(o[0], o[1], o[2], o[3]);
    g.SFo[sf_offset(m, n0 >> 5, g.N >> 7)] = ok ? (uint8_t)by0 : (uint8_t)0;
  }
}

// PLAIN epilogue of one 32-column chunk in the row layout: the thread writes 64 (16-bit) or 128 (fp32) contiguous bytes.
__device__ __forceinline__ void plain_chunk(const GemmArgs& g, const uint32_t (&r)[32], float ts, uint8_t* dst_row, int n0, const float* bsm /* the chunk's 32 bias values in shared memory */) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float v[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 bb = g.bias ? *reinterpret_cast<const float4*>(bsm + 8 * q + 4 * h) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float b4[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = __uint_as_float(r[8 * q + 4 * h + e]);
        float x = (g.flags & KF_G_PRE_ROUND_BF16) ? bf16_round(a * ts) + b4[e] : fmaf(a, ts, b4[e]);   // the result may be rounded to bf16 before the bias
        if (g.flags & KF_G_GELU) x = gelu_erf(x);
        if (g.flags & KF_G_ROUND_BF16) x = bf16_round(x);
        v[4 * h + e] = x;
      }
    }
    if (dst_row) {
      if (g.out_dtype == KF_F32) {
        float4* d = reinterpret_cast<float4*>(dst_row + (size_t)(n0 + 8 * q) * 4);
        d[0] = make_float4(v[0], v[1], v[2], v[3]);
        d[1] = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        const uint2 lo = pack4(make_float4(v[0], v[1], v[2], v[3]), g.out_dtype), hi = pack4(make_float4(v[4], v[5], v[6], v[7]), g.out_dtype);
        *reinterpret_cast<uint4*>(dst_row + (size_t)(n0 + 8 * q) * 2) = make_uint4(lo.x, lo.y, hi.x, hi.y);
      }
    }
  }
}

// PLAIN / QUANT: the 64 bias values of the warp's columns go to its shared-memory slice (one coalesced load per tile,
// issued before the wait for the accumulator so that its L2 latency runs under that wait); the chunk loops then read
// them as broadcast float4s.
template <int EPI>
__device__ __forceinline__ void epilogue_bias_stage(const GemmArgs& g, int n0, float* stg, int lane) {
  if constexpr (!Pipe<EPI>::STAGING) {
    if (g.bias && n0 < g.N) {
      const float2 b2 = __ldg(reinterpret_cast<const float2*>(g.bias + n0) + lane);
      __syncwarp();                                // every lane has finished reading the previous tile's values
      reinterpret_cast<float2*>(stg)[lane] = b2;
      __syncwarp();
    }
  }
}

// ------------------------------------------------------------------------------------------------ the fused epilogues
// One epilogue warp's share of a tile: rows rbase..rbase+31 (thread `lane` holds row rbase + lane of the accumulator),
// columns n0..n0+63 (r0 = first 32, r1 = last 32).  `stg` is the warp's private 32 x 32 fp32 staging tile.
// What an epilogue can fetch before its accumulator exists: ROPE takes its two bias vectors, which then land during the
// wait for the accumulator instead of in front of the first arithmetic (qkv 90 -> 86 us).  The same for the first round
// of residual loads of RES was measured slower (proj 55 -> 59 us): 24 more registers live across the accumulator load
// spill under the 96-register cap of the 608-thread CTA.
struct EpiPre {
  float4 b0, b1;
};
template <int EPI>
__device__ __forceinline__ void epilogue_prefetch(const GemmArgs& g, int n0, int lane, EpiPre& p) {
  if constexpr (EPI == KF_EPI_ROPE) {
    const int c4 = 4 * (lane & 7);
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n0 >= g.N) return;
    p.b0 = g.bias ? ldg4(g.bias + n0 + c4) : z4;
    p.b1 = g.bias ? ldg4(g.bias + n0 + 32 + c4) : z4;
  }
}

template <int EPI>
__device__ __forceinline__ void epilogue_math(const GemmArgs& g, uint32_t (&r0)[32], uint32_t (&r1)[32], float ts, const Nv4Scale& sco, int rbase, int n0, float* stg,
                                              int lane, const EpiPre& pre) {
  const int c4 = 4 * (lane & 7);                // coalesced layout: this lane's 4 columns inside a 32-column chunk
  const int rsub = lane >> 3;                   // coalesced layout: row 4*i + rsub in pass i
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (EPI == KF_EPI_ROPE) {
    // the 64 columns of this warp are one head of q, k or v: r0 = first half, r1 = second half.  Both halves go
    // through the staging tile into the coalesced layout (the first stays in registers, the second is read back
    // pass by pass), where the rotary tables and the output rows are read / written 4 rows x 128 bytes at a time.
    const int which = n0 / g.d, h = (n0 - which * g.d) >> 6;
    const int nbatch = g.M / g.Ntok;
    const int b0 = rbase / g.Ntok, t0 = rbase - b0 * g.Ntok;   // one division per tile; rows advance from here
    const float4 b_lo = pre.b0, b_hi = pre.b1;
    float4 lo[8];
    stg_put(stg, lane, r0);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) lo[i] = fma4(stg_get(stg, lane, i), ts, b_lo);
    __syncwarp();
    stg_put(stg, lane, r1);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = rbase + 4 * i + rsub;
      if (m < g.M) {
        int b = b0, t = t0 + 4 * i + rsub;
        while (t >= g.Ntok) {
          t -= g.Ntok;
          ++b;
        }
        const float4 hi = fma4(stg_get(stg, lane, i), ts, b_hi);
        float4 ol = lo[i], oh = hi;
        if (which < 2 && t >= g.prefix) {
          const float* tab = g.sin + (size_t)(t - g.prefix) * 64 + c4;
          const float* tabc = g.cos + (size_t)(t - g.prefix) * 64 + c4;
          const float4 sl = ldg4(tab), cl = ldg4(tabc), sh = ldg4(tab + 32), ch = ldg4(tabc + 32);
          // lo' = lo*cos - hi*sin (tables of columns 0..31), hi' = hi*cos + lo*sin (tables of columns 32..63)
          ol = fma4v(hi, make_float4(-sl.x, -sl.y, -sl.z, -sl.w), mul4v(lo[i], cl));
          oh = fma4v(hi, ch, mul4v(lo[i], sh));
        }
        uint8_t* dst = static_cast<uint8_t*>(g.C) + (((((size_t)which * nbatch + b) * g.Ntok + t) * g.H + h) * 64 + c4) * 2;
        *reinterpret_cast<uint2*>(dst) = pack4(ol, g.out_dtype);
        *reinterpret_cast<uint2*>(dst + 64) = pack4(oh, g.out_dtype);
      }
    }
    __syncwarp();                                             // the staging tile is reused by the next tile
  } else if (EPI == KF_EPI_RES) {
    // two 32-column chunks, each restaged so that the fp32 residual is read and written 128 contiguous bytes per row.
    // Four rounds (chunk, half of the 8 passes); the residual loads of round r + 1 are in flight while round r is worked
    // out, so only the first round waits for its loads.
    auto load_round = [&](int r, float4 (&rr)[4]) {
      const int n = n0 + 32 * (r >> 1) + c4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = rbase + 4 * (4 * (r & 1) + i) + rsub;
        rr[i] = m < g.M ? ld4_stream(g.R + (size_t)m * g.N + n) : z4;
      }
    };
    auto do_round = [&](int r, const float4 (&rr)[4], const float4& b4, const float4& g4) {
      const int n = n0 + 32 * (r >> 1) + c4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = rbase + 4 * (4 * (r & 1) + i) + rsub;
        const float4 v = fma4(stg_get(stg, lane, 4 * (r & 1) + i), ts, b4);
        if (m < g.M)
          *reinterpret_cast<float4*>(static_cast<float*>(g.C) + (size_t)m * g.N + n) =
              fma4v(g4, v, rr[i]);
      }
    };
    float4 rra[4], rrb[4];
    load_round(0, rra);
    const float4 b40 = g.bias ? ldg4(g.bias + n0 + c4) : z4, g40 = ldg4(g.gamma + n0 + c4);
    const float4 b41 = g.bias ? ldg4(g.bias + n0 + 32 + c4) : z4, g41 = ldg4(g.gamma + n0 + 32 + c4);
    stg_put(stg, lane, r0);
    __syncwarp();
    load_round(1, rrb);
    do_round(0, rra, b40, g40);
    load_round(2, rra);
    do_round(1, rrb, b40, g40);
    __syncwarp();                                             // the staging tile is reused by the second chunk
    stg_put(stg, lane, r1);
    __syncwarp();
    load_round(3, rrb);
    do_round(2, rra, b41, g41);
    do_round(3, rrb, b41, g41);
    __syncwarp();                                             // ... and by the next tile
  } else if (EPI == KF_EPI_PLAIN) {
    const int m = rbase + lane;
    uint8_t* dst_row = nullptr;
    if (m < g.M) {
      const int64_t orow = g.row_group > 0 ? (int64_t)(m / g.row_group) * g.row_stride + g.row_offset + m % g.row_group : m;
      dst_row = static_cast<uint8_t*>(g.C) + (size_t)orow * g.N * (g.out_dtype == KF_F32 ? 4 : 2);
    }
    plain_chunk(g, r0, ts, dst_row, n0, stg);
    plain_chunk(g, r1, ts, dst_row, n0 + 32, stg + 32);
  } else {   // KF_EPI_QUANT: gelu(acc*ts + bias) -> codes + blocked scales of format out_fmt
    quant_chunk(g, r0, ts, sco, rbase + lane, n0, stg);
    quant_chunk(g, r1, ts, sco, rbase + lane, n0 + 32, stg + 32);
  }
}

}  // namespace kf
