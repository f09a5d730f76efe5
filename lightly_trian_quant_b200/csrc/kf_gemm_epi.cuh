// Shared pieces of the block-scaled GEMM kernels: argument block, per-format traits and the fused epilogues
// (PLAIN / RES / ROPE / QUANT) as one device function that works on a 32-row x 64-column piece of the accumulator held in
// registers.  Epilogue math per infer-opt/round13_mxfp8_full/impl/mgx_core.cu:308-426 and
// infer-opt/round14_fp4_full/impl/fp4g_core.cu:309-382.
//
// Every epilogue works in the layout tcgen05.ld delivers: thread `lane` of a warp owns 64 consecutive columns of ONE
// output row.  That is 128 contiguous bytes of a 16-bit output (exactly one [token, head] row of the q/k/v layout) or
// 256 contiguous bytes of an fp32 one, which the thread moves with 256-bit global loads / stores (ld/st.global.v8): every
// access is a whole 32-byte sector, so nothing is restaged through shared memory; the only shared memory the epilogue
// warps use holds the bias (and LayerScale) values: the whole vector of the launch, loaded once per CTA, or a 64-value
// slice per warp and tile where the operand ring leaves no room for the vector.
#pragma once
#include "kf_sm100.cuh"

namespace kf {

constexpr int KIND_MX8 = KF_FMT_MX8, KIND_NV4 = KF_FMT_NV4, KIND_MX4 = KF_FMT_MX4, KIND_BF16 = KF_FMT_BF16;
constexpr int BM = 128, BN = 256, BKB = 128;          // tile rows, tile columns, K bytes per stage
constexpr int A_BYTES = BM * BKB, TILE_BYTES = (BM + BN) * BKB;   // 16 KB of A, then 32 KB of W per stage
constexpr int SF_STAGE_BYTES = 6144;                   // up to 4 atoms for A, then up to 4 + 4 for the two 128-row halves of W
constexpr int EPI_WARPS = 16;
constexpr int EPI_WARP0 = 4;                           // warps 0..3: TMA producer, MMA issuer, scale-factor copier, spare
constexpr int GEMM_THREADS = 32 * (EPI_WARP0 + EPI_WARPS);
constexpr int SF_BUFS = 4;                             // scale-factor buffers in TMEM, 48 columns each (A at +0, W at +16)
constexpr int SF_BUF_COLS = 48;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_SF_COL = 256;                       // accumulator: columns [0,256); scale factors from 256
constexpr int SLICE_FLOATS = 128;                      // per epilogue warp: 64 bias values, then 64 LayerScale values (RES)
constexpr int ROPE_SLAB_FLOATS = 32 * 64;              // per TMEM lane quarter: 32 rows x (32 sin | 32 cos) values of the rotary tables
static_assert(TMEM_SF_COL + SF_BUFS * SF_BUF_COLS <= TMEM_COLS, "TMEM budget");

struct GemmArgs {
  const uint8_t *sfa, *sfw;
  const float *ts_a, *ts_w, *bias, *gamma, *R, *sin, *cos, *tso;
  void* C;
  uint8_t *Qo, *SFo;
  int M, N, K;
  int Ntok, prefix, H, d;
  int out_dtype, flags, out_fmt;
  int m_tiles, n_tiles, k_tiles, nkb4, stages;
  int row_group, row_stride, row_offset;   // PLAIN, RES: output row = (m / group) * stride + offset + m % group (group 0: identity)
  int m_tiles_pb, a_rows_pb, w_rows_pb;    // batched products (m_tiles_pb > 0): row tiles, A rows and W rows per product
  int vec_floats;                          // > 0: the whole bias vector (and for RES the LayerScale vector behind it) sits in shared memory for the launch
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

// ------------------------------------------------------------------------------------------------ 256-bit global accesses
struct F8 {
  float v[8];
};
__device__ __forceinline__ F8 ldg8_stream(const float* p) {   // 32-byte aligned; read once: do not keep the line in L1
  F8 r;
  asm volatile("ld.global.L1::no_allocate.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ F8 ldg8_nc(const float* p) {       // read-only data shared by several warps (rotary tables)
  F8 r;
  asm volatile("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ float4 ldg4_nc(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void stg8(void* p, float a, float b, float c, float d, float e, float f, float g, float h) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d), "f"(e), "f"(f), "f"(g), "f"(h)
               : "memory");
}
__device__ __forceinline__ void stg8w(void* p, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]),
               "r"(w[6]), "r"(w[7])
               : "memory");
}
// two fp32 -> one 32-bit word of two bf16 / f16 values (first value in the low half)
__device__ __forceinline__ uint32_t pack2(float a, float b, int out_dtype) {
  if (out_dtype == KF_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------------------ QUANT
// QUANT epilogue of one 32-column chunk: the thread owns columns n0..n0+31 of row m = two nv4 blocks or one mx block, so
// block maxima need no shuffles and the per-block scale arithmetic is paid once per 16 / 32 values.
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
    uint32_t o[4];
    float va[16], vb[16];
    const float am0 = quant_values16(g, r, 0, ts, bsm, dbg, va), am1 = quant_values16(g, r, 1, ts, bsm, dbg, vb);
    if (g.flags & KF_Q_FAST_NV4) {
      quant_nv4_fast<16>(va, am0, sco.ts, sco.rcp_ts, o, by0);
      quant_nv4_fast<16>(vb, am1, sco.ts, sco.rcp_ts, o + 2, by1);
    } else {
      quant_nv4_pair16(va, am0, vb, am1, sco, div_true, o, by0, by1);
    }
    if (ok) *reinterpret_cast<uint4*>(g.Qo + (size_t)m * (g.N >> 1) + (n0 >> 1)) = make_uint4(o[0], o[1], o[2], o[3]);
    // two scale bytes of this row for the chunk (rows beyond M inside the last tile get zeros)
    *reinterpret_cast<uint16_t*>(g.SFo + sf_offset(m, n0 >> 4, g.N >> 6)) = ok ? (uint16_t)(by0 | (by1 << 8)) : (uint16_t)0;
    return;
  }
  float va[16], vb[16];
  const float am = amax_nan(quant_values16(g, r, 0, ts, bsm, dbg, va), quant_values16(g, r, 1, ts, bsm, dbg, vb));
  if (g.out_fmt == KF_FMT_MX8) {
    uint32_t o[8];
    quant_mx8<16>(va, am, div_true, o, by0);
    quant_mx8<16>(vb, am, div_true, o + 4, by0);
    if (ok) stg8w(g.Qo + (size_t)m * g.N + n0, o);
    g.SFo[sf_offset(m, n0 >> 5, g.N >> 7)] = ok ? (uint8_t)by0 : (uint8_t)0;
  } else {
    uint32_t o[4];
    quant_mx4<16>(va, am, div_true, o, by0);
    quant_mx4<16>(vb, am, div_true, o + 2, by0);
    if (ok) *reinterpret_cast<uint4*>(g.Qo + (size_t)m * (g.N >> 1) + (n0 >> 1)) = make_uint4(o[0], o[1], o[2], o[3]);
    g.SFo[sf_offset(m, n0 >> 5, g.N >> 7)] = ok ? (uint8_t)by0 : (uint8_t)0;
  }
}

// ------------------------------------------------------------------------------------------------ PLAIN
// PLAIN epilogue of one 32-column chunk: the thread writes 64 (16-bit) or 128 (fp32) contiguous bytes of its row.
__device__ __forceinline__ void plain_chunk(const GemmArgs& g, const uint32_t (&r)[32], float ts, uint8_t* dst_row, int n0, const float* bsm /* the chunk's 32 bias values in shared memory */) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {                 // 16 columns at a time
    float v[16];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float4 bb = g.bias ? *reinterpret_cast<const float4*>(bsm + 16 * q + 4 * h) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float b4[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = __uint_as_float(r[16 * q + 4 * h + e]);
        float x = (g.flags & KF_G_PRE_ROUND_BF16) ? bf16_round(a * ts) + b4[e] : fmaf(a, ts, b4[e]);   // the result may be rounded to bf16 before the bias
        if (g.flags & KF_G_GELU) x = gelu_erf(x);
        if (g.flags & KF_G_ROUND_BF16) x = bf16_round(x);
        v[4 * h + e] = x;
      }
    }
    if (dst_row) {
      if (g.out_dtype == KF_F32) {
        float* d = reinterpret_cast<float*>(dst_row) + n0 + 16 * q;
        stg8(d, v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]);
        stg8(d + 8, v[8], v[9], v[10], v[11], v[12], v[13], v[14], v[15]);
      } else {
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = pack2(v[2 * e], v[2 * e + 1], g.out_dtype);
        stg8w(dst_row + (size_t)(n0 + 16 * q) * 2, w);
      }
    }
  }
}

// Fallback when the launch has no room for the whole vectors: the bias values (and for RES the LayerScale values) of the
// warp's 64 columns go to its shared-memory slice with one coalesced load per tile (the kernel's shared memory leaves
// little L1: a load inside the chunk loops would be an L2 round trip); the chunk loops then read them as broadcast
// float4s.  The store into the slice waits for the load, an L2 round trip at the head of the tile.
template <int EPI>
__device__ __forceinline__ void epilogue_slice_stage(const GemmArgs& g, int n0, float* slice, int lane) {
  if (n0 >= g.N) return;
  float2 b2 = make_float2(0.f, 0.f), g2 = make_float2(0.f, 0.f);
  if (g.bias) b2 = __ldg(reinterpret_cast<const float2*>(g.bias + n0) + lane);
  if (EPI == KF_EPI_RES) g2 = __ldg(reinterpret_cast<const float2*>(g.gamma + n0) + lane);
  __syncwarp();                                // every lane has finished reading the previous tile's values
  reinterpret_cast<float2*>(slice)[lane] = b2;
  if (EPI == KF_EPI_RES) reinterpret_cast<float2*>(slice + 64)[lane] = g2;
  __syncwarp();
}

// ------------------------------------------------------------------------------------------------ ROPE table slab
// Rotary tables whose columns 32..63 repeat columns 0..31 (KF_G_ROPE_HALF; true for the axial tables of DINOv3, where the
// angle vector is concatenated with itself): the 4 warps that share a TMEM lane quarter (the 4 heads of a 256-column tile)
// need the same 32 table rows.  Together they fetch them with coalesced loads BEFORE the wait for the accumulator (the L2
// latency runs under that wait, 4 float4 per thread held in registers), then park them in the quarter's slab:
// row j = [sin 0..31 | cos 0..31] of token rbase + j, 16-byte pieces XOR-swizzled by the row so that the row-layout reads
// of the epilogue (lane = row) are free of bank conflicts.
struct RopeSlabRegs {
  float4 v[4];
};
__device__ __forceinline__ void rope_slab_fetch(const GemmArgs& g, int rbase, int tid /* 0..127 within the quarter */, RopeSlabRegs& x) {
  const int f = tid & 15;                                            // piece of the row: 0..7 sin, 8..15 cos
  const float* tab = (f < 8 ? g.sin : g.cos) + ((f & 7) << 2);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int m = rbase + (tid >> 4) + 8 * u;
    x.v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < g.M) {
      const int t = m % g.Ntok;
      if (t >= g.prefix) x.v[u] = __ldg(reinterpret_cast<const float4*>(tab + (size_t)(t - g.prefix) * 64));
    }
  }
}
__device__ __forceinline__ void rope_slab_store(float* slab, int tid, const RopeSlabRegs& x) {
  const int f = tid & 15;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int row = (tid >> 4) + 8 * u;
    *reinterpret_cast<float4*>(slab + row * 64 + ((f ^ (row & 7)) << 2)) = x.v[u];
  }
}
__device__ __forceinline__ void quarter_barrier(int quarter) { asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory"); }

// ------------------------------------------------------------------------------------------------ the fused epilogues
// One epilogue warp's share of a tile: rows rbase..rbase+31 (thread `lane` holds row rbase + lane of the accumulator),
// columns n0..n0+63 (r0 = first 32, r1 = last 32).  `slice` / `gslice` point at the bias / LayerScale values of these 64 columns in shared memory.
template <int EPI>
__device__ __forceinline__ void epilogue_math(const GemmArgs& g, uint32_t (&r0)[32], uint32_t (&r1)[32], float ts, const Nv4Scale& sco, int rbase, int n0,
                                              const float* slice, const float* gslice /* RES: the LayerScale values of the warp's 64 columns */,
                                              const float* slab /* ROPE: the quarter's table rows in shared memory, or null */, int lane,
                                              int m_end /* first row past the product: M, or the end of the tile's product in a batched launch */) {
  const int m = rbase + lane;
  if (EPI == KF_EPI_ROPE) {
    // the 64 columns of this warp are one head of q, k or v and the thread's 64 values are one [token, head] row of the
    // output: r0 = first half, r1 = second half of the rotation pairs, so the rotary embedding needs no data exchange:
    //   lo' = lo*cos_lo - hi*sin_lo (tables of columns 0..31), hi' = hi*cos_hi + lo*sin_hi (tables of columns 32..63).
    // With KF_G_ROPE_HALF the table row of every token of the warp's quarter is already in shared memory (rope_slab_*).
    if (m >= g.M) return;
    const int which = n0 / g.d, h = (n0 - which * g.d) >> 6;
    const int b = m / g.Ntok, t = m - b * g.Ntok;
    const int nbatch = g.M / g.Ntok;
    const bool rot = which < 2 && t >= g.prefix;
    const float* sn = g.sin + (size_t)(rot ? t - g.prefix : 0) * 64;
    const float* cs = g.cos + (size_t)(rot ? t - g.prefix : 0) * 64;
    const float* srow = slab + lane * 64;
    uint8_t* dst = static_cast<uint8_t*>(g.C) + ((((size_t)which * nbatch + b) * g.Ntok + t) * g.H + h) * 128;
    uint32_t wlo[8], whi[8];                    // 16 output columns of each half: stored as soon as they are complete
    const float2 ts2 = splat2(ts);
#pragma unroll
    for (int c = 0; c < 8; ++c) {               // 4 rotation pairs at a time (few values live: the thread already holds 64 accumulators)
      float2 lo[2], hi[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 4 * c + 2 * e;
        lo[e] = fma2(make_float2(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1])), ts2, *reinterpret_cast<const float2*>(slice + j));
        hi[e] = fma2(make_float2(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1])), ts2, *reinterpret_cast<const float2*>(slice + 32 + j));
      }
      float2 ol[2] = {lo[0], lo[1]}, oh[2] = {hi[0], hi[1]};
      if (rot) {
        float4 s4, c4;                          // sin / cos of the 4 pairs: first for the lo outputs, then for the hi outputs
        if (slab != nullptr) {                  // both halves of the tables are the same 32 values
          s4 = *reinterpret_cast<const float4*>(srow + ((c ^ (lane & 7)) << 2));
          c4 = *reinterpret_cast<const float4*>(srow + (((c + 8) ^ (lane & 7)) << 2));
        } else {
          s4 = ldg4_nc(sn + 4 * c);
          c4 = ldg4_nc(cs + 4 * c);
        }
        ol[0] = fma2(hi[0], make_float2(-s4.x, -s4.y), mul2(lo[0], make_float2(c4.x, c4.y)));
        ol[1] = fma2(hi[1], make_float2(-s4.z, -s4.w), mul2(lo[1], make_float2(c4.z, c4.w)));
        if (slab == nullptr) {
          s4 = ldg4_nc(sn + 32 + 4 * c);
          c4 = ldg4_nc(cs + 32 + 4 * c);
        }
        oh[0] = fma2(hi[0], make_float2(c4.x, c4.y), mul2(lo[0], make_float2(s4.x, s4.y)));
        oh[1] = fma2(hi[1], make_float2(c4.z, c4.w), mul2(lo[1], make_float2(s4.z, s4.w)));
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        wlo[2 * (c & 3) + e] = pack2(ol[e].x, ol[e].y, g.out_dtype);
        whi[2 * (c & 3) + e] = pack2(oh[e].x, oh[e].y, g.out_dtype);
      }
      if ((c & 3) == 3) {
        stg8w(dst + 32 * (c >> 2), wlo);
        stg8w(dst + 64 + 32 * (c >> 2), whi);
      }
    }
  } else if (EPI == KF_EPI_RES) {
    // out = R + gamma * (acc*ts + bias) on the thread's 256 contiguous bytes of the fp32 residual row: eight 32-byte pieces,
    // four residual loads in flight ahead of the arithmetic.
    if (m >= g.M) return;
    const float* rrow = g.R + (size_t)m * g.N + n0;
    const int64_t orow = g.row_group > 0 ? (int64_t)(m / g.row_group) * g.row_stride + g.row_offset + m % g.row_group : m;   // the output may be a longer stream
    float* crow = static_cast<float*>(g.C) + (size_t)orow * g.N + n0;
    const float2 ts2 = splat2(ts);
    F8 rr[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) rr[c] = ldg8_stream(rrow + 8 * c);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint32_t* acc = c < 4 ? &r0[8 * c] : &r1[8 * (c - 4)];
      const F8 cur = rr[c & 3];
      if (c + 4 < 8) rr[c & 3] = ldg8_stream(rrow + 8 * (c + 4));
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const float2 bb = *reinterpret_cast<const float2*>(slice + 8 * c + e), gg = *reinterpret_cast<const float2*>(gslice + 8 * c + e);
        const float2 v = fma2(make_float2(__uint_as_float(acc[e]), __uint_as_float(acc[e + 1])), ts2, bb);
        const float2 w = fma2(gg, v, make_float2(cur.v[e], cur.v[e + 1]));
        o[e] = w.x;
        o[e + 1] = w.y;
      }
      stg8(crow + 8 * c, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
    }
  } else if (EPI == KF_EPI_PLAIN) {
    uint8_t* dst_row = nullptr;
    if (m < m_end) {
      const int64_t orow = g.row_group > 0 ? (int64_t)(m / g.row_group) * g.row_stride + g.row_offset + m % g.row_group : m;
      dst_row = static_cast<uint8_t*>(g.C) + (size_t)orow * g.N * (g.out_dtype == KF_F32 ? 4 : 2);
    }
    plain_chunk(g, r0, ts, dst_row, n0, slice);
    plain_chunk(g, r1, ts, dst_row, n0 + 32, slice + 32);
  } else {   // KF_EPI_QUANT: gelu(acc*ts + bias) -> codes + blocked scales of format out_fmt
    quant_chunk(g, r0, ts, sco, m, n0, slice);
    quant_chunk(g, r1, ts, sco, m, n0 + 32, slice + 32);
  }
}

// First A / C row of row tile m_blk and the first row past its product (batched launches: row tiles never straddle two
// products, the last tile of a product is cut at the product's end); the first W row of column tile n_blk.
__device__ __forceinline__ int tile_row0(const GemmArgs& g, int m_blk, int& row_end) {
  if (g.m_tiles_pb > 0) {
    const int b = m_blk / g.m_tiles_pb, mt = m_blk - b * g.m_tiles_pb;
    row_end = (b + 1) * g.a_rows_pb;
    return b * g.a_rows_pb + mt * BM;
  }
  row_end = g.M;
  return m_blk * BM;
}
__device__ __forceinline__ int tile_wrow0(const GemmArgs& g, int m_blk, int n_blk) {
  return (g.m_tiles_pb > 0 ? (m_blk / g.m_tiles_pb) * g.w_rows_pb : 0) + n_blk * BN;
}

// ------------------------------------------------------------------------------------------------ tile schedules and the epilogue warps' loop
// The i-th tile of a persistent CTA: tiles start, start + step, ... of the row-major tile grid (n_fixed < 0), or a fixed
// column block with the row blocks start, start + step, ... (a weight-stationary schedule).
struct TileSched {
  int start, step, total, n_tiles, n_fixed;     // n_fixed < 0: row-major walk over (m, n); else the column block every tile uses
  __device__ __forceinline__ bool get(int i, int& m_blk, int& n_blk) const {
    const int idx = start + i * step;
    if (idx >= total) return false;
    if (n_fixed >= 0) {
      m_blk = idx;
      n_blk = n_fixed;
    } else {
      m_blk = idx / n_tiles;
      n_blk = idx - m_blk * n_tiles;
    }
    return true;
  }
};

// Body of the 16 epilogue warps (warp = (TMEM lane quarter, 64-column group)): per tile, stage the bias slice (and fetch the
// rotary-table rows), wait for the accumulator, take the warp's 32 x 64 piece into registers, hand TMEM back at once and
// run the fused epilogue on the registers while the next tile's main loop fills the accumulator again.
template <int EPI>
__device__ __forceinline__ void epilogue_warps(const GemmArgs& g, const TileSched& sched, uint32_t tmem_base, uint64_t* tfull, uint64_t* tempty, float* slices,
                                               float* slabs, const WaitCtx& ctx, int warp, int lane) {
  const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31 are the ones this warp may read
  const int cg = (warp - EPI_WARP0) >> 2;       // which 64-column group of the 256-column tile
  float* slice = slices + (warp - EPI_WARP0) * SLICE_FLOATS;
  // Where the launch left room for it, the bias vector (and the LayerScale vector) is brought into shared memory once per
  // CTA instead of 64 values per warp and tile: that load was an L2 round trip (400-700 clk) at the head of every tile of
  // warps that are the busy role of these kernels.
  const bool vec = g.vec_floats > 0;
  if (vec) {
    const int tid = (warp - EPI_WARP0) * 32 + lane;
    for (int i = tid; i < g.N; i += EPI_WARPS * 32) {
      slices[i] = g.bias ? __ldg(g.bias + i) : 0.f;
      if (EPI == KF_EPI_RES) slices[g.N + i] = __ldg(g.gamma + i);
    }
    asm volatile("bar.sync 5, %0;" ::"r"(EPI_WARPS * 32) : "memory");
  }
  float ts = 1.f;
  if (g.ts_a) ts *= __ldg(g.ts_a);
  if (g.ts_w) ts *= __ldg(g.ts_w);
  const Nv4Scale sco = nv4_scale((EPI == KF_EPI_QUANT && g.out_fmt == KF_FMT_NV4) ? __ldg(g.tso) : 1.f);   // once per CTA: every global load here is an L2 round trip
  const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + cg * 64;
  int m_blk, n_blk;
  for (int lt = 0; sched.get(lt, m_blk, n_blk); ++lt) {
    int row_end;
    const int rbase = tile_row0(g, m_blk, row_end) + quarter * 32;
    const int n0 = n_blk * BN + cg * 64;        // first column of this warp's group
    uint32_t r0[32], r1[32];
    if (!vec) epilogue_slice_stage<EPI>(g, n0, slice, lane);
    const float* bsl = vec ? slices + n0 : slice;
    const float* gsl = vec ? slices + g.N + n0 : slice + 64;
    // ROPE with half tables: the quarter's table rows are fetched now and parked in shared memory after the wait
    const bool use_slab = EPI == KF_EPI_ROPE && (g.flags & KF_G_ROPE_HALF) != 0 && n_blk * BN < 2 * g.d;   // the tile holds q or k columns
    RopeSlabRegs tab;
    if (EPI == KF_EPI_ROPE && use_slab) rope_slab_fetch(g, rbase, cg * 32 + lane, tab);
    if (!mbar_wait(tfull, lt & 1, ctx, 4)) break;
    tc_fence_after();
    tmem_ld32(taddr, r0);
    tmem_ld32(taddr + 32, r1);
    tmem_ld_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(tempty);                       // the accumulator is in registers: hand TMEM back
    float* slab = nullptr;
    if (EPI == KF_EPI_ROPE && use_slab) {                      // all 4 warps of the quarter take this path together (it depends on the tile only)
      slab = slabs + quarter * ROPE_SLAB_FLOATS;
      quarter_barrier(quarter);                                // the previous tile's rows have been read by all four warps
      rope_slab_store(slab, cg * 32 + lane, tab);
      quarter_barrier(quarter);
    }
    if (n0 >= g.N) continue;                                   // column group past N in the last column tile
    epilogue_math<EPI>(g, r0, r1, ts, sco, rbase, n0, bsl, gsl, slab, lane, row_end);
  }
}

constexpr int REGS_LEAN = 40, REGS_EPI = 104;          // 128 * 40 + 512 * 104 <= 640 * 96, the allocation at launch
constexpr int REGS_LEAN_ROPE = 32, REGS_EPI_ROPE = 112; // the ROPE epilogue spills at 104 registers (64 accumulators + packed outputs + table values)

}  // namespace kf
