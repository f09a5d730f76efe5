// Memory-bound producers of the block-scaled operands: the stand-alone row quantiser (optionally bias + GELU first),
// LayerNorm fused with quantisation, and LayerNorm to a 16-bit tensor.  All three stream each input element once
// from HBM with 16-byte loads issued up front, keep the row segment in registers and write codes with 8/16-byte
// stores and scale factors as whole 32-bit words of the 128x4 blocked layout.
//
// Bit rules (identical to the reference's torch quantiser, infer-opt/round10_lowp_probe/impl/quant_ref.py:92-154):
//   mx8  byte = min(exp(fl32(amax/448)) + (mant != 0), 255);  q = e4m3_rn_sat(clamp(x * 2^(127 - max(byte,1)), +-448))
//   mx4  byte = min(exp(fl32(amax/6))   + (mant != 0), 254);  q = e2m1_rn_sat(x * 2^(127 - byte))
//   nv4  sf = e4m3_rn(min((amax/6)/ts, 448));  q = e2m1_rn_sat(x / (float(sf) * ts)), 0 when the scale is 0
// LN + quant is persistent (warps stride over the rows) with the LayerNorm weight and bias of the lane's columns held
// in registers, so the only per-row loads are the row itself.
#include "kf_sm100.cuh"

namespace kf {

// ------------------------------------------------------------------------------------------------ loads
template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
  const float4* p4 = reinterpret_cast<const float4*>(p);
  float4 a = __ldg(p4), b = __ldg(p4 + 1), c = __ldg(p4 + 2), d = __ldg(p4 + 3);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  v[8] = c.x; v[9] = c.y; v[10] = c.z; v[11] = c.w; v[12] = d.x; v[13] = d.y; v[14] = d.z; v[15] = d.w;
}

template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4* p4 = reinterpret_cast<const uint4*>(p);
  uint4 a = __ldg(p4), b = __ldg(p4 + 1);
  uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

template <>
__device__ __forceinline__ void load16<__half>(const __half* p, float (&v)[16]) {
  const uint4* p4 = reinterpret_cast<const uint4*>(p);
  uint4 a = __ldg(p4), b = __ldg(p4 + 1);
  uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// Gathers the scale bytes of 4 consecutive k-blocks (held by lanes lane0, lane0+STEP, ...) into one word on lane0.
template <int STEP>
__device__ __forceinline__ uint32_t gather_sf_word(int byte, int lane) {
  int base = lane & ~(4 * STEP - 1);
  uint32_t b0 = __shfl_sync(0xffffffffu, byte, base);
  uint32_t b1 = __shfl_sync(0xffffffffu, byte, base + STEP);
  uint32_t b2 = __shfl_sync(0xffffffffu, byte, base + 2 * STEP);
  uint32_t b3 = __shfl_sync(0xffffffffu, byte, base + 3 * STEP);
  return (b0 & 0xFF) | ((b1 & 0xFF) << 8) | ((b2 & 0xFF) << 16) | ((b3 & 0xFF) << 24);
}

// ------------------------------------------------------------------------------------------------ row quantiser
// One thread = 16 consecutive elements of one row.  mx8 / mx4: two adjacent lanes share a 1x32 block, eight lanes one
// scale word; nv4: one lane = one 1x16 block, four lanes one scale word.
template <typename T, int FMT>
__global__ void __launch_bounds__(256) quant_rows_kernel(const T* __restrict__ x, int64_t ldx, int M, int K, const float* __restrict__ ts_ptr,
                                                         const float* __restrict__ bias, int flags, uint8_t* __restrict__ q,
                                                         uint8_t* __restrict__ sf, int64_t items_valid, int64_t items_total) {
  const int lane = threadIdx.x & 31;
  const int per_row = K >> 4;
  int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool in_pad = w < items_total;          // inside the padded row range (scale bytes must be written)
  const bool valid = w < items_valid;           // a real row
  // 32-bit index arithmetic (the host checks that the item count fits); a power-of-two row length needs no division
  const uint32_t w32 = (uint32_t)w;
  int row, c16;
  if ((per_row & (per_row - 1)) == 0) {
    row = (int)(w32 >> (31 - __clz(per_row)));
    c16 = (int)(w32 & (uint32_t)(per_row - 1));
  } else {
    row = (int)(w32 / (uint32_t)per_row);
    c16 = (int)(w32 - (uint32_t)row * (uint32_t)per_row);
  }
  float v[16];
  if (valid) {
    load16<T>(x + (int64_t)row * ldx + c16 * 16, v);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  const Nv4Scale ts = nv4_scale(FMT == KF_FMT_NV4 ? __ldg(ts_ptr) : 1.f);
  if (flags & KF_Q_GELU) {
    if (valid) {
      const float4* b4 = reinterpret_cast<const float4*>(bias + c16 * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 bb = __ldg(b4 + i);
        v[4 * i] = gelu_erf(v[4 * i] + bb.x);
        v[4 * i + 1] = gelu_erf(v[4 * i + 1] + bb.y);
        v[4 * i + 2] = gelu_erf(v[4 * i + 2] + bb.z);
        v[4 * i + 3] = gelu_erf(v[4 * i + 3] + bb.w);
      }
    }
  }
  if (flags & KF_Q_ROUND_BF16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = bf16_round(v[i]);
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = amax_nan(amax, fabsf(v[i]));
  const bool div_true = !(flags & KF_Q_RECIP_DIV);
  int byte;
  if (FMT == KF_FMT_MX8) {
    amax = amax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    uint32_t o[4];
    quant_mx8<16>(v, amax, div_true, o, byte);
    if (valid) *reinterpret_cast<uint4*>(q + (int64_t)row * K + c16 * 16) = make_uint4(o[0], o[1], o[2], o[3]);
  } else if (FMT == KF_FMT_MX4) {
    amax = amax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    uint32_t o[2];
    quant_mx4<16>(v, amax, div_true, o, byte);
    if (valid) *reinterpret_cast<uint2*>(q + (int64_t)row * (K >> 1) + c16 * 8) = make_uint2(o[0], o[1]);
  } else {
    uint32_t o[2];
    quant_nv4<16>(v, amax, ts, div_true, o, byte);
    if (valid) *reinterpret_cast<uint2*>(q + (int64_t)row * (K >> 1) + c16 * 8) = make_uint2(o[0], o[1]);
  }
  if (!valid) byte = 0;
  constexpr int STEP = (FMT == KF_FMT_NV4) ? 1 : 2;                 // lanes per k-block
  uint32_t word = gather_sf_word<STEP>(byte, lane);
  if (in_pad && (lane & (4 * STEP - 1)) == 0) {
    int kb = (FMT == KF_FMT_NV4) ? c16 : (c16 >> 1);
    int nkb4 = (FMT == KF_FMT_NV4) ? (K >> 6) : (K >> 7);
    *reinterpret_cast<uint32_t*>(sf + sf_offset(row, kb, nkb4)) = word;
  }
}

// ------------------------------------------------------------------------------------------------ LayerNorm (+ quant)
// One warp per row; lane l holds the 8 consecutive elements [i*256 + l*8, +8) for i < NV (d = NV*256), as two pieces of
// four.  With BLK16 the lane's chunks pair up into runs of 16 consecutive elements (whole NVFP4 blocks): chunks 2h and
// 2h + 1 are [h*512 + l*16, +16).  The lane then reads the four pieces of a run in the rotated order
// (k + (l >> 1)) & 3, k = 0..3: with a lane stride of 64 bytes the eight lanes of a 128-bit shared-memory access would
// otherwise meet in two bank groups (four passes per load); rotated they cover all eight.  LayerNorm does not care about
// the order, the affine parameters are loaded in the same order, and the quantiser undoes it on its packed output.
// LAY_SWAP is the chunk layout read from shared memory: lanes 4..7 of every eight take the two pieces of a chunk in the
// other order (at a lane stride of 32 bytes lanes l and l + 4 would otherwise share their banks: two passes per load).
constexpr int LAY_CHUNK = 0, LAY_BLK16 = 1, LAY_SWAP = 2;
template <int LAY>
__device__ __forceinline__ int ln_piece_offset(int i, int half, int lane) {
  if (LAY == LAY_BLK16) return (i >> 1) * 512 + lane * 16 + (((2 * (i & 1) + half) + ((lane >> 1) & 3)) & 3) * 4;
  if (LAY == LAY_SWAP) return i * 256 + lane * 8 + (half ^ ((lane >> 2) & 1)) * 4;
  return i * 256 + lane * 8 + half * 4;
}

template <int NV, int LAY = LAY_CHUNK>
__device__ __forceinline__ void ln_affine_load(const float* __restrict__ w, const float* __restrict__ b, int lane, float (&ww)[NV][8], float (&bb)[NV][8]) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + ln_piece_offset<LAY>(i, 0, lane)));
    const float4 w1 = __ldg(reinterpret_cast<const float4*>(w + ln_piece_offset<LAY>(i, 1, lane)));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + ln_piece_offset<LAY>(i, 0, lane)));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(b + ln_piece_offset<LAY>(i, 1, lane)));
    ww[i][0] = w0.x; ww[i][1] = w0.y; ww[i][2] = w0.z; ww[i][3] = w0.w; ww[i][4] = w1.x; ww[i][5] = w1.y; ww[i][6] = w1.z; ww[i][7] = w1.w;
    bb[i][0] = b0.x; bb[i][1] = b0.y; bb[i][2] = b0.z; bb[i][3] = b0.w; bb[i][4] = b1.x; bb[i][5] = b1.y; bb[i][6] = b1.z; bb[i][7] = b1.w;
  }
}

// LayerNorm of one row with the affine parameters already in registers (the persistent kernels load them once per
// warp: re-reading them per row doubles the load instructions of a kernel that is otherwise one pass over x).
template <int NV, bool FROM_SMEM = false, int LAY = LAY_CHUNK>
__device__ __forceinline__ void ln_row(const float* xr, const float (&ww)[NV][8], const float (&bb)[NV][8], float eps,
                                       int lane, bool valid, float (&v)[NV][8]) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (valid) {
      const float4* pa = reinterpret_cast<const float4*>(xr + ln_piece_offset<LAY>(i, 0, lane));
      const float4* pc = reinterpret_cast<const float4*>(xr + ln_piece_offset<LAY>(i, 1, lane));
      float4 a, c;
      if (FROM_SMEM) {
        a = *pa;
        c = *pc;
      } else {
        a = __ldg(pa);
        c = __ldg(pc);
      }
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w; v[i][4] = c.x; v[i][5] = c.y; v[i][6] = c.z; v[i][7] = c.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }
  // statistics and affine step on packed pairs, the sums in one chain per 256-element group
  constexpr float inv_d = 1.0f / (NV * 256);
  float2 sp[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    sp[i] = add2(add2(make_float2(v[i][0], v[i][1]), make_float2(v[i][2], v[i][3])), add2(make_float2(v[i][4], v[i][5]), make_float2(v[i][6], v[i][7])));
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) s += sp[i].x + sp[i].y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float mean = s * inv_d;
  const float2 nmean = splat2(-mean);
  float2 c[NV][4], qp[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) c[i][j] = add2(make_float2(v[i][2 * j], v[i][2 * j + 1]), nmean);
    qp[i] = mul2(c[i][0], c[i][0]);
#pragma unroll
    for (int j = 1; j < 4; ++j) qp[i] = fma2(c[i][j], c[i][j], qp[i]);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) ss += qp[i].x + qp[i].y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float2 rstd = splat2(rsqrtf(ss * inv_d + eps));
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 y = fma2(mul2(c[i][j], rstd), make_float2(ww[i][2 * j], ww[i][2 * j + 1]), make_float2(bb[i][2 * j], bb[i][2 * j + 1]));
      v[i][2 * j] = y.x;
      v[i][2 * j + 1] = y.y;
    }
}

// Rows are streamed through shared memory: each warp owns a ring of LNQ_RING row buffers filled by 1-D bulk copies
// (cp.async.bulk + mbarrier), so two to three rows per warp (8-12 KB) are in flight while the warp normalises and
// quantises the current one; with 16 warps per SM that keeps well over 100 KB of HBM reads outstanding per SM, which
// register-staged loads cannot (they stop while the warp computes).
constexpr int LNQ_RING = 3;

template <int NV, int FMT>
__global__ void __launch_bounds__(128, NV <= 4 ? 4 : 1) ln_quant_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                                       int M, int rows_pad, const float* __restrict__ ts_ptr, int flags, uint8_t* __restrict__ q,
                                                       uint8_t* __restrict__ sf, float* __restrict__ y_dbg, unsigned int* err) {
  constexpr int D = NV * 256;
  extern __shared__ __align__(128) uint8_t lsm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* ring = reinterpret_cast<float*>(lsm) + (size_t)warp * LNQ_RING * D;
  uint64_t* bars = reinterpret_cast<uint64_t*>(lsm + (size_t)4 * LNQ_RING * D * 4) + warp * LNQ_RING;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(lsm + (size_t)4 * LNQ_RING * D * 4 + 4 * LNQ_RING * 8);
  pdl_launch_dependents();                        // the next kernel of the stream may take the SMs this grid leaves
  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int i = 0; i < LNQ_RING; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();                                     // from here on global memory of the predecessors is read and written
  const WaitCtx ctx{abort_flag, err};
  const int W = gridDim.x * 4, gw = blockIdx.x * 4 + warp;
  auto issue = [&](int k) {                       // lane 0: start the copy of this warp's k-th row into slot k % RING
    const int r = gw + k * W;
    if (r < M) {
      mbar_expect_tx(&bars[k % LNQ_RING], D * 4);
      bulk_load_1d(ring + (size_t)(k % LNQ_RING) * D, x + (int64_t)r * D, D * 4, &bars[k % LNQ_RING]);
    }
  };
  if (lane == 0)
    for (int k = 0; k < LNQ_RING; ++k) issue(k);
  constexpr bool BLK16 = FMT == KF_FMT_NV4 && NV == 4;   // d = 1024 in NVFP4: a lane owns whole 16-value blocks
  constexpr int LAY = BLK16 ? LAY_BLK16 : LAY_SWAP;
  float ww[NV][8], bb[NV][8];
  ln_affine_load<NV, LAY>(w, b, lane, ww, bb);
  const Nv4Scale ts = nv4_scale(FMT == KF_FMT_NV4 ? __ldg(ts_ptr) : 1.f);
  const bool div_true = !(flags & KF_Q_RECIP_DIV);
  const bool rb = flags & KF_Q_ROUND_BF16;
  // persistent: warp gw of the grid takes rows gw, gw + W, gw + 2W, ... (rows M..rows_pad only get zero scale words)
  int k = 0;
  for (int row = gw; row < rows_pad; row += W, ++k) {
  const bool valid = row < M;
  const int slot = k % LNQ_RING;
  if (valid && !mbar_wait(&bars[slot], (k / LNQ_RING) & 1, ctx, 30)) break;
  float v[NV][8];
  ln_row<NV, true, LAY>(ring + (size_t)slot * D, ww, bb, eps, lane, valid, v);
  __syncwarp();                                   // every lane has its part of the row: the slot can be refilled
  if (lane == 0) {
    fence_proxy_async_smem();
    issue(k + LNQ_RING);
  }
  if constexpr (BLK16) {
    // d = 1024 in NVFP4 (the block path of the model).  The lane holds two whole blocks: elements [16 l, +16) in chunks
    // 0 and 1 and [512 + 16 l, +16) in chunks 2 and 3, so the block maxima and scalars need no exchange between lanes.
    // Both blocks are quantised together, their scalars on packed pairs; the two scale bytes of a lane are the same
    // byte of two scale words, put together over the four lanes of a word with two shuffles.
    float am[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      am[h] = 0.f;
#pragma unroll
      for (int i = 2 * h; i < 2 * h + 2; ++i) {
        if (rb) {
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const float2 t = bf16_round2(make_float2(v[i][j], v[i][j + 1]));
            v[i][j] = t.x;
            v[i][j + 1] = t.y;
          }
        }
        if (y_dbg && valid) {
          *reinterpret_cast<float4*>(y_dbg + (int64_t)row * D + ln_piece_offset<LAY_BLK16>(i, 0, lane)) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          *reinterpret_cast<float4*>(y_dbg + (int64_t)row * D + ln_piece_offset<LAY_BLK16>(i, 1, lane)) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
#pragma unroll
        for (int j = 0; j < 8; j += 2) am[h] = max3(am[h], fabsf(v[i][j]), fabsf(v[i][j + 1]));
      }
    }
    const float(&blk0)[16] = *reinterpret_cast<const float(*)[16]>(&v[0][0]);
    const float(&blk1)[16] = *reinterpret_cast<const float(*)[16]>(&v[2][0]);
    uint32_t o[4];
    int by0, by1;
    quant_nv4_pair16(blk0, am[0], blk1, am[1], ts, div_true, o, by0, by1);
    {
      // piece k of the registers is piece (k + s) & 3 of the block: rotate the four 16-bit code groups of each block left by s
      const int sr = (lane >> 1) & 3;
      const uint32_t sh = (uint32_t)(sr & 1) * 16;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = (sr & 2) ? o[2 * h + 1] : o[2 * h], hi = (sr & 2) ? o[2 * h] : o[2 * h + 1];
        o[2 * h] = __funnelshift_l(hi, lo, sh);
        o[2 * h + 1] = __funnelshift_l(lo, hi, sh);
      }
    }
    if (valid) {
      uint8_t* qr = q + (int64_t)row * (D / 2) + lane * 8;
      *reinterpret_cast<uint2*>(qr) = make_uint2(o[0], o[1]);
      *reinterpret_cast<uint2*>(qr + D / 4) = make_uint2(o[2], o[3]);
    }
    // lanes 4g .. 4g+3 hold the bytes of k-blocks 4g .. 4g+3 (first half of the row) and 32 + 4g .. (second half)
    uint32_t pk = valid ? ((uint32_t)by0 | ((uint32_t)by1 << 16)) : 0u;              // byte 0: first word, byte 2: second
    pk |= __shfl_xor_sync(0xffffffffu, pk, 1) << 8;                                   // on even lanes: the bytes of lanes l, l + 1
    const uint32_t up = __shfl_xor_sync(0xffffffffu, pk, 2);                          // on lane 4g: the pairs of lanes 4g + 2, 4g + 3
    if ((lane & 3) == 0) {
      const uint32_t w0 = __byte_perm(pk, up, 0x5410), w1 = __byte_perm(pk, up, 0x7632);
      *reinterpret_cast<uint32_t*>(sf + sf_offset(row, lane, D >> 6)) = w0;
      *reinterpret_cast<uint32_t*>(sf + sf_offset(row, 32 + lane, D >> 6)) = w1;
    }
  } else {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (rb) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float2 t = bf16_round2(make_float2(v[i][j], v[i][j + 1]));
        v[i][j] = t.x;
        v[i][j + 1] = t.y;
      }
    }
    if (y_dbg && valid) {
      *reinterpret_cast<float4*>(y_dbg + (int64_t)row * D + ln_piece_offset<LAY_SWAP>(i, 0, lane)) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      *reinterpret_cast<float4*>(y_dbg + (int64_t)row * D + ln_piece_offset<LAY_SWAP>(i, 1, lane)) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
    }
    const bool swapped = (lane >> 2) & 1;                            // this lane holds the two pieces of the chunk in the other order
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j += 2) amax = max3(amax, fabsf(v[i][j]), fabsf(v[i][j + 1]));
    amax = amax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (FMT != KF_FMT_NV4) amax = amax_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int byte;
    const int col = i * 256 + lane * 8;
    if (FMT == KF_FMT_MX8) {
      uint32_t o[2];
      quant_mx8<8>(v[i], amax, div_true, o, byte);
      if (valid) *reinterpret_cast<uint2*>(q + (int64_t)row * D + col) = swapped ? make_uint2(o[1], o[0]) : make_uint2(o[0], o[1]);
    } else if (FMT == KF_FMT_MX4) {
      uint32_t o[1];
      quant_mx4<8>(v[i], amax, div_true, o, byte);
      if (valid) *reinterpret_cast<uint32_t*>(q + (int64_t)row * (D / 2) + (col >> 1)) = swapped ? __funnelshift_l(o[0], o[0], 16) : o[0];
    } else {
      uint32_t o[1];
      quant_nv4<8>(v[i], amax, ts, div_true, o, byte);
      if (valid) *reinterpret_cast<uint32_t*>(q + (int64_t)row * (D / 2) + (col >> 1)) = swapped ? __funnelshift_l(o[0], o[0], 16) : o[0];
    }
    if (!valid) byte = 0;
    constexpr int STEP = (FMT == KF_FMT_NV4) ? 2 : 4;               // lanes per k-block
    uint32_t word = gather_sf_word<STEP>(byte, lane);
    if ((lane & (4 * STEP - 1)) == 0) {
      int kb = col / ((FMT == KF_FMT_NV4) ? 16 : 32);
      constexpr int nkb4 = (FMT == KF_FMT_NV4) ? (D >> 6) : (D >> 7);
      *reinterpret_cast<uint32_t*>(sf + sf_offset(row, kb, nkb4)) = word;
    }
  }
  }
  }
}

template <int NV, typename TO>
__global__ void __launch_bounds__(128) ln_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                                      int M, TO* __restrict__ y) {
  constexpr int D = NV * 256;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= M) return;
  float v[NV][8], ww[NV][8], bb[NV][8];
  ln_affine_load<NV>(w, b, lane, ww, bb);
  ln_row<NV>(x + (int64_t)row * D, ww, bb, eps, lane, true, v);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if constexpr (sizeof(TO) == 2 && std::is_same<TO, __nv_bfloat16>::value) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[i][2 * j], v[i][2 * j + 1]);
        o[j] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(v[i][2 * j], v[i][2 * j + 1]);
        o[j] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(y + (int64_t)row * D + i * 256 + lane * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Final LayerNorm of the token stream [B, Ntok, D] with the row gather of the EoMT head: the first Q rows of every
// image (queries) go to qb [B*Q, D], rows >= Q + npre (patch tokens) go to xb [B*(Ntok-Q-npre), D], the cls / register
// rows in between are skipped.
template <int NV>
__global__ void __launch_bounds__(128) ln_tail_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                                      int M, int Ntok, int Q, int npre, __nv_bfloat16* __restrict__ qb, __nv_bfloat16* __restrict__ xb,
                                                      const __nv_bfloat16* __restrict__ wcls, const float* __restrict__ bcls, int ncls1,
                                                      __nv_bfloat16* __restrict__ cl) {
  constexpr int D = NV * 256;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int img = row / Ntok, t = row - img * Ntok;
  if (t >= Q && t < Q + npre) return;
  float v[NV][8], ww[NV][8], bb[NV][8];
  ln_affine_load<NV>(w, b, lane, ww, bb);
  ln_row<NV>(x + (int64_t)row * D, ww, bb, eps, lane, true, v);
  const int P = Ntok - Q - npre;
  __nv_bfloat16* y = t < Q ? qb + ((int64_t)img * Q + t) * D : xb + ((int64_t)img * P + (t - Q - npre)) * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[i][2 * j], v[i][2 * j + 1]);
      o[j] = *reinterpret_cast<uint32_t*>(&h);
      const float2 r = __bfloat1622float2(h);          // the class head sees the bf16 values that were stored
      v[i][2 * j] = r.x;
      v[i][2 * j + 1] = r.y;
    }
    *reinterpret_cast<uint4*>(y + i * 256 + lane * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // class head on the query rows: logits[c] = bf16(sum_k q[k] * W[c][k] + bias[c]), fp32 accumulation
  if (wcls != nullptr && t < Q) {
    for (int c = 0; c < ncls1; ++c) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const uint4 wq = __ldg(reinterpret_cast<const uint4*>(wcls + (int64_t)c * D + i * 256 + lane * 8));
        const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv[j]));
          acc = fmaf(v[i][2 * j], f.x, acc);
          acc = fmaf(v[i][2 * j + 1], f.y, acc);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) cl[((int64_t)img * Q + t) * ncls1 + c] = __float2bfloat16_rn(acc + bcls[c]);
    }
  }
}

// Copies a block of fp32 rows into every image of a token stream: dst[b, row_offset + r, :] = src[r, :] for r < R.
// The query rows that join the stream for the last blocks and the cls / register rows in front of the patch tokens.
__global__ void __launch_bounds__(256) broadcast_rows_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int R, int d4, int B, int64_t img_stride4,
                                                             int64_t row_offset4) {
  const int64_t n = (int64_t)R * d4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * B; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t bimg = i / n, e = i - bimg * n;
    dst[bimg * img_stride4 + row_offset4 + e] = __ldg(src + e);
  }
}

// ------------------------------------------------------------------------------------------------ host launchers
template <typename T>
static int launch_quant_rows(int fmt, const void* x, int64_t ldx, int M, int K, const float* ts, const float* bias, int flags, void* q, void* sf,
                             cudaStream_t st) {
  int64_t per_row = K / 16;
  int64_t valid = (int64_t)M * per_row, total = (int64_t)((M + 127) / 128 * 128) * per_row;
  KF_REQUIRE(total + 256 < (1ll << 32), "kf_quant_rows: M*K/16 = %lld work items do not fit the 32-bit index", (long long)total);
  unsigned grid = (unsigned)((total + 255) / 256);
  const T* xp = static_cast<const T*>(x);
  uint8_t *qp = static_cast<uint8_t*>(q), *sp = static_cast<uint8_t*>(sf);
  if (fmt == KF_FMT_MX8) quant_rows_kernel<T, KF_FMT_MX8><<<grid, 256, 0, st>>>(xp, ldx, M, K, ts, bias, flags, qp, sp, valid, total);
  else if (fmt == KF_FMT_NV4) quant_rows_kernel<T, KF_FMT_NV4><<<grid, 256, 0, st>>>(xp, ldx, M, K, ts, bias, flags, qp, sp, valid, total);
  else quant_rows_kernel<T, KF_FMT_MX4><<<grid, 256, 0, st>>>(xp, ldx, M, K, ts, bias, flags, qp, sp, valid, total);
  return cuda_status(cudaGetLastError(), "kf_quant_rows launch");
}

template <int NV>
static int launch_ln_quant(int fmt, const float* x, const float* w, const float* b, float eps, int M, const float* ts, int flags, void* q, void* sf,
                           float* y_dbg, cudaStream_t st) {
  int rows_pad = (M + 127) / 128 * 128;
  int sms = 0;
  int rc = device_sm_count(&sms);                        // of the CURRENT device
  if (rc != KF_OK) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  unsigned grid = (unsigned)((rows_pad + 3) / 4);
  uint8_t *qp = static_cast<uint8_t*>(q), *sp = static_cast<uint8_t*>(sf);
  unsigned int* err = dev_error_ptr();
  KF_REQUIRE(err != nullptr, "kf_ln_quant: device error word unavailable");
  const size_t smem = (size_t)4 * LNQ_RING * NV * 256 * 4 + 4 * LNQ_RING * 8 + 16;
  static int per_sm_cached[3][64] = {};                  // per (format, device) of this row width
  auto go = [&](auto kern) {
    // persistent: as many CTAs of 4 warps as are resident at once (4 per SM up to d = 1024, fewer for wider rows); a
    // grid beyond that would run its surplus as a second, nearly empty wave.  The attribute and the occupancy query are
    // per (kernel instance, device): worked out at the first call and kept.
    int per_sm = dev < 64 ? per_sm_cached[fmt][dev] : 0;
    if (per_sm == 0) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(ln_quant_kernel)");
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 128, smem);
      if (e != cudaSuccess) return cuda_status(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor(ln_quant_kernel)");
      if (per_sm < 1) per_sm = 1;
      if (per_sm > 4) per_sm = 4;
      if (dev < 64) per_sm_cached[fmt][dev] = per_sm;
    }
    if (grid > (unsigned)(sms * per_sm)) grid = (unsigned)(sms * per_sm);
    return cuda_status(launch_maybe_pdl(kern, dim3(grid), dim3(128), smem, st, x, w, b, eps, M, rows_pad, ts, flags, qp, sp, y_dbg, err), "kf_ln_quant launch");
  };
  if (fmt == KF_FMT_MX8) return go(ln_quant_kernel<NV, KF_FMT_MX8>);
  if (fmt == KF_FMT_NV4) return go(ln_quant_kernel<NV, KF_FMT_NV4>);
  return go(ln_quant_kernel<NV, KF_FMT_MX4>);
}

template <int NV>
static int launch_ln_rows(const float* x, const float* w, const float* b, float eps, int M, int out_dtype, void* y, cudaStream_t st) {
  unsigned grid = (unsigned)((M + 3) / 4);
  if (out_dtype == KF_BF16) ln_rows_kernel<NV, __nv_bfloat16><<<grid, 128, 0, st>>>(x, w, b, eps, M, static_cast<__nv_bfloat16*>(y));
  else ln_rows_kernel<NV, __half><<<grid, 128, 0, st>>>(x, w, b, eps, M, static_cast<__half*>(y));
  return cuda_status(cudaGetLastError(), "kf_ln_rows launch");
}

template <int NV>
static int launch_ln_tail(const float* x, const float* w, const float* b, float eps, int M, int Ntok, int Q, int npre, void* qb, void* xb, const void* wcls,
                          const float* bcls, int ncls1, void* cl, cudaStream_t st) {
  ln_tail_kernel<NV><<<(unsigned)((M + 3) / 4), 128, 0, st>>>(x, w, b, eps, M, Ntok, Q, npre, static_cast<__nv_bfloat16*>(qb), static_cast<__nv_bfloat16*>(xb),
                                                              static_cast<const __nv_bfloat16*>(wcls), bcls, ncls1, static_cast<__nv_bfloat16*>(cl));
  return cuda_status(cudaGetLastError(), "kf_ln_tail launch");
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace kf

using namespace kf;

extern "C" int kf_quant_rows(int fmt, int in_dtype, const void* x, int64_t ldx, int M, int K, const float* ts, const float* bias, int flags, void* q,
                             void* sf, void* stream) {
  KF_REQUIRE(fmt == KF_FMT_MX8 || fmt == KF_FMT_NV4 || fmt == KF_FMT_MX4, "kf_quant_rows: unknown format %d", fmt);
  KF_REQUIRE(in_dtype == KF_F32 || in_dtype == KF_BF16 || in_dtype == KF_F16, "kf_quant_rows: unknown input dtype %d", in_dtype);
  KF_REQUIRE(M >= 0 && K > 0 && K % 128 == 0, "kf_quant_rows: K=%d must be a positive multiple of 128 (M=%d)", K, M);
  if (M == 0) return KF_OK;
  KF_REQUIRE(x && q && sf, "kf_quant_rows: null tensor pointer");
  KF_REQUIRE(ldx >= K && ldx % 8 == 0, "kf_quant_rows: row stride %lld must be >= K and a multiple of 8", (long long)ldx);
  KF_REQUIRE(aligned16(x) && aligned16(q) && aligned16(sf), "kf_quant_rows: tensors must be 16-byte aligned");
  KF_REQUIRE(fmt != KF_FMT_NV4 || ts, "kf_quant_rows: nv4 needs the per-tensor scale pointer");
  KF_REQUIRE(!(flags & KF_Q_GELU) || (bias && aligned16(bias)), "kf_quant_rows: KF_Q_GELU needs a 16-byte aligned bias");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (in_dtype == KF_F32) return launch_quant_rows<float>(fmt, x, ldx, M, K, ts, bias, flags, q, sf, st);
  if (in_dtype == KF_BF16) return launch_quant_rows<__nv_bfloat16>(fmt, x, ldx, M, K, ts, bias, flags, q, sf, st);
  return launch_quant_rows<__half>(fmt, x, ldx, M, K, ts, bias, flags, q, sf, st);
}

extern "C" int kf_ln_quant(int fmt, const float* x, const float* w, const float* b, float eps, int M, int d, const float* ts, int flags, void* q,
                           void* sf, float* y_dbg, void* stream) {
  KF_REQUIRE(fmt == KF_FMT_MX8 || fmt == KF_FMT_NV4 || fmt == KF_FMT_MX4, "kf_ln_quant: unknown format %d", fmt);
  KF_REQUIRE(M >= 0 && d > 0 && d % 256 == 0 && d <= 2048, "kf_ln_quant: d=%d must be a multiple of 256 up to 2048", d);
  if (M == 0) return KF_OK;
  KF_REQUIRE(x && w && b && q && sf, "kf_ln_quant: null tensor pointer");
  KF_REQUIRE(aligned16(x) && aligned16(w) && aligned16(b) && aligned16(q) && aligned16(sf) && aligned16(y_dbg), "kf_ln_quant: tensors must be 16-byte aligned");
  KF_REQUIRE(fmt != KF_FMT_NV4 || ts, "kf_ln_quant: nv4 needs the per-tensor scale pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (d / 256) {
    case 1: return launch_ln_quant<1>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    case 2: return launch_ln_quant<2>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    case 3: return launch_ln_quant<3>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    case 4: return launch_ln_quant<4>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    case 5: return launch_ln_quant<5>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    case 6: return launch_ln_quant<6>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    case 7: return launch_ln_quant<7>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
    default: return launch_ln_quant<8>(fmt, x, w, b, eps, M, ts, flags, q, sf, y_dbg, st);
  }
}

extern "C" int kf_ln_rows(const float* x, const float* w, const float* b, float eps, int M, int d, int out_dtype, void* y, void* stream) {
  KF_REQUIRE(out_dtype == KF_BF16 || out_dtype == KF_F16, "kf_ln_rows: output dtype must be bf16 or f16");
  KF_REQUIRE(M >= 0 && d > 0 && d % 256 == 0 && d <= 2048, "kf_ln_rows: d=%d must be a multiple of 256 up to 2048", d);
  if (M == 0) return KF_OK;
  KF_REQUIRE(x && w && b && y, "kf_ln_rows: null tensor pointer");
  KF_REQUIRE(aligned16(x) && aligned16(w) && aligned16(b) && aligned16(y), "kf_ln_rows: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (d / 256) {
    case 1: return launch_ln_rows<1>(x, w, b, eps, M, out_dtype, y, st);
    case 2: return launch_ln_rows<2>(x, w, b, eps, M, out_dtype, y, st);
    case 3: return launch_ln_rows<3>(x, w, b, eps, M, out_dtype, y, st);
    case 4: return launch_ln_rows<4>(x, w, b, eps, M, out_dtype, y, st);
    case 5: return launch_ln_rows<5>(x, w, b, eps, M, out_dtype, y, st);
    case 6: return launch_ln_rows<6>(x, w, b, eps, M, out_dtype, y, st);
    case 7: return launch_ln_rows<7>(x, w, b, eps, M, out_dtype, y, st);
    default: return launch_ln_rows<8>(x, w, b, eps, M, out_dtype, y, st);
  }
}

extern "C" int kf_ln_tail(const float* x, const float* w, const float* b, float eps, int B, int Ntok, int Q, int npre, int d, void* qb, void* xb,
                          const void* wcls, const float* bcls, int ncls1, void* cl, void* stream) {
  KF_REQUIRE(B >= 0 && Ntok > 0 && Q >= 0 && npre >= 0 && Q + npre <= Ntok, "kf_ln_tail: bad token counts Ntok=%d Q=%d npre=%d", Ntok, Q, npre);
  KF_REQUIRE(d > 0 && d % 256 == 0 && d <= 2048, "kf_ln_tail: d=%d must be a multiple of 256 up to 2048", d);
  if (B == 0) return KF_OK;
  KF_REQUIRE(x && w && b && xb && (qb || Q == 0), "kf_ln_tail: null tensor pointer");
  KF_REQUIRE(aligned16(x) && aligned16(w) && aligned16(b) && aligned16(qb) && aligned16(xb), "kf_ln_tail: tensors must be 16-byte aligned");
  KF_REQUIRE(wcls == nullptr || (bcls && cl && ncls1 > 0 && ncls1 <= 64 && aligned16(wcls)), "kf_ln_tail: the class head needs wcls (16-byte aligned), bcls, cl and 1..64 logits");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int M = B * Ntok;
  switch (d / 256) {
    case 1: return launch_ln_tail<1>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    case 2: return launch_ln_tail<2>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    case 3: return launch_ln_tail<3>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    case 4: return launch_ln_tail<4>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    case 5: return launch_ln_tail<5>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    case 6: return launch_ln_tail<6>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    case 7: return launch_ln_tail<7>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
    default: return launch_ln_tail<8>(x, w, b, eps, M, Ntok, Q, npre, qb, xb, wcls, bcls, ncls1, cl, st);
  }
}

extern "C" int kf_broadcast_rows(const float* src, float* dst, int R, int d, int B, int64_t img_stride, int64_t row_offset, void* stream) {
  KF_REQUIRE(R >= 0 && B >= 0 && d > 0 && d % 4 == 0, "kf_broadcast_rows: d=%d must be a positive multiple of 4", d);
  KF_REQUIRE(img_stride % 4 == 0 && row_offset >= 0 && row_offset + (int64_t)R <= img_stride / d, "kf_broadcast_rows: rows %lld..%lld do not fit an image of %lld values",
             (long long)row_offset, (long long)(row_offset + R), (long long)img_stride);
  if (R == 0 || B == 0) return KF_OK;
  KF_REQUIRE(src && dst && aligned16(src) && aligned16(dst), "kf_broadcast_rows: tensors must be non-null and 16-byte aligned");
  const int64_t n = (int64_t)R * (d / 4) * B;
  int grid = (int)((n + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  broadcast_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst), R, d / 4, B, img_stride / 4,
                                                                            row_offset * (d / 4));
  return cuda_status(cudaGetLastError(), "kf_broadcast_rows launch");
}
