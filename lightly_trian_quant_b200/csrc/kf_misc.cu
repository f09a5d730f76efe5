// Memory-bound kernels around the transformer blocks of the DINOv3 + EoMT path: patch gathering for the patch-embed
// GEMM, the ScaleBlock tail (bias + GELU + pixel shuffle + depthwise 3x3 + LayerNorm2D), the per-pixel semantic
// scores / argmax, and frame resize + normalisation.
#include "kf_common.cuh"

namespace kf {

// ------------------------------------------------------------------------------------------------ patch gathering
// x [B, 3, S, S] bf16 -> rows [B*g*g, 768] bf16 with k = c*256 + py*16 + px: the K-major A operand of the patch-embed
// GEMM against the Conv2d weight [d, 3, 16, 16] viewed as [d, 768].  One thread moves 16 pixels (32 bytes) of one
// patch row.
__global__ void __launch_bounds__(256) im2col16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int B, int S) {
  const int g = S >> 4;
  const int64_t total = (int64_t)B * g * g * 48;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int seg = (int)(i % 48);
  const int64_t patch = i / 48;
  const int c = seg >> 4, py = seg & 15;
  const int gx = (int)(patch % g), gy = (int)((patch / g) % g), b = (int)(patch / ((int64_t)g * g));
  const uint4* src = reinterpret_cast<const uint4*>(x + (((int64_t)b * 3 + c) * S + gy * 16 + py) * S + gx * 16);
  uint4* dst = reinterpret_cast<uint4*>(out + patch * 768 + seg * 16);
  uint4 a = __ldg(src), d = __ldg(src + 1);
  dst[0] = a;
  dst[1] = d;
}

// ------------------------------------------------------------------------------------------------ ScaleBlock tail
// g [B*Hs*Ws, 4C] bf16 is the ConvTranspose2d(k=2, s=2) GEMM output with column (dy*2+dx)*C + c.  For each output
// pixel (Y, X) = (2y+dy, 2x+dx):  a = bf16(gelu(g + bias[c]))  (skipped when the GEMM epilogue already applied it:
// pre_act != 0);  o = bf16(sum over the 3x3 taps of a * dww[tap][c]) with zero padding, fp32 accumulation in tap
// order;  out = bf16(LayerNorm over c of o) in NHWC, two-pass statistics on the rounded conv outputs.
//
// Channel-stationary threads, rows streamed: a CTA has C/4 threads and thread t owns channels 4t..4t+3 for the whole
// launch, so its 36 tap weights and 8 LayerNorm parameters are loaded once and stay in registers.  A work item is a
// strip of 8 output pixels in x and seg_rows rows in y of one image; persistent CTAs take items round-robin.  The
// halo rows of a strip (10 pixels x C channels, C*20 bytes) stream through a 5-slot shared-memory ring filled by
// 16-byte cp.async copies (zero fill outside the image) that run two rows ahead, across item boundaries too; every
// row is fetched once per strip and used for three output rows.  Per output row a thread reads its 4 channels of the
// 3 x 10 window (30 8-byte shared loads), accumulates the 8 pixels in tap order on packed fp32 pairs, rounds to bf16,
// and the LayerNorm sums of the 8 pixels are reduced over the CTA (a transposing butterfly inside the warp, then one
// shared-memory exchange per statistic); the thread normalises and stores its own 8 bytes of each pixel, so no conv
// result goes through shared memory and a warp's stores are 256 contiguous bytes.
constexpr int DW_SW = 8, DW_HALO = DW_SW + 2, DW_RING = 5;

__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_dst, const void* gsrc, bool valid) {
  const int n = valid ? 16 : 0;                          // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(n) : "memory");
}

// shared-memory accesses by 32-bit address: with a compile-time C the pixel offsets fold into the instruction
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint2 v) { asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory"); }

struct DwItem {
  int b, X0, Y0, rows;                                   // rows: output rows of the item (its halo has rows + 2)
};
__device__ __forceinline__ DwItem dw_item(int item, int strips, int segs, int seg_rows, int Ho) {
  DwItem r;
  const int seg = item % segs;
  const int q = item / segs;
  r.X0 = (q % strips) * DW_SW;
  r.b = q / strips;
  r.Y0 = seg * seg_rows;
  r.rows = min(seg_rows, Ho - r.Y0);
  return r;
}

// sums of v[0..7] over all threads of the CTA, returned in v for every thread.  red: 64 floats of shared memory that no
// other exchange uses between the two barriers around this call.
__device__ __forceinline__ void dw_block_sum8(float (&v)[8], float* red, int warp, int lane, int nwarps) {
  // transposing butterfly: after the three halving steps lane l holds the partial sum of pixel l >> 2
  float a[4], b[2];
  bool hi = lane & 16;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float keep = hi ? v[j + 4] : v[j], send = hi ? v[j] : v[j + 4];
    a[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
  hi = lane & 8;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float keep = hi ? a[j + 2] : a[j], send = hi ? a[j] : a[j + 2];
    b[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  hi = lane & 4;
  float c = (hi ? b[1] : b[0]) + __shfl_xor_sync(0xffffffffu, hi ? b[0] : b[1], 4);
  c += __shfl_xor_sync(0xffffffffu, c, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 1);
  if ((lane & 3) == 0) red[warp * 8 + (lane >> 2)] = c;
  __syncthreads();
  float tot = 0.f;
  if (lane < 8) {
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < nwarps) tot += red[w * 8 + lane];
  }
#pragma unroll
  for (int p = 0; p < 8; ++p) v[p] = __shfl_sync(0xffffffffu, tot, p);
}

// CT: the channel count as a compile-time constant (0 = use the run-time argument)
template <int CT>
__global__ void __launch_bounds__(256, 2)
dw_ln_kernel(const __nv_bfloat16* __restrict__ g, const float* __restrict__ bias, const float* __restrict__ dww, const float* __restrict__ lnw,
             const float* __restrict__ lnb, __nv_bfloat16* __restrict__ out, int Hs, int Ws, int C_arg, float eps, int pre_act, int strips, int segs,
             int seg_rows, int total_items) {
  extern __shared__ __align__(16) uint8_t dsm[];
  const int C = CT ? CT : C_arg;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, nwarps = blockDim.x >> 5;
  const int Ho = 2 * Hs, Wo = 2 * Ws;
  const int row_bytes = DW_HALO * C * 2;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dsm);
  float* red = reinterpret_cast<float*>(dsm + DW_RING * row_bytes);       // two exchange areas of 64 floats

  // the thread's channels: tap weights, LayerNorm parameters, bias
  float2 w[9][2];
#pragma unroll
  for (int k = 0; k < 9; ++k) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(dww + (size_t)k * C) + t);
    w[k][0] = make_float2(v.x, v.y);
    w[k][1] = make_float2(v.z, v.w);
  }
  const float4 gw = __ldg(reinterpret_cast<const float4*>(lnw) + t), gb = __ldg(reinterpret_cast<const float4*>(lnb) + t);
  const float2 gw0 = make_float2(gw.x, gw.y), gw1 = make_float2(gw.z, gw.w), gb0 = make_float2(gb.x, gb.y), gb1 = make_float2(gb.z, gb.w);
  const float invC = 1.0f / (float)C;

  // ---- issue cursor: one halo row per call, two rows ahead of the row being consumed, running on into the next item.
  // A halo row is 10 pixels x C/8 pieces of 16 bytes; with C/4 threads thread t copies piece q = t mod C/8 of the pixels
  // 2k + hi (hi = t >= C/8), k = 0..4.  Those pixels have the same x parity, so their sources are 4C elements apart.
  const int C8 = C >> 3;
  const int i_hi = t >= C8 ? 1 : 0, i_q = t - i_hi * C8;
  int i_item = blockIdx.x, i_hr = 0, i_slot = 0;
  DwItem I = dw_item(i_item < total_items ? i_item : 0, strips, segs, seg_rows, Ho);
  auto issue = [&]() {
    if (i_item < total_items) {
      const int Y = I.Y0 - 1 + i_hr;
      const bool y_in = Y >= 0 && Y < Ho;
      const int xs = (I.X0 >> 1) + i_hi - 1;               // source column of k = 0;  X = 2*(xs + k) + (1 - i_hi)
      const int64_t src0 = ((((int64_t)I.b * Hs + (y_in ? (Y >> 1) : 0)) * Ws + xs) * 4 + (Y & 1) * 2 + (1 - i_hi)) * C + i_q * 8;
      const uint32_t dst0 = ring + i_slot * row_bytes + i_hi * (C * 2) + i_q * 16;
#pragma unroll
      for (int k = 0; k < 5; ++k) {
        const int xk = xs + k;
        const bool valid = y_in && xk >= 0 && xk < Ws;
        cp_async16_zfill(dst0 + k * (C * 4), g + (valid ? src0 + (int64_t)k * 4 * C : 0), valid);
      }
      if (++i_hr == I.rows + 2) {
        i_hr = 0;
        i_item += gridDim.x;
        if (i_item < total_items) I = dw_item(i_item, strips, segs, seg_rows, Ho);
      }
      if (++i_slot == DW_RING) i_slot = 0;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // every thread commits one group per call, copies or not
  };
  issue();
  issue();

  int c_slot = 0;                                            // slot of the halo row consumed by the current step
  float4 bia = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!pre_act) bia = __ldg(reinterpret_cast<const float4*>(bias) + t);
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const DwItem T = dw_item(item, strips, segs, seg_rows, Ho);
    for (int hr = 0; hr < T.rows + 2; ++hr) {
      asm volatile("cp.async.wait_group 1;" ::: "memory");   // this thread's copies of halo row hr have landed
      __syncthreads();                                        // ... and everybody's; the previous step has left the slot refilled next
      issue();
      const uint32_t own = t * 8;                             // the thread's 4 channels inside a pixel
      if (!pre_act) {                                         // bias + GELU on the new row, in place; only this thread reads these bytes later
        const int Y = T.Y0 - 1 + hr;
        if (Y >= 0 && Y < Ho) {
          const uint32_t rowp = ring + c_slot * row_bytes + own;
#pragma unroll
          for (int hx = 0; hx < DW_HALO; ++hx) {
            const int X = T.X0 - 1 + hx;
            if (X >= 0 && X < Wo) {
              const uint2 u = lds64(rowp + hx * (C * 2));
              float2 f0 = make_float2(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u));
              float2 f1 = make_float2(__uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
              f0 = make_float2(gelu_erf(f0.x + bia.x), gelu_erf(f0.y + bia.y));
              f1 = make_float2(gelu_erf(f1.x + bia.z), gelu_erf(f1.y + bia.w));
              const __nv_bfloat162 h0 = __float22bfloat162_rn(f0), h1 = __float22bfloat162_rn(f1);
              sts64(rowp + hx * (C * 2), make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1)));
            }
          }
        }
      }
      if (hr >= 2) {
        // ---- output row Y of the strip: halo rows hr-2, hr-1, hr sit in the slots c_slot-2, c_slot-1, c_slot
        const int Y = T.Y0 + hr - 2;
        float2 acc[DW_SW][2];
#pragma unroll
        for (int p = 0; p < DW_SW; ++p) acc[p][0] = acc[p][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
          int s = c_slot - 2 + ky;
          if (s < 0) s += DW_RING;
          const uint32_t rowp = ring + s * row_bytes + own;
#pragma unroll
          for (int hx = 0; hx < DW_HALO; ++hx) {
            const uint2 u = lds64(rowp + hx * (C * 2));
            const float2 f0 = make_float2(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u));
            const float2 f1 = make_float2(__uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
#pragma unroll
            for (int kx = 2; kx >= 0; --kx) {                 // pixel hx - kx receives tap (ky, kx): per pixel the taps arrive in (ky, kx) order
              const int p = hx - kx;
              if (p >= 0 && p < DW_SW) {
                acc[p][0] = fma2(f0, w[ky * 3 + kx][0], acc[p][0]);
                acc[p][1] = fma2(f1, w[ky * 3 + kx][1], acc[p][1]);
              }
            }
          }
        }
        // ---- LayerNorm over the channels of each of the 8 pixels, statistics on the bf16-rounded conv outputs
        float s8[8];
#pragma unroll
        for (int p = 0; p < DW_SW; ++p) {
          acc[p][0] = bf16_round2(acc[p][0]);
          acc[p][1] = bf16_round2(acc[p][1]);
          const float2 s2 = add2(acc[p][0], acc[p][1]);
          s8[p] = s2.x + s2.y;
        }
        dw_block_sum8(s8, red, warp, lane, nwarps);
#pragma unroll
        for (int p = 0; p < DW_SW; ++p) {
          const float2 nm = splat2(-s8[p] * invC);
          acc[p][0] = add2(acc[p][0], nm);
          acc[p][1] = add2(acc[p][1], nm);
          const float2 q2 = fma2(acc[p][1], acc[p][1], mul2(acc[p][0], acc[p][0]));
          s8[p] = q2.x + q2.y;
        }
        dw_block_sum8(s8, red + 64, warp, lane, nwarps);
        __nv_bfloat16* orow = out + (((int64_t)T.b * Ho + Y) * Wo + T.X0) * C + t * 4;
#pragma unroll
        for (int p = 0; p < DW_SW; ++p) {
          if (T.X0 + p < Wo) {
            const float2 rstd = splat2(rsqrtf(s8[p] * invC + eps));
            const __nv_bfloat162 h0 = __float22bfloat162_rn(fma2(mul2(acc[p][0], rstd), gw0, gb0));
            const __nv_bfloat162 h1 = __float22bfloat162_rn(fma2(mul2(acc[p][1], rstd), gw1, gb1));
            *reinterpret_cast<uint2*>(orow + (int64_t)p * C) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
          }
        }
      }
      if (++c_slot == DW_RING) c_slot = 0;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------ semantic scores
// scores[b, c, p] = sum_q sigmoid(mask_logits[b, q, p]) * softmax(class_logits[b, q, :])[c]   (all ncls+1 classes kept),
// labels[b, p] = argmax over the ncls real classes.  One thread per pixel pair; the class probabilities sit in shared
// memory.  NC1 = ncls + 1 is a compile-time constant, and the mask logits of eight queries are requested before the
// first is used (the loop is otherwise one dependent L2 / HBM round trip per query).
template <int NC1>
__global__ void __launch_bounds__(256) semantic_kernel(const __nv_bfloat16* __restrict__ ml, const __nv_bfloat16* __restrict__ cl, int Q, int HW,
                                                       float* __restrict__ scores, uint8_t* __restrict__ labels) {
  extern __shared__ float prob[];                     // [Q][NC1]
  const int b = blockIdx.y;
  for (int q = threadIdx.x; q < Q; q += blockDim.x) {
    float v[NC1], mx = -INFINITY, s = 0.f;
#pragma unroll
    for (int c = 0; c < NC1; ++c) {
      v[c] = __bfloat162float(cl[((int64_t)b * Q + q) * NC1 + c]);
      mx = fmaxf(mx, v[c]);
    }
#pragma unroll
    for (int c = 0; c < NC1; ++c) {
      v[c] = expf(v[c] - mx);
      s += v[c];
    }
#pragma unroll
    for (int c = 0; c < NC1; ++c) prob[q * NC1 + c] = v[c] / s;
  }
  __syncthreads();
  // two adjacent pixels per thread (one 32-bit load per query when HW is even); sigmoid by exp2 / reciprocal approximations
  const int p = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (p >= HW) return;
  const bool two = p + 1 < HW, vec = two && (HW & 1) == 0;
  float acc0[NC1], acc1[NC1];
#pragma unroll
  for (int c = 0; c < NC1; ++c) acc0[c] = acc1[c] = 0.f;
  const __nv_bfloat16* m = ml + (int64_t)b * Q * HW + p;
  constexpr int QB = 8;
  for (int q0 = 0; q0 < Q; q0 += QB) {
    uint32_t u[QB];
#pragma unroll
    for (int k = 0; k < QB; ++k) {
      u[k] = 0;
      if (q0 + k < Q) {
        const __nv_bfloat16* mq = m + (int64_t)(q0 + k) * HW;
        if (vec) {
          u[k] = __ldg(reinterpret_cast<const uint32_t*>(mq));
        } else {
          u[k] = (uint32_t)__bfloat16_as_ushort(mq[0]);
          if (two) u[k] |= (uint32_t)__bfloat16_as_ushort(mq[1]) << 16;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < QB; ++k) {
      if (q0 + k < Q) {
        const float x0 = __uint_as_float(u[k] << 16), x1 = __uint_as_float(u[k] & 0xFFFF0000u);
        float e0, e1, s0, s1;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(x0 * -1.4426950408889634f));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(x1 * -1.4426950408889634f));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s0) : "f"(1.0f + e0));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s1) : "f"(1.0f + e1));
#pragma unroll
        for (int c = 0; c < NC1; ++c) {
          const float pr = prob[(q0 + k) * NC1 + c];
          acc0[c] = fmaf(s0, pr, acc0[c]);
          acc1[c] = fmaf(s1, pr, acc1[c]);
        }
      }
    }
  }
  int best0 = 0, best1 = 0;
  float bv0 = acc0[0], bv1 = acc1[0];
#pragma unroll
  for (int c = 0; c < NC1; ++c) {
    if (scores) {
      scores[((int64_t)b * NC1 + c) * HW + p] = acc0[c];
      if (two) scores[((int64_t)b * NC1 + c) * HW + p + 1] = acc1[c];
    }
    if (c < NC1 - 1 && acc0[c] > bv0) { bv0 = acc0[c]; best0 = c; }      // first maximum wins, as torch.argmax
    if (c < NC1 - 1 && acc1[c] > bv1) { bv1 = acc1[c]; best1 = c; }
  }
  if (labels) {
    labels[(int64_t)b * HW + p] = (uint8_t)best0;
    if (two) labels[(int64_t)b * HW + p + 1] = (uint8_t)best1;
  }
}

// ------------------------------------------------------------------------------------------------ resize + normalise
// frames uint8 [B, Hi, Wi, 3] (HWC) -> bf16 [B, 3, So, So]: separable triangle filter with support scaled by the
// down-sampling factor (bilinear with antialiasing, align_corners = false), then (v/255 - mean[c]) / std[c].
// One CTA = 256 consecutive pixels of one output row.  Pass 1: the vertical filter over the input rows of the window, for
// every input byte of the CTA's horizontal span (threads walk the span four bytes at a time, so the loads are coalesced
// 32-bit words), result as floats in shared memory.  Pass 2: each thread applies its horizontal taps to the three
// channels from shared memory.  Spans that do not fit the buffer (extreme down-scaling) take the direct path.
constexpr int RS_ROWS = 6;                               // window rows whose loads are in flight together
constexpr int RS_SPAN = 4096;                            // bytes of one input row a CTA can stage (256 outputs at up to 5x down-scaling)

// One aligned 32-bit word of the frame batch; a word that straddles the end of the batch is put together from the bytes
// that belong to it, one that starts past the end reads as zero (the host checks that the batch starts on a word boundary).
__device__ __forceinline__ uint32_t rs_load_word(const uint32_t* wp, uintptr_t buf_end) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(wp);
  if (a + 4 <= buf_end) return __ldg(wp);
  uint32_t w = 0;
  const uint8_t* bp = reinterpret_cast<const uint8_t*>(wp);
  for (int i = 0; i < 3; ++i)
    if (a + i < buf_end) w |= (uint32_t)__ldg(bp + i) << (8 * i);
  return w;
}

__global__ void __launch_bounds__(256) resize_norm_kernel(const uint8_t* __restrict__ src, __nv_bfloat16* __restrict__ dst, int Hi, int Wi, int So,
                                                          float m0, float m1, float m2, float s0, float s1, float s2) {
  __shared__ float vbuf[RS_SPAN];
  const int ox = blockIdx.x * blockDim.x + threadIdx.x, oy = blockIdx.y, b = blockIdx.z;
  const float sy = (float)Hi / So, sx = (float)Wi / So;
  const float supy = fmaxf(sy, 1.f), supx = fmaxf(sx, 1.f);
  const float isx = 1.0f / supx, isy = 1.0f / supy;
  const float cy = (oy + 0.5f) * sy;
  const int y0 = max((int)(cy - supy + 0.5f), 0), y1 = min((int)(cy + supy + 0.5f), Hi);
  auto xwin = [&](int o, int& a, int& e, float& c) {
    c = (o + 0.5f) * sx;
    a = max((int)(c - supx + 0.5f), 0);
    e = min((int)(c + supx + 0.5f), Wi);
  };
  // horizontal span of the CTA in input pixels, its byte range rounded out to 4-byte words of the row
  const int o_first = blockIdx.x * blockDim.x, o_last = min(o_first + (int)blockDim.x, So) - 1;
  int xa, xe, xt;
  float ct;
  xwin(o_first, xa, xt, ct);
  xwin(o_last, xt, xe, ct);
  float wsum = 0.f;
  for (int y = y0; y < y1; ++y) wsum += fmaxf(0.f, 1.f - fabsf((y + 0.5f - cy) * isy));
  const int64_t row0 = ((int64_t)b * Hi) * Wi * 3;       // byte offset of the image
  const int64_t byte_a = (int64_t)xa * 3, byte_e = (int64_t)xe * 3;
  // word alignment is decided on absolute byte offsets (src is 16-byte aligned per frame batch; rows need not be)
  const bool staged = (byte_e - byte_a) + 8 <= RS_SPAN;
  const uintptr_t buf_end = reinterpret_cast<uintptr_t>(src) + (uintptr_t)gridDim.z * Hi * Wi * 3;
  if (staged) {
    const int nbytes = (int)(byte_e - byte_a);
    // every word this CTA may touch lies inside the batch (all CTAs but the ones on the last rows of the last frame)
    const bool interior = reinterpret_cast<uintptr_t>(src) + (uintptr_t)(row0 + (int64_t)(y1 - 1) * Wi * 3 + byte_e) + 12 <= buf_end;
    for (int j4 = threadIdx.x * 4; j4 < nbytes + 3; j4 += blockDim.x * 4) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      // four consecutive bytes of every window row from two aligned 32-bit words (rows are not word aligned in
      // general); words that start past the end of the whole batch are not read.  The rows go six at a time with all
      // their loads issued before the first use: one L2 round trip per group instead of one per row.
      for (int yb = y0; yb < y1; yb += RS_ROWS) {
        uint32_t w0[RS_ROWS], w1[RS_ROWS];
        const int64_t off0 = row0 + (int64_t)yb * Wi * 3 + byte_a + j4;
        const uintptr_t ad0 = reinterpret_cast<uintptr_t>(src) + off0;
#pragma unroll
        for (int k = 0; k < RS_ROWS; ++k) {
          if (yb + k < y1) {
            const uintptr_t ad = ad0 + (uintptr_t)k * Wi * 3;
            const uint32_t* wp = reinterpret_cast<const uint32_t*>(ad & ~(uintptr_t)3);
            if (interior) {
              w0[k] = __ldg(wp);
              w1[k] = __ldg(wp + 1);
            } else {
              w0[k] = rs_load_word(wp, buf_end);
              w1[k] = rs_load_word(wp + 1, buf_end);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < RS_ROWS; ++k) {
          if (yb + k < y1) {
            const float wy = fmaxf(0.f, 1.f - fabsf((yb + k + 0.5f - cy) * isy));
            const uintptr_t ad = ad0 + (uintptr_t)k * Wi * 3;
            const uint32_t four = __funnelshift_r(w0[k], w1[k], (uint32_t)(ad & 3) * 8);
            // byte -> float without the conversion unit: the byte becomes the low mantissa bits of 2^23 (one byte
            // permute), and 2^23 is subtracted exactly
            const float v0 = __uint_as_float(__byte_perm(four, 0x4B000000u, 0x7650)) - 8388608.f;
            const float v1 = __uint_as_float(__byte_perm(four, 0x4B000000u, 0x7651)) - 8388608.f;
            const float v2 = __uint_as_float(__byte_perm(four, 0x4B000000u, 0x7652)) - 8388608.f;
            const float v3 = __uint_as_float(__byte_perm(four, 0x4B000000u, 0x7653)) - 8388608.f;
            a0 = fmaf(wy, v0, a0);
            a1 = fmaf(wy, v1, a1);
            a2 = fmaf(wy, v2, a2);
            a3 = fmaf(wy, v3, a3);
          }
        }
      }
      vbuf[j4] = a0; vbuf[j4 + 1] = a1; vbuf[j4 + 2] = a2; vbuf[j4 + 3] = a3;
    }
    __syncthreads();
  }
  if (ox >= So) return;
  int x0, x1;
  float cx;
  xwin(ox, x0, x1, cx);
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, wxs = 0.f;
  if (staged) {
    const float* vb = vbuf + (x0 - xa) * 3;
    for (int x = x0; x < x1; ++x, vb += 3) {
      const float wx = fmaxf(0.f, 1.f - fabsf((x + 0.5f - cx) * isx));
      wxs += wx;
      acc0 = fmaf(wx, vb[0], acc0);
      acc1 = fmaf(wx, vb[1], acc1);
      acc2 = fmaf(wx, vb[2], acc2);
    }
  } else {
    for (int x = x0; x < x1; ++x) wxs += fmaxf(0.f, 1.f - fabsf((x + 0.5f - cx) * isx));
    for (int y = y0; y < y1; ++y) {
      const float wy = fmaxf(0.f, 1.f - fabsf((y + 0.5f - cy) * isy));
      const uint8_t* row = src + row0 + (int64_t)y * Wi * 3;
      float r0 = 0.f, r1 = 0.f, r2 = 0.f;
      for (int x = x0; x < x1; ++x) {
        const float wx = fmaxf(0.f, 1.f - fabsf((x + 0.5f - cx) * isx));
        r0 = fmaf(wx, (float)row[x * 3], r0);
        r1 = fmaf(wx, (float)row[x * 3 + 1], r1);
        r2 = fmaf(wx, (float)row[x * 3 + 2], r2);
      }
      acc0 = fmaf(wy, r0, acc0);
      acc1 = fmaf(wy, r1, acc1);
      acc2 = fmaf(wy, r2, acc2);
    }
  }
  const float inv = 1.0f / (wsum * wxs * 255.f);
  const int64_t plane = (int64_t)So * So;
  __nv_bfloat16* o = dst + (int64_t)b * 3 * plane + (int64_t)oy * So + ox;
  o[0] = __float2bfloat16_rn((acc0 * inv - m0) / s0);
  o[plane] = __float2bfloat16_rn((acc1 * inv - m1) / s1);
  o[2 * plane] = __float2bfloat16_rn((acc2 * inv - m2) / s2);
}

static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace kf

using namespace kf;

extern "C" int kf_im2col_patch16(const void* x, void* out, int B, int S, void* stream) {
  KF_REQUIRE(B >= 0 && S > 0 && S % 16 == 0, "kf_im2col_patch16: image side %d must be a positive multiple of 16", S);
  if (B == 0) return KF_OK;
  KF_REQUIRE(x && out && al16(x) && al16(out), "kf_im2col_patch16: tensors must be non-null and 16-byte aligned");
  const int64_t total = (int64_t)B * (S / 16) * (S / 16) * 48;
  im2col16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                                                static_cast<__nv_bfloat16*>(out), B, S);
  return cuda_status(cudaGetLastError(), "kf_im2col_patch16 launch");
}

extern "C" int kf_dw_ln(const void* g, const float* bias, const float* dww, const float* lnw, const float* lnb, void* out, int B, int Hs, int Ws, int C,
                        float eps, int pre_act, void* stream) {
  KF_REQUIRE(B >= 0 && Hs > 0 && Ws > 0, "kf_dw_ln: bad shape B=%d Hs=%d Ws=%d", B, Hs, Ws);
  KF_REQUIRE(C > 0 && C % 128 == 0 && C <= 1024, "kf_dw_ln: C=%d must be a multiple of 128 up to 1024", C);
  if (B == 0) return KF_OK;
  KF_REQUIRE(g && (bias || pre_act) && dww && lnw && lnb && out && al16(g) && al16(out) && al16(lnw) && al16(lnb) && al16(dww) && al16(bias),
             "kf_dw_ln: tensors must be non-null and 16-byte aligned");
  const size_t smem = (size_t)DW_RING * DW_HALO * C * 2 + 2 * 64 * sizeof(float);
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    const int big = (int)((size_t)DW_RING * DW_HALO * 1024 * 2 + 2 * 64 * sizeof(float));
    cudaError_t e = cudaFuncSetAttribute(dw_ln_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dw_ln_kernel<768>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dw_ln_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(dw_ln_kernel)");
    if (dev < 64) attr_set[dev] = true;
  }
  int sms = 0;
  int st = device_sm_count(&sms);
  if (st != KF_OK) return st;
  // items: strips of 8 output pixels in x, cut in y into segments of about 40 rows (each segment re-reads two halo rows:
  // 5 %); fewer, longer segments when the image count alone fills the CTAs several times over
  const int Ho = 2 * Hs, strips = (2 * Ws + DW_SW - 1) / DW_SW;
  const int segs = (Ho + 39) / 40, seg_rows = (Ho + segs - 1) / segs;
  const int64_t total = (int64_t)strips * segs * B;
  KF_REQUIRE(total < (1ll << 31), "kf_dw_ln: too many strips");
  const int grid = (int)(total < 2 * sms ? total : 2 * sms);
  // the channel counts of the ViT-L and ViT-B heads are compiled in (pixel offsets become instruction immediates)
  auto kern = C == 1024 ? dw_ln_kernel<1024> : C == 768 ? dw_ln_kernel<768> : dw_ln_kernel<0>;
  kern<<<grid, C / 4, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(g), bias, dww, lnw, lnb, static_cast<__nv_bfloat16*>(out), Hs,
                                                                 Ws, C, eps, pre_act, strips, segs, seg_rows, (int)total);
  return cuda_status(cudaGetLastError(), "kf_dw_ln launch");
}

extern "C" int kf_semantic(const void* mask_logits, const void* class_logits, int B, int Q, int ncls, int HW, float* scores, uint8_t* labels, void* stream) {
  KF_REQUIRE(B >= 0 && Q > 0 && HW > 0 && ncls >= 1 && ncls <= 7, "kf_semantic: bad shape B=%d Q=%d ncls=%d HW=%d", B, Q, ncls, HW);
  if (B == 0) return KF_OK;
  KF_REQUIRE(mask_logits && class_logits && (scores || labels), "kf_semantic: null tensor pointer");
  dim3 grid((HW + 511) / 512, B);
  const __nv_bfloat16* mlp = static_cast<const __nv_bfloat16*>(mask_logits);
  const __nv_bfloat16* clp = static_cast<const __nv_bfloat16*>(class_logits);
  const size_t smem = (size_t)Q * (ncls + 1) * 4;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  switch (ncls + 1) {                                   // one instantiation per class count (ncls real classes + the void class)
    case 2: semantic_kernel<2><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
    case 3: semantic_kernel<3><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
    case 4: semantic_kernel<4><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
    case 5: semantic_kernel<5><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
    case 6: semantic_kernel<6><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
    case 7: semantic_kernel<7><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
    default: semantic_kernel<8><<<grid, 256, smem, cs>>>(mlp, clp, Q, HW, scores, labels); break;
  }
  return cuda_status(cudaGetLastError(), "kf_semantic launch");
}

extern "C" int kf_resize_norm(const uint8_t* frames, void* out, int B, int Hi, int Wi, int So, const float* mean3, const float* std3, void* stream) {
  KF_REQUIRE(B >= 0 && Hi > 0 && Wi > 0 && So > 0, "kf_resize_norm: bad shape");
  if (B == 0) return KF_OK;
  KF_REQUIRE(frames && out && mean3 && std3, "kf_resize_norm: null pointer (mean3 / std3 are host arrays of 3 floats)");
  KF_REQUIRE((reinterpret_cast<uintptr_t>(frames) & 3) == 0, "kf_resize_norm: frames must start on a 4-byte boundary (the kernel reads aligned words)");
  dim3 grid((So + 255) / 256, So, B);
  resize_norm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(frames, static_cast<__nv_bfloat16*>(out), Hi, Wi, So, mean3[0], mean3[1], mean3[2],
                                                                          std3[0], std3[1], std3[2]);
  return cuda_status(cudaGetLastError(), "kf_resize_norm launch");
}

// ------------------------------------------------------------------------------------------------ patch embed without a caller-provided scratch buffer
// The patch-embed path is two launches with a scratch tensor between them: the gather kernel writes the patch rows
// [B*(S/16)^2, 768] bf16 and the tensor-core GEMM reads them as its A operand.  Everywhere else in this library the caller
// allocates that tensor.  Some callers cannot: a plug-in that runs inside another program's frame loop and is handed its
// inputs and outputs but no allocator, or a real-time path in which a cudaMalloc (it synchronises the whole device) would
// stall the copy streams.  For them the rows live in this fixed array inside the library image; every GPU that loads the
// library carries it until the process exits, so it is kept to what one 1024 x 1024 image (or two 640 x 640 ones) needs.
static __device__ __align__(256) unsigned char g_patch_rows[(size_t)KF_PATCH_STATIC_MAX_ROWS * 768 * 2];

namespace kf {
// Device address of the array on the CURRENT device.  On the host the array's name is only a handle: cudaGetSymbolAddress turns
// it into the pointer kernels and tensor maps can use.  Looked up once per device and kept.
static int patch_rows_address(void** out) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
  if (dev >= 0 && dev < 64 && cached[dev] != nullptr) {
    *out = cached[dev];
    return KF_OK;
  }
  void* p = nullptr;
  e = cudaGetSymbolAddress(&p, g_patch_rows);
  if (e != cudaSuccess) return cuda_status(e, "cudaGetSymbolAddress(patch rows)");
  if (p == nullptr) {
    set_error("kf_patch_embed_static: the scratch array has no device address");
    return KF_ERR_UNSUPPORTED;
  }
  if (dev >= 0 && dev < 64) cached[dev] = p;
  *out = p;
  return KF_OK;
}
}  // namespace kf

extern "C" int kf_patch_embed_static(const void* x, const void* w, const float* bias, float* tokens, int B, int S, int d, int tokens_per_image, int row_offset,
                                     int flags, void* stream) {
  KF_REQUIRE(B >= 0 && S > 0 && S % 16 == 0, "kf_patch_embed_static: image side %d must be a positive multiple of 16", S);
  KF_REQUIRE(d > 0 && d % 128 == 0, "kf_patch_embed_static: d=%d must be a positive multiple of 128", d);
  const int64_t P = (int64_t)(S / 16) * (S / 16), rows = P * B;
  KF_REQUIRE(rows <= KF_PATCH_STATIC_MAX_ROWS,
             "kf_patch_embed_static: %lld patch rows exceed the built-in scratch of %d rows (one 1024 x 1024 image); use kf_im2col_patch16 + kf_gemm_bs with your own buffer",
             (long long)rows, KF_PATCH_STATIC_MAX_ROWS);
  KF_REQUIRE(row_offset >= 0 && (int64_t)row_offset + P <= tokens_per_image, "kf_patch_embed_static: %lld patch rows behind %d do not fit %d tokens per image", (long long)P,
             row_offset, tokens_per_image);
  KF_REQUIRE((flags & ~KF_G_ROUND_BF16) == 0, "kf_patch_embed_static: only KF_G_ROUND_BF16 is a valid flag");
  if (B == 0) return KF_OK;
  KF_REQUIRE(x && w && tokens && al16(x) && al16(w), "kf_patch_embed_static: tensors must be non-null and 16-byte aligned");
  void* scratch = nullptr;
  int rc = patch_rows_address(&scratch);
  if (rc != KF_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * 48;
  im2col16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(scratch), B, S);
  rc = cuda_status(cudaGetLastError(), "kf_patch_embed_static gather launch");
  if (rc != KF_OK) return rc;
  kf_gemm_params p = {};
  p.fmt = KF_FMT_BF16;
  p.epi = KF_EPI_PLAIN;
  p.M = (int)rows;
  p.N = d;
  p.K = 768;
  p.out_dtype = KF_F32;
  p.flags = flags;
  p.A = scratch;
  p.W = w;
  p.bias = bias;
  p.C = tokens;
  p.out_row_group = (int)P;
  p.out_row_stride = tokens_per_image;
  p.out_row_offset = row_offset;
  return kf_gemm_bs(&p, stream);
}
