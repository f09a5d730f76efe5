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
// order;  out = bf16(LayerNorm over c of o) in NHWC.
// Persistent CTAs, one tile of 4 x 8 output pixels at a time.  The channels go through in slabs of 128: the 6 x 10 halo
// of a slab (256 contiguous bytes per pixel) is fetched with 16-byte cp.async copies (zero fill outside the image) into
// a 3-deep shared-memory ring that runs ahead across slabs AND tiles, so two slabs are always in flight while a third is
// convolved; each thread convolves 8 channels of 2 adjacent pixels (one 3 x 4 window read for both) with the 72 tap weights
// held in registers; the conv results of all C channels stay in shared memory for the two-pass LayerNorm statistics, which
// each lane then works out on register-resident values.
constexpr int DW_TH = 4, DW_TW = 8, DW_HW = (DW_TH + 2) * (DW_TW + 2), DW_CH = 128, DW_RING = 3;
constexpr int DW_SLAB_BYTES = DW_HW * DW_CH * 2;        // 15 KB

__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;                          // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}

struct DwTile {
  int b, Y0, X0;
};
__device__ __forceinline__ DwTile dw_tile(int tile, int tiles_x, int tiles_y) {
  DwTile t;
  t.X0 = (tile % tiles_x) * DW_TW;
  const int r = tile / tiles_x;
  t.Y0 = (r % tiles_y) * DW_TH;
  t.b = r / tiles_y;
  return t;
}

__global__ void __launch_bounds__(256, 2)
dw_ln_kernel(const __nv_bfloat16* __restrict__ g, const float* __restrict__ bias, const float* __restrict__ dww, const float* __restrict__ lnw,
             const float* __restrict__ lnb, __nv_bfloat16* __restrict__ out, int Hs, int Ws, int C, float eps, int pre_act, int tiles_x, int tiles_y,
             int total_tiles) {
  extern __shared__ __align__(16) uint8_t dsm[];
  uint4* res = reinterpret_cast<uint4*>(dsm + DW_RING * DW_SLAB_BYTES);     // [32 pixels][C/8]
  const int t = threadIdx.x;
  const int Ho = 2 * Hs, Wo = 2 * Ws;
  const int C8 = C >> 3, S = C / DW_CH;
  // conv work item of this thread: 8 channels (grp) of two horizontally adjacent pixels (oy, ox0), (oy, ox0 + 1): the 3 x 4
  // input window is read and unpacked once for both
  const int grp = t & 15, strip = t >> 4;
  const int oy = strip >> 2, ox0 = (strip & 3) * 2;

  // issue cursor (runs two slabs ahead of the consume cursor, across tile boundaries).  The (pixel, 16-byte piece)
  // pairs a thread copies are the same for every slab of a tile: their source offsets are worked out once per tile.
  int i_tile = blockIdx.x, i_slab = 0, i_slot = 0;
  int64_t i_src[4];
  bool i_in[4];
  auto issue = [&]() {
    if (i_tile < total_tiles) {
      if (i_slab == 0) {
        const DwTile T = dw_tile(i_tile, tiles_x, tiles_y);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int idx = t + 256 * k;
          const int px = idx >> 4, q = idx & 15;
          const int hy = px / (DW_TW + 2), hx = px - hy * (DW_TW + 2);
          const int Y = T.Y0 + hy - 1, X = T.X0 + hx - 1;
          i_in[k] = idx < DW_HW * 16 && Y >= 0 && Y < Ho && X >= 0 && X < Wo;
          const int64_t row = i_in[k] ? ((int64_t)T.b * Hs + (Y >> 1)) * Ws + (X >> 1) : 0;
          i_src[k] = row * 4 * C + (i_in[k] ? ((Y & 1) * 2 + (X & 1)) * C : 0) + q * 8;
        }
      }
      uint4* act = reinterpret_cast<uint4*>(dsm + i_slot * DW_SLAB_BYTES);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (t + 256 * k < DW_HW * 16) cp_async16_zfill(act + t + 256 * k, g + i_src[k] + i_slab * DW_CH, i_in[k]);
      if (++i_slab == S) {
        i_slab = 0;
        i_tile += gridDim.x;
      }
      if (++i_slot == DW_RING) i_slot = 0;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // every thread commits one group per call, copies or not
  };
  issue();
  issue();

  int c_slot = 0;
  const int warp = t >> 5, lane = t & 31;
  const float invC = 1.0f / (float)C;
  const int nk = C8 >> 5;                                    // 256-channel steps of the LayerNorm: lane owns 8 channels in each
  for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const DwTile T = dw_tile(tile, tiles_x, tiles_y);
    for (int sl = 0; sl < S; ++sl) {
      const int ch = sl * DW_CH;
      asm volatile("cp.async.wait_group 1;" ::: "memory");   // this thread's copies of the slab to consume have landed
      __syncthreads();                                        // ... and everybody's; the previous slab's conv is finished everywhere
      issue();                                                // refill the slot that conv just left (two slabs stay in flight)
      uint4* act = reinterpret_cast<uint4*>(dsm + c_slot * DW_SLAB_BYTES);
      if (!pre_act) {                                         // bias + GELU once per halo element, in place
        for (int idx = t; idx < DW_HW * 16; idx += 256) {
          const int px = idx >> 4, q = idx & 15;
          const int hy = px / (DW_TW + 2), hx = px - hy * (DW_TW + 2);
          const int Y = T.Y0 + hy - 1, X = T.X0 + hx - 1;
          if (Y >= 0 && Y < Ho && X >= 0 && X < Wo) {
            float f[8];
            bf16x8_to_f32(act[idx], f);
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + ch + q * 8)), b1 = __ldg(reinterpret_cast<const float4*>(bias + ch + q * 8) + 1);
            const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = gelu_erf(f[k] + bb[k]);
            act[idx] = f32_to_bf16x8(f);
          }
        }
        __syncthreads();
      }
      // ---- depthwise 3x3 of the two pixels: taps accumulate in (ky, kx) order for each of them; the 3 x 8 tap weights of
      // a kernel row are fetched when that row is due (72 weights at once would not fit the register budget)
      // (packed pairs: a 16-bit pair unpacks into the two halves of one operand, and one FFMA2 serves two channels)
      float2 acc0[4], acc1[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) acc0[k] = acc1[k] = make_float2(0.f, 0.f);
#pragma unroll
      for (int ky = 0; ky < 3; ++ky) {
        float2 w[3][4];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const float4* wp = reinterpret_cast<const float4*>(dww + (ky * 3 + k) * C + ch + grp * 8);
          const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
          w[k][0] = make_float2(w0.x, w0.y); w[k][1] = make_float2(w0.z, w0.w); w[k][2] = make_float2(w1.x, w1.y); w[k][3] = make_float2(w1.z, w1.w);
        }
#pragma unroll
        for (int cx = 0; cx < 4; ++cx) {
          const uint4 a = act[((oy + ky) * (DW_TW + 2) + ox0 + cx) * 16 + grp];
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
          float2 f[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) f[k] = make_float2(__uint_as_float(aw[k] << 16), __uint_as_float(aw[k] & 0xFFFF0000u));
          if (cx < 3) {
#pragma unroll
            for (int k = 0; k < 4; ++k) acc0[k] = fma2(f[k], w[cx][k], acc0[k]);
          }
          if (cx > 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) acc1[k] = fma2(f[k], w[cx - 1][k], acc1[k]);
          }
        }
      }
      {
        const float o0[8] = {acc0[0].x, acc0[0].y, acc0[1].x, acc0[1].y, acc0[2].x, acc0[2].y, acc0[3].x, acc0[3].y};
        const float o1[8] = {acc1[0].x, acc1[0].y, acc1[1].x, acc1[1].y, acc1[2].x, acc1[2].y, acc1[3].x, acc1[3].y};
        res[(oy * DW_TW + ox0) * C8 + (ch >> 3) + grp] = f32_to_bf16x8(o0);
        res[(oy * DW_TW + ox0 + 1) * C8 + (ch >> 3) + grp] = f32_to_bf16x8(o1);
      }
      if (++c_slot == DW_RING) c_slot = 0;
    }
    __syncthreads();                                          // all conv results of the tile are in res

    // ---- LayerNorm over the channels of each pixel: 8 warps x 4 pixels; the lane's channels stay in registers
    for (int px = warp; px < DW_TH * DW_TW; px += 8) {
      const int py = px / DW_TW, pxx = px - py * DW_TW;
      const int Y = T.Y0 + py, X = T.X0 + pxx;
      const uint4* r = res + px * C8;
      float2 v[4][4];                                         // packed pairs: one instruction per two channels
      float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (k < nk) {
          const uint4 a = r[lane + 32 * k];
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[k][e] = make_float2(__uint_as_float(aw[e] << 16), __uint_as_float(aw[e] & 0xFFFF0000u));
            s2 = add2(s2, v[k][e]);
          }
        }
      }
      float s = s2.x + s2.y;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s * invC;
      const float2 nmean = splat2(-mean);
      float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (k < nk) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[k][e] = add2(v[k][e], nmean);
            q2 = fma2(v[k][e], v[k][e], q2);
          }
        }
      }
      float ss = q2.x + q2.y;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float2 rstd = splat2(rsqrtf(ss * invC + eps));
      if (Y < Ho && X < Wo) {
        uint4* dst = reinterpret_cast<uint4*>(out + (((int64_t)T.b * Ho + Y) * Wo + X) * C);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (k < nk) {
            const int i = lane + 32 * k;
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(lnw) + 2 * i), w1 = __ldg(reinterpret_cast<const float4*>(lnw) + 2 * i + 1);
            const float4 c0 = __ldg(reinterpret_cast<const float4*>(lnb) + 2 * i), c1 = __ldg(reinterpret_cast<const float4*>(lnb) + 2 * i + 1);
            const float2 ww[4] = {make_float2(w0.x, w0.y), make_float2(w0.z, w0.w), make_float2(w1.x, w1.y), make_float2(w1.z, w1.w)};
            const float2 cc[4] = {make_float2(c0.x, c0.y), make_float2(c0.z, c0.w), make_float2(c1.x, c1.y), make_float2(c1.z, c1.w)};
            float f[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 y = fma2(mul2(v[k][e], rstd), ww[e], cc[e]);
              f[2 * e] = y.x;
              f[2 * e + 1] = y.y;
            }
            dst[i] = f32_to_bf16x8(f);
          }
        }
      }
    }
    // the next tile's first conv writes res only after the next __syncthreads, which every warp reaches after its LayerNorm
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------ semantic scores
// scores[b, c, p] = sum_q sigmoid(mask_logits[b, q, p]) * softmax(class_logits[b, q, :])[c]   (all ncls+1 classes kept),
// labels[b, p] = argmax over the ncls real classes.  One thread per pixel; the class probabilities sit in shared memory.
__global__ void __launch_bounds__(256) semantic_kernel(const __nv_bfloat16* __restrict__ ml, const __nv_bfloat16* __restrict__ cl, int Q, int ncls1,
                                                       int HW, float* __restrict__ scores, uint8_t* __restrict__ labels) {
  extern __shared__ float prob[];                     // [Q][ncls1]
  const int b = blockIdx.y;
  for (int q = threadIdx.x; q < Q; q += blockDim.x) {
    float v[8], mx = -INFINITY, s = 0.f;
    for (int c = 0; c < ncls1; ++c) {
      v[c] = __bfloat162float(cl[((int64_t)b * Q + q) * ncls1 + c]);
      mx = fmaxf(mx, v[c]);
    }
    for (int c = 0; c < ncls1; ++c) {
      v[c] = expf(v[c] - mx);
      s += v[c];
    }
    for (int c = 0; c < ncls1; ++c) prob[q * ncls1 + c] = v[c] / s;
  }
  __syncthreads();
  // two adjacent pixels per thread (one 32-bit load per query when HW is even); sigmoid by exp2 / reciprocal approximations
  const int p = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (p >= HW) return;
  const bool two = p + 1 < HW, vec = two && (HW & 1) == 0;
  float acc0[8], acc1[8];                      // static indices only (loops over 8 with a guard) so that they stay in registers
#pragma unroll
  for (int c = 0; c < 8; ++c) acc0[c] = acc1[c] = 0.f;
  const __nv_bfloat16* m = ml + (int64_t)b * Q * HW + p;
  for (int q = 0; q < Q; ++q) {
    float x0, x1 = 0.f;
    if (vec) {
      const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(m + (int64_t)q * HW));
      x0 = __uint_as_float(u << 16);
      x1 = __uint_as_float(u & 0xFFFF0000u);
    } else {
      x0 = __bfloat162float(m[(int64_t)q * HW]);
      if (two) x1 = __bfloat162float(m[(int64_t)q * HW + 1]);
    }
    float e0, e1, s0, s1;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(x0 * -1.4426950408889634f));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(x1 * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s0) : "f"(1.0f + e0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s1) : "f"(1.0f + e1));
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (c < ncls1) {
        const float pr = prob[q * ncls1 + c];
        acc0[c] = fmaf(s0, pr, acc0[c]);
        acc1[c] = fmaf(s1, pr, acc1[c]);
      }
    }
  }
  int best0 = 0, best1 = 0;
  float bv0 = acc0[0], bv1 = acc1[0];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    if (c < ncls1) {
      if (scores) {
        scores[((int64_t)b * ncls1 + c) * HW + p] = acc0[c];
        if (two) scores[((int64_t)b * ncls1 + c) * HW + p + 1] = acc1[c];
      }
      if (c < ncls1 - 1 && acc0[c] > bv0) { bv0 = acc0[c]; best0 = c; }      // first maximum wins, as torch.argmax
      if (c < ncls1 - 1 && acc1[c] > bv1) { bv1 = acc1[c]; best1 = c; }
    }
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
    for (int j4 = threadIdx.x * 4; j4 < nbytes + 3; j4 += blockDim.x * 4) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      for (int y = y0; y < y1; ++y) {
        const float wy = fmaxf(0.f, 1.f - fabsf((y + 0.5f - cy) * isy));
        // four consecutive bytes from two aligned 32-bit words (rows are not word aligned in general); words that start
        // past the end of the whole batch are not read
        const int64_t off = row0 + (int64_t)y * Wi * 3 + byte_a + j4;
        const uintptr_t ad = reinterpret_cast<uintptr_t>(src) + off;
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(ad & ~(uintptr_t)3);
        const uint32_t w0 = rs_load_word(wp, buf_end), w1 = rs_load_word(wp + 1, buf_end);
        const uint32_t four = __funnelshift_r(w0, w1, (uint32_t)(ad & 3) * 8);
        const uint32_t v0 = four & 0xFF, v1 = (four >> 8) & 0xFF, v2 = (four >> 16) & 0xFF, v3 = four >> 24;
        a0 = fmaf(wy, (float)v0, a0);
        a1 = fmaf(wy, (float)v1, a1);
        a2 = fmaf(wy, (float)v2, a2);
        a3 = fmaf(wy, (float)v3, a3);
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
  KF_REQUIRE(C > 0 && C % 256 == 0 && C <= 1024, "kf_dw_ln: C=%d must be a multiple of 256 up to 1024", C);
  if (B == 0) return KF_OK;
  KF_REQUIRE(g && (bias || pre_act) && dww && lnw && lnb && out && al16(g) && al16(out) && al16(lnw) && al16(lnb) && al16(dww) && al16(bias),
             "kf_dw_ln: tensors must be non-null and 16-byte aligned");
  const size_t smem = (size_t)DW_RING * DW_SLAB_BYTES + (size_t)DW_TH * DW_TW * C * 2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(dw_ln_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)DW_RING * DW_SLAB_BYTES + DW_TH * DW_TW * 1024 * 2));
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(dw_ln_kernel)");
    if (dev < 64) attr_set[dev] = true;
  }
  int sms = 0;
  int st = device_sm_count(&sms);
  if (st != KF_OK) return st;
  const int tiles_x = (2 * Ws + DW_TW - 1) / DW_TW, tiles_y = (2 * Hs + DW_TH - 1) / DW_TH;
  const int64_t total = (int64_t)tiles_x * tiles_y * B;
  KF_REQUIRE(total < (1ll << 31), "kf_dw_ln: too many tiles");
  const int grid = (int)(total < 2 * sms ? total : 2 * sms);
  dw_ln_kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(g), bias, dww, lnw, lnb,
                                                                       static_cast<__nv_bfloat16*>(out), Hs, Ws, C, eps, pre_act, tiles_x, tiles_y, (int)total);
  return cuda_status(cudaGetLastError(), "kf_dw_ln launch");
}

extern "C" int kf_semantic(const void* mask_logits, const void* class_logits, int B, int Q, int ncls, int HW, float* scores, uint8_t* labels, void* stream) {
  KF_REQUIRE(B >= 0 && Q > 0 && HW > 0 && ncls >= 1 && ncls <= 7, "kf_semantic: bad shape B=%d Q=%d ncls=%d HW=%d", B, Q, ncls, HW);
  if (B == 0) return KF_OK;
  KF_REQUIRE(mask_logits && class_logits && (scores || labels), "kf_semantic: null tensor pointer");
  dim3 grid((HW + 511) / 512, B);
  semantic_kernel<<<grid, 256, (size_t)Q * (ncls + 1) * 4, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(mask_logits), static_cast<const __nv_bfloat16*>(class_logits), Q, ncls + 1, HW, scores, labels);
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
