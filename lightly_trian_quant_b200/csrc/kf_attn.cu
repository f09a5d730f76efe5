// FlashAttention-style forward on the sm_100a tensor cores (tcgen05.mma kind::f16, fp32 S and O in TMEM), head
// dimension 64, no mask, RoPE already applied by the qkv epilogue.
//
//   input    qkv [3, B, N, H, 64] bf16 | f16 (the physical layout the qkv GEMM epilogue writes)
//   output   O [B, N, H*64] bf16 | f16, or directly the quantised operand of the proj GEMM (kf_attn_fwd_quant)
//   CTA      persistent, two per SM; an item is 128 query rows of one (batch, head), key tiles of 64; a CTA takes the
//            items blockIdx.x, blockIdx.x + gridDim.x, ... and keeps every barrier phase running across them
//   roles    warps 0..3: softmax, one query row per thread (tcgen05.ld of the S row, running max / sum in fp32,
//            P -> 16 bit -> tensor memory by tcgen05.st); warp 4: TMA producer (Q in two buffers, K / V in a 4-deep
//            ring, 4-D tensor maps so rows past N read zero); warp 5 issues the PV products (O += P V: 4 MMAs of K=16
//            with P as the A operand from tensor memory and V as the MN-major B operand), warp 6 the S products
//            (S = Q K^T: 4 MMAs of K=16 from shared memory); warp 7 idles (it completes the second warp group, whose
//            registers setmaxnreg hands to the softmax warps: 200 against 56).  One thread issuing both products was
//            busy for about 1450 of the 1670 clk of a step (each MMA costs it ~55 clk, each commit ~80, each barrier
//            round trip 60-80 even when the phase completed long ago); with two issuers each waits for its operands
//            first and for the hand-over last.
//   pipeline S and P are double buffered in TMEM: S(j+2) is issued when PV(j) has completed (so a softmax that sees
//            S(j+2) knows that P buffer j & 1 has been read), also across the end of an item (the next item's Q and
//            first K tiles are loaded by then).  O accumulates in TMEM over all key tiles.  The exponentials of a tile
//            use the running maximum as it is; the tile's own row sum tells whether that was safe (below 2^15 no
//            element exceeded 2^15), so no maximum is tracked in the common case; only a row whose sum came out larger
//            finds its maximum, recomputes its P and has its O rescaled (TMEM load, multiply, store), which happens on
//            the first tiles and then almost never; the O barriers are waited only then and at the end of an item.
//   numerics softmax scale 1/8 folded into exp2 (fp32; three of every four element pairs by the special-function unit,
//            the fourth by a cubic on the FMA pipe: the unit is shared by the softmax warps of both CTAs and is the
//            busiest pipe of the step; more than a quarter costs more issue slots than it frees); the exponent
//            arguments and the row sums as packed fp32 pairs; m, l, O in fp32; P rounded to the input 16-bit type.
//            Every mbarrier wait is bounded.
//
// Replaces a16::fwd_kernel / attn16_fwd (infer-opt/round12_lowp_stack/impl/attn16o.cu:126-404; mma.sync m16n8k16 +
// TMA on sm_120).  The power-of-two Q pre-scale `pre` of the reference protects its fp16 accumulators
// (attn16o.cu:184-194); with fp32 accumulation it is mathematically neutral and is accepted but not applied.
#include <type_traits>

#include "kf_sm100.cuh"

namespace kf {

constexpr int AT_BM = 128, AT_BN = 64, AT_D = 64;
constexpr int AT_THREADS = 256;                        // warps 0..3 softmax, 4 TMA, 5 PV issuer, 6 S issuer, 7 idle
constexpr int AT_REGS_SOFTMAX = 200, AT_REGS_LEAN = 56; // 128 * 200 + 128 * 56 <= 256 * 128, the allocation at launch
constexpr int AT_KV = 4;                               // K / V ring depth
constexpr int AT_QTILE = AT_BM * AT_D * 2;             // 16 KB
constexpr int AT_KTILE = AT_BN * AT_D * 2;             // 8 KB
constexpr int AT_OFF_Q = 0, AT_OFF_K = 2 * AT_QTILE, AT_OFF_V = AT_OFF_K + AT_KV * AT_KTILE, AT_OFF_BAR = AT_OFF_V + AT_KV * AT_KTILE;
constexpr size_t AT_SMEM = (size_t)AT_OFF_BAR + 256;
constexpr float AT_SUM_LIMIT = 32768.f;                  // a tile's row sum above this sends the row to the exact-maximum path (the largest finite f16 is 65504)
constexpr int AT_POLY_K = 3;                             // which of every four element pairs takes the polynomial exponential
constexpr int AT_TMEM_COLS = 256, AT_COL_S = 0, AT_COL_O = 128, AT_COL_P = 192;   // S buffers at columns 0 and 64, P (16-bit pairs) at 192 and 224

struct AttnArgs {
  void* O;
  int B, N, H;
  int f16;          // 0 = bf16, 1 = f16
  float scale_log2; // softmax scale * log2(e)
  unsigned int* err;
  // optional fused quantisation of the output (the proj GEMM's A operand): out_fmt < 0 = off
  int out_fmt, flags;
  uint8_t *Qo, *SFo;
  const float* tso;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^t for a pair without the special-function unit: t = n + f with n = round(t) taken from the low mantissa bits of
// t + 1.5 * 2^23 and f in [-0.5, 0.5]; 2^f by a cubic (minimax for the relative error on that interval: 7.6e-5, far
// below the rounding of the 16-bit P it feeds); n goes into the exponent field by an integer add.  t is clamped at -126
// (the result is then 2^-126 instead of 0: it vanishes in the 16-bit P and in the row sum alike).  All of it runs on the
// FMA and integer pipes, as packed pairs where the operation exists.
__device__ __forceinline__ float2 ex2_poly2(float2 t) {
  t.x = fmaxf(t.x, -126.f);
  t.y = fmaxf(t.y, -126.f);
  const float2 r = add2(t, splat2(12582912.f));
  const float2 n = add2(r, splat2(-12582912.f));
  const float2 f = fma2(n, splat2(-1.f), t);
  float2 p = fma2(f, splat2(0x1.c43e56p-5f), splat2(0x1.f0df98p-3f));
  p = fma2(p, f, splat2(0x1.62f24ap-1f));
  p = fma2(p, f, splat2(0x1.fff686p-1f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(r.x) << 23)), __int_as_float(__float_as_int(p.y) + (__float_as_int(r.y) << 23)));
}

__device__ __forceinline__ uint32_t pack16(float a, float b, int f16) {
  if (f16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// F16: 16-bit type of q / k / v / P / O (0 = bf16); OUT: -1 = plain 16-bit output, else the KF_FMT_* of the fused
// output quantisation.  Compile-time so that the softmax loop carries one copy of its code.
template <int F16, int OUT>
__global__ void __launch_bounds__(AT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ AttnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AT_OFF_BAR);
  uint64_t *q_full = bars, *q_empty = bars + 2, *k_full = bars + 4, *v_full = k_full + AT_KV, *kv_empty = v_full + AT_KV, *s_full = kv_empty + AT_KV,
           *p_full = s_full + 2, *o_full = p_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  pdl_launch_dependents();                               // the next kernel of the stream may take the SMs this grid leaves
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent: this CTA works through the (image, head, query tile) items blockIdx.x, blockIdx.x + gridDim.x, ...  All
  // barriers keep running across items: K / V ring stages, S / P buffers and the O barrier are indexed by the CTA's global
  // key-tile count G, the two Q buffers by the item count, so the loads and the first S products of the next item are
  // under way while the current one finishes and writes its output.
  const int q_tiles = (a.N + AT_BM - 1) / AT_BM;
  const int n_kt = (a.N + AT_BN - 1) / AT_BN;
  const int items = a.B * a.H * q_tiles;
  const int n_my = (int)blockIdx.x < items ? (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  struct Item {
    int qt, h, b;
  };
  auto item_of = [&](int it) {
    const int item = blockIdx.x + it * gridDim.x;
    Item r;
    r.qt = item % q_tiles;
    const int bh = item / q_tiles;
    r.h = bh % a.H;
    r.b = bh / a.H;
    return r;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < AT_KV; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
    }
    mbar_init(&o_full[0], 1);                             // PV(G) completes o_full[G & 1]: a waiter is never more than one phase behind
    mbar_init(&o_full[1], 1);
    *abort_flag = (smem_u32(smem) & 1023u) ? 1u : 0u;   // the swizzled tiles need a 1024-byte aligned base
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_holder, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();                                            // set-up done: from here on global memory of the predecessors is read and written
  const uint32_t tmem_base = *tmem_holder;
  const WaitCtx ctx{abort_flag, a.err};
  const bool bad_align = *abort_flag != 0 || a.err[0] != 0;   // misaligned tiles, or an earlier CTA / launch already failed: skip the work
  if (*abort_flag != 0 && threadIdx.x == 0 && atomicCAS(&a.err[0], 0u, 99u) == 0u) {
    a.err[1] = 100;
    a.err[2] = blockIdx.x;
  }

  if (warp >= 4) {
  setmaxnreg_dec<AT_REGS_LEAN>();
  if (bad_align) {
    // nothing was issued; fall through to the teardown
  } else if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      uint32_t G = 0;
      bool ok = true;
      for (int it = 0; it < n_my && ok; ++it) {
        const Item I = item_of(it);
        const int qb = it & 1;
        if (!mbar_wait(&q_empty[qb], ((it >> 1) & 1) ^ 1, ctx, 10)) break;          // the S products of item it - 2 are done with this buffer
        mbar_expect_tx(&q_full[qb], AT_QTILE);
        tma_load_4d(smem + AT_OFF_Q + qb * AT_QTILE, &tmQ, 0, I.h, I.qt * AT_BM, I.b, &q_full[qb]);
        for (int j = 0; j < n_kt; ++j, ++G) {
          const int st = G % AT_KV;
          if (!mbar_wait(&kv_empty[st], ((G / AT_KV) & 1) ^ 1, ctx, 11)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], AT_KTILE);
          tma_load_4d(smem + AT_OFF_K + st * AT_KTILE, &tmK, 0, I.h, j * AT_BN, I.b, &k_full[st]);
          mbar_expect_tx(&v_full[st], AT_KTILE);
          tma_load_4d(smem + AT_OFF_V + st * AT_KTILE, &tmV, 0, I.h, j * AT_BN, I.b, &v_full[st]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ issuer of the PV products
    if (lane == 0) {
      const uint32_t idesc_o = idesc_f16(F16 ? 0u : 1u, AT_D) | (1u << 16);   // B (= V) is MN-major
      const uint32_t t_o = tmem_base + AT_COL_O;
      const uint32_t total = (uint32_t)n_my * (uint32_t)n_kt;                // key-tile steps of this CTA over all its items
      uint32_t j = 0;
      for (uint32_t G = 0; G < total; ++G) {
        const uint32_t st = G % AT_KV;
        if (!mbar_wait(&v_full[st], (G / AT_KV) & 1, ctx, 15)) break;      // V lands long before P: its barrier round trip is off the chain P -> PV -> S
        if (!mbar_wait(&p_full[G & 1], (G >> 1) & 1, ctx, 14)) break;
        tc_fence_after();
        const uint32_t t_p = tmem_base + AT_COL_P + (G & 1) * (AT_BN / 2);
        const uint64_t vdesc = smem_desc_sw128(smem_u32(smem + AT_OFF_V + st * AT_KTILE));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)       // A: 16 keys = 8 TMEM columns of P; B: 16 key rows of V = two 8-row groups of 1024 bytes
          mma_f16_ta(t_o, t_p + 8 * kk, vdesc + (uint64_t)(kk * (2048 >> 4)), idesc_o, (j | (uint32_t)kk) != 0);
        tc_commit(&o_full[G & 1]);
        tc_commit(&kv_empty[st]);            // K of this stage was read by S(G), which completed before the softmax of step G began
        if (++j == (uint32_t)n_kt) j = 0;
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------------------------------------------ issuer of the S products
    // A second issuing thread: one thread issuing both products of a step (eight MMAs, three or four commits, three
    // barrier round trips) was busy for about 1450 of the 1670 clk of a step.  S(G + 2) goes into the S buffer that the
    // softmax of step G has read, once PV(G) has completed: then a softmax that sees S(G + 2) also knows that P buffer
    // G & 1 has been read and may be overwritten, as it did when one thread issued S(G + 2) behind PV(G).
    if (lane == 0) {
      const uint32_t idesc_s = idesc_f16(F16 ? 0u : 1u, AT_BN);
      const uint32_t total = (uint32_t)n_my * (uint32_t)n_kt;
      uint32_t it = 0, j = 0;
      for (uint32_t G = 0; G < total; ++G) {                               // issues S(G)
        if (j == 0 && !mbar_wait(&q_full[it & 1], (it >> 1) & 1, ctx, 12)) break;   // the operands first: they land long before PV(G - 2) completes
        if (!mbar_wait(&k_full[G % AT_KV], (G / AT_KV) & 1, ctx, 13)) break;
        if (G >= 2 && !mbar_wait(&o_full[G & 1], ((G - 2) >> 1) & 1, ctx, 20)) break;   // PV(G - 2); the barrier's next completion, PV(G), needs this S(G)
        tc_fence_after();
        const uint64_t qdesc = smem_desc_sw128(smem_u32(smem + AT_OFF_Q + (it & 1) * AT_QTILE));
        const uint64_t kdesc = smem_desc_sw128(smem_u32(smem + AT_OFF_K + (G % AT_KV) * AT_KTILE));
        const uint32_t t_s = tmem_base + AT_COL_S + (G & 1) * AT_BN;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_f16(t_s, qdesc + 2 * kk, kdesc + 2 * kk, idesc_s, kk != 0);
        tc_commit(&s_full[G & 1]);
        if (++j == (uint32_t)n_kt) {
          tc_commit(&q_empty[it & 1]);                                     // the item's last S product: its Q buffer is free once it completes
          j = 0;
          ++it;
        }
      }
    }
    __syncwarp();
  }   // warp 7 is idle: it completes the second warp group, whose registers go to the softmax warps
  } else {
    setmaxnreg_inc<AT_REGS_SOFTMAX>();
    if (!bad_align) {
    // ------------------------------------------------------------------ softmax: thread = query row
    const int row = warp * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
    const float sc = a.scale_log2;
    bool ok = true;
    uint32_t G = 0;                                              // key-tile steps of this CTA so far, over all its items
    // per-tensor scale of an NVFP4 output, its reciprocal and range check: one L2 round trip per CTA, not per item
    const Nv4Scale tsc = nv4_scale(OUT == KF_FMT_NV4 ? __ldg(a.tso) : 1.f);
    for (int it = 0; it < n_my && ok; ++it) {
    const Item I = item_of(it);
    const int qt = I.qt, h = I.h, b = I.b;
    float m_run = -INFINITY, l_run = 0.f;
    for (int j = 0; j < n_kt; ++j, ++G) {
      const int sb = G & 1;
      if (!mbar_wait(&s_full[sb], (G >> 1) & 1, ctx, 17)) { ok = false; break; }
      tc_fence_after();
      const int kbase = j * AT_BN;
      uint32_t r[2][32];
      tmem_ld32(t_lane + AT_COL_S + sb * AT_BN, r[0]);
      tmem_ld32(t_lane + AT_COL_S + sb * AT_BN + 32, r[1]);
      tmem_ld_wait();
      if (kbase + AT_BN > a.N) {                                // key tail: columns past N never win the max and give P = 0
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kbase + c * 32 + i >= a.N) r[c][i] = 0xff800000u;
      }
      // the P row of this tile goes to tensor memory (the A operand of the PV product): 64 keys = 32 columns of 16-bit pairs
      const uint32_t t_p = t_lane + AT_COL_P + sb * (AT_BN / 2);
      // P = exp2(s*sc + mneg) into tensor memory; returns the row sum.  The exponent arguments and the row sum run as
      // packed pairs: half the issue slots of the scalar form.
      auto exp_row = [&](auto is_f16, float mneg) -> float {
        constexpr int F = decltype(is_f16)::value;
        const float2 sc2 = splat2(sc), mn2 = splat2(mneg);
        float2 s0 = make_float2(0.f, 0.f), s1 = s0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 p[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 t = fma2(make_float2(__uint_as_float(r[c][8 * i + 2 * k]), __uint_as_float(r[c][8 * i + 2 * k + 1])), sc2, mn2);
              p[k] = k == AT_POLY_K ? ex2_poly2(t) : make_float2(ex2(t.x), ex2(t.y));   // one pair in four off the special-function unit
            }
            s0 = add2(s0, add2(p[0], p[1]));
            s1 = add2(s1, add2(p[2], p[3]));
#pragma unroll
            for (int k = 0; k < 4; ++k) w[4 * i + k] = pack16(p[k].x, p[k].y, F);
          }
          tmem_st16(t_p + 16 * c, w);
        }
        return (s0.x + s0.y) + (s1.x + s1.y);
      };
      auto run = [&](float mneg) -> float {
        return exp_row(std::integral_constant<int, F16>{}, mneg);
      };
      // Lazy maximum without a maximum: the exponentials of tile j > 0 use the running maximum as it is, and the tile's
      // own row sum tells whether that was safe: while it stays below 2^15 no element exceeded 2^15 (bf16 / f16 P, the
      // fp32 sums and O have room for that), so the maximum of the tile is not needed at all.  Only a row whose sum came
      // out larger (or infinite) finds its maximum, raises the running maximum, recomputes its P and has its O rescaled.
      // The first tile has no running maximum yet and finds its own first.
      float sum = 0.f, alpha = 1.f;
      bool need = true;
      if (j > 0) {
        sum = run(-m_run * sc);
        need = sum > AT_SUM_LIMIT;
      }
      const uint32_t any_need = __ballot_sync(0xffffffffu, need);
      if (any_need) {                                            // warp-uniform: the tensor-memory stores need the whole warp
        if (need) {
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 16; ++i) mx4[i & 3] = max3(mx4[i & 3], __uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          if (mx > m_run) {
            alpha = ex2((m_run - mx) * sc);                      // 0 on the first tile
            m_run = mx;
          }
        }
        sum = run(-m_run * sc);
      }
      const uint32_t any = j > 0 ? any_need : 0u;
      l_run = l_run * alpha + sum;
      // O is only touched when a row of this warp raised its maximum: PV(G-1) must have landed first.  It completes
      // o_full[(G-1) & 1], whose next completion, PV(G+1), cannot come before this thread's arrivals of steps G and G+1.
      // The item's last step always waits, so that the epilogue's wait for the last product is covered as well.
      if ((any || j == n_kt - 1) && j > 0 && !mbar_wait(&o_full[(G - 1) & 1], ((G - 1) >> 1) & 1, ctx, 18)) { ok = false; break; }
      if (any) {                                                 // rescale O in TMEM
        tc_fence_after();
        tmem_ld32(t_lane + AT_COL_O, r[0]);
        tmem_ld32(t_lane + AT_COL_O + 32, r[1]);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          r[0][i] = __float_as_uint(__uint_as_float(r[0][i]) * alpha);
          r[1][i] = __float_as_uint(__uint_as_float(r[1][i]) * alpha);
        }
        tmem_st32(t_lane + AT_COL_O, r[0]);
        tmem_st32(t_lane + AT_COL_O + 32, r[1]);
        tmem_st_wait();
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[sb]);
    }
    if (ok) ok = mbar_wait(&o_full[(G - 1) & 1], ((G - 1) >> 1) & 1, ctx, 19);     // the item's last PV product
    const int n = qt * AT_BM + row;
    if (ok) {
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld32(t_lane + AT_COL_O, r0);
      tmem_ld32(t_lane + AT_COL_O + 32, r1);
      tmem_ld_wait();
      if (n < a.N && OUT >= 0) {
        // O row of this head (64 values) -> rounded to the 16-bit type -> 4 nv4 blocks or 2 mx blocks, written as the
        // codes and scale bytes of row b*N + n, columns h*64.. of the [B*N, H*64] operand
        const float inv = 1.0f / l_run;
        const bool div_true = !(a.flags & KF_Q_RECIP_DIV);
        float v[64];
        const float2 inv2 = splat2(inv);
        auto norm_round = [&](auto is_f16) {                       // O / l rounded to the 16-bit type, as packed pairs
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float2 x = mul2(make_float2(__uint_as_float(r0[i]), __uint_as_float(r0[i + 1])), inv2);
            float2 y = mul2(make_float2(__uint_as_float(r1[i]), __uint_as_float(r1[i + 1])), inv2);
            if (decltype(is_f16)::value) {
              x = __half22float2(__float22half2_rn(x));
              y = __half22float2(__float22half2_rn(y));
            } else {
              x = bf16_round2(x);
              y = bf16_round2(y);
            }
            v[i] = x.x;
            v[i + 1] = x.y;
            v[32 + i] = y.x;
            v[33 + i] = y.y;
          }
        };
        norm_round(std::integral_constant<int, F16>{});
        const size_t m = (size_t)b * a.N + n;
        const int d = a.H * AT_D;
        if (OUT == KF_FMT_NV4) {
          uint32_t o[8];
          float am[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            am[k] = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i += 2) am[k] = max3(am[k], fabsf(v[16 * k + i]), fabsf(v[16 * k + i + 1]));
          }
          int by[4];
#pragma unroll
          for (int k = 0; k < 4; k += 2) {                       // two blocks at a time: their scalars on packed pairs
            const float(&b0)[16] = *reinterpret_cast<const float(*)[16]>(&v[16 * k]);
            const float(&b1)[16] = *reinterpret_cast<const float(*)[16]>(&v[16 * k + 16]);
            quant_nv4_pair16(b0, am[k], b1, am[k + 1], tsc, div_true, o + 2 * k, by[k], by[k + 1]);
          }
          const uint32_t word = (uint32_t)by[0] | ((uint32_t)by[1] << 8) | ((uint32_t)by[2] << 16) | ((uint32_t)by[3] << 24);
          uint4* dst = reinterpret_cast<uint4*>(a.Qo + m * (d >> 1) + h * 32);
          dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
          dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          *reinterpret_cast<uint32_t*>(a.SFo + sf_offset((int)m, h * 4, d >> 6)) = word;
        } else {
          uint32_t half = 0;
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const float(&va)[16] = *reinterpret_cast<const float(*)[16]>(&v[32 * k]);
            const float(&vb)[16] = *reinterpret_cast<const float(*)[16]>(&v[32 * k + 16]);
            float am = 0.f;
#pragma unroll
            for (int i = 0; i < 32; i += 2) am = max3(am, fabsf(v[32 * k + i]), fabsf(v[32 * k + i + 1]));
            int by;
            if (OUT == KF_FMT_MX8) {
              uint32_t o[8];
              quant_mx8<16>(va, am, div_true, o, by);
              quant_mx8<16>(vb, am, div_true, o + 4, by);
              uint4* dst = reinterpret_cast<uint4*>(a.Qo + m * d + h * 64 + k * 32);
              dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
              dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
            } else {
              uint32_t o[4];
              quant_mx4<16>(va, am, div_true, o, by);
              quant_mx4<16>(vb, am, div_true, o + 2, by);
              *reinterpret_cast<uint4*>(a.Qo + m * (d >> 1) + h * 32 + k * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            half |= (uint32_t)by << (8 * k);
          }
          *reinterpret_cast<uint16_t*>(a.SFo + sf_offset((int)m, h * 2, d >> 7)) = (uint16_t)half;
        }
      } else if (n < a.N) {
        const float inv = 1.0f / l_run;
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          w[i] = pack16(__uint_as_float(r0[2 * i]) * inv, __uint_as_float(r0[2 * i + 1]) * inv, F16);
          w[16 + i] = pack16(__uint_as_float(r1[2 * i]) * inv, __uint_as_float(r1[2 * i + 1]) * inv, F16);
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.O) + (((size_t)b * a.N + n) * a.H + h) * (AT_D * 2));
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
    }   // items
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && !bad_align) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

// 4-D tensor map over one of q / k / v: dims (64, H, N, B) of 16-bit elements, box (64, 1, rows, 1), 128-byte swizzle;
// rows past N are out of bounds in their own dimension and read as zero.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_tmap_qkv(CUtensorMap* map, const void* base, int B, int N, int H, int box_rows) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return KF_ERR_UNSUPPORTED;
  }
  EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(p);
  cuuint64_t dims[4] = {64, (cuuint64_t)H, (cuuint64_t)N, (cuuint64_t)B};
  cuuint64_t strides[3] = {128, (cuuint64_t)H * 128, (cuuint64_t)N * H * 128};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (qkv) failed with CUresult %d", (int)r);
    return KF_ERR_BAD_ARGUMENT;
  }
  return KF_OK;
}

}  // namespace kf

using namespace kf;

static int attn_launch(int dtype, const void* qkv, void* O, int B, int N, int H, int out_fmt, void* Qo, void* SFo, const float* tso, int flags,
                       void* stream) {
  KF_REQUIRE(dtype == KF_BF16 || dtype == KF_F16, "kf_attn_fwd: dtype must be bf16 or f16");
  KF_REQUIRE(B >= 0 && N > 0 && H > 0, "kf_attn_fwd: bad shape B=%d N=%d H=%d", B, N, H);
  if (B == 0) return KF_OK;
  KF_REQUIRE(qkv && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0, "kf_attn_fwd: qkv must be non-null and 16-byte aligned");
  if (out_fmt < 0) {
    KF_REQUIRE(O && (reinterpret_cast<uintptr_t>(O) & 15) == 0, "kf_attn_fwd: O must be non-null and 16-byte aligned");
  } else {
    KF_REQUIRE(out_fmt == KF_FMT_MX8 || out_fmt == KF_FMT_NV4 || out_fmt == KF_FMT_MX4, "kf_attn_fwd_quant: bad output format %d", out_fmt);
    KF_REQUIRE(Qo && SFo && (reinterpret_cast<uintptr_t>(Qo) & 15) == 0 && (reinterpret_cast<uintptr_t>(SFo) & 15) == 0,
               "kf_attn_fwd_quant: Qo and SFo must be non-null and 16-byte aligned");
    KF_REQUIRE(out_fmt != KF_FMT_NV4 || tso, "kf_attn_fwd_quant: nv4 needs the per-tensor scale");
    KF_REQUIRE((H * 64) % 128 == 0, "kf_attn_fwd_quant: H*64 must be a multiple of 128");
  }
  const size_t plane = (size_t)B * N * H * 64 * 2;
  const uint8_t* base = static_cast<const uint8_t*>(qkv);
  CUtensorMap tq, tk, tv;
  int st = make_tmap_qkv(&tq, base, B, N, H, AT_BM);
  if (st != KF_OK) return st;
  st = make_tmap_qkv(&tk, base + plane, B, N, H, AT_BN);
  if (st != KF_OK) return st;
  st = make_tmap_qkv(&tv, base + 2 * plane, B, N, H, AT_BN);
  if (st != KF_OK) return st;
  // one instantiation per 16-bit type and output form
  using KernelFn = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, AttnArgs);
  static const KernelFn table[2][4] = {
      {attn_fwd_kernel<0, -1>, attn_fwd_kernel<0, KF_FMT_MX8>, attn_fwd_kernel<0, KF_FMT_NV4>, attn_fwd_kernel<0, KF_FMT_MX4>},
      {attn_fwd_kernel<1, -1>, attn_fwd_kernel<1, KF_FMT_MX8>, attn_fwd_kernel<1, KF_FMT_NV4>, attn_fwd_kernel<1, KF_FMT_MX4>}};
  const int oi = out_fmt < 0 ? 0 : out_fmt == KF_FMT_MX8 ? 1 : out_fmt == KF_FMT_NV4 ? 2 : 3;
  const KernelFn kern = table[dtype == KF_F16 ? 1 : 0][oi];
  static bool attr_set[64][2][4] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev][dtype == KF_F16 ? 1 : 0][oi]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(attn_fwd_kernel)");
    if (dev < 64) attr_set[dev][dtype == KF_F16 ? 1 : 0][oi] = true;
  }
  AttnArgs a{};
  a.O = O; a.B = B; a.N = N; a.H = H; a.f16 = dtype == KF_F16;
  a.scale_log2 = 0.125f * 1.4426950408889634f;
  a.err = dev_error_ptr();
  a.out_fmt = out_fmt; a.flags = flags; a.Qo = static_cast<uint8_t*>(Qo); a.SFo = static_cast<uint8_t*>(SFo); a.tso = tso;
  KF_REQUIRE(a.err != nullptr, "kf_attn_fwd: device error word unavailable");
  const int q_tiles = (N + AT_BM - 1) / AT_BM;
  const long long items = (long long)B * H * q_tiles;
  KF_REQUIRE(items < (1ll << 30), "kf_attn_fwd: too many (image, head, query tile) items");
  int sms = 0;
  const int sst = device_sm_count(&sms);
  if (sst != KF_OK) return sst;
  const int slots = 2 * sms;                                  // two CTAs are resident per SM
  const int grid = items < slots ? (int)items : slots;
  return cuda_status(launch_maybe_pdl(kern, dim3(grid), dim3(AT_THREADS), (size_t)AT_SMEM, static_cast<cudaStream_t>(stream), tq, tk, tv, a),
                     "kf_attn_fwd launch");
}

extern "C" int kf_attn_fwd(int dtype, const void* qkv, void* O, int B, int N, int H, float pre, void* stream) {
  (void)pre;
  return attn_launch(dtype, qkv, O, B, N, H, -1, nullptr, nullptr, nullptr, 0, stream);
}

extern "C" int kf_attn_fwd_quant(int dtype, const void* qkv, int B, int N, int H, float pre, int out_fmt, void* Qo, void* SFo, const float* tso, int flags,
                                 void* stream) {
  (void)pre;
  return attn_launch(dtype, qkv, nullptr, B, N, H, out_fmt, Qo, SFo, tso, flags, stream);
}
