// Block-scaled GEMM  C[M,N] = A[M,K] * W[N,K]^T  on the sm_100a tensor cores (tcgen05.mma, fp32 accumulators in
// TMEM) with the epilogues of the ViT block fused in.
//
//   operands   K-major codes: e4m3 bytes (mx8), packed e2m1 nibbles (nv4 / mx4) or plain bf16; scale factors in
//              the 128x4 blocked layout, one 512-byte atom per 128 rows x 4 k-blocks
//   tile       128 x 256 output tile per CTA step (one MMA instruction is 128 x 256 x 32 K-bytes), 128 bytes of K per
//              pipeline stage.  The tile shape is set by shared-memory bandwidth: a 128 x 128 MMA reads its 8 KB of
//              operands in the ~68 clk it executes, which alone saturates the 128 B/clk of the shared-memory array,
//              and the TMA writes of the next stages need the same array (measured: main loop at half the instruction
//              rate).  At 128 x 256 an MMA reads 12 KB per ~136 clk.
//   pipeline   20 warps.  Warp group 0: warp 0 = TMA producer (operand tiles by tensor map, scale atoms by 1-D bulk copy),
//              warp 1 = MMA issuer (4 MMAs per stage), warp 2 = scale-factor copier (tcgen05.cp atoms smem -> TMEM; the
//              copies take tensor-pipe time but overlap the MMAs when another warp issues them), warp 3 idle.  Warp groups
//              1..4 = 16 epilogue warps.  Registers are re-balanced between the roles (setmaxnreg, per epilogue kind): the three single-thread
//              roles give theirs up and every epilogue thread holds its 64 accumulator values plus loads in flight
//              without spilling.
//              One 256-column accumulator in TMEM: each epilogue warp takes (32-row TMEM quarter, 64 columns) into
//              registers and hands TMEM back at once, so the next tile's main loop runs under the epilogue math;
//              persistent CTAs, one per SM, static round-robin over tiles
//   epilogues  PLAIN  out = act(acc*ts + bias)                       -> f32 | bf16 | f16 [M,N]
//              RES    out = R + gamma * (acc*ts + bias)              -> f32 [M,N]         (proj, fc2)
//              ROPE   bias + rotary embedding of q,k + relayout      -> bf16 | f16 [3,B,Ntok,H,64]   (qkv)
//              QUANT  gelu(acc*ts + bias) quantised again            -> codes [M,N] + blocked scales (fc1 -> fc2)
//              all four work in the TMEM row layout (a thread owns 64 consecutive columns of one row) and touch global
//              memory in whole 32-byte sectors (kf_gemm_epi.cuh)
//
// Replaces (reference checkout paths): infer-opt/round13_mxfp8_full/impl/mgx_core.cu:118-444 (MXFP8, mma.sync) and
// infer-opt/round14_fp4_full/impl/fp4g_core.cu:153-470 (NVFP4 / MXFP4, mma.sync); epilogue math per
// mgx_core.cu:308-426 and fp4g_core.cu:309-382.
#include <mutex>

#include "kf_gemm_epi.cuh"

namespace kf {

// Depth of the operand ring, chosen per launch.  A fourth stage (54 KB) helps where the main loop is the longer chain
// (measured at M = 22 470: fc2 K 4096 79 -> 76 us, MXFP8 fc2 116 -> 108 us, PLAIN 73 -> 69 us) and hurts where the epilogue is
// (proj 51 -> 53 us, fc1 93 -> 98 us: the stage's shared memory comes out of the L1 the epilogue's global accesses use);
// the ROPE kernel's table slabs leave no room for one.
constexpr int MAX_STAGES = 4;
static int gemm_stages(int epi, int k_tiles, int flags) {
  if (epi == KF_EPI_PLAIN) return (flags & KF_G_GELU) ? 3 : 4;      // PLAIN with GELU (the head's ConvTranspose GEMMs) is epilogue-bound too
  if (epi == KF_EPI_RES && k_tiles >= 8) return 4;
  return 3;
}
constexpr size_t GEMM_SMEM_MAX = 227 * 1024;
template <int EPI>
constexpr size_t gemm_smem(int stages, int vec_floats = 0) {   // operand ring + scale atoms + bias slices or vectors (+ the rotary-table slabs) + barriers
  const size_t sl = (size_t)(vec_floats > EPI_WARPS * SLICE_FLOATS ? vec_floats : EPI_WARPS * SLICE_FLOATS) * 4;
  return (size_t)stages * (TILE_BYTES + SF_STAGE_BYTES) + sl + (EPI == KF_EPI_ROPE ? 4 * ROPE_SLAB_FLOATS * 4 : 0) + 256;
}

// ------------------------------------------------------------------------------------------------ the kernel
template <int KIND, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const GemmArgs g) {
  constexpr int ATOMS = KindTraits<KIND>::ATOMS;
  constexpr bool SCALED = KIND != KIND_BF16;
  const int STAGES = g.stages;                            // 3 or 4: the ring depth this launch was given shared memory for

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* tiles = smem;
  uint8_t* sfs = smem + (size_t)STAGES * TILE_BYTES;
  float* slices = reinterpret_cast<float*>(sfs + (size_t)STAGES * SF_STAGE_BYTES);
  float* slabs = slices + (g.vec_floats > EPI_WARPS * SLICE_FLOATS ? g.vec_floats : EPI_WARPS * SLICE_FLOATS);   // ROPE only
  uint64_t* bars = reinterpret_cast<uint64_t*>(slabs + (EPI == KF_EPI_ROPE ? 4 * ROPE_SLAB_FLOATS : 0));
  uint64_t *full = bars, *empty = bars + MAX_STAGES, *tfull = bars + 2 * MAX_STAGES, *tempty = tfull + 1;
  uint64_t *sf_full = tempty + 1, *sf_empty = sf_full + SF_BUFS;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(sf_empty + SF_BUFS);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  pdl_launch_dependents();                               // the next kernel of the stream may take the SMs this grid leaves
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < SF_BUFS; ++b) {
      mbar_init(&sf_full[b], 1);
      mbar_init(&sf_empty[b], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, EPI_WARPS);
    *abort_flag = (smem_u32(smem) & 1023u) ? 1u : 0u;     // the swizzled operand tiles need a 1024-byte aligned base
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();                                            // set-up done: from here on global memory of the predecessors is read and written
  const uint32_t tmem_base = *tmem_holder;
  const WaitCtx ctx{abort_flag, g.err};
  const int total_tiles = g.m_tiles * g.n_tiles;
  const bool bad_align = *abort_flag != 0 || g.err[0] != 0;   // misaligned tiles, or an earlier CTA / launch already failed: skip the work
  if (*abort_flag != 0 && threadIdx.x == 0 && atomicCAS(&g.err[0], 0u, (unsigned)(-KF_ERR_DEVICE_WAIT)) == 0u) {
    g.err[1] = 100;
    g.err[2] = blockIdx.x;
  }

  if (warp < EPI_WARP0) {
    setmaxnreg_dec<EPI == KF_EPI_ROPE ? REGS_LEAN_ROPE : REGS_LEAN>();
    if (bad_align) {
      // nothing is issued; fall through to the teardown
    } else if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
          const int m_blk = tile / g.n_tiles, n_blk = tile - m_blk * g.n_tiles;
          const int w_halves = (n_blk * BN + 128 < g.N) ? 2 : 1;              // the last column tile may hold only 128 columns
          int row_end;
          const int a_row0 = tile_row0(g, m_blk, row_end), w_row0 = tile_wrow0(g, m_blk, n_blk);
          const uint32_t tx = TILE_BYTES + (SCALED ? (1 + w_halves) * ATOMS * 512 : 0);
          for (int kt = 0; kt < g.k_tiles; ++kt) {
            if (!mbar_wait(&empty[s], ph ^ 1, ctx, 1)) { ok = false; break; }
            mbar_expect_tx(&full[s], tx);
            uint8_t* ta = tiles + (size_t)s * TILE_BYTES;
            tma_load_2d(ta, &tmA, kt * BKB, a_row0, &full[s]);
            tma_load_2d(ta + A_BYTES, &tmW, kt * BKB, w_row0, &full[s]);       // rows past the end of W are filled with zeros
            if (SCALED) {
              uint8_t* sa = sfs + (size_t)s * SF_STAGE_BYTES;
              bulk_load_1d(sa, g.sfa + ((size_t)m_blk * g.nkb4 + (size_t)kt * ATOMS) * 512, ATOMS * 512, &full[s]);
              for (int h = 0; h < w_halves; ++h)
                bulk_load_1d(sa + (1 + h) * ATOMS * 512, g.sfw + ((size_t)(2 * n_blk + h) * g.nkb4 + (size_t)kt * ATOMS) * 512, ATOMS * 512, &full[s]);
            }
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t IDESC = KIND == KIND_BF16 ? idesc_f16(1, BN)
                                   : KIND == KIND_MX8 ? idesc_bs(0, 1, BN)
                                   : KIND == KIND_NV4 ? idesc_bs(1, 0, BN)
                                                      : idesc_bs(1, 1, BN);
        uint32_t s = 0, ph = 0, lt = 0, sb = 0, sph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++lt) {
          if (!mbar_wait(tempty, (lt & 1) ^ 1, ctx, 2)) break;                  // the epilogue has taken the previous tile out of TMEM
          tc_fence_after();
          const uint32_t d_tmem = tmem_base;
          for (int kt = 0; kt < g.k_tiles; ++kt) {
            if (!mbar_wait(&full[s], ph, ctx, 3)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(tiles + (size_t)s * TILE_BYTES);
            const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(a_addr + A_BYTES);
            // scale factors of this stage: A at +0 (4 columns per atom), W at +16 (8 columns per atom pair: the atom of
            // columns 0..127 of the tile, then the atom of columns 128..255)
            const uint32_t sf_t = tmem_base + TMEM_SF_COL + sb * SF_BUF_COLS;
            if (SCALED) {                          // copied into TMEM by the scale-copy warp, which runs ahead of the MMAs
              if (!mbar_wait(&sf_full[sb], sph, ctx, 5)) { ok = false; break; }
              tc_fence_after();
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {                                       // 32 K-bytes per MMA
              const uint32_t acc = (kt | j) != 0;
              const uint64_t ad = adesc + 2 * j, bd = bdesc + 2 * j;
              if (KIND == KIND_BF16) {
                mma_f16(d_tmem, ad, bd, IDESC, acc);
              } else if (KIND == KIND_MX8) {      // one scale per row per MMA: byte j of the atom's 32-bit word
                mma_mxf8(d_tmem, ad, bd, idesc_with_sf_id(IDESC, j, j), acc, sf_t, sf_t + 16);
              } else if (KIND == KIND_NV4) {      // four scales per row per MMA: atom j
                mma_nvf4(d_tmem, ad, bd, IDESC, acc, sf_t + 4 * j, sf_t + 16 + 8 * j);
              } else {                            // two scales per row per MMA: half-word (j & 1) of atom j / 2
                mma_mxf4(d_tmem, ad, bd, idesc_with_sf_id(IDESC, 2 * (j & 1), 2 * (j & 1)), acc, sf_t + 4 * (j >> 1), sf_t + 16 + 8 * (j >> 1));
              }
            }
            tc_commit(&empty[s]);
            if (SCALED) {
              tc_commit(&sf_empty[sb]);
              if (++sb == SF_BUFS) { sb = 0; sph ^= 1; }
            }
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
          if (ok) tc_commit(tfull);
        }
      }
      __syncwarp();
    } else if (warp == 2) {
      // ------------------------------------------------------------------ scale-factor copier
      // tcgen05.cp of one 512-byte atom costs about as much tensor-pipe time as a 128 x 128 MMA, but it overlaps with
      // the MMAs when it is issued from another warp; issued from the MMA thread the two serialise.  This warp therefore
      // moves the atoms of stage s (shared memory -> one of SF_BUFS TMEM buffers) as soon as the TMA has landed them and
      // hands the buffer to the MMA warp through an mbarrier.
      if (SCALED && lane == 0) {
        uint32_t s = 0, ph = 0, sb = 0, sph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
          const int n_blk = tile % g.n_tiles;
          const int w_halves = (n_blk * BN + 128 < g.N) ? 2 : 1;
          for (int kt = 0; kt < g.k_tiles; ++kt) {
            if (!mbar_wait(&sf_empty[sb], sph ^ 1, ctx, 6)) { ok = false; break; }
            if (!mbar_wait(&full[s], ph, ctx, 7)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sf_t = tmem_base + TMEM_SF_COL + sb * SF_BUF_COLS;
            const uint32_t sa = smem_u32(sfs + (size_t)s * SF_STAGE_BYTES);
#pragma unroll
            for (int a = 0; a < ATOMS; ++a) {
              tc_cp_sf(sf_t + 4 * a, smem_desc_sf(sa + a * 512));
              tc_cp_sf(sf_t + 16 + 8 * a, smem_desc_sf(sa + (ATOMS + a) * 512));
              if (w_halves == 2) tc_cp_sf(sf_t + 16 + 8 * a + 4, smem_desc_sf(sa + (2 * ATOMS + a) * 512));
            }
            tc_commit(&sf_full[sb]);
            if (++sb == SF_BUFS) { sb = 0; sph ^= 1; }
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 16 warps, warp = (TMEM lane quarter, 64-column group)
    setmaxnreg_inc<EPI == KF_EPI_ROPE ? REGS_EPI_ROPE : REGS_EPI>();
    if (!bad_align) {
      const TileSched sched{(int)blockIdx.x, (int)gridDim.x, total_tiles, g.n_tiles, -1};
      epilogue_warps<EPI>(g, sched, tmem_base, tfull, tempty, slices, slabs, ctx, warp, lane);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {                 // a wait ran out: give copies still in flight time to land before the CTA exits
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Encoding a tensor map costs about a microsecond of host time; an eager caller (the Linear swap) issues the same few
// (pointer, shape) combinations over and over, so the encoded maps are kept in a small per-thread direct-mapped cache.
struct TmapKey {
  const void* base;
  uint64_t rows, row_bytes, pitch_bytes;
  uint32_t box_rows;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && row_bytes == o.row_bytes && pitch_bytes == o.pitch_bytes && box_rows == o.box_rows;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};

int make_tmap_2d_bytes(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch_bytes, uint32_t box_rows) {
  constexpr int SLOTS = 256;
  static thread_local TmapSlot cache[SLOTS] = {};
  const TmapKey key{base, rows, row_bytes, pitch_bytes, box_rows};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 8;
  h ^= rows * 0x9E3779B97F4A7C15ull;
  h ^= (row_bytes << 7) ^ box_rows;
  TmapSlot& slot = cache[(h ^ (h >> 17)) % SLOTS];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    return KF_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return KF_ERR_UNSUPPORTED;
  }
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (base %p rows %llu row_bytes %llu)", (int)r, base, (unsigned long long)rows,
              (unsigned long long)row_bytes);
    return KF_ERR_BAD_ARGUMENT;
  }
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return KF_OK;
}

int device_sm_count(int* sms) {
  static int cached[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
  if (dev < 64 && cached[dev]) {
    *sms = cached[dev];
    return KF_OK;
  }
  int n = 0;
  e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_status(e, "cudaDeviceGetAttribute");
  if (dev < 64) cached[dev] = n;
  *sms = n;
  return KF_OK;
}

template <int KIND, int EPI>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmW, const GemmArgs& g, int grid, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<KIND, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_MAX);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(gemm_kernel)");
    if (dev < 64) attr_set[dev] = true;
  }
  return cuda_status(launch_maybe_pdl(gemm_kernel<KIND, EPI>, dim3(grid), dim3(GEMM_THREADS), gemm_smem<EPI>(g.stages, g.vec_floats), st, tmA, tmW, g), "kf_gemm_bs launch");
}

template <int KIND>
static int launch_gemm_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmW, const GemmArgs& g, int grid, cudaStream_t st) {
  switch (epi) {
    case KF_EPI_PLAIN: return launch_gemm<KIND, KF_EPI_PLAIN>(tmA, tmW, g, grid, st);
    case KF_EPI_RES: return launch_gemm<KIND, KF_EPI_RES>(tmA, tmW, g, grid, st);
    case KF_EPI_ROPE: return launch_gemm<KIND, KF_EPI_ROPE>(tmA, tmW, g, grid, st);
    default: return launch_gemm<KIND, KF_EPI_QUANT>(tmA, tmW, g, grid, st);
  }
}

static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool al32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }   // 256-bit global accesses of the epilogues

}  // namespace kf

using namespace kf;

extern "C" int kf_gemm_bs(const kf_gemm_params* p, void* stream) {
  KF_REQUIRE(p != nullptr, "kf_gemm_bs: null parameter block");
  const int fmt = p->fmt, epi = p->epi;
  KF_REQUIRE(fmt >= KF_FMT_MX8 && fmt <= KF_FMT_BF16, "kf_gemm_bs: unknown operand format %d", fmt);
  KF_REQUIRE(epi >= KF_EPI_PLAIN && epi <= KF_EPI_QUANT, "kf_gemm_bs: unknown epilogue %d", epi);
  KF_REQUIRE(p->M >= 0 && p->N > 0 && p->K > 0, "kf_gemm_bs: bad shape M=%d N=%d K=%d", p->M, p->N, p->K);
  KF_REQUIRE(p->N % 128 == 0, "kf_gemm_bs: N=%d must be a multiple of 128", p->N);
  const int kelems = fmt == KF_FMT_MX8 ? 128 : (fmt == KF_FMT_BF16 ? 64 : 256);   // K elements per 128-byte stage
  KF_REQUIRE(p->K % kelems == 0, "kf_gemm_bs: K=%d must be a multiple of %d for this format", p->K, kelems);
  if (p->M == 0) return KF_OK;
  KF_REQUIRE(p->A && p->W && al16(p->A) && al16(p->W), "kf_gemm_bs: A and W must be non-null and 16-byte aligned");
  if (fmt != KF_FMT_BF16) KF_REQUIRE(p->SFA && p->SFW && al16(p->SFA) && al16(p->SFW), "kf_gemm_bs: scale tensors must be non-null and 16-byte aligned");
  KF_REQUIRE(!p->bias || al16(p->bias), "kf_gemm_bs: bias must be 16-byte aligned");
  if (epi == KF_EPI_PLAIN) {
    KF_REQUIRE(p->C && al32(p->C), "kf_gemm_bs: PLAIN needs a 32-byte aligned output C");
    KF_REQUIRE(p->out_row_group >= 0 && (p->out_row_group == 0 || (p->out_row_stride >= p->out_row_group && p->out_row_offset >= 0)),
               "kf_gemm_bs: bad output row mapping group=%d stride=%d offset=%d", p->out_row_group, p->out_row_stride, p->out_row_offset);
    KF_REQUIRE(p->out_dtype == KF_F32 || p->out_dtype == KF_BF16 || p->out_dtype == KF_F16, "kf_gemm_bs: bad out_dtype %d", p->out_dtype);
  } else if (epi == KF_EPI_RES) {
    KF_REQUIRE(p->C && p->R && p->gamma && al32(p->C) && al32(p->R) && al16(p->gamma), "kf_gemm_bs: RES needs 32-byte aligned C and R and a 16-byte aligned gamma");
    KF_REQUIRE(p->out_row_group >= 0 && (p->out_row_group == 0 || (p->out_row_stride >= p->out_row_group && p->out_row_offset >= 0)),
               "kf_gemm_bs: bad output row mapping group=%d stride=%d offset=%d", p->out_row_group, p->out_row_stride, p->out_row_offset);
    KF_REQUIRE(p->out_row_group == 0 || p->C != p->R, "kf_gemm_bs: RES with an output row mapping cannot run in place");
  } else if (epi == KF_EPI_ROPE) {
    KF_REQUIRE(p->C && al32(p->C) && p->sin && p->cos && al32(p->sin) && al32(p->cos), "kf_gemm_bs: ROPE needs 32-byte aligned C, sin and cos");
    KF_REQUIRE(p->out_dtype == KF_BF16 || p->out_dtype == KF_F16, "kf_gemm_bs: ROPE output must be bf16 or f16");
    KF_REQUIRE(p->H > 0 && p->N == 3 * p->H * 64, "kf_gemm_bs: ROPE needs N = 3*H*64 (N=%d, H=%d)", p->N, p->H);
    KF_REQUIRE(p->Ntok > 0 && p->M % p->Ntok == 0 && p->prefix >= 0 && p->prefix <= p->Ntok, "kf_gemm_bs: ROPE needs M %% Ntok == 0 and 0 <= prefix <= Ntok");
  } else {
    KF_REQUIRE(p->out_fmt == KF_FMT_MX8 || p->out_fmt == KF_FMT_NV4 || p->out_fmt == KF_FMT_MX4, "kf_gemm_bs: bad quantise-out format %d", p->out_fmt);
    KF_REQUIRE(p->Qo && p->SFo && al32(p->Qo) && al16(p->SFo), "kf_gemm_bs: QUANT needs a 32-byte aligned Qo and a 16-byte aligned SFo");
    KF_REQUIRE(p->out_fmt != KF_FMT_NV4 || p->tso, "kf_gemm_bs: nv4 quantise-out needs the per-tensor scale tso");
    KF_REQUIRE(!p->y_dbg || al16(p->y_dbg), "kf_gemm_bs: y_dbg must be 16-byte aligned");
  }
  KF_REQUIRE(p->batch >= 0, "kf_gemm_bs: negative batch");
  if (p->batch > 0) {
    KF_REQUIRE(fmt == KF_FMT_BF16 && epi == KF_EPI_PLAIN && p->out_row_group == 0, "kf_gemm_bs: batched products need bf16 operands, the PLAIN epilogue and no output row mapping");
    KF_REQUIRE(p->a_rows_per_batch > 0 && (long long)p->batch * p->a_rows_per_batch == p->M && p->w_rows_per_batch >= p->N,
               "kf_gemm_bs: batched products need M = batch * a_rows_per_batch and w_rows_per_batch >= N (batch=%d, rows=%d, M=%d, w rows=%d, N=%d)",
               p->batch, p->a_rows_per_batch, p->M, p->w_rows_per_batch, p->N);
  }
  const uint64_t kbytes = fmt == KF_FMT_MX8 ? (uint64_t)p->K : (fmt == KF_FMT_BF16 ? 2ull * p->K : (uint64_t)p->K / 2);
  const uint64_t w_rows = p->batch > 0 ? (uint64_t)p->batch * p->w_rows_per_batch : (uint64_t)p->N;
  CUtensorMap tmA, tmW;
  int st = make_tmap_2d_bytes(&tmA, p->A, (uint64_t)p->M, kbytes, kbytes, BM);
  if (st != KF_OK) return st;
  st = make_tmap_2d_bytes(&tmW, p->W, w_rows, kbytes, kbytes, BN);
  if (st != KF_OK) return st;
  GemmArgs g{};
  g.sfa = static_cast<const uint8_t*>(p->SFA);
  g.sfw = static_cast<const uint8_t*>(p->SFW);
  g.ts_a = p->ts_a; g.ts_w = p->ts_w; g.bias = p->bias; g.gamma = p->gamma; g.R = p->R; g.sin = p->sin; g.cos = p->cos; g.tso = p->tso;
  g.C = p->C; g.Qo = static_cast<uint8_t*>(p->Qo); g.SFo = static_cast<uint8_t*>(p->SFo);
  g.M = p->M; g.N = p->N; g.K = p->K;
  g.Ntok = p->Ntok; g.prefix = p->prefix; g.H = p->H; g.d = p->H * 64;
  g.out_dtype = p->out_dtype; g.flags = p->flags; g.out_fmt = p->out_fmt;
  g.m_tiles = (p->M + BM - 1) / BM; g.n_tiles = (p->N + BN - 1) / BN; g.k_tiles = (int)(kbytes / BKB);
  if (p->batch > 0) {
    g.m_tiles_pb = (p->a_rows_per_batch + BM - 1) / BM;
    g.a_rows_pb = p->a_rows_per_batch;
    g.w_rows_pb = p->w_rows_per_batch;
    g.m_tiles = p->batch * g.m_tiles_pb;
  }
  g.nkb4 = fmt == KF_FMT_BF16 ? 0 : p->K / (4 * fmt_vec(fmt));
  g.stages = gemm_stages(epi, g.k_tiles, p->flags);
  {
    // the whole bias (+ LayerScale) vector in shared memory where the ring depth of this launch leaves room for it
    const int want = (p->bias || epi == KF_EPI_RES) ? p->N * (epi == KF_EPI_RES ? 2 : 1) : 0;
    const size_t rest = (size_t)g.stages * (TILE_BYTES + SF_STAGE_BYTES) + (epi == KF_EPI_ROPE ? 4 * ROPE_SLAB_FLOATS * 4 : 0) + 256;
    const size_t vec_bytes = (size_t)(want > EPI_WARPS * SLICE_FLOATS ? want : EPI_WARPS * SLICE_FLOATS) * 4;
    g.vec_floats = (want > 0 && rest + vec_bytes <= GEMM_SMEM_MAX) ? want : 0;
  }
  const bool maps_rows = epi == KF_EPI_PLAIN || epi == KF_EPI_RES;
  g.row_group = maps_rows ? p->out_row_group : 0; g.row_stride = p->out_row_stride; g.row_offset = p->out_row_offset;
  g.y_dbg = epi == KF_EPI_QUANT ? p->y_dbg : nullptr;
  g.err = dev_error_ptr();
  KF_REQUIRE(g.err != nullptr, "kf_gemm_bs: device error word unavailable");
  int sms = 0;
  st = device_sm_count(&sms);
  if (st != KF_OK) return st;
  const int total = g.m_tiles * g.n_tiles;
  const int grid = total < sms ? total : sms;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  switch (fmt) {
    case KF_FMT_MX8: return launch_gemm_epi<KIND_MX8>(epi, tmA, tmW, g, grid, cs);
    case KF_FMT_NV4: return launch_gemm_epi<KIND_NV4>(epi, tmA, tmW, g, grid, cs);
    case KF_FMT_MX4: return launch_gemm_epi<KIND_MX4>(epi, tmA, tmW, g, grid, cs);
    default: return launch_gemm_epi<KIND_BF16>(epi, tmA, tmW, g, grid, cs);
  }
}
