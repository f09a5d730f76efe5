// Block-scaled GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs on two SMs computes one 256 x 256 output
// tile.  Each CTA loads its own 128 rows of A and its own 128 rows of W (= 128 of the 256 tile columns) per stage, the
// leader CTA issues one M = 256, N = 256 MMA per 32 K-bytes, every SM reads only its half of the operands from its own
// shared memory and accumulates its 128 rows x 256 columns in its own tensor memory.  Against the one-CTA kernel
// (kf_gemm.cu, 128 x 256 tiles) this halves the W bytes each SM writes and reads per FLOP, which is what bounds that
// kernel's main loop.  Epilogues, operand formats and the C-ABI are the same (kf_gemm_epi.cuh, kf_gemm_bs).
//
//   hand-shakes   full[s]       leader only: the TMA loads of BOTH CTAs complete on it (cta_group::2 loads signal a barrier
//                               of either CTA of the pair); operand tiles and scale atoms all go through tensor maps
//                 empty[s]      per CTA: the leader's MMA thread commits once to its own and once to the follower's barrier
//                 sf_full/empty leader only: scale-factor buffers in tensor memory (copied for both CTAs by the leader)
//                 tfull         per CTA: committed like empty[s]
//                 tempty        leader only, 32 arrivals: the epilogue warps of both CTAs have the accumulator in registers
//   Every wait is bounded; the two cluster barriers (start, teardown) are reached by every thread on every path.
//
// Replaces the same reference kernels as kf_gemm.cu: infer-opt/round13_mxfp8_full/impl/mgx_core.cu:118-444 and
// infer-opt/round14_fp4_full/impl/fp4g_core.cu:153-470.
#include "kf_gemm_epi.cuh"
#include "kf_sm100_pair.cuh"

namespace kf {

constexpr int P_TILE_BYTES = 2 * 128 * BKB;              // 16 KB of A rows + 16 KB of W rows per CTA and stage
template <int EPI>
struct PairPipe {                                        // as many stages as fit beside the staging tiles of RES / ROPE: 4, or 5 without
  static constexpr int STG_BYTES = Pipe<EPI>::STG_BYTES;
  static constexpr int STAGES = (227 * 1024 - 512 - STG_BYTES) / (P_TILE_BYTES + SF_STAGE_BYTES);
  static constexpr int SMEM = STAGES * (P_TILE_BYTES + SF_STAGE_BYTES) + STG_BYTES + 512;
};

template <int KIND, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmSA,
                 const __grid_constant__ CUtensorMap tmSW, const GemmArgs g) {
  constexpr int ATOMS = KindTraits<KIND>::ATOMS;
  constexpr bool SCALED = KIND != KIND_BF16;
  constexpr int P_STAGES = PairPipe<EPI>::STAGES;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* tiles = smem;
  uint8_t* sfs = smem + (size_t)P_STAGES * P_TILE_BYTES;
  uint8_t* stg_all = sfs + (size_t)P_STAGES * SF_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg_all + PairPipe<EPI>::STG_BYTES);
  uint64_t *full = bars, *empty = full + P_STAGES, *tfull = empty + P_STAGES, *tempty = tfull + 1;
  uint64_t *sf_full = tempty + 1, *sf_empty = sf_full + SF_BUFS;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(sf_empty + SF_BUFS);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  uint32_t* bad_flag = tmem_holder + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                 // 0 = leader (issues the MMAs), 1 = follower
  const uint32_t peer = rank ^ 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < SF_BUFS; ++b) {
      mbar_init(&sf_full[b], 1);
      mbar_init(&sf_empty[b], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, 2 * EPI_WARPS);
    *abort_flag = 0;
    *bad_flag = ((smem_u32(smem) & 1023u) ? 1u : 0u) | (g.err[0] != 0 ? 2u : 0u);   // misaligned tiles, or an earlier failure
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmW);
    if (SCALED) {
      prefetch_tmap(&tmSA);
      prefetch_tmap(&tmSW);
    }
  }
  __syncthreads();
  cluster_sync_all();                                      // both CTAs' barriers exist before anything arrives remotely
  const uint32_t bad = *bad_flag | ld_shared_cluster_u32(map_to_rank(bad_flag, peer));   // the same value in both CTAs
  if (bad) {
    if ((bad & 1) && threadIdx.x == 0 && atomicCAS(&g.err[0], 0u, (unsigned)(-KF_ERR_DEVICE_WAIT)) == 0u) {
      g.err[1] = 100;
      g.err[2] = blockIdx.x;
    }
    cluster_sync_all();                                    // the peer may still be reading this CTA's flag
    return;
  }
  if (warp == 1) {
    tmem_alloc2(tmem_holder, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const WaitCtx ctx{abort_flag, g.err};
  const int m_pairs = (g.m_tiles + 1) >> 1;
  const int total_tiles = m_pairs * g.n_tiles;
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs, own halves)
    if (lane == 0) {
      const uint32_t leader_full = map_to_rank(&full[0], 0);               // every load of the pair reports to the leader's barrier
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
        const int m_pair = tile / g.n_tiles, n_blk = tile - m_pair * g.n_tiles;
        const int m_blk = 2 * m_pair + (int)rank;                             // this CTA's 128 rows of A / of the output
        const int w_halves = (n_blk * BN + 128 < g.N) ? 2 : 1;              // the last column tile may hold only 128 columns
        const uint32_t tx = 2 * (P_TILE_BYTES + (SCALED ? (1 + w_halves) * ATOMS * 512 : 0));   // both CTAs' bytes
        for (int kt = 0; kt < g.k_tiles; ++kt) {
          if (!mbar_wait_cluster(&empty[s], ph ^ 1, ctx, 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(&full[s], tx);
          const uint32_t bar = leader_full + s * 8;
          uint8_t* ta = tiles + (size_t)s * P_TILE_BYTES;
          tma_load_2d_pair(ta, &tmA, kt * BKB, m_blk * 128, bar);               // rows past M are filled with zeros
          tma_load_2d_pair(ta + 128 * BKB, &tmW, kt * BKB, n_blk * BN + (int)rank * 128, bar);   // rows past N likewise
          if (SCALED) {
            uint8_t* sa = sfs + (size_t)s * SF_STAGE_BYTES;
            const int m_sf = m_blk < g.m_tiles ? m_blk : g.m_tiles - 1;         // a row block past M has no scale atoms: any valid ones do (codes are zero)
            tma_load_2d_pair(sa, &tmSA, 0, m_sf * g.nkb4 + kt * ATOMS, bar);
            for (int h = 0; h < w_halves; ++h) tma_load_2d_pair(sa + (1 + h) * ATOMS * 512, &tmSW, 0, (2 * n_blk + h) * g.nkb4 + kt * ATOMS, bar);
          }
          if (++s == P_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t IDESC = KIND == KIND_BF16 ? idesc2_f16(1, BN)
                                 : KIND == KIND_MX8 ? idesc2_bs(0, 1, BN)
                                 : KIND == KIND_NV4 ? idesc2_bs(1, 0, BN)
                                                    : idesc2_bs(1, 1, BN);
      const uint32_t peer_empty = map_to_rank(&empty[0], 1), peer_tfull = map_to_rank(tfull, 1);
      uint32_t s = 0, ph = 0, lt = 0, sb = 0, sph = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs, ++lt) {
        if (!mbar_wait_cluster(tempty, (lt & 1) ^ 1, ctx, 2)) break;          // both CTAs' epilogues have taken the previous tile out of TMEM
        tc_fence_after();
        const uint32_t d_tmem = tmem_base;
        for (int kt = 0; kt < g.k_tiles; ++kt) {
          if (!mbar_wait_cluster(&full[s], ph, ctx, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * P_TILE_BYTES);
          const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(a_addr + 128 * BKB);
          const uint32_t sf_t = tmem_base + TMEM_SF_COL + sb * SF_BUF_COLS;
          if (SCALED) {
            if (!mbar_wait(&sf_full[sb], sph, ctx, 5)) { ok = false; break; }
            tc_fence_after();
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {                                       // 32 K-bytes per MMA
            const uint32_t acc = (kt | j) != 0;
            const uint64_t ad = adesc + 2 * j, bd = bdesc + 2 * j;
            if (KIND == KIND_BF16) {
              mma2_f16(d_tmem, ad, bd, IDESC, acc);
            } else if (KIND == KIND_MX8) {
              mma2_mxf8(d_tmem, ad, bd, idesc_with_sf_id(IDESC, j, j), acc, sf_t, sf_t + 16);
            } else if (KIND == KIND_NV4) {
              mma2_nvf4(d_tmem, ad, bd, IDESC, acc, sf_t + 4 * j, sf_t + 16 + 8 * j);
            } else {
              mma2_mxf4(d_tmem, ad, bd, idesc_with_sf_id(IDESC, 2 * (j & 1), 2 * (j & 1)), acc, sf_t + 4 * (j >> 1), sf_t + 16 + 8 * (j >> 1));
            }
          }
          tc_commit2(&empty[s]);                                             // the stage is free again, in both CTAs
          tc_commit2_to(peer_empty + s * 8);
          if (SCALED) {
            tc_commit2(&sf_empty[sb]);
            if (++sb == SF_BUFS) { sb = 0; sph ^= 1; }
          }
          if (++s == P_STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) {
          tc_commit2(tfull);
          tc_commit2_to(peer_tfull);
        }
      }
    }
    __syncwarp();
  } else if (warp == SF_WARP) {
    if (SCALED && lane == 0 && rank == 0) {
      // ---------------------------------------------------------------- leader: scale atoms shared memory -> tensor memory, in both CTAs
      uint32_t s = 0, ph = 0, sb = 0, sph = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
        const int n_blk = tile % g.n_tiles;
        const int w_halves = (n_blk * BN + 128 < g.N) ? 2 : 1;
        for (int kt = 0; kt < g.k_tiles; ++kt) {
          if (!mbar_wait(&sf_empty[sb], sph ^ 1, ctx, 6)) { ok = false; break; }
          if (!mbar_wait_cluster(&full[s], ph, ctx, 7)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sf_t = tmem_base + TMEM_SF_COL + sb * SF_BUF_COLS;
          const uint32_t sa = smem_u32(sfs + (size_t)s * SF_STAGE_BYTES);
#pragma unroll
          for (int a = 0; a < ATOMS; ++a) {
            tc_cp_sf2(sf_t + 4 * a, smem_desc_sf(sa + a * 512));
            tc_cp_sf2(sf_t + 16 + 8 * a, smem_desc_sf(sa + (ATOMS + a) * 512));
            if (w_halves == 2) tc_cp_sf2(sf_t + 16 + 8 * a + 4, smem_desc_sf(sa + (2 * ATOMS + a) * 512));
          }
          tc_commit2(&sf_full[sb]);
          if (++sb == SF_BUFS) { sb = 0; sph ^= 1; }
          if (++s == P_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue: 16 warps per CTA, warp = (TMEM lane quarter, 64-column group)
    const int quarter = warp & 3;
    const int cg = (warp - 2) >> 2;
    float* stg = reinterpret_cast<float*>(stg_all + (size_t)(warp - 2) * Pipe<EPI>::STG_STRIDE);   // staging tile, or the warp's bias slice
    float ts = 1.f;
    if (g.ts_a) ts *= __ldg(g.ts_a);
    if (g.ts_w) ts *= __ldg(g.ts_w);
    const Nv4Scale sco = nv4_scale((EPI == KF_EPI_QUANT && g.out_fmt == KF_FMT_NV4) ? __ldg(g.tso) : 1.f);   // once per CTA: every global load here is an L2 round trip
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + cg * 64;
    const uint32_t leader_tempty = map_to_rank(tempty, 0);
    uint32_t lt = 0;
    for (int tile = pair_id; tile < total_tiles; tile += n_pairs, ++lt) {
      const int m_pair = tile / g.n_tiles, n_blk = tile - m_pair * g.n_tiles;
      const int rbase = (2 * m_pair + (int)rank) * 128 + quarter * 32;
      const int n0 = n_blk * BN + cg * 64;
      uint32_t r0[32], r1[32];
      epilogue_bias_stage<EPI>(g, n0, stg, lane);
      EpiPre pre;
      epilogue_prefetch<EPI>(g, n0, lane, pre);
      if (!mbar_wait_cluster(tfull, lt & 1, ctx, 4)) break;
      tc_fence_after();
      tmem_ld32(taddr, r0);
      tmem_ld32(taddr + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(leader_tempty);          // the accumulator is in registers: hand TMEM back (to the leader's MMA warp)
      if (n0 >= g.N || rbase >= g.m_tiles * 128) continue;        // column group past N, or the follower's row block past the last one
      epilogue_math<EPI>(g, r0, r1, ts, sco, rbase, n0, stg, lane, pre);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {                 // a wait ran out: give copies still in flight time to land before the CTA exits
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  cluster_sync_all();                // no remote arrival or pair MMA may target a CTA that has already left
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <int KIND, int EPI>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmSA, const CUtensorMap& tmSW, const GemmArgs& g, int grid,
                       cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<KIND, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairPipe<EPI>::SMEM);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(gemm_pair_kernel)");
    if (dev < 64) attr_set[dev] = true;
  }
  gemm_pair_kernel<KIND, EPI><<<grid, GEMM_THREADS, PairPipe<EPI>::SMEM, st>>>(tmA, tmW, tmSA, tmSW, g);
  return cuda_status(cudaGetLastError(), "kf_gemm_bs (pair) launch");
}

template <int KIND>
static int launch_pair_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmSA, const CUtensorMap& tmSW, const GemmArgs& g,
                           int grid, cudaStream_t st) {
  switch (epi) {
    case KF_EPI_PLAIN: return launch_pair<KIND, KF_EPI_PLAIN>(tmA, tmW, tmSA, tmSW, g, grid, st);
    case KF_EPI_RES: return launch_pair<KIND, KF_EPI_RES>(tmA, tmW, tmSA, tmSW, g, grid, st);
    case KF_EPI_ROPE: return launch_pair<KIND, KF_EPI_ROPE>(tmA, tmW, tmSA, tmSW, g, grid, st);
    default: return launch_pair<KIND, KF_EPI_QUANT>(tmA, tmW, tmSA, tmSW, g, grid, st);
  }
}

// Scale atoms as a 2-D tensor: one row = one 512-byte atom (128 x u32), box = the `atoms` consecutive atoms of one stage.
static int make_tmap_atoms(CUtensorMap* map, const void* base, uint64_t n_atoms, uint32_t atoms) {
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                         CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<Fn>(p);
  }
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return KF_ERR_UNSUPPORTED;
  }
  cuuint64_t dims[2] = {128, n_atoms};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, atoms};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (scale atoms) failed with CUresult %d", (int)r);
    return KF_ERR_BAD_ARGUMENT;
  }
  return KF_OK;
}

// Called by kf_gemm_bs with validated arguments; tmW must have a 128-row box.
int launch_gemm_pair(int fmt, int epi, const CUtensorMap& tmA, const CUtensorMap& tmW, const GemmArgs& g, int sms, cudaStream_t st) {
  CUtensorMap tmSA = tmA, tmSW = tmW;                    // unused by the bf16 kind
  if (fmt != KF_FMT_BF16) {
    const uint32_t atoms = fmt == KF_FMT_NV4 ? 4 : (fmt == KF_FMT_MX4 ? 2 : 1);
    int rc = make_tmap_atoms(&tmSA, g.sfa, (uint64_t)g.m_tiles * g.nkb4, atoms);
    if (rc != KF_OK) return rc;
    rc = make_tmap_atoms(&tmSW, g.sfw, (uint64_t)((g.N + 127) / 128) * g.nkb4, atoms);
    if (rc != KF_OK) return rc;
  }
  const int m_pairs = (g.m_tiles + 1) / 2;
  const int total = m_pairs * g.n_tiles;
  int pairs = sms / 2;
  if (pairs > total) pairs = total;
  const int grid = 2 * pairs;
  switch (fmt) {
    case KF_FMT_MX8: return launch_pair_epi<KIND_MX8>(epi, tmA, tmW, tmSA, tmSW, g, grid, st);
    case KF_FMT_NV4: return launch_pair_epi<KIND_NV4>(epi, tmA, tmW, tmSA, tmSW, g, grid, st);
    case KF_FMT_MX4: return launch_pair_epi<KIND_MX4>(epi, tmA, tmW, tmSA, tmSW, g, grid, st);
    default: return launch_pair_epi<KIND_BF16>(epi, tmA, tmW, tmSA, tmSW, g, grid, st);
  }
}

}  // namespace kf
