// Instruction-rate probe of the sm_100a tensor core: every SM issues tcgen05.mma back to back on operands that stay
// in shared memory (zero-filled, no TMA traffic) and accumulators that stay in TMEM.  The host times the launch; the
// resulting FLOP rate is the ceiling a GEMM main loop of the same instruction shape can reach on this part at the
// clocks it actually runs at, which is the denominator used for the FP8 / FP4 roofline fractions.
// N = 64 shows what the attention products (64 keys or 64 head columns per MMA) can reach: 1.30 of 2.2 PFLOP/s for bf16.
// Same idea as the reference's register-resident mma.sync probe (infer-opt/round10_lowp_probe/peak_extra.cu).
#include "kf_sm100.cuh"
#include "../../include/kf_b200_dev.h"

namespace kf {

constexpr int PK_SMEM = 1024 + 16384 + 32768 + 4096 + 64;

template <int KIND, int N>
__global__ void __launch_bounds__(128, 1) peak_kernel(int iters, int sf_copies, unsigned int* err) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  uint8_t *a = smem, *b = smem + 16384, *sf = smem + 16384 + 32768;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sf + 4096);
  uint32_t* holder = reinterpret_cast<uint32_t*>(bar + 1);
  volatile uint32_t* abort_flag = holder + 1;
  for (int i = threadIdx.x; i < (16384 + 32768 + 4096) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init(bar + 2, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc(holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  const WaitCtx ctx{abort_flag, err};
  if (threadIdx.x == 0) {
    constexpr uint32_t IDESC = KIND == KF_FMT_BF16 ? idesc_f16(1, N) : KIND == KF_FMT_MX8 ? idesc_bs(0, 1, N) : KIND == KF_FMT_NV4 ? idesc_bs(1, 0, N) : idesc_bs(1, 1, N);
    const uint64_t ad = smem_desc_sw128(smem_u32(a)), bd = smem_desc_sw128(smem_u32(b));
    const uint32_t sft = tmem + 256 + (N > 128 ? 128 : 0);
    if (KIND != KF_FMT_BF16) {
      for (int i = 0; i < 8; ++i) tc_cp_sf(sft + 4 * i, smem_desc_sf(smem_u32(sf) + i * 512));
    }
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tmem + ((N <= 128) ? (it & 1) * N : 0);
      if (KIND != KF_FMT_BF16) {           // optionally re-copy scale atoms every stage, as a real main loop must
        for (int c = 0; c < (sf_copies <= 8 ? sf_copies : 0); ++c)
          tc_cp_sf(sft + 32 * (it & 1) + 4 * (c & 7), smem_desc_sf(smem_u32(sf) + (c & 7) * 512));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (KIND == KF_FMT_BF16) mma_f16(d, ad + 2 * j, bd + 2 * j, IDESC, 1);
        else if (KIND == KF_FMT_MX8) mma_mxf8(d, ad + 2 * j, bd + 2 * j, idesc_with_sf_id(IDESC, j, j), 1, sft, sft + 16);
        else if (KIND == KF_FMT_NV4) mma_nvf4(d, ad + 2 * j, bd + 2 * j, IDESC, 1, sft, sft + 16);
        else mma_mxf4(d, ad + 2 * j, bd + 2 * j, idesc_with_sf_id(IDESC, 2 * (j & 1), 2 * (j & 1)), 1, sft, sft + 16);
      }
    }
    tc_commit(bar);
    mbar_wait(bar, 0, ctx, 50);
  } else if (threadIdx.x == 32 && sf_copies > 8 && KIND != KF_FMT_BF16) {
    // sf_copies = 8 + c: the c copies per stage are issued by a second warp into a scratch TMEM region, with no
    // ordering against the MMA stream: shows whether tcgen05.cp and tcgen05.mma overlap in the hardware
    const uint32_t scratch = tmem + 256 + (N > 128 ? 128 : 0) + 64;
    for (int it = 0; it < iters; ++it)
      for (int c = 0; c < sf_copies - 8; ++c) tc_cp_sf(scratch + 4 * (c & 7), smem_desc_sf(smem_u32(sf) + (c & 7) * 512));
    tc_commit(bar + 2);
    mbar_wait(bar + 2, 0, ctx, 51);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int KIND>
static int launch_peak(int n, int iters, int sf_copies, int sms, unsigned int* err, cudaStream_t st) {
  auto go = [&](auto kern) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(peak_kernel)");
    kern<<<sms, 128, PK_SMEM, st>>>(iters, sf_copies, err);
    return cuda_status(cudaGetLastError(), "kf_tensor_peak_probe launch");
  };
  return n == 256 ? go(peak_kernel<KIND, 256>) : n == 128 ? go(peak_kernel<KIND, 128>) : go(peak_kernel<KIND, 64>);
}

// ------------------------------------------------------------------------------------------------ fill-rate probe
// What a GEMM main loop can be fed: every SM streams `iters` stages of `stage_bytes` from global memory into a
// three-stage shared-memory ring with 1-D bulk copies (16 KB pieces, completion on an mbarrier), refilling a stage as
// soon as it has landed; nothing consumes the data.  The source window of `span` bytes is walked by all CTAs at
// staggered offsets (the walks overlap): with a window that fits L2 this is the L2 -> shared-memory rate.
constexpr int FILL_STAGES = 3, FILL_MAX_STAGE = 65536, FILL_SMEM = FILL_STAGES * FILL_MAX_STAGE + 64;

__global__ void __launch_bounds__(128, 1) fill_kernel(const uint8_t* __restrict__ src, size_t span, int stage_bytes, int iters, unsigned int* err) {
  extern __shared__ __align__(128) uint8_t fsm[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(fsm + FILL_STAGES * FILL_MAX_STAGE);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + FILL_STAGES);
  if (threadIdx.x == 0) {
    for (int i = 0; i < FILL_STAGES; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const WaitCtx ctx{abort_flag, err};
    const size_t slots = span / (size_t)stage_bytes;            // the host guarantees slots >= 1
    size_t slot = ((size_t)blockIdx.x * 7919u) % slots;
    bool ok = true;
    for (int it = 0; it < iters + FILL_STAGES && ok; ++it) {
      const int s = it % FILL_STAGES;
      if (it >= FILL_STAGES) ok = mbar_wait(&bars[s], ((it / FILL_STAGES) - 1) & 1, ctx, 40);   // the stage's previous fill has landed
      if (ok && it < iters) {
        mbar_expect_tx(&bars[s], (uint32_t)stage_bytes);
        const uint8_t* g = src + slot * (size_t)stage_bytes;
        for (int off = 0; off < stage_bytes; off += 16384) {
          const int n = stage_bytes - off < 16384 ? stage_bytes - off : 16384;
          bulk_load_1d(fsm + (size_t)s * FILL_MAX_STAGE + off, g + off, (uint32_t)n, &bars[s]);
        }
        if (++slot == slots) slot = 0;
      }
    }
    if (!ok) {                                                    // a wait ran out: give copies in flight time to land
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------ reciprocal self-test
// Every significand of one binade: the three-instruction correctly rounded reciprocal of the quantisers (rcp_rn_pair)
// against __frcp_rn.  Significands that are all ones are outside its contract (callers route them to __fdiv_rn).
__global__ void rcp_selftest_kernel(int exponent, unsigned int* mismatches) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;           // 2^23 threads
  if (i >= (1u << 23) - 1u) return;
  const float d = __uint_as_float(((uint32_t)(exponent + 127) << 23) | i);
  const float2 r = rcp_rn_pair(make_float2(d, -d));
  const float ref = __frcp_rn(d);
  if (r.x != ref || r.y != -ref) atomicAdd(mismatches, 1u);
}

}  // namespace kf

using namespace kf;

extern "C" int kf_fill_rate_probe(const void* src, long long span, int stage_bytes, int iters, double* bytes_per_launch, void* stream) {
  KF_REQUIRE(src && (reinterpret_cast<uintptr_t>(src) & 15) == 0, "kf_fill_rate_probe: src must be non-null and 16-byte aligned");
  KF_REQUIRE(stage_bytes >= 1024 && stage_bytes <= FILL_MAX_STAGE && stage_bytes % 1024 == 0, "kf_fill_rate_probe: stage_bytes must be a multiple of 1024 up to 65536");
  KF_REQUIRE(span >= stage_bytes, "kf_fill_rate_probe: span must hold at least one stage");
  KF_REQUIRE(iters > 0 && iters <= (1 << 22), "kf_fill_rate_probe: iters out of range");
  int sms = 0;
  int st = device_sm_count(&sms);
  if (st != KF_OK) return st;
  unsigned int* err = dev_error_ptr();
  KF_REQUIRE(err != nullptr, "kf_fill_rate_probe: device error word unavailable");
  cudaError_t e = cudaFuncSetAttribute(fill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FILL_SMEM);
  if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(fill_kernel)");
  if (bytes_per_launch) *bytes_per_launch = (double)stage_bytes * iters * sms;
  fill_kernel<<<sms, 128, FILL_SMEM, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(src), (size_t)span, stage_bytes, iters, err);
  return cuda_status(cudaGetLastError(), "kf_fill_rate_probe launch");
}

extern "C" int kf_tensor_peak_probe(int fmt, int n, int iters, int sf_copies, double* flops_per_launch, void* stream) {
  KF_REQUIRE(fmt >= KF_FMT_MX8 && fmt <= KF_FMT_BF16, "kf_tensor_peak_probe: unknown format %d", fmt);
  KF_REQUIRE(n == 64 || n == 128 || n == 256, "kf_tensor_peak_probe: n must be 64, 128 or 256");
  KF_REQUIRE(iters > 0 && iters <= (1 << 22), "kf_tensor_peak_probe: iters out of range");
  KF_REQUIRE(sf_copies >= 0 && sf_copies <= 16, "kf_tensor_peak_probe: sf_copies must be 0..16");
  int sms = 0;
  int st = device_sm_count(&sms);
  if (st != KF_OK) return st;
  unsigned int* err = dev_error_ptr();
  KF_REQUIRE(err != nullptr, "kf_tensor_peak_probe: device error word unavailable");
  const double k_per_mma = fmt == KF_FMT_MX8 ? 32.0 : (fmt == KF_FMT_BF16 ? 16.0 : 64.0);
  if (flops_per_launch) *flops_per_launch = 2.0 * 128.0 * n * k_per_mma * 4.0 * iters * sms;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  switch (fmt) {
    case KF_FMT_MX8: return launch_peak<KF_FMT_MX8>(n, iters, sf_copies, sms, err, cs);
    case KF_FMT_NV4: return launch_peak<KF_FMT_NV4>(n, iters, sf_copies, sms, err, cs);
    case KF_FMT_MX4: return launch_peak<KF_FMT_MX4>(n, iters, sf_copies, sms, err, cs);
    default: return launch_peak<KF_FMT_BF16>(n, iters, sf_copies, sms, err, cs);
  }
}

extern "C" int kf_selftest_rcp(int exponent, unsigned int* mismatches, void* stream) {
  KF_REQUIRE(exponent >= -59 && exponent <= 59, "kf_selftest_rcp: exponent must be within -59..59 (the range the quantisers use the routine in)");
  KF_REQUIRE(mismatches != nullptr, "kf_selftest_rcp: null counter");
  rcp_selftest_kernel<<<(1 << 23) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(exponent, mismatches);
  return cuda_status(cudaGetLastError(), "kf_selftest_rcp launch");
}
