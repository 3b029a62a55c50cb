// bf16 GEMM for a few hundred rows (decode with 128 < M <= 512 running sequences): 256 x 256 output tiles on CTA
// pairs (`tcgen05.mma.cta_group::2`) with the K range split over the pairs of one thread-block cluster.
//
//   C[M,N] = epilogue( A[M,K] * B[N,K]^T ),  A and B K-major
//
// Why. At these sizes the weight matrix B is read once, but the activation panel A is re-read by every n tile, and
// the traffic between L2 and the SMs, not HBM, bounds the kernel: with 128 x 64 tiles a 256 x 4096 x 4096 problem
// moves 196 MB through the SMs for 33.5 MB of weights. A CTA pair computes a 256 x 256 tile while each CTA stages only
// 128 rows of A and 128 rows of B per k block (32 KiB for 256 x 256 x 64 multiply-adds); the K split supplies the
// parallelism that the few tiles lack (16 n tiles x 4 splits = 64 pairs for that problem, 65 MB through the SMs).
//
//   * grid (2 * n tiles, m tiles, S), cluster (2, 1, S): cluster rank = p + 2 z with p the pair member, z the split
//   * per pair the gemm_2cta.cu protocol (own A / B halves by TMA with `.cta_group::2` completion on the leader's
//     barrier, MMAs by one thread of the leader, commits to both CTAs); no TMA multicast
//   * epilogue warps spill the CTA's 128 x 256 fp32 partial from TMEM into the idle ring, cluster barrier, then CTA
//     (p, z) sums column slice z of the S partials of member p through distributed shared memory and writes C
//   * every mbarrier wait bounded; a timeout sets *status and falls through to the cluster barriers
//
// Measured on B200 against the kernels it was meant to replace (CUDA events, L2 flushed): 256 x 4096 x 4096 38.9 us
// against 23.6 us (128 x 64 tiles of the persistent kernel), 256 x 6144 x 4096 49.2 against 29.7, 256 x 4096 x 12288
// 63.5 against 47.1 (128 x 256 tiles with cluster split-K), 512 x 4096 x 4096 32.8 against 26.6; rollout at 256
// sequences 18.9 k against 23.8 k tokens/s. Halving the L2 -> SM traffic does not pay for a pair that runs only 16
// k blocks and then spills, synchronises the cluster and reduces 128 KiB per CTA. The kernel is numerically checked
// (tests/test_pair_splitk_gpu.py) and stays opt-in (TUNIX_B200_PAIR_SPLITK=1); nothing selects it by default.
#include "common.cuh"
#include <cstdlib>

using namespace tb;

namespace {

constexpr int BM = 256, BN = 256, BK = 64, UMMA_K = 16;
constexpr int HM = 128, HN = 128;
constexpr int STAGES = 6;
constexpr int A_BYTES = HM * BK * 2, B_BYTES = HN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int PART_BYTES = HM * BN * 4;            // 128 KiB, overlays the ring
static_assert(PART_BYTES <= STAGES * STAGE_BYTES, "partial tile must fit in the ring");

enum { GF_OUT_F32 = 4, GF_ACCUM = 8, GF_BIAS = 16, GF_RESIDUAL = 32 };

struct PsArgs {
  int M, N, K, flags, S;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  long long ldr;
  float alpha;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(uint32_t smem_dst, const CUtensorMap* tm, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// partial tile: 16-byte chunk c4 (of 64) of row r, XOR-swizzled by row (row-wise writers, chunk-wise readers)
__device__ __forceinline__ uint32_t part_off(int r, int c4) { return (uint32_t)((r * 64 + (c4 ^ (r & 63))) << 4); }

__global__ void __launch_bounds__(192, 1)
gemm_pair_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PsArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                  // used in the pair's leader only
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };      // one per CTA
  const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);                   // one per CTA
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_al + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = args.M, N = args.N, S = args.S;
  const uint32_t rank = cluster_ctarank();            // p + 2 z
  const uint32_t p = rank & 1u, z = rank >> 1;
  const uint32_t leader_rank = rank & ~1u;
  const bool leader = p == 0;
  const int m0 = blockIdx.y * BM + (int)p * HM, n0 = (blockIdx.x >> 1) * BN;
  const int num_kb = (args.K + BK - 1) / BK;
  const int kb_begin = (int)((long long)z * num_kb / S), kb_end = (int)((long long)(z + 1) * num_kb / S);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32((const void*)tmem_ptr_smem), BN);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();                    // every CTA's barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (own halves of A and B)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_PRODUCER)) break;
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint32_t fb = mapa_u32(full_bar(stage), leader_rank);
        if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
        tma2_load_2d(sa, &tmA, fb, kb * BK, m0);
        tma2_load_2d(sa + A_BYTES, &tmB, fb, kb * BK, n0 + (int)p * HN);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (pair leader only)
    if (leader && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint32_t sb = sa + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t ad = make_smem_desc(sa + k * 32u, 16u, 1024);
          const uint64_t bd = make_smem_desc(sb + k * 32u, 16u, 1024);
          umma2_f16_ss(tmem_base, ad, bd, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
        }
        umma2_commit(empty_bar(stage));                               // frees the stage here ...
        umma2_commit(mapa_u32(empty_bar(stage), rank | 1u));          // ... and in the peer
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok && kb_end > kb_begin) {
        umma2_commit(tfull_bar);
        umma2_commit(mapa_u32(tfull_bar, rank | 1u));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------- spill this CTA's 128 x 256 partial into the ring
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const bool have = kb_end > kb_begin;
    bool ok = true;
    if (have) ok = mbar_wait_bounded(tfull_bar, 0, abort_flag, args.status, ST_TIMEOUT_EPILOGUE);
    tc_fence_after();
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      if (n0 + c * 32 >= N) break;
      uint32_t v[32];
      if (have && ok) {
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (m0 + r < M) {
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<uint4*>(smem_al + part_off(r, c * 8 + g)) = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
      }
    }
    tc_fence_before();
  }

  cluster_sync_all();

  {
    // CTA (p, z) reduces chunks [c_begin, c_end) of the rows of member p over the S partial tiles
    const int rows = max(0, min(HM, M - m0));
    const int chunks_total = (min(BN, N - n0) + 3) / 4;
    const int c_begin = (int)((long long)z * chunks_total / S), c_end = (int)((long long)(z + 1) * chunks_total / S);
    const int nch = c_end - c_begin;
    const bool out_f32 = args.flags & GF_OUT_F32, accum = args.flags & GF_ACCUM;
    const bool has_bias = args.flags & GF_BIAS, has_res = args.flags & GF_RESIDUAL;
    for (int it = threadIdx.x; it < rows * nch; it += blockDim.x) {
      const int r = it / nch, c4 = c_begin + (it - r * nch);
      const uint32_t local = smem_base + part_off(r, c4);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < S; ++s) {
        const float4 v = ld_dsmem_f4(mapa_u32(local, p + 2u * (uint32_t)s));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      float o[4] = {acc.x * args.alpha, acc.y * args.alpha, acc.z * args.alpha, acc.w * args.alpha};
      const int row = m0 + r, col = n0 + c4 * 4;
      const int nv = min(4, N - col);
      if (has_bias)
        for (int i = 0; i < nv; ++i) o[i] += __bfloat162float(args.bias[col + i]);
      if (has_res) {
        const __nv_bfloat16* rp = args.resid + (long long)row * args.ldr + col;
        for (int i = 0; i < nv; ++i) o[i] += __bfloat162float(rp[i]);
      }
      if (out_f32) {
        float* cp = reinterpret_cast<float*>(args.C) + (long long)row * args.ldc + col;
        if (accum)
          for (int i = 0; i < nv; ++i) o[i] += cp[i];
        if (nv == 4 && (reinterpret_cast<uintptr_t>(cp) & 15) == 0) *reinterpret_cast<float4*>(cp) = make_float4(o[0], o[1], o[2], o[3]);
        else
          for (int i = 0; i < nv; ++i) cp[i] = o[i];
      } else {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc + col;
        if (accum)
          for (int i = 0; i < nv; ++i) o[i] += __bfloat162float(cp[i]);
        if (nv == 4 && (reinterpret_cast<uintptr_t>(cp) & 7) == 0) *reinterpret_cast<uint2*>(cp) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
        else
          for (int i = 0; i < nv; ++i) cp[i] = __float2bfloat16(o[i]);
      }
    }
  }

  cluster_sync_all();                    // nobody leaves while a peer still reads its shared memory

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let TMA copies that may still be in flight land
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, BN);
  }
}

int g_ps_sms = 0;

}  // namespace

// Returns 1 when the problem was launched here, 0 when it is left to the other kernels, negative on error.
// A and B K-major, conventions of tb_gemm_bf16. Taken: 128 < M <= 512 rows, N >= 256, at least 16 k blocks, and so
// few 256 x 256 tiles that the pairs of the device are not filled without splitting K.
int tb_gemm_pair_splitk_try(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                            int* status, cudaStream_t stream) {
  static const bool off = getenv("TUNIX_B200_PAIR_SPLITK") == nullptr;     // opt-in until measured
  if (off || (flags & 3)) return 0;                      // MN-major operands stay on the other kernels
  if (M <= 128 || M > 512 || N < 256 || K < 16 * BK) return 0;
  static DeviceOnce once;
  if (once.first()) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_ps_sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm_pair_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -5;
  }
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN, num_kb = (K + BK - 1) / BK;
  const int tiles = num_m * num_n, pairs = g_ps_sms / 2;
  if (tiles > pairs) return 0;                           // enough tiles for the persistent two-SM kernel
  int S = 1;
  for (int s = 2; s <= 4; ++s)
    if (tiles * s <= pairs && num_kb / s >= 8) S = s;
  if (S == 1 && tiles * 2 > pairs) return 0;
  CUtensorMap tmA, tmB;
  if (tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, HM, BK, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tmB, B, N, K, ldb, HN, BK, 1)) return -4;
  PsArgs a;
  a.M = M; a.N = N; a.K = K; a.flags = flags; a.S = S; a.C = C; a.ldc = ldc;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  a.ldr = ldr; a.alpha = alpha; a.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * num_n, num_m, S);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = S;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_pair_splitk_kernel, tmA, tmB, a) != cudaSuccess) {
    cudaGetLastError();
    return 0;                                            // cluster shape not schedulable here: other kernels take it
  }
  return 1;
}
