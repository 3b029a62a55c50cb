// Split-K bf16 GEMM for skinny problems (decode: M = running sequences, a few hundred rows at most).
//
//   C[M,N] = epilogue( A[M,K] * B[N,K]^T ),  A and B K-major
//
// With few output tiles the persistent kernel in gemm.cu either leaves most SMs idle (wide tiles) or, with
// narrow tiles, makes every CTA re-read the whole A panel, and the L2 -> SM traffic of those re-reads, not
// HBM, bounds the kernel. Here the tile stays 128 x 256 (A is re-read once per 256 weight rows) and the K
// range is split over the S CTAs of a thread-block cluster instead:
//
//   * grid (n tiles, m tiles, S), cluster (1, 1, S); CTA z owns k blocks [z*KB/S, (z+1)*KB/S)
//   * per CTA the gemm.cu pipeline: TMA producer warp -> smem ring -> one-thread tcgen05.mma -> TMEM
//   * the four epilogue warps spill the fp32 partial tile from TMEM into the (now idle) ring memory
//   * cluster barrier; CTA z sums column slice z of all S partial tiles through distributed shared memory
//     (mapa + ld.shared::cluster), applies alpha / bias / residual / accumulate and writes C
//   * cluster barrier (nobody leaves while a peer still reads its shared memory); TMEM freed
//
// Every mbarrier wait is bounded; a timeout sets *status and falls through to the cluster barriers, which
// every thread of every CTA reaches on every path.
#include "common.cuh"

using namespace tb;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int PART_BYTES = BM * BN * 4;   // 128 KiB, overlays the ring
static_assert(PART_BYTES <= STAGES * STAGE_BYTES, "partial tile must fit in the ring");

enum { GF_OUT_F32 = 4, GF_ACCUM = 8, GF_BIAS = 16, GF_RESIDUAL = 32 };

struct SkArgs {
  int M, N, K, flags, S;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  long long ldr;
  float alpha;
  int* status;
  const uint8_t* b_packed;   // B pre-tiled in 256-row blocks by tb_pack_weight (null: B through tmB)
};

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// partial tile: 16-byte chunk c4 (of 64) of row r, chunks XOR-swizzled by row so that row-wise writers
// (one thread per row) and chunk-wise readers both spread over the banks
__device__ __forceinline__ uint32_t part_off(int r, int c4) { return (uint32_t)((r * 64 + (c4 ^ (r & 63))) << 4); }

__global__ void __launch_bounds__(192, 1)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const SkArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_al + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = args.M, N = args.N, S = args.S;
  const int z = blockIdx.z;                       // rank in the cluster (cluster = (1,1,S))
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
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
    tmem_alloc(smem_u32((const void*)tmem_ptr_smem), BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_PRODUCER)) break;
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        mbar_expect_tx(full_bar(stage), STAGE_BYTES);
        tma_load_2d(sa, &tmA, full_bar(stage), kb * BK, m0);
        if (args.b_packed != nullptr)
          bulk_load(sa + A_BYTES, args.b_packed + ((size_t)blockIdx.x * num_kb + kb) * (size_t)B_BYTES, B_BYTES, full_bar(stage));
        else
          tma_load_2d(sa + A_BYTES, &tmB, full_bar(stage), kb * BK, n0);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
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
          umma_f16_ss(tmem_base, ad, bd, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(tfull_bar);
    }
    __syncwarp();
  } else {
    // spill this CTA's partial tile (rows that exist) into the ring memory
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
    // CTA z reduces chunks [c_begin, c_end) of every existing row over the S partial tiles
    const int rows = min(BM, M - m0);
    const int chunks_total = (min(BN, N - n0) + 3) / 4;
    const int c_begin = (int)((long long)z * chunks_total / S), c_end = (int)((long long)(z + 1) * chunks_total / S);
    const int nch = c_end - c_begin;
    const bool out_f32 = args.flags & GF_OUT_F32, accum = args.flags & GF_ACCUM;
    const bool has_bias = args.flags & GF_BIAS, has_res = args.flags & GF_RESIDUAL;
    for (int it = threadIdx.x; it < rows * nch; it += blockDim.x) {
      const int r = it / nch, c4 = c_begin + (it - r * nch);
      const uint32_t local = smem_base + part_off(r, c4);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < S; ++p) {
        const float4 v = ld_dsmem_f4(map_to_cta(local, (uint32_t)p));
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

  cluster_sync_all();

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let TMA copies that may still be in flight land
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

int g_sk_sms = 0;

}  // namespace

// Returns 1 when the problem was launched here, 0 when it is not a split-K case (the caller runs the persistent
// kernel), a negative code on error. A and B K-major, same conventions as tb_gemm_bf16.
int tb_gemm_splitk_try(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                       int* status, cudaStream_t stream, const void* b_packed) {
  if (flags & 3) return 0;                              // MN-major operands stay on the persistent kernel
  // Measured on B200 against the persistent kernel's narrow tiles: the split pays once the K loop is long
  // (down projections, K >= 8192: 40 -> 28 us at 64 x 4096 x 12288); at K = 4096 it wins up to 64 rows
  // (64 x 4096 x 4096: 23.6 -> 20.5 us, 16 rows: 23.6 -> 18.5 us) and loses from 128 rows on.
  if (M > 512 || N < 256 || K < (M <= 64 ? 4096 : 8192)) return 0;
  static DeviceOnce once;
  if (once.first()) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sk_sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -5;
  }
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN, num_kb = (K + BK - 1) / BK;
  const int tiles = num_m * num_n;
  if (tiles * 2 > g_sk_sms) return 0;
  // smallest split whose wave efficiency is within 8% of the best one (each extra split re-reads A and adds
  // a partial tile to the reduction)
  double eff[9], best = 0.0;
  static int max_clusters[9] = {0};                     // co-resident clusters per size, asked of the runtime once
  for (int s = 1; s <= 8; ++s) {
    eff[s] = 0.0;
    if (num_kb / s < 4) continue;
    if (max_clusters[s] == 0) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(1, 1, s);
      q.blockDim = dim3(192, 1, 1);
      q.dynamicSmemBytes = SMEM_BYTES;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 1;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = s;
      q.attrs = qa;
      q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_splitk_kernel, &q) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = -1;
      }
      max_clusters[s] = n;
    }
    if (max_clusters[s] < 0) continue;
    const long long waves = (tiles + max_clusters[s] - 1) / max_clusters[s];
    eff[s] = (double)tiles * s / (double)(waves * g_sk_sms);
    if (eff[s] > best) best = eff[s];
  }
  if (best == 0.0) return 0;
  int S = 1;
  for (int s = 1; s <= 8; ++s)
    if (eff[s] >= 0.92 * best) { S = s; break; }
  if (S == 1 && tiles >= g_sk_sms) return 0;            // enough tiles for the persistent kernel
  CUtensorMap tmA, tmB;
  if (tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, BM, BK, 1)) return -3;
  if (b_packed != nullptr) tmB = tmA;                  // unused by the kernel
  else if (tb_make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN, BK, 1)) return -4;
  SkArgs a;
  a.b_packed = reinterpret_cast<const uint8_t*>(b_packed);
  a.M = M; a.N = N; a.K = K; a.flags = flags; a.S = S; a.C = C; a.ldc = ldc;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  a.ldr = ldr; a.alpha = alpha; a.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_n, num_m, S);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = S;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_splitk_kernel, tmA, tmB, a) != cudaSuccess) return -5;
  return 1;
}
