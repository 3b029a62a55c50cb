// Two-SM bf16 GEMM for sm_100a: a pair of CTAs (a 2-CTA cluster) computes one 256 x 256 output tile with
// `tcgen05.mma.cta_group::2`.
//
//   C[M,N] = epilogue( A[M,K] * B[N,K]^T )            fp32 accumulation in TMEM
//
// Why: with one CTA per tile a 128 x 256 tile has to pull 48 KiB of operands through the SM's L2 port for every
// 512 tensor-core cycles, more than the port delivers, and the tensor pipe idles a quarter of the time (ncu:
// 74 % active on the single-CTA kernel). In a CTA pair each CTA stages its own 128 rows of A and only HALF of
// the B tile (128 of its 256 rows); the pair's MMA reads both halves, so every CTA moves 32 KiB per 512 cycles
// for the same math. No TMA multicast is involved: each CTA loads its own halves.
//
//   * cluster (2,1,1); CTA rank 0 is the leader and issues every MMA, rank 1 contributes shared memory and TMEM
//   * warp 0 (both CTAs): TMA producer for the CTA's own A / B halves; the loads carry `.cta_group::2` so that
//     their transaction bytes complete on the LEADER's full barrier, which the leader's producer arms with the
//     bytes of both CTAs
//   * warp 1 (leader): one thread issues 4 MMAs (M 256, N 256, K 16) per stage, then commits the stage's empty
//     barrier in both CTAs (two plain commits, own and peer address) and, per tile, the accumulator-full barrier
//     in both CTAs
//   * warps 2..5 (both CTAs): epilogue for the CTA's 128 rows, TMEM double-buffered; "accumulator free" arrives
//     on the leader's barrier from all eight epilogue warps (remote mbarrier arrive for the peer)
//   * 6 stages x 32 KiB, TMEM 2 x 256 columns per CTA, every wait bounded, cluster barrier before teardown
//
// Operand layouts (K-major / MN-major) and epilogue flags are those of gemm.cu.
#include "common.cuh"
#include <cstdlib>

using namespace tb;

namespace {

constexpr int BM = 256, BN = 256, BK = 64, UMMA_K = 16;
constexpr int HM = 128, HN = 128;                  // rows of A and of B staged by one CTA
constexpr int STAGES = 6;
constexpr int A_BYTES = HM * BK * 2, B_BYTES = HN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int GROUP_M = 8;

enum { GF_A_MN = 1, GF_B_MN = 2, GF_OUT_F32 = 4, GF_ACCUM = 8, GF_BIAS = 16, GF_RESIDUAL = 32 };

struct Args2 {
  int M, N, K, flags;
  // second contraction segment accumulated into the same TMEM tile: C += A2[M, K2] * B2[N, K2]^T with the layouts of
  // A and B (a low-rank adapter update x A^T B^T carried by the base projection's GEMM); K2 = 0 when absent
  int K2;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  long long ldr;
  float alpha;
  int* status;
  // log-softmax epilogue (lm_head): instead of writing C, every tile leaves per row the online-softmax state of its
  // 256 columns and the target column's value, so logits never reach memory. partial: fp32 [M, num_n, 4] =
  // (max, sum exp(z - max), sum exp(z - max) z, z[target] or -inf when the target is in another tile).
  const int* targets;
  float* partial;
  float inv_temp, softcap;
  // logit-gradient epilogue (lm_head backward): the accumulator z is turned in registers into
  //   dz = dlogp (1[j == target] - p_j) - dent p_j (z_j - lse + entropy),  p_j = exp(z_j - lse),
  // chained through temperature and soft-cap, and written as bf16; the fp32 logits never reach memory.
  // dz_lse != nullptr selects it; dz_dlogp / dz_dent / dz_ent may be null.
  const float* dz_lse;
  const float* dz_dlogp;
  const float* dz_dent;
  const float* dz_ent;
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
__device__ __forceinline__ void umma2_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on a barrier (own or peer, cluster address) when the MMAs issued so far by this thread have retired
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory whose bytes complete on a barrier given by cluster address
__device__ __forceinline__ void tma2_load_2d(uint32_t smem_dst, const CUtensorMap* tm, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__global__ void __launch_bounds__(192, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, const Args2 args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // used in the leader only
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };           // one per CTA
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };       // one per CTA
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };  // used in the leader only
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_al + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int M = args.M, N = args.N, K = args.K;
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
  const int num_kb1 = (K + BK - 1) / BK;                         // k-blocks of the main operands ...
  const int num_kb = num_kb1 + (args.K2 + BK - 1) / BK;          // ... followed by those of the second segment
  const int num_tiles = num_m * num_n;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const bool a_mn = args.flags & GF_A_MN, b_mn = args.flags & GF_B_MN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 8);       // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    if (args.K2 > 0) {
      prefetch_tensormap(&tmA2);
      prefetch_tensormap(&tmB2);
    }
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32((const void*)tmem_ptr_smem), 2 * BN);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();                    // barriers of both CTAs exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  auto tile_coords = [&](int t, int& mt, int& nt) {
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, num_m - first_m);
    const int r = t - g * per_group;
    mt = first_m + (r % gsz);
    nt = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (own halves of A and B)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int mt, nt;
        tile_coords(t, mt, nt);
        const int m0 = mt * BM + (int)rank * HM, n0 = nt * BN + (int)rank * HN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t fb = mapa_u32(full_bar(stage), 0);           // the leader's barrier for this stage
          if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          // the second segment's maps zero-fill past K2, so a rank below 64 costs one padded k-block
          const bool seg2 = kb >= num_kb1;
          const CUtensorMap* ta = seg2 ? &tmA2 : &tmA;
          const CUtensorMap* tb_ = seg2 ? &tmB2 : &tmB;
          const int k0 = (seg2 ? kb - num_kb1 : kb) * BK;
          if (!a_mn) {
            tma2_load_2d(sa, ta, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < HM / 64; ++j) tma2_load_2d(sa + j * 8192, ta, fb, m0 + 64 * j, k0);
          }
          if (!b_mn) {
            tma2_load_2d(sb, tb_, fb, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < HN / 64; ++j) tma2_load_2d(sb + j * 8192, tb_, fb, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, a_mn ? 1 : 0, b_mn ? 1 : 0);
      const uint32_t a_lbo = a_mn ? 8192u : 16u, b_lbo = b_mn ? 8192u : 16u;
      const uint32_t a_kstep = a_mn ? 2048u : 32u, b_kstep = b_mn ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1, abort_flag, args.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc(sb + k * b_kstep, b_lbo, 1024);
            umma2_f16_ss(tmem_d, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma2_commit(empty_bar(stage));                              // frees the stage here ...
          umma2_commit(mapa_u32(empty_bar(stage), 1));                 // ... and in the peer
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit(tfull_bar(acc));
        umma2_commit(mapa_u32(tfull_bar(acc), 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (own 128 rows)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = args.flags & GF_OUT_F32, accum = args.flags & GF_ACCUM;
    const bool has_bias = args.flags & GF_BIAS, has_res = args.flags & GF_RESIDUAL;
    const float alpha = args.alpha;
    const bool c_al16 = (reinterpret_cast<uintptr_t>(args.C) & 15) == 0;
    const bool r_al16 = (reinterpret_cast<uintptr_t>(args.resid) & 15) == 0;
    const uint32_t tempty_leader0 = mapa_u32(tempty_bar(0), 0), tempty_leader1 = mapa_u32(tempty_bar(1), 0);
    const bool lse_mode = args.partial != nullptr;
    const bool dz_mode = args.dz_lse != nullptr;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int mt, nt;
      tile_coords(t, mt, nt);
      const int row = mt * BM + (int)rank * HM + q * 32 + lane;
      const int n0 = nt * BN;
      float dz_l = 0.f, dz_gl = 0.f, dz_ge = 0.f, dz_en = 0.f;
      int dz_t = -1;
      if (dz_mode && row < M) {
        dz_l = args.dz_lse[row];
        dz_ge = args.dz_dent ? args.dz_dent[row] : 0.f;
        dz_en = (args.dz_dent && args.dz_ent) ? args.dz_ent[row] : 0.f;
        dz_t = args.targets ? args.targets[row] : -1;
        if (dz_t < 0 || dz_t >= N) dz_t = -1;
        dz_gl = (dz_t >= 0 && args.dz_dlogp) ? args.dz_dlogp[row] : 0.f;
      }
      if (!mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, args.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      if (lse_mode) {
        // one thread owns one row of the tile: the softmax statistics of its 256 columns need no communication
        float mx = -INFINITY, sm = 0.f, sz = 0.f, zt = -INFINITY;
        const int tgt = row < M ? args.targets[row] : -1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          float cm = -INFINITY;
          float z[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(r[i]) * alpha;
            if (args.softcap > 0.f) v = args.softcap * tanhf(v / args.softcap);
            v *= args.inv_temp;
            z[i] = (col0 + i < N) ? v : -INFINITY;
            cm = fmaxf(cm, z[i]);
          }
          if (tgt >= col0 && tgt < col0 + 32) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i == tgt) zt = z[i];
          }
          const float nm = fmaxf(mx, cm);
          const float corr = (mx == -INFINITY) ? 0.f : __expf(mx - nm);
          float s2 = 0.f, z2 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float e = (z[i] == -INFINITY) ? 0.f : __expf(z[i] - nm);
            s2 += e;
            z2 += e * (z[i] == -INFINITY ? 0.f : z[i]);
          }
          sm = sm * corr + s2;
          sz = sz * corr + z2;
          mx = nm;
        }
        if (row < M)
          *reinterpret_cast<float4*>(args.partial + ((long long)row * num_n + nt) * 4) = make_float4(mx, sm, sz, zt);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc == 0 ? tempty_leader0 : tempty_leader1);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row < M) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
          const bool full = (col0 + 32 <= N);
          if (dz_mode) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float capped = v[i], chain = args.inv_temp;
              if (args.softcap > 0.f) {
                const float th = tanhf(v[i] / args.softcap);
                capped = args.softcap * th;
                chain *= (1.f - th * th);
              }
              const float z = capped * args.inv_temp;
              const float p = __expf(z - dz_l);
              float d = dz_gl * ((col0 + i == dz_t ? 1.f : 0.f) - p);
              if (dz_ge != 0.f) d -= dz_ge * p * (z - dz_l + dz_en);
              v[i] = d * chain;
            }
          }
          if (has_bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (full || col0 + i < N) v[i] += __bfloat162float(args.bias[col0 + i]);
          }
          if (has_res) {
            const __nv_bfloat16* rp = args.resid + (long long)row * args.ldr + col0;
            if (full && (args.ldr % 8 == 0) && r_al16) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const uint4 u = reinterpret_cast<const uint4*>(rp)[g];
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[g * 8 + 2 * j] += bf16_lo(w[j]);
                  v[g * 8 + 2 * j + 1] += bf16_hi(w[j]);
                }
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) v[i] += __bfloat162float(rp[i]);
            }
          }
          if (out_f32) {
            float* cp = reinterpret_cast<float*>(args.C) + (long long)row * args.ldc + col0;
            if (full && (args.ldc % 4 == 0) && c_al16) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                float4 o = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                if (accum) {
                  const float4 p = reinterpret_cast<float4*>(cp)[g];
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                reinterpret_cast<float4*>(cp)[g] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) cp[i] = accum ? cp[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc + col0;
            if (full && (args.ldc % 8 == 0) && c_al16) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (accum) {
                  const uint4 u = reinterpret_cast<uint4*>(cp)[g];
                  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    v[g * 8 + 2 * j] += bf16_lo(w[j]);
                    v[g * 8 + 2 * j + 1] += bf16_hi(w[j]);
                  }
                }
                uint4 o;
                o.x = pack_bf16(v[g * 8 + 0], v[g * 8 + 1]);
                o.y = pack_bf16(v[g * 8 + 2], v[g * 8 + 3]);
                o.z = pack_bf16(v[g * 8 + 4], v[g * 8 + 5]);
                o.w = pack_bf16(v[g * 8 + 6], v[g * 8 + 7]);
                reinterpret_cast<uint4*>(cp)[g] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) cp[i] = __float2bfloat16(v[i] + (accum ? __bfloat162float(cp[i]) : 0.f));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? tempty_leader0 : tempty_leader1);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let TMA copies that may still be in flight land
  }
  cluster_sync_all();                    // the peer may still read this CTA's shared memory / write its TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 2 * BN);
  }
}

int g_sms2 = 0;
struct LseArgs {           // log-softmax epilogue request; partial == nullptr for a plain GEMM
  const int* targets = nullptr;
  float* partial = nullptr;
  float inv_temp = 1.f, softcap = 0.f;
  const float* dz_lse = nullptr;       // logit-gradient epilogue when set
  const float* dz_dlogp = nullptr;
  const float* dz_dent = nullptr;
  const float* dz_ent = nullptr;
};
struct Seg2 {              // second contraction segment; K2 == 0 when absent
  const void* A2 = nullptr;
  const void* B2 = nullptr;
  int K2 = 0;
  long long lda2 = 0, ldb2 = 0;
};

// partial [M, num_n, 4] -> logp[row] = z[target] - lse (0 for targets outside [0, V)), lse, entropy = lse - E[z]
__global__ void lse_combine_kernel(const float* __restrict__ partial, const int* __restrict__ targets, int M, int num_n,
                                   int V, float* __restrict__ logp, float* __restrict__ lse_out, float* __restrict__ ent_out) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY, sm = 0.f, sz = 0.f, zt = -INFINITY;
  for (int j = lane; j < num_n; j += 32) {
    const float4 p = *reinterpret_cast<const float4*>(partial + ((long long)row * num_n + j) * 4);
    const float nm = fmaxf(mx, p.x);
    const float a = (mx == -INFINITY) ? 0.f : __expf(mx - nm), b = (p.x == -INFINITY) ? 0.f : __expf(p.x - nm);
    sm = sm * a + p.y * b;
    sz = sz * a + p.z * b;
    mx = nm;
    zt = fmaxf(zt, p.w);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, o), os = __shfl_xor_sync(0xffffffffu, sm, o);
    const float oz = __shfl_xor_sync(0xffffffffu, sz, o), ot = __shfl_xor_sync(0xffffffffu, zt, o);
    const float nm = fmaxf(mx, om);
    const float a = (mx == -INFINITY) ? 0.f : __expf(mx - nm), b = (om == -INFINITY) ? 0.f : __expf(om - nm);
    sm = sm * a + os * b;
    sz = sz * a + oz * b;
    mx = nm;
    zt = fmaxf(zt, ot);
  }
  if (lane == 0) {
    const float lse = mx + logf(sm);
    const int t = targets[row];
    if (logp) logp[row] = (t >= 0 && t < V) ? zt - lse : 0.f;
    if (lse_out) lse_out[row] = lse;
    if (ent_out) ent_out[row] = lse - sz / sm;
  }
}

}  // namespace

namespace {
int launch_2cta(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                int flags, const void* bias, const void* resid, long long ldr, float alpha, int* status,
                cudaStream_t stream, const LseArgs& lse, const Seg2& seg = Seg2{}) {
  static const bool off = getenv("TUNIX_B200_NO_2CTA") != nullptr;
  if (off) return 0;
  static DeviceOnce once;
  if (once.first()) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms2, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -5;
  }
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
  const int pairs = g_sms2 / 2;
  // worth it when the pairs have at least a wave of 256 x 256 tiles and the K loop amortises the prologue
  if (N < 256 || M < 256 || K < 256 || (long long)num_m * num_n < (pairs * 3) / 5) return 0;
  const bool a_mn = flags & GF_A_MN, b_mn = flags & GF_B_MN;
  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn) r = tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, HM, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmA, A, K, M, lda, BK, 64, 1);
  if (r) return -3;
  if (!b_mn) r = tb_make_tmap_2d_bf16(&tmB, B, N, K, ldb, HN, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, 64, 1);
  if (r) return -4;
  CUtensorMap tmA2 = tmA, tmB2 = tmB;
  if (seg.K2 > 0) {
    if ((seg.lda2 % 8) || (seg.ldb2 % 8) || (reinterpret_cast<uintptr_t>(seg.A2) & 15) ||
        (reinterpret_cast<uintptr_t>(seg.B2) & 15))
      return -2;
    if (!a_mn) r = tb_make_tmap_2d_bf16(&tmA2, seg.A2, M, seg.K2, seg.lda2, HM, BK, 1);
    else       r = tb_make_tmap_2d_bf16(&tmA2, seg.A2, seg.K2, M, seg.lda2, BK, 64, 1);
    if (r) return -3;
    if (!b_mn) r = tb_make_tmap_2d_bf16(&tmB2, seg.B2, N, seg.K2, seg.ldb2, HN, BK, 1);
    else       r = tb_make_tmap_2d_bf16(&tmB2, seg.B2, seg.K2, N, seg.ldb2, BK, 64, 1);
    if (r) return -4;
  }
  Args2 a;
  a.K2 = seg.K2;
  a.M = M; a.N = N; a.K = K; a.flags = flags; a.C = C; a.ldc = ldc;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  a.ldr = ldr; a.alpha = alpha; a.status = status;
  a.targets = lse.targets; a.partial = lse.partial; a.inv_temp = lse.inv_temp; a.softcap = lse.softcap;
  a.dz_lse = lse.dz_lse; a.dz_dlogp = lse.dz_dlogp; a.dz_dent = lse.dz_dent; a.dz_ent = lse.dz_ent;
  const int tiles = num_m * num_n;
  const int use_pairs = tiles < pairs ? tiles : pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * use_pairs, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm2_kernel, tmA, tmB, tmA2, tmB2, a) != cudaSuccess) return -5;
  return 1;
}
}  // namespace

// Returns 1 when the problem was launched here, 0 when it is left to the single-CTA kernel, negative on error.
int tb_gemm_2cta_try(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                     int* status, cudaStream_t stream) {
  return launch_2cta(A, B, C, M, N, K, lda, ldb, ldc, flags, bias, resid, ldr, alpha, status, stream, LseArgs{});
}

// C = epilogue(A * B^T + A2 * B2^T): the base projection with a low-rank update accumulated into the same TMEM tile
// (A2 [M, K2] or [K2, M], B2 [N, K2] or [K2, N], laid out like A and B; K2 is the adapter rank, any multiple of 8).
// Returns 1 when launched, 0 when the problem is too small for the two-SM kernel (the caller then runs the two
// products separately), negative on error.
TB_API int tb_gemm_bf16_ext(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                            const void* A2, const void* B2, int K2, long long lda2, long long ldb2, int* status,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K2 <= 0 || (K2 % 8) || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  Seg2 seg;
  seg.A2 = A2; seg.B2 = B2; seg.K2 = K2; seg.lda2 = lda2; seg.ldb2 = ldb2;
  return launch_2cta(A, B, C, M, N, K, lda, ldb, ldc, flags, bias, resid, ldr, alpha, status, stream, LseArgs{}, seg);
}

// log p(target) (and optionally lse / entropy) of z = softcap(h W^T) / temperature without materialising z:
// the two-SM GEMM's epilogue leaves per-tile softmax statistics, a small kernel merges them.
// h [M, K] bf16 (row stride ldh), w [V, K] bf16 (row stride ldw), targets int32 [M] (negative = ignored),
// partial: fp32 scratch of M * ceil(V / 256) * 4 elements. Returns 1 when run here, 0 when the problem does not
// qualify for the two-SM kernel (the caller uses its chunked path), negative on error.
TB_API int tb_lm_head_lse(const void* h, long long ldh, const void* w, long long ldw, int M, int V, int K,
                          const int* targets, float inv_temp, float softcap, float* partial, float* logp, float* lse,
                          float* entropy, int* status, cudaStream_t stream) {
  LseArgs lse_args;
  lse_args.targets = targets; lse_args.partial = partial; lse_args.inv_temp = inv_temp; lse_args.softcap = softcap;
  const int rc = launch_2cta(h, w, nullptr, M, V, K, ldh, ldw, 0, 0, nullptr, nullptr, 0, 1.0f, status, stream, lse_args);
  if (rc != 1) return rc;
  const int num_n = (V + BN - 1) / BN;
  lse_combine_kernel<<<(M + 7) / 8, 256, 0, stream>>>(partial, targets, M, num_n, V, logp, lse, entropy);
  return cudaGetLastError() == cudaSuccess ? 1 : -5;
}

// dz [M, V] (bf16, row stride ldo) = gradient of sum_rows(dlogp * logp + dent * entropy) with respect to the raw
// logits h W^T, computed in the epilogue of the two-SM GEMM that recomputes those logits: lse (and entropy, when dent
// is given) are the row statistics saved by the forward pass. dlogp / dent / entropy may be null. Returns 1 when run
// here, 0 when the problem does not qualify for the two-SM kernel, negative on error.
TB_API int tb_lm_head_dlogits(const void* h, long long ldh, const void* w, long long ldw, int M, int V, int K,
                              const int* targets, const float* lse, const float* entropy, const float* dlogp,
                              const float* dent, float inv_temp, float softcap, void* out, long long ldo, int* status,
                              cudaStream_t stream) {
  if (!lse || !out) return -2;
  LseArgs e;
  e.targets = targets; e.inv_temp = inv_temp; e.softcap = softcap;
  e.dz_lse = lse; e.dz_dlogp = dlogp; e.dz_dent = dent; e.dz_ent = entropy;
  return launch_2cta(h, w, out, M, V, K, ldh, ldw, ldo, 0, nullptr, nullptr, 0, 1.0f, status, stream, e);
}
