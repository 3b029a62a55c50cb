// Flash-attention forward for sm_100a on tcgen05 tensor cores.
//
//   O = softmax(mask(softcap(scale * Q K^T))) V      per (batch, query head), GQA aware
//
// One CTA handles 128 query rows of one head. Five warps:
//   warps 0..3 : one thread per query row. S is read from TMEM (tcgen05.ld), masked and
//                exponentiated in registers (row max / row sum are thread-local: no shuffles),
//                P is written to shared memory in the 128-byte-swizzled K-major layout,
//                O stays in TMEM and is rescaled there only when a row max grows by > 2^8.
//   warp 4     : one elected thread issues every TMA load (no multicast) and every
//                tcgen05.mma: S_{j+1} = Q K_{j+1}^T is in flight while the softmax of block j runs.
// Masks: causal (with offset for Tq != Tk), sliding window, segment ids (packing / padding),
// key length. Logit soft-cap (Gemma-2). Head dim 64 / 128 / 256.
// Every mbarrier wait is bounded; a timeout sets *status and the CTA unwinds.
//
// Replaces the eager [B,N,T,S] attention and the TPU-only splash attention of the reference
// (tunix/models/llama3/model.py:379-396, tunix/models/qwen3/model.py:607-793,
//  tunix/models/gemma/model.py:442-483).
#include "common.cuh"
#include <cstdlib>

using namespace tb;

namespace {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 64;   // keys per iteration
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

struct AttnArgs {
  int B, Tq, Tk, N, KH;      // query heads N, kv heads KH
  float scale, softcap;
  int causal, window;        // window <= 0: unlimited
  int q_off;                 // kv position of query row i is i + q_off
  const int* seg_q;          // [B, Tq] or null
  const int* seg_k;          // [B, Tk] or null
  __nv_bfloat16* O;          // [B*Tq, N*H]
  long long ldo;
  float* lse;                // [B, N, Tq]
  int* status;
};

template <int H>
struct FwdCfg {
  static constexpr int HS = H / 64;                 // 64-column slabs along the head dim
  static constexpr int Q_BYTES = HS * BQ * 128;     // K-major slabs [128 x 128B]
  static constexpr int KV_BYTES = HS * BKV * 128;   // slabs [64 x 128B]
  static constexpr int P_BYTES = BQ * 128;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_BYTES;    // two V buffers
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024;
  static constexpr int TMEM_S = 0;                  // two S buffers of 64 columns
  static constexpr int TMEM_O = 128;
  static constexpr int TMEM_COLS = (128 + H) <= 256 ? 256 : 512;
};

template <int H>
__global__ void __launch_bounds__(160, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using C_ = FwdCfg<H>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sptr = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t sQ = sbase + C_::OFF_Q, sK = sbase + C_::OFF_K, sV = sbase + C_::OFF_V,
                 sP = sbase + C_::OFF_P, bars = sbase + C_::OFF_BAR;
  // barriers: 0 Q, 1 K, 2-3 V[2], 4-5 S[2], 6 P, 7 PV
  const uint32_t barQ = bars, barK = bars + 8, barV0 = bars + 16, barS0 = bars + 32,
                 barP = bars + 48, barPV = bars + 56;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sptr + C_::OFF_BAR + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sptr + C_::OFF_BAR + 68);

  const int warp = threadIdx.x >> 5;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int n = blockIdx.y, b = blockIdx.z;
  const int kvh = n / (a.N / a.KH);
  const int q0 = qt * BQ;

  // key-block range of this query tile
  int kv_end = a.Tk;
  if (a.causal) kv_end = min(a.Tk, q0 + BQ + a.q_off);
  int kv_start = 0;
  if (a.window > 0) kv_start = max(0, q0 + a.q_off - a.window + 1);
  const int jb0 = kv_start / BKV;
  const int nblk = kv_end > jb0 * BKV ? (kv_end - jb0 * BKV + BKV - 1) / BKV : 0;

  if (threadIdx.x == 0) {
    mbar_init(barQ, 1);
    mbar_init(barK, 1);
    mbar_init(barV0, 1);
    mbar_init(barV0 + 8, 1);
    mbar_init(barS0, 1);
    mbar_init(barS0 + 8, 1);
    mbar_init(barP, 128);
    mbar_init(barPV, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32((const void*)tmem_slot), C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------ issuer warp
    if (nblk > 0 && elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(BQ, H, 0, 1);
      auto load_k = [&](int j) {
        mbar_expect_tx(barK, C_::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C_::HS; ++c)
          tma_load_2d(sK + c * (BKV * 128), &tmK, barK, kvh * H + 64 * c, b * a.Tk + (jb0 + j) * BKV);
      };
      auto load_v = [&](int j) {
        const uint32_t bar = barV0 + 8 * (j & 1);
        mbar_expect_tx(bar, C_::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C_::HS; ++c)
          tma_load_2d(sV + (j & 1) * C_::KV_BYTES + c * (BKV * 128), &tmV, bar, kvh * H + 64 * c,
                      b * a.Tk + (jb0 + j) * BKV);
      };
      auto issue_s = [&](int j) {
        const uint32_t d = tmem + C_::TMEM_S + (j & 1) * BKV;
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint64_t ad = make_smem_desc(sQ + (kk >> 2) * (BQ * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(sK + (kk >> 2) * (BKV * 128) + (kk & 3) * 32, 16, 1024);
          umma_f16_ss(d, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(barS0 + 8 * (j & 1));
      };
      bool ok = true;
      mbar_expect_tx(barQ, C_::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C_::HS; ++c)
        tma_load_2d(sQ + c * (BQ * 128), &tmQ, barQ, n * H + 64 * c, b * a.Tq + q0);
      load_k(0);
      load_v(0);
      ok = ok && mbar_wait_bounded(barQ, 0, abort_flag, a.status, ST_TIMEOUT_PRODUCER);
      ok = ok && mbar_wait_bounded(barK, 0, abort_flag, a.status, ST_TIMEOUT_PRODUCER);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          // S_j retired -> the K buffer is free again
          if (!mbar_wait_bounded(barS0 + 8 * (j & 1), (j >> 1) & 1, abort_flag, a.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          load_k(j + 1);
          if (!mbar_wait_bounded(barK, (j + 1) & 1, abort_flag, a.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
          // V buffer (j+1)&1 was last read by PV_{j-1}
          if (j >= 1 && !mbar_wait_bounded(barPV, (j - 1) & 1, abort_flag, a.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          load_v(j + 1);
        }
        if (!mbar_wait_bounded(barP, j & 1, abort_flag, a.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        if (!mbar_wait_bounded(barV0 + 8 * (j & 1), (j >> 1) & 1, abort_flag, a.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
        tc_fence_after();
        const uint32_t vb = sV + (j & 1) * C_::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t ad = make_smem_desc(sP + kk * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(vb + kk * 2048, BKV * 128, 1024);
          umma_f16_ss(tmem + C_::TMEM_O, ad, bd, idesc_o, (j | kk) != 0);
        }
        umma_commit(barPV);
      }
    }
  } else {
    // ---------------------------------------------------------- softmax warps
    const int r = threadIdx.x;             // row inside the tile == TMEM lane
    const int qi = q0 + r;                 // query index in the sequence
    const bool row_valid = qi < a.Tq;
    const int qpos = qi + a.q_off;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const int my_seg = (a.seg_q && row_valid) ? a.seg_q[(long long)b * a.Tq + qi] : 0;
    const float sc2 = a.scale * LOG2E;
    float m_used = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      if (!mbar_wait_bounded(barS0 + 8 * (j & 1), (j >> 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      uint32_t sraw[64];
      {
        uint32_t t0[32], t1[32];
        tmem_ld_32x32(tmem + lane_addr + C_::TMEM_S + (j & 1) * BKV, t0);
        tmem_ld_32x32(tmem + lane_addr + C_::TMEM_S + (j & 1) * BKV + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sraw[i] = t0[i]; sraw[32 + i] = t1[i]; }
      }
      const int k0 = (jb0 + j) * BKV;
      float z[64];
      float mx = -INFINITY;
      const int* segk = a.seg_k ? a.seg_k + (long long)b * a.Tk + k0 : nullptr;
      // most key blocks of a causal tile lie fully below the diagonal: skip the per-element mask there
      const bool need_mask = (k0 + BKV > a.Tk) || (segk != nullptr) ||
                             (a.causal && (k0 + BKV - 1 > q0 + a.q_off)) ||
                             (a.window > 0 && (k0 <= q0 + BQ - 1 + a.q_off - a.window));
      if (!need_mask && a.softcap <= 0.f) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          z[i] = __uint_as_float(sraw[i]) * sc2;
          mx = fmaxf(mx, z[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int kp = k0 + i;
          float s = __uint_as_float(sraw[i]);
          if (a.softcap > 0.f) s = a.softcap * tanhf(s * a.scale / a.softcap) * LOG2E;
          else s *= sc2;
          bool keep = kp < a.Tk;
          if (a.causal) keep = keep && (kp <= qpos);
          if (a.window > 0) keep = keep && (kp > qpos - a.window);
          if (segk) keep = keep && (kp < a.Tk) && (__ldg(segk + (kp < a.Tk ? i : 0)) == my_seg);
          s = keep ? s : -INFINITY;
          z[i] = s;
          mx = fmaxf(mx, s);
        }
      }
      float alpha = 1.f;
      bool need = false;
      if (mx != -INFINITY) {
        if (l == 0.f) {
          m_used = mx;  // nothing accumulated yet for this row: O is exactly zero
        } else if (mx > m_used + RESCALE_THRESHOLD) {
          alpha = exp2f(m_used - mx);
          m_used = mx;
          need = true;
        }
      }
      const bool warp_need = __any_sync(0xffffffffu, need);
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = exp2f(z[2 * i] - m_used);
        const float p1 = exp2f(z[2 * i + 1] - m_used);
        psum += p0 + p1;
        pk[i] = pack_bf16(p0, p1);
      }
      l = l * alpha + psum;
      if (j > 0) {
        // PV_{j-1} retired: P buffer reusable and O consistent
        if (!mbar_wait_bounded(barPV, (j - 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
        if (warp_need) {
#pragma unroll 1
          for (int c = 0; c < H / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(tmem + lane_addr + C_::TMEM_O + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(tmem + lane_addr + C_::TMEM_O + c * 16, o);
          }
          tmem_st_wait();
        }
      }
      // P row -> smem, K-major 128-byte swizzle: 16-byte chunk c of row r lands at c ^ (r & 7)
      uint8_t* prow = sptr + C_::OFF_P + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 v = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(barP);
    }
    // ------------------------------------------------------------- epilogue
    if (ok && nblk > 0)
      ok = mbar_wait_bounded(barPV, (nblk - 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE);
    tc_fence_after();
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    __nv_bfloat16* orow = a.O + ((long long)b * a.Tq + qi) * a.ldo + (long long)n * H;
#pragma unroll 1
    for (int c = 0; c < H / 32; ++c) {
      uint32_t o[32];
      if (nblk > 0 && ok) {
        tmem_ld_32x32(tmem + lane_addr + C_::TMEM_O + c * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0;
      }
      if (row_valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(o[8 * g + 0]) * inv_l, __uint_as_float(o[8 * g + 1]) * inv_l);
          v.y = pack_bf16(__uint_as_float(o[8 * g + 2]) * inv_l, __uint_as_float(o[8 * g + 3]) * inv_l);
          v.z = pack_bf16(__uint_as_float(o[8 * g + 4]) * inv_l, __uint_as_float(o[8 * g + 5]) * inv_l);
          v.w = pack_bf16(__uint_as_float(o[8 * g + 6]) * inv_l, __uint_as_float(o[8 * g + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
        }
      }
    }
    if (row_valid && a.lse)
      a.lse[((long long)b * a.N + n) * a.Tq + qi] = (l > 0.f) ? (m_used / LOG2E + logf(l)) : INFINITY;
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, C_::TMEM_COLS);
  }
}

template <int H>
int launch_fwd(const void* q, const void* k, const void* v, const AttnArgs& a, long long ldq,
               long long ldk, long long ldv, cudaStream_t stream) {
  using C_ = FwdCfg<H>;
  CUtensorMap tq, tk, tv;
  if (tb_make_tmap_2d_bf16(&tq, q, (uint64_t)a.B * a.Tq, (uint64_t)a.N * H, ldq, BQ, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tk, k, (uint64_t)a.B * a.Tk, (uint64_t)a.KH * H, ldk, BKV, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tv, v, (uint64_t)a.B * a.Tk, (uint64_t)a.KH * H, ldv, BKV, 64, 1)) return -3;
  static DeviceOnce once;
  if (once.first() &&
      cudaFuncSetAttribute(attn_fwd_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES) != cudaSuccess)
    return -5;
  dim3 grid((a.Tq + BQ - 1) / BQ, a.N, a.B);
  attn_fwd_kernel<H><<<grid, 160, C_::SMEM_BYTES, stream>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}


// ---------------------------------------------------------------------------------------------
// Two query tiles per CTA (head dim 64 / 128, more than 128 query rows).
//
// The one-tile kernel above leaves the tensor pipe idle most of the time: its four softmax warps
// sit one per scheduler, every K tile is fetched only after the previous S = Q K^T has retired
// (one K buffer), and the P buffer is single. Here a CTA owns 256 query rows of one head as two
// 128-row tiles a and b:
//   warps 0-7 / 8-15 : softmax of tile a / b. TWO threads per query row: warps 0-3 take key columns
//                      0-31 of a block, warps 4-7 columns 32-63 (same TMEM lanes, other columns); the
//                      two halves of a row exchange their maxima through shared memory once per block
//                      and each rescales / writes back its half of O. With one thread per row an SM
//                      holds two softmax warps per scheduler and the kernel is bound by instruction
//                      latency (ncu: 0.32 instructions per cycle and scheduler, tensor pipe 29 %).
//   warp 16          : one thread issues every tcgen05.mma: S_a, S_b of key block j+1 are queued
//                      before it waits for P_a(j), P_b(j), so the tensor pipe always has work
//                      from one tile while the other tile's rows are in the softmax
//   warp 17          : one thread runs the TMA ring (K_0 V_0 K_1 V_1 ... over NSTG stages, three
//                      key blocks ahead); a stage is handed back by a tcgen05.commit
// TMEM: S_a[2] | S_b[2] | O_a | O_b = 4*64 + 2*H columns. K / V tiles are read once per 256 rows.
// ---------------------------------------------------------------------------------------------
template <int H>
struct Fwd2Cfg {
  static constexpr int HS = H / 64;
  static constexpr int Q_BYTES = HS * 128 * 128;    // one 128-row tile
  static constexpr int KV_BYTES = HS * BKV * 128;
  static constexpr int P_BYTES = 128 * 128;
  static constexpr int NSTG = H == 128 ? 6 : 8;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_RING = 2 * Q_BYTES;
  static constexpr int OFF_P = OFF_RING + NSTG * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int OFF_MX = OFF_BAR + 256;      // row maxima / sums exchanged between the two column halves
  static constexpr int SMEM_BYTES = OFF_MX + 2 * 2 * 2 * 128 * 4 + 1024;
  static constexpr int TMEM_COLS = 512;
  __host__ __device__ static constexpr int tm_s(int x, int buf) { return x * 128 + buf * 64; }
  __host__ __device__ static constexpr int tm_o(int x) { return 256 + x * H; }
};

template <int H>
__global__ void __launch_bounds__(576, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using C_ = Fwd2Cfg<H>;
  constexpr int NSTG = C_::NSTG;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sptr = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t sQ = sbase + C_::OFF_Q, sRing = sbase + C_::OFF_RING, sP = sbase + C_::OFF_P,
                 bars = sbase + C_::OFF_BAR;
  // barriers (8 bytes each): 0 Q | 1..NSTG full | 9..8+NSTG free | 17-20 S[x][buf] | 21-22 P[x] | 23-24 PV[x] |
  //                          25-26 row-max exchange[x]
  const uint32_t barQ = bars, barFull0 = bars + 8, barFree0 = bars + 72, barS0 = bars + 136, barP0 = bars + 168,
                 barPV0 = bars + 184, barX0 = bars + 200;
  float* s_mx = reinterpret_cast<float*>(sptr + C_::OFF_MX);     // [2 parities][2 tiles][2 halves][128 rows]
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sptr + C_::OFF_BAR + 224);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sptr + C_::OFF_BAR + 228);

  const int warp = threadIdx.x >> 5;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int n = blockIdx.y, b = blockIdx.z;
  const int kvh = n / (a.N / a.KH);
  const int q0 = qt * 256;

  // key-block range of each tile, relative to the first block the CTA touches
  int kstart[2], kend[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int q0x = q0 + x * 128;
    int ke = a.Tk, ks = 0;
    if (a.causal) ke = min(a.Tk, q0x + 128 + a.q_off);
    if (a.window > 0) ks = max(0, q0x + a.q_off - a.window + 1);
    if (q0x >= a.Tq || ke <= ks) { ks = 0; ke = 0; }
    kstart[x] = ks;
    kend[x] = ke;
  }
  int jb0 = 1 << 30;
#pragma unroll
  for (int x = 0; x < 2; ++x)
    if (kend[x] > 0) jb0 = min(jb0, kstart[x] / BKV);
  int lo[2], hi[2], nblk = 0;
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    lo[x] = hi[x] = 0;
    if (kend[x] > 0) {
      lo[x] = kstart[x] / BKV - jb0;
      hi[x] = (kend[x] + BKV - 1) / BKV - jb0;
      nblk = max(nblk, hi[x]);
    }
  }

  if (threadIdx.x == 0) {
    mbar_init(barQ, 1);
    for (int s = 0; s < NSTG; ++s) {
      mbar_init(barFull0 + 8 * s, 1);
      mbar_init(barFree0 + 8 * s, 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(barS0 + 8 * i, 1);
    for (int x = 0; x < 2; ++x) {
      mbar_init(barP0 + 8 * x, 256);
      mbar_init(barPV0 + 8 * x, 1);
      mbar_init(barX0 + 8 * x, 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 16) {
    tmem_alloc(smem_u32((const void*)tmem_slot), C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 17) {
    // ------------------------------------------------------------------ TMA ring
    if (nblk > 0 && elect_one()) {
      mbar_expect_tx(barQ, 2 * C_::Q_BYTES);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int c = 0; c < C_::HS; ++c)
          tma_load_2d(sQ + x * C_::Q_BYTES + c * (128 * 128), &tmQ, barQ, n * H + 64 * c, b * a.Tq + q0 + x * 128);
      const int ntiles = 2 * nblk;
      for (int t = 0; t < ntiles; ++t) {
        const int s = t % NSTG, use = t / NSTG;
        if (use > 0 &&
            !mbar_wait_bounded(barFree0 + 8 * s, (use - 1) & 1, abort_flag, a.status, ST_TIMEOUT_PRODUCER))
          break;
        const uint32_t bar = barFull0 + 8 * s;
        const CUtensorMap* tm = (t & 1) ? &tmV : &tmK;
        mbar_expect_tx(bar, C_::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C_::HS; ++c)
          tma_load_2d(sRing + s * C_::KV_BYTES + c * (BKV * 128), tm, bar, kvh * H + 64 * c,
                      b * a.Tk + (jb0 + (t >> 1)) * BKV);
      }
    }
  } else if (warp == 16) {
    // ---------------------------------------------------------------- MMA issuer
    if (nblk > 0 && elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(128, BKV, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, H, 0, 1);
      // Descriptors are built once: the start-address field sits in the low bits, so the descriptor of a tile
      // further along is the base plus (byte offset >> 4). The issuing thread is the one serial resource both
      // tiles share; every instruction it does not spend on descriptor arithmetic goes to issuing MMAs.
      const uint64_t qd0 = make_smem_desc(sQ, 16, 1024);
      const uint64_t kd0 = make_smem_desc(sRing, 16, 1024);
      const uint64_t pd0 = make_smem_desc(sP, 16, 1024);
      const uint64_t vd0 = make_smem_desc(sRing, BKV * 128, 1024);
      auto wait_full = [&](int t) {
        return mbar_wait_bounded(barFull0 + 8 * (t % NSTG), (t / NSTG) & 1, abort_flag, a.status, ST_TIMEOUT_MMA);
      };
      auto issue_s = [&](int x, int j) {
        const int i = j - lo[x];
        const uint32_t d = tmem + C_::tm_s(x, i & 1);
        const uint64_t qd = qd0 + (uint64_t)((x * C_::Q_BYTES) >> 4);
        const uint64_t kd = kd0 + (uint64_t)((((2 * j) % NSTG) * C_::KV_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk)
          umma_f16_ss(d, qd + (uint64_t)(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4),
                      kd + (uint64_t)(((kk >> 2) * (BKV * 128) + (kk & 3) * 32) >> 4), idesc_s, kk != 0);
        umma_commit(barS0 + 8 * (2 * x + (i & 1)));
      };
      auto issue_s_block = [&](int j) {        // both tiles' S of key block j; the K stage goes back when they retire
#pragma unroll
        for (int x = 0; x < 2; ++x)
          if (j >= lo[x] && j < hi[x]) issue_s(x, j);
        umma_commit(barFree0 + 8 * ((2 * j) % NSTG));
      };
      bool ok = mbar_wait_bounded(barQ, 0, abort_flag, a.status, ST_TIMEOUT_MMA) && wait_full(0);
      if (ok) {
        tc_fence_after();
        issue_s_block(0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          if (!wait_full(2 * j + 2)) { ok = false; break; }
          tc_fence_after();
          issue_s_block(j + 1);
        }
        if (!wait_full(2 * j + 1)) { ok = false; break; }
        const uint64_t vd = vd0 + (uint64_t)((((2 * j + 1) % NSTG) * C_::KV_BYTES) >> 4);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (j < lo[x] || j >= hi[x]) continue;
          const int i = j - lo[x];
          if (!mbar_wait_bounded(barP0 + 8 * x, i & 1, abort_flag, a.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint64_t pd = pd0 + (uint64_t)((x * C_::P_BYTES) >> 4);
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk)
            umma_f16_ss(tmem + C_::tm_o(x), pd + (uint64_t)((kk * 32) >> 4), vd + (uint64_t)((kk * 2048) >> 4), idesc_o,
                        (i | kk) != 0);
          umma_commit(barPV0 + 8 * x);
        }
        if (ok) umma_commit(barFree0 + 8 * ((2 * j + 1) % NSTG));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int x = warp >> 3;               // tile
    const int half = (warp >> 2) & 1;      // which 32 of the block's 64 key columns
    const int r = ((warp & 3) << 5) | (threadIdx.x & 31);   // row inside the tile == TMEM lane
    const int qi = q0 + x * 128 + r;
    const bool row_valid = qi < a.Tq;
    const int qpos = qi + a.q_off;
    const int q0x = q0 + x * 128;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int my_seg = (a.seg_q && row_valid) ? a.seg_q[(long long)b * a.Tq + qi] : 0;
    const float sc2 = a.scale * LOG2E;
    const int lo_x = x ? lo[1] : lo[0];
    const int nx = (x ? hi[1] : hi[0]) - lo_x;
    const uint32_t barS = barS0 + 16 * x, barP = barP0 + 8 * x, barPV = barPV0 + 8 * x, barX = barX0 + 8 * x;
    constexpr int HH = H / 2;              // this thread's columns of O
    const uint32_t tO = tmem + lane_addr + C_::tm_o(x) + half * HH;
    float m_used = 0.f, l = 0.f;           // l: this half's share of the row sum
    bool seen = false;                     // a key was visible to this row (decided on the maximum both halves share)
    bool ok = true;
    for (int i = 0; i < nx && ok; ++i) {
      const int j = lo_x + i;
      if (!mbar_wait_bounded(barS + 8 * (i & 1), (i >> 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      uint32_t sraw[32];
      tmem_ld_32x32(tmem + lane_addr + C_::tm_s(x, i & 1) + half * 32, sraw);
      tmem_ld_wait();
      const int k0 = (jb0 + j) * BKV;
      const int kh = k0 + half * 32;
      const int* segk = a.seg_k ? a.seg_k + (long long)b * a.Tk + kh : nullptr;
      const bool need_mask = (k0 + BKV > a.Tk) || (segk != nullptr) ||
                             (a.causal && (k0 + BKV - 1 > q0x + a.q_off)) ||
                             (a.window > 0 && (k0 <= q0x + 127 + a.q_off - a.window));
      const bool fast = !need_mask && a.softcap <= 0.f;
      float mx = -INFINITY;
      if (fast) {
        // raw scores: the scale is folded into the exponent's FMA below (scale > 0 keeps the max where it is);
        // four independent chains instead of one of 32
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          m0 = fmaxf(m0, __uint_as_float(sraw[c]));
          m1 = fmaxf(m1, __uint_as_float(sraw[c + 1]));
          m2 = fmaxf(m2, __uint_as_float(sraw[c + 2]));
          m3 = fmaxf(m3, __uint_as_float(sraw[c + 3]));
        }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * sc2;
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int kp = kh + c;
          float sv = __uint_as_float(sraw[c]);
          if (a.softcap > 0.f) sv = a.softcap * tanhf(sv * a.scale / a.softcap) * LOG2E;
          else sv *= sc2;
          bool keep = kp < a.Tk;
          if (a.causal) keep = keep && (kp <= qpos);
          if (a.window > 0) keep = keep && (kp > qpos - a.window);
          if (segk) keep = keep && (kp < a.Tk) && (__ldg(segk + (kp < a.Tk ? c : 0)) == my_seg);
          sv = keep ? sv : -INFINITY;
          sraw[c] = __float_as_uint(sv);
          mx = fmaxf(mx, sv);
        }
      }
      // the row's maximum over both halves: both threads then take the same rescaling decision
      float* slot = s_mx + (((i & 1) * 2 + x) * 2) * 128;
      slot[half * 128 + r] = mx;
      mbar_arrive(barX);
      if (!mbar_wait_bounded(barX, i & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      mx = fmaxf(mx, slot[(half ^ 1) * 128 + r]);
      float alpha = 1.f;
      bool need = false;
      if (mx != -INFINITY) {
        if (!seen) {
          m_used = mx;  // no key has been visible to this row yet: O and both halves' sums are exactly zero
          seen = true;
        } else if (mx > m_used + RESCALE_THRESHOLD) {
          alpha = exp2f(m_used - mx);
          m_used = mx;
          need = true;
        }
      }
      const bool warp_need = __any_sync(0xffffffffu, need);
      float p0s = 0.f, p1s = 0.f, p2s = 0.f, p3s = 0.f;
      uint32_t pk[16];
      const float mul = fast ? sc2 : 1.f;
      const float neg_m = -m_used;
#pragma unroll
      for (int c = 0; c < 16; c += 2) {
        const float e0 = exp2f(fmaf(__uint_as_float(sraw[2 * c]), mul, neg_m));
        const float e1 = exp2f(fmaf(__uint_as_float(sraw[2 * c + 1]), mul, neg_m));
        const float e2 = exp2f(fmaf(__uint_as_float(sraw[2 * c + 2]), mul, neg_m));
        const float e3 = exp2f(fmaf(__uint_as_float(sraw[2 * c + 3]), mul, neg_m));
        p0s += e0; p1s += e1; p2s += e2; p3s += e3;
        pk[c] = pack_bf16(e0, e1);
        pk[c + 1] = pack_bf16(e2, e3);
      }
      l = l * alpha + ((p0s + p1s) + (p2s + p3s));
      if (i > 0) {
        // PV(i-1) retired: P buffer reusable and O consistent
        if (!mbar_wait_bounded(barPV, (i - 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
        if (warp_need) {
#pragma unroll 1
          for (int c = 0; c < HH / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(tO + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x16(tO + c * 16, o);
          }
          tmem_st_wait();
        }
      }
      // this half of the P row -> smem, K-major 128-byte swizzle: 16-byte chunk c of row r lands at c ^ (r & 7)
      uint8_t* prow = sptr + C_::OFF_P + x * C_::P_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 v = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        *reinterpret_cast<uint4*>(prow + (((half * 4 + c) ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(barP);
    }
    // ------------------------------------------------------------- epilogue
    if (ok && nx > 0) ok = mbar_wait_bounded(barPV, (nx - 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE);
    tc_fence_after();
    // the row sum is the two halves' shares together
    float* lslot = s_mx + ((nx & 1) * 2 + x) * 2 * 128;
    lslot[half * 128 + r] = l;
    mbar_arrive(barX);
    if (ok) ok = mbar_wait_bounded(barX, nx & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE);
    if (ok) l += lslot[(half ^ 1) * 128 + r];
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    __nv_bfloat16* orow = a.O + ((long long)b * a.Tq + qi) * a.ldo + (long long)n * H + half * HH;
#pragma unroll 1
    for (int c = 0; c < HH / 32; ++c) {
      uint32_t o[32];
      if (nx > 0 && ok) {
        tmem_ld_32x32(tO + c * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0;
      }
      if (row_valid) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(o[8 * g + 0]) * inv_l, __uint_as_float(o[8 * g + 1]) * inv_l);
          v.y = pack_bf16(__uint_as_float(o[8 * g + 2]) * inv_l, __uint_as_float(o[8 * g + 3]) * inv_l);
          v.z = pack_bf16(__uint_as_float(o[8 * g + 4]) * inv_l, __uint_as_float(o[8 * g + 5]) * inv_l);
          v.w = pack_bf16(__uint_as_float(o[8 * g + 6]) * inv_l, __uint_as_float(o[8 * g + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
        }
      }
    }
    if (row_valid && a.lse && half == 0)
      a.lse[((long long)b * a.N + n) * a.Tq + qi] = (l > 0.f) ? (m_used / LOG2E + logf(l)) : INFINITY;
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // copies in flight land before the CTA's memory goes away
  }
  if (warp == 16) {
    tc_fence_after();
    tmem_dealloc(tmem, C_::TMEM_COLS);
  }
}

template <int H>
int launch_fwd2(const void* q, const void* k, const void* v, const AttnArgs& a, long long ldq,
                long long ldk, long long ldv, cudaStream_t stream) {
  using C_ = Fwd2Cfg<H>;
  CUtensorMap tq, tk, tv;
  if (tb_make_tmap_2d_bf16(&tq, q, (uint64_t)a.B * a.Tq, (uint64_t)a.N * H, ldq, 128, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tk, k, (uint64_t)a.B * a.Tk, (uint64_t)a.KH * H, ldk, BKV, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tv, v, (uint64_t)a.B * a.Tk, (uint64_t)a.KH * H, ldv, BKV, 64, 1)) return -3;
  static DeviceOnce once;
  if (once.first() &&
      cudaFuncSetAttribute(attn_fwd2_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES) != cudaSuccess)
    return -5;
  dim3 grid((a.Tq + 255) / 256, a.N, a.B);
  attn_fwd2_kernel<H><<<grid, 576, C_::SMEM_BYTES, stream>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// The two-tile kernel is opt-in (TUNIX_B200_ATTN_TWO_TILE=1, read at every call): measured on B200 at B = 8, T = 2048,
// 32 / 8 heads of 128 it reaches 580 TFLOP/s against 630 for two co-resident one-tile CTAs per SM, so the one-tile
// kernel stays the default. What was ruled out on the way: the single K buffer (the ring made no difference), the
// number of softmax warps (one or two threads per row: 568 vs 581), descriptor arithmetic in the issuing thread
// (precomputed: 578).
bool use_two_tiles(int H, int Tq) {
  const char* on = getenv("TUNIX_B200_ATTN_TWO_TILE");
  return on != nullptr && on[0] == '1' && H <= 128 && Tq > 128;
}

}  // namespace

// q: [B*Tq, N*H] row stride ldq; k, v: [B*Tk, KH*H]; o: [B*Tq, N*H]; lse: [B, N, Tq] fp32 (may be null).
// seg_q / seg_k: int32 [B,Tq] / [B,Tk] or null. Rows of k/v past Tk must hold finite values.
TB_API int tb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq,
                       int Tk, int N, int KH, int H, long long ldq, long long ldk, long long ldv,
                       long long ldo, float scale, float softcap, int causal, int window, int q_off,
                       const int* seg_q, const int* seg_k, int* status, cudaStream_t stream) {
  if (B <= 0 || Tq <= 0 || N <= 0) return 0;
  if (KH <= 0 || N % KH || (ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -2;
  AttnArgs a;
  a.B = B; a.Tq = Tq; a.Tk = Tk; a.N = N; a.KH = KH;
  a.scale = scale; a.softcap = softcap; a.causal = causal; a.window = window; a.q_off = q_off;
  a.seg_q = seg_q; a.seg_k = seg_k;
  a.O = reinterpret_cast<__nv_bfloat16*>(o); a.ldo = ldo; a.lse = lse; a.status = status;
  if (use_two_tiles(H, Tq))
    return H == 64 ? launch_fwd2<64>(q, k, v, a, ldq, ldk, ldv, stream) : launch_fwd2<128>(q, k, v, a, ldq, ldk, ldv, stream);
  switch (H) {
    case 64: return launch_fwd<64>(q, k, v, a, ldq, ldk, ldv, stream);
    case 128: return launch_fwd<128>(q, k, v, a, ldq, ldk, ldv, stream);
    case 256: return launch_fwd<256>(q, k, v, a, ldq, ldk, ldv, stream);
    default: return -2;
  }
}
