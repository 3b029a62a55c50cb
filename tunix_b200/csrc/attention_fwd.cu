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
  switch (H) {
    case 64: return launch_fwd<64>(q, k, v, a, ldq, ldk, ldv, stream);
    case 128: return launch_fwd<128>(q, k, v, a, ldq, ldk, ldv, stream);
    case 256: return launch_fwd<256>(q, k, v, a, ldq, ldk, ldv, stream);
    default: return -2;
  }
}
