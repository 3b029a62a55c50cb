// Flash-attention backward for sm_100a on tcgen05 tensor cores.
//
// One CTA owns 128 keys of one kv head and walks over every (query head of the group,
// 64-row query tile) that can see them. All five GEMMs of the backward run on tcgen05 with
// the accumulators in TMEM; the transposed orientation (keys on TMEM lanes) makes every
// element-wise step thread-local (one thread per key row):
//
//   St  = K  Q^T          [128 keys x 64 queries]     P  = exp(z - lse)
//   dPt = V  dO^T         [128 x 64]                  dS = P * (dP - delta) * scale
//   dV += Pt  dO          [128 x HO]   (accumulates in TMEM over all query tiles / heads)
//   dK += dSt Q           [128 x HO]
//   dQt = K^T dS^T        [HO  x 64]   -> fp32 atomics into dQ (coalesced along the head dim)
//
// HO = min(H, 128): for head_dim 256 two CTAs share the keys, each producing one 128-column
// half of dK / dV / dQ (S and dP need the full contraction and are computed by both).
// Masks and soft-cap as in the forward kernel. Waits are bounded (common.cuh).
//
// Counterpart in the reference: autodiff of the attention in tunix/models/*/model.py
// (e.g. tunix/models/llama3/model.py:379-396); no hand-written backward exists there.
#include "common.cuh"
#include <cstdlib>

using namespace tb;

namespace {

constexpr int BK_ = 128;  // keys per CTA
constexpr int BQ_ = 64;   // queries per iteration
constexpr float LOG2E = 1.4426950408889634f;

struct BwdArgs {
  int B, Tq, Tk, N, KH;
  float scale, softcap;
  int causal, window, q_off;
  const int* seg_q;
  const int* seg_k;
  const float* lse;     // [B, N, Tq]
  const float* delta;   // [B, N, Tq]
  float* dQ;            // fp32 [B*Tq, N*H], zero-initialised by the caller
  __nv_bfloat16* dK;    // [B*Tk, KH*H]
  __nv_bfloat16* dV;
  long long lddk, lddv;
  int* status;
};

template <int H>
struct BwdCfg {
  static constexpr bool PIPE = (H <= 128);          // software-pipelined schedule (needs double buffers)
  static constexpr int HS = H / 64;
  static constexpr int HO = H < 128 ? H : 128;
  static constexpr int NHALF = H / HO;
  static constexpr int NST = PIPE ? 3 : 1;          // Q / dO tile stages
  static constexpr int NPB = PIPE ? 2 : 1;          // Pt / dSt staging buffers
  static constexpr int KV_BYTES = HS * BK_ * 128;
  static constexpr int Q_BYTES = HS * BQ_ * 128;
  static constexpr int P_BYTES = BK_ * 128;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_BYTES;
  static constexpr int OFF_Q = OFF_V + KV_BYTES;
  static constexpr int OFF_DO = OFF_Q + NST * Q_BYTES;
  static constexpr int OFF_PT = OFF_DO + NST * Q_BYTES;
  static constexpr int OFF_DST = OFF_PT + NPB * P_BYTES;
  static constexpr int OFF_STAT = OFF_DST + NPB * P_BYTES;   // [2][3][64] 4-byte values
  static constexpr int OFF_BAR = OFF_STAT + 2 * 3 * 64 * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 192 + 1024;
  // TMEM columns. PIPE: St/dQt buffers at 0 and 64, dPt buffers at 128 and 192, dV at 256, dK after it.
  // Otherwise: St 0, dPt 64, dQt 128, dV 192, dK after it.
  static constexpr int TM_DV = PIPE ? 256 : 192;
  static constexpr int TM_DK = TM_DV + HO;
  static constexpr int TMEM_COLS = 512;
  __host__ __device__ static constexpr int tm_st(int buf) { return PIPE ? buf * 64 : 0; }
  __host__ __device__ static constexpr int tm_dpt(int buf) { return PIPE ? 128 + buf * 64 : 64; }
  __host__ __device__ static constexpr int tm_dqt(int buf) { return PIPE ? buf * 64 : 128; }
};

// Schedule (PIPE): while the row threads work on query tile `it` (P, then dS), the tensor core already
// holds St/dPt of tile it+1 (issued at mid-iteration) and finishes dV/dK/dQt of tile it-1; the dQt of
// tile it-1 is drained between the two phases of tile it. Handoffs never wait on a just-issued MMA.
// RG_: row-thread groups. The BQ_ query columns of a key row are split over RG_ threads (one per warpgroup), so the
// element-wise work between the MMAs runs on 128 * RG_ threads.
template <int H, int RG_>
__global__ void __launch_bounds__(128 * RG_ + 32, 1)   // 9 warps are allocated as 12: 168 registers per thread
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const BwdArgs a) {
  using C_ = BwdCfg<H>;
  constexpr int CW_ = BQ_ / RG_;           // query columns per row thread
  constexpr int NROW_ = 128 * RG_;         // row threads per CTA (plus the issuer warp)
  constexpr int HO = C_::HO;
  constexpr int NST = C_::NST;
  constexpr bool PIPE = C_::PIPE;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sptr = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t sK = sbase + C_::OFF_K, sV = sbase + C_::OFF_V, sQ = sbase + C_::OFF_Q,
                 sdO = sbase + C_::OFF_DO, sPt = sbase + C_::OFF_PT, sdSt = sbase + C_::OFF_DST,
                 bars = sbase + C_::OFF_BAR;
  // barriers (8 bytes each): 0 KV | 1-3 Q[3] | 4-6 Qfree[3] | 7-8 St[2] | 9-10 dPt[2] | 11 Pt | 12 dSt |
  //                          13 dQ | 14 dQ drained | 15 row-thread sync ; then tmem slot + abort flag
  const uint32_t barKV = bars, barQ0 = bars + 8, barQF0 = bars + 32, barSt0 = bars + 56, bardPt0 = bars + 72,
                 barPt = bars + 88, bardSt = bars + 96, bardQ = bars + 104, barDQfree = bars + 112,
                 barSync = bars + 120;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sptr + C_::OFF_BAR + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sptr + C_::OFF_BAR + 132);
  float* s_stat = reinterpret_cast<float*>(sptr + C_::OFF_STAT);

  const int warp = threadIdx.x >> 5;
  const int kt = blockIdx.x;
  const int half = (C_::NHALF > 1) ? (blockIdx.y % C_::NHALF) : 0;
  const int kvh = blockIdx.y / C_::NHALF;
  const int b = blockIdx.z;
  const int G = a.N / a.KH;
  const int k0 = kt * BK_;

  // query tiles that can see keys [k0, k0+128)
  int q_lo = 0, q_hi = a.Tq;
  if (a.causal) q_lo = max(0, k0 - a.q_off);
  if (a.window > 0) q_hi = min(a.Tq, k0 + BK_ + a.window - 1 - a.q_off);
  const int qt0 = q_lo / BQ_;
  const int nq = q_hi > qt0 * BQ_ ? (q_hi - qt0 * BQ_ + BQ_ - 1) / BQ_ : 0;
  const int nit = nq * G;

  if (threadIdx.x == 0) {
    mbar_init(barKV, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(barQ0 + 8 * s, 1);
      mbar_init(barQF0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(barSt0 + 8 * s, 1);
      mbar_init(bardPt0 + 8 * s, 1);
    }
    mbar_init(barPt, NROW_);
    mbar_init(bardSt, NROW_);
    mbar_init(bardQ, 1);
    mbar_init(barDQfree, NROW_);
    mbar_init(barSync, NROW_);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 * RG_) {
    tmem_alloc(smem_u32((const void*)tmem_slot), C_::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM buffer / barrier index and parity of the per-tile St and dPt results
  auto sbuf = [&](int it) { return PIPE ? (it & 1) : 0; };
  auto spar = [&](int it) { return PIPE ? ((it >> 1) & 1) : (it & 1); };

  if (warp == 4 * RG_) {
    // ------------------------------------------------------------ issuer warp
    if (nit > 0 && elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(128, BQ_, 0, 0);     // K-major x K-major, N = 64
      const uint32_t idesc_dv = make_idesc_bf16(128, HO, 0, 1);     // A K-major, B MN-major, N = HO
      const uint32_t idesc_dq = make_idesc_bf16(128, BQ_, 1, 1);    // both MN-major, N = 64
      const uint32_t col_off = half * (HO / 64) * (BQ_ * 128);      // slab offset of this half in Q/dO tiles
      const uint32_t k_half = sK + half * (HO / 64) * (BK_ * 128);
      auto load_q = [&](int it) {
        const int st = it % NST;
        const int g = it / nq, qt = qt0 + it % nq;
        const int n = kvh * G + g;
        const uint32_t bar = barQ0 + 8 * st;
        mbar_expect_tx(bar, 2 * C_::Q_BYTES);
#pragma unroll
        for (int c = 0; c < C_::HS; ++c) {
          tma_load_2d(sQ + st * C_::Q_BYTES + c * (BQ_ * 128), &tmQ, bar, n * H + 64 * c, b * a.Tq + qt * BQ_);
          tma_load_2d(sdO + st * C_::Q_BYTES + c * (BQ_ * 128), &tmdO, bar, n * H + 64 * c, b * a.Tq + qt * BQ_);
        }
      };
      // St = K Q^T ; dPt = V dO^T  (contraction over the full head dim)
      auto issue_s_dp = [&](int it) {
        const int st = it % NST;
        const uint32_t q_s = sQ + st * C_::Q_BYTES, do_s = sdO + st * C_::Q_BYTES;
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint64_t ad = make_smem_desc(sK + (kk >> 2) * (BK_ * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(q_s + (kk >> 2) * (BQ_ * 128) + (kk & 3) * 32, 16, 1024);
          umma_f16_ss(tmem + C_::tm_st(sbuf(it)), ad, bd, idesc_s, kk != 0);
        }
        umma_commit(barSt0 + 8 * sbuf(it));
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint64_t ad = make_smem_desc(sV + (kk >> 2) * (BK_ * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(do_s + (kk >> 2) * (BQ_ * 128) + (kk & 3) * 32, 16, 1024);
          umma_f16_ss(tmem + C_::tm_dpt(sbuf(it)), ad, bd, idesc_s, kk != 0);
        }
        umma_commit(bardPt0 + 8 * sbuf(it));
      };
      // dV += Pt dO   (A = Pt K-major over 64 queries, B = dO MN-major, this CTA's column half)
      auto issue_dv = [&](int it) {
        const uint32_t do_s = sdO + (it % NST) * C_::Q_BYTES;
        const uint32_t pt = sPt + (PIPE ? (it & 1) : 0) * C_::P_BYTES;
#pragma unroll
        for (int kk = 0; kk < BQ_ / 16; ++kk) {
          const uint64_t ad = make_smem_desc(pt + kk * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(do_s + col_off + kk * 2048, BQ_ * 128, 1024);
          umma_f16_ss(tmem + C_::TM_DV, ad, bd, idesc_dv, (it | kk) != 0);
        }
      };
      // dK += dSt Q ; dQt = K^T dS^T
      auto issue_dk_dq = [&](int it) {
        const uint32_t q_s = sQ + (it % NST) * C_::Q_BYTES;
        const uint32_t ds = sdSt + (PIPE ? (it & 1) : 0) * C_::P_BYTES;
#pragma unroll
        for (int kk = 0; kk < BQ_ / 16; ++kk) {
          const uint64_t ad = make_smem_desc(ds + kk * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(q_s + col_off + kk * 2048, BQ_ * 128, 1024);
          umma_f16_ss(tmem + C_::TM_DK, ad, bd, idesc_dv, (it | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < BK_ / 16; ++kk) {
          // A = K^T: M (head dim) contiguous, 64-wide M chunks BK_*128 bytes apart; 16 keys per step
          const uint64_t ad = make_smem_desc(k_half + kk * 2048, BK_ * 128, 1024);
          const uint64_t bd = make_smem_desc(ds + kk * 2048, BK_ * 128, 1024);
          umma_f16_ss(tmem + C_::tm_dqt(sbuf(it)), ad, bd, idesc_dq, kk != 0);
        }
        umma_commit(barQF0 + 8 * (it % NST));
        umma_commit(bardQ);
      };
#define BWD_WAIT(bar, par, code) \
  if (!mbar_wait_bounded((bar), (par), abort_flag, a.status, (code))) { ok = false; break; }
      bool ok = true;
      mbar_expect_tx(barKV, 2 * C_::KV_BYTES);
#pragma unroll
      for (int c = 0; c < C_::HS; ++c) {
        tma_load_2d(sK + c * (BK_ * 128), &tmK, barKV, kvh * H + 64 * c, b * a.Tk + k0);
        tma_load_2d(sV + c * (BK_ * 128), &tmV, barKV, kvh * H + 64 * c, b * a.Tk + k0);
      }
      for (int i = 0; i < NST && i < nit; ++i) load_q(i);
      ok = mbar_wait_bounded(barKV, 0, abort_flag, a.status, ST_TIMEOUT_PRODUCER);
      if (PIPE) {
        ok = ok && mbar_wait_bounded(barQ0, 0, abort_flag, a.status, ST_TIMEOUT_PRODUCER);
        if (ok) {
          tc_fence_after();
          issue_s_dp(0);
        }
        for (int it = 0; it < nit && ok; ++it) {
          BWD_WAIT(barPt, it & 1, ST_TIMEOUT_MMA);
          tc_fence_after();
          issue_dv(it);
          if (it + 1 < nit) {
            BWD_WAIT(barQ0 + 8 * ((it + 1) % NST), ((it + 1) / NST) & 1, ST_TIMEOUT_PRODUCER);
            // St_{it+1} overwrites the TMEM buffer that held dQt_{it-1}: wait until it was drained
            if (it >= 1) BWD_WAIT(barDQfree, (it - 1) & 1, ST_TIMEOUT_MMA);
            tc_fence_after();
            issue_s_dp(it + 1);
          }
          if (it >= 1 && it + 2 < nit) {
            // the stage of tile it-1 is free once its dK / dQt retired
            BWD_WAIT(barQF0 + 8 * ((it - 1) % NST), ((it - 1) / NST) & 1, ST_TIMEOUT_MMA);
            load_q(it + 2);
          }
          BWD_WAIT(bardSt, it & 1, ST_TIMEOUT_MMA);
          tc_fence_after();
          issue_dk_dq(it);
        }
      } else {
        for (int it = 0; it < nit && ok; ++it) {
          if (it >= 1) {
            BWD_WAIT(barQF0, (it - 1) & 1, ST_TIMEOUT_MMA);
            load_q(it);
          }
          BWD_WAIT(barQ0, it & 1, ST_TIMEOUT_PRODUCER);
          tc_fence_after();
          issue_s_dp(it);
          BWD_WAIT(barPt, it & 1, ST_TIMEOUT_MMA);
          tc_fence_after();
          issue_dv(it);
          BWD_WAIT(bardSt, it & 1, ST_TIMEOUT_MMA);
          tc_fence_after();
          issue_dk_dq(it);
        }
      }
    }
  } else {
    // ------------------------------------------------------- per-key-row math
    const int r = threadIdx.x & 127;     // key row in tile == TMEM lane
    const int hq = threadIdx.x >> 7;     // which CW_ query columns of the row this thread works on
    const int c0 = hq * CW_;
    const int kp = k0 + r;
    const bool key_valid = kp < a.Tk;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int my_seg = (a.seg_k && key_valid) ? a.seg_k[(long long)b * a.Tk + kp] : 0;
    bool ok = true;
    auto stat_ptr = [&](int buf, int which) { return s_stat + (buf * 3 + which) * 64; };
    auto tile_of = [&](int it, int& n, int& qbase) {
      n = kvh * G + it / nq;
      qbase = (qt0 + it % nq) * BQ_;
    };
    auto fetch_stats = [&](int it, float& v_lse, float& v_delta, int& v_seg) {
      int n, qbase;
      tile_of(it, n, qbase);
      const int qi = qbase + (int)threadIdx.x;
      if (threadIdx.x < 64 && qi < a.Tq) {
        const long long o = ((long long)b * a.N + n) * a.Tq + qi;
        v_lse = a.lse[o] * LOG2E;
        v_delta = a.delta[o];
        v_seg = a.seg_q ? a.seg_q[(long long)b * a.Tq + qi] : 0;
      } else {
        v_lse = INFINITY;
        v_delta = 0.f;
        v_seg = -1;
      }
    };
    // dQt tile of `it`: lane = head-dim index (within this CTA's half), column = query
    auto drain_dq = [&](int it) {
      int n, qbase;
      tile_of(it, n, qbase);
      uint32_t t[CW_ / 32][32];
#pragma unroll
      for (int j = 0; j < CW_ / 32; ++j) tmem_ld_32x32(tmem + lane_addr + C_::tm_dqt(sbuf(it)) + c0 + 32 * j, t[j]);
      tmem_ld_wait();
      if (r < HO) {
        float* dq = a.dQ + ((long long)b * a.Tq + qbase + c0) * ((long long)a.N * H) + (long long)n * H + half * HO + r;
        const long long ld = (long long)a.N * H;
        if (qbase + 64 <= a.Tq) {
#pragma unroll
          for (int i = 0; i < CW_; ++i) atomicAdd(dq + i * ld, __uint_as_float(t[i >> 5][i & 31]));
        } else {
#pragma unroll
          for (int i = 0; i < CW_; ++i)
            if (qbase + c0 + i < a.Tq) atomicAdd(dq + i * ld, __uint_as_float(t[i >> 5][i & 31]));
        }
      }
    };
    if (nit > 0) {
      float f0, f1;
      int i2;
      fetch_stats(0, f0, f1, i2);
      if (threadIdx.x < 64) {
        stat_ptr(0, 0)[threadIdx.x] = f0;
        stat_ptr(0, 1)[threadIdx.x] = f1;
        reinterpret_cast<int*>(stat_ptr(0, 2))[threadIdx.x] = i2;
      }
    }
    for (int it = 0; it < nit && ok; ++it) {
      // stats of tile `it` visible to every row thread; previous tile's stats fully consumed
      mbar_arrive(barSync);
      BWD_WAIT(barSync, it & 1, ST_TIMEOUT_EPILOGUE);
      float nx_lse = INFINITY, nx_delta = 0.f;
      int nx_seg = -1;
      if (it + 1 < nit) fetch_stats(it + 1, nx_lse, nx_delta, nx_seg);
      int n, qbase;
      tile_of(it, n, qbase);
      const float* st_lse = stat_ptr(it & 1, 0) + c0;          // this thread's columns
      const float* st_delta = stat_ptr(it & 1, 1) + c0;
      const int* st_seg = reinterpret_cast<const int*>(stat_ptr(it & 1, 2)) + c0;
      const int pb = PIPE ? (it & 1) : 0;
      // does any (key, query) pair of this tile need masking?
      const int qpos_lo = qbase + a.q_off, qpos_hi = qbase + BQ_ - 1 + a.q_off;
      const bool need_mask = (k0 + BK_ > a.Tk) || (qbase + BQ_ > a.Tq) || (a.seg_k != nullptr) ||
                             (a.causal && (k0 + BK_ - 1 > qpos_lo)) ||
                             (a.window > 0 && (k0 <= qpos_hi - a.window));

      BWD_WAIT(barSt0 + 8 * sbuf(it), spar(it), ST_TIMEOUT_EPILOGUE);
      tc_fence_after();
      float p[CW_];
      {
        uint32_t t[CW_ / 32][32];
#pragma unroll
        for (int j = 0; j < CW_ / 32; ++j) tmem_ld_32x32(tmem + lane_addr + C_::tm_st(sbuf(it)) + c0 + 32 * j, t[j]);
        tmem_ld_wait();
        const float sc2 = a.scale * LOG2E;
        if (!need_mask && a.softcap <= 0.f) {
#pragma unroll
          for (int i = 0; i < CW_; ++i)
            p[i] = exp2f(__uint_as_float(t[i >> 5][i & 31]) * sc2 - st_lse[i]);
        } else {
#pragma unroll
          for (int i = 0; i < CW_; ++i) {
            const float s = __uint_as_float(t[i >> 5][i & 31]);
            const int qpos = qbase + c0 + i + a.q_off;
            float z;
            if (a.softcap > 0.f) z = a.softcap * tanhf(s * a.scale / a.softcap) * LOG2E;
            else z = s * sc2;
            bool keep = key_valid && (qbase + c0 + i < a.Tq);
            if (a.causal) keep = keep && (kp <= qpos);
            if (a.window > 0) keep = keep && (kp > qpos - a.window);
            if (a.seg_k) keep = keep && (st_seg[i] == my_seg);
            p[i] = keep ? exp2f(z - st_lse[i]) : 0.f;
          }
        }
      }
      {
        uint8_t* prow = sptr + C_::OFF_PT + pb * C_::P_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < CW_ / 8; ++c) {
          uint4 v;
          v.x = pack_bf16(p[8 * c + 0], p[8 * c + 1]);
          v.y = pack_bf16(p[8 * c + 2], p[8 * c + 3]);
          v.z = pack_bf16(p[8 * c + 4], p[8 * c + 5]);
          v.w = pack_bf16(p[8 * c + 6], p[8 * c + 7]);
          *reinterpret_cast<uint4*>(prow + (((c + c0 / 8) ^ (r & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(barPt);
      }
      if (PIPE && it >= 1) {
        // drain dQt of the previous tile while the tensor core works on dV of this one
        BWD_WAIT(bardQ, (it - 1) & 1, ST_TIMEOUT_EPILOGUE);
        tc_fence_after();
        drain_dq(it - 1);
        tc_fence_before();
        mbar_arrive(barDQfree);
      }
      BWD_WAIT(bardPt0 + 8 * sbuf(it), spar(it), ST_TIMEOUT_EPILOGUE);
      tc_fence_after();
      {
        uint32_t t[CW_ / 32][32];
#pragma unroll
        for (int j = 0; j < CW_ / 32; ++j) tmem_ld_32x32(tmem + lane_addr + C_::tm_dpt(sbuf(it)) + c0 + 32 * j, t[j]);
        tmem_ld_wait();
        if (a.softcap > 0.f) {
          uint32_t sv[CW_ / 32][32];
#pragma unroll
          for (int j = 0; j < CW_ / 32; ++j) tmem_ld_32x32(tmem + lane_addr + C_::tm_st(sbuf(it)) + c0 + 32 * j, sv[j]);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < CW_; ++i) {
            const float s = __uint_as_float(sv[i >> 5][i & 31]);
            const float t = tanhf(s * a.scale / a.softcap);
            p[i] *= (1.f - t * t);
          }
        }
        uint8_t* drow = sptr + C_::OFF_DST + pb * C_::P_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < CW_ / 8; ++c) {
          float d[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int i = 8 * c + e;
            const float dp = __uint_as_float(t[i >> 5][i & 31]);
            d[e] = p[i] * (dp - st_delta[i]) * a.scale;
          }
          uint4 v;
          v.x = pack_bf16(d[0], d[1]);
          v.y = pack_bf16(d[2], d[3]);
          v.z = pack_bf16(d[4], d[5]);
          v.w = pack_bf16(d[6], d[7]);
          *reinterpret_cast<uint4*>(drow + (((c + c0 / 8) ^ (r & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(bardSt);
      }
      if (!PIPE) {
        BWD_WAIT(bardQ, it & 1, ST_TIMEOUT_EPILOGUE);
        tc_fence_after();
        drain_dq(it);
        tc_fence_before();
      }
      if (it + 1 < nit && threadIdx.x < 64) {
        stat_ptr((it + 1) & 1, 0)[threadIdx.x] = nx_lse;
        stat_ptr((it + 1) & 1, 1)[threadIdx.x] = nx_delta;
        reinterpret_cast<int*>(stat_ptr((it + 1) & 1, 2))[threadIdx.x] = nx_seg;
      }
    }
    if (PIPE && nit > 0 && ok) {
      // last tile's dQt; its completion also means every dV / dK MMA has retired
      ok = mbar_wait_bounded(bardQ, (nit - 1) & 1, abort_flag, a.status, ST_TIMEOUT_EPILOGUE);
      tc_fence_after();
      if (ok) drain_dq(nit - 1);
    }
#undef BWD_WAIT
    // ------------------------------------------------------------- dK / dV
    tc_fence_after();
    __nv_bfloat16* dkrow = a.dK + ((long long)b * a.Tk + kp) * a.lddk + (long long)kvh * H + half * HO;
    __nv_bfloat16* dvrow = a.dV + ((long long)b * a.Tk + kp) * a.lddv + (long long)kvh * H + half * HO;
#pragma unroll 1
    for (int c = hq; c < HO / 32; c += RG_) {      // the row's output columns are shared out between its threads
      uint32_t o[32];
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        if (nit > 0 && ok) {
          tmem_ld_32x32(tmem + lane_addr + (which ? C_::TM_DK : C_::TM_DV) + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
        if (key_valid) {
          __nv_bfloat16* dst = (which ? dkrow : dvrow) + c * 32;
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[8 * g4 + 0]), __uint_as_float(o[8 * g4 + 1]));
            v.y = pack_bf16(__uint_as_float(o[8 * g4 + 2]), __uint_as_float(o[8 * g4 + 3]));
            v.z = pack_bf16(__uint_as_float(o[8 * g4 + 4]), __uint_as_float(o[8 * g4 + 5]));
            v.w = pack_bf16(__uint_as_float(o[8 * g4 + 6]), __uint_as_float(o[8 * g4 + 7]));
            *reinterpret_cast<uint4*>(dst + g4 * 8) = v;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (warp == 4 * RG_) {
    tc_fence_after();
    tmem_dealloc(tmem, C_::TMEM_COLS);
  }
}

// delta[b, n, t] = sum_h dO * O
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo,
                                  const __nv_bfloat16* __restrict__ dout, long long lddo,
                                  float* __restrict__ delta, int B, int T, int N, int H) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * T * N;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
       w += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int n = (int)(w % N);
    const long long bt = w / N;
    const int t = (int)(bt % T);
    const int b = (int)(bt / T);
    const __nv_bfloat16* po = o + bt * ldo + (long long)n * H;
    const __nv_bfloat16* pd = dout + bt * lddo + (long long)n * H;
    float acc = 0.f;
    for (int c = lane * 2; c < H; c += 64) {
      const uint32_t x = *reinterpret_cast<const uint32_t*>(po + c);
      const uint32_t y = *reinterpret_cast<const uint32_t*>(pd + c);
      acc += bf16_lo(x) * bf16_lo(y) + bf16_hi(x) * bf16_hi(y);
    }
    acc = warp_sum(acc);
    if (lane == 0) delta[((long long)b * N + n) * T + t] = acc;
  }
}

template <int H>
int launch_bwd(const void* q, const void* k, const void* v, const void* dout, const BwdArgs& a,
               long long ldq, long long ldk, long long ldv, long long lddo, cudaStream_t stream) {
  using C_ = BwdCfg<H>;
  CUtensorMap tq, tk, tv, tdo;
  if (tb_make_tmap_2d_bf16(&tq, q, (uint64_t)a.B * a.Tq, (uint64_t)a.N * H, ldq, BQ_, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tdo, dout, (uint64_t)a.B * a.Tq, (uint64_t)a.N * H, lddo, BQ_, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tk, k, (uint64_t)a.B * a.Tk, (uint64_t)a.KH * H, ldk, BK_, 64, 1)) return -3;
  if (tb_make_tmap_2d_bf16(&tv, v, (uint64_t)a.B * a.Tk, (uint64_t)a.KH * H, ldv, BK_, 64, 1)) return -3;
  static DeviceOnce once;
  if (once.first() &&
      (cudaFuncSetAttribute(attn_bwd_kernel<H, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES) != cudaSuccess ||
       cudaFuncSetAttribute(attn_bwd_kernel<H, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM_BYTES) != cudaSuccess))
    return -5;
  dim3 grid((a.Tk + BK_ - 1) / BK_, a.KH * C_::NHALF, a.B);
  // two row-thread groups (288 threads; B = 8, T = 2048, 32 / 8 heads, H = 128: 1.55 ms against 1.77 ms with one group);
  // TUNIX_B200_ATTN_BWD_GROUPS=1 selects the single-warpgroup form for comparison
  static const bool one_group = [] { const char* e = getenv("TUNIX_B200_ATTN_BWD_GROUPS"); return e && atoi(e) == 1; }();
  if (one_group) attn_bwd_kernel<H, 1><<<grid, 160, C_::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, a);
  else attn_bwd_kernel<H, 2><<<grid, 288, C_::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

TB_API int tb_attn_delta(const void* o, long long ldo, const void* dout, long long lddo, float* delta,
                         int B, int T, int N, int H, cudaStream_t stream) {
  const long long total = (long long)B * T * N;
  if (total <= 0) return 0;
  long long blocks = (total + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  attn_delta_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, ldo, (const __nv_bfloat16*)dout,
                                                     lddo, delta, B, T, N, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// dq_accum: fp32 [B*Tq, N*H] zero-initialised; dk, dv: bf16 [B*Tk, KH*H] (fully written).
TB_API int tb_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                       const float* delta, float* dq_accum, void* dk, void* dv, int B, int Tq, int Tk,
                       int N, int KH, int H, long long ldq, long long ldk, long long ldv, long long lddo,
                       long long lddk, long long lddv, float scale, float softcap, int causal, int window,
                       int q_off, const int* seg_q, const int* seg_k, int* status, cudaStream_t stream) {
  if (B <= 0 || Tk <= 0 || KH <= 0) return 0;
  if (N % KH || (ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddk % 8) || (lddv % 8)) return -2;
  BwdArgs a;
  a.B = B; a.Tq = Tq; a.Tk = Tk; a.N = N; a.KH = KH;
  a.scale = scale; a.softcap = softcap; a.causal = causal; a.window = window; a.q_off = q_off;
  a.seg_q = seg_q; a.seg_k = seg_k; a.lse = lse; a.delta = delta; a.dQ = dq_accum;
  a.dK = reinterpret_cast<__nv_bfloat16*>(dk); a.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  a.lddk = lddk; a.lddv = lddv; a.status = status;
  switch (H) {
    case 64: return launch_bwd<64>(q, k, v, dout, a, ldq, ldk, ldv, lddo, stream);
    case 128: return launch_bwd<128>(q, k, v, dout, a, ldq, ldk, ldv, lddo, stream);
    case 256: return launch_bwd<256>(q, k, v, dout, a, ldq, ldk, ldv, lddo, stream);
    default: return -2;
  }
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in noalloc.h; it has no counterpart in the reference).
//
// tb_attn_bwd above expects its caller to hand it two scratch buffers (delta and the fp32 dQ
// accumulator), which in this package come from torch's caching allocator. Some callers cannot
// allocate device memory at all: code running inside a CUDA-graph capture or a stream-ordered
// region where cudaMalloc is illegal, a serving process whose memory pool is owned and fully
// reserved by another component, or a plain C/C++ host that links this library without torch.
// For them the scratch lives in the library image itself.
// ---------------------------------------------------------------------------------------------
#include "noalloc.h"
#include <cstdio>
#include <mutex>

namespace {

// Fixed scratch, resident on every GPU that loads this library until the process exits.
static __device__ __align__(256) float g_noalloc_dq_scratch[TB_NOALLOC_MAX_DQ_ELEMS];
static __device__ __align__(256) float g_noalloc_delta_scratch[TB_NOALLOC_MAX_ROWS];

constexpr int kMaxDevices = 64;
float* g_noalloc_dq_ptr[kMaxDevices] = {nullptr};
float* g_noalloc_delta_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_setup_mutex;          // two host threads may make the first call on a device at once
thread_local char g_noalloc_error[256] = "";   // each host thread reads the message of its own last call

__global__ void noalloc_zero_kernel(float* p, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = 0.f;
}
__global__ void noalloc_cast_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

int noalloc_fail(int code, const char* msg) {
  snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s", msg);
  return code;
}

// In host code the array names above are host-side stand-ins, not device addresses; the real
// addresses are looked up once per device, with that device current.
int noalloc_setup(int dev) {
  std::lock_guard<std::mutex> lock(g_noalloc_setup_mutex);
  if (g_noalloc_dq_ptr[dev] && g_noalloc_delta_ptr[dev]) return 0;
  float* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_dq_scratch);
  if (e != cudaSuccess || !p) return noalloc_fail(-10, "cudaGetSymbolAddress(dq scratch) failed");
  g_noalloc_dq_ptr[dev] = p;
  p = nullptr;
  e = cudaGetSymbolAddress((void**)&p, g_noalloc_delta_scratch);
  if (e != cudaSuccess || !p) return noalloc_fail(-10, "cudaGetSymbolAddress(delta scratch) failed");
  g_noalloc_delta_ptr[dev] = p;
  return 0;
}

}  // namespace

TB_API const char* tb_noalloc_last_error() { return g_noalloc_error; }

TB_API int tb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const float* lse, void* dq, void* dk, void* dv, int B, int Tq, int Tk, int N,
                               int KH, int H, float scale, float softcap, int causal, int window,
                               int* status, cudaStream_t stream) {
  g_noalloc_error[0] = 0;
  if (B <= 0 || Tq <= 0 || Tk <= 0 || N <= 0 || KH <= 0 || N % KH) return noalloc_fail(-2, "bad shape");
  if (H != 64 && H != 128 && H != 256) return noalloc_fail(-2, "head dim must be 64, 128 or 256");
  const long long dq_elems = (long long)B * Tq * N * H;
  const long long rows = (long long)B * N * Tq;
  if (dq_elems > TB_NOALLOC_MAX_DQ_ELEMS || rows > TB_NOALLOC_MAX_ROWS) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "problem too large for the built-in scratch: B*Tq*N*H = %lld (max %lld), B*N*Tq = %lld (max %lld)",
             dq_elems, (long long)TB_NOALLOC_MAX_DQ_ELEMS, rows, (long long)TB_NOALLOC_MAX_ROWS);
    return -11;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return noalloc_fail(-10, "no current device");
  if (int rc = noalloc_setup(dev)) return rc;
  float* dq32 = g_noalloc_dq_ptr[dev];
  float* delta = g_noalloc_delta_ptr[dev];
  const long long ldq = (long long)N * H, ldkv = (long long)KH * H;
  // The scratch keeps the previous call's contents: the dQ accumulator must start at zero.
  noalloc_zero_kernel<<<592, 256, 0, stream>>>(dq32, dq_elems);
  long long blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  attn_delta_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, ldq, (const __nv_bfloat16*)dout, ldq,
                                                     delta, B, Tq, N, H);
  BwdArgs a;
  a.B = B; a.Tq = Tq; a.Tk = Tk; a.N = N; a.KH = KH;
  a.scale = scale; a.softcap = softcap; a.causal = causal; a.window = window; a.q_off = Tk - Tq;
  a.seg_q = nullptr; a.seg_k = nullptr; a.lse = lse; a.delta = delta; a.dQ = dq32;
  a.dK = reinterpret_cast<__nv_bfloat16*>(dk); a.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  a.lddk = ldkv; a.lddv = ldkv; a.status = status;
  int rc;
  switch (H) {
    case 64: rc = launch_bwd<64>(q, k, v, dout, a, ldq, ldkv, ldkv, ldq, stream); break;
    case 128: rc = launch_bwd<128>(q, k, v, dout, a, ldq, ldkv, ldkv, ldq, stream); break;
    default: rc = launch_bwd<256>(q, k, v, dout, a, ldq, ldkv, ldkv, ldq, stream); break;
  }
  if (rc) return noalloc_fail(rc, "backward launch failed");
  noalloc_cast_kernel<<<592, 256, 0, stream>>>(dq32, (__nv_bfloat16*)dq, dq_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : noalloc_fail(-5, "kernel launch failed");
}
