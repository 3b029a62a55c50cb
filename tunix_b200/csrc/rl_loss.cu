// Token-level RL objective math in one pass over [B, T] (replaces a chain of ~25 elementwise XLA ops per
// micro-batch in tunix/rl/algo_core.py:400-763 and tunix/rl/common.py:145-204), and the GAE reverse scan
// (tunix/rl/algo_core.py:33-110).
//
//  policy_loss : per token, from the new / old / reference log-probabilities, the advantage, the mask and an
//                optional importance weight:
//                    r = exp(clamp(new - old, -20, 20))
//                    pg = max(-A r, -A clamp(r, 1 - eps_lo, 1 + eps_hi));  dual clip: A < 0 -> min(pg, -eps_c A)
//                    kl = new - ref | 0.5 (new - ref)^2 | exp(d) - d - 1 with d = clamp(ref - new, -20, 20)
//                and their derivatives with respect to `new`, which the autograd wrapper multiplies by the
//                aggregation weights. Inactive tokens (mask 0 or non-finite inputs) produce zeros.
//  gae_scan    : one thread per sequence walks the time axis backwards:
//                    delta_t = r_t + gamma V_{t+1} - V_t,  A_t = delta_t + gamma lambda A_{t+1}, returns = A + V
#include "common.cuh"

using namespace tb;

namespace {

__global__ void policy_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_logp,
                                   const float* __restrict__ ref_logp, const float* __restrict__ adv, int adv_per_token,
                                   const float* __restrict__ mask, const float* __restrict__ is_w, int B, int T,
                                   float eps_lo, float eps_hi, float eps_c, int kl_mode, float kl_clamp,
                                   float* __restrict__ pg, float* __restrict__ dpg, float* __restrict__ kl,
                                   float* __restrict__ dkl, float* __restrict__ flags) {
  const long long n = (long long)B * T;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float nw = logp[i];
    const float od = old_logp ? old_logp[i] : nw;
    const bool active = mask[i] > 0.f && isfinite(nw) && isfinite(od);
    float a = adv_per_token ? adv[i] : adv[i / T];
    if (!active || !isfinite(a)) a = 0.f;
    float p = 0.f, dp = 0.f, clipped = 0.f, lower = 0.f;
    if (active) {
      const float lr_raw = nw - od;
      const float lr = fminf(fmaxf(lr_raw, -20.f), 20.f);
      const float dlr = (lr_raw > -20.f && lr_raw < 20.f) ? 1.f : 0.f;
      const float r = __expf(lr);
      const float rc = fminf(fmaxf(r, 1.f - eps_lo), 1.f + eps_hi);
      const float l1 = -a * r, l2 = -a * rc;
      const bool use2 = l2 > l1;
      p = use2 ? l2 : l1;
      // d/d new: l1 -> -a r dlr; l2 -> -a r dlr when r is inside the clip range, else 0
      const bool inside = r > 1.f - eps_lo && r < 1.f + eps_hi;
      dp = use2 ? (inside ? -a * r * dlr : 0.f) : -a * r * dlr;
      clipped = use2 ? 1.f : 0.f;
      if (eps_c > 0.f && a < 0.f) {
        const float l3 = -eps_c * a;
        if (p > l3) {
          p = l3;
          dp = 0.f;
          lower = 1.f;
        }
      }
      if (is_w) {
        const float w = is_w[i];
        p *= w;
        dp *= w;
      }
    }
    pg[i] = p;
    dpg[i] = dp;
    if (flags) {
      flags[i] = clipped;
      flags[n + i] = lower;
    }
    if (kl) {
      float k = 0.f, dk = 0.f;
      if (active && ref_logp) {
        float nn = isnan(nw) ? -100.f : fminf(fmaxf(nw, -100.f), 100.f);
        const float rr_raw = ref_logp[i];
        const float rr = isnan(rr_raw) ? -100.f : fminf(fmaxf(rr_raw, -100.f), 100.f);
        const float dn = (nw > -100.f && nw < 100.f) ? 1.f : 0.f;
        if (kl_mode == 0) {
          k = nn - rr;
          dk = dn;
        } else if (kl_mode == 1) {
          k = 0.5f * (nn - rr) * (nn - rr);
          dk = (nn - rr) * dn;
        } else {
          const float d_raw = rr - nn;
          const float d = fminf(fmaxf(d_raw, -20.f), 20.f);
          const float dd = (d_raw > -20.f && d_raw < 20.f) ? -dn : 0.f;
          k = __expf(d) - d - 1.f;
          dk = (__expf(d) - 1.f) * dd;
        }
        if (kl_clamp > 0.f) {
          if (k > kl_clamp) { k = kl_clamp; dk = 0.f; }
          if (k < -kl_clamp) { k = -kl_clamp; dk = 0.f; }
        }
      }
      kl[i] = k;
      dkl[i] = dk;
    }
  }
}

__global__ void gae_scan_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                                const float* __restrict__ mask, int B, int T, float gamma, float lam,
                                float* __restrict__ advantages, float* __restrict__ returns) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float next_v = 0.f, run = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const long long i = (long long)b * T + t;
    const float m = mask ? mask[i] : 1.f;
    const float v = values[i];
    if (m > 0.f) {
      const float delta = rewards[i] + gamma * next_v - v;
      run = delta + gamma * lam * run;
      next_v = v;
    }
    // masked positions pass the running state through; the caller masks the advantages after whitening
    advantages[i] = run;
    returns[i] = run + v;
  }
}

}  // namespace

// All tensors fp32 [B, T] contiguous. old_logp / ref_logp / is_w / flags / kl may be null. adv is [B] (adv_per_token = 0)
// or [B, T]. eps_c <= 0 disables the dual clip, kl_clamp <= 0 the KL clamp. flags: [2, B, T] (clipped, clipped-lower).
TB_API int tb_policy_loss(const float* logp, const float* old_logp, const float* ref_logp, const float* adv,
                          int adv_per_token, const float* mask, const float* is_w, int B, int T, float eps_lo,
                          float eps_hi, float eps_c, int kl_mode, float kl_clamp, float* pg, float* dpg, float* kl,
                          float* dkl, float* flags, cudaStream_t stream) {
  const long long n = (long long)B * T;
  if (n <= 0) return 0;
  if (kl_mode < 0 || kl_mode > 2) return -2;
  int grid = (int)((n + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  policy_loss_kernel<<<grid, 256, 0, stream>>>(logp, old_logp, ref_logp, adv, adv_per_token, mask, is_w, B, T, eps_lo, eps_hi,
                                               eps_c, kl_mode, kl_clamp, pg, dpg, kl, dkl, flags);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_gae_scan(const float* rewards, const float* values, const float* mask, int B, int T, float gamma, float lam,
                       float* advantages, float* returns, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  gae_scan_kernel<<<(B + 63) / 64, 64, 0, stream>>>(rewards, values, mask, B, T, gamma, lam, advantages, returns);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
