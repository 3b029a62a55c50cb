// Fused token sampling for the rollout engine: temperature, top-k, top-p, categorical draw and the
// chosen token's log-probability, one thread block per sequence, logits read straight from the lm_head
// output (fp32 [B, V]).
//
//  * softmax statistics by an online max/sum pass;
//  * top-k / top-p as probability thresholds found by bisection (count(p >= t) >= k, mass(p >= t) >= top_p):
//    no sort, no [B, V] scratch; each iteration re-reads the row, which stays in L2;
//  * the draw is Gumbel-max over the kept tokens with a counter-based Philox stream keyed by
//    (seed, step, row, token), so a sequence's randomness does not depend on batch composition;
//  * the final logit soft-cap (cap * tanh(z / cap), Gemma-2/3) and a list of forbidden token ids
//    (tunix/generate/sampler.py:84-85,407) are applied to the row in place by the first pass, so the
//    engine needs no [B, V] element-wise kernel in front of this one and the returned log-probability
//    is the one of the distribution that was sampled from.
//
// Replaces lax.top_k + softmax + cumsum mask + categorical of the reference (tunix/generate/sampler.py:112-168).
#include "common.cuh"

using namespace tb;

namespace {

__device__ __forceinline__ uint32_t mulhilo(uint32_t a, uint32_t b, uint32_t& hi) {
  const unsigned long long p = (unsigned long long)a * b;
  hi = (uint32_t)(p >> 32);
  return (uint32_t)p;
}
// Philox-4x32-10
__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, hi1;
    const uint32_t lo0 = mulhilo(0xD2511F53u, ctr.x, hi0);
    const uint32_t lo1 = mulhilo(0xCD9E8D57u, ctr.z, hi1);
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}
__device__ __forceinline__ float u01(uint32_t x) { return ((x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax amax(ArgMax a, ArgMax b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

__global__ void __launch_bounds__(1024)
sample_kernel(float* __restrict__ logits, long long ld, int V, float inv_temp, int top_k, float top_p,
              unsigned long long seed, int step_host, const int* __restrict__ step_dev, int greedy,
              long long* __restrict__ tokens, float* __restrict__ logprobs, float softcap,
              const int* __restrict__ forbidden, int n_forbidden) {
  pdl_trigger();
  pdl_wait();
  const int step = step_dev ? *step_dev : step_host;  // device-resident step keeps the launch graph-capturable
  __shared__ float red[33];
  __shared__ float s_a[32];
  __shared__ int s_i[32];
  const int row = blockIdx.x;
  float* z = logits + (long long)row * ld;
  const int tid = threadIdx.x, nt = blockDim.x;

  if (softcap > 0.f) {
    const float inv_cap = 1.f / softcap;
    for (int i = tid; i < V; i += nt) z[i] = softcap * tanhf(z[i] * inv_cap);
  }
  if (n_forbidden > 0) {
    __syncthreads();                                    // the capped values are in place before they are overwritten
    for (int j = tid; j < n_forbidden; j += nt) {
      const int t = forbidden[j];
      if (t >= 0 && t < V) z[t] = -INFINITY;
    }
  }
  if (softcap > 0.f || n_forbidden > 0) __syncthreads();

  const bool filtered = !greedy && ((top_k > 0 && top_k < V) || (top_p > 0.f && top_p < 1.f));
  if (!filtered) {
    // No top-k / top-p: one pass over the row. Every thread keeps a running (max, sum exp) pair and its best
    // Gumbel-perturbed score; the pairs are merged after the loop. The row is read once, four values per load.
    float lm = -INFINITY, ls = 0.f;
    ArgMax best{-INFINITY, 0x7fffffff};
    const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
    const bool vec = (reinterpret_cast<uintptr_t>(z) & 15) == 0;
    for (int i4 = tid * 4; i4 < V; i4 += nt * 4) {
      float zz[4];
      if (vec && i4 + 4 <= V) {
        const float4 q = *reinterpret_cast<const float4*>(z + i4);
        zz[0] = q.x; zz[1] = q.y; zz[2] = q.z; zz[3] = q.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) zz[j] = (i4 + j < V) ? z[i4 + j] : -INFINITY;
      }
      uint4 r = make_uint4(0, 0, 0, 0);
      if (!greedy) r = philox(make_uint4((uint32_t)(i4 >> 2), (uint32_t)row, (uint32_t)step, 0x5A17u), key);
      const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
      float cm = lm;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        zz[j] *= inv_temp;
        cm = fmaxf(cm, zz[j]);
      }
      if (cm > lm) {
        ls *= __expf(lm - cm);          // exp(-inf) = 0 on the first group
        lm = cm;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (i4 + j >= V) break;
        if (zz[j] > -INFINITY) ls += __expf(zz[j] - lm);      // a forbidden token (-inf) adds nothing
        const float score = greedy ? zz[j] : zz[j] - __logf(-__logf(u01(rr[j])));
        best = amax(best, ArgMax{score, i4 + j});
      }
    }
    const float m = block_max(lm, red);
    const float s = block_sum(lm == -INFINITY ? 0.f : ls * __expf(lm - m), red);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = amax(best, other);
    }
    if ((tid & 31) == 0) {
      s_a[tid >> 5] = best.v;
      s_i[tid >> 5] = best.i;
    }
    __syncthreads();
    if (tid < 32) {
      ArgMax b = (tid < (nt >> 5)) ? ArgMax{s_a[tid], s_i[tid]} : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = amax(b, other);
      }
      if (tid == 0) {
        const int tok = b.i < V ? b.i : 0;
        tokens[row] = tok;
        if (logprobs) logprobs[row] = z[tok] * inv_temp - m - logf(s);
      }
    }
    return;
  }

  float m = -INFINITY;
  for (int i = tid; i < V; i += nt) m = fmaxf(m, z[i] * inv_temp);
  m = block_max(m, red);
  float s = 0.f;
  for (int i = tid; i < V; i += nt) s += __expf(z[i] * inv_temp - m);
  s = block_sum(s, red);
  const float log_s = logf(s);

  // threshold on the unnormalised probability e_i = exp(z_i - m) in (0, 1]
  float thr = 0.f;
  float kept_mass = s;
  if (!greedy && top_k > 0 && top_k < V) {
    float lo = 0.f, hi = 1.f;  // count(e >= lo) >= k always; find the largest such lo
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = tid; i < V; i += nt) c += (__expf(z[i] * inv_temp - m) >= mid) ? 1.f : 0.f;
      c = block_sum(c, red);
      if (c >= (float)top_k) lo = mid; else hi = mid;
    }
    thr = lo;
    float km = 0.f;
    for (int i = tid; i < V; i += nt) {
      const float e = __expf(z[i] * inv_temp - m);
      km += (e >= thr) ? e : 0.f;
    }
    kept_mass = block_sum(km, red);
  }
  if (!greedy && top_p > 0.f && top_p < 1.f) {
    const float target = top_p * kept_mass;
    float lo = thr, hi = 1.f;   // mass(e >= lo) >= target; find the largest such lo
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = tid; i < V; i += nt) {
        const float e = __expf(z[i] * inv_temp - m);
        c += (e >= mid) ? e : 0.f;
      }
      c = block_sum(c, red);
      if (c >= target) lo = mid; else hi = mid;
    }
    thr = lo;
  }

  ArgMax best{-INFINITY, 0x7fffffff};
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  for (int i4 = tid * 4; i4 < V; i4 += nt * 4) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (!greedy) r = philox(make_uint4((uint32_t)(i4 >> 2), (uint32_t)row, (uint32_t)step, 0x5A17u), key);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i4 + j;
      if (i >= V) break;
      const float zi = z[i] * inv_temp;
      float score = zi;
      if (!greedy) {
        if (__expf(zi - m) < thr) continue;
        score = zi - __logf(-__logf(u01(rr[j])));
      }
      best = amax(best, ArgMax{score, i});
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = amax(best, other);
  }
  if ((tid & 31) == 0) {
    s_a[tid >> 5] = best.v;
    s_i[tid >> 5] = best.i;
  }
  __syncthreads();
  if (tid < 32) {
    ArgMax b = (tid < (nt >> 5)) ? ArgMax{s_a[tid], s_i[tid]} : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = amax(b, other);
    }
    if (tid == 0) {
      const int tok = b.i < V ? b.i : 0;
      tokens[row] = tok;
      if (logprobs) logprobs[row] = z[tok] * inv_temp - m - log_s;
    }
  }
}

}  // namespace

// logits fp32 [B, V] (row stride ld). tokens int64 [B]; logprobs fp32 [B] or null.
// temperature <= 0 selects greedy decoding. top_k <= 0 and top_p >= 1 disable the filters.
TB_API int tb_sample(const float* logits, long long ld, int B, int V, float temperature, int top_k, float top_p,
                     unsigned long long seed, int step, const int* step_dev, long long* tokens, float* logprobs,
                     cudaStream_t stream) {
  if (B <= 0) return 0;
  const int greedy = temperature <= 0.f;
  const float inv_temp = greedy ? 1.f : 1.f / temperature;
  return launch_pdl(sample_kernel, dim3(B), dim3(1024), 0, stream, const_cast<float*>(logits), ld, V, inv_temp, top_k, top_p,
                    seed, step, step_dev, greedy, tokens, logprobs, 0.f, (const int*)nullptr, 0) == cudaSuccess ? 0 : -5;
}

// The same with the final logit soft-cap and forbidden token ids applied inside the kernel. The logits row is
// MODIFIED in place (capped values, -inf at the forbidden ids): it is the caller's scratch.
// softcap <= 0 disables the cap; forbidden: device int32 [n_forbidden] or null.
TB_API int tb_sample_ex(float* logits, long long ld, int B, int V, float temperature, int top_k, float top_p,
                        unsigned long long seed, int step, const int* step_dev, long long* tokens, float* logprobs,
                        float softcap, const int* forbidden, int n_forbidden, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (n_forbidden < 0 || (n_forbidden > 0 && !forbidden)) return -2;
  const int greedy = temperature <= 0.f;
  const float inv_temp = greedy ? 1.f : 1.f / temperature;
  return launch_pdl(sample_kernel, dim3(B), dim3(1024), 0, stream, logits, ld, V, inv_temp, top_k, top_p, seed, step, step_dev,
                    greedy, tokens, logprobs, softcap, forbidden, n_forbidden) == cudaSuccess ? 0 : -5;
}
