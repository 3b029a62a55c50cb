// Optimizer-side kernels over flat parameter buffers: global grad-norm, fused AdamW with
// fp32 master weights (clip factor read from device memory, bf16 working copy written in the
// same pass), and dtype casts / scaling for gradient buckets.
//
// Replaces the optax update + clip_by_global_norm chain of the reference trainer
// (tunix/sft/peft_trainer.py:517-548, tunix/cli/config.py:286-378).
#include "common.cuh"

using namespace tb;

namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// out[0] += sum(g^2)
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[33];
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f<T>(g[i]);
    acc += v * v;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^t
  float grad_scale;     // multiplies every gradient (e.g. 1 / accumulated denominator)
  float max_norm;       // <= 0 disables clipping
  const float* sumsq;   // device scalar holding sum(g^2) of the *unscaled* grads (may be null)
  const float* denom;   // device scalar; when non-null grads are divided by max(*denom, 1e-8)
};

// AdamW as optax.adamw: p -= lr * (m_hat / (sqrt(v_hat) + eps) + wd * p).
// Clipping as optax.clip_by_global_norm: g *= max_norm / max(norm, max_norm).
template <typename G>
__device__ __forceinline__ void load4g(const G* g, long long i, float (&o)[4]);
template <>
__device__ __forceinline__ void load4g<float>(const float* g, long long i, float (&o)[4]) {
  const float4 q = *reinterpret_cast<const float4*>(g + i);
  o[0] = q.x; o[1] = q.y; o[2] = q.z; o[3] = q.w;
}
template <>
__device__ __forceinline__ void load4g<__nv_bfloat16>(const __nv_bfloat16* g, long long i, float (&o)[4]) {
  const uint2 q = *reinterpret_cast<const uint2*>(g + i);
  o[0] = bf16_lo(q.x); o[1] = bf16_hi(q.x); o[2] = bf16_lo(q.y); o[3] = bf16_hi(q.y);
}

// Four elements per thread with 16-byte accesses; buffers come from flat allocations, so every pointer is
// 16-byte aligned and only the last n % 4 elements take the scalar tail.
template <typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
             const G* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n, AdamArgs a) {
  float scale = a.grad_scale;
  if (a.denom) scale /= fmaxf(*a.denom, 1e-8f);
  if (a.max_norm > 0.f && a.sumsq) {
    const float norm = sqrtf(*a.sumsq) * fabsf(scale);
    scale *= a.max_norm / fmaxf(norm, a.max_norm);
  }
  const float ib1 = 1.f / a.bc1, ib2 = 1.f / a.bc2;
  const long long n4 = n >> 2;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < n4;
       q += (long long)gridDim.x * blockDim.x) {
    const long long i = q << 2;
    float gi[4];
    load4g<G>(g, i, gi);
    float4 mm = *reinterpret_cast<float4*>(m + i);
    float4 vv = *reinterpret_cast<float4*>(v + i);
    float4 pp = *reinterpret_cast<float4*>(p32 + i);
    float* mp = &mm.x; float* vp = &vv.x; float* p = &pp.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = gi[k] * scale;
      mp[k] = a.beta1 * mp[k] + (1.f - a.beta1) * gk;
      vp[k] = a.beta2 * vp[k] + (1.f - a.beta2) * gk * gk;
      const float upd = (mp[k] * ib1) / (sqrtf(vp[k] * ib2) + a.eps) + a.weight_decay * p[k];
      p[k] -= a.lr * upd;
    }
    *reinterpret_cast<float4*>(m + i) = mm;
    *reinterpret_cast<float4*>(v + i) = vv;
    *reinterpret_cast<float4*>(p32 + i) = pp;
    if (p16) {
      uint2 o;
      o.x = pack_bf16(p[0], p[1]);
      o.y = pack_bf16(p[2], p[3]);
      *reinterpret_cast<uint2*>(p16 + i) = o;
    }
  }
  // scalar tail
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gk = to_f<G>(g[i]) * scale;
    const float mi = a.beta1 * m[i] + (1.f - a.beta1) * gk;
    const float vi = a.beta2 * v[i] + (1.f - a.beta2) * gk * gk;
    m[i] = mi;
    v[i] = vi;
    float p = p32[i];
    p -= a.lr * ((mi * ib1) / (sqrtf(vi * ib2) + a.eps) + a.weight_decay * p);
    p32[i] = p;
    if (p16) p16[i] = __float2bfloat16(p);
  }
}

// SGD with optional momentum, same flat-buffer contract.
template <typename G>
__global__ void sgd_kernel(float* __restrict__ p32, float* __restrict__ mom,
                           const G* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n,
                           float lr, float momentum, float weight_decay, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float p = p32[i];
    float gi = to_f<G>(g[i]) * scale + weight_decay * p;
    if (mom) {
      gi = momentum * mom[i] + gi;
      mom[i] = gi;
    }
    p -= lr * gi;
    p32[i] = p;
    if (p16) p16[i] = __float2bfloat16(p);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                        long long n, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out,
                                        long long n, float scale, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(in[i]) * scale;
    out[i] = accumulate ? out[i] + v : v;
  }
}

inline int grid_for(long long n, int block) {
  long long g = (n + block - 1) / block;
  const long long cap = 148LL * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

TB_API int tb_sumsq(const void* g, long long n, int is_bf16, float* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (is_bf16)
    sumsq_kernel<__nv_bfloat16><<<grid_for(n, 512), 512, 0, stream>>>((const __nv_bfloat16*)g, n, out);
  else
    sumsq_kernel<float><<<grid_for(n, 512), 512, 0, stream>>>((const float*)g, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_adamw(float* p32, float* m, float* v, const void* g, int g_is_bf16, void* p16,
                    long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                    float bc1, float bc2, float grad_scale, float max_norm, const float* sumsq,
                    const float* denom, cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, max_norm, sumsq, denom};
  const uintptr_t align = reinterpret_cast<uintptr_t>(p32) | reinterpret_cast<uintptr_t>(m) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(g) |
                          (reinterpret_cast<uintptr_t>(p16) << 1);
  if (align & 15) return -2;  // flat buffers are always 16-byte aligned
  if (g_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid_for((n + 3) / 4, 256), 256, 0, stream>>>(
        p32, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)p16, n, a);
  else
    adamw_kernel<float><<<grid_for((n + 3) / 4, 256), 256, 0, stream>>>(p32, m, v, (const float*)g,
                                                              (__nv_bfloat16*)p16, n, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_sgd(float* p32, float* mom, const void* g, int g_is_bf16, void* p16, long long n,
                  float lr, float momentum, float weight_decay, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (g_is_bf16)
    sgd_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>(
        p32, mom, (const __nv_bfloat16*)g, (__nv_bfloat16*)p16, n, lr, momentum, weight_decay, scale);
  else
    sgd_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>(p32, mom, (const float*)g,
                                                            (__nv_bfloat16*)p16, n, lr, momentum,
                                                            weight_decay, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_cast_f32_bf16(const float* in, void* out, long long n, float scale,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>(in, (__nv_bfloat16*)out, n, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
TB_API int tb_cast_bf16_f32(const void* in, float* out, long long n, float scale, int accumulate,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, stream>>>((const __nv_bfloat16*)in, out, n,
                                                                scale, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// ------------------------------------------------------------------ NF4 dequantisation (QLoRA base weights)
// packed: two 4-bit codes per byte (high nibble first), absmax: one fp32 per `block` values. Writes bf16.
// One thread expands 8 bytes = 16 values and writes two 16-byte vectors; the 16-entry codebook sits in registers
// through a constant table. The frozen base weight is expanded once per use into a scratch tensor that the GEMM
// reads; nothing else of the 4-bit weight is ever materialised.
namespace {
__constant__ float kNf4Code[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                   -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                   0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                   0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

__global__ void nf4_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ absmax, int block,
                                   __nv_bfloat16* __restrict__ out, long long numel) {
  const long long n16 = (numel + 15) / 16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const long long base = i * 16;
    const uint2 bytes = *reinterpret_cast<const uint2*>(packed + i * 8);
    const uint32_t w[2] = {bytes.x, bytes.y};
    float v[16];
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t byte = (w[b >> 2] >> ((b & 3) * 8)) & 0xFFu;
      v[2 * b] = kNf4Code[byte >> 4];
      v[2 * b + 1] = kNf4Code[byte & 0xF];
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] *= absmax[(base + j) / block];
    if (base + 16 <= numel) {
      uint4 o0, o1;
      o0.x = pack_bf16(v[0], v[1]); o0.y = pack_bf16(v[2], v[3]); o0.z = pack_bf16(v[4], v[5]); o0.w = pack_bf16(v[6], v[7]);
      o1.x = pack_bf16(v[8], v[9]); o1.y = pack_bf16(v[10], v[11]); o1.z = pack_bf16(v[12], v[13]); o1.w = pack_bf16(v[14], v[15]);
      reinterpret_cast<uint4*>(out + base)[0] = o0;
      reinterpret_cast<uint4*>(out + base)[1] = o1;
    } else {
      for (int j = 0; j < 16 && base + j < numel; ++j) out[base + j] = __float2bfloat16(v[j]);
    }
  }
}
}  // namespace

// packed holds ceil(numel / 2) bytes padded to a multiple of 8; any block size works (absmax is looked up per value).
TB_API int tb_nf4_dequant(const void* packed, const float* absmax, int block, void* out, long long numel,
                          cudaStream_t stream) {
  if (numel <= 0) return 0;
  if (block <= 0 || (reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  const long long n16 = (numel + 15) / 16;
  int grid = (int)((n16 + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  nf4_dequant_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)packed, absmax, block, (__nv_bfloat16*)out, numel);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
