// Vocabulary-sized reductions for the lm_head: log-softmax statistics, chosen-token
// log-probability, entropy, and the matching gradient w.r.t. the logits. They run on
// one row-chunk of logits at a time (the caller produces the chunk with the tcgen05 GEMM),
// so the [tokens, vocab] tensor is never resident as a whole.
//
// Replaces the full-logits log_softmax + one-hot / take_along_axis of the reference
// (tunix/sft/peft_trainer.py:1208-1227, tunix/rl/common.py:207-226, 1213-1300).
#include "common.cuh"

using namespace tb;

namespace {

// Transform applied to raw head outputs: optional tanh soft-cap, then 1/temperature.
__device__ __forceinline__ float z_of(float raw, float softcap, float inv_temp) {
  if (softcap > 0.f) raw = softcap * tanhf(raw / softcap);
  return raw * inv_temp;
}

struct Online {
  float m, s, sz;  // running max, sum exp(z-m), sum exp(z-m)*z
  __device__ __forceinline__ void add(float z) {
    if (z > m) {
      const float c = __expf(m - z);
      s = s * c + 1.f;
      sz = sz * c + z;
      m = z;
    } else {
      const float e = __expf(z - m);
      s += e;
      sz += e * z;
    }
  }
  __device__ __forceinline__ void merge(const Online& o) {
    const float nm = fmaxf(m, o.m);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);
    const float b = (o.m == -INFINITY) ? 0.f : __expf(o.m - nm);
    s = s * a + o.s * b;
    sz = sz * a + o.sz * b;
    m = nm;
  }
};

// One block per row. logits fp32 [rows, V] with row stride ld.
// Outputs (any may be null): logp[row] = z[target]-lse, lse[row], entropy[row].
// target < 0 or >= V yields logp = 0.
__global__ void __launch_bounds__(512)
logsoftmax_gather_kernel(const float* __restrict__ logits, long long ld,
                         const int* __restrict__ targets, float* __restrict__ logp,
                         float* __restrict__ lse_out, float* __restrict__ ent_out, int V,
                         float softcap, float inv_temp) {
  __shared__ float sm[3][16];
  const long long row = blockIdx.x;
  const float* zr = logits + row * ld;
  Online st{-INFINITY, 0.f, 0.f};
  const bool vec = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  if (vec) {
    const int V4 = V >> 2;
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
      const float4 q = reinterpret_cast<const float4*>(zr)[i];
      st.add(z_of(q.x, softcap, inv_temp));
      st.add(z_of(q.y, softcap, inv_temp));
      st.add(z_of(q.z, softcap, inv_temp));
      st.add(z_of(q.w, softcap, inv_temp));
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x)
      st.add(z_of(zr[i], softcap, inv_temp));
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) st.add(z_of(zr[i], softcap, inv_temp));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Online other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.sz = __shfl_xor_sync(0xffffffffu, st.sz, o);
    st.merge(other);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) {
    sm[0][w] = st.m;
    sm[1][w] = st.s;
    sm[2][w] = st.sz;
  }
  __syncthreads();
  if (w == 0) {
    Online t{-INFINITY, 0.f, 0.f};
    if (lane < nw) {
      t.m = sm[0][lane];
      t.s = sm[1][lane];
      t.sz = sm[2][lane];
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      Online other;
      other.m = __shfl_xor_sync(0xffffffffu, t.m, o);
      other.s = __shfl_xor_sync(0xffffffffu, t.s, o);
      other.sz = __shfl_xor_sync(0xffffffffu, t.sz, o);
      t.merge(other);
    }
    if (lane == 0) {
      const float lse = t.m + logf(t.s);
      if (lse_out) lse_out[row] = lse;
      if (ent_out) ent_out[row] = lse - t.sz / t.s;
      if (logp) {
        const int tg = targets[row];
        logp[row] = (tg >= 0 && tg < V) ? z_of(zr[tg], softcap, inv_temp) - lse : 0.f;
      }
    }
  }
}

// dlogits[row, j] (bf16) = d/d raw_j of ( dlogp*logp + dent*entropy ), with
//   d logp / dz_j = 1[j==t] - p_j ;  d entropy / dz_j = -p_j * (z_j - lse + entropy)
// chained through temperature and the optional soft-cap. grid = (col_blocks, rows).
__global__ void __launch_bounds__(256)
dlogits_kernel(const float* __restrict__ logits, long long ld, const int* __restrict__ targets,
               const float* __restrict__ lse_in, const float* __restrict__ ent_in,
               const float* __restrict__ dlogp, const float* __restrict__ dent,
               __nv_bfloat16* __restrict__ out, long long ldo, int V, float softcap,
               float inv_temp) {
  const long long row = blockIdx.y;
  const float* zr = logits + row * ld;
  __nv_bfloat16* orow = out + row * ldo;
  const float lse = lse_in[row];
  const float gl = dlogp ? dlogp[row] : 0.f;
  const float ge = dent ? dent[row] : 0.f;
  const float ent = (dent && ent_in) ? ent_in[row] : 0.f;
  int tg = targets ? targets[row] : -1;
  if (tg < 0 || tg >= V) tg = -1;
  const float gl_eff = (tg >= 0) ? gl : 0.f;
  const int start = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int stride = gridDim.x * blockDim.x * 4;
  const bool vec = ((ld & 3) == 0) && ((ldo & 3) == 0);
  for (int j0 = start; j0 < V; j0 += stride) {
    float r[4];
    if (vec && j0 + 4 <= V) {
      const float4 q = *reinterpret_cast<const float4*>(zr + j0);
      r[0] = q.x; r[1] = q.y; r[2] = q.z; r[3] = q.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) r[k] = (j0 + k < V) ? zr[j0 + k] : 0.f;
    }
    float g[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float raw = r[k], chain = inv_temp, capped = raw;
      if (softcap > 0.f) {
        const float t = tanhf(raw / softcap);
        capped = softcap * t;
        chain *= (1.f - t * t);
      }
      const float z = capped * inv_temp;
      const float p = __expf(z - lse);
      float d = gl_eff * (((j0 + k) == tg ? 1.f : 0.f) - p);
      if (ge != 0.f) d -= ge * p * (z - lse + ent);
      g[k] = d * chain;
    }
    if (vec && j0 + 4 <= V) {
      uint2 o;
      o.x = pack_bf16(g[0], g[1]);
      o.y = pack_bf16(g[2], g[3]);
      *reinterpret_cast<uint2*>(orow + j0) = o;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (j0 + k < V) orow[j0 + k] = __float2bfloat16(g[k]);
    }
  }
}

}  // namespace

TB_API int tb_logsoftmax_gather(const float* logits, long long ld, const int* targets, float* logp,
                                float* lse, float* entropy, int rows, int V, float softcap,
                                float temperature, cudaStream_t stream) {
  if (rows <= 0) return 0;
  logsoftmax_gather_kernel<<<rows, 512, 0, stream>>>(logits, ld, targets, logp, lse, entropy, V,
                                                    softcap, 1.f / temperature);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_dlogits(const float* logits, long long ld, const int* targets, const float* lse,
                      const float* entropy, const float* dlogp, const float* dent, void* out,
                      long long ldo, int rows, int V, float softcap, float temperature,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  int col_blocks = (V + 256 * 4 * 8 - 1) / (256 * 4 * 8);
  if (col_blocks < 1) col_blocks = 1;
  dim3 grid(col_blocks, rows);
  dlogits_kernel<<<grid, 256, 0, stream>>>(logits, ld, targets, lse, entropy, dlogp, dent,
                                           (__nv_bfloat16*)out, ldo, V, softcap,
                                           1.f / temperature);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
