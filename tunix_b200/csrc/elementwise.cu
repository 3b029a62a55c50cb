// Memory-bound transformer ops for sm_100a: RMSNorm, RoPE, gated activations, embedding.
// All tensors bf16 with fp32 math; 16-byte vector accesses; one warp per row for the
// row-wise ops so a row's two passes stay in L1/L2.
//
// Replaces the XLA elementwise fusions of the reference models
// (RMSNorm: tunix/models/llama3/model.py:290-297, gemma (1+w): tunix/models/gemma/model.py:730-740,
//  RoPE: tunix/models/llama3/model.py:249-270, SwiGLU/GeGLU: llama3/model.py:489-496, gemma/model.py:592-601).
#include "common.cuh"

using namespace tb;

namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = bf16_lo(w[j]);
    v[2 * j + 1] = bf16_hi(w[j]);
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]);
  o.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// ------------------------------------------------------------------ RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * (w + add_one). D % 8 == 0. One warp per row.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                   const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, long long ldy,
                                   float* __restrict__ rstd_out, int rows, int D, float eps,
                                   float add_one) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const __nv_bfloat16* xr = x + row * ldx;
    float ss = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8];
      load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    __nv_bfloat16* yr = y + row * ldy;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8], g[8];
      load8(xr + c, v);
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * (g[i] + add_one);
      store8(yr + c, v);
    }
  }
}

// Same, one CTA per row: with few rows (decode) the warp-per-row kernel is a handful of warps each walking a
// whole row twice, and latency, not bandwidth, sets its time. The row is held in registers between the passes.
template <int VPT>   // 8-element vectors per thread
__global__ void __launch_bounds__(128)
rmsnorm_fwd_row_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, long long ldy, float* __restrict__ rstd_out, int D, float eps,
                       float add_one) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ldx;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c = (threadIdx.x + j * 128) * 8;
    if (c < D) {
      load8(xr + c, v[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[j][i] * v[j][i];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)D + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  __nv_bfloat16* yr = y + row * ldy;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c = (threadIdx.x + j * 128) * 8;
    if (c < D) {
      float g[8];
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j][i] = v[j][i] * rstd * (g[i] + add_one);
      store8(yr + c, v[j]);
    }
  }
}

// dx = rstd * (dy*w' - xhat * mean(dy*w'*xhat)), xhat = x*rstd, w' = w + add_one.
// If accumulate != 0, dx += (used when the residual stream's gradient is folded in).
__global__ void rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy,
                                      const __nv_bfloat16* __restrict__ x, long long ldx,
                                      const __nv_bfloat16* __restrict__ w,
                                      const float* __restrict__ rstd_in,
                                      __nv_bfloat16* __restrict__ dx, long long lddx, int rows,
                                      int D, float add_one, int accumulate) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const __nv_bfloat16* xr = x + row * ldx;
    const __nv_bfloat16* dyr = dy + row * lddy;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8], g[8], d[8];
      load8(xr + c, v);
      load8(w + c, g);
      load8(dyr + c, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += d[i] * (g[i] + add_one) * v[i] * rstd;
    }
    dot = warp_sum(dot) / (float)D;
    __nv_bfloat16* dxr = dx + row * lddx;
    for (int c = lane * 8; c < D; c += 256) {
      float v[8], g[8], d[8], o[8];
      load8(xr + c, v);
      load8(w + c, g);
      load8(dyr + c, d);
      if (accumulate) load8(dxr + c, o);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float r = rstd * (d[i] * (g[i] + add_one) - v[i] * rstd * dot);
        o[i] = accumulate ? o[i] + r : r;
      }
      store8(dxr + c, o);
    }
  }
}

// dw[c] += sum_rows dy[r,c] * x[r,c] * rstd[r]   (fp32 atomics into a zeroed buffer)
__global__ void rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy,
                                      const __nv_bfloat16* __restrict__ x, long long ldx,
                                      const float* __restrict__ rstd_in, float* __restrict__ dw,
                                      int rows, int D) {
  __shared__ float red[4][128];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
  const int col = blockIdx.x * 128 + tx * 2;
  float a0 = 0.f, a1 = 0.f;
  if (col < D) {
    for (long long r = (long long)blockIdx.y * 4 + ty; r < rows; r += (long long)gridDim.y * 4) {
      uint32_t dv = *reinterpret_cast<const uint32_t*>(dy + r * lddy + col);
      uint32_t xv = *reinterpret_cast<const uint32_t*>(x + r * ldx + col);
      const float rs = rstd_in[r];
      a0 += bf16_lo(dv) * bf16_lo(xv) * rs;
      a1 += bf16_hi(dv) * bf16_hi(xv) * rs;
    }
  }
  red[ty][tx * 2] = a0;
  red[ty][tx * 2 + 1] = a1;
  __syncthreads();
  if (ty == 0 && col < D) {
    float s0 = red[0][tx * 2] + red[1][tx * 2] + red[2][tx * 2] + red[3][tx * 2];
    float s1 = red[0][tx * 2 + 1] + red[1][tx * 2 + 1] + red[2][tx * 2 + 1] + red[3][tx * 2 + 1];
    atomicAdd(dw + col, s0);
    atomicAdd(dw + col + 1, s1);
  }
}

// --------------------------------------------------------------------- RoPE
// In-place half-split rotation on x[tokens, heads, H] (row stride ld between tokens, heads
// contiguous). cos/sin tables are [max_pos, H/2] fp32; pos[token] selects the row.
// sign = +1 forward, -1 backward (the transpose of a rotation is the opposite rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, long long ld, const int* __restrict__ pos,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            long long tokens, int heads, int H, float sign) {
  const int half = H >> 1;
  const int pairs_per_token = heads * (half >> 1);  // each thread rotates 2 adjacent pairs
  const long long total = tokens * pairs_per_token;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long tok = i / pairs_per_token;
    const int rem = (int)(i - tok * pairs_per_token);
    const int h = rem / (half >> 1);
    const int j = (rem - h * (half >> 1)) * 2;
    const int p = pos[tok];
    const float2 c = *reinterpret_cast<const float2*>(cos_t + (long long)p * half + j);
    float2 s = *reinterpret_cast<const float2*>(sin_t + (long long)p * half + j);
    s.x *= sign;
    s.y *= sign;
    __nv_bfloat16* base = x + tok * ld + (long long)h * H;
    uint32_t lo = *reinterpret_cast<uint32_t*>(base + j);
    uint32_t hi = *reinterpret_cast<uint32_t*>(base + half + j);
    const float a0 = bf16_lo(lo), a1 = bf16_hi(lo), b0 = bf16_lo(hi), b1 = bf16_hi(hi);
    *reinterpret_cast<uint32_t*>(base + j) = pack_bf16(a0 * c.x - b0 * s.x, a1 * c.y - b1 * s.y);
    *reinterpret_cast<uint32_t*>(base + half + j) =
        pack_bf16(b0 * c.x + a0 * s.x, b1 * c.y + a1 * s.y);
  }
}

// ------------------------------------------------------------- gated activation
__device__ __forceinline__ float act_fwd(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));  // SiLU
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;  // tanh-approximate GELU
  return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
}
__device__ __forceinline__ float act_bwd(float g, int kind) {
  if (kind == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
}

// h = act(g) * u ; all [rows, F] with row strides. F % 8 == 0.
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ g, long long ldg,
                               const __nv_bfloat16* __restrict__ u, long long ldu,
                               __nv_bfloat16* __restrict__ h, long long ldh, long long rows, int F,
                               int kind) {
  pdl_trigger();
  pdl_wait();
  const int vec_per_row = F >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) << 3;
    float a[8], b[8];
    load8(g + r * ldg + c, a);
    load8(u + r * ldu + c, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = act_fwd(a[k], kind) * b[k];
    store8(h + r * ldh + c, a);
  }
}
// dg = dh * u * act'(g) ; du = dh * act(g). dg/du may alias g/u (in-place).
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, long long lddh,
                               const __nv_bfloat16* g, long long ldg, const __nv_bfloat16* u,
                               long long ldu, __nv_bfloat16* dg, long long lddg, __nv_bfloat16* du,
                               long long lddu, long long rows, int F, int kind) {
  const int vec_per_row = F >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) << 3;
    float a[8], b[8], d[8], og[8], ou[8];
    load8(g + r * ldg + c, a);
    load8(u + r * ldu + c, b);
    load8(dh + r * lddh + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      og[k] = d[k] * b[k] * act_bwd(a[k], kind);
      ou[k] = d[k] * act_fwd(a[k], kind);
    }
    store8(dg + r * lddg + c, og);
    store8(du + r * lddu + c, ou);
  }
}

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] * scale
__global__ void embedding_fwd_kernel(const int* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ table, long long ldt,
                                     __nv_bfloat16* __restrict__ out, long long ldo,
                                     long long tokens, int D, int vocab, float scale) {
  pdl_trigger();
  pdl_wait();
  const int vec_per_row = D >> 3;
  const long long total = tokens * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = (int)(i - t * vec_per_row) << 3;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    float v[8];
    load8(table + (long long)id * ldt + c, v);
    if (scale != 1.f) {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= scale;
    }
    store8(out + t * ldo + c, v);
  }
}
// dtable[ids[t], :] += dout[t, :] * scale  (bf16x2 atomics)
__global__ void embedding_bwd_kernel(const int* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dout, long long ldo,
                                     __nv_bfloat16* __restrict__ dtable, long long ldt,
                                     long long tokens, int D, int vocab, float scale) {
  const int pairs = D >> 1;
  const long long total = tokens * pairs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / pairs;
    const int c = (int)(i - t * pairs) << 1;
    const int id = ids[t];
    if (id < 0 || id >= vocab) continue;
    uint32_t d = *reinterpret_cast<const uint32_t*>(dout + t * ldo + c);
    __nv_bfloat162 v = __floats2bfloat162_rn(bf16_lo(d) * scale, bf16_hi(d) * scale);
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + (long long)id * ldt + c), v);
  }
}

// y = a + b (bf16), n % 8 == 0
__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* y,
                           long long n) {
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n;
       i += (long long)gridDim.x * blockDim.x * 8) {
    float x[8], z[8];
    load8(a + i, x);
    load8(b + i, z);
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] += z[k];
    store8(y + i, x);
  }
}

inline int grid_for(long long work_items, int block, int cap = 148 * 16) {
  long long g = (work_items + block - 1) / block;
  if (g < 1) g = 1;
  return (int)(g > cap ? cap : g);
}

}  // namespace

TB_API int tb_rmsnorm_fwd(const void* x, long long ldx, const void* w, void* y, long long ldy,
                          float* rstd, int rows, int D, float eps, float add_one,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8) return -2;
  if (rows <= 2048 && D >= 1024 && D <= 8192) {
    auto xx = (const __nv_bfloat16*)x;
    auto ww = (const __nv_bfloat16*)w;
    auto yy = (__nv_bfloat16*)y;
    cudaError_t e;
    if (D <= 2048) e = launch_pdl(rmsnorm_fwd_row_kernel<2>, dim3(rows), dim3(128), 0, stream, xx, ldx, ww, yy, ldy, rstd, D, eps, add_one);
    else if (D <= 4096) e = launch_pdl(rmsnorm_fwd_row_kernel<4>, dim3(rows), dim3(128), 0, stream, xx, ldx, ww, yy, ldy, rstd, D, eps, add_one);
    else e = launch_pdl(rmsnorm_fwd_row_kernel<8>, dim3(rows), dim3(128), 0, stream, xx, ldx, ww, yy, ldy, rstd, D, eps, add_one);
    return e == cudaSuccess ? 0 : -5;
  }
  const int block = 256;
  rmsnorm_fwd_kernel<<<grid_for((long long)rows * 32, block), block, 0, stream>>>(
      (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, ldy, rstd, rows, D,
      eps, add_one);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_rmsnorm_bwd(const void* dy, long long lddy, const void* x, long long ldx,
                          const void* w, const float* rstd, void* dx, long long lddx, float* dw,
                          int rows, int D, float add_one, int accumulate_dx, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8) return -2;
  const int block = 256;
  if (dx)
    rmsnorm_bwd_dx_kernel<<<grid_for((long long)rows * 32, block), block, 0, stream>>>(
        (const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, rstd,
        (__nv_bfloat16*)dx, lddx, rows, D, add_one, accumulate_dx);
  if (dw) {
    dim3 grid((D + 127) / 128, (unsigned)min(128, (rows + 3) / 4));
    rmsnorm_bwd_dw_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, lddy,
                                                    (const __nv_bfloat16*)x, ldx, rstd, dw, rows, D);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_rope(void* x, long long ld, const int* pos, const float* cos_t, const float* sin_t,
                   long long tokens, int heads, int H, int backward, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H % 4) return -2;
  const long long total = tokens * heads * (H / 4);
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>((__nv_bfloat16*)x, ld, pos, cos_t, sin_t,
                                                       tokens, heads, H, backward ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_glu_fwd(const void* g, long long ldg, const void* u, long long ldu, void* h,
                      long long ldh, long long rows, int F, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (F % 8) return -2;
  return launch_pdl(glu_fwd_kernel, dim3(grid_for(rows * (F / 8), 256)), dim3(256), 0, stream, (const __nv_bfloat16*)g, ldg,
                    (const __nv_bfloat16*)u, ldu, (__nv_bfloat16*)h, ldh, rows, F, kind) == cudaSuccess ? 0 : -5;
}

TB_API int tb_glu_bwd(const void* dh, long long lddh, const void* g, long long ldg, const void* u,
                      long long ldu, void* dg, long long lddg, void* du, long long lddu,
                      long long rows, int F, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (F % 8) return -2;
  glu_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)dh, lddh, (const __nv_bfloat16*)g, ldg, (const __nv_bfloat16*)u, ldu,
      (__nv_bfloat16*)dg, lddg, (__nv_bfloat16*)du, lddu, rows, F, kind);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_embedding_fwd(const int* ids, const void* table, long long ldt, void* out,
                            long long ldo, long long tokens, int D, int vocab, float scale,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (D % 8) return -2;
  return launch_pdl(embedding_fwd_kernel, dim3(grid_for(tokens * (D / 8), 256)), dim3(256), 0, stream, ids,
                    (const __nv_bfloat16*)table, ldt, (__nv_bfloat16*)out, ldo, tokens, D, vocab, scale) == cudaSuccess ? 0 : -5;
}

TB_API int tb_embedding_bwd(const int* ids, const void* dout, long long ldo, void* dtable,
                            long long ldt, long long tokens, int D, int vocab, float scale,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (D % 2) return -2;
  embedding_bwd_kernel<<<grid_for(tokens * (D / 2), 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)dout, ldo, (__nv_bfloat16*)dtable, ldt, tokens, D, vocab, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_add_bf16(const void* a, const void* b, void* y, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)a,
                                                       (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
