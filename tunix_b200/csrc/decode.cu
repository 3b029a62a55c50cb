// Paged KV cache kernels for the rollout engine.
//
//  * kv_write      : scatter new K / V rows of a step (decode) or of a whole prompt (prefill) into the pages
//                    named by the page table; sequence ids and positions are read from device memory, so
//                    the launch is identical every step and can live in a CUDA graph.
//  * paged_decode  : single-query attention over a paged cache with GQA: one CTA per (sequence, kv head,
//                    context split). A warp streams 4 keys per iteration (8 lanes per key, 16 head dims per
//                    lane, 16-byte loads), keeps running max / sum per query head and accumulates P*V in
//                    registers; partial results of the splits are merged by `paged_decode_combine`.
//                    Sliding window and logit soft-cap supported. Memory-bound by construction: every K / V
//                    byte of the sequence is read exactly once per kv head.
//
// The reference keeps only host-side page-table logic (tunix/experimental/generate/*) and runs decode on a
// dense cache through XLA (tunix/generate/sampler.py:732-793); these kernels are the device side of the
// in-framework engine that replaces its vLLM / SGLang integrations.
#include "common.cuh"

using namespace tb;

namespace {

constexpr int MAX_G = 8;        // query heads per kv head handled by one CTA
constexpr int SPLIT_TOKENS = 256;

// k_new/v_new: [n_tok, KH*H] rows. seq_ids[n_tok] = row of page_table, pos[n_tok] = position in the sequence
// (negative = padding, skipped). Pools: [num_pages, page_size, KH*H].
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                long long ld_new, const int* __restrict__ seq_ids, const int* __restrict__ pos,
                                const int* __restrict__ page_table, int max_pages, int page_size,
                                __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                                int n_tok, int row_elems) {
  const int vec = row_elems >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n_tok * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec);
    const int c = (int)(i - (long long)t * vec) << 3;
    const int p = pos[t];
    if (p < 0) continue;
    const int page = page_table[(long long)seq_ids[t] * max_pages + p / page_size];
    if (page < 0) continue;
    const long long dst = ((long long)page * page_size + p % page_size) * row_elems + c;
    *reinterpret_cast<uint4*>(k_pool + dst) = *reinterpret_cast<const uint4*>(k_new + (long long)t * ld_new + c);
    *reinterpret_cast<uint4*>(v_pool + dst) = *reinterpret_cast<const uint4*>(v_new + (long long)t * ld_new + c);
  }
}

template <int H, int G>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long ldq,        // [B, N*H]
                    const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                    const int* __restrict__ page_table, int max_pages, int page_size,
                    const int* __restrict__ seq_ids, const int* __restrict__ seq_lens, int KH, float scale,
                    float softcap, int window, int num_splits, float* __restrict__ part_acc,  // [B, N, splits, H]
                    float* __restrict__ part_ml) {                                              // [B, N, splits, 2]
  constexpr int DPL = H / 8;                     // head dims per lane (8 lanes share a key)
  const int b = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, l8 = lane & 7;      // which of the 4 keys of this warp iteration; lane within the key
  const int N = KH * G;
  const int len = seq_lens[b];
  int lo = split * SPLIT_TOKENS, hi = min(len, lo + SPLIT_TOKENS);
  if (window > 0) lo = max(lo, len - window);
  const int* pt = page_table + (long long)seq_ids[b] * max_pages;
  const long long row = (long long)KH * H;

  float qf[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + (long long)b * ldq + (long long)(kh * G + g) * H + l8 * DPL;
#pragma unroll
    for (int d = 0; d < DPL; d += 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(qp + d);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        qf[g][d + 2 * j] = bf16_lo(w[j]) * scale;
        qf[g][d + 2 * j + 1] = bf16_hi(w[j]) * scale;
      }
    }
  }
  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;
  }
  for (int t0 = lo + warp * 4; t0 < hi; t0 += 16) {
    const int t = t0 + sub;
    const bool valid = t < hi;
    float kf[DPL], vf[DPL];
    if (valid) {
      const int page = pt[t / page_size];
      const long long off = ((long long)page * page_size + t % page_size) * row + (long long)kh * H + l8 * DPL;
#pragma unroll
      for (int d = 0; d < DPL; d += 8) {
        const uint4 ku = *reinterpret_cast<const uint4*>(k_pool + off + d);
        const uint4 vu = *reinterpret_cast<const uint4*>(v_pool + off + d);
        const uint32_t kw[4] = {ku.x, ku.y, ku.z, ku.w}, vw[4] = {vu.x, vu.y, vu.z, vu.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          kf[d + 2 * j] = bf16_lo(kw[j]);
          kf[d + 2 * j + 1] = bf16_hi(kw[j]);
          vf[d + 2 * j] = bf16_lo(vw[j]);
          vf[d + 2 * j + 1] = bf16_hi(vw[j]);
        }
      }
    } else {
#pragma unroll
      for (int d = 0; d < DPL; ++d) kf[d] = vf[d] = 0.f;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int d = 0; d < DPL; ++d) s += qf[g][d] * kf[d];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      if (!valid) s = -INFINITY;
      const float mn = fmaxf(m[g], s);
      const float corr = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn);
      const float p = (s == -INFINITY) ? 0.f : __expf(s - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[g][d] = acc[g][d] * corr + p * vf[d];
      m[g] = mn;
    }
  }
  // merge the 4 key groups of the warp, then the 4 warps through shared memory
  __shared__ float sm_m[4][MAX_G], sm_l[4][MAX_G];
  __shared__ float sm_acc[4][MAX_G][H];
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo_ = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float ca = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn);
      const float cb = (mo == -INFINITY) ? 0.f : __expf(mo - mn);
      l[g] = l[g] * ca + lo_ * cb;
#pragma unroll
      for (int d = 0; d < DPL; ++d) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][d], o);
        acc[g][d] = acc[g][d] * ca + ao * cb;
      }
      m[g] = mn;
    }
    if (sub == 0) {
      if (l8 == 0) {
        sm_m[warp][g] = m[g];
        sm_l[warp][g] = l[g];
      }
#pragma unroll
      for (int d = 0; d < DPL; ++d) sm_acc[warp][g][l8 * DPL + d] = acc[g][d];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * H; idx += blockDim.x) {
    const int g = idx / H, d = idx - g * H;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (sm_m[w][g] == -INFINITY) ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * c;
      aa += sm_acc[w][g][d] * c;
    }
    const long long o = (((long long)b * N + kh * G + g) * num_splits + split);
    part_acc[o * H + d] = aa;
    if (d == 0) {
      part_ml[o * 2] = mm;
      part_ml[o * 2 + 1] = ll;
    }
  }
}

// out[b, n, :] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)
__global__ void paged_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                            const int* __restrict__ seq_lens, int N, int H, int num_splits, int window,
                                            __nv_bfloat16* __restrict__ out, long long ldo) {
  const int b = blockIdx.x, n = blockIdx.y;
  const int len = seq_lens[b];
  const int used = min(num_splits, (len + SPLIT_TOKENS - 1) / SPLIT_TOKENS);
  const long long base = ((long long)b * N + n) * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < used; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < used; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) L += part_ml[(base + s) * 2 + 1] * __expf(ms - M);
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < used; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) a += part_acc[(base + s) * H + d] * __expf(ms - M);
    }
    out[(long long)b * ldo + (long long)n * H + d] = __float2bfloat16(a * inv);
  }
}

template <int H>
int launch_decode(int G, dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, long long ldq,
                  const __nv_bfloat16* kp, const __nv_bfloat16* vp, const int* pt, int max_pages, int page_size,
                  const int* seq_ids, const int* seq_lens, int KH, float scale, float softcap, int window, int splits,
                  float* pa, float* pml) {
#define LAUNCH(GV)                                                                                              \
  paged_decode_kernel<H, GV><<<grid, 128, 0, stream>>>(q, ldq, kp, vp, pt, max_pages, page_size, seq_ids,      \
                                                       seq_lens, KH, scale, softcap, window, splits, pa, pml); \
  return 0;
  switch (G) {
    case 1: LAUNCH(1)
    case 2: LAUNCH(2)
    case 4: LAUNCH(4)
    case 8: LAUNCH(8)
    default: return -2;
  }
#undef LAUNCH
}

}  // namespace

TB_API int tb_kv_write(const void* k_new, const void* v_new, long long ld_new, const int* seq_ids, const int* pos,
                       const int* page_table, int max_pages, int page_size, void* k_pool, void* v_pool, int n_tok,
                       int row_elems, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  if (row_elems % 8 || ld_new % 8) return -2;
  long long work = (long long)n_tok * (row_elems / 8);
  int grid = (int)((work + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  kv_write_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, ld_new, seq_ids,
                                            pos, page_table, max_pages, page_size, (__nv_bfloat16*)k_pool,
                                            (__nv_bfloat16*)v_pool, n_tok, row_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// q [B, N*H]; pools [num_pages, page_size, KH*H]; page_table [*, max_pages]; seq_ids [B]; seq_lens [B];
// workspace: part_acc fp32 [B*N*splits*H], part_ml fp32 [B*N*splits*2] with splits = ceil(max_ctx / 256).
TB_API int tb_paged_decode(const void* q, long long ldq, const void* k_pool, const void* v_pool,
                           const int* page_table, int max_pages, int page_size, const int* seq_ids,
                           const int* seq_lens, int B, int N, int KH, int H, int max_ctx, float scale, float softcap,
                           int window, float* part_acc, float* part_ml, void* out, long long ldo,
                           cudaStream_t stream) {
  if (B <= 0) return 0;
  if (KH <= 0 || N % KH || (ldq % 8)) return -2;
  const int G = N / KH;
  const int splits = (max_ctx + SPLIT_TOKENS - 1) / SPLIT_TOKENS;
  dim3 grid(B, KH, splits);
  int rc;
  auto qq = (const __nv_bfloat16*)q;
  auto kp = (const __nv_bfloat16*)k_pool;
  auto vp = (const __nv_bfloat16*)v_pool;
  switch (H) {
    case 64: rc = launch_decode<64>(G, grid, stream, qq, ldq, kp, vp, page_table, max_pages, page_size, seq_ids, seq_lens, KH, scale, softcap, window, splits, part_acc, part_ml); break;
    case 128: rc = launch_decode<128>(G, grid, stream, qq, ldq, kp, vp, page_table, max_pages, page_size, seq_ids, seq_lens, KH, scale, softcap, window, splits, part_acc, part_ml); break;
    case 256: rc = launch_decode<256>(G, grid, stream, qq, ldq, kp, vp, page_table, max_pages, page_size, seq_ids, seq_lens, KH, scale, softcap, window, splits, part_acc, part_ml); break;
    default: return -2;
  }
  if (rc) return rc;
  paged_decode_combine_kernel<<<dim3(B, N), 128, 0, stream>>>(part_acc, part_ml, seq_lens, N, H, splits, window,
                                                               (__nv_bfloat16*)out, ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
