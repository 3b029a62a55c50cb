// Mixture-of-experts data movement and tile planning around the grouped tcgen05 GEMM (gemm.cu, TileDesc).
//
// Tokens routed to an expert occupy one contiguous row segment of a permuted buffer; segments start on
// multiples of 128 rows and are zero padded, so that a 128-row output tile never spans two experts and the
// weight-gradient contraction over a segment sees zeros in the padding. Everything below reads the routing
// from device memory: the host never learns the per-expert counts, so one training step has no host sync.
//
//   moe_zero_pad      : zero the padding rows of every segment
//   moe_scatter_rows  : dst[pos[t, j]] = scale[t, j] * src[t]          (dispatch; combine backward)
//   moe_gather_sum    : out[t] = sum_j w[t, j] * src[pos[t, j]] (+ res) (combine; dispatch backward with w = 1)
//   moe_dot_rows      : dw[t, j] = <a[t], b[pos[t, j]]>                 (gradient of the routing weights)
//   moe_pull_rows     : dst[r] = peer[src_rank[r]][src_row[r]]        (expert-parallel dispatch over NVLink, P2P loads)
//   moe_gather_sum_peer: out[t] = sum_j peer[dst_rank[t, j]][pos[t, j]] (expert-parallel combine, P2P loads)
//   moe_row_scale / moe_row_dot : per-row routing weight applied on the expert's side, and its gradient
//   moe_tiles_rows    : tile list for GEMMs whose output rows are the permuted rows (forward, dgrad)
//   moe_tiles_expert  : tile list for GEMMs with one output matrix per expert (wgrad), k range = the segment
//
// Replaces the sort / ragged_dot / unsort path of the reference's sparse MoE block
// (tunix/models/qwen3/model.py:941-1149).
#include "common.cuh"

using namespace tb;

namespace {

struct TileDesc {          // must match gemm.cu
  int m0, n0, m_end, kb0, kb1, b_row0;
  long long c_off;
};

__global__ void moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, long long ld, const int* __restrict__ seg_off,
                                    const int* __restrict__ counts, int E, int D) {
  const int e = blockIdx.x;
  const int first = seg_off[e] + counts[e], last = seg_off[e + 1];
  const int vec = D >> 3;
  for (long long i = threadIdx.x + (long long)blockIdx.y * blockDim.x; i < (long long)(last - first) * vec;
       i += (long long)blockDim.x * gridDim.y) {
    const int r = (int)(i / vec), c = (int)(i - (long long)r * vec) << 3;
    *reinterpret_cast<uint4*>(buf + (long long)(first + r) * ld + c) = make_uint4(0, 0, 0, 0);
  }
}

// one warp per (token, slot)
__global__ void moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                        const int* __restrict__ pos, const float* __restrict__ scale,
                                        __nv_bfloat16* __restrict__ dst, long long ldd, long long n_slots, int k, int D) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_slots) return;
  const int lane = threadIdx.x & 31;
  const int p = pos[w];
  if (p < 0) return;
  const __nv_bfloat16* s = src + (w / k) * lds;
  __nv_bfloat16* d = dst + (long long)p * ldd;
  if (scale == nullptr) {
    for (int c = lane * 8; c < D; c += 256) *reinterpret_cast<uint4*>(d + c) = *reinterpret_cast<const uint4*>(s + c);
  } else {
    const float f = scale[w];
    for (int c = lane * 8; c < D; c += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(s + c);
      const uint32_t in[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = pack_bf16(bf16_lo(in[j]) * f, bf16_hi(in[j]) * f);
      *reinterpret_cast<uint4*>(d + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// one CTA of 128 threads per token; D % 8 == 0
__global__ void __launch_bounds__(128)
moe_gather_sum_kernel(const __nv_bfloat16* __restrict__ src, long long lds, const int* __restrict__ pos,
                      const float* __restrict__ wts, const __nv_bfloat16* __restrict__ res, long long ldr,
                      __nv_bfloat16* __restrict__ out, long long ldo, int k, int D) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < D; c += 128 * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (res != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(res + t * ldr + c);
      const uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = bf16_lo(in[j]);
        acc[2 * j + 1] = bf16_hi(in[j]);
      }
    }
    for (int j = 0; j < k; ++j) {
      const int p = pos[t * k + j];
      if (p < 0) continue;
      const float f = wts ? wts[t * k + j] : 1.f;
      const uint4 u = *reinterpret_cast<const uint4*>(src + (long long)p * lds + c);
      const uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += f * bf16_lo(in[q]);
        acc[2 * q + 1] += f * bf16_hi(in[q]);
      }
    }
    *reinterpret_cast<uint4*>(out + t * ldo + c) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

// one warp per (token, slot)
__global__ void moe_dot_rows_kernel(const __nv_bfloat16* __restrict__ a, long long lda,
                                    const __nv_bfloat16* __restrict__ b, long long ldb, const int* __restrict__ pos,
                                    float* __restrict__ out, long long n_slots, int k, int D) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_slots) return;
  const int lane = threadIdx.x & 31;
  const int p = pos[w];
  float s = 0.f;
  if (p >= 0) {
    const __nv_bfloat16* ar = a + (w / k) * lda;
    const __nv_bfloat16* br = b + (long long)p * ldb;
    for (int c = lane * 8; c < D; c += 256) {
      const uint4 ua = *reinterpret_cast<const uint4*>(ar + c), ub = *reinterpret_cast<const uint4*>(br + c);
      const uint32_t x[4] = {ua.x, ua.y, ua.z, ua.w}, y[4] = {ub.x, ub.y, ub.z, ub.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) s += bf16_lo(x[j]) * bf16_lo(y[j]) + bf16_hi(x[j]) * bf16_hi(y[j]);
    }
  }
  s = warp_sum(s);
  if (lane == 0) out[w] = s;
}

constexpr int MAX_RANKS = 8;
struct PeerPtrs {
  const void* p[MAX_RANKS];
};

// one warp per destination row; rows whose source rank is negative are left alone
__global__ void moe_pull_rows_kernel(PeerPtrs src, long long lds, const int* __restrict__ src_rank,
                                     const int* __restrict__ src_row, __nv_bfloat16* __restrict__ dst, long long ldd,
                                     long long n_rows, int D) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const int r = src_rank[w];
  if (r < 0) return;
  const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + (long long)src_row[w] * lds;
  __nv_bfloat16* d = dst + w * ldd;
  for (int c = lane * 8; c < D; c += 256) *reinterpret_cast<uint4*>(d + c) = *reinterpret_cast<const uint4*>(s + c);
}

__global__ void __launch_bounds__(128)
moe_gather_sum_peer_kernel(PeerPtrs src, long long lds, const int* __restrict__ dst_rank, const int* __restrict__ pos,
                           const __nv_bfloat16* __restrict__ res, long long ldr, __nv_bfloat16* __restrict__ out,
                           long long ldo, int k, int D) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < D; c += 128 * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (res != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(res + t * ldr + c);
      const uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = bf16_lo(in[j]);
        acc[2 * j + 1] = bf16_hi(in[j]);
      }
    }
    for (int j = 0; j < k; ++j) {
      const int r = dst_rank[t * k + j];
      if (r < 0) continue;
      const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + (long long)pos[t * k + j] * lds;
      const uint4 u = *reinterpret_cast<const uint4*>(row + c);
      const uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += bf16_lo(in[q]);
        acc[2 * q + 1] += bf16_hi(in[q]);
      }
    }
    *reinterpret_cast<uint4*>(out + t * ldo + c) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

// one warp per row: buf[r] *= scale[r] (out of place when dst != buf)
__global__ void moe_row_scale_kernel(const __nv_bfloat16* __restrict__ src, long long lds, const float* __restrict__ scale,
                                     __nv_bfloat16* __restrict__ dst, long long ldd, long long n_rows, int D) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const float f = scale[w];
  for (int c = lane * 8; c < D; c += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(src + w * lds + c);
    const uint32_t in[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16(bf16_lo(in[j]) * f, bf16_hi(in[j]) * f);
    *reinterpret_cast<uint4*>(dst + w * ldd + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// one warp per row: out[r] = <a[r], b[r]>
__global__ void moe_row_dot_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const __nv_bfloat16* __restrict__ b,
                                   long long ldb, float* __restrict__ out, long long n_rows, int D) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    const uint4 ua = *reinterpret_cast<const uint4*>(a + w * lda + c), ub = *reinterpret_cast<const uint4*>(b + w * ldb + c);
    const uint32_t x[4] = {ua.x, ua.y, ua.z, ua.w}, y[4] = {ub.x, ub.y, ub.z, ub.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) s += bf16_lo(x[j]) * bf16_lo(y[j]) + bf16_hi(x[j]) * bf16_hi(y[j]);
  }
  s = warp_sum(s);
  if (lane == 0) out[w] = s;
}

// single CTA: tiles [expert][m tile of its segment][n tile]
__global__ void moe_tiles_rows_kernel(const int* __restrict__ seg_off, int E, int num_n, int bn, int kblocks,
                                      int b_rows_per_expert, TileDesc* __restrict__ tiles, int* __restrict__ num_tiles) {
  __shared__ int base[1025];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      base[e] = acc;
      acc += ((seg_off[e + 1] - seg_off[e]) >> 7) * num_n;
    }
    base[E] = acc;
    *num_tiles = acc;
  }
  __syncthreads();
  for (int e = 0; e < E; ++e) {
    const int n = base[e + 1] - base[e];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int mt = i / num_n, nt = i - mt * num_n;
      TileDesc d;
      d.m0 = seg_off[e] + mt * 128;
      d.n0 = nt * bn;
      d.m_end = d.m0 + 128;
      d.kb0 = 0;
      d.kb1 = kblocks;
      d.b_row0 = e * b_rows_per_expert;
      d.c_off = 0;
      tiles[base[e] + i] = d;
    }
  }
}

// tiles [expert][m tile][n tile] of a per-expert [M, N] output, contraction over the expert's row segment
__global__ void moe_tiles_expert_kernel(const int* __restrict__ seg_off, int E, int M, int num_m, int num_n, int bn,
                                        long long c_stride, TileDesc* __restrict__ tiles, int* __restrict__ num_tiles) {
  const int per = num_m * num_n;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < E * per; i += gridDim.x * blockDim.x) {
    const int e = i / per, r = i - e * per;
    const int mt = r / num_n, nt = r - mt * num_n;
    TileDesc d;
    d.m0 = mt * 128;
    d.n0 = nt * bn;
    d.m_end = M;
    d.kb0 = seg_off[e] >> 6;
    d.kb1 = seg_off[e + 1] >> 6;
    d.b_row0 = 0;
    d.c_off = (long long)e * c_stride;
    tiles[i] = d;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *num_tiles = E * per;
}

}  // namespace

TB_API int tb_moe_zero_pad(void* buf, long long ld, const int* seg_off, const int* counts, int E, int D,
                           cudaStream_t stream) {
  if (E <= 0) return 0;
  if (D % 8 || ld % 8) return -2;
  moe_zero_pad_kernel<<<dim3(E, 2), 256, 0, stream>>>((__nv_bfloat16*)buf, ld, seg_off, counts, E, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_scatter_rows(const void* src, long long lds, const int* pos, const float* scale, void* dst,
                               long long ldd, long long n_tokens, int k, int D, cudaStream_t stream) {
  const long long n = n_tokens * k;
  if (n <= 0) return 0;
  if (D % 8 || lds % 8 || ldd % 8) return -2;
  moe_scatter_rows_kernel<<<(unsigned)((n + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)src, lds, pos, scale,
                                                                        (__nv_bfloat16*)dst, ldd, n, k, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_gather_sum(const void* src, long long lds, const int* pos, const float* wts, const void* res,
                             long long ldr, void* out, long long ldo, long long n_tokens, int k, int D,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (D % 8 || lds % 8 || ldo % 8 || (res && ldr % 8)) return -2;
  moe_gather_sum_kernel<<<(unsigned)n_tokens, 128, 0, stream>>>((const __nv_bfloat16*)src, lds, pos, wts,
                                                                (const __nv_bfloat16*)res, ldr, (__nv_bfloat16*)out,
                                                                ldo, k, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_dot_rows(const void* a, long long lda, const void* b, long long ldb, const int* pos, float* out,
                           long long n_tokens, int k, int D, cudaStream_t stream) {
  const long long n = n_tokens * k;
  if (n <= 0) return 0;
  if (D % 8 || lda % 8 || ldb % 8) return -2;
  moe_dot_rows_kernel<<<(unsigned)((n + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)a, lda,
                                                                    (const __nv_bfloat16*)b, ldb, pos, out, n, k, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

static PeerPtrs make_peer_ptrs(const void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

// dst[r, :D] = peer[src_rank[r]][src_row[r], :D]; src_ptrs: `world` device pointers (host array), row stride lds.
TB_API int tb_moe_pull_rows(const void* const* src_ptrs, int world, long long lds, const int* src_rank,
                            const int* src_row, void* dst, long long ldd, long long n_rows, int D, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || D % 8 || lds % 8 || ldd % 8) return -2;
  moe_pull_rows_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, stream>>>(make_peer_ptrs(src_ptrs, world), lds, src_rank,
                                                                          src_row, (__nv_bfloat16*)dst, ldd, n_rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_gather_sum_peer(const void* const* src_ptrs, int world, long long lds, const int* dst_rank,
                                  const int* pos, const void* res, long long ldr, void* out, long long ldo,
                                  long long n_tokens, int k, int D, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || D % 8 || lds % 8 || ldo % 8 || (res && ldr % 8)) return -2;
  moe_gather_sum_peer_kernel<<<(unsigned)n_tokens, 128, 0, stream>>>(make_peer_ptrs(src_ptrs, world), lds, dst_rank, pos,
                                                                     (const __nv_bfloat16*)res, ldr, (__nv_bfloat16*)out,
                                                                     ldo, k, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_row_scale(const void* src, long long lds, const float* scale, void* dst, long long ldd,
                            long long n_rows, int D, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (D % 8 || lds % 8 || ldd % 8) return -2;
  moe_row_scale_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)src, lds, scale,
                                                                          (__nv_bfloat16*)dst, ldd, n_rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_row_dot(const void* a, long long lda, const void* b, long long ldb, float* out, long long n_rows,
                          int D, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (D % 8 || lda % 8 || ldb % 8) return -2;
  moe_row_dot_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)a, lda,
                                                                        (const __nv_bfloat16*)b, ldb, out, n_rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// seg_off int32 [E + 1], multiples of 128. tiles: room for (seg_off[E] / 128) * num_n descriptors of 32 bytes.
TB_API int tb_moe_tiles_rows(const int* seg_off, int E, int num_n, int bn, int kblocks, int b_rows_per_expert,
                             void* tiles, int* num_tiles, cudaStream_t stream) {
  if (E <= 0 || E > 1024) return -2;
  moe_tiles_rows_kernel<<<1, 1024, 0, stream>>>(seg_off, E, num_n, bn, kblocks, b_rows_per_expert,
                                                reinterpret_cast<TileDesc*>(tiles), num_tiles);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_moe_tiles_expert(const int* seg_off, int E, int M, int N, int bn, long long c_stride, void* tiles,
                               int* num_tiles, cudaStream_t stream) {
  if (E <= 0) return -2;
  const int num_m = (M + 127) / 128, num_n = (N + bn - 1) / bn;
  const int total = E * num_m * num_n;
  moe_tiles_expert_kernel<<<(total + 255) / 256, 256, 0, stream>>>(seg_off, E, M, num_m, num_n, bn, c_stride,
                                                                   reinterpret_cast<TileDesc*>(tiles), num_tiles);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
