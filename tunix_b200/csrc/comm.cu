// Collective kernels over peer memory (NVLink 5 / NVSwitch), used by the sharded optimizer.
//
// Every rank maps every peer's symmetric buffers; kernels receive the table of peer base
// pointers by value and move data with plain 16-byte peer loads (P2P). No TMA multicast, no
// multimem in this file, so a rank that disappears cannot fault its peers.
//
//  * symm_barrier       : flag barrier across ranks with a bounded wait (status word on expiry)
//  * reduce_scatter_pull: out32[shard] = scale * sum_p grad_p[shard]  + sum of squares, in one pass
//                         (gradient reduce-scatter fused with cast/scale and the grad-norm partial)
//  * allgather_pull     : full_params[all shards] = peers' updated bf16 shards
//  * pull_blocks        : dst block = a peer's block, for a table of 2-D blocks (trainer -> rollout weight reshard)
//
// Parameters are sharded per tensor along dim 0: a tensor of `len` elements at `full_off` in the
// flat buffer is owned in W contiguous pieces of `rank_stride = len / W`; rank r keeps piece r at
// `shard_off` of its local shard buffers. Work is described by a chunk table built on the host.
//
// Replaces the GSPMD-inserted reduce-scatter / all-gather of the reference's FSDP sharding
// (tunix/models/llama3/model.py:65-82, tunix/sft/peft_trainer.py:609-650).
#include "common.cuh"

using namespace tb;

namespace {

constexpr int MAX_RANKS = 8;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

struct Chunk {
  long long full_off;     // element offset of this chunk inside piece 0 of the tensor (flat full buffer)
  long long shard_off;    // element offset inside a rank's shard buffer
  long long rank_stride;  // elements between the pieces of consecutive ranks
  int len;                // elements in this chunk (multiple of 8)
  int pad;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// flags[r] points at rank r's flag words; slot s uses words [s*world, (s+1)*world).
__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int slot, unsigned epoch,
                                    long long timeout_ns, int* status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<unsigned*>(flags.p[p]) + slot * world + rank, epoch);
  const unsigned* mine = reinterpret_cast<const unsigned*>(flags.p[rank]) + slot * world + p;
  const unsigned long long t0 = globaltimer_ns();
  while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
    if ((long long)(globaltimer_ns() - t0) > timeout_ns) {
      if (status) {
        atomicCAS(status, 0, ST_TIMEOUT_FLAG);
        status[1] = p;                 // the peer that never arrived
        status[2] = (int)epoch;
      }
      break;
    }
    __nanosleep(200);
  }
}

template <typename G>
__device__ __forceinline__ void load8f(const G* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8f<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = bf16_lo(w[j]);
    v[2 * j + 1] = bf16_hi(w[j]);
  }
}
template <>
__device__ __forceinline__ void load8f<float>(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0];
  const float4 b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename G>
__global__ void __launch_bounds__(512)
reduce_scatter_pull_kernel(PeerPtrs grads, const Chunk* __restrict__ chunks, int nchunks, int rank,
                           int world, float* __restrict__ out32, float scale, float* __restrict__ sumsq) {
  __shared__ float red[33];
  float ss = 0.f;
  for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const Chunk ch = chunks[c];
    const long long base = ch.full_off + (long long)rank * ch.rank_stride;
    for (int i = threadIdx.x * 8; i < ch.len; i += blockDim.x * 8) {
      float v[MAX_RANKS][8];
#pragma unroll
      for (int pp = 0; pp < MAX_RANKS; ++pp) {
        if (pp < world) {
          const int p = (rank + pp) % world;  // local piece first, peers rotated to spread load
          load8f<G>(reinterpret_cast<const G*>(grads.p[p]) + base + i, v[pp]);
        }
      }
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
      for (int pp = 0; pp < MAX_RANKS; ++pp) {
        if (pp < world) {
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += v[pp][k];
        }
      }
      float4 o0, o1;
      o0.x = acc[0] * scale; o0.y = acc[1] * scale; o0.z = acc[2] * scale; o0.w = acc[3] * scale;
      o1.x = acc[4] * scale; o1.y = acc[5] * scale; o1.z = acc[6] * scale; o1.w = acc[7] * scale;
      float* dst = out32 + ch.shard_off + i;
      reinterpret_cast<float4*>(dst)[0] = o0;
      reinterpret_cast<float4*>(dst)[1] = o1;
      ss += o0.x * o0.x + o0.y * o0.y + o0.z * o0.z + o0.w * o0.w + o1.x * o1.x + o1.y * o1.y +
            o1.z * o1.z + o1.w * o1.w;
    }
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0 && sumsq) atomicAdd(sumsq, ss);
}

// full[full_off + p*rank_stride + i] = shard_p[shard_off + i] for every rank p (bf16).
__global__ void __launch_bounds__(512)
allgather_pull_kernel(PeerPtrs shards, const Chunk* __restrict__ chunks, int nchunks, int rank, int world,
                      __nv_bfloat16* __restrict__ full) {
  const int total = nchunks * world;
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
    const int c = w / world;
    const int p = (rank + 1 + w % world) % world;  // peers first, own piece last
    const Chunk ch = chunks[c];
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(shards.p[p]) + ch.shard_off;
    __nv_bfloat16* dst = full + ch.full_off + (long long)p * ch.rank_stride;
    for (int i = threadIdx.x * 8; i < ch.len; i += blockDim.x * 8)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  }
}

// shard32[shard_off + i] = float(full[full_off + rank*rank_stride + i])  (initial master weights)
__global__ void gather_shard_kernel(const __nv_bfloat16* __restrict__ full, const Chunk* __restrict__ chunks,
                                    int nchunks, int rank, float* __restrict__ shard32,
                                    __nv_bfloat16* __restrict__ shard16) {
  for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const Chunk ch = chunks[c];
    const __nv_bfloat16* src = full + ch.full_off + (long long)rank * ch.rank_stride;
    for (int i = threadIdx.x; i < ch.len; i += blockDim.x) {
      const __nv_bfloat16 v = src[i];
      if (shard32) shard32[ch.shard_off + i] = __bfloat162float(v);
      if (shard16) shard16[ch.shard_off + i] = v;
    }
  }
}

// One 2-D block of a weight transfer: `rows` runs of `cols` bf16 elements (cols % 8 == 0), read from rank
// `src_rank`'s staging buffer at element offset src_off (row stride src_ld) and written to the local
// destination at dst_off (row stride dst_ld). A contiguous slice is a block with one row.
struct Block2D {
  long long src_off, dst_off, src_ld, dst_ld;
  int src_rank, rows, cols, pad;
};

__global__ void __launch_bounds__(512)
pull_blocks_kernel(PeerPtrs src, const Block2D* __restrict__ blocks, int nblocks, __nv_bfloat16* __restrict__ dst) {
  // the whole grid walks every block: NVLink latency is covered by the bytes in flight (4 vectors per thread)
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int b = 0; b < nblocks; ++b) {
    const Block2D bl = blocks[b];
    const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[bl.src_rank]) + bl.src_off;
    __nv_bfloat16* d = dst + bl.dst_off;
    const int vpr = bl.cols >> 3;
    const long long total = (long long)bl.rows * vpr;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long i = i0 + j * stride;
        if (i < total) {
          const long long r = i / vpr;
          v[j] = *reinterpret_cast<const uint4*>(s + r * bl.src_ld + ((int)(i - r * vpr) << 3));
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long i = i0 + j * stride;
        if (i < total) {
          const long long r = i / vpr;
          *reinterpret_cast<uint4*>(d + r * bl.dst_ld + ((int)(i - r * vpr) << 3)) = v[j];
        }
      }
    }
  }
}

PeerPtrs make_ptrs(const void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}

}  // namespace

// flag_ptrs: host array of `world` device pointers (uint32 words, zero-initialised, symmetric).
TB_API int tb_symm_barrier(const void* const* flag_ptrs, int rank, int world, int slot, unsigned epoch,
                           long long timeout_ms, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -2;
  symm_barrier_kernel<<<1, 32, 0, stream>>>(make_ptrs(flag_ptrs, world), rank, world, slot, epoch,
                                            timeout_ms * 1000000LL, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_reduce_scatter_pull(const void* const* grad_ptrs, int grads_are_bf16, const void* chunks,
                                  int nchunks, int rank, int world, float* out32, float scale, float* sumsq,
                                  int max_ctas, cudaStream_t stream) {
  if (nchunks <= 0) return 0;
  if (world < 1 || world > MAX_RANKS) return -2;
  int grid = nchunks < 148 * 2 ? nchunks : 148 * 2;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  PeerPtrs pp = make_ptrs(grad_ptrs, world);
  if (grads_are_bf16)
    reduce_scatter_pull_kernel<__nv_bfloat16><<<grid, 512, 0, stream>>>(
        pp, reinterpret_cast<const Chunk*>(chunks), nchunks, rank, world, out32, scale, sumsq);
  else
    reduce_scatter_pull_kernel<float><<<grid, 512, 0, stream>>>(
        pp, reinterpret_cast<const Chunk*>(chunks), nchunks, rank, world, out32, scale, sumsq);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_allgather_pull(const void* const* shard_ptrs, const void* chunks, int nchunks, int rank,
                             int world, void* full, int max_ctas, cudaStream_t stream) {
  if (nchunks <= 0) return 0;
  if (world < 1 || world > MAX_RANKS) return -2;
  int grid = nchunks * world < 148 * 2 ? nchunks * world : 148 * 2;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  allgather_pull_kernel<<<grid, 512, 0, stream>>>(make_ptrs(shard_ptrs, world),
                                                  reinterpret_cast<const Chunk*>(chunks), nchunks, rank,
                                                  world, reinterpret_cast<__nv_bfloat16*>(full));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

TB_API int tb_gather_shard(const void* full, const void* chunks, int nchunks, int rank, float* shard32,
                           void* shard16, cudaStream_t stream) {
  if (nchunks <= 0) return 0;
  const int grid = nchunks < 148 * 4 ? nchunks : 148 * 4;
  gather_shard_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(full),
                                                reinterpret_cast<const Chunk*>(chunks), nchunks, rank,
                                                shard32, reinterpret_cast<__nv_bfloat16*>(shard16));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// dst[block] = peer[block.src_rank][block] for a device-resident table of Block2D (48 bytes each).
TB_API int tb_pull_blocks(const void* const* src_ptrs, int world, const void* blocks, int nblocks, void* dst,
                          cudaStream_t stream) {
  if (nblocks <= 0) return 0;
  if (world < 1 || world > MAX_RANKS) return -2;
  pull_blocks_kernel<<<296, 512, 0, stream>>>(make_ptrs(src_ptrs, world), reinterpret_cast<const Block2D*>(blocks),
                                               nblocks, reinterpret_cast<__nv_bfloat16*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
