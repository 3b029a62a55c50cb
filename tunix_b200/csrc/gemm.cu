// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = epilogue( A[M,K] * B[N,K]^T )            fp32 accumulation in TMEM
//
// * one CTA per SM, tile 128 x BN (BN = 256 or 128), K block 64 (one 128-byte swizzle row)
// * warp 0      : TMA producer (cp.async.bulk.tensor, no multicast) into a 4/6-stage smem ring
// * warp 1      : single-thread tcgen05.mma issue, accumulators double-buffered in TMEM
// * warps 2..5  : epilogue, tcgen05.ld -> registers -> (bias / residual / accumulate) -> global
// * A and B may each be "K-major" (contraction dimension contiguous) or "MN-major"
//   (the M or N dimension contiguous), which covers forward, dgrad and wgrad of a
//   linear layer without any transposed copy of activations or weights.
// * every mbarrier wait is bounded (common.cuh); a timeout sets *status and unwinds.
//
// Role in the framework: replaces the XLA dot -> cuBLAS lowering of the reference's dense
// projections and gated MLP (tunix/models/llama3/model.py:311-334, 489-496).
#include "common.cuh"
#include <mutex>
#include <unordered_map>
#include <cstring>
#include <cstdio>
#include <cstdlib>

using namespace tb;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GROUP_M = 16;  // rasterisation: 16 M-tiles share one sweep over N (L2 reuse)

enum GemmFlags : int {
  GF_A_MN = 1,         // A stored [K, M] (M contiguous)
  GF_B_MN = 2,         // B stored [K, N] (N contiguous)
  GF_OUT_F32 = 4,      // C is fp32 (else bf16)
  GF_ACCUM = 8,        // C += result (reads C)
  GF_BIAS = 16,        // + bias[N] (bf16)
  GF_RESIDUAL = 32,    // + R[M,N] (bf16, row stride ldr)
  // Gated activation in the epilogue (pre-tiled weights only): the N columns are gate / up projections interleaved in
  // groups of 16 = [8 gate | 8 up] (tb_pack_weight_glu); the kernel writes act(gate) * up, N / 2 bf16 columns.
  GF_GLU_SILU = 64,
  GF_GLU_GELU = 128,
};

// Grouped mode (mixture-of-experts): the tile list lives in device memory, built by a planning kernel from
// per-expert token counts that the host never sees. A tile names its output block, its k-block range, a row
// offset into B (the expert's slice of the stacked weights) and an element offset into C (the expert's slice of
// a stacked weight gradient).
struct TileDesc {
  int m0, n0;          // output block origin
  int m_end;           // rows >= m_end are not written
  int kb0, kb1;        // k-block range [kb0, kb1)
  int b_row0;          // added to the row coordinate of every B load
  long long c_off;     // added (in elements) to C
};

constexpr int MAX_RANKS = 8;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

// Fused all-gather: CTAs past `gemm_ctas` pull the peers' row blocks of the gathered operand into the local
// copy (TMA bulk loads from peer memory into shared memory, bulk stores from there to local memory) and
// publish one flag per 128-row block; GEMM tiles wait for the flags of the rows they read.
struct CopyArgs {
  PeerPtrs src;               // every rank's gathered buffer (symmetric); rank p owns rows [p, p+1) * rows/world
  char* dst;                  // this rank's gathered buffer
  long long rank_bytes;       // bytes owned by one rank
  long long job_bytes;        // bytes of one 128-row block
  int jobs_per_rank;
  int piece_bytes;            // bulk copy granularity (divides job_bytes, multiple of 16, <= 32 KiB)
  unsigned* flags;            // [world * jobs_per_rank], local
  unsigned epoch;
};
// Fused reduce-scatter: every rank leaves its partial product in its own symmetric buffer and counts finished
// tiles per 128-row block; CTAs past `gemm_ctas` wait for the blocks of this rank's rows on every peer, pull
// them (TMA bulk loads), add them up in fp32 and write the reduced rows.
struct ReduceArgs {
  PeerPtrs part;              // every rank's partial C [M, N] bf16, contiguous
  PeerPtrs done;              // every rank's per-block counters
  __nv_bfloat16* out;         // [M / world, N] contiguous
  const __nv_bfloat16* resid; // optional, same layout as out
  int tiles_per_rank;
  unsigned target;            // counter value that marks a finished block in this call
  int* work;                  // local counter handing out row blocks to reducer CTAs (zero at launch)
};

struct GemmArgs {
  int M, N, K;
  int flags;
  const TileDesc* tiles;      // null = dense problem
  const int* num_tiles_dev;
  int a_rows_rt;              // K-major A, one tile high, no MN-major B: rows of A that are loaded (16 / 32 / 64; 0 = all
                              // 128) and the ring is packed tightly, see the kernel
  int bn_rt;                  // dense problems only: tile width actually used (multiple of 16, <= BN; 0 = BN). A width
                              // picked at run time lets a skinny problem cover the SMs in whole waves.
  const uint8_t* b_packed;    // dense problems only: B pre-tiled by tb_pack_weight (one contiguous, pre-swizzled
                              // block per n tile and k block, fetched with one bulk copy); null = B through tmB
  // --- fused collectives (all zero for a plain GEMM)
  int gemm_ctas;              // CTAs that run GEMM tiles; the rest of the grid runs the aux role
  int aux_kind;               // 0 none, 1 copier (all-gather), 2 reducer (reduce-scatter)
  int rank, world;
  int rot_m, rot_n;           // tile order starts at this m / n tile (own rows first, or own rows last)
  int wait_mode;              // 0 none; a tile waits for the flags of 1: its A rows, 2: its B rows,
                              // 3: each 128 rows of the contraction (gathered dimension = K, both operands MN-major)
  int rot_k;                  // mode 3: k blocks start here (own rows first)
  int own_lo, own_hi;         // flag range that is local and needs no wait
  const unsigned* wait_flags;
  unsigned wait_epoch;
  unsigned* done_flags;       // per m tile, += 1 per epilogue warp and tile
  CopyArgs copy;
  ReduceArgs red;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  long long ldr;
  float alpha;
  int* status;
};

constexpr int MAX_STAGES = 16;   // barrier slots per kind; the compact ring of skinny problems (GemmArgs::a_rows_rt) uses up to this many

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // fill ~200 KiB of shared memory: deeper rings for the narrow tiles that stream weights at small M
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : (BN == 64) ? 8 : 10;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulator stages
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/;
};

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}
constexpr long long FLAG_WAIT_NS = 4000000000ll;   // a flag another CTA or rank sets: give up after 4 s

// Bounded wait for *flag to reach `target` (wrap-safe). `sys` = the flag lives in a peer's memory.
__device__ __forceinline__ bool flag_wait_bounded(const unsigned* flag, unsigned target, bool sys,
                                                  volatile int* abort_flag, int* status) {
  const unsigned long long t0 = gtimer_ns();
  int polls = 0;
  while (true) {
    const unsigned v = sys ? ld_acquire_sys_u32(flag) : ld_acquire_gpu_u32(flag);
    if ((int)(v - target) >= 0) return true;
    if ((++polls & 15) == 0) {
      if (*abort_flag) return false;
      if ((long long)(gtimer_ns() - t0) > FLAG_WAIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, ST_TIMEOUT_FLAG);
        return false;
      }
    }
    __nanosleep(sys ? 500 : 100);
  }
}

// All-gather copier (one elected thread): peers' 128-row blocks, nearest ring neighbour first.
__device__ void copier_role(const CopyArgs& ca, int rank, int world, int aux_id, int n_aux, uint32_t smem_base,
                            uint32_t bar_base, int ring_bytes, volatile int* abort_flag, int* status) {
  const int piece = ca.piece_bytes;
  int nbuf = ring_bytes / piece;
  if (nbuf > 6) nbuf = 6;
  uint32_t phase_bits = 0;                                   // parity per buffer
  const int total_jobs = (world - 1) * ca.jobs_per_rank;
  for (int j = aux_id; j < total_jobs; j += n_aux) {
    const int step = j / ca.jobs_per_rank, within = j - step * ca.jobs_per_rank;
    const int peer = (rank + 1 + step) % world;
    const long long off = (long long)peer * ca.rank_bytes + (long long)within * ca.job_bytes;
    const char* src = reinterpret_cast<const char*>(ca.src.p[peer]) + off;
    char* dst = ca.dst + off;
    const int np = (int)(ca.job_bytes / piece);
    for (int i = 0; i < np && i < nbuf; ++i) {
      mbar_expect_tx(bar_base + 8u * i, piece);
      bulk_load(smem_base + i * piece, src + (long long)i * piece, piece, bar_base + 8u * i);
    }
    bool ok = true;
    for (int i = 0; i < np; ++i) {
      const int b = i % nbuf;
      if (!mbar_wait_bounded(bar_base + 8u * b, (phase_bits >> b) & 1u, abort_flag, status, ST_TIMEOUT_PRODUCER)) {
        ok = false;
        break;
      }
      phase_bits ^= 1u << b;
      bulk_store(dst + (long long)i * piece, smem_base + b * piece, piece);
      tma_store_commit();
      if (i + nbuf < np) {
        tma_store_wait_read<0>();                            // the buffer may be overwritten
        mbar_expect_tx(bar_base + 8u * b, piece);
        bulk_load(smem_base + b * piece, src + (long long)(i + nbuf) * piece, piece, bar_base + 8u * b);
      }
    }
    if (!ok) return;
    tma_store_wait<0>();
    fence_proxy_async_all();
    __threadfence();
    st_release_gpu_u32(ca.flags + peer * ca.jobs_per_rank + within, ca.epoch);
  }
}

// Reduce-scatter reducer (whole CTA): this rank's row blocks, summed over all ranks' partial products.
// A block (128 rows x N) is walked in 16 KiB chunks; for each chunk the `world` source pieces stream through a
// ring of 11 shared-memory buffers (TMA bulk loads, peers over NVLink) and every thread keeps the fp32 sums of
// its vectors in registers until the last source has arrived. full / empty mbarriers per buffer, no CTA-wide
// barrier inside the stream.
__device__ void reducer_role(const ReduceArgs& ra, int rank, int world, int N, int aux_id, int n_aux,
                             uint8_t* smem_al, uint32_t smem_base, uint32_t bar_base, volatile int* abort_flag,
                             int* status) {
  constexpr int PIECE = 16384, NBUF = 11, VEC = PIECE / 16, MAXV = (VEC + 191) / 192;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const long long block_bytes = 128ll * N * 2;
  const int nchunk = (int)(block_bytes / PIECE);
  // 11 buffers (176 KiB in flight per CTA against NVLink latency); their barriers sit behind them in the ring,
  // which every tile configuration sizes at 192 KiB or more
  (void)bar_base;
  const uint32_t rbar = smem_base + NBUF * PIECE;
  auto full = [&](int b) { return rbar + 8u * b; };
  auto empty = [&](int b) { return rbar + 8u * (NBUF + b); };
  __syncthreads();
  if (tid == 0) {
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(full(b), 1);
      mbar_init(empty(b), nthr >> 5);                          // one arrival per warp
    }
    mbar_fence_init();
  }
  __syncthreads();
  uint32_t ph_full = 0u, ph_empty = 0u;                      // parity bits per buffer (ph_empty: thread 0 only)
  long long issued = 0;                                      // pieces issued so far (thread 0), over all blocks
  long long consumed = 0;
  volatile int* s_blk = reinterpret_cast<volatile int*>(smem_al + NBUF * PIECE + 8 * (2 * NBUF));
  const int parts = (nchunk % 4 == 0) ? 4 : 1;               // work unit: a quarter of a block's chunks
  (void)aux_id; (void)n_aux;
  while (true) {
    // row blocks are handed out by a counter: dedicated reducer CTAs start while the tiles still run, the tile
    // CTAs join when their tiles are done
    __syncthreads();
    if (tid == 0) *s_blk = atomicAdd(ra.work, 1);
    __syncthreads();
    const int unit = *s_blk;                                 // (row block, part of its chunks)
    if (unit >= ra.tiles_per_rank * parts) break;
    const int blk = unit / parts, part = unit - blk * parts;
    const int c_first = part * (nchunk / parts);
    const int gmt = rank * ra.tiles_per_rank + blk;
    if (tid == 0) {
      for (int s = 0; s < world; ++s) {
        const int p = (rank - 1 - s + 2 * world) % world;    // the peer that computes this rank's rows first
        const unsigned* f = reinterpret_cast<const unsigned*>(ra.done.p[p]) + gmt;
        if (!flag_wait_bounded(f, ra.target, p != rank, abort_flag, status)) break;
      }
      fence_proxy_async_all();
    }
    __syncthreads();
    if (*abort_flag) return;
    const int npieces = (nchunk / parts) * world;
    int next = 0;                                            // next piece of this block to issue (thread 0)
    auto issue_upto = [&](int limit) {
      while (next < npieces && next < limit) {
        const int b = (int)(issued % NBUF);
        if (issued >= NBUF) {
          if (!mbar_wait_bounded(empty(b), (ph_empty >> b) & 1u, abort_flag, status, ST_TIMEOUT_PRODUCER)) return;
          ph_empty ^= 1u << b;
        }
        const int c = c_first + next / world, s = next % world;
        const int p = (rank + 1 + s) % world;                // own partial product last
        const char* src = reinterpret_cast<const char*>(ra.part.p[p]) + (long long)gmt * block_bytes + (long long)c * PIECE;
        mbar_expect_tx(full(b), PIECE);
        bulk_load(smem_base + b * PIECE, src, PIECE, full(b));
        ++issued;
        ++next;
      }
    };
    if (tid == 0) issue_upto(NBUF - 1);
    float acc[MAXV][8];
    for (int q = 0; q < npieces; ++q) {
      const int c = c_first + q / world, s = q % world;
      if (tid == 0) issue_upto(q + NBUF);
      const int b = (int)(consumed % NBUF);
      if (!mbar_wait_bounded(full(b), (ph_full >> b) & 1u, abort_flag, status, ST_TIMEOUT_EPILOGUE)) return;
      ph_full ^= 1u << b;
      ++consumed;
      const uint8_t* buf = smem_al + b * PIECE;
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int v = tid + j * 192;
        if (v < VEC) {
          const uint4 u = *reinterpret_cast<const uint4*>(buf + v * 16);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
          if (s == 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              acc[j][2 * k] = bf16_lo(w[k]);
              acc[j][2 * k + 1] = bf16_hi(w[k]);
            }
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              acc[j][2 * k] += bf16_lo(w[k]);
              acc[j][2 * k + 1] += bf16_hi(w[k]);
            }
          }
        }
      }
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(empty(b));
      if (s == world - 1) {
        const long long out_off = ((long long)blk * block_bytes + (long long)c * PIECE) >> 1;   // elements
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int v = tid + j * 192;
          if (v < VEC) {
            if (ra.resid != nullptr) {
              const uint4 u = *reinterpret_cast<const uint4*>(ra.resid + out_off + v * 8);
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                acc[j][2 * k] += bf16_lo(w[k]);
                acc[j][2 * k + 1] += bf16_hi(w[k]);
              }
            }
            *reinterpret_cast<uint4*>(ra.out + out_off + v * 8) =
                make_uint4(pack_bf16(acc[j][0], acc[j][1]), pack_bf16(acc[j][2], acc[j][3]),
                           pack_bf16(acc[j][4], acc[j][5]), pack_bf16(acc[j][6], acc[j][7]));
          }
        }
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmArgs args) {
  using C_ = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C_::STAGES * C_::STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tfull[2], tempty[2], then tmem ptr, abort
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * MAX_STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * MAX_STAGES + 2 + s); };
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_al + C_::STAGES * C_::STAGE_BYTES + 8 * (2 * MAX_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int M = args.M, N = args.N, K = args.K;
  const int num_m = (M + BM - 1) / BM;
  const int bn = args.bn_rt > 0 ? args.bn_rt : BN;        // tile width in use
  const int num_n = (N + bn - 1) / bn;
  const int num_kb = (K + BK - 1) / BK;
  const int num_tiles = num_m * num_n;
  const bool a_mn = args.flags & GF_A_MN;
  const bool b_mn = args.flags & GF_B_MN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_ptr_smem), C_::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  pdl_wait();            // everything above overlapped the previous kernel's tail; from here on memory is read

  const bool grouped = args.tiles != nullptr;
  // Ring geometry. Normally STAGES slots of a 128-row A tile and a BN-row B tile. A one-tile-high problem with
  // M <= 64 (a_rows_rt) loads only the rows of A that exist and packs the slots tightly (a_rows_rt * 128 bytes of
  // A, then bn rows of B): the same shared memory holds more stages, which is what a kernel that only streams
  // weights is short of. The MMA still reads 128 rows of A; rows past a_rows_rt are whatever follows in the ring
  // (the slot's B tile, the next slot), and the accumulator rows they produce are never stored.
  const int a_bytes = args.a_rows_rt > 0 ? args.a_rows_rt * BK * 2 : C_::A_BYTES;
  const int stage_bytes = args.a_rows_rt > 0 ? a_bytes + bn * BK * 2 : C_::STAGE_BYTES;
  int nstages = C_::STAGES;
  if (args.a_rows_rt > 0) {
    // the last slot's 128-row A read must end inside the ring
    nstages = (C_::STAGES * C_::STAGE_BYTES - C_::A_BYTES) / stage_bytes + 1;
    if (nstages * stage_bytes > C_::STAGES * C_::STAGE_BYTES) --nstages;
    nstages = max(1, min(nstages, MAX_STAGES));
  }
  const int total_tiles = grouped ? *args.num_tiles_dev : num_tiles;
  const int n_gemm = args.gemm_ctas > 0 ? args.gemm_ctas : (int)gridDim.x;   // CTAs that walk the tile list
  auto tile_info = [&](int t) -> TileDesc {
    if (grouped) return args.tiles[t];
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, num_m - first_m);
    const int r = t - g * per_group;
    TileDesc d;
    d.m0 = ((first_m + (r % gsz) + args.rot_m) % num_m) * BM;
    d.n0 = ((r / gsz + args.rot_n) % num_n) * bn;
    if (args.wait_mode == 2) {
      // gathered B rows: walk N in groups of 8 tiles (own rows first), all of M inside a group, so that the
      // tiles of a peer's rows come up only after everything that needs no transfer
      constexpr int GROUP_N = 8;
      const int per_gn = GROUP_N * num_m;
      const int gn = t / per_gn;
      const int first_n = gn * GROUP_N;
      const int gszn = min(GROUP_N, num_n - first_n);
      const int rn = t - gn * per_gn;
      d.m0 = (rn / gszn) * BM;
      d.n0 = ((first_n + (rn % gszn) + args.rot_n) % num_n) * BN;
    }
    d.m_end = M;
    d.kb0 = 0;
    d.kb1 = num_kb;
    d.b_row0 = 0;
    d.c_off = 0;
    return d;
  };

  if ((int)blockIdx.x >= n_gemm) {
    // ------------------------------------------------ aux role of a fused collective (no tiles, no TMEM use)
    const int aux_id = (int)blockIdx.x - n_gemm, n_aux = (int)gridDim.x - n_gemm;
    if (args.aux_kind == 1) {
      if (warp == 0 && elect_one())
        copier_role(args.copy, args.rank, args.world, aux_id, n_aux, smem_base, bar_base, C_::STAGES * C_::STAGE_BYTES,
                    abort_flag, args.status);
    } else if (args.aux_kind == 2) {
      reducer_role(args.red, args.rank, args.world, N, aux_id, n_aux, smem_al, smem_base, bar_base, abort_flag,
                   args.status);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += n_gemm) {
        const TileDesc td = tile_info(t);
        const int m0 = td.m0, n0 = td.n0;
        if (args.wait_mode == 1 || args.wait_mode == 2) {
          // rows this tile reads from the gathered operand must have landed (copier CTAs of this kernel)
          const int f_lo = (args.wait_mode == 1 ? m0 : n0) >> 7;
          const int ext = args.wait_mode == 1 ? min(BM, M - m0) : min(BN, N - n0);
          const int f_hi = f_lo + ((ext + 127) >> 7);
          for (int f = f_lo; f < f_hi && ok; ++f) {
            if (f >= args.own_lo && f < args.own_hi) continue;
            ok = flag_wait_bounded(args.wait_flags + f, args.wait_epoch, false, abort_flag, args.status);
          }
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kbi = td.kb0; kbi < td.kb1; ++kbi) {
          int kb = kbi;
          if (args.wait_mode == 3) {
            kb = (kbi + args.rot_k) % num_kb;
            const int f = (kb * BK) >> 7;
            if ((kbi == td.kb0 || (kb & 1) == 0) && !(f >= args.own_lo && f < args.own_hi)) {
              if (!flag_wait_bounded(args.wait_flags + f, args.wait_epoch, false, abort_flag, args.status)) {
                ok = false;
                break;
              }
              fence_proxy_async_all();
            }
          }
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1, abort_flag, args.status,
                                 ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + a_bytes;
          mbar_expect_tx(full_bar(stage), a_bytes + (b_mn ? C_::B_BYTES : bn * BK * 2));
          const int k0 = kb * BK;
          if (!a_mn) {
            tma_load_2d(sa, &tmA, full_bar(stage), k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &tmA, full_bar(stage), m0 + 64 * j, k0);
          }
          if (args.b_packed != nullptr) {
            const size_t blk = (size_t)(n0 / bn) * num_kb + kb;
            bulk_load(sb, args.b_packed + blk * (size_t)(bn * BK * 2), bn * BK * 2, full_bar(stage));
          } else if (!b_mn) {
            tma_load_2d(sb, &tmB, full_bar(stage), k0, n0 + td.b_row0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmB, full_bar(stage), n0 + 64 * j, k0 + td.b_row0);
          }
          if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, bn, a_mn ? 1 : 0, b_mn ? 1 : 0);
      const uint32_t a_lbo = a_mn ? 8192u : 16u, b_lbo = b_mn ? 8192u : 16u;
      const uint32_t a_kstep = a_mn ? 2048u : 32u, b_kstep = b_mn ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += n_gemm) {
        int kb0 = 0, kb1 = num_kb;
        if (grouped) {
          kb0 = args.tiles[t].kb0;
          kb1 = args.tiles[t].kb1;
          if (kb1 <= kb0) continue;                 // empty contraction: the epilogue writes zeros on its own
        }
        if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1, abort_flag, args.status,
                               ST_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + a_bytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc(sb + k * b_kstep, b_lbo, 1024);
            umma_f16_ss(tmem_d, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // frees the smem slot when these MMAs retire
          if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = args.flags & GF_OUT_F32;
    const bool accum = args.flags & GF_ACCUM;
    const bool has_bias = args.flags & GF_BIAS;
    const bool has_res = args.flags & GF_RESIDUAL;
    const int glu_kind = (args.flags & GF_GLU_SILU) ? 1 : (args.flags & GF_GLU_GELU) ? 2 : 0;
    const float alpha = args.alpha;
    const bool c_al16 = (reinterpret_cast<uintptr_t>(args.C) & 15) == 0;      // vector paths need aligned bases
    const bool r_al16 = (reinterpret_cast<uintptr_t>(args.resid) & 15) == 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += n_gemm) {
      const TileDesc td = tile_info(t);
      const int row = td.m0 + q * 32 + lane;
      const int n0 = td.n0;
      const int N = min(args.N, n0 + bn);           // shadows the problem's N: columns of this tile that exist
      const int M = td.m_end;                       // shadows the problem's M: rows of this tile that exist
      const long long c_off = td.c_off;
      const bool empty_k = td.kb1 <= td.kb0;        // nothing was accumulated: the tile's value is zero
      if (!empty_k && !mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, args.status,
                                         ST_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) break;  // warp-uniform
        uint32_t r[32];
        if (!empty_k) {
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row < M) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
          const bool full = (col0 + 32 <= N);
          if (glu_kind) {
            // two groups of [8 gate | 8 up] -> 16 outputs at column col0 / 2
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.C) + c_off + (long long)row * args.ldc + (col0 >> 1);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              if (col0 + 16 * g >= N) break;
              float o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float gt = v[16 * g + j], up = v[16 * g + 8 + j];
                float act;
                if (glu_kind == 1) {
                  act = gt / (1.f + __expf(-gt));
                } else {
                  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
                  act = 0.5f * gt * (1.f + tanhf(k0 * (gt + k1 * gt * gt * gt)));
                }
                o[j] = act * up;
              }
              uint4 pk;
              pk.x = pack_bf16(o[0], o[1]);
              pk.y = pack_bf16(o[2], o[3]);
              pk.z = pack_bf16(o[4], o[5]);
              pk.w = pack_bf16(o[6], o[7]);
              *reinterpret_cast<uint4*>(cp + 8 * g) = pk;       // ldc % 8 == 0 and col0 % 32 == 0: 16-byte aligned
            }
            continue;
          }
          if (has_bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (full || col0 + i < N) v[i] += __bfloat162float(args.bias[col0 + i]);
          }
          if (has_res) {
            const __nv_bfloat16* rp = args.resid + (long long)row * args.ldr + col0;
            if (full && (args.ldr % 8 == 0) && r_al16) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint4 u = reinterpret_cast<const uint4*>(rp)[g];
                uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[g * 8 + 2 * j] += bf16_lo(w[j]);
                  v[g * 8 + 2 * j + 1] += bf16_hi(w[j]);
                }
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) v[i] += __bfloat162float(rp[i]);
            }
          }
          if (out_f32) {
            float* cp = reinterpret_cast<float*>(args.C) + c_off + (long long)row * args.ldc + col0;
            if (full && (args.ldc % 4 == 0) && c_al16) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                float4 o = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                if (accum) {
                  float4 p = reinterpret_cast<float4*>(cp)[g];
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                reinterpret_cast<float4*>(cp)[g] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) cp[i] = accum ? cp[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* cp =
                reinterpret_cast<__nv_bfloat16*>(args.C) + c_off + (long long)row * args.ldc + col0;
            if (full && (args.ldc % 8 == 0) && c_al16) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (accum) {
                  uint4 u = reinterpret_cast<uint4*>(cp)[g];
                  uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    v[g * 8 + 2 * j] += bf16_lo(w[j]);
                    v[g * 8 + 2 * j + 1] += bf16_hi(w[j]);
                  }
                }
                uint4 o;
                o.x = pack_bf16(v[g * 8 + 0], v[g * 8 + 1]);
                o.y = pack_bf16(v[g * 8 + 2], v[g * 8 + 3]);
                o.z = pack_bf16(v[g * 8 + 4], v[g * 8 + 5]);
                o.w = pack_bf16(v[g * 8 + 6], v[g * 8 + 7]);
                reinterpret_cast<uint4*>(cp)[g] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) {
                  float o = v[i] + (accum ? __bfloat162float(cp[i]) : 0.f);
                  cp[i] = __float2bfloat16(o);
                }
            }
          }
        }
      }
      if (args.done_flags != nullptr) {
        __threadfence_system();                     // this tile's rows are visible to peers before the count moves
        __syncwarp();
        if (lane == 0) red_release_sys_add(args.done_flags + (td.m0 >> 7), 1u);
      }
      tc_fence_before();
      __syncwarp();
      if (empty_k) continue;                        // the MMA warp skipped this tile too: no accumulator used
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  if (args.aux_kind == 2 && (int)blockIdx.x < n_gemm) {
    // reduce-scatter: tile CTAs whose tiles are done help the reducer CTAs with the remaining row blocks
    tc_fence_before();
    __syncthreads();
    if (!*abort_flag)
      reducer_role(args.red, args.rank, args.world, N, 0, 1, smem_al, smem_base, bar_base, abort_flag, args.status);
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give TMA copies that may still be in flight time to land before smem is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C_::TMEM_COLS);
  }
}

struct TmapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && box_cols == o.box_cols;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1315423911u ^ k.rows;
    h = h * 1315423911u ^ k.cols;
    h = h * 1315423911u ^ k.ld;
    h = h * 1315423911u ^ (((uint64_t)k.box_rows << 32) | k.box_cols);
    return h;
  }
};
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
int g_sm_count = 0;
void set_gemm_attrs();
// CTAs to give to the copier role: enough to move `bytes` while the local share of `flops` is computed, assuming
// about 30 GB/s per CTA (measured: bulk copies with ~190 KiB in flight per CTA over NVLink) and 1.3 PFLOP/s for the tiles.
// Measured on 8 ranks against a sizing that only keeps pace with the tile walk (4 CTAs instead of 19 for a
// 14336 x 4096 weight): 1.553 instead of 1.610 ms for that shape, but 1.827 instead of 1.618 ms (4096 x 14336) and 0.543
// instead of 0.472 ms (4096 x 4096), and 1057 instead of 1017 ms for the weight-sharded training step: the early
// finish is kept.
int aux_ctas_for(double bytes, double flops, int world) {
  const double t = flops / 1.3e15 / world;      // the transfer should be over when the local tiles are
  int n = (int)(bytes / (t * 30e9) + 0.999);
  if (n < 2) n = 2;
  if (n > 24) n = 24;
  return n;
}
void clear_fused(GemmArgs& a) {
  a.gemm_ctas = 0; a.aux_kind = 0; a.rank = 0; a.world = 1; a.rot_m = 0; a.rot_n = 0; a.wait_mode = 0;
  a.own_lo = 0; a.own_hi = 0; a.rot_k = 0; a.a_rows_rt = 0; a.bn_rt = 0; a.b_packed = nullptr; a.wait_flags = nullptr; a.wait_epoch = 0; a.done_flags = nullptr;
  memset(&a.copy, 0, sizeof(a.copy));
  memset(&a.red, 0, sizeof(a.red));
}

}  // namespace

int tb_gemm_splitk_try(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                       int* status, cudaStream_t stream, const void* b_packed = nullptr);

int tb_gemm_2cta_try(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                     int* status, cudaStream_t stream);

int tb_gemm_pair_splitk_try(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                            int* status, cudaStream_t stream);

tb_encode_tiled_fn tb_get_encode_tiled() {
  static tb_encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<tb_encode_tiled_fn>(p);
  });
  return fn;
}

int tb_make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t ld, uint32_t box_rows, uint32_t box_cols, int swizzle128) {
  tb_encode_tiled_fn enc = tb_get_encode_tiled();
  if (!enc) return -1;
  TmapKey key{base, rows, cols, ld, box_rows, box_cols | (swizzle128 ? 0x80000000u : 0)};
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  auto encode = [&] {
    return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r != CUDA_SUCCESS) {
    // A thread that has not touched the runtime yet (an autograd worker whose first operation is one of these
    // kernels) has no current context, and the driver's encoder refuses to work without one: bind the device's
    // primary context to this thread and try once more.
    cudaFree(nullptr);
    r = encode();
  }
  if (r != CUDA_SUCCESS) return (int)r;
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  if (g_tmap_cache.size() > 65536) g_tmap_cache.clear();
  g_tmap_cache.emplace(key, *out);
  return 0;
}

namespace {
bool g_pdl = false;
}
bool tb_pdl_enabled() { return g_pdl; }
// Programmatic dependent launch for the kernels that support it (decode path): 1 = on.
TB_API void tb_set_pdl(int on) { g_pdl = on != 0; }

// Forget cached tensor maps (call when device memory is released back to the driver).
TB_API void tb_tmap_cache_clear() {
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  g_tmap_cache.clear();
}

// C[M,N] = alpha * A*B^T (+bias)(+resid)(+C). Strides in elements.
//   A: K-major -> [M,K] ld=lda ; MN-major (flags&1) -> [K,M] ld=lda
//   B: K-major -> [N,K] ld=ldb ; MN-major (flags&2) -> [K,N] ld=ldb
// Requirements: bf16 operands 16-byte aligned, lda/ldb multiples of 8, K > 0.
// max_ctas <= 0 means one CTA per SM. Returns 0 or a negative error code.
TB_API int tb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                        long long ldb, long long ldc, int flags, const void* bias,
                        const void* resid, long long ldr, float alpha, int* status, int max_ctas,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool a_mn = flags & GF_A_MN, b_mn = flags & GF_B_MN;
  static const bool no_splitk = getenv("TUNIX_B200_NO_SPLITK") != nullptr;
  if (max_ctas <= 0 && !no_splitk && !(flags & (GF_GLU_SILU | GF_GLU_GELU))) {
    // a few hundred rows: 256x256 tiles on CTA pairs with the K range split over a cluster (gemm_pair_splitk.cu)
    const int ps = tb_gemm_pair_splitk_try(A, B, C, M, N, K, lda, ldb, ldc, flags, bias, resid, ldr, alpha, status, stream);
    if (ps != 0) return ps < 0 ? ps : 0;
  }
  if (max_ctas <= 0 && !no_splitk) {
    // skinny problems: 128x256 tiles with the K range split over a cluster (gemm_splitk.cu)
    const int sk = tb_gemm_splitk_try(A, B, C, M, N, K, lda, ldb, ldc, flags, bias, resid, ldr, alpha, status, stream);
    if (sk != 0) return sk < 0 ? sk : 0;
  }
  if (max_ctas <= 0) {
    // large problems: 256x256 tiles on CTA pairs (gemm_2cta.cu)
    const int tc = tb_gemm_2cta_try(A, B, C, M, N, K, lda, ldb, ldc, flags, bias, resid, ldr, alpha, status, stream);
    if (tc != 0) return tc < 0 ? tc : 0;
  }
  // Tile width: the widest N tile that still gives every SM work. Large problems use 128x256; skinny
  // ones (decode: M <= 128) fall to 128x64 / 128x32 so that >= 100 CTAs stream the weight matrix.
  const int num_m = (M + BM - 1) / BM;
  int BN = 32;
  for (int cand : {256, 128, 64, 32}) {
    if (cand > 128 && N < 256) continue;
    if (cand < 64 && b_mn) continue;          // MN-major B is loaded in 64-wide swizzled boxes
    BN = cand;
    if ((long long)num_m * ((N + cand - 1) / cand) >= (g_sm_count * 3) / 5) break;
  }
  if (b_mn && BN < 64) BN = 64;
  // Skinny problems (one row of tiles, K-major B): a run-time tile width, a multiple of 16, chosen so that the
  // tiles fill the SMs in whole waves (24576 columns: 140 tiles of 176 instead of 96 of 256).
  int bn_rt = 0;
  static const bool fixed_bn = getenv("TUNIX_B200_FIXED_BN") != nullptr;
  if (num_m == 1 && !b_mn && N >= 1024 && max_ctas <= 0 && !fixed_bn) {
    double best = 0.0;
    for (int w = 32; w <= 256; w += 16) {
      const int tiles = (N + w - 1) / w;
      const int waves = (tiles + g_sm_count - 1) / g_sm_count;
      // wave efficiency, with a mild preference for wide tiles (fewer re-reads of A)
      const double eff = (double)tiles / (waves * g_sm_count) * (1.0 + 0.0004 * w) * ((double)N / ((double)tiles * w));
      if (eff > best) { best = eff; bn_rt = w; }
    }
    BN = bn_rt > 128 ? 256 : bn_rt > 64 ? 128 : bn_rt > 32 ? 64 : 32;
    if (bn_rt == BN) bn_rt = 0;
  }
  CUtensorMap tmA, tmB;
  int r;
  static const bool no_compact = getenv("TUNIX_B200_NO_COMPACT_RING") != nullptr;
  const int a_rows = (num_m == 1 && M <= 64 && !a_mn && !b_mn && max_ctas <= 0 && !no_compact) ? (M <= 16 ? 16 : M <= 32 ? 32 : 64) : 0;
  if (!a_mn) r = tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, a_rows > 0 ? a_rows : BM, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmA, A, K, M, lda, BK, 64, 1);
  if (r) return -3;
  if (!b_mn) r = tb_make_tmap_2d_bf16(&tmB, B, N, K, ldb, bn_rt > 0 ? bn_rt : BN, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, 64, 1);
  if (r) return -4;
  GemmArgs args;
  args.M = M; args.N = N; args.K = K; args.flags = flags;
  args.C = C; args.ldc = ldc;
  args.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  args.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  args.ldr = ldr; args.alpha = alpha; args.status = status;
  args.tiles = nullptr; args.num_tiles_dev = nullptr;
  clear_fused(args);
  args.bn_rt = bn_rt;
  args.a_rows_rt = a_rows;
  const int tiles = num_m * ((N + (bn_rt > 0 ? bn_rt : BN) - 1) / (bn_rt > 0 ? bn_rt : BN));
  int ctas = g_sm_count;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles < ctas) ctas = tiles;
  set_gemm_attrs();
  cudaError_t err;
  switch (BN) {
    case 256: err = launch_pdl(gemm_bf16_kernel<256>, dim3(ctas), dim3(192), Cfg<256>::SMEM_BYTES, stream, tmA, tmB, args); break;
    case 128: err = launch_pdl(gemm_bf16_kernel<128>, dim3(ctas), dim3(192), Cfg<128>::SMEM_BYTES, stream, tmA, tmB, args); break;
    case 64: err = launch_pdl(gemm_bf16_kernel<64>, dim3(ctas), dim3(192), Cfg<64>::SMEM_BYTES, stream, tmA, tmB, args); break;
    default: err = launch_pdl(gemm_bf16_kernel<32>, dim3(ctas), dim3(192), Cfg<32>::SMEM_BYTES, stream, tmA, tmB, args); break;
  }
  return err == cudaSuccess ? 0 : -5;
}

// ------------------------------------------------------------------ pre-tiled weights for skinny GEMMs
// A K-major weight [N, K] read through a 2-D tensor map arrives as 128-byte row pieces that lie K*2 bytes apart:
// at decode sizes (M <= 128) the kernel is a pure weight stream, and that access pattern reaches about half of
// the copy bandwidth. tb_pack_weight re-tiles the weight once: block (n tile, k block) holds `w` rows x 64
// columns contiguously, already in the 128-byte-swizzled order the MMA descriptors expect, and the blocks of
// one n tile follow each other, so a CTA streams one contiguous range with one bulk copy per pipeline stage.
// glu_f > 0: W holds glu_f gate rows followed by glu_f up rows; packed row n takes gate row 8 * (n / 16) + n % 16 when
// n % 16 < 8 and up row 8 * (n / 16) + n % 16 - 8 otherwise, so that every 16 packed rows pair 8 gate rows with
// their 8 up rows (the GF_GLU_* epilogue of the GEMM).
__global__ void pack_weight_kernel(const __nv_bfloat16* __restrict__ W, long long ldw, int N, int K, int w, int num_kb,
                                   uint4* __restrict__ P, long long total, int glu_f) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx & 7);
    const long long rr = idx >> 3;
    const int r = (int)(rr % w);
    const long long blk = rr / w;
    const int kb = (int)(blk % num_kb);
    const long long nt = blk / num_kb;
    long long n = nt * w + r;
    const int k = kb * BK + c * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    const bool in_range = n < N;
    if (glu_f > 0 && in_range) {
      const long long grp = n >> 4;
      const int w16 = (int)(n & 15);
      n = w16 < 8 ? grp * 8 + w16 : (long long)glu_f + grp * 8 + (w16 - 8);
    }
    if (in_range && k < K) v = *reinterpret_cast<const uint4*>(W + n * ldw + k);
    P[blk * (long long)w * 8 + (long long)r * 8 + (c ^ (r & 7))] = v;
  }
}

// Tile width a weight [N, K] is packed with: 256 where the cluster split-K kernel takes the problem (long
// contraction, few tiles), otherwise the multiple of 16 that fills the SMs in whole waves.
TB_API int tb_packed_width(int N, int K) {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (K >= 8192 && N >= 256 && ((N + 255) / 256) * 2 <= g_sm_count) return 256;
  double best = 0.0;
  int bw = 32;
  for (int w = 32; w <= 256; w += 16) {
    const int tiles = (N + w - 1) / w;
    const int waves = (tiles + g_sm_count - 1) / g_sm_count;
    const double eff = (double)tiles / (waves * g_sm_count) * (1.0 + 0.0004 * w) * ((double)N / ((double)tiles * w));
    if (eff > best) { best = eff; bw = w; }
  }
  return bw;
}

// P must hold ceil(N/w) * ceil(K/64) * w * 128 bytes. W: [N, K] bf16, 16-byte aligned, ldw and K multiples of 8.
TB_API int tb_pack_weight(const void* W, long long ldw, int N, int K, int w, void* P, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || w < 16 || w > 256 || (w % 16) || (ldw % 8) || (K % 8) ||
      (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(P) & 127))
    return -2;
  const int num_kb = (K + BK - 1) / BK;
  const long long total = (long long)((N + w - 1) / w) * num_kb * w * 8;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  pack_weight_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(W), ldw, N, K, w, num_kb,
                                                     reinterpret_cast<uint4*>(P), total, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// The same for a fused gate / up weight W = [gate (F rows); up (F rows)] with the rows interleaved for the gated
// epilogue (see pack_weight_kernel). N = 2 F must be a multiple of 16; w a multiple of 32.
TB_API int tb_pack_weight_glu(const void* W, long long ldw, int N, int K, int w, void* P, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || (N % 16) || w < 32 || w > 256 || (w % 16) || (ldw % 8) || (K % 8) ||
      (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(P) & 127))
    return -2;
  const int num_kb = (K + BK - 1) / BK;
  const long long total = (long long)((N + w - 1) / w) * num_kb * w * 8;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  pack_weight_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(W), ldw, N, K, w, num_kb,
                                                     reinterpret_cast<uint4*>(P), total, N / 2);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// C[M,N] = alpha * A[M,K] * W^T (+bias)(+resid)(+C) with W given as the packed copy P of width w.
TB_API int tb_gemm_packed_bf16(const void* A, long long lda, const void* P, int w, void* C, long long ldc, int M, int N,
                               int K, int flags, const void* bias, const void* resid, long long ldr, float alpha,
                               int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(P) & 127) ||
      w < 16 || w > 256 || (w % 16) || (flags & (GF_A_MN | GF_B_MN)))
    return -2;
  const bool glu = flags & (GF_GLU_SILU | GF_GLU_GELU);
  // gated epilogue: bf16 output of N / 2 columns, nothing else in the epilogue, 16-byte aligned rows
  if (glu && ((flags & (GF_OUT_F32 | GF_ACCUM | GF_BIAS | GF_RESIDUAL)) || (N % 16) || (ldc % 8) ||
              (reinterpret_cast<uintptr_t>(C) & 15) || alpha != 1.0f))
    return -2;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  static const bool no_splitk = getenv("TUNIX_B200_NO_SPLITK") != nullptr;
  if (w == 256 && !no_splitk && !glu) {
    const int sk = tb_gemm_splitk_try(A, nullptr, C, M, N, K, lda, 8, ldc, flags, bias, resid, ldr, alpha, status, stream, P);
    if (sk != 0) return sk < 0 ? sk : 0;
  }
  const int BN = w > 128 ? 256 : w > 64 ? 128 : w > 32 ? 64 : 32;
  CUtensorMap tmA;
  static const bool no_compact = getenv("TUNIX_B200_NO_COMPACT_RING") != nullptr;
  const int a_rows = (M <= 64 && !no_compact) ? (M <= 16 ? 16 : M <= 32 ? 32 : 64) : 0;
  if (tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, a_rows > 0 ? a_rows : BM, BK, 1)) return -3;
  GemmArgs args;
  args.M = M; args.N = N; args.K = K; args.flags = flags;
  args.C = C; args.ldc = ldc;
  args.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  args.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  args.ldr = ldr; args.alpha = alpha; args.status = status;
  args.tiles = nullptr; args.num_tiles_dev = nullptr;
  clear_fused(args);
  args.bn_rt = w == BN ? 0 : w;
  args.a_rows_rt = a_rows;
  args.b_packed = reinterpret_cast<const uint8_t*>(P);
  const int tiles = ((M + BM - 1) / BM) * ((N + w - 1) / w);
  const int ctas = tiles < g_sm_count ? tiles : g_sm_count;
  set_gemm_attrs();
  cudaError_t err;
  switch (BN) {
    case 256: err = launch_pdl(gemm_bf16_kernel<256>, dim3(ctas), dim3(192), Cfg<256>::SMEM_BYTES, stream, tmA, tmA, args); break;
    case 128: err = launch_pdl(gemm_bf16_kernel<128>, dim3(ctas), dim3(192), Cfg<128>::SMEM_BYTES, stream, tmA, tmA, args); break;
    case 64: err = launch_pdl(gemm_bf16_kernel<64>, dim3(ctas), dim3(192), Cfg<64>::SMEM_BYTES, stream, tmA, tmA, args); break;
    default: err = launch_pdl(gemm_bf16_kernel<32>, dim3(ctas), dim3(192), Cfg<32>::SMEM_BYTES, stream, tmA, tmA, args); break;
  }
  return err == cudaSuccess ? 0 : -5;
}

// Grouped GEMM over a device-resident tile list (see TileDesc). The arrays are described by their full
// extents: A is [a_rows, a_cols], B is [b_rows, b_cols] (row-major, leading strides lda / ldb); which of the
// two dimensions is contracted follows from the MN-major flags exactly as in tb_gemm_bf16. N is the column
// limit of one group's output, `bn` the tile width the list was planned for (256, 128 or 64).
TB_API int tb_gemm_grouped_bf16(const void* A, long long a_rows, long long a_cols, long long lda, const void* B,
                                long long b_rows, long long b_cols, long long ldb, void* C, long long ldc, int N,
                                int flags, int bn, const void* tiles, const int* num_tiles_dev, int max_tiles,
                                float alpha, int* status, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  if (bn != 256 && bn != 128 && bn != 64) return -2;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool a_mn = flags & GF_A_MN, b_mn = flags & GF_B_MN;
  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn) r = tb_make_tmap_2d_bf16(&tmA, A, a_rows, a_cols, lda, BM, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmA, A, a_rows, a_cols, lda, BK, 64, 1);
  if (r) return -3;
  if (!b_mn) r = tb_make_tmap_2d_bf16(&tmB, B, b_rows, b_cols, ldb, bn, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmB, B, b_rows, b_cols, ldb, BK, 64, 1);
  if (r) return -4;
  GemmArgs args;
  args.M = 0; args.N = N; args.K = 0; args.flags = flags;
  args.C = C; args.ldc = ldc; args.bias = nullptr; args.resid = nullptr; args.ldr = 0;
  args.alpha = alpha; args.status = status;
  args.tiles = reinterpret_cast<const TileDesc*>(tiles);
  args.num_tiles_dev = num_tiles_dev;
  clear_fused(args);
  const int ctas = max_tiles < g_sm_count ? max_tiles : g_sm_count;
  set_gemm_attrs();
  switch (bn) {
    case 256: gemm_bf16_kernel<256><<<ctas, 192, Cfg<256>::SMEM_BYTES, stream>>>(tmA, tmB, args); break;
    case 128: gemm_bf16_kernel<128><<<ctas, 192, Cfg<128>::SMEM_BYTES, stream>>>(tmA, tmB, args); break;
    default: gemm_bf16_kernel<64><<<ctas, 192, Cfg<64>::SMEM_BYTES, stream>>>(tmA, tmB, args); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// ------------------------------------------------------------------ fused collectives
// C = epilogue(A * B^T) where one operand (or the contraction) is all-gathered from the peers inside the kernel.
//   gathered: `world` pointers (host array) to every rank's copy of the gathered array [rows, cols], contiguous
//   bf16, symmetric memory; rank r has already written rows [r, r+1) * rows / world of its own copy, and a
//   cross-rank barrier has run since. The local copy is complete when the kernel ends.
//   mode 1: gathered array is A [M, K] (K-major);  mode 2: gathered array is B [N, K] (K-major);
//   mode 3: gathered array is B [K, N] (MN-major, gathered along the contraction); A is local in full, [K, M]
//           with GF_A_MN (weight gradient of a sequence-parallel layer) or [M, K] without (input gradient
//           through row-sharded weights).
//   other / ld_other: the operand that is not gathered. flags: GF_* epilogue bits (operand layout bits are
//   implied by the mode). ready: unsigned [rows / 128], local scratch that persists between calls; epoch: a
//   value that grows by one per call on this buffer.
TB_API int tb_gemm_ag_bf16(const void* const* gathered, int rank, int world, int mode, long long rows, long long cols,
                           const void* other, long long ld_other, void* C, long long ldc, int M, int N, int K,
                           int flags, const void* bias, const void* resid, long long ldr, unsigned* ready,
                           unsigned epoch, int n_aux, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || mode < 1 || mode > 3) return -2;
  if (rows % (128ll * world) || (cols % 8) || (ld_other % 8)) return -2;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  // the gathered operand's layout is fixed by the mode; the other operand keeps the caller's layout bit
  if (mode == 1) flags &= ~GF_A_MN;
  if (mode == 2) flags &= ~GF_B_MN;
  if (mode == 3) flags |= GF_B_MN;       // A keeps the caller's layout: [K, M] (wgrad) or [M, K] (dgrad)
  const bool a_mn = flags & GF_A_MN, b_mn = flags & GF_B_MN;
  const void* local = gathered[rank];
  const void* A = mode == 1 ? local : other;
  const void* B = mode == 1 ? other : local;
  const long long lda = mode == 1 ? cols : ld_other, ldb = mode == 1 ? ld_other : cols;
  const int num_m = (M + BM - 1) / BM;
  if (world == 1) n_aux = 0;
  else if (n_aux <= 0) n_aux = aux_ctas_for((double)(rows - rows / world) * cols * 2.0, 2.0 * M * N * K, world);
  if (n_aux > g_sm_count / 2) n_aux = g_sm_count / 2;
  const int avail = g_sm_count - n_aux;
  int BN = 64;
  for (int cand : {256, 128, 64}) {
    if (cand > 128 && N < 256) continue;
    BN = cand;
    if ((long long)num_m * ((N + cand - 1) / cand) >= (avail * 3) / 5) break;
  }
  const int num_n = (N + BN - 1) / BN;
  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn) r = tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, BM, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmA, A, K, M, lda, BK, 64, 1);
  if (r) return -3;
  if (!b_mn) r = tb_make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, 64, 1);
  if (r) return -4;
  GemmArgs a;
  a.M = M; a.N = N; a.K = K; a.flags = flags; a.C = C; a.ldc = ldc;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  a.ldr = ldr; a.alpha = 1.f; a.status = status; a.tiles = nullptr; a.num_tiles_dev = nullptr;
  clear_fused(a);
  const int tiles = num_m * num_n;
  int n_gemm = tiles < avail ? tiles : avail;
  a.rank = rank; a.world = world;
  if (world > 1) {
    const int jpr = (int)(rows / world / 128);
    a.gemm_ctas = n_gemm; a.aux_kind = 1; a.wait_mode = mode; a.wait_flags = ready; a.wait_epoch = epoch;
    a.own_lo = rank * jpr; a.own_hi = (rank + 1) * jpr;
    if (mode == 1) a.rot_m = (rank * jpr) % num_m;
    if (mode == 2) a.rot_n = (int)((rank * (rows / world)) / BN) % num_n;
    if (mode == 3) a.rot_k = (int)((rank * (rows / world)) / BK);
    for (int p = 0; p < world; ++p) a.copy.src.p[p] = const_cast<void*>(gathered[p]);
    a.copy.dst = reinterpret_cast<char*>(const_cast<void*>(local));
    a.copy.rank_bytes = (rows / world) * cols * 2;
    a.copy.job_bytes = 128 * cols * 2;
    a.copy.jobs_per_rank = jpr;
    int piece = 32768;
    while (a.copy.job_bytes % piece) piece >>= 1;
    a.copy.piece_bytes = piece;
    a.copy.flags = ready;
    a.copy.epoch = epoch;
  }
  set_gemm_attrs();
  const int grid = n_gemm + (world > 1 ? n_aux : 0);
  switch (BN) {
    case 256: gemm_bf16_kernel<256><<<grid, 192, Cfg<256>::SMEM_BYTES, stream>>>(tmA, tmB, a); break;
    case 128: gemm_bf16_kernel<128><<<grid, 192, Cfg<128>::SMEM_BYTES, stream>>>(tmA, tmB, a); break;
    default: gemm_bf16_kernel<64><<<grid, 192, Cfg<64>::SMEM_BYTES, stream>>>(tmA, tmB, a); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// out[M / world, N] = sum over ranks of (A_r * B_r^T)[this rank's rows] (+ resid), the reduce-scatter of a
// row-parallel product, in one kernel. part / done: `world` pointers (host arrays) to every rank's partial
// product buffer ([M, N] bf16 contiguous) and per-block counters (unsigned [M / 128]); both symmetric, a
// cross-rank barrier has run since the previous use of `part`. *total (host) carries the counter target from
// call to call and must evolve identically on all ranks (same shapes in the same order). work: one local int.
TB_API int tb_gemm_rs_bf16(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int flags,
                           const void* const* part, const void* const* done, void* out, const void* resid, int rank,
                           int world, unsigned* total, int* work, int n_aux, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -2;
  if (M % (128 * world) || (N % 64) || (lda % 8) || (ldb % 8) || K <= 0) return -2;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool a_mn = flags & GF_A_MN, b_mn = flags & GF_B_MN;
  flags &= (GF_A_MN | GF_B_MN);
  const int num_m = M / BM;
  if (n_aux <= 0) n_aux = 4;     // a few dedicated reducers overlap with the tiles; all CTAs reduce once tiles end
  if (n_aux > g_sm_count / 2) n_aux = g_sm_count / 2;
  const int avail = g_sm_count - n_aux;
  int BN = 64;
  for (int cand : {256, 128, 64}) {
    if (cand > 128 && N < 256) continue;
    BN = cand;
    if ((long long)num_m * ((N + cand - 1) / cand) >= (avail * 3) / 5) break;
  }
  const int num_n = (N + BN - 1) / BN;
  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn) r = tb_make_tmap_2d_bf16(&tmA, A, M, K, lda, BM, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmA, A, K, M, lda, BK, 64, 1);
  if (r) return -3;
  if (!b_mn) r = tb_make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN, BK, 1);
  else       r = tb_make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, 64, 1);
  if (r) return -4;
  GemmArgs a;
  a.M = M; a.N = N; a.K = K; a.flags = flags;
  a.C = const_cast<void*>(part[rank]); a.ldc = N;
  a.bias = nullptr; a.resid = nullptr; a.ldr = 0; a.alpha = 1.f; a.status = status;
  a.tiles = nullptr; a.num_tiles_dev = nullptr;
  clear_fused(a);
  const int tiles = num_m * num_n;
  const int n_gemm = tiles < avail ? tiles : avail;
  const int tpr = num_m / world;
  *total += 4u * (unsigned)num_n;
  a.gemm_ctas = n_gemm; a.aux_kind = 2; a.rank = rank; a.world = world;
  a.rot_m = (((rank + 1) % world) * tpr) % num_m;
  a.done_flags = reinterpret_cast<unsigned*>(const_cast<void*>(done[rank]));
  for (int p = 0; p < world; ++p) {
    a.red.part.p[p] = const_cast<void*>(part[p]);
    a.red.done.p[p] = const_cast<void*>(done[p]);
  }
  a.red.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.red.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  a.red.tiles_per_rank = tpr;
  a.red.target = *total;
  a.red.work = work;
  if (cudaMemsetAsync(work, 0, sizeof(int), stream) != cudaSuccess) return -5;
  set_gemm_attrs();
  const int grid = n_gemm + n_aux;
  switch (BN) {
    case 256: gemm_bf16_kernel<256><<<grid, 192, Cfg<256>::SMEM_BYTES, stream>>>(tmA, tmB, a); break;
    case 128: gemm_bf16_kernel<128><<<grid, 192, Cfg<128>::SMEM_BYTES, stream>>>(tmA, tmB, a); break;
    default: gemm_bf16_kernel<64><<<grid, 192, Cfg<64>::SMEM_BYTES, stream>>>(tmA, tmB, a); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

namespace {
void set_gemm_attrs() {
  static DeviceOnce once;
  if (once.first()) {
    cudaFuncSetAttribute(gemm_bf16_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Cfg<256>::SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Cfg<128>::SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Cfg<64>::SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Cfg<32>::SMEM_BYTES);
  }
}
}  // namespace
