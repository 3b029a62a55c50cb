// Paged KV cache kernels for the rollout engine.
//
//  * kv_write      : scatter new K / V rows of a step (decode) or of a whole prompt (prefill) into the pages
//                    named by the page table; sequence ids and positions are read from device memory, so
//                    the launch is identical every step and can live in a CUDA graph.
//  * qkv_post      : what sits between the fused q/k/v projection and attention in a decode step, in one
//                    launch: per-head RMS norm of q and k (when the model has it), RoPE of q and k, q back in
//                    place, k and v rows straight into their pages.
//  * paged_decode  : single-query attention over a paged cache with GQA: one CTA per (sequence, kv head,
//                    context split). The query heads of a kv head are the rows of a 16-row mma.sync tile, K / V
//                    stream through a double-buffered cp.async stage and are read with ldmatrix; running
//                    max / sum per query head, partial results of the splits merged by `paged_decode_combine`.
//                    Sliding window and logit soft-cap supported. Memory-bound by construction: every K / V
//                    byte of the sequence is read exactly once per kv head.
//
// The reference keeps only host-side page-table logic (tunix/experimental/generate/*) and runs decode on a
// dense cache through XLA (tunix/generate/sampler.py:732-793); these kernels are the device side of the
// in-framework engine that replaces its vLLM / SGLang integrations.
#include "common.cuh"

using namespace tb;

namespace {

constexpr int MAX_G = 16;       // query heads per kv head handled by one CTA (rows of one mma tile)
constexpr int MAX_SPLIT_TOKENS = 2048;  // context tokens per CTA: a multiple of 64 up to this, chosen by the caller

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

// qkv: [n_tok, (N + 2 KH) * H] rows (q heads, then k heads, then v heads). One warp per (token, head).
template <int H>
__global__ void __launch_bounds__(256)
qkv_post_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, const int* __restrict__ seq_ids,
                const int* __restrict__ pos, const __nv_bfloat16* __restrict__ qw,
                const __nv_bfloat16* __restrict__ kw, float eps, float add_one, const float* __restrict__ cos_t,
                const float* __restrict__ sin_t, const int* __restrict__ page_table, int max_pages, int page_size,
                __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int n_tok, int N, int KH) {
  constexpr int HALF = H / 2, E = H / 64;          // elements per lane in each half
  pdl_trigger();
  pdl_wait();
  const int heads = N + 2 * KH;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)n_tok * heads) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(wid / heads), hh = (int)(wid - (long long)t * heads);
  const int p = pos[t];
  __nv_bfloat16* src = qkv + (long long)t * ld + (long long)hh * H;
  __nv_bfloat16* dst = src;
  if (hh >= N) {
    if (p < 0) return;
    const int page = page_table[(long long)seq_ids[t] * max_pages + p / page_size];
    if (page < 0) return;
    const bool is_k = hh < N + KH;
    const int kvh = is_k ? hh - N : hh - N - KH;
    dst = (is_k ? k_pool : v_pool) + ((long long)page * page_size + p % page_size) * ((long long)KH * H) + (long long)kvh * H;
    if (!is_k) {
      for (int c = lane * 8; c < H; c += 256)
        *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
      return;
    }
  }
  float a[E], b[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    a[e] = __bfloat162float(src[lane * E + e]);
    b[e] = __bfloat162float(src[HALF + lane * E + e]);
  }
  const __nv_bfloat16* w = hh < N ? qw : kw;
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) ss += a[e] * a[e] + b[e] * b[e];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int e = 0; e < E; ++e) {   // rounded to bf16 like the stand-alone norm kernel, so both paths agree
      a[e] = __bfloat162float(__float2bfloat16(a[e] * rstd * (__bfloat162float(w[lane * E + e]) + add_one)));
      b[e] = __bfloat162float(__float2bfloat16(b[e] * rstd * (__bfloat162float(w[HALF + lane * E + e]) + add_one)));
    }
  }
  const int pp = p < 0 ? 0 : p;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float c = cos_t[(long long)pp * HALF + lane * E + e], sn = sin_t[(long long)pp * HALF + lane * E + e];
    dst[lane * E + e] = __float2bfloat16(a[e] * c - b[e] * sn);
    dst[HALF + lane * E + e] = __float2bfloat16(b[e] * c + a[e] * sn);
  }
}

// ---- tensor-core fragments (warp-level mma.sync: with at most 16 query rows per kv head there is no 64/128-row
// tile to give to tcgen05, and the kernel is bound by the K/V stream, not by math) --------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int TILE_KEYS = 64;   // keys staged per pipeline stage; 16 per warp

// byte offset of 16-byte chunk c of row r in a [rows, H] bf16 tile whose 128-byte groups are XOR-swizzled by row
template <int H>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * (H * 2) + (((c & ~7) | ((c ^ r) & 7)) << 4));
}

// byte offset of chunk c of key row r inside a staged K or V tile. TMA stages a tile as H/64 slabs of [64 rows x
// 128 bytes] with the hardware's 128-byte swizzle; the cp.async path keeps whole rows together.
template <int H, bool TMA>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  if (TMA) return (uint32_t)((c >> 3) * (TILE_KEYS * 128) + r * 128 + (((c ^ r) & 7) << 4));
  return swz<H>(r, c);
}

// One CTA per (sequence, kv head, context split): the G (<= 16) query heads of the kv head are the 16 rows of the
// A operand, a warp owns 16 keys of each 64-key stage, S = Q K^T and O += P V run on mma.sync and read K / V with
// ldmatrix; every K / V byte is read once. Staging: with pages of a multiple of 64 tokens a tile lies in one page
// and one thread fetches it with TMA (two tensor-map boxes per 64 head dims, STAGES deep, mbarrier completion);
// otherwise all threads gather rows with cp.async (double buffered). The TMA path reads whole 64-token tiles, so
// the unused tail of a page must hold finite values (pages start zeroed and only ever receive K / V rows).
template <int H, bool TMA, int STAGES>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __nv_bfloat16* __restrict__ q, long long ldq,        // [B, N*H]
                    const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                    const int* __restrict__ page_table, int max_pages, int page_size,
                    const int* __restrict__ seq_ids, const int* __restrict__ seq_lens, int KH, int G, float scale,
                    float softcap, int window, int num_splits, int split_tokens,
                    float* __restrict__ part_acc,                                               // [B, N, splits, H]
                    float* __restrict__ part_ml,                                                // [B, N, splits, 2]
                    __nv_bfloat16* __restrict__ out, long long ldo,   // written directly when there is one split
                    int* __restrict__ status) {
  constexpr int CPR = H / 8;                       // 16-byte chunks per row
  constexpr int TILE_BYTES = TILE_KEYS * H * 2;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(128) uint8_t q_s[16 * H * 2];
  __shared__ __align__(8) unsigned long long full_bars[STAGES];
  __shared__ int abort_flag;
  // TMA tiles are 1024-byte aligned (the launch adds the slack for it)
  uint8_t* smem = smem_raw + (TMA ? ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u) : 0u);
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = KH * G;
  const int len = seq_lens[b];
  int lo = split * split_tokens;
  if (lo >= len) {                // past the end of this sequence: the combine kernel never reads this split
    if (num_splits == 1)          // (an empty slot with a single split: its output row is zero)
      for (int idx = threadIdx.x; idx < G * H; idx += 128)
        out[(long long)b * ldo + (long long)(kh * G) * H + idx] = __float2bfloat16(0.f);
    return;
  }
  const int hi = min(len, lo + split_tokens);
  if (window > 0) lo = max(lo, len - window);
  const int* pt = page_table + (long long)seq_ids[b] * max_pages;
  const long long row_elems = (long long)KH * H;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t q_base = smem_u32(q_s);

  // queries -> shared (rows >= G are zero)
  for (int idx = tid; idx < 16 * CPR; idx += 128) {
    const int r = idx / CPR, c = idx - r * CPR;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < G) u = *reinterpret_cast<const uint4*>(q + (long long)b * ldq + (long long)(kh * G + r) * H + c * 8);
    *reinterpret_cast<uint4*>(q_s + swz<H>(r, c)) = u;
  }

  const int t_first = split * split_tokens + ((max(lo - split * split_tokens, 0)) / TILE_KEYS) * TILE_KEYS;
  const int n_tiles = hi > t_first ? (hi - t_first + TILE_KEYS - 1) / TILE_KEYS : 0;

  if (TMA) {
    if (tid == 0) {
      for (int i = 0; i < STAGES; ++i) mbar_init(smem_u32(&full_bars[i]), 1);
      abort_flag = 0;
      mbar_fence_init();
    }
    __syncthreads();
  }
  // one thread, one tile: the tile's 64 tokens lie in one page
  auto issue_tma = [&](int tile, int buf) {
    const int t0 = t_first + tile * TILE_KEYS;
    const int row = pt[t0 / page_size] * page_size + t0 % page_size;
    const uint32_t kb = smem_base + buf * 2 * TILE_BYTES, vb = kb + TILE_BYTES;
    const uint32_t bar = smem_u32(&full_bars[buf]);
    mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
    for (int j = 0; j < H / 64; ++j) {
      tma_load_2d(kb + j * (TILE_KEYS * 128), &tmK, bar, kh * H + j * 64, row);
      tma_load_2d(vb + j * (TILE_KEYS * 128), &tmV, bar, kh * H + j * 64, row);
    }
  };
  auto issue = [&](int tile, int buf) {
    const int t0 = t_first + tile * TILE_KEYS;
    const uint32_t kb = smem_base + buf * 2 * TILE_BYTES, vb = kb + TILE_BYTES;
    for (int idx = tid; idx < TILE_KEYS * CPR; idx += 128) {
      const int r = idx / CPR, c = idx - r * CPR;
      const int t = t0 + r;
      const bool ok = t >= lo && t < hi;
      long long off = 0;
      if (ok) {
        const int page = pt[t / page_size];
        off = ((long long)page * page_size + t % page_size) * row_elems + (long long)kh * H + c * 8;
      }
      const uint32_t d = swz<H>(r, c);
      cp_async16(kb + d, k_pool + off, ok ? 16 : 0);
      cp_async16(vb + d, v_pool + off, ok ? 16 : 0);
    }
    cp_async_commit();
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[H / 8][4];
#pragma unroll
  for (int i = 0; i < H / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  if (TMA) {
    if (tid == 0)
      for (int i = 0; i < STAGES - 1 && i < n_tiles; ++i) issue_tma(i, i);
  } else if (n_tiles > 0) {
    issue(0, 0);
  }
  const int li = lane >> 3, lr = lane & 7;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = TMA ? tile % STAGES : (tile & 1);
    if (TMA) {
      // the buffer of tile + STAGES - 1 was read in the previous iteration, which ended with a barrier
      if (tid == 0 && tile + STAGES - 1 < n_tiles) issue_tma(tile + STAGES - 1, (tile + STAGES - 1) % STAGES);
      if (!mbar_wait_bounded(smem_u32(&full_bars[buf]), (tile / STAGES) & 1, &abort_flag, status, ST_TIMEOUT_PRODUCER)) break;
    } else {
      if (tile + 1 < n_tiles) {
        issue(tile + 1, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
    }
    const uint32_t kb = smem_base + buf * 2 * TILE_BYTES, vb = kb + TILE_BYTES;
    const int kr0 = warp * 16;
    const int tw = t_first + tile * TILE_KEYS + kr0;      // first key of this warp's slice
    if (tw < hi) {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < H / 16; ++ks) {
        uint32_t a[4], kf[4];
        ldsm_x4(a, q_base + swz<H>((li & 1) * 8 + lr, ks * 2 + (li >> 1)));
        ldsm_x4(kf, kb + tile_off<H, TMA>(kr0 + (li >> 1) * 8 + lr, ks * 2 + (li & 1)));
        mma_16816(s[0], a, kf[0], kf[1]);
        mma_16816(s[1], a, kf[2], kf[3]);
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int t = tw + nb * 8 + 2 * (lane & 3) + (j & 1);
          float v = s[nb][j] * scale;
          if (softcap > 0.f) v = softcap * tanhf(v / softcap);
          if (t < lo || t >= hi) v = -INFINITY;
          s[nb][j] = v;
          if (j < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float c0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - mn0);
      const float c1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mn1);
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        s[nb][0] = (s[nb][0] == -INFINITY) ? 0.f : __expf(s[nb][0] - mn0);
        s[nb][1] = (s[nb][1] == -INFINITY) ? 0.f : __expf(s[nb][1] - mn0);
        s[nb][2] = (s[nb][2] == -INFINITY) ? 0.f : __expf(s[nb][2] - mn1);
        s[nb][3] = (s[nb][3] == -INFINITY) ? 0.f : __expf(s[nb][3] - mn1);
        ps0 += s[nb][0] + s[nb][1];
        ps1 += s[nb][2] + s[nb][3];
      }
      l0 = l0 * c0 + ps0;
      l1 = l1 * c1 + ps1;
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int d2 = 0; d2 < H / 16; ++d2) {
        uint32_t vf[4];
        ldsm_x4_t(vf, vb + tile_off<H, TMA>(kr0 + (li & 1) * 8 + lr, d2 * 2 + (li >> 1)));
        float* oa = o[2 * d2];
        float* ob = o[2 * d2 + 1];
        oa[0] *= c0; oa[1] *= c0; oa[2] *= c1; oa[3] *= c1;
        ob[0] *= c0; ob[1] *= c0; ob[2] *= c1; ob[3] *= c1;
        mma_16816(o[2 * d2], pa, vf[0], vf[1]);
        mma_16816(o[2 * d2 + 1], pa, vf[2], vf[3]);
      }
    }
    __syncthreads();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // merge the four warps' partial states through shared memory (the stage buffers are free now)
  float* sm_acc = reinterpret_cast<float*>(smem);             // [4][16][H]
  __shared__ float sm_m[4][16], sm_l[4][16];
  const int r0 = lane >> 2, r1 = r0 + 8, cq = 2 * (lane & 3);
  if ((lane & 3) == 0) {
    sm_m[warp][r0] = m0; sm_l[warp][r0] = l0;
    sm_m[warp][r1] = m1; sm_l[warp][r1] = l1;
  }
#pragma unroll
  for (int db = 0; db < H / 8; ++db) {
    float* a0 = sm_acc + ((warp * 16 + r0) * H + db * 8 + cq);
    float* a1 = sm_acc + ((warp * 16 + r1) * H + db * 8 + cq);
    a0[0] = o[db][0]; a0[1] = o[db][1];
    a1[0] = o[db][2]; a1[1] = o[db][3];
  }
  __syncthreads();
  for (int idx = tid; idx < G * H; idx += 128) {
    const int g = idx / H, d = idx - g * H;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (sm_m[w][g] == -INFINITY) ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * c;
      aa += sm_acc[(w * 16 + g) * H + d] * c;
    }
    if (num_splits == 1) {                 // the whole context in this CTA: no partial state, no combine kernel
      out[(long long)b * ldo + (long long)(kh * G + g) * H + d] = __float2bfloat16(ll > 0.f ? aa / ll : 0.f);
      continue;
    }
    const long long oidx = (((long long)b * N + kh * G + g) * num_splits + split);
    part_acc[oidx * H + d] = aa;
    if (d == 0) {
      part_ml[oidx * 2] = mm;
      part_ml[oidx * 2 + 1] = ll;
    }
  }
}

// out[b, n, :] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)
__global__ void paged_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                            const int* __restrict__ seq_lens, int N, int H, int num_splits, int split_tokens,
                                            int window, __nv_bfloat16* __restrict__ out, long long ldo) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, n = blockIdx.y;
  const int len = seq_lens[b];
  const int used = min(num_splits, (len + split_tokens - 1) / split_tokens);
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

template <int H, bool TMA, int STAGES>
int launch_decode_v(int G, dim3 grid, cudaStream_t stream, const CUtensorMap& tmK, const CUtensorMap& tmV,
                    const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* kp, const __nv_bfloat16* vp, const int* pt,
                    int max_pages, int page_size, const int* seq_ids, const int* seq_lens, int KH, float scale, float softcap,
                    int window, int splits, int split_tokens, float* pa, float* pml, __nv_bfloat16* out, long long ldo,
                    int* status) {
  constexpr int TILE2 = 2 * TILE_KEYS * H * 2;                       // one stage: a K tile and a V tile
  constexpr int SMEM = STAGES * TILE2 + (TMA ? 1024 : 0);
  static DeviceOnce once;
  if (once.first() &&
      cudaFuncSetAttribute(paged_decode_kernel<H, TMA, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
    return -5;
  // a split of one 64-key tile needs one stage only: more CTAs fit on an SM
  const int smem = split_tokens > TILE_KEYS ? SMEM : TILE2 + (TMA ? 1024 : 0);
  return launch_pdl(paged_decode_kernel<H, TMA, STAGES>, grid, dim3(128), smem, stream, tmK, tmV, q, ldq, kp, vp, pt, max_pages,
                    page_size, seq_ids, seq_lens, KH, G, scale, softcap, window, splits, split_tokens, pa, pml, out, ldo,
                    status) == cudaSuccess ? 0 : -5;
}

// TMA staging needs tiles that lie inside one page.
template <int H>
int launch_decode(int G, dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, long long ldq,
                  const __nv_bfloat16* kp, const __nv_bfloat16* vp, long long pool_rows, const int* pt, int max_pages,
                  int page_size, const int* seq_ids, const int* seq_lens, int KH, float scale, float softcap, int window,
                  int splits, int split_tokens, float* pa, float* pml, __nv_bfloat16* out, long long ldo, int* status) {
  static const bool no_tma = getenv("TUNIX_B200_DECODE_NO_TMA") != nullptr;
  static const char* stages_env = getenv("TUNIX_B200_DECODE_STAGES");
  CUtensorMap tmK, tmV;
  memset(&tmK, 0, sizeof(tmK));
  memset(&tmV, 0, sizeof(tmV));
  const bool tma = !no_tma && page_size % TILE_KEYS == 0 && pool_rows > 0 &&
                   tb_make_tmap_2d_bf16(&tmK, kp, (uint64_t)pool_rows, (uint64_t)KH * H, (uint64_t)KH * H, TILE_KEYS, 64, 1) == 0 &&
                   tb_make_tmap_2d_bf16(&tmV, vp, (uint64_t)pool_rows, (uint64_t)KH * H, (uint64_t)KH * H, TILE_KEYS, 64, 1) == 0;
#define LD(T, S) launch_decode_v<H, T, S>(G, grid, stream, tmK, tmV, q, ldq, kp, vp, pt, max_pages, page_size, seq_ids, seq_lens, \
                                         KH, scale, softcap, window, splits, split_tokens, pa, pml, out, ldo, status)
  if (!tma) return LD(false, 2);
  // measured at head dim 128 (8 kv heads, 256 sequences x 768 tokens): 2 / 3 / 4 stages take 157 / 161 / 194 us,
  // cp.async staging 190 us: three CTAs per SM with two stages each beat deeper rings on fewer CTAs
  const int want = stages_env ? atoi(stages_env) : 2;
  if (want <= 2) return LD(true, 2);
  if (want == 3 || H >= 256) return LD(true, 3);
  return LD(true, 4);
#undef LD
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

// Fused decode-side epilogue of the q/k/v projection (see qkv_post_kernel). qw / kw null = no QK norm.
TB_API int tb_qkv_post(void* qkv, long long ld, const int* seq_ids, const int* pos, const void* qw, const void* kw,
                       float eps, float add_one, const float* cos_t, const float* sin_t, const int* page_table,
                       int max_pages, int page_size, void* k_pool, void* v_pool, int n_tok, int N, int KH, int H,
                       cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  if (ld % 8) return -2;
  const long long warps = (long long)n_tok * (N + 2 * KH);
  const int grid = (int)((warps + 7) / 8);
  cudaError_t err = cudaSuccess;
#define QP(HV)                                                                                                     \
  err = launch_pdl(qkv_post_kernel<HV>, dim3(grid), dim3(256), 0, stream, (__nv_bfloat16*)qkv, ld, seq_ids, pos,     \
                   (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, eps, add_one, cos_t, sin_t, page_table,       \
                   max_pages, page_size, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_tok, N, KH)
  switch (H) {
    case 64: QP(64); break;
    case 128: QP(128); break;
    case 256: QP(256); break;
    default: return -2;
  }
#undef QP
  return err == cudaSuccess ? 0 : -5;
}

// q [B, N*H]; pools [num_pages, page_size, KH*H]; page_table [*, max_pages]; seq_ids [B]; seq_lens [B];
// workspace: part_acc fp32 [B*N*splits*H], part_ml fp32 [B*N*splits*2] with splits = ceil(max_ctx / split_tokens);
// split_tokens = context tokens per CTA, a multiple of 64 in [64, 2048] (0 = 256). CTAs of splits that lie past the
// end of their sequence return at once. pool_rows = num_pages * page_size (rows of the pools, for the tensor maps;
// 0 = no TMA staging). status: word that a bounded mbarrier wait writes its code to.
TB_API int tb_paged_decode(const void* q, long long ldq, const void* k_pool, const void* v_pool,
                           const int* page_table, int max_pages, int page_size, const int* seq_ids,
                           const int* seq_lens, int B, int N, int KH, int H, int max_ctx, float scale, float softcap,
                           int window, int split_tokens, long long pool_rows, float* part_acc, float* part_ml, void* out,
                           long long ldo, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (KH <= 0 || N % KH || (ldq % 8)) return -2;
  const int G = N / KH;
  if (G > MAX_G) return -2;
  if (split_tokens <= 0) split_tokens = 256;
  if (split_tokens % TILE_KEYS || split_tokens > MAX_SPLIT_TOKENS) return -2;
  const int splits = (max_ctx + split_tokens - 1) / split_tokens;
  dim3 grid(B, KH, splits);
  int rc;
  auto qq = (const __nv_bfloat16*)q;
  auto kp = (const __nv_bfloat16*)k_pool;
  auto vp = (const __nv_bfloat16*)v_pool;
  switch (H) {
    case 64: rc = launch_decode<64>(G, grid, stream, qq, ldq, kp, vp, pool_rows, page_table, max_pages, page_size, seq_ids, seq_lens, KH, scale, softcap, window, splits, split_tokens, part_acc, part_ml, (__nv_bfloat16*)out, ldo, status); break;
    case 128: rc = launch_decode<128>(G, grid, stream, qq, ldq, kp, vp, pool_rows, page_table, max_pages, page_size, seq_ids, seq_lens, KH, scale, softcap, window, splits, split_tokens, part_acc, part_ml, (__nv_bfloat16*)out, ldo, status); break;
    case 256: rc = launch_decode<256>(G, grid, stream, qq, ldq, kp, vp, pool_rows, page_table, max_pages, page_size, seq_ids, seq_lens, KH, scale, softcap, window, splits, split_tokens, part_acc, part_ml, (__nv_bfloat16*)out, ldo, status); break;
    default: return -2;
  }
  if (rc) return rc;
  if (splits == 1) return 0;
  return launch_pdl(paged_decode_combine_kernel, dim3(B, N), dim3(128), 0, stream, (const float*)part_acc,
                    (const float*)part_ml, seq_lens, N, H, splits, split_tokens, window, (__nv_bfloat16*)out, ldo) == cudaSuccess ? 0 : -5;
}

// ------------------------------------------------------------------ per-step bookkeeping of the decode loop
// One thread per running slot does what the continuous-batching loop needs after a token was sampled:
//   a finished (or empty) slot writes the padding token to the spare last column and stays idle;
//   a live slot appends (token, log-prob) at its output cursor, advances the cursor, and finishes when the token is
//   an end-of-sequence id or the cursor reaches the slot's limit; a slot that is still live is fed the token at the
//   next step (position = its current length, length + 1), a finished one idles (position -1, length 0).
// The step counter (Philox offset of the sampling kernel) advances by one.
namespace {
__global__ void decode_advance_kernel(const long long* __restrict__ next, const float* __restrict__ next_lp,
                                      bool* __restrict__ done, long long* __restrict__ out_tokens,
                                      float* __restrict__ out_lp, long long ld_out, long long* __restrict__ out_pos,
                                      const long long* __restrict__ limit, const long long* __restrict__ eos, int n_eos,
                                      long long pad_id, long long* __restrict__ tokens, int* __restrict__ positions,
                                      int* __restrict__ seq_lens, int* __restrict__ step, int B) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *step += 1;
  if (i >= B) return;
  const bool was_done = done[i];
  const long long tok = was_done ? pad_id : next[i];
  long long pos = out_pos[i];
  const long long col = was_done ? ld_out - 1 : pos;
  out_tokens[(long long)i * ld_out + col] = tok;
  out_lp[(long long)i * ld_out + col] = next_lp[i];
  if (!was_done) out_pos[i] = ++pos;
  bool fin = was_done || pos >= limit[i];
  for (int e = 0; e < n_eos; ++e) fin = fin || (tok == eos[e]);
  done[i] = fin;
  tokens[i] = tok;
  const int len = seq_lens[i];
  positions[i] = fin ? -1 : len;
  seq_lens[i] = fin ? 0 : len + 1;
}
}  // namespace

TB_API int tb_decode_advance(const long long* next, const float* next_lp, void* done, long long* out_tokens, float* out_lp,
                             long long ld_out, long long* out_pos, const long long* limit, const long long* eos, int n_eos,
                             long long pad_id, long long* tokens, int* positions, int* seq_lens, int* step, int B,
                             cudaStream_t stream) {
  if (B <= 0) return 0;
  return launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, next, next_lp,
                    reinterpret_cast<bool*>(done), out_tokens, out_lp, ld_out, out_pos, limit, eos, n_eos, pad_id, tokens,
                    positions, seq_lens, step, B) == cudaSuccess ? 0 : -5;
}
