// Paged causal attention for bfloat16 on the tensor cores (mma.sync m16n8k16, float accumulation),
// one kernel for prompt portions and for decoded tokens.
//
// Work is cut per (request, kv head): the G = H / Hkv query heads that share a kv head are folded into the
// row dimension, row m of a request's tile standing for (token m / G, head hk*G + m % G), so a key/value
// tile is fetched once for the whole group. Two shapes of thread block exist:
//   * "wide" (4 warps x 16 rows = 64 rows, every warp walks all keys of a 64-key tile): prompt portions;
//   * "deep" (16 rows, the warps deal the keys out among themselves, each with a pipeline of its own, results
//     merged through shared memory; the key range may also be split over several blocks whose partial
//     results the block that finishes last merges): requests that bring at most 16 / G tokens, i.e. decoding.
// A request is handled by the shape its row count fits; the other shape's blocks leave it alone.
//
// Scores, running maxima, sums and outputs are float; probabilities are rounded to bfloat16 for the
// second product, as the reference does (serve/kernels/attn_prefill.py:71, attn_decode.py:110). The
// recurrences are those of attn_prefill.py:58-72 with exp2 and a folded log2(e) (attn_prefill.py:330-331).
// Compile with -DSB_HEAD_DIM=<multiple of 16, 16..256>.
#include <algorithm>
#include <type_traits>

#include "common.cuh"

#ifndef SB_HEAD_DIM
#error "define SB_HEAD_DIM"
#endif

using namespace sb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int D = SB_HEAD_DIM;
constexpr int BN = 64;               // keys per tile
constexpr int LDS = D + 8;           // row stride in shared memory (elements): 16 bytes of padding
constexpr int THREADS = 128;
constexpr int CHUNKS = D / 8;        // 16-byte pieces per row
constexpr float LOG2E = 1.4426950408889634f;

static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head_dim must be a multiple of 16 in 16..256");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // 0: nothing is read, the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct Params {
  const bf16* qkv; int q_stride;
  const bf16* kc; const bf16* vc;
  const int* block_table; int bt_width;
  const int* cu_q; const int* kv_len;
  int H, Hkv, G, ps, num_pages;
  int ps_shift;     // log2(ps) if ps is a power of two, else -1: a shift in place of a division in the key loops
  float scale_log2; int window;
  bf16* out;
  // deep shape only
  int split_size, num_splits;
  float* part_o;    // [R, Hkv, splits, 16, D]
  float* part_ml;   // [R, Hkv, splits, 16, 2]
  int* tickets;     // [R, Hkv] zero before the launch and again after it; nullptr: a separate kernel merges
  // wide shape only
  const int* wide_rows;   // requests the launch covers (blockIdx.z indexes it); nullptr: all, in order
  int heads_in_x;         // wide shape: grid (kv heads, row tiles, requests) rather than (row tiles, kv heads, requests)
};

constexpr int MAX_SPLITS = 32;

// Partial results of all key splits of (request r, kv head hk) -> the output rows. Reads bypass L1: the
// partials were written by other SMs. First the (max, sum) pairs of all splits are fetched at once and turned
// into one factor per (split, row); then every output element adds its S scaled partials, loads unrolled.
// ``work``: (2 * MAX_SPLITS + 1) * 16 floats of shared memory nobody else uses any more.
__device__ __forceinline__ void merge_splits(const Params& p, int r, int hk, int q0, int M, int nthreads, float* work) {
  float (*f_s)[16] = reinterpret_cast<float (*)[16]>(work);
  float* inv_s = work + MAX_SPLITS * 16;
  float* l_s = inv_s + 16;                               // [S][16] sums, beside their maxima
  const int S = p.num_splits;
  const size_t base = ((size_t)r * p.Hkv + hk) * S;
  // With few splits everything is asked for at once: the partial rows of this thread's first element go out together
  // with the (max, sum) pairs, so the merge costs one trip to L2, not three one after the other (this code is the tail
  // of the whole launch: the block that arrives last runs it alone).
  constexpr int EARLY = 16;
  const bool early = S <= EARLY && (int)threadIdx.x < M * D;
  float v[EARLY];
  if (early) {
    const int row = threadIdx.x / D, d = threadIdx.x - row * D;
#pragma unroll
    for (int s_ = 0; s_ < EARLY; ++s_)
      v[s_] = s_ < S ? __ldcg(p.part_o + ((base + s_) * 16 + row) * D + d) : 0.f;
  }
  for (int idx = threadIdx.x; idx < S * 16; idx += nthreads) {
    const int s_ = idx >> 4, row = idx & 15;
    float2 ml = make_float2(-INFINITY, 0.f);
    if (row < M) ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((base + s_) * 16 + row) * 2));
    f_s[s_][row] = ml.x;
    l_s[s_ * 16 + row] = ml.y;
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int row = threadIdx.x;
    float mm = -INFINITY;
    for (int s_ = 0; s_ < S; ++s_) mm = fmaxf(mm, f_s[s_][row]);
    float ll = 0.f;
    for (int s_ = 0; s_ < S; ++s_) {
      const float ms = f_s[s_][row];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      if (f != 0.f) ll += l_s[s_ * 16 + row] * f;
      f_s[s_][row] = f;
    }
    inv_s[row] = ll > 0.f ? 1.f / ll : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < M * D; idx += nthreads) {
    const int row = idx / D, d = idx - row * D;
    float acc = 0.f;
    if (early && idx == (int)threadIdx.x) {
      // a split without keys wrote no partial output: its factor is 0 and its (stale) values are not touched
#pragma unroll
      for (int s_ = 0; s_ < EARLY; ++s_) {
        const float f = s_ < S ? f_s[s_][row] : 0.f;
        acc = f != 0.f ? fmaf(v[s_], f, acc) : acc;
      }
    } else {
      for (int s_ = 0; s_ < S; ++s_) {
        const float f = f_s[s_][row];
        if (f != 0.f) acc = fmaf(__ldcg(p.part_o + ((base + s_) * 16 + row) * D + d), f, acc);
      }
    }
    const int tok = row / p.G, hd = hk * p.G + (row - tok * p.G);
    p.out[(size_t)(q0 + tok) * p.H * D + (size_t)hd * D + d] = __float2bfloat16_rn(acc * inv_s[row]);
  }
}

// Called by every block of a split launch once its partial results are written: the block that arrives last
// merges. Nobody waits for anybody.
__device__ __forceinline__ void finish_split(const Params& p, int r, int hk, int q0, int M, int nthreads, float* work) {
  if (p.tickets == nullptr) return;
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(p.tickets + (size_t)r * p.Hkv + hk, 1);
    s_last = (t == p.num_splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  merge_splits(p, r, hk, q0, M, nthreads, work);
  if (threadIdx.x == 0) p.tickets[(size_t)r * p.Hkv + hk] = 0;
}

constexpr int BT_CACHE = 256;        // block-table entries a thread block keeps in shared memory

// Fetch keys [kt, kt+BN) of kv head hk into one stage of shared memory; keys outside [lo, hi) become zeros.
// bt points at the table entry of block bt_first (shared memory copy, or the table itself with bt_first 0).
__device__ __forceinline__ void load_kv_tile(const Params& p, const int* bt, int bt_first, int hk, int kt, int lo, int hi, bf16* Ks,
                                             bf16* Vs) {
#pragma unroll
  for (int idx = threadIdx.x; idx < BN * CHUNKS; idx += THREADS) {
    const int row = idx / CHUNKS, ch = idx - row * CHUNKS;
    const int key = kt + row;
    bool ok = key >= lo && key < hi;
    size_t off = 0;
    if (ok) {
      const int blk = p.ps_shift >= 0 ? (key >> p.ps_shift) : key / p.ps;
      const int page = blk < p.bt_width ? bt[blk - bt_first] : -1;
      ok = page >= 0 && page < p.num_pages;
      if (ok) off = (((size_t)page * p.Hkv + hk) * p.ps + (key - blk * p.ps)) * D + ch * 8;
    }
    cp_async16(Ks + row * LDS + ch * 8, p.kc + off, ok);
    cp_async16(Vs + row * LDS + ch * 8, p.vc + off, ok);
  }
}

// WM warps along rows, WN warps along the keys of a tile (WM * WN == 4).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The wide shape: requests with more than 16 rows (prompt portions). grid (row tiles of 64, Hkv, R), 4 warps,
// each warp 16 rows against all 64 keys of a tile; two stages of keys/values. Tiles wholly below every row's
// position (and inside every row's window) skip the mask; the heaviest row tiles (the last ones) start first.
constexpr bool WQ_IN_REGS = D <= 128;

__global__ void __launch_bounds__(THREADS, (D <= 64 ? 4 : 1)) attention_wide_kernel(const Params p) {
  constexpr int BM = 64;
  constexpr int NT = BN / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int bt_s[BT_CACHE];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);     // [BM][LDS]
  bf16* KVs = Qs + BM * LDS;                        // 2 stages x (K [BN][LDS], V [BN][LDS])

  // blocks start in the order of blockIdx.x, then y: with the heads in x the longest tiles of all heads start first
  const int r = p.wide_rows ? p.wide_rows[blockIdx.z] : (int)blockIdx.z;
  const int hk = p.heads_in_x ? blockIdx.x : blockIdx.y, bx = p.heads_in_x ? blockIdx.y : blockIdx.x;
  const int q0 = p.cu_q[r], qn = p.cu_q[r + 1] - q0;
  const int G = p.G;
  const int M = qn * G;                             // rows of this (request, kv head)
  if (M <= 16) return;                              // the deep shape takes this request
  const int n_mtiles = (M + BM - 1) / BM;
  if (bx >= n_mtiles) return;
  const int m0 = (n_mtiles - 1 - bx) * BM;          // later rows see more keys: they go first
  const int L = p.kv_len[r];
  const int p0 = L - qn;                            // position of the request's first query
  const int tok_first = m0 / G, row_last = min(m0 + BM, M) - 1;
  const int lo = p.window > 0 ? max(0, p0 + tok_first - p.window + 1) : 0;
  const int hi = p0 + row_last / G + 1;             // exclusive, <= L
  // keys every row of the tile may see without a mask
  const int free_lo = p.window > 0 ? max(lo, p0 + row_last / G - p.window + 1) : lo;
  const int free_hi = min(hi, p0 + tok_first + 1);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int* bt = p.block_table + (size_t)r * p.bt_width;
  int bt_first = 0;

  for (int idx = tid; idx < BM * CHUNKS; idx += THREADS) {
    const int row = idx / CHUNKS, ch = idx - row * CHUNKS;
    const int m = m0 + row;
    const bool ok = m < M;
    const int tok = ok ? m / G : 0, hd = ok ? hk * G + (m - tok * G) : 0;
    cp_async16(Qs + row * LDS + ch * 8, p.qkv + (size_t)(q0 + tok) * p.q_stride + (size_t)hd * D + ch * 8, ok);
  }
  const int kt0 = (lo / BN) * BN;
  const int n_tiles = (hi - kt0 + BN - 1) / BN;
  {
    const int b_lo = lo / p.ps, b_hi = min((hi - 1) / p.ps, p.bt_width - 1);
    if (b_hi - b_lo + 1 <= BT_CACHE) {
      for (int i = tid; i <= b_hi - b_lo; i += THREADS) bt_s[i] = bt[b_lo + i];
      __syncthreads();
      bt = bt_s;
      bt_first = b_lo;
    }
  }
  load_kv_tile(p, bt, bt_first, hk, kt0, lo, hi, KVs, KVs + BN * LDS);
  cp_async_commit();

  const int row_a = m0 + warp * 16 + g, row_b = row_a + 8;
  const int pos_a = row_a < M ? p0 + row_a / G : -1, pos_b = row_b < M ? p0 + row_b / G : -1;
  uint32_t qf[WQ_IN_REGS ? D / 16 : 1][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    const int kt = kt0 + it * BN;
    bf16* Ks = KVs + (it & 1) * 2 * BN * LDS;
    bf16* Vs = Ks + BN * LDS;
    if (it + 1 < n_tiles) {
      bf16* Kn = KVs + ((it + 1) & 1) * 2 * BN * LDS;
      load_kv_tile(p, bt, bt_first, hk, kt + BN, lo, hi, Kn, Kn + BN * LDS);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (WQ_IN_REGS && it == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], Qs + (warp * 16 + (lane & 15)) * LDS + kk * 16 + (lane >> 4) * 8);
    }
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      if (WQ_IN_REGS) {
        a0 = qf[kk][0]; a1 = qf[kk][1]; a2 = qf[kk][2]; a3 = qf[kk][3];
      } else {
        ldmatrix_x4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 15)) * LDS + kk * 16 + (lane >> 4) * 8);
      }
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane >> 4) * 8 + (lane & 7)) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    float mx_a = -INFINITY, mx_b = -INFINITY;
    if (kt >= free_lo && kt + BN <= free_hi) {
      // (rows beyond M hold zero queries; what they compute is finite and never stored)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        s[j][0] *= p.scale_log2; s[j][1] *= p.scale_log2; s[j][2] *= p.scale_log2; s[j][3] *= p.scale_log2;
        mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = kt + j * 8 + tq * 2 + e;
          const bool in_range = key >= lo && key < hi;
          const bool ok_a = in_range && key <= pos_a && (p.window <= 0 || key > pos_a - p.window);
          const bool ok_b = in_range && key <= pos_b && (p.window <= 0 || key > pos_b - p.window);
          s[j][e] = ok_a ? s[j][e] * p.scale_log2 : -INFINITY;
          s[j][2 + e] = ok_b ? s[j][2 + e] * p.scale_log2 : -INFINITY;
          mx_a = fmaxf(mx_a, s[j][e]);
          mx_b = fmaxf(mx_b, s[j][2 + e]);
        }
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a, use_b = (mn_b == -INFINITY) ? 0.f : mn_b;
    const float al_a = ex2(m_a - use_a), al_b = ex2(m_b - use_b);   // ex2(-inf) = 0: nothing was accumulated yet
    m_a = mn_a; m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t pa[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const float p0_ = ex2(s[j][0] - use_a), p1_ = ex2(s[j][1] - use_a);
      const float p2_ = ex2(s[j][2] - use_b), p3_ = ex2(s[j][3] - use_b);
      sum_a += p0_ + p1_;
      sum_b += p2_ + p3_;
      pa[j][0] = pack_bf16(p0_, p1_);
      pa[j][1] = pack_bf16(p2_, p3_);
    }
    l_a = l_a * al_a + sum_a;
    l_b = l_b * al_b + sum_b;
    if (__any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b;
      }
    }
#pragma unroll
    for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
      for (int i = 0; i < D / 8; i += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + i * 8 + (lane >> 4) * 8);
        mma_bf16(o[i], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b0, b1);
        mma_bf16(o[i + 1], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b2, b3);
      }
    }
    __syncthreads();   // the stage may be overwritten by the next iteration's fetch
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  if (row_a < M) {
    const int tok = row_a / G, hd = hk * G + (row_a - tok * G);
    bf16* dst = p.out + (size_t)(q0 + tok) * p.H * D + (size_t)hd * D + tq * 2;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
  }
  if (row_b < M) {
    const int tok = row_b / G, hd = hk * G + (row_b - tok * G);
    bf16* dst = p.out + (size_t)(q0 + tok) * p.H * D + (size_t)hd * D + tq * 2;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
  }
}

size_t wide_smem_bytes() { return (size_t)(64 + 2 * 2 * BN) * LDS * sizeof(bf16); }

// The deep shape, for requests with at most 16 rows (decoding). grid (splits, Hkv, R), 4 warps. The keys of the
// block's split are dealt to the warps in sub-tiles of DKW (warp w takes sub-tiles w, w+4, ...); every warp runs
// a cp.async pipeline of its own over private shared memory, so no block-wide barrier sits in the loop and
// the warps hide one another's latencies. The four partial results meet in shared memory at the end.
// The loop is written for few instructions per byte: a sub-tile lies in one page whenever the page size is a
// multiple of DKW (one table lookup, contiguous source rows); tiles away from the edges of the key range skip
// the mask; rows 8..15 of the tile are only computed when the request has that many (UPPER).
constexpr int DKW = D <= 64 ? 32 : 16;                    // keys per warp per step
constexpr int DNT = DKW / 8;                              // score n-tiles per step
constexpr int DSTAGES = 2;                                 // steps in flight per warp
constexpr bool DQ_IN_REGS = D <= 128;                     // query fragments live in registers
constexpr int DCOPIES = DKW * CHUNKS / 32;                // 16-byte copies per lane per sub-tile and tensor

// Sub-tile of keys [k0, k0 + DKW) of kv head hk -> one stage. Keys outside [lo, hi) become zeros.
__device__ __forceinline__ void load_kv_subtile(const Params& p, const int* bt, int bt_first, int hk, int k0, int lo, int hi,
                                                bool same_page, bf16* Ks, bf16* Vs, int lane) {
  if (same_page) {
    const int blk = p.ps_shift >= 0 ? (k0 >> p.ps_shift) : k0 / p.ps;
    const int page = blk < p.bt_width ? bt[blk - bt_first] : -1;
    const bool page_ok = page >= 0 && page < p.num_pages;
    const size_t base = (((size_t)(page_ok ? page : 0) * p.Hkv + hk) * p.ps + (k0 - blk * p.ps)) * D;
    const bool inner = page_ok && k0 >= lo && k0 + DKW <= hi;
#pragma unroll
    for (int i = 0; i < DCOPIES; ++i) {
      const int c = lane + 32 * i;
      const int row = c / CHUNKS, ch = c - row * CHUNKS;
      const bool ok = inner || (page_ok && k0 + row >= lo && k0 + row < hi);
      cp_async16(Ks + row * LDS + ch * 8, p.kc + base + (size_t)c * 8, ok);
      cp_async16(Vs + row * LDS + ch * 8, p.vc + base + (size_t)c * 8, ok);
    }
    return;
  }
  if (DKW == 32 && p.ps == 16) {
    // pages of 16 tokens under sub-tiles of 32 keys: two pages, looked up once each; which of the two a copy belongs
    // to is known when the loop is unrolled (row = (lane + 32 i) / CHUNKS)
    const int blk = k0 >> 4;
    const int page_a = blk < p.bt_width ? bt[blk - bt_first] : -1, page_b = blk + 1 < p.bt_width ? bt[blk + 1 - bt_first] : -1;
    const bool ok_a = page_a >= 0 && page_a < p.num_pages, ok_b = page_b >= 0 && page_b < p.num_pages;
    const size_t base_a = ((size_t)(ok_a ? page_a : 0) * p.Hkv + hk) * 16 * D, base_b = ((size_t)(ok_b ? page_b : 0) * p.Hkv + hk) * 16 * D;
    const bool inner = k0 >= lo && k0 + DKW <= hi;
#pragma unroll
    for (int i = 0; i < DCOPIES; ++i) {
      const int c = lane + 32 * i;
      const int row = c / CHUNKS, ch = c - row * CHUNKS;
      const bool second = row >= 16;
      const bool ok = (second ? ok_b : ok_a) && (inner || (k0 + row >= lo && k0 + row < hi));
      const size_t off = (second ? base_b : base_a) + (size_t)(row & 15) * D + ch * 8;
      cp_async16(Ks + row * LDS + ch * 8, p.kc + off, ok);
      cp_async16(Vs + row * LDS + ch * 8, p.vc + off, ok);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < DCOPIES; ++i) {
    const int c = lane + 32 * i;
    const int row = c / CHUNKS, ch = c - row * CHUNKS;
    const int key = k0 + row;
    bool ok = key >= lo && key < hi;
    size_t off = 0;
    if (ok) {
      const int blk = p.ps_shift >= 0 ? (key >> p.ps_shift) : key / p.ps;
      const int page = blk < p.bt_width ? bt[blk - bt_first] : -1;
      ok = page >= 0 && page < p.num_pages;
      if (ok) off = (((size_t)page * p.Hkv + hk) * p.ps + (key - blk * p.ps)) * D + ch * 8;
    }
    cp_async16(Ks + row * LDS + ch * 8, p.kc + off, ok);
    cp_async16(Vs + row * LDS + ch * 8, p.vc + off, ok);
  }
}

// NWARPS: 4 when many blocks share an SM, 8 when a block has an SM to itself (small batches).
template <bool UPPER, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32) attention_deep_kernel(const Params p) {
  constexpr int NTHR = NWARPS * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int bt_s[BT_CACHE];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][LDS]
  bf16* KVs = Qs + 16 * LDS;                                    // [NWARPS][DSTAGES][K DKWxLDS, V DKWxLDS]

  const int r = blockIdx.z, hk = blockIdx.y, split = blockIdx.x;
  const int q0 = p.cu_q[r], qn = p.cu_q[r + 1] - q0;
  const int G = p.G;
  const int M = qn * G;
  // A block with nothing to do still waits for the kernel before this one: the kernel after this one waits only for
  // this one, so a launch whose blocks all left at once would let it run ahead of everything before.
  if (M > 16 || M <= 0) { pdl_wait(); return; }                 // the wide shape takes this request
  if (UPPER != (M > 8)) { pdl_wait(); return; }                 // the other instantiation takes this request
  const int L = p.kv_len[r];
  const int p0 = L - qn;
  int lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
  int hi = p0 + (M - 1) / G + 1;
  {
    // the request's keys are shared out evenly over the launch's splits, in units of one step of all the block's
    // warps. The splits start at the unit boundary at or below the first key, so their size is taken from there:
    // sized from the first key itself they could end before the last one.
    constexpr int UNIT = NWARPS * DKW;
    const int base = (lo / UNIT) * UNIT;
    const int split_size = max(UNIT, ((hi - base + p.num_splits - 1) / p.num_splits + UNIT - 1) / UNIT * UNIT);
    lo = max(lo, base + split * split_size);
    hi = min(hi, base + (split + 1) * split_size);
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int* bt = p.block_table + (size_t)r * p.bt_width;
  int bt_first = 0;

  if (lo >= hi) {
    pdl_launch_dependents();
    pdl_wait();
    if (p.num_splits > 1) {
      if (tid < 16) {
        float* ml = p.part_ml + ((((size_t)r * p.Hkv + hk) * p.num_splits + split) * 16 + tid) * 2;
        ml[0] = -INFINITY; ml[1] = 0.f;
      }
      finish_split(p, r, hk, q0, M, NTHR, reinterpret_cast<float*>(smem_raw));
    } else {
      // no key at all (a length below the token count): the rows are zeros, as a sum over nothing
      for (int idx = tid; idx < M * D; idx += NTHR) {
        const int row = idx / D, d = idx - row * D;
        const int tok = row / G, hd = hk * G + (row - tok * G);
        p.out[(size_t)(q0 + tok) * p.H * D + (size_t)hd * D + d] = __float2bfloat16_rn(0.f);
      }
    }
    return;
  }
  {
    // lengths and block tables are the step's own inputs: fetched while the kernel before this one finishes
    const int b_lo = lo / p.ps, b_hi = min((hi - 1) / p.ps, p.bt_width - 1);
    if (b_hi - b_lo + 1 <= BT_CACHE) {
      for (int i = tid; i <= b_hi - b_lo; i += NTHR) bt_s[i] = bt[b_lo + i];
      bt = bt_s;
      bt_first = b_lo;
    }
  }
  pdl_launch_dependents();
  pdl_wait();                                                   // queries and this step's keys/values come from earlier kernels
  for (int idx = tid; idx < 16 * CHUNKS; idx += NTHR) {
    const int row = idx / CHUNKS, ch = idx - row * CHUNKS;
    const bool ok = row < M;
    const int tok = ok ? row / G : 0, hd = ok ? hk * G + (row - tok * G) : 0;
    cp_async16(Qs + row * LDS + ch * 8, p.qkv + (size_t)(q0 + tok) * p.q_stride + (size_t)hd * D + ch * 8, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();                                              // queries and table entries are in shared memory

  const bool same_page = (p.ps % DKW) == 0;
  const int k_first = (lo / DKW) * DKW;
  const int n_sub = (hi - k_first + DKW - 1) / DKW;             // sub-tiles of the split
  const int my_n = (n_sub - warp + NWARPS - 1) / NWARPS;        // this warp's share: sub-tiles warp, warp+NWARPS, ...
  bf16* myKV = KVs + (size_t)warp * DSTAGES * 2 * DKW * LDS;
#pragma unroll
  for (int s = 0; s < DSTAGES - 1; ++s) {
    if (s < my_n) load_kv_subtile(p, bt, bt_first, hk, k_first + (warp + NWARPS * s) * DKW, lo, hi, same_page, myKV + s * 2 * DKW * LDS,
                                  myKV + s * 2 * DKW * LDS + DKW * LDS, lane);
    cp_async_commit();
  }
  uint32_t qf[DQ_IN_REGS ? D / 16 : 1][4];
  if (DQ_IN_REGS) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], Qs + (lane & 15) * LDS + kk * 16 + (lane >> 4) * 8);
  }
  const int pos_a = g < M ? p0 + g / G : -1;
  const int pos_b = (UPPER && g + 8 < M) ? p0 + (g + 8) / G : -1;
  // a sub-tile all of whose keys every row may see needs no mask: keys in [free_lo, free_hi)
  const int free_lo = max(lo, p.window > 0 ? p0 + (M - 1) / G - p.window + 1 : 0);
  const int free_hi = min(hi, p0 + 1);
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  for (int it = 0; it < my_n; ++it) {
    {
      const int nx = it + DSTAGES - 1;
      if (nx < my_n) {
        bf16* Kn = myKV + (nx % DSTAGES) * 2 * DKW * LDS;
        load_kv_subtile(p, bt, bt_first, hk, k_first + (warp + NWARPS * nx) * DKW, lo, hi, same_page, Kn, Kn + DKW * LDS, lane);
      }
      cp_async_commit();
      cp_async_wait<DSTAGES - 1>();
    }
    __syncwarp();
    const bf16* Ks = myKV + (it % DSTAGES) * 2 * DKW * LDS;
    const bf16* Vs = Ks + DKW * LDS;
    const int kbase = k_first + (warp + NWARPS * it) * DKW;
    float s[DNT][4];
#pragma unroll
    for (int j = 0; j < DNT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      if (DQ_IN_REGS) {
        a0 = qf[kk][0]; a1 = qf[kk][1]; a2 = qf[kk][2]; a3 = qf[kk][3];
      } else {
        ldmatrix_x4(a0, a1, a2, a3, Qs + (lane & 15) * LDS + kk * 16 + (lane >> 4) * 8);
      }
#pragma unroll
      for (int j = 0; j < DNT; j += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane >> 4) * 8 + (lane & 7)) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // (rows beyond M hold zero queries; what they compute is finite and never stored)
    const bool unmasked = kbase >= free_lo && kbase + DKW <= free_hi;
    float mx_a = -INFINITY, mx_b = -INFINITY;
    if (unmasked) {
#pragma unroll
      for (int j = 0; j < DNT; ++j) {
        s[j][0] *= p.scale_log2; s[j][1] *= p.scale_log2;
        mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
        if (UPPER) {
          s[j][2] *= p.scale_log2; s[j][3] *= p.scale_log2;
          mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < DNT; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = kbase + j * 8 + tq * 2 + e;
          const bool in_range = key >= lo && key < hi;
          const bool ok_a = in_range && key <= pos_a && (p.window <= 0 || key > pos_a - p.window);
          s[j][e] = ok_a ? s[j][e] * p.scale_log2 : -INFINITY;
          mx_a = fmaxf(mx_a, s[j][e]);
          if (UPPER) {
            const bool ok_b = in_range && key <= pos_b && (p.window <= 0 || key > pos_b - p.window);
            s[j][2 + e] = ok_b ? s[j][2 + e] * p.scale_log2 : -INFINITY;
            mx_b = fmaxf(mx_b, s[j][2 + e]);
          }
        }
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    const float mn_a = fmaxf(m_a, mx_a);
    const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a;       // ex2(-inf - 0) = 0: masked entries vanish by themselves
    const float al_a = ex2(m_a - use_a);
    m_a = mn_a;
    float mn_b = m_b, use_b = 0.f, al_b = 1.f;
    if (UPPER) {
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      mn_b = fmaxf(m_b, mx_b);
      use_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      al_b = ex2(m_b - use_b);
      m_b = mn_b;
    }
    uint32_t pa[DNT][2];
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int j = 0; j < DNT; ++j) {
      const float p0_ = ex2(s[j][0] - use_a), p1_ = ex2(s[j][1] - use_a);
      sum_a += p0_ + p1_;
      pa[j][0] = pack_bf16(p0_, p1_);
      if (UPPER) {
        const float p2_ = ex2(s[j][2] - use_b), p3_ = ex2(s[j][3] - use_b);
        sum_b += p2_ + p3_;
        pa[j][1] = pack_bf16(p2_, p3_);
      } else {
        pa[j][1] = 0u;
      }
    }
    l_a = l_a * al_a + sum_a;
    if (UPPER) l_b = l_b * al_b + sum_b;
    // rescale the output only when some row's maximum moved (warp-uniform decision)
    if (__any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= al_a; o[i][1] *= al_a;
        if (UPPER) { o[i][2] *= al_b; o[i][3] *= al_b; }
      }
    }
#pragma unroll
    for (int ks = 0; ks < DKW / 16; ++ks) {
#pragma unroll
      for (int i = 0; i < D / 8; i += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + i * 8 + (lane >> 4) * 8);
        mma_bf16(o[i], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b0, b1);
        mma_bf16(o[i + 1], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b2, b3);
      }
    }
    __syncwarp();   // all lanes have read this stage before a later fetch overwrites it
  }
  cp_async_wait<0>();
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  __syncthreads();                                              // every warp is done with its stages: reuse the memory
  float* Om = reinterpret_cast<float*>(smem_raw);               // [NWARPS][16][D]
  float* MLm = Om + NWARPS * 16 * D;                            // [NWARPS][16][2]
  // only rows that exist are merged below: the others are not written
  const bool row_a = g < M, row_b = UPPER && g + 8 < M;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    float* d0 = Om + ((size_t)warp * 16 + g) * D + i * 8 + tq * 2;
    float* d1 = Om + ((size_t)warp * 16 + g + 8) * D + i * 8 + tq * 2;
    if (row_a) { d0[0] = o[i][0]; d0[1] = o[i][1]; }
    if (row_b) { d1[0] = o[i][2]; d1[1] = o[i][3]; }
  }
  if (tq == 0) {
    if (row_a) { MLm[(warp * 16 + g) * 2] = m_a; MLm[(warp * 16 + g) * 2 + 1] = l_a; }
    if (row_b) { MLm[(warp * 16 + g + 8) * 2] = m_b; MLm[(warp * 16 + g + 8) * 2 + 1] = l_b; }
  }
  __syncthreads();
  const bool last = p.num_splits == 1;
  for (int idx = tid; idx < M * D; idx += NTHR) {
    const int row = idx / D, d = idx - row * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) mm = fmaxf(mm, MLm[(w * 16 + row) * 2]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = MLm[(w * 16 + row) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      ll += MLm[(w * 16 + row) * 2 + 1] * f;
      acc += Om[((size_t)w * 16 + row) * D + d] * f;
    }
    if (last) {
      const int tok = row / G, hd = hk * G + (row - tok * G);
      p.out[(size_t)(q0 + tok) * p.H * D + (size_t)hd * D + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    } else {
      const size_t base = (((size_t)r * p.Hkv + hk) * p.num_splits + split) * 16 + row;
      p.part_o[base * D + d] = acc;
      if (d == 0) { p.part_ml[base * 2] = mm; p.part_ml[base * 2 + 1] = ll; }
    }
  }
  if (!last) finish_split(p, r, hk, q0, M, NTHR, reinterpret_cast<float*>(smem_raw));
}

size_t deep_smem_bytes(int nwarps) {
  const size_t tiles = (size_t)(16 + nwarps * DSTAGES * 2 * DKW) * LDS * sizeof(bf16);
  const size_t merge = (size_t)(nwarps * 16 * D + nwarps * 16 * 2) * sizeof(float);
  return tiles > merge ? tiles : merge;
}

template <bool UPPER, int NWARPS>
int launch_deep(const Params& p, int n_rows, cudaStream_t stream) {
  auto k = attention_deep_kernel<UPPER, NWARPS>;
  const size_t smem = deep_smem_bytes(NWARPS);
  if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  SB_PDL_CHECK(launch_pdl(k, dim3(p.num_splits, p.Hkv, n_rows), dim3(NWARPS * 32), smem, stream, p));
  return 0;
}

// Merge the partial results of the key splits of the deep shape. grid (Hkv, R), 128 threads.
__global__ void __launch_bounds__(THREADS) attention_merge_kernel(const Params p) {
  const int r = blockIdx.y, hk = blockIdx.x;
  const int q0 = p.cu_q[r], qn = p.cu_q[r + 1] - q0;
  const int M = qn * p.G;
  if (M > 16 || M <= 0) return;
  __shared__ float work[(2 * MAX_SPLITS + 1) * 16];
  merge_splits(p, r, hk, q0, M, THREADS, work);
}

}  // namespace

SB_EXPORT int sb_attention_mma_head_dim() { return D; }

// Bytes of scratch the deep shape needs for (n_rows, Hkv, num_splits): partial outputs, then (max, sum) pairs.
SB_EXPORT long long sb_attention_mma_scratch_bytes(int n_rows, int Hkv, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)n_rows * Hkv * num_splits * 16 * (D + 2) * (long long)sizeof(float);
}

// which: bit 0 launch the wide shape (for the n_wide requests listed in wide_rows if that is given, else for all:
// a step of hundreds of decoding requests and a few prompt portions then launches blocks for the portions only),
// bit 1 launch the deep shape. ``longest``: no sequence of the step is longer (0: not known). With num_splits > 1 the deep shape needs
// ``scratch`` (sb_attention_mma_scratch_bytes) and merges either in the block that finishes last (tickets: n_rows * Hkv
// ints, zero before the first launch; every launch leaves them zero) or, with tickets == nullptr, in a second kernel.
SB_EXPORT int sb_attention_mma(const void* qkv, int q_stride, const void* kc, const void* vc, const int* block_table, int bt_width,
                               const int* cu_q, const int* kv_len, int H, int Hkv, int ps, int num_pages, float scale, int window,
                               void* out, int n_rows, int max_q, int which, int longest, int num_splits, void* scratch,
                               int* tickets, const int* wide_rows, int n_wide, cudaStream_t stream) {
  if (n_rows <= 0 || max_q <= 0) return 0;
  if (H <= 0 || Hkv <= 0 || H % Hkv || ps <= 0 || bt_width <= 0) return SB_ERR_SHAPE;
  if (Hkv > 65535 || n_rows > 65535) return SB_ERR_LIMIT;
  if ((q_stride % 8) || !aligned16(qkv) || !aligned16(kc) || !aligned16(vc) || !aligned16(out)) return SB_ERR_ALIGN;
  Params p;
  p.qkv = (const bf16*)qkv; p.q_stride = q_stride; p.kc = (const bf16*)kc; p.vc = (const bf16*)vc;
  p.block_table = block_table; p.bt_width = bt_width; p.cu_q = cu_q; p.kv_len = kv_len;
  p.H = H; p.Hkv = Hkv; p.G = H / Hkv; p.ps = ps; p.num_pages = num_pages;
  p.ps_shift = (ps & (ps - 1)) == 0 ? __builtin_ctz((unsigned)ps) : -1;
  p.scale_log2 = scale * LOG2E; p.window = window; p.out = (bf16*)out;
  p.split_size = 0; p.num_splits = num_splits; p.part_o = nullptr; p.part_ml = nullptr; p.tickets = nullptr;
  p.wide_rows = wide_rows; p.heads_in_x = 0;
  if (which & 1) {
    auto k = attention_wide_kernel;
    const size_t smem = wide_smem_bytes();
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const long long tiles = ((long long)max_q * p.G + 63) / 64;
    if (tiles > 2147483647LL) return SB_ERR_LIMIT;
    const int z = wide_rows ? n_wide : n_rows;
    p.heads_in_x = tiles <= 65535 ? 1 : 0;
    if (z > 0) k<<<p.heads_in_x ? dim3(Hkv, (unsigned)tiles, z) : dim3((unsigned)tiles, Hkv, z), THREADS, smem, stream>>>(p);
    SB_LAUNCH_CHECK();
  }
  if (which & 2) {
    if (p.G > 16) return SB_ERR_SHAPE;   // the caller sends such groups to the wide shape
    if (num_splits < 1 || num_splits > MAX_SPLITS) return SB_ERR_SHAPE;
    if (num_splits > 1) {
      if (!scratch) return SB_ERR_SHAPE;
      p.part_o = (float*)scratch;
      p.part_ml = p.part_o + (size_t)n_rows * Hkv * num_splits * 16 * D;
      p.tickets = tickets;
    }
    // bit 2 of ``which``: some request has more than 8 rows (the caller knows the largest token count).
    // Few blocks (at most one per SM): 8 warps each, so that an SM still has warps to switch between.
    const bool roomy = (long long)n_rows * Hkv * num_splits <= sm_count() && deep_smem_bytes(8) <= 227 * 1024;
    // Otherwise the block shape follows from what fits the SMs at once (two four-warp blocks an SM at head_dim 64, five
    // two-warp blocks, ten one-warp blocks) and from how long the sequences can be (``longest``, 0 if the caller does
    // not say). A block's fixed part (table, queries, first loads, merge, store) is 4-5 us: it should overlap with
    // other blocks' key loops, and a round of blocks that is mostly empty costs a whole block's time. Measured with 8 kv
    // heads of 64 (`profiles/steps_other_sizes_and_contexts.md`):
    //  - four warps while one round of them holds all blocks, for very long sequences, and for a few hundred pairs of
    //    1,024 to 4,096 tokens whose last round is not thin (64 requests x 2,048 tokens: 48.4 us against 49.5 with two);
    //  - one warp per pair only for a thousand and more pairs of at most 256 tokens (1,000 requests x 192: 76.9 us
    //    against 84.1 with two warps and 135.6 with four); with longer sequences one-warp blocks lose badly (192
    //    requests x 2,048: 176 us against 137 with two warps);
    //  - two warps otherwise (90 requests x 512: 21.0 against 25.5 us with four; 40 x 2,048, where four-warp blocks are
    //    296 + 24: 35.2 against 42.8), unless their own last round would be thin and one-warp blocks fit at once
    //    (100 requests x 300 tokens: 17.1 us with one warp, 20.2 with two).
    const long long pairs = (long long)n_rows * Hkv, blocks = pairs * num_splits;
    auto at_once = [&](int nw) { return (long long)sm_count() * (long long)std::max<size_t>(1, (227 * 1024) / (deep_smem_bytes(nw) + 2048)); };
    const long long cap4 = at_once(4), cap2 = at_once(2), cap1 = at_once(1);
    auto thin_last_round = [&](long long cap) {          // the last round of blocks would be under 70 % full
      const long long rounds = (blocks + cap - 1) / cap;
      return blocks * 10 < rounds * cap * 7;
    };
    int warps = 2;
    if (roomy) warps = 8;
    else if (blocks <= cap4) warps = 4;
    else if (num_splits == 1 && pairs >= 1024 && longest > 0 && longest <= 256) warps = thin_last_round(cap1) ? 2 : 1;
    else if (longest <= 0 || longest >= 4096) warps = (thin_last_round(cap4) && blocks <= cap2) ? 2 : 4;
    else if (longest > 1024 && blocks <= 2 * cap4 && !thin_last_round(cap4)) warps = 4;
    else if (num_splits == 1 && longest <= 1024 && blocks > cap2 && blocks <= cap1 && thin_last_round(cap2)) warps = 1;
    auto launch = [&](auto upper) -> int {
      constexpr bool U = decltype(upper)::value;
      if (warps == 8) return launch_deep<U, 8>(p, n_rows, stream);
      if (warps == 1) return launch_deep<U, 1>(p, n_rows, stream);
      if (warps == 2) return launch_deep<U, 2>(p, n_rows, stream);
      return launch_deep<U, 4>(p, n_rows, stream);
    };
    int rc = launch(std::false_type{});
    if (rc) return rc;
    if (which & 4) {
      rc = launch(std::true_type{});
      if (rc) return rc;
    }
    if (num_splits > 1 && tickets == nullptr) {
      attention_merge_kernel<<<dim3(Hkv, n_rows), THREADS, 0, stream>>>(p);
      SB_LAUNCH_CHECK();
    }
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// Decoding attention with built-in scratch memory, for callers that must not allocate (attention_noalloc.h).
#include "attention_noalloc.h"

namespace {
constexpr size_t kNoallocPartialFloats = (size_t)SB_NOALLOC_MAX_TILES * 16 * (D + 2);
// partial outputs and (max, sum) pairs of the key splits, then one arrival counter per (request, kv head)
static __device__ __align__(256) float g_noalloc_scratch[kNoallocPartialFloats + SB_NOALLOC_MAX_TILES];
// In host code the name above is only a handle; the device address is looked up once per device.
constexpr int kNoallocMaxDevices = 64;
void* g_noalloc_addr[kNoallocMaxDevices];
}  // namespace

SB_EXPORT int sb_attention_decode_noalloc_max_tiles(void) { return SB_NOALLOC_MAX_TILES; }

SB_EXPORT int sb_attention_decode_noalloc(const void* qkv, int q_stride, const void* kc, const void* vc, const int* block_table,
                                          int bt_width, const int* cu_q, const int* kv_len, int H, int Hkv, int ps, int num_pages,
                                          float scale, int window, void* out, int n_rows, int max_q, int num_splits,
                                          cudaStream_t stream) {
  if (n_rows <= 0 || max_q <= 0) return 0;
  if (H <= 0 || Hkv <= 0 || H % Hkv || ps <= 0 || bt_width <= 0) return SB_ERR_SHAPE;
  const int G = H / Hkv;
  if (G > 16 || (long long)max_q * G > 16) return SB_ERR_SHAPE;
  if (num_splits < 1 || num_splits > MAX_SPLITS) return SB_ERR_SHAPE;
  if (Hkv > 65535 || n_rows > 65535) return SB_ERR_LIMIT;
  if ((long long)n_rows * Hkv * num_splits > SB_NOALLOC_MAX_TILES) return SB_ERR_LIMIT;
  if ((q_stride % 8) || !aligned16(qkv) || !aligned16(kc) || !aligned16(vc) || !aligned16(out)) return SB_ERR_ALIGN;

  // set-up, once per device, with that device current: the array's address on this device
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return SB_ERR_LIMIT;
  if (g_noalloc_addr[dev] == nullptr) {
    void* addr = nullptr;
    e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_addr[dev] = addr;
  }
  float* scratch = static_cast<float*>(g_noalloc_addr[dev]);
  int* tickets = reinterpret_cast<int*>(scratch + kNoallocPartialFloats);

  Params p;
  p.qkv = (const bf16*)qkv; p.q_stride = q_stride; p.kc = (const bf16*)kc; p.vc = (const bf16*)vc;
  p.block_table = block_table; p.bt_width = bt_width; p.cu_q = cu_q; p.kv_len = kv_len;
  p.H = H; p.Hkv = Hkv; p.G = G; p.ps = ps; p.num_pages = num_pages;
  p.ps_shift = (ps & (ps - 1)) == 0 ? __builtin_ctz((unsigned)ps) : -1;
  p.scale_log2 = scale * LOG2E; p.window = window; p.out = (bf16*)out;
  p.split_size = 0; p.num_splits = num_splits; p.part_o = nullptr; p.part_ml = nullptr; p.tickets = nullptr;
  p.wide_rows = nullptr;
  if (num_splits > 1) {
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)n_rows * Hkv * num_splits * 16 * D;
    p.tickets = tickets;
    // the array keeps the last call's contents; the arrival counters are what has to start at zero
    e = cudaMemsetAsync(tickets, 0, (size_t)n_rows * Hkv * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
  }
  const bool roomy = (long long)n_rows * Hkv * num_splits <= sm_count() && deep_smem_bytes(8) <= 227 * 1024;
  int rc = roomy ? launch_deep<false, 8>(p, n_rows, stream) : launch_deep<false, 4>(p, n_rows, stream);
  if (rc) return rc;
  if ((long long)max_q * G > 8 || G > 8) {
    rc = roomy ? launch_deep<true, 8>(p, n_rows, stream) : launch_deep<true, 4>(p, n_rows, stream);
    if (rc) return rc;
  }
  return 0;
}
