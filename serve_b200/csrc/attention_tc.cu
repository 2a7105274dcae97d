// Paged causal attention for prompt portions on the fifth-generation tensor cores (head_dim 64 or 128, bfloat16).
//
// Work is cut as in attention_mma.cu: per (request, kv head), with the G = H / Hkv query heads that share the kv
// head folded into the row dimension: row m stands for (token m / G, head hk*G + m % G). A CTA owns 128 such
// rows (128 / G tokens) and walks over the request's keys in tiles of 64:
//   warp 0     one thread feeds shared memory with TMA: the query tile once (a 4-d box over the q/k/v buffer),
//              then per tile the key and value pages named by the block table (4-d boxes over the caches,
//              128-byte swizzle), three stages; the thread's loop is kept free of divisions, it is on the critical path;
//   warp 1     one thread issues tcgen05.mma: S = Q K^T (128 x 64 x 64) into one of two score buffers in tensor
//              memory, and, once the probabilities of a tile are in shared memory, O += P V (128 x 64 x 64, V read
//              MN-major) into the output accumulator, which stays in tensor memory for the whole walk;
//              tcgen05.commit signals the readers and frees stages and buffers;
//   warps 2..5 one thread per row: reads its row of S from tensor memory (tcgen05.ld), scale, causal mask on
//              the diagonal tiles, exp2 against a reference maximum, writes the probabilities as bfloat16 into the
//              swizzled layout the second product reads (two buffers). The reference maximum only follows the
//              running maximum when that has moved by more than 8 (a factor 256, harmless in bfloat16 and float);
//              then, and only then, the accumulator in tensor memory is rescaled (tcgen05.ld / tcgen05.st) after
//              the products issued so far have finished. So in the steady state nobody waits for the second
//              product. At the end each thread divides its output row by the row's sum and stores its row.
// Two CTAs share an SM at head_dim 64 (96 KB of shared memory, 256 columns of tensor memory each).
// At head_dim 128 an operand row is two 128-byte swizzle atoms: queries, keys and values arrive as two TMA boxes of 64
// elements each, the first product walks over both atoms of Q and K, the second product covers the 128 output
// columns in one instruction (the descriptor's leading byte offset names the distance between the atoms of V);
// shared memory then holds one CTA per SM.
// The recurrences are those of serve/kernels/attn_prefill.py:58-72 with exp2 and a folded log2(e)
// (attn_prefill.py:330-331); probabilities are rounded to bfloat16 before the second product (attn_prefill.py:71).
// Every wait is bounded; a wait that runs out raises *error and the CTA still frees its tensor memory.
#include <cuda.h>

#include "common.cuh"

#if SB_HEAD_DIM == 64 || SB_HEAD_DIM == 128

using namespace sb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int D = SB_HEAD_DIM;
constexpr int KA = D / 64;            // 128-byte swizzle atoms (64 elements) per operand row
constexpr int CTAS_PER_SM = D == 64 ? 2 : 1;
constexpr int BM = 128;              // rows per CTA
constexpr int BN = 64;               // keys per tile (one 128-byte row of probabilities: one k-block of P)
constexpr int NS = 3;                // key/value stages
constexpr int BT_CACHE = 1024;       // block-table entries kept in shared memory
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 256;  // S0, S1 (BN columns each), O (64), rounded up to a power of two; two CTAs share an SM
constexpr unsigned WAIT_LIMIT = 1u << 26;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int Q_BYTES = BM * D * 2, KV_BYTES = BN * D * 2, P_BYTES = BM * BN * 2;
constexpr int TILE_BYTES = Q_BYTES + 2 * NS * KV_BYTES + 2 * P_BYTES;  // 96 KB at head_dim 64, 160 KB at 128
constexpr int SMEM_BYTES = TILE_BYTES + 256 + BT_CACHE * 4;             // + barriers + table entries; two CTAs fit an SM

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  const uint32_t addr = smem_u32(bar);
  for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 columns: thread i of the warp gets lane (base + i), 32 consecutive columns. No wait: several loads
// may be in flight; tc_wait_ld() before the registers are read.
__device__ __forceinline__ void tc_load32(uint32_t taddr, float* r) {
  uint32_t* u = reinterpret_cast<uint32_t*>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]),
        "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]), "=r"(u[17]), "=r"(u[18]),
        "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]),
        "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_store32(uint32_t taddr, const float* r) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]),
        "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]),
        "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]),
        "r"(u[30]), "r"(u[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart; ``lbo`` is the distance between
// 64-element swizzle atoms along the non-k dimension of an MN-major operand (not used by K-major operands).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: float accumulator, bfloat16 operands; b_mn_major: the second operand has its
// non-k dimension contiguous in shared memory (values: rows are keys, head elements contiguous)
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct TcParams {
  const int* block_table; int bt_width;
  const int* cu_q; const int* kv_len;
  int H, Hkv, G, ps;
  float scale_log2;
  bf16* out;
  int* error;
  const int* rows;      // requests this launch covers (blockIdx.z indexes it); nullptr: all, in order
  int heads_in_x;       // grid (kv heads, row tiles, requests) rather than (row tiles, kv heads, requests)
};

__global__ void __launch_bounds__(THREADS, CTAS_PER_SM) attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                               const __grid_constant__ CUtensorMap map_k,
                                                               const __grid_constant__ CUtensorMap map_v, const TcParams p) {
  // Blocks start in the order of blockIdx.x, then y: with the heads in x, the tiles that see the most keys start first
  // for all heads. The other way round the last heads' longest tiles would start when a third of the time is over
  // and end last: 2,048 tokens, 32/8 heads took 53 us so, against 32 key tiles x ~1.1 us for the longest tile itself.
  const int r = p.rows ? p.rows[blockIdx.z] : (int)blockIdx.z;
  const int hk = p.heads_in_x ? blockIdx.x : blockIdx.y, bx = p.heads_in_x ? blockIdx.y : blockIdx.x;
  const int q0 = p.cu_q[r], qn = p.cu_q[r + 1] - q0;
  const int G = p.G;
  const int M = qn * G;
  // (a block with nothing to do still waits for the kernel before this one: see attention_deep_kernel)
  if (M <= 16) { pdl_wait(); return; }                  // the deep shape takes this request
  const int tok_per_tile = BM / G;
  const int n_mtiles = (qn + tok_per_tile - 1) / tok_per_tile;
  if (bx >= n_mtiles) { pdl_wait(); return; }
  const int tile = n_mtiles - 1 - bx;                   // later rows see more keys: they go first
  const int tok0 = tile * tok_per_tile;
  const int L = p.kv_len[r];
  const int p0 = L - qn;                                // position of the request's first query
  const int tok_last = min(tok0 + tok_per_tile, qn) - 1;
  const int hi = p0 + tok_last + 1;                     // keys [0, hi) are seen by some row of the tile
  const int n_tiles = (hi + BN - 1) / BN;

  // all shared memory is dynamic, so that the tiles start at the CTA's (1024-byte aligned) window base: the
  // 128-byte swizzle needs that alignment, and a padded request would not let two CTAs share an SM
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* base = smem;
  unsigned char* Qs = base;
  unsigned char* Ks = Qs + Q_BYTES;                     // NS stages
  unsigned char* Vs = Ks + NS * KV_BYTES;               // NS stages
  unsigned char* Ps = Vs + NS * KV_BYTES;               // 2 buffers of [128 rows][128 bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + TILE_BYTES);
  uint64_t& q_full = bars[0];
  uint64_t* kv_full = bars + 1;                         // NS: a stage's keys and values have landed
  uint64_t* kv_empty = bars + 1 + NS;                   // NS: the products that read the stage have finished
  uint64_t* s_full = bars + 1 + 2 * NS;                 // 2: a score buffer is complete
  uint64_t* s_empty = bars + 3 + 2 * NS;                // 2: the softmax threads hold it in registers
  uint64_t* p_full = bars + 5 + 2 * NS;                 // 2: a buffer of probabilities is written
  uint64_t* p_empty = bars + 7 + 2 * NS;                // 2: the second product that read it has finished
  uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(bars + 9 + 2 * NS);
  int* bt_s = reinterpret_cast<int*>(base + TILE_BYTES + 256);
  if ((smem_u32(base) & 1023u) != 0) {                  // never seen; refuse rather than compute with a wrong swizzle
    if (threadIdx.x == 0) atomicExch(p.error, 1);
    pdl_wait();
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
#pragma unroll
    for (int s = 0; s < NS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4); mbar_init(&p_full[b], 4); mbar_init(&p_empty[b], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // set up; queries, this step's keys and values, and the right to overwrite out come with the end of the kernel before
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_s;
  bool failed = false;

  if (warp == 0) {
    // the table entries of the tile's keys, fetched once by the whole warp instead of one dependent load per page
    const int* bt = p.block_table + (size_t)r * p.bt_width;
    const int n_blocks = min((hi + p.ps - 1) / p.ps, p.bt_width);
    if (n_blocks <= BT_CACHE) {
      for (int i = lane; i < n_blocks; i += 32) bt_s[i] = bt[i];
      __syncwarp();
      bt = bt_s;
    }
    if (lane == 0) {
      // queries: box {64 elements, G heads, 1 kv head, tokens of the tile} -> rows (token, head)
      mbar_expect_tx(&q_full, (unsigned)(tok_per_tile * G * D * 2));
#pragma unroll
      for (int a = 0; a < KA; ++a) tma_load_4d(Qs + (size_t)a * BM * 128, &map_q, &q_full, a * 64, 0, hk, q0 + tok0);
      const bool big_pages = p.ps > BN;                  // a page holds several tiles (a multiple of BN keys)
      const int pages_per_tile = big_pages ? 0 : BN / p.ps;
      int big_blk = 0, big_at = 0;                        // big pages: the tile's page, and where in it the tile starts
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % NS;
        if (!mbar_wait(&kv_empty[s], ((j / NS) & 1) ^ 1)) { failed = true; break; }
        const int kt = j * BN, blk0 = j * pages_per_tile;   // pages tile the stage: no division in this thread's loop
        if (big_pages) {
          const bool there = kt < hi && big_blk < p.bt_width;
          mbar_expect_tx(&kv_full[s], there ? (unsigned)(BN * D * 2 * 2) : 0u);
          if (there) {
            const int page = bt[big_blk];
#pragma unroll
            for (int a = 0; a < KA; ++a) {
              const size_t off = (size_t)s * KV_BYTES + (size_t)a * BN * 128;
              tma_load_4d(Ks + off, &map_k, &kv_full[s], a * 64, big_at, hk, page);
              tma_load_4d(Vs + off, &map_v, &kv_full[s], a * 64, big_at, hk, page);
            }
          }
          big_at += BN;
          if (big_at == p.ps) { big_at = 0; ++big_blk; }
          continue;
        }
        int n_pages = 0;
        for (int i = 0; i < pages_per_tile; ++i)
          if (kt + i * p.ps < hi && blk0 + i < p.bt_width) ++n_pages;
        mbar_expect_tx(&kv_full[s], (unsigned)(n_pages * p.ps * D * 2 * 2));
        for (int i = 0; i < n_pages; ++i) {
          const int page = bt[blk0 + i];
#pragma unroll
          for (int a = 0; a < KA; ++a) {
            // atom a of a stage: 64 keys x 128 bytes; the page's keys at their rows of it
            const size_t off = (size_t)s * KV_BYTES + (size_t)a * BN * 128 + (size_t)i * p.ps * 128;
            tma_load_4d(Ks + off, &map_k, &kv_full[s], a * 64, 0, hk, page);
            tma_load_4d(Vs + off, &map_v, &kv_full[s], a * 64, 0, hk, page);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN, false);
      constexpr uint32_t idesc_o = make_idesc(BM, D, true);
      const uint64_t dq = make_desc(smem_u32(Qs), 0);
      auto issue_s = [&](int t) {
        const uint64_t dk = make_desc(smem_u32(Ks + (size_t)(t % NS) * KV_BYTES), 0);
        const uint32_t acc = tmem_base + (uint32_t)((t & 1) * BN);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // 16 k-values further: 32 bytes within an atom (4 steps), then the next atom of Q (128 rows) and K (64 rows)
          const uint64_t qo = (uint64_t)((kk >> 2) * (BM * 128 >> 4) + (kk & 3) * 2);
          const uint64_t ko = (uint64_t)((kk >> 2) * (BN * 128 >> 4) + (kk & 3) * 2);
          tc_mma(acc, dq + qo, dk + ko, idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[t & 1]);
      };
      do {
        if (!mbar_wait(&q_full, 0) || !mbar_wait(&kv_full[0], 0)) { failed = true; break; }
        tc_fence_after();
        issue_s(0);
        for (int j = 0; j < n_tiles; ++j) {
          const int b = j & 1;
          if (j + 1 < n_tiles) {
            // the next tile's scores, as soon as its keys are there and its score buffer has been read
            const int t = j + 1;
            if (!mbar_wait(&kv_full[t % NS], (t / NS) & 1) || !mbar_wait(&s_empty[t & 1], ((t >> 1) & 1) ^ 1)) { failed = true; break; }
            tc_fence_after();
            issue_s(t);
          }
          if (!mbar_wait(&p_full[b], (j >> 1) & 1)) { failed = true; break; }
          tc_fence_after();
          // O += P V: P is K-major (one block of 64 keys); V is MN-major, 16 keys = 2048 bytes further per step
          const uint32_t pa = smem_u32(Ps + (size_t)b * P_BYTES), va = smem_u32(Vs + (size_t)(j % NS) * KV_BYTES);
          const uint32_t acc = tmem_base + (uint32_t)(2 * BN);
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            const uint64_t dp = make_desc(pa + (uint32_t)(kk * 32), 0);
            const uint64_t dv = make_desc(va + (uint32_t)(kk * 2048), BN * 128);
            tc_mma(acc, dp, dv, idesc_o, (j | kk) != 0 ? 1u : 0u);
          }
          tc_commit(&p_empty[b]);            // also: "the products up to tile j have finished"
          tc_commit(&kv_empty[j % NS]);
        }
      } while (false);
    }
  } else {
    const int q = warp & 3;                              // the 32 tensor-memory lanes this warp may touch
    const int row = q * 32 + lane;
    const int m = tok0 * G + row;
    const bool row_ok = row < tok_per_tile * G && m < M;
    const int tok = row_ok ? m / G : 0, head = row_ok ? hk * G + (m - tok * G) : 0;
    const int pos = row_ok ? p0 + tok : -1;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t o_addr = lane_addr + (uint32_t)(2 * BN);
    float m_ref = -INFINITY;                             // what the exponentials are taken against (log2 domain)
    float l_run = 0.f;
    const int first_pos = p0 + tok0;                     // smallest position of the tile's rows

    for (int j = 0; j < n_tiles && !failed; ++j) {
      const int b = j & 1, kt = j * BN;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1)) { failed = true; break; }
      tc_fence_after();
      const bool masked = kt + BN - 1 > first_pos;       // the tile reaches beyond what the first row may see
      float sv[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tc_load32(lane_addr + (uint32_t)(b * BN + c * 32), sv + c * 32);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[b]);           // the scores are in registers: the buffer may be reused
      if (masked) {
#pragma unroll
        for (int i = 0; i < BN; ++i) sv[i] = (kt + i <= pos) ? sv[i] : -INFINITY;
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        mx0 = fmaxf(mx0, sv[i]); mx1 = fmaxf(mx1, sv[i + 1]); mx2 = fmaxf(mx2, sv[i + 2]); mx3 = fmaxf(mx3, sv[i + 3]);
      }
      const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      // the reference follows the maximum only when that has run ahead by more than 8 (or there was none yet)
      const bool moved = m_tile > m_ref + 8.0f;           // false for m_tile = -inf; true for m_ref = -inf, m_tile finite
      if (__any_sync(0xffffffffu, moved && m_ref != -INFINITY)) {
        // rare: rescale the accumulator in tensor memory, once the products issued so far (up to tile j-1) are done
        const int pb = (j - 1) & 1;
        if (!mbar_wait(&p_empty[pb], ((j - 1) >> 1) & 1)) { failed = true; break; }
        tc_fence_after();
        const float f = (moved && m_ref != -INFINITY) ? ex2(m_ref - m_tile) : 1.f;
        float ov[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tc_load32(o_addr + (uint32_t)(c * 32), ov + c * 32);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < D; ++i) ov[i] *= f;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tc_store32(o_addr + (uint32_t)(c * 32), ov + c * 32);
        tc_wait_st();
        l_run *= f;
      }
      if (moved) m_ref = m_tile;                         // (with no reference yet, accumulator and sum are still zero)
      const float use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // the buffer of probabilities must have been read by the product of two tiles ago
      if (j >= 2 && !mbar_wait(&p_empty[b], ((j - 2) >> 1) & 1)) { failed = true; break; }
      // probabilities -> shared memory (bfloat16, the swizzled K-major layout of the second product);
      // ex2(-inf) = 0 takes care of masked entries
      float sum0 = 0.f, sum1 = 0.f;
      unsigned char* prow = Ps + (size_t)b * P_BYTES + (size_t)row * 128;
#pragma unroll
      for (int c = 0; c < BN / 8; ++c) {                 // 16-byte pieces of 8 keys
        uint32_t pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float e0 = ex2(fmaf(sv[c * 8 + 2 * i], p.scale_log2, -use));
          const float e1 = ex2(fmaf(sv[c * 8 + 2 * i + 1], p.scale_log2, -use));
          sum0 += e0;
          sum1 += e1;
          pk[i] = pack_bf16(e0, e1);
        }
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run += sum0 + sum1;
      // values of keys beyond the sequence (never written, or another tile's leftovers) must not meet a zero
      // probability as NaN: the rows of this stage beyond hi are cleared
      if (kt + BN > hi) {
        if (!mbar_wait(&kv_full[j % NS], (j / NS) & 1)) { failed = true; break; }
        unsigned char* vt = Vs + (size_t)(j % NS) * KV_BYTES;
        const int first = hi - kt;                       // rows [first, BN)
        for (int idx = (warp - 2) * 32 + lane; idx < (BN - first) * 8 * KA; idx += 128) {
          const int a = idx / ((BN - first) * 8), rest = idx - a * (BN - first) * 8;
          *reinterpret_cast<uint4*>(vt + (size_t)a * BN * 128 + (size_t)(first + (rest >> 3)) * 128 + ((rest & 7) << 4)) =
              make_uint4(0u, 0u, 0u, 0u);
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these writes are read by the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }
    if (!failed) {
      // all products have finished when the last one has
      const int pb = (n_tiles - 1) & 1;
      if (!mbar_wait(&p_empty[pb], ((n_tiles - 1) >> 1) & 1)) failed = true;
      tc_fence_after();
      if (!failed) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        float ov[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tc_load32(o_addr + (uint32_t)(c * 32), ov + c * 32);
        tc_wait_ld();
        if (row_ok) {
          bf16* dst = p.out + (size_t)(q0 + tok) * p.H * D + (size_t)head * D;
#pragma unroll
          for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<uint4*>(dst + i * 8) =
                make_uint4(pack_bf16(ov[8 * i] * inv, ov[8 * i + 1] * inv), pack_bf16(ov[8 * i + 2] * inv, ov[8 * i + 3] * inv),
                           pack_bf16(ov[8 * i + 4] * inv, ov[8 * i + 5] * inv), pack_bf16(ov[8 * i + 6] * inv, ov[8 * i + 7] * inv));
        }
      }
    }
  }
  if (failed) atomicExch(p.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int encode4(CUtensorMap* map, const void* basep, const cuuint64_t dims[4], const cuuint64_t strides[3], const cuuint32_t box[4]) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn) return -300;
    g_encode = (EncodeTiledFn)fn;
  }
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult rc = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(basep), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -301 - (int)rc;
}

}  // namespace

// 1 if sb_attention_tc takes this geometry (else the caller uses the mma.sync kernel).
SB_EXPORT int sb_attention_tc_supports(int H, int Hkv, int ps, int window, int q_stride) {
  if (H <= 0 || Hkv <= 0 || H % Hkv) return 0;
  const int G = H / Hkv;
  if (G > 128) return 0;                                // a tile holds whole tokens: 128 / G of them (rows beyond stay unused)
  if (ps < 8) return 0;
  if (ps <= BN ? (BN % ps) != 0 : ((ps % BN) != 0 || ps > 256)) return 0;   // pages tile a stage of keys (in whole swizzle atoms), or stages tile a page
  if (window > 0) return 0;
  if (q_stride % 8) return 0;
  return 1;
}

// The wide shape of sb_attention_mma (requests with more than 16 rows) on tcgen05; arguments as there.
// n_tokens: rows of qkv; num_pages: pages of kc / vc. rows (may be null): the n_rows requests to cover, so that a
// step of hundreds of decoding requests and a few prompt portions launches blocks for the portions only.
SB_EXPORT int sb_attention_tc(const void* qkv, int q_stride, int n_tokens, const void* kc, const void* vc, const int* block_table,
                              int bt_width, const int* cu_q, const int* kv_len, int H, int Hkv, int ps, int num_pages, float scale,
                              void* out, int n_rows, int max_q, const int* rows, int* error, cudaStream_t stream) {
  if (n_rows <= 0 || max_q <= 0) return 0;
  if (!sb_attention_tc_supports(H, Hkv, ps, 0, q_stride)) return SB_ERR_SHAPE;
  if (Hkv > 65535 || n_rows > 65535) return SB_ERR_LIMIT;
  if (!aligned16(qkv) || !aligned16(kc) || !aligned16(vc) || !aligned16(out) || !error) return SB_ERR_ALIGN;
  const int G = H / Hkv;
  CUtensorMap map_q, map_k, map_v;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)G, (cuuint64_t)Hkv, (cuuint64_t)n_tokens};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)G * D * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)(BM / G)};   // one swizzle atom of the head
    int rc = encode4(&map_q, qkv, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)ps, (cuuint64_t)Hkv, (cuuint64_t)num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)ps * D * 2, (cuuint64_t)Hkv * ps * D * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)(ps < BN ? ps : BN), 1, 1};
    int rc = encode4(&map_k, kc, dims, strides, box);
    if (rc) return rc;
    rc = encode4(&map_v, vc, dims, strides, box);
    if (rc) return rc;
  }
  TcParams p;
  p.block_table = block_table; p.bt_width = bt_width; p.cu_q = cu_q; p.kv_len = kv_len;
  p.H = H; p.Hkv = Hkv; p.G = G; p.ps = ps; p.scale_log2 = scale * LOG2E; p.out = (bf16*)out; p.error = error; p.rows = rows;
  const int tok_per_tile = BM / G;
  const int m_tiles = (max_q + tok_per_tile - 1) / tok_per_tile;
  auto k = attention_tc_kernel;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  p.heads_in_x = m_tiles <= 65535 ? 1 : 0;
  const dim3 grid = p.heads_in_x ? dim3(Hkv, m_tiles, n_rows) : dim3(m_tiles, Hkv, n_rows);
  SB_PDL_CHECK(launch_pdl(k, grid, dim3(THREADS), (size_t)SMEM_BYTES, stream, map_q, map_k, map_v, p));
  return 0;
}

#else

SB_EXPORT int sb_attention_tc_supports(int, int, int, int, int) { return 0; }

#endif
