// Matrix products for many rows (prompt portions) on the fifth-generation tensor cores:
// out[M,N] = a[M,K] * w[N,K]^T, bfloat16 in, float accumulation in tensor memory, bfloat16 out.
// With gate_up, w is [2N, K] (gate rows, then up rows) and out[m,n] = silu(gate) * up (serve/model.py:85):
// the activation is applied while the accumulator leaves tensor memory, and the [M, 2N] intermediate of the
// unfused path is never written. A third epilogue is the q/k/v product's (serve/model.py:120-124, 234-244): query and
// key columns are rotated by their token's position, queries go to out, keys and values straight into the
// request's cache pages, so the rotary kernel and its pass over q, k and v are not needed.
//
// A persistent CTA per SM walks over 128 x 256 tiles of the accumulator (with gate_up: 128 gate columns and
// their 128 up columns, i.e. 128 output columns). Warp 0 feeds a ring of four shared-memory stages with TMA
// (cp.async.bulk.tensor, 128-byte swizzle: one 128 x 64 box of a and a 256 x 64 box, or two 128 x 64 boxes, of
// w per stage, completion counted on an mbarrier); one thread of warp 1 issues tcgen05.mma (128 x 256 x 16,
// operands read from shared memory through matrix descriptors, accumulator in tensor memory) and releases
// stages with tcgen05.commit; warps 2..17 read a finished accumulator back with tcgen05.ld, apply the epilogue
// and store. Tensor memory holds two accumulators (2 x 256 columns), so the epilogue of one tile runs while
// the products of the next are issued. Tiles that share a panel of w run at the same time on neighbouring
// CTAs, so w comes from HBM once. Rows beyond M and k-values beyond K are zero-filled by TMA; stores are guarded.
//
// Every wait is bounded; a wait that runs out raises *error, and the CTA still frees its tensor memory.
#include <cuda.h>

#include "common.cuh"

using namespace sb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;      // accumulator tile and k-values per stage
constexpr int NSTAGE = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 16;                    // two warps per quarter of the tensor-memory lanes: even and odd column chunks
constexpr int THREADS = 64 + 32 * EPI_WARPS;     // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..9: epilogue
constexpr unsigned WAIT_LIMIT = 1u << 26;
constexpr uint32_t TMEM_COLS = 512;              // two accumulators of BN columns

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
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
// 32 lanes x 32 columns of 32-bit accumulator: thread i of the warp gets lane (base lane + i), 32 consecutive columns
__device__ __forceinline__ void tc_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored by TMA with the 128-byte swizzle: rows of 128 bytes,
// 8 rows to a 1024-byte atom, atoms one after the other (stride 1024 bytes); version 1, layout type 2.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);            // start address, 16-byte units
  d |= (uint64_t)0 << 16;                                 // leading byte offset: not used by this layout
  d |= (uint64_t)(1024 >> 4) << 32;                       // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                                 // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                                 // 128-byte swizzle
  return d;
}

// kind::f16 instruction descriptor: float accumulator, bfloat16 a and b, both K-major, N x M of the tile
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

constexpr int EPI_STORE = 0, EPI_GATE_UP = 1, EPI_ROPE = 2;

// What the q/k/v epilogue needs: columns are [q heads | k heads | v heads] x D, D a multiple of 32 so that the 32
// columns a thread holds at a time lie in one head. Adjacent pairs (2j, 2j+1) turn by position * inv_freq[j]; the
// cosine and sine of that angle come from a table [rot/2, rows] made once per step (sb_rope_angles): an epilogue
// warp has its scheduler to itself, so every instruction of a sincosf would be paid at full latency, 16 times per
// 32 columns, and the epilogue, not the tensor core, would set the kernel's pace.
struct RopeEpilogue {
  const int* positions;
  const int* token_row;
  const float2* cos_sin;
  const int* block_table;
  bf16* kc;
  bf16* vc;
  int* errors;
  int rot, H, Hkv, D, bt_width, ps, num_pages, write_cache;
};

// Where the keys and values of this thread's row go: element offset of (page, kv head 0, slot, 0) or -1.
__device__ __forceinline__ long long rope_row_slot(const RopeEpilogue& ra, int row, int pos) {
  const int blk = pos / ra.ps;
  const int page = (blk < ra.bt_width && pos >= 0) ? ra.block_table[(size_t)ra.token_row[row] * ra.bt_width + blk] : -1;
  if (page < 0 || page >= ra.num_pages) return -1;
  return ((long long)page * ra.Hkv * ra.ps + (pos - blk * ra.ps)) * ra.D;
}

// 32 accumulator columns n .. n+31 of one row: rounded to bfloat16 as the unfused path stores them, q and k pairs
// rotated, then q to out and k, v to the row's slot in the cache.
__device__ __forceinline__ void rope_store_chunk(const RopeEpilogue& ra, const uint32_t (&v)[32], int row, int n, int M, int N,
                                                 long long slot, bf16* __restrict__ out) {
  const int head = n / ra.D, d0 = n - head * ra.D;
  uint32_t packed[16];
  const bool turns = head < ra.H + ra.Hkv;
  // the table is [pair][row]: the 32 rows of a warp read 256 consecutive bytes per pair. All loads first, so that
  // their latencies overlap (a warp alone on its scheduler has nothing else to run meanwhile).
  float2 a[16];
  const float2* angles = ra.cos_sin + (size_t)(d0 >> 1) * M + row;
#pragma unroll
  for (int i = 0; i < 16; ++i) a[i] = (turns && d0 + 2 * i < ra.rot) ? __ldg(angles + (size_t)i * M) : make_float2(1.f, 0.f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float x = to_float(__float2bfloat16_rn(__uint_as_float(v[2 * i]))), y = to_float(__float2bfloat16_rn(__uint_as_float(v[2 * i + 1])));
    __nv_bfloat162 o;
    if (turns && d0 + 2 * i < ra.rot) o = __floats2bfloat162_rn(x * a[i].x - y * a[i].y, y * a[i].x + x * a[i].y);
    else o = __floats2bfloat162_rn(x, y);
    packed[i] = *reinterpret_cast<uint32_t*>(&o);
  }
  bf16* dst;
  if (head < ra.H) {
    dst = out + (size_t)row * N + n;
  } else {
    if (!ra.write_cache) return;
    if (slot < 0) {
      if (n == ra.H * ra.D) atomicAdd(ra.errors, 1);       // once per token
      return;
    }
    const bool is_k = turns;
    const int kvh = is_k ? head - ra.H : head - ra.H - ra.Hkv;
    dst = (is_k ? ra.kc : ra.vc) + slot + (long long)kvh * ra.ps * ra.D + d0;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
}

template <int EPI>
__global__ void __launch_bounds__(THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_w, bf16* __restrict__ out,
                                                               int M, int N, int K, int bn, int* __restrict__ error,
                                                               const RopeEpilogue ra) {
  constexpr bool GU = EPI == EPI_GATE_UP;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[NSTAGE];
  __shared__ __align__(8) uint64_t empty_bar[NSTAGE];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  // the dynamic region is aligned by hand: the 128-byte swizzle wants 1024-byte aligned tiles
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // bn: accumulator columns of a tile (a multiple of 32, at most BN), chosen by the host so that the tiles
  // fill whole waves of CTAs
  const int OUT_COLS = GU ? bn / 2 : bn;             // output columns of one tile
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + OUT_COLS - 1) / OUT_COLS;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPI_WARPS);       // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // barriers, tensor memory and descriptors are ready; the activations (and the right to overwrite out) come with
  // the end of the kernel before this one
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_s;
  bool failed = false;

  // tile t of this CTA: consecutive CTAs take the row tiles of one panel of w
  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                      // stages issued so far, over all tiles
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * OUT_COLS;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % NSTAGE;
          // a fresh barrier passes a wait on parity 1: the first round finds every stage free
          if (!mbar_wait(&empty_bar[s], ((it / NSTAGE) & 1) ^ 1)) { failed = true; break; }
          unsigned char* a_dst = tiles + (size_t)s * STAGE_BYTES;
          unsigned char* b_dst = a_dst + A_BYTES;
          mbar_expect_tx(&full_bar[s], (unsigned)(A_BYTES + bn * BK * 2));
          tma_load_2d(a_dst, &map_a, &full_bar[s], kb * BK, m0);
          if (GU) {
            tma_load_2d(b_dst, &map_w, &full_bar[s], kb * BK, n0);                       // 128 gate rows
            tma_load_2d(b_dst + (size_t)(bn / 2) * BK * 2, &map_w, &full_bar[s], kb * BK, N + n0);   // their up rows
          } else {
            tma_load_2d(b_dst, &map_w, &full_bar[s], kb * BK, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, bn);
      int it = 0, local = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue must have emptied this accumulator (first use of each: passes at once)
        if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1)) { failed = true; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % NSTAGE;
          if (!mbar_wait(&full_bar[s], (it / NSTAGE) & 1)) { failed = true; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t da = make_desc(a_addr), db = make_desc(a_addr + A_BYTES);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            // 16 k-values further along the swizzled row: 32 bytes, two 16-byte units of the start address
            tc_mma(acc, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (kb | j) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);          // the stage is free once these products have read it
        }
        tc_commit(&acc_full[buf]);           // the accumulator is complete once all products are done
      }
    }
  } else {
    // epilogue warps: a warp may touch the 32 tensor-memory lanes of its rank modulo 4; the warps of a quarter take
    // the chunks of 32 columns in turn. With a tile or two per CTA the last tile's epilogue is not hidden behind any
    // product, and a warp alone on its scheduler pays every instruction's latency in full: with four warps (one per
    // quarter) the q/k/v product with rotation took 41.7 us inside a 2,048-token step, with eight 40.7, with sixteen 35.6.
    const int q = warp & 3, c_first = ((warp - 2) >> 2) * 32;
    int local = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local) {
      const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * OUT_COLS;
      const int buf = local & 1;
      if (!mbar_wait(&acc_full[buf], (local >> 1) & 1)) { failed = true; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      int pos = 0;
      long long slot = -1;
      if (EPI == EPI_ROPE && row < M) {
        pos = ra.positions[row];
        if (ra.write_cache && n0 + OUT_COLS > ra.H * ra.D) slot = rope_row_slot(ra, row, pos);
      }
#pragma unroll 1
      for (int c = c_first; c < OUT_COLS; c += 32 * (EPI_WARPS / 4)) {
        if (n0 + c >= N) break;
        uint32_t v[32];
        tc_load32(acc + (uint32_t)c, v);
        if (EPI == EPI_ROPE) {
          if (row < M) rope_store_chunk(ra, v, row, n0 + c, M, N, slot, out);
          continue;
        }
        uint32_t packed[16];
        if (GU) {
          uint32_t u[32];
          tc_load32(acc + (uint32_t)(OUT_COLS + c), u);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // both halves rounded to the activation type first, as the unfused path stores them
            const float g0 = to_float(__float2bfloat16_rn(__uint_as_float(v[2 * i]))), g1 = to_float(__float2bfloat16_rn(__uint_as_float(v[2 * i + 1])));
            const float u0 = to_float(__float2bfloat16_rn(__uint_as_float(u[2 * i]))), u1 = to_float(__float2bfloat16_rn(__uint_as_float(u[2 * i + 1])));
            __nv_bfloat162 o = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
            packed[i] = *reinterpret_cast<uint32_t*>(&o);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            packed[i] = *reinterpret_cast<uint32_t*>(&o);
          }
        }
        if (row < M) {
          bf16* dst = out + (size_t)row * N + n0 + c;
          if (n0 + c + 32 <= N) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          } else {
            for (int i = 0; i < 32; ++i)
              if (n0 + c + i < N) dst[i] = reinterpret_cast<const bf16*>(packed)[i];
          }
        }
      }
      // this warp has read its part of the accumulator: the next tile but one may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
    }
  }
  if (failed) atomicExch(error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------------------
// The same product with two CTAs (a cluster of two, on neighbouring SMs) working on one 256 x bn tile:
// tcgen05.mma.cta_group::2. CTA r of the pair holds rows 128 r .. 128 r + 127 of the tile's a operand and the r-th
// half of its w operand in its own shared memory, and its 128 rows of the accumulator in its own tensor memory.
// One thread of the first CTA issues the products for both; each product reads both shared memories, so every CTA
// loads (and the tensor core reads) only half of w per tile: shared-memory traffic per flop is 2/3 of the
// one-CTA kernel's, which is what that kernel is bound by. A stage is 16 KB of a + at most 16 KB of w, six stages.
//
// Barriers: both CTAs' TMA loads count their bytes on the first CTA's full barrier (its address with the pair bit
// cleared); tcgen05.commit arrives on the empty / accumulator-full barriers of both CTAs at once (multicast);
// the epilogue warps of both CTAs arrive on the first CTA's accumulator-empty barrier (a remote arrive for the second).
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_A_BYTES = 128 * BK * 2, PAIR_STAGE_BYTES = PAIR_A_BYTES + 128 * BK * 2;
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;   // clears the bit of a shared-memory address that tells the two CTAs apart

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the products issued so far are done, on the barrier at this address in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void cluster_sync_all_threads() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS)
    gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                             bf16* __restrict__ out, int M, int N, int K, int bn, int* __restrict__ error,
                             const RopeEpilogue ra) {
  constexpr bool GU = EPI == EPI_GATE_UP;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[PAIR_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[PAIR_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int OUT_COLS = GU ? bn / 2 : bn;
  const int half = bn / 2;                              // rows of w this CTA loads per stage
  const int m_tiles = (M + 255) / 256, n_tiles = (N + OUT_COLS - 1) / OUT_COLS;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * EPI_WARPS);   // one arrival per epilogue warp of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }
  if (warp == 1) {
    // the same warp of both CTAs allocates: the accumulators get the same address in both tensor memories
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all_threads();            // the other CTA's barriers exist before anything arrives on them
  tc_fence_after();
  pdl_launch_dependents();
  pdl_wait();                            // as in the one-CTA kernel
  const uint32_t tmem_base = tmem_base_s;
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      for (int tile = pair; tile < total_tiles && !failed; tile += num_pairs) {
        const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * OUT_COLS;
        // with gate_up the first CTA loads the gate rows and the second their up rows: accumulator columns
        // 0 .. half-1 are gate, half .. bn-1 are up, for the rows of both CTAs
        const int w_row = GU ? (rank == 0 ? n0 : N + n0) : n0 + (int)rank * half;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % PAIR_STAGES;
          if (!mbar_wait(&empty_bar[s], ((it / PAIR_STAGES) & 1) ^ 1)) { failed = true; break; }
          unsigned char* a_dst = tiles + (size_t)s * PAIR_STAGE_BYTES;
          const uint32_t leader_bar = smem_u32(&full_bar[s]) & PAIR_LEADER_MASK;
          if (rank == 0) mbar_expect_tx(&full_bar[s], (unsigned)(2 * (PAIR_A_BYTES + half * BK * 2)));
          tma_load_2d_pair(a_dst, &map_a, leader_bar, kb * BK, m0);
          tma_load_2d_pair(a_dst + PAIR_A_BYTES, &map_w, leader_bar, kb * BK, w_row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(256, bn);
      int it = 0, local = 0;
      for (int tile = pair; tile < total_tiles && !failed; tile += num_pairs, ++local) {
        const int buf = local & 1;
        if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1)) { failed = true; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % PAIR_STAGES;
          if (!mbar_wait(&full_bar[s], (it / PAIR_STAGES) & 1)) { failed = true; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * PAIR_STAGE_BYTES);
          const uint64_t da = make_desc(a_addr), db = make_desc(a_addr + PAIR_A_BYTES);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j)
            tc_mma_pair(acc, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (kb | j) != 0 ? 1u : 0u);
          tc_commit_pair(&empty_bar[s]);
        }
        tc_commit_pair(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3, c_first = ((warp - 2) >> 2) * 32;
    uint32_t leader_acc_empty[2];
#pragma unroll
    for (int b = 0; b < 2; ++b)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(leader_acc_empty[b]) : "r"(smem_u32(&acc_empty[b])), "r"(0u));
    int local = 0;
    for (int tile = pair; tile < total_tiles && !failed; tile += num_pairs, ++local) {
      const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * OUT_COLS;
      const int buf = local & 1;
      if (!mbar_wait(&acc_full[buf], (local >> 1) & 1)) { failed = true; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      int pos = 0;
      long long slot = -1;
      if (EPI == EPI_ROPE && row < M) {
        pos = ra.positions[row];
        if (ra.write_cache && n0 + OUT_COLS > ra.H * ra.D) slot = rope_row_slot(ra, row, pos);
      }
#pragma unroll 1
      for (int c = c_first; c < OUT_COLS; c += 32 * (EPI_WARPS / 4)) {
        if (n0 + c >= N) break;
        uint32_t v[32];
        tc_load32(acc + (uint32_t)c, v);
        if (EPI == EPI_ROPE) {
          if (row < M) rope_store_chunk(ra, v, row, n0 + c, M, N, slot, out);
          continue;
        }
        uint32_t packed[16];
        if (GU) {
          uint32_t u[32];
          tc_load32(acc + (uint32_t)(OUT_COLS + c), u);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g0 = to_float(__float2bfloat16_rn(__uint_as_float(v[2 * i]))), g1 = to_float(__float2bfloat16_rn(__uint_as_float(v[2 * i + 1])));
            const float u0 = to_float(__float2bfloat16_rn(__uint_as_float(u[2 * i]))), u1 = to_float(__float2bfloat16_rn(__uint_as_float(u[2 * i + 1])));
            __nv_bfloat162 o = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
            packed[i] = *reinterpret_cast<uint32_t*>(&o);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            packed[i] = *reinterpret_cast<uint32_t*>(&o);
          }
        }
        if (row < M) {
          bf16* dst = out + (size_t)row * N + n0 + c;
          if (n0 + c + 32 <= N) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          } else {
            for (int i = 0; i < 32; ++i)
              if (n0 + c + i < N) dst[i] = reinterpret_cast<const bf16*>(packed)[i];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(leader_acc_empty[buf]) : "memory");
    }
  }
  if (failed) atomicExch(error, 1);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all_threads();            // neither CTA leaves, or frees tensor memory, while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// rows x cols bfloat16, row-major; box of box_rows x 64 columns, 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn) return -300;
    g_encode = (EncodeTiledFn)fn;
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -301 - (int)r;
}

int g_pair_enabled = 1;
int g_forced_width = 0;      // tests: accumulator columns per tile instead of the tile plan's choice
int g_pair_capacity[3] = {0, 0, 0};

bool pair_mode(int M) { return g_pair_enabled && M > 128; }

template <int EPI>
int pair_capacity_of(int sms) {
  const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms / 2 * 2, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  int clusters = 0;
  cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<EPI>, &cfg);
  if (e != cudaSuccess || clusters < 1) { cudaGetLastError(); clusters = sms / 2; }
  return clusters > sms / 2 ? sms / 2 : clusters;
}

// CTA pairs of the two-CTA kernel that the device holds at a time (the persistent grid's size)
int pair_capacity(int epi, int sms) {
  int& cached = g_pair_capacity[epi];
  if (cached > 0) return cached;
  cached = epi == EPI_GATE_UP ? pair_capacity_of<EPI_GATE_UP>(sms) : epi == EPI_ROPE ? pair_capacity_of<EPI_ROPE>(sms)
                                                                                      : pair_capacity_of<EPI_STORE>(sms);
  return cached;
}

template <int EPI>
cudaError_t launch_single(dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_w, bf16* out,
                          int M, int N, int K, int bn, int* error, const RopeEpilogue& ra) {
  auto k = gemm_tcgen05_kernel<EPI>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_pdl(k, grid, dim3(THREADS), smem, stream, map_a, map_w, out, M, N, K, bn, error, ra);
}

template <int EPI>
cudaError_t launch_pair(dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_w, bf16* out,
                        int M, int N, int K, int bn, int* error, const RopeEpilogue& ra) {
  return launch_pdl(gemm_tcgen05_pair_kernel<EPI>, grid, dim3(THREADS), smem, stream, map_a, map_w, out, M, N, K, bn, error, ra);
}

int supports(int M, int N, int K, int epi) {
  if (M < 1 || N < 8 || K < 8 || (K % 8) || (N % 8)) return 0;     // 16-byte row pitch for TMA, vector stores
  if (epi == EPI_GATE_UP && (N % 128)) return 0;                    // a tile's 128 gate rows must not reach into the up rows
  return 1;
}

// a [M,K], w [N,K] (or [2N,K] with gate/up), out [M,N]; all bfloat16, row-major, 16-byte aligned.
int run_product(const void* a, const void* w, void* out, int M, int N, int K, int epi, const RopeEpilogue& ra, int* error,
                cudaStream_t stream) {
  if (!supports(M, N, K, epi)) return SB_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(w) || !aligned16(out) || !error) return SB_ERR_ALIGN;
  const bool gate_up = epi == EPI_GATE_UP;
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, a, (uint64_t)M, (uint64_t)K, BM);
  if (rc) return rc;
  const int sms = sm_count();
  // Tile plan. A wave of tiles takes about (tile width + a fixed part worth 32 columns) whether its tiles are 128 rows
  // on one CTA or 256 rows on a CTA pair (each SM works on 128 rows either way), so the two kernels' costs compare
  // directly: whole waves needed x that time, for the best width of each. Ragged row counts decide it: 330 rows are
  // three 128-row tiles but two 256-row ones (512 rows of work).
  const bool forced = g_forced_width >= 32 && g_forced_width <= BN && (g_forced_width % 32) == 0 && !gate_up;
  const int widest = forced ? g_forced_width : BN, narrowest = forced ? g_forced_width : (gate_up ? BN : 128);
  long long cost_single = -1, cost_pair = -1, waves_pair = 0;
  int bn_single = BN, bn_pair = BN;
  const int pairs = pair_mode(M) ? pair_capacity(epi, sms) : 0;
  for (int cand = widest; cand >= narrowest; cand -= 32) {
    const int out_cols = gate_up ? cand / 2 : cand;
    const long long n_tiles = (N + out_cols - 1) / out_cols;
    const long long w1 = (((M + 127) / 128) * n_tiles + sms - 1) / sms;
    if (cost_single < 0 || w1 * (cand + 32) < cost_single) { cost_single = w1 * (cand + 32); bn_single = cand; }
    if (pairs > 0) {
      const long long w2 = (((M + 255) / 256) * n_tiles + pairs - 1) / pairs;
      if (cost_pair < 0 || w2 * (cand + 32) < cost_pair) { cost_pair = w2 * (cand + 32); bn_pair = cand; waves_pair = w2; }
    }
  }
  cudaError_t e;
  // At equal cost the pair kernel wins only where a CTA has enough to do: starting and ending a cluster costs it about
  // 2 us more than the one-CTA kernel (2,048 rows: q/k/v 32.5 against 29.8 us, output projection 20.5 against 18.7, but
  // down projection, four times as many k-values, 53.3 against 54.8).
  const long long k_blocks = (K + BK - 1) / BK;
  const bool pair_wins = cost_pair < cost_single || (cost_pair == cost_single && waves_pair * k_blocks >= 96);
  if (pairs > 0 && (pair_wins || g_pair_enabled == 2)) {
    const long long m_tiles = (M + 255) / 256;
    const int bn = bn_pair;
    rc = make_map(&map_w, w, (uint64_t)(gate_up ? 2 * N : N), (uint64_t)K, bn / 2);
    if (rc) return rc;
    const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024;
    const int out_cols = gate_up ? bn / 2 : bn;
    const long long tiles = (long long)((N + out_cols - 1) / out_cols) * m_tiles;
    dim3 grid((unsigned)(2 * (tiles < pairs ? tiles : pairs)));
    e = epi == EPI_GATE_UP ? launch_pair<EPI_GATE_UP>(grid, smem, stream, map_a, map_w, (bf16*)out, M, N, K, bn, error, ra)
        : epi == EPI_ROPE  ? launch_pair<EPI_ROPE>(grid, smem, stream, map_a, map_w, (bf16*)out, M, N, K, bn, error, ra)
                           : launch_pair<EPI_STORE>(grid, smem, stream, map_a, map_w, (bf16*)out, M, N, K, bn, error, ra);
    SB_PDL_CHECK(e);
    return 0;
  }
  const long long m_tiles = (M + BM - 1) / BM;
  const int bn = bn_single;
  rc = make_map(&map_w, w, (uint64_t)(gate_up ? 2 * N : N), (uint64_t)K, gate_up ? bn / 2 : bn);
  if (rc) return rc;
  const size_t smem = (size_t)NSTAGE * STAGE_BYTES + 1024;
  const int out_cols = gate_up ? bn / 2 : bn;
  const long long tiles = (long long)((N + out_cols - 1) / out_cols) * m_tiles;
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  e = epi == EPI_GATE_UP ? launch_single<EPI_GATE_UP>(grid, smem, stream, map_a, map_w, (bf16*)out, M, N, K, bn, error, ra)
      : epi == EPI_ROPE  ? launch_single<EPI_ROPE>(grid, smem, stream, map_a, map_w, (bf16*)out, M, N, K, bn, error, ra)
                         : launch_single<EPI_STORE>(grid, smem, stream, map_a, map_w, (bf16*)out, M, N, K, bn, error, ra);
  SB_PDL_CHECK(e);
  return 0;
}

}  // namespace

// 0 keeps every product on the one-CTA kernel, 1 (the default) lets products of more than 128 rows go to CTA pairs
// where the tile plan says they are no slower, 2 sends all of those to CTA pairs (tests).
SB_EXPORT void sb_gemm_tcgen05_use_pairs(int on) { g_pair_enabled = on; }
// 0: the tile plan chooses; a multiple of 32 up to 256: every product without gate/up uses tiles of that many columns
SB_EXPORT void sb_gemm_tcgen05_force_width(int bn) { g_forced_width = bn; }
SB_EXPORT int sb_gemm_tcgen05_pair_capacity(int gate_up) { return pair_capacity(gate_up ? EPI_GATE_UP : EPI_STORE, sm_count()); }

// 1 if sb_gemm_tcgen05 takes these sizes (else the caller uses the library product).
SB_EXPORT int sb_gemm_tcgen05_supports(int M, int N, int K, int gate_up) { return supports(M, N, K, gate_up ? EPI_GATE_UP : EPI_STORE); }

// error: device int set to 1 if a bounded wait inside the kernel ran out.
SB_EXPORT int sb_gemm_tcgen05(const void* a, const void* w, void* out, int M, int N, int K, int gate_up, int* error,
                              cudaStream_t stream) {
  return run_product(a, w, out, M, N, K, gate_up ? EPI_GATE_UP : EPI_STORE, RopeEpilogue{}, error, stream);
}

// 1 if sb_gemm_tcgen05_qkv_rope takes these sizes: whole heads of a multiple of 32 elements, an even rotary width.
SB_EXPORT int sb_gemm_tcgen05_qkv_rope_supports(int M, int K, int rot, int H, int Hkv, int D) {
  if (H < 1 || Hkv < 1 || D < 32 || (D % 32) || rot < 0 || rot > D || (rot & 1)) return 0;
  return supports(M, (H + 2 * Hkv) * D, K, EPI_ROPE);
}

// The q/k/v product of an attention layer: out[M, (H + 2 Hkv) D] gets the rotated queries (its key and value columns
// are left untouched); rotated keys and the values go to kc / vc [pages, Hkv, ps, D] at each token's position, through
// its request's row of the block table. cos_sin [rot/2, M] pairs of floats from sb_rope_angles for the same positions. errors counts tokens without a page; wait_error as in sb_gemm_tcgen05.
SB_EXPORT int sb_gemm_tcgen05_qkv_rope(const void* a, const void* w, void* out, int M, int K, const int* positions,
                                       const int* token_row, const float* cos_sin, int rot, int H, int Hkv, int D, void* kc,
                                       void* vc, const int* block_table, int bt_width, int ps, int num_pages, int write_cache,
                                       int* errors, int* wait_error, cudaStream_t stream) {
  if (!sb_gemm_tcgen05_qkv_rope_supports(M, K, rot, H, Hkv, D) || ps <= 0) return SB_ERR_SHAPE;
  if (!positions || !errors || (rot > 0 && (!cos_sin || ((uintptr_t)cos_sin & 7)))) return SB_ERR_ALIGN;
  if (write_cache && (!kc || !vc || !block_table || !token_row || !aligned16(kc) || !aligned16(vc))) return SB_ERR_ALIGN;
  RopeEpilogue ra;
  ra.positions = positions;
  ra.token_row = token_row;
  ra.cos_sin = (const float2*)cos_sin;
  ra.block_table = block_table;
  ra.kc = (bf16*)kc;
  ra.vc = (bf16*)vc;
  ra.errors = errors;
  ra.rot = rot; ra.H = H; ra.Hkv = Hkv; ra.D = D;
  ra.bt_width = bt_width; ra.ps = ps; ra.num_pages = num_pages; ra.write_cache = write_cache;
  return run_product(a, w, out, M, (H + 2 * Hkv) * D, K, EPI_ROPE, ra, wait_error, stream);
}
