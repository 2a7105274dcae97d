// A run of decoder layers for a decoding step (one token per request, at most 16 requests) as ONE persistent kernel.
//
// A decoding step of a small batch is a chain of short kernels per layer (norm, q/k/v product, attention, output
// projection, norm, gate/up product, down projection), each of which reads a few megabytes of weights and then hands
// over to the next: most of a layer's time is hand-over, not bytes. Here one thread block per SM stays resident for
// the whole run of layers. The five phases of a layer are separated by barriers across the grid, and what makes the
// barriers cheap is that the weights do not depend on the activations: every warp walks one fixed list of weight
// chunks for the whole kernel (all phases of all layers) and keeps a ring of cp.async copies running ahead of what it
// consumes, across phase boundaries and barrier waits, so the memory system keeps streaming while the blocks meet.
//
// Work of a phase: the output columns (rows of the weight matrix) are dealt out evenly over the blocks, in pairs.
// Inside a block the rows form tiles of 8, each tile's K range is cut into slices, and the (tile, slice) units are
// dealt to the 8 warps; a warp multiplies its unit on the tensor cores (mma.sync m16n8k16: activation rows are the
// 16-row operand, resident in shared memory; 8 weight rows the 8-column operand, from the ring). Slices of a tile
// meet in shared memory and are added in a fixed order, so a row's result does not depend on the other rows.
//   phase 1  x' = x + pending, h = rmsnorm(x'), q/k/v = h Wqkv^T, rotation of q and k, k and v into the cache pages
//   phase 2  attention of each (request, kv head[, key split]) over the cache (split results merged by the last arriver)
//   phase 3  delta = attn Wo^T
//   phase 4  x'' = x' + delta, h = rmsnorm(x''), act = silu(h Wg^T) * (h Wu^T)
//   phase 5  pending = act Wd^T
// Rounding points are those of the separate kernels (activations bfloat16, residual stream float32, norms, rotation
// angles and softmax statistics float32). Formulas: serve/model.py:63-68 (norm), :80-85 (SwiGLU), :104-134 (attention
// layer), :146-149 (block), :234-244 (rotation); serve/kernels/attn_decode.py:92-111 (online softmax).
//
// Every wait is bounded: a grid barrier that does not complete within its iteration limit sets the error flag, and
// the block runs on without waiting (its results are then not valid, which the flag says). Blocks wait only for
// blocks of this same launch, which is cooperative: all of them are resident.
// Compile with -DSB_HEAD_DIM=<multiple of 16, 16..256>.
#include "common.cuh"
#include "decode_stack.h"

#ifndef SB_HEAD_DIM
#error "define SB_HEAD_DIM"
#endif

using namespace sb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int D = SB_HEAD_DIM;
constexpr int NWARPS = 8;
constexpr int NTHR = NWARPS * 32;
constexpr int CK = 128;                          // k-values of a weight chunk (one ring stage: 8 rows x 128 k = 2 KB)
constexpr int STAGE_ELEMS = 8 * CK;
constexpr int NST = 8;                           // ring stages per warp
constexpr int MAX_UNITS = 64;                    // (tile, slice) units of a block in one phase
constexpr int ACAP_FULL = 2048, ACAP_HALF = 4096;  // k-values of the activation operand resident at a time (16 / 8 rows)
constexpr int APAD = 8;
constexpr int MAX_SPLITS = 32;

constexpr size_t A_BYTES = (size_t)16 * (ACAP_FULL + APAD) * sizeof(bf16);      // = 8 * (ACAP_HALF + 8) * 2 (rounded up)
constexpr size_t RING_BYTES = (size_t)NWARPS * NST * STAGE_ELEMS * sizeof(bf16);
constexpr size_t RED_BYTES = (size_t)MAX_UNITS * 128 * sizeof(float);
constexpr size_t SMEM_BYTES = A_BYTES + RED_BYTES + RING_BYTES;
static_assert((size_t)8 * (ACAP_HALF + APAD) * sizeof(bf16) <= A_BYTES, "the half-height operand must fit the same space");

// attention phase: keys per warp step, stages per warp, and as many warps as fit the operand + reduction space
constexpr int AKW = 16;
constexpr int ASTAGES = 2;
constexpr int ALDS = D + 8;
constexpr size_t ATT_STAGE_BYTES = (size_t)2 * AKW * ALDS * sizeof(bf16);
constexpr size_t ATT_Q_BYTES = (size_t)16 * ALDS * sizeof(bf16);
constexpr int att_warps_for(size_t space) {
  int w = NWARPS;
  while (w > 1 && ATT_Q_BYTES + (size_t)w * ASTAGES * ATT_STAGE_BYTES > space) w >>= 1;
  return w;
}
constexpr int ATT_WARPS = att_warps_for(A_BYTES + RED_BYTES);
static_assert(ATT_Q_BYTES + (size_t)ATT_WARPS * ASTAGES * ATT_STAGE_BYTES <= A_BYTES + RED_BYTES, "attention tiles do not fit");
static_assert((size_t)ATT_WARPS * 16 * (D + 2) * sizeof(float) + (2 * MAX_SPLITS + 1) * 16 * sizeof(float) <= A_BYTES + RED_BYTES,
              "attention merge space does not fit");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
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
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct Params {
  const SbStackLayer* layers;
  int n_layers, M;
  int hidden, H, Hkv, inter;
  const int* positions;           // [M]
  const int* kv_len;              // [M] lengths after this step
  const int* block_tables[SB_STACK_MAX_GROUPS];
  int bt_width[SB_STACK_MAX_GROUPS];
  int ps, ps_shift;
  float* xa;                      // [M, hidden] residual stream (in and out)
  float* xb;                      // [M, hidden] scratch
  const bf16* first_delta;        // pending delta of whatever ran before, or null
  bf16* delta_o;                  // [M, hidden]
  bf16* delta_down;               // [M, hidden]: the pending delta after the last layer
  bf16* qkv;                      // [M, (H + 2 Hkv) D] (query columns used)
  bf16* attn;                     // [M, H D]
  bf16* act;                      // [M, inter]
  float* part_o;                  // [M, Hkv, splits, 16, D]
  float* part_ml;                 // [M, Hkv, splits, 16, 2]
  int* tickets;                   // [M, Hkv], zero before and after
  int num_splits;
  unsigned* barrier;              // [0] arrivals at barriers, [1] blocks that have left: zero before the launch and after it
  int* errors;                    // [0] cache writes that met a missing page, [1] a wait ran out
  long long* timing;              // null, or [n_layers][10] nanosecond stamps of block 0: after each phase and each barrier
};

__device__ __forceinline__ void stamp(const Params& p, int layer, int slot) {
  if (p.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.timing[layer * 10 + slot] = t;
  }
}

// ---- the grid barrier -------------------------------------------------------------------------------------------
struct Grid {
  unsigned* counter;
  unsigned arrived;     // barriers passed so far
  int* errors;
  bool aborted;
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All blocks of the launch meet. What a block wrote before is visible to every block after. The wait is bounded.
__device__ __forceinline__ void grid_barrier(Grid& g) {
  __syncthreads();
  g.arrived += 1;
  if (threadIdx.x == 0 && !g.aborted) {
    __threadfence();
    atomicAdd(g.counter, 1u);
    const unsigned target = g.arrived * gridDim.x;
    unsigned spins = 0;
    while (ld_acquire(g.counter) < target) {
      if (++spins > (1u << 24)) {                  // about a second: something is badly wrong
        atomicExch(g.errors + 1, 1);
        g.aborted = true;
        break;
      }
      if (spins > 64) __nanosleep(32);
    }
    __threadfence();
  }
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = g.aborted ? 1 : 0;
  __syncthreads();
  g.aborted = s_abort != 0;
}

// ---- geometry of a product phase for one block --------------------------------------------------------------------
enum { PH_QKV = 0, PH_O = 1, PH_GU = 2, PH_DOWN = 3, N_PHASES = 4 };

struct Geo {
  const bf16* w;
  int K;            // row length of w
  int row_lo;       // first output column of this block
  int n_rows;       // its columns (for gate/up: columns of the activation; gate and up rows both)
  int tiles;        // 8-row tiles (gate tiles then up tiles for gate/up)
  int gate_tiles;   // tiles / 2 for gate/up, else tiles
  int up_off;       // row offset of the up half in w (inter) for gate/up, else 0
  int ks;           // K slices of a tile inside a segment
  int slice;        // k-values of a slice
  int kseg;         // k-values of a segment (resident activation operand)
  int nseg;
};

template <bool HALF>
__device__ __forceinline__ Geo make_geo(const Params& p, const SbStackLayer& L, int phase) {
  Geo g;
  const int acap = HALF ? ACAP_HALF : ACAP_FULL;
  int n_total;
  g.up_off = 0;
  if (phase == PH_QKV) { g.w = (const bf16*)L.wqkv; g.K = p.hidden; n_total = (p.H + 2 * p.Hkv) * D; }
  else if (phase == PH_O) { g.w = (const bf16*)L.wo; g.K = p.H * D; n_total = p.hidden; }
  else if (phase == PH_GU) { g.w = (const bf16*)L.wgu; g.K = p.hidden; n_total = p.inter; g.up_off = p.inter; }
  else { g.w = (const bf16*)L.wdown; g.K = p.inter; n_total = p.hidden; }
  const long long pairs = n_total / 2;
  const int lo = 2 * (int)((long long)blockIdx.x * pairs / gridDim.x);
  const int hi = 2 * (int)((long long)(blockIdx.x + 1) * pairs / gridDim.x);
  g.row_lo = lo;
  g.n_rows = hi - lo;
  g.gate_tiles = (g.n_rows + 7) / 8;
  g.tiles = phase == PH_GU ? 2 * g.gate_tiles : g.gate_tiles;
  g.kseg = g.K < acap ? g.K : acap;
  g.nseg = g.K / g.kseg;
  int ks = g.tiles >= 32 ? 1 : (g.tiles >= 16 ? 2 : (g.tiles >= 8 ? 4 : 8));
  while (ks > 1 && ((g.kseg % (ks * CK)) != 0 || g.tiles * ks > MAX_UNITS)) ks >>= 1;
  g.ks = ks;
  g.slice = g.kseg / ks;
  return g;
}

// Ask for this block's rows of a later phase's weights to be brought into the L2 cache (rows of a block are one
// contiguous range; gate and up rows are two). Nothing waits for it: it keeps the memory system streaming through
// barriers, norms and attention, when the ring of copies stands still. which: 0 all, 1 gate rows only, 2 up rows only.
constexpr int PF_PIECE = 16384;
#ifndef SB_STACK_L2_PREFETCH
#define SB_STACK_L2_PREFETCH 0
#endif
template <bool HALF>
__device__ __forceinline__ void prefetch_phase(const Params& p, int layer, int phase, int which) {
  if (!SB_STACK_L2_PREFETCH || layer >= p.n_layers) return;
  const Geo g = make_geo<HALF>(p, p.layers[layer], phase);
  const size_t bytes = (size_t)g.n_rows * g.K * sizeof(bf16);
  const int pieces = (int)((bytes + PF_PIECE - 1) / PF_PIECE);
  for (int part = 0; part < (phase == PH_GU ? 2 : 1); ++part) {
    if (phase == PH_GU && which != 0 && which != part + 1) continue;
    const char* base = reinterpret_cast<const char*>(g.w + (size_t)((part ? g.up_off : 0) + g.row_lo) * g.K);
    for (int i = threadIdx.x; i < pieces; i += NTHR) {
      const size_t off = (size_t)i * PF_PIECE;
      const unsigned n = (unsigned)(bytes - off < (size_t)PF_PIECE ? bytes - off : (size_t)PF_PIECE);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(base + off), "r"(n) : "memory");
    }
  }
}

// ---- a warp's walk over its weight chunks: one list for the whole kernel -------------------------------------------
template <bool HALF>
struct Cursor {
  int layer, phase, seg, unit, ck;
  bool done;
  Geo g;

  __device__ __forceinline__ void settle(const Params& p, int warp) {
    // move on to the next phase (segment) in which this warp has a unit
    while (!done) {
      if (unit < g.tiles * g.ks) return;
      unit = warp;
      ck = 0;
      if (++seg < g.nseg) continue;
      seg = 0;
      if (++phase == N_PHASES) {
        phase = 0;
        if (++layer >= p.n_layers) { done = true; return; }
      }
      g = make_geo<HALF>(p, p.layers[layer], phase);
    }
  }
  __device__ __forceinline__ void start(const Params& p, int warp) {
    layer = 0; phase = 0; seg = 0; unit = warp; ck = 0; done = p.n_layers <= 0;
    if (!done) g = make_geo<HALF>(p, p.layers[0], 0);
    settle(p, warp);
  }
  __device__ __forceinline__ void advance(const Params& p, int warp) {
    if (done) return;
    if (++ck * CK >= g.slice) {
      ck = 0;
      unit += NWARPS;
      settle(p, warp);
    }
  }
  // issue the copies of the current chunk into ``stage`` (8 rows x 128 k, 16-byte pieces swizzled by row)
  __device__ __forceinline__ void issue(bf16* stage, int lane) const {
    if (done) return;
    const int t = unit / g.ks, s = unit - t * g.ks;
    const bool up = t >= g.gate_tiles;
    const int tt = up ? t - g.gate_tiles : t;
    const int r0 = (up ? g.up_off : 0) + g.row_lo + 8 * tt;
    const int valid = min(8, g.n_rows - 8 * tt);
    const int k0 = seg * g.kseg + s * g.slice + ck * CK;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j;
      const int row = i >> 4, c16 = i & 15;
      const bool ok = row < valid;
      const bf16* src = g.w + (size_t)(r0 + (ok ? row : 0)) * g.K + k0 + c16 * 8;
      cp_async16(stage + row * CK + ((c16 ^ row) & 15) * 8, src, ok);
    }
  }
};

// ---- phases -----------------------------------------------------------------------------------------------------

// x_out = x_in + delta (all rows, this block's share of the columns); A_s[m] = bf16(rmsnorm(x_in[m] + delta[m]) * w).
// One warp per row; a lane's loads go out together (16 float4 at a time), sums in index order within a lane, then a
// fixed shuffle tree. Rows of up to 2,048 values stay in registers between the sum and the scaling.
#ifndef SB_STACK_NV
#define SB_STACK_NV 4
#endif
constexpr int NV = SB_STACK_NV;

__device__ __forceinline__ void norm_load_tile(const float* xr, const bf16* dr, int base, int n4, int lane, float4 (&v)[NV]) {
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = base + lane + 32 * j;
    v[j] = i < n4 ? __ldcg(reinterpret_cast<const float4*>(xr) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dr) {
    uint2 u[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = base + lane + 32 * j;
      u[j] = i < n4 ? __ldcg(reinterpret_cast<const uint2*>(dr) + i) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u[j].x), b = *reinterpret_cast<const __nv_bfloat162*>(&u[j].y);
      v[j].x += __low2float(a); v[j].y += __high2float(a); v[j].z += __low2float(b); v[j].w += __high2float(b);
    }
  }
}

__device__ __forceinline__ void norm_store_tile(const float4 (&v)[NV], int base, int n4, int lane, float inv, const void* weight, bool w_f32,
                                                float* xo_row, int own_lo, int own_hi, bf16* arow) {
  float4 wv[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = base + lane + 32 * j;
    if (i >= n4) { wv[j] = make_float4(0.f, 0.f, 0.f, 0.f); continue; }
    if (w_f32) {
      wv[j] = __ldg(reinterpret_cast<const float4*>(weight) + i);
    } else {
      const uint2 u = __ldg(reinterpret_cast<const uint2*>(weight) + i);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
      wv[j] = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = base + lane + 32 * j;
    if (i >= n4) continue;
    if (i >= own_lo && i < own_hi) reinterpret_cast<float4*>(xo_row)[i] = v[j];
    uint2 o;
    o.x = pack_bf16(v[j].x * inv * wv[j].x, v[j].y * inv * wv[j].y);
    o.y = pack_bf16(v[j].z * inv * wv[j].z, v[j].w * inv * wv[j].w);
    *reinterpret_cast<uint2*>(arow + i * 4) = o;
  }
}

template <bool HALF>
__device__ __forceinline__ void norm_into_operand(const Params& p, const float* x_in, const bf16* delta, float* x_out, const void* weight,
                                                  bool w_f32, float eps, bf16* A_s, int ald) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n4 = p.hidden >> 2;
  const int own_lo = (int)((long long)blockIdx.x * n4 / gridDim.x), own_hi = (int)((long long)(blockIdx.x + 1) * n4 / gridDim.x);
  constexpr int ROWS = HALF ? 8 : 16;
  constexpr int TILE = 32 * NV;
  for (int m = warp; m < ROWS; m += NWARPS) {
    bf16* arow = A_s + (size_t)m * ald;
    if (m >= p.M) {
      for (int i = lane; i < n4; i += 32) *reinterpret_cast<uint2*>(arow + i * 4) = make_uint2(0u, 0u);
      continue;
    }
    const float* xr = x_in + (size_t)m * p.hidden;
    const bf16* dr = delta ? delta + (size_t)m * p.hidden : nullptr;
    float* xo = x_out + (size_t)m * p.hidden;
    float4 v[NV];
    float ss = 0.f;
    for (int base = 0; base < n4; base += TILE) {
      norm_load_tile(xr, dr, base, n4, lane, v);
#pragma unroll
      for (int j = 0; j < NV; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)p.hidden + eps);
    if (n4 <= TILE) {
      norm_store_tile(v, 0, n4, lane, inv, weight, w_f32, xo, own_lo, own_hi, arow);
    } else {
      for (int base = 0; base < n4; base += TILE) {
        norm_load_tile(xr, dr, base, n4, lane, v);
        norm_store_tile(v, base, n4, lane, inv, weight, w_f32, xo, own_lo, own_hi, arow);
      }
    }
  }
}

// A_s[m][0..kseg) = src[m][k0..k0+kseg) for m < M, zeros for the other rows. src was written by other blocks.
// A thread's loads go out eight at a time.
template <bool HALF>
__device__ __forceinline__ void load_operand(const Params& p, const bf16* src, int K, int k0, int kseg, bf16* A_s, int ald) {
  constexpr int ROWS = HALF ? 8 : 16;
  const int per_row = kseg >> 3;                      // 16-byte pieces per row
  const int total = ROWS * per_row;
  for (int base = 0; base < total; base += 8 * NTHR) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = base + threadIdx.x + j * NTHR;
      v[j] = make_uint4(0u, 0u, 0u, 0u);
      if (i < total) {
        const int m = i / per_row, c = i - m * per_row;
        if (m < p.M) v[j] = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)m * K + k0) + c);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = base + threadIdx.x + j * NTHR;
      if (i < total) {
        const int m = i / per_row, c = i - m * per_row;
        *reinterpret_cast<uint4*>(A_s + (size_t)m * ald + c * 8) = v[j];
      }
    }
  }
}

// The products of this block's units for one segment: every warp consumes its chunks from its ring (issuing the
// chunks NST - 1 ahead, whatever phase they belong to) and leaves each unit's 16 x 8 partial sums in red[unit].
template <bool HALF>
__device__ __forceinline__ void run_units(const Params& p, const Geo& g, int seg, const bf16* A_s, int ald, float* red, bf16* ring,
                                          Cursor<HALF>& prod, int& cons_slot, int warp, int lane) {
  const int gq = lane >> 2, tq = lane & 3;
  const int n_units = g.tiles * g.ks;
  const int chunks = g.slice / CK;
  for (int unit = warp; unit < n_units; unit += NWARPS) {
    const int s = unit % g.ks;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ck = 0; ck < chunks; ++ck) {
      // keep the ring full: the chunk NST - 1 ahead of this one goes into the slot consumed last
      prod.issue(ring + (size_t)((cons_slot + NST - 1) % NST) * STAGE_ELEMS, lane);
      prod.advance(p, warp);
      cp_async_commit();
      cp_async_wait<NST - 1>();
      __syncwarp();
      const bf16* stage = ring + (size_t)cons_slot * STAGE_ELEMS;
      const int ka = s * g.slice + ck * CK;             // k inside the segment
#pragma unroll
      for (int kk2 = 0; kk2 < CK / 32; ++kk2) {
        uint32_t b0, b1, b2, b3;
        {
          const int row = lane & 7, c16 = kk2 * 4 + (lane >> 3);
          ldmatrix_x4(b0, b1, b2, b3, stage + row * CK + ((c16 ^ row) & 15) * 8);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int k = ka + kk2 * 32 + h * 16;
          uint32_t a0, a1 = 0u, a2, a3 = 0u;
          if (HALF) {
            ldmatrix_x2(a0, a2, A_s + (size_t)(lane & 7) * ald + k + ((lane >> 3) & 1) * 8);
          } else {
            ldmatrix_x4(a0, a1, a2, a3, A_s + (size_t)(lane & 15) * ald + k + (lane >> 4) * 8);
          }
          if (h == 0) mma_bf16(c, a0, a1, a2, a3, b0, b1); else mma_bf16(c, a0, a1, a2, a3, b2, b3);
        }
      }
      __syncwarp();                                     // all lanes have read the slot before a later copy lands in it
      cons_slot = (cons_slot + 1) % NST;
    }
    float* r = red + (size_t)unit * 128;
    if (seg == 0) {
      r[gq * 8 + tq * 2] = c[0]; r[gq * 8 + tq * 2 + 1] = c[1];
      if (!HALF) { r[(gq + 8) * 8 + tq * 2] = c[2]; r[(gq + 8) * 8 + tq * 2 + 1] = c[3]; }
    } else {
      r[gq * 8 + tq * 2] += c[0]; r[gq * 8 + tq * 2 + 1] += c[1];
      if (!HALF) { r[(gq + 8) * 8 + tq * 2] += c[2]; r[(gq + 8) * 8 + tq * 2 + 1] += c[3]; }
    }
  }
}

// sum of a tile's slices for element (m, nn), in slice order
__device__ __forceinline__ float tile_sum(const float* red, int tile, int ks, int m, int nn) {
  float s = 0.f;
  for (int i = 0; i < ks; ++i) s += red[(size_t)(tile * ks + i) * 128 + m * 8 + nn];
  return s;
}

// ---- attention over the cache for this block's (request, kv head, split) items -----------------------------------
constexpr int BT_CACHE = 256;

struct AttArgs {
  const bf16* kc; const bf16* vc;
  const int* block_table; int bt_width;
  int num_pages, window;
  float scale_log2;
};

__device__ __forceinline__ void att_load_subtile(const Params& p, const AttArgs& a, const int* bt, int bt_first, int hk, int k0, int lo, int hi,
                                                 bool same_page, bf16* Ks, bf16* Vs, int lane) {
  constexpr int CHUNKS = D / 8;
  constexpr int COPIES = (AKW * CHUNKS + 31) / 32;
  if (same_page) {
    const int blk = p.ps_shift >= 0 ? (k0 >> p.ps_shift) : k0 / p.ps;
    const int page = blk < a.bt_width ? bt[blk - bt_first] : -1;
    const bool page_ok = page >= 0 && page < a.num_pages;
    const size_t base = (((size_t)(page_ok ? page : 0) * p.Hkv + hk) * p.ps + (k0 - blk * p.ps)) * D;
#pragma unroll
    for (int i = 0; i < COPIES; ++i) {
      const int c = lane + 32 * i;
      if (c < AKW * CHUNKS) {
        const int row = c / CHUNKS, ch = c - row * CHUNKS;
        const bool ok = page_ok && k0 + row >= lo && k0 + row < hi;
        cp_async16(Ks + row * ALDS + ch * 8, a.kc + base + (size_t)c * 8, ok);
        cp_async16(Vs + row * ALDS + ch * 8, a.vc + base + (size_t)c * 8, ok);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < COPIES; ++i) {
    const int c = lane + 32 * i;
    if (c < AKW * CHUNKS) {
      const int row = c / CHUNKS, ch = c - row * CHUNKS;
      const int key = k0 + row;
      bool ok = key >= lo && key < hi;
      size_t off = 0;
      if (ok) {
        const int blk = key / p.ps;
        const int page = blk < a.bt_width ? bt[blk - bt_first] : -1;
        ok = page >= 0 && page < a.num_pages;
        if (ok) off = (((size_t)page * p.Hkv + hk) * p.ps + (key - blk * p.ps)) * D + ch * 8;
      }
      cp_async16(Ks + row * ALDS + ch * 8, a.kc + off, ok);
      cp_async16(Vs + row * ALDS + ch * 8, a.vc + off, ok);
    }
  }
}

// Partial results of all key splits of (request r, kv head hk) -> the output rows (reads bypass L1).
__device__ __forceinline__ void att_merge_splits(const Params& p, int r, int hk, int G, float* work) {
  float (*f_s)[16] = reinterpret_cast<float (*)[16]>(work);
  float* inv_s = work + MAX_SPLITS * 16;
  float* l_s = inv_s + 16;
  const int S = p.num_splits;
  const size_t base = ((size_t)r * p.Hkv + hk) * S;
  for (int idx = threadIdx.x; idx < S * 16; idx += NTHR) {
    const int s_ = idx >> 4, row = idx & 15;
    float2 ml = make_float2(-INFINITY, 0.f);
    if (row < G) ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((base + s_) * 16 + row) * 2));
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
  for (int idx = threadIdx.x; idx < G * D; idx += NTHR) {
    const int row = idx / D, d = idx - row * D;
    float acc = 0.f;
    for (int s_ = 0; s_ < S; ++s_) {
      const float f = f_s[s_][row];
      if (f != 0.f) acc = fmaf(__ldcg(p.part_o + ((base + s_) * 16 + row) * D + d), f, acc);
    }
    p.attn[(size_t)r * p.H * D + (size_t)(hk * G + row) * D + d] = __float2bfloat16_rn(acc * inv_s[row]);
  }
  __syncthreads();
}

template <bool UPPER>
__device__ __forceinline__ void att_item(const Params& p, const AttArgs& a, int r, int hk, int split, unsigned char* space, int* bt_s) {
  constexpr int CHUNKS = D / 8;
  constexpr int ANT = AKW / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int G = p.H / p.Hkv;                                   // rows of the tile: one token, G query heads
  bf16* Qs = reinterpret_cast<bf16*>(space);
  bf16* KVs = Qs + 16 * ALDS;
  const int L = p.kv_len[r];
  const int pos = L - 1;
  int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  int hi = L;
  {
    constexpr int UNIT = ATT_WARPS * AKW;
    const int base = (lo / UNIT) * UNIT;
    const int split_size = max(UNIT, ((hi - base + p.num_splits - 1) / p.num_splits + UNIT - 1) / UNIT * UNIT);
    lo = max(lo, base + split * split_size);
    hi = min(hi, base + (split + 1) * split_size);
  }
  const bool last = p.num_splits == 1;
  const size_t pbase = (((size_t)r * p.Hkv + hk) * p.num_splits + split) * 16;
  if (lo >= hi) {
    if (!last) {
      if (tid < 16) { p.part_ml[(pbase + tid) * 2] = -INFINITY; p.part_ml[(pbase + tid) * 2 + 1] = 0.f; }
    } else {
      for (int idx = tid; idx < G * D; idx += NTHR)
        p.attn[(size_t)r * p.H * D + (size_t)(hk * G + idx / D) * D + (idx % D)] = __float2bfloat16_rn(0.f);
    }
  } else {
    const int* bt = a.block_table + (size_t)r * a.bt_width;
    int bt_first = 0;
    {
      const int b_lo = lo / p.ps, b_hi = min((hi - 1) / p.ps, a.bt_width - 1);
      if (b_hi - b_lo + 1 <= BT_CACHE) {
        for (int i = tid; i <= b_hi - b_lo; i += NTHR) bt_s[i] = bt[b_lo + i];
        bt = bt_s;
        bt_first = b_lo;
      }
    }
    // queries of this step were written by other blocks in the phase before
    for (int idx = tid; idx < 16 * CHUNKS; idx += NTHR) {
      const int row = idx / CHUNKS, ch = idx - row * CHUNKS;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < G) v = __ldcg(reinterpret_cast<const uint4*>(p.qkv + (size_t)r * ((p.H + 2 * p.Hkv) * D) + (size_t)(hk * G + row) * D) + ch);
      *reinterpret_cast<uint4*>(Qs + row * ALDS + ch * 8) = v;
    }
    __syncthreads();
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    if (warp < ATT_WARPS) {
      const bool same_page = (p.ps % AKW) == 0;
      const int k_first = (lo / AKW) * AKW;
      const int n_sub = (hi - k_first + AKW - 1) / AKW;
      const int my_n = (n_sub - warp + ATT_WARPS - 1) / ATT_WARPS;
      bf16* myKV = KVs + (size_t)warp * ASTAGES * 2 * AKW * ALDS;
#pragma unroll
      for (int s = 0; s < ASTAGES - 1; ++s) {
        if (s < my_n) att_load_subtile(p, a, bt, bt_first, hk, k_first + (warp + ATT_WARPS * s) * AKW, lo, hi, same_page,
                                       myKV + s * 2 * AKW * ALDS, myKV + s * 2 * AKW * ALDS + AKW * ALDS, lane);
        cp_async_commit();
      }
      for (int it = 0; it < my_n; ++it) {
        {
          const int nx = it + ASTAGES - 1;
          if (nx < my_n) {
            bf16* Kn = myKV + (nx % ASTAGES) * 2 * AKW * ALDS;
            att_load_subtile(p, a, bt, bt_first, hk, k_first + (warp + ATT_WARPS * nx) * AKW, lo, hi, same_page, Kn, Kn + AKW * ALDS, lane);
          }
          cp_async_commit();
          cp_async_wait<ASTAGES - 1>();
        }
        __syncwarp();
        const bf16* Ks = myKV + (it % ASTAGES) * 2 * AKW * ALDS;
        const bf16* Vs = Ks + AKW * ALDS;
        const int kbase = k_first + (warp + ATT_WARPS * it) * AKW;
        float s[ANT][4];
#pragma unroll
        for (int j = 0; j < ANT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4(a0, a1, a2, a3, Qs + (lane & 15) * ALDS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int j = 0; j < ANT; j += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane >> 4) * 8 + (lane & 7)) * ALDS + kk * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
            mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
          }
        }
        // one token per request: every row sees every key of [lo, hi); only the edges of the range need a mask
        const bool unmasked = kbase >= lo && kbase + AKW <= hi;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < ANT; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = kbase + j * 8 + tq * 2 + e;
            const bool ok = unmasked || (key >= lo && key < hi);
            s[j][e] = ok ? s[j][e] * a.scale_log2 : -INFINITY;
            mx_a = fmaxf(mx_a, s[j][e]);
            if (UPPER) {
              s[j][2 + e] = ok ? s[j][2 + e] * a.scale_log2 : -INFINITY;
              mx_b = fmaxf(mx_b, s[j][2 + e]);
            }
          }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        const float mn_a = fmaxf(m_a, mx_a);
        const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a;
        const float al_a = ex2(m_a - use_a);
        m_a = mn_a;
        float use_b = 0.f, al_b = 1.f;
        if (UPPER) {
          mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
          mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
          const float mn_b = fmaxf(m_b, mx_b);
          use_b = (mn_b == -INFINITY) ? 0.f : mn_b;
          al_b = ex2(m_b - use_b);
          m_b = mn_b;
        }
        uint32_t pa[ANT][2];
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int j = 0; j < ANT; ++j) {
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
        if (__any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
          for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= al_a; o[i][1] *= al_a;
            if (UPPER) { o[i][2] *= al_b; o[i][3] *= al_b; }
          }
        }
#pragma unroll
        for (int ks = 0; ks < AKW / 16; ++ks) {
#pragma unroll
          for (int i = 0; i < D / 8; i += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ALDS + i * 8 + (lane >> 4) * 8);
            mma_bf16(o[i], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b0, b1);
            mma_bf16(o[i + 1], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1], b2, b3);
          }
        }
        __syncwarp();
      }
      cp_async_wait<0>();
      l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
      l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
      l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
      l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    }
    __syncthreads();                                            // every warp is done with its stages: reuse the space
    float* Om = reinterpret_cast<float*>(space);                // [ATT_WARPS][16][D]
    float* MLm = Om + ATT_WARPS * 16 * D;                       // [ATT_WARPS][16][2]
    if (warp < ATT_WARPS) {
      const bool row_a = g < G, row_b = UPPER && g + 8 < G;
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
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += NTHR) {
      const int row = idx / D, d = idx - row * D;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, MLm[(w * 16 + row) * 2]);
      float ll = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) {
        const float mw = MLm[(w * 16 + row) * 2];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
        ll += MLm[(w * 16 + row) * 2 + 1] * f;
        acc += Om[((size_t)w * 16 + row) * D + d] * f;
      }
      if (last) {
        p.attn[(size_t)r * p.H * D + (size_t)(hk * G + row) * D + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
      } else {
        p.part_o[(pbase + row) * D + d] = acc;
        if (d == 0) { p.part_ml[(pbase + row) * 2] = mm; p.part_ml[(pbase + row) * 2 + 1] = ll; }
      }
    }
  }
  if (!last) {
    // the block that arrives last for (r, hk) merges the splits; nobody waits for anybody
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int t = atomicAdd(p.tickets + (size_t)r * p.Hkv + hk, 1);
      s_last = (t == p.num_splits - 1);
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      att_merge_splits(p, r, hk, G, reinterpret_cast<float*>(space));
      if (tid == 0) p.tickets[(size_t)r * p.Hkv + hk] = 0;
    }
  }
  __syncthreads();                                              // the space is free for the next item
}

// ---- the kernel ---------------------------------------------------------------------------------------------------
template <bool HALF>
__global__ void __launch_bounds__(NTHR, 1) decode_stack_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int bt_s[BT_CACHE];
  bf16* A_s = reinterpret_cast<bf16*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw + A_BYTES);
  bf16* ring_all = reinterpret_cast<bf16*>(smem_raw + A_BYTES + RED_BYTES);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  bf16* ring = ring_all + (size_t)warp * NST * STAGE_ELEMS;
  const int ald = (HALF ? ACAP_HALF : ACAP_FULL) + APAD;
  const int n_qkv = (p.H + 2 * p.Hkv) * D;
  const int G = p.H / p.Hkv;

  Grid grid;
  grid.counter = p.barrier; grid.arrived = 0; grid.errors = p.errors; grid.aborted = false;

  // the ring starts NST - 1 chunks ahead, before anything else happens
  Cursor<HALF> prod;
  prod.start(p, warp);
  int cons_slot = 0;
#pragma unroll
  for (int s = 0; s < NST - 1; ++s) {
    prod.issue(ring + (size_t)s * STAGE_ELEMS, lane);
    prod.advance(p, warp);
    cp_async_commit();
  }

  for (int l = 0; l < p.n_layers; ++l) {
    const SbStackLayer L = p.layers[l];
    const int* block_table = p.block_tables[L.group];
    const int bt_width = p.bt_width[L.group];

    // ---- phase 1: norm, q/k/v product, rotation, cache write ----
    {
      const Geo g = make_geo<HALF>(p, L, PH_QKV);
      if (l == 0) prefetch_phase<HALF>(p, 0, PH_QKV, 0);
      prefetch_phase<HALF>(p, l, PH_O, 0);
      norm_into_operand<HALF>(p, p.xa, l == 0 ? p.first_delta : p.delta_down, p.xb, L.norm1, (L.norm_f32 & 1) != 0, L.eps1, A_s, ald);
      __syncthreads();
      run_units<HALF>(p, g, 0, A_s, ald, red, ring, prod, cons_slot, warp, lane);
      __syncthreads();
      for (int idx = tid; idx < g.tiles * 8 * p.M; idx += NTHR) {
        const int t = idx / (8 * p.M), rem = idx - t * 8 * p.M;
        const int m = rem >> 3, nn = rem & 7;
        if (8 * t + nn >= g.n_rows) continue;
        const int n = g.row_lo + 8 * t + nn;
        const int head = n / D, i = n - head * D;
        float v = round_bf16(tile_sum(red, t, g.ks, m, nn));     // as the separate kernels store q/k/v before rotating
        const int pos = p.positions[m];
        if (head < p.H + p.Hkv && i < L.rot) {
          const float sp = round_bf16(tile_sum(red, t, g.ks, m, nn ^ 1));
          float sn, cs;
          sincosf((float)pos * L.inv_freq[i >> 1], &sn, &cs);
          v = (i & 1) ? (v * cs + sp * sn) : (v * cs - sp * sn);
        }
        if (head < p.H) {
          p.qkv[(size_t)m * n_qkv + n] = __float2bfloat16_rn(v);
        } else if (L.write_cache) {
          const int blk = pos / p.ps;
          const int page = (blk < bt_width && pos >= 0) ? block_table[(size_t)m * bt_width + blk] : -1;
          if (page >= 0 && page < L.num_pages) {
            const bool is_k = head < p.H + p.Hkv;
            const int kvh = is_k ? head - p.H : head - p.H - p.Hkv;
            bf16* dst = (is_k ? (bf16*)L.kc : (bf16*)L.vc) + (((size_t)page * p.Hkv + kvh) * p.ps + (pos - blk * p.ps)) * D + i;
            *dst = __float2bfloat16_rn(v);
          } else if (n == p.H * D) {
            atomicAdd(p.errors, 1);
          }
        }
      }
    }
    stamp(p, l, 0);
    grid_barrier(grid);
    stamp(p, l, 1);

    // ---- phase 2: attention ----
    {
      prefetch_phase<HALF>(p, l, PH_GU, 1);
      AttArgs a;
      a.kc = (const bf16*)L.kc; a.vc = (const bf16*)L.vc; a.block_table = block_table; a.bt_width = bt_width;
      a.num_pages = L.num_pages; a.window = L.window; a.scale_log2 = L.scale_log2;
      const int items = p.M * p.Hkv * p.num_splits;
      for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int r = it / (p.Hkv * p.num_splits), rem = it - r * p.Hkv * p.num_splits;
        const int hk = rem / p.num_splits, split = rem - hk * p.num_splits;
        if (G > 8) att_item<true>(p, a, r, hk, split, smem_raw, bt_s);
        else att_item<false>(p, a, r, hk, split, smem_raw, bt_s);
      }
    }
    stamp(p, l, 2);
    grid_barrier(grid);
    stamp(p, l, 3);

    // ---- phase 3: output projection ----
    {
      const Geo g = make_geo<HALF>(p, L, PH_O);
      prefetch_phase<HALF>(p, l, PH_GU, 2);
      for (int seg = 0; seg < g.nseg; ++seg) {
        if (seg) __syncthreads();
        load_operand<HALF>(p, p.attn, g.K, seg * g.kseg, g.kseg, A_s, ald);
        __syncthreads();
        run_units<HALF>(p, g, seg, A_s, ald, red, ring, prod, cons_slot, warp, lane);
      }
      __syncthreads();
      for (int idx = tid; idx < g.tiles * 8 * p.M; idx += NTHR) {
        const int t = idx / (8 * p.M), rem = idx - t * 8 * p.M;
        const int m = rem >> 3, nn = rem & 7;
        if (8 * t + nn >= g.n_rows) continue;
        p.delta_o[(size_t)m * p.hidden + g.row_lo + 8 * t + nn] = __float2bfloat16_rn(tile_sum(red, t, g.ks, m, nn));
      }
    }
    stamp(p, l, 4);
    grid_barrier(grid);
    stamp(p, l, 5);

    // ---- phase 4: norm, gate/up product, SwiGLU ----
    {
      const Geo g = make_geo<HALF>(p, L, PH_GU);
      prefetch_phase<HALF>(p, l, PH_DOWN, 0);
      norm_into_operand<HALF>(p, p.xb, p.delta_o, p.xa, L.norm2, (L.norm_f32 & 2) != 0, L.eps2, A_s, ald);
      __syncthreads();
      run_units<HALF>(p, g, 0, A_s, ald, red, ring, prod, cons_slot, warp, lane);
      __syncthreads();
      for (int idx = tid; idx < g.gate_tiles * 8 * p.M; idx += NTHR) {
        const int t = idx / (8 * p.M), rem = idx - t * 8 * p.M;
        const int m = rem >> 3, nn = rem & 7;
        if (8 * t + nn >= g.n_rows) continue;
        // both halves are rounded to the activation type first, as if the [M, 2 inter] intermediate had been stored
        const float gte = round_bf16(tile_sum(red, t, g.ks, m, nn));
        const float up = round_bf16(tile_sum(red, g.gate_tiles + t, g.ks, m, nn));
        p.act[(size_t)m * p.inter + g.row_lo + 8 * t + nn] = __float2bfloat16_rn(gte / (1.0f + expf(-gte)) * up);
      }
    }
    stamp(p, l, 6);
    grid_barrier(grid);
    stamp(p, l, 7);

    // ---- phase 5: down projection ----
    {
      const Geo g = make_geo<HALF>(p, L, PH_DOWN);
      prefetch_phase<HALF>(p, l + 1, PH_QKV, 0);
      for (int seg = 0; seg < g.nseg; ++seg) {
        if (seg) __syncthreads();
        load_operand<HALF>(p, p.act, g.K, seg * g.kseg, g.kseg, A_s, ald);
        __syncthreads();
        run_units<HALF>(p, g, seg, A_s, ald, red, ring, prod, cons_slot, warp, lane);
      }
      __syncthreads();
      for (int idx = tid; idx < g.tiles * 8 * p.M; idx += NTHR) {
        const int t = idx / (8 * p.M), rem = idx - t * 8 * p.M;
        const int m = rem >> 3, nn = rem & 7;
        if (8 * t + nn >= g.n_rows) continue;
        p.delta_down[(size_t)m * p.hidden + g.row_lo + 8 * t + nn] = __float2bfloat16_rn(tile_sum(red, t, g.ks, m, nn));
      }
    }
    stamp(p, l, 8);
    if (l + 1 < p.n_layers) grid_barrier(grid);
    stamp(p, l, 9);
  }
  cp_async_wait<0>();
  // The block that leaves last puts the barrier's counters back to zero for the next launch. (Every block that is here
  // has passed the last barrier, so all blocks have left its wait once the leaving count is complete.)
  if (tid == 0 && !grid.aborted) {
    const unsigned t = atomicAdd(p.barrier + 1, 1u);
    if (t == gridDim.x - 1) {
      p.barrier[0] = 0u;
      p.barrier[1] = 0u;
      __threadfence();
    }
  }
}

int supports(int M, int hidden, int H, int Hkv, int inter, int n_ctas) {
  if (M < 1 || M > 16 || n_ctas < 1) return 0;
  if (H <= 0 || Hkv <= 0 || H % Hkv || H / Hkv > 16) return 0;
  const int acap = M <= 8 ? ACAP_HALF : ACAP_FULL;
  if (hidden % CK || hidden > acap) return 0;                   // the norm phases keep a whole row resident
  if ((H * D) % CK || inter % CK) return 0;
  if ((H * D) > acap && (H * D) % acap) return 0;
  if (inter > acap && inter % acap) return 0;
  // tiles of a block in any phase (gate and up tiles both) must fit the reduction space even without slicing
  const int widest = 2 * (((inter / 2 + n_ctas - 1) / n_ctas * 2 + 2 + 7) / 8);
  const int qkv_tiles = ((((H + 2 * Hkv) * D / 2 + n_ctas - 1) / n_ctas) * 2 + 2 + 7) / 8;
  if (widest > MAX_UNITS || qkv_tiles > MAX_UNITS) return 0;
  return 1;
}

}  // namespace

SB_EXPORT int sb_decode_stack_head_dim(void) { return D; }
SB_EXPORT int sb_decode_stack_layer_bytes(void) { return (int)sizeof(SbStackLayer); }

// Thread blocks of the kernel that are resident at once on the current device (one per SM), or 0.
SB_EXPORT int sb_decode_stack_blocks(void) {
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (cudaFuncSetAttribute(decode_stack_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess) return 0;
  if (cudaFuncSetAttribute(decode_stack_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess) return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel<false>, NTHR, SMEM_BYTES) != cudaSuccess) return 0;
  return per_sm >= 1 ? sms : 0;
}

SB_EXPORT int sb_decode_stack_supports(int M, int hidden, int H, int Hkv, int inter, int n_ctas) {
  return supports(M, hidden, H, Hkv, inter, n_ctas);
}

// Floats of scratch for the partial results of split keys: [M, Hkv, splits, 16, D + 2].
SB_EXPORT long long sb_decode_stack_partial_floats(int M, int Hkv, int num_splits) {
  return num_splits > 1 ? (long long)M * Hkv * num_splits * 16 * (D + 2) : 0;
}

// Runs layers[0..n_layers) on the M tokens of a decoding step. x [M, hidden] float is the residual stream (updated in
// place, without the last layer's feed-forward delta, which is left in delta_down as the pending delta); first_delta
// (may be null) is a pending delta to add first. block_tables / bt_widths: one per cache group the layers name.
// barrier: two zeroed uint32 (left zero); tickets: M * Hkv zeroed ints (left zero). n_ctas: sb_decode_stack_blocks().
// timing: null, or n_layers * 10 int64 that receive block 0's clock after each phase and each barrier (for profiles).
SB_EXPORT int sb_decode_stack(const void* layers, int n_layers, int M, int hidden, int H, int Hkv, int inter, const int* positions,
                              const int* kv_len, const int* const* block_tables, const int* bt_widths, int n_groups, int ps, float* x,
                              float* x_scratch, const void* first_delta, void* delta_o, void* delta_down, void* qkv, void* attn,
                              void* act, float* partials, int* tickets, int num_splits, unsigned* barrier, int* errors, int n_ctas,
                              long long* timing, cudaStream_t stream) {
  if (n_layers <= 0) return 0;
  if (!supports(M, hidden, H, Hkv, inter, n_ctas)) return SB_ERR_SHAPE;
  if (n_groups < 1 || n_groups > SB_STACK_MAX_GROUPS || ps <= 0) return SB_ERR_SHAPE;
  if (num_splits < 1 || num_splits > MAX_SPLITS || (num_splits > 1 && (!partials || !tickets))) return SB_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(x_scratch) || !aligned16(delta_o) || !aligned16(delta_down) || !aligned16(qkv) || !aligned16(attn) ||
      !aligned16(act) || (first_delta && !aligned16(first_delta)))
    return SB_ERR_ALIGN;
  Params p;
  p.layers = (const SbStackLayer*)layers; p.n_layers = n_layers; p.M = M;
  p.hidden = hidden; p.H = H; p.Hkv = Hkv; p.inter = inter;
  p.positions = positions; p.kv_len = kv_len;
  for (int i = 0; i < SB_STACK_MAX_GROUPS; ++i) {
    p.block_tables[i] = i < n_groups ? block_tables[i] : nullptr;
    p.bt_width[i] = i < n_groups ? bt_widths[i] : 0;
  }
  p.ps = ps; p.ps_shift = (ps & (ps - 1)) == 0 ? __builtin_ctz((unsigned)ps) : -1;
  p.xa = x; p.xb = x_scratch; p.first_delta = (const bf16*)first_delta; p.delta_o = (bf16*)delta_o; p.delta_down = (bf16*)delta_down;
  p.qkv = (bf16*)qkv; p.attn = (bf16*)attn; p.act = (bf16*)act;
  p.part_o = partials;
  p.part_ml = partials ? partials + (size_t)M * Hkv * num_splits * 16 * D : nullptr;
  p.tickets = tickets; p.num_splits = num_splits; p.barrier = barrier; p.errors = errors; p.timing = timing;
  void* args[] = {(void*)&p};
  cudaError_t e;
  if (M <= 8) {
    e = cudaFuncSetAttribute(decode_stack_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaLaunchCooperativeKernel((const void*)decode_stack_kernel<true>, dim3(n_ctas), dim3(NTHR), args, SMEM_BYTES, stream);
  } else {
    e = cudaFuncSetAttribute(decode_stack_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaLaunchCooperativeKernel((const void*)decode_stack_kernel<false>, dim3(n_ctas), dim3(NTHR), args, SMEM_BYTES, stream);
  }
  if (e != cudaSuccess) return (int)e;
  return 0;
}
