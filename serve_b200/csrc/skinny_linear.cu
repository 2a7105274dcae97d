// Matrix products for a handful of rows (decoding): out[M,N] = a[M,K] * w[N,K]^T with M <= 16, bfloat16 in,
// float accumulation, bfloat16 or float out. The work is reading w once at memory speed; the reference
// leaves this to cuBLAS (nn.Linear, serve/model.py:95-97,80-82,159), whose kernels for such shapes do not
// fill the memory system at N = 2048.
//
// On the tensor cores (mma.sync m16n8k16) the activation rows are the 16-row operand and 8 rows of w the
// 8-column operand. A block of 8 warps owns 8 output columns and splits K eight ways; partial sums meet in
// shared memory and are added in a fixed order, so a row's result does not depend on how many other rows the
// step has. Each thread fetches 16 contiguous bytes of a w row per 32 k-values straight into registers; both
// operands use the same permutation of k inside such a group of 32, which a dot product does not notice.
//
// With gate_up set, w is [2*N, K] (gate rows, then up rows) and the block also owns rows N + n of it:
// out[m, n] = silu(gate) * up  (serve/model.py:85), saving a pass over the [M, 2N] intermediate.
#include "common.cuh"

using namespace sb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What the q/k/v product of an attention layer does with its columns instead of storing them all (ROPE):
// columns are [q heads | k heads | v heads] x head_dim; q and k are rotated in adjacent pairs (2j, 2j+1) by
// position * inv_freq[j] (serve/model.py:234-244), q goes to ``out``, rotated k and plain v go straight into
// the request's cache page (serve/model.py:120-124), as the separate rotary kernel does.
struct RopeArgs {
  const int* positions;
  const int* token_row;
  const float* inv_freq;
  int rot, H, Hkv, D;
  bf16* kc;
  bf16* vc;
  const int* block_table;
  int bt_width, ps, num_pages, write_cache;
  int* errors;
  int late_trigger;    // let the kernel after this one start only when this kernel's products are done (see launch_mt)
};

// MT: tiles of 16 activation rows (M <= 16*MT); HALF: only rows 0..7 of the single tile exist (M <= 8).
// NT: tiles of 8 output columns per block (2 for very wide outputs: fewer, fatter blocks).
// GU: fused gate/up with SwiGLU epilogue. OutT: bf16 or float.
template <int MT, bool HALF, int NT, bool GU, bool ROPE, typename OutT>
__global__ void __launch_bounds__(THREADS, 2) skinny_linear_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w,
                                                                OutT* __restrict__ out, int M, int N, int K, const RopeArgs ra) {
  constexpr int NW = GU ? 2 : 1;
  constexpr int NB = NW * NT;                        // 8-column tiles of w rows a lane streams
  constexpr int BN = 8 * NT;                         // output columns per block
  // groups of 32 k-values whose loads are issued together: 8 where the registers allow it (one or, with at most 8 rows,
  // two tiles of w: at hidden 2048 a warp's whole share of q/k/v or of the output projection is then asked for before the wait)
  // (four tiles of w and up to 16 rows, the wide gate/up product: 2, or the registers spill; 0.965 -> 0.932 ms a decoding
  // step at batch 16)
  constexpr int UNROLL = (MT * NB > 2 && !HALF) ? 2 : ((MT * NB > 2 || (MT * NB > 1 && !HALF)) ? 4 : 8);
  __shared__ float red[WARPS][NB][MT][16 * 8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int n0 = blockIdx.x * BN;
  // this warp's share of K, in groups of 32
  const int groups = K / 32;
  const int per = (groups + WARPS - 1) / WARPS;
  const int g_lo = warp * per, g_hi = min(groups, g_lo + per);

  const bf16* wp[NB];   // tile u*NT + v: half u (gate/up), column tile v
#pragma unroll
  for (int v = 0; v < NT; ++v) {
    const int rn = min(n0 + v * 8 + g, N - 1);   // clamped: columns beyond N are computed and dropped
    wp[v] = w + (size_t)rn * K + tq * 8;
    if (GU) wp[NT + v] = w + (size_t)(N + rn) * K + tq * 8;
  }
  const bf16* xg[MT];
  const bf16* xh[MT];
  bool okg[MT], okh[MT];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    okg[t] = t * 16 + g < M;
    okh[t] = !HALF && (t * 16 + g + 8 < M);
    xg[t] = a + (size_t)(okg[t] ? t * 16 + g : 0) * K + tq * 8;
    xh[t] = a + (size_t)(okh[t] ? t * 16 + g + 8 : 0) * K + tq * 8;
  }

  float c[NB][MT][4];
#pragma unroll
  for (int u = 0; u < NB; ++u)
#pragma unroll
    for (int t = 0; t < MT; ++t) c[u][t][0] = c[u][t][1] = c[u][t][2] = c[u][t][3] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 vw[UNROLL][NB];
  // the weights do not depend on the kernel before this one: their first loads go out before the wait
  if (g_lo < g_hi) {
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      const size_t off = (size_t)(g_lo + j < g_hi ? g_lo + j : g_lo) * 32;
#pragma unroll
      for (int u = 0; u < NB; ++u) vw[j][u] = ld_stream(wp[u] + off);
    }
  }
  if (!ra.late_trigger) pdl_launch_dependents();
  pdl_wait();
  for (int gi = g_lo; gi < g_hi; gi += UNROLL) {
    uint4 vg[UNROLL][MT], vh[UNROLL][MT];
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      const bool in = gi + j < g_hi;
      const size_t off = (size_t)(in ? gi + j : g_lo) * 32;
      if (gi != g_lo) {
#pragma unroll
        for (int u = 0; u < NB; ++u) vw[j][u] = ld_stream(wp[u] + off);
      }
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        vg[j][t] = ld_cached(xg[t] + off);       // always a valid address; masked below
        if (!HALF) vh[j][t] = ld_cached(xh[t] + off);
      }
    }
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      const bool in = gi + j < g_hi;
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (!(in && okg[t])) vg[j][t] = zero;
        if (HALF || !(in && okh[t])) vh[j][t] = zero;
      }
    }
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
#pragma unroll
      for (int u = 0; u < NB; ++u) {
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          mma_bf16(c[u][t], vg[j][t].x, vh[j][t].x, vg[j][t].y, vh[j][t].y, vw[j][u].x, vw[j][u].y);
          mma_bf16(c[u][t], vg[j][t].z, vh[j][t].z, vg[j][t].w, vh[j][t].w, vw[j][u].z, vw[j][u].w);
        }
      }
    }
  }
  if (ra.late_trigger) pdl_launch_dependents();
  // partial sums of the 8 warps -> shared memory; element (m_local, n_local) of a tile at m_local*8 + n_local
#pragma unroll
  for (int u = 0; u < NB; ++u)
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      float* r = red[warp][u][t];
      r[g * 8 + tq * 2] = c[u][t][0];
      r[g * 8 + tq * 2 + 1] = c[u][t][1];
      if (!HALF) {
        r[(g + 8) * 8 + tq * 2] = c[u][t][2];
        r[(g + 8) * 8 + tq * 2 + 1] = c[u][t][3];
      }
    }
  __syncthreads();
  for (int idx = tid; idx < MT * 16 * BN; idx += THREADS) {
    const int m = idx / BN, nl = idx - m * BN;
    const int n = n0 + nl;
    if (m >= M || n >= N) continue;
    const int t = m >> 4, ml = m & 15;
    const int vt = nl >> 3, nn = nl & 7;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int wv = 0; wv < WARPS; ++wv) {
      s0 += red[wv][vt][t][ml * 8 + nn];
      if (GU) s1 += red[wv][NB - NT + vt][t][ml * 8 + nn];
    }
    float v = s0;
    if (GU) {
      // both halves are rounded to the activation type first, as if the [M, 2N] intermediate had been stored
      const float gte = to_float(__float2bfloat16_rn(s0)), up = to_float(__float2bfloat16_rn(s1));
      v = gte / (1.0f + expf(-gte)) * up;
    }
    if (ROPE) {
      const int head = n / ra.D, i = n - head * ra.D;
      v = to_float(__float2bfloat16_rn(v));            // as the unfused path stores q/k/v before rotating
      const int pos = ra.positions[m];
      if (head < ra.H + ra.Hkv && i < ra.rot) {
        // the partner of the pair sits in the neighbouring column of the same tile
        float sp = 0.f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) sp += red[wv][vt][t][ml * 8 + (nn ^ 1)];
        sp = to_float(__float2bfloat16_rn(sp));
        float sn, cs;
        sincosf((float)pos * ra.inv_freq[i >> 1], &sn, &cs);
        v = (i & 1) ? (v * cs + sp * sn) : (v * cs - sp * sn);
      }
      if (head < ra.H) {
        out[(size_t)m * N + n] = from_float<OutT>(v);
      } else if (ra.write_cache) {
        const int blk = pos / ra.ps;
        const int page = (blk < ra.bt_width && pos >= 0) ? ra.block_table[(size_t)ra.token_row[m] * ra.bt_width + blk] : -1;
        if (page >= 0 && page < ra.num_pages) {
          const bool is_k = head < ra.H + ra.Hkv;
          const int kvh = is_k ? head - ra.H : head - ra.H - ra.Hkv;
          bf16* dst = (is_k ? ra.kc : ra.vc) + (((size_t)page * ra.Hkv + kvh) * ra.ps + (pos - blk * ra.ps)) * ra.D + i;
          *dst = __float2bfloat16_rn(v);
        } else if (n == (ra.H * ra.D)) {
          atomicAdd(ra.errors, 1);
        }
      }
      continue;
    }
    out[(size_t)m * N + n] = from_float<OutT>(v);
  }
}

template <int MT, bool HALF, int NT, bool GU, bool ROPE, typename OutT>
int launch(const void* a, const void* w, void* out, int M, int N, int K, const RopeArgs& ra, cudaStream_t stream) {
  SB_PDL_CHECK(launch_pdl(skinny_linear_kernel<MT, HALF, NT, GU, ROPE, OutT>, dim3((N + 8 * NT - 1) / (8 * NT)), dim3(THREADS), 0,
                          stream, (const bf16*)a, (const bf16*)w, (OutT*)out, M, N, K, ra));
  return 0;
}

// Blocks of 8 columns (NT 1) or of 16 (NT 2)? Two blocks fit an SM. If 8-column blocks need more than one round of
// them, 16-column blocks do the same work in fewer, fatter blocks (each pays its fixed part once): measured on the 1B
// shapes, q/k/v (384 -> 192 blocks) and gate/up (1024 -> 512) gained 4 % of a decoding step each.
inline bool wide_blocks(int N) {
  int sms = sm_count();
  return (N + 7) / 8 > 2 * sms;
}

template <bool GU, typename OutT>
int launch_mt(const void* a, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
  RopeArgs none = {};
  // A plain product with bfloat16 output is followed by the add + norm kernel (a handful of blocks). If that kernel
  // is launched ahead, it should come in when this kernel's products are done, not when they start: it would release
  // its own successor at once, and blocks of kernels two and three launches ahead would take the places of running ones.
  static const bool late = getenv("SERVE_B200_EARLY_TRIGGER") == nullptr;
  none.late_trigger = (late && !GU && sizeof(OutT) == 2) ? 1 : 0;
  const bool wide = wide_blocks(N);
  if (M <= 8) {
    if (wide) return launch<1, true, 2, GU, false, OutT>(a, w, out, M, N, K, none, stream);
    return launch<1, true, 1, GU, false, OutT>(a, w, out, M, N, K, none, stream);
  }
  if (wide) return launch<1, false, 2, GU, false, OutT>(a, w, out, M, N, K, none, stream);
  return launch<1, false, 1, GU, false, OutT>(a, w, out, M, N, K, none, stream);
}

// The same product in true 32-bit arithmetic (plain fused multiply-adds, no tensor-core mode), for the float32 path's
// decoding steps: a warp owns NC output columns and MB activation rows, its lanes share K out among themselves in
// steps of four values, partial sums meet by a shuffle tree of fixed order. The weights are read once from memory at
// streaming speed (KU steps' loads per column go out together); the activation rows come from the L1 cache. NC is chosen
// so that there are blocks for every SM (narrow outputs: one column a warp). A row's result does not depend on the other rows.
constexpr int F32_MB = 8, F32_WARPS = 8;

__device__ __forceinline__ float4 ld_stream_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

template <int NC, int KU>
__global__ void __launch_bounds__(F32_WARPS * 32, 2) skinny_linear_f32_kernel(const float* __restrict__ a, const float* __restrict__ w,
                                                                               float* __restrict__ out, int M, int N, int K) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.x * F32_WARPS + warp) * NC;
  const int m0 = blockIdx.y * F32_MB;
  const float* wp[NC];
  const float* ap[F32_MB];
#pragma unroll
  for (int c = 0; c < NC; ++c) wp[c] = w + (size_t)min(n0 + c, N - 1) * K;      // clamped: computed and dropped
#pragma unroll
  for (int i = 0; i < F32_MB; ++i) ap[i] = a + (size_t)min(m0 + i, M - 1) * K;
  float acc[NC][F32_MB];
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int i = 0; i < F32_MB; ++i) acc[c][i] = 0.f;
  // the weights do not depend on the kernel before this one: their first loads go out before the wait
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 wv[KU][NC];
  const int k_first = lane * 4;
#pragma unroll
  for (int u = 0; u < KU; ++u)
#pragma unroll
    for (int c = 0; c < NC; ++c) wv[u][c] = (k_first + u * 128 < K && n0 < N) ? ld_stream_f4(wp[c] + k_first + u * 128) : zero4;
  pdl_launch_dependents();
  pdl_wait();
  if (n0 >= N) return;
  for (int k = k_first; k < K; k += 128 * KU) {
    float4 wn[KU][NC];
#pragma unroll
    for (int u = 0; u < KU; ++u)
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int kn = k + 128 * KU + u * 128;
        wn[u][c] = kn < K ? ld_stream_f4(wp[c] + kn) : zero4;
      }
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      const int ku = k + u * 128;
      if (ku < K) {
        float4 av[F32_MB];
#pragma unroll
        for (int i = 0; i < F32_MB; ++i) av[i] = __ldg(reinterpret_cast<const float4*>(ap[i] + ku));
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
          for (int i = 0; i < F32_MB; ++i) {
            acc[c][i] = fmaf(wv[u][c].x, av[i].x, acc[c][i]);
            acc[c][i] = fmaf(wv[u][c].y, av[i].y, acc[c][i]);
            acc[c][i] = fmaf(wv[u][c].z, av[i].z, acc[c][i]);
            acc[c][i] = fmaf(wv[u][c].w, av[i].w, acc[c][i]);
          }
      }
    }
#pragma unroll
    for (int u = 0; u < KU; ++u)
#pragma unroll
      for (int c = 0; c < NC; ++c) wv[u][c] = wn[u][c];
  }
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int i = 0; i < F32_MB; ++i) {
      const float s = warp_sum(acc[c][i]);
      if (lane == 0 && n0 + c < N && m0 + i < M) out[(size_t)(m0 + i) * N + n0 + c] = s;
    }
}

}  // namespace

// 1 if sb_skinny_linear_f32 takes these sizes, else 0 (the caller then uses the library product).
SB_EXPORT int sb_skinny_linear_f32_supports(int M, int N, int K) {
  if (M < 1 || M > 32 || N < 1 || K < 4 || (K % 4)) return 0;
  return 1;
}

// a [M,K] float, w [N,K] float, out [M,N] float; M <= 32, K a multiple of 4.
SB_EXPORT int sb_skinny_linear_f32(const void* a, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
  if (!sb_skinny_linear_f32_supports(M, N, K)) return SB_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(w)) return SB_ERR_ALIGN;
  const int mt = (M + F32_MB - 1) / F32_MB;
  const int want = 2 * sm_count();                     // two blocks fit an SM
  const float *af = (const float*)a, *wf = (const float*)w;
  float* of = (float*)out;
  // columns per warp: as many as still leave blocks for every SM
  if ((long long)((N + F32_WARPS * 4 - 1) / (F32_WARPS * 4)) * mt >= want) {
    SB_PDL_CHECK(launch_pdl(skinny_linear_f32_kernel<4, 1>, dim3((N + F32_WARPS * 4 - 1) / (F32_WARPS * 4), mt), dim3(F32_WARPS * 32), 0,
                            stream, af, wf, of, M, N, K));
  } else if ((long long)((N + F32_WARPS * 2 - 1) / (F32_WARPS * 2)) * mt >= want) {
    SB_PDL_CHECK(launch_pdl(skinny_linear_f32_kernel<2, 2>, dim3((N + F32_WARPS * 2 - 1) / (F32_WARPS * 2), mt), dim3(F32_WARPS * 32), 0,
                            stream, af, wf, of, M, N, K));
  } else {
    SB_PDL_CHECK(launch_pdl(skinny_linear_f32_kernel<1, 4>, dim3((N + F32_WARPS - 1) / F32_WARPS, mt), dim3(F32_WARPS * 32), 0, stream,
                            af, wf, of, M, N, K));
  }
  return 0;
}

// Up to 16 rows (one tile of the 16-row operand). A second tile of rows was measured on the Llama-3.2-1B shapes
// against the library, in a graph: 17..32 rows took 9.4 / 5.2 / 14.4 us (q/k/v, output, down projection) against
// 5.9 / 5.1 / 12.9 us, and 32 us against 15 for gate/up, because every block re-reads all activation rows; at 12..16
// rows this kernel wins (4.6 / 3.6 / 9.6 us against 5.5 / 4.9 / 12.8).
SB_EXPORT int sb_skinny_linear_supports(int M, int N, int K, int gate_up) {
  (void)gate_up;
  if (M < 1 || M > 16 || N < 1 || K < 32 || (K % 32)) return 0;
  return 1;
}

// a [M,K] bf16, w [N,K] bf16 (or [2N,K] with gate_up), out [M,N] bf16 (out_dtype 1) or float (0).
SB_EXPORT int sb_skinny_linear(const void* a, const void* w, void* out, int M, int N, int K, int out_dtype, int gate_up,
                               cudaStream_t stream) {
  if (!sb_skinny_linear_supports(M, N, K, gate_up)) return SB_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(w)) return SB_ERR_ALIGN;
  if (gate_up) {
    if (out_dtype != SB_DTYPE_BF16) return SB_ERR_DTYPE;
    return launch_mt<true, bf16>(a, w, out, M, N, K, stream);
  }
  if (out_dtype == SB_DTYPE_BF16) return launch_mt<false, bf16>(a, w, out, M, N, K, stream);
  if (out_dtype == SB_DTYPE_F32) return launch_mt<false, float>(a, w, out, M, N, K, stream);
  return SB_ERR_DTYPE;
}

// The q/k/v product of an attention layer with rotation and cache write in its epilogue (see RopeArgs):
// a [M,K], w [(H + 2 Hkv) * D, K]; out [M, (H + 2 Hkv) * D] receives the rotated queries (its k and v columns are
// left as they were); rotated keys and values go to kc, vc [num_pages, Hkv, ps, D]. Pairs are adjacent columns.
SB_EXPORT int sb_skinny_qkv_rope(const void* a, const void* w, void* out, int M, int K, const int* positions, const int* token_row,
                                 const float* inv_freq, int rot, int H, int Hkv, int D, void* kc, void* vc, const int* block_table,
                                 int bt_width, int ps, int num_pages, int write_cache, int* errors, cudaStream_t stream) {
  const int N = (H + 2 * Hkv) * D;
  if (!sb_skinny_linear_supports(M, N, K, 0)) return SB_ERR_SHAPE;
  if (H <= 0 || Hkv <= 0 || D <= 0 || (D % 8) || rot < 0 || rot > D || (rot & 1) || ps <= 0) return SB_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(w)) return SB_ERR_ALIGN;
  RopeArgs ra;
  ra.positions = positions; ra.token_row = token_row; ra.inv_freq = inv_freq; ra.rot = rot; ra.H = H; ra.Hkv = Hkv; ra.D = D;
  ra.kc = (bf16*)kc; ra.vc = (bf16*)vc; ra.block_table = block_table; ra.bt_width = bt_width; ra.ps = ps; ra.num_pages = num_pages;
  ra.write_cache = write_cache; ra.errors = errors; ra.late_trigger = 0;
  const bool wide = wide_blocks(N);
  if (M <= 8) {
    if (wide) return launch<1, true, 2, false, true, bf16>(a, w, out, M, N, K, ra, stream);
    return launch<1, true, 1, false, true, bf16>(a, w, out, M, N, K, ra, stream);
  }
  if (wide) return launch<1, false, 2, false, true, bf16>(a, w, out, M, N, K, ra, stream);
  return launch<1, false, 1, false, true, bf16>(a, w, out, M, N, K, ra, stream);
}
