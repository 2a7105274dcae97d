// Paged causal attention in plain float arithmetic (no tensor cores): the true
// 32-bit path, and the reference the faster kernels are checked against.
//
// One kernel serves prompt portions and decoded tokens alike. Row r of the
// step brings n = cu_q[r+1] - cu_q[r] query tokens at positions
// kv_len[r] - n .. kv_len[r] - 1; a query at position p attends the cached
// keys max(0, p - window + 1) .. p of its request (window 0: all of them).
// Scores, running maximum, sum and the output accumulator are float; the
// online-softmax recurrences are those of serve/kernels/attn_prefill.py:58-72,
// in base e. Compile with -DSB_HEAD_DIM=<multiple of 16>.
#include "common.cuh"

#ifndef SB_HEAD_DIM
#error "define SB_HEAD_DIM"
#endif

using namespace sb;

namespace {

constexpr int D = SB_HEAD_DIM;
constexpr int BM = 16;        // query rows per block
constexpr int BN = 32;        // keys per tile
constexpr int THREADS = 128;  // 16 rows x 8 threads
constexpr int KSTRIDE = D + 1;

static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head_dim must be a multiple of 16 in 16..256");

template <typename T>
__global__ void __launch_bounds__(THREADS) attention_simt_kernel(
    const T* __restrict__ qkv, int q_stride, const T* __restrict__ kc, const T* __restrict__ vc,  // caches [P, Hkv, ps, D]
    const int* __restrict__ block_table, int bt_width, const int* __restrict__ cu_q, const int* __restrict__ kv_len, int H,
    int Hkv, int ps, int num_pages, float scale, int window, T* __restrict__ out, int decode_apart) {
  extern __shared__ float smem[];
  float* Qs = smem;                 // [BM][D]
  float* Ks = Qs + BM * D;          // [BN][KSTRIDE]
  float* Vs = Ks + BN * KSTRIDE;    // [BN][D]
  float* Ps = Vs + BN * D;          // [BM][BN]

  const int r = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int q0 = cu_q[r], qn = cu_q[r + 1] - q0;
  const int m0 = tile * BM;
  if (m0 >= qn) return;
  if (decode_apart && H / Hkv <= 16 && qn * (H / Hkv) <= 16) return;     // the decoding shape below takes this request
  const int L = kv_len[r];
  const int p0 = L - qn;            // position of the row's first query
  const int hk = h / (H / Hkv);
  const int tid = threadIdx.x;
  const int i = tid >> 3, jj = tid & 7;

  for (int w = tid; w < BM * D; w += THREADS) {
    const int mi = w / D, d = w - mi * D;
    Qs[w] = (m0 + mi < qn) ? to_float(qkv[(size_t)(q0 + m0 + mi) * q_stride + (size_t)h * D + d]) : 0.f;
  }

  const int pi = p0 + m0 + i;                       // this thread's query position
  const bool row_ok = (m0 + i) < qn;
  const int first_pos = p0 + m0, last_pos = p0 + min(m0 + BM, qn) - 1;
  const int lo = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int hi = last_pos + 1;                      // exclusive; <= L

  float m_run = -INFINITY, l_run = 0.f;
  float acc[D / 8];
#pragma unroll
  for (int c = 0; c < D / 8; ++c) acc[c] = 0.f;

  const int* bt = block_table + (size_t)r * bt_width;
  for (int kt = (lo / BN) * BN; kt < hi; kt += BN) {
    __syncthreads();  // previous tile fully consumed (and Qs written, first time round)
    for (int w = tid; w < BN * D; w += THREADS) {
      const int kj = w / D, d = w - kj * D;
      const int key = kt + kj;
      float kvv = 0.f, vvv = 0.f;
      if (key >= lo && key < hi) {
        const int blk = key / ps;
        const int page = blk < bt_width ? bt[blk] : -1;
        if (page >= 0 && page < num_pages) {
          const size_t off = (((size_t)page * Hkv + hk) * ps + (key - blk * ps)) * D + d;
          kvv = to_float(kc[off]);
          vvv = to_float(vc[off]);
        }
      }
      Ks[kj * KSTRIDE + d] = kvv;
      Vs[kj * D + d] = vvv;
    }
    __syncthreads();

    float s[BN / 8];
#pragma unroll
    for (int c = 0; c < BN / 8; ++c) s[c] = 0.f;
    for (int d = 0; d < D; ++d) {
      const float qv = Qs[i * D + d];
#pragma unroll
      for (int c = 0; c < BN / 8; ++c) s[c] += qv * Ks[(jj + 8 * c) * KSTRIDE + d];
    }
    float tmax = -INFINITY;
#pragma unroll
    for (int c = 0; c < BN / 8; ++c) {
      const int key = kt + jj + 8 * c;
      const bool ok = row_ok && key <= pi && (window <= 0 || key > pi - window);
      s[c] = ok ? s[c] * scale : -INFINITY;
      tmax = fmaxf(tmax, s[c]);
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
    const float m_new = fmaxf(m_run, tmax);
    const float alpha = (m_new == -INFINITY) ? 1.f : expf(m_run - m_new);
    float psum = 0.f;
#pragma unroll
    for (int c = 0; c < BN / 8; ++c) {
      const float p = (s[c] == -INFINITY) ? 0.f : expf(s[c] - m_new);
      Ps[i * BN + jj + 8 * c] = p;
      psum += p;
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    psum += __shfl_xor_sync(0xffffffffu, psum, 4);
    l_run = l_run * alpha + psum;
    m_run = m_new;
    __syncwarp();  // the 8 threads of a row are in one warp; Ps row i is read only by them
#pragma unroll
    for (int c = 0; c < D / 8; ++c) acc[c] *= alpha;
    for (int kj = 0; kj < BN; ++kj) {
      const float p = Ps[i * BN + kj];
#pragma unroll
      for (int c = 0; c < D / 8; ++c) acc[c] += p * Vs[kj * D + jj + 8 * c];
    }
  }
  if (row_ok) {
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    T* orow = out + (size_t)(q0 + m0 + i) * H * D + (size_t)h * D;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) orow[jj + 8 * c] = from_float<T>(acc[c] * inv);
  }
}

// The decoding shape: requests that bring at most 16 / G tokens (G = H / Hkv query heads per kv head). One block per
// (request, kv head); the G heads of every token are rows of one tile, so a key or value is fetched once for the
// whole group. The 8 warps deal the keys out among themselves; a warp's
// lanes share the head's elements, a score is a shuffle-tree sum of fixed order, and every warp keeps its own
// running maximum, sum and output for up to DEC_ROWS rows at a time (more rows: more passes over the keys); a warp
// takes KU consecutive keys per step (warp w: keys lo + w KU .. lo + w KU + KU - 1, then 8 KU further on). The
// warps' results meet in shared memory and are merged in warp order. Same recurrences as above, base e, full-
// precision expf.
constexpr int DEC_WARPS = 8;
constexpr int DEC_ROWS = 4;
constexpr int DPL = (D + 31) / 32;   // elements of a head vector per lane
constexpr int KU = DPL <= 2 ? 8 : (DPL <= 4 ? 4 : 2);   // keys a warp asks for at a time

template <typename T>
__global__ void __launch_bounds__(DEC_WARPS * 32) attention_simt_decode_kernel(
    const T* __restrict__ qkv, int q_stride, const T* __restrict__ kc, const T* __restrict__ vc,
    const int* __restrict__ block_table, int bt_width, const int* __restrict__ cu_q, const int* __restrict__ kv_len, int H,
    int Hkv, int ps, int num_pages, float scale, int window, T* __restrict__ out) {
  extern __shared__ float smem[];
  float* Qs = smem;                                                                          // [16][D]
  float (*Om)[DEC_ROWS][D] = reinterpret_cast<float (*)[DEC_ROWS][D]>(Qs + 16 * D);          // [DEC_WARPS][DEC_ROWS][D]
  float (*MLm)[DEC_ROWS][2] = reinterpret_cast<float (*)[DEC_ROWS][2]>(Qs + 16 * D + DEC_WARPS * DEC_ROWS * D);
  const int r = blockIdx.y, hk = blockIdx.x;
  const int q0 = cu_q[r], qn = cu_q[r + 1] - q0;
  const int G = H / Hkv;
  const int M = qn * G;
  if (M > 16 || M <= 0) return;                     // the tile kernel takes this request
  const int L = kv_len[r];
  const int p0 = L - qn;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int w = tid; w < M * D; w += DEC_WARPS * 32) {
    const int row = w / D, d = w - row * D;
    const int tok = row / G, hd = hk * G + (row - tok * G);
    Qs[w] = to_float(qkv[(size_t)(q0 + tok) * q_stride + (size_t)hd * D + d]) * scale;
  }
  __syncthreads();
  const int* bt = block_table + (size_t)r * bt_width;
  for (int m0 = 0; m0 < M; m0 += DEC_ROWS) {
    float q[DEC_ROWS][DPL], acc[DEC_ROWS][DPL], m_run[DEC_ROWS], l_run[DEC_ROWS];
    int pos[DEC_ROWS];
#pragma unroll
    for (int i = 0; i < DEC_ROWS; ++i) {
      const bool valid = m0 + i < M;
      pos[i] = valid ? p0 + (m0 + i) / G : -1;
      m_run[i] = -INFINITY;
      l_run[i] = 0.f;
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int d = lane + 32 * e;
        q[i][e] = (valid && d < D) ? Qs[(m0 + i) * D + d] : 0.f;
        acc[i][e] = 0.f;
      }
    }
    const int last_row = min(m0 + DEC_ROWS, M) - 1;
    const int lo = window > 0 ? max(0, p0 + m0 / G - window + 1) : 0;
    const int hi = p0 + last_row / G + 1;             // exclusive; <= L
    // KU keys at a time, their table entries, keys and values asked for together: one trip to memory per KU keys
    for (int key0 = lo + warp * KU; key0 < hi; key0 += DEC_WARPS * KU) {
      size_t off[KU];
      bool there[KU];
#pragma unroll
      for (int j = 0; j < KU; ++j) {
        const int key = key0 + j;
        const int blk = key / ps;
        const int page = (key < hi && blk < bt_width) ? bt[blk] : -1;
        there[j] = page >= 0 && page < num_pages;           // (a missing page: nothing to read; warp-uniform)
        off[j] = there[j] ? (((size_t)page * Hkv + hk) * ps + (key - blk * ps)) * D : 0;
      }
      float kv[KU][DPL], vv[KU][DPL];
#pragma unroll
      for (int j = 0; j < KU; ++j)
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
          const int d = lane + 32 * e;
          kv[j][e] = (there[j] && d < D) ? to_float(kc[off[j] + d]) : 0.f;
          vv[j][e] = (there[j] && d < D) ? to_float(vc[off[j] + d]) : 0.f;
        }
#pragma unroll
      for (int j = 0; j < KU; ++j) {
        const int key = key0 + j;
        if (!there[j]) continue;
#pragma unroll
        for (int i = 0; i < DEC_ROWS; ++i) {
          float sc = 0.f;
#pragma unroll
          for (int e = 0; e < DPL; ++e) sc += q[i][e] * kv[j][e];
          sc = warp_sum(sc);
          const bool ok = key <= pos[i] && (window <= 0 || key > pos[i] - window);
          if (ok) {
            const float m_new = fmaxf(m_run[i], sc);
            const float alpha = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
            const float pr = expf(sc - m_new);
            l_run[i] = l_run[i] * alpha + pr;
#pragma unroll
            for (int e = 0; e < DPL; ++e) acc[i][e] = acc[i][e] * alpha + pr * vv[j][e];
            m_run[i] = m_new;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < DEC_ROWS; ++i) {
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int d = lane + 32 * e;
        if (d < D) Om[warp][i][d] = acc[i][e];
      }
      if (lane == 0) { MLm[warp][i][0] = m_run[i]; MLm[warp][i][1] = l_run[i]; }
    }
    __syncthreads();
    for (int w = tid; w < DEC_ROWS * D; w += DEC_WARPS * 32) {
      const int i = w / D, d = w - i * D;
      if (m0 + i >= M) continue;
      float mm = -INFINITY;
#pragma unroll
      for (int wv = 0; wv < DEC_WARPS; ++wv) mm = fmaxf(mm, MLm[wv][i][0]);
      float ll = 0.f, o = 0.f;
#pragma unroll
      for (int wv = 0; wv < DEC_WARPS; ++wv) {
        const float mw = MLm[wv][i][0];
        const float f = (mw == -INFINITY) ? 0.f : expf(mw - mm);
        ll += MLm[wv][i][1] * f;
        o += Om[wv][i][d] * f;
      }
      const int row = m0 + i, tok = row / G, hd = hk * G + (row - tok * G);
      out[(size_t)(q0 + tok) * H * D + (size_t)hd * D + d] = from_float<T>(ll > 0.f ? o / ll : 0.f);
    }
    __syncthreads();
  }
}

}  // namespace

SB_EXPORT int sb_attention_simt_head_dim() { return D; }

SB_EXPORT int sb_attention_simt(const void* qkv, int q_stride, const void* kc, const void* vc, const int* block_table, int bt_width,
                                const int* cu_q, const int* kv_len, int H, int Hkv, int ps, int num_pages, float scale, int window,
                                void* out, int n_rows, int max_q, int dtype, cudaStream_t stream) {
  if (n_rows <= 0 || max_q <= 0) return 0;
  if (H <= 0 || Hkv <= 0 || H % Hkv || ps <= 0 || bt_width <= 0) return SB_ERR_SHAPE;
  if (H > 65535 || n_rows > 65535) return SB_ERR_LIMIT;
  const size_t smem = (size_t)(BM * D + BN * KSTRIDE + BN * D + BM * BN) * sizeof(float);
  // Requests with at most 16 rows (tokens x query heads per kv head) go to the decoding shape, the others to the
  // tile kernel; each kernel's blocks leave the other's requests alone. A step of decoded tokens only launches no tiles.
  const int G = H / Hkv;
  const bool decode_shape = G <= 16 && Hkv <= 65535;
  const bool tiles_needed = !decode_shape || (long long)max_q * G > 16;
  dim3 grid((max_q + BM - 1) / BM, H, n_rows);
  dim3 dgrid(Hkv, n_rows);
  const size_t dsmem = (size_t)(16 * D + DEC_WARPS * DEC_ROWS * D + DEC_WARPS * DEC_ROWS * 2) * sizeof(float);
  if (dtype == SB_DTYPE_F32) {
    if (tiles_needed) {
      auto k = attention_simt_kernel<float>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      k<<<grid, THREADS, smem, stream>>>((const float*)qkv, q_stride, (const float*)kc, (const float*)vc, block_table, bt_width, cu_q,
                                         kv_len, H, Hkv, ps, num_pages, scale, window, (float*)out, decode_shape ? 1 : 0);
      SB_LAUNCH_CHECK();
    }
    if (decode_shape) {
      auto kd = attention_simt_decode_kernel<float>;
      if (dsmem > 48 * 1024) cudaFuncSetAttribute(kd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsmem);
    }
    if (decode_shape)
      attention_simt_decode_kernel<float><<<dgrid, DEC_WARPS * 32, dsmem, stream>>>(
          (const float*)qkv, q_stride, (const float*)kc, (const float*)vc, block_table, bt_width, cu_q, kv_len, H, Hkv, ps, num_pages,
          scale, window, (float*)out);
  } else if (dtype == SB_DTYPE_BF16) {
    if (tiles_needed) {
      auto k = attention_simt_kernel<__nv_bfloat16>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      k<<<grid, THREADS, smem, stream>>>((const __nv_bfloat16*)qkv, q_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                         block_table, bt_width, cu_q, kv_len, H, Hkv, ps, num_pages, scale, window,
                                         (__nv_bfloat16*)out, decode_shape ? 1 : 0);
      SB_LAUNCH_CHECK();
    }
    if (decode_shape) {
      auto kd = attention_simt_decode_kernel<__nv_bfloat16>;
      if (dsmem > 48 * 1024) cudaFuncSetAttribute(kd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsmem);
    }
    if (decode_shape)
      attention_simt_decode_kernel<__nv_bfloat16><<<dgrid, DEC_WARPS * 32, dsmem, stream>>>(
          (const __nv_bfloat16*)qkv, q_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, bt_width, cu_q, kv_len, H,
          Hkv, ps, num_pages, scale, window, (__nv_bfloat16*)out);
  } else {
    return SB_ERR_DTYPE;
  }
  SB_LAUNCH_CHECK();
  return 0;
}
