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
// whole group. LPK lanes share a key (each holds EPL <= 16 elements of the head vector), so a warp works on
// KPW = 32 / LPK keys at a time and a score costs log2(LPK) shuffles; the 8 warps x KPW lane groups are 8 KPW
// independent streams over the keys (stream s takes keys lo + s, lo + s + 8 KPW, ...), each with its own running
// maximum, sum and output for up to DEC_ROWS rows at a time (more rows: more passes over the keys). The streams meet
// in shared memory and are merged in stream order. Same recurrences as above, base e, full-precision expf.
constexpr int DEC_WARPS = 8;
constexpr int DEC_ROWS = 4;
constexpr int LPK = D <= 16 ? 1 : (D <= 32 ? 2 : (D <= 64 ? 4 : (D <= 128 ? 8 : 16)));
constexpr int NCH = D / 4;                         // a head vector in chunks of four elements
constexpr int CPL = (NCH + LPK - 1) / LPK;         // chunks per lane: lane `sub` of a key's lanes takes chunks sub, sub + LPK, ...
constexpr int EPL = CPL * 4;                       // so neighbouring lanes read neighbouring 16 bytes of a key
constexpr int KPW = 32 / LPK;
constexpr int DEC_STREAMS = DEC_WARPS * KPW;
static_assert(D % 4 == 0 && EPL <= 16, "at most 16 elements of a head vector per lane");

__device__ __forceinline__ void load4(const float* p, float* x) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* x) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x), b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
  x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
}

// element e of lane `sub` is element dec_index(sub, e) of the head vector
__device__ __forceinline__ int dec_index(int sub, int e) { return ((e >> 2) * LPK + sub) * 4 + (e & 3); }

template <typename T>
__device__ __forceinline__ void dec_load(const T* __restrict__ base, size_t off, int sub, bool there, float (&x)[EPL]) {
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    if (there && c * LPK + sub < NCH) load4(base + off + (size_t)(c * LPK + sub) * 4, &x[c * 4]);
    else { x[c * 4] = 0.f; x[c * 4 + 1] = 0.f; x[c * 4 + 2] = 0.f; x[c * 4 + 3] = 0.f; }
  }
}

template <typename T>
__global__ void __launch_bounds__(DEC_WARPS * 32) attention_simt_decode_kernel(
    const T* __restrict__ qkv, int q_stride, const T* __restrict__ kc, const T* __restrict__ vc,
    const int* __restrict__ block_table, int bt_width, const int* __restrict__ cu_q, const int* __restrict__ kv_len, int H,
    int Hkv, int ps, int num_pages, float scale, int window, T* __restrict__ out) {
  extern __shared__ float smem[];
  float* Qs = smem;                                        // [16][D]
  float* Om = Qs + 16 * D;                                 // [DEC_STREAMS][DEC_ROWS][LPK * EPL]
  float* MLm = Om + DEC_STREAMS * DEC_ROWS * LPK * EPL;    // [DEC_STREAMS][DEC_ROWS][2]
  const int r = blockIdx.y, hk = blockIdx.x;
  const int q0 = cu_q[r], qn = cu_q[r + 1] - q0;
  const int G = H / Hkv;
  const int M = qn * G;
  if (M > 16 || M <= 0) return;                     // the tile kernel takes this request
  const int L = kv_len[r];
  const int p0 = L - qn;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gk = lane / LPK, sub = lane - gk * LPK;
  const int stream = warp * KPW + gk;
  for (int w = tid; w < M * D; w += DEC_WARPS * 32) {
    const int row = w / D, d = w - row * D;
    const int tok = row / G, hd = hk * G + (row - tok * G);
    Qs[w] = to_float(qkv[(size_t)(q0 + tok) * q_stride + (size_t)hd * D + d]) * scale;
  }
  __syncthreads();
  const int* bt = block_table + (size_t)r * bt_width;
  for (int m0 = 0; m0 < M; m0 += DEC_ROWS) {
    float q[DEC_ROWS][EPL], acc[DEC_ROWS][EPL], m_run[DEC_ROWS], l_run[DEC_ROWS];
    int pos[DEC_ROWS];
#pragma unroll
    for (int i = 0; i < DEC_ROWS; ++i) {
      const bool valid = m0 + i < M;
      pos[i] = valid ? p0 + (m0 + i) / G : -1;
      m_run[i] = -INFINITY;
      l_run[i] = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        q[i][e] = (valid && dec_index(sub, e) < D) ? Qs[(m0 + i) * D + dec_index(sub, e)] : 0.f;
        acc[i][e] = 0.f;
      }
    }
    const int last_row = min(m0 + DEC_ROWS, M) - 1;
    const int lo = window > 0 ? max(0, p0 + m0 / G - window + 1) : 0;
    const int hi = p0 + last_row / G + 1;             // exclusive; <= L
    // this stream's keys: lo + stream, then DEC_STREAMS further on; the next key's loads go out before this key's sums
    auto locate = [&](int key, size_t& off) -> bool {
      if (key >= hi) return false;
      const int blk = key / ps;
      const int page = blk < bt_width ? bt[blk] : -1;
      if (page < 0 || page >= num_pages) return false;          // (a missing page: nothing to read)
      off = (((size_t)page * Hkv + hk) * ps + (key - blk * ps)) * D;
      return true;
    };
    float kn[EPL], vn[EPL];
    size_t off = 0;
    int key = lo + stream;
    bool there = locate(key, off);
    dec_load(kc, off, sub, there, kn);
    dec_load(vc, off, sub, there, vn);
    for (int base = lo; base < hi; base += DEC_STREAMS) {
      float kv[EPL], vv[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) { kv[e] = kn[e]; vv[e] = vn[e]; }
      const int this_key = key;
      const bool this_there = there;
      key += DEC_STREAMS;
      there = locate(key, off);
      dec_load(kc, off, sub, there, kn);
      dec_load(vc, off, sub, there, vn);
#pragma unroll
      for (int i = 0; i < DEC_ROWS; ++i) {
        float sc = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) sc += q[i][e] * kv[e];
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        const bool ok = this_there && this_key <= pos[i] && (window <= 0 || this_key > pos[i] - window);
        if (ok) {
          const float m_new = fmaxf(m_run[i], sc);
          const float alpha = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
          const float pr = expf(sc - m_new);
          l_run[i] = l_run[i] * alpha + pr;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[i][e] = acc[i][e] * alpha + pr * vv[e];
          m_run[i] = m_new;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < DEC_ROWS; ++i) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) Om[((size_t)stream * DEC_ROWS + i) * (LPK * EPL) + dec_index(sub, e)] = acc[i][e];
      if (sub == 0) { MLm[(stream * DEC_ROWS + i) * 2] = m_run[i]; MLm[(stream * DEC_ROWS + i) * 2 + 1] = l_run[i]; }
    }
    __syncthreads();
    for (int w = tid; w < DEC_ROWS * D; w += DEC_WARPS * 32) {
      const int i = w / D, d = w - i * D;
      if (m0 + i >= M) continue;
      float mm = -INFINITY;
      for (int st = 0; st < DEC_STREAMS; ++st) mm = fmaxf(mm, MLm[(st * DEC_ROWS + i) * 2]);
      float ll = 0.f, o = 0.f;
      for (int st = 0; st < DEC_STREAMS; ++st) {
        const float mw = MLm[(st * DEC_ROWS + i) * 2];
        const float f = (mw == -INFINITY) ? 0.f : expf(mw - mm);
        ll += MLm[(st * DEC_ROWS + i) * 2 + 1] * f;
        o += Om[((size_t)st * DEC_ROWS + i) * (LPK * EPL) + d] * f;
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
  const size_t dsmem = (size_t)(16 * D + DEC_STREAMS * DEC_ROWS * LPK * EPL + DEC_STREAMS * DEC_ROWS * 2) * sizeof(float);
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
