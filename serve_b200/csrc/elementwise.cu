// Embedding gather, residual-add + RMSNorm, SwiGLU activation, rotary + cache
// write, and sampling. All arithmetic is float; T is the storage type of
// activations and weights.
//
// Formulas: serve/model.py:63-68 (RMSNorm), :85 (SwiGLU), :234-244 (rotation),
// :120-124 (cache write), serve/run.py:47-60 (sampling).
#include "common.cuh"

using namespace sb;

// ---------------------------------------------------------------- embedding
// A token id below zero, -(s+1), stands for "the token last sampled for state slot s": it is read from
// last_token[s], where the sampling kernel left it, so that a decode step can be launched before the host has
// seen the previous step's tokens.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ out,
                                 int dim, int vocab, const int* __restrict__ last_token, int n_slots) {
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  int tok = tokens[t];
  if (tok < 0 && last_token != nullptr && -tok - 1 < n_slots) tok = last_token[-tok - 1];
  const bool ok = tok >= 0 && tok < vocab;
  const T* src = table + (size_t)(ok ? tok : 0) * dim;
  float* dst = out + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = ok ? to_float(src[i]) : 0.f;
}

// A step's packed integer inputs, from pinned host memory to the device buffer the kernels read, copied by a kernel:
// a few KB through the device's view of the host buffer. (As a memcpy the copy costs the same microseconds but sits
// between two switches of engine, ~9 us of idle each, in a decoding step of under a millisecond.)
__global__ void fetch_ints_kernel(const int4* __restrict__ src, int4* __restrict__ dst, int n4) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// src: pinned host memory (device-accessible), dst: device; n: ints, a multiple of 4; both 16-byte aligned.
SB_EXPORT int sb_fetch_ints(const int* src, int* dst, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n % 4) || !aligned16(src) || !aligned16(dst)) return SB_ERR_ALIGN;
  const int n4 = n / 4;
  const int blocks = n4 <= 1024 ? 1 : (n4 + 1023) / 1024 > 64 ? 64 : (n4 + 1023) / 1024;
  fetch_ints_kernel<<<blocks, 256, 0, stream>>>((const int4*)src, (int4*)dst, n4);
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_embedding(const int* tokens, const void* table, float* out, int n_tokens, int dim, int vocab, int dtype,
                           const int* last_token, int n_slots, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || vocab <= 0) return SB_ERR_SHAPE;
  const int threads = dim >= 1024 ? 256 : 128;
  if (dtype == SB_DTYPE_F32)
    SB_PDL_CHECK(launch_pdl(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, out, dim, vocab,
                            last_token, n_slots));
  else if (dtype == SB_DTYPE_BF16)
    SB_PDL_CHECK(launch_pdl(embedding_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                            (const __nv_bfloat16*)table, out, dim, vocab, last_token, n_slots));
  else
    return SB_ERR_DTYPE;
  return 0;
}

// ---------------------------------------------------------- add + RMSNorm
// One block per row. x (float residual) += delta if given (and is written back
// when update_x); out = x * rsqrt(mean(x^2) + eps) * weight, rounded once.
// With rows != nullptr, row b of the output comes from x[rows[b]] and x is not
// written.
template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const int* __restrict__ rows,
                                   const W* __restrict__ weight, T* __restrict__ out, int dim, float eps) {
  __shared__ float red[32];
  extern __shared__ float rowbuf[];  // dim floats
  const int b = blockIdx.x;
  const int src_row = rows ? rows[b] : b;
  float* xr = x + (size_t)src_row * dim;
  const T* dr = delta ? delta + (size_t)src_row * dim : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    if (dr) v += to_float(dr[i]);
    rowbuf[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  T* orow = out + (size_t)b * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = rowbuf[i];
    if (!rows && dr) xr[i] = v;
    orow[i] = from_float<T>(v * inv * to_float(weight[i]));
  }
}

// The same for widths that are a multiple of 4 and fit 8 float4 per thread: the row stays in registers, the
// weight is fetched before the reduction, loads are 16 bytes (8 for bfloat16).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <typename T, typename W, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta, const int* __restrict__ rows,
                                       const W* __restrict__ weight, T* __restrict__ out, int dim, float eps) {
  __shared__ float red[32];
  const int b = blockIdx.x;
  const int src_row = rows ? rows[b] : b;
  float* xr = x + (size_t)src_row * dim;
  const T* dr = delta ? delta + (size_t)src_row * dim : nullptr;
  const int nvec = dim >> 2;
  float4 v[VPT], wv[VPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) wv[k] = Vec4<W>::load(weight + i * 4);    // not written by any kernel of the step
  }
  pdl_launch_dependents();
  pdl_wait();
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      v[k] = Vec4<float>::load(xr + i * 4);
      if (dr) {
        const float4 d = Vec4<T>::load(dr + i * 4);
        v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
      }
    }
  }
  // the sum of squares is taken in index order within a thread and in a fixed tree across threads
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  T* orow = out + (size_t)b * dim;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      if (!rows && dr) Vec4<float>::store(xr + i * 4, v[k]);
      Vec4<T>::store(orow + i * 4, make_float4(v[k].x * inv * wv[k].x, v[k].y * inv * wv[k].y, v[k].z * inv * wv[k].z,
                                               v[k].w * inv * wv[k].w));
    }
  }
}

template <typename T>
static int launch_add_rmsnorm(float* x, const void* delta, const int* rows, const void* weight, int weight_dtype, void* out,
                              int n_rows, int dim, float eps, cudaStream_t stream) {
  if ((dim % 4) == 0 && aligned16(x) && aligned16(out) && aligned16(weight) && (!delta || aligned16(delta))) {
    // vector path: threads so that each holds at most 2 (or 8) float4
    const int nvec = dim / 4;
    int threads = nvec <= 128 ? 128 : (nvec <= 256 ? 256 : 512);
    const int vpt = (nvec + threads - 1) / threads;
    if (vpt <= 8) {
    // The kernel is launched ahead of its predecessor's end (its blocks then wait inside). With the few rows of a
    // decoding step that once hurt: this kernel lets its own successor in at once, so blocks of products two and three
    // launches ahead sat on the SMs, waiting, in place of blocks of the product that was running (1.23 ms a step against
    // 0.89 ms with this kernel as a full stop). The products that come before a norm therefore let their successor in
    // only when their own work is done (skinny_linear.cu, late_trigger); with that, launching this kernel ahead gains
    // 1-1.5 % of a decoding step (0.802 -> 0.791 ms at batch 8). SERVE_B200_EARLY_TRIGGER=1 brings the full stop back.
    static const bool late = getenv("SERVE_B200_EARLY_TRIGGER") == nullptr;
    const bool ahead = n_rows > 32 || late;
#define SB_NORM_VEC(WT, VPT)                                                                                              \
  do {                                                                                                                    \
    if (ahead) {                                                                                                          \
      SB_PDL_CHECK(launch_pdl(add_rmsnorm_vec_kernel<T, WT, VPT>, dim3(n_rows), dim3(threads), 0, stream, x,              \
                              (const T*)delta, rows, (const WT*)weight, (T*)out, dim, eps));                              \
    } else {                                                                                                              \
      add_rmsnorm_vec_kernel<T, WT, VPT><<<n_rows, threads, 0, stream>>>(x, (const T*)delta, rows, (const WT*)weight,     \
                                                                         (T*)out, dim, eps);                              \
    }                                                                                                                     \
  } while (0)
      if (weight_dtype == SB_DTYPE_F32) {
        if (vpt <= 1) SB_NORM_VEC(float, 1); else if (vpt <= 2) SB_NORM_VEC(float, 2); else SB_NORM_VEC(float, 8);
      } else if (weight_dtype == SB_DTYPE_BF16) {
        if (vpt <= 1) SB_NORM_VEC(__nv_bfloat16, 1); else if (vpt <= 2) SB_NORM_VEC(__nv_bfloat16, 2); else SB_NORM_VEC(__nv_bfloat16, 8);
      } else {
        return SB_ERR_DTYPE;
      }
#undef SB_NORM_VEC
      return 0;
    }
  }
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  const size_t smem = (size_t)dim * sizeof(float);
  if (smem > 200 * 1024) return SB_ERR_LIMIT;
  if (weight_dtype == SB_DTYPE_F32) {
    auto k = add_rmsnorm_kernel<T, float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<n_rows, threads, smem, stream>>>(x, (const T*)delta, rows, (const float*)weight, (T*)out, dim, eps);
  } else if (weight_dtype == SB_DTYPE_BF16) {
    auto k = add_rmsnorm_kernel<T, __nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<n_rows, threads, smem, stream>>>(x, (const T*)delta, rows, (const __nv_bfloat16*)weight, (T*)out, dim, eps);
  } else {
    return SB_ERR_DTYPE;
  }
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_add_rmsnorm(float* x, const void* delta, const int* rows, const void* weight, int weight_dtype, void* out,
                             int n_rows, int dim, float eps, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0) return SB_ERR_SHAPE;
  if (dtype == SB_DTYPE_F32) return launch_add_rmsnorm<float>(x, delta, rows, weight, weight_dtype, out, n_rows, dim, eps, stream);
  if (dtype == SB_DTYPE_BF16)
    return launch_add_rmsnorm<__nv_bfloat16>(x, delta, rows, weight, weight_dtype, out, n_rows, dim, eps, stream);
  return SB_ERR_DTYPE;
}

// ---------------------------------------------------------------- SwiGLU
// gate_up: [T, 2*I] (gate columns first, then up); out[t,i] = silu(gate)*up.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gate_up[t * 2 * inter + i]);
    const float u = to_float(gate_up[t * 2 * inter + inter + i]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(s * u);
  }
}

// bfloat16, 8 elements (16 bytes of gate, 16 of up) per thread; needs inter % 8 == 0 and aligned pointers
__global__ void swiglu_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter8,
                                       size_t total8) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter8;
    const int i = (int)(idx - t * inter8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + (t * 2 * inter8 + i) * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + (t * 2 * inter8 + inter8 + i) * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = ov;
  }
}

SB_EXPORT int sb_swiglu(const void* gate_up, void* out, int n_tokens, int inter, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (inter <= 0) return SB_ERR_SHAPE;
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  if (dtype == SB_DTYPE_BF16 && (inter % 8) == 0 && aligned16(gate_up) && aligned16(out)) {
    const size_t total8 = total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    const int blocks = (int)(want < sm_count() * 16 ? want : sm_count() * 16);
    swiglu_bf16_vec_kernel<<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter / 8, total8);
    SB_LAUNCH_CHECK();
    return 0;
  }
  const int blocks = (int)((total + threads - 1) / threads < sm_count() * 16 ? (total + threads - 1) / threads : sm_count() * 16);
  if (dtype == SB_DTYPE_F32)
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
  else if (dtype == SB_DTYPE_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------ rotary + cache write
// qkv: [T, (H + 2*Hkv) * D]. Queries and keys are rotated (angle = position *
// inv_freq[j], float); queries in place, rotated keys and plain values go to
// the request's pages: cache[page, kv_head, pos % ps, :], page =
// block_table[row, pos / ps]. pairing 0: pairs (j, j + rot/2); 1: (2j, 2j+1).
// A page id < 0 or a block index beyond the table is counted in *errors and
// the write is skipped.
constexpr int ROPE_THREADS = 128;

// grid (tokens, y): blocks y < rot_blocks each rotate ROPE_THREADS (head, pair) items of q and k; the
// remaining blocks copy v (and the part of k beyond the rotary width) into the page.
template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS) rope_cache_write_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_row, const float* __restrict__ inv_freq,
    int pairing, int rot, int H, int Hkv, int D, T* __restrict__ kc, T* __restrict__ vc, const int* __restrict__ block_table,
    int bt_width, int ps, int num_pages, int write_cache, int rot_blocks, int* __restrict__ errors) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  T* row = qkv + (size_t)t * (H + 2 * Hkv) * D;
  size_t cache_base = 0;
  bool cache_ok = false;
  if (write_cache) {
    const int blk = pos / ps;
    const int r = token_row[t];
    const int page = (blk < bt_width && pos >= 0) ? block_table[(size_t)r * bt_width + blk] : -1;
    cache_ok = page >= 0 && page < num_pages;
    if (!cache_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicAdd(errors, 1);
    cache_base = (size_t)(cache_ok ? page : 0) * Hkv * ps * D + (size_t)(pos % ps) * D;   // + kv_head * ps * D
  }
  if ((int)blockIdx.y < rot_blocks) {
    const int w = blockIdx.y * ROPE_THREADS + threadIdx.x;
    if (w >= (H + Hkv) * half) return;
    const int h = w / half, j = w - h * half;
    const int i0 = pairing == 0 ? j : 2 * j;
    const int i1 = pairing == 0 ? j + half : 2 * j + 1;
    T* hv = row + (size_t)h * D;
    const float ang = (float)pos * inv_freq[j];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    pdl_launch_dependents();
    pdl_wait();                      // positions, tables and angles came before; q and k come from the kernel before
    const float a = to_float(hv[i0]), b = to_float(hv[i1]);
    const T o0 = from_float<T>(a * cs - b * sn);
    const T o1 = from_float<T>(b * cs + a * sn);
    if (h < H) {
      hv[i0] = o0;
      hv[i1] = o1;
    } else if (cache_ok) {
      T* dst = kc + cache_base + (size_t)(h - H) * ps * D;
      dst[i0] = o0;
      dst[i1] = o1;
    }
    return;
  }
  pdl_launch_dependents();
  pdl_wait();
  if (!cache_ok) return;
  // copy blocks: all value elements, then key elements beyond the rotary width
  const int tail = D - rot;
  const int n_v = Hkv * D, n_tail = Hkv * tail;
  const int stride = (gridDim.y - rot_blocks) * ROPE_THREADS;
  const T* vrow = row + (size_t)(H + Hkv) * D;
  for (int w = (blockIdx.y - rot_blocks) * ROPE_THREADS + threadIdx.x; w < n_v + n_tail; w += stride) {
    if (w < n_v) {
      const int h = w / D, i = w - h * D;
      vc[cache_base + (size_t)h * ps * D + i] = vrow[w];
    } else {
      const int u = w - n_v;
      const int h = u / tail, i = rot + (u - h * tail);
      kc[cache_base + (size_t)h * ps * D + i] = row[(size_t)(H + h) * D + i];
    }
  }
}

// bfloat16, adjacent pairs, 8 elements (16 bytes) per thread: one thread rotates four pairs of a q or k head, or
// copies 8 elements of a v head; q back in place, k and v into the page. For prompt portions, where the one-item-
// per-thread kernel above is far from memory speed. Needs D % 8 == 0, rot % 8 == 0 and 16-byte aligned rows.
__global__ void __launch_bounds__(256) rope_cache_write_vec_kernel(
    __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_row,
    const float* __restrict__ inv_freq, int rot, int H, int Hkv, int D, __nv_bfloat16* __restrict__ kc,
    __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int bt_width, int ps, int num_pages, int write_cache,
    int n_tokens, int* __restrict__ errors) {
  const int chunks_per_head = D >> 3;
  const int heads_all = H + 2 * Hkv;
  const int chunks_per_token = heads_all * chunks_per_head;
  const long long total = (long long)n_tokens * chunks_per_token;
  pdl_launch_dependents();
  pdl_wait();                          // q, k and v come from the product before this kernel
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / chunks_per_token);
    const int c = (int)(idx - (long long)t * chunks_per_token);
    const int head = c / chunks_per_head, ch = c - head * chunks_per_head;
    if (head >= H && !write_cache) continue;
    const int pos = positions[t];
    __nv_bfloat16* src = qkv + (size_t)t * heads_all * D + (size_t)head * D + ch * 8;
    uint4 v = *reinterpret_cast<const uint4*>(src);
    if (head < H + Hkv && ch * 8 < rot) {
      __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 ab = __bfloat1622float2(p2[k]);
        float sn, cs;
        sincosf((float)pos * inv_freq[ch * 4 + k], &sn, &cs);
        p2[k] = __floats2bfloat162_rn(ab.x * cs - ab.y * sn, ab.y * cs + ab.x * sn);
      }
    }
    if (head < H) {
      *reinterpret_cast<uint4*>(src) = v;
      continue;
    }
    const int blk = pos / ps;
    const int page = (blk < bt_width && pos >= 0) ? block_table[(size_t)token_row[t] * bt_width + blk] : -1;
    if (page < 0 || page >= num_pages) {
      if (c == H * chunks_per_head) atomicAdd(errors, 1);
      continue;
    }
    const bool is_k = head < H + Hkv;
    const int kvh = is_k ? head - H : head - H - Hkv;
    __nv_bfloat16* dst = (is_k ? kc : vc) + (((size_t)page * Hkv + kvh) * ps + (pos - blk * ps)) * D + ch * 8;
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

SB_EXPORT int sb_rope_cache_write(void* qkv, const int* positions, const int* token_row, const float* inv_freq, int pairing,
                                  int rot, int H, int Hkv, int D, void* kc, void* vc, const int* block_table, int bt_width,
                                  int ps, int num_pages, int write_cache, int* errors, int n_tokens, int dtype,
                                  cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || Hkv <= 0 || D <= 0 || rot < 0 || rot > D || (rot & 1) || ps <= 0) return SB_ERR_SHAPE;
  if (dtype == SB_DTYPE_BF16 && pairing == 1 && n_tokens >= 64 && (D % 8) == 0 && (rot % 8) == 0 && aligned16(qkv) &&
      (!write_cache || (aligned16(kc) && aligned16(vc)))) {
    const long long total = (long long)n_tokens * (H + 2 * Hkv) * (D / 8);
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < sm_count() * 16 ? want : sm_count() * 16);
    SB_PDL_CHECK(launch_pdl(rope_cache_write_vec_kernel, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)qkv, positions, token_row,
                            inv_freq, rot, H, Hkv, D, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, block_table, bt_width, ps, num_pages,
                            write_cache, n_tokens, errors));
    return 0;
  }
  const int rot_blocks = ((H + Hkv) * (rot / 2) + ROPE_THREADS - 1) / ROPE_THREADS;
  int copy_blocks = 0;
  if (write_cache) {
    copy_blocks = (Hkv * (2 * D - rot) + ROPE_THREADS * 4 - 1) / (ROPE_THREADS * 4);
    if (copy_blocks < 1) copy_blocks = 1;
    if (copy_blocks > 64) copy_blocks = 64;
  }
  if (rot_blocks + copy_blocks == 0) return 0;
  if (rot_blocks + copy_blocks > 65535) return SB_ERR_LIMIT;
  dim3 grid(n_tokens, rot_blocks + copy_blocks);
  if (dtype == SB_DTYPE_F32)
    SB_PDL_CHECK(launch_pdl(rope_cache_write_kernel<float>, grid, dim3(ROPE_THREADS), 0, stream, (float*)qkv, positions, token_row,
                            inv_freq, pairing, rot, H, Hkv, D, (float*)kc, (float*)vc, block_table, bt_width, ps, num_pages,
                            write_cache, rot_blocks, errors));
  else if (dtype == SB_DTYPE_BF16)
    SB_PDL_CHECK(launch_pdl(rope_cache_write_kernel<__nv_bfloat16>, grid, dim3(ROPE_THREADS), 0, stream, (__nv_bfloat16*)qkv,
                            positions, token_row, inv_freq, pairing, rot, H, Hkv, D, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc,
                            block_table, bt_width, ps, num_pages, write_cache, rot_blocks, errors));
  else
    return SB_ERR_DTYPE;
  return 0;
}

// (cos, sin) of position * inv_freq[j] for every rotary pair and every token of a step: float2 [half, n_tokens]
// (pair-major: the threads of a warp that hold consecutive rows of a product read consecutive entries).
// The angle is the float32 product that the rotary kernels form, so a value taken from here is the one they compute.
__global__ void __launch_bounds__(256) rope_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                                          int half, int n_tokens, float2* __restrict__ out) {
  const long long total = (long long)n_tokens * half;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(idx / n_tokens), t = (int)(idx - (long long)j * n_tokens);
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
    out[idx] = make_float2(cs, sn);
  }
}

SB_EXPORT int sb_rope_angles(const int* positions, const float* inv_freq, int rot, int n_tokens, float* out, cudaStream_t stream) {
  if (n_tokens <= 0 || rot <= 0) return 0;
  if ((rot & 1) || !positions || !inv_freq || !out || ((uintptr_t)out & 7)) return SB_ERR_SHAPE;
  const long long total = (long long)n_tokens * (rot / 2);
  const long long want = (total + 255) / 256;
  rope_angles_kernel<<<(int)(want < sm_count() * 8 ? want : sm_count() * 8), 256, 0, stream>>>(positions, inv_freq, rot / 2, n_tokens, (float2*)out);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- sampling
// One block per row of float logits [L, V]. temperature 0: the largest logit,
// lowest index on ties (serve/run.py:56-57). Otherwise the Gumbel-max form of
// run.py:48-60: argmax_i softmax(l/T)_i / q_i with q ~ Exp(1), which is
// argmax_i (l_i / T - log q_i). The uniform behind q_i comes from a counter
// hash of (seed, request id, index of the token in its request, i), so a draw
// does not depend on what else is in the batch.
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

__device__ __forceinline__ float counter_uniform(uint32_t seed_lo, uint32_t seed_hi, uint32_t req, uint32_t tok, uint32_t i) {
  uint32_t h = mix32(seed_lo ^ 0x9E3779B9U);
  h = mix32(h ^ seed_hi);
  h = mix32(h + req * 0x85EBCA6BU);
  h = mix32(h ^ (tok * 0xC2B2AE35U));
  h = mix32(h + i);
  return ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);  // in (0, 1)
}

// Order-preserving key of (score, index): a larger score gives a larger key, and among equal scores the lower
// index does. Key 0 is below every real key.
__device__ __forceinline__ unsigned long long sample_key(float s, int i) {
  uint32_t u = __float_as_uint(s);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
}

// grid (rows, chunks): every block scans its share of the vocabulary and folds its best (score, index) into the
// row's key with one atomicMax; the block that arrives last (a counter per row) turns the key into the token
// and leaves key and counter zero for the next call. Nobody waits for anybody.
__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                              const int* __restrict__ req_ids, const int* __restrict__ tok_index, uint32_t seed_lo,
                              uint32_t seed_hi, int vocab, int* __restrict__ out, unsigned long long* __restrict__ keys,
                              int* __restrict__ counters, const int* __restrict__ slots, int* __restrict__ last_token) {
  __shared__ unsigned long long skey[32];
  const int r = blockIdx.x;
  const float* lr = logits + (size_t)r * vocab;
  pdl_launch_dependents();
  pdl_wait();
  const float temp = temperature[r];
  const uint32_t req = (uint32_t)req_ids[r], tok = (uint32_t)tok_index[r];
  const int per = (vocab + gridDim.y - 1) / gridDim.y;
  const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
  unsigned long long best = 0ull;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float s = lr[i];
    if (temp > 0.f) {
      const float u = counter_uniform(seed_lo, seed_hi, req, tok, (uint32_t)i);
      const float q = -logf(u);             // Exp(1)
      s = s / temp - logf(q);
    }
    if (s == s) {                           // a NaN is never chosen
      const unsigned long long k = sample_key(s, i);
      best = k > best ? k : best;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) skey[warp] = best;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? skey[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    if (lane == 0) {
      if (best) atomicMax(keys + r, best);
      __threadfence();
      if (atomicAdd(counters + r, 1) == (int)gridDim.y - 1) {
        __threadfence();
        const unsigned long long k = atomicExch(keys + r, 0ull);
        const int chosen = k ? (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull)) : 0;
        out[r] = chosen;
        if (slots != nullptr && last_token != nullptr) last_token[slots[r]] = chosen;   // for the next step's embedding
        counters[r] = 0;
      }
    }
  }
}

// work: n_rows 64-bit keys followed by n_rows int counters (16-byte aligned), all zero before the first call;
// every call leaves them zero.
// slots / last_token (both or neither): the chosen token of row r is also left in last_token[slots[r]].
SB_EXPORT int sb_sample(const float* logits, const float* temperature, const int* req_ids, const int* tok_index,
                        unsigned long long seed, int n_rows, int vocab, int* out, void* work, const int* slots, int* last_token,
                        cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0 || !work) return SB_ERR_SHAPE;
  if (n_rows > 65535) return SB_ERR_LIMIT;
  const int threads = 256;
  // few rows: more, smaller chunks, so that the launch still fills the GPU (at least 4 values per thread)
  const int per_chunk = n_rows <= 16 ? 1024 : 4096;
  int chunks = (vocab + per_chunk - 1) / per_chunk;
  if (chunks > 128) chunks = 128;
  unsigned long long* keys = (unsigned long long*)work;
  int* counters = (int*)(keys + n_rows);
  SB_PDL_CHECK(launch_pdl(sample_kernel, dim3(n_rows, chunks), dim3(threads), 0, stream, logits, temperature, req_ids, tok_index,
                          (uint32_t)(seed & 0xffffffffULL), (uint32_t)(seed >> 32), vocab, out, keys, counters, slots, last_token));
  return 0;
}
