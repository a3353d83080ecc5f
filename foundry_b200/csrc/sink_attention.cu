// Grouped-query attention over the paged cache with a distance bias, a sliding
// window that keeps the first tokens, and a softmax with a sink; with a norm
// of the whole query and key projections in front of it.
//
//   q' = q / sqrt(mean(q^2) + eps) * wq     over ALL query rows of a token at once
//   k' = k / sqrt(mean(k^2) + eps) * wk     (before the split into heads)
//   s_ij = (q'_i . k'_j) * scale - slope_h * (i - j),  slope_h = 2^(-steep (h+1) / H)
//   j visible to i  iff  j <= i and (i - j < window or j < keep_first)
//   p_ij = exp(s_ij) / (sink + sum_j exp(s_ij)),  sink = 1 or 0: one more term exp(0)
//          in the sum, which adds nothing to the output
//   o_i = sum_j p_ij v_j
//
// Every constant is a parameter: window 0 = all earlier keys, steep 0 = no bias,
// sink 0 = the plain softmax. Keys have `dim` elements and values `vdim`; the
// two caches have strides of their own. Positions are the tokens' own, so the
// bias of a kept token is by the distance it really has.
//
// This file holds the CUDA-core forms (32-bit arithmetic, any sizes): one warp
// per (token, query head) walking the kept prefix and then the window.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// ------------------------------------------------ whole-projection norm + cache
template <typename T>
__global__ void qk_norm_cache_kernel(const float* qkv, long long ld, T* __restrict__ q_out,
                                     const float* __restrict__ wq, const float* __restrict__ wk,
                                     float eps, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int max_pages,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     long long k_page, long long k_head, long long v_page,
                                     long long v_head, int H, int G, int dim, int vdim,
                                     int write_cache) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int nq = H * dim, nk = G * dim, nv = G * vdim;
  const float* row = qkv + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) {
    const float v = __ldcg(row + i);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const float v = __ldcg(row + nq + i);
    sk += v * v;
  }
  sq = fb_block_sum(sq, scratch);
  sk = fb_block_sum(sk, scratch);
  const float rq = 1.0f / sqrtf(sq / (float)nq + eps);
  const float rk = 1.0f / sqrtf(sk / (float)nk + eps);
  T* qo = q_out + (size_t)t * nq;
  for (int i = threadIdx.x; i < nq; i += blockDim.x)
    qo[i] = fb_from_float<T>(__ldcg(row + i) * rq * wq[i]);
  if (!write_cache || seq < 0) return;
  const int pos = positions[t];
  const long long page = page_table[(size_t)seq * max_pages + pos / FB_PAGE];
  const int r = pos % FB_PAGE;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int g = i / dim, d = i - g * dim;
    k_cache[page * k_page + g * k_head + (long long)r * dim + d] =
        fb_from_float<T>(__ldcg(row + nq + i) * rk * wk[i]);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int g = i / vdim, d = i - g * vdim;
    v_cache[page * v_page + g * v_head + (long long)r * vdim + d] =
        fb_from_float<T>(__ldcg(row + nq + nk + i));
  }
}

// ---------------------------------------------------------------- attention
struct SinkMask {
  int window, keep_first, sink;
  float scale, steep;
};

// VEC (value size a multiple of 8, 16-byte aligned value rows): a value row is
// read as 16-byte pieces by `lpr` neighbouring lanes and 32 / lpr keys are worked at
// a time, every lane's loads of a chunk independent of one another; the lanes that
// share a piece add their sums up once, at the end. Otherwise a lane owns the
// elements lane, lane + 32, ... and keys go one by one.
template <typename T, bool VEC>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_kernel(const T* q, long long q_stride, T* __restrict__ out, long long out_stride,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ page_table, int max_pages, const T* k_cache,
                      const T* v_cache, long long k_page, long long k_head, long long v_page,
                      long long v_head, SinkMask mask, int H, int G, int D, int VD, int splits,
                      float* __restrict__ partial, int lpr, int kvec) {
  fb_pdl_wait();
  __shared__ float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int a = blockIdx.y * WARPS + warp;
  if (a >= H) return;
  const int seq = seq_of_token[t];
  T* o = out + (size_t)t * out_stride + (size_t)a * VD;
  if (seq < 0) {  // padding token: defined output, no cache access
    for (int d = lane; d < VD; d += 32) o[d] = fb_from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int g = a / (H / G);
  const T* qrow = q + (size_t)t * q_stride + (size_t)a * D;
  for (int d = lane; d < D; d += 32) qs[warp][d] = fb_load_coherent<T>(qrow + d);
  __syncwarp();
  const float slope = mask.steep > 0.f ? exp2f(-mask.steep * (float)(a + 1) / (float)H) : 0.f;
  const int lo = (mask.window > 0 && pos - mask.window + 1 > 0) ? pos - mask.window + 1 : 0;
  const int kept = min(mask.keep_first, lo);  // keys [0, kept) lie in front of the window
  const int* pages = page_table + (size_t)seq * max_pages;
  const T* kbase = k_cache + (long long)g * k_head;
  const T* vbase = v_cache + (long long)g * v_head;

  // With `splits` > 1 the visible keys (the kept ones, then the window's) are cut into
  // that many runs; block z takes run z and leaves (max, sum, weighted values) for
  // `attention_sink_merge_kernel`, which also adds the sink.
  const int total = kept + (pos + 1 - lo);
  const int i0 = (int)((long long)total * blockIdx.z / splits);
  const int i1 = (int)((long long)total * (blockIdx.z + 1) / splits);
  // the sink is the term exp(0) of the sum: the running maximum starts at 0, the sum at 1
  const bool own_sink = mask.sink && splits == 1;
  float m = own_sink ? 0.f : -INFINITY, l = own_sink ? 1.f : 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int range = 0; range < 2; ++range) {
    const int begin = range == 0 ? min(i0, kept) : lo + max(i0 - kept, 0);
    const int end = range == 0 ? min(i1, kept) : lo + max(i1 - kept, 0);  // exclusive
    for (int j0 = begin; j0 < end; j0 += 32) {
      const int j = j0 + lane;
      float s = -INFINITY;
      long long k_off = 0, v_off = 0;
      if (j < end) {
        const long long page = pages[j / FB_PAGE];
        const int r = j % FB_PAGE;
        k_off = page * k_page + (long long)r * D;
        v_off = page * v_page + (long long)r * VD;
        const T* krow = kbase + k_off;
        float dot = 0.f;
        if (kvec) {  // key rows of whole 16-byte pieces
          for (int d = 0; d < D; d += 8) {
            float kv[8];
            load8<T>(krow + d, kv);
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(qs[warp][d + e], kv[e], dot);
          }
        } else {
          for (int d = 0; d < D; ++d) dot = fmaf(qs[warp][d], fb_load_coherent<T>(krow + d), dot);
        }
        s = dot * mask.scale - slope * (float)(pos - j);
      }
      const float m_new = fmaxf(m, fb_warp_max(s));
      const float corr = expf(m - m_new);  // exp(-inf) = 0 on a first chunk without sink
      const float p = (j < end) ? expf(s - m_new) : 0.f;
      l = l * corr + fb_warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
      const int n = min(32, end - j0);
      if (VEC) {
        const int d0 = (lane % lpr) * 8, sub = lane / lpr, ks = 32 / lpr;
        for (int jj = 0; jj < n; jj += ks) {  // uniform trip count; lanes past n add nothing
          const int key = jj + sub;
          const float pj = __shfl_sync(0xffffffffu, p, key & 31);
          const long long off = __shfl_sync(0xffffffffu, v_off, key & 31);
          if (key < n && d0 < VD) {
            float vv[8];
            load8<T>(vbase + off + d0, vv);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(pj, vv[e], acc[e]);
          }
        }
      } else {
        for (int jj = 0; jj < n; ++jj) {
          const float pj = __shfl_sync(0xffffffffu, p, jj);
          const long long off = __shfl_sync(0xffffffffu, v_off, jj);
          const T* vrow = vbase + off;
#pragma unroll
          for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < VD) acc[i] = fmaf(pj, fb_load_coherent<T>(vrow + d), acc[i]);
          }
        }
      }
    }
  }
  if (VEC) {
    // the lanes that hold the same piece of the row (one per key worked at a time)
#pragma unroll
    for (int e = 0; e < 8; ++e)
      for (int off = lpr; off < 32; off <<= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
    const int d0 = lane * 8;  // after the sum every group of lpr lanes holds the whole row
    if (splits > 1) {
      float* dst = partial + (((size_t)t * H + a) * splits + blockIdx.z) * (VD + 2);
      if (lane == 0) { dst[0] = m; dst[1] = l; }
      if (lane < lpr && d0 < VD)
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[2 + d0 + e] = acc[e];
      return;
    }
    const float inv = 1.0f / l;
    if (lane < lpr && d0 < VD)
#pragma unroll
      for (int e = 0; e < 8; ++e) o[d0 + e] = fb_from_float<T>(acc[e] * inv);
    return;
  }
  if (splits > 1) {
    float* dst = partial + (((size_t)t * H + a) * splits + blockIdx.z) * (VD + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < VD) dst[2 + d] = acc[i];
    }
    return;
  }
  const float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < VD) o[d] = fb_from_float<T>(acc[i] * inv_l);
  }
}

// One warp per (token, head): the runs' partial results become the output.
template <typename T>
__global__ void attention_sink_merge_kernel(const float* partial, T* __restrict__ out,
                                            long long out_stride, const int* __restrict__ seq_of_token,
                                            int H, int VD, int splits, int sink) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, a = blockIdx.y * WARPS + warp;
  if (a >= H || seq_of_token[t] < 0) return;  // padding rows were written by the first kernel
  const float* src = partial + ((size_t)t * H + a) * splits * (VD + 2);
  float M = sink ? 0.f : -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, __ldcg(src + (size_t)s * (VD + 2)));
  float L = sink ? expf(-M) : 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* ps = src + (size_t)s * (VD + 2);
    const float ms = __ldcg(ps);
    if (ms == -INFINITY) continue;  // an empty run
    const float f = expf(ms - M);
    L = fmaf(__ldcg(ps + 1), f, L);
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < VD) acc[i] = fmaf(__ldcg(ps + 2 + d), f, acc[i]);
    }
  }
  const float inv = 1.0f / L;
  T* o = out + (size_t)t * out_stride + (size_t)a * VD;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < VD) o[d] = fb_from_float<T>(acc[i] * inv);
  }
}
}  // namespace

FB_API int fb_qk_norm_cache_write(const float* qkv, long long ld, void* q_out, int dtype,
                                  const float* wq, const float* wk, float eps,
                                  const int* positions, const int* seq_of_token,
                                  const int* page_table, int max_pages, void* k_cache,
                                  void* v_cache, long long k_page, long long k_head,
                                  long long v_page, long long v_head, int T, int H, int G, int dim,
                                  int vdim, int write_cache, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G > 0 && dim > 0 && vdim > 0, "qk_norm_cache_write: bad sizes");
  FB_REQUIRE(ld >= (long long)H * dim + (long long)G * (dim + vdim),
             "qk_norm_cache_write: rows of %lld hold no q, k and v", ld);
  FB_REQUIRE(!write_cache || (k_cache && v_cache && page_table && max_pages > 0),
             "qk_norm_cache_write: no cache to write");
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(qk_norm_cache_kernel<E>, dim3(T), dim3(256), 0, stream,
      qkv, ld, (E*)q_out, wq, wk, eps, positions, seq_of_token, page_table, max_pages,
      (E*)k_cache, (E*)v_cache, k_page, k_head, v_page, v_head, H, G, dim, vdim, write_cache)));
  return fb_check_launch("qk_norm_cache_write");
}

FB_API int fb_attention_sink(const void* q, long long q_stride, void* out, long long out_stride,
                             int dtype, const int* positions, const int* seq_of_token,
                             const int* page_table, int max_pages, const void* k_cache,
                             const void* v_cache, long long k_page, long long k_head,
                             long long v_page, long long v_head, int window, int keep_first,
                             int sink, float scale, float steep, int T, int H, int G, int D, int VD,
                             int splits, float* partial, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G > 0 && D > 0 && VD > 0, "attention_sink: bad sizes");
  FB_REQUIRE(H % G == 0, "attention_sink: %d query heads are not a multiple of %d key-value heads",
             H, G);
  FB_REQUIRE(D <= MAX_D && VD <= MAX_D, "attention_sink: key size %d and value size %d must be "
             "at most %d", D, VD, MAX_D);
  const int kvec = D % 8 == 0 && k_page % 8 == 0 && k_head % 8 == 0 && ((uintptr_t)k_cache % 32) == 0;
  FB_REQUIRE(window >= 0 && keep_first >= 0 && max_pages > 0, "attention_sink: bad mask");
  FB_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || partial != nullptr),
             "attention_sink: %d runs need a workspace", splits);
  if (T == 0) return 0;
  SinkMask mask{window, keep_first, sink ? 1 : 0, scale, steep};
  dim3 grid(T, (H + WARPS - 1) / WARPS, splits);
  const bool vec = VD % 8 == 0 && v_page % 8 == 0 && v_head % 8 == 0 && ((uintptr_t)v_cache % 32) == 0;
  int lpr = 1;
  while (lpr * 8 < VD) lpr *= 2;  // lanes that share a value row: a power of two, at most 32
  if (vec) {
    FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_kernel<E, true>, dim3(grid),
        dim3(WARPS * 32), 0, stream, (const E*)q, q_stride, (E*)out, out_stride, positions,
        seq_of_token, page_table, max_pages, (const E*)k_cache, (const E*)v_cache, k_page, k_head,
        v_page, v_head, mask, H, G, D, VD, splits, partial, lpr, kvec)));
  } else {
    FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_kernel<E, false>, dim3(grid),
        dim3(WARPS * 32), 0, stream, (const E*)q, q_stride, (E*)out, out_stride, positions,
        seq_of_token, page_table, max_pages, (const E*)k_cache, (const E*)v_cache, k_page, k_head,
        v_page, v_head, mask, H, G, D, VD, splits, partial, lpr, kvec)));
  }
  if (splits > 1) {
    int rc = fb_check_launch("attention_sink");
    if (rc) return rc;
    FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_merge_kernel<E>,
        dim3(T, (H + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream, (const float*)partial,
        (E*)out, out_stride, seq_of_token, H, VD, splits, sink ? 1 : 0)));
  }
  return fb_check_launch("attention_sink");
}
