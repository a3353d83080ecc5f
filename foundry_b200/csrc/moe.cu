// A feed-forward of routed experts.
//
//   z = W_router h + b (32-bit);  the `top` experts of largest z are chosen
//   (the lower index among equals);  their weights are softmax over the chosen
//   z only;  y = sum_c weight_c * expert_c(h)
//   expert:  g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit)
//            a = g * sigmoid(alpha g) * (u + 1);  out = W_down a
//
// The experts' matrices are stacked: gate_up [E, 2 ff, W] (gate rows, then up
// rows) and down [E, W, ff]. `limit`, `alpha` and the counts are parameters.
//
// `fb_moe_route` makes the choice per token. `fb_moe_experts_rows` is the form
// for a handful of tokens: one block per token streams the weights of that
// token's experts (each chosen expert's matrices once, 16-byte loads along K),
// with the hidden activations in shared memory and 32-bit sums throughout.
#include "common.cuh"

namespace {

__global__ void moe_route_kernel(const float* z, long long ld, const float* __restrict__ bias,
                                 int E, int top, int* __restrict__ chosen,
                                 float* __restrict__ weights) {
  fb_pdl_launch();
  fb_pdl_wait();
  // one warp per token; each lane keeps the experts lane, lane + 32, ... (up to 8 of them)
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? __ldcg(z + (size_t)t * ld + e) + bias[e] : -INFINITY;
  }
  float first = 0.f, sum = 0.f, mine = 0.f;
  for (int c = 0; c < top; ++c) {  // top <= 32: lane c keeps the c-th chosen value
    float best = -INFINITY;
    int at = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v[i] > best) { best = v[i]; at = lane + 32 * i; }
    // the largest value, and among equals the lowest index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (c == 0) first = best;  // values are chosen in falling order: the first is the largest
    const float e = expf(best - first);
    sum += e;
    if (lane == c) mine = e;
    if (at >= E) at = 0;  // only when every value left is NaN: any expert, never a wild index
    if (lane == 0) chosen[(size_t)t * top + c] = at;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (at == lane + 32 * i) v[i] = -INFINITY;
  }
  if (lane < top) weights[(size_t)t * top + lane] = mine / sum;
}

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* x, int K, int lane);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ w, const float* x, int K,
                                                int lane) {
  float acc = 0.f;
  for (int k = lane; k < K; k += 32) acc = fmaf(w[k], x[k], acc);
  return fb_warp_sum(acc);
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w,
                                                        const float* x, int K, int lane) {
  float acc = 0.f;
  if (K % 8 == 0 && ((uintptr_t)w % 16) == 0) {
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + k);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc = fmaf(f.x, x[k + 2 * i], acc);
        acc = fmaf(f.y, x[k + 2 * i + 1], acc);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(w[k]), x[k], acc);
  }
  return fb_warp_sum(acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_experts_rows_kernel(const T* h, const T* __restrict__ gate_up, const T* __restrict__ down,
                        const int* chosen, const float* weights, float* __restrict__ out, int W,
                        int ff, int top, int E, float limit, float alpha) {
  fb_pdl_wait();
  extern __shared__ float smem[];  // x [W] | act [ff] | acc [W]
  float* x = smem;
  float* act = smem + W;
  float* acc = act + ff;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    x[i] = fb_load_coherent<T>(h + (size_t)t * W + i);
    acc[i] = 0.f;
  }
  __syncthreads();
  for (int c = 0; c < top; ++c) {
    const int e = __ldcg(chosen + (size_t)t * top + c);
    if (e < 0 || e >= E) continue;  // uniform over the block
    const float wt = __ldcg(weights + (size_t)t * top + c);
    const T* gu = gate_up + (size_t)e * 2 * ff * W;
    for (int f = warp; f < ff; f += nwarps) {
      float g = dot_row<T>(gu + (size_t)f * W, x, W, lane);
      float u = dot_row<T>(gu + (size_t)(ff + f) * W, x, W, lane);
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      if (lane == 0) act[f] = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
    }
    __syncthreads();
    const T* dn = down + (size_t)e * W * ff;
    for (int r = warp; r < W; r += nwarps) {
      const float y = dot_row<T>(dn + (size_t)r * ff, act, ff, lane);
      if (lane == 0) acc[r] = fmaf(wt, y, acc[r]);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)t * W + i] = acc[i];
}
}  // namespace

FB_API int fb_moe_route(const float* z, long long ld, const float* bias, int E, int top,
                        int* chosen, float* weights, int T, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && E > 0 && E <= 256 && top > 0 && top <= E && top <= 32 && ld >= E,
             "moe_route: %d experts (at most 256), %d chosen (at most 32)", E, top);
  if (T == 0) return 0;
  // a warp per token
  fb_launch(moe_route_kernel, dim3(T), dim3(32), 0, stream, z, ld, bias, E, top, chosen, weights);
  return fb_check_launch("moe_route");
}

FB_API int fb_moe_experts_rows(const void* h, int dtype, const void* gate_up, const void* down,
                               const int* chosen, const float* weights, float* out, int T, int W,
                               int ff, int top, int E, float limit, float alpha,
                               cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && W > 0 && ff > 0 && top > 0, "moe_experts_rows: bad sizes");
  const size_t smem = (size_t)(2 * W + ff) * 4;
  FB_REQUIRE(smem <= 200 * 1024, "moe_experts_rows: width %d and %d hidden units do not fit "
             "shared memory", W, ff);
  if (T == 0) return 0;
#define FB_MOE_ROWS(E_)                                                                         \
  do {                                                                                          \
    static bool seen[64];                                                                       \
    if (smem > 48 * 1024 && fb_first_use_on_device(seen))                                       \
      cudaFuncSetAttribute(moe_experts_rows_kernel<E_>,                                         \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);            \
    fb_launch(moe_experts_rows_kernel<E_>, dim3(T), dim3(256), smem, stream, (const E_*)h,      \
              (const E_*)gate_up, (const E_*)down, chosen, weights, out, W, ff, top, E, limit,  \
              alpha);                                                                           \
  } while (0)
  FB_DISPATCH_DTYPE(dtype, E_, FB_MOE_ROWS(E_));
#undef FB_MOE_ROWS
  return fb_check_launch("moe_experts_rows");
}
