// A routed feed-forward: every row goes through `top` of `n_expert` small two-layer experts.
//   z = W_router h   (32-bit),  s = softmax(z) over all experts,  the `top` largest s are chosen
//   (ties to the lower index), their weights are those s themselves or, with `renorm`, divided by
//   their sum;  out = sum over the chosen e of s_e * W_down[e] act(W_up[e] h).
//   moe_route : a block per row -> ids [T, top], weights [T, top]
//   moe_up    : a block per (row, chosen expert, slice of the inner width): inner = act(W_up[e] h)
//   moe_down  : a block per (row, slice of the width): x += sum_j s_j W_down[e_j] inner_j   (one block owns
//               an output, so the sum has a fixed order and needs no atomics)
// Expert weights are stacked [n_expert, out, in].  A warp makes an output at a time: its lanes walk the
// input dimension, which is how the weight rows lie in memory.  Accumulation and activation are 32-bit.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int MOE_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_route_kernel(const T* h, int ldh, const T* __restrict__ wr, int C, int n_expert, int top, int renorm, int* ids,
                 float* weights) {
  pdl_trigger();
  extern __shared__ float smem[];
  float* row = smem;               // [C]
  float* prob = smem + C;          // [n_expert]
  __shared__ float scratch[32];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = to_float(h[(size_t)t * ldh + c]);
  __syncthreads();
  for (int e = warp; e < n_expert; e += MOE_WARPS) {
    const T* w = wr + (size_t)e * C;
    float s = 0.0f;
    for (int c = lane; c < C; c += 32) s += row[c] * to_float(w[c]);
    s = warp_sum(s);
    if (lane == 0) prob[e] = s;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int e = threadIdx.x; e < n_expert; e += blockDim.x) mx = fmaxf(mx, prob[e]);
  mx = block_max(mx, scratch);
  float sum = 0.0f;
  for (int e = threadIdx.x; e < n_expert; e += blockDim.x) sum += expf(prob[e] - mx);
  sum = block_sum(sum, scratch);
  __syncthreads();
  for (int e = threadIdx.x; e < n_expert; e += blockDim.x) prob[e] = expf(prob[e] - mx) / sum;
  __syncthreads();
  if (warp == 0) {
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
      float best = -1.0f;
      int at = -1;
      for (int e = lane; e < n_expert; e += 32) {
        const float p = prob[e];
        if (p > best) { best = p; at = e; }      // (a taken expert holds -2; a NaN is never larger)
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
      }
      if (at < 0) { at = k % n_expert; best = 0.0f; }   // rows that hold no numbers (rows of no request)
      if (lane == 0) {
        ids[(size_t)t * top + k] = at;
        weights[(size_t)t * top + k] = best;
        prob[at] = -2.0f;
      }
      total += best;
      __syncwarp();
    }
    if (renorm && total > 0.0f)
      for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] /= total;
  }
}

constexpr int MOE_PER_WARP = 8;   // outputs a warp makes one after the other

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_up_kernel(const T* h, int ldh, const T* __restrict__ w_up, const int* ids, T* inner, int C, int F, int top,
              int act) {
  pdl_trigger();
  extern __shared__ float row[];   // [C]
  const int p = blockIdx.x, t = p / top, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int e = ids[p];
  for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = to_float(h[(size_t)t * ldh + c]);
  __syncthreads();
  const int f0 = (blockIdx.y * MOE_WARPS + warp) * MOE_PER_WARP;
  for (int f = f0; f < min(F, f0 + MOE_PER_WARP); ++f) {
    const T* w = w_up + ((size_t)e * F + f) * C;
    float s = 0.0f;
    for (int c = lane; c < C; c += 32) s += row[c] * to_float(w[c]);
    s = warp_sum(s);
    if (lane == 0) inner[(size_t)p * F + f] = from_float<T>(apply_act(s, act));
  }
}

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* inner, const T* __restrict__ w_down, const int* ids, const float* weights, float* x, int C,
                int F, int top) {
  pdl_trigger();
  extern __shared__ float rows[];  // [top][F]
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  for (int i = threadIdx.x; i < top * F; i += blockDim.x) rows[i] = to_float(inner[(size_t)t * top * F + i]);
  __syncthreads();
  const int c0 = (blockIdx.y * MOE_WARPS + warp) * MOE_PER_WARP;
  for (int c = c0; c < min(C, c0 + MOE_PER_WARP); ++c) {
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
      const T* w = w_down + ((size_t)ids[(size_t)t * top + k] * C + c) * F;
      const float* r = rows + k * F;
      float s = 0.0f;
      for (int f = lane; f < F; f += 32) s += r[f] * to_float(w[f]);
      total += weights[(size_t)t * top + k] * warp_sum(s);
    }
    if (lane == 0) x[(size_t)t * C + c] += total;
  }
}

}  // namespace nib

using namespace nib;

extern "C" int nib_moe_route(int dtype, const void* h, int ldh, const void* w_router, int T, int C, int n_expert,
                             int top, int renorm, int* ids, float* weights, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || top > n_expert || C <= 0) return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)(C + n_expert) * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_route_kernel<float>, dim3(T), dim3(MOE_WARPS * 32), smem, stream, (const float*)h, ldh,
               (const float*)w_router, C, n_expert, top, renorm, ids, weights);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_route_kernel<bf16>, dim3(T), dim3(MOE_WARPS * 32), smem, stream, (const bf16*)h, ldh,
               (const bf16*)w_router, C, n_expert, top, renorm, ids, weights);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// inner: [T * top, F] in `dtype`; act: an activation code of the linear epilogues.
extern "C" int nib_moe_up(int dtype, const void* h, int ldh, const void* w_up, const int* ids, void* inner, int T,
                          int C, int F, int top, int act, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const dim3 grid(T * top, (F + MOE_WARPS * MOE_PER_WARP - 1) / (MOE_WARPS * MOE_PER_WARP));
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_up_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)h, ldh,
               (const float*)w_up, ids, (float*)inner, C, F, top, act);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_up_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)h, ldh, (const bf16*)w_up,
               ids, (bf16*)inner, C, F, top, act);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// x: the 32-bit residual stream [T, C]; the experts' weighted outputs are added to it.
extern "C" int nib_moe_down(int dtype, const void* inner, const void* w_down, const int* ids, const float* weights,
                            float* x, int T, int C, int F, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)top * F * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const dim3 grid(T, (C + MOE_WARPS * MOE_PER_WARP - 1) / (MOE_WARPS * MOE_PER_WARP));
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_down_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)inner,
               (const float*)w_down, ids, weights, x, C, F, top);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_down_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)inner,
               (const bf16*)w_down, ids, weights, x, C, F, top);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}
