// The generalised delta rule: a recurrent mixer whose state per head is a matrix S [key channel, value
// channel] that every token first decays per key channel, then partly erases along its own unit key,
// then writes its key/value pair into:
//   w   = exp(-exp(-1/2) * sigmoid(w_logit))           decay per head and key channel, in (0.545, 1)
//   a   = sigmoid(a_logit)                              removal rate per head and key channel
//   u   = k / sqrt(sum(k^2) + 1e-6)                     the head's unit key
//   S_t = diag(w) S_(t-1) - (a * u) (u^T S_(t-1)) + k v^T        (both terms read the old state)
//   o_t = S_t^T r
// then each head's o is divided by its root mean square, multiplied by a weight and by sigmoid(gate).
// One block per (batch entry, head) walks the entry's rows in order; thread j owns value channel j, the
// state lives in shared memory as 32-bit floats and goes back to the request's slot at the end.  The
// projections come in as 32-bit floats; everything here is 32-bit.
#include "api.h"
#include "common.cuh"

namespace nib {

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T>
__global__ void delta_rule_kernel(const float* proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off,
                                  const float* wl, int ld_w, const float* __restrict__ w0,
                                  const float* __restrict__ a_bias, const float* __restrict__ norm_w, float* state,
                                  const int* __restrict__ entry_start, const int* __restrict__ entry_slot,
                                  int n_head, int dim, float eps, T* out, int ldo) {
  pdl_trigger();
  extern __shared__ float smem[];
  float* S = smem;                       // [dim][dim]: S[i * dim + j], key channel i, value channel j
  float* sh_r = S + dim * dim;
  float* sh_k = sh_r + dim;
  float* sh_w = sh_k + dim;
  float* sh_au = sh_w + dim;
  float* sh_u = sh_au + dim;
  __shared__ float scratch[32];
  const int e = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const bool on = j < dim;
  const int col = h * dim + j;
  const int t0 = entry_start[e], t1 = entry_start[e + 1];
  float* slot = state + ((size_t)entry_slot[e] * n_head + h) * (size_t)dim * dim;
  const float w0j = on ? w0[col] : 0.f, abj = on ? a_bias[col] : 0.f, nwj = on ? norm_w[col] : 0.f;
  pdl_wait();
  for (int i = threadIdx.x; i < dim * dim; i += blockDim.x) S[i] = slot[i];
  float r = 0.f, k = 0.f, v = 0.f, g = 0.f, al = 0.f, wv = 0.f;
  if (on && t0 < t1) {
    const float* p = proj + (size_t)t0 * ld;
    r = p[r_off + col]; k = p[k_off + col]; v = p[v_off + col]; g = p[g_off + col]; al = p[a_off + col];
    wv = wl[(size_t)t0 * ld_w + col];
  }
  for (int t = t0; t < t1; ++t) {
    const float rc = r, kc = k, vc = v, gc = g, alc = al, wc = wv;
    if (on && t + 1 < t1) {              // the next row's values are asked for while this one is worked on
      const float* p = proj + (size_t)(t + 1) * ld;
      r = p[r_off + col]; k = p[k_off + col]; v = p[v_off + col]; g = p[g_off + col]; al = p[a_off + col];
      wv = wl[(size_t)(t + 1) * ld_w + col];
    }
    const float ksq = block_sum(on ? kc * kc : 0.f, scratch);
    if (on) {
      const float u = kc / sqrtf(ksq + 1e-6f);
      sh_r[j] = rc;
      sh_k[j] = kc;
      sh_w[j] = expf(-0.6065306597126334f * sigmoid_f(wc + w0j));
      sh_au[j] = sigmoid_f(alc + abj) * u;
      sh_u[j] = u;
    }
    __syncthreads();
    float o = 0.f;
    if (on) {
      float sa = 0.f;
      for (int i = 0; i < dim; ++i) sa += sh_u[i] * S[i * dim + j];
      for (int i = 0; i < dim; ++i) {
        const float s = sh_w[i] * S[i * dim + j] - sh_au[i] * sa + sh_k[i] * vc;
        S[i * dim + j] = s;
        o += s * sh_r[i];
      }
    }
    const float osq = block_sum(on ? o * o : 0.f, scratch);   // (its barriers also end this row's reads of sh_*)
    if (on)
      out[(size_t)t * ldo + col] = from_float<T>(o / sqrtf(osq / (float)dim + eps) * nwj * sigmoid_f(gc));
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim * dim; i += blockDim.x) slot[i] = S[i];
}

}  // namespace nib

using namespace nib;

// proj: float [T, ld] holding r, k, v, gate logits and removal logits at the given column offsets (n_head *
// dim columns each); wl: float [T, ld_w] decay logits before their bias w0.  state: float [slots, n_head,
// dim, dim].  out: [T, n_head * dim] in `dtype`.
extern "C" int nib_delta_rule(int dtype, const float* proj, int ld, int r_off, int k_off, int v_off, int g_off,
                              int a_off, const float* wl, int ld_w, const float* w0, const float* a_bias,
                              const float* norm_w, float* state, const int* entry_start, const int* entry_slot,
                              int n_entries, int n_head, int dim, float eps, void* out, int ldo,
                              cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (dim <= 0 || dim > 224 || n_head <= 0) return NIB_ERR_UNSUPPORTED_SIZE;
  const size_t smem = ((size_t)dim * dim + 5 * (size_t)dim) * sizeof(float);
  const int threads = (dim + 31) / 32 * 32;
  const dim3 grid(n_entries, n_head);
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_rule_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(delta_rule_kernel<float>, grid, dim3(threads), smem, stream, proj, ld, r_off, k_off, v_off, g_off,
               a_off, wl, ld_w, w0, a_bias, norm_w, state, entry_start, entry_slot, n_head, dim, eps, (float*)out, ldo);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_rule_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(delta_rule_kernel<bf16>, grid, dim3(threads), smem, stream, proj, ld, r_off, k_off, v_off, g_off,
               a_off, wl, ld_w, w0, a_bias, norm_w, state, entry_start, entry_slot, n_head, dim, eps, (bf16*)out, ldo);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}
