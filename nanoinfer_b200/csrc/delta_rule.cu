// The generalised delta rule: a recurrent mixer whose state per head is a matrix S [key channel, value
// channel] that every token first decays per key channel, then partly erases along its own unit key,
// then writes its key/value pair into:
//   w   = exp(-exp(-1/2) * sigmoid(w_logit))           decay per head and key channel, in (0.545, 1)
//   a   = sigmoid(a_logit)                              removal rate per head and key channel
//   u   = k / sqrt(sum(k^2) + 1e-6)                     the head's unit key
//   S_t = diag(w) S_(t-1) - (a * u) (u^T S_(t-1)) + k v^T        (both terms read the old state)
//   o_t = S_t^T r
// then each head's o is divided by its root mean square, multiplied by a weight and by sigmoid(gate).
// One block per (batch entry, head) walks the entry's rows in order; a column of S belongs to one value
// channel, and the columns do not see one another.  For head sizes that are multiples of 16 up to 128 a
// column lives in the registers of four neighbouring threads, a quarter of the key channels each (u^T S and
// S^T r are then sums over four lanes: two shuffles), every token's per-channel vectors (r, k, w, a u, u) are made by the
// channel's thread for the NEXT token while this one is worked on and passed through a double buffer in
// shared memory (one barrier a token), the raw outputs take the place of the decay logits already used, and
// the division by each head's root mean square is a pass over the rows afterwards (inside the kernel for a
// step of single tokens, else a kernel of its own with a warp a row and head).  Other head sizes keep the
// state in shared memory.  The state goes back to the request's slot at the end.  The projections come in
// as 32-bit floats; everything here is 32-bit.
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

template <int DIM> struct DeltaInputs {
  float r, k, a, w, u, v, ks[(DIM + 31) / 32];
};

// What a token gives the recurrence besides r, k and v does not depend on the state: for a step with prompt
// portions it is made for all rows at once, a warp a (row, head): the decay w takes the place of its logit, a u
// the place of the removal logit, the unit key u goes to a buffer of its own.
__global__ void __launch_bounds__(256)
delta_prepare_kernel(float* proj, int ld, int k_off, int a_off, float* wl, int ld_w, const float* __restrict__ w0,
                     const float* __restrict__ a_bias, float* unit, int n_head, int dim, int n_rows) {
  pdl_trigger();
  const int wi = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();
  if (wi >= n_rows * n_head) return;
  const int t = wi / n_head, h = wi % n_head;
  float* p = proj + (size_t)t * ld;
  float ks = 0.0f;
  for (int i = lane; i < dim; i += 32) {
    const float k = p[k_off + h * dim + i];
    ks += k * k;
  }
  const float inv = 1.0f / sqrtf(warp_sum(ks) + 1e-6f);
  for (int i = lane; i < dim; i += 32) {
    const int col = h * dim + i;
    const float u = p[k_off + col] * inv;
    const size_t at = (size_t)t * ld_w + col;
    wl[at] = expf(-0.6065306597126334f * sigmoid_f(wl[at] + w0[col]));
    p[a_off + col] = sigmoid_f(p[a_off + col] + a_bias[col]) * u;
    unit[(size_t)t * n_head * dim + col] = u;
  }
}

// o[t, head] / rms * weight * sigmoid(gate) for the rows t = first, first + step, ... below `end`; a warp a row.
template <typename T, int DIM>
__device__ __forceinline__ void delta_finish_rows(const float* proj, int ld, int g_off, const float* raw, int ld_w,
                                                  const float* __restrict__ norm_w, int h, float eps, T* out, int ldo,
                                                  int first, int end, int step, int lane) {
  constexpr int M = (DIM + 31) / 32;
  for (int t = first; t < end; t += step) {
    float ov[M], ss = 0.0f;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const int i = lane + 32 * m;
      ov[m] = i < DIM ? raw[(size_t)t * ld_w + h * DIM + i] : 0.0f;
      ss += ov[m] * ov[m];
    }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)DIM + eps);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const int i = lane + 32 * m;
      if (i < DIM) {
        const int col = h * DIM + i;
        out[(size_t)t * ldo + col] =
            from_float<T>(ov[m] * rstd * norm_w[col] * sigmoid_f(proj[(size_t)t * ld + g_off + col]));
      }
    }
  }
}

constexpr int DELTA_PARTS = 4;     // threads that share a column of the state, each a quarter of the key channels

template <typename T, int DIM>
__global__ void __launch_bounds__(DIM * DELTA_PARTS)
delta_rule_reg_kernel(const float* proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off, float* wl,
                      int ld_w, const float* __restrict__ w0, const float* __restrict__ a_bias,
                      const float* __restrict__ norm_w, float* state, const int* __restrict__ entry_start,
                      const int* __restrict__ entry_slot, int n_head, float eps, T* out, int ldo, int finish_inside,
                      const float* unit) {
  pdl_trigger();
  constexpr int KPT = DIM / DELTA_PARTS, NV = (DIM + 31) / 32 * 32, M = (DIM + 31) / 32;
  __shared__ __align__(16) float st[2][5][DIM];     // r, k, w, a u, u of the token at hand and of the next
  const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  // the thread's column, and which 16-byte pieces of a per-channel vector are its own: pieces part, part + 4, ...
  // (the four threads of a column then read 64 bytes side by side: no two of them meet in a bank)
  const int j = tid / DELTA_PARTS, part = tid % DELTA_PARTS;
  const int col = h * DIM + j;
  // the first NV threads (whole warps) also make the per-channel vectors, thread c the channel c
  const bool maker = tid < NV, made = tid < DIM;
  const int mcol = h * DIM + (made ? tid : 0);
  const int t0 = entry_start[e], t1 = entry_start[e + 1];
  float* slot = state + ((size_t)entry_slot[e] * n_head + h) * (size_t)DIM * DIM;
  const float w0c = w0[mcol], abc = a_bias[mcol];
  pdl_wait();
  if (t0 >= t1) return;
  float S[KPT];       // S[4 m + c] is key channel 4 (part + 4 m) + c of column j
#pragma unroll
  for (int i = 0; i < KPT; ++i) S[i] = slot[(4 * (part + DELTA_PARTS * (i / 4)) + i % 4) * DIM + j];

  DeltaInputs<DIM> in;
  auto load = [&](int t) {
    const float* p = proj + (size_t)t * ld;
    in.v = p[v_off + col];
    if (maker) {
      in.r = p[r_off + mcol]; in.k = p[k_off + mcol]; in.a = p[a_off + mcol];
      in.w = wl[(size_t)t * ld_w + mcol];
      if (unit != nullptr) {         // w, a u and u were made for all rows ahead of this kernel
        in.u = unit[(size_t)t * n_head * DIM + mcol];
      } else {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const int i = lane + 32 * m;
          in.ks[m] = i < DIM ? p[k_off + h * DIM + i] : 0.0f;
        }
      }
    }
  };
  auto finish = [&](int buf) {       // every making warp sums the head's k^2 on its own: no barrier
    if (!maker) return;
    if (unit != nullptr) {
      if (made) {
        st[buf][0][tid] = in.r; st[buf][1][tid] = in.k; st[buf][2][tid] = in.w; st[buf][3][tid] = in.a;
        st[buf][4][tid] = in.u;
      }
      return;
    }
    float ks = 0.0f;
#pragma unroll
    for (int m = 0; m < M; ++m) ks += in.ks[m] * in.ks[m];
    ks = warp_sum(ks);
    if (made) {
      const float u = in.k / sqrtf(ks + 1e-6f);
      st[buf][0][tid] = in.r;
      st[buf][1][tid] = in.k;
      st[buf][2][tid] = expf(-0.6065306597126334f * sigmoid_f(in.w + w0c));
      st[buf][3][tid] = sigmoid_f(in.a + abc) * u;
      st[buf][4][tid] = u;
    }
  };
  load(t0);
  finish(0);
  float vc = in.v;
  __syncthreads();
  int cur = 0;
  for (int t = t0; t < t1; ++t) {
    const bool more = t + 1 < t1;
    if (more) load(t + 1);           // asked for now, used after this token's arithmetic
    const float4* r4 = reinterpret_cast<const float4*>(st[cur][0]) + part;
    const float4* k4 = reinterpret_cast<const float4*>(st[cur][1]) + part;
    const float4* w4 = reinterpret_cast<const float4*>(st[cur][2]) + part;
    const float4* a4 = reinterpret_cast<const float4*>(st[cur][3]) + part;
    const float4* u4 = reinterpret_cast<const float4*>(st[cur][4]) + part;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < KPT / 4; ++i) {
      const float4 u = u4[DELTA_PARTS * i];
      s0 += u.x * S[4 * i] + u.z * S[4 * i + 2];
      s1 += u.y * S[4 * i + 1] + u.w * S[4 * i + 3];
    }
    float sa = s0 + s1;              // u^T S over this thread's channels; the column's four threads are neighbours
    sa += __shfl_xor_sync(0xffffffffu, sa, 1);
    sa += __shfl_xor_sync(0xffffffffu, sa, 2);
    float o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int i = 0; i < KPT / 4; ++i) {
      const float4 w = w4[DELTA_PARTS * i], a = a4[DELTA_PARTS * i], k = k4[DELTA_PARTS * i], r = r4[DELTA_PARTS * i];
      S[4 * i] = w.x * S[4 * i] - a.x * sa + k.x * vc;             o0 += S[4 * i] * r.x;
      S[4 * i + 1] = w.y * S[4 * i + 1] - a.y * sa + k.y * vc;     o1 += S[4 * i + 1] * r.y;
      S[4 * i + 2] = w.z * S[4 * i + 2] - a.z * sa + k.z * vc;     o0 += S[4 * i + 2] * r.z;
      S[4 * i + 3] = w.w * S[4 * i + 3] - a.w * sa + k.w * vc;     o1 += S[4 * i + 3] * r.w;
    }
    float o = o0 + o1;
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    if (part == 0) wl[(size_t)t * ld_w + col] = o;                   // the raw output where the decay logit was
    if (more) {
      finish(cur ^ 1);
      vc = in.v;
    }
    __syncthreads();
    cur ^= 1;
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) slot[(4 * (part + DELTA_PARTS * (i / 4)) + i % 4) * DIM + j] = S[i];
  if (finish_inside)
    delta_finish_rows<T, DIM>(proj, ld, g_off, wl, ld_w, norm_w, h, eps, out, ldo, t0 + (tid >> 5), t1,
                              DIM * DELTA_PARTS / 32, lane);
}

template <typename T, int DIM>
__global__ void __launch_bounds__(256)
delta_finish_kernel(const float* proj, int ld, int g_off, const float* raw, int ld_w, const float* __restrict__ norm_w,
                    int n_head, float eps, T* out, int ldo, int n_rows) {
  pdl_trigger();
  const int w = blockIdx.x * 8 + (threadIdx.x >> 5);      // (row, head) pairs, a warp each
  pdl_wait();
  if (w >= n_rows * n_head) return;
  const int t = w / n_head, h = w % n_head;
  delta_finish_rows<T, DIM>(proj, ld, g_off, raw, ld_w, norm_w, h, eps, out, ldo, t, t + 1, 1, threadIdx.x & 31);
}

template <typename T, int DIM>
static int launch_delta_reg(float* proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off, float* wl,
                            int ld_w, const float* w0, const float* a_bias, const float* norm_w, float* state,
                            const int* entry_start, const int* entry_slot, int n_entries, int n_rows, int n_head,
                            float eps, T* out, int ldo, float* unit, cudaStream_t stream) {
  // single tokens: a row's gates and its norm cost less inside the kernel than a launch each
  const int inside = n_rows == n_entries || unit == nullptr;
  if (!inside)
    launch_pdl(delta_prepare_kernel, dim3((n_rows * n_head + 7) / 8), dim3(256), 0, stream, proj, ld, k_off, a_off, wl,
               ld_w, w0, a_bias, unit, n_head, DIM, n_rows);
  launch_pdl(delta_rule_reg_kernel<T, DIM>, dim3(n_entries, n_head), dim3(DIM * DELTA_PARTS), 0, stream, proj, ld,
             r_off, k_off, v_off, g_off, a_off, wl, ld_w, w0, a_bias, norm_w, state, entry_start, entry_slot, n_head,
             eps, out, ldo, inside, inside ? (const float*)nullptr : (const float*)unit);
  if (!inside)
    launch_pdl(delta_finish_kernel<T, DIM>, dim3((n_rows * n_head + 7) / 8), dim3(256), 0, stream, proj, ld, g_off,
               (const float*)wl, ld_w, norm_w, n_head, eps, out, ldo, n_rows);
  NIB_LAUNCH_CHECK();
}

template <typename T>
static int pick_delta_reg(int dim, float* proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off,
                          float* wl, int ld_w, const float* w0, const float* a_bias, const float* norm_w, float* state,
                          const int* entry_start, const int* entry_slot, int n_entries, int n_rows, int n_head,
                          float eps, T* out, int ldo, float* unit, cudaStream_t stream) {
#define NIB_DELTA(D)                                                                                                \
  case D:                                                                                                           \
    return launch_delta_reg<T, D>(proj, ld, r_off, k_off, v_off, g_off, a_off, wl, ld_w, w0, a_bias, norm_w, state, \
                                  entry_start, entry_slot, n_entries, n_rows, n_head, eps, out, ldo, unit, stream)
  switch (dim) {
    NIB_DELTA(16); NIB_DELTA(32); NIB_DELTA(48); NIB_DELTA(64); NIB_DELTA(80); NIB_DELTA(96); NIB_DELTA(112);
    NIB_DELTA(128);
  }
#undef NIB_DELTA
  return NIB_ERR_UNSUPPORTED_SIZE;
}

}  // namespace nib

using namespace nib;

// proj: float [T, ld] holding r, k, v, gate logits and removal logits at the given column offsets (n_head *
// dim columns each); wl: float [T, ld_w] decay logits before their bias w0.  state: float [slots, n_head,
// dim, dim].  out: [T, n_head * dim] in `dtype`.  n_rows: the rows of all entries together.  wl and the
// removal logits of proj are scratch afterwards (the kernel for head sizes in steps of 16 leaves raw outputs
// and, for steps with prompt portions, the rows' gates there); unit: float [n_rows, n_head * dim] of scratch
// for the unit keys (may be null: the gates are then made token by token inside the recurrence).
extern "C" int nib_delta_rule(int dtype, float* proj, int ld, int r_off, int k_off, int v_off, int g_off,
                              int a_off, float* wl, int ld_w, const float* w0, const float* a_bias,
                              const float* norm_w, float* state, const int* entry_start, const int* entry_slot,
                              int n_entries, int n_rows, int n_head, int dim, float eps, void* out, int ldo,
                              float* unit, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (dim <= 0 || dim > 224 || n_head <= 0) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dim % 16 == 0 && dim <= 128) {
    if (dtype == DT_F32)
      return pick_delta_reg<float>(dim, proj, ld, r_off, k_off, v_off, g_off, a_off, wl, ld_w, w0, a_bias, norm_w,
                                   state, entry_start, entry_slot, n_entries, n_rows, n_head, eps, (float*)out, ldo,
                                   unit, stream);
    if (dtype == DT_BF16)
      return pick_delta_reg<bf16>(dim, proj, ld, r_off, k_off, v_off, g_off, a_off, wl, ld_w, w0, a_bias, norm_w,
                                  state, entry_start, entry_slot, n_entries, n_rows, n_head, eps, (bf16*)out, ldo,
                                  unit, stream);
    return NIB_ERR_BAD_ARGUMENT;
  }
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
