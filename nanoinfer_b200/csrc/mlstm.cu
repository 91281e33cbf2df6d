// The matrix memory of xLSTM (mLSTM): a recurrent mixer whose state per head is a matrix S [key channel, value
// channel], a vector n [key channel] and a running maximum mx of the log gates, kept so that the exponentials
// of the gates never overflow.  Per token and head, with log input gate gi and log forget gate gf (both <= cap):
//   gi  = cap * tanh((z_i + b_i) / cap),   gf = logsigmoid(cap * tanh((z_f + b_f) / cap))
//   mx' = max(gf + mx, gi)                                  (mx starts at 0)
//   S'  = exp(gf + mx - mx') S + exp(gi - mx') k v^T,       n' likewise with k alone
//   o   = S'^T q / (max(|n' . q|, exp(-mx')) + 1e-6),       q scaled by dim^(-1/2)
// then each head's o is divided by its root mean square, multiplied by a weight and by sigmoid(gate).
//
// Three kernels:
//   mlstm_gates  : a block per (batch entry, head).  What does not depend on S: the gates of all the entry's rows,
//                  the running maximum (a serial pass of one thread over 256 rows at a time), and from them the two
//                  factors exp(gf + mx - mx'), exp(gi - mx') and the floor exp(-mx') of every row.  mx goes back to
//                  the request's slot.
//   mlstm_scan   : a block per (entry, head, 64 value channels) walks the entry's rows in order.  A column of S
//                  belongs to one value channel and the columns do not see one another; n is one more column whose
//                  value is 1 (the first block of a head carries it).  A column lives in the registers of four
//                  (columns of more than 96 floats: eight) neighbouring threads, which take the 16-byte pieces r,
//                  r + R, r + 2R, ... of q and k (they read side by side: no bank conflicts; S^T q is a sum over
//                  those lanes, two or three shuffles).  The
//                  rows' q, k, v and factors come into shared memory eight rows at a time by `cp.async`, the next
//                  eight while these are worked on: two barriers per eight rows, none between rows.
//                  It leaves the numerators S'^T q and the denominators.
//   mlstm_finish : a warp per (row, head): the division, the head's root mean square, weight and gate.
// The projections come in as 32-bit floats; everything here is 32-bit.  State per slot and head:
// [value channels + 1][dim rounded up to 16] floats (the last column is n), then mx and three unused floats.
#include <cstdint>

#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int ML_GATE_ROWS = 256;
// threads of a block that owns VC value channels: R a column, the column of n, rounded up to whole warps
__host__ __device__ constexpr int ml_threads(int vc, int r) { return (r * (vc + 1) + 31) / 32 * 32; }

__device__ __forceinline__ float ml_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float ml_logsigmoid(float v) { return fminf(v, 0.0f) - log1pf(expf(-fabsf(v))); }

__global__ void __launch_bounds__(ML_GATE_ROWS)
mlstm_gates_kernel(const float* proj, int ld, int i_off, int f_off, const float* __restrict__ bias_i,
                   const float* __restrict__ bias_f, float cap, float* state, long long slot_stride,
                   long long head_stride, const int* __restrict__ entry_start, const int* __restrict__ entry_slot,
                   int n_head, float* gates) {
  pdl_trigger();
  __shared__ float gi[ML_GATE_ROWS], gf[ML_GATE_ROWS], gm[ML_GATE_ROWS + 1];
  const int e = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  const int t0 = entry_start[e], t1 = entry_start[e + 1];
  float* mx_at = state + (size_t)entry_slot[e] * slot_stride + (size_t)(h + 1) * head_stride - 4;
  const float bi = bias_i[h], bf = bias_f[h], inv_cap = 1.0f / cap;
  pdl_wait();
  if (i == 0) gm[0] = *mx_at;
  for (int base = t0; base < t1; base += ML_GATE_ROWS) {
    const int n = min(ML_GATE_ROWS, t1 - base);
    if (i < n) {
      const float* p = proj + (size_t)(base + i) * ld;
      gi[i] = cap * tanhf((p[i_off + h] + bi) * inv_cap);
      gf[i] = ml_logsigmoid(cap * tanhf((p[f_off + h] + bf) * inv_cap));
    }
    __syncthreads();
    if (i == 0) {
      float m = gm[0];
#pragma unroll 8
      for (int j = 0; j < n; ++j) {
        m = fmaxf(gf[j] + m, gi[j]);
        gm[j + 1] = m;
      }
    }
    __syncthreads();
    if (i < n) {
      const float m = gm[i + 1];
      float* g = gates + ((size_t)(base + i) * n_head + h) * 4;
      g[0] = expf(gf[i] + gm[i] - m);
      g[1] = expf(gi[i] - m);
      g[2] = expf(-m);
    }
    const float last = gm[n];
    __syncthreads();
    if (i == 0) gm[0] = last;
  }
  if (i == 0) *mx_at = gm[0];
}

constexpr int ML_CHUNK = 8;                // rows staged at a time

__device__ __forceinline__ void ml_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ml_copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// R: threads a column (4 for columns of up to 96 floats, 8 beyond: a row's time grows with the pieces a thread
// walks, and more lanes a column cost a shuffle more).  NP: 16-byte pieces of q (and of k) a thread
// holds: it walks the pieces r, r + R, r + 2R, ... of a column of dp = 16 * ceil(dim / 16) floats, R * NP >= dp / 4.
// ML_VC: value channels a block (the host takes fewer where that fills more of the device).  aligned: every run of
// values that a row brings starts on a 16-byte boundary and is a multiple of four long (3: and the block has a
// thread for each of a row's 16-byte pieces).
// The entry's rows come in chunks of ML_CHUNK: while one chunk is worked on (no barrier between its rows: what a
// row reads lies in shared memory, what it changes in registers) the next one is on its way (`cp.async`).
template <int NP, int R, int ML_VC>
__global__ void __launch_bounds__(ml_threads(ML_VC, R))
mlstm_scan_kernel(const float* proj, int ld, int q_off, int k_off, int v_off, const float* gates, float* state,
                  long long slot_stride, long long head_stride, const int* __restrict__ entry_start,
                  const int* __restrict__ entry_slot, int n_head, int dim, int vdim, float q_scale, float* num,
                  int ld_num, float* den, int ALIGNED, int dp) {
  pdl_trigger();
  constexpr int ML_THREADS = ml_threads(ML_VC, R);
  constexpr int DP = 4 * R * NP;                    // room for q (and for k) in a staged row
  constexpr int STAGE = 2 * DP + ML_VC + 4;         // q | k | v of the block's channels | the row's three factors
  __shared__ __align__(16) float stage[2][ML_CHUNK][STAGE];
  const int e = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * ML_VC, tid = threadIdx.x;
  const int jc = tid / R, r = tid % R;
  const int t0 = entry_start[e], t1 = entry_start[e + 1];
  // this thread's column: a value channel of the block, or (first block of the head) the column of n
  const bool is_n = jc == ML_VC && blockIdx.z == 0;
  const int col = is_n ? vdim : c0 + jc;
  const bool live = is_n || (jc < ML_VC && col < vdim);
  float* column = state + (size_t)entry_slot[e] * slot_stride + (size_t)h * head_stride + (size_t)col * dp;
  const int n4 = dp / 4;                            // 16-byte pieces of a column: this thread's are r + p * R < n4
  const int nv = min(ML_VC, vdim - c0);             // value channels of this block
  float* out_at = num + (size_t)t0 * ld_num + h * vdim + (is_n ? 0 : col);   // this column's numerator of row t0
  // asks for the rows first .. first + ML_CHUNK - 1 (those below t1) into stage[buf]
  auto fetch = [&](int first, int buf) {
    const int rows = min(ML_CHUNK, t1 - first);
    if (ALIGNED == 3) {
      // a thread owns the same 16-byte piece of every row: no division in the loop (with it, a fifth of a row's
      // instructions went into finding places: 0.40 -> 0.32 ms a prompt of 952 rows)
      const int c = 4 * tid;
      if (c < 2 * dim + nv + 4) {
        const float* src;
        int at;
        if (c < dim) { src = proj + q_off + h * dim + c; at = c; }
        else if (c < 2 * dim) { src = proj + k_off + h * dim + c - dim; at = DP + c - dim; }
        else if (c < 2 * dim + nv) { src = proj + v_off + h * vdim + c0 + c - 2 * dim; at = 2 * DP + c - 2 * dim; }
        else { src = nullptr; at = 2 * DP + ML_VC; }
        if (src != nullptr) {
          src += (size_t)first * ld;
          for (int row = 0; row < rows; ++row, src += ld) ml_copy16(&stage[buf][row][at], src);
        } else {
          const float* g = gates + ((size_t)first * n_head + h) * 4;
          for (int row = 0; row < rows; ++row, g += 4 * n_head) ml_copy16(&stage[buf][row][at], g);
        }
      }
    } else if (ALIGNED) {
      const int per = (2 * dim + nv) / 4 + 1;       // 16-byte pieces a row
      for (int i = tid; i < rows * per; i += ML_THREADS) {
        const int row = i / per, c = 4 * (i % per);
        const float* p = proj + (size_t)(first + row) * ld;
        float* dst = stage[buf][row];
        if (c < dim) ml_copy16(dst + c, p + q_off + h * dim + c);
        else if (c < 2 * dim) ml_copy16(dst + DP + c - dim, p + k_off + h * dim + c - dim);
        else if (c < 2 * dim + nv) ml_copy16(dst + 2 * DP + c - 2 * dim, p + v_off + h * vdim + c0 + c - 2 * dim);
        else ml_copy16(dst + 2 * DP + ML_VC, gates + ((size_t)(first + row) * n_head + h) * 4);
      }
    } else {
      const int per = 2 * dim + nv + 3;
      for (int i = tid; i < rows * per; i += ML_THREADS) {
        const int row = i / per, c = i % per;
        const float* p = proj + (size_t)(first + row) * ld;
        float* dst = stage[buf][row];
        if (c < dim) ml_copy4(dst + c, p + q_off + h * dim + c);
        else if (c < 2 * dim) ml_copy4(dst + DP + c - dim, p + k_off + h * dim + c - dim);
        else if (c < 2 * dim + nv) ml_copy4(dst + 2 * DP + c - 2 * dim, p + v_off + h * vdim + c0 + c - 2 * dim);
        else ml_copy4(dst + 2 * DP + ML_VC + c - 2 * dim - nv, gates + ((size_t)(first + row) * n_head + h) * 4 + c - 2 * dim - nv);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // what no copy writes (q and k beyond dim) stays zero
  for (int i = tid; i < 2 * ML_CHUNK * STAGE; i += ML_THREADS) (&stage[0][0][0])[i] = 0.0f;
  __syncthreads();
  pdl_wait();
  if (t0 >= t1) return;
  fetch(t0, 0);
  float4 S[NP];
#pragma unroll
  for (int p = 0; p < NP; ++p)
    S[p] = live && p * R + r < n4 ? reinterpret_cast<const float4*>(column)[p * R + r] : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int first = t0, buf = 0; first < t1; first += ML_CHUNK, buf ^= 1) {
    if (first + ML_CHUNK < t1) {
      fetch(first + ML_CHUNK, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();                                // the chunk is there for every thread
    const int rows = min(ML_CHUNK, t1 - first);
    // one row: the state's update and the row's numerator (or, in the column of n, its denominator)
    auto row = [&](int i) {
      const float* st = stage[buf][i];
      const float keep = st[2 * DP + ML_VC], take = st[2 * DP + ML_VC + 1];
      const float tv = take * (is_n ? 1.0f : st[2 * DP + (jc < ML_VC ? jc : 0)]);
      const float4* q4 = reinterpret_cast<const float4*>(st);
      const float4* k4 = reinterpret_cast<const float4*>(st + DP);
      float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);   // four chains, not one of 4 * NP links
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        const float4 q = q4[p * R + r], k = k4[p * R + r];
        S[p].x = fmaf(keep, S[p].x, tv * k.x);
        S[p].y = fmaf(keep, S[p].y, tv * k.y);
        S[p].z = fmaf(keep, S[p].z, tv * k.z);
        S[p].w = fmaf(keep, S[p].w, tv * k.w);
        a4.x = fmaf(S[p].x, q.x, a4.x);
        a4.y = fmaf(S[p].y, q.y, a4.y);
        a4.z = fmaf(S[p].z, q.z, a4.z);
        a4.w = fmaf(S[p].w, q.w, a4.w);
      }
      float acc = (a4.x + a4.y) + (a4.z + a4.w);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (R >= 4) acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (R >= 8) acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc *= q_scale;
      if (r == 0 && live) {
        if (is_n)
          den[(size_t)(first + i) * n_head + h] = fmaxf(fabsf(acc), st[2 * DP + ML_VC + 2]) + 1e-6f;
        else
          out_at[(size_t)(first + i - t0) * ld_num] = acc;
      }
    };
    if (rows == ML_CHUNK) {     // unrolled: a row's sums and stores overlap the next row's update (a fifth to a third
#pragma unroll                  // faster than the loop left rolled, measured side by side)
      for (int i = 0; i < ML_CHUNK; ++i) row(i);
    } else {
      for (int i = 0; i < rows; ++i) row(i);
    }
    __syncthreads();                                // before the chunk after next overwrites this one
  }
  if (live) {
#pragma unroll
    for (int p = 0; p < NP; ++p)
      if (p * R + r < n4) reinterpret_cast<float4*>(column)[p * R + r] = S[p];
  }
}

// out[t, h, :] = (num / den) over its root mean square, times the weight, times sigmoid(gate); a warp a (row, head)
template <typename T>
__global__ void __launch_bounds__(256)
mlstm_finish_kernel(const float* num, int ld_num, const float* den, const float* proj, int ld, int g_off,
                    const float* __restrict__ norm_w, float eps, T* out, int ldo, int n_head, int vdim, int n_rows) {
  pdl_trigger();
  const int wi = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();
  if (wi >= n_rows * n_head) return;
  const int t = wi / n_head, h = wi % n_head;
  const float inv = 1.0f / den[(size_t)t * n_head + h];
  const float* src = num + (size_t)t * ld_num + h * vdim;
  float sq = 0.0f;
  for (int j = lane; j < vdim; j += 32) {
    const float o = src[j] * inv;
    sq += o * o;
  }
  const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)vdim + eps);
  for (int j = lane; j < vdim; j += 32) {
    const int c = h * vdim + j;
    out[(size_t)t * ldo + c] = from_float<T>(src[j] * inv * rstd * norm_w[c] * ml_sigmoid(proj[(size_t)t * ld + g_off + c]));
  }
}

template <int NP, int R, int VC>
static cudaError_t launch_scan(dim3 grid, cudaStream_t stream, const float* proj, int ld, int q_off, int k_off, int v_off,
                               const float* gates, float* state, long long slot_stride, long long head_stride,
                               const int* entry_start, const int* entry_slot, int n_head, int dim, int vdim,
                               float q_scale, float* num, int ld_num, float* den) {
  int aligned = ((dim | vdim | ld | q_off | k_off | v_off) & 3) == 0 && (((uintptr_t)proj | (uintptr_t)gates) & 15) == 0;
  // (3: a block has a thread for every 16-byte piece of a row)
  if (aligned && 2 * dim + VC + 4 <= 4 * ml_threads(VC, R)) aligned = 3;
  grid.z = (vdim + VC - 1) / VC;
  if (grid.z > 65535) return cudaErrorInvalidValue;
  return launch_pdl(mlstm_scan_kernel<NP, R, VC>, grid, dim3(ml_threads(VC, R)), 0, stream, proj, ld, q_off, k_off, v_off, gates,
                    state, slot_stride, head_stride, entry_start, entry_slot, n_head, dim, vdim, q_scale, num, ld_num, den,
                    aligned, (dim + 15) / 16 * 16);
}

// Fewer value channels a block where 64 would leave most of the device idle (one prompt, a few heads).
template <int NP, int R>
static cudaError_t launch_scan_np(int n_entries, cudaStream_t stream, const float* proj, int ld, int q_off, int k_off,
                                  int v_off, const float* gates, float* state, long long slot_stride,
                                  long long head_stride, const int* entry_start, const int* entry_slot, int n_head,
                                  int dim, int vdim, float q_scale, float* num, int ld_num, float* den) {
  const dim3 grid(n_entries, n_head, 1);
  const long pairs = (long)n_entries * n_head;
#define NIB_ML_ARGS grid, stream, proj, ld, q_off, k_off, v_off, gates, state, slot_stride, head_stride, entry_start, \
                    entry_slot, n_head, dim, vdim, q_scale, num, ld_num, den
  if (pairs * ((vdim + 63) / 64) >= 120) return launch_scan<NP, R, 64>(NIB_ML_ARGS);
  if (pairs * ((vdim + 31) / 32) >= 120) return launch_scan<NP, R, 32>(NIB_ML_ARGS);
  return launch_scan<NP, R, 16>(NIB_ML_ARGS);
#undef NIB_ML_ARGS
}

}  // namespace nib

using namespace nib;

// Floats of state per head: nib_mlstm_state_floats(dim, vdim) (the slot holds n_head times that).
extern "C" long long nib_mlstm_state_floats(int dim, int vdim) {
  const long long dp = (dim + 15) / 16 * 16;
  return (long long)(vdim + 1) * dp + 4;
}

// proj [rows, ld] float: the projections q, k (n_head x dim each), v, g (n_head x vdim each) and the two gate
// logits (n_head each) at their column offsets.  gates [rows, n_head, 4], num [rows, ld_num >= n_head * vdim] and
// den [rows, n_head] are scratch.  out [rows, ldo] in `dtype` receives n_head * vdim values a row.
extern "C" int nib_mlstm(int dtype, const float* proj, int ld, int q_off, int k_off, int v_off, int g_off, int i_off,
                         int f_off, const float* bias_i, const float* bias_f, float cap, const float* norm_w,
                         float* state, const int* entry_start, const int* entry_slot, int n_entries, int n_rows,
                         int n_head, int dim, int vdim, float eps, float* gates, float* num, int ld_num, float* den,
                         void* out, int ldo, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0 || dim > 256 || vdim <= 0 || n_head <= 0 || n_head > 65535 || !(cap > 0.0f)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_entries > 0) {
    const long long head_stride = nib_mlstm_state_floats(dim, vdim), slot_stride = head_stride * n_head;
    launch_pdl(mlstm_gates_kernel, dim3(n_entries, n_head), dim3(ML_GATE_ROWS), 0, stream, proj, ld, i_off, f_off, bias_i,
               bias_f, cap, state, slot_stride, head_stride, entry_start, entry_slot, n_head, gates);
    const float q_scale = 1.0f / sqrtf((float)dim);
    cudaError_t err;
#define NIB_ML_CASE(NP, R)                                                                                             \
  err = launch_scan_np<NP, R>(n_entries, stream, proj, ld, q_off, k_off, v_off, gates, state, slot_stride, head_stride, \
                              entry_start, entry_slot, n_head, dim, vdim, q_scale, num, ld_num, den)
    const int pieces = (dim + 15) / 16 * 4;   // 16-byte pieces of a column; a thread's share: the next size that is built
    // (measured at 952 rows: columns of 96 floats 0.39 ms with four threads a column, 0.41 with eight, 0.51 with two;
    // columns of 256 floats 0.91 to 1.2 ms with four, 0.79 with eight)
    if (pieces <= 4) NIB_ML_CASE(1, 4);
    else if (pieces <= 8) NIB_ML_CASE(2, 4);
    else if (pieces <= 12) NIB_ML_CASE(3, 4);
    else if (pieces <= 16) NIB_ML_CASE(4, 4);
    else if (pieces <= 24) NIB_ML_CASE(6, 4);
    else if (pieces <= 32) NIB_ML_CASE(4, 8);
    else if (pieces <= 48) NIB_ML_CASE(6, 8);
    else NIB_ML_CASE(8, 8);
#undef NIB_ML_CASE
    if (err != cudaSuccess) return (int)err;
  }
  const dim3 fgrid((n_rows * n_head + 7) / 8);
  if (dtype == DT_F32)
    launch_pdl(mlstm_finish_kernel<float>, fgrid, dim3(256), 0, stream, num, ld_num, den, proj, ld, g_off, norm_w, eps,
               (float*)out, ldo, n_head, vdim, n_rows);
  else if (dtype == DT_BF16)
    launch_pdl(mlstm_finish_kernel<bf16>, fgrid, dim3(256), 0, stream, num, ld_num, den, proj, ld, g_off, norm_w, eps,
               (bf16*)out, ldo, n_head, vdim, n_rows);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
