// Attention through a low-rank latent: what a token leaves in the cache is one row
//   [ c (kv_rank values, RMS-normed) | k_rot (rot_dim values, rotated by the token's position) ]
// shared by all heads.  With W_uk and W_uv the per-head maps from the latent to keys and values,
//   score(h, i, j) = (q_nope[h,i] . W_uk[h] c_j + q_rot[h,i] . k_rot_j) * scale
//                  = ((W_uk[h]^T q_nope[h,i]) . c_j + q_rot[h,i] . k_rot_j) * scale,
//   out[h, i]      = W_uv[h] (sum_j p(h,i,j) c_j),
// so a head's query is carried into the latent space once ("absorbed": kv_rank + rot_dim numbers), every
// head attends over the same rows of the cache, and the weighted sum of latents is mapped to the head's
// values afterwards.  The two per-head maps are products of their own (linear_heads.cu).
//
//   latent_prep      : from the down-projections' output [c_q raw | c raw | k_rot raw] of a row:
//                      c_q = rmsnorm(.) * w_q  -> the up-projection's input;
//                      c = rmsnorm(.) * w_kv and k_rot rotated -> the row's slot of the paged latent cache
//   rope_heads       : rotates the rot part of every head's query and writes it behind the absorbed part
//   latent_attention : softmax attention of rows over the cache, causal, with an optional window
//                      (position i sees j with 0 <= i - j < window)
// Rotation: pairs (2i, 2i+1) of the first rot_dims values, angle = position * freq[i]; the angle and its
// sine and cosine are computed in double precision from a table of frequencies made on the host, the
// rest in 32-bit.  Scores, softmax and the weighted sums are 32-bit.
#include "api.h"
#include "common.cuh"

namespace nib {

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* proj, int ld, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                   const double* __restrict__ freqs, const float* __restrict__ wq, const float* __restrict__ wkv,
                   float eps, T* cq, int ld_cq, T* cache, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ row_entry, const int* __restrict__ positions, int page_size,
                   int n_pages, int has_kv, int* status) {
  pdl_trigger();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int entry = row_entry[t], pos = positions[t];
  pdl_wait();
  const float* src = proj + (size_t)t * ld;
  float s = 0.0f;
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) s += src[c] * src[c];
  const float rq = 1.0f / sqrtf(block_sum(s, scratch) / (float)q_rank + eps);
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
    cq[(size_t)t * ld_cq + c] = from_float<T>(src[c] * rq * wq[c]);
  if (!has_kv || entry < 0) return;    // a layer that reads another's cache; a row of no request
  const int page = block_table[(size_t)entry * max_blocks + pos / page_size];
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0) *status = NIB_STATUS_BAD_PAGE;
    return;
  }
  const float* kv = src + q_rank;
  s = 0.0f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) s += kv[c] * kv[c];
  const float rk = 1.0f / sqrtf(block_sum(s, scratch) / (float)kv_rank + eps);
  T* dst = cache + ((size_t)page * page_size + pos % page_size) * (size_t)(kv_rank + rot_dim);
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) dst[c] = from_float<T>(kv[c] * rk * wkv[c]);
  const float* kr = kv + kv_rank;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    double sn, cs;
    sincos((double)pos * freqs[i], &sn, &cs);
    const float u = kr[2 * i], v = kr[2 * i + 1], c = (float)cs, sf = (float)sn;
    dst[kv_rank + 2 * i] = from_float<T>(u * c - v * sf);
    dst[kv_rank + 2 * i + 1] = from_float<T>(v * c + u * sf);
  }
  for (int c = rot_dims + threadIdx.x; c < rot_dim; c += blockDim.x) dst[kv_rank + c] = from_float<T>(kr[c]);
}

// q: [T, H * (nope + rot_dim)] as the up-projection leaves it; out: float [T, H, out_dim], the rot part of
// head h goes to out[t, h, out_off ...].
template <typename T>
__global__ void __launch_bounds__(128)
rope_heads_kernel(const T* q, int ldq, int nope, int rot_dim, int rot_dims, const double* __restrict__ freqs,
                  const int* __restrict__ positions, float* out, int out_dim, int out_off, int n_head) {
  pdl_trigger();
  extern __shared__ float cs[];   // cos, sin per pair
  const int t = blockIdx.x, half = rot_dims / 2;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, c;
    sincos((double)pos * freqs[i], &sn, &c);
    cs[2 * i] = (float)c;
    cs[2 * i + 1] = (float)sn;
  }
  __syncthreads();
  pdl_wait();
  const int per_head = half + (rot_dim - rot_dims);
  for (int w = threadIdx.x; w < n_head * per_head; w += blockDim.x) {
    const int h = w / per_head, i = w % per_head;
    const T* src = q + (size_t)t * ldq + (size_t)h * (nope + rot_dim) + nope;
    float* dst = out + ((size_t)t * n_head + h) * out_dim + out_off;
    if (i < half) {
      const float u = to_float(src[2 * i]), v = to_float(src[2 * i + 1]), c = cs[2 * i], s = cs[2 * i + 1];
      dst[2 * i] = u * c - v * s;
      dst[2 * i + 1] = v * c + u * s;
    } else {
      const int d = rot_dims + (i - half);
      dst[d] = to_float(src[d]);
    }
  }
}

constexpr int LA_WARPS = 8;     // heads a block takes, one a warp
constexpr int LA_TILE = 32;     // keys a tile, one a lane

// One block per (row, group of LA_WARPS heads).  A tile of 32 keys is brought into shared memory as
// floats (row stride odd: a lane reads its own key's row without bank conflicts), lane j of a warp makes
// the score of key j for the warp's head, the tile's maximum and sum come from warp reductions, and for
// the weighted sum lane l owns the latent's elements l, l + 32, ...
template <typename T, int NACC>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const float* q, const T* cache, T* out, int ldo, const int* __restrict__ block_table,
                        int max_blocks, const int* __restrict__ rows, const int* __restrict__ row_entry,
                        const int* __restrict__ positions, int n_head, int kv_rank, int D, int page_size,
                        int n_pages, float scale, int window, int* status, int n_splits, float* partials) {
  pdl_trigger();
  extern __shared__ float smem[];
  const int Dp = D | 1;
  float* ktile = smem;                          // [LA_TILE][Dp]
  float* qs = smem + LA_TILE * Dp;              // [LA_WARPS][D]
  __shared__ int key_page[LA_TILE];
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  const int entry = row_entry[t];
  if (entry < 0) return;                        // a row of no request
  const int pos = positions[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * LA_WARPS + warp;
  const bool live = h < n_head;
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  int hi = pos;
  if (n_splits > 1) {
    // the row's own key range cut into n_splits equal pieces of whole tiles; this block takes piece blockIdx.z
    const int per = ((pos - lo + n_splits) / n_splits + LA_TILE - 1) / LA_TILE * LA_TILE;
    lo += blockIdx.z * per;
    hi = min(pos, lo + per - 1);
  }
  pdl_wait();
  if (live) {
    const float* src = q + ((size_t)t * n_head + h) * D;
    for (int d = lane; d < D; d += 32) qs[warp * D + d] = src[d];
  }
  float m = -INFINITY, l = 0.0f, acc[NACC];
#pragma unroll
  for (int k = 0; k < NACC; ++k) acc[k] = 0.0f;
  for (int j0 = lo; j0 <= hi; j0 += LA_TILE) {
    __syncthreads();                            // the tile before is done with
    if (threadIdx.x < LA_TILE) {
      const int j = j0 + threadIdx.x;
      int page = -1;
      if (j <= hi) {
        page = block_table[(size_t)entry * max_blocks + j / page_size];
        if (page < 0 || page >= n_pages) {
          *status = NIB_STATUS_BAD_PAGE;
          page = -1;
        }
      }
      key_page[threadIdx.x] = page;
    }
    __syncthreads();
    // every warp brings in its share of the tile's keys, a lane an element: rows of the cache as they lie
#pragma unroll
    for (int i = 0; i < LA_TILE / LA_WARPS; ++i) {
      const int jj = warp * (LA_TILE / LA_WARPS) + i;
      const int page = key_page[jj];
      float* dst = ktile + jj * Dp;
      if (page >= 0) {
        const T* srck = cache + ((size_t)page * page_size + (j0 + jj) % page_size) * (size_t)D;
        for (int d = lane; d < D; d += 32) dst[d] = to_float(srck[d]);
      } else {
        for (int d = lane; d < D; d += 32) dst[d] = 0.0f;
      }
    }
    __syncthreads();
    if (live) {
      const float* kr = ktile + lane * Dp;
      const float* qh = qs + warp * D;
      float s = 0.0f;
      for (int d = 0; d < D; ++d) s += qh[d] * kr[d];
      s = (j0 + lane <= hi && key_page[lane] >= 0) ? s * scale : -INFINITY;
      const float m_new = fmaxf(m, warp_max(s));
      const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
      const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int k = 0; k < NACC; ++k) acc[k] *= corr;
      const int n_keys = min(LA_TILE, hi - j0 + 1);
      for (int jj = 0; jj < n_keys; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const float* row = ktile + jj * Dp;
#pragma unroll
        for (int k = 0; k < NACC; ++k) {
          const int d = lane + 32 * k;
          if (d < kv_rank) acc[k] += pj * row[d];
        }
      }
      m = m_new;
    }
  }
  if (live && n_splits > 1) {
    // (maximum, sum, unscaled weighted sum) of this piece: the merge kernel puts the pieces together
    float* dst = partials + (((size_t)t * n_head + h) * n_splits + blockIdx.z) * (size_t)(kv_rank + 2);
    if (lane == 0) {
      dst[0] = m;
      dst[1] = l;
    }
#pragma unroll
    for (int k = 0; k < NACC; ++k) {
      const int d = lane + 32 * k;
      if (d < kv_rank) dst[2 + d] = acc[k];
    }
  } else if (live) {
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    T* o = out + (size_t)t * ldo + (size_t)h * kv_rank;
#pragma unroll
    for (int k = 0; k < NACC; ++k) {
      const int d = lane + 32 * k;
      if (d < kv_rank) o[d] = from_float<T>(acc[k] * inv);
    }
  }
}

// One block per (row, head): the pieces of a row's keys, each with its own maximum, put together in the
// order of the pieces.
template <typename T>
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* partials, T* out, int ldo, const int* __restrict__ rows,
                    const int* __restrict__ row_entry, int n_head, int kv_rank, int n_splits) {
  pdl_trigger();
  const int t = rows ? rows[blockIdx.x] : blockIdx.x, h = blockIdx.y;
  if (row_entry[t] < 0) return;
  pdl_wait();
  const float* src = partials + ((size_t)t * n_head + h) * n_splits * (size_t)(kv_rank + 2);
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, src[(size_t)s * (kv_rank + 2)]);
  float l = 0.0f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = src[(size_t)s * (kv_rank + 2)];
    if (ms != -INFINITY) l += src[(size_t)s * (kv_rank + 2) + 1] * expf(ms - m);
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
    float a = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = src[(size_t)s * (kv_rank + 2)];
      if (ms != -INFINITY) a += src[(size_t)s * (kv_rank + 2) + 2 + d] * expf(ms - m);
    }
    out[(size_t)t * ldo + (size_t)h * kv_rank + d] = from_float<T>(a * inv);
  }
}

template <typename T, int NACC>
static int launch_latent_attention(const float* q, const T* cache, T* out, int ldo, const int* block_table,
                                   int max_blocks, const int* rows, const int* row_entry, const int* positions,
                                   int n_rows, int n_head, int kv_rank, int D, int page_size, int n_pages,
                                   float scale, int window, int* status, int n_splits, float* partials,
                                   cudaStream_t stream) {
  const size_t smem = ((size_t)LA_TILE * (D | 1) + (size_t)LA_WARPS * D) * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_kernel<T, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(latent_attention_kernel<T, NACC>, dim3(n_rows, (n_head + LA_WARPS - 1) / LA_WARPS, n_splits),
             dim3(LA_WARPS * 32), smem, stream, q, cache, out, ldo, block_table, max_blocks, rows, row_entry, positions,
             n_head, kv_rank, D, page_size, n_pages, scale, window, status, n_splits, partials);
  if (n_splits > 1)
    launch_pdl(latent_merge_kernel<T>, dim3(n_rows, n_head), dim3(128), 0, stream, (const float*)partials, out, ldo,
               rows, row_entry, n_head, kv_rank, n_splits);
  NIB_LAUNCH_CHECK();
}

template <typename T>
static int pick_latent_attention(const float* q, const void* cache, void* out, int ldo, const int* block_table,
                                 int max_blocks, const int* rows, const int* row_entry, const int* positions,
                                 int n_rows, int n_head, int kv_rank, int D, int page_size, int n_pages,
                                 float scale, int window, int* status, int n_splits, float* partials,
                                 cudaStream_t stream) {
#define NIB_LA(N)                                                                                              \
  return launch_latent_attention<T, N>(q, (const T*)cache, (T*)out, ldo, block_table, max_blocks, rows,       \
                                       row_entry, positions, n_rows, n_head, kv_rank, D, page_size, n_pages,  \
                                       scale, window, status, n_splits, partials, stream)
  const int n = (kv_rank + 31) / 32;
  if (n <= 2) NIB_LA(2);
  if (n <= 4) NIB_LA(4);
  if (n <= 8) NIB_LA(8);
  if (n <= 16) NIB_LA(16);
  if (n <= 32) NIB_LA(32);
#undef NIB_LA
  return NIB_ERR_UNSUPPORTED_SIZE;
}

}  // namespace nib

using namespace nib;

extern "C" int nib_latent_prep(int dtype, const float* proj, int ld, int q_rank, int kv_rank, int rot_dim,
                               int rot_dims, const double* freqs, const float* wq, const float* wkv, float eps,
                               void* cq, int ld_cq, void* cache, const int* block_table, int max_blocks,
                               const int* row_entry, const int* positions, int T, int page_size, int n_pages,
                               int has_kv, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank <= 0 || (has_kv && (kv_rank <= 0 || rot_dim < 0 || rot_dims > rot_dim || (rot_dims & 1))))
    return NIB_ERR_BAD_ARGUMENT;
  if (dtype == DT_F32)
    launch_pdl(latent_prep_kernel<float>, dim3(T), dim3(128), 0, stream, proj, ld, q_rank, kv_rank, rot_dim, rot_dims,
               freqs, wq, wkv, eps, (float*)cq, ld_cq, (float*)cache, block_table, max_blocks, row_entry, positions,
               page_size, n_pages, has_kv, status);
  else if (dtype == DT_BF16)
    launch_pdl(latent_prep_kernel<bf16>, dim3(T), dim3(128), 0, stream, proj, ld, q_rank, kv_rank, rot_dim, rot_dims,
               freqs, wq, wkv, eps, (bf16*)cq, ld_cq, (bf16*)cache, block_table, max_blocks, row_entry, positions,
               page_size, n_pages, has_kv, status);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_rope_heads(int dtype, const void* q, int ldq, int nope, int rot_dim, int rot_dims,
                              const double* freqs, const int* positions, float* out, int out_dim, int out_off,
                              int n_head, int T, cudaStream_t stream) {
  if (T <= 0 || rot_dim <= 0) return 0;
  if (rot_dims > rot_dim || (rot_dims & 1)) return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)(rot_dims + 2) * sizeof(float);
  if (dtype == DT_F32)
    launch_pdl(rope_heads_kernel<float>, dim3(T), dim3(128), smem, stream, (const float*)q, ldq, nope, rot_dim,
               rot_dims, freqs, positions, out, out_dim, out_off, n_head);
  else if (dtype == DT_BF16)
    launch_pdl(rope_heads_kernel<bf16>, dim3(T), dim3(128), smem, stream, (const bf16*)q, ldq, nope, rot_dim,
               rot_dims, freqs, positions, out, out_dim, out_off, n_head);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

// q: float [T, n_head, D] (absorbed part, then the rotated part), D = kv_rank + rot_dim; cache: one layer
// [n_pages, page_size, D]; out: [T, n_head * kv_rank] in the cache's dtype.  rows: the step's rows to
// process (nullptr: rows 0..n_rows-1).  n_splits > 1: every row's keys are cut into that many pieces, each a
// block of its own, and merged through `partials` (n_rows * n_head * n_splits * (kv_rank + 2) floats).
extern "C" int nib_latent_attention(int dtype, const float* q, const void* cache, void* out, int ldo,
                                    const int* block_table, int max_blocks, const int* rows, const int* row_entry,
                                    const int* positions, int n_rows, int n_head, int kv_rank, int D,
                                    int page_size, int n_pages, float scale, int window, int* status, int n_splits,
                                    float* partials, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (kv_rank <= 0 || D < kv_rank || n_head <= 0) return NIB_ERR_BAD_ARGUMENT;
  if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && partials == nullptr)) return NIB_ERR_BAD_ARGUMENT;
  if (dtype == DT_F32)
    return pick_latent_attention<float>(q, cache, out, ldo, block_table, max_blocks, rows, row_entry, positions,
                                        n_rows, n_head, kv_rank, D, page_size, n_pages, scale, window, status,
                                        n_splits, partials, stream);
  if (dtype == DT_BF16)
    return pick_latent_attention<bf16>(q, cache, out, ldo, block_table, max_blocks, rows, row_entry, positions,
                                       n_rows, n_head, kv_rank, D, page_size, n_pages, scale, window, status,
                                       n_splits, partials, stream);
  return NIB_ERR_BAD_ARGUMENT;
}
