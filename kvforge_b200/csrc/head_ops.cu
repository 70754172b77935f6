// What lies between an attention layer's input product and its attention kernel when queries and
// keys are normed per head, or when keys and values are made from one small latent per token;
// a logistic gate per head on an attention layer's output; a row added to every row of the
// residual stream.  All arithmetic is float whatever the storage type T; each result is rounded once.
#include "common.cuh"

using namespace kvf;

namespace {

// ---------------------------------------------------------------- per-head norm, rotation, cache write
// Rows of `qkv` hold nh query heads and nkv key heads of dk and nkv value heads of dv.  A warp owns
// one (token, head).  Query and key heads: x <- x / sqrt(mean(x^2) + eps) * w (w of dk floats shared
// by all heads; skipped without w), then the first `rot` dims turn by the angle pos * inv_freq[i], in
// interleaved pairs (2i, 2i+1) or, with split_pairs, in pairs (i, i + rot/2) (skipped when rot == 0).
// Queries are written back in place; keys and values go to their slot of the paged cache
// ([blocks][nkv][block_size][dk] and [...][dv]); a slot below zero (padding) is skipped, one beyond the
// pool raises bit 1 of the error flag.  Values may be mixed with those that an earlier layer of the same
// step left for the same token: with v_keep the values as projected are also copied to v_keep[n][nkv*dv];
// with v_first the value becomes (1 - lambda) v + lambda v_first[n] (lambda = *v_lambda, in float, rounded
// once) before it is cached.
template <typename T>
__global__ void __launch_bounds__(128) head_norm_cache_kernel(T* __restrict__ qkv, long long row_stride,
                                                               const int* __restrict__ positions,
                                                               const float* __restrict__ q_w, const float* __restrict__ k_w,
                                                               float eps, const float* __restrict__ inv_freq, int rot,
                                                               const int* __restrict__ slots, T* __restrict__ kcache,
                                                               T* __restrict__ vcache, int n_tokens, int nh, int nkv, int dk,
                                                               int dv, int block_size, long long num_slots,
                                                               int* __restrict__ err, int split_pairs,
                                                               T* __restrict__ v_keep, const T* __restrict__ v_first,
                                                               const float* __restrict__ v_lambda) {
  pdl_launch();
  pdl_wait();
  const int heads = nh + 2 * nkv;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)n_tokens * heads) return;
  const int n = (int)(unit / heads), h = (int)(unit - (long long)n * heads);
  const int lane = threadIdx.x & 31;
  T* row = qkv + (size_t)n * row_stride;
  const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
  long long slot = -1;
  if (!is_q) {
    slot = slots ? slots[n] : -1;
    if (slot < 0 && !is_k && v_keep) {  // a row without a slot still leaves its values for the layers after
      const int g = h - nh - nkv;
      const T* src = row + (size_t)(nh + nkv) * dk + (size_t)g * dv;
      for (int j = lane; j < dv; j += 32) v_keep[(size_t)n * nkv * dv + (size_t)g * dv + j] = src[j];
    }
    if (slot < 0) return;
    if (slot >= num_slots) {
      if (lane == 0 && err) atomicOr(err, 2);
      return;
    }
  }
  if (!is_q && !is_k) {  // a value head: copied as it is
    const int g = h - nh - nkv;
    const T* src = row + (size_t)(nh + nkv) * dk + (size_t)g * dv;
    T* dst = vcache + (((size_t)(slot / block_size) * nkv + g) * block_size + (size_t)(slot % block_size)) * dv;
    if (v_first) {
      const float lam = v_lambda[0];
      const T* first = v_first + (size_t)n * nkv * dv + (size_t)g * dv;
      for (int j = lane; j < dv; j += 32) dst[j] = from_float<T>(fmaf(lam, to_float<T>(first[j]), (1.f - lam) * to_float<T>(src[j])));
    } else {
      for (int j = lane; j < dv; j += 32) dst[j] = src[j];
    }
    if (v_keep)
      for (int j = lane; j < dv; j += 32) v_keep[(size_t)n * nkv * dv + (size_t)g * dv + j] = src[j];
    return;
  }
  T* x = row + (size_t)h * dk;  // key heads follow the query heads with the same size
  const float* w = is_q ? q_w : k_w;
  if (is_q && !w && rot == 0) return;
  float ss = 0.f;
  if (w) {
    for (int j = lane; j < dk; j += 32) {
      const float v = to_float<T>(x[j]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
  }
  const float r = w ? 1.f / sqrtf(ss / (float)dk + eps) : 1.f;
  const float pos = (float)positions[n];
  T* dst = x;
  if (is_k) {
    const int g = h - nh;
    dst = kcache + (((size_t)(slot / block_size) * nkv + g) * block_size + (size_t)(slot % block_size)) * dk;
  }
  for (int i = lane; i < dk / 2; i += 32) {
    // pair i: dims (2i, 2i+1), or (i, i + rot/2) among the dims that turn in split pairs
    const bool turns = 2 * i < rot;
    const int ia = (turns && split_pairs) ? i : 2 * i, ib = (turns && split_pairs) ? i + rot / 2 : 2 * i + 1;
    float a = to_float<T>(x[ia]), b = to_float<T>(x[ib]);
    if (w) {
      a = a * r * w[ia];
      b = b * r * w[ib];
    }
    if (turns) {
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      float ya, yb;
      rotate_pair(a, b, cs, sn, ya, yb);
      a = ya;
      b = yb;
    }
    dst[ia] = from_float<T>(a);
    dst[ib] = from_float<T>(b);
  }
}

// ---------------------------------------------------------------- RMS norm of a column range
// out[n][:] = x[n][0 .. r) / sqrt(mean(x^2) + eps) * w, a warp per row; x rows may be part of wider rows.
template <typename T>
__global__ void __launch_bounds__(128) row_rmsnorm_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
                                                           float eps, long long n_rows, int r, T* __restrict__ out, long long out_stride) {
  pdl_launch();
  pdl_wait();
  const long long n = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (n >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const T* row = x + (size_t)n * x_stride;
  float ss = 0.f;
  for (int j = lane; j < r; j += 32) {
    const float v = to_float<T>(row[j]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)r + eps);
  T* dst = out + (size_t)n * out_stride;
  for (int j = lane; j < r; j += 32) dst[j] = from_float<T>(to_float<T>(row[j]) * inv * w[j]);
}

// ---------------------------------------------------------------- latent keys and values
// A row of `x` holds, from column q_off, nh query heads of dk + dr numbers (the last dr of each turn
// with the position) and, from column c_off, a latent of r numbers followed by dr numbers of a key
// part that turns and is shared by all heads.  Per token, one CTA:
//   c = latent / sqrt(mean(latent^2) + eps) * c_w  -> cache row [0, r)
//   the shared key part, turned                     -> cache row [r, r + dr)
//   every head's turning query part, turned         -> qa[n][h][r .. r + dr)
// (qa rows hold nh heads of r + dr; their first r numbers are written by whoever folds the key
// up-projection into the queries).  Pairs are interleaved (2i, 2i+1), i < rot/2, rot <= dr, or with
// split_pairs (i, i + rot/2); angles pos * inv_freq[i].  The cache is [blocks][1][block_size][r + dr].
// The query heads may lie in rows of their own (`xq`, row stride q_stride; null: in `x` from q_off).
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const T* __restrict__ x, long long row_stride, int q_off,
                                                              int c_off, const int* __restrict__ positions,
                                                              const float* __restrict__ c_w, float eps,
                                                              const float* __restrict__ inv_freq, int rot,
                                                              const int* __restrict__ slots, T* __restrict__ cache,
                                                              T* __restrict__ qa, int nh, int dk, int dr, int r,
                                                              int block_size, long long num_slots, int* __restrict__ err,
                                                              int split_pairs, const T* __restrict__ xq, long long q_stride) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int n = blockIdx.x;
  const T* row = x + (size_t)n * row_stride;
  const T* qsrc = xq ? xq + (size_t)n * q_stride : row + q_off;
  const float pos = (float)positions[n];
  // queries: every head's turning part
  T* qrow = qa + (size_t)n * nh * (r + dr);
  for (int idx = threadIdx.x; idx < nh * (dr / 2); idx += blockDim.x) {
    const int h = idx / (dr / 2), i = idx - h * (dr / 2);
    const T* src = qsrc + (size_t)h * (dk + dr) + dk;
    const bool split = split_pairs && 2 * i < rot;
    const int ia = split ? i : 2 * i, ib = split ? i + rot / 2 : 2 * i + 1;
    float a = to_float<T>(src[ia]), b = to_float<T>(src[ib]);
    if (2 * i < rot) {
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      float ya, yb;
      rotate_pair(a, b, cs, sn, ya, yb);
      a = ya;
      b = yb;
    }
    T* dst = qrow + (size_t)h * (r + dr) + r;
    dst[ia] = from_float<T>(a);
    dst[ib] = from_float<T>(b);
  }
  const long long slot = slots ? slots[n] : -1;  // uniform over the CTA
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && err) atomicOr(err, 2);
    return;
  }
  const T* lat = row + c_off;
  float ss = 0.f;
  for (int j = threadIdx.x; j < r; j += blockDim.x) {
    const float v = to_float<T>(lat[j]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)r + eps);
  T* dst = cache + (size_t)slot * (r + dr);  // one key head: a slot is a row
  for (int j = threadIdx.x; j < r; j += blockDim.x) dst[j] = from_float<T>(to_float<T>(lat[j]) * inv * c_w[j]);
  for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
    const bool split = split_pairs && 2 * i < rot;
    const int ia = split ? i : 2 * i, ib = split ? i + rot / 2 : 2 * i + 1;
    float a = to_float<T>(lat[r + ia]), b = to_float<T>(lat[r + ib]);
    if (2 * i < rot) {
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      float ya, yb;
      rotate_pair(a, b, cs, sn, ya, yb);
      a = ya;
      b = yb;
    }
    dst[r + ia] = from_float<T>(a);
    dst[r + ib] = from_float<T>(b);
  }
}

// ---------------------------------------------------------------- a logistic gate per head
// y[n][h][:] *= 1 / (1 + exp(-g[n][h])), in place; g is a column range of a wider row.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ y, const T* __restrict__ g, long long g_stride, long long total, int nh,
                                 int dv) {
  pdl_launch();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long nhid = idx / dv;
    const long long n = nhid / nh;
    const int h = (int)(nhid - n * nh);
    const float z = to_float<T>(g[(size_t)n * g_stride + h]);
    y[idx] = from_float<T>(to_float<T>(y[idx]) * (1.f / (1.f + expf(-z))));
  }
}

// ---------------------------------------------------------------- a row added to every row
__global__ void add_row_kernel(float* __restrict__ resid, const float* __restrict__ vec, long long total, int width) {
  pdl_launch();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x)
    resid[idx] += vec[idx % width];
}

inline unsigned grid_for(long long total, int threads) {
  long long g = (total + threads - 1) / threads;
  return (unsigned)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace

#define KVF_HEAD_OPS_API(SUF, T)                                                                                     \
  KVF_API int kvf_head_norm_cache_##SUF(void* qkv, long long row_stride, const int* positions, const float* q_w,     \
                                        const float* k_w, float eps, const float* inv_freq, int rot,                 \
                                        const int* slots, void* kcache, void* vcache, int n_tokens, int nh, int nkv, \
                                        int dk, int dv, int block_size, long long num_slots, int* err,               \
                                        int split_pairs, void* v_keep, const void* v_first, const float* v_lambda,   \
                                        cudaStream_t st) {                                                           \
    if (n_tokens <= 0) return 0;                                                                                     \
    if (dk <= 0 || (dk & 1) || rot < 0 || rot > dk || (rot & 1)) return (int)cudaErrorInvalidValue;                  \
    if (v_first && !v_lambda) return (int)cudaErrorInvalidValue;                                                     \
    const long long units = (long long)n_tokens * (nh + 2 * nkv);                                                    \
    return launch(head_norm_cache_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, st, (T*)qkv,           \
                  row_stride, positions, q_w, k_w, eps, inv_freq, rot, slots, (T*)kcache, (T*)vcache, n_tokens, nh,  \
                  nkv, dk, dv, block_size, num_slots, err, split_pairs, (T*)v_keep, (const T*)v_first, v_lambda);    \
  }                                                                                                                  \
  KVF_API int kvf_row_rmsnorm_##SUF(const void* x, long long x_stride, const float* w, float eps, long long n_rows,  \
                                    int r, void* out, long long out_stride, cudaStream_t st) {                       \
    if (n_rows <= 0) return 0;                                                                                       \
    if (r <= 0 || !w) return (int)cudaErrorInvalidValue;                                                             \
    return launch(row_rmsnorm_kernel<T>, dim3((unsigned)((n_rows + 3) / 4)), dim3(128), 0, st, (const T*)x,          \
                  x_stride, w, eps, n_rows, r, (T*)out, out_stride);                                                 \
  }                                                                                                                  \
  KVF_API int kvf_latent_prepare_##SUF(const void* x, long long row_stride, int q_off, int c_off,                    \
                                       const int* positions, const float* c_w, float eps, const float* inv_freq,     \
                                       int rot, const int* slots, void* cache, void* qa, int n_tokens, int nh,       \
                                       int dk, int dr, int r, int block_size, long long num_slots, int* err,         \
                                       int split_pairs, const void* xq, long long q_stride, cudaStream_t st) {       \
    if (n_tokens <= 0) return 0;                                                                                     \
    if (r <= 0 || dr < 0 || (dr & 1) || rot < 0 || rot > dr || (rot & 1)) return (int)cudaErrorInvalidValue;         \
    return launch(latent_prepare_kernel<T>, dim3(n_tokens), dim3(128), 0, st, (const T*)x, row_stride, q_off,        \
                  c_off, positions, c_w, eps, inv_freq, rot, slots, (T*)cache, (T*)qa, nh, dk, dr, r, block_size,    \
                  num_slots, err, split_pairs, (const T*)xq, q_stride);                                              \
  }                                                                                                                  \
  KVF_API int kvf_head_gate_##SUF(void* y, const void* g, long long g_stride, long long n_tokens, int nh, int dv,    \
                                  cudaStream_t st) {                                                                 \
    const long long total = n_tokens * nh * dv;                                                                      \
    if (total <= 0) return 0;                                                                                        \
    return launch(head_gate_kernel<T>, dim3(grid_for(total, 256)), dim3(256), 0, st, (T*)y, (const T*)g, g_stride,   \
                  total, nh, dv);                                                                                    \
  }

KVF_HEAD_OPS_API(f32, float)
KVF_HEAD_OPS_API(bf16, bf16)

KVF_API int kvf_add_row_f32(float* resid, const float* vec, long long n_rows, int width, cudaStream_t st) {
  const long long total = n_rows * width;
  if (total <= 0) return 0;
  return launch(add_row_kernel, dim3(grid_for(total, 256)), dim3(256), 0, st, resid, vec, total, width);
}

// Turn programmatic dependent launch on or off for every launch of this library (the flag is one per
// shared library).
KVF_API int kvf_routed_set_pdl(int enabled) {
  kvf::g_pdl_enabled = enabled ? 1 : 0;
  return 0;
}
