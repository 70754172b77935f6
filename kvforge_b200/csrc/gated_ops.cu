// What a layer needs around its matrix products when every sublayer's result is gated, normed and only then
// added to the residual stream, and when queries and keys are rotated and then normed per head:
//
//   norm_step    : resid += norm_post(y * sigmoid(z + b)) ; out = norm_next(resid)   (one pass over a row)
//   qk_prepare   : rotation of split pairs, per-head RMS norm without a weight, keys and values to the cache
//   unary_act    : xIELU, squared ReLU or tanh-GELU on the rows of an inner activation
//
// All arithmetic is float whatever the storage type T; each result is rounded once.
#include "common.cuh"

using namespace kvf;

namespace {

// ---------------------------------------------------------------- gated post-norm, residual sum, next norm
struct NormStepParams {
  float* resid;            // [*, W] float residual stream
  const int* rows;         // output row r reads residual row rows[r] (nothing is written back then); null: r
  const void* y;           // pending sublayer result in the storage type [*, y_stride], or null
  const float* y_parts;    // ... or float slices [nsplit][*, W] that are summed in slice order, or null
  long long y_stride, split_stride;
  int nsplit;
  const void* z;           // gate logits in the storage type [*, z_stride] (the gate is sigmoid(z + z_bias)), or null
  long long z_stride;
  const float* z_bias;     // [W] or null
  const float* post_w;     // weight of the norm of the gated result, or null: the result is added as it is
  const float* next_w;     // weight of the norm whose rows go to `out`, or null: `out` gets the stream itself
  void* out;               // [*, out_stride] storage type, or null
  long long out_stride;
  int W;
  int centred;             // 1: layer norm (mean taken off, variance of the deviations); 0: RMS norm
  int store_normed;        // 1: the normed row also replaces the residual row (float)
  float eps;
};

// One statistic pass over `buf` (shared memory, W floats): returns (mean, 1 / sqrt(var + eps)); for an RMS
// norm the mean is zero and var the mean square.  Two passes over shared memory: the variance is the mean of
// the squared deviations from the mean that was taken first.
__device__ __forceinline__ void row_stats(const float* buf, int W, int centred, float eps, float* red, float& mean,
                                          float& rstd) {
  mean = 0.f;
  if (centred) {
    float s = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) s += buf[i];
    mean = block_sum(s, red) / (float)W;
  }
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = buf[i] - mean;
    q = fmaf(d, d, q);
  }
  rstd = 1.f / sqrtf(block_sum(q, red) / (float)W + eps);
}

template <typename T>
__global__ void __launch_bounds__(256) norm_step_kernel(const NormStepParams p) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float rowbuf[];  // 2 W floats
  __shared__ float red[32];
  const int W = p.W;
  float* u = rowbuf;
  float* v = rowbuf + W;
  const int r = blockIdx.x;
  const int src = p.rows ? p.rows[r] : r;
  float* h = p.resid + (size_t)src * W;
  const bool pending = p.y != nullptr || p.y_parts != nullptr;
  if (pending) {
    const T* y = p.y ? (const T*)p.y + (size_t)src * p.y_stride : nullptr;
    const float* yp = p.y_parts ? p.y_parts + (size_t)src * W : nullptr;
    const T* z = p.z ? (const T*)p.z + (size_t)src * p.z_stride : nullptr;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float a = 0.f;
      if (y) a = to_float<T>(y[i]);
      if (yp)
        for (int s = 0; s < p.nsplit; ++s) a += yp[(size_t)s * p.split_stride + i];
      if (z) {
        const float g = to_float<T>(z[i]) + (p.z_bias ? p.z_bias[i] : 0.f);
        a *= 1.f / (1.f + expf(-g));
      }
      u[i] = a;
    }
    __syncthreads();
    float mean = 0.f, rstd = 1.f;
    if (p.post_w) row_stats(u, W, p.centred, p.eps, red, mean, rstd);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float d = p.post_w ? (u[i] - mean) * rstd * p.post_w[i] : u[i];
      const float s = h[i] + d;
      v[i] = s;
      if (!p.rows && !p.store_normed) h[i] = s;
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) v[i] = h[i];
  }
  if (!p.out && !p.store_normed) return;
  __syncthreads();
  float mean = 0.f, rstd = 1.f;
  if (p.next_w) row_stats(v, W, p.centred, p.eps, red, mean, rstd);
  T* o = p.out ? (T*)p.out + (size_t)r * p.out_stride : nullptr;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float x = p.next_w ? (v[i] - mean) * rstd * p.next_w[i] : v[i];
    if (o) o[i] = from_float<T>(x);
    if (p.store_normed && !p.rows) h[i] = x;
  }
}

// The same pass for rows of up to 4 * 256 * NIT numbers whose rows start on 16-byte boundaries: a thread owns
// four neighbouring numbers of each of up to NIT quarters of the row and keeps them in registers; everything a
// row needs from memory is asked for before the first number is used.  The sums run in the same order whatever
// else is in the batch.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* src, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(src);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* dst, const float* f) {
    *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* src, float* f) {
    const uint2 u = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(bf16* dst, const float* f) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = u;
  }
};

template <int NIT>
__device__ __forceinline__ void reg_stats(const float (&x)[NIT][4], const bool (&live)[NIT], int W, int centred, float eps,
                                          float* red, float& mean, float& rstd) {
  mean = 0.f;
  if (centred) {
    float s = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; ++it)
      if (live[it]) s += (x[it][0] + x[it][1]) + (x[it][2] + x[it][3]);
    mean = block_sum(s, red) / (float)W;
  }
  float q = 0.f;
#pragma unroll
  for (int it = 0; it < NIT; ++it)
    if (live[it]) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d = x[it][e] - mean;
        q = fmaf(d, d, q);
      }
    }
  rstd = 1.f / sqrtf(block_sum(q, red) / (float)W + eps);
}

template <typename T, int NIT>
__global__ void __launch_bounds__(256) norm_step_vec_kernel(const NormStepParams p) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int W = p.W;
  const int r = blockIdx.x;
  const int src = p.rows ? p.rows[r] : r;
  float* h = p.resid + (size_t)src * W;
  const bool pending = p.y != nullptr || p.y_parts != nullptr;
  const T* y = p.y ? (const T*)p.y + (size_t)src * p.y_stride : nullptr;
  const float* yp = p.y_parts ? p.y_parts + (size_t)src * W : nullptr;
  const T* z = (pending && p.z) ? (const T*)p.z + (size_t)src * p.z_stride : nullptr;
  bool live[NIT];
  float hv[NIT][4], a[NIT][4], g[NIT][4], pw[NIT][4], nw[NIT][4];
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int i = (it * 256 + threadIdx.x) * 4;
    live[it] = i < W;
#pragma unroll
    for (int e = 0; e < 4; ++e) hv[it][e] = a[it][e] = g[it][e] = 0.f, pw[it][e] = nw[it][e] = 1.f;
    if (!live[it]) continue;
    Vec4<float>::load(h + i, hv[it]);
    if (p.next_w) Vec4<float>::load(p.next_w + i, nw[it]);
    if (!pending) continue;
    if (y) Vec4<T>::load(y + i, a[it]);
    if (z) {
      Vec4<T>::load(z + i, g[it]);
      if (p.z_bias) {
        float zb[4];
        Vec4<float>::load(p.z_bias + i, zb);
#pragma unroll
        for (int e = 0; e < 4; ++e) g[it][e] += zb[e];
      }
    }
    if (p.post_w) Vec4<float>::load(p.post_w + i, pw[it]);
  }
  if (yp) {
    for (int s = 0; s < p.nsplit; ++s) {
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        if (!live[it]) continue;
        float t[4];
        Vec4<float>::load(yp + (size_t)s * p.split_stride + (it * 256 + threadIdx.x) * 4, t);
#pragma unroll
        for (int e = 0; e < 4; ++e) a[it][e] += t[e];
      }
    }
  }
  if (pending) {
    if (z) {
#pragma unroll
      for (int it = 0; it < NIT; ++it)
#pragma unroll
        for (int e = 0; e < 4; ++e) a[it][e] *= 1.f / (1.f + expf(-g[it][e]));
    }
    float mean = 0.f, rstd = 1.f;
    if (p.post_w) reg_stats<NIT>(a, live, W, p.centred, p.eps, red, mean, rstd);
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
#pragma unroll
      for (int e = 0; e < 4; ++e) hv[it][e] += p.post_w ? (a[it][e] - mean) * rstd * pw[it][e] : a[it][e];
      if (live[it] && !p.rows && !p.store_normed) Vec4<float>::store(h + (it * 256 + threadIdx.x) * 4, hv[it]);
    }
  }
  if (!p.out && !p.store_normed) return;
  float mean = 0.f, rstd = 1.f;
  if (p.next_w) reg_stats<NIT>(hv, live, W, p.centred, p.eps, red, mean, rstd);
  T* o = p.out ? (T*)p.out + (size_t)r * p.out_stride : nullptr;
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    if (!live[it]) continue;
    const int i = (it * 256 + threadIdx.x) * 4;
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = p.next_w ? (hv[it][e] - mean) * rstd * nw[it][e] : hv[it][e];
    if (o) Vec4<T>::store(o + i, x);
    if (p.store_normed && !p.rows) Vec4<float>::store(h + i, x);
  }
}

template <typename T>
bool norm_step_vec_ok(const NormStepParams& p) {
  auto al = [](const void* q, size_t n) { return q == nullptr || ((uintptr_t)q % n) == 0; };
  constexpr size_t TB = 4 * sizeof(T);
  return p.W % 4 == 0 && p.W <= 4 * 256 * 4 && al(p.resid, 16) && al(p.y_parts, 16) && al(p.z_bias, 16) && al(p.post_w, 16) &&
         al(p.next_w, 16) && al(p.y, TB) && al(p.z, TB) && al(p.out, TB) && p.y_stride % 4 == 0 && p.z_stride % 4 == 0 &&
         p.out_stride % 4 == 0 && p.split_stride % 4 == 0;
}

// ---------------------------------------------------------------- rotation, head norm, cache write
// A row of `x` holds nh query heads of d numbers from column 0, nkv key heads of d from column k_off, and the
// value heads' sources from column v_off (v_step numbers apart, the first dv of each are the value; with
// v_off == k_off and v_step == d the values are the keys as projected, before rotation and norm).  A warp owns
// one (token, head).  The first `rot` dims turn in split pairs (i, i + rot/2) by the angle pos * inv_freq[i];
// then, with norm != 0, the head is divided by sqrt(mean(x^2) + eps).  Queries are written back in place; keys
// and values go to their slot of the paged cache ([blocks][nkv][block_size][d] and [...][dv]); a slot below
// zero (padding) is skipped, one beyond the pool raises bit 1 of the error flag.
constexpr int PREP_EPL = 8;  // elements a lane holds: heads up to 256 wide

template <typename T>
__global__ void __launch_bounds__(128) qk_prepare_kernel(T* __restrict__ x, long long row_stride, int k_off, int v_off,
                                                          int v_step, const int* __restrict__ positions,
                                                          const float* __restrict__ inv_freq, int rot, int norm, float eps,
                                                          const int* __restrict__ slots, T* __restrict__ kcache,
                                                          T* __restrict__ vcache, int n_tokens, int nh, int nkv, int d, int dv,
                                                          int block_size, long long num_slots, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int heads = nh + nkv;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)n_tokens * heads) return;
  const int n = (int)(unit / heads), h = (int)(unit - (long long)n * heads);
  const int lane = threadIdx.x & 31;
  T* row = x + (size_t)n * row_stride;
  const bool is_q = h < nh;
  const int g = h - nh;
  long long slot = -1;
  if (!is_q) {
    slot = slots ? slots[n] : -1;
    if (slot < 0) return;
    if (slot >= num_slots) {
      if (lane == 0 && err) atomicOr(err, 2);
      return;
    }
    const T* vsrc = row + v_off + (size_t)g * v_step;
    T* vdst = vcache + (((size_t)(slot / block_size) * nkv + g) * block_size + (size_t)(slot % block_size)) * dv;
    for (int j = lane; j < dv; j += 32) vdst[j] = vsrc[j];
  }
  T* src = is_q ? row + (size_t)h * d : row + k_off + (size_t)g * d;
  const float pos = (float)positions[n];
  const int half = rot >> 1;
  float val[PREP_EPL];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PREP_EPL; ++k) {
    const int e = lane + 32 * k;
    float y = 0.f;
    if (e < d) {
      const float a = to_float<T>(src[e]);
      y = a;
      if (e < rot) {
        const int i = e < half ? e : e - half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        float y1, y2;
        if (e < half) {
          rotate_pair(a, to_float<T>(src[e + half]), cs, sn, y1, y2);
          y = y1;
        } else {
          rotate_pair(to_float<T>(src[e - half]), a, cs, sn, y1, y2);
          y = y2;
        }
      }
      ss = fmaf(y, y, ss);
    }
    val[k] = y;
  }
  float r = 1.f;
  if (norm) r = 1.f / sqrtf(warp_sum(ss) / (float)d + eps);
  __syncwarp();
  T* dst = src;
  if (!is_q) dst = kcache + (((size_t)(slot / block_size) * nkv + g) * block_size + (size_t)(slot % block_size)) * d;
#pragma unroll
  for (int k = 0; k < PREP_EPL; ++k) {
    const int e = lane + 32 * k;
    if (e < d) dst[e] = from_float<T>(val[k] * r);
  }
}

// ---------------------------------------------------------------- activations of one input
// kind 0: xIELU with the two numbers (p, q) of `ab`: z > 0: softplus(p) z^2 + z/2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
// kind 1: relu(z)^2     kind 2: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__device__ __forceinline__ float unary_act(float z, int kind, float ap, float aq) {
  if (kind == 0) return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
  if (kind == 1) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256) unary_act_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out,
                                                         long long out_stride, long long rows, int cols, int kind,
                                                         const float* __restrict__ ab) {
  pdl_launch();
  pdl_wait();
  float ap = 0.f, aq = 0.f;
  if (kind == 0) {
    ap = softplus_f(ab[0]);
    aq = 0.5f + softplus_f(ab[1]);
  }
  const long long total = rows * cols;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / cols;
    const int c = (int)(idx - r * cols);
    out[r * out_stride + c] = from_float<T>(unary_act(to_float<T>(in[r * in_stride + c]), kind, ap, aq));
  }
}

unsigned grid_for(long long total) {
  long long g = (total + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return (unsigned)(g < 1 ? 1 : g);
}

}  // namespace

KVF_API int kvf_gated_set_pdl(int enabled) {
  g_pdl_enabled = enabled ? 1 : 0;
  return 0;
}

#define KVF_GATED_API(SUF, T)                                                                                          \
  KVF_API int kvf_norm_step_##SUF(float* resid, const int* rows, const void* y, const float* y_parts, long long y_stride, \
                                  long long split_stride, int nsplit, const void* z, long long z_stride,              \
                                  const float* z_bias, const float* post_w, const float* next_w, void* out,           \
                                  long long out_stride, int n_rows, int W, int centred, int store_normed, float eps,  \
                                  cudaStream_t st) {                                                                  \
    if (n_rows <= 0) return 0;                                                                                        \
    if (W <= 0 || (y && y_parts) || (store_normed && rows)) return (int)cudaErrorInvalidValue;                        \
    NormStepParams p;                                                                                                 \
    p.resid = resid; p.rows = rows; p.y = y; p.y_parts = y_parts; p.y_stride = y_stride; p.split_stride = split_stride; \
    p.nsplit = nsplit; p.z = z; p.z_stride = z_stride; p.z_bias = z_bias; p.post_w = post_w; p.next_w = next_w;       \
    p.out = out; p.out_stride = out_stride; p.W = W; p.centred = centred; p.store_normed = store_normed; p.eps = eps; \
    if (norm_step_vec_ok<T>(p)) {                                                                                     \
      if (W <= 1024) return launch(norm_step_vec_kernel<T, 1>, dim3(n_rows), dim3(256), 0, st, p);                    \
      if (W <= 2048) return launch(norm_step_vec_kernel<T, 2>, dim3(n_rows), dim3(256), 0, st, p);                    \
      return launch(norm_step_vec_kernel<T, 4>, dim3(n_rows), dim3(256), 0, st, p);                                   \
    }                                                                                                                 \
    const size_t smem = (size_t)2 * W * sizeof(float);                                                                \
    auto kern = norm_step_kernel<T>;                                                                                  \
    if (smem > 48 * 1024) {                                                                                           \
      if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;                                                       \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
      if (e != cudaSuccess) return (int)e;                                                                            \
    }                                                                                                                 \
    return launch(kern, dim3(n_rows), dim3(256), smem, st, p);                                                        \
  }                                                                                                                   \
  KVF_API int kvf_qk_prepare_##SUF(void* x, long long row_stride, int k_off, int v_off, int v_step, const int* positions, \
                                   const float* inv_freq, int rot, int norm, float eps, const int* slots, void* kcache, \
                                   void* vcache, int n_tokens, int nh, int nkv, int d, int dv, int block_size,        \
                                   long long num_slots, int* err, cudaStream_t st) {                                  \
    if (n_tokens <= 0) return 0;                                                                                      \
    if (d <= 0 || d > 32 * PREP_EPL || dv <= 0 || dv > v_step || rot < 0 || rot > d || (rot & 1) || nh < 0 || nkv < 0) \
      return (int)cudaErrorInvalidValue;                                                                              \
    const long long units = (long long)n_tokens * (nh + nkv);                                                         \
    return launch(qk_prepare_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, st, (T*)x, row_stride, k_off, \
                  v_off, v_step, positions, inv_freq, rot, norm, eps, slots, (T*)kcache, (T*)vcache, n_tokens, nh,    \
                  nkv, d, dv, block_size, num_slots, err);                                                            \
  }                                                                                                                   \
  KVF_API int kvf_unary_act_##SUF(const void* in, long long in_stride, void* out, long long out_stride, long long rows, \
                                  int cols, int kind, const float* ab, cudaStream_t st) {                             \
    if (rows <= 0 || cols <= 0) return 0;                                                                             \
    if (kind < 0 || kind > 2 || (kind == 0 && !ab)) return (int)cudaErrorInvalidValue;                                \
    return launch(unary_act_kernel<T>, dim3(grid_for(rows * cols)), dim3(256), 0, st, (const T*)in, in_stride, (T*)out, \
                  out_stride, rows, cols, kind, ab);                                                                  \
  }

KVF_GATED_API(f32, float)
KVF_GATED_API(bf16, bf16)
