// A norm without statistics fused with the residual sum:  v = resid + mult * pending,
// out = T(tanh(alpha * v) * w + b), with a learned scalar alpha and vectors w and b.  Nothing is summed
// over a row, so the kernel is elementwise: four neighbouring numbers a thread where rows allow it.
// `pending` is a tensor in the storage type T or the float slices of a split product (summed in slice
// order); `mult` scales what joins the stream.  Without `rows` the sum is written back into resid; with
// `rows` (int32 [R]) output row r comes from row rows[r] and resid is left as it is.  All arithmetic is
// float whatever T; the result is rounded once.
#include "common.cuh"

using namespace kvf;

namespace {

// V numbers that lie side by side, as floats; V == 4 takes one aligned load (rows are multiples of four numbers wide)
template <int V>
__device__ __forceinline__ void load_floats(const float* src, float* dst) {
  if (V == 4) {
    const float4 t = *reinterpret_cast<const float4*>(src);
    dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
  } else {
    dst[0] = src[0];
  }
}
template <int V>
__device__ __forceinline__ void load_floats(const bf16* src, float* dst) {
  if (V == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(src);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
  } else {
    dst[0] = __bfloat162float(src[0]);
  }
}
template <int V>
__device__ __forceinline__ void store_floats(float* dst, const float* v) {
  if (V == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  else dst[0] = v[0];
}
template <int V>
__device__ __forceinline__ void store_floats(bf16* dst, const float* v) {
  if (V == 4) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = t;
  } else {
    dst[0] = __float2bfloat16_rn(v[0]);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) tanh_norm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                                         const float* __restrict__ partials, int nsplit, long long split_stride,
                                                         float mult, const float* __restrict__ alpha, const float* __restrict__ w,
                                                         const float* __restrict__ b, T* __restrict__ out,
                                                         const int* __restrict__ rows, long long n_rows, int W) {
  pdl_launch();
  pdl_wait();
  const float al = alpha[0];
  const int per_row = W / V;
  const long long total = n_rows * per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / per_row;
    const int c = (int)(idx - r * per_row) * V;
    const long long src = rows ? (long long)rows[r] : r;
    float v[V];
    load_floats<V>(resid + (size_t)src * W + c, v);
    if (delta || nsplit > 0) {
      float d[V];
#pragma unroll
      for (int i = 0; i < V; ++i) d[i] = 0.f;
      if (delta) load_floats<V>(delta + (size_t)src * W + c, d);
      for (int s = 0; s < nsplit; ++s) {
        float t[V];
        load_floats<V>(partials + (size_t)s * split_stride + (size_t)src * W + c, t);
#pragma unroll
        for (int i = 0; i < V; ++i) d[i] += t[i];
      }
#pragma unroll
      for (int i = 0; i < V; ++i) v[i] = fmaf(mult, d[i], v[i]);
      if (!rows) store_floats<V>(resid + (size_t)src * W + c, v);
    }
    if (out) {
      float y[V];
#pragma unroll
      for (int i = 0; i < V; ++i) y[i] = fmaf(tanhf(al * v[i]), w[c + i], b[c + i]);
      store_floats<V>(out + (size_t)r * W + c, y);
    }
  }
}

}  // namespace

#define KVF_TANH_NORM_API(SUF, T)                                                                                      \
  KVF_API int kvf_tanh_norm_##SUF(float* resid, const void* delta, const float* partials, int nsplit,                  \
                                  long long split_stride, float mult, const float* alpha, const float* w,              \
                                  const float* b, void* out, const int* rows, long long n_rows, int W,                 \
                                  cudaStream_t st) {                                                                   \
    if (n_rows <= 0 || W <= 0) return 0;                                                                               \
    if (!alpha || !w || !b || nsplit < 0) return (int)cudaErrorInvalidValue;                                           \
    const bool v4 = (W % 4) == 0 && (split_stride % 4) == 0 &&                                                         \
                    ((((uintptr_t)resid) | ((uintptr_t)delta) | ((uintptr_t)partials) | ((uintptr_t)out)) % 16) == 0; \
    long long g = (n_rows * (v4 ? W / 4 : W) + 255) / 256;                                                             \
    if (g > 148 * 16) g = 148 * 16;                                                                                    \
    if (v4)                                                                                                            \
      return launch(tanh_norm_kernel<T, 4>, dim3((unsigned)g), dim3(256), 0, st, resid, (const T*)delta, partials,     \
                    nsplit, split_stride, mult, alpha, w, b, (T*)out, rows, n_rows, W);                                \
    return launch(tanh_norm_kernel<T, 1>, dim3((unsigned)g), dim3(256), 0, st, resid, (const T*)delta, partials,       \
                  nsplit, split_stride, mult, alpha, w, b, (T*)out, rows, n_rows, W);                                  \
  }

KVF_TANH_NORM_API(f32, float)
KVF_TANH_NORM_API(bf16, bf16)

// Turn programmatic dependent launch on or off for every launch of this library (the flag is one per
// shared library).
KVF_API int kvf_decay_set_pdl(int enabled) {
  kvf::g_pdl_enabled = enabled ? 1 : 0;
  return 0;
}
