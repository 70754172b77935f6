// Paged grouped-query attention whose heads talk to one another before the softmax, with an optional
// sink in the softmax, on the FP32 pipes: any head size up to 256, up to 64 heads, any
// grouping, any mix of query lengths in one flat batch.
//
// What it computes, for query i of sequence b at position p = ctx_b - q_b + i and key j <= p
// (and j > p - window when window > 0):
//   s_g(i, j)  = scale * (q_g(i) . k_{c(g)}(j))                 c(g) = g / (nh / nkv)
//   s'_h(i, j) = sum_g talk[h][g] * s_g(i, j)                   (talk == null: s' = s)
//   w_h(i, j)  = exp(s'_h(i, j)) / (exp(sink_h) + sum_j' exp(s'_h(i, j')))     (sink == null: no such term)
//   o_h(i)     = sum_j w_h(i, j) * v_{c(h)}(j)
// The sink has no key and no value: it only takes part in the sum below the line.  Everything is float;
// the output is rounded once to the storage type T.
//
// A CTA owns tq queries of one sequence and ALL heads (a head's weights need every head's scores).  Its rows
// are r = head * tq + query; a warp owns `rpw` neighbouring rows from the scores to the output.  Keys are
// walked in tiles of 32 that start at absolute multiples of 32.  Per tile: the key tiles of the kv heads come
// through shared memory a few at a time and every row's scores are one thread's sequential dot products; the
// heads are mixed (a thread owns four target heads of one (query, key) and adds over the source heads in
// order); the rows' running maxima and sums move on; the value tiles come through the same shared memory
// and the rows add their weighted values.  A fully masked tile leaves a row's state untouched, so a result
// does not depend on how the prompt was cut, on the other rows of its tile, or on the physical pages.
//
// SPLIT: every sequence has one query; grid.x walks key ranges of split_size, partial (m, l, acc) go to
// scratch and a second kernel merges the ranges in order.  The sink belongs to the first range.
//
// Cache layout per layer: K [num_blocks][nkv][block_size][d], V [num_blocks][nkv][block_size][dv].
//
// This header is compiled once per storage type (attention_talking_f32.cu, attention_talking_bf16.cu), so that the
// two build side by side.
#pragma once
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int TK = 32;   // keys per tile = one per lane
constexpr int NW = 8;    // warps per CTA
constexpr int MAXR = 8;  // rows a warp owns at most

struct TalkParams {
  const void* q;
  void* out;
  const void* kcache;
  const void* vcache;
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  const float* talk;  // [nh][nh] (target head, source head) or null
  const float* sink;  // [nh] or null
  float* part_acc;    // split mode: [B][nh][splits][dv]
  float* part_ml;     // split mode: [B][nh][splits][2]
  int q_stride, out_stride, bt_stride;
  int nh, nkv, d, dv, block_size;
  int tq, rpw, gc;  // queries per CTA, rows per warp, kv heads in shared memory at a time
  int window;
  int split_size, max_splits;
  float scale;
};

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<bf16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void load_vec(const T* src, float* dst);
template <> __device__ __forceinline__ void load_vec<float>(const float* src, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
template <> __device__ __forceinline__ void load_vec<bf16>(const bf16* src, float* dst) {
  bf16x8_to_float(*reinterpret_cast<const uint4*>(src), dst);
}

// `count` tiles of TK keys from position t0 on, of kv heads c0 .. c0 + count - 1, `width` numbers a key, as
// float rows of `ld`; keys at or beyond ctx and pages that were given back are zeros.  A width that is no multiple
// of a 16-byte load goes number by number, and the row is filled with zeros up to the next multiple of four.
template <typename T>
__device__ __forceinline__ void stage_tiles(const T* cache, const int* bt, int t0, int ctx, int c0, int count, int width,
                                            int ld, int nkv, int block_size, float* dst) {
  constexpr int VN = Vec<T>::N;
  if (width % VN != 0) {
    const int wpad = (width + 3) & ~3;
    for (int idx = threadIdx.x; idx < count * TK * wpad; idx += blockDim.x) {
      const int cc = idx / (TK * wpad), rem = idx - cc * TK * wpad;
      const int key = rem / wpad, col = rem - key * wpad;
      const int kp = t0 + key;
      const int blk = (kp < ctx && col < width) ? bt[kp / block_size] : -1;
      float f = 0.f;
      if (blk >= 0) f = to_float<T>(cache[(((size_t)blk * nkv + (c0 + cc)) * block_size + (kp % block_size)) * width + col]);
      dst[((size_t)cc * TK + key) * ld + col] = f;
    }
    return;
  }
  const int per = width / VN;
  for (int idx = threadIdx.x; idx < count * TK * per; idx += blockDim.x) {
    const int cc = idx / (TK * per), rem = idx - cc * TK * per;
    const int key = rem / per, col = (rem - key * per) * VN;
    const int kp = t0 + key;
    float f[VN];
    const int blk = kp < ctx ? bt[kp / block_size] : -1;
    if (blk >= 0) {
      const size_t base = (((size_t)blk * nkv + (c0 + cc)) * block_size + (kp % block_size)) * width + col;
      load_vec<T>(cache + base, f);
    } else {
#pragma unroll
      for (int e = 0; e < VN; ++e) f[e] = 0.f;
    }
    float* o = dst + ((size_t)cc * TK + key) * ld + col;
#pragma unroll
    for (int e = 0; e < VN; ++e) o[e] = f[e];
  }
}

template <typename T, int DPL, bool SPLIT>
__global__ void __launch_bounds__(NW * 32) talking_attention_kernel(const TalkParams p) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int d = p.d, dv = p.dv, nh = p.nh, tq = p.tq;
  const int R = nh * tq;
  const int nhp = (nh + 3) & ~3;
  const int dp = (d + 3) & ~3;  // a query row and a key row are walked four numbers at a time: zeros fill them up
  const int ld = (((d > dv ? d : dv) + 3) & ~3) + 4;
  float* Qs = smem;                                  // [R][dp]
  float* Ss = Qs + (size_t)R * dp;                   // [R][TK]
  float* Ps = p.talk ? Ss + (size_t)R * TK : Ss;     // [R][TK]
  float* Tt = Ps + (size_t)R * TK;                   // [nh][nhp]: Tt[g][h] = talk[h][g]
  float* KVs = p.talk ? Tt + (size_t)nh * nhp : Tt;  // [gc][TK][ld]

  const int b = blockIdx.y;
  const int gs = nh / p.nkv;
  const int q_begin = p.qsl[b], q_len = p.qsl[b + 1] - q_begin;
  const int ctx = p.ctx_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (q_len <= 0 || ctx <= 0) return;

  int q0, n_tok, kv_lo, kv_hi;
  if (SPLIT) {
    q0 = q_len - 1;
    n_tok = 1;
    kv_lo = blockIdx.x * p.split_size;
    if (kv_lo >= ctx) return;  // a range past the context: the merge never reads it
    kv_hi = min(ctx, kv_lo + p.split_size);
  } else {
    q0 = blockIdx.x * tq;
    if (q0 >= q_len) return;
    n_tok = min(tq, q_len - q0);
    kv_lo = 0;
    kv_hi = ctx - q_len + q0 + n_tok;
  }

  // ---- stage the queries as float, and the mixing matrix turned (source head first)
  const T* qg = (const T*)p.q;
  for (int idx = threadIdx.x; idx < R * dp; idx += blockDim.x) {
    const int r = idx / dp, j = idx - r * dp;
    const int h = r / tq, i = r - h * tq;
    Qs[idx] = (i < n_tok && j < d) ? to_float<T>(qg[(size_t)(q_begin + q0 + i) * p.q_stride + (size_t)h * d + j]) : 0.f;
  }
  if (p.talk)
    for (int idx = threadIdx.x; idx < nh * nhp; idx += blockDim.x) {
      const int g = idx / nhp, h = idx - g * nhp;
      Tt[idx] = h < nh ? p.talk[(size_t)h * nh + g] : 0.f;
    }

  // ---- the rows this warp owns
  float m[MAXR], l[MAXR], acc[MAXR][DPL];
  int pos[MAXR], kvh[MAXR];
  const int r_first = warp * p.rpw;
  const bool with_sink = p.sink != nullptr && (!SPLIT || blockIdx.x == 0);
#pragma unroll
  for (int k = 0; k < MAXR; ++k) {
    const int r = r_first + k;
    const int h = r / tq, i = r - h * tq;
    const bool valid = k < p.rpw && r < R && i < n_tok;
    pos[k] = valid ? ctx - q_len + q0 + i : -1;  // -1: sees nothing, writes nothing
    kvh[k] = valid ? h / gs : -1;
    m[k] = (valid && with_sink) ? p.sink[h] : -INFINITY;
    l[k] = (valid && with_sink) ? 1.f : 0.f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[k][e] = 0.f;
  }
  // all of this warp's rows on one kv head: they share every value they load
  int c_lo = p.nkv, c_hi = -1;
#pragma unroll
  for (int k = 0; k < MAXR; ++k)
    if (kvh[k] >= 0) {
      c_lo = min(c_lo, kvh[k]);
      c_hi = max(c_hi, kvh[k]);
    }
  const bool one_kv = c_lo == c_hi;

  const T* kc = (const T*)p.kcache;
  const T* vc = (const T*)p.vcache;
  const int* bt = p.block_tables + (size_t)b * p.bt_stride;

  for (int t0 = kv_lo; t0 < kv_hi; t0 += TK) {
    // ---- scores of every head: S[r][key]
    for (int c0 = 0; c0 < p.nkv; c0 += p.gc) {
      const int cn = min(p.gc, p.nkv - c0);
      __syncthreads();  // the tiles in shared memory are consumed (and, the first time, the queries staged)
      stage_tiles<T>(kc, bt, t0, ctx, c0, cn, d, ld, p.nkv, p.block_size, KVs);
      __syncthreads();
      for (int k = 0; k < p.rpw; ++k) {
        const int r = r_first + k;
        const int h = r / tq;
        const int c = h / gs;
        if (r >= R || r - h * tq >= n_tok || c < c0 || c >= c0 + cn) continue;  // warp-uniform
        const float* krow = KVs + ((size_t)(c - c0) * TK + lane) * ld;
        const float* qrow = Qs + (size_t)r * dp;
        float s = 0.f;
        for (int c = 0; c < dp; c += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(krow + c);
          const float4 q4 = *reinterpret_cast<const float4*>(qrow + c);
          s = fmaf(q4.x, k4.x, s);
          s = fmaf(q4.y, k4.y, s);
          s = fmaf(q4.z, k4.z, s);
          s = fmaf(q4.w, k4.w, s);
        }
        Ss[r * TK + lane] = s * p.scale;
      }
    }
    // ---- the heads talk: S'[h] = sum_g talk[h][g] S[g], source heads in order
    if (p.talk) {
      __syncthreads();
      const int per_hq = tq * TK;
      for (int item = threadIdx.x; item < (nhp >> 2) * per_hq; item += blockDim.x) {
        const int hq = item / per_hq, rem = item - hq * per_hq;  // rem = query * TK + key
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int g = 0; g < nh; ++g) {
          const float s = Ss[g * per_hq + rem];
          const float4 t4 = *reinterpret_cast<const float4*>(Tt + g * nhp + hq * 4);
          a.x = fmaf(t4.x, s, a.x);
          a.y = fmaf(t4.y, s, a.y);
          a.z = fmaf(t4.z, s, a.z);
          a.w = fmaf(t4.w, s, a.w);
        }
        const int h0 = hq * 4;
        Ps[(h0 + 0) * per_hq + rem] = a.x;
        if (h0 + 1 < nh) Ps[(h0 + 1) * per_hq + rem] = a.y;
        if (h0 + 2 < nh) Ps[(h0 + 2) * per_hq + rem] = a.z;
        if (h0 + 3 < nh) Ps[(h0 + 3) * per_hq + rem] = a.w;
      }
      __syncthreads();
    } else {
      __syncwarp();
    }
    // ---- running maximum and sum of every row; P[r][key] = exp(s' - m)
    const int kp = t0 + lane;
#pragma unroll
    for (int k = 0; k < MAXR; ++k) {
      if (pos[k] < 0) continue;  // warp-uniform
      const int r = r_first + k;
      bool vis = (kp <= pos[k]) && (kp < kv_hi);
      if (p.window > 0) vis = vis && (kp > pos[k] - p.window);
      if (SPLIT) vis = vis && (kp >= kv_lo);
      const float sc = vis ? Ps[r * TK + lane] : -INFINITY;
      const float m_new = fmaxf(m[k], warp_max(sc));
      float pj = 0.f, corr = 1.f;
      if (m_new != -INFINITY) {  // warp-uniform
        corr = expf(m[k] - m_new);
        pj = vis ? expf(sc - m_new) : 0.f;
        m[k] = m_new;
      }
      l[k] = l[k] * corr + warp_sum(pj);
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[k][e] *= corr;
      Ps[r * TK + lane] = pj;
    }
    __syncwarp();
    // ---- O += P V, the value tiles through the same shared memory
    for (int c0 = 0; c0 < p.nkv; c0 += p.gc) {
      const int cn = min(p.gc, p.nkv - c0);
      __syncthreads();
      stage_tiles<T>(vc, bt, t0, ctx, c0, cn, dv, ld, p.nkv, p.block_size, KVs);
      __syncthreads();
      if (one_kv) {
        if (c_lo < c0 || c_lo >= c0 + cn) continue;  // warp-uniform; every warp still meets the barriers above
        const float* vt = KVs + (size_t)(c_lo - c0) * TK * ld;
        for (int j = 0; j < TK; j += 4) {
          float4 p4[MAXR];
#pragma unroll
          for (int k = 0; k < MAXR; ++k)
            p4[k] = pos[k] >= 0 ? *reinterpret_cast<const float4*>(Ps + (r_first + k) * TK + j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
              const int dim = lane + 32 * e;
              const float v = dim < dv ? vt[(j + jj) * ld + dim] : 0.f;
#pragma unroll
              for (int k = 0; k < MAXR; ++k) {
                const float pv = jj == 0 ? p4[k].x : jj == 1 ? p4[k].y : jj == 2 ? p4[k].z : p4[k].w;
                acc[k][e] = fmaf(pv, v, acc[k][e]);
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < MAXR; ++k) {
          if (kvh[k] < c0 || kvh[k] >= c0 + cn) continue;  // warp-uniform
          const float* vt = KVs + (size_t)(kvh[k] - c0) * TK * ld;
          const float* prow = Ps + (r_first + k) * TK;
          for (int j = 0; j < TK; j += 4) {
            const float4 p4 = *reinterpret_cast<const float4*>(prow + j);
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
              const int dim = lane + 32 * e;
              if (dim < dv) {
                float a = acc[k][e];
                a = fmaf(p4.x, vt[(j + 0) * ld + dim], a);
                a = fmaf(p4.y, vt[(j + 1) * ld + dim], a);
                a = fmaf(p4.z, vt[(j + 2) * ld + dim], a);
                a = fmaf(p4.w, vt[(j + 3) * ld + dim], a);
                acc[k][e] = a;
              }
            }
          }
        }
      }
    }
  }

  // ---- write
#pragma unroll
  for (int k = 0; k < MAXR; ++k) {
    if (pos[k] < 0) continue;
    const int r = r_first + k;
    const int h = r / tq, i = r - h * tq;
    if (SPLIT) {
      const size_t slot = ((size_t)b * nh + h) * p.max_splits + blockIdx.x;
      if (lane == 0) {
        p.part_ml[slot * 2] = m[k];
        p.part_ml[slot * 2 + 1] = l[k];
      }
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int dim = lane + 32 * e;
        if (dim < dv) p.part_acc[slot * dv + dim] = acc[k][e];
      }
    } else {
      const float inv = l[k] > 0.f ? 1.f / l[k] : 0.f;
      T* o = (T*)p.out + (size_t)(q_begin + q0 + i) * p.out_stride + (size_t)h * dv;
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int dim = lane + 32 * e;
        if (dim < dv) o[dim] = from_float<T>(acc[k][e] * inv);
      }
    }
  }
}

// Merge the partial results of the key ranges of one (sequence, head), in range order.
template <typename T>
__global__ void talking_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, T* __restrict__ out,
                                       const int* __restrict__ qsl, const int* __restrict__ ctx_lens, int nh, int dv,
                                       int out_stride, int split_size, int max_splits) {
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.y, head = blockIdx.x;
  const int q_begin = qsl[b], q_len = qsl[b + 1] - q_begin;
  const int ctx = ctx_lens[b];
  if (q_len <= 0 || ctx <= 0) return;
  const int ns = min(max_splits, (ctx + split_size - 1) / split_size);
  const size_t base = ((size_t)b * nh + head) * max_splits;
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) L += expf(ms - M) * part_ml[(base + s) * 2 + 1];
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  T* o = out + (size_t)(q_begin + q_len - 1) * out_stride + (size_t)head * dv;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) a += expf(ms - M) * part_acc[(base + s) * dv + j];
    }
    o[j] = from_float<T>(a * inv);
  }
}

template <typename T, int DPL, bool SPLIT>
int launch_talking(const TalkParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = talking_attention_kernel<T, DPL, SPLIT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, grid, dim3(NW * 32), smem, st, p);
}

template <typename T, bool SPLIT>
int dispatch_dpl(const TalkParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  if (p.dv <= 32) return launch_talking<T, 1, SPLIT>(p, grid, smem, st);
  if (p.dv <= 64) return launch_talking<T, 2, SPLIT>(p, grid, smem, st);
  if (p.dv <= 128) return launch_talking<T, 4, SPLIT>(p, grid, smem, st);
  return launch_talking<T, 8, SPLIT>(p, grid, smem, st);
}

constexpr size_t SMEM_SOFT = 96 * 1024;   // up to here several CTAs share an SM
constexpr size_t SMEM_HARD = 200 * 1024;

template <typename T>
int talking_attention(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables,
                      const int* qsl, const int* ctx_lens, const float* talk, const float* sink, int B, int max_q_len,
                      int q_stride, int out_stride, int bt_stride, int nh, int nkv, int d, int dv, int block_size,
                      float scale, int window, int split_size, int max_splits, int grid_splits, float* part_acc,
                      float* part_ml, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (d <= 0 || d > 256 || dv <= 0 || dv > 256 || nkv <= 0 || nh % nkv != 0 ||
      nh > NW * MAXR || block_size <= 0 || (unsigned)B > 65535u)
    return (int)cudaErrorInvalidValue;
  TalkParams p;
  p.q = q; p.out = out; p.kcache = kcache; p.vcache = vcache;
  p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens;
  p.talk = talk; p.sink = sink; p.part_acc = part_acc; p.part_ml = part_ml;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.nkv = nkv; p.d = d; p.dv = dv; p.block_size = block_size;
  p.window = window; p.scale = scale; p.split_size = split_size; p.max_splits = max_splits;
  const bool split = split_size > 0;
  if (split && (split_size % TK != 0 || max_splits <= 0 || !part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
  const int dp = (d + 3) & ~3;
  const int ld = (((d > dv ? d : dv) + 3) & ~3) + 4;
  const int nhp = (nh + 3) & ~3;
  const size_t tile = (size_t)TK * ld * sizeof(float);
  int tq = split ? 1 : (NW * MAXR) / nh;
  if (tq > 16) tq = 16;
  if (tq > max_q_len) tq = max_q_len;
  size_t fixed = 0;
  for (;; --tq) {  // fewer queries per CTA until the rows and one tile fit
    const size_t R = (size_t)nh * tq;
    fixed = (R * dp + (talk ? 2 : 1) * R * TK + (talk ? (size_t)nh * nhp : 0)) * sizeof(float);
    if (fixed + tile <= SMEM_HARD || tq == 1) break;
  }
  if (fixed + tile > SMEM_HARD) return (int)cudaErrorInvalidValue;
  p.tq = tq;
  const int R = nh * tq;
  p.rpw = (R + NW - 1) / NW;
  const size_t soft = fixed + tile <= SMEM_SOFT ? SMEM_SOFT : SMEM_HARD;
  int gc = (int)((soft - fixed) / tile);
  p.gc = gc < nkv ? gc : nkv;
  const size_t smem = fixed + (size_t)p.gc * tile;
  if (split) {
    dim3 grid(grid_splits > 0 && grid_splits < max_splits ? grid_splits : max_splits, B);
    int rc = dispatch_dpl<T, true>(p, grid, smem, st);
    if (rc) return rc;
    return launch(talking_combine_kernel<T>, dim3(nh, B), dim3(64), 0, st, (const float*)part_acc, (const float*)part_ml,
                  (T*)out, qsl, ctx_lens, nh, dv, out_stride, split_size, max_splits);
  }
  dim3 grid((max_q_len + tq - 1) / tq, B);
  return dispatch_dpl<T, false>(p, grid, smem, st);
}

}  // namespace

#define KVF_TALK_API(SUF, T)                                                                                      \
  KVF_API int kvf_talking_attention_##SUF(                                                                        \
      const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables, const int* qsl,  \
      const int* ctx_lens, const float* talk, const float* sink, int B, int max_q_len, int q_stride,              \
      int out_stride, int bt_stride, int nh, int nkv, int d, int dv, int block_size, float scale, int window,     \
      int split_size, int max_splits, int grid_splits, float* part_acc, float* part_ml, cudaStream_t st) {        \
    return talking_attention<T>(q, out, kcache, vcache, block_tables, qsl, ctx_lens, talk, sink, B, max_q_len,    \
                                q_stride, out_stride, bt_stride, nh, nkv, d, dv, block_size, scale, window,       \
                                split_size, max_splits, grid_splits, part_acc, part_ml, st);                      \
  }

