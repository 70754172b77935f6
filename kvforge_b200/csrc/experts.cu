// A feed-forward made of many small experts of which every token uses a few.
//
//   route   : per token the router's logits (float, plus a bias per expert where the router has one), scores
//             s = 1 / (1 + exp(-z)) (or a softmax over all experts, or the logits themselves with a softmax
//             over the chosen ones alone), the choice among the best groups of neighbouring experts, the
//             chosen experts and their weights
//   sort    : the (token, choice) pairs ordered by expert, and the list of row tiles per expert
//   product : for every tile of one expert's rows a tile of  act(x W_up^T)  or of  h W_down^T; a gated expert's
//             first matrix holds gate and up rows in alternating blocks of 8 and its activation joins the two:
//             g' = min(g, limit), u' = clamp(u, -limit, limit), g' / (1 + exp(-alpha g')) * (u' + shift)
//   combine : resid[token] += sum_k weight_k * y[token, k]   (float, k in order)
//
// A pair's row of a product depends on that row and on its expert's weights alone (its products are
// added in the order of k: by one thread on the FP32 pipes, by the tensor cores' own order in bfloat16),
// so a token's result does not depend on what else is in the batch or on where its pairs land in the order.  Router, scores, choice and the weighted sum are float
// whatever the storage type T.
#include <limits.h>

#include "common.cuh"

using namespace kvf;

namespace {

constexpr int TM = 32;  // rows of a tile of the grouped products on the FP32 pipes
constexpr int TM_MIN = 8;  // the smallest tile any product uses: scratch for the tile list is made for it

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
    if (v2 > v || (v2 == v && i2 < i)) {
      v = v2;
      i = i2;
    }
  }
}

template <typename T> __device__ __forceinline__ void load8(const T* src, float* dst);
template <> __device__ __forceinline__ void load8<float>(const float* src, float* dst) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w; dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* src, float* dst) {
  bf16x8_to_float(*reinterpret_cast<const uint4*>(src), dst);
}

// One CTA of eight warps per RT tokens (one token a CTA while a step has few, four when it has many).  The warps share out the experts: a logit is one warp's dot product (a lane
// adds its products in the order of the columns, then the lanes are summed in a fixed tree), so it does not depend on
// the batch; a row of the router is read once for the CTA's tokens.  Then warp t chooses for token t.  Shared memory
// per token: scores [E], choice scores [E], group scores [G], group flags [G].
template <typename T, int RT>
__global__ void __launch_bounds__(256) moe_route_kernel(const T* __restrict__ x, long long x_stride,
                                                         const float* __restrict__ router, const float* __restrict__ correction,
                                                         int n_tokens, int W, int E, int top, int groups, int keep,
                                                         float norm_eps, int vec, int flags, int* __restrict__ ids, float* __restrict__ wts,
                                                         const float* __restrict__ logit_bias) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * RT;
  const int per_token = 2 * E + 2 * groups;
  for (int e = warp; e < E; e += 8) {
    const float* wr = router + (size_t)e * W;
    float z[RT];
#pragma unroll
    for (int t = 0; t < RT; ++t) z[t] = 0.f;
    if (vec) {
      for (int j = lane * 8; j < W; j += 256) {
        float wv[8];
        load8<float>(wr + j, wv);
#pragma unroll
        for (int t = 0; t < RT; ++t) {
          if (n0 + t >= n_tokens) break;
          float xv[8];
          load8<T>(x + (size_t)(n0 + t) * x_stride + j, xv);
#pragma unroll
          for (int i = 0; i < 8; ++i) z[t] = fmaf(xv[i], wv[i], z[t]);
        }
      }
    } else {
      for (int j = lane; j < W; j += 32) {
        const float wv = wr[j];
#pragma unroll
        for (int t = 0; t < RT; ++t)
          if (n0 + t < n_tokens) z[t] = fmaf(to_float<T>(x[(size_t)(n0 + t) * x_stride + j]), wv, z[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < RT; ++t) {
      const float zt = warp_sum(z[t]) + (logit_bias ? logit_bias[e] : 0.f);
      if (lane == 0) {
        // flags bit 0: the scores are a softmax over all experts, made below from the logits kept here;
        // bit 2: the logits themselves rank the experts, and the weights are a softmax over the chosen logits
        const float s = (flags & 5) ? zt : 1.f / (1.f + expf(-zt));
        sm[t * per_token + e] = s;
        sm[t * per_token + E + e] = s + (correction ? correction[e] : 0.f);
      }
    }
  }
  __syncthreads();
  if (warp >= RT || n0 + warp >= n_tokens) return;
  const int n = n0 + warp;
  float* sc = sm + warp * per_token;
  float* ch = sc + E;
  float* gs = ch + E;
  float* ga = gs + groups;
  if (flags & 1) {
    // softmax over the experts: a lane adds its experts in order, then the lanes are summed in a fixed tree
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, sc[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(sc[e] - mx);
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
      const float s = expf(sc[e] - mx) / sum;
      sc[e] = s;
      ch[e] = s + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
  }
  if (groups > 1 && keep < groups) {
    // a group is ranked by the sum of the top two shifted scores among its members; the `keep` best-ranked stay
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = ch[e];
        if (v > a) {
          b = a;
          a = v;
        } else if (v > b) {
          b = v;
        }
      }
      gs[g] = per > 1 ? a + b : a;
      ga[g] = 0.f;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float v = -INFINITY;
      int i = INT_MAX;
      for (int g = lane; g < groups; g += 32)
        if (ga[g] == 0.f && (gs[g] > v || i == INT_MAX)) {
          v = gs[g];
          i = g;
        }
      warp_argmax(v, i);
      if (lane == 0 && i != INT_MAX) ga[i] = 1.f;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (ga[e / per] == 0.f) ch[e] = -INFINITY;
    __syncwarp();
  }
  int* my_ids = ids + (size_t)n * top;
  float* my_w = wts + (size_t)n * top;
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float v = -INFINITY;
    int i = INT_MAX;
    for (int e = lane; e < E; e += 32) {
      const float c = ch[e];
      if (c != c) continue;  // taken already (marked not-a-number)
      if (c > v || i == INT_MAX) {
        v = c;
        i = e;
      }
    }
    warp_argmax(v, i);
    if (i == INT_MAX) i = 0;  // cannot happen while top <= E
    const float s = sc[i];
    total += s;  // every lane adds the same numbers in the same order
    if (lane == 0) {
      my_ids[k] = i;
      my_w[k] = s;
      ch[i] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  if (flags & 4) {
    // softmax over the chosen logits alone: the first chosen is the largest; every lane adds in the order of k
    const float mx = my_w[0];
    float sum = 0.f;
    for (int k = 0; k < top; ++k) sum += expf(my_w[k] - mx);
    __syncwarp();
    for (int k = lane; k < top; k += 32) my_w[k] = expf(my_w[k] - mx) / sum;
    return;
  }
  if (flags & 2) return;  // the weights are the chosen scores as they are
  const float inv = 1.f / (total + norm_eps);
  for (int k = lane; k < top; k += 32) my_w[k] *= inv;
}

// One CTA.  ids [P] -> order [P] (pairs by expert), tiles: (expert, first sorted row, rows) per tile of
// tm rows, meta[0] = number of tiles.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int P, int E, int tm, int* __restrict__ order,
                                                         int* __restrict__ tiles, int* __restrict__ meta) {
  pdl_launch();
  pdl_wait();
  extern __shared__ int si[];
  int* cnt = si;          // [E]
  int* off = cnt + E;     // [E]
  int* tbase = off + E;   // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      tbase[e] = t;
      run += cnt[e];
      t += (cnt[e] + tm - 1) / tm;
    }
    meta[0] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = cnt[e];
    for (int r0 = 0, t = tbase[e]; r0 < c; r0 += tm, ++t) {
      tiles[3 * t] = e;
      tiles[3 * t + 1] = off[e] + r0;
      tiles[3 * t + 2] = min(tm, c - r0);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;  // now a cursor
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p];
    order[off[e] + atomicAdd(&cnt[e], 1)] = p;
  }
}

__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f)); }
// What an expert applies between its two products.  kind 0: the exact GELU, 1: the square of relu, 2: gated (the
// first matrix holds gate and up rows in alternating blocks of 8; see `gated_act`).
struct ExpertAct {
  int kind;
  float limit, alpha, shift;
};
constexpr int ACT_GATED = 2;
__device__ __forceinline__ float gated_act(float g, float u, const ExpertAct& a) {
  g = fminf(g, a.limit);
  u = fminf(fmaxf(u, -a.limit), a.limit);
  return g / (1.f + expf(-a.alpha * g)) * (u + a.shift);
}
__device__ __forceinline__ float expert_act(float z, int kind) {
  if (kind == 1) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  return gelu_erf(z);
}

// A tile of TM rows of one expert times a tile of 64 of its output columns, on the FP32 pipes.
//   UP:   A row i = x[order[i] / top], B = w[e] [n_out][K], out act[i][col] = T(act(acc))
//   else: A row i = act[i],            B = w[e] [n_out][K], out y[order[i]][col] = acc (float)
template <typename T, bool UP>
__global__ void __launch_bounds__(256) moe_product_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ w,
                                                           const int* __restrict__ order, const int* __restrict__ tiles,
                                                           const int* __restrict__ meta, int top, int K, int n_out,
                                                           T* __restrict__ act, float* __restrict__ y, ExpertAct ea, int act_ld) {
  pdl_launch();
  pdl_wait();
  constexpr int BN = 64, BK = 16;
  if ((int)blockIdx.y >= meta[0]) return;
  __shared__ float As[BK][TM + 1];
  __shared__ float Bs[BK][BN + 1];
  __shared__ int src[TM];
  const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int col0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  if (tid < TM) {
    int s = -1;
    if (tid < rows) s = UP ? order[row0 + tid] / top : row0 + tid;
    src[tid] = s;
  }
  __syncthreads();
  const T* wb = w + (size_t)e * n_out * K;
  // rows ty*2 .. +1; columns cb, cb+1 and cb+8, cb+9 of the tile: with gate and up rows in blocks of 8 a thread
  // holds two gates and their ups
  const int ty = tid >> 4, tx = tid & 15;
  const int cb = (tx >> 2) * 16 + (tx & 3) * 2;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < TM * BK; idx += 256) {
      const int r = idx / BK, kk = idx - r * BK;
      float v = 0.f;
      if (src[r] >= 0 && k0 + kk < K) v = to_float<T>(a[(size_t)src[r] * a_stride + k0 + kk]);
      As[kk][r] = v;
    }
    for (int idx = tid; idx < BN * BK; idx += 256) {
      const int c = idx / BK, kk = idx - c * BK;
      float v = 0.f;
      if (col0 + c < n_out && k0 + kk < K) v = to_float<T>(wb[(size_t)(col0 + c) * K + k0 + kk]);
      Bs[kk][c] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Bs[kk][cb + (j & 1) + 8 * (j >> 1)];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
    if (UP && ea.kind == ACT_GATED) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = col0 + cb + j;  // a gate row of the stacked matrix; its up row is 8 further
        if (c + 8 >= n_out) continue;
        act[(size_t)(row0 + r) * act_ld + (c >> 4) * 8 + (c & 7)] = from_float<T>(gated_act(acc[i][j], acc[i][j + 2], ea));
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + cb + (j & 1) + 8 * (j >> 1);
      if (c >= n_out) continue;
      if (UP)
        act[(size_t)(row0 + r) * act_ld + c] = from_float<T>(expert_act(acc[i][j], ea.kind));
      else
        y[(size_t)order[row0 + r] * n_out + c] = acc[i][j];
    }
  }
}

// ---------------------------------------------------------------- the same products on the tensor cores (bfloat16)
// A tile of up to NT * 8 rows of one expert times 64 of its output columns over the whole of K: the expert's
// weights ride the MMA's 16-row side (mma.sync m16n8k16) and the tile's rows its 8-column side, as in the
// decode product of the dense layers; weights and gathered rows come in through a cp.async pipeline of
// 16-byte chunks in XOR-swizzled rows.  With a few rows an expert (decoding) the kernel streams each chosen
// expert's weights once; with many it reads them once per tile of rows, from L2.
__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cpa16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte chunk `chunk` (0..7) of row `row` in a swizzled tile of 128-byte rows
__device__ __forceinline__ uint32_t toff(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <int NT, int STAGES, bool UP>
__global__ void __launch_bounds__(128) moe_product_mma_kernel(const bf16* __restrict__ a, long long a_stride, const bf16* __restrict__ w,
                                                               const int* __restrict__ order, const int* __restrict__ tiles,
                                                               const int* __restrict__ meta, int top, int K, int n_out,
                                                               bf16* __restrict__ act, float* __restrict__ y, ExpertAct ea, int act_ld) {
  constexpr int BN = 64, BK = 64, THREADS = 128;
  constexpr int W_BYTES = BN * 128, X_ROWS = NT * 8, X_BYTES = X_ROWS * 128, STAGE_BYTES = W_BYTES + X_BYTES;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int src[X_ROWS], dst[X_ROWS];
  pdl_launch();
  pdl_wait();
  if ((int)blockIdx.y >= meta[0]) return;
  const uint32_t smem = s_u32(smem_raw);
  const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int n0 = blockIdx.x * BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < X_ROWS) {
    int s = -1, d = -1;
    if ((int)threadIdx.x < rows) {
      const int pair = order[row0 + threadIdx.x];
      s = UP ? pair / top : row0 + (int)threadIdx.x;
      d = UP ? row0 + (int)threadIdx.x : pair;
    }
    src[threadIdx.x] = s;
    dst[threadIdx.x] = d;
  }
  __syncthreads();
  const bf16* wb = w + (size_t)e * n_out * K;
  const int n_iters = (K + BK - 1) / BK;
  auto load = [&](int stage, int it) {
    const int k0 = it * BK;
    const uint32_t ws = smem + stage * STAGE_BYTES, xs = ws + W_BYTES;
#pragma unroll
    for (int i = 0; i < (BN * 8) / THREADS; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      const int row = idx >> 3, c = idx & 7;
      const int k = k0 + c * 8;
      const bool valid = (n0 + row < n_out) && (k < K);
      cpa16(ws + toff(row, c), wb + (valid ? (size_t)(n0 + row) * K + k : 0), valid);
    }
    for (int idx = threadIdx.x; idx < X_ROWS * 8; idx += THREADS) {
      const int row = idx >> 3, c = idx & 7;
      const int k = k0 + c * 8;
      const bool valid = (src[row] >= 0) && (k < K);
      cpa16(xs + toff(row, c), a + (valid ? (size_t)src[row] * a_stride + k : 0), valid);
    }
  };
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_iters) load(s, s);
    cpa_commit();
  }
  for (int it = 0; it < n_iters; ++it) {
    cpa_wait<STAGES - 2>();
    __syncthreads();  // stage `it` has landed for every thread; stage `it-1` has been consumed
    if (it + STAGES - 1 < n_iters) load((it + STAGES - 1) % STAGES, it + STAGES - 1);
    cpa_commit();
    const uint32_t ws = smem + (it % STAGES) * STAGE_BYTES, xs = ws + W_BYTES;
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      uint32_t af[4];
      ldsm_x4(af, ws + toff(warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4)));
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t b[4];
        const int trow = (NT == 1) ? (lane & 7) : (j * 8 + ((lane >> 4) << 3) + (lane & 7));
        ldsm_x4(b, xs + toff(trow, 2 * kk + ((lane >> 3) & 1)));
        mma16816(acc[j], af, b[0], b[1]);
        if (NT > 1) mma16816(acc[j + 1 < NT ? j + 1 : j], af, b[2], b[3]);
      }
    }
  }
  cpa_wait<0>();
  // acc[j]: c0,c1 -> column f0 = warp*16 + lane/4, rows t, t+1; c2,c3 -> column f0 + 8
  const int f0 = n0 + warp * 16 + (lane >> 2);
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int t = j * 8 + ((lane & 3) << 1) + r;
      if (t >= rows) continue;
      if (UP && ea.kind == ACT_GATED) {
        // stacked rows f0 (a gate) and f0 + 8 (its up): one output column
        if (f0 + 8 < n_out) act[(size_t)dst[t] * act_ld + (f0 >> 4) * 8 + (f0 & 7)] = __float2bfloat16_rn(gated_act(acc[j][r], acc[j][2 + r], ea));
        continue;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int f = f0 + 8 * h;
        if (f >= n_out) continue;
        const float v = acc[j][2 * h + r];
        if (UP)
          act[(size_t)dst[t] * act_ld + f] = __float2bfloat16_rn(expert_act(v, ea.kind));
        else
          y[(size_t)dst[t] * n_out + f] = v;
      }
    }
  }
}

template <int NT, int STAGES, bool UP>
int launch_mma(const bf16* a, long long a_stride, const bf16* w, const int* order, const int* tiles, const int* meta, int top, int K,
               int n_out, int max_tiles, bf16* act, float* y, ExpertAct ea, int act_ld, cudaStream_t st) {
  const size_t smem = (size_t)STAGES * (64 * 128 + NT * 8 * 128);
  auto kern = moe_product_mma_kernel<NT, STAGES, UP>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, dim3((n_out + 63) / 64, max_tiles), dim3(128), smem, st, a, a_stride, w, order, tiles, meta, top, K, n_out, act, y, ea, act_ld);
}

template <bool UP>
int product_mma(int tm, const bf16* a, long long a_stride, const bf16* w, const int* order, const int* tiles, const int* meta, int top, int K,
                int n_out, int max_tiles, bf16* act, float* y, ExpertAct ea, int act_ld, cudaStream_t st) {
  if (tm <= 8) return launch_mma<1, 8, UP>(a, a_stride, w, order, tiles, meta, top, K, n_out, max_tiles, act, y, ea, act_ld, st);
  if (tm <= 16) return launch_mma<2, 8, UP>(a, a_stride, w, order, tiles, meta, top, K, n_out, max_tiles, act, y, ea, act_ld, st);
  if (tm <= 32) return launch_mma<4, 6, UP>(a, a_stride, w, order, tiles, meta, top, K, n_out, max_tiles, act, y, ea, act_ld, st);
  return launch_mma<8, 6, UP>(a, a_stride, w, order, tiles, meta, top, K, n_out, max_tiles, act, y, ea, act_ld, st);
}

// Rows of a tile for P pairs over E experts on the tensor cores: small tiles while an expert has a few rows (the
// weights stream once either way), large ones when it has many (its weights are read once per tile).
inline int mma_tile_rows(int P, int E) {
  if (P <= 2 * E) return 8;
  if (P <= 6 * E) return 16;
  if (P <= 24 * E) return 32;
  return 64;
}

// xs[i, :] = x[order[i] / top, :]: the rows of the pairs in the order of the experts (16-byte copies), for a
// product that wants an expert's rows side by side.
__global__ void moe_gather_kernel(const bf16* __restrict__ x, long long x_stride, const int* __restrict__ order, int top, int P,
                                  int W, bf16* __restrict__ xs) {
  pdl_launch();
  pdl_wait();
  const int chunks = W / 8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (long long)P * chunks; idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx / chunks), c = (int)(idx - (long long)i * chunks);
    const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)(order[i] / top) * x_stride + c * 8);
    *reinterpret_cast<uint4*>(xs + (size_t)i * W + c * 8) = v;
  }
}

__global__ void moe_combine_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ wts,
                                   long long total, int W, int top) {
  pdl_launch();
  pdl_wait();
  if ((W & 3) == 0) {  // four columns a thread; each column's sum is the same chain over k as below
    const int w4 = W >> 2;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (total >> 2); idx += (long long)gridDim.x * blockDim.x) {
      const long long n = idx / w4;
      const int c = (int)(idx - n * w4) * 4;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < top; ++k) {
        const float g = wts[n * top + k];
        const float4 v = *reinterpret_cast<const float4*>(y + ((size_t)n * top + k) * W + c);
        s.x = fmaf(g, v.x, s.x);
        s.y = fmaf(g, v.y, s.y);
        s.z = fmaf(g, v.z, s.z);
        s.w = fmaf(g, v.w, s.w);
      }
      float4* r = reinterpret_cast<float4*>(resid + (size_t)n * W + c);
      float4 o = *r;
      o.x += s.x;
      o.y += s.y;
      o.z += s.z;
      o.w += s.w;
      *r = o;
    }
    return;
  }
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / W;
    const int c = (int)(idx - n * W);
    float s = 0.f;
    for (int k = 0; k < top; ++k) s = fmaf(wts[n * top + k], y[((size_t)n * top + k) * W + c], s);
    resid[idx] += s;
  }
}

}  // namespace

// Rows of tiles that `n_pairs` pairs spread over `E` experts can make at most, whatever the tile size.
KVF_API int kvf_moe_max_tiles(int n_pairs, int E) { return n_pairs / TM_MIN + E; }

template <typename T>
int run_products(const T* x, long long x_stride, const T* w_up, const T* w_down, const int* ids, int P, int W, int ff, int E, int top,
                 int* order, int* tiles, int* meta, T* act, float* y, ExpertAct ea, cudaStream_t st);

template <>
int run_products<float>(const float* x, long long x_stride, const float* w_up, const float* w_down, const int* ids, int P, int W, int ff,
                        int E, int top, int* order, int* tiles, int* meta, float* act, float* y, ExpertAct ea, cudaStream_t st) {
  int rc = launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), st, ids, P, E, TM, order, tiles, meta);
  if (rc) return rc;
  const int max_tiles = P / TM + E;
  const int n_up = ea.kind == ACT_GATED ? 2 * ff : ff;  // rows of an expert's first matrix
  rc = launch(moe_product_kernel<float, true>, dim3((n_up + 63) / 64, max_tiles), dim3(256), 0, st, x, x_stride, w_up, (const int*)order,
              (const int*)tiles, (const int*)meta, top, W, n_up, act, (float*)nullptr, ea, ff);
  if (rc) return rc;
  return launch(moe_product_kernel<float, false>, dim3((W + 63) / 64, max_tiles), dim3(256), 0, st, (const float*)act, (long long)ff,
                w_down, (const int*)order, (const int*)tiles, (const int*)meta, top, ff, W, (float*)nullptr, y, ea, ff);
}

template <>
int run_products<bf16>(const bf16* x, long long x_stride, const bf16* w_up, const bf16* w_down, const int* ids, int P, int W, int ff, int E,
                       int top, int* order, int* tiles, int* meta, bf16* act, float* y, ExpertAct ea, cudaStream_t st) {
  const int n_up = ea.kind == ACT_GATED ? 2 * ff : ff;
  const bool tensor = (W % 8 == 0) && (ff % 8 == 0) && (x_stride % 8 == 0) && ((((uintptr_t)x) & 15) == 0);
  const int tm = tensor ? mma_tile_rows(P, E) : TM;
  int rc = launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), st, ids, P, E, tm, order, tiles, meta);
  if (rc) return rc;
  const int max_tiles = P / tm + E;
  if (tensor) {
    rc = product_mma<true>(tm, x, x_stride, w_up, order, tiles, meta, top, W, n_up, max_tiles, act, nullptr, ea, ff, st);
    if (rc) return rc;
    return product_mma<false>(tm, act, (long long)ff, w_down, order, tiles, meta, top, ff, W, max_tiles, nullptr, y, ea, ff, st);
  }
  rc = launch(moe_product_kernel<bf16, true>, dim3((n_up + 63) / 64, max_tiles), dim3(256), 0, st, x, x_stride, w_up, (const int*)order,
              (const int*)tiles, (const int*)meta, top, W, n_up, act, (float*)nullptr, ea, ff);
  if (rc) return rc;
  return launch(moe_product_kernel<bf16, false>, dim3((W + 63) / 64, max_tiles), dim3(256), 0, st, (const bf16*)act, (long long)ff,
                w_down, (const int*)order, (const int*)tiles, (const int*)meta, top, ff, W, (bf16*)nullptr, y, ea, ff);
}

#define KVF_EXPERTS_API(SUF, T)                                                                                       \
  KVF_API int kvf_moe_route_##SUF(const void* x, long long x_stride, const float* router, const float* correction,    \
                                  int n_tokens, int W, int E, int top, int groups, int keep, float norm_eps,          \
                                  int flags, int* ids, float* wts, const float* logit_bias, cudaStream_t st) {        \
    if (n_tokens <= 0) return 0;                                                                                      \
    if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||                   \
        top > keep * (E / groups))                                                                                    \
      return (int)cudaErrorInvalidValue;                                                                              \
    const int rt = n_tokens <= 256 ? 1 : 4;                                                                           \
    const size_t smem = (size_t)rt * (2 * E + 2 * groups) * sizeof(float);                                            \
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;                                                          \
    const int vec = (W % 8 == 0) && (x_stride % 8 == 0) && ((((uintptr_t)x) | ((uintptr_t)router)) % 16 == 0);        \
    if (rt == 1)                                                                                                      \
      return launch(moe_route_kernel<T, 1>, dim3(n_tokens), dim3(256), smem, st, (const T*)x, x_stride, router,       \
                    correction, n_tokens, W, E, top, groups, keep, norm_eps, vec, flags, ids, wts, logit_bias);       \
    return launch(moe_route_kernel<T, 4>, dim3((n_tokens + 3) / 4), dim3(256), smem, st, (const T*)x, x_stride,       \
                  router, correction, n_tokens, W, E, top, groups, keep, norm_eps, vec, flags, ids, wts, logit_bias); \
  }                                                                                                                   \
  KVF_API int kvf_moe_experts_##SUF(const void* x, long long x_stride, const void* w_up, const void* w_down,          \
                                    const int* ids, const float* wts, int n_tokens, int W, int ff, int E, int top,    \
                                    int* order, int* tiles, int* meta, void* act, float* y, float* resid,             \
                                    int act_kind, float act_limit, float act_alpha, float act_shift,                  \
                                    cudaStream_t st) {                                                                \
    if (n_tokens <= 0) return 0;                                                                                      \
    if (act_kind == ACT_GATED && (ff & 7)) return (int)cudaErrorInvalidValue; /* gate and up rows in blocks of 8 */   \
    const ExpertAct ea{act_kind, act_limit, act_alpha, act_shift};                                                    \
    const int P = n_tokens * top;                                                                                     \
    if ((size_t)3 * E * sizeof(int) > 48 * 1024) return (int)cudaErrorInvalidValue;                                   \
    if (kvf_moe_max_tiles(P, E) > 65535) return (int)cudaErrorInvalidValue;                                           \
    int rc = run_products<T>((const T*)x, x_stride, (const T*)w_up, (const T*)w_down, ids, P, W, ff, E, top, order,   \
                             tiles, meta, (T*)act, y, ea, st);                                                        \
    if (rc) return rc;                                                                                                \
    const long long total = (long long)n_tokens * W;                                                                  \
    long long g = (total + 255) / 256;                                                                                \
    if (g > 148 * 16) g = 148 * 16;                                                                                   \
    return launch(moe_combine_kernel, dim3((unsigned)g), dim3(256), 0, st, resid, (const float*)y, wts, total, W,     \
                  top);                                                                                               \
  }

KVF_EXPERTS_API(f32, float)
KVF_EXPERTS_API(bf16, bf16)

// The steps one by one, for a caller that runs the two products elsewhere (the tensor-memory product of many rows).
KVF_API int kvf_moe_sort(const int* ids, int P, int E, int tm, int* order, int* tiles, int* meta, cudaStream_t st) {
  if (P <= 0) return 0;
  if (tm <= 0 || (size_t)3 * E * sizeof(int) > 48 * 1024) return (int)cudaErrorInvalidValue;
  return launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), st, ids, P, E, tm, order, tiles, meta);
}

KVF_API int kvf_moe_gather_bf16(const void* x, long long x_stride, const int* order, int top, int P, int W, void* xs,
                                cudaStream_t st) {
  if (P <= 0) return 0;
  if ((W & 7) || (x_stride & 7) || ((((uintptr_t)x) | ((uintptr_t)xs)) & 15)) return (int)cudaErrorInvalidValue;
  long long g = ((long long)P * (W / 8) + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return launch(moe_gather_kernel, dim3((unsigned)g), dim3(256), 0, st, (const bf16*)x, x_stride, order, top, P, W, (bf16*)xs);
}

KVF_API int kvf_moe_combine(float* resid, const float* y, const float* wts, int n_tokens, int W, int top, cudaStream_t st) {
  const long long total = (long long)n_tokens * W;
  if (total <= 0) return 0;
  long long g = (total + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return launch(moe_combine_kernel, dim3((unsigned)g), dim3(256), 0, st, resid, y, wts, total, W, top);
}
