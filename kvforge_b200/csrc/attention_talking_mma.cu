// Attention whose heads talk before the softmax, bfloat16 storage, heads of 64 or 128 numbers with values as
// wide as keys: the two products (q . k and weights x values) on the tensor cores (mma.sync m16n8k16, float
// accumulators), the mixing of the heads, the softmax and its sink in float on the FP32 pipes.
//
// A CTA of eight warps owns tq queries of one sequence and ALL heads.  The rows of one kv head (its query
// heads x the CTA's queries, head-major, padded to a multiple of 16) form that head's m-tiles; a warp owns one or
// two m-tiles from the scores to the output.  Keys are walked in tiles of BN that start at absolute multiples
// of BN.  Per tile:
//   1. the key tiles of every kv head are in shared memory (cp.async, issued one tile ahead); every warp
//      computes its rows' scores and writes them, scaled, as floats S[head][query][key];
//   2. the value tiles are on their way; the heads are mixed, S'[h] = sum_g talk[h][g] S[g], source heads in
//      order: a warp owns eight target heads of 32, 64 or 128 (query, key) columns (as many as still leave every
//      warp its share) and keeps the matrix's row in registers while it walks its columns;
//   3. every warp reads its rows of S' back in the accumulator layout, masks, moves the running maximum and
//      sum on (the sink is where they start) and adds weights x values; the weights enter that product as two
//      bfloat16 terms (the rounded weight and the rounded rest), so 16 bits of them count.
// A fully masked tile leaves a row's state untouched, so a result does not depend on how the prompt was cut,
// on the other rows of its tile, or on the physical pages.
//
// SPLIT: every sequence has one query; grid.x walks key ranges of split_size, partial (m, l, acc) go to
// scratch and the merge kernel of the FP32-pipe form adds the ranges in order.  The sink belongs to the first.
#include "attention_talking.cuh"

namespace {
namespace tmma {

constexpr int HC = 8;           // target heads a warp mixes at a time
constexpr float LOG2E = 1.4426950408889634f;
constexpr size_t SMEM_MOST = 220 * 1024;
constexpr size_t TWO_CTAS = 112 * 1024;  // what a CTA may hold for two to share an SM

struct Params {
  const bf16* q;
  bf16* out;
  const bf16* kcache;
  const bf16* vcache;
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  const float* talk;
  const float* sink;
  float* part_acc;
  float* part_ml;
  int q_stride, out_stride, bt_stride;
  int nh, nkv, gs, block_size;
  int tq, mtc;  // queries per CTA, m-tiles per kv head
  int window, split_size, max_splits;
  float scale;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// a float as two bfloat16 terms: the rounded number and the rounded rest
__device__ __forceinline__ void split_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const __nv_bfloat162 l = __floats2bfloat162_rn(a - __low2float(h), b - __high2float(h));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}
// byte offset of the 16-byte chunk `chunk` of row `row` in a swizzled [rows][D] bfloat16 tile
template <int D> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// Where the keys [t0, t0 + BN) lie: koff[key] = (page * nkv * block_size + place in the page) in keys, or -1 for a
// key at or past `ctx` or in a page that was given back.  Written by the first BN threads.
template <int BN>
__device__ __forceinline__ void locate_keys(const int* bt, int t0, int ctx, int nkv, int block_size, int* koff) {
  if (threadIdx.x < BN) {
    const int kp = t0 + threadIdx.x;
    int off = -1;
    if (kp < ctx) {
      const int pg = kp / block_size;
      const int blk = bt[pg];
      if (blk >= 0) off = blk * nkv * block_size + (kp - pg * block_size);
    }
    koff[threadIdx.x] = off;
  }
}

// The keys that `koff` locates, of every kv head, into one swizzled tile a head; keys that are not there are zeros.
template <int D, int BN>
__device__ __forceinline__ void load_tiles(const bf16* cache, const int* koff, int nkv, int block_size, uint32_t dst) {
  constexpr int CH = D / 8;
  const int chunk = threadIdx.x % CH;
  const int key0 = threadIdx.x / CH;
  constexpr int KSTEP = NW * 32 / CH;  // keys between a thread's chunks of one head
  static_assert(BN % KSTEP == 0 || KSTEP % BN == 0, "tile and CTA sizes");
  if (KSTEP <= BN) {
    for (int c = 0; c < nkv; ++c) {
#pragma unroll
      for (int key = key0; key < BN; key += KSTEP) {
        const int off = koff[key];
        const bool valid = off >= 0;
        const size_t base = valid ? ((size_t)off + (size_t)c * block_size) * D + chunk * 8 : 0;
        cp_async16(dst + (uint32_t)c * (BN * D * 2) + tile_off<D>(key, chunk), cache + base, valid);
      }
    }
  } else {  // a pass of the CTA covers several heads
    constexpr int HEADS = KSTEP / BN;
    const int key = key0 % BN, c0 = key0 / BN;
    const int off = koff[key];
    const bool valid = off >= 0;
    for (int c = c0; c < nkv; c += HEADS) {
      const size_t base = valid ? ((size_t)off + (size_t)c * block_size) * D + chunk * 8 : 0;
      cp_async16(dst + (uint32_t)c * (BN * D * 2) + tile_off<D>(key, chunk), cache + base, valid);
    }
  }
}

// S' = talk x S over the source heads in order, for the warp's columns; C columns a lane.
template <int BN, int BNP, int C>
__device__ __forceinline__ void mix_heads(const float* Ss, float* Ps, const float* Tt, int nh, int nhp, int tq, int warp, int lane) {
  const int per_h = tq * BNP;
  const int groups = tq * BN / (32 * C);
  const int items = (nhp / HC) * groups;
  for (int it = warp; it < items; it += NW) {
    const int chunk = it / groups, grp = it - chunk * groups;
    int off[C];
#pragma unroll
    for (int k = 0; k < C; ++k) {
      const int col = (grp * C + k) * 32 + lane;
      off[k] = (col / BN) * BNP + (col % BN);
    }
    float2 acc[C][HC / 2];  // pairs of neighbouring target heads: one packed FMA moves both
#pragma unroll
    for (int k = 0; k < C; ++k)
#pragma unroll
      for (int e = 0; e < HC / 2; ++e) acc[k][e] = make_float2(0.f, 0.f);
    const float* trow = Tt + chunk * HC;
    for (int g = 0; g < nh; ++g) {
      const float4 ta = *reinterpret_cast<const float4*>(trow + g * nhp);
      const float4 tb = *reinterpret_cast<const float4*>(trow + g * nhp + 4);
      const float2 t0 = make_float2(ta.x, ta.y), t1 = make_float2(ta.z, ta.w), t2 = make_float2(tb.x, tb.y), t3 = make_float2(tb.z, tb.w);
      const float* srow = Ss + g * per_h;
#pragma unroll
      for (int k = 0; k < C; ++k) {
        const float s = srow[off[k]];
        const float2 s2 = make_float2(s, s);
        acc[k][0] = __ffma2_rn(t0, s2, acc[k][0]);
        acc[k][1] = __ffma2_rn(t1, s2, acc[k][1]);
        acc[k][2] = __ffma2_rn(t2, s2, acc[k][2]);
        acc[k][3] = __ffma2_rn(t3, s2, acc[k][3]);
      }
    }
#pragma unroll
    for (int e = 0; e < HC; ++e) {
      const int h = chunk * HC + e;
      if (h < nh) {
#pragma unroll
        for (int k = 0; k < C; ++k) Ps[h * per_h + off[k]] = (e & 1) ? acc[k][e / 2].y : acc[k][e / 2].x;
      }
    }
  }
}

template <int D, int BN, int MT, bool SPLIT>
__global__ void __launch_bounds__(NW * 32, (D == 64 && BN == 32 && MT == 1) ? 2 : 1) talking_mma_kernel(const Params p) {
  pdl_launch();
  pdl_wait();
  constexpr int BNP = BN + 8;  // row stride of the score tiles: rows eight apart fall into other banks
  constexpr int NT = BN / 8;
  constexpr int ND = D / 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int nh = p.nh, nkv = p.nkv, gs = p.gs, tq = p.tq;
  const int nhp = (nh + HC - 1) / HC * HC;
  const int per_h = tq * BNP;
  unsigned char* Kb = smem_raw;                                   // [nkv][BN][D] bfloat16, swizzled
  unsigned char* Vb = Kb + (size_t)nkv * BN * D * 2;
  float* Ss = reinterpret_cast<float*>(Vb + (size_t)nkv * BN * D * 2);  // [nh][tq][BNP]
  float* Ps = p.talk ? Ss + (size_t)nh * per_h : Ss;
  float* Tt = Ps + (size_t)nh * per_h;                            // [nh][nhp]: Tt[g][h] = talk[h][g]
  int* koff = reinterpret_cast<int*>(Tt + (p.talk ? (size_t)nh * nhp : 0));  // [2][BN]: where a tile's keys lie
  const uint32_t kb = smem_u32(Kb), vb = smem_u32(Vb);

  const int b = blockIdx.y;
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
    q0 = (gridDim.x - 1 - blockIdx.x) * tq;  // the queries with the most keys first
    if (q0 >= q_len) return;
    n_tok = min(tq, q_len - q0);
    kv_lo = 0;
    kv_hi = ctx - q_len + q0 + n_tok;
  }
  const int* bt = p.block_tables + (size_t)b * p.bt_stride;

  locate_keys<BN>(bt, kv_lo, ctx, nkv, p.block_size, koff);
  if (p.talk)
    for (int idx = threadIdx.x; idx < nh * nhp; idx += NW * 32) {
      const int g = idx / nhp, h = idx - g * nhp;
      Tt[idx] = h < nh ? p.talk[(size_t)h * nh + g] : 0.f;
    }
  __syncthreads();
  load_tiles<D, BN>(p.kcache, koff, nkv, p.block_size, kb);
  cp_async_commit();

  // ---- the rows this warp owns: m-tile mt = warp + k * NW of kv head mt / mtc; a thread holds rows lane/4 and lane/4 + 8
  const int n_mt = nkv * p.mtc;
  const int rows_c = gs * tq;  // rows of one kv head before padding
  int kvh[MT], srow[MT][2], pos[MT][2], head[MT][2];
  uint32_t qf[MT][D / 16][4];
  float m[MT][2], l[MT][2], o[MT][ND][4];
  const bool with_sink = p.sink != nullptr && (!SPLIT || blockIdx.x == 0);
#pragma unroll
  for (int k = 0; k < MT; ++k) {
    const int mt = warp + k * NW;
    const bool live = mt < n_mt;
    kvh[k] = live ? mt / p.mtc : -1;
    const int lt = live ? mt - kvh[k] * p.mtc : 0;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int lr = lt * 16 + (lane >> 2) + 8 * rr;
      const bool in_rows = live && lr < rows_c;
      const int hl = in_rows ? lr / tq : 0, qi = in_rows ? lr - hl * tq : 0;
      head[k][rr] = in_rows ? kvh[k] * gs + hl : -1;
      srow[k][rr] = in_rows ? (head[k][rr] * tq + qi) * BNP : -1;
      const bool valid = in_rows && qi < n_tok;
      pos[k][rr] = valid ? ctx - q_len + q0 + qi : -1;  // -1: sees nothing, writes nothing
      m[k][rr] = (valid && with_sink) ? p.sink[head[k][rr]] * LOG2E : -INFINITY;
      l[k][rr] = (valid && with_sink) ? 1.f : 0.f;
      const bf16* qrow = p.q + (size_t)(q_begin + q0 + qi) * p.q_stride + (size_t)(in_rows ? head[k][rr] : 0) * D + (lane & 3) * 2;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        qf[k][kk][rr] = valid ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16) : 0u;
        qf[k][kk][rr + 2] = valid ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8) : 0u;
      }
    }
#pragma unroll
    for (int nd = 0; nd < ND; ++nd)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[k][nd][e] = 0.f;
  }
  const float scale2 = p.scale * LOG2E;  // scores in units of log 2: the mixing is linear, so the factor may come first

  int cur = 0;
  for (int t0 = kv_lo; t0 < kv_hi; t0 += BN, cur ^= 1) {
    cp_async_wait<0>();
    __syncthreads();  // the key tiles have landed; the value tiles and score tiles of the tile before are consumed
    load_tiles<D, BN>(p.vcache, koff + cur * BN, nkv, p.block_size, vb);
    cp_async_commit();
    const bool more = t0 + BN < kv_hi;
    if (more) locate_keys<BN>(bt, t0 + BN, ctx, nkv, p.block_size, koff + (cur ^ 1) * BN);
    // ---- 1. scores
#pragma unroll
    for (int k = 0; k < MT; ++k) {
      if (kvh[k] < 0) continue;  // warp-uniform
      float s[NT][4];
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
      const uint32_t ks = kb + (uint32_t)kvh[k] * (BN * D * 2);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t bb[4];
          const int key = j * 8 + ((lane >> 4) << 3) + (lane & 7);
          const int chunk = 2 * kk + ((lane >> 3) & 1);
          ldmatrix_x4(bb, ks + tile_off<D>(key, chunk));
          mma_16816(s[j], qf[k][kk], bb[0], bb[1]);
          mma_16816(s[j + 1], qf[k][kk], bb[2], bb[3]);
        }
      }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (srow[k][rr] < 0) continue;
        float* dst = Ss + srow[k][rr] + (lane & 3) * 2;
#pragma unroll
        for (int j = 0; j < NT; ++j)
          *reinterpret_cast<float2*>(dst + j * 8) = make_float2(s[j][2 * rr] * scale2, s[j][2 * rr + 1] * scale2);
      }
    }
    __syncthreads();  // every head's scores are written; the key tiles are consumed
    if (more) {
      load_tiles<D, BN>(p.kcache, koff + (cur ^ 1) * BN, nkv, p.block_size, kb);
      cp_async_commit();
    }
    // ---- 2. the heads talk
    if (p.talk) {  // as many columns a lane as still leave every warp an item
      const int cols32 = tq * BN / 32, chunks = nhp / HC;
      if (cols32 % 4 == 0 && chunks * (cols32 / 4) >= NW)
        mix_heads<BN, BNP, 4>(Ss, Ps, Tt, nh, nhp, tq, warp, lane);
      else if (cols32 % 2 == 0 && chunks * (cols32 / 2) >= NW)
        mix_heads<BN, BNP, 2>(Ss, Ps, Tt, nh, nhp, tq, warp, lane);
      else
        mix_heads<BN, BNP, 1>(Ss, Ps, Tt, nh, nhp, tq, warp, lane);
    }
    if (more)
      cp_async_wait<1>();
    else
      cp_async_wait<0>();
    __syncthreads();  // mixed scores and value tiles are there
    // ---- 3. softmax step and O += P V
#pragma unroll
    for (int k = 0; k < MT; ++k) {
      if (kvh[k] < 0) continue;  // warp-uniform
      float pr[NT][4];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const float* src = Ps + (srow[k][rr] < 0 ? 0 : srow[k][rr]) + (lane & 3) * 2;
        const int ps = pos[k][rr];
        float mx = -INFINITY;
        if (ps >= t0 + BN - 1 && t0 + BN <= kv_hi && p.window <= 0) {  // the row sees the whole tile
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            const float2 v = *reinterpret_cast<const float2*>(src + j * 8);
            pr[j][2 * rr] = v.x;
            pr[j][2 * rr + 1] = v.y;
            mx = fmaxf(mx, fmaxf(v.x, v.y));
          }
        } else {
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            const float2 v = ps >= 0 ? *reinterpret_cast<const float2*>(src + j * 8) : make_float2(0.f, 0.f);
            const int key = t0 + j * 8 + (lane & 3) * 2;
            bool v0 = key <= ps && key < kv_hi, v1 = key + 1 <= ps && key + 1 < kv_hi;
            if (p.window > 0) {
              v0 = v0 && key > ps - p.window;
              v1 = v1 && key + 1 > ps - p.window;
            }
            pr[j][2 * rr] = v0 ? v.x : -INFINITY;
            pr[j][2 * rr + 1] = v1 ? v.y : -INFINITY;
            mx = fmaxf(mx, fmaxf(pr[j][2 * rr], pr[j][2 * rr + 1]));
          }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[k][rr], mx);
        float corr = 1.f, sum = 0.f;
        if (m_new == -INFINITY) {
#pragma unroll
          for (int j = 0; j < NT; ++j) pr[j][2 * rr] = pr[j][2 * rr + 1] = 0.f;
        } else {
          corr = ex2(m[k][rr] - m_new);
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            pr[j][2 * rr] = ex2(pr[j][2 * rr] - m_new);
            pr[j][2 * rr + 1] = ex2(pr[j][2 * rr + 1] - m_new);
            sum += pr[j][2 * rr] + pr[j][2 * rr + 1];
          }
          m[k][rr] = m_new;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[k][rr] = l[k][rr] * corr + sum;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
          o[k][nd][2 * rr] *= corr;
          o[k][nd][2 * rr + 1] *= corr;
        }
      }
      const uint32_t vs = vb + (uint32_t)kvh[k] * (BN * D * 2);
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
        uint32_t ah[4], al[4];
        split_pair(pr[2 * ks][0], pr[2 * ks][1], ah[0], al[0]);
        split_pair(pr[2 * ks][2], pr[2 * ks][3], ah[1], al[1]);
        split_pair(pr[2 * ks + 1][0], pr[2 * ks + 1][1], ah[2], al[2]);
        split_pair(pr[2 * ks + 1][2], pr[2 * ks + 1][3], ah[3], al[3]);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
          uint32_t bb[4];
          const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
          const int chunk = 2 * dp + (lane >> 4);
          ldmatrix_x4_trans(bb, vs + tile_off<D>(key, chunk));
          mma_16816(o[k][2 * dp], ah, bb[0], bb[1]);
          mma_16816(o[k][2 * dp + 1], ah, bb[2], bb[3]);
          mma_16816(o[k][2 * dp], al, bb[0], bb[1]);
          mma_16816(o[k][2 * dp + 1], al, bb[2], bb[3]);
        }
      }
    }
  }

  // ---- write
#pragma unroll
  for (int k = 0; k < MT; ++k) {
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      if (pos[k][rr] < 0) continue;
      const int h = head[k][rr];
      if (SPLIT) {
        const size_t slot = ((size_t)b * nh + h) * p.max_splits + blockIdx.x;
        if ((lane & 3) == 0) {
          p.part_ml[slot * 2] = m[k][rr] * (1.f / LOG2E);  // back to natural units: the merge uses expf
          p.part_ml[slot * 2 + 1] = l[k][rr];
        }
        float* dst = p.part_acc + slot * D + (lane & 3) * 2;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) *reinterpret_cast<float2*>(dst + nd * 8) = make_float2(o[k][nd][2 * rr], o[k][nd][2 * rr + 1]);
      } else {
        const int qi = (srow[k][rr] / BNP) - h * tq;
        const float inv = l[k][rr] > 0.f ? 1.f / l[k][rr] : 0.f;
        bf16* dst = p.out + (size_t)(q_begin + q0 + qi) * p.out_stride + (size_t)h * D + (lane & 3) * 2;
#pragma unroll
        for (int nd = 0; nd < ND; ++nd)
          *reinterpret_cast<__nv_bfloat162*>(dst + nd * 8) = __floats2bfloat162_rn(o[k][nd][2 * rr] * inv, o[k][nd][2 * rr + 1] * inv);
      }
    }
  }
}

struct Plan {
  int tq, mtc, bn, mt;
  size_t smem;
};

inline size_t smem_need(int nh, int nkv, int d, int tq, int bn, bool talk) {
  const int nhp = (nh + HC - 1) / HC * HC;
  return (size_t)2 * nkv * bn * d * 2 + (size_t)(talk ? 2 : 1) * nh * tq * (bn + 8) * 4 + (talk ? (size_t)nh * nhp * 4 : 0) + (size_t)2 * bn * 4;
}

// The most queries a CTA that fit: every m-tile has a warp (two a warp for heads of 64), everything in shared memory.
inline bool make_plan(int nh, int nkv, int d, int dv, bool split, int max_q_len, bool talk, Plan& pl) {
  if (d != dv || (d != 64 && d != 128) || nkv <= 0 || nh % nkv != 0 || nh > NW * MAXR) return false;
  const int gs = nh / nkv;
  const int mt_most = d == 64 ? 2 : 1;
  int bn = (d == 64 && !split) ? 64 : 32;
  int tq_first = split ? 1 : 16;
  while (tq_first > 1 && tq_first / 2 >= max_q_len) tq_first /= 2;
  for (int tq = tq_first; tq >= 1; tq /= 2) {
    const int mtc = (gs * tq + 15) / 16;
    const int n_mt = nkv * mtc;
    if (n_mt > NW * mt_most) continue;
    const size_t need = smem_need(nh, nkv, d, tq, bn, talk);
    if (need > SMEM_MOST) continue;
    pl.tq = tq; pl.mtc = mtc; pl.bn = bn; pl.mt = (n_mt + NW - 1) / NW; pl.smem = need;
    // heads of 64, one m-tile a warp: with tiles of 32 keys two CTAs share an SM (one mixes while the other multiplies)
    if (bn == 64 && pl.mt == 1 && smem_need(nh, nkv, d, tq, 32, talk) <= TWO_CTAS) {
      pl.bn = 32;
      pl.smem = smem_need(nh, nkv, d, tq, 32, talk);
    }
    return true;
  }
  return false;
}

template <int D, int BN, int MT, bool SPLIT>
int launch_mma(const Params& p, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = talking_mma_kernel<D, BN, MT, SPLIT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, grid, dim3(NW * 32), smem, st, p);
}

}  // namespace tmma
}  // namespace

// 1 when the tensor-core form takes this shape (bfloat16 storage), 0 when the FP32-pipe form has to.
KVF_API int kvf_talking_mma_ok(int nh, int nkv, int d, int dv, int split, int with_talk) {
  tmma::Plan pl;
  return tmma::make_plan(nh, nkv, d, dv, split != 0, split ? 1 : 16, with_talk != 0, pl) &&
                 tmma::make_plan(nh, nkv, d, dv, split != 0, 1, with_talk != 0, pl)
             ? 1
             : 0;
}

KVF_API int kvf_talking_attention_mma_bf16(
    const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables, const int* qsl,
    const int* ctx_lens, const float* talk, const float* sink, int B, int max_q_len, int q_stride, int out_stride,
    int bt_stride, int nh, int nkv, int d, int dv, int block_size, float scale, int window, int split_size,
    int max_splits, int grid_splits, float* part_acc, float* part_ml, cudaStream_t st) {
  using namespace tmma;
  if (B <= 0 || max_q_len <= 0) return 0;
  const bool split = split_size > 0;
  Plan pl;
  if (block_size <= 0 || (unsigned)B > 65535u || (q_stride % 2) != 0 || (out_stride % 2) != 0 ||
      !make_plan(nh, nkv, d, dv, split, max_q_len, talk != nullptr, pl))
    return (int)cudaErrorInvalidValue;
  if (split && (split_size % pl.bn != 0 || max_splits <= 0 || !part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
  Params p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache;
  p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens; p.talk = talk; p.sink = sink;
  p.part_acc = part_acc; p.part_ml = part_ml;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.nkv = nkv; p.gs = nh / nkv; p.block_size = block_size;
  p.tq = pl.tq; p.mtc = pl.mtc; p.window = window; p.split_size = split_size; p.max_splits = max_splits; p.scale = scale;
  int rc;
  if (split) {
    dim3 grid(grid_splits > 0 && grid_splits < max_splits ? grid_splits : max_splits, B);
    if (d == 64)
      rc = pl.mt == 1 ? launch_mma<64, 32, 1, true>(p, grid, pl.smem, st) : launch_mma<64, 32, 2, true>(p, grid, pl.smem, st);
    else
      rc = launch_mma<128, 32, 1, true>(p, grid, pl.smem, st);
    if (rc) return rc;
    return launch(talking_combine_kernel<bf16>, dim3(nh, B), dim3(64), 0, st, (const float*)part_acc, (const float*)part_ml,
                  (bf16*)out, qsl, ctx_lens, nh, dv, out_stride, split_size, max_splits);
  }
  dim3 grid((max_q_len + pl.tq - 1) / pl.tq, B);
  if (d == 64 && pl.bn == 32) return launch_mma<64, 32, 1, false>(p, grid, pl.smem, st);
  if (d == 64)
    return pl.mt == 1 ? launch_mma<64, 64, 1, false>(p, grid, pl.smem, st) : launch_mma<64, 64, 2, false>(p, grid, pl.smem, st);
  return launch_mma<128, 32, 1, false>(p, grid, pl.smem, st);
}
