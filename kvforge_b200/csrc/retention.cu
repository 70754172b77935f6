// Retention: linear attention with one fixed decay a head, no softmax and no denominator.
//
//   S_t = a_h S_(t-1) + k_t v_t^T        (S: [dk][dv] floats per head, in the request's state slot)
//   o_t = S_t^T q_t
//
// q and k turn with the position on their first `rot` dims (pairs (i, i + rot/2), or (2i, 2i+1)); k is then
// multiplied by k_scale.  Everything from the rotation on is float whatever the storage type T of the projections.
//
//   prepare : a warp per (token, head of q, k or v): rotation, scaling, widening to float.  Nothing here depends
//             on the state, so it runs over all tokens at once.
//   walk    : a CTA owns (sequence, head, tile of CT value columns) and walks the sequence's tokens in order.  A
//             column's dk rows are spread over KS neighbouring lanes, R rows each in registers (in runs of four: rows
//             4 (j KS + s) .. + 3 for lane s, so that q and k come from shared memory four at a time).  Per token a
//             lane makes  S <- a S + k v  and its part of  S^T q  in one pass; the parts are added in a tree whose
//             shape follows dk alone.  Chunks of TC tokens come in through a cp.async double buffer; the state tile passes through
//             shared memory so that global memory sees whole rows.
//   gate    : every head's read-out divided by its root mean square and multiplied by act(gate).
//
// The state after a token is the same bits however the sequence was cut into steps (the walk is token by token,
// and every sum has an order fixed by dk alone, however many rows a lane holds), so a token's output does not
// depend on the cut, the batch or the slot.  A sequence without rows, or with a slot below zero (padding), touches nothing.
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int TC = 16;  // tokens per chunk of the walk, at most

template <typename T>
__global__ void __launch_bounds__(128) retention_prepare_kernel(const T* __restrict__ x, long long x_stride, int q_off, int k_off,
                                                                 int v_off, const int* __restrict__ positions,
                                                                 const float* __restrict__ inv_freq, int rot, int split_pairs,
                                                                 float k_scale, long long n_tokens, int H, int dk, int dv,
                                                                 float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vn) {
  pdl_launch();
  pdl_wait();
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= n_tokens * 3 * H) return;
  const long long n = unit / (3 * H);
  const int u = (int)(unit - n * 3 * H), kind = u / H, h = u - kind * H;
  const int lane = threadIdx.x & 31;
  const T* row = x + (size_t)n * x_stride;
  if (kind == 2) {
    const T* src = row + v_off + (size_t)h * dv;
    float* dst = vn + ((size_t)n * H + h) * dv;
    for (int j = lane; j < dv; j += 32) dst[j] = to_float<T>(src[j]);
    return;
  }
  const T* src = row + (kind == 0 ? q_off : k_off) + (size_t)h * dk;
  float* dst = (kind == 0 ? qn : kn) + ((size_t)n * H + h) * dk;
  const float mul = kind == 0 ? 1.f : k_scale;
  const float pos = (float)positions[n];
  for (int i = lane; i < dk / 2; i += 32) {
    const bool turns = 2 * i < rot;
    const int ia = (turns && split_pairs) ? i : 2 * i, ib = (turns && split_pairs) ? i + rot / 2 : 2 * i + 1;
    float a = to_float<T>(src[ia]), b = to_float<T>(src[ib]);
    if (turns) {
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      float ya, yb;
      rotate_pair(a, b, cs, sn, ya, yb);
      a = ya;
      b = yb;
    }
    dst[ia] = a * mul;
    dst[ib] = b * mul;
  }
  if ((dk & 1) && lane == 0) dst[dk - 1] = to_float<T>(src[dk - 1]) * mul;
}

__device__ __forceinline__ void cp_async(float* dst, const float* src, bool wide) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  if (wide)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}

// R rows a lane (a multiple of four); blockDim.x = KS * CT (a multiple of 32, at most 256); KS a power of two, at most 32.
// The sum over a column's rows has one order whatever R is: runs of four rows are added in order, and the runs are then
// added in a binary tree that joins the halves of the (padded) row range first and neighbouring runs last; a lane's own runs
// are the upper levels of that tree and the shuffles over the KS lanes the lower ones.  So R can follow the batch (few
// sequences: fewer rows a lane and more lanes) without changing a bit of the result.
template <int R>
__global__ void __launch_bounds__(256) retention_walk_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
                                                              const float* __restrict__ vn, const float* __restrict__ decay,
                                                              float* __restrict__ state, long long state_stride,
                                                              float* __restrict__ out, long long out_stride,
                                                              const int* __restrict__ qsl, const int* __restrict__ state_slots,
                                                              int H, int dk, int dv, int KS, int CT, int tc) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  constexpr int NJ = R / 4;  // runs of four rows a lane
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * CT;
  const int q_begin = qsl[b], q_len = qsl[b + 1] - q_begin;
  const int slot = state_slots[b];
  if (q_len <= 0 || slot < 0) return;
  const int dkp = KS * R, tid = threadIdx.x, nthreads = blockDim.x;
  const int s = tid & (KS - 1), col = tid / KS;
  const int ncol = min(CT, dv - c0);
  const int lds = CT + 1;
  float* St = sm;                       // [dkp][CT + 1]: the state tile on its way in and out
  const int st_floats = (dkp * lds + 3) & ~3;
  // tc tokens a chunk (16, or as many as the step's longest sequence brings when that is fewer)
  const int stage = tc * (2 * dkp + CT);  // q [tc][dkp], k [tc][dkp], v [tc][CT]
  float* buf = sm + st_floats;
  const float a = decay[h];

  float* sbase = state + (size_t)slot * state_stride + (size_t)h * dk * dv + c0;
  // whole tiles of whole rows go four numbers at a time
  const bool tile4 = dkp == dk && ncol == CT && (CT & 3) == 0 && (dv & 3) == 0 && (((uintptr_t)sbase) & 15) == 0;
  if (tile4) {
    const int c4 = CT >> 2;
    for (int idx = tid; idx < dk * c4; idx += nthreads) {
      const int r = idx / c4, c = (idx - r * c4) << 2;
      const float4 t4 = *reinterpret_cast<const float4*>(sbase + (size_t)r * dv + c);
      float* d = St + r * lds + c;
      d[0] = t4.x; d[1] = t4.y; d[2] = t4.z; d[3] = t4.w;
    }
  } else {
    for (int idx = tid; idx < dkp * CT; idx += nthreads) {
      const int r = idx / CT, c = idx - r * CT;
      St[r * lds + c] = (r < dk && c < ncol) ? sbase[(size_t)r * dv + c] : 0.f;
    }
    // what no copy ever writes is zero for good: rows of q and k beyond dk, value columns beyond the tile's
    for (int idx = tid; idx < 2 * stage; idx += nthreads) buf[idx] = 0.f;
  }
  __syncthreads();
  // register i of lane s holds row ((i / 4) * KS + s) * 4 + i % 4: run i / 4 of the lane is run (i / 4) * KS + s of the column
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = St[(((i >> 2) * KS + s) * 4 + (i & 3)) * lds + col];

  const bool wide_qk = (dk & 3) == 0, wide_v = (dv & 3) == 0 && (c0 & 3) == 0 && (ncol & 3) == 0;
  auto issue = [&](int chunk) {
    float* bq = buf + (chunk & 1) * stage;
    float* bk = bq + tc * dkp;
    float* bv = bk + tc * dkp;
    const int t0 = chunk * tc, nt = min(tc, q_len - t0);
    const int per = wide_qk ? dk / 4 : dk;
    for (int idx = tid; idx < nt * per; idx += nthreads) {
      const int t = idx / per, j = (idx - t * per) * (wide_qk ? 4 : 1);
      const size_t g = ((size_t)(q_begin + t0 + t) * H + h) * dk + j;
      cp_async(bq + t * dkp + j, qn + g, wide_qk);
      cp_async(bk + t * dkp + j, kn + g, wide_qk);
    }
    const int perv = wide_v ? ncol / 4 : ncol;
    for (int idx = tid; idx < nt * perv; idx += nthreads) {
      const int t = idx / perv, j = (idx - t * perv) * (wide_v ? 4 : 1);
      cp_async(bv + t * CT + j, vn + ((size_t)(q_begin + t0 + t) * H + h) * dv + c0 + j, wide_v);
    }
  };

  const int nchunks = (q_len + tc - 1) / tc;
  issue(0);
  asm volatile("cp.async.commit_group;\n" ::);
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) issue(c + 1);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    const float* bq = buf + (c & 1) * stage;
    const float* bk = bq + tc * dkp;
    const float* bv = bk + tc * dkp;
    const int t0 = c * tc, nt = min(tc, q_len - t0);
    float* orow = out + (size_t)(q_begin + t0) * out_stride + (size_t)h * dv + c0 + col;
    const float4* q = reinterpret_cast<const float4*>(bq) + s;
    const float4* k = reinterpret_cast<const float4*>(bk) + s;
    const float* v = bv + col;
    const bool writes = s == 0 && col < ncol;
#pragma unroll(R >= 32 ? 2 : 4)
    for (int t = 0; t < nt; ++t) {
      const float vv = *v;
      float pg[NJ];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float4 k4 = k[j * KS], q4 = q[j * KS];
        S[4 * j] = fmaf(a, S[4 * j], __fmul_rn(k4.x, vv));
        S[4 * j + 1] = fmaf(a, S[4 * j + 1], __fmul_rn(k4.y, vv));
        S[4 * j + 2] = fmaf(a, S[4 * j + 2], __fmul_rn(k4.z, vv));
        S[4 * j + 3] = fmaf(a, S[4 * j + 3], __fmul_rn(k4.w, vv));
        pg[j] = fmaf(S[4 * j + 3], q4.w, fmaf(S[4 * j + 2], q4.z, fmaf(S[4 * j + 1], q4.y, __fmul_rn(S[4 * j], q4.x))));
      }
#pragma unroll
      for (int half = NJ / 2; half > 0; half >>= 1) {
#pragma unroll
        for (int j = 0; j < half; ++j) pg[j] = __fadd_rn(pg[j], pg[j + half]);
      }
      float p = pg[0];
      // the lanes' parts, the halves of the row range first; levels a column has no lanes for are skipped (KS is one for the CTA)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        if (o < KS) p = __fadd_rn(p, __shfl_xor_sync(0xffffffffu, p, o));
      if (writes) *orow = p;
      q += dkp / 4;
      k += dkp / 4;
      v += CT;
      orow += out_stride;
    }
    __syncthreads();  // the chunk is used up: the copy after next may overwrite it
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
  for (int i = 0; i < R; ++i) St[(((i >> 2) * KS + s) * 4 + (i & 3)) * lds + col] = S[i];
  __syncthreads();
  if (tile4) {
    const int c4 = CT >> 2;
    for (int idx = tid; idx < dk * c4; idx += nthreads) {
      const int r = idx / c4, c = (idx - r * c4) << 2;
      const float* d = St + r * lds + c;
      *reinterpret_cast<float4*>(sbase + (size_t)r * dv + c) = make_float4(d[0], d[1], d[2], d[3]);
    }
    return;
  }
  for (int idx = tid; idx < dk * ncol; idx += nthreads) {
    const int r = idx / ncol, c = idx - r * ncol;
    sbase[(size_t)r * dv + c] = St[r * lds + c];
  }
}

// What follows the walk: every head's read-out divided by its root mean square (no weight) and multiplied by
// act(gate), a warp per (token, head).  act: 0 none, 1 silu, 2 the logistic function; float arithmetic, one rounding.
template <typename T>
__global__ void __launch_bounds__(128) retention_gate_kernel(const float* __restrict__ o, long long o_stride, const T* __restrict__ gate,
                                                              long long gate_stride, float eps, int act, long long pairs, int H, int dv,
                                                              T* __restrict__ out, long long out_stride) {
  pdl_launch();
  pdl_wait();
  const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long n = pair / H;
  const int h = (int)(pair - n * H);
  const float* row = o + (size_t)n * o_stride + (size_t)h * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  const T* g = gate ? gate + (size_t)n * gate_stride + (size_t)h * dv : nullptr;
  T* dst = out + (size_t)n * out_stride + (size_t)h * dv;
  for (int j = lane; j < dv; j += 32) {
    float y = row[j] * inv;
    if (act) {
      const float z = to_float<T>(g[j]), sg = 1.f / (1.f + expf(-z));
      y *= act == 1 ? z * sg : sg;
    }
    dst[j] = from_float<T>(y);
  }
}

inline int pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

template <int R>
int launch_walk(const float* qn, const float* kn, const float* vn, const float* decay, float* state, long long state_stride, float* out,
                long long out_stride, const int* qsl, const int* state_slots, int B, int H, int dk, int dv, int tc, cudaStream_t st) {
  const int KS = pow2_at_least((dk + R - 1) / R);
  if (KS > 32) return (int)cudaErrorInvalidValue;
  int CT = (R >= 32 ? 128 : 256) / KS;  // 32 rows a lane take 128 registers: smaller CTAs fit an SM better
  const int cols = pow2_at_least(dv);
  if (CT > cols) CT = cols;
  if (CT * KS < 32) CT = 32 / KS;
  // few (sequence, head) pairs: narrower tiles, so that there are CTAs for every SM
  while (CT * KS > 64 && CT > 4 && (long long)B * H * ((dv + CT - 1) / CT) < 148) CT >>= 1;
  const int dkp = KS * R;
  const size_t smem = (size_t)(((dkp * (CT + 1) + 3) & ~3) + 2 * tc * (2 * dkp + CT)) * sizeof(float);
  auto kern = retention_walk_kernel<R>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, dim3((dv + CT - 1) / CT, H, B), dim3(KS * CT), smem, st, qn, kn, vn, decay, state, state_stride, out, out_stride,
                qsl, state_slots, H, dk, dv, KS, CT, tc);
}

// Rows a lane: as many (up to 32) as still leave a warp for every warp scheduler of the device; a state of few heads in a
// step of few sequences is spread thin instead, since the walk over a sequence is a chain that only other lanes can hide
// (one sequence of 2,048 tokens, 16 heads of 128 x 128: 536 us with 32 rows a lane, 460 us with 16 or 8, 480 us with 4;
// eight sequences of 256 tokens: 219, 244, 247 and 336 us).
inline int rows_per_lane(int B, int H, int dk, int dv) {
  int best = 32;
  for (int r = 32; r >= 4; r >>= 1) {
    if ((dk + r - 1) / r > 32) break;  // more lanes a column than a warp has
    best = r;
    if ((long long)B * H * dv * pow2_at_least((dk + r - 1) / r) / 32 >= 4 * 148) break;
  }
  return best;
}

}  // namespace

// x: rows of the projections (q heads from q_off, k heads from k_off, v heads from v_off; H heads each of dk, dk, dv).
// qn, kn [N][H*dk] and vn [N][H*dv]: float scratch.  state: float, slot i at state + i * state_stride, [H][dk][dv].
// out: float [N][H*dv] (row stride out_stride).  decay: float [H].  max_q_len: the most rows a sequence of the step brings
// (0: unknown); a step of single tokens stages one token, not sixteen.  Two launches.
#define KVF_RETENTION_API(SUF, T)                                                                                       \
  KVF_API int kvf_retention_##SUF(const void* x, long long x_stride, int q_off, int k_off, int v_off,                   \
                                  const int* positions, const float* inv_freq, int rot, int split_pairs,                \
                                  float k_scale, const float* decay, float* state, long long state_stride, float* out,  \
                                  long long out_stride, const int* qsl, const int* state_slots, int B, long long N,     \
                                  int H, int dk, int dv, float* qn, float* kn, float* vn, int max_q_len,                \
                                  cudaStream_t st) {                                                                    \
    if (B <= 0 || N <= 0) return 0;                                                                                     \
    if (H <= 0 || dk <= 0 || dk > 512 || dv <= 0 || rot < 0 || rot > dk || (rot & 1) || (unsigned)B > 65535u ||         \
        (unsigned)H > 65535u)                                                                                           \
      return (int)cudaErrorInvalidValue;                                                                                \
    const long long units = N * 3 * H;                                                                                  \
    int rc = launch(retention_prepare_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, st, (const T*)x,      \
                    x_stride, q_off, k_off, v_off, positions, inv_freq, rot, split_pairs, k_scale, N, H, dk, dv, qn,    \
                    kn, vn);                                                                                            \
    if (rc) return rc;                                                                                                  \
    const int r = rows_per_lane(B, H, dk, dv);                                                                          \
    const int tc = max_q_len > 0 && max_q_len < TC ? max_q_len : TC;                                                    \
    if (r == 4)                                                                                                         \
      return launch_walk<4>(qn, kn, vn, decay, state, state_stride, out, out_stride, qsl, state_slots, B, H, dk, dv,    \
                            tc, st);                                                                                        \
    if (r == 8)                                                                                                         \
      return launch_walk<8>(qn, kn, vn, decay, state, state_stride, out, out_stride, qsl, state_slots, B, H, dk, dv,    \
                            tc, st);                                                                                        \
    if (r == 16)                                                                                                        \
      return launch_walk<16>(qn, kn, vn, decay, state, state_stride, out, out_stride, qsl, state_slots, B, H, dk, dv,   \
                             tc, st);                                                                                       \
    return launch_walk<32>(qn, kn, vn, decay, state, state_stride, out, out_stride, qsl, state_slots, B, H, dk, dv,     \
                           tc, st);                                                                                         \
  }

#define KVF_RETENTION_GATE_API(SUF, T)                                                                                  \
  KVF_API int kvf_retention_gate_##SUF(const float* o, long long o_stride, const void* gate, long long gate_stride,     \
                                       float eps, int act, long long N, int H, int dv, void* out, long long out_stride, \
                                       cudaStream_t st) {                                                               \
    const long long pairs = N * H;                                                                                      \
    if (pairs <= 0) return 0;                                                                                           \
    if ((act && !gate) || act < 0 || act > 2 || dv <= 0) return (int)cudaErrorInvalidValue;                             \
    return launch(retention_gate_kernel<T>, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, st, o, o_stride,           \
                  (const T*)gate, gate_stride, eps, act, pairs, H, dv, (T*)out, out_stride);                            \
  }

KVF_RETENTION_GATE_API(f32, float)
KVF_RETENTION_GATE_API(bf16, bf16)
KVF_RETENTION_API(f32, float)
KVF_RETENTION_API(bf16, bf16)
