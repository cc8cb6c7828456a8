// The gated delta rule: a recurrent mixer whose state per head is a matrix S [d x e] (float32) that is decayed,
// corrected towards the token's value along the token's key, and read with the token's query:
//
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
//
// with g in (0, 1) a decay and beta in (0, 1) a step size per token and head.  Two kernels: `delta_prepare` (queries and
// keys to unit vectors, the queries times d^(-1/2); beta = sigmoid(.), g = exp(-exp(A_log) softplus(. + dt_bias))) and
// `delta_scan` (the recurrence over the step's tokens of every sequence, from and to the sequence's state row).
// Everything here is float32 in both precisions.
//
// Tokens of all sequences are packed along the first axis; `seq_tok0[s] .. seq_tok0[s + 1] - 1` are the packed rows of
// the batch's sequence s, `seq_slot[s]` the row of its state.
#include "common.cuh"

namespace edgelm {

__device__ __forceinline__ float dr_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

// qkv [tokens][G d | G d | H e] (after the convolution): every query and key head x <- x / sqrt(sum(x^2) + unit_eps),
// queries also times q_scale.  bg [tokens][2 H]: beta, then the decay, from the raw projections u[t][b_off + h], u[t][a_off + h].
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qkv, int C, const float* __restrict__ u, int ldu, int b_off, int a_off,
                     const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ bg, int H, int G, int d,
                     float unit_eps, float q_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, NW = blockDim.x >> 5;
  float* row = qkv + (size_t)t * C;
  for (int v = blockIdx.y * NW + warp; v < 2 * G; v += gridDim.y * NW) {          // the vectors: G query heads, then G key heads
    float* x = row + (size_t)v * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float inv = (1.0f / sqrtf(ss + unit_eps)) * (v < G ? q_scale : 1.0f);
    for (int i = lane; i < d; i += 32) x[i] *= inv;
  }
  const float* ur = u + (size_t)t * ldu;
  for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < H; h += gridDim.y * blockDim.x) {
    bg[(size_t)t * 2 * H + h] = 1.0f / (1.0f + expf(-ur[b_off + h]));
    bg[(size_t)t * 2 * H + H + h] = expf(-expf(A_log[h]) * dr_softplus(ur[a_off + h] + dt_bias[h]));
  }
}

// A block = 16 CPT columns of one head's state for one sequence.  Eight lanes share CPT neighbouring columns, each lane with
// RPT of their rows in registers (row = sublane * RPT + r; rows beyond d are zeros); S^T k and S^T q are sums over a lane's
// rows and three shuffles.  With CPT > 1 the token's key and query rows are read once for the CPT columns and the columns'
// chains of dependent operations run side by side: fewer instructions a column, for steps with enough (sequence, head) pairs
// to fill the device; for one sequence the chain from one token's state to the next is what takes the time, and one column a
// thread is fastest (measured at the launch).  The step's queries, keys, values, betas and decays come through shared
// memory, DS_TC tokens a stage, the next stage on its way (cp.async) while this one is computed.  State layout:
// [slot][H][e][d] (a column's rows side by side).
constexpr int DS_SUB = 8, DS_GROUPS = 16, DS_THREADS = DS_SUB * DS_GROUPS, DS_TC = 8;

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int RPT, int CPT>
__global__ void __launch_bounds__(DS_THREADS)
delta_scan_kernel(const float* __restrict__ qkv, int C, const float* __restrict__ bg, float* __restrict__ state, float* __restrict__ o,
                  const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot, int H, int G, int d, int e) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DP = DS_SUB * RPT;                       // padded rows
  constexpr int COLS = DS_GROUPS * CPT;                  // columns a block
  constexpr int NV = RPT / 4;
  constexpr int STAGE = DS_TC * (2 * DP + COLS + 2);     // floats a stage: q, k [DS_TC][DP]; v [DS_TC][COLS]; beta, g [DS_TC]
  __shared__ __align__(16) float sm[2 * STAGE];
  const int s = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * COLS;
  const int g = h / (H / G);
  const int sub = threadIdx.x & (DS_SUB - 1), grp = threadIdx.x >> 3, mycol = col0 + grp * CPT;
  const int t0 = seq_tok0[s], n = seq_tok0[s + 1] - t0;
  float* st = state + ((size_t)seq_slot[s] * H + h) * e * d;
  float S[CPT][RPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int i = sub * RPT + r;
      S[c][r] = (mycol + c < e && i < d) ? st[(size_t)(mycol + c) * d + i] : 0.f;
    }
  for (int i = threadIdx.x; i < 2 * STAGE; i += DS_THREADS) sm[i] = 0.f;   // (rows beyond d and columns beyond e stay zero)
  __syncthreads();
  const int q_off = g * d, k_off = G * d + g * d, v_off = 2 * G * d + h * e + col0;
  auto load = [&](int chunk) {
    float* b = sm + (chunk & 1) * STAGE;
    const int c0 = chunk * DS_TC, nt = min(DS_TC, n - c0);
    for (int i = threadIdx.x; i < nt * d; i += DS_THREADS) {
      const int tt = i / d, j = i - tt * d;
      const float* src = qkv + (size_t)(t0 + c0 + tt) * C;
      cp_async4(b + tt * DP + j, src + q_off + j);
      cp_async4(b + DS_TC * DP + tt * DP + j, src + k_off + j);
    }
    const int ncol = min(COLS, e - col0);
    for (int i = threadIdx.x; i < nt * ncol; i += DS_THREADS) {
      const int tt = i / ncol, j = i - tt * ncol;
      cp_async4(b + 2 * DS_TC * DP + tt * COLS + j, qkv + (size_t)(t0 + c0 + tt) * C + v_off + j);
    }
    if (threadIdx.x < 2 * nt) {
      const int tt = threadIdx.x >> 1, which = threadIdx.x & 1;
      cp_async4(b + 2 * DS_TC * DP + DS_TC * COLS + which * DS_TC + tt, bg + (size_t)(t0 + c0 + tt) * 2 * H + which * H + h);
    }
    cp_async_commit();
  };
  const int n_chunks = (n + DS_TC - 1) / DS_TC;
  if (n_chunks > 0) load(0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) { load(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const float* b = sm + (c & 1) * STAGE;
    const int nt = min(DS_TC, n - c * DS_TC);
    for (int tt = 0; tt < nt; ++tt) {
      const float* qs = b + tt * DP + sub * RPT;
      const float* kk = b + DS_TC * DP + tt * DP + sub * RPT;
      const float beta = b[2 * DS_TC * DP + DS_TC * COLS + tt], dec = b[2 * DS_TC * DP + DS_TC * COLS + DS_TC + tt];
      float4 k4[NV], q4[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) { k4[i] = *reinterpret_cast<const float4*>(kk + 4 * i); q4[i] = *reinterpret_cast<const float4*>(qs + 4 * i); }
      float v[CPT], ks[CPT], ov[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) v[cc] = b[2 * DS_TC * DP + tt * COLS + grp * CPT + cc];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int r = 4 * i;
          S[cc][r] *= dec; S[cc][r + 1] *= dec; S[cc][r + 2] *= dec; S[cc][r + 3] *= dec;
          a0 = fmaf(S[cc][r], k4[i].x, a0); a1 = fmaf(S[cc][r + 1], k4[i].y, a1);
          a0 = fmaf(S[cc][r + 2], k4[i].z, a0); a1 = fmaf(S[cc][r + 3], k4[i].w, a1);
        }
        ks[cc] = a0 + a1;
      }
#pragma unroll
      for (int off = 1; off < DS_SUB; off <<= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) ks[cc] += __shfl_xor_sync(0xffffffffu, ks[cc], off);
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const float uu = beta * (v[cc] - ks[cc]);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int r = 4 * i;
          S[cc][r] = fmaf(k4[i].x, uu, S[cc][r]); S[cc][r + 1] = fmaf(k4[i].y, uu, S[cc][r + 1]);
          S[cc][r + 2] = fmaf(k4[i].z, uu, S[cc][r + 2]); S[cc][r + 3] = fmaf(k4[i].w, uu, S[cc][r + 3]);
          a0 = fmaf(S[cc][r], q4[i].x, a0); a1 = fmaf(S[cc][r + 1], q4[i].y, a1);
          a0 = fmaf(S[cc][r + 2], q4[i].z, a0); a1 = fmaf(S[cc][r + 3], q4[i].w, a1);
        }
        ov[cc] = a0 + a1;
      }
#pragma unroll
      for (int off = 1; off < DS_SUB; off <<= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) ov[cc] += __shfl_xor_sync(0xffffffffu, ov[cc], off);
      if (sub == 0) {
        float* orow = o + (size_t)(t0 + c * DS_TC + tt) * H * e + (size_t)h * e;
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc)
          if (mycol + cc < e) orow[mycol + cc] = ov[cc];
      }
    }
    __syncthreads();     // the stage is free for the load after the next
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int i = sub * RPT + r;
      if (mycol + c < e && i < d) st[(size_t)(mycol + c) * d + i] = S[c][r];
    }
}

}  // namespace edgelm

using namespace edgelm;

static int g_delta_columns = 0;
// Columns of the state a thread of `delta_scan` holds (1, 2 or 4; 0: the kernel's own choice).  For measurements.
extern "C" int edgelm_delta_scan_columns(int n) {
  g_delta_columns = (n == 1 || n == 2 || n == 4) ? n : 0;
  return 0;
}

extern "C" int edgelm_delta_prepare(float* qkv, int C, const float* u, int ldu, int b_off, int a_off, const float* A_log,
                                    const float* dt_bias, float* bg, int n_tokens, int H, int G, int d, int e, float unit_eps,
                                    float q_scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0 && C == 2 * G * d + H * e, "delta_prepare: sizes do not fit (heads %d over %d, %d x %d, channels %d)", H, G, d, e, C);
  EL_REFUSE(b_off >= 0 && a_off >= 0 && b_off + H <= ldu && a_off + H <= ldu, "delta_prepare: rows of %d values are too short", ldu);
  const int vec_blocks = n_tokens >= 256 ? 1 : (2 * G + 3) / 4;    // a step of few tokens: a warp a vector
  launch_pdl(pdl_bit_for_tokens(n_tokens), delta_prepare_kernel, dim3(n_tokens, vec_blocks), dim3(128), (size_t)0, stream, qkv, C, u, ldu, b_off, a_off, A_log,
             dt_bias, bg, H, G, d, unit_eps, q_scale);
  EL_LAUNCH_CHECK("delta_prepare");
  return 0;
}

extern "C" int edgelm_delta_scan(const float* qkv, int C, const float* bg, float* state, float* o, const int32_t* seq_tok0,
                                 const int32_t* seq_slot, int n_seqs, int n_tokens, int H, int G, int d, int e, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && n_seqs <= 65535 && H > 0 && H <= 65535 && G > 0 && H % G == 0 && C == 2 * G * d + H * e, "delta_scan: sizes do not fit (heads %d over %d, channels %d)", H, G, C);
  EL_REFUSE(d >= 1 && d <= 256 && e >= 1, "delta_scan: a state of %d rows per head is not taken (1 to 256)", d);
  // Columns a thread.  Measured (keys and values of 64, 32 heads): one sequence of 2,048 tokens 0.66 / 0.73 / 0.87 ms with 1 / 2 /
  // 4 columns; eight sequences of 512 tokens 0.39 / 0.30 / 0.29 ms.  (Fewer lanes a column, down to a whole column a thread
  // without any shuffle, were measured too: 0.87 to 0.97 ms for the one sequence.)  So one column while the warps leave the
  // device room, else four (two where a column's rows fill the registers), fewer for value heads so narrow that lanes would
  // idle.  `edgelm_delta_scan_columns` overrides, for measurements.
  const int cpt_max = d <= 128 ? 4 : 2;
  const long long warps1 = (long long)n_seqs * H * ((e + 3) / 4);      // warps with one column a thread
  int cpt = g_delta_columns > 0 ? (g_delta_columns < cpt_max ? g_delta_columns : cpt_max) : (warps1 <= 148 * 16 ? 1 : cpt_max);
  while (cpt > 1 && e <= DS_GROUPS * (cpt / 2)) cpt >>= 1;
  const dim3 grid((e + DS_GROUPS * cpt - 1) / (DS_GROUPS * cpt), H, n_seqs), block(DS_THREADS);
  const int bit = pdl_bit_for_tokens(n_tokens);
#define EL_DS2(RPT, CPT) launch_pdl(bit, delta_scan_kernel<RPT, CPT>, grid, block, (size_t)0, stream, qkv, C, bg, state, o, seq_tok0, seq_slot, H, G, d, e)
#define EL_DS(RPT) do { if (cpt == 4) EL_DS2(RPT, 4); else if (cpt == 2) EL_DS2(RPT, 2); else EL_DS2(RPT, 1); } while (0)
  if (d <= 32) EL_DS(4);
  else if (d <= 64) EL_DS(8);
  else if (d <= 128) EL_DS(16);
  else { if (cpt == 2) EL_DS2(32, 2); else EL_DS2(32, 1); }
#undef EL_DS
#undef EL_DS2
  EL_LAUNCH_CHECK("delta_scan");
  return 0;
}
