// Kernels of mixers that carry a fixed-size state from token to token: the blend of a token with the one
// before it (token shift), a short causal convolution over channels, the selective state-space recurrence
// (state N x P per head, scalar decay per head and token), the decayed outer-product recurrence with a bonus
// for the current token (state K x V per head, decay per key channel and token), the decay's low-rank
// projection, and the gated group RMS norm that follows both recurrences.
//
// Tokens of all sequences are packed along the first axis; `seq_tok0[s] .. seq_tok0[s + 1] - 1` are the packed
// rows of the batch's sequence s, `seq_slot[s]` the row of its state.  States, decays, step sizes, norms and the
// recurrences themselves are float32 in both precisions; `T*` names the storage type of activations that feed a
// matrix product (float or bfloat16).
#include "common.cuh"

namespace edgelm {

__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_exact(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

// ------------------------------------------------------------------ blend with the previous token
// out[m][t][:] = a + (prev - a) * mu[m][:], a = in[t], prev = in[t - 1], or the state row for the first token
// that a sequence brings to this step (zeros at a sequence's start).
template <typename TIn, typename TOut>
__global__ void shift_mix_kernel(const TIn* __restrict__ in, const float* __restrict__ state, const float* __restrict__ mu,
                                 TOut* __restrict__ out, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_tok0,
                                 const int32_t* __restrict__ seq_slot, int n_tokens, int dim, int n_mix) {
  const int t = blockIdx.x;
  const int s = tok_seq[t];
  const bool first = t == seq_tok0[s];
  const float* st = state + (size_t)seq_slot[s] * dim;
  const TIn* cur = in + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float a = to_f32(cur[i]);
    const float p = first ? st[i] : to_f32(cur[i - dim]);
    const float d = p - a;
    for (int m = 0; m < n_mix; ++m) out[((size_t)m * n_tokens + t) * dim + i] = from_f32<TOut>(a + d * mu[(size_t)m * dim + i]);
  }
}

// state[slot(s)][:] = in[last row of s][:]
template <typename TIn>
__global__ void save_last_rows_kernel(const TIn* __restrict__ in, float* __restrict__ state, const int32_t* __restrict__ seq_tok0,
                                      const int32_t* __restrict__ seq_slot, int dim) {
  const int s = blockIdx.x;
  const int t = seq_tok0[s + 1] - 1;
  float* st = state + (size_t)seq_slot[s] * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) st[i] = to_f32(in[(size_t)t * dim + i]);
}

// ------------------------------------------------------------------ short causal convolution + silu
// Channel c of token t: silu(b[c] + sum_j w[c][j] * in[t - (taps - 1) + j][c]); inputs before the step come from
// the state [slot][taps - 1][C] (oldest first; zeros before a sequence's start).  `u` holds the inputs at column
// `off + c` of rows of `ldu` floats.
__global__ void conv_silu_kernel(const float* __restrict__ u, int ldu, int off, const float* __restrict__ w,
                                 const float* __restrict__ b, const float* __restrict__ state, float* __restrict__ out,
                                 const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_tok0,
                                 const int32_t* __restrict__ seq_slot, int C, int taps) {
  const int t = blockIdx.x;
  const int s = tok_seq[t];
  const int t0 = seq_tok0[s];
  const int k = t - t0;
  const float* st = state + (size_t)seq_slot[s] * (taps - 1) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = b[c];
    for (int j = 0; j < taps; ++j) {
      const int r = k - (taps - 1) + j;
      const float v = r >= 0 ? u[(size_t)(t0 + r) * ldu + off + c] : st[(size_t)(taps - 1 + r) * C + c];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)t * C + c] = silu_exact(acc);
  }
}

// The state after the step: the last taps - 1 inputs of each sequence.  A thread owns a channel and walks the
// rows upwards, so that a row it still has to read (one further on) is never overwritten before.
__global__ void conv_state_update_kernel(const float* __restrict__ u, int ldu, int off, float* __restrict__ state,
                                         const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot, int C, int taps) {
  const int s = blockIdx.x;
  const int t0 = seq_tok0[s], n = seq_tok0[s + 1] - t0;
  float* st = state + (size_t)seq_slot[s] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x)
    for (int j = 0; j < taps - 1; ++j) {
      const int r = n - (taps - 1) + j;
      st[(size_t)j * C + c] = r >= 0 ? u[(size_t)(t0 + r) * ldu + off + c] : st[(size_t)(j + n) * C + c];
    }
}

// ------------------------------------------------------------------ selective state-space recurrence
// Per head h (group g = h / (H / G)) and token t, with dt = softplus(dt_raw + dt_bias[h]) and a = exp(-exp(A_log[h]) dt):
//   S <- a S + dt B_t x_t^T      (S is N x P)
//   y_t = S^T C_t + D[h] x_t
// A warp owns one column p of one head of one sequence; lane l holds the rows n = l, l + 32, ... (NK of them) in
// registers, so a token costs a handful of multiply-adds and one warp sum, and nothing is exchanged between warps.
// Tokens are taken U at a time: their inputs are requested together, the warp sums are done together.
constexpr int SCAN_WARPS = 8;

template <int NK, int U>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
ssm_scan_kernel(const float* __restrict__ xbc, int C, int inner, int G, int N, const float* __restrict__ u, int ldu, int dt_off,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dp,
                float* __restrict__ state, float* __restrict__ y, const int32_t* __restrict__ seq_tok0,
                const int32_t* __restrict__ seq_slot, int H, int P) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x / H, h = blockIdx.x - s * H;
  const int p = blockIdx.y * SCAN_WARPS + warp;
  if (p >= P) return;
  const int g = h / (H / G);
  const int t0 = seq_tok0[s], t1 = seq_tok0[s + 1];
  float* sp = state + (((size_t)seq_slot[s] * H + h) * P + p) * N;
  float S[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) S[k] = lane + 32 * k < N ? sp[lane + 32 * k] : 0.f;
  const float A = -expf(A_log[h]), Dh = Dp[h], bias = dt_bias[h];
  const int xo = h * P + p, bo = inner + g * N, co = inner + G * N + g * N;
  for (int tb = t0; tb < t1; tb += U) {
    float dtr[U], xv[U], Bn[U][NK], Cn[U][NK], acc[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int t = min(tb + i, t1 - 1);
      const float* row = xbc + (size_t)t * C;
      dtr[i] = u[(size_t)t * ldu + dt_off + h];
      xv[i] = row[xo];
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const int n = lane + 32 * k;
        Bn[i][k] = n < N ? row[bo + n] : 0.f;
        Cn[i][k] = n < N ? row[co + n] : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      acc[i] = 0.f;
      if (tb + i < t1) {
        const float dt = softplus_exact(dtr[i] + bias);
        const float a = expf(A * dt), dx = dt * xv[i];
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          S[k] = fmaf(a, S[k], dx * Bn[i][k]);
          acc[i] = fmaf(S[k], Cn[i][k], acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < U; ++i) acc[i] = warp_sum(acc[i]);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < U; ++i)
        if (tb + i < t1) y[(size_t)(tb + i) * inner + xo] = acc[i] + Dh * xv[i];
    }
  }
#pragma unroll
  for (int k = 0; k < NK; ++k)
    if (lane + 32 * k < N) sp[lane + 32 * k] = S[k];
}

// ------------------------------------------------------------------ decayed outer-product recurrence with a bonus
// Per head, key channel i and value channel j:
//   o_t[j] = sum_i (S[i][j] + bonus[i] k_t[i] v_t[j]) r_t[i]
//   S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
// A warp owns one value channel j; lane l holds the key channels i = l, l + 32, ...  r, k, v, w: [tokens][H * K]
// (value size = key size K); state [slot][H][K (j)][K (i)].
template <int NK, int U>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ kk, const float* __restrict__ v, const float* __restrict__ w,
                const float* __restrict__ bonus, float* __restrict__ state, float* __restrict__ o,
                const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot, int H, int K) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x / H, h = blockIdx.x - s * H;
  const int j = blockIdx.y * SCAN_WARPS + warp;
  if (j >= K) return;
  const int t0 = seq_tok0[s], t1 = seq_tok0[s + 1];
  float* sp = state + (((size_t)seq_slot[s] * H + h) * K + j) * K;
  float S[NK], bn[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int i = lane + 32 * k;
    S[k] = i < K ? sp[i] : 0.f;
    bn[k] = i < K ? bonus[h * K + i] : 0.f;
  }
  const int ld = H * K, ho = h * K;
  for (int tb = t0; tb < t1; tb += U) {
    float vj[U], rr[U][NK], kv[U][NK], ww[U][NK], acc[U];
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const size_t row = (size_t)min(tb + q, t1 - 1) * ld + ho;
      vj[q] = v[row + j];
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const int i = lane + 32 * k;
        rr[q][k] = i < K ? r[row + i] : 0.f;
        kv[q][k] = i < K ? kk[row + i] : 0.f;
        ww[q][k] = i < K ? w[row + i] : 0.f;
      }
    }
#pragma unroll
    for (int q = 0; q < U; ++q) {
      acc[q] = 0.f;
      if (tb + q < t1) {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          const float x = kv[q][k] * vj[q];
          acc[q] = fmaf(fmaf(bn[k], x, S[k]), rr[q][k], acc[q]);
          S[k] = fmaf(ww[q][k], S[k], x);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < U; ++q) acc[q] = warp_sum(acc[q]);
    if (lane == 0) {
#pragma unroll
      for (int q = 0; q < U; ++q)
        if (tb + q < t1) o[(size_t)(tb + q) * ld + ho + j] = acc[q];
    }
  }
#pragma unroll
  for (int k = 0; k < NK; ++k)
    if (lane + 32 * k < K) sp[lane + 32 * k] = S[k];
}

// ------------------------------------------------------------------ the decay from its low-rank projection
// out[t][c] = exp(-exp(w0[c] + sum_l W2[c][l] tanh(a[t][l]))), all in float32 (W2 in its storage type).
template <typename TW>
__global__ void lowrank_decay_kernel(const float* __restrict__ a, const TW* __restrict__ w2, const float* __restrict__ w0,
                                     float* __restrict__ out, int C, int L) {
  extern __shared__ float th[];
  const int t = blockIdx.x;
  for (int l = threadIdx.x; l < L; l += blockDim.x) th[l] = tanhf(a[(size_t)t * L + l]);
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = w0[c];
    const TW* row = w2 + (size_t)c * L;
    for (int l = 0; l < L; ++l) acc = fmaf(to_f32(row[l]), th[l], acc);
    out[(size_t)t * C + c] = expf(-expf(acc));
  }
}

// ------------------------------------------------------------------ gated RMS norm in equal groups
// A row of `inner` values in `groups` equal parts, each divided by its own root mean square.
//   gate_first:  v = y * silu(gate); out = v / rms(v) * w
//   else:        out = y / rms(y) * w * silu(gate)
template <typename TOut>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ldg,
                                        const float* __restrict__ w, TOut* __restrict__ out, int inner, int groups, float eps,
                                        int gate_first) {
  __shared__ float red[33];
  const int t = blockIdx.x, g = blockIdx.y, gs = inner / groups;
  const float* yr = y + (size_t)t * inner + (size_t)g * gs;
  const float* gr = gate + (size_t)t * ldg + (size_t)g * gs;
  const float* wr = w + (size_t)g * gs;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float v = gate_first ? yr[i] * silu_exact(gr[i]) : yr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
  TOut* orow = out + (size_t)t * inner + (size_t)g * gs;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float sg = silu_exact(gr[i]);
    orow[i] = from_f32<TOut>(gate_first ? yr[i] * sg * inv * wr[i] : yr[i] * inv * wr[i] * sg);
  }
}

// ------------------------------------------------------------------ x += rmsnorm(a y1 + b y2) * w  (+ a copy of x in the compute type)
template <typename TCast>
__global__ void rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y1, float a, const float* __restrict__ y2, float b,
                                   const float* __restrict__ w, TCast* __restrict__ xc, int dim, float eps) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* r1 = y1 + (size_t)t * dim;
  const float* r2 = y2 ? y2 + (size_t)t * dim : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = r2 ? a * r1[i] + b * r2[i] : a * r1[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  float* xr = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = r2 ? a * r1[i] + b * r2[i] : a * r1[i];
    const float nx = xr[i] + v * inv * w[i];
    xr[i] = nx;
    if (xc) xc[(size_t)t * dim + i] = from_f32<TCast>(nx);
  }
}

// out = a y1 + b y2
__global__ void scaled_sum_kernel(const float* __restrict__ y1, float a, const float* __restrict__ y2, float b, float* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = a * y1[i] + b * y2[i];
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_scaled_sum(const float* y1, float a, const float* y2, float b, float* out, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  EL_REFUSE(n > 0, "scaled_sum: bad size");
  const long long blocks = (n + 255) / 256;
  scaled_sum_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, stream>>>(y1, a, y2, b, out, (size_t)n);
  EL_LAUNCH_CHECK("scaled_sum");
  return 0;
}

static inline int row_threads(int dim) { return dim >= 1024 ? 256 : 128; }

extern "C" int edgelm_shift_mix(const void* in, int in_dtype, const float* state, const float* mu, void* out, int out_dtype,
                                const int32_t* tok_seq, const int32_t* seq_tok0, const int32_t* seq_slot, int n_tokens, int dim,
                                int n_mix, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && dim > 0 && n_mix > 0, "shift_mix: bad sizes tokens=%d dim=%d mixes=%d", n_tokens, dim, n_mix);
  const dim3 grid(n_tokens), block(row_threads(dim));
#define EL_SM(TI, TO) shift_mix_kernel<TI, TO><<<grid, block, 0, stream>>>((const TI*)in, state, mu, (TO*)out, tok_seq, seq_tok0, seq_slot, n_tokens, dim, n_mix)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) EL_SM(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) EL_SM(float, __nv_bfloat16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) EL_SM(__nv_bfloat16, __nv_bfloat16);
  else EL_REFUSE(false, "shift_mix: dtype codes %d -> %d are not taken", in_dtype, out_dtype);
#undef EL_SM
  EL_LAUNCH_CHECK("shift_mix");
  return 0;
}

extern "C" int edgelm_save_last_rows(const void* in, int in_dtype, float* state, const int32_t* seq_tok0, const int32_t* seq_slot,
                                     int n_seqs, int dim, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && dim > 0, "save_last_rows: bad sizes");
  if (in_dtype == DT_F32) save_last_rows_kernel<float><<<n_seqs, row_threads(dim), 0, stream>>>((const float*)in, state, seq_tok0, seq_slot, dim);
  else if (in_dtype == DT_BF16) save_last_rows_kernel<__nv_bfloat16><<<n_seqs, row_threads(dim), 0, stream>>>((const __nv_bfloat16*)in, state, seq_tok0, seq_slot, dim);
  else EL_REFUSE(false, "save_last_rows: unknown dtype code %d", in_dtype);
  EL_LAUNCH_CHECK("save_last_rows");
  return 0;
}

// The convolution over the step's tokens and, after it, the state for the next step (two launches).
extern "C" int edgelm_conv_silu(const float* u, int ldu, int off, const float* w, const float* b, float* state, float* out,
                                const int32_t* tok_seq, const int32_t* seq_tok0, const int32_t* seq_slot, int n_tokens, int n_seqs,
                                int C, int taps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && n_seqs > 0 && C > 0 && taps >= 1 && off >= 0 && off + C <= ldu, "conv_silu: bad sizes C=%d taps=%d", C, taps);
  conv_silu_kernel<<<n_tokens, row_threads(C), 0, stream>>>(u, ldu, off, w, b, state, out, tok_seq, seq_tok0, seq_slot, C, taps);
  EL_LAUNCH_CHECK("conv_silu");
  if (taps > 1) {
    conv_state_update_kernel<<<dim3(n_seqs, (C + 255) / 256), 256, 0, stream>>>(u, ldu, off, state, seq_tok0, seq_slot, C, taps);
    EL_LAUNCH_CHECK("conv_state_update");
  }
  return 0;
}

extern "C" int edgelm_ssm_scan(const float* xbc, int C, int inner, int G, int N, const float* u, int ldu, int dt_off,
                               const float* dt_bias, const float* A_log, const float* Dp, float* state, float* y,
                               const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, int H, int P, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && H > 0 && P > 0 && G > 0 && H % G == 0 && inner == H * P && C == inner + 2 * G * N,
            "ssm_scan: sizes do not fit (heads %d, groups %d, head size %d, inner %d, channels %d)", H, G, P, inner, C);
  EL_REFUSE(N >= 1 && N <= 256, "ssm_scan: a state of %d rows per head is not taken (1 to 256)", N);
  const dim3 grid(n_seqs * H, (P + SCAN_WARPS - 1) / SCAN_WARPS), block(SCAN_WARPS * 32);
#define EL_SCAN(NK, U) ssm_scan_kernel<NK, U><<<grid, block, 0, stream>>>(xbc, C, inner, G, N, u, ldu, dt_off, dt_bias, A_log, Dp, state, y, seq_tok0, seq_slot, H, P)
  if (N <= 32) EL_SCAN(1, 8);
  else if (N <= 64) EL_SCAN(2, 4);
  else if (N <= 128) EL_SCAN(4, 4);
  else EL_SCAN(8, 2);
#undef EL_SCAN
  EL_LAUNCH_CHECK("ssm_scan");
  return 0;
}

extern "C" int edgelm_wkv_scan(const float* r, const float* k, const float* v, const float* w, const float* bonus, float* state,
                               float* o, const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, int H, int K,
                               cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && H > 0, "wkv_scan: bad sizes");
  EL_REFUSE(K >= 1 && K <= 256, "wkv_scan: a head size of %d is not taken (1 to 256)", K);
  const dim3 grid(n_seqs * H, (K + SCAN_WARPS - 1) / SCAN_WARPS), block(SCAN_WARPS * 32);
#define EL_SCAN(NK, U) wkv_scan_kernel<NK, U><<<grid, block, 0, stream>>>(r, k, v, w, bonus, state, o, seq_tok0, seq_slot, H, K)
  if (K <= 32) EL_SCAN(1, 8);
  else if (K <= 64) EL_SCAN(2, 4);
  else if (K <= 128) EL_SCAN(4, 2);
  else EL_SCAN(8, 1);
#undef EL_SCAN
  EL_LAUNCH_CHECK("wkv_scan");
  return 0;
}

extern "C" int edgelm_lowrank_decay(const float* a, const void* w2, int w_dtype, const float* w0, float* out, int n_tokens, int C,
                                    int L, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && C > 0 && L > 0 && L <= 8192, "lowrank_decay: bad sizes C=%d L=%d", C, L);
  const size_t smem = (size_t)L * sizeof(float);
  if (w_dtype == DT_F32) lowrank_decay_kernel<float><<<n_tokens, row_threads(C), smem, stream>>>(a, (const float*)w2, w0, out, C, L);
  else if (w_dtype == DT_BF16) lowrank_decay_kernel<__nv_bfloat16><<<n_tokens, row_threads(C), smem, stream>>>(a, (const __nv_bfloat16*)w2, w0, out, C, L);
  else EL_REFUSE(false, "lowrank_decay: unknown dtype code %d", w_dtype);
  EL_LAUNCH_CHECK("lowrank_decay");
  return 0;
}

extern "C" int edgelm_gated_group_norm(const float* y, const float* gate, int ldg, const float* w, void* out, int out_dtype,
                                       int n_tokens, int inner, int groups, float eps, int gate_first, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && inner > 0 && groups > 0 && inner % groups == 0, "gated_group_norm: %d values do not split into %d equal groups", inner, groups);
  const dim3 grid(n_tokens, groups), block(inner / groups >= 1024 ? 256 : (inner / groups >= 128 ? 128 : 32));
  if (out_dtype == DT_F32) gated_group_norm_kernel<float><<<grid, block, 0, stream>>>(y, gate, ldg, w, (float*)out, inner, groups, eps, gate_first);
  else if (out_dtype == DT_BF16) gated_group_norm_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(y, gate, ldg, w, (__nv_bfloat16*)out, inner, groups, eps, gate_first);
  else EL_REFUSE(false, "gated_group_norm: unknown dtype code %d", out_dtype);
  EL_LAUNCH_CHECK("gated_group_norm");
  return 0;
}

// x += rmsnorm(a y1 + b y2) * w; y2 may be null; `xc` (may be null) receives x in `cast_dtype` as well.
extern "C" int edgelm_rmsnorm_add(float* x, const float* y1, float a, const float* y2, float b, const float* w, void* xc, int cast_dtype,
                                  int n_tokens, int dim, float eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && dim > 0, "rmsnorm_add: bad sizes");
  const dim3 grid(n_tokens), block(row_threads(dim));
  if (xc == nullptr || cast_dtype == DT_F32) rmsnorm_add_kernel<float><<<grid, block, 0, stream>>>(x, y1, a, y2, b, w, (float*)xc, dim, eps);
  else if (cast_dtype == DT_BF16) rmsnorm_add_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(x, y1, a, y2, b, w, (__nv_bfloat16*)xc, dim, eps);
  else EL_REFUSE(false, "rmsnorm_add: unknown dtype code %d", cast_dtype);
  EL_LAUNCH_CHECK("rmsnorm_add");
  return 0;
}
