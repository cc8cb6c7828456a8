// Sliding-window attention with pooled blocks behind the window, over the paged cache.
//
// A token at position i sees the keys j with 0 <= i - j < window, and one pooled key and value per block of P
// consecutive positions that lies wholly before the window (block b = positions bP .. bP + P - 1 is seen iff
// bP + P - 1 <= i - window).  A pooled key (value) is the mean of the block's P keys (values) as the cache holds
// them.  Tokens and blocks share one softmax.
//
// Cache layout: keys [page][kv_head][PAGE][dk], values [page][kv_head][PAGE][dv] in the compute type, as the other
// attention kernels keep them; pooled keys and values in float32, [page][kv_head][R][dk or dv], where a block's
// row lives in the page that holds the block's LAST position e = bP + P - 1: page e / PAGE, row b - (PAGE * (e / PAGE)) / P
// (R = ceil(PAGE / P) rows a page are enough: that many block ends fall into one page at most).
//
// Three kernels: (1) bias, partial rotation, per-head unit RMS norm of q and k, append of k and v; (2) the pooled
// rows of the blocks that the step's tokens complete; (3) attention.  Scores, softmax, norms, angles: float32.
#include "common.cuh"

namespace edgelm {

constexpr int PW_WARPS = 4;

// qkv: [tokens][H dk + G dk + G dv] float32 (the stacked projection), biases float32 (may be null).
// The first `rot` dimensions of each query and key head are rotated: (u, v) = (x[i], x[i + rot/2]) becomes
// (u cos a - v sin a, v cos a + u sin a), a = position * freq[i]; then the head is divided by its root mean square.
template <typename T>
__global__ void __launch_bounds__(PW_WARPS * 32)
qk_rope_norm_append_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, T* __restrict__ q_out,
                           const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ tok_seq,
                           const int32_t* __restrict__ page_table, int table_stride, int n_pages, T* __restrict__ kcache,
                           T* __restrict__ vcache, int H, int G, int dk, int dv, int rot, const double* __restrict__ freq,
                           float eps, int unit_norm, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  extern __shared__ float stage[];   // PW_WARPS rows of dk floats
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = tok_pos[t];
  if (pos < 0) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, ERR_POSITION_RANGE);
    return;
  }
  const int page = page_table[(size_t)tok_seq[t] * table_stride + pos / PAGE];
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, ERR_PAGE_RANGE);
    return;
  }
  const int in_page = pos % PAGE, half = rot >> 1;
  const int ld = H * dk + G * dk + G * dv;
  const float* row = qkv + (size_t)t * ld;
  float* sh = stage + warp * dk;
  const double dpos = (double)pos;
  // a warp a head (query heads, then key heads); the blocks of a token stand side by side over the heads
  for (int head = blockIdx.y * PW_WARPS + warp; head < H + G; head += gridDim.y * PW_WARPS) {
    const float* src = row + (size_t)head * dk;
    const float* b = bias ? bias + (size_t)head * dk : nullptr;
    for (int i = lane; i < dk; i += 32) sh[i] = src[i] + (b ? b[i] : 0.f);
    __syncwarp();
    float ss = 0.f;
    float val[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const int i = lane + 32 * m;
      float x = 0.f;
      if (i < dk) {
        x = sh[i];
        if (i < rot) {
          const int f = i < half ? i : i - half;
          // the angle position * f is formed exactly and brought into [-pi, pi] before it is rounded to float32: at
          // position 1,000 a float32 product alone is off by up to 3e-5 rad, which is most of a float32 model's error
          double a = dpos * freq[f];
          a -= 6.283185307179586477 * rint(a * 0.15915494309189533577);
          float sn, cs;
          sincosf((float)a, &sn, &cs);
          x = i < half ? sh[i] * cs - sh[i + half] * sn : sh[i] * cs + sh[i - half] * sn;
        }
      }
      val[m] = x;
      ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = unit_norm ? 1.0f / sqrtf(ss / (float)dk + eps) : 1.0f;
    T* dst = head < H ? q_out + ((size_t)t * H + head) * dk : kcache + (((size_t)page * G + (head - H)) * PAGE + in_page) * dk;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const int i = lane + 32 * m;
      if (i < dk) dst[i] = from_f32<T>(val[m] * inv);
    }
    __syncwarp();
  }
  const float* vrow = row + (size_t)(H + G) * dk;
  const float* vb = bias ? bias + (size_t)(H + G) * dk : nullptr;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < G * dv; i += gridDim.y * blockDim.x) {
    const int g = i / dv, j = i - g * dv;
    vcache[(((size_t)page * G + g) * PAGE + in_page) * dv + j] = from_f32<T>(vrow[i] + (vb ? vb[i] : 0.f));
  }
}

// The pooled rows of the blocks that end at a token of this step.
template <typename T>
__global__ void pool_blocks_kernel(const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ tok_seq,
                                   const int32_t* __restrict__ page_table, int table_stride, int n_pages,
                                   const T* __restrict__ kcache, const T* __restrict__ vcache, float* __restrict__ pk,
                                   float* __restrict__ pv, int G, int dk, int dv, int P, int R, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  if (pos < 0 || (pos + 1) % P != 0) return;
  const int b = (pos + 1) / P - 1;
  const int32_t* table = page_table + (size_t)tok_seq[t] * table_stride;
  const int dst_page = table[pos / PAGE];
  if (dst_page < 0 || dst_page >= n_pages) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, ERR_PAGE_RANGE);
    return;
  }
  const int rowi = b - (PAGE * (pos / PAGE)) / P;
  const float invP = 1.0f / (float)P;
  // a block per (token that ends a block, key/value head); a thread a channel of the key, then of the value: the rows
  // of a block lie side by side in a page, so neighbouring threads read neighbouring addresses, eight rows in flight
  const int g = blockIdx.y;
  for (int i = threadIdx.x; i < dk + dv; i += blockDim.x) {
    const bool is_k = i < dk;
    const int d = is_k ? dk : dv, c = is_k ? i : i - dk;
    const T* base = is_k ? kcache : vcache;
    float acc = 0.f;
#pragma unroll 8
    for (int j = 0; j < P; ++j) {
      const int p = b * P + j;
      const int page = table[p / PAGE];
      if (page < 0 || page >= n_pages) continue;   // (flagged by the append of that token's step)
      acc += to_f32(base[(((size_t)page * G + g) * PAGE + p % PAGE) * d + c]);
    }
    float* dst = is_k ? pk : pv;
    dst[(((size_t)dst_page * G + g) * R + rowi) * d + c] = acc * invP;
  }
}

// ---- the attention kernel
// A block per (token, query head); its NW warps take the keys in turns of 32 (a lane a key: pooled blocks first, then
// the window's tokens), each with its own running maximum, denominator and weighted values (float32), merged at the end
// through shared memory.  A lane reads its key 16 bytes at a time where the layout allows; for the weighted values the
// lanes stand side by side over the value's dimensions, two each.

// q . k over n dimensions, q float32 in shared memory; four running sums.
template <typename TK>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const TK* __restrict__ k, int n, bool vec);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int n, bool vec) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int i = 0;
  if (vec) {
    for (; i + 4 <= n; i += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + i);
      const float4 qv = *reinterpret_cast<const float4*>(q + i);
      a0 = fmaf(qv.x, kv.x, a0); a1 = fmaf(qv.y, kv.y, a1); a2 = fmaf(qv.z, kv.z, a2); a3 = fmaf(qv.w, kv.w, a3);
    }
  }
  for (; i < n; ++i) a0 = fmaf(q[i], k[i], a0);
  return (a0 + a1) + (a2 + a3);
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int n, bool vec) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int i = 0;
  if (vec) {
    for (; i + 8 <= n; i += 8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(k + i);
      const float4 q0 = *reinterpret_cast<const float4*>(q + i), q1 = *reinterpret_cast<const float4*>(q + i + 4);
      a0 = fmaf(q0.x, __uint_as_float(kv.x << 16), a0); a1 = fmaf(q0.y, __uint_as_float(kv.x & 0xffff0000u), a1);
      a2 = fmaf(q0.z, __uint_as_float(kv.y << 16), a2); a3 = fmaf(q0.w, __uint_as_float(kv.y & 0xffff0000u), a3);
      a0 = fmaf(q1.x, __uint_as_float(kv.z << 16), a0); a1 = fmaf(q1.y, __uint_as_float(kv.z & 0xffff0000u), a1);
      a2 = fmaf(q1.z, __uint_as_float(kv.w << 16), a2); a3 = fmaf(q1.w, __uint_as_float(kv.w & 0xffff0000u), a3);
    }
  }
  for (; i < n; ++i) a0 = fmaf(q[i], __bfloat162float(k[i]), a0);
  return (a0 + a1) + (a2 + a3);
}

// two neighbouring values of a row
__device__ __forceinline__ float2 load_pair(const float* p, bool pair) {
  return pair ? *reinterpret_cast<const float2*>(p) : make_float2(p[0], 0.f);
}
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p, bool pair) {
  if (!pair) return make_float2(__bfloat162float(p[0]), 0.f);
  const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}

constexpr int PW_MAX_WARPS = 8;

// Dynamic shared memory: the query (dk floats, 16-byte aligned), then per warp its maximum, its denominator and dv values.
// (Eight lanes sharing a key, so that a load instruction of the warp covers four whole rows, was built and measured: 5.2 ms
// against 3.8 ms for 2,048 tokens of 32 heads with a window of 1,024: the extra shuffles cost more than the loads save.)
// DVR: how many pairs of value dimensions a lane holds (value heads of up to 64 DVR dimensions).
template <typename T, int DVR>
__global__ void __launch_bounds__(PW_MAX_WARPS * 32)
pooled_window_attn_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
                          const float* __restrict__ pk, const float* __restrict__ pv, const int32_t* __restrict__ tok_pos,
                          const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ page_table, int table_stride,
                          int n_pages, int H, int G, int dk, int dv, float scale, int window, int P, int R, int vec_k, int pair_v) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  extern __shared__ __align__(16) float smem[];
  const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, NW = blockDim.x >> 5;
  const int dkp = (dk + 3) & ~3;
  float* qh = smem;
  float* wm = smem + dkp;          // [NW] maxima
  float* wl = wm + NW;             // [NW] denominators
  float* wo = wl + NW;             // [NW][dv]
  const int pos = tok_pos[t];
  if (pos < 0) return;
  const int g = h / (H / G);
  const int32_t* table = page_table + (size_t)tok_seq[t] * table_stride;
  const T* qrow = q + ((size_t)t * H + h) * dk;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) qh[i] = to_f32(qrow[i]) * scale;
  __syncthreads();
  const int lo = max(0, pos - window + 1), n_win = pos - lo + 1;
  const int n_blocks = (P > 0 && pos - window >= 0) ? (pos - window + 1) / P : 0;
  const int blk_chunks = (n_blocks + 31) >> 5, n_chunks = blk_chunks + ((n_win + 31) >> 5);
  float m = -INFINITY, l = 0.f;
  float o[2 * DVR];                // dimensions 2 lane + 64 r and the one after it
#pragma unroll
  for (int r = 0; r < 2 * DVR; ++r) o[r] = 0.f;
  for (int c = warp; c < n_chunks; c += NW) {
    const bool pooled = c < blk_chunks;
    const int e0 = pooled ? c * 32 : (c - blk_chunks) * 32;
    const int n_here = min(32, (pooled ? n_blocks : n_win) - e0);
    float sc = -INFINITY;
    int vrow = -1;                 // this lane's key: the row of its value
    if (lane < n_here) {
      if (pooled) {
        const int e = e0 + lane, end = e * P + P - 1;
        const int page = table[end / PAGE];
        if (page >= 0 && page < n_pages) {
          vrow = (page * G + g) * R + (e - (PAGE * (end / PAGE)) / P);
          sc = dot_row<float>(qh, pk + (size_t)vrow * dk, dk, (dk & 3) == 0);
        }
      } else {
        const int p = lo + e0 + lane;
        const int page = table[p / PAGE];
        if (page >= 0 && page < n_pages) {
          vrow = (page * G + g) * PAGE + p % PAGE;
          sc = dot_row<T>(qh, kcache + (size_t)vrow * dk, dk, vec_k != 0);
        }
      }
    }
    const float m_new = fmaxf(m, warp_max(sc));
    if (m_new == -INFINITY) continue;
    const float w = sc == -INFINITY ? 0.f : expf(sc - m_new);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(w);
    m = m_new;
#pragma unroll
    for (int r = 0; r < 2 * DVR; ++r) o[r] *= corr;
    if (pooled) {
      const bool pair = (dv & 1) == 0;
      for (int j = 0; j < n_here; ++j) {
        const float wj = __shfl_sync(0xffffffffu, w, j);
        const int vr_i = __shfl_sync(0xffffffffu, vrow, j);
        if (vr_i < 0) continue;
        const float* vr = pv + (size_t)vr_i * dv;
#pragma unroll
        for (int r = 0; r < DVR; ++r) {
          const int d = 2 * lane + 64 * r;
          if (d < dv) {
            const float2 x = load_pair(vr + d, pair);
            o[2 * r] = fmaf(wj, x.x, o[2 * r]);
            if (d + 1 < dv) o[2 * r + 1] = fmaf(wj, pair ? x.y : vr[d + 1], o[2 * r + 1]);
          }
        }
      }
    } else {
#pragma unroll 4
      for (int j = 0; j < n_here; ++j) {
        const float wj = __shfl_sync(0xffffffffu, w, j);
        const int vr_i = __shfl_sync(0xffffffffu, vrow, j);
        if (vr_i < 0) continue;
        const T* vr = vcache + (size_t)vr_i * dv;
#pragma unroll
        for (int r = 0; r < DVR; ++r) {
          const int d = 2 * lane + 64 * r;
          if (d < dv) {
            const float2 x = load_pair(vr + d, pair_v != 0);
            o[2 * r] = fmaf(wj, x.x, o[2 * r]);
            if (d + 1 < dv) o[2 * r + 1] = fmaf(wj, pair_v ? x.y : to_f32(vr[d + 1]), o[2 * r + 1]);
          }
        }
      }
    }
  }
  // merge the warps' partial results in a fixed order
  if (lane == 0) { wm[warp] = m; wl[warp] = l; }
#pragma unroll
  for (int r = 0; r < DVR; ++r) {
    const int d = 2 * lane + 64 * r;
    if (d < dv) wo[warp * dv + d] = o[2 * r];
    if (d + 1 < dv) wo[warp * dv + d + 1] = o[2 * r + 1];
  }
  __syncthreads();
  float M = -INFINITY;
  for (int w2 = 0; w2 < NW; ++w2) M = fmaxf(M, wm[w2]);
  float L = 0.f;
  for (int w2 = 0; w2 < NW; ++w2) L += wm[w2] == -INFINITY ? 0.f : wl[w2] * expf(wm[w2] - M);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float acc = 0.f;
    for (int w2 = 0; w2 < NW; ++w2)
      if (wm[w2] != -INFINITY) acc = fmaf(wo[w2 * dv + d], expf(wm[w2] - M), acc);
    out[((size_t)t * H + h) * dv + d] = from_f32<T>(acc * inv);
  }
}

// ---- the attention kernel of prompt steps
// A block = up to 32 (token, query head) rows of one key/value head and of one run of consecutive tokens (a tile of the
// step's metadata); 64 keys with their values are staged in shared memory as float32 once for all the rows: first the
// pooled rows that the tile's last token sees (gathered through the page table), then the window's pages.  A warp owns
// four rows, so a key element read from shared memory serves four multiply-adds; lanes own keys for the scores and
// value dimensions for the weighted sum.  Scores, maxima, exponentials, sums and weighted values are float32.  A row sees
// pooled block e iff e < its own count of seen blocks, and key p iff first <= p <= its position.
constexpr int TW_RW = 4, TW_WARPS = 8, TW_ROWS = TW_RW * TW_WARPS, TW_KEYS = PAGE;

template <typename T, int NC>    // NC = ceil(dv / 32): value dimensions a lane owns
__global__ void __launch_bounds__(TW_WARPS * 32)
pooled_window_attn_tiled_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
                                const float* __restrict__ pk, const float* __restrict__ pv, const int32_t* __restrict__ page_table,
                                int table_stride, int n_pages, const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_tok0,
                                const int32_t* __restrict__ tile_ntok, const int32_t* __restrict__ tile_pos0, int H, int G, int dk,
                                int dv, float scale, int window, int P, int R) {
  extern __shared__ float tw_smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int ks = dk + 1;                        // padded key row: lanes read different rows
  float* Ks = tw_smem;                          // [TW_KEYS][dk + 1]
  float* Vs = Ks + TW_KEYS * ks;                // [TW_KEYS][dv]
  float* Qs = Vs + TW_KEYS * dv;                // [TW_ROWS][dk]
  float* Ps = Qs + TW_ROWS * dk;                // [TW_ROWS][TW_KEYS]
  const int tile = blockIdx.x, g = blockIdx.y, grp = H / G;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  const int32_t* pages = page_table + (size_t)seq * table_stride;
  const int rows_total = ntok * grp, row_base = blockIdx.z * TW_ROWS;
  if (row_base >= rows_total) return;
  const int rows_here = min(TW_ROWS, rows_total - row_base);
  const int last_pos = pos0 + (row_base + rows_here - 1) / grp, first_pos = pos0 + row_base / grp;
  for (int i = threadIdx.x; i < rows_here * dk; i += blockDim.x) {
    const int r = i / dk, d = i - r * dk;
    const int rr = row_base + r, tok = rr / grp, head = g * grp + rr % grp;
    Qs[r * dk + d] = to_f32(q[((size_t)(tok0 + tok) * H + head) * dk + d]);
  }
  float m[TW_RW], l[TW_RW], acc[TW_RW][NC];
  int limit[TW_RW], first[TW_RW], seen[TW_RW];
#pragma unroll
  for (int r = 0; r < TW_RW; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
    const int rr = row_base + warp * TW_RW + r;
    limit[r] = rr < rows_total ? pos0 + rr / grp : -1;                       // the row's own position; -1: no row
    first[r] = max(0, limit[r] - window + 1);
    seen[r] = (P > 0 && limit[r] - window >= 0) ? (limit[r] - window + 1) / P : 0;   // pooled blocks wholly before its window
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
  }
  // what a warp does with the 64 staged keys whose indices (block numbers, or positions) start at `base`: row r sees
  // index i iff lo[r] <= i <= hi[r]
  auto process = [&](int base, const int (&lo)[TW_RW], const int (&hi)[TW_RW], int valid) {
    int any_hi = -1, any_lo = 0x7fffffff;
#pragma unroll
    for (int r = 0; r < TW_RW; ++r)
      if (hi[r] >= lo[r]) { any_hi = max(any_hi, hi[r]); any_lo = min(any_lo, lo[r]); }
    if (base > any_hi || base + TW_KEYS - 1 < any_lo) return;     // none of this warp's rows sees any of these keys
    const int i0 = base + lane, i1 = i0 + 32;
    float s0[TW_RW] = {}, s1[TW_RW] = {};
    const float* k0 = Ks + lane * ks;
    const float* k1 = Ks + (lane + 32) * ks;
    const float* qw = Qs + warp * TW_RW * dk;
    for (int d = 0; d < dk; ++d) {
      const float a = k0[d], b = k1[d];
#pragma unroll
      for (int r = 0; r < TW_RW; ++r) {
        const float qv = qw[r * dk + d];
        s0[r] = fmaf(qv, a, s0[r]);
        s1[r] = fmaf(qv, b, s1[r]);
      }
    }
    float corr[TW_RW];
#pragma unroll
    for (int r = 0; r < TW_RW; ++r) {
      const float a = i0 >= lo[r] && i0 <= hi[r] ? s0[r] * scale : -INFINITY;
      const float b = i1 >= lo[r] && i1 <= hi[r] ? s1[r] * scale : -INFINITY;
      const float mx = fmaxf(m[r], warp_max(fmaxf(a, b)));
      float p0 = 0.f, p1 = 0.f;
      corr[r] = 1.f;
      if (mx != -INFINITY) {      // uniform over the warp
        corr[r] = expf(m[r] - mx);
        p0 = expf(a - mx);
        p1 = expf(b - mx);
        l[r] = l[r] * corr[r] + warp_sum(p0 + p1);
        m[r] = mx;
      }
      Ps[(warp * TW_RW + r) * TW_KEYS + lane] = p0;
      Ps[(warp * TW_RW + r) * TW_KEYS + lane + 32] = p1;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < TW_RW; ++r)
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[r][c] *= corr[r];
    const float* pw = Ps + warp * TW_RW * TW_KEYS;
    for (int j = 0; j < valid; ++j) {
      float v[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int d = lane + 32 * c;
        v[c] = d < dv ? Vs[j * dv + d] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < TW_RW; ++r) {
        const float pj = pw[r * TW_KEYS + j];
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = fmaf(pj, v[c], acc[r][c]);
      }
    }
    __syncwarp();
  };
  // 1. the pooled rows that the block's last token sees
  const int blocks_seen = (P > 0 && last_pos - window >= 0) ? (last_pos - window + 1) / P : 0;
  int zero[TW_RW], top[TW_RW];
#pragma unroll
  for (int r = 0; r < TW_RW; ++r) { zero[r] = 0; top[r] = limit[r] < 0 ? -1 : seen[r] - 1; }
  for (int e0 = 0; e0 < blocks_seen; e0 += TW_KEYS) {
    const int valid = min(TW_KEYS, blocks_seen - e0);
    __syncthreads();              // the keys staged before are no longer read (and the queries are staged)
    for (int i = threadIdx.x; i < TW_KEYS * (dk + dv); i += blockDim.x) {
      const int j = i / (dk + dv), c = i - j * (dk + dv);
      float val = 0.f;
      if (j < valid) {
        const int e = e0 + j, end = e * P + P - 1;
        const int page = pages[end / PAGE];
        if (page >= 0 && page < n_pages) {
          const size_t rowi = ((size_t)page * G + g) * R + (e - (PAGE * (end / PAGE)) / P);
          val = c < dk ? pk[rowi * dk + c] : pv[rowi * dv + (c - dk)];
        }
      }
      if (c < dk) Ks[j * ks + c] = val; else Vs[j * dv + (c - dk)] = val;
    }
    __syncthreads();
    process(e0, zero, top, valid);
  }
  // 2. the window's pages: from the page of the first row's first key to the page of the last row's position
  const int kt_begin = max(0, first_pos - window + 1) / PAGE, kt_end = last_pos / PAGE;
  for (int kt = kt_begin; kt <= kt_end; ++kt) {
    const int page = pages[kt];
    const bool held = page >= 0 && page < n_pages;
    const T* kp = kcache + ((size_t)(held ? page : 0) * G + g) * PAGE * dk;
    const T* vp = vcache + ((size_t)(held ? page : 0) * G + g) * PAGE * dv;
    const int valid = held ? min(PAGE, last_pos + 1 - kt * PAGE) : 0;   // rows of the page that hold this block's keys
    __syncthreads();
    for (int i = threadIdx.x; i < PAGE * dk; i += blockDim.x) {
      const int j = i / dk, d = i - j * dk;
      Ks[j * ks + d] = j < valid ? to_f32(kp[i]) : 0.f;   // what lies behind is not this sequence's: never let it in
    }
    for (int i = threadIdx.x; i < PAGE * dv; i += blockDim.x) Vs[i] = i / dv < valid ? to_f32(vp[i]) : 0.f;
    __syncthreads();
    process(kt * PAGE, first, limit, valid);
  }
#pragma unroll
  for (int r = 0; r < TW_RW; ++r) {
    const int rr = row_base + warp * TW_RW + r;
    if (rr >= rows_total) continue;
    const int tok = rr / grp, head = g * grp + rr % grp;
    const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = lane + 32 * c;
      if (d < dv) out[((size_t)(tok0 + tok) * H + head) * dv + d] = from_f32<T>(acc[r][c] * inv);
    }
  }
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_qk_rope_norm_append(const float* qkv, const float* bias, void* q_out, int dtype, const int32_t* tok_pos,
                                          const int32_t* tok_seq, const int32_t* page_table, int table_stride, int n_pages,
                                          void* kcache, void* vcache, int n_tokens, int H, int G, int dk, int dv, int rot,
                                          const double* freq, float eps, int unit_norm, int* err, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && H > 0 && G > 0 && H % G == 0, "qk_rope_norm_append: %d query heads over %d key/value heads", H, G);
  EL_REFUSE(dk >= 1 && dk <= 256 && dv >= 1 && dv <= 256, "qk_rope_norm_append: head sizes %d / %d are not taken (1 to 256)", dk, dv);
  EL_REFUSE(rot >= 0 && rot <= dk && rot % 2 == 0, "qk_rope_norm_append: %d rotated dimensions of %d", rot, dk);
  const size_t smem = (size_t)PW_WARPS * dk * sizeof(float);
  if (dtype == DT_F32)
    launch_pdl(pdl_bit_for_tokens(n_tokens), qk_rope_norm_append_kernel<float>, dim3(n_tokens, (H + G + PW_WARPS - 1) / PW_WARPS), dim3(PW_WARPS * 32), (size_t)(smem), stream, qkv, bias, (float*)q_out, tok_pos, tok_seq, page_table, table_stride, n_pages,
                                                                              (float*)kcache, (float*)vcache, H, G, dk, dv, rot, freq, eps, unit_norm, err);
  else if (dtype == DT_BF16)
    launch_pdl(pdl_bit_for_tokens(n_tokens), qk_rope_norm_append_kernel<__nv_bfloat16>, dim3(n_tokens, (H + G + PW_WARPS - 1) / PW_WARPS), dim3(PW_WARPS * 32), (size_t)(smem), stream, qkv, bias, (__nv_bfloat16*)q_out, tok_pos, tok_seq, page_table, table_stride, n_pages,
                                                                                      (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, H, G, dk, dv, rot, freq, eps, unit_norm, err);
  else
    EL_REFUSE(false, "qk_rope_norm_append: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("qk_rope_norm_append");
  return 0;
}

extern "C" int edgelm_pool_blocks(const int32_t* tok_pos, const int32_t* tok_seq, const int32_t* page_table, int table_stride,
                                  int n_pages, const void* kcache, const void* vcache, int dtype, float* pk, float* pv,
                                  int n_tokens, int G, int dk, int dv, int P, int R, int* err, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && G > 0 && dk > 0 && dv > 0 && P >= 1 && R == (PAGE + P - 1) / P, "pool_blocks: bad sizes (block %d, rows a page %d)", P, R);
  if (dtype == DT_F32)
    launch_pdl(pdl_bit_for_tokens(n_tokens), pool_blocks_kernel<float>, dim3(n_tokens, G), dim3(128), (size_t)(0), stream, tok_pos, tok_seq, page_table, table_stride, n_pages, (const float*)kcache, (const float*)vcache, pk, pv, G, dk, dv, P, R, err);
  else if (dtype == DT_BF16)
    launch_pdl(pdl_bit_for_tokens(n_tokens), pool_blocks_kernel<__nv_bfloat16>, dim3(n_tokens, G), dim3(128), (size_t)(0), stream, tok_pos, tok_seq, page_table, table_stride, n_pages, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, pk, pv, G, dk, dv, P, R, err);
  else
    EL_REFUSE(false, "pool_blocks: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("pool_blocks");
  return 0;
}

extern "C" int edgelm_pooled_window_attn(const void* q, void* out, const void* kcache, const void* vcache, int dtype, const float* pk,
                                         const float* pv, const int32_t* tok_pos, const int32_t* tok_seq, const int32_t* page_table,
                                         int table_stride, int n_pages, int n_tokens, int H, int G, int dk, int dv, float scale,
                                         int window, int P, int R, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && H > 0 && G > 0 && H % G == 0, "pooled_window_attn: %d query heads over %d key/value heads", H, G);
  EL_REFUSE(dk >= 1 && dk <= 256 && dv >= 1 && dv <= 256, "pooled_window_attn: head sizes %d / %d are not taken (1 to 256)", dk, dv);
  EL_REFUSE(window >= 1 && P >= 0 && (P == 0 || R == (PAGE + P - 1) / P), "pooled_window_attn: window %d, block %d, rows a page %d", window, P, R);
  // few (token, head) pairs (a decode step): more warps a block share one query's keys
  const int nw = (long long)n_tokens * H >= 2 * 148 * 4 ? 4 : PW_MAX_WARPS;
  const dim3 grid(n_tokens, H), block(nw * 32);
  const size_t smem = (size_t)(((dk + 3) & ~3) + 2 * nw + nw * dv) * sizeof(float);
  const int esz = dtype == DT_F32 ? 4 : 2;
  const int vec_k = ((size_t)dk * esz) % 16 == 0 && (uintptr_t)kcache % 16 == 0;
  const int pair_v = dv % 2 == 0 && (uintptr_t)vcache % 8 == 0;
  EL_REFUSE(P == 0 || ((uintptr_t)pk % 16 == 0 && (uintptr_t)pv % 8 == 0), "pooled_window_attn: the pooled rows are not 16-byte aligned");
  EL_REFUSE((long long)n_pages * G * (PAGE > R ? PAGE : R) < (1ll << 31), "pooled_window_attn: more cache rows than a 32-bit index counts");
  const int dvr = dv <= 64 ? 1 : (dv <= 128 ? 2 : 4);
#define EL_PWA(TT, DVR) launch_pdl(pdl_bit_for_tokens(n_tokens), pooled_window_attn_kernel<TT, DVR>, dim3(grid), dim3(block), (size_t)(smem), stream, (const TT*)q, (TT*)out, (const TT*)kcache, (const TT*)vcache, pk, pv, \
      tok_pos, tok_seq, page_table, table_stride, n_pages, H, G, dk, dv, scale, window, P, R, vec_k, pair_v)
  if (dtype == DT_F32) {
    if (dvr == 1) EL_PWA(float, 1); else if (dvr == 2) EL_PWA(float, 2); else EL_PWA(float, 4);
  } else if (dtype == DT_BF16) {
    if (dvr == 1) EL_PWA(__nv_bfloat16, 1); else if (dvr == 2) EL_PWA(__nv_bfloat16, 2); else EL_PWA(__nv_bfloat16, 4);
  } else
    EL_REFUSE(false, "pooled_window_attn: unknown dtype code %d", dtype);
#undef EL_PWA
  EL_LAUNCH_CHECK("pooled_window_attn");
  return 0;
}

// The same attention for prompt steps: tiles (runs of at most `max_tile_tokens` consecutive tokens of one sequence, as
// the step's metadata lists them) instead of single tokens; `max_tile_tokens` x (H / G) rows are dealt to blocks of 32.
template <typename T, int NC>
static int launch_tiled(const void* q, void* out, const void* kc, const void* vc, const float* pk, const float* pv,
                        const int32_t* page_table, int table_stride, int n_pages, const int32_t* tile_seq, const int32_t* tile_tok0,
                        const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles, int max_tile_tokens, int H, int G, int dk, int dv,
                        float scale, int window, int P, int R, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)TW_KEYS * (dk + 1) + (size_t)TW_KEYS * dv + (size_t)TW_ROWS * dk + (size_t)TW_ROWS * TW_KEYS);
  auto kern = pooled_window_attn_tiled_kernel<T, NC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("pooled_window_attn_tiled: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return -2;
  }
  const dim3 grid(n_tiles, G, (max_tile_tokens * (H / G) + TW_ROWS - 1) / TW_ROWS);
  kern<<<grid, TW_WARPS * 32, smem, stream>>>((const T*)q, (T*)out, (const T*)kc, (const T*)vc, pk, pv, page_table, table_stride, n_pages, tile_seq,
                                             tile_tok0, tile_ntok, tile_pos0, H, G, dk, dv, scale, window, P, R);
  return 0;
}

extern "C" int edgelm_pooled_window_attn_tiled(const void* q, void* out, const void* kcache, const void* vcache, int dtype, const float* pk,
                                               const float* pv, const int32_t* page_table, int table_stride, int n_pages,
                                               const int32_t* tile_seq, const int32_t* tile_tok0, const int32_t* tile_ntok,
                                               const int32_t* tile_pos0, int n_tiles, int max_tile_tokens, int H, int G, int dk, int dv,
                                               float scale, int window, int P, int R, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  EL_REFUSE(n_tiles > 0 && max_tile_tokens > 0 && H > 0 && G > 0 && H % G == 0, "pooled_window_attn_tiled: %d query heads over %d key/value heads", H, G);
  EL_REFUSE(dk >= 1 && dk <= 256 && dv >= 1 && dv <= 256, "pooled_window_attn_tiled: head sizes %d / %d are not taken (1 to 256)", dk, dv);
  EL_REFUSE(window >= 1 && P >= 0 && (P == 0 || R == (PAGE + P - 1) / P), "pooled_window_attn_tiled: window %d, block %d, rows a page %d", window, P, R);
  EL_REFUSE(dtype == DT_F32 || dtype == DT_BF16, "pooled_window_attn_tiled: unknown dtype code %d", dtype);
  int rc;
#define EL_TW(NC)                                                                                                                                  \
  rc = dtype == DT_F32 ? launch_tiled<float, NC>(q, out, kcache, vcache, pk, pv, page_table, table_stride, n_pages, tile_seq, tile_tok0, tile_ntok, \
                                                 tile_pos0, n_tiles, max_tile_tokens, H, G, dk, dv, scale, window, P, R, stream)                    \
                       : launch_tiled<__nv_bfloat16, NC>(q, out, kcache, vcache, pk, pv, page_table, table_stride, n_pages, tile_seq, tile_tok0,   \
                                                         tile_ntok, tile_pos0, n_tiles, max_tile_tokens, H, G, dk, dv, scale, window, P, R, stream)
  if (dv <= 32) { EL_TW(1); } else if (dv <= 64) { EL_TW(2); } else if (dv <= 128) { EL_TW(4); } else { EL_TW(8); }
#undef EL_TW
  if (rc != 0) return rc;
  EL_LAUNCH_CHECK("pooled_window_attn_tiled");
  return 0;
}
