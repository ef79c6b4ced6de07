// Kernels of the parts that sit around the products of a gated pre-norm layer with a latent
// cache.  Everything here is memory-bound and computes in 32-bit; activations are read and
// written in the compute type (float or bfloat16), the residual stream is float.
//
//   embed_pair_norm   x_t = E[tok_t] * s + G[row(tok_{t-1}, tok_t)], then x / sqrt(mean(x^2) + eps) * w
//                     row(a, b) = (a * mul_prev + b * mul_cur) mod buckets; a sequence's first token
//                     takes row `buckets`.  The previous token of a step's first token comes from a
//                     two-place ring per slot that is indexed by position parity.
//   canon_conv        u_t = h_t + sum_j w[j, :] * h_{t - taps + 1 + j} per channel, causal (w is handed over
//                     as [taps, width], a tap's weights side by side).  Rows before
//                     the step's first come from a ring of `taps` rows per slot, indexed by
//                     position mod taps; rows before the sequence's start are zero.
//   latent_keep       c = rmsnorm(d) * w into the layer's latent page at the token's position, and
//                     the last taps - 1 rows of h of every sequence into its ring.
//   head_product      per head: q'_h = W_h^T q_h (the keys' up-projection taken into the query), or
//                     o_h = W_h a_h times sigmoid(gate_h) (the values' up-projection after the sum).
//   head_gate         o[t, h, :] *= sigmoid(gate[t, h])
//   gated_add         x += y * sigmoid(g + b), optionally followed by the RMS norm of the new x
//   xielu             a z^2 + z/2 above zero, (1/2 + b)(exp(z) - 1 - z) + z/2 below, a and b the
//                     softplus of two learned numbers
//
// Rings are indexed by position, never by step: a decode step that is taken back and run again
// at the same position reads what the step before it read.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// embedding with a pair table and a norm
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void __launch_bounds__(256)
embed_pair_norm_kernel(const TW *__restrict__ table, const TW *__restrict__ pairs,
                       const int *__restrict__ ids, const int *__restrict__ tok_pos,
                       const int *__restrict__ tok_seq, const int *__restrict__ seq_slots,
                       const int *__restrict__ seq_meta, int *__restrict__ ring,
                       const float *__restrict__ norm_w, float *__restrict__ out, int T, int H,
                       int V, float scale, long long buckets, long long mul_prev,
                       long long mul_cur, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ int prev_s;
  const int t = blockIdx.x;
  const int b = tok_seq[t], pos = tok_pos[t];
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;                     // the host validates ids; never read outside
  if (threadIdx.x == 0) {
    const bool first_of_step = (t == 0) || (tok_seq[t - 1] != b);
    int prev = -1;
    int *my_ring = ring + 2 * (size_t)seq_slots[b];
    if (pos > 0) prev = first_of_step ? my_ring[(pos - 1) & 1] : ids[t - 1];
    if (first_of_step) {
      // this block alone reads and writes the slot's ring in this launch: the read above comes first
      const int n = seq_meta ? seq_meta[4 * b + 1] : 1;
      my_ring[(pos + n - 1) & 1] = ids[t + n - 1];
    }
    prev_s = prev;
  }
  __syncthreads();
  const int prev = prev_s;
  long long row = buckets;
  if (prev >= 0) {
    row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  const TW *e = table + (size_t)id * H;
  const TW *g = pairs + (size_t)row * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = fmaf(to_f32(e[j]), scale, to_f32(g[j]));
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  float *o = out + (size_t)t * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = fmaf(to_f32(e[j]), scale, to_f32(g[j]));
    o[j] = (v * inv) * norm_w[j];
  }
}

extern "C" int g2b_embed_pair_norm(const void *table, const void *pairs, int table_dtype,
                                   const int *ids, const int *tok_pos, const int *tok_seq,
                                   const int *seq_slots, const int *seq_meta, int *ring,
                                   const float *norm_w, float *out, int T, int H, int V,
                                   float scale, long long buckets, long long mul_prev,
                                   long long mul_cur, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0 || buckets <= 0) G2B_REFUSE("embed_pair_norm: bad sizes H=%d V=%d buckets=%lld", H, V, buckets);
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  if (table_dtype == G2B_F32)
    g2b_launch(embed_pair_norm_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float *)table,
               (const float *)pairs, ids, tok_pos, tok_seq, seq_slots, seq_meta, ring, norm_w, out, T, H,
               V, scale, buckets, mul_prev, mul_cur, eps);
  else if (table_dtype == G2B_BF16)
    g2b_launch(embed_pair_norm_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16 *)table,
               (const bf16 *)pairs, ids, tok_pos, tok_seq, seq_slots, seq_meta, ring, norm_w, out, T, H,
               V, scale, buckets, mul_prev, mul_cur, eps);
  else
    G2B_REFUSE("embed_pair_norm: unknown table dtype %d", table_dtype);
  return g2b_check_launch("embed_pair_norm");
}

// ---------------------------------------------------------------------------
// causal convolution over time on each channel, added to its input.  One block per token; a
// thread takes eight neighbouring channels (16-byte loads) when the width allows, else one.
// ---------------------------------------------------------------------------
#define CANON_MAX_TAPS 16
#define CANON_TOKENS 8        // tokens of a block in a long step, a warp each (their set-up is shared)

template <typename TA> struct Vec8;
template <> struct Vec8<bf16> {
  uint4 raw;
  __device__ __forceinline__ void load(const bf16 *p) { raw = *reinterpret_cast<const uint4 *>(p); }
  __device__ __forceinline__ void store(bf16 *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
  __device__ __forceinline__ float get(int i) const {
    const uint32_t w = (&raw.x)[i >> 1];
    return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
  }
  __device__ __forceinline__ void set(const float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      (&raw.x)[i] = *reinterpret_cast<uint32_t *>(&p2);
    }
  }
};
template <> struct Vec8<float> {
  float4 lo, hi;
  __device__ __forceinline__ void load(const float *p) {
    lo = *reinterpret_cast<const float4 *>(p);
    hi = *reinterpret_cast<const float4 *>(p + 4);
  }
  __device__ __forceinline__ void store(float *p) const {
    *reinterpret_cast<float4 *>(p) = lo;
    *reinterpret_cast<float4 *>(p + 4) = hi;
  }
  __device__ __forceinline__ float get(int i) const { return i < 4 ? (&lo.x)[i] : (&hi.x)[i - 4]; }
  __device__ __forceinline__ void set(const float (&v)[8]) {
    lo = make_float4(v[0], v[1], v[2], v[3]);
    hi = make_float4(v[4], v[5], v[6], v[7]);
  }
};

template <typename TA, bool VEC>
__global__ void __launch_bounds__(256)
canon_conv_kernel(const TA *__restrict__ h, const float *__restrict__ w, const TA *__restrict__ ring,
                  const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                  const int *__restrict__ seq_slots, TA *__restrict__ out, int T, int H, int taps,
                  int per_block) {
  pdl_launch();
  pdl_wait();
  // the row that lies k steps back of each of the block's tokens; nullptr: before the start
  __shared__ const TA *all_src[CANON_TOKENS][CANON_MAX_TAPS];
  const int first = blockIdx.x * per_block;
  for (int i = threadIdx.x; i < per_block * taps; i += blockDim.x) {
    const int t = first + i / taps, k = i % taps;
    const TA *p = nullptr;
    if (t < T) {
      const int b = tok_seq[t], pos = tok_pos[t];
      if (pos - k >= 0) {
        if (t - k >= 0 && tok_seq[t - k] == b) p = h + (size_t)(t - k) * H;
        else p = ring + ((size_t)seq_slots[b] * taps + (pos - k) % taps) * H;
      }
    }
    all_src[i / taps][k] = p;
  }
  __syncthreads();
  // one token per block: all threads on its row; several: a warp per token, so that every warp
  // has its own row's loads in flight
  const int ti = per_block > 1 ? (int)(threadIdx.x >> 5) : 0;
  const int me = per_block > 1 ? (int)(threadIdx.x & 31) : (int)threadIdx.x;
  const int team = per_block > 1 ? 32 : (int)blockDim.x;
  const int t = first + ti;
  if (ti >= per_block || t >= T) return;
  const TA *const *src = all_src[ti];
  if (VEC) {
    for (int j = 8 * me; j < H; j += 8 * team) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int k = taps - 1; k >= 0; --k) {            // oldest first: the order of the taps
        if (!src[k]) continue;
        Vec8<TA> v;
        v.load(src[k] + j);
        Vec8<float> wk;                                // the tap's weights of these eight channels
        wk.load(w + (size_t)(taps - 1 - k) * H + j);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(wk.get(i), v.get(i), acc[i]);
      }
      Vec8<TA> own;
      own.load(src[0] + j);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += own.get(i);
      own.set(acc);
      own.store(out + (size_t)t * H + j);
    }
  } else {
    for (int j = me; j < H; j += team) {
      float acc = 0.f;
      for (int k = taps - 1; k >= 0; --k)
        if (src[k]) acc = fmaf(w[(size_t)(taps - 1 - k) * H + j], to_f32(src[k][j]), acc);
      out[(size_t)t * H + j] = from_f32<TA>(to_f32(src[0][j]) + acc);
    }
  }
}

extern "C" int g2b_canon_conv(const void *h, const float *w, const void *ring, int dtype,
                              const int *tok_pos, const int *tok_seq, const int *seq_slots,
                              void *out, int T, int H, int taps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || taps > CANON_MAX_TAPS) G2B_REFUSE("canon_conv: %d taps outside 1..%d", taps, CANON_MAX_TAPS);
  const bool vec = H % 8 == 0 && (((uintptr_t)h | (uintptr_t)ring | (uintptr_t)out | (uintptr_t)w) & 15) == 0;
  const int per = vec ? 8 : 1;
  int threads = (H / per + 31) / 32 * 32;
  threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
  const int per_block = T >= 256 ? CANON_TOKENS : 1;
  if (per_block > 1) threads = 32 * CANON_TOKENS;
  const dim3 grid((T + per_block - 1) / per_block);
  if (dtype == G2B_F32) {
    auto k = vec ? canon_conv_kernel<float, true> : canon_conv_kernel<float, false>;
    g2b_launch(k, grid, dim3(threads), 0, stream, (const float *)h, w, (const float *)ring, tok_pos,
               tok_seq, seq_slots, (float *)out, T, H, taps, per_block);
  } else if (dtype == G2B_BF16) {
    auto k = vec ? canon_conv_kernel<bf16, true> : canon_conv_kernel<bf16, false>;
    g2b_launch(k, grid, dim3(threads), 0, stream, (const bf16 *)h, w, (const bf16 *)ring, tok_pos,
               tok_seq, seq_slots, (bf16 *)out, T, H, taps, per_block);
  } else {
    G2B_REFUSE("canon_conv: unknown dtype %d", dtype);
  }
  return g2b_check_launch("canon_conv");
}

// The same for a step of one token per sequence, with the norm in front of it and the ring's
// update behind it in one launch: h = x / sqrt(mean(x^2) + eps) * g (rounded to the compute type,
// as the other path stores it), u = h + conv(h) with the earlier rows from the ring, and h into
// the ring at the token's position.  A slot's ring is read and written by its token's block only.
// With `y`: the gated addition that the layer in front left undone comes first, x += y * sigmoid(ga + gb).
template <typename TA>
__global__ void __launch_bounds__(1024)
norm_canon_single_kernel(float *__restrict__ x, const float *__restrict__ g, float eps,
                         const float *__restrict__ w, TA *__restrict__ ring,
                         const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                         const int *__restrict__ seq_slots, TA *__restrict__ h_out,
                         TA *__restrict__ u_out, int H, int taps, const float *__restrict__ y,
                         const TA *__restrict__ ga, int ga_stride, const float *__restrict__ gb) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  TA *my_ring = ring + (size_t)seq_slots[tok_seq[t]] * taps * H;
  float *xr = x + (size_t)t * H;
  float ss = 0.f;
  if (y) {
    const float *yr = y + (size_t)t * H;
    const TA *gr = ga + (size_t)t * ga_stride;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      const float v = fmaf(yr[j], sigmoid_f(to_f32(gr[j]) + (gb ? gb[j] : 0.f)), xr[j]);
      xr[j] = v;                                       // read back below by the thread that wrote it
      ss = fmaf(v, v, ss);
    }
  } else {
    for (int j = threadIdx.x; j < H; j += blockDim.x) ss = fmaf(xr[j], xr[j], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const TA hr = from_f32<TA>((g[j] * xr[j]) * inv);
    const float hv = to_f32(hr);
    float acc = 0.f;
    for (int k = taps - 1; k >= 1; --k)               // oldest first; rows before the start are zero
      if (pos - k >= 0) acc = fmaf(w[(size_t)(taps - 1 - k) * H + j], to_f32(my_ring[(size_t)((pos - k) % taps) * H + j]), acc);
    acc = fmaf(w[(size_t)(taps - 1) * H + j], hv, acc);
    h_out[(size_t)t * H + j] = hr;
    u_out[(size_t)t * H + j] = from_f32<TA>(hv + acc);
    if (taps > 1) my_ring[(size_t)(pos % taps) * H + j] = hr;
  }
}

extern "C" int g2b_norm_canon_single(float *x, const float *g, float eps, const float *w, void *ring,
                                     int dtype, const int *tok_pos, const int *tok_seq,
                                     const int *seq_slots, void *h_out, void *u_out, int T, int H,
                                     int taps, const float *y, const void *ga, int ga_stride,
                                     const float *gb, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || taps > CANON_MAX_TAPS) G2B_REFUSE("norm_canon: %d taps outside 1..%d", taps, CANON_MAX_TAPS);
  int threads = (H / 2 + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  if (dtype == G2B_F32)
    g2b_launch(norm_canon_single_kernel<float>, dim3(T), dim3(threads), 0, stream, x, g, eps, w, (float *)ring,
               tok_pos, tok_seq, seq_slots, (float *)h_out, (float *)u_out, H, taps, y, (const float *)ga,
               ga_stride, gb);
  else if (dtype == G2B_BF16)
    g2b_launch(norm_canon_single_kernel<bf16>, dim3(T), dim3(threads), 0, stream, x, g, eps, w, (bf16 *)ring,
               tok_pos, tok_seq, seq_slots, (bf16 *)h_out, (bf16 *)u_out, H, taps, y, (const bf16 *)ga,
               ga_stride, gb);
  else
    G2B_REFUSE("norm_canon: unknown dtype %d", dtype);
  return g2b_check_launch("norm_canon");
}

// ---------------------------------------------------------------------------
// what a layer keeps of a token: its normed latent in the page of its position, and (the last
// taps - 1 tokens of each sequence in the step) the row the convolution will need next
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128)
latent_keep_kernel(const TA *__restrict__ d, int d_stride, int rank, const float *__restrict__ norm_w,
                   float eps, TA *__restrict__ pages, const int *__restrict__ page_table, int P,
                   int page_size, const TA *__restrict__ h, TA *__restrict__ ring, int H, int taps,
                   const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                   const int *__restrict__ seq_slots, int T) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int b = tok_seq[t], pos = tok_pos[t];
  if (d) {
    const TA *dr = d + (size_t)t * d_stride;
    float ss = 0.f;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) {
      const float v = to_f32(dr[j]);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    const int page = page_table[(size_t)b * P + pos / page_size];
    TA *row = pages + ((size_t)page * page_size + pos % page_size) * rank;
    for (int j = threadIdx.x; j < rank; j += blockDim.x)
      row[j] = from_f32<TA>((to_f32(dr[j]) * inv) * norm_w[j]);
  }
  if (ring && taps > 1) {
    // among the last taps - 1 tokens of its sequence in this step?
    const int ahead = t + taps - 1;
    if (ahead >= T || tok_seq[ahead] != b) {
      TA *row = ring + ((size_t)seq_slots[b] * taps + pos % taps) * H;
      const TA *hr = h + (size_t)t * H;
      for (int j = threadIdx.x; j < H; j += blockDim.x) row[j] = hr[j];
    }
  }
}

extern "C" int g2b_latent_keep(const void *d, int d_stride, int rank, const float *norm_w, float eps,
                               void *pages, const int *page_table, int P, int page_size,
                               const void *h, void *ring, int H, int taps, int dtype,
                               const int *tok_pos, const int *tok_seq, const int *seq_slots, int T,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d && (rank <= 0 || page_size <= 0)) G2B_REFUSE("latent_keep: bad sizes rank=%d page=%d", rank, page_size);
  if (dtype == G2B_F32)
    g2b_launch(latent_keep_kernel<float>, dim3(T), dim3(128), 0, stream, (const float *)d, d_stride, rank,
               norm_w, eps, (float *)pages, page_table, P, page_size, (const float *)h, (float *)ring, H,
               taps, tok_pos, tok_seq, seq_slots, T);
  else if (dtype == G2B_BF16)
    g2b_launch(latent_keep_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16 *)d, d_stride, rank,
               norm_w, eps, (bf16 *)pages, page_table, P, page_size, (const bf16 *)h, (bf16 *)ring, H,
               taps, tok_pos, tok_seq, seq_slots, T);
  else
    G2B_REFUSE("latent_keep: unknown dtype %d", dtype);
  return g2b_check_launch("latent_keep");
}

// ---------------------------------------------------------------------------
// products with one small matrix per head.  W [heads * n, r] (rows of head h: h*n .. h*n+n-1).
//   absorb: out[t, h, 0..r)  = sum_i W[h*n + i, :] * in[t, h, i]        (W_h^T applied; in has n per head)
//   expand: out[t, h, 0..n)  = W[h*n + i, :] . in[t, h, :], times sigmoid(gate[t, h]) when gate
// One block per (head, tile of HP_ROWS tokens); the sum over the inner index always runs in
// the same order, so a token's result does not depend on its tile.
// ---------------------------------------------------------------------------
#define HP_ROWS 8
#define HP_THREADS 256
#define HP_COLS 64            // absorb: output columns per block (two per lane), the inner index dealt to the 8 warps

template <typename TA>
__global__ void __launch_bounds__(HP_THREADS)
head_absorb_kernel(const TA *__restrict__ in, int in_stride, const TA *__restrict__ W,
                   TA *__restrict__ out, int out_stride, int T, int heads, int n, int r) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float hp_smem[];                  // [HP_ROWS][n], then [8 warps][HP_ROWS][HP_COLS]
  float *part = hp_smem + HP_ROWS * n;
  const int h = blockIdx.x, t0 = blockIdx.y * HP_ROWS, c0 = blockIdx.z * HP_COLS;
  const int rows = min(HP_ROWS, T - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < HP_ROWS * n; i += blockDim.x) {
    const int m = i / n, k = i % n;
    hp_smem[i] = m < rows ? to_f32(in[(size_t)(t0 + m) * in_stride + (size_t)h * n + k]) : 0.f;
  }
  __syncthreads();
  const TA *Wh = W + (size_t)h * n * r;
  const int ca = c0 + 2 * lane, cb = ca + 1;
  float acc[HP_ROWS][2];
#pragma unroll
  for (int m = 0; m < HP_ROWS; ++m) acc[m][0] = acc[m][1] = 0.f;
  for (int k = warp; k < n; k += HP_THREADS / 32) {    // warp w: inner indices w, w + 8, ...
    const float wa = ca < r ? to_f32(Wh[(size_t)k * r + ca]) : 0.f;
    const float wb = cb < r ? to_f32(Wh[(size_t)k * r + cb]) : 0.f;
#pragma unroll
    for (int m = 0; m < HP_ROWS; ++m) {
      const float x = hp_smem[m * n + k];
      acc[m][0] = fmaf(wa, x, acc[m][0]);
      acc[m][1] = fmaf(wb, x, acc[m][1]);
    }
  }
#pragma unroll
  for (int m = 0; m < HP_ROWS; ++m) {
    part[(warp * HP_ROWS + m) * HP_COLS + 2 * lane] = acc[m][0];
    part[(warp * HP_ROWS + m) * HP_COLS + 2 * lane + 1] = acc[m][1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < HP_ROWS * HP_COLS; i += blockDim.x) {     // the warps' parts in warp order
    const int m = i / HP_COLS, c = i % HP_COLS;
    if (m >= rows || c0 + c >= r) continue;
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < HP_THREADS / 32; ++wi) v += part[(wi * HP_ROWS + m) * HP_COLS + c];
    out[(size_t)(t0 + m) * out_stride + (size_t)h * r + c0 + c] = from_f32<TA>(v);
  }
}

// expand: a warp per output number of a head (8 per block), lanes over the rank
template <typename TA>
__global__ void __launch_bounds__(HP_THREADS)
head_expand_kernel(const TA *__restrict__ in, int in_stride, const TA *__restrict__ W,
                   const TA *__restrict__ gate, int gate_stride, TA *__restrict__ out,
                   int out_stride, int T, int heads, int n, int r) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float hp_smem[];                  // [HP_ROWS][r]
  const int h = blockIdx.x, t0 = blockIdx.y * HP_ROWS;
  const int rows = min(HP_ROWS, T - t0);
  for (int i = threadIdx.x; i < HP_ROWS * r; i += blockDim.x) {
    const int m = i / r, k = i % r;
    hp_smem[i] = m < rows ? to_f32(in[(size_t)(t0 + m) * in_stride + (size_t)h * r + k]) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.z * (HP_THREADS / 32) + warp;
  if (i >= n) return;
  const TA *wr = W + ((size_t)h * n + i) * r;
  float acc[HP_ROWS];
#pragma unroll
  for (int m = 0; m < HP_ROWS; ++m) acc[m] = 0.f;
  for (int k = lane; k < r; k += 32) {
    const float w = to_f32(wr[k]);
#pragma unroll
    for (int m = 0; m < HP_ROWS; ++m) acc[m] = fmaf(w, hp_smem[m * r + k], acc[m]);
  }
#pragma unroll
  for (int m = 0; m < HP_ROWS; ++m) acc[m] = warp_sum(acc[m]);
  if (lane < rows) {
    float v = acc[0];
#pragma unroll
    for (int m = 1; m < HP_ROWS; ++m) v = lane == m ? acc[m] : v;
    if (gate) v *= sigmoid_f(to_f32(gate[(size_t)(t0 + lane) * gate_stride + h]));
    out[(size_t)(t0 + lane) * out_stride + (size_t)h * n + i] = from_f32<TA>(v);
  }
}

extern "C" int g2b_head_product(const void *in, int in_stride, const void *W, const void *gate,
                                int gate_stride, void *out, int out_stride, int T, int heads, int n,
                                int r, int expand, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || n <= 0 || r <= 0) G2B_REFUSE("head_product: bad sizes heads=%d n=%d r=%d", heads, n, r);
  const size_t smem = sizeof(float) * HP_ROWS * (size_t)(expand ? r : n + (HP_THREADS / 32) * HP_COLS);
  if (smem > 48 * 1024) G2B_REFUSE("head_product: %d values per head and token are more than fit", expand ? r : n);
  const dim3 grid(heads, (T + HP_ROWS - 1) / HP_ROWS,
                  expand ? (n + HP_THREADS / 32 - 1) / (HP_THREADS / 32) : (r + HP_COLS - 1) / HP_COLS);
  if (grid.y > 65535 || grid.z > 65535) G2B_REFUSE("head_product: %d tokens or %d outputs per head are too many", T, expand ? n : r);
  if (dtype == G2B_F32) {
    if (expand)
      g2b_launch(head_expand_kernel<float>, grid, dim3(HP_THREADS), smem, stream, (const float *)in, in_stride,
                 (const float *)W, (const float *)gate, gate_stride, (float *)out, out_stride, T, heads, n, r);
    else
      g2b_launch(head_absorb_kernel<float>, grid, dim3(HP_THREADS), smem, stream, (const float *)in, in_stride,
                 (const float *)W, (float *)out, out_stride, T, heads, n, r);
  } else if (dtype == G2B_BF16) {
    if (expand)
      g2b_launch(head_expand_kernel<bf16>, grid, dim3(HP_THREADS), smem, stream, (const bf16 *)in, in_stride,
                 (const bf16 *)W, (const bf16 *)gate, gate_stride, (bf16 *)out, out_stride, T, heads, n, r);
    else
      g2b_launch(head_absorb_kernel<bf16>, grid, dim3(HP_THREADS), smem, stream, (const bf16 *)in, in_stride,
                 (const bf16 *)W, (bf16 *)out, out_stride, T, heads, n, r);
  } else {
    G2B_REFUSE("head_product: unknown dtype %d", dtype);
  }
  return g2b_check_launch("head_product");
}

// o[t, h, :] *= sigmoid(gate[t, h]); o [T, heads * n] contiguous.  A block per token.
template <typename TA, bool VEC>
__global__ void __launch_bounds__(256)
head_gate_kernel(TA *__restrict__ o, const TA *__restrict__ gate, int gate_stride, int heads, int n) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float hg_smem[];                  // sigmoid of the token's gates
  const int t = blockIdx.x, W = heads * n;
  for (int h = threadIdx.x; h < heads; h += blockDim.x)
    hg_smem[h] = sigmoid_f(to_f32(gate[(size_t)t * gate_stride + h]));
  __syncthreads();
  TA *row = o + (size_t)t * W;
  if (VEC) {                                           // n is a multiple of 8: a vector lies inside one head
    for (int j = 8 * threadIdx.x; j < W; j += 8 * blockDim.x) {
      Vec8<TA> v;
      v.load(row + j);
      const float g = hg_smem[j / n];
      float r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) r[i] = v.get(i) * g;
      v.set(r);
      v.store(row + j);
    }
  } else {
    for (int j = threadIdx.x; j < W; j += blockDim.x) row[j] = from_f32<TA>(to_f32(row[j]) * hg_smem[j / n]);
  }
}

extern "C" int g2b_head_gate(void *o, const void *gate, int gate_stride, int T, int heads, int n,
                             int dtype, cudaStream_t stream) {
  if (T <= 0 || heads <= 0 || n <= 0) return 0;
  const bool vec = n % 8 == 0 && ((uintptr_t)o & 15) == 0;
  int threads = (heads * n / (vec ? 8 : 1) + 31) / 32 * 32;
  threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
  const size_t smem = sizeof(float) * heads;
  if (smem > 48 * 1024) G2B_REFUSE("head_gate: %d heads", heads);
  if (dtype == G2B_F32) {
    auto k = vec ? head_gate_kernel<float, true> : head_gate_kernel<float, false>;
    g2b_launch(k, dim3(T), dim3(threads), smem, stream, (float *)o, (const float *)gate, gate_stride, heads, n);
  } else if (dtype == G2B_BF16) {
    auto k = vec ? head_gate_kernel<bf16, true> : head_gate_kernel<bf16, false>;
    g2b_launch(k, dim3(T), dim3(threads), smem, stream, (bf16 *)o, (const bf16 *)gate, gate_stride, heads, n);
  } else {
    G2B_REFUSE("head_gate: unknown dtype %d", dtype);
  }
  return g2b_check_launch("head_gate");
}

// ---------------------------------------------------------------------------
// x += y * sigmoid(g + b); then, when `normed` is given, normed = x / sqrt(mean(x^2) + eps) * w
// (the norm in front of the next sublayer).  One block per row.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(1024)
gated_add_kernel(float *__restrict__ x, const float *__restrict__ y, const TA *__restrict__ g,
                 int g_stride, const float *__restrict__ bias, int H, const float *__restrict__ norm_w,
                 float eps, TA *__restrict__ normed) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float *xr = x + (size_t)t * H;
  const float *yr = y + (size_t)t * H;
  const TA *gr = g + (size_t)t * g_stride;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float z = to_f32(gr[j]) + (bias ? bias[j] : 0.f);
    const float v = fmaf(yr[j], sigmoid_f(z), xr[j]);
    xr[j] = v;
    ss = fmaf(v, v, ss);
  }
  if (!normed) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TA *o = normed + (size_t)t * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x)   // a thread reads back what it wrote itself
    o[j] = from_f32<TA>(((norm_w ? norm_w[j] : 1.f) * xr[j]) * inv);          // the order of the norm kernels
}

extern "C" int g2b_gated_add(float *x, const float *y, const void *g, int g_stride, const float *bias,
                             int T, int H, const float *norm_w, float eps, void *normed, int dtype,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  // few rows (a decode step): two elements a thread, the row's latency is what counts; many rows: eight
  int threads = (H / (T <= 256 ? 2 : 8) + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  if (dtype == G2B_F32)
    g2b_launch(gated_add_kernel<float>, dim3(T), dim3(threads), 0, stream, x, y, (const float *)g, g_stride,
               bias, H, norm_w, eps, (float *)normed);
  else if (dtype == G2B_BF16)
    g2b_launch(gated_add_kernel<bf16>, dim3(T), dim3(threads), 0, stream, x, y, (const bf16 *)g, g_stride,
               bias, H, norm_w, eps, (bf16 *)normed);
  else
    G2B_REFUSE("gated_add: unknown dtype %d", dtype);
  return g2b_check_launch("gated_add");
}

// ---------------------------------------------------------------------------
// xIELU on the first F columns of a [T, stride] buffer
// ---------------------------------------------------------------------------
// exp(z) - 1 for z <= 0.  Where the result is rounded to bfloat16 the absolute error of
// exp(z) - 1 by the fast exponential (1e-7) is far below half a unit of z / 2, the term beside it.
template <typename TA> __device__ __forceinline__ float exp_minus_one(float z) { return expm1f(z); }
template <> __device__ __forceinline__ float exp_minus_one<bf16>(float z) { return __expf(z) - 1.f; }

template <typename TA, bool VEC>
__global__ void __launch_bounds__(256)
xielu_kernel(const TA *__restrict__ in, int in_stride, const float *__restrict__ pq,
             TA *__restrict__ out, int F) {
  pdl_launch();
  pdl_wait();
  __shared__ float coef[2];
  if (threadIdx.x < 2) coef[threadIdx.x] = (threadIdx.x ? 0.5f : 0.f) + softplus_f(pq[threadIdx.x]);
  __syncthreads();
  const float a = coef[0], bq = coef[1];
  const TA *row = in + (size_t)blockIdx.x * in_stride;           // rows along x: a step may have any number of them
  TA *orow = out + (size_t)blockIdx.x * F;
  if (VEC) {
    const int j = 8 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (j >= F) return;
    Vec8<TA> v;
    v.load(row + j);
    float r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float z = v.get(i);
      r[i] = z > 0.f ? fmaf(a * z, z, 0.5f * z) : fmaf(bq, exp_minus_one<TA>(z) - z, 0.5f * z);
    }
    v.set(r);
    v.store(orow + j);
  } else {
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= F) return;
    const float z = to_f32(row[j]);
    orow[j] = from_f32<TA>(z > 0.f ? fmaf(a * z, z, 0.5f * z) : fmaf(bq, expm1f(z) - z, 0.5f * z));
  }
}

extern "C" int g2b_xielu(const void *in, int in_stride, const float *pq, void *out, int T, int F,
                         int dtype, cudaStream_t stream) {
  if (T <= 0 || F <= 0) return 0;
  const size_t es = dtype == G2B_F32 ? 4 : 2;
  const bool vec = F % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                   ((size_t)in_stride * es) % 16 == 0;
  const int per = vec ? 8 : 1;
  const dim3 grid(T, ((F + per - 1) / per + 255) / 256);
  if (grid.y > 65535) G2B_REFUSE("xielu: %d columns are too many", F);
  if (dtype == G2B_F32) {
    auto k = vec ? xielu_kernel<float, true> : xielu_kernel<float, false>;
    g2b_launch(k, grid, dim3(256), 0, stream, (const float *)in, in_stride, pq, (float *)out, F);
  } else if (dtype == G2B_BF16) {
    auto k = vec ? xielu_kernel<bf16, true> : xielu_kernel<bf16, false>;
    g2b_launch(k, grid, dim3(256), 0, stream, (const bf16 *)in, in_stride, pq, (bf16 *)out, F);
  } else {
    G2B_REFUSE("xielu: unknown dtype %d", dtype);
  }
  return g2b_check_launch("xielu");
}
