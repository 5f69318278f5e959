// layered_blocks.cuh — device code of the layered-model engine for models whose layers are  x += norm(sublayer(x))  (the sublayer
// reads the residual stream itself; a layer norm with weight and bias, or an RMS norm with a weight stored around zero, closes it),
// with a learned position table or a computed sine/cosine position vector, short causal convolutions in front of a gated delta
// rule, the two-sided xIELU activation and mixtures of experts (gated silu or relu^2 experts, two routing rules).
// Also the pre-norm block form whose norm weights are one number each: the stream kept in several copies mixed by
// hyper-connections, and a causal convolution added to every sublayer input (embed_streams_kernel, hc_open_kernel, short_conv_kernel).
//
// Number formats as in layered_kernels.cuh: T is the storage type of weights and GEMM inputs (bf16 serving, float in the 32-bit
// mode); the residual stream, norms, router, decays, step sizes, unit vectors and every state are fp32 whatever T is.
#pragma once
#include "layered_kernels.cuh"

namespace xl {

// sum over the block (all threads get it); `red` holds 32 floats; ends with a barrier so `red` can be reused at once
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ---------------------------------------------------------------------------------------------------------------------------
// embedding with a learned position table:  x[m, :] = embed[token[m], :] + pos[row_pos[m], :]  (fp32), and its T copy h (the
// operand of the first sublayer's products).  pos_table may be NULL.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_pos_rows_kernel(const T* __restrict__ embed, const T* __restrict__ pos_table, const int* __restrict__ tokens,
                                      const int* __restrict__ row_pos, float* __restrict__ x, T* __restrict__ h, int D) {
  const int m = blockIdx.x;
  const T* src = embed + (size_t)tokens[m] * D;
  const T* ps = pos_table ? pos_table + (size_t)row_pos[m] * D : nullptr;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = ldf(src + d) + (ps ? ldf(ps + d) : 0.f);
    x[(size_t)m * D + d] = v;
    if (h) stf(h + (size_t)m * D + d, v);
  }
}
// the T copy of an fp32 stream (a later shard starts from the residual stream it is given)
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ h, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) stf(h + i, x[i]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Layer norm that closes a sublayer:   x[m] += (t - mean) / sqrt(var + eps) * w + b,  t = y[m] + y_bias ;   h[m] = T(x[m])     (y != NULL)
// or norms gathered rows of the stream: h[m] = T((x[src_rows[m]] - mean) / sqrt(var + eps) * w + b)            (y == NULL)
// var = mean of the squared deviations (two passes over the row, which waits in shared memory).  One block per row;
// dynamic shared memory: D floats.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void residual_layernorm_kernel(float* __restrict__ x, const float* __restrict__ y, const T* __restrict__ y_bias, const T* __restrict__ w,
                                          const T* __restrict__ b, T* __restrict__ h, const int* __restrict__ src_rows, int D, float eps) {
  extern __shared__ float ln_row[];
  __shared__ float red[32];
  const int m = blockIdx.x;
  const float* in = y ? y + (size_t)m * D : x + (size_t)(src_rows ? src_rows[m] : m) * D;
  float s = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = in[d] + (y && y_bias ? ldf(y_bias + d) : 0.f); ln_row[d] = v; s += v; }
  const float mean = block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = ln_row[d] - mean; q = fmaf(c, c, q); }
  const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = (ln_row[d] - mean) * rstd * ldf(w + d) + ldf(b + d);
    if (y) {
      v += x[(size_t)m * D + d];
      x[(size_t)m * D + d] = v;
    }
    if (h) stf(h + (size_t)m * D + d, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// embedding with a computed position vector:  e[d] = embed[token[m], d] + (d even ? sin : cos)(row_pos[m] * freqs[d / 2]), the
// angle in fp32 (freqs are rounded once from double on the host; NULL = no such vector), + pos_table[row_pos[m], d] when there is
// a learned table; then, when w_norm != NULL, the RMS norm x = e / sqrt(mean(e^2) + eps) * (w_offset + w_norm).  Writes the fp32
// stream x and its T copy h.  One block per row; dynamic shared memory: D floats.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_sinusoid_rows_kernel(const T* __restrict__ embed, const T* __restrict__ pos_table, const float* __restrict__ freqs,
                                           const int* __restrict__ tokens, const int* __restrict__ row_pos, const T* __restrict__ w_norm, float w_offset,
                                           float eps, float* __restrict__ x, T* __restrict__ h, int D) {
  extern __shared__ float ln_row[];
  __shared__ float red[32];
  const int m = blockIdx.x;
  const T* src = embed + (size_t)tokens[m] * D;
  const T* ps = pos_table ? pos_table + (size_t)row_pos[m] * D : nullptr;
  const float p = (float)row_pos[m];
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = ldf(src + d) + (ps ? ldf(ps + d) : 0.f);
    if (freqs) {
      const float ang = p * freqs[d >> 1];
      v += (d & 1) ? cosf(ang) : sinf(ang);
    }
    ln_row[d] = v;                                             // read back by the same thread only
    ss = fmaf(v, v, ss);
  }
  const float r = w_norm ? 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps) : 1.0f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = w_norm ? ln_row[d] * r * (w_offset + ldf(w_norm + d)) : ln_row[d];
    x[(size_t)m * D + d] = v;
    if (h) stf(h + (size_t)m * D + d, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// RMS norm that closes a sublayer:   t = y[m] + y_bias ;  x[m] += t / sqrt(mean(t^2) + eps) * (w_offset + w) ;  h[m] = T(x[m])
// or norms gathered rows of the stream: h[m] = T(x[src_rows[m]] / sqrt(mean(.^2) + eps) * (w_offset + w))        (y == NULL)
// w_offset = 1 for weights stored around zero, 0 for plain weights; y_bias (may be NULL) is the bias of the projection that made
// y, added here so that it costs no pass of its own.  One block per row; dynamic shared memory: D floats.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void residual_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const T* __restrict__ y_bias, const T* __restrict__ w,
                                        float w_offset, T* __restrict__ h, const int* __restrict__ src_rows, int D, float eps) {
  extern __shared__ float ln_row[];
  __shared__ float red[32];
  const int m = blockIdx.x;
  const float* in = y ? y + (size_t)m * D : x + (size_t)(src_rows ? src_rows[m] : m) * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = in[d] + (y && y_bias ? ldf(y_bias + d) : 0.f);
    ln_row[d] = v;                                             // read back by the same thread only
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = ln_row[d] * r * (w_offset + ldf(w + d));
    if (y) {
      v += x[(size_t)m * D + d];
      x[(size_t)m * D + d] = v;
    }
    if (h) stf(h + (size_t)m * D + d, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Short causal convolution on C channels of an fp32 matrix (a projection output, or a normed sublayer input):
//   out[m, c] = act( bias[c] + sum_{i < taps} w[c, i] * in(pos_m - (taps - 1 - i), c) )  (+ in(pos_m, c) when `residual`)
// act: 0 none, 1 silu.  in(p, c) is the input of the request's token at position p: a row of this step when p >= the step's first
// position of the request, else one of the last taps-1 inputs of earlier steps, kept per slot in `state` ([taps - 1][C] fp32, zero
// at the start of a request, so positions before 0 read as zero).  TO = float or the storage type (the operand of a product).
// grid (requests, ceil(C / 256), row stretches): stretch z takes rows [z * per, (z + 1) * per) with per >= taps - 1, so only stretch 0
// reads the state — and the thread that read channel c's state moves that channel's window on afterwards (the last taps - 1 inputs
// of the request so far), in the same launch.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T, typename TO>
__global__ void short_conv_kernel(const float* __restrict__ proj, int ld, int col0, int C, const T* __restrict__ w, const T* __restrict__ bias, int taps,
                                  int act, int residual, const Item* __restrict__ seqs, float* __restrict__ state, size_t state_slot_stride,
                                  TO* __restrict__ out, int ld_out) {
  const Item sq = seqs[blockIdx.x];
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float* st = state + (size_t)sq.slot * state_slot_stride;
  const float b = bias ? ldf(bias + c) : 0.f;
  const int per = max((sq.n_rows + (int)gridDim.z - 1) / (int)gridDim.z, taps - 1);
  const int t_begin = blockIdx.z * per, t_end = min(sq.n_rows, t_begin + per);
  // in(p, c) for a row offset src of this step (negative: before it)
  auto input = [&](int src) { return src >= 0 ? proj[(size_t)(sq.row0 + src) * ld + col0 + c] : st[(size_t)(src + taps - 1) * C + c]; };
  constexpr int RT = 8;                                        // up to RT taps: weights and the sliding window stay in registers, one load per row
  if (taps <= RT) {
    float wr[RT], win[RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) {
      wr[i] = i < taps ? ldf(w + (size_t)c * taps + i) : 0.f;
      win[i] = (i < taps - 1 && t_begin < t_end) ? input(t_begin - (taps - 1) + i) : 0.f;
    }
    for (int t = t_begin; t < t_end; ++t) {
      const float cur = proj[(size_t)(sq.row0 + t) * ld + col0 + c];
      float acc = b;
#pragma unroll
      for (int i = 0; i < RT; ++i) {
        if (i == taps - 1) win[i] = cur;
        if (i < taps) acc = fmaf(wr[i], win[i], acc);
      }
#pragma unroll
      for (int i = 0; i + 1 < RT; ++i) win[i] = win[i + 1];
      if (act == 1) acc = siluf_(acc);
      if (residual) acc += cur;
      stf(out + (size_t)(sq.row0 + t) * ld_out + c, acc);
    }
  } else {
    for (int t = t_begin; t < t_end; ++t) {
      float acc = b;
      for (int i = 0; i < taps; ++i) acc = fmaf(ldf(w + (size_t)c * taps + i), input(t - (taps - 1 - i)), acc);
      if (act == 1) acc = siluf_(acc);
      if (residual) acc += proj[(size_t)(sq.row0 + t) * ld + col0 + c];
      stf(out + (size_t)(sq.row0 + t) * ld_out + c, acc);
    }
  }
  if (blockIdx.z == 0)
    for (int i = 0; i < taps - 1; ++i) {                       // increasing i: entry i + n_rows is still the old one when it is read
      const int src = sq.n_rows + i - (taps - 1);
      st[(size_t)i * C + c] = src >= 0 ? proj[(size_t)(sq.row0 + src) * ld + col0 + c] : st[(size_t)(i + sq.n_rows) * C + c];
    }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Per-token vectors of the gated delta rule, in the form delta_rule_kernel takes (S <- diag(w) S - au (u^T S) + kk v^T, o = S^T r,
// both products on the old S).  With unit key k, step size beta and decay g of the head:
//   S <- g S;  S += k (beta (v - S^T k))^T      ==      w = g (all rows),  u = k,  au = beta g k,  kk = beta k.
// cv [M, C] holds the filtered q (G * dk), k (G * dk), v (H * dv) channels; value head a reads query/key head a / (H / G).
// proj columns col_b + a / col_a + a are the step-size and decay logits.  One warp per (row, value head).
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_delta_prepare_kernel(const float* __restrict__ cv, int C, const float* __restrict__ proj, int ld, int col_b, int col_a,
                                           const T* __restrict__ a_log, const T* __restrict__ dt_bias, float* __restrict__ w_out,
                                           float* __restrict__ u_out, float* __restrict__ au_out, float* __restrict__ kk_out,
                                           float* __restrict__ r_out, int H, int G, int dk, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const size_t m = idx / H;
  const int a = idx % H, kh = a / (H / G);
  const float* q = cv + m * C + (size_t)kh * dk;
  const float* k = cv + m * C + (size_t)G * dk + (size_t)kh * dk;
  float sq = 0.f, sk = 0.f;
  for (int i = lane; i < dk; i += 32) { sq = fmaf(q[i], q[i], sq); sk = fmaf(k[i], k[i], sk); }
  const float iq = 1.0f / (sqrtf(warp_sum(sq) + 1e-6f) * sqrtf((float)dk)), ik = 1.0f / sqrtf(warp_sum(sk) + 1e-6f);
  const float beta = sigmoidf_(proj[m * ld + col_b + a]);
  const float g = expf(-expf(ldf(a_log + a)) * softplusf_(proj[m * ld + col_a + a] + ldf(dt_bias + a)));
  for (int i = lane; i < dk; i += 32) {
    const size_t o = m * (size_t)(H * dk) + (size_t)a * dk + i;
    const float ku = k[i] * ik;
    w_out[o] = g;
    u_out[o] = ku;
    au_out[o] = beta * g * ku;
    kk_out[o] = beta * ku;
    r_out[o] = q[i] * iq;
  }
}

// dot product of a weight row (T, global) with a row held in shared memory (fp32), 16 bytes per lane per load when `vec`
template <typename T>
__device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* __restrict__ xs, int n, int lane, bool vec) {
  constexpr int VEC = 16 / sizeof(T);
  float acc = 0.f;
  if (vec) {
    for (int k = lane * VEC; k < n; k += 32 * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + k);
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc = fmaf(ldf(reinterpret_cast<const T*>(&raw) + v), xs[k + v], acc);
    }
  } else {
    for (int k = lane; k < n; k += 32) acc = fmaf(ldf(w + k), xs[k], acc);
  }
  return warp_sum(acc);
}

// two rows at once (w0 . x0 and w1 . x1): twice the loads in flight
template <typename T>
__device__ __forceinline__ void row_dot2(const T* __restrict__ w0, const T* __restrict__ w1, const float* __restrict__ x0, const float* __restrict__ x1,
                                         int n, int lane, bool vec, float& r0, float& r1) {
  constexpr int VEC = 16 / sizeof(T);
  float a0 = 0.f, a1 = 0.f;
  if (vec) {
    for (int k = lane * VEC; k < n; k += 64 * VEC) {
      const int k2 = k + 32 * VEC;
      const uint4 z = make_uint4(0, 0, 0, 0);
      const uint4 p0 = *reinterpret_cast<const uint4*>(w0 + k), p1 = *reinterpret_cast<const uint4*>(w1 + k);
      const uint4 q0 = k2 < n ? *reinterpret_cast<const uint4*>(w0 + k2) : z, q1 = k2 < n ? *reinterpret_cast<const uint4*>(w1 + k2) : z;
      const int kk = k2 < n ? k2 : k;                  // past the end the weights read as zero; the index stays inside x
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        a0 = fmaf(ldf(reinterpret_cast<const T*>(&p0) + v), x0[k + v], a0);
        a1 = fmaf(ldf(reinterpret_cast<const T*>(&p1) + v), x1[k + v], a1);
        a0 = fmaf(ldf(reinterpret_cast<const T*>(&q0) + v), x0[kk + v], a0);
        a1 = fmaf(ldf(reinterpret_cast<const T*>(&q1) + v), x1[kk + v], a1);
      }
    }
  } else {
    for (int k = lane; k < n; k += 32) { a0 = fmaf(ldf(w0 + k), x0[k], a0); a1 = fmaf(ldf(w1 + k), x1[k], a1); }
  }
  r0 = warp_sum(a0);
  r1 = warp_sum(a1);
}

// four rows at once
template <typename T>
__device__ __forceinline__ void row_dot4(const T* const (&w)[4], const float* const (&x)[4], int n, int lane, bool vec, float (&r)[4]) {
  constexpr int VEC = 16 / sizeof(T);
  float a[4] = {0.f, 0.f, 0.f, 0.f};
  if (vec) {
    for (int k = lane * VEC; k < n; k += 32 * VEC) {
      uint4 p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = *reinterpret_cast<const uint4*>(w[i] + k);
#pragma unroll
      for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = fmaf(ldf(reinterpret_cast<const T*>(&p[i]) + v), x[i][k + v], a[i]);
    }
  } else {
    for (int k = lane; k < n; k += 32)
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = fmaf(ldf(w[i] + k), x[i][k], a[i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) r[i] = warp_sum(a[i]);
}

// four rows of x against two sets of four weight rows (wa[i] . x[i] and wb[i] . x[i])
template <typename T>
__device__ __forceinline__ void row_dot4x2(const T* const (&wa)[4], const T* const (&wb)[4], const float* const (&x)[4], int n, int lane, bool vec,
                                           float (&ra)[4], float (&rb)[4]) {
  constexpr int VEC = 16 / sizeof(T);
  float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
  if (vec) {
    for (int k = lane * VEC; k < n; k += 64 * VEC) {           // two pieces of every row per pass: sixteen loads in flight per lane
      const int k2 = k + 32 * VEC;
      const bool more = k2 < n;
      const int kk = more ? k2 : k;                            // past the end the weights read as zero; the index stays inside x
      const uint4 z = make_uint4(0, 0, 0, 0);
      uint4 p[4], q[4], p2[4], q2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        p[i] = *reinterpret_cast<const uint4*>(wa[i] + k);
        q[i] = *reinterpret_cast<const uint4*>(wb[i] + k);
        p2[i] = more ? *reinterpret_cast<const uint4*>(wa[i] + k2) : z;
        q2[i] = more ? *reinterpret_cast<const uint4*>(wb[i] + k2) : z;
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float xv = x[i][k + v], xw = x[i][kk + v];
          a[i] = fmaf(ldf(reinterpret_cast<const T*>(&p[i]) + v), xv, a[i]);
          b[i] = fmaf(ldf(reinterpret_cast<const T*>(&q[i]) + v), xv, b[i]);
          a[i] = fmaf(ldf(reinterpret_cast<const T*>(&p2[i]) + v), xw, a[i]);
          b[i] = fmaf(ldf(reinterpret_cast<const T*>(&q2[i]) + v), xw, b[i]);
        }
    }
  } else {
    for (int k = lane; k < n; k += 32)
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = fmaf(ldf(wa[i] + k), x[i][k], a[i]); b[i] = fmaf(ldf(wb[i] + k), x[i][k], b[i]); }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) { ra[i] = warp_sum(a[i]); rb[i] = warp_sum(b[i]); }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Mixture of experts, router: logits z = W_r h (+ bias) in fp32 (h in T).
//   kind 0: scores s = softmax(z) over all E experts; experts form `groups` equal groups of neighbours, a group's score is its best
//           expert's, only experts of the `keep` best groups can be chosen; the `top` best of those are the token's experts,
//           weighted by their s (not renormalised);
//   kind 1: the `top` largest logits are the token's experts, weighted by the softmax over those `top` logits only.
// Ties go to the lower index.  One block per row (its warps share the experts' logits, warp 0 selects); dynamic shared memory:
// D + E floats.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ h, int D, const T* __restrict__ w_router, const T* __restrict__ bias, int kind, int E,
                                  int groups, int keep, int top, int* __restrict__ ids, float* __restrict__ wts, int M) {
  extern __shared__ __align__(16) float rsm[];                 // [D] the row (fp32), then [E] scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int m = blockIdx.x;
  float* hs = rsm;
  float* s = rsm + ((D + 3) & ~3);
  for (int d = threadIdx.x; d < D; d += blockDim.x) hs[d] = ldf(h + (size_t)m * D + d);
  __syncthreads();
  const bool vec = D % (16 / sizeof(T)) == 0 && (reinterpret_cast<uintptr_t>(w_router) & 15) == 0;
  for (int e = warp; e < E; e += nw) {                         // the warps share the experts; logits in fp32
    const float z = row_dot(w_router + (size_t)e * D, hs, D, lane, vec);
    if (lane == 0) s[e] = z + (bias ? ldf(bias + e) : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  if (kind == 1) {
    if (lane == 0) {
      float den = 0.f, first = 0.f;
      for (int k = 0; k < top; ++k) {                          // serial selection; the first chosen logit is the largest
        int bi = 0;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e)
          if (s[e] > bv) { bv = s[e]; bi = e; }
        if (k == 0) first = bv;
        const float w = expf(bv - first);
        ids[(size_t)m * top + k] = bi;
        wts[(size_t)m * top + k] = w;
        den += w;
        s[bi] = -INFINITY;                                     // taken
      }
      for (int k = 0; k < top; ++k) wts[(size_t)m * top + k] /= den;
    }
    return;
  }
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
  mx = warp_max(mx);
  float den = 0.f;
  for (int e = lane; e < E; e += 32) den += expf(s[e] - mx);
  den = warp_sum(den);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = expf(s[e] - mx) / den;
  __syncwarp();
  if (lane == 0) {
    // serial selection (E and top are small next to the products).  Scores are in [0, 1]; an expert of a dropped group is marked
    // by s <- -1 - s, a chosen expert by s <- -3, so `s >= 0` means "can still be chosen".
    const int gs = groups > 1 ? E / groups : E;
    if (groups > 1) {
      for (int r = 0; r < groups - keep; ++r) {                // drop the group with the smallest best score, groups - keep times
        int worst = -1;
        float wv = INFINITY;
        for (int g = groups - 1; g >= 0; --g) {                // ties: the higher index is dropped first
          if (s[(size_t)g * gs] < 0.f) continue;               // already dropped
          float best = -1.f;
          for (int e = 0; e < gs; ++e) best = fmaxf(best, s[(size_t)g * gs + e]);
          if (best < wv) { wv = best; worst = g; }
        }
        if (worst < 0) break;
        for (int e = 0; e < gs; ++e) s[(size_t)worst * gs + e] = -1.f - s[(size_t)worst * gs + e];
      }
    }
    for (int k = 0; k < top; ++k) {
      int bi = 0;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e)
        if (s[e] >= 0.f && s[e] > bv) { bv = s[e]; bi = e; }
      ids[(size_t)m * top + k] = bi;
      wts[(size_t)m * top + k] = bv;
      s[bi] = -3.f;                                            // taken
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Mixture of experts: layout of an expert's gate and up matrices.  w_gu is [E][2 F, D]; with il8 (F a multiple of 8) gate row f
// and up row f sit at rows (f / 8) * 16 + f % 8 and (f / 8) * 16 + 8 + f % 8, so that a 16-column fragment of a product's output
// holds 8 gate values next to their 8 up values and silu(gate) * up is formed in the epilogue; else gate rows come first, then up.
// ---------------------------------------------------------------------------------------------------------------------------
__device__ __host__ __forceinline__ size_t moe_gate_row(int f, int F, int il8) { return il8 ? (size_t)(f / 8) * 16 + f % 8 : (size_t)f; }
__device__ __host__ __forceinline__ size_t moe_up_row(int f, int F, int il8) { return il8 ? (size_t)(f / 8) * 16 + 8 + f % 8 : (size_t)F + f; }

// ---------------------------------------------------------------------------------------------------------------------------
// Mixture of experts, row form (few rows, and the 32-bit mode): every (row, chosen expert) streams that expert's matrices.
//   moe_rows_up_kernel   act[m, k, f] = silu(W_gate[e] h_m)[f] * (W_up[e] h_m)[f],  e = ids[m, k]        one warp per f
//                        ungated experts (w_gu is then [E][F, D], up rows only): act[m, k, f] = relu(W_up[e] h_m)[f]^2
//   moe_rows_down_kernel y[m, d] (+)= sum_k wts[m, k] * (W_down[e_k] act[m, k, :])[d]                    one warp per d
// w_down: [E][D, F].  With `accumulate` the sum is added to what y holds (a shared expert's output made by ordinary products).
// A shared expert of ungated form can also ride along: w_shared [Fs, D] is one more "expert" of moe_rows_up_kernel (grid y = top,
// its activations go to act_shared [M, Fs]), and moe_rows_down_kernel adds W_sdown act_shared with weight one (w_sdown [D, Fs]).
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_rows_up_kernel(const T* __restrict__ h, int D, const T* __restrict__ w_gu, int F, int il8, int gated, const int* __restrict__ ids,
                                   int top, T* __restrict__ act, const T* __restrict__ w_shared, int Fs, T* __restrict__ act_shared) {
  extern __shared__ __align__(16) float hs[];                  // the row, fp32
  const int m = blockIdx.x, k = blockIdx.y;
  for (int d = threadIdx.x; d < D; d += blockDim.x) hs[d] = ldf(h + (size_t)m * D + d);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool vec = D % (16 / sizeof(T)) == 0 && (reinterpret_cast<uintptr_t>(w_gu) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_shared) & 15) == 0;
  if (!gated) {                                                // four up rows per pass: four loads in flight per lane
    const bool sh = k == top;                                  // the shared expert rides along as grid row `top`
    const T* we = sh ? w_shared : w_gu + (size_t)ids[(size_t)m * top + k] * F * D;
    T* out = sh ? act_shared + (size_t)m * Fs : act + ((size_t)m * top + k) * F;
    if (sh) F = Fs;
    const int step = gridDim.z * nw;
    for (int f = blockIdx.z * nw + warp; f < F; f += 4 * step) {
      const T* w4[4];
      const float* x4[4] = {hs, hs, hs, hs};
      float u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) w4[i] = we + (size_t)(f + i * step < F ? f + i * step : f) * D;   // past the end: row f again, not stored
      row_dot4(w4, x4, D, lane, vec, u);
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (f + i * step < F) { const float r = fmaxf(u[i], 0.f); stf(out + f + i * step, r * r); }
      }
    }
    return;
  }
  const T* we = w_gu + (size_t)ids[(size_t)m * top + k] * 2 * F * D;
  for (int f = blockIdx.z * nw + warp; f < F; f += gridDim.z * nw) {
    float g, u;
    row_dot2(we + moe_gate_row(f, F, il8) * D, we + moe_up_row(f, F, il8) * D, hs, hs, D, lane, vec, g, u);
    if (lane == 0) stf(act + ((size_t)m * top + k) * F + f, siluf_(g) * u);
  }
}
template <typename T>
__global__ void moe_rows_down_kernel(const T* __restrict__ act, int F, const T* __restrict__ w_down, int D, const int* __restrict__ ids,
                                     const float* __restrict__ wts, int top, int accumulate, float* __restrict__ y, const T* __restrict__ act_shared,
                                     const T* __restrict__ w_sdown, int Fs) {
  extern __shared__ __align__(16) float as[];                  // [top][F] fp32, then [Fs] of the shared expert (from a 16-byte boundary)
  const int m = blockIdx.x;
  float* as_s = as + (((size_t)top * F + 3) & ~(size_t)3);
  for (int i = threadIdx.x; i < top * F; i += blockDim.x) as[i] = ldf(act + (size_t)m * top * F + i);
  if (w_sdown)
    for (int i = threadIdx.x; i < Fs; i += blockDim.x) as_s[i] = ldf(act_shared + (size_t)m * Fs + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool vec = F % (16 / sizeof(T)) == 0 && (reinterpret_cast<uintptr_t>(w_down) & 15) == 0;
  const bool vec_s = Fs % (16 / sizeof(T)) == 0 && (reinterpret_cast<uintptr_t>(w_sdown) & 15) == 0;
  // two output entries per warp and pass (d and d + dstep), the experts of a row four by four, then two by two, in their order:
  // eight weight rows in flight per lane
  const int dstep = gridDim.y * nw;
  for (int d = blockIdx.y * nw + warp; d < D; d += 2 * dstep) {
    const bool two = d + dstep < D;
    const int d2 = two ? d + dstep : d;                // past the end: entry d again, not stored
    float out = 0.f, out2 = 0.f;
    int k = 0;
    for (; k + 3 < top; k += 4) {
      const T* w4[4];
      const T* v4[4];
      const float* x4[4];
      float r4[4], s4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const size_t ex = (size_t)ids[(size_t)m * top + k + i] * D;
        w4[i] = w_down + (ex + d) * F;
        v4[i] = w_down + (ex + d2) * F;
        x4[i] = as + (k + i) * F;
      }
      row_dot4x2(w4, v4, x4, F, lane, vec, r4, s4);
#pragma unroll
      for (int i = 0; i < 4; ++i) { out = fmaf(wts[(size_t)m * top + k + i], r4[i], out); out2 = fmaf(wts[(size_t)m * top + k + i], s4[i], out2); }
    }
    for (; k + 1 < top; k += 2) {
      const size_t e0 = (size_t)ids[(size_t)m * top + k] * D, e1 = (size_t)ids[(size_t)m * top + k + 1] * D;
      const T* w4[4] = {w_down + (e0 + d) * F, w_down + (e1 + d) * F, w_down + (e0 + d2) * F, w_down + (e1 + d2) * F};
      const float* x4[4] = {as + k * F, as + (k + 1) * F, as + k * F, as + (k + 1) * F};
      float r4[4];
      row_dot4(w4, x4, F, lane, vec, r4);
      out = fmaf(wts[(size_t)m * top + k], r4[0], out);
      out = fmaf(wts[(size_t)m * top + k + 1], r4[1], out);
      out2 = fmaf(wts[(size_t)m * top + k], r4[2], out2);
      out2 = fmaf(wts[(size_t)m * top + k + 1], r4[3], out2);
    }
    if (k < top) {
      const size_t ex = (size_t)ids[(size_t)m * top + k] * D;
      float r0, r1;
      row_dot2(w_down + (ex + d) * F, w_down + (ex + d2) * F, as + k * F, as + k * F, F, lane, vec, r0, r1);
      out = fmaf(wts[(size_t)m * top + k], r0, out);
      out2 = fmaf(wts[(size_t)m * top + k], r1, out2);
    }
    if (w_sdown) {                                             // the shared expert: weight one
      float r0, r1;
      row_dot2(w_sdown + (size_t)d * Fs, w_sdown + (size_t)d2 * Fs, as_s, as_s, Fs, lane, vec_s, r0, r1);
      out += r0;
      out2 += r1;
    }
    if (lane == 0) {
      y[(size_t)m * D + d] = accumulate ? y[(size_t)m * D + d] + out : out;
      if (two) y[(size_t)m * D + d2] = accumulate ? y[(size_t)m * D + d2] + out2 : out2;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Mixture of experts, grouped form (many rows, bf16): the (row, expert) pairs are sorted by expert on the device, every expert's
// run padded to whole 128-row tiles, and two tensor-core products run over the tiles with the expert's matrices chosen per tile.
//   moe_plan_kernel    (one block)  counts -> padded run starts, tile -> expert map (-1 beyond the last run), cursors reset
//   moe_scatter_kernel (one warp per pair) takes the pair's place in its expert's run, remembers it, copies the row there
//   moe_combine_kernel y[m, :] (+)= sum_k wts[m, k] * yg[place[m, k], :]
// ints: counts[E], starts[E + 1], cursor[E], then tile_expert[n_tiles].  The order of pairs inside a run depends on scheduling; a
// pair's result does not (rows of a product are independent).
// ---------------------------------------------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_pairs, int* __restrict__ counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_pairs) atomicAdd(counts + ids[i], 1);
}
__global__ void moe_plan_kernel(int* __restrict__ counts, int E, int tile_rows, int n_tiles, int* __restrict__ starts, int* __restrict__ cursor,
                                int* __restrict__ tile_expert) {
  __shared__ int s_total;
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      starts[e] = at;
      at += (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
      cursor[e] = 0;
    }
    starts[E] = at;
    s_total = at;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
    const int r = t * tile_rows;
    int ex = -1;
    if (r < s_total) {
      int lo = 0, hi = E - 1;                                  // the last expert whose run starts at or before r and is not empty there
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (starts[mid] <= r) lo = mid; else hi = mid - 1;
      }
      ex = lo;
    }
    tile_expert[t] = ex;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;   // ready for the next layer
}
template <typename T>
__global__ void moe_scatter_kernel(const T* __restrict__ h, int D, const int* __restrict__ ids, int n_pairs, int top, const int* __restrict__ starts,
                                   int* __restrict__ cursor, int* __restrict__ place, T* __restrict__ xg) {
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= n_pairs) return;
  int p = 0;
  if (lane == 0) {
    const int e = ids[i];
    p = starts[e] + atomicAdd(cursor + e, 1);
    place[i] = p;
  }
  p = __shfl_sync(0xffffffffu, p, 0);
  const T* src = h + (size_t)(i / top) * D;
  T* dst = xg + (size_t)p * D;
  constexpr int VEC = 16 / sizeof(T);
  if (D % VEC == 0) {
    for (int d = lane * VEC; d < D; d += 32 * VEC) *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(src + d);
  } else {
    for (int d = lane; d < D; d += 32) dst[d] = src[d];
  }
}
__global__ void moe_combine_kernel(const float* __restrict__ yg, const int* __restrict__ place, const float* __restrict__ wts, int top, int D,
                                   int accumulate, float* __restrict__ y) {
  const size_t m = blockIdx.x;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(wts[m * top + k], yg[(size_t)place[m * top + k] * D + d], acc);
    y[m * D + d] = accumulate ? y[m * D + d] + acc : acc;
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Pre-norm block with one-number norm weights and hyper-connections (XOTB200_LM_BLOCK_PRE_SCALAR).
// The stream of row m is kept in S copies X[m][s][:] (S = 1: the plain residual stream).
//
// embed_streams_kernel:  e = embed[token]; e <- e / sqrt(mean(e^2) + eps) * g; every copy starts as e.
//
// hc_open_kernel closes the pending sublayer and opens the next in one pass over the row:
//   close (y != NULL):  X_t <- sum_s mix[s, t] X_s + mult * out[t] * (ya * y + yb * y2)    for all t at once   (mix, out NULL: X += ...)
//   open              :  u = sum_s in[s] X_s  (in NULL: the sum of the copies);
//                        with g: h = u / sqrt(mean(u^2) + eps) * g  -> out_f32 (fp32; a convolution follows) or out_t (a product follows);
//                        without g: u itself -> out_f32 (the model's stream after a layer).
// src_rows != NULL gathers (the final norm of the rows whose logits are wanted): row m reads X row src_rows[m]; the closed copies
// are then not written back (the stream is not needed again).  One block per row; dynamic shared memory: D floats.  S <= 8.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int HC_MAX_STREAMS = 8;

template <typename T>
__global__ void embed_streams_kernel(const T* __restrict__ embed, const int* __restrict__ tokens, const T* __restrict__ g, float eps, float* __restrict__ X,
                                     int S, int D) {
  __shared__ float red[32];
  const int m = blockIdx.x;
  const T* src = embed + (size_t)tokens[m] * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = ldf(src + d); ss = fmaf(v, v, ss); }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps) * (g ? ldf(g) : 1.0f);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = ldf(src + d) * r;
    for (int s = 0; s < S; ++s) X[((size_t)m * S + s) * D + d] = v;
  }
}

template <typename T, int SM, int VEC>   // SM: copies held per entry (>= S); VEC: entries per thread and pass (4: 16-byte loads, D % 4 == 0)
__global__ void hc_open_kernel(float* __restrict__ X, int S, const float* __restrict__ y, const float* __restrict__ y2, float ya, float yb, float mult,
                               const T* __restrict__ mix, const T* __restrict__ outc, const T* __restrict__ inc, const T* __restrict__ g, float eps,
                               const int* __restrict__ src_rows, float* __restrict__ out_f32, T* __restrict__ out_t, int D) {
  extern __shared__ __align__(16) float hc_row[];
  __shared__ float red[32];
  __shared__ float c_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], c_out[HC_MAX_STREAMS], c_in[HC_MAX_STREAMS];
  const int m = blockIdx.x;
  const size_t xm = src_rows ? src_rows[m] : m;
  if (threadIdx.x < S * S) c_mix[threadIdx.x] = mix ? ldf(mix + threadIdx.x) : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = (outc ? ldf(outc + threadIdx.x) : 1.f) * mult;
    c_in[threadIdx.x] = inc ? ldf(inc + threadIdx.x) : 1.f;
  }
  __syncthreads();
  float* xr = X + xm * S * D;
  float ss = 0.f;
  for (int d = threadIdx.x * VEC; d < D; d += blockDim.x * VEC) {
    float xs[SM][VEC];
#pragma unroll
    for (int s = 0; s < SM; ++s) {
      if (s < S) {
        if constexpr (VEC == 4) {
          const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * D + d);
          xs[s][0] = v.x; xs[s][1] = v.y; xs[s][2] = v.z; xs[s][3] = v.w;
        } else {
          xs[s][0] = xr[(size_t)s * D + d];
        }
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) xs[s][v] = 0.f;
      }
    }
    if (y) {
      float yv[VEC];
#pragma unroll
      for (int v = 0; v < VEC; ++v) yv[v] = ya * y[xm * D + d + v] + (y2 ? yb * y2[xm * D + d + v] : 0.f);
      float nx[SM][VEC];
#pragma unroll
      for (int t = 0; t < SM; ++t)
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          float a = 0.f;
          if (t < S) {
#pragma unroll
            for (int s = 0; s < SM; ++s)
              if (s < S) a = fmaf(c_mix[s * S + t], xs[s][v], a);
            a = fmaf(c_out[t], yv[v], a);
          }
          nx[t][v] = a;
        }
#pragma unroll
      for (int t = 0; t < SM; ++t) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) xs[t][v] = nx[t][v];
        if (t < S && !src_rows) {
          if constexpr (VEC == 4) *reinterpret_cast<float4*>(xr + (size_t)t * D + d) = make_float4(nx[t][0], nx[t][1], nx[t][2], nx[t][3]);
          else xr[(size_t)t * D + d] = nx[t][0];
        }
      }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < SM; ++s)
        if (s < S) u = fmaf(c_in[s], xs[s][v], u);
      hc_row[d + v] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!out_f32 && !out_t) return;
  float r = 1.0f;
  if (g) r = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps) * ldf(g);
  for (int d = threadIdx.x * VEC; d < D; d += blockDim.x * VEC) {   // every thread reads back what it wrote
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const float o = hc_row[d + v] * r;
      if (out_f32) out_f32[(size_t)m * D + d + v] = o;
      if (out_t) stf(out_t + (size_t)m * D + d + v, o);
    }
  }
}

}  // namespace xl
