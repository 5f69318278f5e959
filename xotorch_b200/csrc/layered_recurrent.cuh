// layered_recurrent.cuh — the per-token vectors of two more linear recurrences, in the form delta_rule_kernel (layered_kernels.cuh)
// takes:  S <- diag(w) S + kk v^T,  o = S^T r  (no removal term: its u / au vectors are absent).
//
//   matrix LSTM (XOTB200_LM_MIX_MATRIX_LSTM).  Per head: log input gate i = cap tanh((W_i h + b_i) / cap), log forget gate
//     f = logsigmoid(cap tanh((W_f h + b_f) / cap)), running maximum m_t = max(f_t + m_(t-1), i_t) with m = 0 before the first token;
//     S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T,  n_t the same with k alone,  o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6).
//     mlstm_gates_kernel walks the tokens of a request once per head (the maximum is a sequential scan; the transcendental functions
//     of 32 tokens are taken in parallel before each stretch of it) and leaves decay, input weight and e^(-m) per (row, head);
//     mlstm_expand_kernel writes the vectors; mlstm_normaliser_kernel carries n (a vector per head, kept apart from S so that the
//     matrix keeps its power-of-two shape) and leaves n . q per (row, head).
//   state-space layer (XOTB200_LM_MIX_MAMBA2).  Per head: dt = softplus(dt_raw + dt_bias), S <- e^(-e^A_log dt) S + dt B x^T,
//     y = S^T C (+ D x, added by mamba2_out_kernel):  w = e^(-e^A_log dt), kk = dt B, r = C, v = x.
//     mamba2_out_kernel: (y + D x) * silu(z), RMS norm in equal consecutive parts, times the norm weight -> the output product's operand.
//
// Everything here is fp32 whatever the storage type T of the weights is.
#pragma once
#include "layered_kernels.cuh"

namespace xl {

__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// One warp per (request of the step, head).  proj[m, col_i + a], proj[m, col_f + a]: the gate logits before bias and cap.
// m_state[slot * stride + a]: the running maximum, carried between steps.  Outputs per (row, head): decay, inw, floor = e^(-m).
template <typename T>
__global__ void mlstm_gates_kernel(const float* __restrict__ proj, int ld, int col_i, int col_f, const T* __restrict__ b_i, const T* __restrict__ b_f,
                                   float cap, const Item* __restrict__ seqs, int n_seq, int H, float* __restrict__ m_state, size_t state_slot_stride,
                                   float* __restrict__ decay, float* __restrict__ inw, float* __restrict__ floor_out) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_seq * H) return;
  const Item sq = seqs[idx / H];
  const int a = idx % H;
  float* mp = m_state + (size_t)sq.slot * state_slot_stride + a;
  float mrun = *mp;
  const float bi = ldf(b_i + a), bf = ldf(b_f + a);
  for (int t0 = 0; t0 < sq.n_rows; t0 += 32) {
    const int t = t0 + lane;
    float ig = 0.f, fg = 0.f;
    if (t < sq.n_rows) {
      const float* pr = proj + (size_t)(sq.row0 + t) * ld;
      ig = cap * tanhf((pr[col_i + a] + bi) / cap);
      fg = logsigmoidf_(cap * tanhf((pr[col_f + a] + bf) / cap));
    }
    float m_prev = 0.f, m_new = 0.f;
    const int n = min(32, sq.n_rows - t0);
    for (int l = 0; l < n; ++l) {                              // the scan itself: every lane follows it, lane l keeps its token's pair
      const float fl = __shfl_sync(0xffffffffu, fg, l), il = __shfl_sync(0xffffffffu, ig, l);
      const float nm = fmaxf(fl + mrun, il);
      if (l == lane) { m_prev = mrun; m_new = nm; }
      mrun = nm;
    }
    if (t < sq.n_rows) {
      const size_t o = (size_t)(sq.row0 + t) * H + a;
      decay[o] = expf(fg + m_prev - m_new);
      inw[o] = expf(ig - m_new);
      floor_out[o] = expf(-m_new);
    }
  }
  if (lane == 0) *mp = mrun;
}

// One warp per (row, head): w = decay (all dk rows), kk = inw * k, r = q / sqrt(dk).
__global__ void mlstm_expand_kernel(const float* __restrict__ proj, int ld, int col_q, int col_k, const float* __restrict__ decay,
                                    const float* __restrict__ inw, float* __restrict__ w_out, float* __restrict__ kk_out, float* __restrict__ r_out,
                                    int H, int dk, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const size_t m = idx / H;
  const int a = idx % H;
  const float* pr = proj + m * ld;
  const float dc = decay[idx], iw = inw[idx], qs = 1.0f / sqrtf((float)dk);
  for (int i = lane; i < dk; i += 32) {
    const size_t o = m * (size_t)(H * dk) + (size_t)a * dk + i;
    w_out[o] = dc;
    kk_out[o] = iw * pr[col_k + a * dk + i];
    r_out[o] = pr[col_q + a * dk + i] * qs;
  }
}

// The normaliser: n_t = decay_t n_(t-1) + inw_t k_t, nq[row, head] = n_t . r_t.  One block per (request of the step, head); a lane
// keeps dk / 32 entries of n (dk <= 256).  kk = inw * k and r = q / sqrt(dk) are the expanded vectors [M, H * dk].
// Every entry of n is a linear recurrence of its own, so the step's tokens are cut into one stretch per warp: each warp first runs its
// stretch from zero (leaving the stretch's product of decays and its local n in shared memory), then takes its true start —
// the state pushed through the stretches before it, in order — and runs the stretch again, now writing n . r.  The last warp leaves
// the new state.  (One row per request, decoding: one warp, one pass.)
__global__ void mlstm_normaliser_kernel(const float* __restrict__ kk, const float* __restrict__ r, const float* __restrict__ decay, const Item* __restrict__ seqs,
                                        int H, int dk, float* __restrict__ n_state, size_t state_slot_stride, float* __restrict__ nq) {
  constexpr int E = 8, TB = 4;
  __shared__ float seg_n[32][E * 32];
  __shared__ float seg_p[32];
  const Item sq = seqs[blockIdx.x / H];
  const int a = blockIdx.x % H, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int per = (sq.n_rows + nw - 1) / nw, t_begin = min(sq.n_rows, warp * per), t_end = min(sq.n_rows, t_begin + per);
  float* np = n_state + (size_t)sq.slot * state_slot_stride + (size_t)a * dk;
  float n[E];
  // one pass over the warp's stretch from the n given; write_out: leave n . r per token
  auto pass = [&](bool write_out, float& prod) {
    for (int t0 = t_begin; t0 < t_end; t0 += TB) {
      float kv[TB][E], rv[TB][E], dc[TB];
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        const bool on = t0 + t < t_end;
        const size_t row = (size_t)sq.row0 + (on ? t0 + t : t_begin);
        dc[t] = on ? decay[row * H + a] : 1.0f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const bool in = on && e * 32 + lane < dk;
          kv[t][e] = in ? kk[row * (size_t)(H * dk) + (size_t)a * dk + e * 32 + lane] : 0.f;
          rv[t][e] = in && write_out ? r[row * (size_t)(H * dk) + (size_t)a * dk + e * 32 + lane] : 0.f;
        }
      }
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        float d = 0.f;
        prod *= dc[t];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          n[e] = fmaf(dc[t], n[e], kv[t][e]);
          d = fmaf(n[e], rv[t][e], d);
        }
        if (write_out) {
          d = warp_sum(d);
          if (lane == 0 && t0 + t < t_end) nq[((size_t)sq.row0 + t0 + t) * H + a] = d;
        }
      }
    }
  };
  float prod = 1.0f;
  if (nw > 1) {
#pragma unroll
    for (int e = 0; e < E; ++e) n[e] = 0.f;
    pass(false, prod);
#pragma unroll
    for (int e = 0; e < E; ++e) seg_n[warp][e * 32 + lane] = n[e];
    if (lane == 0) seg_p[warp] = prod;
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < E; ++e) n[e] = e * 32 + lane < dk ? np[e * 32 + lane] : 0.f;
  for (int u = 0; u < warp; ++u)                            // the state pushed through the stretches before this one, in order
#pragma unroll
    for (int e = 0; e < E; ++e) n[e] = fmaf(seg_p[u], n[e], seg_n[u][e * 32 + lane]);
  if (nw > 1) __syncthreads();                               // every warp has read the old state before the last one replaces it
  pass(true, prod);
  if (warp == nw - 1)
#pragma unroll
    for (int e = 0; e < E; ++e)
      if (e * 32 + lane < dk) np[e * 32 + lane] = n[e];
}

// One warp per (row, head).  cv [M, C]: the filtered channels [x (H * dv) | B (G * N) | C (G * N)]; proj[m, col_dt + a]: raw step size.
template <typename T>
__global__ void mamba2_prepare_kernel(const float* __restrict__ cv, int C, const float* __restrict__ proj, int ld, int col_dt, const T* __restrict__ a_log,
                                      const T* __restrict__ dt_bias, float* __restrict__ w_out, float* __restrict__ kk_out, float* __restrict__ r_out,
                                      int H, int G, int N, int dv, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const size_t m = idx / H;
  const int a = idx % H, g = a / (H / G);
  const float dt = softplusf_(proj[m * ld + col_dt + a] + ldf(dt_bias + a));
  const float dec = expf(-expf(ldf(a_log + a)) * dt);
  const float* B = cv + m * C + (size_t)H * dv + (size_t)g * N;
  const float* Cm = B + (size_t)G * N;
  for (int i = lane; i < N; i += 32) {
    const size_t o = m * (size_t)(H * N) + (size_t)a * N + i;
    w_out[o] = dec;
    kk_out[o] = dt * B[i];
    r_out[o] = Cm[i];
  }
}

// One block per (row, norm part): part p covers entries [p * n, (p + 1) * n) of the row's H * dv outputs.
//   t = (o + D[head] x) * silu(z);  out = t / sqrt(mean_part(t^2) + eps) * w
// The gated entries wait in dynamic shared memory (n floats) between the two passes.
template <typename T>
__global__ void mamba2_out_kernel(const float* __restrict__ o_raw, const float* __restrict__ cv, int C, const float* __restrict__ proj, int ld, int col_z,
                                  const T* __restrict__ Dskip, const T* __restrict__ w_norm, int H, int dv, int parts, float eps, T* __restrict__ out) {
  extern __shared__ float gated[];
  __shared__ float red[32];
  const size_t m = blockIdx.x / parts;
  const int p = blockIdx.x % parts, inner = H * dv, n = inner / parts, c0 = p * n;
  const float* o = o_raw + m * inner + c0;
  const float* x = cv + m * C + c0;
  const float* z = proj + m * ld + col_z + c0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float t = (o[c] + ldf(Dskip + (c0 + c) / dv) * x[c]) * siluf_(z[c]);
    gated[c] = t;
    ss = fmaf(t, t, ss);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  const float rs = 1.0f / sqrtf(warp_sum(lane < nw ? red[lane] : 0.f) / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf(out + m * inner + c0 + c, gated[c] * rs * ldf(w_norm + c0 + c));
}

}  // namespace xl
