// layered_recurrent.cuh — the per-token vectors of two more linear recurrences, in the form delta_rule_kernel (layered_kernels.cuh)
// takes:  S <- diag(w) S + kk v^T,  o = S^T r  (no removal term: its u / au vectors are absent).
//
//   matrix LSTM (XOTB200_LM_MIX_MATRIX_LSTM).  Per head: log input gate i = cap tanh((W_i h + b_i) / cap), log forget gate
//     f = logsigmoid(cap tanh((W_f h + b_f) / cap)), running maximum m_t = max(f_t + m_(t-1), i_t) with m = 0 before the first token;
//     S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T,  n_t the same with k alone,  o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6).
//     The normaliser n rides along as ONE MORE VALUE COLUMN whose value is 1 for every token: the state is [dk, dv + 1] per head, the
//     read-out's last entry is n . q.  mlstm_gates_kernel walks the tokens of a request once per head (the maximum is a sequential
//     scan; the transcendental functions of 32 tokens are taken in parallel before each stretch of it) and leaves decay, input
//     weight and e^(-m) per (row, head); mlstm_expand_kernel writes the vectors.
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

// One warp per (row, head): w = decay (all dk rows), kk = inw * k, r = q / sqrt(dk), v_aug = [v | 1].
__global__ void mlstm_expand_kernel(const float* __restrict__ proj, int ld, int col_q, int col_k, int col_v, const float* __restrict__ decay,
                                    const float* __restrict__ inw, float* __restrict__ w_out, float* __restrict__ kk_out, float* __restrict__ r_out,
                                    float* __restrict__ v_out, int H, int dk, int dv, int M) {
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
  float* vo = v_out + m * (size_t)(H * (dv + 1)) + (size_t)a * (dv + 1);
  for (int d = lane; d <= dv; d += 32) vo[d] = d < dv ? pr[col_v + a * dv + d] : 1.0f;
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

// One warp per (row, norm part): part p covers entries [p * n, (p + 1) * n) of the row's H * dv outputs.
//   t = (o + D[head] x) * silu(z);  out = t / sqrt(mean_part(t^2) + eps) * w
template <typename T>
__global__ void mamba2_out_kernel(const float* __restrict__ o_raw, const float* __restrict__ cv, int C, const float* __restrict__ proj, int ld, int col_z,
                                  const T* __restrict__ Dskip, const T* __restrict__ w_norm, int H, int dv, int parts, float eps, T* __restrict__ out, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * parts) return;
  const size_t m = idx / parts;
  const int p = idx % parts, inner = H * dv, n = inner / parts, c0 = p * n;
  const float* o = o_raw + m * inner;
  const float* x = cv + m * C;
  const float* z = proj + m * ld + col_z;
  float ss = 0.f;
  for (int c = c0 + lane; c < c0 + n; c += 32) {
    const float t = (o[c] + ldf(Dskip + c / dv) * x[c]) * siluf_(z[c]);
    ss = fmaf(t, t, ss);
  }
  const float rs = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
  for (int c = c0 + lane; c < c0 + n; c += 32) {
    const float t = (o[c] + ldf(Dskip + c / dv) * x[c]) * siluf_(z[c]);
    stf(out + m * inner + c, t * rs * ldf(w_norm + c));
  }
}

}  // namespace xl
