// layered_kernels.cuh — device code of the layered-model engine (libxotb200_lm.so): decoder models given as a LIST of layers,
// each a token mixer (latent attention over a paged latent cache, or a generalised delta-rule recurrence over a per-request
// state) and an optional feed-forward, with grouped RMS norms before and after every sublayer.  The products, the recurrence
// and the small helpers here also serve the mixers and block forms of layered_gqa.cuh and layered_blocks.cuh.
//
// Number formats: every kernel is a template over T, the storage type of weights, GEMM inputs and the latent cache
// (__nv_bfloat16 when serving, float for the all-32-bit mode).  Whatever T is, these are fp32: the residual stream, every norm,
// positions / angles / rotations, attention scores and softmax, gates, decays, unit keys, the recurrent state, GEMM accumulators.
//
// A step works on a PACKED batch: M token rows of several requests back to back (no padding); row_slot[m] / row_pos[m] say which
// request a row belongs to and where it stands in it.  The same kernels serve prompts (many rows per request) and decoding (one
// row per request); the small-M projection kernel (gemv_rows_kernel) is the decode specialisation.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xl {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }
// xIELU:  z > 0: softplus(p) z^2 + z / 2;   z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2.   ap = softplus(p), aq = 1/2 + softplus(q).
__device__ __forceinline__ float xielu_f(float z, float ap, float aq) {
  return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
}

// the exact gelu: z (1 + erf(z / sqrt 2)) / 2
__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); }

// Where a request's token lives in a paged pool: page_table[slot * pages_per_slot + pos / P] * P + pos % P.
struct Paging {
  const int* page_table;
  int pages_per_slot;
  int page_size;
  __device__ __forceinline__ size_t row(int slot, int pos) const {
    return (size_t)page_table[(size_t)slot * pages_per_slot + pos / page_size] * page_size + pos % page_size;
  }
};

// ---------------------------------------------------------------------------------------------------------------------------
// embedding:  x[m, :] = embed[token[m], :]   (fp32 residual)
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ embed, const int* __restrict__ tokens, float* __restrict__ x, int D) {
  const int m = blockIdx.x;
  const T* src = embed + (size_t)tokens[m] * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) x[(size_t)m * D + d] = ldf(src + d);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Fused "close one sublayer, open the next":   x += groupnorm(y) * w_post ;  h = groupnorm(x) * w_pre
// groupnorm: the row is cut into G equal consecutive parts, each divided by sqrt(mean(part^2) + eps).  A part is shared by a few warps of the row's block.  y / w_post may be NULL (first sublayer), h / w_pre may be NULL (no
// sublayer follows).  src_rows (may be NULL) gathers: output row m reads x row src_rows[m] and does not write x (used for the
// final norm on the rows whose logits are wanted).
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void residual_groupnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const T* __restrict__ w_post,
                                          const T* __restrict__ w_pre, T* __restrict__ h, const int* __restrict__ src_rows, int D, int G,
                                          float eps) {
  // `wpg` warps share one part (each a slice of it); their sums of squares meet in shared memory.  All warps walk the same
  // number of rounds, so the barriers are uniform.
  __shared__ float red[2][32];
  const int m = blockIdx.x;
  const int xm = src_rows ? src_rows[m] : m;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int Dg = D / G;
  const int wpg = max(1, nw / G), gpr = nw / wpg;    // warps per part, parts per round
  const int sub = warp % wpg, gsel = warp / wpg;
  const int sl = (Dg + wpg - 1) / wpg, d0 = sub * sl, d1 = min(Dg, d0 + sl);
  for (int g0 = 0; g0 < G; g0 += gpr) {
    const int g = g0 + gsel;
    const bool on = gsel < gpr && g < G;
    float* xr = x + (size_t)xm * D + (size_t)(on ? g : 0) * Dg;
    const float* yr = y ? y + (size_t)m * D + (size_t)(on ? g : 0) * Dg : nullptr;
    float ry = 0.f;
    if (y) {
      float s = 0.f;
      if (on)
        for (int d = d0 + lane; d < d1; d += 32) { const float v = yr[d]; s = fmaf(v, v, s); }
      s = warp_sum(s);
      if (lane == 0) red[0][warp] = s;
      __syncthreads();
      float t = 0.f;
      for (int k = 0; k < wpg; ++k) t += red[0][(warp / wpg) * wpg + k];
      ry = 1.0f / sqrtf(t / (float)Dg + eps);
    }
    float s2 = 0.f;
    if (on)
      for (int d = d0 + lane; d < d1; d += 32) {
        float v = xr[d];
        if (y) {
          v += yr[d] * ry * ldf(w_post + (size_t)g * Dg + d);
          xr[d] = v;
        }
        s2 = fmaf(v, v, s2);
      }
    if (h) {
      s2 = warp_sum(s2);
      if (lane == 0) red[1][warp] = s2;
      __syncthreads();
      float t = 0.f;
      for (int k = 0; k < wpg; ++k) t += red[1][(warp / wpg) * wpg + k];
      const float rx = 1.0f / sqrtf(t / (float)Dg + eps);
      if (on)
        for (int d = d0 + lane; d < d1; d += 32) stf(h + (size_t)m * D + (size_t)g * Dg + d, xr[d] * rx * ldf(w_pre + (size_t)g * Dg + d));
    }
    __syncthreads();                                 // `red` is reused by the next round
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Plain RMS norm of n columns of an fp32 matrix (a projection's output) into a T matrix:  out[m, :] = in[m, col0:col0+n] / rms * w
// One warp per row.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_cols_kernel(const float* __restrict__ in, int ld_in, int col0, int n, const T* __restrict__ w, T* __restrict__ out,
                                    int ld_out, int M, float eps) {
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (m >= M) return;
  const float* r = in + (size_t)m * ld_in + col0;
  float s = 0.f;
  for (int d = lane; d < n; d += 32) s = fmaf(r[d], r[d], s);
  const float rs = 1.0f / sqrtf(warp_sum(s) / (float)n + eps);
  for (int d = lane; d < n; d += 32) stf(out + (size_t)m * ld_out + d, r[d] * rs * ldf(w + d));
}

// Rotation of one pair by the angle pos * freq (fp32 throughout).  layout 0: pairs (2i, 2i+1); 1: pairs (i, i + dims/2).
__device__ __forceinline__ void rot_pair_index(int i, int dims, int layout, int& a, int& b) {
  if (layout == 0) { a = 2 * i; b = 2 * i + 1; }
  else { a = i; b = i + dims / 2; }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Latent cache append.  proj[m, col0 : col0 + R + dr] is the down-projection of row m: the first R columns are RMS-normed (weight
// w_norm) into the latent, the last dr are the shared key part, of which the first rot_dims entries are rotated by the row's
// position.  Both go to the row's place in the paged pool: pool[(page * P + offset) * (R + dr) + ...].  One warp per row.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_append_kernel(const float* __restrict__ proj, int ld, int col0, int R, int dr, const T* __restrict__ w_norm, float eps,
                                     const float* __restrict__ freqs, int rot_dims, int layout, const int* __restrict__ row_slot,
                                     const int* __restrict__ row_pos, Paging pg, T* __restrict__ pool, int M) {
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (m >= M) return;
  const float* r = proj + (size_t)m * ld + col0;
  T* dst = pool + pg.row(row_slot[m], row_pos[m]) * (size_t)(R + dr);
  float s = 0.f;
  for (int d = lane; d < R; d += 32) s = fmaf(r[d], r[d], s);
  const float rs = 1.0f / sqrtf(warp_sum(s) / (float)R + eps);
  for (int d = lane; d < R; d += 32) stf(dst + d, r[d] * rs * ldf(w_norm + d));
  const float p = (float)row_pos[m];
  const float* kr = r + R;
  for (int i = lane; i < rot_dims / 2; i += 32) {
    int a, b;
    rot_pair_index(i, rot_dims, layout, a, b);
    const float ang = p * freqs[i], c = cosf(ang), sn = sinf(ang);
    const float u = kr[a], v = kr[b];
    stf(dst + R + a, u * c - v * sn);
    stf(dst + R + b, v * c + u * sn);
  }
  for (int d = rot_dims + lane; d < dr; d += 32) stf(dst + R + d, kr[d]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Query split.  qraw[m, h * (dn + dr) + ...] (fp32 projection output, leading dimension ld, first column col0) is cut per head
// into the unrotated part -> qn[m, h, dn] (T: the operand of the key-absorption product) and the rotated part, turned by the
// row's position -> qfull[m, h, R : R + dr] (fp32; columns [0, R) are filled by the absorption product).  One warp per (row, head).
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void query_split_kernel(const float* __restrict__ qraw, int ld, int col0, int H, int dn, int dr, int R, const float* __restrict__ freqs,
                                   int rot_dims, int layout, const int* __restrict__ row_pos, T* __restrict__ qn, float* __restrict__ qfull,
                                   int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const int m = idx / H, h = idx % H;
  const float* q = qraw + (size_t)m * ld + col0 + (size_t)h * (dn + dr);
  for (int d = lane; d < dn; d += 32) stf(qn + ((size_t)m * H + h) * dn + d, q[d]);
  float* out = qfull + ((size_t)m * H + h) * (R + dr) + R;
  const float p = (float)row_pos[m];
  const float* qr = q + dn;
  for (int i = lane; i < rot_dims / 2; i += 32) {
    int a, b;
    rot_pair_index(i, rot_dims, layout, a, b);
    const float ang = p * freqs[i], c = cosf(ang), sn = sinf(ang);
    const float u = qr[a], v = qr[b];
    out[a] = u * c - v * sn;
    out[b] = v * c + u * sn;
  }
  for (int d = rot_dims + lane; d < dr; d += 32) out[d] = qr[d];
}

// ---------------------------------------------------------------------------------------------------------------------------
// Latent attention over the paged pool, in the ABSORBED form: with q~ = W_uk[h]^T q_unrotated (R numbers per head, computed by a
// batched product before this kernel) the score of query (m, h) against cached token j is (q~ . c_j + q_rot . kr_j) * scale, and
// the head's output is W_uv[h] (sum_j p_j c_j) — so every head reads the SAME cached rows [c_j | kr_j] and nothing per head is
// ever expanded or stored.  Key range of a query at position i: max(0, i - window + 1) .. i (window == 0: 0 .. i).
//
// One CTA serves one work item = up to `q_per_item` consecutive rows of one request, all H heads; one WARP owns one (row, head)
// pair: lane j scores key j of a 32-key tile held in shared memory (fp32, row stride padded odd), the softmax statistics are
// exchanged by shuffles, and the lanes then split the R latent columns of the running sum sum_j p_j c_j between them
// (NACC = ceil(R / 32) registers).  Output: olat[m, h, R] (T), times sigmoid(gate[m, h]) when the mixer has an output gate.
// ---------------------------------------------------------------------------------------------------------------------------
struct Item {
  int row0;     // first packed row
  int n_rows;   // rows of this item (consecutive positions of one request)
  int slot;     // request
  int pos0;     // position of row0
};

// Key splits: with gridDim.z > 1 the keys of an item are cut into gridDim.z runs of `chunk` keys (a multiple of 32); CTA z handles
// run z and parks its unnormalised result {running max, sum, accumulator[R]} in `part` ([M * H][gridDim.z][2 + R] fp32), and
// latent_attention_combine_kernel merges the runs.  That is what keeps a single decoded row over a long context from running on
// one SM.  With gridDim.z == 1 the kernel normalises, gates and stores itself.
template <typename T, int NACC>
__global__ void latent_attention_kernel(const float* __restrict__ qfull, const T* __restrict__ pool, Paging pg, const Item* __restrict__ items,
                                        int H, int R, int dr, float scale, int window, const float* __restrict__ gate, int gate_ld,
                                        int gate_col0, T* __restrict__ olat, int chunk, float* __restrict__ part) {
  extern __shared__ float smem[];
  const Item it = items[blockIdx.x];
  const int W = R + dr, WS = W | 1;                 // odd row stride: lane j reading row j is conflict-free
  float* ktile = smem;                              // [32][WS]
  float* qs = smem + 32 * WS;                       // [warps][W]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int pair = blockIdx.y * nw + warp;         // (row, head) pair of this warp
  const bool active = pair < it.n_rows * H;
  const int qi = active ? pair / H : 0, h = active ? pair % H : 0;
  const int m = it.row0 + qi, pos = it.pos0 + qi;
  float* q = qs + (size_t)warp * W;
  if (active) {
    const float* src = qfull + ((size_t)m * H + h) * W;
    for (int d = lane; d < W; d += 32) q[d] = src[d];
  }
  int last = it.pos0 + it.n_rows - 1;
  int first = window > 0 ? max(0, it.pos0 - window + 1) : 0;
  if (gridDim.z > 1) {
    first += blockIdx.z * chunk;
    last = min(last, first + chunk - 1);
  }
  float acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  float mx = -INFINITY, den = 0.f;
  for (int j0 = first; j0 <= last; j0 += 32) {
    __syncthreads();
    // stage 32 cached rows (fp32), one warp per row — rows past `last` are zero-filled
    for (int jr = warp; jr < 32; jr += nw) {
      const int j = j0 + jr;
      float* dst = ktile + jr * WS;
      if (j <= last) {
        const T* src = pool + pg.row(it.slot, j) * (size_t)W;
        for (int d = lane; d < W; d += 32) dst[d] = ldf(src + d);
      } else {
        for (int d = lane; d < W; d += 32) dst[d] = 0.f;
      }
    }
    __syncthreads();
    if (!active) continue;
    const int j = j0 + lane;
    const bool vis = j <= pos && j <= last && (window == 0 || pos - j < window);
    float s = 0.f;
    const float* kr = ktile + lane * WS;
    for (int d = 0; d < W; ++d) s = fmaf(q[d], kr[d], s);
    s = vis ? s * scale : -INFINITY;
    const float tmax = warp_max(s);
    if (tmax == -INFINITY) continue;                // no visible key in this tile (warp-uniform)
    const float nmx = fmaxf(mx, tmax);
    const float corr = expf(mx - nmx);              // mx == -inf: exp(-inf) = 0
    const float p = vis ? expf(s - nmx) : 0.f;
    den = den * corr + warp_sum(p);
    mx = nmx;
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] *= corr;
    for (int jr = 0; jr < 32; ++jr) {
      const float pj = __shfl_sync(0xffffffffu, p, jr);
      if (pj == 0.f) continue;                      // warp-uniform
      const float* c = ktile + jr * WS;
#pragma unroll
      for (int a = 0; a < NACC; ++a) {
        const int d = a * 32 + lane;
        if (d < R) acc[a] = fmaf(pj, c[d], acc[a]);
      }
    }
  }
  if (!active) return;
  if (gridDim.z > 1) {
    float* dst = part + (((size_t)m * H + h) * gridDim.z + blockIdx.z) * (size_t)(2 + R);
    if (lane == 0) { dst[0] = mx; dst[1] = den; }
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int d = a * 32 + lane;
      if (d < R) dst[2 + d] = acc[a];
    }
    return;
  }
  float g = 1.0f / den;
  if (gate) g *= sigmoidf_(gate[(size_t)m * gate_ld + gate_col0 + h]);
  T* out = olat + ((size_t)m * H + h) * R;
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    const int d = a * 32 + lane;
    if (d < R) stf(out + d, acc[a] * g);
  }
}

// merges the key runs of latent_attention_kernel: one warp per (row, head) pair of the listed items (grid.y covers the pairs);
// lane z first turns run z's {max, sum} into its weight exp(max_z - max) (at most 32 runs), then the lanes split the R columns
template <typename T>
__global__ void latent_attention_combine_kernel(const float* __restrict__ part, const Item* __restrict__ items, int H, int R, int splits,
                                                const float* __restrict__ gate, int gate_ld, int gate_col0, T* __restrict__ olat) {
  const Item it = items[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int pair = blockIdx.y * nw + warp;
  if (pair >= it.n_rows * H) return;
  const int m = it.row0 + pair / H, h = pair % H;
  const float* src = part + ((size_t)m * H + h) * splits * (size_t)(2 + R);
  const float mz = lane < splits ? src[(size_t)lane * (2 + R)] : -INFINITY;
  const float mx = warp_max(mz);
  const float wz = mz == -INFINITY ? 0.f : expf(mz - mx);
  const float den = warp_sum(lane < splits ? src[(size_t)lane * (2 + R) + 1] * wz : 0.f);
  float g = 1.0f / den;
  if (gate) g *= sigmoidf_(gate[(size_t)m * gate_ld + gate_col0 + h]);
  for (int d0 = 0; d0 < R; d0 += 32) {
    const int d = d0 + lane;
    float a = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float w = __shfl_sync(0xffffffffu, wz, z);
      if (w != 0.f && d < R) a = fmaf(src[(size_t)z * (2 + R) + 2 + d], w, a);
    }
    if (d < R) stf(olat + ((size_t)m * H + h) * R + d, a * g);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Generalised delta rule.  Per head, with key size dk and value size dv, the state S [dk, dv] (fp32, one per request and layer)
// moves per token as   S <- diag(w) S - (a * u)(u^T S) + k v^T   (both products read the old S),   o = S^T r,
// where u = k / sqrt(|k|^2 + 1e-6), w = exp(-exp(-1/2) * sigmoid(decay logit + bias)) and a = sigmoid(removal logit + bias).
// The COLUMNS of S (value index) never mix, so a column lives in the registers of `P` cooperating lanes (KPT key rows each,
// row i = e * P + part) and the only exchange per token is a P-lane shuffle reduction of u^T S and of S^T r.
// One CTA = one (request, head, group of value columns); tokens of the step are staged CH at a time in shared memory, where
// w, a * u, u are computed once per token for all columns.
//   proj: fp32 [M, ld] projection output with the r / k / v / a blocks (H * d columns each) at the given column offsets;
//   wlog: fp32 [M, H * dk] decay logits (low-rank branch output), to which w_bias is added;   o_raw: fp32 [M, H * dv].
// ---------------------------------------------------------------------------------------------------------------------------
// The per-token vectors are made for all rows at once by delta_prepare_kernel (one warp per (row, head)): in place w <- decay
// (wlog), and u, a * u into two fp32 buffers.  delta_rule_kernel then only carries the recurrence: the six vectors of 16 tokens
// at a time (fewer for wide heads) come into shared memory with cp.async, double-buffered, while the previous 16 tokens are being applied.
template <typename T>
__global__ void delta_prepare_kernel(const float* __restrict__ proj, int ld, int col_k, int col_a, float* __restrict__ wlog, const T* __restrict__ w_bias,
                                     const T* __restrict__ a_bias, float* __restrict__ u_out, float* __restrict__ au_out, int H, int dk, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const size_t m = idx / H;
  const int h = idx % H;
  const float* pr = proj + m * ld;
  float ss = 0.f;
  for (int i = lane; i < dk; i += 32) { const float kv = pr[col_k + h * dk + i]; ss = fmaf(kv, kv, ss); }
  const float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
  for (int i = lane; i < dk; i += 32) {
    const size_t o = m * (size_t)(H * dk) + h * dk + i;
    const float u = pr[col_k + h * dk + i] * inv;
    u_out[o] = u;
    au_out[o] = sigmoidf_(pr[col_a + h * dk + i] + ldf(a_bias + h * dk + i)) * u;
    wlog[o] = expf(-0.60653065971263342f * sigmoidf_(wlog[o] + ldf(w_bias + h * dk + i)));
  }
}

__device__ __forceinline__ void cp_async4(float* dst_smem, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}

// A thread owns NC value columns x KPT key rows of the state (row i = e * P + part), so the token's vectors, read from shared
// memory once, serve NC columns and the NC recurrences run as independent chains.  vec4: every source row is 16-byte aligned
// (sizes and offsets multiples of 4 floats), so the staging uses 16-byte cp.async.
// uvec == NULL: the rule has no removal term (S <- diag(w) S + k v^T): u and a * u are neither staged nor applied.
// The write key k, the read-out vector r and the value v each come from their own fp32 matrix (pointer, leading dimension, first
// column; head a's vector at column a * dk, resp. a * dv): a projection output or a prepared buffer.
struct DeltaSrc {
  const float* p;
  int ld, col;
};
template <int KPT, int P, int NC>
__global__ void delta_rule_kernel(DeltaSrc ksrc, DeltaSrc rsrc, DeltaSrc vsrc, const float* __restrict__ wdec,
                                  const float* __restrict__ uvec, const float* __restrict__ auvec, const Item* __restrict__ seqs, int H, int dk,
                                  int dv, float* __restrict__ state, size_t state_slot_stride, float* __restrict__ o_raw, int vec4) {
  constexpr int DKP = KPT * P;                       // padded size: >= dk and >= dv
  constexpr int CH = DKP <= 64 ? 16 : DKP <= 128 ? 8 : 4;   // tokens per buffer: two buffers fill the 48 KB of static shared memory
  __shared__ __align__(16) float buf[2][CH][6][DKP]; // per token: w, a*u, u, k, r, v
  const Item sq = seqs[blockIdx.x / H];
  const int h = blockIdx.x % H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int CPW = (32 / P) * NC;                 // columns per warp
  const int col0 = (blockIdx.y * (blockDim.x >> 5) + warp) * CPW + (lane / P) * NC, part = lane % P;   // grid.y splits the value columns
  float* S = state + (size_t)sq.slot * state_slot_stride + (size_t)h * dk * dv;
  float s[KPT][NC];
#pragma unroll
  for (int e = 0; e < KPT; ++e)
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int i = e * P + part;
      s[e][c] = (col0 + c < dv && i < dk) ? S[(size_t)i * dv + col0 + c] : 0.f;
    }
  for (int e = threadIdx.x; e < 2 * CH * 6 * DKP; e += blockDim.x) (&buf[0][0][0][0])[e] = 0.f;   // the padding stays zero
  __syncthreads();
  const int HD = H * dk;
  // A thread copies the same pieces (vector, offset) of every token of a chunk: which pieces is worked out per piece, not per copy
  // (the divisions stay out of the token loop), and the token loop only adds the source's row stride.
  const int perk = vec4 ? dk / 4 : dk, perv = vec4 ? dv / 4 : dv;   // copies per key-sized vector / per value vector
  const int per_tok = 5 * perk + perv;
  auto issue = [&](int c) {
    const int t0 = c * CH, nt = min(CH, sq.n_rows - t0);
    const size_t m0 = (size_t)sq.row0 + t0;
    for (int piece = threadIdx.x; piece < per_tok; piece += blockDim.x) {
      const int vec = piece / perk < 5 ? piece / perk : 5, i = (piece - vec * perk) * (vec4 ? 4 : 1);
      const float* src;
      size_t stride;
      if (!uvec && (vec == 1 || vec == 2)) continue;          // no removal term: these two stay zero
      if (vec == 0) { src = wdec + m0 * HD + h * dk + i; stride = HD; }
      else if (vec == 1) { src = auvec + m0 * HD + h * dk + i; stride = HD; }
      else if (vec == 2) { src = uvec + m0 * HD + h * dk + i; stride = HD; }
      else if (vec == 3) { src = ksrc.p + m0 * ksrc.ld + ksrc.col + h * dk + i; stride = ksrc.ld; }
      else if (vec == 4) { src = rsrc.p + m0 * rsrc.ld + rsrc.col + h * dk + i; stride = rsrc.ld; }
      else { src = vsrc.p + m0 * vsrc.ld + vsrc.col + h * dv + i; stride = vsrc.ld; }
      float* dst = &buf[c & 1][0][vec][i];
      if (vec4) {
        for (int t = 0; t < nt; ++t) cp_async16(dst + (size_t)t * 6 * DKP, src + t * stride);
      } else {
        for (int t = 0; t < nt; ++t) cp_async4(dst + (size_t)t * 6 * DKP, src + t * stride);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int nch = (sq.n_rows + CH - 1) / CH;
  issue(0);
  for (int c = 0; c < nch; ++c) {
    if (c + 1 < nch) {
      issue(c + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int nt = min(CH, sq.n_rows - c * CH);
    float(*b)[6][DKP] = buf[c & 1];
    for (int t = 0; t < nt; ++t) {
      float dot[NC], out[NC], vj[NC];
#pragma unroll
      for (int x = 0; x < NC; ++x) { dot[x] = 0.f; out[x] = 0.f; vj[x] = col0 + x < DKP ? b[t][5][col0 + x] : 0.f; }
      if (uvec) {                                          // block-uniform
#pragma unroll
        for (int e = 0; e < KPT; ++e) {
          const float u = b[t][2][e * P + part];
#pragma unroll
          for (int x = 0; x < NC; ++x) dot[x] = fmaf(u, s[e][x], dot[x]);
        }
#pragma unroll
        for (int o = P / 2; o > 0; o >>= 1)
#pragma unroll
          for (int x = 0; x < NC; ++x) dot[x] += __shfl_xor_sync(0xffffffffu, dot[x], o);
      }
#pragma unroll
      for (int e = 0; e < KPT; ++e) {
        const int i = e * P + part;
        const float w = b[t][0][i], au = b[t][1][i], kk = b[t][3][i], rr = b[t][4][i];
#pragma unroll
        for (int x = 0; x < NC; ++x) {
          s[e][x] = fmaf(w, s[e][x], fmaf(-au, dot[x], kk * vj[x]));
          out[x] = fmaf(s[e][x], rr, out[x]);
        }
      }
#pragma unroll
      for (int o = P / 2; o > 0; o >>= 1)
#pragma unroll
        for (int x = 0; x < NC; ++x) out[x] += __shfl_xor_sync(0xffffffffu, out[x], o);
      if (part == 0) {
        float* dst = o_raw + ((size_t)sq.row0 + c * CH + t) * (size_t)(H * dv) + h * dv + col0;
#pragma unroll
        for (int x = 0; x < NC; ++x)
          if (col0 + x < dv) dst[x] = out[x];
      }
    }
    __syncthreads();                                 // the buffer is refilled two chunks later
  }
#pragma unroll
  for (int e = 0; e < KPT; ++e)
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int i = e * P + part;
      if (col0 + c < dv && i < dk) S[(size_t)i * dv + col0 + c] = s[e][c];
    }
}

// Output side of the recurrent mixers: per (row, head) o / rms(o) * w_norm * sigmoid(gate) -> T, the operand of the output product.
// w_head_stride: dv when every head has its own norm weight, 0 when the heads share one of size dv.  gate_silu: 0 = sigmoid(gate),
// 1 = silu(gate).  nq != NULL (with den_floor, both [M, H]): the head's read-out is first divided by max(|nq|, den_floor) + 1e-6
// (a normaliser n . q that must not fall below a floor).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o_raw, const float* __restrict__ nq, const float* __restrict__ den_floor,
                                      const T* __restrict__ w_norm, int w_head_stride, const float* __restrict__ gate, int gate_ld, int gate_col0, int gate_silu,
                                      T* __restrict__ out, int H, int dv, float eps, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const int m = idx / H, h = idx % H;
  const float* o = o_raw + (size_t)m * H * dv + (size_t)h * dv;
  const float pre = nq ? 1.0f / (fmaxf(fabsf(nq[idx]), den_floor[idx]) + 1e-6f) : 1.0f;
  float s = 0.f;
  for (int d = lane; d < dv; d += 32) { const float v = o[d] * pre; s = fmaf(v, v, s); }
  const float rs = pre / sqrtf(warp_sum(s) / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) {
    const float z = gate[(size_t)m * gate_ld + gate_col0 + h * dv + d];
    stf(out + (size_t)m * H * dv + (size_t)h * dv + d, o[d] * rs * ldf(w_norm + h * w_head_stride + d) * (gate_silu ? z * sigmoidf_(z) : sigmoidf_(z)));
  }
}

// out[m, :n] = tanh(in[m, col0 : col0 + n])  (fp32 in, T out): the low-rank decay branch between its two products
template <typename T>
__global__ void tanh_cols_kernel(const float* __restrict__ in, int ld, int col0, int n, T* __restrict__ out, int M) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)M * n) return;
  const size_t m = i / n, d = i % n;
  stf(out + i, tanhf(in[m * ld + col0 + d]));
}

// ---------------------------------------------------------------------------------------------------------------------------
// Products.  C[z][m, n] = sum_k A[z][m, k] * B[z][n, k]   with fp32 accumulation; A row-major (lda), B addressed by two strides
// (sbn, sbk) so that a weight stored [K, N] is used without a transposed copy, z = batch (per-head products) via element offsets.
// EPI 1: C = relu(C)^2.  EPI 2: C = xIELU(C) with the two raw parameters p, q at `epi` (in the weights' type).  EPI 4: C = gelu(C), exact.
// gemm_tiled_kernel: 64 x 64 x 16 shared-memory tiles, 256 threads, 4 x 4 outputs per thread, fp32 FMA (exact fp32 in the 32-bit mode).
// ---------------------------------------------------------------------------------------------------------------------------
template <typename TA, typename TB, typename TC, int EPI>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const TA* __restrict__ A, long lda, long a_batch, const TB* __restrict__ B, long sbn, long sbk, long b_batch, TC* __restrict__ C,
                  long ldc, long c_batch, int M, int N, int K, const TB* __restrict__ epi) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4], Bs[BK][BN + 4];
  A += (size_t)blockIdx.z * a_batch;
  B += (size_t)blockIdx.z * b_batch;
  C += (size_t)blockIdx.z * c_batch;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int r = e / BK, k = e % BK;
      As[k][r] = (m0 + r < M && k0 + k < K) ? ldf(A + (size_t)(m0 + r) * lda + k0 + k) : 0.f;
    }
    if (sbk == 1) {
      for (int e = threadIdx.x; e < BN * BK; e += 256) {
        const int r = e / BK, k = e % BK;
        Bs[k][r] = (n0 + r < N && k0 + k < K) ? ldf(B + (size_t)(n0 + r) * sbn + k0 + k) : 0.f;
      }
    } else {
      for (int e = threadIdx.x; e < BN * BK; e += 256) {
        const int k = e / BN, r = e % BN;
        Bs[k][r] = (n0 + r < N && k0 + k < K) ? ldf(B + (size_t)(n0 + r) * sbn + (size_t)(k0 + k) * sbk) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float ap = 0.f, aq = 0.f;
  if (EPI == 2) { ap = softplusf_(ldf(epi)); aq = 0.5f + softplusf_(ldf(epi + 1)); }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) {
        float v = acc[i][j];
        if (EPI == 1) { v = fmaxf(v, 0.f); v *= v; }
        if (EPI == 2) v = xielu_f(v, ap, aq);
        if (EPI == 4) v = gelu_erf_f(v);
        stf(C + (size_t)m * ldc + n, v);
      }
    }
}

// gemv_rows_kernel: the decode form (M <= MR activation rows, B contiguous along k).  The weights are read ONCE, 16 bytes per
// lane per load, and multiplied into all M activation rows (held in shared memory as fp32).  To keep enough loads in flight for
// HBM, a warp works on RB = 4 weight rows at a time (four independent loads per step) and `wsplit` warps share a row group by
// cutting K into slices (a [N small, K large] matrix still fills the GPU); the slices meet in shared memory.
template <typename TA, typename TB, typename TC, int EPI, int MR>
__global__ void __launch_bounds__(256)
gemv_rows_kernel(const TA* __restrict__ A, long lda, long a_batch, const TB* __restrict__ B, long sbn, long b_batch, TC* __restrict__ C, long ldc,
                 long c_batch, int M, int N, int K, int wsplit, const TB* __restrict__ epi) {
  constexpr int RB = 4;
  extern __shared__ float a_s[];                     // [M][K], then the slice sums [8 warps][RB][MR]
  A += (size_t)blockIdx.z * a_batch;
  B += (size_t)blockIdx.z * b_batch;
  C += (size_t)blockIdx.z * c_batch;
  for (int m = 0; m < M; ++m)
    for (int k = threadIdx.x; k < K; k += blockDim.x) a_s[m * K + k] = ldf(A + (size_t)m * lda + k);
  float* red = a_s + (size_t)M * K;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gpb = 8 / wsplit, grp = warp / wsplit, slice = warp % wsplit;
  constexpr int VEC = 16 / sizeof(TB);
  const bool vec_ok = (K % VEC == 0) && (sbn % VEC == 0) && ((reinterpret_cast<uintptr_t>(B) & 15) == 0);
  const int step = vec_ok ? 32 * VEC : 32;
  const int ksl = ((K + wsplit - 1) / wsplit + step - 1) / step * step;
  const int kbeg = slice * ksl, kend = min(K, kbeg + ksl);
  for (int nb = blockIdx.x * gpb * RB; nb < N; nb += gridDim.x * gpb * RB) {   // uniform trip count for the whole block
    const int n0 = nb + grp * RB;
    float acc[RB][MR];
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;
    if (vec_ok) {
      // two steps of the slice at a time: 2 x RB independent 16-byte loads per lane are in flight before the first FMA
      for (int k = kbeg + lane * VEC; k < kend; k += 64 * VEC) {
        uint4 raw[2][RB];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int r = 0; r < RB; ++r)
            raw[u][r] = (n0 + r < N && k + u * 32 * VEC < kend) ? *reinterpret_cast<const uint4*>(B + (size_t)(n0 + r) * sbn + k + u * 32 * VEC)
                                                                : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int ku = min(k + u * 32 * VEC, K - VEC);     // past the slice the weights read as zero; the index stays inside a_s
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            float av[MR];
#pragma unroll
            for (int m = 0; m < MR; ++m) av[m] = m < M ? a_s[m * K + ku + v] : 0.f;
#pragma unroll
            for (int r = 0; r < RB; ++r) {
              const float w = ldf(reinterpret_cast<const TB*>(&raw[u][r]) + v);
#pragma unroll
              for (int m = 0; m < MR; ++m) acc[r][m] = fmaf(av[m], w, acc[r][m]);
            }
          }
        }
      }
    } else {
      for (int k = kbeg + lane; k < kend; k += 32) {
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          const float w = n0 + r < N ? ldf(B + (size_t)(n0 + r) * sbn + k) : 0.f;
#pragma unroll
          for (int m = 0; m < MR; ++m)
            if (m < M) acc[r][m] = fmaf(a_s[m * K + k], w, acc[r][m]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float v = warp_sum(acc[r][m]);
        if (lane == 0) red[(warp * RB + r) * MR + m] = v;
      }
    __syncthreads();
    if (slice == 0 && lane < RB * MR) {
      const int r = lane / MR, m = lane % MR;
      float v = 0.f;
      for (int sidx = 0; sidx < wsplit; ++sidx) v += red[((warp + sidx) * RB + r) * MR + m];   // fixed order: deterministic
      if (m < M && n0 + r < N) {
        if (EPI == 1) { v = fmaxf(v, 0.f); v *= v; }
        if (EPI == 2) v = xielu_f(v, softplusf_(ldf(epi)), 0.5f + softplusf_(ldf(epi + 1)));
        if (EPI == 4) v = gelu_erf_f(v);
        stf(C + (size_t)m * ldc + n0 + r, v);
      }
    }
    __syncthreads();
  }
}

// finishes the logits of every row in place — l <- l * scale, then l <- cap * tanh(l / cap) when cap > 0 — and takes the
// lowest-index argmax of the row (greedy sampling on the device)
__global__ void argmax_rows_kernel(float* __restrict__ logits, int V, float scale, float cap, int* __restrict__ out) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  float* r = logits + (size_t)blockIdx.x * V;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = r[i];
    if (scale != 1.0f || cap > 0.f) {
      v *= scale;
      if (cap > 0.f) v = cap * tanhf(v / cap);
      r[i] = v;
    }
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
    out[blockIdx.x] = idx;
  }
}

// weights arrive as bf16 bit patterns: widen (or copy) rows into their place in the T-typed blob
template <typename T>
__global__ void store_rows_kernel(const bf16* __restrict__ src, T* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    stf(dst + i, __bfloat162float(src[i]));
}
// rows of src [rows, cols] go to dst rows (r / 8) * 16 + half * 8 + r % 8: two matrices interleaved in groups of 8 rows
template <typename T>
__global__ void store_rows_interleaved8_kernel(const bf16* __restrict__ src, T* __restrict__ dst, int rows, int cols, int half) {
  const size_t n = (size_t)rows * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols, c = i % cols;
    stf(dst + ((r / 8) * 16 + (size_t)half * 8 + r % 8) * cols + c, __bfloat162float(src[i]));
  }
}
// synthetic weights: element i = mean + dev * (uniform in [-sqrt 3, sqrt 3)) from a counter hash — for benchmarks and smoke runs
template <typename T>
__global__ void fill_random_kernel(T* __restrict__ dst, size_t n, uint64_t seed, float mean, float dev) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint64_t z = (i + 1) * 0x9E3779B97F4A7C15ull + seed;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u = (float)(z >> 40) * (1.0f / 16777216.0f);          // [0, 1)
    stf(dst + i, mean + dev * 3.4641016f * (u - 0.5f));
  }
}

// src [heads * d, cols] (row-major, bf16 bits) -> dst [heads][cols][d]: each head's block transposed
template <typename T>
__global__ void store_heads_transposed_kernel(const bf16* __restrict__ src, T* __restrict__ dst, int heads, int d, int cols) {
  const size_t n = (size_t)heads * d * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t h = i / ((size_t)d * cols), r = i % ((size_t)d * cols);
    const size_t c = r / d, k = r % d;
    stf(dst + i, __bfloat162float(src[(h * d + k) * cols + c]));
  }
}
// the inverse: src [heads][cols][d] -> dst [heads * d, cols]
template <typename T>
__global__ void untranspose_heads_kernel(const T* __restrict__ src, T* __restrict__ dst, int heads, int d, int cols) {
  const size_t n = (size_t)heads * d * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t h = i / ((size_t)d * cols), r = i % ((size_t)d * cols);
    const size_t c = r / d, k = r % d;
    dst[(h * d + k) * cols + c] = src[i];
  }
}
__global__ void copy_rows_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, int ld_src, int ld_dst, int n, int M) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)M * n) return;
  dst[(i / n) * ld_dst + i % n] = src[(i / n) * ld_src + i % n];
}


// ===========================================================================================================================
// Prompt attention on the tensor cores (bf16 serving path; requests that bring FLASH_MIN_ROWS rows or more).
//
// For many query rows the EXPANDED form is cheaper than the absorbed one: the visible cached rows of the request are gathered
// from the paged pool into a contiguous buffer (latent_gather_kernel), expanded once per step by two tensor-core products into
// per-head unrotated keys kn = c W_uk^T and values v = c W_uv^T, and latent_flash_kernel then runs a streaming-softmax attention
// per (64-row tile, head) with mma.sync.m16n8k16 (bf16 operands, fp32 accumulators): scores = [q_unrot | q_rot] . [kn | kr],
// fp32 scale / mask / running max and sum, and the weights enter the value product as a bf16 PAIR (high part + remainder, two
// MMAs) so that they keep 16 mantissa bits instead of 8.  Key range as in the absorbed kernel: j <= i and (window == 0 or
// i - j < window).  Output: o[m, h * dv + :] (bf16), times sigmoid(gate[m, h]) when the mixer is gated.
// ===========================================================================================================================
constexpr int FLASH_MIN_ROWS = 16;

struct GatherReq {
  int slot;      // request
  int kfirst;    // first cached position that any row of the step can see
  int nkeys;     // positions kfirst .. kfirst + nkeys - 1 (up to the request's last row of this step)
  int kbase;     // index of position kfirst in the gathered buffers
};

struct FlashTile {
  int row0;      // first packed row
  int n_rows;    // <= 64 consecutive rows of one request
  int pos0;      // position of row0
  int kbase;     // as in GatherReq
  int kfirst;
};

template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pool, Paging pg, const GatherReq* __restrict__ reqs, int W, T* __restrict__ cbuf) {
  const GatherReq rq = reqs[blockIdx.y];
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= rq.nkeys) return;
  const T* src = pool + pg.row(rq.slot, rq.kfirst + i) * (size_t)W;
  T* dst = cbuf + (size_t)(rq.kbase + i) * W;
  for (int d = lane; d < W; d += 32) dst[d] = src[d];
}

// Query in 16 bits for the expanded form: q16[m, h, 0:dn] = unrotated part, q16[m, h, dn:dn+dr] = rotated part turned by the position
__global__ void query_rotate16_kernel(const float* __restrict__ qraw, int ld, int H, int dn, int dr, const float* __restrict__ freqs, int rot_dims,
                                      int layout, const int* __restrict__ row_pos, bf16* __restrict__ q16, int M) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * H) return;
  const int m = idx / H, h = idx % H;
  const float* q = qraw + (size_t)m * ld + (size_t)h * (dn + dr);
  bf16* out = q16 + ((size_t)m * H + h) * (dn + dr);
  for (int d = lane; d < dn; d += 32) out[d] = __float2bfloat16_rn(q[d]);
  const float p = (float)row_pos[m];
  const float* qr = q + dn;
  for (int i = lane; i < rot_dims / 2; i += 32) {
    int a, b;
    rot_pair_index(i, rot_dims, layout, a, b);
    const float ang = p * freqs[i], c = cosf(ang), sn = sinf(ang);
    const float u = qr[a], v = qr[b];
    out[dn + a] = __float2bfloat16_rn(u * c - v * sn);
    out[dn + b] = __float2bfloat16_rn(v * c + u * sn);
  }
  for (int d = rot_dims + lane; d < dr; d += 32) out[dn + d] = __float2bfloat16_rn(qr[d]);
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
// 8 consecutive bf16 from p (n_valid of them exist, the rest read as zero) -> dst (16-byte aligned shared memory)
__device__ __forceinline__ void stage8(bf16* dst, const bf16* p, int n_valid, bool vec) {
  if (n_valid >= 8 && vec) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[e] = e < n_valid ? p[e] : __float2bfloat16_rn(0.f);
  }
}

template <int DVT>   // value columns held per warp row: DVT tiles of 8 (dv <= 8 * DVT)
__global__ void __launch_bounds__(128)
latent_flash_kernel(const bf16* __restrict__ q16, const bf16* __restrict__ kn, const bf16* __restrict__ cbuf, const bf16* __restrict__ vx,
                    const FlashTile* __restrict__ tiles, int H, int dn, int dr, int dv, int R, float scale, int window, const float* __restrict__ gate,
                    int gate_ld, int gate_col0, bf16* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t fsm[];
  const FlashTile tl = tiles[blockIdx.x];
  const int h = blockIdx.y;
  const int DQ = dn + dr, DQP = (DQ + 15) & ~15, QS = DQP + 8;       // padded row length and row stride (elements) of the Q / K tiles
  constexpr int VS = 64 + 8;                                         // row stride of the transposed V tile [value column][key]
  bf16* Qs = reinterpret_cast<bf16*>(fsm);
  bf16* Ks = Qs + 64 * QS;
  bf16* Vt = Ks + 64 * QS;                                           // [8 * DVT][VS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const bool vq = (DQ % 8 == 0), vk = (dn % 8 == 0) && ((H * dn) % 8 == 0), vr = (dr % 8 == 0) && (R % 8 == 0) && dn % 8 == 0,
             vv = (dv % 8 == 0);

  // ---- Q tile (rows beyond n_rows and the padding read as zero)
  for (int e = threadIdx.x; e < 64 * (DQP / 8); e += 128) {
    const int r = e / (DQP / 8), c = (e % (DQP / 8)) * 8;
    const int nv = r < tl.n_rows ? max(0, min(8, DQ - c)) : 0;
    stage8(Qs + r * QS + c, q16 + ((size_t)(tl.row0 + r) * H + h) * DQ + c, nv, vq);
  }
  float o[DVT][4];
#pragma unroll
  for (int i = 0; i < DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mx[2] = {-INFINITY, -INFINITY}, den[2] = {0.f, 0.f};
  const int pos_lo = tl.pos0 + warp * 16 + g, pos_hi = pos_lo + 8;   // positions of this thread's two rows
  const int last = tl.pos0 + tl.n_rows - 1;
  const int first = window > 0 ? max(0, tl.pos0 - window + 1) : 0;

  for (int j0 = first; j0 <= last; j0 += 64) {
    __syncthreads();
    // ---- K tile: [kn(h) | kr] per key, V tile transposed
    for (int e = threadIdx.x; e < 64 * (DQP / 8); e += 128) {
      const int r = e / (DQP / 8), c = (e % (DQP / 8)) * 8, j = j0 + r;
      bf16* dst = Ks + r * QS + c;
      const size_t idx = (size_t)(tl.kbase + (j - tl.kfirst));
      if (j > last || c >= DQ) stage8(dst, kn, 0, false);
      else if (c + 8 <= dn) stage8(dst, kn + idx * ((size_t)H * dn) + (size_t)h * dn + c, 8, vk);
      else if (c >= dn) stage8(dst, cbuf + idx * (size_t)(R + dr) + R + (c - dn), min(8, DQ - c), vr);
      else {   // a chunk that straddles the two sources (dn not a multiple of 8)
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const int d = c + x;
          dst[x] = d < dn ? kn[idx * ((size_t)H * dn) + (size_t)h * dn + d] : d < DQ ? cbuf[idx * (size_t)(R + dr) + R + (d - dn)] : __float2bfloat16_rn(0.f);
        }
      }
    }
    for (int e = threadIdx.x; e < 64 * DVT; e += 128) {
      const int r = e / DVT, c = (e % DVT) * 8, j = j0 + r;
      __align__(16) bf16 tmp[8];
      const int nv = j <= last ? max(0, min(8, dv - c)) : 0;
      stage8(tmp, vx + (size_t)(tl.kbase + (j - tl.kfirst)) * ((size_t)H * dv) + (size_t)h * dv + c, nv, vv);
#pragma unroll
      for (int x = 0; x < 8; ++x) Vt[(c + x) * VS + r] = tmp[x];
    }
    __syncthreads();
    // ---- scores of this warp's 16 rows against the 64 keys
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    const bf16* qa = Qs + (warp * 16 + g) * QS + 2 * t;
    for (int k0 = 0; k0 < DQP; k0 += 16) {
      const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa + k0), a1 = *reinterpret_cast<const uint32_t*>(qa + 8 * QS + k0);
      const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qa + k0 + 8), a3 = *reinterpret_cast<const uint32_t*>(qa + 8 * QS + k0 + 8);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const bf16* kb = Ks + (n * 8 + g) * QS + k0 + 2 * t;
        mma_bf16_16816(s[n], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
      }
    }
    // ---- scale, mask, running max
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int j = j0 + n * 8 + 2 * t + (x & 1), pos = (x < 2) ? pos_lo : pos_hi;
        const bool vis = j <= pos && j <= last && (window == 0 || pos - j < window);
        s[n][x] = vis ? s[n][x] * scale : -INFINITY;
        tmax[x >> 1] = fmaxf(tmax[x >> 1], s[n][x]);
      }
    float corr[2], nmx[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      nmx[r] = fmaxf(mx[r], tmax[r]);
      corr[r] = (mx[r] == -INFINITY) ? 0.f : expf(mx[r] - nmx[r]);
      mx[r] = nmx[r];
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float p = (s[n][x] == -INFINITY) ? 0.f : expf(s[n][x] - nmx[x >> 1]);
        s[n][x] = p;
        psum[x >> 1] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      den[r] = den[r] * corr[r] + psum[r];
    }
#pragma unroll
    for (int i = 0; i < DVT; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
    // ---- o += P V with P as (high, remainder) bf16 pairs
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float p0 = s[2 * kk + (x >> 1)][(x & 1) * 2], p1 = s[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
        const float h0 = __bfloat162float(__float2bfloat16_rn(p0)), h1 = __bfloat162float(__float2bfloat16_rn(p1));
        ah[x] = pack_bf16x2(h0, h1);
        al[x] = pack_bf16x2(p0 - h0, p1 - h1);
      }
#pragma unroll
      for (int i = 0; i < DVT; ++i) {
        const bf16* vb = Vt + (i * 8 + g) * VS + kk * 16 + 2 * t;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(vb), b1 = *reinterpret_cast<const uint32_t*>(vb + 8);
        mma_bf16_16816(o[i], ah[0], ah[1], ah[2], ah[3], b0, b1);
        mma_bf16_16816(o[i], al[0], al[1], al[2], al[3], b0, b1);
      }
    }
  }
  // ---- normalise, gate, store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qi = warp * 16 + g + r * 8;
    if (qi >= tl.n_rows) continue;
    const int m = tl.row0 + qi;
    float sc = 1.0f / den[r];
    if (gate) sc *= sigmoidf_(gate[(size_t)m * gate_ld + gate_col0 + h]);
    bf16* dst = out + (size_t)m * ((size_t)H * dv) + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < DVT; ++i)
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int c = i * 8 + 2 * t + x;
        if (c < dv) dst[c] = __float2bfloat16_rn(o[i][r * 2 + x] * sc);
      }
  }
}

// The same attention for sizes whose rows are whole 16-byte chunks (dn, dr, R, dv multiples of 8): K and V tiles arrive by 16-byte
// cp.async into two buffers each (the next tile is in flight while this one is multiplied), V stays in its natural [key][column]
// layout and is transposed on the way into registers by ldmatrix.trans; Q and K fragments come from ldmatrix too.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const bf16* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void cp_async16_b(bf16* dst_smem, const bf16* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}

template <int DVT>
__global__ void __launch_bounds__(128)
latent_flash_aligned_kernel(const bf16* __restrict__ q16, const bf16* __restrict__ kn, const bf16* __restrict__ cbuf, const bf16* __restrict__ vx,
                            const FlashTile* __restrict__ tiles, int H, int dn, int dr, int dv, int R, float scale, int window,
                            const float* __restrict__ gate, int gate_ld, int gate_col0, bf16* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t fsm[];
  const FlashTile tl = tiles[blockIdx.x];
  const int h = blockIdx.y;
  const int DQ = dn + dr, DQP = (DQ + 15) & ~15, QS = DQP + 8;
  constexpr int VS = 8 * DVT + 8;
  bf16* Qs = reinterpret_cast<bf16*>(fsm);          // [64][QS]
  bf16* Ks = Qs + 64 * QS;                          // [2][64][QS]
  bf16* Vs = Ks + 2 * 64 * QS;                      // [2][64][VS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  const int last = tl.pos0 + tl.n_rows - 1;
  const int first = window > 0 ? max(0, tl.pos0 - window + 1) : 0;
  const int qc = DQP / 8;

  auto issue = [&](int j0, int bsel) {
    bf16* kd = Ks + bsel * 64 * QS;
    for (int e = threadIdx.x; e < 64 * qc; e += 128) {
      const int r = e / qc, c = (e % qc) * 8, j = j0 + r;
      bf16* dst = kd + r * QS + c;
      const size_t idx = (size_t)(tl.kbase + (j - tl.kfirst));
      if (j > last || c >= DQ) *reinterpret_cast<uint4*>(dst) = zero4;
      else if (c < dn) cp_async16_b(dst, kn + idx * ((size_t)H * dn) + (size_t)h * dn + c);
      else cp_async16_b(dst, cbuf + idx * (size_t)(R + dr) + R + (c - dn));
    }
    bf16* vd = Vs + bsel * 64 * VS;
    for (int e = threadIdx.x; e < 64 * DVT; e += 128) {
      const int r = e / DVT, c = (e % DVT) * 8, j = j0 + r;
      bf16* dst = vd + r * VS + c;
      if (j > last || c >= dv) *reinterpret_cast<uint4*>(dst) = zero4;
      else cp_async16_b(dst, vx + (size_t)(tl.kbase + (j - tl.kfirst)) * ((size_t)H * dv) + (size_t)h * dv + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // Q tile (plain 16-byte copies; rows beyond n_rows and the padding are zero)
  for (int e = threadIdx.x; e < 64 * qc; e += 128) {
    const int r = e / qc, c = (e % qc) * 8;
    uint4 v = zero4;
    if (r < tl.n_rows && c < DQ) v = *reinterpret_cast<const uint4*>(q16 + ((size_t)(tl.row0 + r) * H + h) * DQ + c);
    *reinterpret_cast<uint4*>(Qs + r * QS + c) = v;
  }
  float o[DVT][4];
#pragma unroll
  for (int i = 0; i < DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mx[2] = {-INFINITY, -INFINITY}, den[2] = {0.f, 0.f};
  const int pos_lo = tl.pos0 + warp * 16 + g, pos_hi = pos_lo + 8;
  const int ntile = (last - first) / 64 + 1;
  issue(first, 0);
  for (int it = 0; it < ntile; ++it) {
    const int j0 = first + it * 64, bsel = it & 1;
    if (it + 1 < ntile) {
      issue(j0 + 64, bsel ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* kt = Ks + bsel * 64 * QS;
    const bf16* vt = Vs + bsel * 64 * VS;
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    for (int k0 = 0; k0 < DQP; k0 += 16) {
      uint32_t a[4];
      ldsm_x4(a, Qs + (warp * 16 + (lane & 15)) * QS + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n < 8; n += 2) {
        uint32_t b[4];
        ldsm_x4(b, kt + (n * 8 + (lane & 7) + ((lane >> 4) << 3)) * QS + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(s[n], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_bf16_16816(s[n + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
      }
    }
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int j = j0 + n * 8 + 2 * t + (x & 1), pos = (x < 2) ? pos_lo : pos_hi;
        const bool vis = j <= pos && j <= last && (window == 0 || pos - j < window);
        s[n][x] = vis ? s[n][x] * scale : -INFINITY;
        tmax[x >> 1] = fmaxf(tmax[x >> 1], s[n][x]);
      }
    float corr[2], nmx[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      nmx[r] = fmaxf(mx[r], tmax[r]);
      corr[r] = (mx[r] == -INFINITY) ? 0.f : expf(mx[r] - nmx[r]);
      mx[r] = nmx[r];
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float p = (s[n][x] == -INFINITY) ? 0.f : expf(s[n][x] - nmx[x >> 1]);
        s[n][x] = p;
        psum[x >> 1] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      den[r] = den[r] * corr[r] + psum[r];
    }
#pragma unroll
    for (int i = 0; i < DVT; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float p0 = s[2 * kk + (x >> 1)][(x & 1) * 2], p1 = s[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
        const float h0 = __bfloat162float(__float2bfloat16_rn(p0)), h1 = __bfloat162float(__float2bfloat16_rn(p1));
        ah[x] = pack_bf16x2(h0, h1);
        al[x] = pack_bf16x2(p0 - h0, p1 - h1);
      }
#pragma unroll
      for (int i = 0; i < DVT; i += 2) {
        uint32_t b[4];
        ldsm_x4_trans(b, vt + (kk * 16 + (lane & 15)) * VS + i * 8 + (lane >> 4) * 8);
        mma_bf16_16816(o[i], ah[0], ah[1], ah[2], ah[3], b[0], b[1]);
        mma_bf16_16816(o[i], al[0], al[1], al[2], al[3], b[0], b[1]);
        mma_bf16_16816(o[i + 1], ah[0], ah[1], ah[2], ah[3], b[2], b[3]);
        mma_bf16_16816(o[i + 1], al[0], al[1], al[2], al[3], b[2], b[3]);
      }
    }
    __syncthreads();                                 // this buffer is refilled by the next iteration's issue
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qi = warp * 16 + g + r * 8;
    if (qi >= tl.n_rows) continue;
    const int m = tl.row0 + qi;
    float sc = 1.0f / den[r];
    if (gate) sc *= sigmoidf_(gate[(size_t)m * gate_ld + gate_col0 + h]);
    bf16* dst = out + (size_t)m * ((size_t)H * dv) + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < DVT; ++i) {
      const int c = i * 8 + 2 * t;
      if (c < dv) *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16x2(o[i][r * 2] * sc, o[i][r * 2 + 1] * sc);
    }
  }
}

}  // namespace xl
