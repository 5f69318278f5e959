// layered_gqa.cuh — grouped-query attention over a paged key/value cache (mixer XOTB200_LM_MIX_ATTENTION of the layered engine).
//
// H query heads of size dk share G key/value heads (query head a reads key/value head a / (H / G)); values have size dv.  The cache
// of a layer is one paged pool whose row for a token is [keys of all G heads, after their norm | values of all G heads] in T; a layer
// may read another layer's pool (shared keys/values) with its own queries and mask.
//
//   score(i, j) = q_i . k_j * scale                       fp32
//                 -> cap * tanh(score / cap)              when cap > 0
//                 -> - r1[a] * ln(1 + r2[a] * (i - j))    when the head has a distance penalty
//                 -> + rel[a][min(i - j, rel_n - 1)]      when the layer has a learned bias per distance bucket (tabulated per
//                                                         distance; from rel_n - 1 on every distance is in the last bucket)
//   visible     : j <= i,  i - j < window (window > 0),  floor(i / chunk) == floor(j / chunk) (chunk > 0; blocks are counted from
//                 position 0 of the request, whatever portion of it a step brings);
//                 keep_first > 0: the first keep_first tokens stay visible beyond the window;
//                 pool > 0: every block of `pool` tokens that ends at or before i - window is seen as ONE key / value, the means of
//                 its cached keys / values (made by gqa_pool_blocks_kernel when the block's last token is appended; they live in
//                 the second half of the layer's pool, block b of a request at the place token b has in the first half)
//   weights     = softmax over the visible keys (fp32); with a sink the denominator also holds exp(sink[a]), a term that has no
//                 key, no value, no scale and no bias and counts once; output = sum_j p_j v_j, times sigmoid(gate) per head or
//                 per entry.
// Queries and keys may be rotated by position before they are used / cached (first rot_dims entries of a head, fp32 angle).
// Queries may carry a temperature: the query at position p is multiplied by 1 + coef * ln(1 + (p + 1) / every), integer quotient.
//
// Kernels: gqa_prepare_kernel (bias, per-head RMS norm, temperature, cache append), gqa_prepare_row_kernel (the same with ONE norm
// over the whole query / key projection), gqa_attention_kernel + gqa_combine_kernel (one warp per (row, query head); decode,
// short portions and the 32-bit mode), gqa_flash_kernel (tensor cores, bf16, long portions).
#pragma once
#include "layered_kernels.cuh"
#include "layered_blocks.cuh"

namespace xl {

struct GqaScore {
  float scale, cap;
  int window, chunk;
  const void* r1;    // per query head, T; NULL = no distance penalty
  const void* r2;
  const float* rel;  // [H][rel_n] fp32: learned bias per distance, the last entry for every larger distance; NULL = none
  int rel_n;
  const void* sink;  // per query head, T; NULL = no sink
  int keep_first;    // > 0: the first tokens of a request that every later row sees
  int pool;          // > 0: tokens per pooled block
  size_t pool_rows;  // rows of the pool's first half (token rows); pooled block b of a request lives at pool_rows + row(slot, b)
};

// Keys a work item meets come in two stretches: `extra` keys in front (kept first tokens that lie before the item's token range, or
// the pooled blocks its last row sees), then the tokens first .. last.  A VIRTUAL index v runs over both: v < extra -> extra key v.
__device__ __host__ __forceinline__ int gqa_extra_keys(int first, int pos_last, int window, int keep_first, int pool) {
  if (keep_first > 0) return keep_first < first ? keep_first : first;
  if (pool > 0 && window > 0) return pos_last - window + 1 > 0 ? (pos_last - window + 1) / pool : 0;
  return 0;
}
// pooled blocks the row at `pos` sees: those with (b + 1) * pool <= pos - window + 1
__device__ __forceinline__ int gqa_blocks_seen(int pos, int window, int pool) { return pos - window + 1 > 0 ? (pos - window + 1) / pool : 0; }

// multiplier of the query at position pos (1 when coef == 0)
__device__ __forceinline__ float gqa_query_temperature(float coef, int every, int pos) {
  return coef != 0.f ? 1.0f + coef * logf((float)((pos + 1) / every + 1)) : 1.0f;
}
// folds a sink into finished softmax statistics: returns the factor for the accumulator, updates the denominator
__device__ __forceinline__ float gqa_apply_sink(float sink, float mx, float& den) {
  const float nmx = fmaxf(mx, sink);
  const float corr = mx == -INFINITY ? 0.f : expf(mx - nmx);
  den = den * corr + expf(sink - nmx);
  return corr;
}

template <typename T>
__device__ __forceinline__ float gqa_adjust(float dot, const GqaScore& sc, float r1, float r2, const float* __restrict__ rel_head, int dist) {
  float s = dot * sc.scale;
  if (sc.cap > 0.f) s = sc.cap * tanhf(s / sc.cap);
  if (sc.r1) s -= r1 * log1pf(r2 * (float)dist);
  if (rel_head) s += rel_head[min(dist, sc.rel_n - 1)];
  return s;
}
// the same in the tensor-core prompt kernel: fp32 with the fast exponential and division units (tanh x = (e^2x - 1) / (e^2x + 1))
__device__ __forceinline__ float gqa_adjust_fast(float dot, const GqaScore& sc, float inv_cap, const float* __restrict__ dist_bias, int dist) {
  float s = dot * sc.scale;
  if (sc.cap > 0.f) {
    const float t = __expf(2.0f * fminf(fmaxf(s * inv_cap, -15.f), 15.f));
    s = sc.cap * __fdividef(t - 1.0f, t + 1.0f);
  }
  if (dist_bias) s += dist_bias[dist];                         // learned bias - r1 * ln(1 + r2 * distance), staged per tile; the caller's index
  return s;
}
__device__ __forceinline__ bool gqa_visible(int pos, int j, int window, int chunk, int keep_first = 0) {
  return j <= pos && (window == 0 || pos - j < window || j < keep_first) && (chunk == 0 || j / chunk == pos / chunk);
}
// first key any row of positions pos0 .. can see
__device__ __host__ __forceinline__ int gqa_first_key(int pos0, int window, int chunk) {
  int f = 0;
  if (window > 0 && pos0 - window + 1 > f) f = pos0 - window + 1;
  if (chunk > 0 && (pos0 / chunk) * chunk > f) f = (pos0 / chunk) * chunk;
  return f;
}

// ---------------------------------------------------------------------------------------------------------------------------
// After the input projection: proj[m, :] (fp32) holds q (H * dk) at col_q and, for a layer with keys/values of its own, k (G * dk)
// at col_k and v (G * dv) at col_v.  Adds the projection biases, RMS-norms every query and key head over dk (weight of size dk
// shared by the heads; w == NULL: no norm) and stores queries as fp32 [M, H, dk] (+ a bf16 copy for the tensor-core kernel) and
// keys / values into the row's place of the paged pool; queries are multiplied by their temperature.  norm_on without weights: the
// heads are only divided by their root mean square.  freqs != NULL: after the norm, the first rot_dims entries of every query and key
// head are rotated by angle pos * freqs[i] (rot_layout 1: entry i pairs with i + rot_dims / 2; 0: entries 2i, 2i + 1):
// (u, v) -> (u cos - v sin, v cos + u sin).  One warp per (row, head slot): slots 0..H-1 queries, H..H+G-1 keys, H+G..H+2G-1 values.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gqa_prepare_kernel(const float* __restrict__ proj, int ld, int col_q, int col_k, int col_v, const T* __restrict__ bias,
                                   const T* __restrict__ q_norm, const T* __restrict__ k_norm, float eps, int H, int G, int dk, int dv, int own_kv,
                                   float q_temp_coef, int q_temp_every, const int* __restrict__ row_slot, const int* __restrict__ row_pos, Paging pg,
                                   T* __restrict__ pool, float* __restrict__ qf, bf16* __restrict__ q16, int M, int norm_on,
                                   const float* __restrict__ freqs, int rot_dims, int rot_layout) {
  const int slots = H + (own_kv ? 2 * G : 0);
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= M * slots) return;
  const int m = idx / slots, sl = idx % slots;
  const float* pr = proj + (size_t)m * ld;
  if (sl >= H + G) {                                           // a value head: bias, store
    const int g = sl - H - G, c0 = col_v + g * dv;
    T* dst = pool + pg.row(row_slot[m], row_pos[m]) * (size_t)(G * (dk + dv)) + (size_t)G * dk + (size_t)g * dv;
    for (int d = lane; d < dv; d += 32) stf(dst + d, pr[c0 + d] + (bias ? ldf(bias + c0 + d) : 0.f));
    return;
  }
  const bool is_q = sl < H;
  const int hd = is_q ? sl : sl - H, c0 = (is_q ? col_q : col_k) + hd * dk;
  const T* w = is_q ? q_norm : k_norm;
  float ss = 0.f;
  for (int d = lane; d < dk; d += 32) { const float v = pr[c0 + d] + (bias ? ldf(bias + c0 + d) : 0.f); ss = fmaf(v, v, ss); }
  const float rs = (norm_on ? 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps) : 1.0f) * (is_q ? gqa_query_temperature(q_temp_coef, q_temp_every, row_pos[m]) : 1.0f);
  T* kdst = is_q ? nullptr : pool + pg.row(row_slot[m], row_pos[m]) * (size_t)(G * (dk + dv)) + (size_t)hd * dk;
  const float fpos = (float)row_pos[m];
  const int half = rot_dims >> 1;
  for (int d = lane; d < dk; d += 32) {
    float v = (pr[c0 + d] + (bias ? ldf(bias + c0 + d) : 0.f)) * rs * (w ? ldf(w + d) : 1.f);
    if (freqs && d < rot_dims) {
      const bool lo = rot_layout ? d < half : (d & 1) == 0;   // the pair's first member
      const int dp = rot_layout ? (lo ? d + half : d - half) : (d ^ 1), fi = rot_layout ? (lo ? d : d - half) : (d >> 1);
      const float o = (pr[c0 + dp] + (bias ? ldf(bias + c0 + dp) : 0.f)) * rs * (w ? ldf(w + dp) : 1.f);
      const float ang = fpos * freqs[fi], cs = cosf(ang), sn = sinf(ang);
      v = lo ? v * cs - o * sn : v * cs + o * sn;
    }
    if (is_q) {
      qf[((size_t)m * H + hd) * dk + d] = v;
      if (q16) q16[((size_t)m * H + hd) * dk + d] = __float2bfloat16_rn(v);
    } else {
      stf(kdst + d, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// The same step for layers whose query / key norm runs over the WHOLE projection: q (all H * dk entries of the row, bias added)
// is divided by its root mean square and multiplied by a weight of that size, and so is k (G * dk entries).  One block per row.
// First pass: every load the row needs (projection, biases, norm weights) is issued at once — the sums of squares are taken, the
// entries wait in shared memory already multiplied by their norm weight, the values go straight to the pool; one block-wide
// reduction of both sums; second pass: scale and write q (fp32, + bf16 copy) and k (paged pool).  Dynamic shared memory:
// (H + G) * dk floats.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gqa_prepare_row_kernel(const float* __restrict__ proj, int ld, int col_q, int col_k, int col_v, const T* __restrict__ bias,
                                       const T* __restrict__ q_norm, const T* __restrict__ k_norm, float eps, int H, int G, int dk, int dv, int own_kv,
                                       float q_temp_coef, int q_temp_every, const int* __restrict__ row_slot, const int* __restrict__ row_pos, Paging pg,
                                       T* __restrict__ pool, float* __restrict__ qf, bf16* __restrict__ q16) {
  extern __shared__ float qk_row[];                            // [nq] q * q_norm, then [nk] k * k_norm; read back by the writing thread only
  __shared__ float red[2][32];
  const int m = blockIdx.x, nq = H * dk, nk = own_kv ? G * dk : 0, nv = own_kv ? G * dv : 0;
  const float* pr = proj + (size_t)m * ld;
  T* dst = own_kv ? pool + pg.row(row_slot[m], row_pos[m]) * (size_t)(nk + nv) : nullptr;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < nq; c += blockDim.x) {
    const float v = pr[col_q + c] + (bias ? ldf(bias + col_q + c) : 0.f);
    sq = fmaf(v, v, sq);
    qk_row[c] = v * ldf(q_norm + c);
  }
  for (int c = threadIdx.x; c < nk; c += blockDim.x) {
    const float v = pr[col_k + c] + (bias ? ldf(bias + col_k + c) : 0.f);
    sk = fmaf(v, v, sk);
    qk_row[nq + c] = v * ldf(k_norm + c);
  }
  for (int c = threadIdx.x; c < nv; c += blockDim.x) stf(dst + nk + c, pr[col_v + c] + (bias ? ldf(bias + col_v + c) : 0.f));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
  __syncthreads();
  sq = warp_sum(lane < nw ? red[0][lane] : 0.f);
  sk = warp_sum(lane < nw ? red[1][lane] : 0.f);
  const float rq = 1.0f / sqrtf(sq / (float)nq + eps) * gqa_query_temperature(q_temp_coef, q_temp_every, row_pos[m]);
  for (int c = threadIdx.x; c < nq; c += blockDim.x) {
    const float v = qk_row[c] * rq;
    qf[(size_t)m * nq + c] = v;
    if (q16) q16[(size_t)m * nq + c] = __float2bfloat16_rn(v);
  }
  if (nk) {
    const float rk = 1.0f / sqrtf(sk / (float)nk + eps);
    for (int c = threadIdx.x; c < nk; c += blockDim.x) stf(dst + c, qk_row[nq + c] * rk);
  }
}

// table[a][d] = rel[bucket_of[d], a] for d < n: the learned bias of head a at distance d (rel is [buckets, H] as stored)
template <typename T>
__global__ void gqa_rel_table_kernel(const T* __restrict__ rel, const int* __restrict__ bucket_of, int H, int n, float* __restrict__ table) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)H * n) return;
  const int a = (int)(i / n), d = (int)(i % n);
  table[i] = ldf(rel + (size_t)bucket_of[d] * H + a);
}

// how the mixer output is gated: 0 none, 1 sigmoid(gate[m, col0 + head]), 2 sigmoid(gate[m, col0 + head * dv + d])
__device__ __forceinline__ float gqa_gate(const float* gate, int mode, size_t m, int ld, int col0, int h, int dv, int d) {
  if (mode == 0) return 1.f;
  return sigmoidf_(gate[m * ld + col0 + (mode == 1 ? h : h * dv + d)]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Pooled blocks: when a step appends the last token of block b (tokens b * P .. b * P + P - 1) of a request, the block's pooled row
// — the mean over its P cached rows, keys and values alike, fp32 sum — is stored at pool_rows + row(slot, b).  grid (requests of the
// step, blocks a request can complete in it, 128-entry pieces of the row).
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gqa_pool_blocks_kernel(T* __restrict__ pool, Paging pg, size_t pool_rows, const Item* __restrict__ seqs, int P, int rowlen) {
  const Item sq = seqs[blockIdx.x];
  const int b = sq.pos0 / P + blockIdx.y;
  if (b >= (sq.pos0 + sq.n_rows) / P) return;
  T* dst = pool + (pool_rows + pg.row(sq.slot, b)) * (size_t)rowlen;
  const float inv = 1.0f / (float)P;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  if (c >= rowlen) return;
  float a = 0.f;
  for (int t = 0; t < P; ++t) a += ldf(pool + pg.row(sq.slot, b * P + t) * (size_t)rowlen + c);
  stf(dst + c, a * inv);
}

// ---------------------------------------------------------------------------------------------------------------------------
// One CTA = one work item (up to q_per_item consecutive rows of one request) x one key/value head; one WARP owns one (row, query
// head of the group) pair.  32 cached keys + values of the head wait in shared memory (fp32, odd row stride): lane j scores key j,
// the softmax statistics go round by shuffles, then the lanes split the dv value columns (NACC = ceil(dv / 32) registers).
// The keys are walked by their virtual index (extra keys first, see gqa_extra_keys).
// gridDim.z > 1: the keys are cut into runs of `chunk_keys` (a multiple of 32); run z parks {max, sum, accumulator[dv]} in `part`
// ([M * H][gridDim.z][2 + dv]) and gqa_combine_kernel merges them.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T, int NACC>
__global__ void gqa_attention_kernel(const float* __restrict__ qf, const T* __restrict__ pool, Paging pg, const Item* __restrict__ items, int H,
                                     int G, int dk, int dv, GqaScore sc, const float* __restrict__ gate, int gate_mode, int gate_ld, int gate_col0,
                                     T* __restrict__ out, int chunk_keys, float* __restrict__ part) {
  extern __shared__ float smem[];
  const Item it = items[blockIdx.x];
  const int rep = H / G, W = dk + dv, WS = W | 1;
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_y = (it.n_rows * rep + nw - 1) / nw;         // blockIdx.y = kv head * y-tiles + tile
  const int ypg = gridDim.y / G;
  const int g = blockIdx.y / ypg, ytile = blockIdx.y % ypg;
  if (ytile >= tiles_y) return;                                // whole CTA: no barrier has been passed yet
  float* ktile = smem;                                         // [32][WS]
  float* qs = smem + 32 * WS;                                  // [warps][dk]
  const int pair = ytile * nw + warp;
  const bool active = pair < it.n_rows * rep;
  const int qi = active ? pair / rep : 0, h = g * rep + (active ? pair % rep : 0);
  const int m = it.row0 + qi, pos = it.pos0 + qi;
  float* q = qs + (size_t)warp * dk;
  if (active) {
    const float* src = qf + ((size_t)m * H + h) * dk;
    for (int d = lane; d < dk; d += 32) q[d] = src[d];
  }
  const float r1 = sc.r1 ? ldf(static_cast<const T*>(sc.r1) + h) : 0.f, r2 = sc.r1 ? ldf(static_cast<const T*>(sc.r2) + h) : 0.f;
  const float* rel_head = sc.rel ? sc.rel + (size_t)h * sc.rel_n : nullptr;
  const int first = gqa_first_key(it.pos0, sc.window, sc.chunk), pos_last = it.pos0 + it.n_rows - 1;
  const int extra = gqa_extra_keys(first, pos_last, sc.window, sc.keep_first, sc.pool);
  int vfirst = 0, vlast = extra + pos_last - first;           // virtual key range of the item
  if (gridDim.z > 1) {
    vfirst = blockIdx.z * chunk_keys;
    vlast = min(vlast, vfirst + chunk_keys - 1);
  }
  float acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  float mx = -INFINITY, den = 0.f;
  const size_t rowlen = (size_t)G * W;
  const int seen = sc.pool > 0 ? gqa_blocks_seen(pos, sc.window, sc.pool) : 0;
  for (int j0 = vfirst; j0 <= vlast; j0 += 32) {
    __syncthreads();
    for (int jr = warp; jr < 32; jr += nw) {
      const int v = j0 + jr;
      float* dst = ktile + jr * WS;
      if (v <= vlast) {
        const size_t prow = v >= extra ? pg.row(it.slot, first + v - extra) : sc.pool > 0 ? sc.pool_rows + pg.row(it.slot, v) : pg.row(it.slot, v);
        const T* src = pool + prow * rowlen;
        for (int d = lane; d < dk; d += 32) dst[d] = ldf(src + (size_t)g * dk + d);
        for (int d = lane; d < dv; d += 32) dst[dk + d] = ldf(src + (size_t)G * dk + (size_t)g * dv + d);
      } else {
        for (int d = lane; d < W; d += 32) dst[d] = 0.f;
      }
    }
    __syncthreads();
    if (!active) continue;
    const int v = j0 + lane;
    const int j = v >= extra ? first + v - extra : v;         // a token's position (kept first tokens keep theirs); a pooled block's index
    const bool vis = v <= vlast && (v >= extra ? gqa_visible(pos, j, sc.window, sc.chunk, sc.keep_first) : (sc.pool > 0 ? v < seen : true));
    float s = 0.f;
    const float* kr = ktile + lane * WS;
    for (int d = 0; d < dk; ++d) s = fmaf(q[d], kr[d], s);
    s = vis ? gqa_adjust<T>(s, sc, r1, r2, rel_head, pos - j) : -INFINITY;
    const float tmax = warp_max(s);
    if (tmax == -INFINITY) continue;                           // warp-uniform
    const float nmx = fmaxf(mx, tmax);
    const float corr = expf(mx - nmx);
    const float p = vis ? expf(s - nmx) : 0.f;
    den = den * corr + warp_sum(p);
    mx = nmx;
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] *= corr;
    for (int jr = 0; jr < 32; ++jr) {
      const float pj = __shfl_sync(0xffffffffu, p, jr);
      if (pj == 0.f) continue;                                 // warp-uniform
      const float* v = ktile + jr * WS + dk;
#pragma unroll
      for (int a = 0; a < NACC; ++a) {
        const int d = a * 32 + lane;
        if (d < dv) acc[a] = fmaf(pj, v[d], acc[a]);
      }
    }
  }
  if (!active) return;
  if (gridDim.z > 1) {
    float* dst = part + (((size_t)m * H + h) * gridDim.z + blockIdx.z) * (size_t)(2 + dv);
    if (lane == 0) { dst[0] = mx; dst[1] = den; }
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int d = a * 32 + lane;
      if (d < dv) dst[2 + d] = acc[a];
    }
    return;
  }
  const float corr = sc.sink ? gqa_apply_sink(ldf(static_cast<const T*>(sc.sink) + h), mx, den) : 1.0f;
  const float inv = corr / den;
  T* o = out + (size_t)m * H * dv + (size_t)h * dv;
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    const int d = a * 32 + lane;
    if (d < dv) stf(o + d, acc[a] * inv * gqa_gate(gate, gate_mode, m, gate_ld, gate_col0, h, dv, d));
  }
}

// merges the key runs: one warp per (row, query head) of the listed items; at most 32 runs.  A sink (per head, may be NULL) joins
// here, once, like a run that holds the weight exp(sink) and no values.
template <typename T>
__global__ void gqa_combine_kernel(const float* __restrict__ part, const Item* __restrict__ items, int H, int dv, int splits, const T* __restrict__ sink,
                                   const float* __restrict__ gate, int gate_mode, int gate_ld, int gate_col0, T* __restrict__ out) {
  const Item it = items[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int pair = blockIdx.y * nw + warp;
  if (pair >= it.n_rows * H) return;
  const int m = it.row0 + pair / H, h = pair % H;
  const float* src = part + ((size_t)m * H + h) * splits * (size_t)(2 + dv);
  const float mz = lane < splits ? src[(size_t)lane * (2 + dv)] : -INFINITY;
  const float sk = sink ? ldf(sink + h) : -INFINITY;
  const float mx = fmaxf(warp_max(mz), sk);
  const float wz = mz == -INFINITY ? 0.f : expf(mz - mx);
  const float den = warp_sum(lane < splits ? src[(size_t)lane * (2 + dv) + 1] * wz : 0.f) + (sink ? expf(sk - mx) : 0.f);
  const float inv = 1.0f / den;
  for (int d0 = 0; d0 < dv; d0 += 32) {
    const int d = d0 + lane;
    float a = 0.f;
#pragma unroll 8
    for (int z = 0; z < splits; ++z) {                         // loads without a branch, so that several are in flight: a run
      const float w = __shfl_sync(0xffffffffu, wz, z);         // that saw no key has parked zeros and weighs zero
      const float v = d < dv ? src[(size_t)z * (2 + dv) + 2 + d] : 0.f;
      a = fmaf(v, w, a);
    }
    if (d < dv) stf(out + (size_t)m * H * dv + (size_t)h * dv + d, a * inv * gqa_gate(gate, gate_mode, m, gate_ld, gate_col0, h, dv, d));
  }
}

// ===========================================================================================================================
// Prompt attention on the tensor cores (bf16 serving path; requests that bring FLASH_MIN_ROWS rows or more; sizes whose rows are
// whole 16-byte chunks: dk, dv multiples of 8, dk <= 256, dv <= 128).  One CTA = one tile of up to 64 consecutive rows of one
// request x one query head.  Keys and values of the head's key/value group come straight from the paged pool by 16-byte cp.async
// into two buffers each (the next 64 keys are in flight while these are multiplied); Q, K fragments by ldmatrix, V transposed on
// the way into registers by ldmatrix.trans; scores by mma.sync.m16n8k16 (bf16 operands, fp32 accumulators), then in fp32: scale,
// soft cap, distance penalty, mask, running max and sum.  The softmax weights enter the value product as a bf16 PAIR (high part +
// remainder, two MMAs) so that they keep 16 mantissa bits.  The keys are walked by their virtual index (kept first tokens or pooled
// blocks in front of the token stretch, see gqa_extra_keys); distance terms go with layers that have no such keys.
// ===========================================================================================================================
// dist_table[a][d] = r1[a] * ln(1 + r2[a] * d) for d < n: the distance penalty of head a, made once per step and layer so that the
// prompt kernel reads it instead of taking a logarithm per score
__global__ void gqa_dist_table_kernel(const bf16* __restrict__ r1, const bf16* __restrict__ r2, int H, int n, float* __restrict__ table) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)H * n) return;
  const int a = (int)(i / n), d = (int)(i % n);
  table[i] = __bfloat162float(r1[a]) * log1pf(__bfloat162float(r2[a]) * (float)d);
}

struct GqaTile {
  int row0;      // first packed row
  int n_rows;    // <= 64 consecutive rows of one request
  int pos0;      // position of row0
  int slot;      // request
};

template <int DVT>   // value columns per warp row: DVT tiles of 8 (dv <= 8 * DVT)
__global__ void __launch_bounds__(128)
gqa_flash_kernel(const bf16* __restrict__ q16, const bf16* __restrict__ pool, Paging pg, const GqaTile* __restrict__ tiles, int H, int G, int dk, int dv,
                 GqaScore sc, const float* __restrict__ dist_table, int dist_n, const float* __restrict__ gate, int gate_mode, int gate_ld, int gate_col0,
                 bf16* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t gsm[];
  __shared__ size_t krow[2][64];                    // pool rows of the keys of the tile in flight / in use
  __shared__ float dpen[2][128];                    // distance terms (learned bias - penalty) a (64 rows x 64 keys) tile can meet: distance = dbase + index
  const GqaTile tl = tiles[gridDim.x - 1 - blockIdx.x];   // later tiles of a request see more keys: the long ones start first
  const int h = blockIdx.y, g = h / (H / G);
  const int DQP = (dk + 15) & ~15, QS = DQP + 8;
  constexpr int VS = 8 * DVT + 8;
  bf16* Qs = reinterpret_cast<bf16*>(gsm);          // [64][QS]
  bf16* Ks = Qs + 64 * QS;                          // [2][64][QS]
  bf16* Vs = Ks + 2 * 64 * QS;                      // [2][64][VS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  const int last = tl.pos0 + tl.n_rows - 1;
  const int first = gqa_first_key(tl.pos0, sc.window, sc.chunk);
  const int extra = gqa_extra_keys(first, last, sc.window, sc.keep_first, sc.pool);   // keys in front of the token stretch (virtual index < extra)
  const int vlast = extra + last - first;
  const int qc = DQP / 8;
  const size_t rowlen = (size_t)G * (dk + dv);
  const float* dtab = dist_table ? dist_table + (size_t)h * dist_n : nullptr;
  const float* rtab = sc.rel ? sc.rel + (size_t)h * sc.rel_n : nullptr;
  const bool dist_terms = dtab || rtab;

  // the page walk is done once per key (64 threads), then every thread copies 16-byte pieces from the rows it names
  auto locate = [&](int v0, int bsel) {
    if (threadIdx.x < 64) {
      const int v = v0 + (int)threadIdx.x;
      size_t r = 0;
      if (v <= vlast) r = v >= extra ? pg.row(tl.slot, first + v - extra) : sc.pool > 0 ? sc.pool_rows + pg.row(tl.slot, v) : pg.row(tl.slot, v);
      krow[bsel][threadIdx.x] = r * rowlen;
    }
  };
  auto issue = [&](int j0, int bsel) {                   // j0: virtual index of the tile's first key
    bf16* kd = Ks + bsel * 64 * QS;
    for (int e = threadIdx.x; e < 64 * qc; e += 128) {
      const int r = e / qc, c = (e % qc) * 8, j = j0 + r;
      bf16* dst = kd + r * QS + c;
      if (j > vlast || c >= dk) *reinterpret_cast<uint4*>(dst) = zero4;
      else cp_async16_b(dst, pool + krow[bsel][r] + (size_t)g * dk + c);
    }
    bf16* vd = Vs + bsel * 64 * VS;
    for (int e = threadIdx.x; e < 64 * DVT; e += 128) {
      const int r = e / DVT, c = (e % DVT) * 8, j = j0 + r;
      bf16* dst = vd + r * VS + c;
      if (j > vlast || c >= dv) *reinterpret_cast<uint4*>(dst) = zero4;
      else cp_async16_b(dst, pool + krow[bsel][r] + (size_t)G * dk + (size_t)g * dv + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  for (int e = threadIdx.x; e < 64 * qc; e += 128) {
    const int r = e / qc, c = (e % qc) * 8;
    uint4 v = zero4;
    if (r < tl.n_rows && c < dk) v = *reinterpret_cast<const uint4*>(q16 + ((size_t)(tl.row0 + r) * H + h) * dk + c);
    *reinterpret_cast<uint4*>(Qs + r * QS + c) = v;
  }
  float o[DVT][4];
#pragma unroll
  for (int i = 0; i < DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mx[2] = {-INFINITY, -INFINITY}, den[2] = {0.f, 0.f};
  const int pos_lo = tl.pos0 + warp * 16 + gq, pos_hi = pos_lo + 8;
  // visible keys of this thread's two rows: [lo, pos] (the divisions of the block rule are done once, here)
  const int vis_lo[2] = {gqa_first_key(pos_lo, sc.window, sc.chunk), gqa_first_key(pos_hi, sc.window, sc.chunk)};
  const int seen[2] = {sc.pool > 0 ? gqa_blocks_seen(pos_lo, sc.window, sc.pool) : 0, sc.pool > 0 ? gqa_blocks_seen(pos_hi, sc.window, sc.pool) : 0};
  const float inv_cap = sc.cap > 0.f ? 1.0f / sc.cap : 0.f;
  const int ntile = vlast / 64 + 1;
  locate(0, 0);
  locate(64, 1);
  __syncthreads();
  issue(0, 0);
  for (int it = 0; it < ntile; ++it) {
    const int v0 = it * 64, bsel = it & 1;
    const int j0 = first + v0 - extra;                  // position of the tile's first key where it is a token (distance terms: extra == 0)
    if (dist_terms) {                                // distances pos0 - (j0 + 63) + index; negative ones belong to keys after the row (masked)
      const int d = tl.pos0 - j0 - 63 + (int)threadIdx.x;
      float b = 0.f;
      if (dtab && d >= 0 && d < dist_n) b = -dtab[d];
      if (rtab && d >= 0) b += rtab[min(d, sc.rel_n - 1)];
      dpen[bsel][threadIdx.x] = b;
    }
    if (it + 1 < ntile) {
      issue(v0 + 64, bsel ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    locate(v0 + 128, bsel);                          // krow[bsel] was last read by the issue of this tile; the next reader is two barriers away
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
        const int v = v0 + n * 8 + 2 * t + (x & 1), j = first + v - extra, pos = (x < 2) ? pos_lo : pos_hi;
        const bool vis = v < extra ? (sc.pool > 0 ? v < seen[x >> 1] : true) : (j <= last && j <= pos && (j >= vis_lo[x >> 1] || j < sc.keep_first));
        s[n][x] = vis ? gqa_adjust_fast(s[n][x], sc, inv_cap, dist_terms ? dpen[bsel] : nullptr, (pos - tl.pos0) - (j - j0) + 63) : -INFINITY;
        tmax[x >> 1] = fmaxf(tmax[x >> 1], s[n][x]);
      }
    float corr[2], nmx[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      nmx[r] = fmaxf(mx[r], tmax[r]);
      corr[r] = (mx[r] == -INFINITY) ? 0.f : __expf(mx[r] - nmx[r]);
      mx[r] = nmx[r];
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float p = (s[n][x] == -INFINITY) ? 0.f : __expf(s[n][x] - nmx[x >> 1]);
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
    const int qi = warp * 16 + gq + r * 8;
    if (qi >= tl.n_rows) continue;
    const size_t m = tl.row0 + qi;
    const float corr = sc.sink ? gqa_apply_sink(__bfloat162float(static_cast<const bf16*>(sc.sink)[h]), mx[r], den[r]) : 1.0f;
    const float inv = corr / den[r];
    bf16* dst = out + m * ((size_t)H * dv) + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < DVT; ++i) {
      const int c = i * 8 + 2 * t;
      if (c < dv)
        *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16x2(o[i][r * 2] * inv * gqa_gate(gate, gate_mode, m, gate_ld, gate_col0, h, dv, c),
                                                            o[i][r * 2 + 1] * inv * gqa_gate(gate, gate_mode, m, gate_ld, gate_col0, h, dv, c + 1));
    }
  }
}

}  // namespace xl
