// layered.cu — host side of libxotb200_lm.so (include/xotb200_lm.h): the layered-model engine.
//
//   model     : a table of layers (xotb200_lm_layer); weights in ONE blob of T (bf16 or fp32), input projections of a mixer that
//               read the same normed input are stored as one concatenated matrix so they are one product;
//   loader    : strict safetensors reader (mmap -> device staging -> widen/copy kernel into the blob);
//   state     : paged cache (one pool per attention layer that owns keys/values or latents, page table per slot, host free list)
//               + fp32 recurrent states and convolution inputs per slot; slots are emptied and reused, pages return to the pool;
//   step      : a packed batch of rows through the layers on one stream (kernels in layered_kernels.cuh; the second mixer of a
//               two-mixer layer on a side stream beside the first), logits / argmax of the wanted rows back to the host.
#include <cuda_runtime.h>
#include <dirent.h>
#include <fcntl.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <type_traits>
#include <map>
#include <string>
#include <vector>

#include "../../include/xotb200_lm.h"
#include "layered_kernels.cuh"
#include "layered_blocks.cuh"
#include "layered_gqa.cuh"
#include "layered_recurrent.cuh"
#include "layered_tc.cuh"
#include "st_header.h"

using namespace xl;

static thread_local char g_err[1024] = "";
static void set_err(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
#define CK(call)                                                                           \
  do {                                                                                     \
    cudaError_t _e = (call);                                                               \
    if (_e != cudaSuccess) {                                                               \
      set_err("%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return XOTB200_ECUDA;                                                                \
    }                                                                                      \
  } while (0)
#define REQUIRE(cond, ...)   \
  do {                       \
    if (!(cond)) {           \
      set_err(__VA_ARGS__);  \
      return XOTB200_EINVAL; \
    }                        \
  } while (0)
#define TRY(call)           \
  do {                      \
    int _r = (call);        \
    if (_r < 0) return _r;  \
  } while (0)

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static int cdiv(long a, long b) { return (int)((a + b - 1) / b); }

// where a tensor of the file goes: rows [row_off, row_off + rows) of a [*, cols] matrix in the blob
struct Dest {
  size_t elem_off;   // element offset of the matrix in the blob
  int rows, cols, row_off;
  bool loaded;
  bool has2 = false;  // a second, untransposed copy at elem_off2 (W_uk: the expanded prompt attention reads it row-major)
  size_t elem_off2 = 0;
  int tr_heads = 0;   // > 0: the file's [heads * d, cols] matrix is stored head by head TRANSPOSED, [heads][cols][d]
  int il8 = -1;       // 0 / 1: row r goes to row (r / 8) * 16 + il8 * 8 + r % 8 of the matrix at elem_off (gate / up rows of an expert)
};

struct LmLayer {
  xotb200_lm_layer s;
  size_t norm1, norm1b, norm2, norm2b;                 // element offsets into the blob
  size_t w_in;                                         // concatenated input projections [n_in, D]
  int n_in;
  int c_q, c_kv, c_g;                                  // latent attention: columns of the projection output
  size_t dq_norm, uq, dkv_norm, uk, uk_rows, uv, wo;
  int c_r, c_k, c_v, c_a, c_w1;                        // delta rule: columns (gate shares c_g)
  size_t w2, w0, a_b, onorm;
  size_t up, down;
  // grouped-query attention: columns of q / k / v (gate: c_g), bias vector over the projection's columns, norm weights, penalties
  int c_kk = 0, c_vv = 0;
  size_t b_in = 0, q_norm = 0, k_norm = 0, r1 = 0, r2 = 0, o_b = 0, sink = 0, rel = 0;
  int rel_n = 0;                                       // distances tabulated for the learned bias: every distance >= rel_n - 1 is in the last bucket
  int* rel_bucket = nullptr;                           // [rel_n] bucket of every tabulated distance (device; made on the host in double)
  float* rel_tab = nullptr;                            // [heads][rel_n] the bias per head and distance (device; remade when weights change)
  int kv_src = -1;                                     // local index of the layer whose pool this layer reads (itself when it has keys/values)
  // gated delta rule: filter weights [channels, taps] (q, k, v channels in the projection's order), decay constants, column of beta
  size_t conv_w = 0, a_log = 0, dt_bias = 0;
  int c_b = 0, conv_ch = 0;
  size_t conv_off = 0;                                 // float offset of the filter inputs inside a slot's state block
  // feed-forward forms: xIELU parameters; mixture of experts: router [E, D], experts' [E][2 F, D] (gate rows, up rows) and [E][D, F]
  size_t act_p = 0, router = 0, router_b = 0, w_gu = 0, w_edown = 0;   // a shared expert's matrices are `up` / `down`
  // matrix LSTM: gate biases, float offset of the running maxima in a slot's block; state-space layer: filter bias, skip weights
  size_t i_b = 0, f_b = 0, conv_b = 0, d_skip = 0, m_off = 0, n_off = 0;
  int c_i = 0, c_f = 0, c_z = 0, c_dt = 0;
  int ld_in = 0;                                       // leading dimension of the projection output this mixer reads (all mixers of the layer)
  std::vector<LmLayer> par;                            // the layer's second mixer (0 or 1 entries): reads the same input, output added
  // pre-norm block with one-number weights: convolutions on the sublayer inputs ([D, taps]), their inputs' place in a slot's state
  // block, hyper-connection coefficients (in [S], out [S], mix [S, S]) of the two sublayers
  size_t canon[2] = {0, 0}, canon_off[2] = {0, 0}, hc_in[2] = {0, 0}, hc_out[2] = {0, 0}, hc_mix[2] = {0, 0};
  float* freqs = nullptr;                              // [rot_dims / 2] fp32 on the device
  void* pool = nullptr;                                // paged pool [n_pages * P, row] of T: latent + rotated key part, or keys + values
  size_t state_off = 0;                                // delta rules: float offset of this layer's state inside a slot's block
};

struct GraphSlot {
  int seen = 0;
  cudaGraphExec_t exec = nullptr;
  int64_t launches = 0;
};

struct xotb200_lm {
  xotb200_lm_cfg cfg;
  std::vector<LmLayer> layers;                         // local layers
  int device = 0, sm_count = 148;
  bool first = false, last = false;
  size_t esz = 2;
  cudaStream_t stream = nullptr;                       // the stream every launch goes to (the second mixer of a layer swaps in `side`)
  cudaStream_t side = nullptr;                         // second mixer of a two-mixer layer: runs beside the first, joined before the layer goes on
  cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev_fork = nullptr, ev_join = nullptr;
  char* blob = nullptr;
  size_t blob_elems = 0;
  size_t embed = 0, final_norm = 0, head = 0, embed_norm = 0;
  float* pos_freqs = nullptr;                          // [ceil(width / 2)] frequencies of the computed position vector (device)
  bool tables_stale = true;                            // tables derived from weights (learned distance bias) have to be remade
  std::map<std::string, Dest> dests;
  // request state
  int max_requests = 0, page_size = 0, n_pages = 0, pages_per_slot = 0;
  std::vector<int> free_pages, slot_len, slot_pages;
  int* h_table = nullptr;                              // pinned [max_requests, pages_per_slot]
  int* d_table = nullptr;
  float* state = nullptr;                              // [max_requests][state_floats]
  size_t state_floats = 0;
  // per-step staging
  int* h_stage = nullptr;
  int* d_stage = nullptr;
  size_t stage_cap = 0;
  // scratch (rows capacity m_cap)
  int m_cap = 0, want_cap = 0;
  float *x = nullptr, *y = nullptr, *proj = nullptr, *qraw = nullptr, *qfull = nullptr, *wlog = nullptr, *oraw = nullptr, *du = nullptr, *dau = nullptr, *logits = nullptr;
  float *dkk = nullptr, *drr = nullptr, *cvb = nullptr, *moe_wts = nullptr;   // gated delta rule: write keys, read-out vectors, filtered channels; expert weights
  int* moe_ids = nullptr;
  void* mact = nullptr;                                // experts' inner activations [rows, top, F] of T (grouped form: [padded pairs, F])
  void* moe_xg = nullptr;                              // grouped form: the rows sorted by expert [padded pairs, D] (bf16)
  float* moe_yg = nullptr;                             // grouped form: the experts' outputs [padded pairs, D]
  int* moe_plan = nullptr;                             // counts[E], starts[E + 1], cursor[E], place[rows * top], tile_expert[tiles]
  int moe_tiles_cap = 0;
  float* dist_tab = nullptr;                           // prompt attention: distance penalties per head and distance, remade per layer
  size_t dist_cap = 0;
  int max_conv = 0, max_top = 0, max_eff = 0, max_experts = 0;
  float *y2 = nullptr, *h0 = nullptr, *gdec = nullptr, *ginw = nullptr, *gfloor = nullptr, *gnq = nullptr;   // second mixer's output, normed input
                                                       // before its convolution, matrix-LSTM decay / input weight / floor / n . q per (row, head)
  int max_heads_rec = 0;
  bool pre_scalar = false;
  size_t final_norm_b = 0, pos_table = 0;
  void* oh2 = nullptr;                                 // the second mixer's operand of its output product
  void *h = nullptr, *cqn = nullptr, *qn = nullptr, *olat = nullptr, *oh = nullptr, *act = nullptr, *th = nullptr, *hw = nullptr;
  void *q16 = nullptr, *cbuf = nullptr, *knx = nullptr, *vxx = nullptr;   // expanded prompt attention (bf16)
  size_t flash_keys_cap = 0;
  float* part = nullptr;                               // key-run partial results of the absorbed attention kernel
  size_t part_cap = 0;
  int max_w = 0;                                       // widest cached row (kv_rank + rot_dim)
  int* d_argmax = nullptr;
  float* h_out = nullptr;                              // pinned staging for results
  size_t h_out_cap = 0;
  int max_in = 0, max_q = 0, max_qfull = 0, max_qr = 0, max_hdn = 0, max_olat = 0, max_oh = 0, max_ff = 0, max_hd = 0, max_lr = 0;
  bool trace = false;
  float* trace_buf = nullptr;
  size_t trace_floats = 0, trace_cap = 0;
  int gemm_mode = 0;
  bool graphs_on = true;                               // decode steps are replayed from CUDA graphs
  std::map<std::array<long, 5>, GraphSlot> graphs;
  int64_t graph_replays = 0;
  bool flash_fits = true;                              // every attention layer fits the expanded kernel's tile sizes
  bool gqa_flash_fits = true;                          // every key/value-cache attention layer fits the tensor-core prompt kernel (16-byte rows)
  bool flash_on = true;                                // bf16: prompt portions of FLASH_MIN_ROWS rows or more use the expanded tensor-core attention
  std::vector<int> stage_build;
  int64_t launches = 0, tc_launches = 0, flash_launches = 0;
  int* d_err = nullptr;                                // sticky device error word (3 = a bounded wait of a tensor-core product expired)
  int* h_err = nullptr;                                // pinned copy, read after every step
  float last_ms = 0.f;
};

template <typename T> static T* at(xotb200_lm* e, size_t off) { return reinterpret_cast<T*>(e->blob) + off; }

// ---------------------------------------------------------------------------------------------------------------------------
// layout
// ---------------------------------------------------------------------------------------------------------------------------
// columns of the projection a mixer reads (every matrix that multiplies the sublayer's input)
static int mixer_columns(const xotb200_lm_layer& s) {
  switch (s.mixer) {
    case XOTB200_LM_MIX_ATTENTION:
      return s.heads * s.dim + (s.kv_from < 0 ? s.kv_heads * (s.dim + s.vdim) : 0) + (s.out_gate == 2 ? s.heads * s.vdim : s.out_gate == 1 ? s.heads : 0);
    case XOTB200_LM_MIX_GATED_DELTA: return 2 * s.kv_heads * s.dim + 2 * s.heads * s.vdim + 2 * s.heads;
    case XOTB200_LM_MIX_MATRIX_LSTM: return 2 * s.heads * s.dim + 2 * s.heads * s.vdim + 2 * s.heads;
    case XOTB200_LM_MIX_MAMBA2: return 2 * s.heads * s.vdim + 2 * s.kv_heads * s.dim + s.heads;
    default: return 0;
  }
}

static int build_layout(xotb200_lm* e, const xotb200_lm_layer* all) {
  const int D = e->cfg.width, V = e->cfg.vocab;
  size_t cur = 0;
  const size_t al = 256 / e->esz;
  auto take = [&](size_t n) { size_t o = cur; cur = align_up(cur + n, al); return o; };
  auto dest = [&](const std::string& name, size_t off, int rows, int cols, int row_off) { e->dests[name] = Dest{off, rows, cols, row_off, false}; };
  const bool post_ln = e->cfg.block == XOTB200_LM_BLOCK_POST_LN, post_rms = e->cfg.block == XOTB200_LM_BLOCK_POST_RMS;
  const bool pre_scalar = e->cfg.block == XOTB200_LM_BLOCK_PRE_SCALAR;
  const int NW = pre_scalar ? 1 : D;                   // entries of a block norm's weight
  const int S = e->cfg.streams, CT = e->cfg.canon_taps;
  e->pre_scalar = pre_scalar;
  // what a sublayer of the pre-scalar block owns besides its norm: input convolution and hyper-connection coefficients
  auto sublayer_extras = [&](LmLayer& L, const std::string& p, int q) {
    const std::string n = std::to_string(q + 1);
    if (CT > 0) {
      L.canon[q] = take((size_t)D * CT); dest(p + "canon" + n, L.canon[q], D, CT, 0);
      L.canon_off[q] = e->state_floats;
      e->state_floats += (size_t)(CT - 1) * D;
    }
    if (S > 0) {
      L.hc_in[q] = take(S); dest(p + "hc" + n + ".in", L.hc_in[q], 1, S, 0);
      L.hc_out[q] = take(S); dest(p + "hc" + n + ".out", L.hc_out[q], 1, S, 0);
      L.hc_mix[q] = take((size_t)S * S); dest(p + "hc" + n + ".mix", L.hc_mix[q], S, S, 0);
    }
  };
  // the weight after a sublayer: a second grouped RMS norm ("norm1b"), or the bias of the closing layer norm ("norm1.b"); a closing
  // RMS norm has one weight only
  const std::string nb = post_ln ? ".b" : "b";
  if (e->first) {
    e->embed = take((size_t)V * D); dest("embed", e->embed, V, D, 0);
    if (e->cfg.embed_norm) { e->embed_norm = take(NW); dest("embed.norm", e->embed_norm, 1, NW, 0); }
    if (e->cfg.max_positions > 0) { e->pos_table = take((size_t)e->cfg.max_positions * D); dest("pos", e->pos_table, e->cfg.max_positions, D, 0); }
  }
  for (int li = e->cfg.start_layer; li <= e->cfg.end_layer; ++li) {
    LmLayer L{};
    L.s = all[li];
    const xotb200_lm_layer& s = L.s;
    const std::string p = "l" + std::to_string(li) + ".";
    REQUIRE(s.heads >= 1 && s.dim >= 1, "layer %d: heads and dim must be positive", li);
    L.norm1 = take(NW); dest(p + "norm1", L.norm1, 1, NW, 0);
    if (!post_rms && !pre_scalar) { L.norm1b = take(D); dest(p + "norm1" + nb, L.norm1b, 1, D, 0); }
    if (pre_scalar) sublayer_extras(L, p, 0);
    // one mixer: its projection columns start at column cb of the layer's projection output; `shared`: the projection matrix of
    // the layer's mixers is one allocation (w_shared) and this mixer's rows follow the first mixer's
    auto layout_mixer = [&](LmLayer& L, const std::string& mp, int cb, bool shared, size_t w_shared) -> int {
    const xotb200_lm_layer& s = L.s;
    REQUIRE(!shared || (s.mixer != XOTB200_LM_MIX_LATENT_ATTN && s.mixer != XOTB200_LM_MIX_DELTA_RULE), "layer %d: this mixer kind cannot share a layer", li);
    if (s.mixer == XOTB200_LM_MIX_LATENT_ATTN) {
      const int H = s.heads, dn = s.dim, dr = s.rot_dim, dv = s.vdim, R = s.kv_rank, HQ = H * (dn + dr);
      REQUIRE(R >= 1 && R <= 512, "layer %d: kv_rank %d outside 1..512", li, R);
      REQUIRE(dv >= 1 && dr >= 0 && s.rot_dims <= dr && s.rot_dims % 2 == 0 && s.rot_dims >= 0, "layer %d: bad rotation sizes", li);
      REQUIRE(s.rot_layout == XOTB200_LM_ROT_INTERLEAVED || s.rot_layout == XOTB200_LM_ROT_HALF, "layer %d: unknown rotation layout %d", li, s.rot_layout);
      REQUIRE(s.window >= 0, "layer %d: negative window", li);
      const int nq = s.q_rank > 0 ? s.q_rank : HQ;
      L.c_q = 0; L.c_kv = nq; L.c_g = nq + R + dr;
      L.n_in = nq + R + dr + (s.out_gate ? H : 0);
      L.w_in = shared ? w_shared : take((size_t)L.n_in * D);
      if (s.q_rank > 0) {
        dest(mp + "dq", L.w_in, s.q_rank, D, 0);
        L.dq_norm = take(s.q_rank); dest(mp + "dq.norm", L.dq_norm, 1, s.q_rank, 0);
        L.uq = take((size_t)HQ * s.q_rank); dest(mp + "uq", L.uq, HQ, s.q_rank, 0);
      } else {
        dest(mp + "q", L.w_in, HQ, D, 0);
      }
      dest(mp + "dkv", L.w_in, R + dr, D, L.c_kv);
      if (s.out_gate) dest(mp + "g", L.w_in, H, D, L.c_g);
      L.dkv_norm = take(R); dest(mp + "dkv.norm", L.dkv_norm, 1, R, 0);
      // W_uk is kept per head as [R, dn]: the absorption product q~ = W_uk[h]^T q then reads it K-major like every other weight
      L.uk = take((size_t)H * dn * R); dest(mp + "uk", L.uk, H * dn, R, 0); e->dests[mp + "uk"].tr_heads = H;
      L.uk_rows = take((size_t)H * dn * R); e->dests[mp + "uk"].has2 = true; e->dests[mp + "uk"].elem_off2 = L.uk_rows;
      L.uv = take((size_t)H * dv * R); dest(mp + "uv", L.uv, H * dv, R, 0);
      L.wo = take((size_t)D * H * dv); dest(mp + "o", L.wo, D, H * dv, 0);
      e->max_q = std::max(e->max_q, HQ);
      e->max_qfull = std::max(e->max_qfull, H * (R + dr));
      e->max_qr = std::max(e->max_qr, s.q_rank);
      e->max_hdn = std::max(e->max_hdn, H * dn);
      e->max_olat = std::max(e->max_olat, H * R);
      e->max_oh = std::max(e->max_oh, H * dv);
      e->max_w = std::max(e->max_w, R + dr);
      // the expanded prompt attention holds dv <= 128 value columns per warp row and 256 query/key entries per tile row; a model with
      // a wider layer keeps ALL its attention on the absorbed kernel (the split into few-row and many-row requests is per step)
      if (dv > 128 || ((dn + dr + 15) & ~15) > 256) e->flash_fits = false;
    } else if (s.mixer == XOTB200_LM_MIX_DELTA_RULE) {
      const int HD = s.heads * s.dim;
      REQUIRE(s.vdim == s.dim, "layer %d: the delta rule uses one size for keys and values", li);
      REQUIRE(s.dim <= 256, "layer %d: delta-rule head size %d above 256", li, s.dim);
      REQUIRE(s.low_rank >= 1, "layer %d: the decay branch needs an inner size", li);
      L.c_r = 0; L.c_k = HD; L.c_v = 2 * HD; L.c_g = 3 * HD; L.c_a = 4 * HD; L.c_w1 = 5 * HD;
      L.n_in = 5 * HD + s.low_rank;
      L.w_in = shared ? w_shared : take((size_t)L.n_in * D);
      dest(mp + "r", L.w_in, HD, D, L.c_r);
      dest(mp + "k", L.w_in, HD, D, L.c_k);
      dest(mp + "v", L.w_in, HD, D, L.c_v);
      dest(mp + "g", L.w_in, HD, D, L.c_g);
      dest(mp + "a", L.w_in, HD, D, L.c_a);
      dest(mp + "w1", L.w_in, s.low_rank, D, L.c_w1);
      L.w2 = take((size_t)HD * s.low_rank); dest(mp + "w2", L.w2, HD, s.low_rank, 0);
      L.w0 = take(HD); dest(mp + "w0", L.w0, 1, HD, 0);
      L.a_b = take(HD); dest(mp + "a.b", L.a_b, 1, HD, 0);
      L.onorm = take(HD); dest(mp + "norm", L.onorm, 1, HD, 0);
      L.wo = take((size_t)D * HD); dest(mp + "o", L.wo, D, HD, 0);
      L.state_off = e->state_floats;
      e->state_floats += (size_t)s.heads * s.dim * s.dim;
      e->max_hd = std::max(e->max_hd, HD);
      e->max_lr = std::max(e->max_lr, s.low_rank);
      e->max_oh = std::max(e->max_oh, HD);
    } else if (s.mixer == XOTB200_LM_MIX_ATTENTION) {
      const int H = s.heads, G = s.kv_heads, dk = s.dim, dv = s.vdim;
      const bool own = s.kv_from < 0;
      REQUIRE(G >= 1 && H % G == 0, "layer %d: %d query heads do not divide into %d key/value heads", li, H, G);
      REQUIRE(dv >= 1 && dv <= 512 && dk <= 1024, "layer %d: attention sizes dim %d (<= 1024) / vdim %d (1..512)", li, dk, dv);
      REQUIRE(s.window >= 0 && s.chunk >= 0 && s.softcap >= 0.f, "layer %d: negative window, chunk or softcap", li);
      REQUIRE(s.out_gate >= 0 && s.out_gate <= 2, "layer %d: unknown output gate %d", li, s.out_gate);
      REQUIRE(s.qk_norm >= XOTB200_LM_QKNORM_NONE && s.qk_norm <= XOTB200_LM_QKNORM_HEAD_PLAIN, "layer %d: unknown query/key norm %d", li, s.qk_norm);
      REQUIRE(s.rot_dims >= 0 && s.rot_dims <= dk && s.rot_dims % 2 == 0, "layer %d: %d rotated entries of a head of %d", li, s.rot_dims, dk);
      REQUIRE(s.rot_dims == 0 || (s.rot_base > 0.f && (s.rot_layout == XOTB200_LM_ROT_INTERLEAVED || s.rot_layout == XOTB200_LM_ROT_HALF)),
              "layer %d: rotation needs a positive base and a known layout", li);
      REQUIRE(s.rot_dims == 0 || s.qk_norm != XOTB200_LM_QKNORM_ROW, "layer %d: rotation is implemented with per-head query/key norms (or none)", li);
      REQUIRE(s.rot_scale_factor == 0.f || (s.rot_scale_factor > 0.f && s.rot_scale_high > s.rot_scale_low && s.rot_scale_low > 0.f && s.rot_scale_original > 0.f),
              "layer %d: frequency scaling needs factor > 0, 0 < low < high and the original length", li);
      REQUIRE(s.keep_first >= 0 && s.pool >= 0 && !(s.keep_first > 0 && s.pool > 0), "layer %d: kept first tokens and pooled blocks exclude each other", li);
      REQUIRE((s.keep_first == 0 && s.pool == 0) || (s.window > 0 && s.chunk == 0 && !s.dist_bias && s.rel_buckets == 0 && own),
              "layer %d: kept first tokens / pooled blocks go with a sliding window, keys of the layer's own and no block mask or distance terms", li);
      REQUIRE(!s.out_bias || post_ln || post_rms, "layer %d: a bias of the output projection is added by the closing norm of the post-norm block forms only", li);
      REQUIRE(s.qk_norm != XOTB200_LM_QKNORM_ROW || (size_t)(H + G) * dk * 4 <= 200 * 1024,
              "layer %d: a query/key norm over the whole projection holds the row in shared memory: (heads + kv_heads) * dim <= 51200", li);
      REQUIRE(s.q_temp_coef == 0.f || s.q_temp_every >= 1, "layer %d: query temperature every %d positions", li, s.q_temp_every);
      REQUIRE(s.rel_buckets == 0 || (s.rel_buckets >= 2 && s.rel_buckets <= 65536 && s.rel_max > (float)(s.rel_buckets / 2) && s.rel_max <= 4194304.f),
              "layer %d: %d distance buckets up to distance %g (2..65536 buckets, the largest distance above half their number and <= 4194304)", li,
              s.rel_buckets, (double)s.rel_max);
      if (!own) {
        REQUIRE(s.kv_from >= e->cfg.start_layer && s.kv_from < li, "layer %d reads the keys/values of layer %d, which is not an earlier layer of this shard", li,
                s.kv_from);
        const xotb200_lm_layer& o = all[s.kv_from];
        REQUIRE(o.mixer == XOTB200_LM_MIX_ATTENTION && o.kv_from < 0 && o.kv_heads == G && o.dim == dk && o.vdim == dv,
                "layer %d: layer %d does not hold keys/values of its shape", li, s.kv_from);
        L.kv_src = s.kv_from - e->cfg.start_layer;
      } else {
        L.kv_src = li - e->cfg.start_layer;
      }
      // projection columns: q | k | v | gate   (k, v only with keys/values of its own)
      L.c_q = cb; L.c_kk = cb + H * dk; L.c_vv = L.c_kk + (own ? G * dk : 0); L.c_g = L.c_vv + (own ? G * dv : 0);
      const int ng = s.out_gate == 2 ? H * dv : s.out_gate == 1 ? H : 0;
      L.n_in = L.c_g + ng - cb;
      L.w_in = shared ? w_shared : take((size_t)L.n_in * D);
      dest(mp + "q", L.w_in, H * dk, D, L.c_q);
      if (own) { dest(mp + "k", L.w_in, G * dk, D, L.c_kk); dest(mp + "v", L.w_in, G * dv, D, L.c_vv); }
      if (ng) dest(mp + "g", L.w_in, ng, D, L.c_g);
      if (s.proj_bias) {
        L.b_in = take(cb + L.n_in);                            // zero where a projection has no bias (the blob starts zeroed)
        dest(mp + "q.b", L.b_in + L.c_q, 1, H * dk, 0);
        if (own) { dest(mp + "k.b", L.b_in + L.c_kk, 1, G * dk, 0); dest(mp + "v.b", L.b_in + L.c_vv, 1, G * dv, 0); }
      }
      if (s.qk_norm && s.qk_norm != XOTB200_LM_QKNORM_HEAD_PLAIN) {
        const bool whole = s.qk_norm == XOTB200_LM_QKNORM_ROW;
        const int nq = whole ? H * dk : dk, nk = whole ? G * dk : dk;
        L.q_norm = take(nq); dest(mp + "q.norm", L.q_norm, 1, nq, 0);
        if (own) { L.k_norm = take(nk); dest(mp + "k.norm", L.k_norm, 1, nk, 0); }
      }
      if (s.out_bias) { L.o_b = take(D); dest(mp + "o.b", L.o_b, 1, D, 0); }
      if (s.sink) { L.sink = take(H); dest(mp + "sink", L.sink, 1, H, 0); }
      if (s.rel_buckets > 0) { L.rel = take((size_t)s.rel_buckets * H); dest(mp + "rel", L.rel, s.rel_buckets, H, 0); }
      if (s.dist_bias) {
        L.r1 = take(H); dest(mp + "r1", L.r1, 1, H, 0);
        L.r2 = take(H); dest(mp + "r2", L.r2, 1, H, 0);
      }
      L.wo = take((size_t)D * H * dv); dest(mp + "o", L.wo, D, H * dv, 0);
      e->max_q = std::max(e->max_q, H * dk);
      e->max_qfull = std::max(e->max_qfull, H * dk);
      e->max_oh = std::max(e->max_oh, H * dv);
      if (dk % 8 || dv % 8 || dk > 256 || dv > 128) e->gqa_flash_fits = false;
    } else if (s.mixer == XOTB200_LM_MIX_GATED_DELTA) {
      const int H = s.heads, G = s.kv_heads, dk = s.dim, dv = s.vdim, C = 2 * G * dk + H * dv;
      REQUIRE(G >= 1 && H % G == 0, "layer %d: %d value heads do not divide into %d query/key heads", li, H, G);
      REQUIRE(dk <= 256 && dv >= 1 && dv <= 256, "layer %d: delta-rule head sizes %d / %d above 256", li, dk, dv);
      REQUIRE(s.conv_taps >= 1 && s.conv_taps <= 64, "layer %d: %d convolution taps (1..64)", li, s.conv_taps);
      // projection columns: q | k | v (the filtered channels, in this order) | output gate | beta | decay logit
      L.c_r = cb; L.c_k = cb + G * dk; L.c_v = cb + 2 * G * dk; L.c_g = cb + C; L.c_b = L.c_g + H * dv; L.c_a = L.c_b + H;
      L.conv_ch = C;
      L.n_in = L.c_a + H - cb;
      L.w_in = shared ? w_shared : take((size_t)L.n_in * D);
      dest(mp + "q", L.w_in, G * dk, D, L.c_r);
      dest(mp + "k", L.w_in, G * dk, D, L.c_k);
      dest(mp + "v", L.w_in, H * dv, D, L.c_v);
      dest(mp + "g", L.w_in, H * dv, D, L.c_g);
      dest(mp + "b", L.w_in, H, D, L.c_b);
      dest(mp + "a", L.w_in, H, D, L.c_a);
      L.conv_w = take((size_t)C * s.conv_taps);
      dest(mp + "q.conv", L.conv_w, G * dk, s.conv_taps, 0);
      dest(mp + "k.conv", L.conv_w, G * dk, s.conv_taps, G * dk);
      dest(mp + "v.conv", L.conv_w, H * dv, s.conv_taps, 2 * G * dk);
      L.a_log = take(H); dest(mp + "A_log", L.a_log, 1, H, 0);
      L.dt_bias = take(H); dest(mp + "dt_bias", L.dt_bias, 1, H, 0);
      L.onorm = take(dv); dest(mp + "norm", L.onorm, 1, dv, 0);
      L.wo = take((size_t)D * H * dv); dest(mp + "o", L.wo, D, H * dv, 0);
      L.state_off = e->state_floats;
      e->state_floats += (size_t)H * dk * dv;
      L.conv_off = e->state_floats;
      e->state_floats += (size_t)(s.conv_taps - 1) * C;
      e->max_hd = std::max(e->max_hd, H * std::max(dk, dv));
      e->max_oh = std::max(e->max_oh, H * dv);
      e->max_conv = std::max(e->max_conv, C);
    } else if (s.mixer == XOTB200_LM_MIX_MATRIX_LSTM) {
      const int H = s.heads, dk = s.dim, dv = s.vdim;
      REQUIRE(dk <= 256 && dv >= 1 && dv <= 256, "layer %d: matrix-LSTM head sizes %d / %d above 256", li, dk, dv);
      REQUIRE(s.gate_cap > 0.f, "layer %d: the gates' cap must be positive", li);
      // projection columns: q | k | v | output gate | input-gate logits | forget-gate logits
      L.c_r = cb; L.c_k = cb + H * dk; L.c_v = cb + 2 * H * dk; L.c_g = L.c_v + H * dv; L.c_i = L.c_g + H * dv; L.c_f = L.c_i + H;
      L.n_in = L.c_f + H - cb;
      L.w_in = shared ? w_shared : take((size_t)L.n_in * D);
      dest(mp + "q", L.w_in, H * dk, D, L.c_r);
      dest(mp + "k", L.w_in, H * dk, D, L.c_k);
      dest(mp + "v", L.w_in, H * dv, D, L.c_v);
      dest(mp + "g", L.w_in, H * dv, D, L.c_g);
      dest(mp + "i", L.w_in, H, D, L.c_i);
      dest(mp + "f", L.w_in, H, D, L.c_f);
      L.i_b = take(H); dest(mp + "i.b", L.i_b, 1, H, 0);
      L.f_b = take(H); dest(mp + "f.b", L.f_b, 1, H, 0);
      L.onorm = take((size_t)H * dv); dest(mp + "norm", L.onorm, 1, H * dv, 0);
      L.wo = take((size_t)D * H * dv); dest(mp + "o", L.wo, D, H * dv, 0);
      L.state_off = e->state_floats;                       // per head the matrix [dk, dv], then the normalisers [H, dk], then the maxima [H]
      e->state_floats += (size_t)H * dk * dv;
      L.n_off = e->state_floats;
      e->state_floats += (size_t)H * dk;
      L.m_off = e->state_floats;
      e->state_floats += (size_t)H;
      e->max_hd = std::max(e->max_hd, H * std::max(dk, dv));
      e->max_oh = std::max(e->max_oh, H * dv);
      e->max_heads_rec = std::max(e->max_heads_rec, H);
    } else if (s.mixer == XOTB200_LM_MIX_MAMBA2) {
      const int H = s.heads, G = s.kv_heads, N = s.dim, dv = s.vdim, inner = H * dv, C = inner + 2 * G * N;
      REQUIRE(G >= 1 && H % G == 0, "layer %d: %d heads do not divide into %d groups", li, H, G);
      REQUIRE(N <= 256 && dv >= 1 && dv <= 256, "layer %d: state size %d / head size %d above 256", li, N, dv);
      REQUIRE(s.conv_taps >= 1 && s.conv_taps <= 64, "layer %d: %d convolution taps (1..64)", li, s.conv_taps);
      REQUIRE(s.out_norm_groups >= 1 && inner % s.out_norm_groups == 0, "layer %d: %d channels do not divide into %d norm parts", li, inner, s.out_norm_groups);
      // projection columns as stored: z | x | B | C (x, B, C are the filtered channels) | dt
      L.c_z = cb; L.c_v = cb + inner; L.c_k = L.c_v + inner; L.c_r = L.c_k + G * N; L.c_dt = L.c_r + G * N;
      L.conv_ch = C;
      L.n_in = L.c_dt + H - cb;
      L.w_in = shared ? w_shared : take((size_t)L.n_in * D);
      dest(mp + "in", L.w_in, L.n_in, D, cb);
      L.conv_w = take((size_t)C * s.conv_taps); dest(mp + "conv", L.conv_w, C, s.conv_taps, 0);
      L.conv_b = take(C); dest(mp + "conv.b", L.conv_b, 1, C, 0);
      L.dt_bias = take(H); dest(mp + "dt_bias", L.dt_bias, 1, H, 0);
      L.a_log = take(H); dest(mp + "A_log", L.a_log, 1, H, 0);
      L.d_skip = take(H); dest(mp + "D", L.d_skip, 1, H, 0);
      L.onorm = take(inner); dest(mp + "norm", L.onorm, 1, inner, 0);
      L.wo = take((size_t)D * inner); dest(mp + "o", L.wo, D, inner, 0);
      L.state_off = e->state_floats;
      e->state_floats += (size_t)H * N * dv;
      L.conv_off = e->state_floats;
      e->state_floats += (size_t)(s.conv_taps - 1) * C;
      e->max_hd = std::max(e->max_hd, H * std::max(N, dv));
      e->max_oh = std::max(e->max_oh, inner);
      e->max_conv = std::max(e->max_conv, C);
    } else {
      REQUIRE(false, "layer %d: unknown mixer kind %d", li, s.mixer);
    }
    return 0;
    };
    if (s.par_on) {
      REQUIRE(pre_scalar, "layer %d: a second mixer in a layer goes with the pre-norm block form with one-number weights", li);
      REQUIRE(s.mixer == XOTB200_LM_MIX_ATTENTION || s.mixer == XOTB200_LM_MIX_GATED_DELTA || s.mixer == XOTB200_LM_MIX_MATRIX_LSTM || s.mixer == XOTB200_LM_MIX_MAMBA2,
              "layer %d: mixer kind %d cannot share a layer", li, s.mixer);
      REQUIRE(s.par_mixer == XOTB200_LM_MIX_GATED_DELTA || s.par_mixer == XOTB200_LM_MIX_MATRIX_LSTM || s.par_mixer == XOTB200_LM_MIX_MAMBA2,
              "layer %d: the second mixer of a layer is a recurrent one (gated delta rule, matrix LSTM, state-space), not kind %d", li, s.par_mixer);
      LmLayer R{};
      R.s = xotb200_lm_layer{};
      R.s.mixer = s.par_mixer; R.s.heads = s.par_heads; R.s.kv_heads = s.par_kv_heads; R.s.dim = s.par_dim; R.s.vdim = s.par_vdim;
      R.s.conv_taps = s.par_conv_taps; R.s.out_norm_groups = s.par_out_norm_groups; R.s.gate_cap = s.par_gate_cap; R.s.kv_from = -1;
      REQUIRE(R.s.heads >= 1 && R.s.dim >= 1, "layer %d: heads and dim of the second mixer must be positive", li);
      const int n_left = mixer_columns(s), n_right = mixer_columns(R.s);
      const size_t w_all = take((size_t)(n_left + n_right) * D);   // the rows of both mixers' projections: one product
      TRY(layout_mixer(L, p + "mix.left.", 0, true, w_all));
      TRY(layout_mixer(R, p + "mix.right.", n_left, true, w_all));
      REQUIRE(L.n_in == n_left && R.n_in == n_right, "internal: projection columns of layer %d", li);
      L.ld_in = R.ld_in = n_left + n_right;
      L.par.push_back(R);
    } else {
      TRY(layout_mixer(L, p + "mix.", 0, false, 0));
      L.ld_in = L.n_in;
    }
    e->max_in = std::max(e->max_in, L.ld_in);
    const bool has_ff = s.ff_kind == XOTB200_LM_FF_MOE ? s.experts > 0 : s.ff > 0;
    if (has_ff) {
      L.norm2 = take(NW); dest(p + "norm2", L.norm2, 1, NW, 0);
      if (!post_rms && !pre_scalar) { L.norm2b = take(D); dest(p + "norm2" + nb, L.norm2b, 1, D, 0); }
      if (pre_scalar) sublayer_extras(L, p, 1);
    }
    if (s.ff_kind == XOTB200_LM_FF_MOE && has_ff) {
      const int E = s.experts, F = s.expert_ff;
      REQUIRE(F >= 1 && s.top >= 1 && s.top <= E && E <= 4096, "layer %d: %d experts of size %d, %d per token", li, E, F, s.top);
      if (s.groups > 1)
        REQUIRE(E % s.groups == 0 && s.groups_keep >= 1 && s.groups_keep <= s.groups && s.groups_keep * (E / s.groups) >= s.top,
                "layer %d: %d experts in %d groups of which %d are kept cannot give %d experts per token", li, E, s.groups, s.groups_keep, s.top);
      REQUIRE(s.expert_act == XOTB200_LM_EXPERT_SILU_GATED || s.expert_act == XOTB200_LM_EXPERT_RELU2, "layer %d: unknown expert form %d", li, s.expert_act);
      REQUIRE(s.router_kind == XOTB200_LM_ROUTER_SOFTMAX_ALL || s.router_kind == XOTB200_LM_ROUTER_TOPK_SOFTMAX, "layer %d: unknown routing rule %d", li, s.router_kind);
      REQUIRE(s.shared_ff >= 0, "layer %d: negative size of the shared expert", li);
      const bool gated = s.expert_act == XOTB200_LM_EXPERT_SILU_GATED;
      L.router = take((size_t)E * D); dest(p + "mlp.router", L.router, E, D, 0);
      if (s.router_bias) { L.router_b = take(E); dest(p + "mlp.router.b", L.router_b, 1, E, 0); }
      L.w_gu = take((size_t)E * (gated ? 2 : 1) * F * D);
      L.w_edown = take((size_t)E * D * F);
      for (int x = 0; x < E; ++x) {
        const std::string ep = p + "mlp.e" + std::to_string(x) + ".";
        if (gated) {
          dest(ep + "gate", L.w_gu, F, D, x * 2 * F);
          dest(ep + "up", L.w_gu, F, D, x * 2 * F + (F % 8 ? F : 0));
          if (F % 8 == 0) { e->dests[ep + "gate"].il8 = 0; e->dests[ep + "up"].il8 = 1; }   // gate and up rows interleaved in eights
        } else {
          dest(ep + "up", L.w_gu, F, D, x * F);
        }
        dest(ep + "down", L.w_edown, D, F, x * D);
      }
      if (s.shared_ff > 0) {
        REQUIRE(!gated, "layer %d: a shared expert is implemented for relu^2 experts only", li);
        L.up = take((size_t)s.shared_ff * D); dest(p + "mlp.shared.up", L.up, s.shared_ff, D, 0);
        L.down = take((size_t)D * s.shared_ff); dest(p + "mlp.shared.down", L.down, D, s.shared_ff, 0);
        e->max_ff = std::max(e->max_ff, s.shared_ff);
      }
      e->max_top = std::max(e->max_top, s.top);
      e->max_eff = std::max(e->max_eff, F);
      e->max_experts = std::max(e->max_experts, E);
    } else if (has_ff) {
      REQUIRE(s.ff_kind == XOTB200_LM_FF_RELU2 || s.ff_kind == XOTB200_LM_FF_XIELU || s.ff_kind == XOTB200_LM_FF_GELU, "layer %d: unknown feed-forward kind %d", li,
              s.ff_kind);
      L.up = take((size_t)s.ff * D); dest(p + "mlp.up", L.up, s.ff, D, 0);
      L.down = take((size_t)D * s.ff); dest(p + "mlp.down", L.down, D, s.ff, 0);
      if (s.ff_kind == XOTB200_LM_FF_XIELU) { L.act_p = take(2); dest(p + "mlp.act", L.act_p, 1, 2, 0); }
      e->max_ff = std::max(e->max_ff, s.ff);
    }
    e->layers.push_back(L);
  }
  if (e->last) {
    e->final_norm = take(NW); dest("final.norm", e->final_norm, 1, NW, 0);
    if (post_ln) { e->final_norm_b = take(D); dest("final.norm.b", e->final_norm_b, 1, D, 0); }   // a final RMS norm has a weight only
    e->head = take((size_t)V * D); dest("head", e->head, V, D, 0);
  }
  e->blob_elems = cur;
  return 0;
}

static int upload_tensor(xotb200_lm* e, Dest& d, const void* host_bf16) {
  const size_t n = (size_t)d.rows * d.cols;
  bf16* tmp = nullptr;
  CK(cudaMalloc(&tmp, n * 2));
  cudaError_t er = cudaMemcpyAsync(tmp, host_bf16, n * 2, cudaMemcpyHostToDevice, e->stream);
  if (er == cudaSuccess) {
    const int grid = (int)std::min<size_t>(4096, (n + 255) / 256);
    const size_t off = d.elem_off + (size_t)d.row_off * d.cols;
    if (d.tr_heads > 0) {
      const int dh = d.rows / d.tr_heads;
      if (e->esz == 2) store_heads_transposed_kernel<bf16><<<grid, 256, 0, e->stream>>>(tmp, at<bf16>(e, off), d.tr_heads, dh, d.cols);
      else store_heads_transposed_kernel<float><<<grid, 256, 0, e->stream>>>(tmp, at<float>(e, off), d.tr_heads, dh, d.cols);
    } else if (d.il8 >= 0) {
      if (e->esz == 2) store_rows_interleaved8_kernel<bf16><<<grid, 256, 0, e->stream>>>(tmp, at<bf16>(e, off), d.rows, d.cols, d.il8);
      else store_rows_interleaved8_kernel<float><<<grid, 256, 0, e->stream>>>(tmp, at<float>(e, off), d.rows, d.cols, d.il8);
    } else if (e->esz == 2) store_rows_kernel<bf16><<<grid, 256, 0, e->stream>>>(tmp, at<bf16>(e, off), n);
    else store_rows_kernel<float><<<grid, 256, 0, e->stream>>>(tmp, at<float>(e, off), n);
    if (d.has2) {
      if (e->esz == 2) store_rows_kernel<bf16><<<grid, 256, 0, e->stream>>>(tmp, at<bf16>(e, d.elem_off2), n);
      else store_rows_kernel<float><<<grid, 256, 0, e->stream>>>(tmp, at<float>(e, d.elem_off2), n);
      e->launches++;
    }
    er = cudaGetLastError();
    e->launches++;
  }
  cudaError_t er2 = cudaStreamSynchronize(e->stream);
  cudaFree(tmp);
  CK(er);
  CK(er2);
  d.loaded = true;
  e->tables_stale = true;
  return 0;
}

// does a tensor name belong to this shard? (so that an unknown name there is an error, and anything else is skipped)
static bool owned_name(const xotb200_lm* e, const std::string& name) {
  if (name == "embed" || name == "pos" || name == "embed.norm") return e->first;
  if (name == "head" || name == "final.norm" || name == "final.norm.b") return e->last;
  if (name.size() > 1 && name[0] == 'l' && isdigit((unsigned char)name[1])) {
    const int li = atoi(name.c_str() + 1);
    return li >= e->cfg.start_layer && li <= e->cfg.end_layer;
  }
  return true;   // not a name of this model family at all: strict
}

// ---------------------------------------------------------------------------------------------------------------------------
// products
// ---------------------------------------------------------------------------------------------------------------------------
static const size_t GEMV_SMEM_MAX = 160 * 1024;
// Rows up to which 16-bit products run on the one-warp-per-row-group kernel.  Beyond two rows its fp32 FMAs (8 per weight at 8
// rows) fall behind the weight stream, and the tensor-core tiles — mostly empty, but they read each weight once — are faster.
static const int GEMV_MAX_ROWS = 2;

template <typename K>
static int opt_in_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) CK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return 0;
}

// ---- tensor-core path of the bf16 products (layered_tc.cuh) ---------------------------------------------------------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_tiled_fn get_encode_tiled() {
  static encode_tiled_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_fn>(p);
  }
  return fn;
}
// bf16 matrix [batch][rows, K] with row stride ld and batch stride bs (elements) as a 3-D map {K, rows, batch}, box {64, box_rows, 1},
// 128-byte swizzle, zero fill outside.  False when the operand cannot be described (alignment) — the caller then uses the FMA tiles.
static bool make_map3(CUtensorMap* m, const void* ptr, long rows, long K, long ld, long bs, int batch, int box_rows) {
  encode_tiled_fn enc = get_encode_tiled();
  if (!enc || (reinterpret_cast<uintptr_t>(ptr) & 15) || ld % 8 || (batch > 1 && bs % 8) || K < 1 || rows < 1) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? bs : ld * rows) * 2};
  const cuuint32_t box[3] = {(cuuint32_t)LTC_BK, (cuuint32_t)box_rows, 1};
  const cuuint32_t es[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT, int EPI, typename TC>
static int launch_ltc(xotb200_lm* e, const CUtensorMap& ma, const CUtensorMap& mb, const LtcArgs& a, int batch) {
  constexpr int NS = 3;
  auto kern = ltc_gemm_kernel<NT, EPI, NS, TC>;
  CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ltc_smem_bytes(NT, NS)));
  const dim3 grid = a.cols_first ? dim3(cdiv(a.N, NT), cdiv(a.M, LTC_M), batch) : dim3(cdiv(a.M, LTC_M), cdiv(a.N, NT), batch);
  kern<<<grid, LTC_THREADS, ltc_smem_bytes(NT, NS), e->stream>>>(ma, mb, a);
  CK(cudaGetLastError());
  e->launches++;
  e->tc_launches++;
  return 0;
}

// 1 = launched, 0 = not eligible (the caller falls back), < 0 = error
template <typename TC, int EPI>
static int product_tc(xotb200_lm* e, const bf16* A, long lda, long a_batch, const bf16* B, long ldb, long b_batch, TC* C, long ldc, long c_batch, int M,
                      int N, int K, int batch, const void* epi) {
  const int nt = (N > 64 && M > LTC_M) ? 128 : 64;   // one row tile: narrower column tiles, twice the CTAs streaming weights
  CUtensorMap ma, mb;
  if (!make_map3(&ma, A, M, K, lda, a_batch, batch, LTC_M) || !make_map3(&mb, B, N, K, ldb, b_batch, batch, nt)) return 0;
  LtcArgs a{M, N, K, C, ldc, c_batch, e->d_err, static_cast<const bf16*>(epi), nullptr, 0};
  if (nt == 128) TRY((launch_ltc<128, EPI, TC>(e, ma, mb, a, batch)));
  else TRY((launch_ltc<64, EPI, TC>(e, ma, mb, a, batch)));
  return 1;
}

template <typename TA, typename TB, typename TC, int EPI>
static int product(xotb200_lm* e, const TA* A, long lda, long a_batch, const TB* B, long sbn, long sbk, long b_batch, TC* C, long ldc, long c_batch,
                   int M, int N, int K, int batch, const void* epi = nullptr) {
  if (M == 0 || N == 0) return 0;
  const size_t smem = (size_t)M * K * 4;
  if constexpr (std::is_same<TA, bf16>::value && std::is_same<TB, bf16>::value && (EPI == 0 || !std::is_same<TC, float>::value)) {
    // 16-bit operands with more rows than the decode kernel takes: the tensor cores, when the operands can be described to TMA
    if (sbk == 1 && ((e->gemm_mode == 0 && M > GEMV_MAX_ROWS) || e->gemm_mode == 2)) {
      const int r = product_tc<TC, EPI>(e, A, lda, a_batch, B, sbn, b_batch, C, ldc, c_batch, M, N, K, batch, epi);
      if (r != 0) return r < 0 ? r : 0;
    }
  }
  if (e->gemm_mode == 0 && M <= 8 && sbk == 1 && smem <= GEMV_SMEM_MAX) {
    // warps per row group: enough K per warp to keep its lanes busy, more slices when there are few rows
    int wsplit = 1;
    while (wsplit < 8 && K / (wsplit * 2) >= 256 && (long)cdiv(N, 4 * (8 / wsplit)) * batch < 4L * e->sm_count) wsplit *= 2;
    const int blocks = std::max(1, std::min(cdiv(N, 4 * (8 / wsplit)), e->sm_count * 8 / std::max(1, batch)));
    const size_t sm = smem + 8 * 4 * 8 * 4;
#define LAUNCH_GEMV(MR)                                                                                                        \
  do {                                                                                                                         \
    auto kern = gemv_rows_kernel<TA, TB, TC, EPI, MR>;                                                                         \
    TRY(opt_in_smem(kern, sm));                                                                                                \
    kern<<<dim3(blocks, 1, batch), 256, sm, e->stream>>>(A, lda, a_batch, B, sbn, b_batch, C, ldc, c_batch, M, N, K, wsplit,    \
                                                         static_cast<const TB*>(epi));                                        \
  } while (0)
    if (M == 1) LAUNCH_GEMV(1);
    else if (M == 2) LAUNCH_GEMV(2);
    else if (M <= 4) LAUNCH_GEMV(4);
    else LAUNCH_GEMV(8);
#undef LAUNCH_GEMV
  } else {
    gemm_tiled_kernel<TA, TB, TC, EPI><<<dim3(cdiv(N, 64), cdiv(M, 64), batch), 256, 0, e->stream>>>(A, lda, a_batch, B, sbn, sbk, b_batch, C, ldc,
                                                                                                  c_batch, M, N, K, static_cast<const TB*>(epi));
  }
  CK(cudaGetLastError());
  e->launches++;
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------------
// scratch
// ---------------------------------------------------------------------------------------------------------------------------
template <typename P> static int regrow(P*& p, size_t bytes) {
  if (p) { cudaFree(p); p = nullptr; }
  if (bytes == 0) return 0;
  CK(cudaMalloc(&p, bytes));
  return 0;
}

// captured decode steps hold device pointers: whenever a buffer they name is replaced they are dropped
static void drop_graphs(xotb200_lm* e) {
  for (auto& kv : e->graphs)
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
  e->graphs.clear();
}

static int ensure_scratch(xotb200_lm* e, int M, int n_want) {
  const int D = e->cfg.width;
  if (M > e->m_cap) {
    drop_graphs(e);
    const size_t m = (size_t)std::max(M, 64), z = e->esz;
    TRY(regrow(e->x, m * D * 4 * (e->pre_scalar ? std::max(1, e->cfg.streams) : 1)));
    TRY(regrow(e->y, m * D * 4));
    if (e->pre_scalar) {
      TRY(regrow(e->y2, m * D * 4));
      TRY(regrow(e->h0, m * D * 4));
    }
    if (e->max_heads_rec) {
      TRY(regrow(e->gdec, m * e->max_heads_rec * 4));
      TRY(regrow(e->ginw, m * e->max_heads_rec * 4));
      TRY(regrow(e->gfloor, m * e->max_heads_rec * 4));
      TRY(regrow(e->gnq, m * e->max_heads_rec * 4));
    }
    TRY(regrow(e->proj, m * e->max_in * 4));
    TRY(regrow(e->qraw, m * e->max_q * 4));
    TRY(regrow(e->qfull, m * e->max_qfull * 4));
    TRY(regrow(e->wlog, m * e->max_hd * 4));
    TRY(regrow(e->oraw, m * e->max_hd * 4));
    TRY(regrow(e->du, m * e->max_hd * 4));
    TRY(regrow(e->dau, m * e->max_hd * 4));
    if (e->max_conv || e->max_heads_rec) {
      TRY(regrow(e->dkk, m * e->max_hd * 4));
      TRY(regrow(e->drr, m * e->max_hd * 4));
      TRY(regrow(e->cvb, m * std::max(1, e->max_conv) * 4));
    }
    if (e->max_top) {
      TRY(regrow(e->moe_ids, m * e->max_top * 4));
      TRY(regrow(e->moe_wts, m * e->max_top * 4));
      // the grouped form pads every expert's run to whole 128-row tiles
      const size_t tiles = (m * e->max_top + LTC_M - 1) / LTC_M + e->max_experts, pairs_pad = tiles * LTC_M;
      TRY(regrow(e->mact, pairs_pad * e->max_eff * z));
      if (z == 2) {
        TRY(regrow(e->moe_xg, pairs_pad * D * 2));
        TRY(regrow(e->moe_yg, pairs_pad * D * 4));
        const size_t ints = 3 * (size_t)e->max_experts + 1 + m * e->max_top + tiles;
        TRY(regrow(e->moe_plan, ints * 4));
        CK(cudaMemsetAsync(e->moe_plan, 0, ints * 4, e->stream));
        e->moe_tiles_cap = (int)tiles;
      }
    }
    TRY(regrow(e->h, m * D * z));
    TRY(regrow(e->cqn, m * e->max_qr * z));
    TRY(regrow(e->qn, m * e->max_hdn * z));
    if (z == 2) TRY(regrow(e->q16, m * e->max_q * 2));
    TRY(regrow(e->olat, m * e->max_olat * z));
    TRY(regrow(e->oh, m * e->max_oh * z));
    if (e->pre_scalar) TRY(regrow(e->oh2, m * e->max_oh * z));
    TRY(regrow(e->act, m * e->max_ff * z));
    TRY(regrow(e->th, m * e->max_lr * z));
    e->m_cap = (int)m;
    e->trace_cap = 0;
  }
  if (n_want > e->want_cap) {
    drop_graphs(e);
    const size_t w = (size_t)std::max(n_want, 16);
    TRY(regrow(e->hw, w * D * e->esz));
    TRY(regrow(e->logits, w * e->cfg.vocab * 4));
    TRY(regrow(e->d_argmax, w * 4));
    e->want_cap = (int)w;
  }
  if (e->trace && e->trace_cap < (size_t)e->layers.size() * e->m_cap * D) {
    e->trace_cap = (size_t)e->layers.size() * e->m_cap * D;
    TRY(regrow(e->trace_buf, e->trace_cap * 4));
  }
  return 0;
}

static int ensure_host_out(xotb200_lm* e, size_t floats) {
  if (floats <= e->h_out_cap) return 0;
  drop_graphs(e);
  if (e->h_out) { cudaFreeHost(e->h_out); e->h_out = nullptr; }
  CK(cudaHostAlloc(&e->h_out, floats * 4, cudaHostAllocDefault));
  e->h_out_cap = floats;
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------------
// the step
// ---------------------------------------------------------------------------------------------------------------------------
struct StepPlan {
  int M = 0, n_seq = 0;
  const int *tokens = nullptr, *row_slot = nullptr, *row_pos = nullptr, *want = nullptr;   // device
  const Item* seqs = nullptr;
  std::map<int, std::pair<const Item*, int>> items;   // rows per attention work item -> (device list, count)
  // expanded prompt attention (bf16): per distinct window of the model's attention layers, the requests that bring many rows
  struct Flash {
    const GatherReq* reqs = nullptr;
    const FlashTile* tiles = nullptr;
    int n_reqs = 0, n_tiles = 0, n_keys = 0, max_keys = 0;
  };
  std::map<int, Flash> flash;
  int max_len = 0;                                     // longest request after this step (bounds every key range)
  int max_rows = 0;                                    // most rows one request brings
  const GqaTile* gqa_tiles = nullptr;                  // key/value-cache attention, long portions (bf16): 64-row tiles
  int n_gqa_tiles = 0;
  bool any_short = true;                               // some request goes through the absorbed kernel
};

template <typename T>
static int attention_layer(xotb200_lm* e, LmLayer& L, const StepPlan& sp) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M, H = s.heads, dn = s.dim, dr = s.rot_dim, dv = s.vdim, R = s.kv_rank, HQ = H * (dn + dr);
  const float eps = e->cfg.norm_eps;
  T* h = static_cast<T*>(e->h);
  // every projection that reads the normed input, as one product
  TRY((product<T, T, float, 0>(e, h, D, 0, at<T>(e, L.w_in), D, 1, 0, e->proj, L.n_in, 0, M, L.n_in, D, 1)));
  const float* qraw = e->proj;
  int q_ld = L.n_in;
  if (s.q_rank > 0) {
    rmsnorm_cols_kernel<T><<<cdiv(M, 8), 256, 0, e->stream>>>(e->proj, L.n_in, L.c_q, s.q_rank, at<T>(e, L.dq_norm), static_cast<T*>(e->cqn), s.q_rank, M, eps);
    CK(cudaGetLastError());
    e->launches++;
    TRY((product<T, T, float, 0>(e, static_cast<T*>(e->cqn), s.q_rank, 0, at<T>(e, L.uq), s.q_rank, 1, 0, e->qraw, HQ, 0, M, HQ, s.q_rank, 1)));
    qraw = e->qraw;
    q_ld = HQ;
  }
  const Paging pg{e->d_table, e->pages_per_slot, e->page_size};
  latent_append_kernel<T><<<cdiv(M, 8), 256, 0, e->stream>>>(e->proj, L.n_in, L.c_kv, R, dr, at<T>(e, L.dkv_norm), eps, L.freqs, s.rot_dims, s.rot_layout,
                                                             sp.row_slot, sp.row_pos, pg, static_cast<T*>(L.pool), M);
  CK(cudaGetLastError());
  e->launches++;
  // ---- which rows take which form
  const StepPlan::Flash* fl = nullptr;
  if constexpr (std::is_same<T, bf16>::value) {
    auto f = sp.flash.find(s.window);
    if (f != sp.flash.end() && f->second.n_tiles > 0) fl = &f->second;
  }
  const float* gate = s.out_gate ? e->proj : nullptr;
  if (sp.any_short || !fl) {
    // absorbed form (few rows per request, and everything in the 32-bit mode)
    query_split_kernel<T><<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(qraw, q_ld, 0, H, dn, dr, R, L.freqs, s.rot_dims, s.rot_layout, sp.row_pos,
                                                                        static_cast<T*>(e->qn), e->qfull, M);
    CK(cudaGetLastError());
    e->launches++;
    // key absorption: qfull[m, h, 0:R] = sum_d qn[m, h, d] * W_uk[h][:, d]
    TRY((product<T, T, float, 0>(e, static_cast<T*>(e->qn), (long)H * dn, dn, at<T>(e, L.uk), dn, 1, (long)dn * R, e->qfull, (long)H * (R + dr), R + dr, M, R,
                                 dn, H)));
    const int qpi = std::max(1, 32 / H);
    const auto& it = sp.items.at(qpi);
    if (it.second > 0) {
      const int pairs = qpi * H, nw = std::min(R > 256 ? 16 : 32, pairs);   // the widest accumulator variant needs 70 registers: 16 warps at most
      const size_t smem = ((size_t)32 * ((R + dr) | 1) + (size_t)nw * (R + dr)) * 4;
      // few work items (decoding): cut the keys into runs so that the GPU is filled; each run at least one 32-key tile
      const int span = s.window > 0 ? std::min(sp.max_len, s.window + qpi) : sp.max_len;
      int splits = 1;
      if (it.second * cdiv(pairs, nw) < e->sm_count)
        splits = std::max(1, std::min(std::min(32, cdiv(span, 32)), cdiv(2 * e->sm_count, it.second * cdiv(pairs, nw))));
      const int chunk = cdiv(cdiv(span, splits), 32) * 32;
      splits = cdiv(span, chunk);
      if (splits > 1) {
        const size_t need = (size_t)M * H * splits * (2 + R);
        if (need > e->part_cap) { drop_graphs(e); TRY(regrow(e->part, need * 4)); e->part_cap = need; }
      }
      const dim3 grid(it.second, cdiv(pairs, nw), splits);
#define LAUNCH_ATTN(NACC)                                                                                                                       \
  do {                                                                                                                                          \
    auto kern = latent_attention_kernel<T, NACC>;                                                                                               \
    TRY(opt_in_smem(kern, smem));                                                                                                               \
    kern<<<grid, nw * 32, smem, e->stream>>>(e->qfull, static_cast<const T*>(L.pool), pg, it.first, H, R, dr, s.scale, s.window, gate, L.n_in, \
                                             L.c_g, static_cast<T*>(e->olat), chunk, e->part);                                                  \
  } while (0)
      if (R <= 64) LAUNCH_ATTN(2);
      else if (R <= 128) LAUNCH_ATTN(4);
      else if (R <= 256) LAUNCH_ATTN(8);
      else LAUNCH_ATTN(16);
#undef LAUNCH_ATTN
      CK(cudaGetLastError());
      e->launches++;
      if (splits > 1) {
        latent_attention_combine_kernel<T><<<dim3(it.second, cdiv(pairs, 8)), 256, 0, e->stream>>>(e->part, it.first, H, R, splits, gate, L.n_in, L.c_g, static_cast<T*>(e->olat));
        CK(cudaGetLastError());
        e->launches++;
      }
    }
    // value expansion per head
    TRY((product<T, T, T, 0>(e, static_cast<T*>(e->olat), (long)H * R, R, at<T>(e, L.uv), R, 1, (long)dv * R, static_cast<T*>(e->oh), (long)H * dv, dv, M, dv,
                             R, H)));
  }
  if constexpr (std::is_same<T, bf16>::value) {
    if (fl) {
      // expanded form for the requests that bring many rows (it overwrites their rows of `oh`)
      bf16 *q16 = static_cast<bf16*>(e->q16), *cbuf = static_cast<bf16*>(e->cbuf), *knx = static_cast<bf16*>(e->knx), *vxx = static_cast<bf16*>(e->vxx);
      query_rotate16_kernel<<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(qraw, q_ld, H, dn, dr, L.freqs, s.rot_dims, s.rot_layout, sp.row_pos, q16, M);
      CK(cudaGetLastError());
      latent_gather_kernel<bf16><<<dim3(cdiv(fl->max_keys, 8), fl->n_reqs), 256, 0, e->stream>>>(static_cast<const bf16*>(L.pool), pg, fl->reqs, R + dr, cbuf);
      CK(cudaGetLastError());
      e->launches += 2;
      TRY((product<bf16, bf16, bf16, 0>(e, cbuf, R + dr, 0, at<bf16>(e, L.uk_rows), R, 1, 0, knx, (long)H * dn, 0, fl->n_keys, H * dn, R, 1)));
      TRY((product<bf16, bf16, bf16, 0>(e, cbuf, R + dr, 0, at<bf16>(e, L.uv), R, 1, 0, vxx, (long)H * dv, 0, fl->n_keys, H * dv, R, 1)));
      const int dqp = (dn + dr + 15) & ~15, dvt = dv <= 64 ? 8 : 16;
      const dim3 grid(fl->n_tiles, H);
      const bool aligned = dn % 8 == 0 && dr % 8 == 0 && R % 8 == 0 && dv % 8 == 0;
#define LAUNCH_FLASH(KERN, SMEM)                                                                                                                  \
  do {                                                                                                                                            \
    auto kern = KERN;                                                                                                                             \
    TRY(opt_in_smem(kern, SMEM));                                                                                                                 \
    kern<<<grid, 128, SMEM, e->stream>>>(q16, knx, cbuf, vxx, fl->tiles, H, dn, dr, dv, R, s.scale, s.window, gate, L.n_in, L.c_g,               \
                                         static_cast<bf16*>(e->oh));                                                                              \
  } while (0)
      if (aligned) {   // whole 16-byte chunks: cp.async double buffering, ldmatrix fragments
        const size_t smem = ((size_t)3 * 64 * (dqp + 8) + (size_t)2 * 64 * (8 * dvt + 8)) * 2;
        if (dvt == 8) LAUNCH_FLASH(latent_flash_aligned_kernel<8>, smem);
        else LAUNCH_FLASH(latent_flash_aligned_kernel<16>, smem);
      } else {
        const size_t smem = ((size_t)2 * 64 * (dqp + 8) + (size_t)8 * dvt * 72) * 2;
        if (dvt == 8) LAUNCH_FLASH(latent_flash_kernel<8>, smem);
        else LAUNCH_FLASH(latent_flash_kernel<16>, smem);
      }
#undef LAUNCH_FLASH
      CK(cudaGetLastError());
      e->launches++;
      e->flash_launches++;
    }
  }
  // the output projection
  TRY((product<T, T, float, 0>(e, static_cast<T*>(e->oh), (long)H * dv, 0, at<T>(e, L.wo), (long)H * dv, 1, 0, e->y, D, 0, M, D, H * dv, 1)));
  return 0;
}

template <int KPT, int P, int NC>
static int launch_delta(xotb200_lm* e, LmLayer& L, const StepPlan& sp, DeltaSrc ks, DeltaSrc rs, DeltaSrc vs, int dk, int dv, bool removal) {
  const xotb200_lm_layer& s = L.s;
  constexpr int CPW = (32 / P) * NC;
  const int warps = std::max(1, std::min(4, cdiv(dv, CPW)));
  const dim3 grid(sp.n_seq * s.heads, cdiv(dv, warps * CPW));
  const int HD = s.heads * dk;
  const int vec4 = (dk % 4 == 0 && dv % 4 == 0 && HD % 4 == 0 && (ks.ld | ks.col | rs.ld | rs.col | vs.ld | vs.col) % 4 == 0) ? 1 : 0;
  delta_rule_kernel<KPT, P, NC><<<grid, warps * 32, 0, e->stream>>>(ks, rs, vs, e->wlog, removal ? e->du : nullptr, removal ? e->dau : nullptr, sp.seqs, s.heads, dk, dv,
                                                                    e->state + L.state_off, e->state_floats, e->oraw, vec4);
  CK(cudaGetLastError());
  e->launches++;
  return 0;
}
// The recurrence is bound by the instructions one warp issues per token (measured: ~2.8 cycles each with one warp per scheduler):
// key rows over 4 or 8 lanes, few columns per thread, four warps per block.  The variant is chosen by the larger of the key and
// value sizes; of the columns-per-thread choices the widest that still gives CTAs for three quarters of the SMs (a single prompt has only
// heads x column groups CTAs: narrower threads mean more CTAs and more warps per scheduler to hide the dependent latency).
// dk x dv: the state of a head (the mixers that ride on this kernel say what that is); removal: the rule has its - au (u^T S) term
static int run_delta(xotb200_lm* e, LmLayer& L, const StepPlan& sp, DeltaSrc ks, DeltaSrc rs, DeltaSrc vs, int dk, int dv, bool removal) {
  const int d = std::max(dk, dv);
  auto fills = [&](int P, int NC) {                    // CTAs of a variant against the SMs
    const int cpw = (32 / P) * NC, warps = std::max(1, std::min(4, cdiv(dv, cpw)));
    return 4L * sp.n_seq * L.s.heads * cdiv(dv, warps * cpw) >= 3L * e->sm_count;
  };
  if (d <= 16) return launch_delta<4, 4, 2>(e, L, sp, ks, rs, vs, dk, dv, removal);
  if (d <= 32) return fills(4, 2) ? launch_delta<8, 4, 2>(e, L, sp, ks, rs, vs, dk, dv, removal) : launch_delta<8, 4, 1>(e, L, sp, ks, rs, vs, dk, dv, removal);
  if (d <= 64)
    return fills(8, 4) ? launch_delta<8, 8, 4>(e, L, sp, ks, rs, vs, dk, dv, removal)
         : fills(8, 2) ? launch_delta<8, 8, 2>(e, L, sp, ks, rs, vs, dk, dv, removal)
                       : launch_delta<8, 8, 1>(e, L, sp, ks, rs, vs, dk, dv, removal);
  if (d <= 128) return fills(8, 2) ? launch_delta<16, 8, 2>(e, L, sp, ks, rs, vs, dk, dv, removal) : launch_delta<16, 8, 1>(e, L, sp, ks, rs, vs, dk, dv, removal);
  return launch_delta<32, 8, 1>(e, L, sp, ks, rs, vs, dk, dv, removal);
}

template <typename T>
static int delta_layer(xotb200_lm* e, LmLayer& L, const StepPlan& sp) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M, HD = s.heads * s.dim;
  T* h = static_cast<T*>(e->h);
  TRY((product<T, T, float, 0>(e, h, D, 0, at<T>(e, L.w_in), D, 1, 0, e->proj, L.n_in, 0, M, L.n_in, D, 1)));
  tanh_cols_kernel<T><<<cdiv((long)M * s.low_rank, 256), 256, 0, e->stream>>>(e->proj, L.n_in, L.c_w1, s.low_rank, static_cast<T*>(e->th), M);
  CK(cudaGetLastError());
  e->launches++;
  TRY((product<T, T, float, 0>(e, static_cast<T*>(e->th), s.low_rank, 0, at<T>(e, L.w2), s.low_rank, 1, 0, e->wlog, HD, 0, M, HD, s.low_rank, 1)));
  delta_prepare_kernel<T><<<cdiv((long)M * s.heads, 8), 256, 0, e->stream>>>(e->proj, L.n_in, L.c_k, L.c_a, e->wlog, at<T>(e, L.w0), at<T>(e, L.a_b), e->du, e->dau,
                                                                              s.heads, s.dim, M);
  CK(cudaGetLastError());
  e->launches++;
  TRY(run_delta(e, L, sp, DeltaSrc{e->proj, L.n_in, L.c_k}, DeltaSrc{e->proj, L.n_in, L.c_r}, DeltaSrc{e->proj, L.n_in, L.c_v}, s.dim, s.vdim, true));
  head_norm_gate_kernel<T><<<cdiv((long)M * s.heads, 8), 256, 0, e->stream>>>(e->oraw, nullptr, nullptr, at<T>(e, L.onorm), s.vdim, e->proj, L.n_in, L.c_g, 0,
                                                                               static_cast<T*>(e->oh), s.heads, s.vdim, e->cfg.norm_eps, M);
  CK(cudaGetLastError());
  e->launches++;
  TRY((product<T, T, float, 0>(e, static_cast<T*>(e->oh), HD, 0, at<T>(e, L.wo), HD, 1, 0, e->y, D, 0, M, D, HD, 1)));
  return 0;
}

// rows of one request that share a CTA of the warp-per-(row, head) attention kernel: about 32 (row, head) pairs
static int gqa_rows_per_item(const xotb200_lm_layer& s) { return std::max(1, 32 / (s.heads / s.kv_heads)); }
// warps of its CTA (one per (row, head) pair): the widest accumulator variant (values above 256) needs too many registers for 32
static int gqa_item_warps(const xotb200_lm_layer& s, int pairs) { return std::min(s.vdim > 256 ? 16 : 32, pairs); }

// Few CTAs (decoding): the keys of an item are cut into runs so that the GPU is filled; each run at least one 32-key tile.
// Returns the number of runs and their length.
static int gqa_key_runs(const xotb200_lm* e, const xotb200_lm_layer& s, int n_items, int max_len, int* run) {
  const int rep = s.heads / s.kv_heads, qpi = gqa_rows_per_item(s), pairs = qpi * rep, nw = gqa_item_warps(s, pairs), ytiles = cdiv(pairs, nw);
  int span = std::max(1, max_len);
  if (s.window > 0) span = std::min(span, s.window + qpi);
  if (s.chunk > 0) span = std::min(span, s.chunk + qpi - 1);   // an item's rows may straddle two blocks: its keys start at the first row's block
  if (s.keep_first > 0) span += std::min(s.keep_first, std::max(1, max_len));   // extra keys in front of the token stretch
  if (s.pool > 0) span += std::max(1, max_len) / s.pool;
  int splits = 1;
  const long ctas = (long)n_items * s.kv_heads * ytiles;
  if (ctas > 0 && ctas < e->sm_count) splits = std::max(1, std::min(std::min(32, cdiv(span, 32)), cdiv(2 * e->sm_count, ctas)));
  *run = cdiv(cdiv(span, splits), 32) * 32;
  return cdiv(span, *run);
}

// (the projection of the layer's mixers is in e->proj, leading dimension L.ld_in; the mixer's output goes to yout)
template <typename T>
static int gqa_layer(xotb200_lm* e, LmLayer& L, const StepPlan& sp, float* yout) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M, H = s.heads, G = s.kv_heads, dk = s.dim, dv = s.vdim, rep = H / G;
  const bool own = s.kv_from < 0;
  const Paging pg{e->d_table, e->pages_per_slot, e->page_size};
  T* pool = static_cast<T*>(e->layers[L.kv_src].pool);
  const int slots = H + (own ? 2 * G : 0);
  bf16* q16 = sp.n_gqa_tiles > 0 ? static_cast<bf16*>(e->q16) : nullptr;
  const bool weighted = s.qk_norm == XOTB200_LM_QKNORM_HEAD || s.qk_norm == XOTB200_LM_QKNORM_ROW;
  if (s.qk_norm == XOTB200_LM_QKNORM_ROW) {
    const int nt = std::min(1024, std::max(128, cdiv(H * dk, 4 * 32) * 32));
    auto pk = gqa_prepare_row_kernel<T>;
    const size_t psm = (size_t)(H + (own ? G : 0)) * dk * 4;
    TRY(opt_in_smem(pk, psm));
    pk<<<M, nt, psm, e->stream>>>(e->proj, L.ld_in, L.c_q, L.c_kk, L.c_vv, s.proj_bias ? at<T>(e, L.b_in) : nullptr, at<T>(e, L.q_norm),
                                                        own ? at<T>(e, L.k_norm) : nullptr, e->cfg.norm_eps, H, G, dk, dv, own ? 1 : 0, s.q_temp_coef,
                                                        s.q_temp_every, sp.row_slot, sp.row_pos, pg, pool, e->qfull, q16);
  } else {
    gqa_prepare_kernel<T><<<cdiv((long)M * slots, 8), 256, 0, e->stream>>>(
        e->proj, L.ld_in, L.c_q, L.c_kk, L.c_vv, s.proj_bias ? at<T>(e, L.b_in) : nullptr, weighted ? at<T>(e, L.q_norm) : nullptr,
        weighted && own ? at<T>(e, L.k_norm) : nullptr, e->cfg.norm_eps, H, G, dk, dv, own ? 1 : 0, s.q_temp_coef, s.q_temp_every, sp.row_slot, sp.row_pos,
        pg, pool, e->qfull, q16, M, s.qk_norm != XOTB200_LM_QKNORM_NONE ? 1 : 0, s.rot_dims > 0 ? L.freqs : nullptr, s.rot_dims, s.rot_layout);
  }
  CK(cudaGetLastError());
  e->launches++;
  const size_t pool_rows = (size_t)e->n_pages * e->page_size;
  if (s.pool > 0) {
    // blocks whose last token this step appended get their pooled row (after the append, before any reader)
    gqa_pool_blocks_kernel<T><<<dim3(sp.n_seq, sp.max_rows / s.pool + 1, cdiv(G * (dk + dv), 128)), 128, 0, e->stream>>>(pool, pg, pool_rows, sp.seqs, s.pool,
                                                                                                                       G * (dk + dv));
    CK(cudaGetLastError());
    e->launches++;
  }
  const GqaScore sc{s.scale, s.softcap, s.window, s.chunk, s.dist_bias ? at<T>(e, L.r1) : nullptr, s.dist_bias ? at<T>(e, L.r2) : nullptr,
                    s.rel_buckets > 0 ? L.rel_tab : nullptr, L.rel_n, s.sink ? at<T>(e, L.sink) : nullptr, s.keep_first, s.pool, pool_rows};
  const float* gate = s.out_gate ? e->proj : nullptr;
  const int qpi = gqa_rows_per_item(s);
  const auto& it = sp.items.at(-qpi);   // the lists of this mixer have negative keys
  if (it.second > 0) {
    const int pairs = qpi * rep, nw = gqa_item_warps(s, pairs), ytiles = cdiv(pairs, nw);
    const size_t smem = ((size_t)32 * ((dk + dv) | 1) + (size_t)nw * dk) * 4;
    int run = 0;
    const int splits = gqa_key_runs(e, s, it.second, sp.max_len, &run);
    REQUIRE(splits == 1 || (size_t)M * H * splits * (2 + dv) <= e->part_cap, "internal: the key-run buffer was not sized for this step");
    const dim3 grid(it.second, G * ytiles, splits);
#define LAUNCH_GQA(NACC)                                                                                                                     \
  do {                                                                                                                                       \
    auto kern = gqa_attention_kernel<T, NACC>;                                                                                               \
    TRY(opt_in_smem(kern, smem));                                                                                                            \
    kern<<<grid, nw * 32, smem, e->stream>>>(e->qfull, pool, pg, it.first, H, G, dk, dv, sc, gate, s.out_gate, L.ld_in, L.c_g,               \
                                             static_cast<T*>(e->oh), run, e->part);                                                          \
  } while (0)
    if (dv <= 32) LAUNCH_GQA(1);
    else if (dv <= 64) LAUNCH_GQA(2);
    else if (dv <= 128) LAUNCH_GQA(4);
    else if (dv <= 256) LAUNCH_GQA(8);
    else LAUNCH_GQA(16);
#undef LAUNCH_GQA
    CK(cudaGetLastError());
    e->launches++;
    if (splits > 1) {
      gqa_combine_kernel<T><<<dim3(it.second, cdiv(qpi * H, 8)), 256, 0, e->stream>>>(e->part, it.first, H, dv, splits, s.sink ? at<T>(e, L.sink) : nullptr, gate,
                                                                                     s.out_gate, L.ld_in, L.c_g, static_cast<T*>(e->oh));
      CK(cudaGetLastError());
      e->launches++;
    }
  }
  if constexpr (std::is_same<T, bf16>::value) {
    if (sp.n_gqa_tiles > 0) {
      // long portions: streaming softmax on the tensor cores, keys and values straight from the pages
      const int dqp = (dk + 15) & ~15, dvt = dv <= 64 ? 8 : 16;
      const size_t fsm = ((size_t)3 * 64 * (dqp + 8) + (size_t)2 * 64 * (8 * dvt + 8)) * 2;
      const dim3 grid(sp.n_gqa_tiles, H);
      // distances a tile can meet: up to the longest request, less under a block or window rule (a 64-row tile reaches 63 further back)
      int dist_n = sp.max_len;
      if (s.chunk > 0) dist_n = std::min(dist_n, s.chunk + 64);
      if (s.window > 0) dist_n = std::min(dist_n, s.window + 64);
      if (s.dist_bias) {
        if ((size_t)H * dist_n > e->dist_cap) { TRY(regrow(e->dist_tab, (size_t)H * dist_n * 4)); e->dist_cap = (size_t)H * dist_n; }
        gqa_dist_table_kernel<<<cdiv((long)H * dist_n, 256), 256, 0, e->stream>>>(at<bf16>(e, L.r1), at<bf16>(e, L.r2), H, dist_n, e->dist_tab);
        CK(cudaGetLastError());
        e->launches++;
      }
#define LAUNCH_GQA_FLASH(DVT)                                                                                                              \
  do {                                                                                                                                     \
    auto kern = gqa_flash_kernel<DVT>;                                                                                                     \
    TRY(opt_in_smem(kern, fsm));                                                                                                           \
    kern<<<grid, 128, fsm, e->stream>>>(static_cast<const bf16*>(e->q16), pool, pg, sp.gqa_tiles, H, G, dk, dv, sc,                        \
                                        s.dist_bias ? e->dist_tab : nullptr, dist_n, gate, s.out_gate, L.ld_in, L.c_g, static_cast<bf16*>(e->oh)); \
  } while (0)
      if (dvt == 8) LAUNCH_GQA_FLASH(8);
      else LAUNCH_GQA_FLASH(16);
#undef LAUNCH_GQA_FLASH
      CK(cudaGetLastError());
      e->launches++;
      e->flash_launches++;
    }
  }
  TRY((product<T, T, float, 0>(e, static_cast<T*>(e->oh), (long)H * dv, 0, at<T>(e, L.wo), (long)H * dv, 1, 0, yout, D, 0, M, D, H * dv, 1)));
  return 0;
}

// short causal convolution of C projection columns starting at col0 (filter inputs of earlier steps from the slot's state, which
// the same launch then moves on) -> e->cvb [M, C]
template <typename T>
static int filter_channels(xotb200_lm* e, LmLayer& L, const StepPlan& sp, int col0, int C, const T* bias) {
  const xotb200_lm_layer& s = L.s;
  float* cstate = e->state + L.conv_off;
  const int zrows = std::max(1, std::min(128, cdiv(sp.max_rows, 8)));
  short_conv_kernel<T, float><<<dim3(sp.n_seq, cdiv(C, 256), zrows), 256, 0, e->stream>>>(e->proj, L.ld_in, col0, C, at<T>(e, L.conv_w), bias, s.conv_taps, 1, 0,
                                                                                          sp.seqs, cstate, e->state_floats, e->cvb, C);
  CK(cudaGetLastError());
  e->launches++;
  return 0;
}

template <typename T>
static int gated_delta_layer(xotb200_lm* e, LmLayer& L, const StepPlan& sp, float* yout, void* ohbuf) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M, H = s.heads, G = s.kv_heads, dk = s.dim, dv = s.vdim, C = L.conv_ch;
  TRY(filter_channels<T>(e, L, sp, L.c_r, C, nullptr));
  gated_delta_prepare_kernel<T><<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(e->cvb, C, e->proj, L.ld_in, L.c_b, L.c_a, at<T>(e, L.a_log), at<T>(e, L.dt_bias), e->wlog,
                                                                            e->du, e->dau, e->dkk, e->drr, H, G, dk, M);
  CK(cudaGetLastError());
  e->launches++;
  TRY(run_delta(e, L, sp, DeltaSrc{e->dkk, H * dk, 0}, DeltaSrc{e->drr, H * dk, 0}, DeltaSrc{e->cvb, C, 2 * G * dk}, dk, dv, true));
  head_norm_gate_kernel<T><<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(e->oraw, nullptr, nullptr, at<T>(e, L.onorm), 0, e->proj, L.ld_in, L.c_g, 1, static_cast<T*>(ohbuf),
                                                                       H, dv, e->cfg.norm_eps, M);
  CK(cudaGetLastError());
  e->launches++;
  TRY((product<T, T, float, 0>(e, static_cast<T*>(ohbuf), (long)H * dv, 0, at<T>(e, L.wo), (long)H * dv, 1, 0, yout, D, 0, M, D, H * dv, 1)));
  return 0;
}

// matrix LSTM: gates (a scan per request and head), vectors, the normaliser's own small recurrence, the shared recurrence kernel on
// the [dk, dv] states, normaliser + head norm + sigmoid gate, output product
template <typename T>
static int matrix_lstm_layer(xotb200_lm* e, LmLayer& L, const StepPlan& sp, float* yout, void* ohbuf) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M, H = s.heads, dk = s.dim, dv = s.vdim;
  mlstm_gates_kernel<T><<<cdiv((long)sp.n_seq * H, 4), 128, 0, e->stream>>>(e->proj, L.ld_in, L.c_i, L.c_f, at<T>(e, L.i_b), at<T>(e, L.f_b), s.gate_cap, sp.seqs, sp.n_seq, H,
                                                                          e->state + L.m_off, e->state_floats, e->gdec, e->ginw, e->gfloor);
  CK(cudaGetLastError());
  mlstm_expand_kernel<<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(e->proj, L.ld_in, L.c_r, L.c_k, e->gdec, e->ginw, e->wlog, e->dkk, e->drr, H, dk, M);
  CK(cudaGetLastError());
  mlstm_normaliser_kernel<<<sp.n_seq * H, 32 * std::max(1, std::min(16, sp.max_rows / 16)), 0, e->stream>>>(e->dkk, e->drr, e->gdec, sp.seqs, H, dk, e->state + L.n_off,
                                                                                                        e->state_floats, e->gnq);
  CK(cudaGetLastError());
  e->launches += 3;
  TRY(run_delta(e, L, sp, DeltaSrc{e->dkk, H * dk, 0}, DeltaSrc{e->drr, H * dk, 0}, DeltaSrc{e->proj, L.ld_in, L.c_v}, dk, dv, false));
  head_norm_gate_kernel<T><<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(e->oraw, e->gnq, e->gfloor, at<T>(e, L.onorm), dv, e->proj, L.ld_in, L.c_g, 0,
                                                                       static_cast<T*>(ohbuf), H, dv, e->cfg.norm_eps, M);
  CK(cudaGetLastError());
  e->launches++;
  TRY((product<T, T, float, 0>(e, static_cast<T*>(ohbuf), (long)H * dv, 0, at<T>(e, L.wo), (long)H * dv, 1, 0, yout, D, 0, M, D, H * dv, 1)));
  return 0;
}

// state-space layer: filter + silu on [x | B | C], step sizes and decays, the shared recurrence kernel, skip + gate + grouped norm,
// output product
template <typename T>
static int mamba2_layer(xotb200_lm* e, LmLayer& L, const StepPlan& sp, float* yout, void* ohbuf) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M, H = s.heads, G = s.kv_heads, N = s.dim, dv = s.vdim, C = L.conv_ch, inner = H * dv;
  TRY(filter_channels<T>(e, L, sp, L.c_v, C, at<T>(e, L.conv_b)));
  mamba2_prepare_kernel<T><<<cdiv((long)M * H, 8), 256, 0, e->stream>>>(e->cvb, C, e->proj, L.ld_in, L.c_dt, at<T>(e, L.a_log), at<T>(e, L.dt_bias), e->wlog, e->dkk, e->drr,
                                                                       H, G, N, dv, M);
  CK(cudaGetLastError());
  e->launches++;
  TRY(run_delta(e, L, sp, DeltaSrc{e->dkk, H * N, 0}, DeltaSrc{e->drr, H * N, 0}, DeltaSrc{e->cvb, C, 0}, N, dv, false));
  {
    const int part = inner / s.out_norm_groups;
    auto ok = mamba2_out_kernel<T>;
    TRY(opt_in_smem(ok, (size_t)part * 4));
    ok<<<M * s.out_norm_groups, std::min(1024, std::max(32, cdiv(part, 4 * 32) * 32)), (size_t)part * 4, e->stream>>>(
        e->oraw, e->cvb, C, e->proj, L.ld_in, L.c_z, at<T>(e, L.d_skip), at<T>(e, L.onorm), H, dv, s.out_norm_groups, e->cfg.norm_eps, static_cast<T*>(ohbuf));
  }
  CK(cudaGetLastError());
  e->launches++;
  TRY((product<T, T, float, 0>(e, static_cast<T*>(ohbuf), (long)inner, 0, at<T>(e, L.wo), (long)inner, 1, 0, yout, D, 0, M, D, inner, 1)));
  return 0;
}

// Rows sorted by expert, every run padded to whole row tiles: C[p, :] = A[p, :] B[tile_batch[p / 128]]^T on the tensor cores.
// 1 = launched, 0 = the operands cannot be described to TMA
template <int EPI, typename TC>
static int grouped_product(xotb200_lm* e, const bf16* A, long lda, const bf16* B, long ldb, long b_batch, int n_batch, TC* C, long ldc, int m_pad, int N,
                           int K, const int* tile_batch) {
  const int nt = N > 64 ? 128 : 64;
  CUtensorMap ma, mb;
  if (!make_map3(&ma, A, m_pad, K, lda, 0, 1, LTC_M) || !make_map3(&mb, B, N, K, ldb, b_batch, n_batch, nt)) return 0;
  LtcArgs a{m_pad, N, K, C, ldc, 0, e->d_err, nullptr, tile_batch, 1};
  if (nt == 128) TRY((launch_ltc<128, EPI, TC>(e, ma, mb, a, 1)));
  else TRY((launch_ltc<64, EPI, TC>(e, ma, mb, a, 1)));
  return 1;
}

// Rows from which the experts run as grouped tensor-core products (below: every (row, expert) pair streams its expert).  Measured
// on decode batches: from 4 rows on the grouped form is faster (each chosen expert is streamed once, however many rows chose it).
static const int MOE_GROUPED_MIN_ROWS = 3;

static bool layer_has_ff(const xotb200_lm_layer& s) { return s.ff_kind == XOTB200_LM_FF_MOE ? s.experts > 0 : s.ff > 0; }

// the feed-forward of a layer: h (T) -> y (fp32)
template <typename T>
static int feed_forward(xotb200_lm* e, LmLayer& L, const StepPlan& sp) {
  const xotb200_lm_layer& s = L.s;
  const int D = e->cfg.width, M = sp.M;
  T* h = static_cast<T*>(e->h);
  if (s.ff_kind == XOTB200_LM_FF_MOE) {
    const int E = s.experts, F = s.expert_ff, top = s.top;
    const bool gated = s.expert_act == XOTB200_LM_EXPERT_SILU_GATED;
    const int Fs = s.shared_ff;
    const bool grouped_ok = std::is_same<T, bf16>::value && M >= MOE_GROUPED_MIN_ROWS && e->gemm_mode != 1 && F % 8 == 0 && D % 8 == 0;
    // Few rows (and the 32-bit mode): the shared expert rides along in the experts' row kernels — no launches and no pass over y of
    // its own — when the activations of a row fit in shared memory.  Otherwise it runs first as two ordinary products and the
    // chosen experts' weighted outputs are added to its output.
    const bool ride = Fs > 0 && !gated && !grouped_ok && ((size_t)top * F + Fs + 4) * 4 <= 200 * 1024;
    const int shared = Fs > 0 && !ride ? 1 : 0;
    if (shared) {
      TRY((product<T, T, T, 1>(e, h, D, 0, at<T>(e, L.up), D, 1, 0, static_cast<T*>(e->act), s.shared_ff, 0, M, s.shared_ff, D, 1)));
      TRY((product<T, T, float, 0>(e, static_cast<T*>(e->act), s.shared_ff, 0, at<T>(e, L.down), s.shared_ff, 1, 0, e->y, D, 0, M, D, s.shared_ff, 1)));
    }
    {
      auto kern = moe_router_kernel<T>;
      const size_t rsm = ((size_t)((D + 3) & ~3) + E) * 4;
      TRY(opt_in_smem(kern, rsm));
      kern<<<M, std::min(1024, std::max(64, cdiv(E, 2) * 32)), rsm, e->stream>>>(h, D, at<T>(e, L.router), s.router_bias ? at<T>(e, L.router_b) : nullptr,
                                                                                 s.router_kind, E, s.groups, s.groups_keep, top, e->moe_ids, e->moe_wts, M);
    }
    CK(cudaGetLastError());
    e->launches++;
    const int il8 = gated && F % 8 == 0 ? 1 : 0;
    if constexpr (std::is_same<T, bf16>::value) {
      if (grouped_ok) {
        const int pairs = M * top, tiles = cdiv(pairs, LTC_M) + E, m_pad = tiles * LTC_M;
        REQUIRE(tiles <= e->moe_tiles_cap, "internal: the expert tile list was not sized for this step");
        int *counts = e->moe_plan, *starts = counts + e->max_experts, *cursor = starts + e->max_experts + 1, *place = cursor + e->max_experts,
            *tile_expert = place + (size_t)e->m_cap * e->max_top;
        bf16* xg = static_cast<bf16*>(e->moe_xg);
        moe_count_kernel<<<cdiv(pairs, 256), 256, 0, e->stream>>>(e->moe_ids, pairs, counts);
        moe_plan_kernel<<<1, 256, 0, e->stream>>>(counts, E, LTC_M, tiles, starts, cursor, tile_expert);
        moe_scatter_kernel<bf16><<<cdiv(pairs, 8), 256, 0, e->stream>>>(h, D, e->moe_ids, pairs, top, starts, cursor, place, xg);
        CK(cudaGetLastError());
        e->launches += 3;
        int r = gated ? grouped_product<3, bf16>(e, xg, D, at<bf16>(e, L.w_gu), D, (long)2 * F * D, E, static_cast<bf16*>(e->mact), F, m_pad, 2 * F, D, tile_expert)
                      : grouped_product<1, bf16>(e, xg, D, at<bf16>(e, L.w_gu), D, (long)F * D, E, static_cast<bf16*>(e->mact), F, m_pad, F, D, tile_expert);
        if (r < 0) return r;
        if (r == 1) r = grouped_product<0, float>(e, static_cast<bf16*>(e->mact), F, at<bf16>(e, L.w_edown), F, (long)D * F, E, e->moe_yg, D, m_pad, D, F, tile_expert);
        if (r < 0) return r;
        if (r == 1) {
          moe_combine_kernel<<<M, 256, 0, e->stream>>>(e->moe_yg, place, e->moe_wts, top, D, shared, e->y);
          CK(cudaGetLastError());
          e->launches++;
          return 0;
        }
      }
    }
    {
      auto kern = moe_rows_up_kernel<T>;
      TRY(opt_in_smem(kern, (size_t)D * 4));
      // a warp takes two weight rows per pass with gated experts (a gate row and its up row), four with ungated ones
      kern<<<dim3(M, top + (ride ? 1 : 0), std::max(1, std::min(cdiv(std::max(F, ride ? Fs : 0), gated ? 8 : 32), M <= 16 ? 1024 : 16))), 256, (size_t)D * 4, e->stream>>>(
          h, D, at<T>(e, L.w_gu), F, il8, gated ? 1 : 0, e->moe_ids, top, static_cast<T*>(e->mact), ride ? at<T>(e, L.up) : nullptr, Fs, static_cast<T*>(e->act));
      CK(cudaGetLastError());
      e->launches++;
    }
    {
      auto kern = moe_rows_down_kernel<T>;
      const size_t dsm = ((size_t)top * F + (ride ? Fs + 4 : 0)) * 4;
      TRY(opt_in_smem(kern, dsm));
      kern<<<dim3(M, std::max(1, std::min(cdiv(D, 16), M <= 16 ? 1024 : 16))), 256, dsm, e->stream>>>(static_cast<T*>(e->mact), F, at<T>(e, L.w_edown), D, e->moe_ids, e->moe_wts, top,
                                                                                                   shared, e->y, static_cast<T*>(e->act), ride ? at<T>(e, L.down) : nullptr, Fs);
      CK(cudaGetLastError());
      e->launches++;
    }
    return 0;
  }
  if (s.ff_kind == XOTB200_LM_FF_GELU)
    TRY((product<T, T, T, 4>(e, h, D, 0, at<T>(e, L.up), D, 1, 0, static_cast<T*>(e->act), s.ff, 0, M, s.ff, D, 1)));
  else if (s.ff_kind == XOTB200_LM_FF_XIELU)
    TRY((product<T, T, T, 2>(e, h, D, 0, at<T>(e, L.up), D, 1, 0, static_cast<T*>(e->act), s.ff, 0, M, s.ff, D, 1, at<T>(e, L.act_p))));
  else
    TRY((product<T, T, T, 1>(e, h, D, 0, at<T>(e, L.up), D, 1, 0, static_cast<T*>(e->act), s.ff, 0, M, s.ff, D, 1)));
  TRY((product<T, T, float, 0>(e, static_cast<T*>(e->act), s.ff, 0, at<T>(e, L.down), s.ff, 1, 0, e->y, D, 0, M, D, s.ff, 1)));
  return 0;
}

template <typename T>
static int run_branch(xotb200_lm* e, LmLayer& L, const StepPlan& sp, float* yout, void* ohbuf) {
  switch (L.s.mixer) {
    case XOTB200_LM_MIX_ATTENTION: return gqa_layer<T>(e, L, sp, yout);
    case XOTB200_LM_MIX_GATED_DELTA: return gated_delta_layer<T>(e, L, sp, yout, ohbuf);
    case XOTB200_LM_MIX_MATRIX_LSTM: return matrix_lstm_layer<T>(e, L, sp, yout, ohbuf);
    default: return mamba2_layer<T>(e, L, sp, yout, ohbuf);
  }
}

// the layer's mixer(s): h (T) -> y (fp32), and y2 for a second mixer.  Every projection that reads h — of both mixers — is one product.
template <typename T>
static int run_mixer(xotb200_lm* e, LmLayer& L, const StepPlan& sp) {
  if (L.s.mixer == XOTB200_LM_MIX_LATENT_ATTN) return attention_layer<T>(e, L, sp);
  if (L.s.mixer == XOTB200_LM_MIX_DELTA_RULE) return delta_layer<T>(e, L, sp);
  TRY((product<T, T, float, 0>(e, static_cast<T*>(e->h), e->cfg.width, 0, at<T>(e, L.w_in), e->cfg.width, 1, 0, e->proj, L.ld_in, 0, sp.M, L.ld_in, e->cfg.width, 1)));
  if (L.par.empty()) return run_branch<T>(e, L, sp, e->y, e->oh);
  // Two mixers: they share the projection and nothing else (each has its scratch, its state, its operand buffer), so the second runs
  // on the side stream beside the first — a recurrence walks the tokens with few CTAs, the attention fills the rest of the GPU — and
  // the layer goes on when both are done.  Inside a captured decode step the two streams become two branches of the graph.
  CK(cudaEventRecord(e->ev_fork, e->stream));
  CK(cudaStreamWaitEvent(e->side, e->ev_fork, 0));
  cudaStream_t main_stream = e->stream;
  e->stream = e->side;
  int rc = run_branch<T>(e, L.par[0], sp, e->y2, e->oh2);
  e->stream = main_stream;
  if (rc == 0) rc = run_branch<T>(e, L, sp, e->y, e->oh);
  // joined also after a failed launch: a capture must not end with the side stream still forked
  cudaError_t j1 = cudaEventRecord(e->ev_join, e->side), j2 = cudaStreamWaitEvent(e->stream, e->ev_join, 0);
  if (rc < 0) return rc;
  CK(j1);
  CK(j2);
  return 0;
}

static void finish_logits(xotb200_lm* e, int n_want) {
  const float scale = e->cfg.logit_scale != 0.f ? e->cfg.logit_scale : 1.0f;
  argmax_rows_kernel<<<n_want, 1024, 0, e->stream>>>(e->logits, e->cfg.vocab, scale, e->cfg.logit_softcap, e->d_argmax);
  e->launches++;
}

// layers of the form x += norm(sublayer(x)): the sublayer reads the stream itself (its T copy h); a layer norm (weight and bias)
// or an RMS norm (weight stored around zero) closes it and adds the bias of the mixer's output projection on the way
template <typename T>
static int run_layers_post(xotb200_lm* e, const StepPlan& sp, int n_want) {
  const int D = e->cfg.width, M = sp.M;
  const float eps = e->cfg.norm_eps;
  const bool rms = e->cfg.block == XOTB200_LM_BLOCK_POST_RMS;
  T* h = static_cast<T*>(e->h);
  const int nt = std::min(1024, std::max(128, cdiv(D, 4 * 32) * 32));
  auto kern = residual_layernorm_kernel<T>;
  auto kern_rms = residual_rmsnorm_kernel<T>;
  TRY(opt_in_smem(kern, (size_t)D * 4));
  TRY(opt_in_smem(kern_rms, (size_t)D * 4));
  auto close = [&](size_t w, size_t b, const T* y_bias) -> int {
    if (rms) kern_rms<<<M, nt, (size_t)D * 4, e->stream>>>(e->x, e->y, y_bias, at<T>(e, w), 1.0f, h, nullptr, D, eps);
    else kern<<<M, nt, (size_t)D * 4, e->stream>>>(e->x, e->y, y_bias, at<T>(e, w), at<T>(e, b), h, nullptr, D, eps);
    CK(cudaGetLastError());
    e->launches++;
    return 0;
  };
  if (e->first) {
    if (e->cfg.pos_sinusoid || e->cfg.embed_norm) {
      auto ek = embed_sinusoid_rows_kernel<T>;
      TRY(opt_in_smem(ek, (size_t)D * 4));
      ek<<<M, nt, (size_t)D * 4, e->stream>>>(at<T>(e, e->embed), e->cfg.max_positions > 0 ? at<T>(e, e->pos_table) : nullptr, e->pos_freqs, sp.tokens, sp.row_pos,
                                              e->cfg.embed_norm ? at<T>(e, e->embed_norm) : nullptr, 1.0f, eps, e->x, h, D);
    } else {
      embed_pos_rows_kernel<T><<<M, 128, 0, e->stream>>>(at<T>(e, e->embed), e->cfg.max_positions > 0 ? at<T>(e, e->pos_table) : nullptr, sp.tokens, sp.row_pos,
                                                         e->x, h, D);
    }
  } else {
    cast_rows_kernel<T><<<std::min(4096, cdiv((long)M * D, 256)), 256, 0, e->stream>>>(e->x, h, (size_t)M * D);
  }
  CK(cudaGetLastError());
  e->launches++;
  for (size_t li = 0; li < e->layers.size(); ++li) {
    LmLayer& L = e->layers[li];
    TRY(run_mixer<T>(e, L, sp));
    TRY(close(L.norm1, L.norm1b, L.s.mixer == XOTB200_LM_MIX_ATTENTION && L.s.out_bias ? at<T>(e, L.o_b) : nullptr));
    if (layer_has_ff(L.s)) {
      TRY(feed_forward<T>(e, L, sp));
      TRY(close(L.norm2, L.norm2b, nullptr));
    }
    if (e->trace) CK(cudaMemcpyAsync(e->trace_buf + li * (size_t)M * D, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToDevice, e->stream));
  }
  if (e->trace) e->trace_floats = e->layers.size() * (size_t)M * D;
  if (e->last && n_want > 0) {
    T* hw = static_cast<T*>(e->hw);
    if (rms) kern_rms<<<n_want, nt, (size_t)D * 4, e->stream>>>(e->x, nullptr, nullptr, at<T>(e, e->final_norm), 1.0f, hw, sp.want, D, eps);
    else kern<<<n_want, nt, (size_t)D * 4, e->stream>>>(e->x, nullptr, nullptr, at<T>(e, e->final_norm), at<T>(e, e->final_norm_b), hw, sp.want, D, eps);
    CK(cudaGetLastError());
    e->launches++;
    TRY((product<T, T, float, 0>(e, hw, D, 0, at<T>(e, e->head), D, 1, 0, e->logits, e->cfg.vocab, 0, n_want, e->cfg.vocab, D, 1)));
    finish_logits(e, n_want);
    CK(cudaGetLastError());
  }
  return 0;
}

// Pre-norm layers with one-number norm weights: x += mult * sublayer(c(rms(x) * g)), the stream kept in `streams` copies mixed by
// hyper-connections, c(h) = h + causal convolution of h.  hc_open_kernel closes the pending sublayer and opens the next in one
// pass; the convolution (whose inputs of earlier steps are part of a slot's state, moved on by the same launch) follows.
template <typename T>
static int run_layers_pre_scalar(xotb200_lm* e, const StepPlan& sp, int n_want) {
  const int D = e->cfg.width, M = sp.M, S = std::max(1, e->cfg.streams), CT = e->cfg.canon_taps;
  const bool hc = e->cfg.streams > 0;
  const float eps = e->cfg.norm_eps, mult = e->cfg.residual_mult != 0.f ? e->cfg.residual_mult : 1.0f;
  T* h = static_cast<T*>(e->h);
  const int nt = std::min(512, std::max(64, cdiv(D, 4 * 32) * 32));    // the row kernels keep all copies of an entry in registers
  // copies held per entry: the smallest of 1, 2, 4, 8 that holds them; 16-byte loads when the rows allow
  auto okern = D % 4 == 0 ? (S <= 1 ? hc_open_kernel<T, 1, 4> : S <= 2 ? hc_open_kernel<T, 2, 4> : S <= 4 ? hc_open_kernel<T, 4, 4> : hc_open_kernel<T, 8, 4>)
                          : (S <= 1 ? hc_open_kernel<T, 1, 1> : S <= 2 ? hc_open_kernel<T, 2, 1> : S <= 4 ? hc_open_kernel<T, 4, 1> : hc_open_kernel<T, 8, 1>);
  TRY(opt_in_smem(okern, (size_t)D * 4));
  // the pending sublayer: its output(s), their scales and its hyper-connection coefficients
  struct Pending { const float *y = nullptr, *y2 = nullptr; float ya = 1.f, yb = 0.f; const T *mix = nullptr, *out = nullptr; } pend;
  // closes the pending sublayer; then, with a norm weight g, opens sublayer q of layer L (h <- c(norm(u))), else writes the sum of the copies to `sum_out`
  auto open = [&](LmLayer* L, int q, float* sum_out) -> int {
    if (!pend.y && !L && !sum_out) return 0;
    const T* g = L ? at<T>(e, q ? L->norm2 : L->norm1) : nullptr;
    const T* inc = L && hc ? at<T>(e, L->hc_in[q]) : nullptr;
    const bool conv = L && CT > 0;
    okern<<<M, nt, (size_t)D * 4, e->stream>>>(e->x, S, pend.y, pend.y2, pend.ya, pend.yb, mult, pend.mix, pend.out, inc, g, eps, nullptr,
                                               L ? (conv ? e->h0 : nullptr) : sum_out, L && !conv ? h : nullptr, D);
    CK(cudaGetLastError());
    e->launches++;
    pend = Pending{};
    if (conv) {
      float* cstate = e->state + L->canon_off[q];
      const int zrows = std::max(1, std::min(128, cdiv(sp.max_rows, 8)));
      short_conv_kernel<T, T><<<dim3(sp.n_seq, cdiv(D, 256), zrows), 256, 0, e->stream>>>(e->h0, D, 0, D, at<T>(e, L->canon[q]), nullptr, CT, 0, 1, sp.seqs, cstate,
                                                                                          e->state_floats, h, D);
      CK(cudaGetLastError());
      e->launches++;
    }
    return 0;
  };
  if (e->first) {
    embed_streams_kernel<T><<<M, nt, 0, e->stream>>>(at<T>(e, e->embed), sp.tokens, e->cfg.embed_norm ? at<T>(e, e->embed_norm) : nullptr, eps, e->x, S, D);
    CK(cudaGetLastError());
    e->launches++;
  }
  for (size_t li = 0; li < e->layers.size(); ++li) {
    LmLayer& L = e->layers[li];
    TRY(open(&L, 0, nullptr));
    TRY(run_mixer<T>(e, L, sp));
    pend.y = e->y;
    pend.ya = L.s.mix_scale != 0.f ? L.s.mix_scale : 1.0f;
    if (!L.par.empty()) { pend.y2 = e->y2; pend.yb = L.s.par_scale; }
    if (hc) { pend.mix = at<T>(e, L.hc_mix[0]); pend.out = at<T>(e, L.hc_out[0]); }
    if (layer_has_ff(L.s)) {
      TRY(open(&L, 1, nullptr));
      TRY(feed_forward<T>(e, L, sp));
      pend.y = e->y;
      if (hc) { pend.mix = at<T>(e, L.hc_mix[1]); pend.out = at<T>(e, L.hc_out[1]); }
    }
    if (e->trace) TRY(open(nullptr, 0, e->trace_buf + li * (size_t)M * D));
  }
  if (e->trace) e->trace_floats = e->layers.size() * (size_t)M * D;
  if (e->last && n_want > 0) {
    // the final norm of the wanted rows closes the last sublayer for them on the way (the other rows' streams are not needed again)
    T* hw = static_cast<T*>(e->hw);
    okern<<<n_want, nt, (size_t)D * 4, e->stream>>>(e->x, S, pend.y, pend.y2, pend.ya, pend.yb, mult, pend.mix, pend.out, nullptr, at<T>(e, e->final_norm), eps, sp.want,
                                                    nullptr, hw, D);
    CK(cudaGetLastError());
    e->launches++;
    TRY((product<T, T, float, 0>(e, hw, D, 0, at<T>(e, e->head), D, 1, 0, e->logits, e->cfg.vocab, 0, n_want, e->cfg.vocab, D, 1)));
    finish_logits(e, n_want);
    CK(cudaGetLastError());
  }
  return 0;
}

// threads of a row's norm block: about one warp per 256 elements, at least one warp per part while parts <= 32, at most 1024
static int norm_threads(int D, int G) {
  int nw = std::max(1, std::min(32, D / 256));
  if (G <= 32) nw = std::max(nw, G) / G * G;
  return std::min(32, std::max(1, nw)) * 32;
}

template <typename T>
static int run_layers(xotb200_lm* e, const StepPlan& sp, int n_want) {
  if (e->cfg.block == XOTB200_LM_BLOCK_PRE_SCALAR) return run_layers_pre_scalar<T>(e, sp, n_want);
  if (e->cfg.block != XOTB200_LM_BLOCK_GROUP_RMS) return run_layers_post<T>(e, sp, n_want);
  const int D = e->cfg.width, G = e->cfg.norm_groups, M = sp.M;
  const float eps = e->cfg.norm_eps;
  T* h = static_cast<T*>(e->h);
  const float* pend_y = nullptr;
  const T* pend_w = nullptr;
  // x += groupnorm(pending sublayer output) * its post-norm weight;  h = groupnorm(x) * w_pre  (either half may be absent)
  auto open = [&](const T* w_pre) -> int {
    if (!pend_y && !w_pre) return 0;
    residual_groupnorm_kernel<T><<<M, norm_threads(D, G), 0, e->stream>>>(e->x, pend_y, pend_w, w_pre, w_pre ? h : nullptr, nullptr, D, G, eps);
    CK(cudaGetLastError());
    e->launches++;
    pend_y = nullptr;
    pend_w = nullptr;
    return 0;
  };
  if (e->first) {
    embed_rows_kernel<T><<<M, 128, 0, e->stream>>>(at<T>(e, e->embed), sp.tokens, e->x, D);
    CK(cudaGetLastError());
    e->launches++;
  }
  for (size_t li = 0; li < e->layers.size(); ++li) {
    LmLayer& L = e->layers[li];
    TRY(open(at<T>(e, L.norm1)));
    TRY(run_mixer<T>(e, L, sp));
    pend_y = e->y;
    pend_w = at<T>(e, L.norm1b);
    if (layer_has_ff(L.s)) {
      TRY(open(at<T>(e, L.norm2)));
      TRY(feed_forward<T>(e, L, sp));
      pend_y = e->y;
      pend_w = at<T>(e, L.norm2b);
    }
    if (e->trace) {
      TRY(open(nullptr));
      CK(cudaMemcpyAsync(e->trace_buf + li * (size_t)M * D, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToDevice, e->stream));
    }
  }
  TRY(open(nullptr));
  if (e->trace) e->trace_floats = e->layers.size() * (size_t)M * D;
  if (e->last && n_want > 0) {
    T* hw = static_cast<T*>(e->hw);
    residual_groupnorm_kernel<T><<<n_want, norm_threads(D, G), 0, e->stream>>>(e->x, nullptr, nullptr, at<T>(e, e->final_norm), hw, sp.want, D, G, eps);
    CK(cudaGetLastError());
    e->launches++;
    TRY((product<T, T, float, 0>(e, hw, D, 0, at<T>(e, e->head), D, 1, 0, e->logits, e->cfg.vocab, 0, n_want, e->cfg.vocab, D, 1)));
    finish_logits(e, n_want);
    CK(cudaGetLastError());
  }
  return 0;
}

static void free_state(xotb200_lm* e) {
  for (auto& L : e->layers)
    if (L.pool) { cudaFree(L.pool); L.pool = nullptr; }
  if (e->h_table) { cudaFreeHost(e->h_table); e->h_table = nullptr; }
  if (e->d_table) { cudaFree(e->d_table); e->d_table = nullptr; }
  if (e->state) { cudaFree(e->state); e->state = nullptr; }
  e->max_requests = 0;
}

// ---------------------------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------------------------
extern "C" {

const char* xotb200_lm_last_error(void) { return g_err; }
const char* xotb200_lm_version(void) { return "xotb200_lm 0.1.0 sm_100a"; }

int xotb200_lm_create(const xotb200_lm_cfg* cfg, const xotb200_lm_layer* layers, int device, xotb200_lm** out) {
  REQUIRE(cfg && layers && out, "null argument");
  REQUIRE(cfg->dtype == XOTB200_LM_DTYPE_BF16 || cfg->dtype == XOTB200_LM_DTYPE_F32, "dtype must be bf16 (0) or f32 (2), got %d", cfg->dtype);
  REQUIRE(cfg->n_layers >= 1 && 0 <= cfg->start_layer && cfg->start_layer <= cfg->end_layer && cfg->end_layer < cfg->n_layers,
          "bad layer range [%d, %d] of %d", cfg->start_layer, cfg->end_layer, cfg->n_layers);
  REQUIRE(cfg->width >= 1 && cfg->vocab >= 1, "width and vocab must be positive");
  REQUIRE(cfg->norm_groups >= 1 && cfg->width % cfg->norm_groups == 0, "width %d is not a multiple of norm_groups %d", cfg->width, cfg->norm_groups);
  REQUIRE(cfg->block == XOTB200_LM_BLOCK_GROUP_RMS || cfg->block == XOTB200_LM_BLOCK_POST_LN || cfg->block == XOTB200_LM_BLOCK_POST_RMS ||
              cfg->block == XOTB200_LM_BLOCK_PRE_SCALAR,
          "unknown block form %d", cfg->block);
  REQUIRE(cfg->block == XOTB200_LM_BLOCK_PRE_SCALAR || (cfg->streams == 0 && cfg->canon_taps == 0 && cfg->residual_mult == 0.f),
          "stream copies, input convolutions and a residual multiplier belong to the pre-norm block with one-number weights");
  REQUIRE(cfg->streams >= 0 && cfg->streams <= HC_MAX_STREAMS && cfg->canon_taps >= 0 && cfg->canon_taps <= 64, "streams 0..%d, convolution taps 0..64", HC_MAX_STREAMS);
  REQUIRE(cfg->block != XOTB200_LM_BLOCK_PRE_SCALAR || (cfg->start_layer == 0 && cfg->end_layer == cfg->n_layers - 1),
          "a model whose stream is kept in several copies runs as one shard");
  REQUIRE(cfg->max_positions >= 0, "negative max_positions");
  REQUIRE(cfg->block != XOTB200_LM_BLOCK_GROUP_RMS || (!cfg->pos_sinusoid && !cfg->embed_norm),
          "a computed position vector and a norm on the embedding belong to the other block forms");
  REQUIRE(cfg->block != XOTB200_LM_BLOCK_PRE_SCALAR || (!cfg->pos_sinusoid && cfg->max_positions == 0), "the one-number pre-norm block form adds no position vector");
  REQUIRE(!cfg->embed_norm || cfg->block == XOTB200_LM_BLOCK_POST_RMS || cfg->block == XOTB200_LM_BLOCK_PRE_SCALAR,
          "the norm on the embedding is the RMS norm of the post-RMS or the one-number pre-norm block form");
  REQUIRE(!cfg->pos_sinusoid || cfg->sinusoid_base > 0.f, "the computed position vector needs a positive base");
  REQUIRE(cfg->logit_softcap >= 0.f, "negative logit soft cap");
  int ndev = 0;
  CK(cudaGetDeviceCount(&ndev));
  REQUIRE(device >= 0 && device < ndev, "device %d out of range (%d visible)", device, ndev);
  CK(cudaSetDevice(device));
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, device));
  REQUIRE(prop.major == 10, "libxotb200_lm is sm_100a-only; device %d is sm_%d%d", device, prop.major, prop.minor);
  xotb200_lm* e = new xotb200_lm();
  e->cfg = *cfg;
  e->device = device;
  e->sm_count = prop.multiProcessorCount;
  e->first = cfg->start_layer == 0;
  e->last = cfg->end_layer == cfg->n_layers - 1;
  e->esz = cfg->dtype == XOTB200_LM_DTYPE_F32 ? 4 : 2;
  int rc = build_layout(e, layers);
  if (rc < 0) { delete e; return rc; }
  auto fail = [&](int code) { xotb200_lm_destroy(e); return code; };
  if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess || cudaStreamCreateWithFlags(&e->side, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&e->ev_fork, cudaEventDisableTiming) != cudaSuccess || cudaEventCreateWithFlags(&e->ev_join, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreate(&e->ev0) != cudaSuccess ||
      cudaEventCreate(&e->ev1) != cudaSuccess || cudaMalloc(&e->blob, e->blob_elems * e->esz) != cudaSuccess) {
    set_err("device allocation of %zu weight bytes failed: %s", e->blob_elems * e->esz, cudaGetErrorString(cudaGetLastError()));
    return fail(XOTB200_ECUDA);
  }
  cudaMemsetAsync(e->blob, 0, e->blob_elems * e->esz, e->stream);
  if (cudaMalloc(&e->d_err, 4) != cudaSuccess || cudaHostAlloc(&e->h_err, 4, cudaHostAllocDefault) != cudaSuccess) {
    set_err("allocation of the error word failed");
    return fail(XOTB200_ECUDA);
  }
  cudaMemsetAsync(e->d_err, 0, 4, e->stream);
  *e->h_err = 0;
  for (auto& L : e->layers) {
    if ((L.s.mixer != XOTB200_LM_MIX_LATENT_ATTN && L.s.mixer != XOTB200_LM_MIX_ATTENTION) || L.s.rot_dims == 0) continue;
    std::vector<float> f(L.s.rot_dims / 2);
    for (int i = 0; i < L.s.rot_dims / 2; ++i) {
      double fi = pow((double)L.s.rot_base, -2.0 * i / L.s.rot_dims);
      if (L.s.mixer == XOTB200_LM_MIX_ATTENTION && L.s.rot_scale_factor > 0.f) {
        // long wavelengths are stretched by `factor`, short ones stay, the band between is blended by where the wavelength lies in it
        const double orig = L.s.rot_scale_original, lo = L.s.rot_scale_low, hi = L.s.rot_scale_high, fac = L.s.rot_scale_factor;
        const double wl = 2.0 * M_PI / fi;
        if (wl > orig / lo) fi = fi / fac;
        else if (wl >= orig / hi) { const double sm = (orig / wl - lo) / (hi - lo); fi = (1.0 - sm) * fi / fac + sm * fi; }
      }
      f[i] = (float)fi;
    }
    if (cudaMalloc(&L.freqs, f.size() * 4) != cudaSuccess ||
        cudaMemcpyAsync(L.freqs, f.data(), f.size() * 4, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
        cudaStreamSynchronize(e->stream) != cudaSuccess) {
      set_err("rotation table allocation failed");
      return fail(XOTB200_ECUDA);
    }
  }
  if (e->first && cfg->pos_sinusoid) {
    const int n = (cfg->width + 1) / 2;
    std::vector<float> f(n);
    for (int i = 0; i < n; ++i) f[i] = (float)pow((double)cfg->sinusoid_base, -2.0 * i / cfg->width);
    if (cudaMalloc(&e->pos_freqs, (size_t)n * 4) != cudaSuccess ||
        cudaMemcpyAsync(e->pos_freqs, f.data(), (size_t)n * 4, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
        cudaStreamSynchronize(e->stream) != cudaSuccess) {
      set_err("position frequency table allocation failed");
      return fail(XOTB200_ECUDA);
    }
  }
  for (auto& L : e->layers) {
    if (L.s.mixer != XOTB200_LM_MIX_ATTENTION || L.s.rel_buckets <= 0) continue;
    // bucket of every distance up to the first one that falls into the last bucket (all larger distances do too), in double
    const int B = L.s.rel_buckets, half = B / 2;
    const double span = log((double)L.s.rel_max / half);
    std::vector<int> bk;
    for (int n = 0;; ++n) {
      int b = n;
      if (n >= half) b = std::min(B - 1, half + (int)floor(log((double)n / half) / span * (B - half)));
      bk.push_back(b);
      if (b == B - 1) break;
    }
    L.rel_n = (int)bk.size();
    if (cudaMalloc(&L.rel_bucket, bk.size() * 4) != cudaSuccess || cudaMalloc(&L.rel_tab, bk.size() * L.s.heads * 4) != cudaSuccess ||
        cudaMemcpyAsync(L.rel_bucket, bk.data(), bk.size() * 4, cudaMemcpyHostToDevice, e->stream) != cudaSuccess ||
        cudaStreamSynchronize(e->stream) != cudaSuccess) {
      set_err("distance bucket table allocation failed");
      return fail(XOTB200_ECUDA);
    }
  }
  cudaStreamSynchronize(e->stream);
  *out = e;
  return 0;
}

// tables that are functions of weights: the learned distance bias per head and distance.  Remade before the first step after any
// weight has changed; never inside a captured step.
static int refresh_tables(xotb200_lm* e) {
  if (!e->tables_stale) return 0;
  for (auto& L : e->layers) {
    if (!L.rel_tab) continue;
    const long n = (long)L.s.heads * L.rel_n;
    if (e->esz == 2) gqa_rel_table_kernel<bf16><<<cdiv(n, 256), 256, 0, e->stream>>>(at<bf16>(e, L.rel), L.rel_bucket, L.s.heads, L.rel_n, L.rel_tab);
    else gqa_rel_table_kernel<float><<<cdiv(n, 256), 256, 0, e->stream>>>(at<float>(e, L.rel), L.rel_bucket, L.s.heads, L.rel_n, L.rel_tab);
    CK(cudaGetLastError());
    e->launches++;
  }
  e->tables_stale = false;
  return 0;
}

int xotb200_lm_destroy(xotb200_lm* e) {
  if (!e) return 0;
  cudaSetDevice(e->device);
  if (e->stream) cudaStreamSynchronize(e->stream);
  drop_graphs(e);
  free_state(e);
  for (auto& L : e->layers) {
    if (L.freqs) cudaFree(L.freqs);
    if (L.rel_bucket) cudaFree(L.rel_bucket);
    if (L.rel_tab) cudaFree(L.rel_tab);
  }
  void* ptrs[] = {e->oh2, e->y2, e->h0, e->gdec, e->ginw, e->gfloor, e->gnq, e->pos_freqs, e->dist_tab, e->moe_xg, e->moe_yg, e->moe_plan, e->dkk, e->drr, e->cvb, e->moe_ids, e->moe_wts, e->mact, e->du, e->dau, e->part, e->q16, e->cbuf, e->knx, e->vxx, e->blob, e->d_stage, e->x, e->y, e->proj, e->qraw, e->qfull, e->wlog, e->oraw, e->logits, e->h, e->cqn, e->qn, e->olat, e->oh, e->act,
                  e->th, e->hw, e->d_argmax, e->trace_buf};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  if (e->h_stage) cudaFreeHost(e->h_stage);
  if (e->h_out) cudaFreeHost(e->h_out);
  if (e->h_err) cudaFreeHost(e->h_err);
  if (e->d_err) cudaFree(e->d_err);
  if (e->ev0) cudaEventDestroy(e->ev0);
  if (e->ev1) cudaEventDestroy(e->ev1);
  if (e->ev_fork) cudaEventDestroy(e->ev_fork);
  if (e->ev_join) cudaEventDestroy(e->ev_join);
  if (e->side) cudaStreamDestroy(e->side);
  if (e->stream) cudaStreamDestroy(e->stream);
  delete e;
  return 0;
}

int xotb200_lm_load_tensor(xotb200_lm* e, const char* name, const void* bits, const int64_t* shape, int ndim) {
  REQUIRE(e && name && bits && shape, "null argument");
  CK(cudaSetDevice(e->device));
  auto it = e->dests.find(name);
  if (it == e->dests.end()) {
    if (!owned_name(e, name)) return 1;
    set_err("tensor '%s' is not part of this model", name);
    return XOTB200_ESTRICT;
  }
  Dest& d = it->second;
  const bool ok = (ndim == 2 && shape[0] == d.rows && shape[1] == d.cols) || (ndim == 1 && d.rows == 1 && shape[0] == d.cols) ||
                  (ndim == 0 && d.rows == 1 && d.cols == 1);
  if (!ok) {
    set_err("tensor '%s': shape [%lld%s%lld] does not fit the model's [%d, %d]", name, (long long)shape[0], ndim > 1 ? ", " : "", ndim > 1 ? (long long)shape[1] : 0LL,
            d.rows, d.cols);
    return XOTB200_ESTRICT;
  }
  return upload_tensor(e, d, bits);
}

int xotb200_lm_init_synthetic(xotb200_lm* e, uint64_t seed) {
  REQUIRE(e, "null engine");
  CK(cudaSetDevice(e->device));
  uint64_t k = 0;
  for (auto& kv : e->dests) {
    Dest& d = kv.second;
    const std::string& name = kv.first;
    const size_t n = (size_t)d.rows * d.cols, off = d.elem_off + (size_t)d.row_off * d.cols + (d.il8 == 1 ? n : 0);   // interleaved pairs: any split will do
    float mean = 0.f, dev = 1.0f / sqrtf((float)d.cols);
    const auto ends = [&](const char* suf) { const size_t n = strlen(suf); return name.size() >= n && name.compare(name.size() - n, n, suf) == 0; };
    const bool block_norm = name.find(".mix.") == std::string::npos && name.find("norm") != std::string::npos;
    if (block_norm && e->cfg.block == XOTB200_LM_BLOCK_POST_RMS) dev = 0.1f;   // closing RMS norms: weights stored around zero
    else if (ends(".r1")) { mean = 0.1f; dev = 0.03f; }              // distance penalties stay positive
    else if (ends(".r2")) { mean = 1.f; dev = 0.2f; }
    else if (ends(".b") && d.rows == 1) dev = 0.1f;            // biases of projections and layer norms
    else if (ends(".A_log")) dev = 0.3f;
    else if (name.find("norm") != std::string::npos) { mean = 1.f; dev = 0.1f; }
    else if (d.rows == 1) dev = 0.5f;                  // biases of the delta-rule gates
    else if (name == "embed") dev = 1.f;
    const int grid = (int)std::min<size_t>(8192, (n + 255) / 256);
    if (e->esz == 2) fill_random_kernel<bf16><<<grid, 256, 0, e->stream>>>(at<bf16>(e, off), n, seed * 1000003ull + (++k), mean, dev);
    else fill_random_kernel<float><<<grid, 256, 0, e->stream>>>(at<float>(e, off), n, seed * 1000003ull + (++k), mean, dev);
    CK(cudaGetLastError());
    e->launches++;
    if (d.has2) {   // the row-major copy is the random one's transpose back: both layouts hold the same matrix
      const int dh = d.rows / d.tr_heads;
      if (e->esz == 2) untranspose_heads_kernel<bf16><<<grid, 256, 0, e->stream>>>(at<bf16>(e, off), at<bf16>(e, d.elem_off2), d.tr_heads, dh, d.cols);
      else untranspose_heads_kernel<float><<<grid, 256, 0, e->stream>>>(at<float>(e, off), at<float>(e, d.elem_off2), d.tr_heads, dh, d.cols);
      CK(cudaGetLastError());
      e->launches++;
    }
    d.loaded = true;
  }
  e->tables_stale = true;
  CK(cudaStreamSynchronize(e->stream));
  return 0;
}

int xotb200_lm_check_loaded(xotb200_lm* e) {
  REQUIRE(e, "null engine");
  for (auto& kv : e->dests)
    if (!kv.second.loaded) {
      set_err("tensor '%s' has not been loaded", kv.first.c_str());
      return XOTB200_ESTRICT;
    }
  return 0;
}

int xotb200_lm_load_dir(xotb200_lm* e, const char* dir) {
  REQUIRE(e && dir, "null argument");
  CK(cudaSetDevice(e->device));
  DIR* dp = opendir(dir);
  if (!dp) { set_err("cannot open directory %s", dir); return XOTB200_EIO; }
  std::vector<std::string> files;
  while (dirent* de = readdir(dp)) {
    const std::string n = de->d_name;
    if (n.size() > 12 && n.substr(n.size() - 12) == ".safetensors") files.push_back(std::string(dir) + "/" + n);
  }
  closedir(dp);
  std::sort(files.begin(), files.end());
  if (files.empty()) { set_err("no *.safetensors in %s", dir); return XOTB200_EIO; }
  for (auto& kv : e->dests) kv.second.loaded = false;
  for (const std::string& path : files) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) { set_err("cannot open %s", path.c_str()); return XOTB200_EIO; }
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); set_err("%s: too short", path.c_str()); return XOTB200_EIO; }
    const char* base = static_cast<const char*>(mmap(nullptr, sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0));
    close(fd);
    if (base == MAP_FAILED) { set_err("%s: mmap failed", path.c_str()); return XOTB200_EIO; }
    int rc = 0;
    uint64_t hlen = 0;
    memcpy(&hlen, base, 8);
    std::map<std::string, StEntry> hdr;
    if (hlen > (uint64_t)sb.st_size - 8 || !parse_st_header(base + 8, hlen, hdr)) {
      set_err("%s: bad safetensors header", path.c_str());
      rc = XOTB200_EIO;
    }
    const char* data = base + 8 + hlen;
    const int64_t data_len = sb.st_size - 8 - (int64_t)hlen;
    for (auto it = hdr.begin(); rc == 0 && it != hdr.end(); ++it) {
      const StEntry& en = it->second;
      auto d = e->dests.find(it->first);
      if (d == e->dests.end()) {
        if (!owned_name(e, it->first)) continue;
        set_err("%s: tensor '%s' is not part of this model", path.c_str(), it->first.c_str());
        rc = XOTB200_ESTRICT;
        break;
      }
      int64_t n = 1;
      for (int64_t v : en.shape) n *= v;
      if (en.dtype != "BF16") { set_err("tensor '%s': dtype %s, expected BF16", it->first.c_str(), en.dtype.c_str()); rc = XOTB200_ESTRICT; break; }
      if (en.begin < 0 || en.end > data_len || en.end - en.begin != n * 2) { set_err("tensor '%s': inconsistent data_offsets", it->first.c_str()); rc = XOTB200_EIO; break; }
      if (en.shape.size() > 2) { set_err("tensor '%s': %zu dimensions", it->first.c_str(), en.shape.size()); rc = XOTB200_ESTRICT; break; }
      const int64_t one = 1;                               // a tensor without dimensions is one number
      rc = xotb200_lm_load_tensor(e, it->first.c_str(), data + en.begin, en.shape.empty() ? &one : en.shape.data(), en.shape.empty() ? 1 : (int)en.shape.size());
    }
    munmap(const_cast<char*>(base), sb.st_size);
    if (rc < 0) return rc;
  }
  return xotb200_lm_check_loaded(e);
}

int xotb200_lm_begin(xotb200_lm* e, int max_tokens, int max_requests, int page_size) {
  REQUIRE(e, "null engine");
  REQUIRE(max_tokens >= 1 && max_requests >= 1 && max_requests <= 4096, "max_tokens >= 1 and 1 <= max_requests <= 4096 required");
  REQUIRE(page_size >= 0 && page_size <= 4096, "page_size out of range");
  CK(cudaSetDevice(e->device));
  CK(cudaStreamSynchronize(e->stream));
  drop_graphs(e);
  free_state(e);
  const int P = page_size > 0 ? page_size : 64;
  e->page_size = P;
  e->max_requests = max_requests;
  // every live request may hold one partly filled page: max_requests pages of slack
  e->n_pages = cdiv(max_tokens, P) + max_requests;
  e->pages_per_slot = cdiv(max_tokens, P) + 1;
  for (auto& L : e->layers) {
    size_t row = 0;                                    // elements a token holds in this layer's pool
    if (L.s.mixer == XOTB200_LM_MIX_LATENT_ATTN) row = (size_t)L.s.kv_rank + L.s.rot_dim;
    else if (L.s.mixer == XOTB200_LM_MIX_ATTENTION && L.s.kv_from < 0) row = (size_t)L.s.kv_heads * (L.s.dim + L.s.vdim);
    if (!row) continue;
    // a layer with pooled blocks keeps them in a second half of the same geometry (block b where token b lives in the first half)
    const size_t bytes = (size_t)e->n_pages * P * row * e->esz * (L.s.mixer == XOTB200_LM_MIX_ATTENTION && L.s.pool > 0 ? 2 : 1);
    CK(cudaMalloc(&L.pool, bytes));
    CK(cudaMemsetAsync(L.pool, 0, bytes, e->stream));
  }
  const size_t tab = (size_t)max_requests * e->pages_per_slot;
  CK(cudaHostAlloc(&e->h_table, tab * 4, cudaHostAllocDefault));
  memset(e->h_table, 0, tab * 4);
  CK(cudaMalloc(&e->d_table, tab * 4));
  CK(cudaMemsetAsync(e->d_table, 0, tab * 4, e->stream));
  if (e->state_floats) {
    CK(cudaMalloc(&e->state, (size_t)max_requests * e->state_floats * 4));
    CK(cudaMemsetAsync(e->state, 0, (size_t)max_requests * e->state_floats * 4, e->stream));
  }
  e->free_pages.clear();
  for (int p = e->n_pages - 1; p >= 0; --p) e->free_pages.push_back(p);   // pages are handed out from the back: 0, 1, 2, ...
  e->slot_len.assign(max_requests, 0);
  e->slot_pages.assign(max_requests, 0);
  CK(cudaStreamSynchronize(e->stream));
  return 0;
}

int xotb200_lm_clear_request(xotb200_lm* e, int slot) {
  REQUIRE(e && e->max_requests > 0, "no request state: call xotb200_lm_begin first");
  REQUIRE(slot >= 0 && slot < e->max_requests, "slot %d out of range (%d)", slot, e->max_requests);
  CK(cudaSetDevice(e->device));
  for (int i = e->slot_pages[slot] - 1; i >= 0; --i) e->free_pages.push_back(e->h_table[(size_t)slot * e->pages_per_slot + i]);
  e->slot_pages[slot] = 0;
  e->slot_len[slot] = 0;
  if (e->state_floats) {
    CK(cudaMemsetAsync(e->state + (size_t)slot * e->state_floats, 0, e->state_floats * 4, e->stream));
    CK(cudaStreamSynchronize(e->stream));
  }
  return 0;
}

int xotb200_lm_request_len(xotb200_lm* e, int slot, int* len) {
  REQUIRE(e && len && slot >= 0 && slot < e->max_requests, "bad argument");
  *len = e->slot_len[slot];
  return 0;
}

int xotb200_lm_step(xotb200_lm* e, int n_seq, const int32_t* slots, const int32_t* counts, const int32_t* tokens, const float* hidden_f32,
                    const int32_t* want_rows, int n_want, float* logits_f32, int32_t* argmax_i32, float* hidden_out_f32) {
  REQUIRE(e && slots && counts && n_seq >= 1, "bad argument");
  REQUIRE(e->max_requests > 0, "no request state: call xotb200_lm_begin first");
  REQUIRE(e->first ? tokens != nullptr : hidden_f32 != nullptr, "the first shard takes token ids, every other shard the hidden state");
  REQUIRE(e->last || hidden_out_f32, "a shard that is not the last returns the hidden state");
  CK(cudaSetDevice(e->device));
  TRY(xotb200_lm_check_loaded(e));
  if (!e->last) n_want = 0;
  const int D = e->cfg.width, V = e->cfg.vocab, P = e->page_size;
  // ---- validate and plan on the host; nothing is changed before every check has passed
  long M = 0;
  int need_pages = 0;
  std::vector<char> seen(e->max_requests, 0);
  for (int i = 0; i < n_seq; ++i) {
    REQUIRE(slots[i] >= 0 && slots[i] < e->max_requests, "slot %d out of range (%d)", slots[i], e->max_requests);
    REQUIRE(!seen[slots[i]], "slot %d appears twice in one step", slots[i]);
    seen[slots[i]] = 1;
    REQUIRE(counts[i] >= 1, "request %d brings %d rows", i, counts[i]);
    const int len = e->slot_len[slots[i]] + counts[i];
    REQUIRE(cdiv(len, P) <= e->pages_per_slot, "slot %d would hold %d tokens, more than the cache was sized for", slots[i], len);
    REQUIRE(e->cfg.max_positions == 0 || len <= e->cfg.max_positions, "slot %d would hold %d tokens, the model has %d positions", slots[i], len,
            e->cfg.max_positions);
    need_pages += cdiv(len, P) - e->slot_pages[slots[i]];
    M += counts[i];
  }
  REQUIRE(M < (1L << 30), "too many rows");
  REQUIRE(need_pages <= (int)e->free_pages.size(), "latent cache full: %d pages needed, %zu free (sized for fewer live tokens)", need_pages,
          e->free_pages.size());
  for (int w = 0; w < n_want; ++w) REQUIRE(want_rows && want_rows[w] >= 0 && want_rows[w] < M, "wanted row out of range");
  if (e->first)
    for (long m = 0; m < M; ++m) REQUIRE(tokens[m] >= 0 && tokens[m] < V, "token id %d outside the vocabulary of %d", tokens[m], V);
  TRY(ensure_scratch(e, (int)M, n_want));
  TRY(refresh_tables(e));
  // ---- commit: pages and lengths; the step's index arrays are built in one host vector and copied once
  const bool use_flash = e->esz == 2 && e->flash_on && e->flash_fits;
  std::vector<int> qpis, windows;
  for (auto& L : e->layers)
    if (L.s.mixer == XOTB200_LM_MIX_LATENT_ATTN) {
      const int q = std::max(1, 32 / L.s.heads);
      if (std::find(qpis.begin(), qpis.end(), q) == qpis.end()) qpis.push_back(q);
      if (use_flash && std::find(windows.begin(), windows.end(), L.s.window) == windows.end()) windows.push_back(L.s.window);
    } else if (L.s.mixer == XOTB200_LM_MIX_ATTENTION) {
      const int q = -gqa_rows_per_item(L.s);             // negative: a list of the key/value-cache attention (its own rule for long portions)
      if (std::find(qpis.begin(), qpis.end(), q) == qpis.end()) qpis.push_back(q);
    }
  std::vector<int>& st = e->stage_build;
  st.assign(3 * (size_t)M + n_want, 0);
  std::vector<Item> seqs(n_seq);
  StepPlan sp;
  sp.M = (int)M;
  sp.n_seq = n_seq;
  int row = 0;
  for (int i = 0; i < n_seq; ++i) {
    const int sl = slots[i], len0 = e->slot_len[sl], len1 = len0 + counts[i];
    const int np0 = e->slot_pages[sl], np1 = cdiv(len1, P);
    for (int p = np0; p < np1; ++p) {
      e->h_table[(size_t)sl * e->pages_per_slot + p] = e->free_pages.back();
      e->free_pages.pop_back();
    }
    if (np1 > np0)
      CK(cudaMemcpyAsync(e->d_table + (size_t)sl * e->pages_per_slot + np0, e->h_table + (size_t)sl * e->pages_per_slot + np0, (size_t)(np1 - np0) * 4,
                         cudaMemcpyHostToDevice, e->stream));
    e->slot_pages[sl] = np1;
    e->slot_len[sl] = len1;
    seqs[i] = Item{row, counts[i], sl, len0};
    sp.max_len = std::max(sp.max_len, len1);
    sp.max_rows = std::max(sp.max_rows, counts[i]);
    for (int t = 0; t < counts[i]; ++t, ++row) {
      st[row] = e->first ? tokens[row] : 0;
      st[M + row] = sl;
      st[2 * M + row] = len0 + t;
    }
  }
  for (int w = 0; w < n_want; ++w) st[3 * M + w] = want_rows[w];
  auto push = [&](const void* p, size_t n_ints) { const size_t o = st.size(); const int* q = static_cast<const int*>(p); st.insert(st.end(), q, q + n_ints); return o; };
  const size_t off_seqs = push(seqs.data(), 4 * (size_t)n_seq);
  auto is_long = [&](int i) { return use_flash && counts[i] >= FLASH_MIN_ROWS; };
  std::map<int, std::pair<size_t, int>> item_off;
  sp.any_short = false;
  const bool use_gqa_flash = e->esz == 2 && e->flash_on && e->gqa_flash_fits;
  auto is_long_gqa = [&](int i) { return use_gqa_flash && counts[i] >= FLASH_MIN_ROWS; };
  for (int qk : qpis) {
    std::vector<Item> it;
    const int q = qk < 0 ? -qk : qk;
    for (int i = 0; i < n_seq; ++i)
      if (qk < 0 ? !is_long_gqa(i) : !is_long(i))
        for (int t = 0; t < counts[i]; t += q) it.push_back(Item{seqs[i].row0 + t, std::min(q, counts[i] - t), seqs[i].slot, seqs[i].pos0 + t});
    item_off[qk] = {push(it.data(), 4 * it.size()), (int)it.size()};
    if (!it.empty() && qk > 0) sp.any_short = true;
  }
  size_t gqa_tiles_off = 0;
  int n_gqa_tiles = 0;
  if (use_gqa_flash && std::any_of(qpis.begin(), qpis.end(), [](int q) { return q < 0; })) {
    std::vector<GqaTile> gt;
    for (int i = 0; i < n_seq; ++i)
      if (is_long_gqa(i))
        for (int t = 0; t < counts[i]; t += 64) gt.push_back(GqaTile{seqs[i].row0 + t, std::min(64, counts[i] - t), seqs[i].pos0 + t, seqs[i].slot});
    gqa_tiles_off = push(gt.data(), 4 * gt.size());
    n_gqa_tiles = (int)gt.size();
  }
  struct FlashOff { size_t reqs, tiles; int n_reqs, n_tiles, n_keys, max_keys; };
  std::map<int, FlashOff> flash_off;
  size_t flash_keys = 0;
  for (int w : windows) {
    std::vector<GatherReq> gr;
    std::vector<FlashTile> ft;
    int kbase = 0, max_keys = 0;
    for (int i = 0; i < n_seq; ++i)
      if (is_long(i)) {
        const int kfirst = w > 0 ? std::max(0, seqs[i].pos0 - w + 1) : 0;
        const int nkeys = seqs[i].pos0 + counts[i] - kfirst;
        gr.push_back(GatherReq{seqs[i].slot, kfirst, nkeys, kbase});
        for (int t = 0; t < counts[i]; t += 64) ft.push_back(FlashTile{seqs[i].row0 + t, std::min(64, counts[i] - t), seqs[i].pos0 + t, kbase, kfirst});
        kbase += nkeys;
        max_keys = std::max(max_keys, nkeys);
      }
    if (gr.empty()) continue;
    flash_off[w] = FlashOff{push(gr.data(), 4 * gr.size()), push(ft.data(), 5 * ft.size()), (int)gr.size(), (int)ft.size(), kbase, max_keys};
    flash_keys = std::max(flash_keys, (size_t)kbase);
  }
  if (flash_keys > e->flash_keys_cap) {
    const size_t cap = std::max<size_t>(flash_keys, 1024);
    TRY(regrow(e->cbuf, cap * e->max_w * 2));
    TRY(regrow(e->knx, cap * e->max_hdn * 2));
    TRY(regrow(e->vxx, cap * e->max_oh * 2));
    e->flash_keys_cap = cap;
  }
  const size_t off = st.size();
  if (off > e->stage_cap) {
    drop_graphs(e);
    CK(cudaStreamSynchronize(e->stream));
    if (e->h_stage) cudaFreeHost(e->h_stage);
    if (e->d_stage) cudaFree(e->d_stage);
    e->h_stage = nullptr; e->d_stage = nullptr; e->stage_cap = 0;
    const size_t cap = std::max<size_t>(off * 2, 4096);
    CK(cudaHostAlloc(&e->h_stage, cap * 4, cudaHostAllocDefault));
    CK(cudaMalloc(&e->d_stage, cap * 4));
    e->stage_cap = cap;
  }
  memcpy(e->h_stage, st.data(), off * 4);
  if (e->last && n_want > 0) TRY(ensure_host_out(e, (size_t)n_want * V + n_want));
  else if (!e->last) TRY(ensure_host_out(e, (size_t)M * D));
  // Decoding — every request brings one row — has the same launches step after step: only the contents of the index arrays and
  // the lengths differ.  Such a step is captured into a CUDA graph the second time its shape is seen and replayed from then on.
  // What the launches depend on is in the key; the key length is a bucket of the longest request (it fixes how the absorbed
  // attention kernel cuts the keys into runs).
  const bool decode_shape = e->graphs_on && e->first && !e->trace && M == n_seq;
  sp.max_len = decode_shape ? cdiv(sp.max_len, 256) * 256 : sp.max_len;
  // the key-run buffer is sized before anything is captured: a captured step must not replace a buffer
  for (auto& L : e->layers)
    if (L.s.mixer == XOTB200_LM_MIX_ATTENTION) {
      int run = 0;
      const int splits = gqa_key_runs(e, L.s, item_off[-gqa_rows_per_item(L.s)].second, sp.max_len, &run);
      const size_t need = splits > 1 ? (size_t)M * L.s.heads * splits * (2 + L.s.vdim) : 0;
      if (need > e->part_cap) { drop_graphs(e); TRY(regrow(e->part, need * 4)); e->part_cap = need; }
    }
  GraphSlot* gs = nullptr;
  if (decode_shape) {
    const std::array<long, 5> key{n_seq, n_want, (logits_f32 ? 1 : 0) | (argmax_i32 ? 2 : 0), sp.max_len, (long)off};
    gs = &e->graphs[key];
  }
  CK(cudaEventRecord(e->ev0, e->stream));
  if (gs && gs->exec) {
    CK(cudaGraphLaunch(gs->exec, e->stream));
    e->launches += gs->launches;
    e->graph_replays++;
  } else {
    const bool capture = gs && gs->seen >= 1;
    if (gs) gs->seen++;
    const int64_t launches0 = e->launches;
    if (capture) CK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
    int rc = 0;
    auto body = [&]() -> int {
      CK(cudaMemcpyAsync(e->d_stage, e->h_stage, off * 4, cudaMemcpyHostToDevice, e->stream));
      sp.tokens = e->d_stage;
      sp.row_slot = e->d_stage + M;
      sp.row_pos = e->d_stage + 2 * M;
      sp.want = e->d_stage + 3 * M;
      sp.seqs = reinterpret_cast<const Item*>(e->d_stage + off_seqs);
      for (auto& kv : item_off) sp.items[kv.first] = {reinterpret_cast<const Item*>(e->d_stage + kv.second.first), kv.second.second};
      sp.gqa_tiles = reinterpret_cast<const GqaTile*>(e->d_stage + gqa_tiles_off);
      sp.n_gqa_tiles = n_gqa_tiles;
      for (auto& kv : flash_off) {
        StepPlan::Flash f;
        f.reqs = reinterpret_cast<const GatherReq*>(e->d_stage + kv.second.reqs);
        f.tiles = reinterpret_cast<const FlashTile*>(e->d_stage + kv.second.tiles);
        f.n_reqs = kv.second.n_reqs; f.n_tiles = kv.second.n_tiles; f.n_keys = kv.second.n_keys; f.max_keys = kv.second.max_keys;
        sp.flash[kv.first] = f;
      }
      if (!e->first) CK(cudaMemcpyAsync(e->x, hidden_f32, (size_t)M * D * 4, cudaMemcpyHostToDevice, e->stream));
      TRY(e->esz == 2 ? run_layers<bf16>(e, sp, n_want) : run_layers<float>(e, sp, n_want));
      if (e->last && n_want > 0) {
        if (logits_f32) CK(cudaMemcpyAsync(e->h_out, e->logits, (size_t)n_want * V * 4, cudaMemcpyDeviceToHost, e->stream));
        if (argmax_i32) CK(cudaMemcpyAsync(e->h_out + (size_t)n_want * V, e->d_argmax, (size_t)n_want * 4, cudaMemcpyDeviceToHost, e->stream));
      } else if (!e->last) {
        CK(cudaMemcpyAsync(e->h_out, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToHost, e->stream));
      }
      CK(cudaMemcpyAsync(e->h_err, e->d_err, 4, cudaMemcpyDeviceToHost, e->stream));
      return 0;
    };
    rc = body();
    if (capture) {
      cudaGraph_t graph = nullptr;
      cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
      if (rc == 0 && ce == cudaSuccess && graph && cudaGraphInstantiate(&gs->exec, graph, 0) == cudaSuccess) {
        gs->launches = e->launches - launches0;
        ce = cudaGraphLaunch(gs->exec, e->stream);
      } else if (rc == 0) {
        gs->exec = nullptr;
        set_err("capturing the decode step into a CUDA graph failed: %s", cudaGetErrorString(ce != cudaSuccess ? ce : cudaGetLastError()));
        rc = XOTB200_ECUDA;
      }
      if (graph) cudaGraphDestroy(graph);
      if (rc == 0 && ce != cudaSuccess) { set_err("launching the captured decode step failed: %s", cudaGetErrorString(ce)); rc = XOTB200_ECUDA; }
    }
    if (rc < 0) { cudaStreamSynchronize(e->stream); return rc; }
  }
  CK(cudaEventRecord(e->ev1, e->stream));
  CK(cudaStreamSynchronize(e->stream));
  CK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
  if (*e->h_err != 0) {
    set_err("a kernel gave up a bounded wait (device error word %d); the step's results are not valid", *e->h_err);
    return XOTB200_ECUDA;
  }
  if (e->last && n_want > 0) {
    if (logits_f32) memcpy(logits_f32, e->h_out, (size_t)n_want * V * 4);
    if (argmax_i32) memcpy(argmax_i32, e->h_out + (size_t)n_want * V, (size_t)n_want * 4);
  } else if (!e->last) {
    memcpy(hidden_out_f32, e->h_out, (size_t)M * D * 4);
  }
  return 0;
}

int xotb200_lm_set_trace(xotb200_lm* e, int on) {
  REQUIRE(e, "null engine");
  e->trace = on != 0;
  e->trace_floats = 0;
  return 0;
}

int xotb200_lm_read_trace(xotb200_lm* e, float* out, int64_t n_floats) {
  REQUIRE(e && out, "null argument");
  REQUIRE(e->trace && e->trace_floats > 0, "no trace recorded: enable it before the step");
  REQUIRE((size_t)n_floats == e->trace_floats, "trace holds %zu floats, caller asked for %lld", e->trace_floats, (long long)n_floats);
  CK(cudaSetDevice(e->device));
  CK(cudaMemcpyAsync(out, e->trace_buf, e->trace_floats * 4, cudaMemcpyDeviceToHost, e->stream));
  CK(cudaStreamSynchronize(e->stream));
  return 0;
}

int xotb200_lm_set_gemm_mode(xotb200_lm* e, int mode) {
  REQUIRE(e && mode >= 0 && mode <= 2, "gemm mode must be 0, 1 or 2");
  drop_graphs(e);
  e->gemm_mode = mode;
  return 0;
}

int xotb200_lm_kernel_launches(xotb200_lm* e, int64_t* count) {
  REQUIRE(e && count, "null argument");
  *count = e->launches;
  return 0;
}

int xotb200_lm_set_graphs(xotb200_lm* e, int on) {
  REQUIRE(e, "null engine");
  drop_graphs(e);
  e->graphs_on = on != 0;
  return 0;
}

int xotb200_lm_graph_replays(xotb200_lm* e, int64_t* count) {
  REQUIRE(e && count, "null argument");
  *count = e->graph_replays;
  return 0;
}

int xotb200_lm_set_attention_mode(xotb200_lm* e, int mode) {
  REQUIRE(e && mode >= 0 && mode <= 1, "attention mode must be 0 or 1");
  drop_graphs(e);
  e->flash_on = mode == 0;
  return 0;
}

int xotb200_lm_prompt_attention_launches(xotb200_lm* e, int64_t* count) {
  REQUIRE(e && count, "null argument");
  *count = e->flash_launches;
  return 0;
}

int xotb200_lm_tensor_core_launches(xotb200_lm* e, int64_t* count) {
  REQUIRE(e && count, "null argument");
  *count = e->tc_launches;
  return 0;
}

int xotb200_lm_weight_bytes(xotb200_lm* e, int64_t* bytes) {
  REQUIRE(e && bytes, "null argument");
  *bytes = (int64_t)(e->blob_elems * e->esz);
  return 0;
}

int xotb200_lm_cache_stats(xotb200_lm* e, int* pages_total, int* pages_free, int* page_size) {
  REQUIRE(e, "null engine");
  if (pages_total) *pages_total = e->n_pages;
  if (pages_free) *pages_free = (int)e->free_pages.size();
  if (page_size) *page_size = e->page_size;
  return 0;
}

int xotb200_lm_last_step_ms(xotb200_lm* e, float* ms) {
  REQUIRE(e && ms, "null argument");
  *ms = e->last_ms;
  return 0;
}

}  // extern "C"
