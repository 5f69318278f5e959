// layered_tc.cuh — the bfloat16 products of the layered-model engine on the 5th-generation tensor cores.
//
//   C[z][m, n] = sum_k A[z][m, k] * B[z][n, k]      A, B bf16 and K-major (row stride a multiple of 8 elements), fp32 accumulation
//
// One CTA computes one 128 x NT output tile: a single thread feeds a ring of shared-memory stages with TMA tensor-map loads
// (cp.async.bulk.tensor.3d, SWIZZLE_128B; coordinates {k, row, batch}), a single thread issues tcgen05.mma.cta_group::1.kind::f16
// into a tensor-memory accumulator, four warps read it back with tcgen05.ld and store it (fp32 or bf16, optionally relu(.)^2).
// Rows beyond M, columns beyond N and the tail of K come from the tensor map's zero fill, so no size has to be a multiple of the
// tile.  EPI 1: relu(.)^2; EPI 2: xIELU; EPI 4: exact gelu; EPI 3: the columns come in groups of 16 = 8 gate values followed by their 8 up values, and
// C [*, N / 2] receives silu(gate) * up.  With `tile_batch` every row tile takes its B matrix from a list (grouped products: rows
// sorted by expert).  The PTX wrappers are those of the shard engine's prefill GEMM (prefill_tc.cuh); what differs is the operand layout
// (plain row-major weights, batched per-head products through the third coordinate), the epilogue and that EVERY wait is bounded:
// a wait that expires sets *err and the CTA drains, frees its tensor memory and returns.
#pragma once
#include "layered_kernels.cuh"
#include "prefill_tc.cuh"

namespace xl {

constexpr int LTC_M = 128, LTC_BK = 64, LTC_THREADS = 256;
constexpr unsigned LTC_SPIN_LIMIT = 1u << 22;   // try_wait rounds (each blocks for a while in hardware): seconds, not forever

__host__ __device__ constexpr int ltc_stage_bytes(int nt) { return LTC_M * LTC_BK * 2 + nt * LTC_BK * 2; }
__host__ __device__ constexpr int ltc_smem_bytes(int nt, int ns) { return ns * ltc_stage_bytes(nt) + 1024 + 256; }
// instruction descriptor of kind::f16: fp32 accumulator (bit 4), bf16 A (bits 7..9 = 1) and B (bits 10..12 = 1), both K-major
__host__ __device__ constexpr uint32_t ltc_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ bool ltc_wait(uint64_t* bar, uint32_t parity, int* err) {
  for (unsigned i = 0; i < LTC_SPIN_LIMIT; ++i)
    if (xb::mbar_try_wait(bar, parity)) return true;
  atomicExch(err, 3);
  return false;
}

struct LtcArgs {
  int M, N, K;
  void* C;          // fp32 or bf16 [*, ldc]
  long ldc, c_batch;
  int* err;
  const __nv_bfloat16* epi;   // EPI 2: the two raw xIELU parameters
  const int* tile_batch;      // not NULL: row tile t reads B's batch tile_batch[t] (A and C are not batched); a negative entry = the tile is empty
  int cols_first;             // 1: blockIdx.x walks the column tiles and blockIdx.y the row tiles (CTAs that run together share few row tiles:
                              // a grouped product then streams an expert's matrix while only that expert's rows are in flight)
};

template <typename TC>
__device__ __forceinline__ void ltc_store(TC* p, float v);
template <> __device__ __forceinline__ void ltc_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void ltc_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int NT, int EPI, int NS, typename TC>
__global__ void __launch_bounds__(LTC_THREADS, 2 * ltc_smem_bytes(NT, NS) <= 226 * 1024 ? 2 : 1)
ltc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const LtcArgs a) {
  extern __shared__ __align__(1024) uint8_t ltc_smem[];
  constexpr int A_BYTES = LTC_M * LTC_BK * 2;
  constexpr int STAGE = ltc_stage_bytes(NT);
  constexpr int TMEM_COLS = NT < 32 ? 32 : NT;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ltc_smem) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(base + NS * STAGE);
  uint64_t* empty = full + NS;
  uint64_t* tmem_full = empty + NS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = a.cols_first ? blockIdx.y : blockIdx.x, ntile = a.cols_first ? blockIdx.x : blockIdx.y;
  const int m0 = mt * LTC_M, n0 = ntile * NT, z = blockIdx.z;
  const int nkb = (a.K + LTC_BK - 1) / LTC_BK;
  const int zb = a.tile_batch ? a.tile_batch[mt] : z;
  if (zb < 0) return;                                  // an empty tile of a grouped product: the whole CTA leaves before anything is set up

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) { xb::mbar_init(&full[i], 1); xb::mbar_init(&empty[i], 1); }
    xb::mbar_init(tmem_full, 1);
    xb::fence_mbar_init();
  }
  if (warp == 2) xb::tmem_alloc(tmem_slot, TMEM_COLS);
  xb::tc_fence_before();
  __syncthreads();
  xb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ===== TMA producer =====
    int issued = 0;
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int st = kb % NS;
      ok = ltc_wait(&empty[st], (((unsigned)kb / NS) & 1u) ^ 1u, a.err);
      if (!ok) break;
      uint8_t* sa = base + (size_t)st * STAGE;
      xb::mbar_expect_tx(&full[st], STAGE);
      xb::tma_load_3d(sa, &tmA, kb * LTC_BK, m0, z, &full[st]);
      xb::tma_load_3d(sa + A_BYTES, &tmB, kb * LTC_BK, n0, zb, &full[st]);
      issued = kb + 1;
    }
    if (!ok)   // gave up: let the copies still in flight land before the CTA's shared memory goes away
      for (int kb = max(0, issued - NS); kb < issued; ++kb) ltc_wait(&full[kb % NS], ((unsigned)kb / NS) & 1u, a.err);
  } else if (warp == 1 && lane == 0) {
    // ===== MMA issuer =====
    constexpr uint32_t idesc = ltc_idesc(LTC_M, NT);
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      const int st = kb % NS;
      ok = ltc_wait(&full[st], ((unsigned)kb / NS) & 1u, a.err);
      if (!ok) break;
      xb::tc_fence_after();
      const uint32_t sa = xb::smem_u32(base + (size_t)st * STAGE);
      const uint32_t sb = sa + A_BYTES;
#pragma unroll
      for (int k = 0; k < LTC_BK / 16; ++k)
        xb::umma_bf16(tmem_base, xb::umma_desc_sw128(sa + k * 32), xb::umma_desc_sw128(sb + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
      xb::umma_commit(&empty[st]);
    }
    if (ok) xb::umma_commit(tmem_full);
  } else if (warp >= 4) {
    // ===== epilogue: warp q reads tensor-memory lanes 32q .. 32q+31 = output rows =====
    const int q = warp - 4;
    const int row = m0 + q * 32 + lane;
    if (ltc_wait(tmem_full, 0, a.err)) {
      xb::tc_fence_after();
      TC* crow = static_cast<TC*>(a.C) + (size_t)z * a.c_batch + (size_t)row * a.ldc;
      const bool vec = (sizeof(TC) == 4) && ((a.ldc | a.c_batch) % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.C) & 15) == 0);
      const bool vec16 = (sizeof(TC) == 2) && ((a.ldc | a.c_batch) % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.C) & 15) == 0);
      float ap = 0.f, aq = 0.f;
      if (EPI == 2) { ap = softplusf_(__bfloat162float(a.epi[0])); aq = 0.5f + softplusf_(__bfloat162float(a.epi[1])); }
#pragma unroll 1
      for (int c0 = 0; c0 < NT; c0 += 16) {
        uint32_t v[16];
        xb::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);   // warp-collective: before any row / column test
        const int n = n0 + c0;
        if (row >= a.M || n >= a.N) continue;
        float f[16];
        if constexpr (EPI == 3) {                      // 8 gate values, then their 8 up values -> 8 outputs at columns n / 2 ..
          const int no = n >> 1;
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = siluf_(__uint_as_float(v[j])) * __uint_as_float(v[j + 8]);
          if (sizeof(TC) == 2 && a.ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(a.C) & 15) == 0) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
              pk[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(crow) + no) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) ltc_store<TC>(crow + no + j, f[j]);
          }
        } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          f[j] = __uint_as_float(v[j]);
          if (EPI == 1) { f[j] = fmaxf(f[j], 0.f); f[j] *= f[j]; }
          if (EPI == 2) f[j] = xielu_f(f[j], ap, aq);
          if (EPI == 4) f[j] = gelu_erf_f(f[j]);
        }
        if (vec && n + 16 <= a.N) {
          float4* d4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(crow) + n);
#pragma unroll
          for (int j = 0; j < 4; ++j) d4[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
        } else if (vec16 && n + 16 <= a.N) {
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            pk[j] = *reinterpret_cast<uint32_t*>(&h2);
          }
          uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(crow) + n);
          d4[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          d4[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (n + j < a.N) ltc_store<TC>(crow + n + j, f[j]);
        }
        }
      }
    }
  }
  xb::tc_fence_before();
  __syncthreads();
  if (warp == 2) xb::tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace xl
