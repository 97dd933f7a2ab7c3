// bf16 GEMM on 5th-generation tensor cores (sm_100a): C[M,N] = A * B^T (+ bias) (+ C), fp32 accumulation in TMEM.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0   : TMA producer  (one elected lane issues cp.async.bulk.tensor loads, 128-byte swizzle, no multicast)
//   warp 1   : MMA issuer    (one elected lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2-5: epilogue      (tcgen05.ld TMEM -> registers -> bf16 -> global), one TMEM lane quarter each
// Tile 128 x 256 x 64, 4-stage shared-memory ring (48 KB per stage), two 256-column TMEM accumulators so
// the epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand layouts ("major" = which dim is contiguous in global memory):
//   A K-major : A[M, K]   (activations in a forward projection, dY in dgrad)
//   A MN-major: A^T[K, M] (dY in wgrad: the reduction dim T is the row index)
//   B K-major : B[N, K]   (weights in a forward projection)
//   B MN-major: B^T[K, N] (weights in dgrad, X in wgrad)
// MN-major tiles are fetched as 64x64 boxes so that the shared-memory image is the canonical
// MN-major 128B-swizzle layout (64-element blocks LBO apart, 8-row groups SBO apart).
//
// All waits are bounded (sm100.cuh); on a timeout the kernel records a status word, every role unwinds,
// TMEM is freed and the kernel returns.
#include <cuda_fp8.h>

#include "sm100.cuh"

namespace sb {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE = BM * BK * 2;              // 16 KB
constexpr int B_STAGE = BN * BK * 2;              // 32 KB
constexpr int STAGE_BYTES = A_STAGE + B_STAGE;    // 48 KB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;                       // raster: 16 m-tiles share the concurrently running n-tiles
constexpr int NUM_THREADS = 192;

struct GemmParams {
  __nv_bfloat16* C;
  const __nv_bfloat16* bias;   // [N] or null
  const __nv_bfloat16* residual;  // [M, N] (leading dim ldr) added in the epilogue, or null
  int M, N, K, ldc, ldr;
  int beta;                    // 1: C += result (bf16 read-modify-write)
  uint32_t* status;
  const float* alpha;          // device scalar multiplied into the accumulator (fp8 de-quantisation), or null
  const float* alpha2;         // second device scalar (the other operand's de-quantisation factor), or null
  int a_fmt, b_fmt;            // fp8 operand formats for the instruction descriptor: 0 = e4m3, 1 = e5m2
  // gated-MLP epilogue of the CTA-pair kernel (GLU mode): B = [w1 ; w2] with F rows each, C = [a | b] (ldc >= 2 F);
  // besides C the epilogue writes q = e4m3(silu(a) * b) [M, F] under delayed scaling (ring `hist` of `slots` floats,
  // this call's slot `cur`, de-quantisation factor to `scale_inv`)
  uint8_t* glu_q;
  int glu_F;
  float* glu_hist;
  int glu_slots, glu_cur;
  float* glu_scale_inv;
  // gate backward in the epilogue of the w3 input-gradient product (GLU = 2): C is not written; with g = the product's
  // result and [a | b] read from glu_ab (leading dimension glu_ld_ab), the epilogue writes q [M, 2 F] =
  // e5m2(g * b * silu'(a) | g * silu(a)) under delayed scaling (same ring protocol)
  const __nv_bfloat16* glu_ab;
  int glu_ld_ab;
};

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, m_tiles - first_m);
  const int r = tile - g * per_group;
  mt = first_m + r % gsz;
  nt = r / gsz;
}

// Epilogue of 32 accumulator columns of one row: scale, + bias, + residual, (+ C), bf16, 16-byte stores.
__device__ __forceinline__ void store_chunk(const GemmParams& p, int row, int col0, const uint32_t (&r)[32], float alpha,
                                            __nv_bfloat16* crow) {
  if (row < p.M && col0 < p.N) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int col = col0 + v * 8;
      if (col + 8 <= p.N) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]) * alpha;
        if (p.bias) {
          const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(b2[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
        }
        if (p.residual) {
          const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * p.ldr + col);
          const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(r2[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
        }
        if (p.beta) {
          const uint4 ov = *reinterpret_cast<const uint4*>(crow + col);
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(o2[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
        }
        uint4 out;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
        *reinterpret_cast<uint4*>(crow + col) = out;
      }
    }
  }
}

// EB = bytes per operand element: 2 = bf16 (kind::f16), 1 = fp8 e4m3 / e5m2 (kind::f8f6f4).  A shared-memory row is
// always 128 bytes, so a k-block holds 64 bf16 or 128 fp8 values and every MMA consumes 32 bytes of K.
template <int A_MN, int B_MN, int EB>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // barrier block after the stages
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  constexpr int BKE = 128 / EB;                      // elements of K per k-block
  constexpr int MNB = 128 / EB;                      // MN elements per 128-byte row of an MN-major box
  constexpr int MN_BOX_BYTES = BKE * 128;            // one MN-major box: BKE k-rows of 128 bytes
  const int num_kb = (p.K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt; tile_coords(tile, m_tiles, n_tiles, mt, nt);
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const int k0 = kb * BKE;
          if (A_MN == 0) {
            tma_load_2d(a_dst, &tmA, k0, m0, full_bar(stage));
          } else {
#pragma unroll
            for (int j = 0; j < BM / MNB; ++j) tma_load_2d(a_dst + j * MN_BOX_BYTES, &tmA, m0 + MNB * j, k0, full_bar(stage));
          }
          if (B_MN == 0) {
            tma_load_2d(b_dst, &tmB, k0, n0, full_bar(stage));
          } else {
#pragma unroll
            for (int j = 0; j < BN / MNB; ++j) tma_load_2d(b_dst + j * MN_BOX_BYTES, &tmB, n0 + MNB * j, k0, full_bar(stage));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // let loads that are still in flight land before the CTA exits
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr int UK = 32 / EB;                       // K elements per MMA (32 bytes)
      const uint32_t idesc = EB == 2 ? umma_idesc_bf16(BM, BN, A_MN, B_MN)
                                     : umma_idesc_fp8(BM, BN, A_MN, B_MN, p.a_fmt, p.b_fmt);
      constexpr uint32_t a_lbo = A_MN ? (uint32_t)MN_BOX_BYTES : 16u, a_step = A_MN ? (UK * 128u) >> 4 : 2u;
      constexpr uint32_t b_lbo = B_MN ? (uint32_t)MN_BOX_BYTES : 16u, b_step = B_MN ? (UK * 128u) >> 4 : 2u;
      int stage = 0; uint32_t phase = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        acc_phase[acc] ^= 1u;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint64_t adesc = umma_smem_desc(a_addr, a_lbo, 1024u);
          const uint64_t bdesc = umma_smem_desc(a_addr + A_STAGE, b_lbo, 1024u);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (EB == 2) umma_bf16(d_tmem, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_fp8(d_tmem, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                         // TMEM lane quarter this warp may access
    uint32_t acc_phase[2] = {0u, 0u};
    int local = 0;
    bool ok = true;
    const float alpha = (p.alpha ? p.alpha[0] : 1.f) * (p.alpha2 ? p.alpha2[0] : 1.f);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      int mt, nt; tile_coords(tile, m_tiles, n_tiles, mt, nt);
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      __nv_bfloat16* crow = p.C + size_t(row) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        store_chunk(p, row, n0 + c * 32, r, alpha, crow);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------ CTA-pair kernel (cta_group::2)
// Two CTAs of a cluster (an SM pair) work on one 256 x 256 output tile.  CTA r of the pair stages rows [128 r, 128 r + 128)
// of the A tile and rows [128 r, 128 r + 128) of the B tile (32 KB per stage instead of 48 KB: six stages, and a third
// less shared-memory traffic per FLOP, which is what bounds one-byte operands on a single SM); its TMEM holds the 128
// accumulator rows of its half.  The even CTA's MMA thread issues tcgen05.mma.cta_group::2 for both; its commits
// arrive on the stage barriers of both CTAs.  Loads complete on the even CTA's `full` barrier.  No multicast loads.
constexpr int P_STAGES = 6;
constexpr int P_A_STAGE = 128 * 128;                 // 16 KB: this CTA's 128 rows of A (128-byte rows)
constexpr int P_B_STAGE = 128 * 128;                 // 16 KB: this CTA's 128 rows of B
constexpr int P_STAGE_BYTES = P_A_STAGE + P_B_STAGE;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
constexpr int P_GROUP_M = 8;

__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = P_GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * P_GROUP_M;
  const int gsz = min(P_GROUP_M, m_tiles - first_m);
  const int r = tile - g * per_group;
  mt = first_m + r % gsz;
  nt = r / gsz;
}

// GLU = 1 (K-major one-byte operands only): output tile t covers features [128 t, 128 t + 128) of BOTH halves of the
// packed gate projection: the even CTA stages the w1 rows of those features, the odd CTA the w2 rows, so accumulator
// columns 0-127 hold a and 128-255 hold b of the same features, and the epilogue applies the gate on the spot: it
// stores a and b (bf16, for the backward) and the e4m3 operand of the following projection, which the separate gate
// kernel otherwise produces by re-reading [a | b] from memory.
template <int A_MN, int B_MN, int EB, int GLU = 0>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + P_STAGES * P_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (P_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * P_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * P_STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + P_STAGES * P_STAGE_BYTES + 8 * (2 * P_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + P_STAGES * P_STAGE_BYTES + 8 * (2 * P_STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();             // 0: issues the MMAs, 1: partner
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int m_tiles = (p.M + 255) / 256, n_tiles = GLU == 1 ? p.glu_F / 128 : (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  constexpr int BKE = 128 / EB;
  constexpr int MNB = 128 / EB;
  constexpr int MN_BOX_BYTES = BKE * 128;
  const int num_kb = (p.K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }   // 4 warps of each CTA
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  // barriers of both CTAs are initialised before either signals the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        int mt, nt; pair_tile_coords(tile, m_tiles, n_tiles, mt, nt);
        const int m0 = mt * 256 + int(rank) * 128;
        const int n0 = GLU == 1 ? nt * 128 + int(rank) * p.glu_F : nt * BN + int(rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * P_STAGE_BYTES;
          const uint32_t b_dst = a_dst + P_A_STAGE;
          const uint32_t bar = map_to_cta(full_bar(stage), 0);         // the even CTA counts both CTAs' bytes
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);
          const int k0 = kb * BKE;
          if (A_MN == 0) {
            tma_load_2d_pair(a_dst, &tmA, k0, m0, bar);
          } else {
#pragma unroll
            for (int j = 0; j < 128 / MNB; ++j) tma_load_2d_pair(a_dst + j * MN_BOX_BYTES, &tmA, m0 + MNB * j, k0, bar);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(b_dst, &tmB, k0, n0, bar);
          } else {
#pragma unroll
            for (int j = 0; j < 128 / MNB; ++j) tma_load_2d_pair(b_dst + j * MN_BOX_BYTES, &tmB, n0 + MNB * j, k0, bar);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (rank == 0 && elect_one()) {
      constexpr int UK = 32 / EB;
      const uint32_t idesc = EB == 2 ? umma_idesc_bf16(256, BN, A_MN, B_MN)
                                     : umma_idesc_fp8(256, BN, A_MN, B_MN, p.a_fmt, p.b_fmt);
      constexpr uint32_t a_lbo = A_MN ? (uint32_t)MN_BOX_BYTES : 16u, a_step = A_MN ? (UK * 128u) >> 4 : 2u;
      constexpr uint32_t b_lbo = B_MN ? (uint32_t)MN_BOX_BYTES : 16u, b_step = B_MN ? (UK * 128u) >> 4 : 2u;
      int stage = 0; uint32_t phase = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local) {
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        acc_phase[acc] ^= 1u;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * P_STAGE_BYTES;
          const uint64_t adesc = umma_smem_desc(a_addr, a_lbo, 1024u);
          const uint64_t bdesc = umma_smem_desc(a_addr + P_A_STAGE, b_lbo, 1024u);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (EB == 2) umma_bf16_pair(d_tmem, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_fp8_pair(d_tmem, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));          // frees this stage in both CTAs
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(acc));      // wakes the epilogue warps of both CTAs
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    uint32_t acc_phase[2] = {0u, 0u};
    int local = 0;
    bool ok = true;
    const float alpha = (p.alpha ? p.alpha[0] : 1.f) * (p.alpha2 ? p.alpha2[0] : 1.f);
    float q_scale = 1.f, q_amax = 0.f;
    if (GLU) {
      // delayed scaling of the gated output: scale from the amax ring (all slots but this call's and the next one's)
      const int nxt = p.glu_cur + 1 == p.glu_slots ? 0 : p.glu_cur + 1;
      float a = 0.f;
      for (int j = 0; j < p.glu_slots; ++j) {
        if (j == p.glu_cur || j == nxt) continue;
        const float h = p.glu_hist[j];
        if (h > a && h < 3.0e38f) a = h;
      }
      const float fmax_q = GLU == 2 ? 57344.f : 448.f;          // e5m2 gradients, e4m3 activations
      if (!(a > 0.f)) a = fmax_q;
      if (blockIdx.x == 0 && warp == 2 && lane == 0) { p.glu_scale_inv[0] = a / fmax_q; p.glu_hist[nxt] = 0.f; }
      q_scale = fmax_q / a;
    }
    for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local) {
      const int acc = local & 1;
      int mt, nt; pair_tile_coords(tile, m_tiles, n_tiles, mt, nt);
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int row = mt * 256 + int(rank) * 128 + q * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      __nv_bfloat16* crow = p.C + size_t(row) * p.ldc;
      if (GLU == 2) {
        const int F = p.glu_F;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          const int f = n0 + c * 32;
          const bool live = row < p.M && f < F;
          uint4 av[4], bv[4];
          if (live) {
            const uint4* pa = reinterpret_cast<const uint4*>(p.glu_ab + size_t(row) * p.glu_ld_ab + f);
            const uint4* pb = reinterpret_cast<const uint4*>(p.glu_ab + size_t(row) * p.glu_ld_ab + F + f);
#pragma unroll
            for (int v = 0; v < 4; ++v) { av[v] = pa[v]; bv[v] = pb[v]; }
          }
          tmem_wait_ld();
          if (live) {
            uint32_t qa[8], qb[8];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av[v]);
              const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv[v]);
              float da[8], db[8];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 af = __bfloat1622float2(a2[j]), bf = __bfloat1622float2(b2[j]);
                // g as the separate product would have stored it (bf16), then the gate backward's arithmetic
                const float g0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[v * 8 + 2 * j]) * alpha));
                const float g1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[v * 8 + 2 * j + 1]) * alpha));
                const float s0 = __fdividef(1.f, 1.f + __expf(-af.x)), s1 = __fdividef(1.f, 1.f + __expf(-af.y));
                const float f0 = af.x * s0, f1 = af.y * s1;
                const float d0 = s0 + f0 * (1.f - s0), d1 = s1 + f1 * (1.f - s1);
                da[2 * j] = __bfloat162float(__float2bfloat16_rn(g0 * bf.x * d0));
                da[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(g1 * bf.y * d1));
                db[2 * j] = __bfloat162float(__float2bfloat16_rn(g0 * f0));
                db[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(g1 * f1));
                q_amax = fmaxf(q_amax, fmaxf(fmaxf(fabsf(da[2 * j]), fabsf(da[2 * j + 1])), fmaxf(fabsf(db[2 * j]), fabsf(db[2 * j + 1]))));
              }
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const unsigned short x0 = __nv_cvt_float2_to_fp8x2(make_float2(da[4 * h] * q_scale, da[4 * h + 1] * q_scale), __NV_SATFINITE, __NV_E5M2);
                const unsigned short x1 = __nv_cvt_float2_to_fp8x2(make_float2(da[4 * h + 2] * q_scale, da[4 * h + 3] * q_scale), __NV_SATFINITE, __NV_E5M2);
                const unsigned short y0 = __nv_cvt_float2_to_fp8x2(make_float2(db[4 * h] * q_scale, db[4 * h + 1] * q_scale), __NV_SATFINITE, __NV_E5M2);
                const unsigned short y1 = __nv_cvt_float2_to_fp8x2(make_float2(db[4 * h + 2] * q_scale, db[4 * h + 3] * q_scale), __NV_SATFINITE, __NV_E5M2);
                qa[2 * v + h] = uint32_t(x0) | (uint32_t(x1) << 16);
                qb[2 * v + h] = uint32_t(y0) | (uint32_t(y1) << 16);
              }
            }
            uint4* da_dst = reinterpret_cast<uint4*>(p.glu_q + size_t(row) * 2 * F + f);
            uint4* db_dst = reinterpret_cast<uint4*>(p.glu_q + size_t(row) * 2 * F + F + f);
            da_dst[0] = make_uint4(qa[0], qa[1], qa[2], qa[3]); da_dst[1] = make_uint4(qa[4], qa[5], qa[6], qa[7]);
            db_dst[0] = make_uint4(qb[0], qb[1], qb[2], qb[3]); db_dst[1] = make_uint4(qb[4], qb[5], qb[6], qb[7]);
          }
        }
      } else if (GLU) {
        const int f0 = nt * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(t_row + c * 32, ra);
          tmem_ld_32x32(t_row + 128 + c * 32, rb);
          tmem_wait_ld();
          if (row < p.M) {
            const int f = f0 + c * 32;
            uint32_t qw[8];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 oa, ob;
              __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&oa);
              __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&ob);
              float o[8];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                a2[j] = __floats2bfloat162_rn(__uint_as_float(ra[v * 8 + 2 * j]) * alpha, __uint_as_float(ra[v * 8 + 2 * j + 1]) * alpha);
                b2[j] = __floats2bfloat162_rn(__uint_as_float(rb[v * 8 + 2 * j]) * alpha, __uint_as_float(rb[v * 8 + 2 * j + 1]) * alpha);
                // the gate on the bf16-rounded a and b (what the backward re-reads), its result rounded to bf16 as the
                // separate gate kernel's is
                const float2 af = __bfloat1622float2(a2[j]), bf = __bfloat1622float2(b2[j]);
                o[2 * j] = __bfloat162float(__float2bfloat16_rn(af.x * __fdividef(1.f, 1.f + __expf(-af.x)) * bf.x));
                o[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(af.y * __fdividef(1.f, 1.f + __expf(-af.y)) * bf.y));
                q_amax = fmaxf(q_amax, fmaxf(fabsf(o[2 * j]), fabsf(o[2 * j + 1])));
              }
              *reinterpret_cast<uint4*>(crow + f + v * 8) = oa;
              *reinterpret_cast<uint4*>(crow + p.glu_F + f + v * 8) = ob;
              const unsigned short h0 = __nv_cvt_float2_to_fp8x2(make_float2(o[0] * q_scale, o[1] * q_scale), __NV_SATFINITE, __NV_E4M3);
              const unsigned short h1 = __nv_cvt_float2_to_fp8x2(make_float2(o[2] * q_scale, o[3] * q_scale), __NV_SATFINITE, __NV_E4M3);
              const unsigned short h2 = __nv_cvt_float2_to_fp8x2(make_float2(o[4] * q_scale, o[5] * q_scale), __NV_SATFINITE, __NV_E4M3);
              const unsigned short h3 = __nv_cvt_float2_to_fp8x2(make_float2(o[6] * q_scale, o[7] * q_scale), __NV_SATFINITE, __NV_E4M3);
              qw[2 * v] = uint32_t(h0) | (uint32_t(h1) << 16);
              qw[2 * v + 1] = uint32_t(h2) | (uint32_t(h3) << 16);
            }
            uint4* qd = reinterpret_cast<uint4*>(p.glu_q + size_t(row) * p.glu_F + f);
            qd[0] = make_uint4(qw[0], qw[1], qw[2], qw[3]);
            qd[1] = make_uint4(qw[4], qw[5], qw[6], qw[7]);
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        store_chunk(p, row, n0 + c * 32, r, alpha, crow);
      }
      }
      tc_fence_before();
      __syncwarp();
      // the MMA thread of the even CTA waits for the four epilogue warps of both CTAs
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
    }
    if (GLU) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) q_amax = fmaxf(q_amax, __shfl_xor_sync(0xffffffffu, q_amax, o));
      if (lane == 0 && q_amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.glu_hist + p.glu_cur), __float_as_uint(q_amax));
    }
  }
  tc_fence_before();
  __syncthreads();
  // neither CTA may free tensor memory or leave while its partner can still signal it or read its shared memory
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

static int g_last_encode_result = 0;

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row stride `ld` elements.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_last_encode_result = (int)r;
  return r == CUDA_SUCCESS ? 0 : -2;
}

// 2-D one-byte tensor map (fp8 operands)
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                    uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_last_encode_result = (int)r;
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int g_num_sms = 0;
static int g_last_detail = 0;   // (which operand << 16) | CUresult of the last failed tensor-map encode

static int g_pair_mode = 2;      // 1: CTA-pair kernel for one-byte operands, 2: for every GEMM, 0: never

// Launch the CTA-pair kernel (cluster of 2) on tensor maps whose boxes are 128 rows (K-major) / 128-byte MN boxes.
template <int EB>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int a_mn, int b_mn,
                       cudaStream_t stream) {
  void (*kern)(const CUtensorMap, const CUtensorMap, GemmParams);
  if (!a_mn && !b_mn) kern = gemm_pair_kernel<0, 0, EB>;
  else if (!a_mn && b_mn) kern = gemm_pair_kernel<0, 1, EB>;
  else if (a_mn && b_mn) kern = gemm_pair_kernel<1, 1, EB>;
  else kern = gemm_pair_kernel<1, 0, EB>;
  static bool attr_set[4] = {false, false, false, false};
  const int idx = a_mn * 2 + b_mn;
  if (!attr_set[idx]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess) return -5;
    attr_set[idx] = true;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + BN - 1) / BN);
  int pairs = g_num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p) == cudaSuccess ? 0 : -6;
}

}  // namespace sb

extern "C" int sb_gemm_last_error_detail() { return sb::g_last_detail; }
// 0: single-CTA tiles only; 1: CTA pairs (cta_group::2) for fp8 operands; 2: CTA pairs for bf16 operands too
extern "C" int sb_gemm_set_pair_mode(int mode) { sb::g_pair_mode = mode; return 0; }

// C = A * B^T (+bias) (+residual) (+C).  a_mn = 0: A is [M, K] row-major with leading dim lda; a_mn = 1: A is stored
// transposed as [K, M] with leading dim lda.  b_mn likewise for B ([N, K] or [K, N]).  All leading dims and
// base addresses must be 16-byte aligned; N a multiple of 8, and K too unless both operands are MN-major.  Returns 0 on a successful launch.
extern "C" int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                            int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, int beta, unsigned int* status,
                            int max_ctas, cudaStream_t stream) {
  using namespace sb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // The tensor-map encoder is a driver call and needs a current context; a thread that has made no runtime call
  // yet (e.g. an autograd worker on its first launch) has none until the runtime binds the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  // K only has to be a multiple of 8 where it is the contiguous dim of an operand (a K-major one)
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldc % 8) || ((!a_mn || !b_mn) && (K % 8))) return -3;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = make_tmap_2d_bf16(&tmA, A, K, M, lda, BK, BM);
  else       rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, 64, BK);
  if (rc) { g_last_detail = (1 << 16) | (g_last_encode_result & 0xffff); return rc; }
  if (!b_mn) rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, BN);
  else       rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, 64, BK);
  if (rc) { g_last_detail = (2 << 16) | (g_last_encode_result & 0xffff); return rc; }
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (residual && ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -4;
  GemmParams p{reinterpret_cast<__nv_bfloat16*>(C), reinterpret_cast<const __nv_bfloat16*>(bias),
               reinterpret_cast<const __nv_bfloat16*>(residual), M, N, K, ldc, ldr, beta, status, nullptr, nullptr, 0, 0};
  if (g_pair_mode >= 2 && max_ctas <= 0) {
    if (!b_mn && (rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, 128))) return rc;     // 128 B rows per CTA of the pair
    return launch_pair<2>(tmA, tmB, p, a_mn, b_mn, stream);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < g_num_sms ? tiles : g_num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  void (*kern)(const CUtensorMap, const CUtensorMap, GemmParams);
  if (!a_mn && !b_mn) kern = gemm_bf16_kernel<0, 0, 2>;
  else if (!a_mn && b_mn) kern = gemm_bf16_kernel<0, 1, 2>;
  else if (a_mn && b_mn) kern = gemm_bf16_kernel<1, 1, 2>;
  else kern = gemm_bf16_kernel<1, 0, 2>;
  static bool attr_set[4] = {false, false, false, false};
  const int idx = a_mn * 2 + b_mn;
  if (!attr_set[idx]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -5;
    attr_set[idx] = true;
  }
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

// Gate projection of the gated MLP with the gate in the epilogue (CTA-pair kernel, GLU mode): AB [M, 2 F] bf16 =
// alpha * A [M, K] * W12 [2 F, K]^T with e4m3 operands, and Q [M, F] = e4m3(silu(a) * b) under delayed scaling (ring
// protocol of sb_quantize_fp8_delayed: `hist` of `slots` floats, slot `cur` collects this call's amax, `scale_inv`
// receives the de-quantisation factor).  F % 128 == 0, K % 16 == 0.
extern "C" int sb_gemm_fp8_glu(const void* A, const void* W12, void* AB, void* Q, const float* alpha, const float* alpha2, int M,
                               int F, int K, int lda, int ldb, int ldab, float* hist, int slots, int cur, float* scale_inv,
                               unsigned int* status, cudaStream_t stream) {
  using namespace sb;
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if ((F % 128) || (K % 16) || (lda % 16) || (ldb % 16) || (ldab % 8) || ldab < 2 * F || slots < 3 || cur < 0 || cur >= slots) return -3;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W12) | reinterpret_cast<uintptr_t>(AB) |
       reinterpret_cast<uintptr_t>(Q)) & 15) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_tmap_2d_u8(&tmA, A, K, M, lda, 128, BM))) return rc;
  if ((rc = make_tmap_2d_u8(&tmB, W12, K, 2 * F, ldb, 128, 128))) return rc;
  if (!g_num_sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev); }
  GemmParams p{reinterpret_cast<__nv_bfloat16*>(AB), nullptr, nullptr, M, 2 * F, K, ldab, 0, 0, status, alpha, alpha2, 0, 0,
               reinterpret_cast<uint8_t*>(Q), F, hist, slots, cur, scale_inv};
  auto kern = gemm_pair_kernel<0, 0, 1, 1>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess) return -5;
    attr_set = true;
  }
  const int tiles = ((M + 255) / 256) * (F / 128);
  int pairs = g_num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p) == cudaSuccess ? 0 : -6;
}

// Input-gradient product of the gated MLP's output projection with the gate backward in the epilogue (GLU = 2):
// g [M, F] = alpha * G [M, D] (e5m2) * W3 [D, F] (e4m3, rows of F contiguous) is not stored; with [a | b] = AB [M, 2 F]
// the epilogue writes Q [M, 2 F] = e5m2(g * b * silu'(a) | g * silu(a)) under delayed scaling.  F % 16 == 0, D % 16 == 0.
extern "C" int sb_gemm_fp8_glu_bwd(const void* G, const void* W3, const void* AB, void* Q, const float* alpha, const float* alpha2,
                                   int M, int F, int D, int ldg, int ldw, int ldab, float* hist, int slots, int cur,
                                   float* scale_inv, unsigned int* status, cudaStream_t stream) {
  using namespace sb;
  if (M <= 0 || F <= 0 || D <= 0) return 0;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if ((F % 32) || (D % 16) || (ldg % 16) || (ldw % 16) || (ldab % 8) || ldab < 2 * F || slots < 3 || cur < 0 || cur >= slots) return -3;
  if ((reinterpret_cast<uintptr_t>(G) | reinterpret_cast<uintptr_t>(W3) | reinterpret_cast<uintptr_t>(AB) |
       reinterpret_cast<uintptr_t>(Q)) & 15) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_tmap_2d_u8(&tmA, G, D, M, ldg, 128, BM))) return rc;
  if ((rc = make_tmap_2d_u8(&tmB, W3, F, D, ldw, 128, 128))) return rc;          // MN-major operand: boxes of 128 x 128
  if (!g_num_sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev); }
  GemmParams p{nullptr, nullptr, nullptr, M, F, D, 0, 0, 0, status, alpha, alpha2, 1, 0,
               reinterpret_cast<uint8_t*>(Q), F, hist, slots, cur, scale_inv, reinterpret_cast<const __nv_bfloat16*>(AB), ldab};
  auto kern = gemm_pair_kernel<0, 1, 1, 2>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess) return -5;
    attr_set = true;
  }
  const int tiles = ((M + 255) / 256) * ((F + BN - 1) / BN);
  int pairs = g_num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p) == cudaSuccess ? 0 : -6;
}

// fp8 GEMM: C[M,N] (bf16) = alpha * A * B^T (+bias) (+residual) (+C) with one-byte operands (e4m3 = 0 / e5m2 = 1) and
// fp32 accumulation; `alpha` and `alpha2` are device scalars (the operands' de-quantisation factors; either may be
// null) whose product scales the accumulator.  Leading dims and contiguous extents must be multiples of 16 elements.
extern "C" int sb_gemm_fp8(const void* A, const void* B, void* C, const void* bias, const void* residual, const float* alpha,
                           const float* alpha2, int M, int N, int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, int a_fmt, int b_fmt,
                           int beta, unsigned int* status, cudaStream_t stream) {
  using namespace sb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if ((N % 8) || (lda % 16) || (ldb % 16) || (ldc % 8) || ((!a_mn || !b_mn) && (K % 16))) return -3;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = make_tmap_2d_u8(&tmA, A, K, M, lda, 128, BM);
  else       rc = make_tmap_2d_u8(&tmA, A, M, K, lda, 128, 128);
  if (rc) { g_last_detail = (1 << 16) | (g_last_encode_result & 0xffff); return rc; }
  if (!b_mn) rc = make_tmap_2d_u8(&tmB, B, K, N, ldb, 128, BN);
  else       rc = make_tmap_2d_u8(&tmB, B, N, K, ldb, 128, 128);
  if (rc) { g_last_detail = (2 << 16) | (g_last_encode_result & 0xffff); return rc; }
  if (!g_num_sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev); }
  if (residual && ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -4;
  GemmParams p{reinterpret_cast<__nv_bfloat16*>(C), reinterpret_cast<const __nv_bfloat16*>(bias),
               reinterpret_cast<const __nv_bfloat16*>(residual), M, N, K, ldc, ldr, beta, status, alpha, alpha2, a_fmt, b_fmt};
  if (g_pair_mode >= 1) {
    if (!b_mn && (rc = make_tmap_2d_u8(&tmB, B, K, N, ldb, 128, 128))) return rc;      // 128 B rows per CTA of the pair
    return launch_pair<1>(tmA, tmB, p, a_mn, b_mn, stream);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < g_num_sms ? tiles : g_num_sms;
  void (*kern)(const CUtensorMap, const CUtensorMap, GemmParams);
  if (!a_mn && !b_mn) kern = gemm_bf16_kernel<0, 0, 1>;
  else if (!a_mn && b_mn) kern = gemm_bf16_kernel<0, 1, 1>;
  else if (a_mn && b_mn) kern = gemm_bf16_kernel<1, 1, 1>;
  else kern = gemm_bf16_kernel<1, 0, 1>;
  static bool attr_set[4] = {false, false, false, false};
  const int idx = a_mn * 2 + b_mn;
  if (!attr_set[idx]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -5;
    attr_set[idx] = true;
  }
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}
