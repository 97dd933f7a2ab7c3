// Flash attention for sm_100a: tcgen05 tensor-core products with TMEM accumulators, TMA-staged operands, online
// softmax by one thread per query row.  Head dimension 128, bf16 in and out, fp32 accumulation and statistics.
//
// Tensors are addressed as [B, L, H, 128] with arbitrary (16-byte aligned) strides for B, L and H, so the q/k/v slices
// of one fused projection output are read in place.  Both kernels load every operand tile the same way: 128 rows of
// one head as two TMA boxes of [128 rows x 64 columns] (128-byte rows, 128-byte swizzle).  Such a tile serves as a
// K-major operand when the contraction runs over the head dimension and as an MN-major operand when it runs over the
// rows, so no tile is ever transposed in memory.
//
// Forward (one CTA = two 128-row query tiles of one head):
//   warp 0      TMA producer   Q tiles once; per key block one K tile and one V tile (single-buffered, separate
//                               barriers, so K[j+1] lands during softmax j and V[j+1] during softmax j+1)
//   warp 1      MMA issuer     S_t = Q_t K^T (TMEM cols t*128), then O_t += P_t V (TMEM cols 256 + t*128); the next S of
//                               a tile is issued right behind its P V product so the two tiles alternate on the tensor
//                               pipe while the other one is in its softmax
//   warps 2-5   softmax of tile 0, warps 6-9 of tile 1: row max, exp2, row sum, P as bf16 into swizzled shared
//               memory, rescale of O in TMEM only when the running maximum grew by more than 2^8
//
// Every wait is bounded (sm100.cuh); on a timeout the CTA records a status code, frees TMEM and returns.
#include "sm100.cuh"

namespace sb {
namespace attn {

constexpr int HD = 128;                 // head dimension
constexpr int BQ = 128;                 // query rows per tile
constexpr int BK = 128;                 // keys per block
constexpr int TILE_BYTES = 128 * HD * 2;   // 32 KB: two boxes of 16 KB
constexpr int BOX_BYTES = 128 * 128;       // 16 KB: 128 rows of 128 bytes
constexpr int FWD_THREADS = 320;
constexpr int FWD_SMEM = 7 * TILE_BYTES + 256 + 1024;
constexpr uint32_t ST_ATTN = 0x20;      // status codes 0x20.. identify attention waits

struct FwdParams {
  __nv_bfloat16* out;        // [B, Lq, H, 128]
  float* lse;                // [B, H, Lq] natural-log sum of exp of the scaled scores
  long long o_sb, o_sl, o_sh;   // element strides of out
  int B, H, Lq, Lk;
  int causal;
  float scale_log2;          // softmax scale * log2(e)
  float scale;
  uint32_t* status;
  int pingpong;              // 1: the two softmax warpgroups take turns on the exponentials (see the kernel)
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// one 128-row tile of head h, batch b, rows l0.. : two boxes (columns 0-63 and 64-127)
__device__ __forceinline__ void load_tile(uint32_t dst, const void* tmap, int l0, int h, int b, uint32_t bar) {
  tma_load_4d(dst, tmap, 0, h, l0, b, bar);
  tma_load_4d(dst + BOX_BYTES, tmap, 64, h, l0, b, bar);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of the 16-byte chunk `cc` (8 bf16 columns, 0..15) of row `r` inside a swizzled [128 x 128] bf16 tile.
__device__ __forceinline__ uint32_t swz_chunk(int r, int cc) {
  return uint32_t(cc >> 3) * BOX_BYTES + uint32_t(r) * 128u + (uint32_t((cc & 7) ^ (r & 7)) << 4);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// K-major operand (contraction over the 128 columns): MMA k-step kk (16 columns) of a tile
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kk) {
  return umma_smem_desc(tile + uint32_t(kk >> 2) * BOX_BYTES + uint32_t(kk & 3) * 32u, 16u, 1024u);
}
// MN-major operand (contraction over the 128 rows; the two 64-column boxes are BOX_BYTES apart): k-step kk = 16 rows
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kk) {
  return umma_smem_desc(tile + uint32_t(kk) * 2048u, BOX_BYTES, 1024u);
}

// P_TMEM: the probabilities go back into tensor memory as packed bf16 over the first 64 columns of their own score
// buffer and enter the P V product as its TMEM operand: no P stores into shared memory and no A-operand reads from it
// (a single-CTA M = 128 product with both operands in shared memory uses the whole shared-memory bandwidth of the SM).
// The price is an ordering constraint: the scores of block j+1 overwrite P(j), so S_t(j+1) is issued behind P_t(j) V(j)
// on the (in-order) tensor pipe instead of during softmax j; the other query tile fills the gap.
template <bool P_TMEM>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // K and V tiles share one ring of three slots, filled in the order they are consumed: K(0) V(0) K(1) V(1) ...
  // (tile number i of that sequence lives in slot i % 3).  K(j)'s slot is free as soon as both score products of block
  // j are done, early in the block, so V(j+1) is already on its way while P V of block j runs; with the same 96 KB as
  // two K stages and one V stage, no TMA latency is left exposed between consecutive P V products.
  const uint32_t sQ = smem_base, sKV = smem_base + 2 * TILE_BYTES, sP = sKV + 3 * TILE_BYTES;
  constexpr uint32_t BAR_OFF = 7 * TILE_BYTES;
  const uint32_t bar_base = smem_base + BAR_OFF;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u + 8u * s; };
  auto kv_free = [&](int s) { return bar_base + 32u + 8u * s; };
  auto s_full = [&](int t) { return bar_base + 56u + 8u * t; };
  auto s_free = [&](int t) { return bar_base + 72u + 8u * t; };
  auto p_ready = [&](int t) { return bar_base + 88u + 8u * t; };
  auto pv_done = [&](int t) { return bar_base + 104u + 8u * t; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + BAR_OFF + 120);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + BAR_OFF + 128);
  // turn(t): "warpgroup t may run its exponentials".  The special-function unit is the shared resource of the two
  // softmax warpgroups: left alone they fall into phase (both in the exponentials, then both waiting on TMEM loads,
  // row maxima and the P V product) and the unit idles half of the time.  Taking turns keeps one warpgroup in its
  // exponentials while the other loads and reduces its next score row.
  auto turn = [&](int t) { return bar_base + 136u + 8u * t; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;          // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qblk * 2 * BQ;
  const int kv_blocks = (p.Lk + BK - 1) / BK;
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * BQ;
    if (r0 >= p.Lq) nb[t] = 0;
    else if (p.causal) nb[t] = min(kv_blocks, r0 / BK + 1);
    else nb[t] = kv_blocks;
  }
  const int n = max(nb[0], nb[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int t = 0; t < 3; ++t) { mbar_init(kv_full(t), 1); mbar_init(kv_free(t), 1); }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1); mbar_init(s_free(t), 128); mbar_init(p_ready(t), 128); mbar_init(pv_done(t), 1);
      mbar_init(turn(t), 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      bool ok = true;
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      load_tile(sQ, &tmQ, q0, h, b, q_full);
      load_tile(sQ + TILE_BYTES, &tmQ, q0 + BQ, h, b, q_full);
      for (int i = 0; i < 2 * n && ok; ++i) {            // i even: K(i/2), i odd: V(i/2)
        const int slot = i % 3;
        const uint32_t use = uint32_t(i / 3);
        if (!mbar_wait(kv_free(slot), (use & 1u) ^ 1u, abort_flag, p.status, ST_ATTN + 1 + (i & 1))) { ok = false; break; }
        mbar_expect_tx(kv_full(slot), TILE_BYTES);
        load_tile(sKV + slot * TILE_BYTES, (i & 1) ? &tmV : &tmK, (i >> 1) * BK, h, b, kv_full(slot));
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n > 0) {
      const uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);     // S = Q K^T: both operands K-major
      const uint32_t idesc_o = umma_idesc_bf16(128, 128, 0, 1);     // O += P V: P K-major, V MN-major
      bool ok = mbar_wait(q_full, 0u, abort_flag, p.status, ST_ATTN + 3);
      // Event loop over both tiles: S_t(js) goes out as soon as K(js) has landed and the softmax warps have read S_t(js-1)
      // out of TMEM; O_t += P_t(jp) V(jp) as soon as P_t(jp) and V(jp) are there.  Each tile's queue is served in order.
      int s_idx[2] = {0, 0}, pv_idx[2] = {0, 0};
      unsigned long long t0 = globaltimer();       // time of the last progress
      uint32_t spins = 0;
      while (ok && (s_idx[0] < nb[0] || s_idx[1] < nb[1] || pv_idx[0] < nb[0] || pv_idx[1] < nb[1])) {
        bool progress = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (pv_idx[t] < nb[t]) {
            const int jp = pv_idx[t];
            const int vslot = (2 * jp + 1) % 3;
            if (mbar_test(p_ready(t), uint32_t(jp) & 1u) && mbar_test(kv_full(vslot), uint32_t((2 * jp + 1) / 3) & 1u)) {
              tc_fence_after();
              const uint32_t sV = sKV + vslot * TILE_BYTES;
#pragma unroll
              for (int kk = 0; kk < 8; ++kk) {
                if (P_TMEM)      // 16 keys = 8 packed columns of the tile's score buffer
                  umma_bf16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, desc_mnmajor(sV, kk), idesc_o,
                               (jp | kk) ? 1u : 0u);
                else
                  umma_bf16(tmem_base + 256 + t * 128, desc_kmajor(sP + t * TILE_BYTES, kk), desc_mnmajor(sV, kk), idesc_o,
                            (jp | kk) ? 1u : 0u);
              }
              umma_commit(pv_done(t));
              pv_idx[t] = jp + 1;
              if (pv_idx[t ^ 1] > jp || jp >= nb[t ^ 1]) umma_commit(kv_free(vslot));   // both tiles are through with V(jp)
              progress = true;
            }
          }
          if (s_idx[t] < nb[t]) {
            const int js = s_idx[t];
            const int kslot = (2 * js) % 3;
            // P_TMEM: P(js-1) lives in the score buffer until its P V product, issued earlier on the in-order pipe, read it
            if (mbar_test(kv_full(kslot), uint32_t((2 * js) / 3) & 1u) &&
                (js == 0 || (P_TMEM ? pv_idx[t] >= js : mbar_test(s_free(t), uint32_t(js - 1) & 1u)))) {
              tc_fence_after();
              const uint32_t sK = sKV + kslot * TILE_BYTES;
#pragma unroll
              for (int kk = 0; kk < 8; ++kk)
                umma_bf16(tmem_base + t * 128, desc_kmajor(sQ + t * TILE_BYTES, kk), desc_kmajor(sK, kk), idesc_s, kk ? 1u : 0u);
              umma_commit(s_full(t));
              s_idx[t] = js + 1;
              if (s_idx[t ^ 1] > js || js >= nb[t ^ 1]) umma_commit(kv_free(kslot));    // both tiles are through with K(js)
              progress = true;
            }
          }
        }
        if (progress) {
          t0 = globaltimer();
        } else {
          if ((++spins & 255u) == 0u) {
            if (*abort_flag) ok = false;
            else if (globaltimer() - t0 > WAIT_BUDGET_NS) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0u, ((ST_ATTN + 6) << 24) | (blockIdx.x & 0xffffffu));
              ok = false;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: one thread per query row
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;                    // TMEM lane quarter this warp may access
    const int r = quarter * 32 + lane;               // row inside the tile
    const int row = q0 + t * BQ + r;                 // query position
    const uint32_t t_s = tmem_base + (uint32_t(quarter * 32) << 16) + t * 128;
    const uint32_t t_o = tmem_base + (uint32_t(quarter * 32) << 16) + 256 + t * 128;
    const uint32_t p_tile = sP + t * TILE_BYTES;
    const float sl2 = p.scale_log2;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nb[t] && ok; ++j) {
      const uint32_t par = uint32_t(j) & 1u;
      if (!mbar_wait(s_full(t), par, abort_flag, p.status, ST_ATTN + 7)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * BK;
      const bool edge = (p.causal && k0 + BK - 1 > q0 + t * BQ) || (k0 + BK > p.Lk);
      const int limit = p.causal ? min(row, p.Lk - 1) : p.Lk - 1;      // last visible key of this row
      // the whole score row into registers, then hand the TMEM buffer back for the next block's scores
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, v[c]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(s_free(t));
      if (edge) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (k0 + c * 32 + i > limit) v[c][i] = 0xff800000u;      // -inf
      }
      // four independent chains keep the dependent-issue latency of the row maximum short
      float bm4[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        bm4[c] = __uint_as_float(v[c][0]);
#pragma unroll
        for (int i = 1; i < 32; ++i) bm4[c] = fmaxf(bm4[c], __uint_as_float(v[c][i]));
      }
      const float bm = fmaxf(fmaxf(bm4[0], bm4[1]), fmaxf(bm4[2], bm4[3]));
      // keep the old reference maximum unless the new one exceeds it by more than 2^8 (P stays below 256)
      float m_new = m;
      if (bm > m && (m == -INFINITY || (bm - m) * sl2 > 8.f)) m_new = bm;
      const float m_ref = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : ex2((m - m_ref) * sl2);
      const bool rescale = (j > 0) && (m_new != m);
      m = m_new;
      if (j > 0) {
        // the previous P V product must have read the P tile (and left O consistent) before either is touched
        if (!mbar_wait(pv_done(t), par ^ 1u, abort_flag, p.status, ST_ATTN + 8)) { ok = false; break; }
        tc_fence_after();
      }
      // my turn on the special-function unit: tile 0 goes first; tile 0's block j follows tile 1's block j-1, tile 1's
      // block j follows tile 0's block j.  A warpgroup whose partner has no such block left does not wait.
      if (p.pingpong) {
        if (t == 0) {
          if (j > 0 && j - 1 < nb[1] &&
              !mbar_wait(turn(0), uint32_t(j - 1) & 1u, abort_flag, p.status, ST_ATTN + 10)) { ok = false; break; }
        } else {
          if (j < nb[0] && !mbar_wait(turn(1), par, abort_flag, p.status, ST_ATTN + 11)) { ok = false; break; }
        }
      }
      // P = exp2((S - m) * scale) as bf16 into the swizzled P tile; row sum in fp32
      const float moff = -m_ref * sl2;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float xa = fmaf(__uint_as_float(v[c][g * 8 + 2 * i]), sl2, moff);
            const float xb = fmaf(__uint_as_float(v[c][g * 8 + 2 * i + 1]), sl2, moff);
            const float ea = ex2(xa), eb = ex2(xb);        // exp2(-inf) = 0 for masked keys
            rs4[i] += ea + eb;
            w[i] = pack_bf16(ea, eb);
          }
          if (P_TMEM) {
            // the score registers of these 8 keys are dead: keep the packed probabilities in their place
#pragma unroll
            for (int i = 0; i < 4; ++i) v[c][g * 4 + i] = w[i];
          } else {
            st_shared_v4(p_tile + swz_chunk(r, c * 4 + g), w[0], w[1], w[2], w[3]);
          }
        }
        if (P_TMEM) {
          uint32_t pw[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pw[i] = v[c][i];
          tmem_st_32x16(t_s + c * 16, pw);                 // keys 32c .. 32c+31 -> packed columns 16c .. 16c+15
        }
      }
      if (P_TMEM) tmem_wait_st();
      if (p.pingpong) mbar_arrive(turn(t ^ 1));               // hand the unit to the other warpgroup
      const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      l = l * alpha + rs;
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(t_o + c * 32, v);
        }
        tmem_wait_st();
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(p_ready(t));
    }
    if (ok && nb[t] > 0) {
      const uint32_t par = uint32_t(nb[t] - 1) & 1u;
      if (mbar_wait(pv_done(t), par, abort_flag, p.status, ST_ATTN + 9)) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.out + (long long)b * p.o_sb + (long long)row * p.o_sl + (long long)h * p.o_sh;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
          tmem_wait_ld();
          if (row < p.Lq) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
              o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
              o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
              o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
            }
          }
        }
        if (row < p.Lq)
          p.lse[((long long)b * p.H + h) * p.Lq + row] = (m == -INFINITY ? 0.f : m) * p.scale + __logf(fmaxf(l, 1e-37f));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------ backward
// One CTA owns a block of 128 keys of one head and walks over the query tiles (64 rows each) that see it.  All five
// products run with M = 128 on the tensor cores, in the transposed form (keys or head dimension on the TMEM lanes):
//   S^T  = K Q^T            [keys x q]   A = K  (K-major),   B = Q_i  (K-major)
//   dP^T = V dO^T           [keys x q]   A = V  (K-major),   B = dO_i (K-major)
//   dV  += P^T dO           [keys x d]   A = P^T (K-major, from shared memory), B = dO_i (MN-major)
//   dK  += dS^T Q           [keys x d]   A = dS^T (K-major),                    B = Q_i  (MN-major)
//   dQ^T = K^T dS^T         [d x q]      A = K (MN-major),   B = dS^T (MN-major)   -> fp32 atomics into dq_acc
// with P = exp(S * scale - lse) and dS = P (dP - delta) * scale computed by one thread per key row and 32 query columns
// (two warpgroups split the 64 columns).  TMEM: S^T (2 x 64 columns, so the scores of the next tile are computed during
// this tile's softmax), dP^T (64), dQ^T (64), dV (128), dK (128).
constexpr int BQ2 = 64;                          // query rows per backward tile
constexpr int QTILE_BYTES = BQ2 * HD * 2;        // 16 KB: two boxes of 8 KB
constexpr int QBOX_BYTES = BQ2 * 128;            // 8 KB
constexpr int PT_BYTES = 128 * 128;              // P^T / dS^T tile: 128 key rows x 64 q columns bf16 = 16 KB
constexpr int BWD_THREADS = 320;
constexpr int STAGE_BYTES = BQ2 * HD * 4;          // dQ^T staging tile: 64 query rows x 128 fp32
constexpr int BWD_SMEM = 2 * TILE_BYTES + 4 * QTILE_BYTES + 4 * PT_BYTES + STAGE_BYTES + 256 + 1024;

struct BwdParams {
  const float* stats;        // [B, H, Lpad, 2]: (-lse * log2(e), scale * (rowsum(dO * O) - dlse)), Lpad = 64 * ceil(Lq / 64)
  __nv_bfloat16* dk;         // [B, Lk, H, 128]; element strides of (batch, key, head) in dk_str / dv_str, unit inner stride
  __nv_bfloat16* dv;
  long long dk_str[3], dv_str[3];
  int B, H, Lq, Lk;
  int causal;
  float scale_log2, scale;
  uint32_t* status;
};

__device__ __forceinline__ void load_qtile(uint32_t dst, const void* tmap, int l0, int h, int b, uint32_t bar) {
  tma_load_4d(dst, tmap, 0, h, l0, b, bar);
  tma_load_4d(dst + QBOX_BYTES, tmap, 64, h, l0, b, bar);
}
// shared -> global reduce-add (fp32) of one box of a 4-D tensor map; completion through the bulk group
__device__ __forceinline__ void tma_reduce_add_4d(const void* tmap, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
      ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(src)
      : "memory");
}
// 64-row tile as K-major operand (contraction over the 128 columns)
__device__ __forceinline__ uint64_t qdesc_kmajor(uint32_t tile, int kk) {
  return umma_smem_desc(tile + uint32_t(kk >> 2) * QBOX_BYTES + uint32_t(kk & 3) * 32u, 16u, 1024u);
}
// 64-row tile as MN-major operand (contraction over its 64 rows, N = 128 columns in two boxes)
__device__ __forceinline__ uint64_t qdesc_mnmajor(uint32_t tile, int kk) {
  return umma_smem_desc(tile + uint32_t(kk) * 2048u, QBOX_BYTES, 1024u);
}
// P^T / dS^T tile [128 rows x 64 columns]: K-major (contraction over the 64 columns) and MN-major (over the 128 rows)
__device__ __forceinline__ uint64_t pdesc_kmajor(uint32_t tile, int kk) { return umma_smem_desc(tile + uint32_t(kk) * 32u, 16u, 1024u); }
__device__ __forceinline__ uint64_t pdesc_mnmajor(uint32_t tile, int kk) { return umma_smem_desc(tile + uint32_t(kk) * 2048u, 16u, 1024u); }

// P_TMEM: P^T stays in tensor memory (written over the consumed S^T columns, two bf16 per 32-bit cell) and feeds the dV
// product as the A operand from TMEM; the shared memory this frees holds a third Q/dO stage, which takes the tile loads
// off the critical path.  Otherwise P^T goes through shared memory like dS^T and there are two Q/dO stages.
template <bool P_TMEM>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmDQ, BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base, sV = sK + TILE_BYTES;
  constexpr int NST = P_TMEM ? 3 : 2;                  // Q/dO stages
  auto sQ = [&](int s) { return smem_base + 2u * TILE_BYTES + uint32_t(s) * 2u * QTILE_BYTES; };
  auto sdO = [&](int s) { return sQ(s) + QTILE_BYTES; };
  const uint32_t pds_base = smem_base + 2u * TILE_BYTES + uint32_t(NST) * 2u * QTILE_BYTES;
  auto sdS = [&](int s) { return pds_base + uint32_t(s) * PT_BYTES; };
  auto sP = [&](int s) { return pds_base + 2u * PT_BYTES + uint32_t(s) * PT_BYTES; };     // only without P_TMEM
  constexpr uint32_t STAGE_OFF = 2 * TILE_BYTES + 4 * QTILE_BYTES + 4 * PT_BYTES;          // both layouts end here
  const uint32_t sStage = smem_base + STAGE_OFF;
  constexpr uint32_t BAR_OFF = STAGE_OFF + STAGE_BYTES;
  const uint32_t bar_base = smem_base + BAR_OFF;
  const uint32_t kv_full = bar_base, dkv_done = bar_base + 8;
  auto qdo_full = [&](int s) { return bar_base + 16u + 8u * s; };
  auto qdo_free = [&](int s) { return bar_base + 40u + 8u * s; };
  auto s_full = [&](int s) { return bar_base + 64u + 8u * s; };
  auto pds_ready = [&](int s) { return bar_base + 80u + 8u * s; };
  const uint32_t dq_full = bar_base + 96u, dq_free = bar_base + 104u;
  const uint32_t stage_ready = bar_base + 112, stage_free = bar_base + 120;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + BAR_OFF + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + BAR_OFF + 136);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * BK, h = blockIdx.y, b = blockIdx.z;
  const int nq = (p.Lq + BQ2 - 1) / BQ2;
  const int i_start = p.causal ? k0 / BQ2 : 0;          // first query tile that sees a key of this block
  const int n = nq - i_start;                            // > 0: the grid only covers key blocks below Lk <= ... (host checks)

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(dkv_done, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(qdo_full(s), 1); mbar_init(qdo_free(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(s_full(s), 1); mbar_init(pds_ready(s), 256); }
    mbar_init(dq_full, 1); mbar_init(dq_free, 256);
    mbar_init(stage_ready, 256); mbar_init(stage_free, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO); prefetch_tmap(&tmDQ);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t T_S = 0, T_DP = 128, T_DQ = 192, T_DV = 256, T_DK = 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n > 0) {
      bool ok = true;
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      load_tile(sK, &tmK, k0, h, b, kv_full);
      load_tile(sV, &tmV, k0, h, b, kv_full);
      for (int it = 0; it < n && ok; ++it) {
        const int s = it % NST;
        if (!mbar_wait(qdo_free(s), (uint32_t(it / NST) & 1u) ^ 1u, abort_flag, p.status, ST_ATTN + 17)) { ok = false; break; }
        mbar_expect_tx(qdo_full(s), 2 * QTILE_BYTES);
        const int i0 = (i_start + it) * BQ2;
        load_qtile(sQ(s), &tmQ, i0, h, b, qdo_full(s));
        load_qtile(sdO(s), &tmdO, i0, h, b, qdo_full(s));
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n > 0) {
      const uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
      const uint32_t idesc_kv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t idesc_dq = umma_idesc_bf16(128, 64, 1, 1);
      // S^T(it) needs Q(it) in shared memory and the S^T buffer of its parity, which the softmax warps finished reading
      // before pds_ready(it-2), a barrier this thread has already passed
      auto issue_s = [&](int it) -> bool {
        const int s = it & 1, qs = it % NST;
        if (!mbar_wait(qdo_full(qs), uint32_t(it / NST) & 1u, abort_flag, p.status, ST_ATTN + 18)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem_base + T_S + s * 64, desc_kmajor(sK, kk), qdesc_kmajor(sQ(qs), kk), idesc_s, kk ? 1u : 0u);
        return true;
      };
      // dP^T(it) goes into the single dP^T buffer: only after the softmax warps have read dP^T(it-1) (pds_ready(it-1))
      auto issue_dp = [&](int it) {
        const int s = it & 1, qs = it % NST;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem_base + T_DP, desc_kmajor(sV, kk), qdesc_kmajor(sdO(qs), kk), idesc_s, kk ? 1u : 0u);
        umma_commit(s_full(s));              // S^T(it) and dP^T(it) are complete
      };
      bool ok = mbar_wait(kv_full, 0u, abort_flag, p.status, ST_ATTN + 20);
      if (ok) ok = issue_s(0);
      if (ok) issue_dp(0);
      for (int it = 0; it < n && ok; ++it) {
        const int s = it & 1, qs = it % NST;
        // the scores of the next tile run while the softmax warps work on this one
        if (it + 1 < n && !issue_s(it + 1)) { ok = false; break; }
        if (!mbar_wait(pds_ready(s), (uint32_t(it) >> 1) & 1u, abort_flag, p.status, ST_ATTN + 21)) { ok = false; break; }
        tc_fence_after();
        if (it + 1 < n) issue_dp(it + 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if (P_TMEM)   // 16 queries = 8 packed columns; each warpgroup wrote its 32 queries over its own S^T columns
            umma_bf16_ts(tmem_base + T_DV, tmem_base + T_S + s * 64 + (kk >> 1) * 32 + (kk & 1) * 8, qdesc_mnmajor(sdO(qs), kk),
                         idesc_kv, (it | kk) ? 1u : 0u);
          else
            umma_bf16(tmem_base + T_DV, pdesc_kmajor(sP(s), kk), qdesc_mnmajor(sdO(qs), kk), idesc_kv, (it | kk) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem_base + T_DK, pdesc_kmajor(sdS(s), kk), qdesc_mnmajor(sQ(qs), kk), idesc_kv, (it | kk) ? 1u : 0u);
        umma_commit(qdo_free(qs));
        // dQ^T(it) into its own buffer once dQ^T(it-1) has been read out (the softmax warps do that after P/dS of tile it)
        if (it >= 1 && !mbar_wait(dq_free, uint32_t(it - 1) & 1u, abort_flag, p.status, ST_ATTN + 19)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem_base + T_DQ, desc_mnmajor(sK, kk), pdesc_mnmajor(sdS(s), kk), idesc_dq, kk ? 1u : 0u);
        umma_commit(dq_full);
      }
      if (ok) umma_commit(dkv_done);
    }
  } else {
    // ------------------------------------------------------------------ P / dS, dQ read-out, dK / dV epilogue
    const int wg = (warp - 2) >> 2;                  // which 32 query columns
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;               // key row of this thread; also head-dimension lane of dQ^T
    const int key = k0 + r;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const float sl2 = p.scale_log2;
    const int tid_c = threadIdx.x - 64;              // 0..255 among the compute threads
    const int lpad = nq * BQ2;
    const float4* stats = reinterpret_cast<const float4*>(p.stats + (((long long)b * p.H + h) * lpad) * 2);
    bool ok = n > 0;
    // dQ^T of tile `it` leaves through shared memory: every thread holds 32 query rows of one head-dimension column,
    // writes them into a [64 x 128] fp32 staging tile, and one thread hands the tile to a TMA reduce-add into dq_acc
    // (rows beyond Lq are clipped by the tensor map).  `cnt` counts the read-outs of this CTA.
    auto read_out_dq = [&](int it, int cnt) -> bool {
      if (!mbar_wait(dq_full, uint32_t(it) & 1u, abort_flag, p.status, ST_ATTN + 22)) return false;
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_32x32(tmem_base + lane_off + T_DQ + wg * 32, v);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(dq_free);
      if (cnt > 0) {
        if (tid_c == 0) { bulk_wait_read<0>(); mbar_arrive(stage_free); }      // the previous reduce has read the tile
        if (!mbar_wait(stage_free, uint32_t(cnt - 1) & 1u, abort_flag, p.status, ST_ATTN + 25)) return false;
      }
      const uint32_t dst = sStage + uint32_t(wg * 32) * 512u + uint32_t(r) * 4u;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + uint32_t(i) * 512u), "r"(v[i]) : "memory");
      fence_proxy_async();
      mbar_arrive(stage_ready);
      if (tid_c == 0) {
        if (!mbar_wait(stage_ready, uint32_t(cnt) & 1u, abort_flag, p.status, ST_ATTN + 26)) return false;
        tma_reduce_add_4d(&tmDQ, sStage, 0, h, (i_start + it) * BQ2, b);
        bulk_commit();
      }
      return true;
    };
    for (int it = 0; it < n && ok; ++it) {
      const int s = it & 1;
      const int qi = (i_start + it) * BQ2 + wg * 32;   // first query of this thread's 32 columns
      // (-lse * log2(e), delta) pairs of the 32 queries: the same addresses in every lane (broadcast loads)
      float4 st[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) st[i] = __ldg(stats + (qi >> 1) + i);
      if (!mbar_wait(s_full(s), (uint32_t(it) >> 1) & 1u, abort_flag, p.status, ST_ATTN + 23)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[32], dp[32];
      tmem_ld_32x32(tmem_base + lane_off + T_S + s * 64 + wg * 32, sv);
      tmem_ld_32x32(tmem_base + lane_off + T_DP + wg * 32, dp);
      tmem_wait_ld();
      uint32_t pw[16], dw[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float pa = ex2(fmaf(__uint_as_float(sv[2 * i]), sl2, st[i].x));
        const float pb = ex2(fmaf(__uint_as_float(sv[2 * i + 1]), sl2, st[i].z));
        const float da = pa * fmaf(__uint_as_float(dp[2 * i]), p.scale, -st[i].y);
        const float db = pb * fmaf(__uint_as_float(dp[2 * i + 1]), p.scale, -st[i].w);
        pw[i] = pack_bf16(pa, pb);
        dw[i] = pack_bf16(da, db);
      }
      if ((p.causal && key > qi) || key >= p.Lk) {
        // some of this row's 32 columns are masked (only the tiles on the diagonal, and the key rows beyond Lk)
        const int vis = key >= p.Lk ? 32 : key - qi;      // columns 0..vis-1 are masked
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (2 * i + 1 < vis) { pw[i] = 0u; dw[i] = 0u; }
          else if (2 * i < vis) { pw[i] &= 0xffff0000u; dw[i] &= 0xffff0000u; }
        }
      }
      // the P^T / dS^T buffers of this parity were last read by the products of tile it-2, which completed before
      // dq_full of tile it-2, and this thread waited for that barrier in read_out_dq(it-2)
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t off = uint32_t(r) * 128u + (uint32_t((wg * 4 + g) ^ (r & 7)) << 4);
        if (!P_TMEM) st_shared_v4(sP(s) + off, pw[4 * g], pw[4 * g + 1], pw[4 * g + 2], pw[4 * g + 3]);
        st_shared_v4(sdS(s) + off, dw[4 * g], dw[4 * g + 1], dw[4 * g + 2], dw[4 * g + 3]);
      }
      if (P_TMEM) {
        tmem_st_32x16(tmem_base + lane_off + T_S + s * 64 + wg * 32, pw);
        tmem_wait_st();
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(pds_ready(s));
      // dQ^T of the previous tile: its product ran while this tile's P and dS were computed
      if (it >= 1 && !read_out_dq(it - 1, it - 1)) { ok = false; break; }
    }
    if (ok && !read_out_dq(n - 1, n - 1)) ok = false;
    if (tid_c == 0) bulk_wait<0>();                     // the last reduce must have left shared memory
    if (ok && mbar_wait(dkv_done, 0u, abort_flag, p.status, ST_ATTN + 24)) {
      tc_fence_after();
      // warpgroup 0 stores dV, warpgroup 1 stores dK: one key row (256 bytes) per thread
      const long long* ds = wg == 0 ? p.dv_str : p.dk_str;
      __nv_bfloat16* dst = (wg == 0 ? p.dv : p.dk) + (long long)b * ds[0] + (long long)key * ds[1] + (long long)h * ds[2];
      const uint32_t t_src = tmem_base + lane_off + (wg == 0 ? T_DV : T_DK);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_src + c * 32, v);
        tmem_wait_ld();
        if (key < p.Lk) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
            o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
            o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
            o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// stats[b, h, i] = (-lse * log2(e), scale * (sum_d dO[b, i, h, d] * O[b, i, h, d] - dlse[b, h, i])) for i < L and (0, 0)
// for the padding rows L <= i < Lpad; one warp per (b, i, h)
__global__ void attn_stats_kernel(const __nv_bfloat16* __restrict__ go, const __nv_bfloat16* __restrict__ o,
                                  const float* __restrict__ lse, const float* __restrict__ glse, float* __restrict__ stats,
                                  int B, int H, int L, int Lpad, float scale, long long g_sb, long long g_sl, long long g_sh,
                                  long long o_sb, long long o_sl, long long o_sh) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * Lpad * H) return;
  const int hh = int(w % H);
  const long long bl = w / H;
  const int i = int(bl % Lpad), bb = int(bl / Lpad);
  float2* dst = reinterpret_cast<float2*>(stats) + ((long long)bb * H + hh) * Lpad + i;
  if (i >= L) {
    if (lane == 0) *dst = make_float2(0.f, 0.f);
    return;
  }
  const uint2 a = *reinterpret_cast<const uint2*>(go + bb * g_sb + i * g_sl + hh * g_sh + lane * 4);
  const uint2 c = *reinterpret_cast<const uint2*>(o + bb * o_sb + i * o_sl + hh * o_sh + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 c0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c.x));
  const float2 c1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c.y));
  float sum = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y;
#pragma unroll
  for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (lane == 0) {
    const long long idx = ((long long)bb * H + hh) * L + i;
    *dst = make_float2(-lse[idx] * 1.4426950408889634f, scale * (sum - (glse ? glse[idx] : 0.f)));
  }
}

// dq[b, i, h, :] (bf16, strided) = dq_acc (fp32, contiguous [B, L, H, 128])
__global__ void attn_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows, int H, int L,
                                    long long sb_, long long sl_, long long sh_) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;     // one thread per 8 values
  if (idx >= rows * 16) return;
  const long long row = idx >> 4;
  const int c = int(idx & 15) * 8;
  const int hh = int(row % H);
  const long long bl = row / H;
  const int i = int(bl % L);
  const long long bb = bl / L;
  const float4 x = *reinterpret_cast<const float4*>(acc + row * HD + c);
  const float4 y = *reinterpret_cast<const float4*>(acc + row * HD + c + 4);
  uint4 o;
  o.x = pack_bf16(x.x, x.y); o.y = pack_bf16(x.z, x.w); o.z = pack_bf16(y.x, y.y); o.w = pack_bf16(y.z, y.w);
  *reinterpret_cast<uint4*>(dq + bb * sb_ + i * sl_ + hh * sh_ + c) = o;
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
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
static int g_last_encode = 0;
static int g_pingpong = 0;     // forward variant: softmax warpgroups take turns on the exponentials (1) or run freely (0)
static int g_p_tmem = 1;       // backward variant: P^T in tensor memory (1) or in shared memory (0)
static int g_fwd_p_tmem = 1;   // forward variant: P as the TMEM operand of P V (1, default) or through shared memory (0)

// [B, L, H, 128] bf16 with element strides (sb, sl, sh); box = 64 columns x 1 head x box_rows rows x 1 batch
static int make_tmap(CUtensorMap* out, const void* base, int B, int L, int H, long long sb, long long sl, long long sh,
                     int box_rows = 128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (sb % 8) || (sl % 8) || (sh % 8)) return -4;
  cuuint64_t dims[4] = {HD, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)sl * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_encode = (int)r; return -2; }
  return 0;
}

}  // namespace attn
}  // namespace sb

extern "C" int sb_attn_last_encode_result() { return sb::attn::g_last_encode; }
extern "C" int sb_attn_set_bwd_variant(int p_in_tmem) { sb::attn::g_p_tmem = p_in_tmem ? 1 : 0; return 0; }
extern "C" int sb_attn_set_fwd_variant(int pingpong) { sb::attn::g_pingpong = pingpong ? 1 : 0; return 0; }
extern "C" int sb_attn_set_fwd_p_tmem(int on) { sb::attn::g_fwd_p_tmem = on ? 1 : 0; return 0; }

// Attention forward.  q [B, Lq, H, 128], k and v [B, Lk, H, 128], out like q: bf16, last dimension contiguous, the
// other strides (in elements) multiples of 8.  lse [B, H, Lq] fp32.  causal needs Lq == Lk (row i sees keys 0..i).
extern "C" int sb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int Lq, int Lk,
                           const long long* q_str, const long long* k_str, const long long* v_str, const long long* o_str,
                           int causal, float scale, unsigned int* status, cudaStream_t stream) {
  using namespace sb;
  using namespace sb::attn;
  if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0) return 0;
  if (causal && Lq != Lk) return -3;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (o_str[0] % 8) || (o_str[1] % 8) || (o_str[2] % 8)) return -4;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap(&tq, q, B, Lq, H, q_str[0], q_str[1], q_str[2]))) return rc;
  if ((rc = make_tmap(&tk, k, B, Lk, H, k_str[0], k_str[1], k_str[2]))) return rc;
  if ((rc = make_tmap(&tv, v, B, Lk, H, v_str[0], v_str[1], v_str[2]))) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) return -5;
    if (cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) return -5;
    attr_set = true;
  }
  FwdParams p{reinterpret_cast<__nv_bfloat16*>(out), lse, o_str[0], o_str[1], o_str[2], B, H, Lq, Lk, causal,
              scale * 1.4426950408889634f, scale, status, g_pingpong};
  dim3 grid((Lq + 2 * BQ - 1) / (2 * BQ), H, B);
  if (g_fwd_p_tmem) attn_fwd_kernel<true><<<grid, FWD_THREADS, FWD_SMEM, stream>>>(tq, tk, tv, p);
  else attn_fwd_kernel<false><<<grid, FWD_THREADS, FWD_SMEM, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

// Attention backward.  go/q/out [B, Lq, H, 128], k/v [B, Lk, H, 128] (bf16, strided as in the forward); lse and the
// optional dlse [B, H, Lq] fp32; scratch: stats (2 * B * H * 64 * ceil(Lq / 64) floats) and dq_acc [B, Lq, H, 128] fp32
// (the kernel adds into it: zero it before the first of the calls that share it).  Results: dq (strided, bf16; null =
// leave the sum in dq_acc), dk and dv (contiguous [B, Lk, H, 128], bf16).  Three launches (two without dq).
extern "C" int sb_attn_bwd(const void* go, const void* q, const void* k, const void* v, const void* out, const float* lse,
                           const float* glse, float* stats, float* dq_acc, void* dq, void* dk, int B, int H, int Lq, int Lk,
                           void* dv, const long long* g_str, const long long* q_str, const long long* k_str,
                           const long long* v_str, const long long* o_str, const long long* dq_str, const long long* dk_str,
                           const long long* dv_str, int causal, float scale, unsigned int* status, cudaStream_t stream) {
  using namespace sb;
  using namespace sb::attn;
  if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0) return 0;
  if (causal && Lq != Lk) return -3;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(go) | reinterpret_cast<uintptr_t>(dq_acc) |
       reinterpret_cast<uintptr_t>(stats)) & 15) return -4;
  for (int i = 0; i < 3; ++i)
    if ((dq_str[i] % 8) || (o_str[i] % 8) || (g_str[i] % 8) || (dk_str[i] % 8) || (dv_str[i] % 8)) return -4;
  CUtensorMap tq, tk, tv, tg, tdq;
  int rc;
  if ((rc = make_tmap(&tq, q, B, Lq, H, q_str[0], q_str[1], q_str[2], BQ2))) return rc;
  if ((rc = make_tmap(&tg, go, B, Lq, H, g_str[0], g_str[1], g_str[2], BQ2))) return rc;
  if ((rc = make_tmap(&tk, k, B, Lk, H, k_str[0], k_str[1], k_str[2]))) return rc;
  if ((rc = make_tmap(&tv, v, B, Lk, H, v_str[0], v_str[1], v_str[2]))) return rc;
  {
    // dq_acc: fp32 [B, Lq, H, 128] contiguous, box = 128 columns x 1 head x 64 rows, no swizzle (dense staging tile)
    EncodeTiledFn enc = get_encode();
    if (!enc) return -1;
    cuuint64_t dims[4] = {HD, (cuuint64_t)H, (cuuint64_t)Lq, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)HD * 4, (cuuint64_t)H * HD * 4, (cuuint64_t)Lq * H * HD * 4};
    cuuint32_t box[4] = {HD, 1, BQ2, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { g_last_encode = (int)r; return -2; }
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return -5;
    if (cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return -5;
    attr_set = true;
  }
  const int lpad = (Lq + BQ2 - 1) / BQ2 * BQ2;
  const long long rows = (long long)B * lpad * H;
  attn_stats_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)go, (const __nv_bfloat16*)out, lse, glse, stats, B, H, Lq, lpad, scale, g_str[0], g_str[1], g_str[2],
      o_str[0], o_str[1], o_str[2]);
  BwdParams p{stats, reinterpret_cast<__nv_bfloat16*>(dk), reinterpret_cast<__nv_bfloat16*>(dv),
              {dk_str[0], dk_str[1], dk_str[2]}, {dv_str[0], dv_str[1], dv_str[2]}, B, H, Lq, Lk,
              causal, scale * 1.4426950408889634f, scale, status};
  dim3 grid((Lk + BK - 1) / BK, H, B);
  if (g_p_tmem) attn_bwd_kernel<true><<<grid, BWD_THREADS, BWD_SMEM, stream>>>(tq, tk, tv, tg, tdq, p);
  else attn_bwd_kernel<false><<<grid, BWD_THREADS, BWD_SMEM, stream>>>(tq, tk, tv, tg, tdq, p);
  const long long orows = (long long)B * Lq * H;
  // dq == null: the caller keeps accumulating into dq_acc over several calls (ring attention) and casts at the end
  if (dq)
    attn_dq_cast_kernel<<<(unsigned)((orows * 16 + 255) / 256), 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, orows, H, Lq,
                                                                                 dq_str[0], dq_str[1], dq_str[2]);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

// ------------------------------------------------------------------------------------ merging partial attention results
// Ring attention computes, per query row, S partial results (o_s, lse_s) over disjoint key sets.  Their combination is
//     lse = log sum_s exp(lse_s),   w_s = exp(lse_s - lse),   o = sum_s w_s o_s
// and its backward  do_s = w_s do,  dlse_s = w_s (do . o_s - do . o).  One warp per (batch, row, head); partials are
// addressed through element strides, so slices of larger attention outputs are read in place.
namespace sb {
namespace attn {
constexpr int MERGE_MAX = 16;
struct MergeArgs {
  const __nv_bfloat16* o[MERGE_MAX];      // [B, L, H, 128] with strides (osb, osl, osh)
  const float* lse[MERGE_MAX];            // [B, H, L] with strides (lsb, lsh, lsl)
  long long osb[MERGE_MAX], osl[MERGE_MAX], osh[MERGE_MAX];
  long long lsb[MERGE_MAX], lsh[MERGE_MAX], lsl[MERGE_MAX];
  int S, B, L, H;
};
struct MergeGrads {
  __nv_bfloat16* go[MERGE_MAX];           // contiguous [B, L, H, 128]
  float* glse[MERGE_MAX];                 // contiguous [B, H, L]
};

__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 q = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&f)[4]) {
  uint2 q;
  q.x = pack_bf16(f[0], f[1]); q.y = pack_bf16(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = q;
}

__global__ void __launch_bounds__(256)
attn_merge_fwd_kernel(MergeArgs a, __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)a.B * a.L * a.H) return;
  const int h = int(w % a.H);
  const long long bl = w / a.H;
  const int l = int(bl % a.L), b = int(bl / a.L);
  float ls[MERGE_MAX], m = -INFINITY;
#pragma unroll
  for (int s = 0; s < MERGE_MAX; ++s)
    if (s < a.S) { ls[s] = a.lse[s][b * a.lsb[s] + h * a.lsh[s] + l * a.lsl[s]]; m = fmaxf(m, ls[s]); }
  float den = 0.f;
#pragma unroll
  for (int s = 0; s < MERGE_MAX; ++s)
    if (s < a.S) den += __expf(ls[s] - m);
  const float lse = m + __logf(den);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < MERGE_MAX; ++s)
    if (s < a.S) {
      const float wgt = __expf(ls[s] - lse);
      float f[4];
      ld4(a.o[s] + b * a.osb[s] + l * a.osl[s] + h * a.osh[s] + lane * 4, f);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += wgt * f[j];
    }
  st4(out + ((long long)(b * a.L + l) * a.H + h) * HD + lane * 4, acc);
  if (lane == 0) lse_out[((long long)b * a.H + h) * a.L + l] = lse;
}

__global__ void __launch_bounds__(256)
attn_merge_bwd_kernel(MergeArgs a, MergeGrads g, const __nv_bfloat16* __restrict__ out, const float* __restrict__ lse_out,
                      const __nv_bfloat16* __restrict__ gout, long long g_sb, long long g_sl, long long g_sh) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)a.B * a.L * a.H) return;
  const int h = int(w % a.H);
  const long long bl = w / a.H;
  const int l = int(bl % a.L), b = int(bl / a.L);
  const long long row = ((long long)(b * a.L + l) * a.H + h) * HD + lane * 4;
  const long long stat = ((long long)b * a.H + h) * a.L + l;
  float go[4], o[4];
  ld4(gout + b * g_sb + l * g_sl + h * g_sh + lane * 4, go);
  ld4(out + row, o);
  float dot_o = go[0] * o[0] + go[1] * o[1] + go[2] * o[2] + go[3] * o[3];
#pragma unroll
  for (int off = 16; off; off >>= 1) dot_o += __shfl_xor_sync(0xffffffffu, dot_o, off);
  const float lse = lse_out[stat];
#pragma unroll
  for (int s = 0; s < MERGE_MAX; ++s)
    if (s < a.S) {
      const float wgt = __expf(a.lse[s][b * a.lsb[s] + h * a.lsh[s] + l * a.lsl[s]] - lse);
      float f[4], d[4];
      ld4(a.o[s] + b * a.osb[s] + l * a.osl[s] + h * a.osh[s] + lane * 4, f);
      float dot = go[0] * f[0] + go[1] * f[1] + go[2] * f[2] + go[3] * f[3];
#pragma unroll
      for (int off = 16; off; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
#pragma unroll
      for (int j = 0; j < 4; ++j) d[j] = wgt * go[j];
      st4(g.go[s] + row, d);
      if (lane == 0) g.glse[s][stat] = wgt * (dot - dot_o);
    }
}
}  // namespace attn
}  // namespace sb

// S partial results -> merged output (bf16, contiguous [B, L, H, 128]) and merged lse (contiguous [B, H, L]).
// o_ptrs / lse_ptrs: S device pointers; o_str: S x 3 element strides (b, l, h); lse_str: S x 3 element strides (b, h, l).
extern "C" int sb_attn_merge_fwd(const void* const* o_ptrs, const void* const* lse_ptrs, const long long* o_str,
                                 const long long* lse_str, int S, int B, int L, int H, void* out, float* lse_out,
                                 cudaStream_t st) {
  using namespace sb::attn;
  if (S < 1 || S > MERGE_MAX) return -1;
  if ((long long)B * L * H == 0) return 0;
  MergeArgs a{};
  for (int s = 0; s < S; ++s) {
    a.o[s] = (const __nv_bfloat16*)o_ptrs[s]; a.lse[s] = (const float*)lse_ptrs[s];
    a.osb[s] = o_str[3 * s]; a.osl[s] = o_str[3 * s + 1]; a.osh[s] = o_str[3 * s + 2];
    a.lsb[s] = lse_str[3 * s]; a.lsh[s] = lse_str[3 * s + 1]; a.lsl[s] = lse_str[3 * s + 2];
    if ((reinterpret_cast<uintptr_t>(o_ptrs[s]) & 7) || (a.osb[s] % 4) || (a.osl[s] % 4) || (a.osh[s] % 4)) return -4;
  }
  a.S = S; a.B = B; a.L = L; a.H = H;
  const long long rows = (long long)B * L * H;
  attn_merge_fwd_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(a, (__nv_bfloat16*)out, lse_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Backward of the merge: go_ptrs[s] (bf16, contiguous [B, L, H, 128]) and glse_ptrs[s] (fp32, contiguous [B, H, L]).
extern "C" int sb_attn_merge_bwd(const void* const* o_ptrs, const void* const* lse_ptrs, const long long* o_str,
                                 const long long* lse_str, int S, int B, int L, int H, const void* out, const float* lse_out,
                                 const void* gout, const long long* g_str, void* const* go_ptrs, void* const* glse_ptrs,
                                 cudaStream_t st) {
  using namespace sb::attn;
  if (S < 1 || S > MERGE_MAX) return -1;
  if ((long long)B * L * H == 0) return 0;
  MergeArgs a{};
  MergeGrads g{};
  for (int s = 0; s < S; ++s) {
    a.o[s] = (const __nv_bfloat16*)o_ptrs[s]; a.lse[s] = (const float*)lse_ptrs[s];
    a.osb[s] = o_str[3 * s]; a.osl[s] = o_str[3 * s + 1]; a.osh[s] = o_str[3 * s + 2];
    a.lsb[s] = lse_str[3 * s]; a.lsh[s] = lse_str[3 * s + 1]; a.lsl[s] = lse_str[3 * s + 2];
    g.go[s] = (__nv_bfloat16*)go_ptrs[s]; g.glse[s] = (float*)glse_ptrs[s];
    if ((reinterpret_cast<uintptr_t>(o_ptrs[s]) & 7) || (a.osb[s] % 4) || (a.osl[s] % 4) || (a.osh[s] % 4)) return -4;
  }
  if ((reinterpret_cast<uintptr_t>(gout) & 7) || (g_str[0] % 4) || (g_str[1] % 4) || (g_str[2] % 4)) return -4;
  a.S = S; a.B = B; a.L = L; a.H = H;
  const long long rows = (long long)B * L * H;
  attn_merge_bwd_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(a, g, (const __nv_bfloat16*)out, lse_out,
                                                                            (const __nv_bfloat16*)gout, g_str[0], g_str[1], g_str[2]);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
