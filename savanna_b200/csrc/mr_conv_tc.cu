// Hyena-MR on tensor cores: the causal FIR of <= 128 taps shared by the 16+ channels of a group is a product
// with a banded Toeplitz matrix, so a [16 time x 16 channel] output block is
//     Y[i0] = sum_{d = 0..8} A_d * U[i0 - 16 d],      A_d[r][c] = h[16 d + r - c]   (zero outside 0..K-1)
// i.e. nine m16n8k16 bf16 MMAs per 8 channels with the A fragments (functions of the filter only) held in
// registers for the whole kernel and the B fragments read from a shared-memory image of u = x2*v with
// ldmatrix.  (The group width of 16 channels is too narrow for a tcgen05 tile — its minimum useful N at M = 128
// would leave the Toeplitz operand, 64 KB per group, as the only thing in shared memory — so this operator uses
// the warp-level MMA path; the wide GEMMs and attention use tcgen05.)  fp32 accumulation; u and h are rounded to
// bf16 for the product, like every other tensor-core operand in the model.
//
//   mr_tc_fwd : z = x1 * (h*u + bias*u)                                  tile 128 time x 64 channels
//   mr_tc_bwd : dfeat = (dz*y, du*v, du*x2), du = h (*) g + bias*g (anticausal), g = dz*x1;
//               dh[s] += sum g[t] u[t-s]  (as P_d = G_blk^T-contracted-over-channels MMAs), dbias += sum g*u
//               tile 64 time x 64 channels, y recomputed instead of saved
// Rows before the sequence start come from `halo` [B, K-1, 3D] (context-parallel shards) or are zero; the
// backward kernel also produces the halo rows' gradient.  Requires dg % 16 == 0 (a warp's 16-channel slab shares
// one filter); other group widths use the CUDA-core kernels in mr_conv.cu.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "halo_src.cuh"

#include "device_info.h"

namespace sb {
typedef __nv_bfloat16 bf16;

constexpr int TC_CH = 64;                 // channels per tile (4 slabs of 16)
constexpr int TC_LD = 72;                 // padded smem row (elements) -> 144 B, conflict-free ldmatrix
constexpr int TC_HALO = 128;              // staged past/future rows
constexpr int TC_THREADS = 256;
constexpr int FWD_TT = 128;
constexpr int BWD_TT = 64;
constexpr int ND = 9;                     // Toeplitz block diagonals d = 0..8

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
__device__ __forceinline__ float tap(const float* h, int K, int s) { return (s >= 0 && s < K) ? h[s] : 0.f; }

// A fragments of the Toeplitz block diagonals for this thread.  transpose = false: A_d[r][c] = h[16d + r - c]
// (causal);  transpose = true: A_d[r][c] = h[16d + c - r] (the anticausal product of the backward pass).
__device__ __forceinline__ void toeplitz_frags(uint32_t (&a)[ND][4], const float* h, int K, int lane, bool transpose) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int d = 0; d < ND; ++d) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = g + ((q & 1) ? 8 : 0), c = 2 * t + ((q & 2) ? 8 : 0);
      const int s0 = transpose ? 16 * d + c - r : 16 * d + r - c;
      const int s1 = transpose ? s0 + 1 : s0 - 1;
      a[d][q] = pack2(tap(h, K, s0), tap(h, K, s1));
    }
  }
}

struct MrArgs {
  const bf16* feat; HaloSrc halo; const float* h; const float* bias;
  int L, D, K, dg;
  // context-parallel backward: rows [L, L + K - 1) of x1 and dz come from the next chunk's staged head (peer memory)
  int ahead_mode; HaloSrc ahead_f, ahead_g;
};

// Loads 8 channels (c0..c0+7) of feature row t (halo-aware): returns false (zeros) outside the sequence.
__device__ __forceinline__ bool load_row8(const MrArgs& a, int b, int t, int c0, float (&x1)[8], float (&x2)[8], float (&v)[8]) {
  const bf16* row = nullptr;
  if (t >= 0 && t < a.L) row = a.feat + ((size_t)b * a.L + t) * 3 * a.D;
  else if (t < 0 && t >= -(a.K - 1)) row = halo_row(a.halo, b, t + a.K - 1, a.K - 1, (size_t)3 * a.D);
  if (!row || c0 >= a.D) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { x1[i] = 0.f; x2[i] = 0.f; v[i] = 0.f; }
    return false;
  }
  const uint4* p = reinterpret_cast<const uint4*>(row + 3 * c0);
  uint4 q0 = p[0], q1 = p[1], q2 = p[2];
  float all[24];
  const uint32_t w[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
#pragma unroll
  for (int i = 0; i < 12; ++i) { float2 f = unpack2(w[i]); all[2 * i] = f.x; all[2 * i + 1] = f.y; }
#pragma unroll
  for (int i = 0; i < 8; ++i) { x1[i] = all[3 * i]; x2[i] = all[3 * i + 1]; v[i] = all[3 * i + 2]; }
  return true;
}
__device__ __forceinline__ void st8(bf16* dst, const float (&f)[8]) {
  uint4 o = make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  *reinterpret_cast<uint4*>(dst) = o;
}

// ------------------------------------------------------------------------------------ forward
// smem: U [(HALO + TT) x LD] bf16 (row r <-> local time r - HALO), X1 [TT x LD] (overwritten with z)
constexpr int FWD_SMEM = ((TC_HALO + FWD_TT) + FWD_TT) * TC_LD * 2;

__global__ void __launch_bounds__(TC_THREADS)
mr_tc_fwd_kernel(MrArgs a, bf16* __restrict__ z) {
  extern __shared__ __align__(16) uint8_t smraw[];
  bf16* sU = reinterpret_cast<bf16*>(smraw);
  bf16* sX = sU + (TC_HALO + FWD_TT) * TC_LD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c_base = blockIdx.x * TC_CH, t0 = blockIdx.y * FWD_TT, b = blockIdx.z;
  // ---- stage u (and x1) : 8 threads per row, 8 channels each
  for (int i = tid; i < (TC_HALO + FWD_TT) * 8; i += TC_THREADS) {
    const int r = i >> 3, cv = i & 7;
    const int t = t0 + r - TC_HALO;
    float x1[8], x2[8], v[8], u[8];
    load_row8(a, b, t, c_base + cv * 8, x1, x2, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = x2[j] * v[j];
    st8(sU + r * TC_LD + cv * 8, u);
    if (r >= TC_HALO) st8(sX + (r - TC_HALO) * TC_LD + cv * 8, x1);
  }
  const int slab = warp & 3, half = warp >> 2;
  const int ch0 = c_base + slab * 16;
  uint32_t A[ND][4];
  {
    const int grp = min(ch0, a.D - 1) / a.dg;
    toeplitz_frags(A, a.h + (size_t)grp * a.K, a.K, lane, false);
  }
  const int nd = min(ND, (a.K - 1) / 16 + 2);
  __syncthreads();
  const int g = lane >> 2, tq = lane & 3;
  // ldmatrix.trans lane address: matrix m = lane/8 -> (time 8*(m&1), channel 8*(m>>1)), row lane%8
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_col = (lane >> 4) * 8;
  const float b_lo0 = ch0 + 2 * tq < a.D ? a.bias[ch0 + 2 * tq] : 0.f, b_lo1 = ch0 + 2 * tq + 1 < a.D ? a.bias[ch0 + 2 * tq + 1] : 0.f;
  const float b_hi0 = ch0 + 8 + 2 * tq < a.D ? a.bias[ch0 + 8 + 2 * tq] : 0.f, b_hi1 = ch0 + 9 + 2 * tq < a.D ? a.bias[ch0 + 9 + 2 * tq] : 0.f;
#pragma unroll 1
  for (int blk = 0; blk < FWD_TT / 32; ++blk) {
    const int i0 = half * (FWD_TT / 2) + blk * 16;            // local output time of the block
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int d = 0; d < ND; ++d) {
      if (d < nd) {
        const int jr = TC_HALO + i0 - 16 * d;                   // smem row of the input block
        uint32_t bf[4];
        ldsm_x4_t(bf, smem_addr(sU + (jr + lm_row) * TC_LD + slab * 16 + lm_col));
        mma16816(acc[0], A[d], bf[0], bf[1]);
        mma16816(acc[1], A[d], bf[2], bf[3]);
      }
    }
    // epilogue in place: z = x1 * (y + bias*u)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = i0 + g + hh * 8, col = slab * 16 + nt * 8 + 2 * tq;
        const float2 u = unpack2(*reinterpret_cast<const uint32_t*>(sU + (TC_HALO + row) * TC_LD + col));
        uint32_t* xp = reinterpret_cast<uint32_t*>(sX + row * TC_LD + col);
        const float2 x = unpack2(*xp);
        const float bi0 = nt ? b_hi0 : b_lo0, bi1 = nt ? b_hi1 : b_lo1;
        *xp = pack2(x.x * (acc[nt][hh * 2] + bi0 * u.x), x.y * (acc[nt][hh * 2 + 1] + bi1 * u.y));
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < FWD_TT * 8; i += TC_THREADS) {
    const int r = i >> 3, cv = i & 7;
    const int t = t0 + r, c = c_base + cv * 8;
    if (t < a.L && c < a.D)
      *reinterpret_cast<uint4*>(z + ((size_t)b * a.L + t) * a.D + c) = *reinterpret_cast<const uint4*>(sX + r * TC_LD + cv * 8);
  }
}

// ------------------------------------------------------------------------------------ backward
// smem rows: U [HALO + TT] (past), G [TT + HALO] (future), tiles X2, V, DZ [TT]; staging for dfeat reuses G.
constexpr int BWD_ROWS = TC_HALO + BWD_TT;
constexpr int BWD_SMEM = (2 * BWD_ROWS + 3 * BWD_TT) * TC_LD * 2 + (4 * 128 + TC_CH) * 4;

__global__ void __launch_bounds__(TC_THREADS, 2)
mr_tc_bwd_kernel(MrArgs a, const bf16* __restrict__ dz, bf16* __restrict__ dfeat, bf16* __restrict__ dhalo,
                 float* __restrict__ dh, float* __restrict__ dbias, int n_halo_tiles) {
  extern __shared__ __align__(16) uint8_t smraw[];
  bf16* sU = reinterpret_cast<bf16*>(smraw);
  bf16* sG = sU + BWD_ROWS * TC_LD;
  bf16* sX2 = sG + BWD_ROWS * TC_LD;
  bf16* sV = sX2 + BWD_TT * TC_LD;
  bf16* sDZ = sV + BWD_TT * TC_LD;
  float* sdh = reinterpret_cast<float*>(sDZ + BWD_TT * TC_LD);      // [4 slabs][128]
  float* sdb = sdh + 4 * 128;                                        // [64]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c_base = blockIdx.x * TC_CH, b = blockIdx.z;
  const int t0 = ((int)blockIdx.y - n_halo_tiles) * BWD_TT;          // halo tiles have negative t0
  for (int i = tid; i < 4 * 128 + TC_CH; i += TC_THREADS) sdh[i] = 0.f;
  // ---- stage U rows [t0-HALO, t0+TT) and G rows [t0, t0+TT+HALO); tile rows also keep x2, v, dz
  float db_part[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) db_part[j] = 0.f;
  for (int i = tid; i < (TC_HALO + BWD_TT + TC_HALO) * 8; i += TC_THREADS) {
    const int r = i >> 3, cv = i & 7;                                // r: 0 .. HALO+TT+HALO-1  <->  t = t0 - HALO + r
    const int t = t0 - TC_HALO + r, c0 = c_base + cv * 8;
    float x1[8], x2[8], v[8], f[8];
    load_row8(a, b, t, c0, x1, x2, v);
    float gz[8];
    const bool in_seq = t >= 0 && t < a.L && c0 < a.D;
    if (in_seq) {
      const uint4 q = *reinterpret_cast<const uint4*>(dz + ((size_t)b * a.L + t) * a.D + c0);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 p = unpack2(w[j]); gz[2 * j] = p.x; gz[2 * j + 1] = p.y; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) gz[j] = 0.f;
    }
    if (r < BWD_ROWS) {                                              // U rows
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = x2[j] * v[j];
      st8(sU + r * TC_LD + cv * 8, f);
    }
    if (r >= TC_HALO) {                                              // G rows
      float gg[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) gg[j] = gz[j] * x1[j];
      st8(sG + (r - TC_HALO) * TC_LD + cv * 8, gg);
      if (r < BWD_ROWS) {                                            // the tile itself
        const int tr = r - TC_HALO;
        st8(sX2 + tr * TC_LD + cv * 8, x2);
        st8(sV + tr * TC_LD + cv * 8, v);
        st8(sDZ + tr * TC_LD + cv * 8, gz);
#pragma unroll
        for (int j = 0; j < 8; ++j) db_part[j] += gg[j] * x2[j] * v[j];
      }
    }
  }
  {
    const int cv = tid & 7;                                          // fixed per thread over the loop above
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&sdb[cv * 8 + j], db_part[j]);
  }
  const int slab = warp & 3, half = warp >> 2;
  const int ch0 = c_base + slab * 16;
  const int grp = min(ch0, a.D - 1) / a.dg;
  const float* hg = a.h + (size_t)grp * a.K;
  const int nd = min(ND, (a.K - 1) / 16 + 2);
  const int g = lane >> 2, tq = lane & 3;
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_col = (lane >> 4) * 8;
  __syncthreads();
  // ---- pass 1: y (causal) and du (anticausal) for this warp's blocks; results parked in registers
  float yacc[2][2][4], dacc[2][2][4];
  {
    uint32_t A[ND][4];
    toeplitz_frags(A, hg, a.K, lane, false);
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int i0 = half * 32 + blk * 16;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) yacc[blk][nt][q] = 0.f;
#pragma unroll
      for (int d = 0; d < ND; ++d) {
        if (d < nd) {
          uint32_t bf[4];
          ldsm_x4_t(bf, smem_addr(sU + (TC_HALO + i0 - 16 * d + lm_row) * TC_LD + slab * 16 + lm_col));
          mma16816(yacc[blk][0], A[d], bf[0], bf[1]);
          mma16816(yacc[blk][1], A[d], bf[2], bf[3]);
        }
      }
    }
    toeplitz_frags(A, hg, a.K, lane, true);
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int i0 = half * 32 + blk * 16;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) dacc[blk][nt][q] = 0.f;
#pragma unroll
      for (int d = 0; d < ND; ++d) {
        if (d < nd) {
          uint32_t bf[4];
          ldsm_x4_t(bf, smem_addr(sG + (i0 + 16 * d + lm_row) * TC_LD + slab * 16 + lm_col));
          mma16816(dacc[blk][0], A[d], bf[0], bf[1]);
          mma16816(dacc[blk][1], A[d], bf[2], bf[3]);
        }
      }
      // du += bias * g  (g is read now: its shared-memory rows are reused as output staging later)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int row = i0 + g + hh * 8, col = slab * 16 + nt * 8 + 2 * tq;
          const float2 gg = unpack2(*reinterpret_cast<const uint32_t*>(sG + row * TC_LD + col));
          const int ca = c_base + col;
          dacc[blk][nt][hh * 2] += (ca < a.D ? a.bias[ca] : 0.f) * gg.x;
          dacc[blk][nt][hh * 2 + 1] += (ca + 1 < a.D ? a.bias[ca + 1] : 0.f) * gg.y;
        }
    }
  }
  // ---- pass 2: filter gradient.  P_d[i][j] = sum_c G[i0+i][c] U[i0-16d+j][c]  ->  dh[16d + i - j]
  if (t0 >= 0) {
    float P[ND][2][4];
#pragma unroll
    for (int d = 0; d < ND; ++d)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) P[d][nt][q] = 0.f;
    // non-transposed ldmatrix lane addresses
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;       // A: (rows 0-7|8-15, k 0-7|8-15)
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;       // B: (time 0-7 k0-7, time 0-7 k8-15, time 8-15 ...)
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int i0 = half * 32 + blk * 16;
      uint32_t af[4];
      ldsm_x4(af, smem_addr(sG + (i0 + a_row) * TC_LD + slab * 16 + a_col));
#pragma unroll
      for (int d = 0; d < ND; ++d) {
        if (d < nd) {
          uint32_t bf[4];
          ldsm_x4(bf, smem_addr(sU + (TC_HALO + i0 - 16 * d + b_row) * TC_LD + slab * 16 + b_col));
          mma16816(P[d][0], af, bf[0], bf[1]);
          mma16816(P[d][1], af, bf[2], bf[3]);
        }
      }
    }
#pragma unroll
    for (int d = 0; d < ND; ++d) {
      if (d < nd) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int i = g + ((q & 2) ? 8 : 0), j = nt * 8 + 2 * tq + (q & 1);
            const int s = 16 * d + i - j;
            if (s >= 0 && s < a.K) atomicAdd(&sdh[slab * 128 + s], P[d][nt][q]);
          }
      }
    }
  }
  __syncthreads();                                                    // all MMAs done: G rows can be reused as staging
  bf16* sOut = sG;                                                    // [TT][3 * 64 (+pad 8)] -> row stride 200 elements
  constexpr int OLD = 3 * TC_CH + 8;
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
    const int i0 = half * 32 + blk * 16;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = i0 + g + hh * 8, col = slab * 16 + nt * 8 + 2 * tq;
        const float2 u = unpack2(*reinterpret_cast<const uint32_t*>(sU + (TC_HALO + row) * TC_LD + col));
        const float2 x2 = unpack2(*reinterpret_cast<const uint32_t*>(sX2 + row * TC_LD + col));
        const float2 v = unpack2(*reinterpret_cast<const uint32_t*>(sV + row * TC_LD + col));
        const float2 gz = unpack2(*reinterpret_cast<const uint32_t*>(sDZ + row * TC_LD + col));
        const int ca = c_base + col;
        const float bi0 = ca < a.D ? a.bias[ca] : 0.f, bi1 = ca + 1 < a.D ? a.bias[ca + 1] : 0.f;
        const float y0 = yacc[blk][nt][hh * 2] + bi0 * u.x, y1 = yacc[blk][nt][hh * 2 + 1] + bi1 * u.y;
        const float du0 = dacc[blk][nt][hh * 2], du1 = dacc[blk][nt][hh * 2 + 1];
        bf16* o = sOut + row * OLD + 3 * col;
        o[0] = __float2bfloat16_rn(gz.x * y0); o[1] = __float2bfloat16_rn(du0 * v.x); o[2] = __float2bfloat16_rn(du0 * x2.x);
        o[3] = __float2bfloat16_rn(gz.y * y1); o[4] = __float2bfloat16_rn(du1 * v.y); o[5] = __float2bfloat16_rn(du1 * x2.y);
      }
  }
  __syncthreads();
  // ---- coalesced write-out: 24 vectors of 16 B per row
  for (int i = tid; i < BWD_TT * 24; i += TC_THREADS) {
    const int r = i / 24, q = i - r * 24;
    const int t = t0 + r, c3 = 3 * c_base + q * 8;
    if (c3 >= 3 * a.D) continue;
    const uint4 val = *reinterpret_cast<const uint4*>(sOut + r * OLD + q * 8);
    if (t >= 0 && t < a.L) *reinterpret_cast<uint4*>(dfeat + ((size_t)b * a.L + t) * 3 * a.D + c3) = val;
    else if (t < 0 && t >= -(a.K - 1) && dhalo) *reinterpret_cast<uint4*>(dhalo + ((size_t)b * (a.K - 1) + (t + a.K - 1)) * 3 * a.D + c3) = val;
  }
  if (t0 >= 0) {
    for (int i = tid; i < 4 * 128; i += TC_THREADS) {
      const int sl = i >> 7, s = i & 127;
      const int c = c_base + sl * 16;
      if (s < a.K && c < a.D) atomicAdd(dh + (size_t)(c / a.dg) * a.K + s, sdh[i]);
    }
    for (int i = tid; i < TC_CH; i += TC_THREADS)
      if (c_base + i < a.D) atomicAdd(dbias + c_base + i, sdb[i]);
  }
}

// ------------------------------------------------------------------------------------ backward, streaming form
// A CTA owns 64 channels and a segment of consecutive 64-row tiles.  The rows of u = x2*v and g = dz*x1 live in two
// shared-memory rings of 320 rows (128 behind the current tile, the tile, 128 ahead); each tile step stages only the
// 64 new rows at the front, so every input row is read once per CTA instead of five times, and the filter-gradient
// accumulators stay in registers over the whole segment (one flush per CTA instead of one per tile).  Per tile: y and
// du by Toeplitz MMAs into a bf16 staging tile, the filter-gradient MMAs (each warp keeps half of the nine block
// diagonals for all 64 rows of its slab), then a coalesced pass that re-reads the tile's features and dz from global
// memory (L2 hits), combines them with y and du and stores dfeat.
constexpr int SB_TT = 64;                         // rows per tile step
constexpr int SB_RING = TC_HALO + SB_TT + TC_HALO; // 320
constexpr int SB_SMEM = (2 * SB_RING + 2 * SB_TT) * TC_LD * 2 + (4 * 128 + TC_CH) * 4;

__device__ __forceinline__ int ring_pos(int p) { return p < 0 ? p + SB_RING : (p >= SB_RING ? p - SB_RING : p); }

__global__ void __launch_bounds__(TC_THREADS, 2)
mr_tc_bwd_stream_kernel(MrArgs a, const bf16* __restrict__ dz, bf16* __restrict__ dfeat, bf16* __restrict__ dhalo,
                        float* __restrict__ dh, float* __restrict__ dbias, int n_halo_tiles, int n_tiles, int tiles_per_seg) {
  extern __shared__ __align__(16) uint8_t smraw[];
  bf16* sU = reinterpret_cast<bf16*>(smraw);
  bf16* sG = sU + SB_RING * TC_LD;
  bf16* sY = sG + SB_RING * TC_LD;                 // [64][LD] y (with the bias term) of the current tile
  bf16* sDU = sY + SB_TT * TC_LD;                  // [64][LD] du
  float* sdh = reinterpret_cast<float*>(sDU + SB_TT * TC_LD);       // [4 slabs][128]
  float* sdb = sdh + 4 * 128;                                        // [64]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c_base = blockIdx.x * TC_CH, b = blockIdx.z;
  const int k0 = blockIdx.y * tiles_per_seg, k1 = min(k0 + tiles_per_seg, n_tiles);
  if (k0 >= k1) return;
  const int seg_t0 = (k0 - n_halo_tiles) * SB_TT, seg_t1 = (k1 - n_halo_tiles) * SB_TT;
  const int base_t = seg_t0 - TC_HALO;             // time of ring row 0 (the ring wraps modulo SB_RING from there)
  for (int i = tid; i < 4 * 128 + TC_CH; i += TC_THREADS) sdh[i] = 0.f;

  float db_part[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) db_part[j] = 0.f;
  // rows [t_first, t_first + count) -> ring; u for every row that exists (sequence or halo), g inside the sequence
  auto stage = [&](int t_first, int count) {
    for (int i = tid; i < count * 8; i += TC_THREADS) {
      const int r = i >> 3, cv = i & 7;
      const int t = t_first + r, c0 = c_base + cv * 8;
      const int pos = (t - base_t) % SB_RING;
      float x1[8], x2[8], v[8], f[8], gg[8];
      load_row8(a, b, t, c0, x1, x2, v);
      const bool in_seq = t >= 0 && t < a.L && c0 < a.D;
      if (in_seq) {
        const uint4 q = *reinterpret_cast<const uint4*>(dz + ((size_t)b * a.L + t) * a.D + c0);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 pq = unpack2(w[j]); gg[2 * j] = pq.x * x1[2 * j]; gg[2 * j + 1] = pq.y * x1[2 * j + 1]; }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) gg[j] = 0.f;
        if (a.ahead_mode && t >= a.L && t < a.L + a.K - 1 && c0 < a.D) {
          // look-ahead of g = dz * x1 past the end of the chunk: the next chunk's first rows, staged by their owner
          const bf16* fr = halo_row(a.ahead_f, b, t - a.L, a.K - 1, (size_t)3 * a.D);
          const bf16* gr = halo_row(a.ahead_g, b, t - a.L, a.K - 1, (size_t)a.D);
          if (fr && gr) {
            const uint4* fp = reinterpret_cast<const uint4*>(fr + 3 * c0);
            const uint4 q0 = fp[0], q1 = fp[1], q2 = fp[2];
            const uint32_t fw[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
            float all[24];
#pragma unroll
            for (int j = 0; j < 12; ++j) { float2 pq = unpack2(fw[j]); all[2 * j] = pq.x; all[2 * j + 1] = pq.y; }
            const uint4 q = *reinterpret_cast<const uint4*>(gr + c0);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { float2 pq = unpack2(w[j]); gg[2 * j] = pq.x * all[6 * j]; gg[2 * j + 1] = pq.y * all[6 * j + 3]; }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = x2[j] * v[j];
      st8(sU + pos * TC_LD + cv * 8, f);
      st8(sG + pos * TC_LD + cv * 8, gg);
      if (in_seq && t >= seg_t0 && t < seg_t1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) db_part[j] += gg[j] * f[j];
      }
    }
  };
  stage(base_t, SB_RING);

  const int slab = warp & 3, half = warp >> 2;
  const int ch0 = c_base + slab * 16;
  const int grp = min(ch0, a.D - 1) / a.dg;
  const float* hg = a.h + (size_t)grp * a.K;
  const int nd = min(ND, (a.K - 1) / 16 + 2);
  const int g = lane >> 2, tq = lane & 3;
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_col = (lane >> 4) * 8;
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
  // filter-gradient accumulators: this warp covers diagonals d = half, half + 2, ... for all four row blocks of the tile
  constexpr int NDH = (ND + 1) / 2;
  float P[NDH][2][4];
#pragma unroll
  for (int dd = 0; dd < NDH; ++dd)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int q = 0; q < 4; ++q) P[dd][nt][q] = 0.f;
  __syncthreads();

  for (int k = k0; k < k1; ++k) {
    const int t0 = (k - n_halo_tiles) * SB_TT;
    const int rel0 = (t0 - base_t) % SB_RING;                 // ring row of the tile's first row
    // ---- y (causal) and du (anticausal) for this warp's two row blocks -> staging tiles
    {
      uint32_t A[ND][4];
      toeplitz_frags(A, hg, a.K, lane, false);
      float acc[2][2][4];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        const int i0 = half * 32 + blk * 16;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[blk][nt][q] = 0.f;
#pragma unroll
        for (int d = 0; d < ND; ++d) {
          if (d < nd) {
            uint32_t bf[4];
            ldsm_x4_t(bf, smem_addr(sU + (ring_pos(rel0 + i0 - 16 * d) + lm_row) * TC_LD + slab * 16 + lm_col));
            mma16816(acc[blk][0], A[d], bf[0], bf[1]);
            mma16816(acc[blk][1], A[d], bf[2], bf[3]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int row = i0 + g + hh * 8, col = slab * 16 + nt * 8 + 2 * tq;
            const float2 u = unpack2(*reinterpret_cast<const uint32_t*>(sU + ring_pos(rel0 + row) * TC_LD + col));
            const int ca = c_base + col;
            const float b0 = ca < a.D ? a.bias[ca] : 0.f, b1 = ca + 1 < a.D ? a.bias[ca + 1] : 0.f;
            *reinterpret_cast<uint32_t*>(sY + row * TC_LD + col) = pack2(acc[blk][nt][hh * 2] + b0 * u.x, acc[blk][nt][hh * 2 + 1] + b1 * u.y);
          }
      }
      toeplitz_frags(A, hg, a.K, lane, true);
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        const int i0 = half * 32 + blk * 16;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[blk][nt][q] = 0.f;
#pragma unroll
        for (int d = 0; d < ND; ++d) {
          if (d < nd) {
            uint32_t bf[4];
            ldsm_x4_t(bf, smem_addr(sG + (ring_pos(rel0 + i0 + 16 * d) + lm_row) * TC_LD + slab * 16 + lm_col));
            mma16816(acc[blk][0], A[d], bf[0], bf[1]);
            mma16816(acc[blk][1], A[d], bf[2], bf[3]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int row = i0 + g + hh * 8, col = slab * 16 + nt * 8 + 2 * tq;
            const float2 gg = unpack2(*reinterpret_cast<const uint32_t*>(sG + ring_pos(rel0 + row) * TC_LD + col));
            const int ca = c_base + col;
            const float b0 = ca < a.D ? a.bias[ca] : 0.f, b1 = ca + 1 < a.D ? a.bias[ca + 1] : 0.f;
            *reinterpret_cast<uint32_t*>(sDU + row * TC_LD + col) = pack2(acc[blk][nt][hh * 2] + b0 * gg.x, acc[blk][nt][hh * 2 + 1] + b1 * gg.y);
          }
      }
    }
    // ---- filter gradient: P_d[i][j] += sum_c G[i0+i][c] U[i0-16d+j][c] over the four row blocks, d = half, half+2, ..
    if (t0 >= 0) {
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        const int i0 = blk * 16;
        uint32_t af[4];
        ldsm_x4(af, smem_addr(sG + (ring_pos(rel0 + i0) + a_row) * TC_LD + slab * 16 + a_col));
#pragma unroll
        for (int dd = 0; dd < NDH; ++dd) {
          const int d = 2 * dd + half;
          if (d < nd) {
            uint32_t bf[4];
            ldsm_x4(bf, smem_addr(sU + (ring_pos(rel0 + i0 - 16 * d) + b_row) * TC_LD + slab * 16 + b_col));
            mma16816(P[dd][0], af, bf[0], bf[1]);
            mma16816(P[dd][1], af, bf[2], bf[3]);
          }
        }
      }
    }
    __syncthreads();                                           // y / du tiles complete, ring reads of this tile done
    // ---- coalesced output pass: (row, 8 channels) per thread and step
    for (int i = tid; i < SB_TT * 8; i += TC_THREADS) {
      const int r = i >> 3, cv = i & 7;
      const int t = t0 + r, c0 = c_base + cv * 8;
      if (c0 >= a.D) continue;
      bf16* dst = nullptr;
      if (t >= 0 && t < a.L) dst = dfeat + ((size_t)b * a.L + t) * 3 * a.D + 3 * c0;
      else if (t < 0 && t >= -(a.K - 1) && dhalo) dst = dhalo + ((size_t)b * (a.K - 1) + (t + a.K - 1)) * 3 * a.D + 3 * c0;
      if (!dst) continue;
      float x1[8], x2[8], v[8], gz[8];
      load_row8(a, b, t, c0, x1, x2, v);
      if (t >= 0) {
        const uint4 q = *reinterpret_cast<const uint4*>(dz + ((size_t)b * a.L + t) * a.D + c0);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { float2 pq = unpack2(w[j]); gz[2 * j] = pq.x; gz[2 * j + 1] = pq.y; }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) gz[j] = 0.f;
      }
      const uint4 yq = *reinterpret_cast<const uint4*>(sY + r * TC_LD + cv * 8);
      const uint4 dq = *reinterpret_cast<const uint4*>(sDU + r * TC_LD + cv * 8);
      const uint32_t yw[4] = {yq.x, yq.y, yq.z, yq.w}, dw[4] = {dq.x, dq.y, dq.z, dq.w};
      float o[24];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 y = unpack2(yw[j]), du = unpack2(dw[j]);
        o[6 * j + 0] = gz[2 * j] * y.x;       o[6 * j + 1] = du.x * v[2 * j];       o[6 * j + 2] = du.x * x2[2 * j];
        o[6 * j + 3] = gz[2 * j + 1] * y.y;   o[6 * j + 4] = du.y * v[2 * j + 1];   o[6 * j + 5] = du.y * x2[2 * j + 1];
      }
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      d4[0] = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
      d4[1] = make_uint4(pack2(o[8], o[9]), pack2(o[10], o[11]), pack2(o[12], o[13]), pack2(o[14], o[15]));
      d4[2] = make_uint4(pack2(o[16], o[17]), pack2(o[18], o[19]), pack2(o[20], o[21]), pack2(o[22], o[23]));
    }
    // ---- advance the rings: the 64 rows that fall out behind are replaced by the 64 rows ahead of the next tile
    if (k + 1 < k1) stage(t0 + SB_TT + TC_HALO, SB_TT);
    __syncthreads();
  }

  // ---- flush: filter gradient (once per CTA), bias gradient
#pragma unroll
  for (int dd = 0; dd < NDH; ++dd) {
    const int d = 2 * dd + half;
    if (d < nd) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = g + ((q & 2) ? 8 : 0), j = nt * 8 + 2 * tq + (q & 1);
          const int s = 16 * d + i - j;
          if (s >= 0 && s < a.K) atomicAdd(&sdh[slab * 128 + s], P[dd][nt][q]);
        }
    }
  }
  {
    const int cv = tid & 7;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&sdb[cv * 8 + j], db_part[j]);
  }
  __syncthreads();
  for (int i = tid; i < 4 * 128; i += TC_THREADS) {
    const int sl = i >> 7, s = i & 127;
    const int c = c_base + sl * 16;
    if (s < a.K && c < a.D) atomicAdd(dh + (size_t)(c / a.dg) * a.K + s, sdh[i]);
  }
  for (int i = tid; i < TC_CH; i += TC_THREADS)
    if (c_base + i < a.D) atomicAdd(dbias + c_base + i, sdb[i]);
}

static int g_mr_bwd_stream = 1;

}  // namespace sb

using namespace sb;

// 1 (default): streaming backward kernel; 0: one independent CTA per 64-row tile
extern "C" int sb_mr_tc_set_bwd_variant(int streaming) { sb::g_mr_bwd_stream = streaming ? 1 : 0; return 0; }

extern "C" int sb_mr_tc_supported(int D, int G, int K) {
  const int dg = D / G;
  return (D % G == 0) && (dg % 16 == 0) && K >= 1 && K <= 128 && (D % 8 == 0);
}

extern "C" int sb_mr_tc_fwd(const void* feat, const void* halo, const float* h, const float* bias, void* z, int B, int L,
                            int D, int G, int K, cudaStream_t st) {
  if (!sb_mr_tc_supported(D, G, K)) return -1;
  if (B * L == 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(mr_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) return -5;
    attr = true;
  }
  MrArgs a{(const bf16*)feat, halo_local(halo), h, bias, L, D, K, D / G, 0, halo_local(nullptr), halo_local(nullptr)};
  dim3 grid((D + TC_CH - 1) / TC_CH, (L + FWD_TT - 1) / FWD_TT, B);
  mr_tc_fwd_kernel<<<grid, TC_THREADS, FWD_SMEM, st>>>(a, (bf16*)z);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Context-parallel forward: feat [2B, L, 3D] (two zigzag chunks per sequence), rows before each chunk read in place
// from the neighbours' staged tails (`before`, see halo_src.cuh).
extern "C" int sb_mr_tc_fwd_cp(const void* feat, const HaloSrc* before, const float* h, const float* bias, void* z, int B2,
                               int L, int D, int G, int K, cudaStream_t st) {
  if (!sb_mr_tc_supported(D, G, K) || !before) return -9;
  if (B2 * L == 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(mr_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) return -5;
    attr = true;
  }
  MrArgs a{(const bf16*)feat, *before, h, bias, L, D, K, D / G, 0, halo_local(nullptr), halo_local(nullptr)};
  dim3 grid((D + TC_CH - 1) / TC_CH, (L + FWD_TT - 1) / FWD_TT, B2);
  mr_tc_fwd_kernel<<<grid, TC_THREADS, FWD_SMEM, st>>>(a, (bf16*)z);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Context-parallel backward (streaming kernel): the look-ahead of dz * x1 past each chunk's end comes from the next
// chunk's staged head (`ahead_feat`, `ahead_dz`), so the gradients of the chunk's tail rows are complete and no halo
// gradient is produced.  L must be a multiple of 64 (whole tiles: a look-ahead row never shares a tile with chunk rows).
extern "C" int sb_mr_tc_bwd_cp(const void* feat, const HaloSrc* before, const float* h, const float* bias, const void* dz,
                               const HaloSrc* ahead_feat, const HaloSrc* ahead_dz, void* dfeat, float* dh, float* dbias, int B2,
                               int L, int D, int G, int K, cudaStream_t st) {
  if (!sb_mr_tc_supported(D, G, K) || !before || !ahead_feat || !ahead_dz || (L % SB_TT)) return -9;
  if (B2 * L == 0) return 0;
  static bool attr2 = false;
  if (!attr2) {
    if (cudaFuncSetAttribute(mr_tc_bwd_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SB_SMEM) != cudaSuccess) return -5;
    attr2 = true;
  }
  MrArgs a{(const bf16*)feat, *before, h, bias, L, D, K, D / G, 1, *ahead_feat, *ahead_dz};
  const int n_tiles = L / SB_TT;
  const int ctiles = (D + TC_CH - 1) / TC_CH;
  int segs = (2 * sb::num_sms()) / (ctiles * B2);
  if (segs > (n_tiles + 7) / 8) segs = (n_tiles + 7) / 8;
  if (segs < 1) segs = 1;
  const int tps = (n_tiles + segs - 1) / segs;
  dim3 sgrid(ctiles, (n_tiles + tps - 1) / tps, B2);
  mr_tc_bwd_stream_kernel<<<sgrid, TC_THREADS, SB_SMEM, st>>>(a, (const bf16*)dz, (bf16*)dfeat, nullptr, dh, dbias, 0, n_tiles, tps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_mr_tc_bwd(const void* feat, const void* halo, const float* h, const float* bias, const void* dz,
                            void* dfeat, void* dhalo, float* dh, float* dbias, int B, int L, int D, int G, int K,
                            cudaStream_t st) {
  if (!sb_mr_tc_supported(D, G, K)) return -1;
  if (B * L == 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(mr_tc_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return -5;
    attr = true;
  }
  MrArgs a{(const bf16*)feat, halo_local(halo), h, bias, L, D, K, D / G, 0, halo_local(nullptr), halo_local(nullptr)};
  const int n_halo = (halo && dhalo) ? (K - 1 + BWD_TT - 1) / BWD_TT : 0;
  if (g_mr_bwd_stream) {
    static bool attr2 = false;
    if (!attr2) {
      if (cudaFuncSetAttribute(mr_tc_bwd_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SB_SMEM) != cudaSuccess) return -5;
      attr2 = true;
    }
    const int n_tiles = (L + SB_TT - 1) / SB_TT + n_halo;
    const int ctiles = (D + TC_CH - 1) / TC_CH;
    // as many segments as fit in one wave of two CTAs per SM (a partial second wave would double the run time),
    // but no shorter than 8 tiles (the ring prologue costs 4 tiles)
    int segs = (2 * sb::num_sms()) / (ctiles * B);
    if (segs > (n_tiles + 7) / 8) segs = (n_tiles + 7) / 8;
    if (segs < 1) segs = 1;
    const int tps = (n_tiles + segs - 1) / segs;
    dim3 sgrid(ctiles, (n_tiles + tps - 1) / tps, B);
    mr_tc_bwd_stream_kernel<<<sgrid, TC_THREADS, SB_SMEM, st>>>(a, (const bf16*)dz, (bf16*)dfeat, (bf16*)dhalo, dh, dbias, n_halo,
                                                               n_tiles, tps);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  dim3 grid((D + TC_CH - 1) / TC_CH, (L + BWD_TT - 1) / BWD_TT + n_halo, B);
  mr_tc_bwd_kernel<<<grid, TC_THREADS, BWD_SMEM, st>>>(a, (const bf16*)dz, (bf16*)dfeat, (bf16*)dhalo, dh, dbias, n_halo);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
