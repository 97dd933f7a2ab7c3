// Block-scaled fp8 (MXFP8) for sm_100a: e4m3 data with one E8M0 (power-of-two) scale per 32 consecutive elements of
// the contraction dimension, consumed by `tcgen05.mma.kind::mxf8f6f4.block_scale`, which applies the scales of both
// operands inside the tensor core.  Role of the block-scaled recipe of the reference's TransformerEngine layers
// (savanna/model/tengine.py builds the fp8 recipe; on Blackwell TE's MXFP8BlockScaling is that recipe).
//
//   quantisers   x [R, C] bf16  ->  q [R, C] e4m3 + scales along C            (row-wise)
//                x [R, C] bf16  ->  q [C, R] e4m3 + scales along R            (transposed: the contraction of a weight-
//                                                                              gradient product runs over the rows)
//   GEMM         C [M, N] bf16 (+)= A [M, K] * B [N, K]^T, both operands K-major with their scale tensors
//
// Scale layout in global memory (what the instruction reads after a 512-byte copy into tensor memory): the scale
// tensor of an operand with R rows and KB = ceil(K / 128) k-blocks is [ceil(R / 128)][KB][512 bytes]; inside a
// 512-byte atom the byte of (row r, 32-element block k4 of the k-block) sits at (r % 32) * 16 + (r / 32) * 4 + k4.
// `tcgen05.cp.32x128b.warpx4` copies an atom into four TMEM columns (replicated over the four lane quarters); the MMA
// of 32-element step k4 selects byte k4 of the column word through the scale ids of its instruction descriptor.
//
// Scale rule: e = ceil(log2(amax / 448)) clamped to [-127, 127], scale byte = e + 127, q = x * 2^-e (so |q| <= 448, the
// largest e4m3 value: no saturation); an all-zero block gets byte 0.
//
// Kernel structure: the single-CTA persistent kernel of gemm_sm100.cu (TMA producer warp, MMA warp, four epilogue
// warps; 128 x 256 tile, four stages) with the scale atoms riding in every stage (bulk copies on the same barrier) and
// one accumulator (256 TMEM columns) plus 12 scale columns; every wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "device_info.h"
#include "sm100.cuh"

namespace sb {

int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                    uint32_t box_outer);

namespace mx {

constexpr int BM = 128, BN = 256, BKE = 128, STAGES = 4;
constexpr int A_STAGE = BM * BKE;                  // 16 KB
constexpr int B_STAGE = BN * BKE;                  // 32 KB
constexpr int SF_ATOM = 512;                       // scales of 128 rows x 128 k
constexpr int SF_STAGE = 3 * SF_ATOM;              // A: one atom, B: two atoms
constexpr int STAGE_BYTES = A_STAGE + B_STAGE + 2048;   // scale atoms in the last 2 KB (keeps stages 1024-byte aligned)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;
constexpr int T_SFA = 256, T_SFB = 260;            // TMEM columns of the scale words (A: 4, B: 8)
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr uint32_t ST_MX = 0x60;

struct Params {
  __nv_bfloat16* C;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int M, N, K, ldc, ldr, beta;
  uint32_t* status;
};

__host__ __device__ inline long long sf_bytes(long long rows, long long k) {
  return ((rows + 127) / 128) * ((k + 127) / 128) * (long long)SF_ATOM;
}
__device__ __forceinline__ long long sf_offset(long long row, long long kblock32, long long kb128_count) {
  const long long mt = row >> 7, m = row & 127, kb = kblock32 >> 2, k4 = kblock32 & 3;
  return (mt * kb128_count + kb) * SF_ATOM + (m & 31) * 16 + (m >> 5) * 4 + k4;
}

// e = ceil(log2(amax / 448)) from the bits of amax / 448; returns the E8M0 byte and 2^-e
__device__ __forceinline__ uint32_t scale_of(float amax, float& inv) {
  if (!(amax > 0.f)) { inv = 0.f; return 0u; }
  const float s = amax * (1.f / 448.f);
  const uint32_t bits = __float_as_uint(s);
  int e = int((bits >> 23) & 0xffu) - 127;
  if (bits & 0x7fffffu) e += 1;
  if (((bits >> 23) & 0xffu) == 0u) e = -126;        // subnormal quotient: smallest normal exponent is plenty
  e = max(-127, min(127, e));
  inv = __uint_as_float(uint32_t(127 - e) << 23);    // 2^-e (e = 127 -> 2^-127 is subnormal: use the exact bit pattern below)
  if (e == 127) inv = __uint_as_float(0x00400000u);
  if (e == -127) inv = __uint_as_float(0x7f000000u); // 2^127
  return uint32_t(e + 127);
}
__device__ __forceinline__ uint32_t to_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

// One thread per (row, 32-column block).  cols % 32 == 0, ld % 8 == 0, 16-byte aligned rows.
__global__ void quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                     long long rows, int cols, long long ld) {
  const int nb = cols >> 5;
  const long long kb128 = (cols + 127) >> 7;
  const long long total = rows * nb;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nb;
    const int b = int(i - r * nb);
    const uint4* src = reinterpret_cast<const uint4*>(x + r * ld + b * 32);
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 u = __ldg(src + j);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = __bfloat1622float2(h[t]);
        v[j * 8 + 2 * t] = f.x; v[j * 8 + 2 * t + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    float inv;
    const uint32_t byte = scale_of(amax, inv);
    uint4 o0, o1;
    o0.x = to_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);     o0.y = to_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
    o0.z = to_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv);   o0.w = to_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv);
    o1.x = to_e4m3x4(v[16] * inv, v[17] * inv, v[18] * inv, v[19] * inv); o1.y = to_e4m3x4(v[20] * inv, v[21] * inv, v[22] * inv, v[23] * inv);
    o1.z = to_e4m3x4(v[24] * inv, v[25] * inv, v[26] * inv, v[27] * inv); o1.w = to_e4m3x4(v[28] * inv, v[29] * inv, v[30] * inv, v[31] * inv);
    uint4* dst = reinterpret_cast<uint4*>(q + r * (long long)cols + b * 32);
    dst[0] = o0; dst[1] = o1;
    sf[sf_offset(r, b, kb128)] = uint8_t(byte);
  }
}

// Transposed: q is [cols, rows_padded] with scales along the rows of x.  A block of 256 threads handles 32 rows x 256
// columns: the loads are coalesced along the columns, every thread owns one column and writes 32 bytes of its output row.
// rows % 32 == 0.
__global__ void quant_transposed_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                        long long rows, int cols, long long ld) {
  const long long rb = blockIdx.x;                       // block of 32 rows
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c >= cols) return;
  const long long kb128 = (rows + 127) >> 7;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v[j] = __bfloat162float(x[(rb * 32 + j) * ld + c]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  float inv;
  const uint32_t byte = scale_of(amax, inv);
  uint4 o0, o1;
  o0.x = to_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);     o0.y = to_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
  o0.z = to_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv);   o0.w = to_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv);
  o1.x = to_e4m3x4(v[16] * inv, v[17] * inv, v[18] * inv, v[19] * inv); o1.y = to_e4m3x4(v[20] * inv, v[21] * inv, v[22] * inv, v[23] * inv);
  o1.z = to_e4m3x4(v[24] * inv, v[25] * inv, v[26] * inv, v[27] * inv); o1.w = to_e4m3x4(v[28] * inv, v[29] * inv, v[30] * inv, v[31] * inv);
  uint4* dst = reinterpret_cast<uint4*>(q + (long long)c * rows + rb * 32);
  dst[0] = o0; dst[1] = o1;
  sf[sf_offset(c, rb, kb128)] = uint8_t(byte);
}

// shared-memory descriptor of one 512-byte scale atom: 32 rows of 16 bytes, no swizzle (8-row groups 128 bytes apart)
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(16u >> 4) << 16;
  d |= static_cast<uint64_t>(128u >> 4) << 32;
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                        uint32_t tsfa, uint32_t tsfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// block-scaled instruction descriptor: e4m3 x e4m3, E8M0 scales, K-major operands, scale ids = 32-element step in the k-block
__host__ __device__ constexpr uint32_t idesc_mx(int M, int N, int sf_id) {
  return (uint32_t(sf_id) << 4) | (0u << 7) | (0u << 10) | (uint32_t(N >> 3) << 17) | (1u << 23) | (uint32_t(M >> 4) << 24) |
         (uint32_t(sf_id) << 29);
}

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, m_tiles - first_m);
  const int r = tile - g * per_group;
  mt = first_m + r % gsz;
  nt = r / gsz;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES), tempty_bar = bar_base + 8u * (2 * STAGES + 1);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 2) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(tfull_bar, 1); mbar_init(tempty_bar, 4);
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
    // ------------------------------------------------------------------ producer: operand tiles by TMA, scale atoms by bulk copies
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      const int n_atoms = (p.N + 127) / 128;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt; tile_coords(tile, m_tiles, n_tiles, mt, nt);
        const int m0 = mt * BM, n0 = nt * BN;
        const bool second = 2 * nt + 1 < n_atoms;       // the tile's second 128 columns exist
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_MX + 1)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE;
          const uint32_t sf_dst = b_dst + B_STAGE;
          mbar_expect_tx(full_bar(stage), A_STAGE + B_STAGE + (second ? 3 : 2) * SF_ATOM);
          tma_load_2d(a_dst, &tmA, kb * BKE, m0, full_bar(stage));
          tma_load_2d(b_dst, &tmB, kb * BKE, n0, full_bar(stage));
          bulk_load(sf_dst, p.sfa + ((long long)mt * num_kb + kb) * SF_ATOM, SF_ATOM, full_bar(stage));
          bulk_load(sf_dst + SF_ATOM, p.sfb + ((long long)(2 * nt) * num_kb + kb) * SF_ATOM, SF_ATOM, full_bar(stage));
          if (second)
            bulk_load(sf_dst + 2 * SF_ATOM, p.sfb + ((long long)(2 * nt + 1) * num_kb + kb) * SF_ATOM, SF_ATOM, full_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar, acc_phase ^ 1u, abort_flag, p.status, ST_MX + 2)) { ok = false; break; }
        acc_phase ^= 1u;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_MX + 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t sf_addr = a_addr + A_STAGE + B_STAGE;
          // the scale words of this k-block: behind the previous block's products on the in-order tensor pipe
          tmem_cp_sf(tmem_base + T_SFA, sf_desc(sf_addr));
          tmem_cp_sf(tmem_base + T_SFB, sf_desc(sf_addr + SF_ATOM));
          tmem_cp_sf(tmem_base + T_SFB + 4, sf_desc(sf_addr + 2 * SF_ATOM));
          const uint64_t adesc = umma_smem_desc(a_addr, 16u, 1024u);
          const uint64_t bdesc = umma_smem_desc(a_addr + A_STAGE, 16u, 1024u);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            // the 32-element step selects byte k of the scale words: in the descriptor's scale ids and, as the
            // instruction's address convention has it, in the two top bits of the scale addresses
            umma_mx(tmem_base, adesc + k * 2u, bdesc + k * 2u, idesc_mx(BM, BN, k), (kb | k) != 0 ? 1u : 0u,
                    (tmem_base + T_SFA) | (uint32_t(k) << 30), (tmem_base + T_SFB) | (uint32_t(k) << 30));
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mt, nt; tile_coords(tile, m_tiles, n_tiles, mt, nt);
      if (!mbar_wait(tfull_bar, acc_phase, abort_flag, p.status, ST_MX + 4)) { ok = false; break; }
      acc_phase ^= 1u;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16);
      __nv_bfloat16* crow = p.C + size_t(row) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col + 8 <= p.N) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace mx
}  // namespace sb

// Bytes of the scale tensor of an operand with `rows` rows and contraction length `k`.
extern "C" long long sb_mx_sf_bytes(long long rows, long long k) { return sb::mx::sf_bytes(rows, k); }

// x [rows, cols] bf16 (row stride ld) -> q e4m3 + scales.  transposed = 0: q [rows, cols], scales along the columns
// (cols % 32 == 0); transposed = 1: q [cols, rows], scales along the rows of x (rows % 32 == 0).  `sf` must hold
// sb_mx_sf_bytes(operand rows, contraction length) bytes and be zero where no block writes (padding rows).
extern "C" int sb_mx_quantize(const void* x, void* q, void* sf, long long rows, int cols, long long ld, int transposed,
                              cudaStream_t stream) {
  using namespace sb::mx;
  if (rows <= 0 || cols <= 0) return 0;
  if ((ld % 8) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15)) return -4;
  if (!transposed) {
    if (cols % 32) return -3;
    const long long total = rows * (cols / 32);
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    const long long cap = (long long)sb::num_sms() * 16;
    if (blocks > cap) blocks = cap;
    quant_rowwise_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)sf, rows, cols, ld);
  } else {
    if (rows % 32) return -3;
    dim3 grid((unsigned)(rows / 32), (cols + 255) / 256);
    quant_transposed_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)sf, rows, cols, ld);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

// C [M, N] bf16 (+)= A [M, K] * B [N, K]^T with block scales.  A, B: e4m3 bytes, rows of K contiguous (lda, ldb in
// bytes, multiples of 16); SFA / SFB in the atom layout described at the top; K % 32 == 0, N % 8 == 0.
extern "C" int sb_gemm_mx(const void* A, const void* SFA, const void* B, const void* SFB, void* C, const void* bias,
                          const void* residual, int M, int N, int K, int lda, int ldb, int ldc, int ldr, int beta,
                          unsigned int* status, cudaStream_t stream) {
  using namespace sb;
  using namespace sb::mx;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  if ((N % 8) || (K % 32) || (lda % 16) || (ldb % 16) || (ldc % 8)) return -3;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB)) & 15) return -4;
  if (residual && ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_tmap_2d_u8(&tmA, A, K, M, lda, 128, BM))) return rc;
  if ((rc = make_tmap_2d_u8(&tmB, B, K, N, ldb, 128, BN))) return rc;
  Params p{reinterpret_cast<__nv_bfloat16*>(C), reinterpret_cast<const __nv_bfloat16*>(bias),
           reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<const uint8_t*>(SFA),
           reinterpret_cast<const uint8_t*>(SFB), M, N, K, ldc, ldr, beta, status};
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -5;
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sms = sb::num_sms();
  gemm_mx_kernel<<<tiles < sms ? tiles : sms, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}
