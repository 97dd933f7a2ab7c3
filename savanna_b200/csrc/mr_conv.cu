// Hyena-MR: z = x1 * ( (h * u)_causal + bias * u ),  u = x2 * v,  filter h [G, K] with K <= 128 taps shared by
// the dg channels of a group.  Channel-last interleaved features, fp32 math on CUDA cores with the input
// tile (and the K-1 rows before it) staged in shared memory and an 8-output register block per thread,
// so each FMA costs 1/8 shared-memory load for the signal and 1/8 for the tap.
//
//   mr_fwd     : z (and y = conv + bias*u, saved for the backward pass)
//   mr_bwd_in  : dfeat = (dz*y, du*v, du*x2) with du[t] = sum_s h[s] dconv[t+s] + bias*dconv[t], dconv = dz*x1
//   mr_bwd_flt : dh[g,s] = sum_{t,c in g} dconv[t] u[t-s],  dbias[c] = sum_t dconv[t] u[t]
// `halo` holds the K-1 feature rows that precede the shard (context parallelism); mr_bwd_in also emits
// their gradient.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {
typedef __nv_bfloat16 bf16;

constexpr int MR_TT = 128;     // time rows per tile
constexpr int MR_TC = 64;      // channels per tile
constexpr int MR_KMAX = 128;
constexpr int MR_THREADS = 256;
constexpr int MR_ROWS = MR_TT + MR_KMAX - 1;                 // 255 staged rows
constexpr int MR_SMEM = MR_ROWS * MR_TC * 4 + MR_TT * MR_TC * 4 + MR_TC * MR_KMAX * 4;  // u | aux | taps

__device__ __forceinline__ float bf(const bf16 v) { return __bfloat162float(v); }

// Feature element (p = 0: x1, 1: x2, 2: v) at row t of batch b; rows in [-(K-1), 0) come from the halo.
struct FeatView {
  const bf16* feat; const bf16* halo; int L, D, K;
  __device__ __forceinline__ const bf16* row(int b, int t) const {
    if (t >= 0 && t < L) return feat + ((size_t)b * L + t) * 3 * D;
    if (t < 0 && t >= -(K - 1) && halo) return halo + ((size_t)b * (K - 1) + (t + K - 1)) * 3 * D;
    return nullptr;
  }
};

// ------------------------------------------------------------------------------------ forward
__global__ void __launch_bounds__(MR_THREADS)
mr_fwd_kernel(FeatView fv, const float* __restrict__ h, const float* __restrict__ bias, bf16* __restrict__ z,
              bf16* __restrict__ ysave, int dg, int G) {
  extern __shared__ float sm[];
  float* su = sm;                                   // [MR_ROWS][MR_TC]  u rows t0-(KMAX-1) .. t0+TT-1
  float* sx1 = sm + MR_ROWS * MR_TC;                // [MR_TT][MR_TC]
  float* sh = sx1 + MR_TT * MR_TC;                  // [MR_TC][K] taps per channel of the tile
  const int K = fv.K, D = fv.D, L = fv.L;
  const int c_base = blockIdx.x * MR_TC, t0 = blockIdx.y * MR_TT, b = blockIdx.z;
  const int tid = threadIdx.x;
  for (int i = tid; i < MR_TC * K; i += MR_THREADS) {
    const int c = i / K, s = i - c * K;
    const int ch = c_base + c;
    sh[c * MR_KMAX + s] = ch < D ? h[(size_t)(ch / dg) * K + s] : 0.f;
  }
  const int first_row = MR_KMAX - K;                // rows before this are never read
  for (int i = tid + first_row * MR_TC; i < MR_ROWS * MR_TC; i += MR_THREADS) {
    const int r = i / MR_TC, c = i - r * MR_TC;
    const int t = t0 - (MR_KMAX - 1) + r, ch = c_base + c;
    float u = 0.f, x1 = 0.f;
    const bf16* row = ch < D ? fv.row(b, t) : nullptr;
    if (row) { x1 = bf(row[3 * ch]); u = bf(row[3 * ch + 1]) * bf(row[3 * ch + 2]); }
    su[i] = u;
    if (r >= MR_KMAX - 1) sx1[(r - (MR_KMAX - 1)) * MR_TC + c] = x1;
  }
  __syncthreads();
  const int c = tid % MR_TC, tb = tid / MR_TC;      // 4 time sub-blocks of 32 outputs
  const int ch = c_base + c;
  const float* hc = sh + c * MR_KMAX;
  const float bi = ch < D ? bias[ch] : 0.f;
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    const int tl = tb * 32 + blk * 8;               // local output row of acc[0]
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // window: win[i] = u[tl + i - s] ; local row index of u[tl+i-s] in su is (KMAX-1) + tl + i - s
    float win[8];
    const float* ub = su + ((MR_KMAX - 1) + tl) * MR_TC + c;
#pragma unroll
    for (int i = 0; i < 8; ++i) win[i] = ub[i * MR_TC];
    for (int s0 = 0; s0 < K; s0 += 8) {
#pragma unroll
      for (int ss = 0; ss < 8; ++ss) {
        const int s = s0 + ss;
        if (s < K) {
          const float hv = hc[s];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += hv * win[i];
          // shift the window one step into the past
#pragma unroll
          for (int i = 7; i > 0; --i) win[i] = win[i - 1];
          win[0] = (s + 1 < K) ? ub[-(s + 1) * MR_TC] : 0.f;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t0 + tl + i;
      if (t < L && ch < D) {
        const float u = su[((MR_KMAX - 1) + tl + i) * MR_TC + c];
        const float y = acc[i] + bi * u;
        const size_t o = ((size_t)b * L + t) * D + ch;
        if (ysave) ysave[o] = __float2bfloat16_rn(y);
        z[o] = __float2bfloat16_rn(sx1[(tl + i) * MR_TC + c] * y);
      }
    }
  }
}

// ------------------------------------------------------------------------------------ backward wrt inputs
// Tile rows t0 .. t0+TT-1 of du need dconv rows t0 .. t0+TT+K-2 ("future" rows; zero beyond L).
// blockIdx.y == gridDim.y-1 extra tile (when halo grads are requested) covers rows [-(K-1), 0).
__global__ void __launch_bounds__(MR_THREADS)
mr_bwd_in_kernel(FeatView fv, const float* __restrict__ h, const float* __restrict__ bias, const bf16* __restrict__ dz,
                 const bf16* __restrict__ ysave, bf16* __restrict__ dfeat, bf16* __restrict__ dhalo, int dg, int n_main_tiles) {
  extern __shared__ float sm[];
  float* sg = sm;                                   // [MR_ROWS][MR_TC] dconv rows t0 .. t0+TT+KMAX-2
  float* sh = sm + MR_ROWS * MR_TC + MR_TT * MR_TC;
  const int K = fv.K, D = fv.D, L = fv.L;
  const bool halo_tile = (int)blockIdx.y >= n_main_tiles;
  const int c_base = blockIdx.x * MR_TC, b = blockIdx.z;
  const int t0 = halo_tile ? -MR_TT : blockIdx.y * MR_TT;
  const int tid = threadIdx.x;
  for (int i = tid; i < MR_TC * K; i += MR_THREADS) {
    const int c = i / K, s = i - c * K;
    const int ch = c_base + c;
    sh[c * MR_KMAX + s] = ch < D ? h[(size_t)(ch / dg) * K + s] : 0.f;
  }
  const int rows_needed = MR_TT + K - 1;
  for (int i = tid; i < rows_needed * MR_TC; i += MR_THREADS) {
    const int r = i / MR_TC, c = i - r * MR_TC;
    const int t = t0 + r, ch = c_base + c;
    float g = 0.f;
    if (t >= 0 && t < L && ch < D) {
      g = bf(dz[((size_t)b * L + t) * D + ch]) * bf(fv.feat[((size_t)b * L + t) * 3 * D + 3 * ch]);
    }
    sg[i] = g;
  }
  __syncthreads();
  const int c = tid % MR_TC, tb = tid / MR_TC;
  const int ch = c_base + c;
  const float* hc = sh + c * MR_KMAX;
  const float bi = ch < D ? bias[ch] : 0.f;
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    const int tl = tb * 32 + blk * 8;
    float acc[8], win[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // du[tl+i] = sum_s h[s] g[tl+i+s]; window win[i] = g[tl+i+s]
    const float* gbp = sg + tl * MR_TC + c;
#pragma unroll
    for (int i = 0; i < 8; ++i) win[i] = gbp[i * MR_TC];
    for (int s0 = 0; s0 < K; s0 += 8) {
#pragma unroll
      for (int ss = 0; ss < 8; ++ss) {
        const int s = s0 + ss;
        if (s < K) {
          const float hv = hc[s];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += hv * win[i];
#pragma unroll
          for (int i = 0; i < 7; ++i) win[i] = win[i + 1];
          win[7] = (tl + 8 + s) < rows_needed ? gbp[(8 + s) * MR_TC] : 0.f;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t0 + tl + i;
      if (ch >= D) continue;
      const bf16* row = fv.row(b, t);
      if (!row) continue;
      const float x2 = bf(row[3 * ch + 1]), v = bf(row[3 * ch + 2]);
      const float du = acc[i] + bi * sg[(tl + i) * MR_TC + c];
      if (t >= 0) {
        const size_t o = ((size_t)b * L + t) * D + ch;
        const float d1 = bf(dz[o]) * bf(ysave[o]);
        bf16* dst = dfeat + ((size_t)b * L + t) * 3 * D + 3 * ch;
        dst[0] = __float2bfloat16_rn(d1); dst[1] = __float2bfloat16_rn(du * v); dst[2] = __float2bfloat16_rn(du * x2);
      } else if (dhalo) {
        bf16* dst = dhalo + ((size_t)b * (K - 1) + (t + K - 1)) * 3 * D + 3 * ch;
        dst[0] = __float2bfloat16_rn(0.f); dst[1] = __float2bfloat16_rn(du * v); dst[2] = __float2bfloat16_rn(du * x2);
      }
    }
  }
}

// ------------------------------------------------------------------------------------ backward wrt filter
// dh[g, s] += sum over the tile's rows t and the tile's channels of group g:  dconv[t] * u[t-s]
__global__ void __launch_bounds__(MR_THREADS)
mr_bwd_flt_kernel(FeatView fv, const bf16* __restrict__ dz, float* __restrict__ dh, float* __restrict__ dbias, int dg) {
  extern __shared__ float sm[];
  float* su = sm;                                   // [MR_ROWS][MR_TC]
  float* sg = sm + MR_ROWS * MR_TC;                 // [MR_TT][MR_TC]
  float* sdh = sg + MR_TT * MR_TC;                  // [MR_TC / min(dg,TC) groups ...] flattened [MR_TC][KMAX] worst case
  const int K = fv.K, D = fv.D, L = fv.L;
  const int c_base = blockIdx.x * MR_TC, t0 = blockIdx.y * MR_TT, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int first_row = MR_KMAX - K;
  for (int i = tid + first_row * MR_TC; i < MR_ROWS * MR_TC; i += MR_THREADS) {
    const int r = i / MR_TC, c = i - r * MR_TC;
    const int t = t0 - (MR_KMAX - 1) + r, ch = c_base + c;
    float u = 0.f, g = 0.f;
    const bf16* row = ch < D ? fv.row(b, t) : nullptr;
    if (row) {
      u = bf(row[3 * ch + 1]) * bf(row[3 * ch + 2]);
      if (t >= 0) g = bf(dz[((size_t)b * L + t) * D + ch]) * bf(row[3 * ch]);
    }
    su[i] = u;
    if (r >= MR_KMAX - 1) sg[(r - (MR_KMAX - 1)) * MR_TC + c] = g;
  }
  // local groups of this tile: channel c belongs to local group c / dg_eff
  const int dg_eff = dg < MR_TC ? dg : MR_TC;
  const int n_local_groups = MR_TC / dg_eff;
  for (int i = tid; i < n_local_groups * MR_KMAX; i += MR_THREADS) sdh[i] = 0.f;
  __syncthreads();
  const int c = tid % MR_TC, q = tid / MR_TC;       // q in 0..3
  const int ch = c_base + c;
  const int n_tapblocks = (K + 7) / 8;
  for (int tbk = q; tbk < n_tapblocks; tbk += 4) {
    const int s0 = tbk * 8;
    float acc[8], win[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // acc[i] = sum_t g[t] * u[t - s0 - i];  window win[i] = u[t - s0 - i]
    const float* ub = su + ((MR_KMAX - 1) - s0) * MR_TC + c;     // row of u[t0 - s0]
#pragma unroll
    for (int i = 1; i < 8; ++i) win[i] = ub[-i * MR_TC];          // u[-s0-i]: the window at t = 0
#pragma unroll 4
    for (int t = 0; t < MR_TT; ++t) {
      win[0] = ub[t * MR_TC];
      const float g = sg[t * MR_TC + c];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += g * win[i];
#pragma unroll
      for (int i = 7; i > 0; --i) win[i] = win[i - 1];
    }
    if (ch < D) {
      const int lg = c / dg_eff;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (s0 + i < K) atomicAdd(&sdh[lg * MR_KMAX + s0 + i], acc[i]);
      if (s0 == 0) atomicAdd(dbias + ch, acc[0]);
    }
  }
  __syncthreads();
  for (int i = tid; i < n_local_groups * MR_KMAX; i += MR_THREADS) {
    const int lg = i / MR_KMAX, s = i - lg * MR_KMAX;
    const int ch0 = c_base + lg * dg_eff;
    if (s < K && ch0 < D) atomicAdd(dh + (size_t)(ch0 / dg) * K + s, sdh[i]);
  }
}

}  // namespace sb

using namespace sb;

static int mr_set_smem() {
  static bool done = false;
  if (!done) {
    if (cudaFuncSetAttribute(mr_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MR_SMEM) != cudaSuccess) return -5;
    if (cudaFuncSetAttribute(mr_bwd_in_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MR_SMEM) != cudaSuccess) return -5;
    if (cudaFuncSetAttribute(mr_bwd_flt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MR_SMEM) != cudaSuccess) return -5;
    done = true;
  }
  return 0;
}

extern "C" int sb_mr_fwd(const void* feat, const void* halo, const float* h, const float* bias, void* z, void* ysave,
                         int B, int L, int D, int G, int K, cudaStream_t st) {
  if (K < 1 || K > MR_KMAX || (D % G)) return -1;
  if (B * L == 0) return 0;
  if (int rc = mr_set_smem()) return rc;
  FeatView fv{(const bf16*)feat, (const bf16*)halo, L, D, K};
  dim3 grid((D + MR_TC - 1) / MR_TC, (L + MR_TT - 1) / MR_TT, B);
  mr_fwd_kernel<<<grid, MR_THREADS, MR_SMEM, st>>>(fv, h, bias, (bf16*)z, (bf16*)ysave, D / G, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_mr_bwd(const void* feat, const void* halo, const float* h, const float* bias, const void* dz,
                         const void* ysave, void* dfeat, void* dhalo, float* dh, float* dbias, int B, int L, int D, int G,
                         int K, cudaStream_t st) {
  if (K < 1 || K > MR_KMAX || (D % G)) return -1;
  if ((MR_TC % (D / G)) && ((D / G) % MR_TC)) return -8;   // tile/group alignment of the filter-gradient kernel
  if (B * L == 0) return 0;
  if (int rc = mr_set_smem()) return rc;
  FeatView fv{(const bf16*)feat, (const bf16*)halo, L, D, K};
  const int n_main = (L + MR_TT - 1) / MR_TT;
  dim3 grid((D + MR_TC - 1) / MR_TC, n_main + ((halo && dhalo) ? 1 : 0), B);
  mr_bwd_in_kernel<<<grid, MR_THREADS, MR_SMEM, st>>>(fv, h, bias, (const bf16*)dz, (const bf16*)ysave, (bf16*)dfeat,
                                                     (bf16*)dhalo, D / G, n_main);
  dim3 grid2((D + MR_TC - 1) / MR_TC, n_main, B);
  mr_bwd_flt_kernel<<<grid2, MR_THREADS, MR_SMEM, st>>>(fv, (const bf16*)dz, dh, dbias, D / G);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
