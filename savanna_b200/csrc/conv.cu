// Short causal depthwise convolutions, channel-last bf16, fp32 math:
//   dwconv_*   : y[b,t,c] = sum_j w[c,j] x[b, t-(K-1)+j, c]           (featuriser, K = short_conv_L)
//   se_*       : z = x1 * conv_K(x2 * v) on interleaved (x1,x2,v) features (Hyena-SE and hyena_mlp)
// A thread owns CH consecutive channels and walks TL consecutive time steps with the filter window in
// registers, so every input element is read once (plus a K-1 overlap per run).  Optional `halo` tensors
// hold the K-1 rows preceding the sequence (context-parallel shards); their gradients are produced too.
// Filter-gradient partial sums stay in registers over the run and are flushed with fp32 atomics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_info.h"
#include "halo_src.cuh"

namespace sb {
typedef __nv_bfloat16 bf16;

template <int CH> struct Vec;
template <> struct Vec<8> { typedef uint4 type; };
template <> struct Vec<4> { typedef uint2 type; };

template <int CH>
__device__ __forceinline__ void load_ch(const bf16* p, float (&f)[CH]) {
  typename Vec<CH>::type v = *reinterpret_cast<const typename Vec<CH>::type*>(p);
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < CH / 2; ++i) { float2 t = __bfloat1622float2(q[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <int CH>
__device__ __forceinline__ void store_ch(bf16* p, const float (&f)[CH]) {
  typename Vec<CH>::type v;
  __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < CH / 2; ++i) q[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<typename Vec<CH>::type*>(p) = v;
}
// interleaved triple load: 3*CH consecutive bf16 -> x1[CH], x2[CH], v[CH]
template <int CH>
__device__ __forceinline__ void load_triple(const bf16* p, float (&x1)[CH], float (&x2)[CH], float (&v)[CH]) {
  float a[CH], b[CH], c[CH];
  load_ch<CH>(p, a); load_ch<CH>(p + CH, b); load_ch<CH>(p + 2 * CH, c);
  float all[3 * CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) { all[i] = a[i]; all[CH + i] = b[i]; all[2 * CH + i] = c[i]; }
#pragma unroll
  for (int i = 0; i < CH; ++i) { x1[i] = all[3 * i]; x2[i] = all[3 * i + 1]; v[i] = all[3 * i + 2]; }
}
template <int CH>
__device__ __forceinline__ void store_triple(bf16* p, const float (&x1)[CH], const float (&x2)[CH], const float (&v)[CH]) {
  float all[3 * CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) { all[3 * i] = x1[i]; all[3 * i + 1] = x2[i]; all[3 * i + 2] = v[i]; }
  float a[CH], b[CH], c[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) { a[i] = all[i]; b[i] = all[CH + i]; c[i] = all[2 * CH + i]; }
  store_ch<CH>(p, a); store_ch<CH>(p + CH, b); store_ch<CH>(p + 2 * CH, c);
}

// 16-byte asynchronous copy global -> shared; nbytes = 0 writes zeros without touching `src` (which must still be a
// valid address).  Used to put a whole tile's loads in flight without holding them in registers.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, int nbytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(nbytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ------------------------------------------------------------------------------------ depthwise conv
template <int K, int CH>
__global__ void dwconv_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ halo, const float* __restrict__ w,
                                  bf16* __restrict__ y, int L, int C, int TL) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * CH >= C) return;
  const int c0 = cv * CH, b = blockIdx.z, t0 = blockIdx.y * TL;
  float wr[CH][K];
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(size_t)(c0 + i) * K + j];
  const bf16* xb = x + (size_t)b * L * C + c0;
  const bf16* hb = halo ? halo + (size_t)b * (K - 1) * C + c0 : nullptr;
  float win[K][CH];                                     // win[j] = x[t-(K-1)+j]
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int t = t0 - (K - 1) + j;
    if (t >= 0) load_ch<CH>(xb + (size_t)t * C, win[j + 1]);
    else if (hb) load_ch<CH>(hb + (size_t)(t + K - 1) * C, win[j + 1]);
    else {
#pragma unroll
      for (int i = 0; i < CH; ++i) win[j + 1][i] = 0.f;
    }
  }
  const int t1 = min(t0 + TL, L);
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < CH; ++i) win[j][i] = win[j + 1][i];
    load_ch<CH>(xb + (size_t)t * C, win[K - 1]);
    float o[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) acc += wr[i][j] * win[j][i];
      o[i] = acc;
    }
    store_ch<CH>(y + ((size_t)b * L + t) * C + c0, o);
  }
}

// dx_ext[t] = sum_j w[j] dy[t+(K-1)-j] for t in [-(K-1), L)   (rows < 0 go to dhalo)
// dw[c,j]  += sum_t dy[t] x_ext[t-(K-1)+j]
template <int K, int CH>
__global__ void dwconv_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ halo, const float* __restrict__ w,
                                  const bf16* __restrict__ dy, bf16* __restrict__ dx, bf16* __restrict__ dhalo,
                                  float* __restrict__ dw, int L, int C, int TL) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * CH >= C) return;
  const int c0 = cv * CH, b = blockIdx.z;
  // block y == 0 additionally covers the halo rows
  const int t_begin = blockIdx.y * TL - (blockIdx.y == 0 ? (K - 1) : 0);
  const int t_end = min((int)(blockIdx.y + 1) * TL, L);
  float wr[CH][K], dwacc[CH][K];
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) { wr[i][j] = w[(size_t)(c0 + i) * K + j]; dwacc[i][j] = 0.f; }
  const bf16* xb = x + (size_t)b * L * C + c0;
  const bf16* gb = dy + (size_t)b * L * C + c0;
  const bf16* hb = halo ? halo + (size_t)b * (K - 1) * C + c0 : nullptr;
  auto load_x_ext = [&](int t, float (&f)[CH]) {
    if (t >= 0 && t < L) load_ch<CH>(xb + (size_t)t * C, f);
    else if (t < 0 && t >= -(K - 1) && hb) load_ch<CH>(hb + (size_t)(t + K - 1) * C, f);
    else {
#pragma unroll
      for (int i = 0; i < CH; ++i) f[i] = 0.f;
    }
  };
  auto load_dy = [&](int t, float (&f)[CH]) {
    if (t >= 0 && t < L) load_ch<CH>(gb + (size_t)t * C, f);
    else {
#pragma unroll
      for (int i = 0; i < CH; ++i) f[i] = 0.f;
    }
  };
  float xw[K][CH];     // xw[j] = x_ext[t-(K-1)+j]
  float gw[K][CH];     // gw[i] = dy[t+i]
#pragma unroll
  for (int j = 0; j < K - 1; ++j) { load_x_ext(t_begin - (K - 1) + j, xw[j + 1]); load_dy(t_begin + j, gw[j + 1]); }
  for (int t = t_begin; t < t_end; ++t) {
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < CH; ++i) { xw[j][i] = xw[j + 1][i]; gw[j][i] = gw[j + 1][i]; }
    load_x_ext(t, xw[K - 1]);
    load_dy(t + K - 1, gw[K - 1]);
    float o[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) { acc += wr[i][j] * gw[K - 1 - j][i]; dwacc[i][j] += gw[0][i] * xw[j][i]; }
      o[i] = acc;
    }
    if (t >= 0) store_ch<CH>(dx + ((size_t)b * L + t) * C + c0, o);
    else if (dhalo) store_ch<CH>(dhalo + ((size_t)b * (K - 1) + (t + K - 1)) * C + c0, o);
  }
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) atomicAdd(dw + (size_t)(c0 + i) * K + j, dwacc[i][j]);
}

constexpr int DW_CT_F = 64, DW_SEG_F = 32, DW_NSEG_F = 4;

// Forward through shared memory: the x tile (DW_T steps + K-1 rows of history, DW_CT channels) is staged with
// asynchronous 16-byte copies, a thread then produces DW_SEG steps of two adjacent channels from shared memory.
template <int K>
__global__ void __launch_bounds__(DW_CT_F / 2 * DW_NSEG_F)
dwconv_fwd_tiled_kernel(const bf16* __restrict__ x, const HaloSrc halo, const float* __restrict__ w,
                        bf16* __restrict__ y, int L, int C) {
  constexpr int H = K - 1, T = DW_SEG_F * DW_NSEG_F, ROWS = T + H, NT = DW_CT_F / 2 * DW_NSEG_F, CHK = DW_CT_F / 8;
  __shared__ __align__(16) bf16 xS[ROWS][DW_CT_F];          // x_ext of times t0-H .. t0+T-1
  const int tid = threadIdx.x, c0 = blockIdx.x * DW_CT_F, b = blockIdx.z, t0 = blockIdx.y * T;
  for (int idx = tid; idx < ROWS * CHK; idx += NT) {
    const int row = idx / CHK, ch = idx % CHK, t = t0 - H + row;
    const bf16* src = x;
    int nb = 0;
    if (t >= 0 && t < L) { src = x + ((size_t)b * L + t) * C + c0 + ch * 8; nb = 16; }
    else if (t < 0 && t >= -H) {
      const bf16* hr = halo_row(halo, b, t + H, H, C);       // local halo tensor or a neighbour's staged tail (peer load)
      if (hr) { src = hr + c0 + ch * 8; nb = 16; }
    }
    cp_async16(&xS[row][ch * 8], src, nb);
  }
  const int cp = tid % (DW_CT_F / 2), seg = tid / (DW_CT_F / 2), r0 = seg * DW_SEG_F;
  float wr[2][K], win[K][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(size_t)(c0 + 2 * cp + i) * K + j];
  cp_async_wait_all();
  __syncthreads();
  auto ld2 = [&](int row, float (&f)[2]) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xS[row][2 * cp]));
    f[0] = v.x; f[1] = v.y;
  };
#pragma unroll
  for (int j = 0; j < H; ++j) ld2(r0 + j, win[j + 1]);
#pragma unroll 8
  for (int i = 0; i < DW_SEG_F; ++i) {
    const int r = r0 + i, t = t0 + r;
#pragma unroll
    for (int j = 0; j < H; ++j) { win[j][0] = win[j + 1][0]; win[j][1] = win[j + 1][1]; }
    ld2(r + H, win[K - 1]);
    float o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) { o0 += wr[0][j] * win[j][0]; o1 += wr[1][j] * win[j][1]; }
    if (t < L) *reinterpret_cast<__nv_bfloat162*>(y + ((size_t)b * L + t) * C + c0 + 2 * cp) = __floats2bfloat162_rn(o0, o1);
  }
}

// Backward through shared memory (same idea as se_bwd_tiled_kernel below): a CTA stages DW_T time steps x DW_CT channels
// of x (with the K-1 rows before) and of dy (with the K-1 rows after) with 16-byte loads that are all in flight at once;
// a thread then walks DW_SEG steps of two adjacent channels with both windows in registers.
constexpr int DW_CT = 64, DW_SEG = 32, DW_NSEG = 4, DW_T = DW_SEG * DW_NSEG;

template <int K>
__global__ void __launch_bounds__(DW_CT / 2 * DW_NSEG)
dwconv_bwd_tiled_kernel(const bf16* __restrict__ x, const HaloSrc halo, const float* __restrict__ w,
                        const bf16* __restrict__ dy, bf16* __restrict__ dx, bf16* __restrict__ dhalo,
                        float* __restrict__ dw, int L, int C, const int ahead_mode, const HaloSrc ahead) {
  constexpr int H = K - 1, ROWS = DW_T + H, NT = DW_CT / 2 * DW_NSEG, CHK = DW_CT / 8;
  __shared__ __align__(16) bf16 xS[ROWS][DW_CT];            // x_ext of times t0-H .. t0+DW_T-1
  __shared__ __align__(16) bf16 gS[ROWS][DW_CT];            // dy of times t0 .. t0+DW_T+H-1
  __shared__ float dwS[DW_CT][K];
  const int tid = threadIdx.x, c0 = blockIdx.x * DW_CT, b = blockIdx.z;
  // Two ways to account for the rows a neighbouring chunk convolved with this chunk's tail.  Default: the first tile
  // starts H rows early and writes the gradient of the halo rows to `dhalo` (the caller routes it to their owner).
  // `ahead_mode`: the H rows of dy that FOLLOW the chunk are read from `ahead` (the next chunk's staged head, peer
  // memory), so dx of the tail rows is complete here and nothing is produced for the halo rows.
  const int t0 = blockIdx.y * DW_T - (ahead_mode ? 0 : H);
  for (int idx = tid; idx < ROWS * CHK; idx += NT) {
    const int row = idx / CHK, ch = idx % CHK;
    int t = t0 - H + row;
    const bf16* src = x;
    int nb = 0;
    if (t >= 0 && t < L) { src = x + ((size_t)b * L + t) * C + c0 + ch * 8; nb = 16; }
    else if (t < 0 && t >= -H) {
      const bf16* hr = halo_row(halo, b, t + H, H, C);
      if (hr) { src = hr + c0 + ch * 8; nb = 16; }
    }
    cp_async16(&xS[row][ch * 8], src, nb);
    t = t0 + row;
    src = dy; nb = 0;
    if (t >= 0 && t < L) { src = dy + ((size_t)b * L + t) * C + c0 + ch * 8; nb = 16; }
    else if (ahead_mode && t >= L && t < L + H) {
      const bf16* ar = halo_row(ahead, b, t - L, H, C);
      if (ar) { src = ar + c0 + ch * 8; nb = 16; }
    }
    cp_async16(&gS[row][ch * 8], src, nb);
  }
  for (int idx = tid; idx < DW_CT * K; idx += NT) (&dwS[0][0])[idx] = 0.f;
  cp_async_wait_all();
  __syncthreads();

  const int cp = tid % (DW_CT / 2), seg = tid / (DW_CT / 2), r0 = seg * DW_SEG;
  float wr[2][K], dwacc[2][K], xw[K][2], gw[K][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) { wr[i][j] = w[(size_t)(c0 + 2 * cp + i) * K + j]; dwacc[i][j] = 0.f; }
  auto ld2 = [&](const bf16 (*tile)[DW_CT], int row, float (&f)[2]) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&tile[row][2 * cp]));
    f[0] = v.x; f[1] = v.y;
  };
#pragma unroll
  for (int j = 0; j < H; ++j) { ld2(xS, r0 + j, xw[j + 1]); ld2(gS, r0 + j, gw[j + 1]); }
#pragma unroll 4
  for (int i = 0; i < DW_SEG; ++i) {
    const int r = r0 + i, t = t0 + r;
#pragma unroll
    for (int j = 0; j < H; ++j) { xw[j][0] = xw[j + 1][0]; xw[j][1] = xw[j + 1][1]; gw[j][0] = gw[j + 1][0]; gw[j][1] = gw[j + 1][1]; }
    ld2(xS, r + H, xw[K - 1]);
    ld2(gS, r + H, gw[K - 1]);
    float o[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      float acc = 0.f;
#pragma unroll
      const float g0 = t < L ? gw[0][q] : 0.f;              // look-ahead rows belong to the next chunk's filter gradient
#pragma unroll
      for (int j = 0; j < K; ++j) { acc += wr[q][j] * gw[K - 1 - j][q]; dwacc[q][j] += g0 * xw[j][q]; }
      o[q] = acc;
    }
    bf16* dst = nullptr;
    if (t >= 0 && t < L) dst = dx + ((size_t)b * L + t) * C + c0 + 2 * cp;
    else if (t < 0 && t >= -H && dhalo) dst = dhalo + ((size_t)b * H + (t + H)) * C + c0 + 2 * cp;
    if (dst) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o[0], o[1]);
  }
#pragma unroll
  for (int q = 0; q < 2; ++q)
#pragma unroll
    for (int j = 0; j < K; ++j) atomicAdd(&dwS[2 * cp + q][j], dwacc[q][j]);
  __syncthreads();
  for (int idx = tid; idx < DW_CT * K; idx += NT) atomicAdd(dw + (size_t)(c0 + idx / K) * K + idx % K, (&dwS[0][0])[idx]);
}

// ------------------------------------------------------------------------------------ Hyena-SE
// feat [B, L, 3D] interleaved; w [G, K] fp32 (conv1d tap order); z [B, L, D].
template <int K, int CH>
__global__ void se_fwd_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ halo, const float* __restrict__ w,
                              bf16* __restrict__ z, int L, int D, int dg, int TL, int pregate, int postgate) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * CH >= D) return;
  const int c0 = cv * CH, b = blockIdx.z, t0 = blockIdx.y * TL;
  float wr[CH][K];
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(size_t)((c0 + i) / dg) * K + j];
  const bf16* fb = feat + (size_t)b * L * 3 * D + 3 * c0;
  const bf16* hb = halo ? halo + (size_t)b * (K - 1) * 3 * D + 3 * c0 : nullptr;
  float win[K][CH];
  float x1[CH], x2[CH], v[CH];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int t = t0 - (K - 1) + j;
    const bf16* src = t >= 0 ? fb + (size_t)t * 3 * D : (hb ? hb + (size_t)(t + K - 1) * 3 * D : nullptr);
    if (src) {
      load_triple<CH>(src, x1, x2, v);
#pragma unroll
      for (int i = 0; i < CH; ++i) win[j + 1][i] = pregate ? x2[i] * v[i] : v[i];
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) win[j + 1][i] = 0.f;
    }
  }
  const int t1 = min(t0 + TL, L);
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < CH; ++i) win[j][i] = win[j + 1][i];
    load_triple<CH>(fb + (size_t)t * 3 * D, x1, x2, v);
    float o[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      win[K - 1][i] = pregate ? x2[i] * v[i] : v[i];
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) acc += wr[i][j] * win[j][i];
      o[i] = postgate ? x1[i] * acc : acc;
    }
    store_ch<CH>(z + ((size_t)b * L + t) * D + c0, o);
  }
}

// Backward.  For every t of the run (plus the halo rows for the first run):
//   conv[t]  = sum_j w[j] u_ext[t-(K-1)+j]           u = x2*v
//   dconv[t] = dz[t] * x1[t]        dx1[t] = dz[t] * conv[t]
//   du[t]    = sum_j w[j] dconv[t+(K-1)-j]           dx2 = du*v, dv = du*x2
//   dw[g,j] += sum_t dconv[t] u_ext[t-(K-1)+j]
template <int K, int CH>
__global__ void se_bwd_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ halo, const float* __restrict__ w,
                              const bf16* __restrict__ dz, bf16* __restrict__ dfeat, bf16* __restrict__ dhalo,
                              float* __restrict__ dw, int L, int D, int dg, int TL, int pregate, int postgate) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * CH >= D) return;
  const int c0 = cv * CH, b = blockIdx.z;
  const int t_begin = blockIdx.y * TL - (blockIdx.y == 0 && halo ? (K - 1) : 0);
  const int t_end = min((int)(blockIdx.y + 1) * TL, L);
  float wr[CH][K], dwacc[CH][K];
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) { wr[i][j] = w[(size_t)((c0 + i) / dg) * K + j]; dwacc[i][j] = 0.f; }
  const bf16* fb = feat + (size_t)b * L * 3 * D + 3 * c0;
  const bf16* hb = halo ? halo + (size_t)b * (K - 1) * 3 * D + 3 * c0 : nullptr;
  const bf16* gb = dz + (size_t)b * L * D + c0;
  auto feat_ptr = [&](int t) -> const bf16* {
    if (t >= 0 && t < L) return fb + (size_t)t * 3 * D;
    if (t < 0 && t >= -(K - 1) && hb) return hb + (size_t)(t + K - 1) * 3 * D;
    return nullptr;
  };
  // dconv at time t (zero outside [0, L): the halo rows produce no output of this shard)
  auto load_dconv = [&](int t, float (&f)[CH]) {
    if (t >= 0 && t < L) {
      float g[CH]; load_ch<CH>(gb + (size_t)t * D, g);
      if (postgate) {
        float a[CH], bb[CH], c[CH]; load_triple<CH>(fb + (size_t)t * 3 * D, a, bb, c);
#pragma unroll
        for (int i = 0; i < CH; ++i) f[i] = g[i] * a[i];
      } else {
#pragma unroll
        for (int i = 0; i < CH; ++i) f[i] = g[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) f[i] = 0.f;
    }
  };
  float uw[K][CH];     // uw[j] = u_ext[t-(K-1)+j]
  float gw[K][CH];     // gw[i] = dconv[t+i]
  float x1[CH], x2[CH], v[CH];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const bf16* src = feat_ptr(t_begin - (K - 1) + j);
    if (src) {
      load_triple<CH>(src, x1, x2, v);
#pragma unroll
      for (int i = 0; i < CH; ++i) uw[j + 1][i] = pregate ? x2[i] * v[i] : v[i];
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) uw[j + 1][i] = 0.f;
    }
    load_dconv(t_begin + j, gw[j + 1]);
  }
  for (int t = t_begin; t < t_end; ++t) {
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < CH; ++i) { uw[j][i] = uw[j + 1][i]; gw[j][i] = gw[j + 1][i]; }
    const bf16* src = feat_ptr(t);
    if (src) load_triple<CH>(src, x1, x2, v);
    else {
#pragma unroll
      for (int i = 0; i < CH; ++i) { x1[i] = 0.f; x2[i] = 0.f; v[i] = 0.f; }
    }
    load_dconv(t + K - 1, gw[K - 1]);
    float g[CH];
    if (t >= 0) load_ch<CH>(gb + (size_t)t * D, g);
    else {
#pragma unroll
      for (int i = 0; i < CH; ++i) g[i] = 0.f;
    }
    float d1[CH], d2[CH], d3[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      uw[K - 1][i] = pregate ? x2[i] * v[i] : v[i];
      float conv = 0.f, du = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        conv += wr[i][j] * uw[j][i];
        du += wr[i][j] * gw[K - 1 - j][i];
        dwacc[i][j] += gw[0][i] * uw[j][i];
      }
      d1[i] = postgate ? g[i] * conv : 0.f;
      if (pregate) { d2[i] = du * v[i]; d3[i] = du * x2[i]; }
      else { d2[i] = 0.f; d3[i] = du; }
    }
    if (t >= 0) store_triple<CH>(dfeat + ((size_t)b * L + t) * 3 * D + 3 * c0, d1, d2, d3);
    else if (dhalo) store_triple<CH>(dhalo + ((size_t)b * (K - 1) + (t + K - 1)) * 3 * D + 3 * c0, d1, d2, d3);
  }
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) atomicAdd(dw + (size_t)((c0 + i) / dg) * K + j, dwacc[i][j]);
}

constexpr int SE_CT = 32, SE_SEG = 32, SE_NSEG = 4, SE_T = SE_SEG * SE_NSEG;

// Forward through shared memory: features of SE_T steps (plus K-1 rows of history) x SE_CT channels staged with
// asynchronous copies, one channel x SE_SEG steps per thread, outputs collected in shared memory and stored as
// 16-byte chunks.
template <int K>
__global__ void __launch_bounds__(SE_CT * SE_NSEG)
se_fwd_tiled_kernel(const bf16* __restrict__ feat, const HaloSrc halo, const float* __restrict__ w,
                    bf16* __restrict__ z, int L, int D, int dg, int pregate, int postgate) {
  constexpr int H = K - 1, ROWS = SE_T + H, NT = SE_CT * SE_NSEG, FCH = 3 * SE_CT / 8, ZCH = SE_CT / 8;
  __shared__ __align__(16) bf16 fS[ROWS][3 * SE_CT];        // features of times t0-H .. t0+SE_T-1
  __shared__ __align__(16) bf16 zS[SE_T][SE_CT];
  const int tid = threadIdx.x, c0 = blockIdx.x * SE_CT, b = blockIdx.z, t0 = blockIdx.y * SE_T;
  for (int idx = tid; idx < ROWS * FCH; idx += NT) {
    const int row = idx / FCH, ch = idx % FCH, t = t0 - H + row;
    const bf16* src = feat;
    int nb = 0;
    if (t >= 0 && t < L) { src = feat + ((size_t)b * L + t) * 3 * D + 3 * c0 + ch * 8; nb = 16; }
    else if (t < 0 && t >= -H) {
      const bf16* hr = halo_row(halo, b, t + H, H, (size_t)3 * D);   // local halo tensor or a neighbour's staged tail
      if (hr) { src = hr + 3 * c0 + ch * 8; nb = 16; }
    }
    cp_async16(&fS[row][ch * 8], src, nb);
  }
  const int c = tid % SE_CT, seg = tid / SE_CT, r0 = seg * SE_SEG;
  float wr[K], win[K];
#pragma unroll
  for (int j = 0; j < K; ++j) wr[j] = w[(size_t)((c0 + c) / dg) * K + j];
  cp_async_wait_all();
  __syncthreads();
  auto u_row = [&](int row) -> float {
    const float x2 = __bfloat162float(fS[row][3 * c + 1]), v = __bfloat162float(fS[row][3 * c + 2]);
    return pregate ? x2 * v : v;
  };
#pragma unroll
  for (int j = 0; j < H; ++j) win[j + 1] = u_row(r0 + j);
#pragma unroll 8
  for (int i = 0; i < SE_SEG; ++i) {
    const int r = r0 + i;
#pragma unroll
    for (int j = 0; j < H; ++j) win[j] = win[j + 1];
    win[K - 1] = u_row(r + H);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) acc += wr[j] * win[j];
    zS[r][c] = __float2bfloat16(postgate ? __bfloat162float(fS[r + H][3 * c]) * acc : acc);
  }
  __syncthreads();
  for (int idx = tid; idx < SE_T * ZCH; idx += NT) {
    const int r = idx / ZCH, ch = idx % ZCH, t = t0 + r;
    if (t < L) *reinterpret_cast<uint4*>(z + ((size_t)b * L + t) * D + c0 + ch * 8) = *reinterpret_cast<const uint4*>(&zS[r][ch * 8]);
  }
}

// Backward through shared memory.  A CTA stages a tile of SE_T time steps x SE_CT channels (plus K-1 rows before, for the
// history of u, and K-1 rows after, for the look-ahead of dconv) with 16-byte loads that are all in flight at once, then
// every thread walks SE_SEG consecutive steps of ONE channel with the two filter windows in registers, reading the tile
// from shared memory.  The run-per-thread kernel above issues its global loads inside the serial time loop and is bound
// by their latency; here the loop only touches shared memory.  Filter gradients are reduced over the lanes of a group
// by shuffles, over the CTA in shared memory, and leave with one atomic per (group, tap) and CTA.

template <int K>
__global__ void __launch_bounds__(SE_CT * SE_NSEG)
se_bwd_tiled_kernel(const bf16* __restrict__ feat, const HaloSrc halo, const int has_halo, const float* __restrict__ w,
                    const bf16* __restrict__ dz, bf16* __restrict__ dfeat, bf16* __restrict__ dhalo,
                    float* __restrict__ dw, int L, int D, int dg, int pregate, int postgate,
                    const int ahead_mode, const HaloSrc ahead_f, const HaloSrc ahead_g) {
  constexpr int H = K - 1, ROWS_F = SE_T + 2 * H, ROWS_G = SE_T + H;
  __shared__ __align__(16) bf16 fS[ROWS_F][3 * SE_CT];      // features of times t0-H .. t0+SE_T+H-1
  __shared__ __align__(16) bf16 gS[ROWS_G][SE_CT];          // dz of times t0 .. t0+SE_T+H-1
  __shared__ float dwS[SE_CT][K];
  const int tid = threadIdx.x, c0 = blockIdx.x * SE_CT, b = blockIdx.z;
  // `ahead_mode`: the H rows after the chunk (features, for x1, and dz) come from the next chunk's staged head in peer
  // memory, so the gradients of this chunk's tail rows are complete here; otherwise the first tile starts H rows early
  // and the gradient of the halo rows goes to `dhalo`.
  const int t0 = blockIdx.y * SE_T - ((has_halo && !ahead_mode) ? H : 0);
  constexpr int FCH = 3 * SE_CT / 8, GCH = SE_CT / 8;       // 16-byte chunks per staged row
  for (int idx = tid; idx < ROWS_F * FCH; idx += SE_CT * SE_NSEG) {
    const int row = idx / FCH, ch = idx % FCH, t = t0 - H + row;
    const bf16* src = feat;
    int nb = 0;
    if (t >= 0 && t < L) { src = feat + ((size_t)b * L + t) * 3 * D + 3 * c0 + ch * 8; nb = 16; }
    else if (t < 0 && t >= -H) {
      const bf16* hr = halo_row(halo, b, t + H, H, (size_t)3 * D);
      if (hr) { src = hr + 3 * c0 + ch * 8; nb = 16; }
    } else if (ahead_mode && t >= L && t < L + H) {
      const bf16* ar = halo_row(ahead_f, b, t - L, H, (size_t)3 * D);
      if (ar) { src = ar + 3 * c0 + ch * 8; nb = 16; }
    }
    cp_async16(&fS[row][ch * 8], src, nb);
  }
  for (int idx = tid; idx < ROWS_G * GCH; idx += SE_CT * SE_NSEG) {
    const int row = idx / GCH, ch = idx % GCH, t = t0 + row;
    const bf16* src = dz;
    int nb = 0;
    if (t >= 0 && t < L) { src = dz + ((size_t)b * L + t) * D + c0 + ch * 8; nb = 16; }
    else if (ahead_mode && t >= L && t < L + H) {
      const bf16* ar = halo_row(ahead_g, b, t - L, H, (size_t)D);
      if (ar) { src = ar + c0 + ch * 8; nb = 16; }
    }
    cp_async16(&gS[row][ch * 8], src, nb);
  }
  for (int idx = tid; idx < SE_CT * K; idx += SE_CT * SE_NSEG) (&dwS[0][0])[idx] = 0.f;
  cp_async_wait_all();
  __syncthreads();

  const int c = tid % SE_CT, seg = tid / SE_CT;
  const int r0 = seg * SE_SEG;                              // first step of this thread, relative to t0
  float wr[K], dwacc[K], uw[K], gw[K];
#pragma unroll
  for (int j = 0; j < K; ++j) { wr[j] = w[(size_t)((c0 + c) / dg) * K + j]; dwacc[j] = 0.f; }
  // u and dconv at relative step r (time t0 + r): feature row r + H, dz row r
  auto u_at = [&](int r) -> float {
    const float x2 = __bfloat162float(fS[r + H][3 * c + 1]), v = __bfloat162float(fS[r + H][3 * c + 2]);
    return pregate ? x2 * v : v;
  };
  auto dconv_at = [&](int r) -> float {
    const float g = __bfloat162float(gS[r][c]);
    return postgate ? g * __bfloat162float(fS[r + H][3 * c]) : g;
  };
#pragma unroll
  for (int j = 0; j < H; ++j) { uw[j + 1] = u_at(r0 - H + j); gw[j + 1] = dconv_at(r0 + j); }
  // The results overwrite this thread's own (x1, x2, v) entries of the tile, so that they can leave with 16-byte
  // stores.  Everything a thread needs from another segment's rows is therefore read before the barrier: the u history
  // above and the dconv look-ahead past the end of the segment here.
  float la[H > 0 ? H : 1];
#pragma unroll
  for (int j = 0; j < H; ++j) la[j] = dconv_at(r0 + SE_SEG + j);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < SE_SEG; ++i) {
    const int r = r0 + i;
#pragma unroll
    for (int j = 0; j < H; ++j) { uw[j] = uw[j + 1]; gw[j] = gw[j + 1]; }
    const float x2 = __bfloat162float(fS[r + H][3 * c + 1]), v = __bfloat162float(fS[r + H][3 * c + 2]);
    const float g = __bfloat162float(gS[r][c]);
    uw[K - 1] = pregate ? x2 * v : v;
    gw[K - 1] = (i + H < SE_SEG) ? dconv_at(r + H) : la[(i + H - SE_SEG) % (H > 0 ? H : 1)];
    float conv = 0.f, du = 0.f;
    const float g0 = (t0 + r) < L ? gw[0] : 0.f;             // look-ahead rows count in the next chunk's filter gradient
#pragma unroll
    for (int j = 0; j < K; ++j) {
      conv += wr[j] * uw[j];
      du += wr[j] * gw[K - 1 - j];
      dwacc[j] += g0 * uw[j];
    }
    fS[r + H][3 * c] = __float2bfloat16(postgate ? g * conv : 0.f);
    fS[r + H][3 * c + 1] = __float2bfloat16(pregate ? du * v : 0.f);
    fS[r + H][3 * c + 2] = __float2bfloat16(pregate ? du * x2 : du);
  }
  // filter gradient: lanes of one group first (groups of 2..32 consecutive channels), then the CTA, then one atomic
  const int span = dg % 32 == 0 ? 32 : (dg < 32 && (dg & (dg - 1)) == 0 ? dg : 0);
  if (span > 0) {
#pragma unroll
    for (int j = 0; j < K; ++j)
      for (int o = span >> 1; o > 0; o >>= 1) dwacc[j] += __shfl_xor_sync(0xffffffffu, dwacc[j], o);
    if ((c & (span - 1)) == 0) {
#pragma unroll
      for (int j = 0; j < K; ++j) atomicAdd(&dwS[c][j], dwacc[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < K; ++j) atomicAdd(&dwS[c][j], dwacc[j]);
  }
  __syncthreads();
  for (int idx = tid; idx < SE_CT * K; idx += SE_CT * SE_NSEG) {
    const float vsum = (&dwS[0][0])[idx];
    if (vsum != 0.f) atomicAdd(dw + (size_t)((c0 + idx / K) / dg) * K + idx % K, vsum);
  }
  for (int idx = tid; idx < SE_T * FCH; idx += SE_CT * SE_NSEG) {
    const int r = idx / FCH, ch = idx % FCH, t = t0 + r;
    bf16* dst = nullptr;
    if (t >= 0 && t < L) dst = dfeat + ((size_t)b * L + t) * 3 * D + 3 * c0 + ch * 8;
    else if (t < 0 && t >= -H && dhalo) dst = dhalo + ((size_t)b * H + (t + H)) * 3 * D + 3 * c0 + ch * 8;
    if (dst) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&fS[r + H][ch * 8]);
  }
}

static int g_se_bwd_tiled = 1;
static int g_conv_fwd_tiled = 1;   // depthwise-conv forward through shared-memory tiles

static inline int pick_tl(int L, int B, int cvecs) {
  // enough CTAs to fill 148 SMs a few times over, runs long enough to amortise the K-1 overlap
  int tl = 64;
  while (tl > 16 && (long long)((L + tl - 1) / tl) * B * ((cvecs + 127) / 128) < sb::num_sms() * 4) tl >>= 1;
  return tl;
}

}  // namespace sb

using namespace sb;

#define K_SWITCH(K, ...)                    \
  switch (K) {                              \
    case 2: { constexpr int KK = 2; __VA_ARGS__; break; } \
    case 3: { constexpr int KK = 3; __VA_ARGS__; break; } \
    case 4: { constexpr int KK = 4; __VA_ARGS__; break; } \
    case 5: { constexpr int KK = 5; __VA_ARGS__; break; } \
    case 6: { constexpr int KK = 6; __VA_ARGS__; break; } \
    case 7: { constexpr int KK = 7; __VA_ARGS__; break; } \
    case 8: { constexpr int KK = 8; __VA_ARGS__; break; } \
    default: return -7;                     \
  }

extern "C" int sb_dwconv_fwd(const void* x, const void* halo, const float* w, void* y, int B, int L, int C, int K,
                             cudaStream_t st) {
  if (C % 8) return -1;
  if (B * L == 0) return 0;
  if (g_conv_fwd_tiled && C % DW_CT_F == 0) {
    constexpr int T = DW_SEG_F * DW_NSEG_F;
    dim3 grid(C / DW_CT_F, (L + T - 1) / T, B);
    K_SWITCH(K, (dwconv_fwd_tiled_kernel<KK><<<grid, DW_CT_F / 2 * DW_NSEG_F, 0, st>>>((const bf16*)x, halo_local(halo), w,
                                                                                     (bf16*)y, L, C)));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int cvecs = C / 8, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (dwconv_fwd_kernel<KK, 8><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)halo, w, (bf16*)y, L, C, tl)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_dwconv_bwd(const void* x, const void* halo, const float* w, const void* dy, void* dx, void* dhalo,
                             float* dw, int B, int L, int C, int K, cudaStream_t st) {
  if (C % 4) return -1;
  if (B * L == 0) return 0;
  if (g_se_bwd_tiled && C % DW_CT == 0) {
    dim3 grid(C / DW_CT, (L + K - 1 + DW_T - 1) / DW_T, B);
    K_SWITCH(K, (dwconv_bwd_tiled_kernel<KK><<<grid, DW_CT / 2 * DW_NSEG, 0, st>>>((const bf16*)x, halo_local(halo), w,
                                                                                 (const bf16*)dy, (bf16*)dx, (bf16*)dhalo, dw, L, C,
                                                                                 0, halo_local(nullptr))));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int cvecs = C / 4, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (dwconv_bwd_kernel<KK, 4><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)halo, w, (const bf16*)dy,
                                                               (bf16*)dx, (bf16*)dhalo, dw, L, C, tl)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// 1: Hyena-SE and depthwise-conv backward through shared-memory tiles; 0: one run per thread straight from global memory.
extern "C" int sb_se_set_bwd_variant(int tiled) { sb::g_se_bwd_tiled = tiled ? 1 : 0; return 0; }
extern "C" int sb_conv_set_fwd_variant(int tiled) { sb::g_conv_fwd_tiled = tiled ? 1 : 0; return 0; }

extern "C" int sb_se_fwd(const void* feat, const void* halo, const float* w, void* z, int B, int L, int D, int G, int K,
                         int pregate, int postgate, cudaStream_t st) {
  if ((D % 8) || (D % G)) return -1;
  if (B * L == 0) return 0;
  if (g_conv_fwd_tiled && D % SE_CT == 0) {
    dim3 grid(D / SE_CT, (L + SE_T - 1) / SE_T, B);
    K_SWITCH(K, (se_fwd_tiled_kernel<KK><<<grid, SE_CT * SE_NSEG, 0, st>>>((const bf16*)feat, halo_local(halo), w, (bf16*)z, L, D,
                                                                         D / G, pregate, postgate)));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int cvecs = D / 8, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (se_fwd_kernel<KK, 8><<<grid, threads, 0, st>>>((const bf16*)feat, (const bf16*)halo, w, (bf16*)z, L, D, D / G, tl,
                                                           pregate, postgate)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_se_bwd(const void* feat, const void* halo, const float* w, const void* dz, void* dfeat, void* dhalo,
                         float* dw, int B, int L, int D, int G, int K, int pregate, int postgate, cudaStream_t st) {
  if ((D % 4) || (D % G)) return -1;
  if (B * L == 0) return 0;
  if (g_se_bwd_tiled && D % SE_CT == 0) {
    const int H = K - 1, steps = L + (halo ? H : 0);
    dim3 grid(D / SE_CT, (steps + SE_T - 1) / SE_T, B);
    K_SWITCH(K, (se_bwd_tiled_kernel<KK><<<grid, SE_CT * SE_NSEG, 0, st>>>((const bf16*)feat, halo_local(halo), halo ? 1 : 0, w,
                                                                         (const bf16*)dz, (bf16*)dfeat, (bf16*)dhalo, dw, L, D, D / G,
                                                                         pregate, postgate, 0, halo_local(nullptr), halo_local(nullptr))));
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int cvecs = D / 4, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (se_bwd_kernel<KK, 4><<<grid, threads, 0, st>>>((const bf16*)feat, (const bf16*)halo, w, (const bf16*)dz,
                                                           (bf16*)dfeat, (bf16*)dhalo, dw, L, D, D / G, tl, pregate, postgate)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}


// ------------------------------------------------------------------------------------ context-parallel entry points
// The same tiled kernels with the edge rows read in place from the neighbours' staged chunk edges (peer memory, see
// halo_src.cuh): x / feat are [2B, L, .] (two zigzag chunks per sequence as consecutive batch rows), `before` describes
// the staged tails (rows preceding each chunk), `ahead*` the staged heads of the tensors whose look-ahead the backward
// needs.  No halo tensor and no halo gradient exist on this path.  Return -9 when the shape has no tiled kernel.
extern "C" int sb_dwconv_fwd_cp(const void* x, const HaloSrc* before, const float* w, void* y, int B2, int L, int C, int K,
                                cudaStream_t st) {
  if (C % DW_CT_F || !before) return -9;
  if (B2 * L == 0) return 0;
  constexpr int T = DW_SEG_F * DW_NSEG_F;
  dim3 grid(C / DW_CT_F, (L + T - 1) / T, B2);
  K_SWITCH(K, (dwconv_fwd_tiled_kernel<KK><<<grid, DW_CT_F / 2 * DW_NSEG_F, 0, st>>>((const bf16*)x, *before, w, (bf16*)y, L, C)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_dwconv_bwd_cp(const void* x, const HaloSrc* before, const float* w, const void* dy, const HaloSrc* ahead_dy,
                                void* dx, float* dw, int B2, int L, int C, int K, cudaStream_t st) {
  if (C % DW_CT || !before || !ahead_dy) return -9;
  if (B2 * L == 0) return 0;
  dim3 grid(C / DW_CT, (L + DW_T - 1) / DW_T, B2);
  K_SWITCH(K, (dwconv_bwd_tiled_kernel<KK><<<grid, DW_CT / 2 * DW_NSEG, 0, st>>>((const bf16*)x, *before, w, (const bf16*)dy,
                                                                               (bf16*)dx, nullptr, dw, L, C, 1, *ahead_dy)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_se_fwd_cp(const void* feat, const HaloSrc* before, const float* w, void* z, int B2, int L, int D, int G, int K,
                            int pregate, int postgate, cudaStream_t st) {
  if ((D % SE_CT) || (D % G) || !before) return -9;
  if (B2 * L == 0) return 0;
  dim3 grid(D / SE_CT, (L + SE_T - 1) / SE_T, B2);
  K_SWITCH(K, (se_fwd_tiled_kernel<KK><<<grid, SE_CT * SE_NSEG, 0, st>>>((const bf16*)feat, *before, w, (bf16*)z, L, D, D / G,
                                                                       pregate, postgate)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_se_bwd_cp(const void* feat, const HaloSrc* before, const float* w, const void* dz, const HaloSrc* ahead_feat,
                            const HaloSrc* ahead_dz, void* dfeat, float* dw, int B2, int L, int D, int G, int K, int pregate,
                            int postgate, cudaStream_t st) {
  if ((D % SE_CT) || (D % G) || !before || !ahead_feat || !ahead_dz) return -9;
  if (B2 * L == 0) return 0;
  dim3 grid(D / SE_CT, (L + SE_T - 1) / SE_T, B2);
  K_SWITCH(K, (se_bwd_tiled_kernel<KK><<<grid, SE_CT * SE_NSEG, 0, st>>>((const bf16*)feat, *before, 1, w, (const bf16*)dz,
                                                                       (bf16*)dfeat, nullptr, dw, L, D, D / G, pregate, postgate,
                                                                       1, *ahead_feat, *ahead_dz)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
