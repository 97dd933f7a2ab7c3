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

static inline int pick_tl(int L, int B, int cvecs) {
  // enough CTAs to fill 148 SMs a few times over, runs long enough to amortise the K-1 overlap
  int tl = 64;
  while (tl > 16 && (long long)((L + tl - 1) / tl) * B * ((cvecs + 127) / 128) < 148 * 4) tl >>= 1;
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
  const int cvecs = C / 8, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (dwconv_fwd_kernel<KK, 8><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)halo, w, (bf16*)y, L, C, tl)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_dwconv_bwd(const void* x, const void* halo, const float* w, const void* dy, void* dx, void* dhalo,
                             float* dw, int B, int L, int C, int K, cudaStream_t st) {
  if (C % 4) return -1;
  if (B * L == 0) return 0;
  const int cvecs = C / 4, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (dwconv_bwd_kernel<KK, 4><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)halo, w, (const bf16*)dy,
                                                               (bf16*)dx, (bf16*)dhalo, dw, L, C, tl)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_se_fwd(const void* feat, const void* halo, const float* w, void* z, int B, int L, int D, int G, int K,
                         int pregate, int postgate, cudaStream_t st) {
  if ((D % 8) || (D % G)) return -1;
  if (B * L == 0) return 0;
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
  const int cvecs = D / 4, threads = 128, tl = pick_tl(L, B, cvecs);
  dim3 grid((cvecs + threads - 1) / threads, (L + tl - 1) / tl, B);
  K_SWITCH(K, (se_bwd_kernel<KK, 4><<<grid, threads, 0, st>>>((const bf16*)feat, (const bf16*)halo, w, (const bf16*)dz,
                                                           (bf16*)dfeat, (bf16*)dhalo, dw, L, D, D / G, tl, pregate, postgate)));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
