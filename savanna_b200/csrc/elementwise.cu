// Memory-bound row / elementwise kernels (bf16 activations, fp32 math): RMSNorm fwd/bwd, gated-MLP
// activation fwd/bwd, rotate-half RoPE, cross-entropy fwd/bwd, squared-norm reduction, fused Adam.
// All use 16-byte vector accesses; grids are sized from the problem, row kernels use one CTA per row
// (forward) or a grid-stride over rows with per-thread column ownership (weight-gradient reductions).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_info.h"

namespace sb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; `red` is a shared array of >= 32 floats; all threads get the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) { t = warp_sum(t); if (lane == 0) red[0] = t; }
  __syncthreads();
  return red[0];
}

// ------------------------------------------------------------------------------------ RMSNorm
// form 0 ("te"):      y = w * x * rsqrt(mean(x^2) + eps);       saved a = rsqrt(mean + eps)
// form 1 ("classic"): y = w * x / (sqrt(mean(x^2)) + eps);      saved a = 1 / (rms + eps)
// Persistent blocks walk over the rows; a row stays in registers (packed) between the sum of squares and the scaling,
// and the next row is in flight meanwhile.
template <int VPT>
__global__ void __launch_bounds__(512, VPT == 1 ? 4 : 2)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                   float* __restrict__ a_out, int T, int D, float eps, int form) {
  __shared__ float red[2][32];
  const int nv = D >> 3;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  uint4 wv[VPT], xn[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    wv[v] = i < nv ? reinterpret_cast<const uint4*>(w)[i] : make_uint4(0, 0, 0, 0);
    xn[v] = make_uint4(0, 0, 0, 0);
  }
  size_t row = blockIdx.x;
  if (row < (size_t)T) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) xn[v] = reinterpret_cast<const uint4*>(x + row * D)[i];
    }
  }
  int it = 0;
  for (; row < (size_t)T; row += gridDim.x, ++it) {
    uint4 xc[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) xc[v] = xn[v];
    const size_t nxt = row + gridDim.x;
    if (nxt < (size_t)T) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        if (i < nv) xn[v] = reinterpret_cast<const uint4*>(x + nxt * D)[i];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float f[8]; unpack8(xc[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    ss = warp_sum(ss);
    float* rr = red[it & 1];
    if (lane == 0) rr[wid] = ss;
    __syncthreads();
    float tot = lane < nw ? rr[lane] : 0.f;
    tot = warp_sum(tot);
    const float mean = tot / D;
    const float a = form == 0 ? rsqrtf(mean + eps) : 1.f / (sqrtf(mean) + eps);
    if (threadIdx.x == 0) a_out[row] = a;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        float f[8], g[8]; unpack8(xc[v], f); unpack8(wv[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * a * g[j];
        reinterpret_cast<uint4*>(y + row * D)[i] = pack8(f);
      }
    }
  }
}

// dx = a * g - x * c * mean(g * x) (+ gres), g = w * dy;  c = a^3 (form 0) or a^2 / rms (form 1); gres is the gradient
// that reached x along the residual branch, added here instead of by a separate kernel
// partial[block, col] = sum over the block's rows of dy * x * a; rmsnorm_dw_reduce_kernel adds the blocks up.
// Each thread owns VPT fixed column-vectors (8 columns each) so its weight-gradient sums stay in registers over the
// row loop; the next row's x and dy are in flight (packed, 8 registers per vector) while this row is reduced and stored.
template <int VPT>
__global__ void __launch_bounds__(512, VPT == 1 ? 2 : 1)
rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ dy,
                   const float* __restrict__ a_in, const bf16* __restrict__ gres, bf16* __restrict__ dx,
                   float* __restrict__ partial,
                   int T, int D, float eps, int form) {
  __shared__ float red[2][32];
  const int nv = D >> 3;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float dwacc[VPT][8];
  uint4 wv[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    wv[v] = i < nv ? reinterpret_cast<const uint4*>(w)[i] : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[v][j] = 0.f;
  }
  uint4 xn[VPT], gn[VPT], rn[VPT];                      // next row: x, dy and (optional) the gradient to add
  size_t row = blockIdx.x;
  if (row < (size_t)T) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        xn[v] = reinterpret_cast<const uint4*>(x + row * D)[i]; gn[v] = reinterpret_cast<const uint4*>(dy + row * D)[i];
        if (gres) rn[v] = reinterpret_cast<const uint4*>(gres + row * D)[i];
      }
    }
  }
  int it = 0;
  for (; row < (size_t)T; row += gridDim.x, ++it) {
    uint4 xc[VPT], gc[VPT], rc[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) { xc[v] = xn[v]; gc[v] = gn[v]; rc[v] = rn[v]; }
    const size_t nxt = row + gridDim.x;
    if (nxt < (size_t)T) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        if (i < nv) {
          xn[v] = reinterpret_cast<const uint4*>(x + nxt * D)[i]; gn[v] = reinterpret_cast<const uint4*>(dy + nxt * D)[i];
          if (gres) rn[v] = reinterpret_cast<const uint4*>(gres + nxt * D)[i];
        }
      }
    }
    const float a = a_in[row];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        float xf[8], gf[8], wf[8];
        unpack8(xc[v], xf); unpack8(gc[v], gf); unpack8(wv[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gx = gf[j] * xf[j];
          dwacc[v][j] += gx * a;
          dot += gx * wf[j];
        }
      }
    }
    // block sum with one barrier per row (two alternating scratch rows)
    dot = warp_sum(dot);
    float* rr = red[it & 1];
    if (lane == 0) rr[wid] = dot;
    __syncthreads();
    float tot = lane < nw ? rr[lane] : 0.f;
    tot = warp_sum(tot);
    float c;
    if (form == 0) c = a * a * a;
    else { const float rms = 1.f / a - eps; c = a * a / fmaxf(rms, 1e-30f); }
    const float k = c * tot / D;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xc[v], xf); unpack8(gc[v], gf); unpack8(wv[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = a * gf[j] * wf[j] - xf[j] * k;
        if (gres) {
          float rf[8]; unpack8(rc[v], rf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rf[j];
        }
        reinterpret_cast<uint4*>(dx + row * D)[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    if (i < nv) {
      float4* dst = reinterpret_cast<float4*>(partial + (size_t)blockIdx.x * D + (size_t)i * 8);
      dst[0] = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
      dst[1] = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
    }
  }
}
// dw[col] = sum_b partial[b, col] as bf16: a block covers 32 groups of four columns, its 8 thread rows split the partial
// rows and are combined through shared memory (no atomics, no zero-initialised output)
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, bf16* __restrict__ dw, int nblk, int D) {
  __shared__ float4 part[8][32];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c4 = blockIdx.x * 32 + cx;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c4 * 4 < D) {
    for (int b = ry; b < nblk; b += 8) {
      const float4 p = *reinterpret_cast<const float4*>(partial + (size_t)b * D + (size_t)c4 * 4);
      s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
    }
  }
  part[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c4 * 4 < D) {
#pragma unroll
    for (int j = 1; j < 8; ++j) { const float4 p = part[j][cx]; s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w; }
    __nv_bfloat162 lo = __floats2bfloat162_rn(s.x, s.y), hi = __floats2bfloat162_rn(s.z, s.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dw + (size_t)c4 * 4) = o;
  }
}

// ------------------------------------------------------------------------------------ gated MLP activation
__device__ __forceinline__ float act_fwd(float a, int act) {
  switch (act) {
    case 0: return a * __fdividef(1.f, 1.f + __expf(-a));                          // silu
    case 1: return 0.5f * a * (1.f + erff(a * 0.70710678118654752f));              // gelu (erf)
    case 2: return fmaxf(a, 0.f);                                                  // relu
    default: return a;                                                             // identity
  }
}
__device__ __forceinline__ float act_grad(float a, int act) {
  switch (act) {
    case 0: { const float s = __fdividef(1.f, 1.f + __expf(-a)); return s * (1.f + a * (1.f - s)); }
    case 1: return 0.5f * (1.f + erff(a * 0.70710678118654752f)) + a * 0.3989422804014327f * __expf(-0.5f * a * a);
    case 2: return a > 0.f ? 1.f : 0.f;
    default: return 1.f;
  }
}
// act(a) and act'(a) together; SILU = true is the compile-time fast path (one exponential and one approximate reciprocal
// for both values), otherwise the run-time `act` selects.
template <bool SILU>
__device__ __forceinline__ void act_both(float a, int act, float& f, float& g) {
  if (SILU) {
    const float s = __fdividef(1.f, 1.f + __expf(-a));
    f = a * s;
    g = s + f * (1.f - s);
  } else {
    f = act_fwd(a, act);
    g = act_grad(a, act);
  }
}
template <bool SILU>
__device__ __forceinline__ float act_only(float a, int act) {
  return SILU ? a * __fdividef(1.f, 1.f + __expf(-a)) : act_fwd(a, act);
}

// ab [T, 2F] = [a | b]  ->  h [T, F] = act(a) * b
__global__ void glu_fwd_kernel(const bf16* __restrict__ ab, bf16* __restrict__ h, size_t T, int F, int act) {
  const int nvF = F >> 3;
  const size_t total = T * nvF;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / nvF; const int i = idx - row * nvF;
    const uint4* r = reinterpret_cast<const uint4*>(ab + row * 2 * F);
    float a[8], b[8], o[8];
    unpack8(r[i], a); unpack8(r[nvF + i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(a[j], act) * b[j];
    reinterpret_cast<uint4*>(h + row * F)[i] = pack8(o);
  }
}
__global__ void glu_bwd_kernel(const bf16* __restrict__ ab, const bf16* __restrict__ dh, bf16* __restrict__ dab,
                               size_t T, int F, int act) {
  const int nvF = F >> 3;
  const size_t total = T * nvF;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / nvF; const int i = idx - row * nvF;
    const uint4* r = reinterpret_cast<const uint4*>(ab + row * 2 * F);
    float a[8], b[8], g[8], da[8], db[8];
    unpack8(r[i], a); unpack8(r[nvF + i], b);
    unpack8(reinterpret_cast<const uint4*>(dh + row * F)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) { da[j] = g[j] * b[j] * act_grad(a[j], act); db[j] = g[j] * act_fwd(a[j], act); }
    uint4* o = reinterpret_cast<uint4*>(dab + row * 2 * F);
    o[i] = pack8(da); o[nvF + i] = pack8(db);
  }
}

// ------------------------------------------------------------------------------------ RoPE (rotate-half)
// x [B, L, H, hd] (arbitrary row stride `xs` between consecutive (b,l,h) rows is NOT assumed: rows are
// addressed as base + ((b*L + l)*H + h) * row_stride), cos/sin [L, rd] fp32, rd <= hd, rd % 16 == 0.
// inverse = 1 applies the transpose rotation (the backward pass).
__global__ void rope_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ cs,
                            const float* __restrict__ sn, int B, int L, int H, int hd, int rd, size_t x_row_stride,
                            size_t y_row_stride, int inverse) {
  const int half = rd >> 1;
  const int vec_per_row = hd >> 3;
  const size_t rows = (size_t)B * L * H;
  const size_t total = rows * vec_per_row;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / vec_per_row; const int vi = idx - row * vec_per_row;
    const int l = (row / H) % L;
    const int c0 = vi * 8;
    const bf16* xr = x + row * x_row_stride;
    bf16* yr = y + row * y_row_stride;
    float f[8]; unpack8(*reinterpret_cast<const uint4*>(xr + c0), f);
    if (c0 < rd) {
      float o[8], other[8];
      const bool lower = c0 < half;
      const int pc = lower ? c0 + half : c0 - half;
      unpack8(*reinterpret_cast<const uint4*>(xr + pc), other);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cs[(size_t)l * rd + c0 + j];
        float s = sn[(size_t)l * rd + c0 + j];
        if (inverse) s = -s;
        // y = x*cos + rotate_half(x)*sin ; rotate_half = [-x2, x1]
        o[j] = f[j] * c + (lower ? -other[j] : other[j]) * s;
      }
      *reinterpret_cast<uint4*>(yr + c0) = pack8(o);
    } else {
      *reinterpret_cast<uint4*>(yr + c0) = pack8(f);
    }
  }
}

// ------------------------------------------------------------------------------------ cross entropy
// One warp per row; V % 8 == 0.  loss = lse - logit[label]; lse saved for the backward pass.
__global__ void ce_fwd_kernel(const bf16* __restrict__ logits, const int64_t* __restrict__ labels,
                              float* __restrict__ loss, float* __restrict__ lse_out, size_t T, int V) {
  const int lane = threadIdx.x & 31;
  const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const uint4* r = reinterpret_cast<const uint4*>(logits + row * V);
  const int nv = V >> 3;
  float m = -INFINITY;
  for (int i = lane; i < nv; i += 32) {
    float f[8]; unpack8(r[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, f[j]);
  }
  m = warp_max(m);
  float s = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float f[8]; unpack8(r[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  s = warp_sum(s);
  const float lse = m + __logf(s);
  if (lane == 0) {
    const int64_t lab = labels[row];
    const float tl = (lab >= 0 && lab < V) ? __bfloat162float(logits[row * V + lab]) : 0.f;
    loss[row] = lse - tl;
    lse_out[row] = lse;
  }
}
// dlogits = (softmax - onehot) * g[row]
__global__ void ce_bwd_kernel(const bf16* __restrict__ logits, const int64_t* __restrict__ labels,
                              const float* __restrict__ lse, const float* __restrict__ g, bf16* __restrict__ dlogits,
                              size_t T, int V) {
  const int lane = threadIdx.x & 31;
  const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const uint4* r = reinterpret_cast<const uint4*>(logits + row * V);
  uint4* o = reinterpret_cast<uint4*>(dlogits + row * V);
  const int nv = V >> 3;
  const float l = lse[row], gr = g[row];
  const int lab = (int)labels[row];
  for (int i = lane; i < nv; i += 32) {
    float f[8]; unpack8(r[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pr = __expf(f[j] - l);
      if (i * 8 + j == lab) pr -= 1.f;
      f[j] = pr * gr;
    }
    o[i] = pack8(f);
  }
}

// ------------------------------------------------------------------------------------ squared norm
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void sqnorm_kernel(const T* __restrict__ x, const float* __restrict__ wgt, float* __restrict__ out, size_t n) {
  __shared__ float red[32];
  float acc = 0.f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = to_f<T>(x[i]);
    acc += wgt ? v * v * wgt[i] : v * v;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}
// bf16 input, 16-byte aligned arrays: eight values per thread and step, two steps in flight
__global__ void __launch_bounds__(512)
sqnorm_bf16_vec_kernel(const uint4* __restrict__ x, const float4* __restrict__ wgt, float* __restrict__ out, size_t n8) {
  __shared__ float red[32];
  float acc0 = 0.f, acc1 = 0.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  auto one = [&](size_t k, float& acc) {
    float f[8]; unpack8(x[k], f);
    if (wgt) {
      const float4 w0 = wgt[2 * k], w1 = wgt[2 * k + 1];
      acc += f[0] * f[0] * w0.x + f[1] * f[1] * w0.y + f[2] * f[2] * w0.z + f[3] * f[3] * w0.w +
             f[4] * f[4] * w1.x + f[5] * f[5] * w1.y + f[6] * f[6] * w1.z + f[7] * f[7] * w1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += f[j] * f[j];
    }
  };
  for (; i + stride < n8; i += 2 * stride) { one(i, acc0); one(i + stride, acc1); }
  if (i < n8) one(i, acc0);
  const float acc = block_sum(acc0 + acc1, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// ------------------------------------------------------------------------------------ fused Adam(W)
// One pass: grad (bf16 or fp32) * scale[0] -> moments -> fp32 master -> low-precision parameter copy.
struct AdamCoef { float lr, b1, b2, eps, wd, inv_bc1, inv_sqrt_bc2, scale; int adamw; };
__device__ __forceinline__ float adam_one(float g, float& w, float& mi, float& vi, const AdamCoef& c) {
  g *= c.scale;
  if (!c.adamw && c.wd != 0.f) g += c.wd * w;
  mi = c.b1 * mi + (1.f - c.b1) * g;
  vi = c.b2 * vi + (1.f - c.b2) * g * g;
  float upd = (mi * c.inv_bc1) / (sqrtf(vi) * c.inv_sqrt_bc2 + c.eps);
  if (c.adamw && c.wd != 0.f) upd += c.wd * w;
  w -= c.lr * upd;
  return w;
}
template <typename G>
__global__ void adam_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                            const G* __restrict__ grad, bf16* __restrict__ param_out, size_t n, float lr, float b1,
                            float b2, float eps, float wd, float bc1, float bc2, int adamw,
                            const float* __restrict__ scale_ptr, float scale_host) {
  const AdamCoef c{lr, b1, b2, eps, wd, 1.f / bc1, rsqrtf(bc2), scale_ptr ? scale_ptr[0] : scale_host, adamw};
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float w = master[i], mi = m[i], vi = v[i];
    adam_one(to_f<G>(grad[i]), w, mi, vi, c);
    m[i] = mi; v[i] = vi; master[i] = w;
    if (param_out) param_out[i] = __float2bfloat16_rn(w);
  }
}
// bf16 gradients, 16-byte aligned arrays, n a multiple of 4: four values per thread and step (16-byte accesses to the
// fp32 state, 8-byte to the bf16 gradient and parameter)
__global__ void __launch_bounds__(512)
adam_bf16_vec_kernel(float4* __restrict__ master, float4* __restrict__ m, float4* __restrict__ v,
                     const uint2* __restrict__ grad, uint2* __restrict__ param_out, size_t n4, float lr, float b1,
                     float b2, float eps, float wd, float bc1, float bc2, int adamw,
                     const float* __restrict__ scale_ptr, float scale_host) {
  const AdamCoef c{lr, b1, b2, eps, wd, 1.f / bc1, rsqrtf(bc2), scale_ptr ? scale_ptr[0] : scale_host, adamw};
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    float4 w = master[i], mi = m[i], vi = v[i];
    const uint2 gq = grad[i];
    const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gq.x));
    const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gq.y));
    adam_one(g01.x, w.x, mi.x, vi.x, c);
    adam_one(g01.y, w.y, mi.y, vi.y, c);
    adam_one(g23.x, w.z, mi.z, vi.z, c);
    adam_one(g23.y, w.w, mi.w, vi.w, c);
    m[i] = mi; v[i] = vi; master[i] = w;
    if (param_out) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
      param_out[i] = o;
    }
  }
}

// ------------------------------------------------------------------------------------ column sums (bias gradients)
// out[c] += sum_rows x[r, c]; each block owns 64 columns x a slab of rows, one fp32 atomic per column per block.
__global__ void __launch_bounds__(256)
colsum_kernel(const bf16* __restrict__ x, float* __restrict__ out, int T, int N, int rows_per_block) {
  __shared__ float part[64];
  const int cv = threadIdx.x & 7;                 // 8 column-vectors of 8 = 64 columns
  const int rl = threadIdx.x >> 3;                // 32 row lanes
  const int c0 = blockIdx.x * 64 + cv * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(r0 + rows_per_block, T);
  if (threadIdx.x < 64) part[threadIdx.x] = 0.f;
  __syncthreads();
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < N) {
    for (int r = r0 + rl; r < r1; r += 32) {
      float f[8]; unpack8(*reinterpret_cast<const uint4*>(x + (size_t)r * N + c0), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
  // a warp holds 4 row lanes x 8 column vectors: fold the row lanes, then one shared atomic per column per warp
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 8);
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
  }
  if ((threadIdx.x & 31) < 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&part[cv * 8 + j], acc[j]);
  }
  __syncthreads();
  if (threadIdx.x < 64) {
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < N) atomicAdd(out + c, part[threadIdx.x]);
  }
}

// ------------------------------------------------------------------------------------ fp8 quantisation (per tensor)
// amax: max |x| over the tensor (atomicMax on the bit pattern of a non-negative float; zero `out` first)
__global__ void amax_kernel(const bf16* __restrict__ x, float* __restrict__ out, size_t n8) {
  float m = 0.f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8]; unpack8(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(m));
}
// q = saturate(x * fmax / amax) in e4m3 (fmt 0) or e5m2 (fmt 1); scale_inv[0] = amax / fmax (the de-quantisation factor)
__global__ void quantize_fp8_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, size_t n8,
                                    const float* __restrict__ amax, float* __restrict__ scale_inv, int fmt) {
  const float fmax = fmt == 0 ? 448.f : 57344.f;
  const float a = fmaxf(amax[0], 1e-12f);
  const float scale = fmax / a;
  if (blockIdx.x == 0 && threadIdx.x == 0) scale_inv[0] = a / fmax;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8]; unpack8(reinterpret_cast<const uint4*>(x)[i], f);
    uint2 o;
    unsigned short h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = make_float2(f[2 * j] * scale, f[2 * j + 1] * scale);
      h[j] = fmt == 0 ? __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, __NV_E4M3) : __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, __NV_E5M2);
    }
    o.x = (unsigned)h[0] | ((unsigned)h[1] << 16);
    o.y = (unsigned)h[2] | ((unsigned)h[3] << 16);
    reinterpret_cast<uint2*>(q)[i] = o;
  }
}

__device__ __forceinline__ uint2 quant8(const float (&f)[8], float scale, int fmt) {
  unsigned short h[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = make_float2(f[2 * j] * scale, f[2 * j + 1] * scale);
    h[j] = fmt == 0 ? __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, __NV_E4M3) : __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, __NV_E5M2);
  }
  return make_uint2((unsigned)h[0] | ((unsigned)h[1] << 16), (unsigned)h[2] | ((unsigned)h[3] << 16));
}
// Delayed scaling in one pass over x.  `hist` is a ring of `slots` = history + 2 floats holding the amax of earlier
// calls at this site: the scale comes from the maximum over the ring except slot `cur` (which collects this call's
// amax by atomicMax and was zeroed by the previous call) and slot `cur + 1` (zeroed here for the next call).
// Values beyond the stale range saturate.  A ring without a finite positive entry leaves x unscaled.
// Each thread converts 16 consecutive values per step (two 16-byte loads, one 16-byte store), two steps in flight.
__global__ void __launch_bounds__(256)
quantize_fp8_delayed_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, size_t n16, size_t n8,
                            float* __restrict__ hist, int slots, int cur, float* __restrict__ scale_inv, int fmt) {
  const float fmax = fmt == 0 ? 448.f : 57344.f;
  const int nxt = cur + 1 == slots ? 0 : cur + 1;
  float a = 0.f;
  for (int j = 0; j < slots; ++j) {
    if (j == cur || j == nxt) continue;
    const float h = hist[j];
    if (h > a && h < 3.0e38f) a = h;
  }
  if (!(a > 0.f)) a = fmax;
  const float scale = fmax / a;
  if (blockIdx.x == 0 && threadIdx.x == 0) { scale_inv[0] = a / fmax; hist[nxt] = 0.f; }
  float m = 0.f;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* qv = reinterpret_cast<uint4*>(q);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  for (; i + stride < n16; i += 2 * stride) {
    const uint4 a0 = xv[2 * i], a1 = xv[2 * i + 1], b0 = xv[2 * (i + stride)], b1 = xv[2 * (i + stride) + 1];
    float f[8];
    uint2 lo, hi;
    unpack8(a0, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    lo = quant8(f, scale, fmt);
    unpack8(a1, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    hi = quant8(f, scale, fmt);
    qv[i] = make_uint4(lo.x, lo.y, hi.x, hi.y);
    unpack8(b0, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    lo = quant8(f, scale, fmt);
    unpack8(b1, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    hi = quant8(f, scale, fmt);
    qv[i + stride] = make_uint4(lo.x, lo.y, hi.x, hi.y);
  }
  for (; i < n16; i += stride) {
    float f[8];
    unpack8(xv[2 * i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    const uint2 lo = quant8(f, scale, fmt);
    unpack8(xv[2 * i + 1], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    const uint2 hi = quant8(f, scale, fmt);
    qv[i] = make_uint4(lo.x, lo.y, hi.x, hi.y);
  }
  // an odd trailing group of 8 values
  if (n8 & 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      float f[8];
      unpack8(xv[n8 - 1], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
      reinterpret_cast<uint2*>(q)[n8 - 1] = quant8(f, scale, fmt);
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(hist + cur), __float_as_uint(m));
}

// ------------------------------------------------------------------------------------ producers with fp8 output
// The scale of a delayed-scaling site is known before its tensor exists, so the kernel that produces the tensor can
// emit the e4m3 bytes for the next GEMM directly (and collect the amax for later calls) instead of writing bf16 that a
// quantiser re-reads.  Ring protocol as in quantize_fp8_delayed_kernel.
__device__ __forceinline__ float delayed_scale(float* hist, int slots, int cur, float* scale_inv, float fmax) {
  const int nxt = cur + 1 == slots ? 0 : cur + 1;
  float a = 0.f;
  for (int j = 0; j < slots; ++j) {
    if (j == cur || j == nxt) continue;
    const float h = hist[j];
    if (h > a && h < 3.0e38f) a = h;
  }
  if (!(a > 0.f)) a = fmax;
  if (blockIdx.x == 0 && threadIdx.x == 0) { scale_inv[0] = a / fmax; hist[nxt] = 0.f; }
  return fmax / a;
}

// RMSNorm whose output goes out as e4m3 (no bf16 copy): q = sat(w * x * a * scale)
template <int VPT>
__global__ void __launch_bounds__(512, VPT == 1 ? 4 : 2)
rmsnorm_fwd_fp8_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, uint8_t* __restrict__ q,
                       float* __restrict__ a_out, int T, int D, float eps, int form, float* __restrict__ hist, int slots,
                       int cur, float* __restrict__ scale_inv) {
  __shared__ float red[2][32];
  const float scale = delayed_scale(hist, slots, cur, scale_inv, 448.f);
  const int nv = D >> 3;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  uint4 wv[VPT], xn[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    wv[v] = i < nv ? reinterpret_cast<const uint4*>(w)[i] : make_uint4(0, 0, 0, 0);
    xn[v] = make_uint4(0, 0, 0, 0);
  }
  size_t row = blockIdx.x;
  if (row < (size_t)T) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) xn[v] = reinterpret_cast<const uint4*>(x + row * D)[i];
    }
  }
  float m = 0.f;
  int it = 0;
  for (; row < (size_t)T; row += gridDim.x, ++it) {
    uint4 xc[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) xc[v] = xn[v];
    const size_t nxt = row + gridDim.x;
    if (nxt < (size_t)T) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        if (i < nv) xn[v] = reinterpret_cast<const uint4*>(x + nxt * D)[i];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float f[8]; unpack8(xc[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    ss = warp_sum(ss);
    float* rr = red[it & 1];
    if (lane == 0) rr[wid] = ss;
    __syncthreads();
    float tot = lane < nw ? rr[lane] : 0.f;
    tot = warp_sum(tot);
    const float mean = tot / D;
    const float a = form == 0 ? rsqrtf(mean + eps) : 1.f / (sqrtf(mean) + eps);
    if (threadIdx.x == 0) a_out[row] = a;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        float f[8], g[8]; unpack8(xc[v], f); unpack8(wv[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // the value the un-fused path would have stored as bf16
          f[j] = __bfloat162float(__float2bfloat16_rn(f[j] * a * g[j]));
          m = fmaxf(m, fabsf(f[j]));
        }
        reinterpret_cast<uint2*>(q + row * D)[i] = quant8(f, scale, 0);
      }
    }
  }
  m = warp_max(m);
  if (lane == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(hist + cur), __float_as_uint(m));
}

// gated activation with e4m3 output: q [T, F] = sat(act(a) * b * scale) for ab [T, 2F] = [a | b]; F % 16 == 0, each
// thread handles 16 columns per step (two 16-byte loads per operand, one 16-byte store)
template <bool SILU>
__global__ void __launch_bounds__(256)
glu_fwd_fp8_kernel(const bf16* __restrict__ ab, uint8_t* __restrict__ q, size_t T, int F, int act, float* __restrict__ hist,
                   int slots, int cur, float* __restrict__ scale_inv) {
  const float scale = delayed_scale(hist, slots, cur, scale_inv, 448.f);
  const int nv = F >> 4;                          // 16-column groups per row
  const size_t total = T * nv;
  float m = 0.f;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / nv; const int i = idx - row * nv;
    const uint4* ra = reinterpret_cast<const uint4*>(ab + row * 2 * F) + 2 * i;
    const uint4* rb = reinterpret_cast<const uint4*>(ab + row * 2 * F + F) + 2 * i;
    const uint4 a0 = ra[0], a1 = ra[1], b0 = rb[0], b1 = rb[1];
    uint2 lo, hi;
    {
      float a[8], b[8], o[8];
      unpack8(a0, a); unpack8(b0, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = __bfloat162float(__float2bfloat16_rn(act_only<SILU>(a[j], act) * b[j])); m = fmaxf(m, fabsf(o[j])); }
      lo = quant8(o, scale, 0);
      unpack8(a1, a); unpack8(b1, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = __bfloat162float(__float2bfloat16_rn(act_only<SILU>(a[j], act) * b[j])); m = fmaxf(m, fabsf(o[j])); }
      hi = quant8(o, scale, 0);
    }
    reinterpret_cast<uint4*>(q + row * F)[i] = make_uint4(lo.x, lo.y, hi.x, hi.y);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(hist + cur), __float_as_uint(m));
}

// gate backward with e5m2 output: dab [T, 2F] = (dh * b * act'(a) | dh * act(a)) as fp8 for the w1|w2 gradient GEMMs;
// F % 16 == 0, 16 columns per thread and step
template <bool SILU>
__global__ void __launch_bounds__(256)
glu_bwd_fp8_kernel(const bf16* __restrict__ ab, const bf16* __restrict__ dh, uint8_t* __restrict__ dq, size_t T, int F,
                   int act, float* __restrict__ hist, int slots, int cur, float* __restrict__ scale_inv) {
  const float scale = delayed_scale(hist, slots, cur, scale_inv, 57344.f);
  const int nv = F >> 4;
  const size_t total = T * nv;
  float m = 0.f;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / nv; const int i = idx - row * nv;
    const uint4* ra = reinterpret_cast<const uint4*>(ab + row * 2 * F) + 2 * i;
    const uint4* rb = reinterpret_cast<const uint4*>(ab + row * 2 * F + F) + 2 * i;
    const uint4* rg = reinterpret_cast<const uint4*>(dh + row * F) + 2 * i;
    const uint4 av[2] = {ra[0], ra[1]}, bv[2] = {rb[0], rb[1]}, gv[2] = {rg[0], rg[1]};
    uint2 qa[2], qb[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float a[8], b[8], g[8], da[8], db[8];
      unpack8(av[h], a); unpack8(bv[h], b); unpack8(gv[h], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float f, dg;
        act_both<SILU>(a[j], act, f, dg);
        da[j] = __bfloat162float(__float2bfloat16_rn(g[j] * b[j] * dg));
        db[j] = __bfloat162float(__float2bfloat16_rn(g[j] * f));
        m = fmaxf(m, fmaxf(fabsf(da[j]), fabsf(db[j])));
      }
      qa[h] = quant8(da, scale, 1); qb[h] = quant8(db, scale, 1);
    }
    reinterpret_cast<uint4*>(dq + row * 2 * F)[i] = make_uint4(qa[0].x, qa[0].y, qa[1].x, qa[1].y);
    reinterpret_cast<uint4*>(dq + row * 2 * F + F)[i] = make_uint4(qb[0].x, qb[0].y, qb[1].x, qb[1].y);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(hist + cur), __float_as_uint(m));
}

static inline int grid_for(size_t work, int threads, int cap = sb::num_sms() * 16) {
  size_t g = (work + threads - 1) / threads;
  if (g > (size_t)cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace sb

using namespace sb;

extern "C" int sb_rmsnorm_fwd(const void* x, const void* w, void* y, float* a_out, int T, int D, float eps, int form,
                              cudaStream_t st) {
  if (D % 8) return -1;
  if (T == 0) return 0;
  const int nv = D / 8;
  const int threads = nv >= 512 ? 512 : (nv >= 256 ? 256 : (nv >= 128 ? 128 : 64));
  const int vpt = (nv + threads - 1) / threads;
  const int grid = T < sb::num_sms() * 4 ? T : sb::num_sms() * 4;
#define LAUNCH(V) rmsnorm_fwd_kernel<V><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)w, (bf16*)y, a_out, T, D, eps, form)
  if (vpt <= 1) LAUNCH(1);
  else if (vpt <= 2) LAUNCH(2);
  else if (vpt <= 4) LAUNCH(4);
  else return -3;
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Blocks of the backward kernel for T rows (also the number of rows of the `partial` scratch).
extern "C" int sb_rmsnorm_bwd_blocks(int T) { return T < sb::num_sms() * 2 ? (T < 1 ? 1 : T) : sb::num_sms() * 2; }

// dw: bf16 [D], written (not accumulated); partial is scratch of sb_rmsnorm_bwd_blocks(T) * D floats.  Two launches.
extern "C" int sb_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* a_in, const void* gres, void* dx,
                              void* dw, float* partial, int T, int D, float eps, int form, cudaStream_t st) {
  if (D % 8) return -1;
  if (T == 0) return 0;
  const int nv = D / 8;
  int threads = nv >= 512 ? 512 : (nv >= 256 ? 256 : (nv >= 128 ? 128 : 64));
  const int vpt = (nv + threads - 1) / threads;
  const int grid = sb_rmsnorm_bwd_blocks(T);
#define LAUNCH(V) rmsnorm_bwd_kernel<V><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, a_in, (const bf16*)gres, (bf16*)dx, partial, T, D, eps, form)
  if (vpt <= 1) LAUNCH(1);
  else if (vpt <= 2) LAUNCH(2);
  else if (vpt <= 4) LAUNCH(4);
  else return -3;
#undef LAUNCH
  rmsnorm_dw_reduce_kernel<<<(D / 4 + 31) / 32, 256, 0, st>>>(partial, (bf16*)dw, grid, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_glu_fwd(const void* ab, void* h, long long T, int F, int act, cudaStream_t st) {
  if (F % 8) return -1;
  if (T == 0) return 0;
  glu_fwd_kernel<<<grid_for((size_t)T * (F / 8), 256), 256, 0, st>>>((const bf16*)ab, (bf16*)h, (size_t)T, F, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
extern "C" int sb_glu_bwd(const void* ab, const void* dh, void* dab, long long T, int F, int act, cudaStream_t st) {
  if (F % 8) return -1;
  if (T == 0) return 0;
  glu_bwd_kernel<<<grid_for((size_t)T * (F / 8), 256), 256, 0, st>>>((const bf16*)ab, (const bf16*)dh, (bf16*)dab, (size_t)T, F, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_rope(const void* x, void* y, const float* cs, const float* sn, int B, int L, int H, int hd, int rd,
                       long long x_row_stride, long long y_row_stride, int inverse, cudaStream_t st) {
  if ((hd % 8) || (rd % 16) || rd > hd || (x_row_stride % 8) || (y_row_stride % 8)) return -1;
  const size_t total = (size_t)B * L * H * (hd / 8);
  if (total == 0) return 0;
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, cs, sn, B, L, H, hd, rd,
                                                    (size_t)x_row_stride, (size_t)y_row_stride, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_ce_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long T, int V,
                         cudaStream_t st) {
  if (V % 8) return -1;
  if (T == 0) return 0;
  const int wpb = 8;
  ce_fwd_kernel<<<(unsigned)((T + wpb - 1) / wpb), wpb * 32, 0, st>>>((const bf16*)logits, (const int64_t*)labels, loss, lse, (size_t)T, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
extern "C" int sb_ce_bwd(const void* logits, const long long* labels, const float* lse, const float* g, void* dlogits,
                         long long T, int V, cudaStream_t st) {
  if (V % 8) return -1;
  if (T == 0) return 0;
  const int wpb = 8;
  ce_bwd_kernel<<<(unsigned)((T + wpb - 1) / wpb), wpb * 32, 0, st>>>((const bf16*)logits, (const int64_t*)labels, lse, g, (bf16*)dlogits, (size_t)T, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// out [N] fp32 must be zeroed by the caller (it is accumulated into); N % 8 == 0
extern "C" int sb_colsum(const void* x, float* out, int T, int N, cudaStream_t st) {
  if (N % 8) return -1;
  if (T == 0 || N == 0) return 0;
  const int cblocks = (N + 63) / 64;
  int rsplit = (sb::num_sms() * 4 + cblocks - 1) / cblocks;
  if (rsplit > (T + 63) / 64) rsplit = (T + 63) / 64;
  if (rsplit < 1) rsplit = 1;
  const int rows_per_block = (T + rsplit - 1) / rsplit;
  dim3 grid(cblocks, (T + rows_per_block - 1) / rows_per_block);
  colsum_kernel<<<grid, 256, 0, st>>>((const bf16*)x, out, T, N, rows_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// out must be zeroed by the caller (it is accumulated into)
extern "C" int sb_sqnorm(const void* x, const float* wgt, float* out, long long n, int is_bf16, cudaStream_t st) {
  if (n == 0) return 0;
  if (is_bf16 && !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wgt)) & 15) && n >= 8) {
    const size_t n8 = (size_t)n / 8;
    sqnorm_bf16_vec_kernel<<<grid_for(n8, 512, sb::num_sms() * 4), 512, 0, st>>>((const uint4*)x, (const float4*)wgt, out, n8);
    const size_t done = n8 * 8;
    if (done < (size_t)n)
      sqnorm_kernel<bf16><<<1, 32, 0, st>>>((const bf16*)x + done, wgt ? wgt + done : nullptr, out, (size_t)n - done);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int grid = grid_for((size_t)n, 512, sb::num_sms() * 4);
  if (is_bf16) sqnorm_kernel<bf16><<<grid, 512, 0, st>>>((const bf16*)x, wgt, out, (size_t)n);
  else sqnorm_kernel<float><<<grid, 512, 0, st>>>((const float*)x, wgt, out, (size_t)n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_adam(float* master, float* m, float* v, const void* grad, void* param_out, long long n, float lr,
                       float b1, float b2, float eps, float wd, float bc1, float bc2, int adamw, const float* scale_ptr,
                       float scale_host, int grad_is_bf16, cudaStream_t st) {
  if (n == 0) return 0;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         (reinterpret_cast<uintptr_t>(grad) << 1) | (reinterpret_cast<uintptr_t>(param_out) << 1);
  if (grad_is_bf16 && !(bits & 15) && (n % 4) == 0) {
    const size_t n4 = (size_t)n / 4;
    adam_bf16_vec_kernel<<<grid_for(n4, 512, sb::num_sms() * 8), 512, 0, st>>>((float4*)master, (float4*)m, (float4*)v, (const uint2*)grad,
                                                                    (uint2*)param_out, n4, lr, b1, b2, eps, wd, bc1, bc2, adamw,
                                                                    scale_ptr, scale_host);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  const int grid = grid_for((size_t)n, 512, sb::num_sms() * 8);
  if (grad_is_bf16)
    adam_kernel<bf16><<<grid, 512, 0, st>>>(master, m, v, (const bf16*)grad, (bf16*)param_out, (size_t)n, lr, b1, b2, eps, wd, bc1, bc2, adamw, scale_ptr, scale_host);
  else
    adam_kernel<float><<<grid, 512, 0, st>>>(master, m, v, (const float*)grad, (bf16*)param_out, (size_t)n, lr, b1, b2, eps, wd, bc1, bc2, adamw, scale_ptr, scale_host);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// x: n bf16 values (n % 8 == 0) -> q: n bytes; amax and scale_inv are device floats (amax is zeroed here).
extern "C" int sb_quantize_fp8(const void* x, void* q, float* amax, float* scale_inv, long long n, int fmt, cudaStream_t st) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  const size_t n8 = (size_t)n / 8;
  const int grid = grid_for(n8, 512, sb::num_sms() * 8);
  if (cudaMemsetAsync(amax, 0, sizeof(float), st) != cudaSuccess) return -2;
  amax_kernel<<<grid, 512, 0, st>>>((const bf16*)x, amax, n8);
  quantize_fp8_kernel<<<grid, 512, 0, st>>>((const bf16*)x, (uint8_t*)q, n8, amax, scale_inv, fmt);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// The two halves of sb_quantize_fp8 as separate calls, for operands that are sharded over several GPUs and need ONE
// scale: every rank computes its amax, the ranks take the maximum (a collective on the same stream), every rank
// quantises with the common value.
extern "C" int sb_amax_bf16(const void* x, float* amax, long long n, cudaStream_t st) {
  if (n % 8) return -1;
  if (cudaMemsetAsync(amax, 0, sizeof(float), st) != cudaSuccess) return -2;
  if (n == 0) return 0;
  const size_t n8 = (size_t)n / 8;
  amax_kernel<<<grid_for(n8, 512, sb::num_sms() * 8), 512, 0, st>>>((const bf16*)x, amax, n8);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_quantize_fp8_with_amax(const void* x, void* q, const float* amax, float* scale_inv, long long n, int fmt,
                                         cudaStream_t st) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  const size_t n8 = (size_t)n / 8;
  quantize_fp8_kernel<<<grid_for(n8, 512, sb::num_sms() * 8), 512, 0, st>>>((const bf16*)x, (uint8_t*)q, n8, amax, scale_inv, fmt);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Delayed-scaling variant (one pass): see quantize_fp8_delayed_kernel.  `hist` has `slots` floats, all zero before the
// first use of a site; the caller advances `cur` by one (mod slots) per call and primes slot 0 with sb_quantize_fp8.
extern "C" int sb_quantize_fp8_delayed(const void* x, void* q, float* hist, int slots, int cur, float* scale_inv,
                                       long long n, int fmt, cudaStream_t st) {
  if ((n % 8) || slots < 3 || cur < 0 || cur >= slots) return -1;
  if (n == 0) return 0;
  const size_t n8 = (size_t)n / 8, n16 = n8 / 2;
  const int grid = grid_for((n16 + 1) / 2 + 1, 256, sb::num_sms() * 8);
  quantize_fp8_delayed_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (uint8_t*)q, n16, n8, hist, slots, cur, scale_inv, fmt);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// RMSNorm with e4m3 output under delayed scaling (ring protocol of sb_quantize_fp8_delayed); a_out as in sb_rmsnorm_fwd.
extern "C" int sb_rmsnorm_fwd_fp8(const void* x, const void* w, void* q, float* a_out, int T, int D, float eps, int form,
                                  float* hist, int slots, int cur, float* scale_inv, cudaStream_t st) {
  if ((D % 8) || slots < 3 || cur < 0 || cur >= slots) return -1;
  if (T == 0) return 0;
  const int nv = D / 8;
  const int threads = nv >= 512 ? 512 : (nv >= 256 ? 256 : (nv >= 128 ? 128 : 64));
  const int vpt = (nv + threads - 1) / threads;
  const int grid = T < sb::num_sms() * 4 ? T : sb::num_sms() * 4;
#define LAUNCH(V) rmsnorm_fwd_fp8_kernel<V><<<grid, threads, 0, st>>>((const bf16*)x, (const bf16*)w, (uint8_t*)q, a_out, T, D, eps, form, hist, slots, cur, scale_inv)
  if (vpt <= 1) LAUNCH(1);
  else if (vpt <= 2) LAUNCH(2);
  else if (vpt <= 4) LAUNCH(4);
  else return -3;
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Gated activation with e4m3 output under delayed scaling.
extern "C" int sb_glu_fwd_fp8(const void* ab, void* q, long long T, int F, int act, float* hist, int slots, int cur,
                              float* scale_inv, cudaStream_t st) {
  if ((F % 16) || slots < 3 || cur < 0 || cur >= slots) return -1;
  if (T == 0) return 0;
  const int g = grid_for((size_t)T * (F / 16), 256);
  if (act == 0) glu_fwd_fp8_kernel<true><<<g, 256, 0, st>>>((const bf16*)ab, (uint8_t*)q, (size_t)T, F, act, hist, slots, cur, scale_inv);
  else glu_fwd_fp8_kernel<false><<<g, 256, 0, st>>>((const bf16*)ab, (uint8_t*)q, (size_t)T, F, act, hist, slots, cur, scale_inv);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Gate backward with e5m2 output under delayed scaling (the gradient operand of the w1|w2 dgrad / wgrad GEMMs).
extern "C" int sb_glu_bwd_fp8(const void* ab, const void* dh, void* dq, long long T, int F, int act, float* hist, int slots,
                              int cur, float* scale_inv, cudaStream_t st) {
  if ((F % 16) || slots < 3 || cur < 0 || cur >= slots) return -1;
  if (T == 0) return 0;
  const int g = grid_for((size_t)T * (F / 16), 256);
  if (act == 0) glu_bwd_fp8_kernel<true><<<g, 256, 0, st>>>((const bf16*)ab, (const bf16*)dh, (uint8_t*)dq, (size_t)T, F, act, hist, slots,
                                                          cur, scale_inv);
  else glu_bwd_fp8_kernel<false><<<g, 256, 0, st>>>((const bf16*)ab, (const bf16*)dh, (uint8_t*)dq, (size_t)T, F, act, hist, slots, cur,
                                                   scale_inv);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
