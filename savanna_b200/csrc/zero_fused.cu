// ZeRO-1 optimizer step fused with its collectives over NVLink peer memory (one process per GPU; every rank's
// flat gradient and flat parameter buffers are mapped into every peer — symmetric memory).
//
//   zero_rs_kernel   : reduce-scatter.  The owner of a shard reads that shard's slice of the bf16 gradients of ALL
//                      ranks straight from their memory (16-byte peer loads), sums in fp32, writes the reduced
//                      slice into its own gradient buffer and accumulates the (weighted) squared norm — gradient
//                      reduction, the cast and the norm partial in one pass, no staging copy.
//   zero_adam_kernel : Adam(W) on the owned fp32 shard, gradient scaled by a device-resident coefficient
//                      (1/world x clip), then the updated bf16 parameters are STORED INTO EVERY RANK's flat
//                      parameter buffer (the all-gather as peer stores in the Adam epilogue).
// The kernels contain no waits: ordering against the peers' backward pass and next forward pass is done by the
// caller with stream-ordered barriers, so nothing here can spin.  Plain peer loads/stores only.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_info.h"

namespace sb {
typedef __nv_bfloat16 bf16;
constexpr int ZMAX = 16;      // max ranks of a partition group on one NVSwitch domain

struct PeerPtrs { const void* p[ZMAX]; };
struct PeerPtrsW { void* p[ZMAX]; };

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(q[i]); acc[2 * i] += t.x; acc[2 * i + 1] += t.y; }
}

__device__ __forceinline__ float block_sum_to(float local, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < 32) {
    t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;
}

// n8 = number of 8-element vectors of the shard; `lo8` = shard offset in vectors inside every rank's buffer.
// `grads` arrives ROTATED by the host (p[0] is this rank's own buffer, p[r] rank me+r), so the unrolled loops index it
// statically and the walk over the peers starts at a different link on every rank.  W = compiled rank slots (>= world),
// U = vectors per thread and pass: W * U 16-byte loads are in flight per thread before the first add.
template <int W, int U>
__global__ void __launch_bounds__(512, (W * U <= 8) ? 2 : 1)
zero_rs_kernel(PeerPtrs grads, int world, size_t lo8, size_t n8, bf16* __restrict__ out,
               const float* __restrict__ norm_weight, float* __restrict__ sqnorm) {
  __shared__ float red[32];
  float local = 0.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i0 < n8; i0 += stride * U) {
    uint4 v[U][W];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + u * stride;
      if (i < n8) {
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < world) v[u][r] = reinterpret_cast<const uint4*>(grads.p[r])[lo8 + i];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= n8) continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < world) add8(acc, v[u][r]);
      uint4 o;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      reinterpret_cast<uint4*>(out)[i] = o;
      if (norm_weight) {
        const float4 w0 = reinterpret_cast<const float4*>(norm_weight)[2 * i], w1 = reinterpret_cast<const float4*>(norm_weight)[2 * i + 1];
        local += acc[0] * acc[0] * w0.x + acc[1] * acc[1] * w0.y + acc[2] * acc[2] * w0.z + acc[3] * acc[3] * w0.w +
                 acc[4] * acc[4] * w1.x + acc[5] * acc[5] * w1.y + acc[6] * acc[6] * w1.z + acc[7] * acc[7] * w1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) local += acc[j] * acc[j];
      }
    }
  }
  const float t = block_sum_to(local, red);                   // one atomic per block
  if (threadIdx.x == 0) atomicAdd(sqnorm, t);
}

__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  return r;
}
__device__ __forceinline__ void mm_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                 "f"(__uint_as_float(v.w)) : "memory");
}

// `params` arrives rotated like the gradient pointers above (p[0] = own buffer).
template <int W>
__global__ void __launch_bounds__(512)
zero_adam_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, const bf16* __restrict__ grad,
                 PeerPtrsW params, void* mc_params, int world, size_t lo8, size_t n8, float lr, float b1, float b2,
                 float eps, float wd, float bc1, float bc2, int adamw, const float* __restrict__ scale_ptr) {
  const float scale = scale_ptr[0];
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 gv = reinterpret_cast<const uint4*>(grad)[i];
    float g[8];
    {
      const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(q[j]); g[2 * j] = t.x * scale; g[2 * j + 1] = t.y * scale; }
    }
    float w[8], mm[8], vv[8];
    float4* mp = reinterpret_cast<float4*>(master) + 2 * i;
    float4* ep = reinterpret_cast<float4*>(m) + 2 * i;
    float4* vp = reinterpret_cast<float4*>(v) + 2 * i;
    {
      float4 a = mp[0], b = mp[1]; w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
      a = ep[0]; b = ep[1]; mm[0] = a.x; mm[1] = a.y; mm[2] = a.z; mm[3] = a.w; mm[4] = b.x; mm[5] = b.y; mm[6] = b.z; mm[7] = b.w;
      a = vp[0]; b = vp[1]; vv[0] = a.x; vv[1] = a.y; vv[2] = a.z; vv[3] = a.w; vv[4] = b.x; vv[5] = b.y; vv[6] = b.z; vv[7] = b.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gj = g[j];
      if (!adamw && wd != 0.f) gj += wd * w[j];
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      float upd = (mm[j] * inv_bc1) / (sqrtf(vv[j]) * inv_sqrt_bc2 + eps);
      if (adamw && wd != 0.f) upd += wd * w[j];
      w[j] -= lr * upd;
    }
    mp[0] = make_float4(w[0], w[1], w[2], w[3]); mp[1] = make_float4(w[4], w[5], w[6], w[7]);
    ep[0] = make_float4(mm[0], mm[1], mm[2], mm[3]); ep[1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    vp[0] = make_float4(vv[0], vv[1], vv[2], vv[3]); vp[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 o;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(w[2 * j], w[2 * j + 1]);
    if (mc_params) {
      mm_st_16(reinterpret_cast<uint4*>(mc_params) + lo8 + i, o);        // one store, replicated by the switch
    } else {
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < world) reinterpret_cast<uint4*>(params.p[r])[lo8 + i] = o;
    }
  }
}

// ---------------------------------------------------------------------------- NVLS (multimem) variants
// With the buffers bound to an NVLink multicast object the switch does the work: one multimem.ld_reduce returns the
// sum of all ranks' gradients for 16 bytes (fp32 accumulation in the switch, so each rank pulls only its own shard
// across NVLink instead of world-1 copies of it), and one multimem.st writes the updated parameters into every rank.
constexpr int MM_U = 4;       // multimem.ld_reduce operations in flight per thread
__global__ void __launch_bounds__(512)
zero_rs_mm_kernel(const uint4* __restrict__ mc_grad, size_t lo8, size_t n8, bf16* __restrict__ out,
                  const float* __restrict__ norm_weight, float* __restrict__ sqnorm) {
  __shared__ float red[32];
  float local = 0.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i0 < n8; i0 += stride * MM_U) {
    uint4 v[MM_U];
#pragma unroll
    for (int u = 0; u < MM_U; ++u) {
      const size_t i = i0 + u * stride;
      if (i < n8) v[u] = mm_ld_reduce_bf16x8(mc_grad + lo8 + i);
    }
#pragma unroll
    for (int u = 0; u < MM_U; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= n8) continue;
      reinterpret_cast<uint4*>(out)[i] = v[u];
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8(acc, v[u]);
      if (norm_weight) {
        const float4 w0 = reinterpret_cast<const float4*>(norm_weight)[2 * i], w1 = reinterpret_cast<const float4*>(norm_weight)[2 * i + 1];
        local += acc[0] * acc[0] * w0.x + acc[1] * acc[1] * w0.y + acc[2] * acc[2] * w0.z + acc[3] * acc[3] * w0.w +
                 acc[4] * acc[4] * w1.x + acc[5] * acc[5] * w1.y + acc[6] * acc[6] * w1.z + acc[7] * acc[7] * w1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) local += acc[j] * acc[j];
      }
    }
  }
  const float t = block_sum_to(local, red);
  if (threadIdx.x == 0) atomicAdd(sqnorm, t);
}

}  // namespace sb

using namespace sb;

// NVLS reduce-scatter: mc_grad = multicast address of the flat gradient buffer (the same object on every rank).
extern "C" int sb_zero_reduce_scatter_mm(const void* mc_grad, long long lo, long long n, void* out, const float* norm_weight,
                                         float* sqnorm, cudaStream_t st) {
  if (!mc_grad || (lo % 8) || (n % 8) || (reinterpret_cast<uintptr_t>(mc_grad) & 15)) return -1;
  if (n == 0) return 0;
  const size_t n8 = (size_t)n / 8;
  size_t g = (n8 + 512 * MM_U - 1) / (512 * MM_U);
  if (g > sb::num_sms() * 4) g = sb::num_sms() * 4;
  zero_rs_mm_kernel<<<(unsigned)g, 512, 0, st>>>((const uint4*)mc_grad, (size_t)lo / 8, n8, (bf16*)out, norm_weight, sqnorm);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// grads[r]: base address of rank r's flat bf16 gradient buffer as mapped in THIS process.  lo / n in elements,
// both multiples of 8; `out` = own gradient buffer + lo.  sqnorm is accumulated into (zero it first).
extern "C" int sb_zero_reduce_scatter(const void* const* grads, int world, int me, long long lo, long long n, void* out,
                                      const float* norm_weight, float* sqnorm, cudaStream_t st) {
  if (world < 1 || world > ZMAX || (lo % 8) || (n % 8)) return -1;
  if (n == 0) return 0;
  PeerPtrs pp;
  for (int r = 0; r < ZMAX; ++r) pp.p[r] = r < world ? grads[(me + r) % world] : nullptr;
  const size_t n8 = (size_t)n / 8;
  auto grid = [&](int u, int per_sm) {
    size_t g = (n8 + 512 * (size_t)u - 1) / (512 * (size_t)u);
    return (unsigned)(g > sb::num_sms() * (size_t)per_sm ? sb::num_sms() * per_sm : g);
  };
  bf16* o = (bf16*)out;
  if (world <= 2)      zero_rs_kernel<2, 4><<<grid(4, 2), 512, 0, st>>>(pp, world, (size_t)lo / 8, n8, o, norm_weight, sqnorm);
  else if (world <= 4) zero_rs_kernel<4, 2><<<grid(2, 2), 512, 0, st>>>(pp, world, (size_t)lo / 8, n8, o, norm_weight, sqnorm);
  else if (world <= 8) zero_rs_kernel<8, 1><<<grid(1, 2), 512, 0, st>>>(pp, world, (size_t)lo / 8, n8, o, norm_weight, sqnorm);
  else                 zero_rs_kernel<16, 1><<<grid(1, 1), 512, 0, st>>>(pp, world, (size_t)lo / 8, n8, o, norm_weight, sqnorm);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// params[r]: base address of rank r's flat bf16 parameter buffer as mapped in this process.
// mc_params: multicast address of the flat parameter buffer (NVLS: one multimem.st per 16 bytes), or null (peer stores).
extern "C" int sb_zero_adam_allgather(float* master, float* m, float* v, const void* grad, void* const* params, void* mc_params,
                                      int world, int me, long long lo, long long n, float lr, float b1, float b2, float eps,
                                      float wd, float bc1, float bc2, int adamw, const float* scale_ptr, cudaStream_t st) {
  if (world < 1 || world > ZMAX || (lo % 8) || (n % 8) || !scale_ptr) return -1;
  if (n == 0) return 0;
  PeerPtrsW pp;
  for (int r = 0; r < ZMAX; ++r) pp.p[r] = r < world ? params[(me + r) % world] : nullptr;
  const size_t n8 = (size_t)n / 8;
  size_t g = (n8 + 511) / 512;
  if (g > sb::num_sms() * 4) g = sb::num_sms() * 4;
#define SB_ADAM(W) zero_adam_kernel<W><<<(unsigned)g, 512, 0, st>>>(master, m, v, (const bf16*)grad, pp, mc_params, world, \
                                                                     (size_t)lo / 8, n8, lr, b1, b2, eps, wd, bc1, bc2, adamw, scale_ptr)
  if (world <= 2) SB_ADAM(2); else if (world <= 4) SB_ADAM(4); else if (world <= 8) SB_ADAM(8); else SB_ADAM(16);
#undef SB_ADAM
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
