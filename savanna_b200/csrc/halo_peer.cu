// Context-parallel halo exchange through NVSwitch peer memory (plain loads from the neighbours' symmetric buffers).
// Under zigzag sharding rank r holds chunks (r, 2cp-1-r) of the sequence back to back.  A causal filter needs the H
// rows before each chunk: the first chunk's come from rank r-1 (zeros on rank 0), the second chunk's from rank r+1
// (on the last rank: from its own first chunk).  Every rank stages its two chunk tails as [B, 2, H, C] in a symmetric
// buffer; after a device barrier `halo_pull` gathers the two neighbour tails into the local halo tensor that the
// convolution kernels read.  Backward runs the other way: every rank stages the halo gradients its convolution
// produced, and `halo_push_add` adds the neighbours' parts onto the tail rows of the local input gradient.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {

// dst [B, 2, H, C]; prev / next: the neighbours' staged [B, 2, H, C] (null: no such neighbour); own: this rank's staging.
// 16-byte vectors; n_vec = H * C / 8 per (b, chunk).
__global__ void halo_pull_kernel(uint4* __restrict__ dst, const uint4* __restrict__ prev, const uint4* __restrict__ next,
                                 const uint4* __restrict__ own, int B, int n_vec) {
  const long long total = (long long)B * 2 * n_vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % n_vec);
    const long long bc = i / n_vec;
    const int chunk = int(bc & 1);
    const long long b = bc >> 1;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (chunk == 0) {
      if (prev) val = prev[(b * 2 + 0) * n_vec + v];          // tail of the first chunk of rank r-1
    } else {
      if (next) val = next[(b * 2 + 1) * n_vec + v];          // tail of the second chunk of rank r+1
      else val = own[(b * 2 + 0) * n_vec + v];                // last rank: its own first chunk precedes the second
    }
    dst[i] = val;
  }
}

__device__ __forceinline__ uint4 add_bf16x8(uint4 a, uint4 b) {
  uint4 r;
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    pr[i] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
  }
  return r;
}

// gx [B, L, C] (two chunks of L/2 rows): rows [L/2 - H, L/2) += the gradient of the halo that rank r+1 took from them
// (next[b, 0]), or on the last rank the gradient of its own second-chunk halo (own[b, 1]); rows [L - H, L) += the
// gradient of the halo rank r-1 took from them (prev[b, 1]).
__global__ void halo_push_add_kernel(uint4* __restrict__ gx, const uint4* __restrict__ prev, const uint4* __restrict__ next,
                                     const uint4* __restrict__ own, int B, int L, int C8, int H) {
  const int n_vec = H * C8;
  const long long total = (long long)B * 2 * n_vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % n_vec);
    const long long bc = i / n_vec;
    const int chunk = int(bc & 1);
    const long long b = bc >> 1;
    const int row = v / C8, col = v % C8;
    const uint4* src = nullptr;
    long long dst_row;
    if (chunk == 0) {                                // tail of my first chunk
      dst_row = L / 2 - H + row;
      if (next) src = next + (b * 2 + 0) * n_vec + v;
      else src = own + (b * 2 + 1) * n_vec + v;
    } else {                                         // tail of my second chunk
      dst_row = L - H + row;
      if (prev) src = prev + (b * 2 + 1) * n_vec + v;
    }
    if (src) {
      uint4* d = gx + (b * L + dst_row) * C8 + col;
      *d = add_bf16x8(*d, *src);
    }
  }
}

// plain 16-byte copy (peer -> local when `src` is a peer mapping)
__global__ void peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n16) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// 2-D copy of `rows` rows of `row16` 16-byte vectors between pitched buffers (pitches in 16-byte units)
__global__ void peer_copy_2d_kernel(uint4* __restrict__ dst, long long dst_pitch, const uint4* __restrict__ src,
                                    long long src_pitch, int row16, long long rows) {
  const long long total = rows * row16;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / row16;
    const int c = int(i - r * row16);
    dst[r * dst_pitch + c] = src[r * src_pitch + c];
  }
}

}  // namespace sb

// Pitched copy (all byte counts multiples of 16, addresses 16-byte aligned); `src` may be a peer GPU's memory.  The
// context-parallel all-to-all is 2*cp of these per rank: every rank pulls its channel block of each sequence chunk
// (or its sequence chunks of each channel block) straight into the final layout.
extern "C" int sb_peer_copy_2d(void* dst, long long dst_pitch, const void* src, long long src_pitch, long long row_bytes,
                               long long rows, int max_blocks, cudaStream_t st) {
  if ((row_bytes % 16) || (dst_pitch % 16) || (src_pitch % 16) ||
      ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15)) return -1;
  if (rows == 0 || row_bytes == 0) return 0;
  const long long total = rows * (row_bytes / 16);
  long long g = (total + 255) / 256;
  const long long cap = max_blocks > 0 ? max_blocks : 592;
  if (g > cap) g = cap;
  sb::peer_copy_2d_kernel<<<(unsigned)g, 256, 0, st>>>((uint4*)dst, dst_pitch / 16, (const uint4*)src, src_pitch / 16,
                                                      (int)(row_bytes / 16), rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Copy `bytes` (a multiple of 16, both addresses 16-byte aligned) with this framework's own kernel; `src` may be a
// peer GPU's memory.  `max_blocks` bounds the grid so that the copy leaves SMs to a kernel running beside it.
extern "C" int sb_peer_copy(void* dst, const void* src, long long bytes, int max_blocks, cudaStream_t st) {
  if ((bytes % 16) || ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15)) return -1;
  if (bytes == 0) return 0;
  const long long n16 = bytes / 16;
  long long g = (n16 + 255) / 256;
  const long long cap = max_blocks > 0 ? max_blocks : 592;
  if (g > cap) g = cap;
  sb::peer_copy_kernel<<<(unsigned)g, 256, 0, st>>>((uint4*)dst, (const uint4*)src, n16);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_halo_pull(void* dst, const void* prev, const void* next, const void* own, int B, int H, int C, cudaStream_t st) {
  if (C % 8) return -1;
  const long long total = (long long)B * 2 * H * (C / 8);
  if (total == 0) return 0;
  const int grid = (int)((total + 255) / 256 > 592 ? 592 : (total + 255) / 256);
  sb::halo_pull_kernel<<<grid, 256, 0, st>>>((uint4*)dst, (const uint4*)prev, (const uint4*)next, (const uint4*)own, B, H * (C / 8));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_halo_push_add(void* gx, const void* prev, const void* next, const void* own, int B, int L, int C, int H,
                                cudaStream_t st) {
  if ((C % 8) || (L % 2) || H > L / 2) return -1;
  const long long total = (long long)B * 2 * H * (C / 8);
  if (total == 0) return 0;
  const int grid = (int)((total + 255) / 256 > 592 ? 592 : (total + 255) / 256);
  sb::halo_push_add_kernel<<<grid, 256, 0, st>>>((uint4*)gx, (const uint4*)prev, (const uint4*)next, (const uint4*)own, B, L, C / 8, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
