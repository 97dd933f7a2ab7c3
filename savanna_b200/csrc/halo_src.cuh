// Where a causal-convolution kernel finds the rows outside its own chunk.
//
// Without context parallelism the K-1 rows before batch row b are row block b of one local tensor [Bk, H, W]
// (`chunked == 0`).  With context parallelism a rank holds two zigzag chunks per sequence, stored as consecutive batch
// rows (b = 2 * sequence + chunk), and every rank stages the edge rows of its chunks as [B, 2, H, W] in a symmetric
// buffer that its neighbours map.  The kernels then read the neighbour's staged rows themselves, with plain loads
// from peer memory, after the stream-ordered barrier that follows the staging: `p0` / `p1` is the staging buffer that
// serves chunk 0 / 1 (a neighbour's, this rank's own, or null when the chunk touches the end of the sequence) and
// `slot0` / `slot1` the staged chunk inside it.
//   rows BEFORE a chunk (forward halo, staged tails):  chunk 0 <- rank-1 slot 0;  chunk 1 <- rank+1 slot 1
//                                                      (last rank: own slot 0)
//   rows AFTER a chunk (look-ahead of the upstream gradient in the backward pass, staged heads):
//                                                      chunk 0 <- rank+1 slot 0 (last rank: own slot 1);
//                                                      chunk 1 <- rank-1 slot 1
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace sb {

struct HaloSrc {
  const void* p0;      // staging buffer serving chunk 0 (or the local halo tensor when `chunked == 0`)
  const void* p1;      // staging buffer serving chunk 1
  int slot0, slot1;    // staged chunk to read inside p0 / p1
  int chunked;
};

static inline HaloSrc halo_local(const void* halo) {
  HaloSrc h;
  h.p0 = halo; h.p1 = halo; h.slot0 = 0; h.slot1 = 0; h.chunked = 0;
  return h;
}

// Row r (0..H-1) of the edge rows serving batch row b, W elements per row; null = no such rows (zeros).
__device__ __forceinline__ const __nv_bfloat16* halo_row(const HaloSrc& h, int b, int r, int H, size_t W) {
  if (!h.chunked) {
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(h.p0);
    return base ? base + ((size_t)b * H + r) * W : nullptr;
  }
  const bool odd = b & 1;
  const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(odd ? h.p1 : h.p0);
  const int slot = odd ? h.slot1 : h.slot0;
  return base ? base + ((size_t)((b >> 1) * 2 + slot) * H + r) * W : nullptr;
}

}  // namespace sb
