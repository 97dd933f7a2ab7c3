// Tensor/sequence-parallel projections fused with their collective (one process per GPU, peers mapped through
// symmetric memory).  Same tcgen05 / TMA / TMEM pipeline as gemm_sm100.cu (tile 128x256x64, 4 stages, two TMEM
// accumulators), with two additions that can be used separately or together:
//
//   all-gather -> GEMM   The A operand is sequence-sharded over the group: rank r holds rows [r*Ms, (r+1)*Ms).
//                        A few CTAs of the grid ("copy CTAs") pull the peers' shards over NVLink with 16-byte peer
//                        loads into a local gather buffer, one 128-row tile at a time, and publish a LOCAL flag per
//                        tile; the GEMM CTAs process the local shard's tiles first and wait (bounded) on those flags
//                        before their TMA producer touches a remote tile.  The transfer therefore overlaps the math
//                        tile by tile and every remote byte crosses NVLink exactly once.
//   GEMM -> reduce-scatter   The epilogue stores each output tile straight into the memory of the rank that owns
//                        those rows (peer stores into slot `me` of the owner's staging buffer [world, Ms, N]); a small
//                        owner-side kernel then sums the `world` slots (+ bias, + residual).  Stores overlap the
//                        remaining tiles' math; the summation order is fixed, so the result is deterministic.
//
// No kernel here waits on another GPU: flags are written and read by CTAs of the same grid (all co-resident: the
// grid never exceeds the SM count and every CTA needs a full SM's shared memory), and the cross-GPU ordering
// (peers' shards complete before the pull, stores landed before the reduction) is established by the caller with
// stream-ordered barriers.  Only plain peer loads/stores are used — no multicast TMA, no remote TMA at all.
#include "sm100.cuh"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

namespace tp {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2, STAGE_BYTES = A_STAGE + B_STAGE;
constexpr int EPI_LD = 72;                                   // staged epilogue row: 64 columns + 8 pad (144 B)
constexpr int EPI_BYTES = 4 * 32 * EPI_LD * 2;               // 4 epilogue warps x 32 rows
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_BYTES;
constexpr int CP_NB = 5, CP_CHUNK = 32768, CP_LAG = 3;        // copy CTAs: ring of bulk-copy buffers
constexpr int TMEM_COLS = 512, GROUP_M = 16, NUM_THREADS = 192, MAXR = 16;

struct Params {
  int M, N, K;
  // plain output (when rs_world == 0)
  __nv_bfloat16* C; int ldc;
  const __nv_bfloat16* bias;
  // all-gather of A
  int ag_world, ag_me, ag_tiles_per_rank, ag_epoch, n_gemm_ctas;
  int* ag_flags;                          // [m_tiles], local; value == ag_epoch means "tile is in the gather buffer"
  const __nv_bfloat16* ag_src[MAXR];      // peers' shards [Ms, K], leading dim ag_src_ld
  int ag_src_ld;
  __nv_bfloat16* ag_dst;                  // local gather buffer [M, K], leading dim K
  // reduce-scatter of C
  int rs_world, rs_me, rs_rows_per_owner;
  __nv_bfloat16* rs_dst[MAXR];            // owners' staging buffers [world, Ms, N]
  uint32_t* status;
};

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, m_tiles - first_m);
  const int r = tile - g * per_group;
  mt = first_m + r % gsz;
  nt = r / gsz;
}

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA_local, const __grid_constant__ CUtensorMap tmA_gather,
               const __grid_constant__ CUtensorMap tmB, Params p) {
  extern __shared__ uint8_t smem_raw[];
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;
  const bool ag = p.ag_world > 1;
  const int n_gemm = ag ? p.n_gemm_ctas : gridDim.x;
  const int n_copy_ctas = gridDim.x - n_gemm;            // copy CTAs take the lowest block indices: scheduled first
  const int first_local_tile = ag ? p.ag_me * p.ag_tiles_per_rank : 0;
  const int gemm_id = (int)blockIdx.x - n_copy_ctas;

  if (ag && (int)blockIdx.x < n_copy_ctas) {
    // ------------------------------------------------------------------ copy CTAs: pull remote tiles, publish local flags
    const int cid = blockIdx.x, n_copy = n_copy_ctas;
    const int n_remote = m_tiles - p.ag_tiles_per_rank;
    const int vec_per_row = p.K >> 3;
    const bool contiguous = p.ag_src_ld == p.K && p.K * 2 <= CP_CHUNK;   // whole rows per bulk chunk
    const uint32_t ring = (smem_u32(smem_raw) + 127u) & ~127u;
    const uint32_t cbar = ring + CP_NB * CP_CHUNK;                       // CP_NB mbarriers
    __shared__ int copy_abort;
    if (threadIdx.x == 0) {
      copy_abort = 0;
      for (int b = 0; b < CP_NB; ++b) mbar_init(cbar + 8u * b, 1);
      fence_barrier_init();
    }
    __syncthreads();
    uint32_t issued = 0, done = 0;                                       // chunk counters over the whole CTA lifetime
    for (int idx = cid; idx < n_remote; idx += n_copy) {
      const int mt = (first_local_tile + p.ag_tiles_per_rank + idx) % m_tiles;     // rotated order: next rank's shard first
      const int src_rank = mt / p.ag_tiles_per_rank;
      const int src_row0 = (mt - src_rank * p.ag_tiles_per_rank) * BM;
      const int rows = min(BM, p.M - mt * BM);
      if (contiguous) {
        // one thread drives a ring of bulk copies: peer memory -> shared -> local gather buffer
        if (threadIdx.x == 0) {
          const char* src = reinterpret_cast<const char*>(p.ag_src[src_rank] + (size_t)src_row0 * p.K);
          char* dst = reinterpret_cast<char*>(p.ag_dst + (size_t)mt * BM * p.K);
          const uint32_t row_bytes = (uint32_t)p.K * 2u;
          const uint32_t rows_per_chunk = max(1u, CP_CHUNK / row_bytes);
          const uint32_t chunk = rows_per_chunk * row_bytes;
          const uint32_t total = (uint32_t)rows * row_bytes;
          const uint32_t n_chunks = (total + chunk - 1) / chunk;
          bool ok = chunk <= (uint32_t)CP_CHUNK;
          for (uint32_t i = 0; ok && i < n_chunks + CP_LAG; ++i) {
            if (i < n_chunks) {
              const uint32_t b = issued % CP_NB;
              bulk_wait_read<CP_NB - CP_LAG - 1>();                      // the store that last used this buffer has read it
              const uint32_t off = i * chunk, sz = min(chunk, total - off);
              mbar_expect_tx(cbar + 8u * b, sz);
              bulk_load(ring + b * CP_CHUNK, src + off, sz, cbar + 8u * b);
              ++issued;
            }
            if (i >= (uint32_t)CP_LAG) {
              const uint32_t j = i - CP_LAG;
              const uint32_t b = done % CP_NB, par = (done / CP_NB) & 1u;
              if (!mbar_wait(cbar + 8u * b, par, &copy_abort, p.status, ST_TIMEOUT_PEER)) { ok = false; break; }
              const uint32_t off = j * chunk, sz = min(chunk, total - off);
              bulk_store(dst + off, ring + b * CP_CHUNK, sz);
              bulk_commit();
              ++done;
            }
          }
          bulk_wait<0>();                                                // all stores of this tile have landed
          if (ok) {
            __threadfence();
            fence_proxy_async();
            st_release(p.ag_flags + mt, p.ag_epoch);
          }
        }
      } else {
        const uint4* src = reinterpret_cast<const uint4*>(p.ag_src[src_rank] + (size_t)src_row0 * p.ag_src_ld);
        uint4* dst = reinterpret_cast<uint4*>(p.ag_dst + (size_t)mt * BM * p.K);
        const int total = rows * vec_per_row;
        const int src_ld8 = p.ag_src_ld >> 3;
        for (int i = threadIdx.x; i < total; i += NUM_THREADS * 8) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int j = i + u * NUM_THREADS;
            if (j < total) { const int r = j / vec_per_row, c = j - r * vec_per_row; v[u] = src[(size_t)r * src_ld8 + c]; }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int j = i + u * NUM_THREADS;
            if (j < total) dst[j] = v[u];
          }
        }
        __threadfence();
        fence_proxy_async();
        __syncthreads();
        if (threadIdx.x == 0) st_release(p.ag_flags + mt, p.ag_epoch);
      }
    }
    return;
  }

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4) + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA_local); prefetch_tmap(&tmA_gather); prefetch_tmap(&tmB);
  }
  if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (actual m tile, n tile): local shard first when the A operand is being gathered
  auto coords = [&](int tile, int& mt, int& nt) {
    int mr; tile_coords(tile, m_tiles, n_tiles, mr, nt);
    mt = ag ? (mr + first_local_tile) % m_tiles : mr;
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = gemm_id; tile < num_tiles && ok; tile += n_gemm) {
        int mt, nt; coords(tile, mt, nt);
        const int n0 = nt * BN;
        const bool local = !ag || (mt >= first_local_tile && mt < first_local_tile + p.ag_tiles_per_rank);
        if (!local) {
          // bounded wait for the copy CTAs
          const unsigned long long t0 = globaltimer();
          uint32_t it = 0;
          while (ld_acquire(p.ag_flags + mt) != p.ag_epoch) {
            if ((++it & 255u) == 0u) {
              if (*abort_flag) { ok = false; break; }
              if (globaltimer() - t0 > WAIT_BUDGET_NS) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0u, (uint32_t(ST_TIMEOUT_PEER) << 24) | uint32_t(mt & 0xffffff));
                ok = false; break;
              }
            }
          }
          if (!ok) break;
          fence_proxy_async();
        }
        const CUtensorMap* tma = local && ag ? &tmA_local : (ag ? &tmA_gather : &tmA_local);
        const int m0 = (local && ag) ? (mt - first_local_tile) * BM : mt * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES, b_dst = a_dst + A_STAGE;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_2d(a_dst, tma, k0, m0, full_bar(stage));
          if (B_MN == 0) tma_load_2d(b_dst, &tmB, k0, n0, full_bar(stage));
          else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, n0 + 64 * j, k0, full_bar(stage));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { const unsigned long long t0 = globaltimer(); while (globaltimer() - t0 < 200000ull) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, B_MN);
      constexpr uint32_t b_lbo = B_MN ? 8192u : 16u, b_step = B_MN ? (UMMA_K * 128u) >> 4 : (UMMA_K * 2u) >> 4;
      int stage = 0; uint32_t phase = 0; uint32_t acc_phase[2] = {0u, 0u}; int local = 0; bool ok = true;
      for (int tile = gemm_id; tile < num_tiles && ok; tile += n_gemm, ++local) {
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        acc_phase[acc] ^= 1u;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint64_t adesc = umma_smem_desc(a_addr, 16u, 1024u);
          const uint64_t bdesc = umma_smem_desc(a_addr + A_STAGE, b_lbo, 1024u);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(d_tmem, adesc + k * 2, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t acc_phase[2] = {0u, 0u}; int local = 0; bool ok = true;
    const bool rs = p.rs_world > 1;
    for (int tile = gemm_id; tile < num_tiles && ok; tile += n_gemm, ++local) {
      const int acc = local & 1;
      int mt, nt; coords(tile, mt, nt);
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      __nv_bfloat16* crow;
      bool staged = false;
      __nv_bfloat16* wbase = nullptr;                 // staged path: destination of row (mt*BM + q*32) of this warp
      if (rs) {
        const int row_w = mt * BM + q * 32;           // rows of one warp never straddle owners (rows_per_owner % 128 == 0)
        const int owner = row_w / p.rs_rows_per_owner, lr = row_w - owner * p.rs_rows_per_owner;
        const int ow = owner < p.rs_world ? owner : 0;
        wbase = p.rs_dst[ow] + ((size_t)p.rs_me * p.rs_rows_per_owner + lr) * p.N;
        crow = wbase + (size_t)lane * p.N;
        staged = ow != p.rs_me;                       // peer rows: coalesce through shared memory into 128-byte row segments
      } else {
        crow = p.C + (size_t)row * p.ldc;
      }
      __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem_gen + STAGES * STAGE_BYTES + 256) + q * 32 * EPI_LD;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (staged) {
          __nv_bfloat16* srow = stg + lane * EPI_LD + (c & 1) * 32;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 out;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
            *reinterpret_cast<uint4*>(srow + v * 8) = out;
          }
          if (c & 1) {
            __syncwarp();
            const int cbase = n0 + (c - 1) * 32;      // first of the 64 staged columns
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3), cv = (lane & 7) * 8;
              if (mt * BM + q * 32 + rr < p.M && cbase + cv + 8 <= p.N)
                *reinterpret_cast<uint4*>(wbase + (size_t)rr * p.N + cbase + cv) = *reinterpret_cast<const uint4*>(stg + rr * EPI_LD + cv);
            }
            __syncwarp();
          }
          continue;
        }
        if (row < p.M && col0 < p.N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col + 8 <= p.N) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              if (p.bias && !rs) {
                const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
                const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
                for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(b2[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
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
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// Owner-side reduction of the staging buffer [world, rows, N] (+ bias + residual) -> out [rows, N]
__global__ void rs_reduce_kernel(const __nv_bfloat16* __restrict__ staging, const __nv_bfloat16* __restrict__ bias,
                                 const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int world,
                                 size_t rows, int N) {
  const int nv = N >> 3;
  const size_t total = rows * nv;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / nv; const int c = idx - r * nv;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < world; ++w) {
      const uint4 v = reinterpret_cast<const uint4*>(staging + ((size_t)w * rows + r) * N)[c];
      const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(q[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
    }
    if (bias) {
      const uint4 v = reinterpret_cast<const uint4*>(bias)[c];
      const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(q[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
    }
    if (residual) {
      const uint4 v = reinterpret_cast<const uint4*>(residual + r * N)[c];
      const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(q[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
    }
    uint4 o;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    reinterpret_cast<uint4*>(out + r * N)[c] = o;
  }
}

// Plain peer gather (used where the gathered operand feeds a reduction dim: weight gradients)
__global__ void gather_rows_kernel(Params p) {
  const int vec_per_row = p.K >> 3;
  const size_t rows_per_rank = (size_t)p.ag_tiles_per_rank * BM;
  const size_t total = (size_t)p.M * vec_per_row;
  const int src_ld8 = p.ag_src_ld >> 3;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / vec_per_row; const int c = idx - r * vec_per_row;
    const int src = r / rows_per_rank;
    const size_t lr = r - src * rows_per_rank;
    reinterpret_cast<uint4*>(p.ag_dst)[idx] = reinterpret_cast<const uint4*>(p.ag_src[src])[lr * src_ld8 + c];
  }
}

}  // namespace tp
}  // namespace sb

using namespace sb;
using namespace sb::tp;

// Fused projection.  A: own shard [Ms, K] (leading dim lda) when ag_world > 1, else the full [M, K].  B: [N, K]
// (b_mn = 0) or [K, N] (b_mn = 1).  ag_src: `ag_world` shard base pointers (index = rank; entry `ag_me` = A);
// gather: local workspace [M, K]; flags: [ceil(M/128)] ints (any contents; `epoch` must differ from the previous
// call's on the same flags).  rs_dst: `rs_world` staging base pointers [rs_world, M/rs_world, N]; with rs_world <= 1
// the result goes to C (ldc) with optional bias.
extern "C" int sb_gemm_tp(const void* A, int lda, const void* B, int ldb, int b_mn, void* C, int ldc, const void* bias,
                          int M, int N, int K, int ag_world, int ag_me, const void* const* ag_src, void* gather, int* flags,
                          int epoch, int n_copy_ctas, int rs_world, int rs_me, void* const* rs_dst, unsigned int* status,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldb % 8)) return -3;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias; p.status = status;
  const bool ag = ag_world > 1, rs = rs_world > 1;
  CUtensorMap tmL, tmG, tmB;
  int rc;
  if (ag) {
    if (ag_world > MAXR || (M % ag_world) || ((M / ag_world) % BM)) return -7;
    const int Ms = M / ag_world;
    p.ag_world = ag_world; p.ag_me = ag_me; p.ag_tiles_per_rank = Ms / BM; p.ag_epoch = epoch; p.ag_flags = flags;
    for (int r = 0; r < ag_world; ++r) p.ag_src[r] = (const __nv_bfloat16*)ag_src[r];
    p.ag_src_ld = lda; p.ag_dst = (__nv_bfloat16*)gather;
    if ((rc = make_tmap_2d_bf16(&tmL, A, K, Ms, lda, BK, BM))) return rc;
    if ((rc = make_tmap_2d_bf16(&tmG, gather, K, M, K, BK, BM))) return rc;
  } else {
    if ((rc = make_tmap_2d_bf16(&tmL, A, K, M, lda, BK, BM))) return rc;
    tmG = tmL;
  }
  if (!b_mn) rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, BK, BN);
  else       rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  if (rs) {
    if (rs_world > MAXR || (M % rs_world) || ((M / rs_world) % BM)) return -8;
    p.rs_world = rs_world; p.rs_me = rs_me; p.rs_rows_per_owner = M / rs_world;
    for (int r = 0; r < rs_world; ++r) p.rs_dst[r] = (__nv_bfloat16*)rs_dst[r];
  } else if (ldc % 8) return -3;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sms = sb::num_sms();
  int n_copy = ag ? (n_copy_ctas > 0 ? n_copy_ctas : 16) : 0;
  int n_gemm = sms - n_copy;
  if (tiles < n_gemm) n_gemm = tiles;
  p.n_gemm_ctas = n_gemm;
  void (*kern)(const CUtensorMap, const CUtensorMap, const CUtensorMap, Params) = b_mn ? gemm_tp_kernel<1> : gemm_tp_kernel<0>;
  static bool attr_set[2] = {false, false};
  if (!attr_set[b_mn ? 1 : 0]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -5;
    attr_set[b_mn ? 1 : 0] = true;
  }
  kern<<<n_gemm + n_copy, NUM_THREADS, SMEM_BYTES, stream>>>(tmL, tmG, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

extern "C" int sb_rs_reduce(const void* staging, const void* bias, const void* residual, void* out, int world, long long rows,
                            int N, cudaStream_t stream) {
  if (N % 8) return -1;
  if (rows == 0) return 0;
  size_t total = (size_t)rows * (N / 8);
  size_t g = (total + 255) / 256;
  if (g > sb::num_sms() * 8) g = sb::num_sms() * 8;
  rs_reduce_kernel<<<(unsigned)g, 256, 0, stream>>>((const __nv_bfloat16*)staging, (const __nv_bfloat16*)bias,
                                                   (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, world, (size_t)rows, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// gather[M, K] <- concat over ranks of src[r][Ms, K] (leading dim ld)
extern "C" int sb_gather_rows(const void* const* src, int world, void* gather, int M, int K, int ld, cudaStream_t stream) {
  if ((K % 8) || (ld % 8) || world > MAXR || (M % world) || ((M / world) % BM)) return -1;
  Params p{};
  p.M = M; p.K = K; p.ag_tiles_per_rank = (M / world) / BM; p.ag_src_ld = ld; p.ag_dst = (__nv_bfloat16*)gather;
  for (int r = 0; r < world; ++r) p.ag_src[r] = (const __nv_bfloat16*)src[r];
  gather_rows_kernel<<<sb::num_sms() * 4, 512, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
