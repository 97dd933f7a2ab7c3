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
// Operands are bf16 (EB = 2) or one-byte e4m3 / e5m2 (EB = 1, kind::f8f6f4; the result is scaled by two device scalars,
// the operands' de-quantisation factors, in the epilogue): a gathered fp8 activation crosses NVLink with half the bytes.
// A micro-batch of `batch` sequences is one launch: rank r's shard is [batch, Ms, K] and the gathered / scattered
// tensor [batch, world, Ms, .], so row block (b, r) of the full tensor belongs to rank r.
//
// No kernel here waits on another GPU: flags are written and read by CTAs of the same grid (all co-resident: the
// grid never exceeds the SM count and every CTA needs a full SM's shared memory), and the cross-GPU ordering
// (peers' shards complete before the pull, stores landed before the reduction) is established by the caller with
// stream-ordered barriers.  Only plain peer loads/stores are used — no multicast TMA, no remote TMA at all.
#include "sm100.cuh"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                    uint32_t box_outer);

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
  // all-gather of A (element size EB bytes)
  int ag_world, ag_me, ag_tiles_per_rank, ag_batch, ag_epoch, n_gemm_ctas;   // tiles per (rank, sequence) block
  int* ag_flags;                          // [m_tiles], local; value == ag_epoch means "tile is in the gather buffer"
  const uint8_t* ag_src[MAXR];            // peers' shards [batch * Ms, K], leading dim ag_src_ld (elements)
  int ag_src_ld;
  uint8_t* ag_dst;                        // local gather buffer [M, K], leading dim K
  // reduce-scatter of C
  int rs_world, rs_me, rs_rows_per_block, rs_batch;
  __nv_bfloat16* rs_dst[MAXR];            // owners' staging buffers [world, batch * Ms, N]
  uint32_t* status;
  const float* alpha; const float* alpha2;  // de-quantisation factors of the two operands (fp8), or null
  int a_fmt, b_fmt;                         // fp8 formats for the instruction descriptor: 0 = e4m3, 1 = e5m2
};

// Row-block bookkeeping of the gathered operand: m-tile `mt` of the full [batch, world, Ms] row space.
__device__ __forceinline__ void ag_tile_source(const Params& p, int mt, int& src_rank, int& src_row0) {
  const int block = mt / p.ag_tiles_per_rank, t = mt - block * p.ag_tiles_per_rank;
  src_rank = block % p.ag_world;
  const int b = block / p.ag_world;
  src_row0 = (b * p.ag_tiles_per_rank + t) * BM;          // row inside the owner's shard [batch * Ms, K]
}
// Processing order: this rank's own blocks first, then the next rank's, ... (index -> m-tile of the full row space)
__device__ __forceinline__ int ag_ordered_tile(const Params& p, int idx) {
  const int per_rank = p.ag_batch * p.ag_tiles_per_rank;
  const int rr = idx / per_rank, rem = idx - rr * per_rank;
  const int b = rem / p.ag_tiles_per_rank, t = rem - b * p.ag_tiles_per_rank;
  const int r = (rr + p.ag_me) % p.ag_world;
  return (b * p.ag_world + r) * p.ag_tiles_per_rank + t;
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

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Copy CTAs of the fused all-gather -> GEMM kernels (the lowest block indices of the grid): pull the remote 128-row tiles
// of the gathered operand into the local gather buffer, next rank's shard first, and publish one flag per tile.  Whole
// rows travel as a ring of untiled bulk copies (peer memory -> shared memory -> local memory) driven by one thread;
// rows with a leading dimension larger than K go through registers.
template <int EB>
__device__ __forceinline__ void tp_copy_cta(const Params& p, uint8_t* smem_raw, int m_tiles, int n_copy_ctas) {
  const int cid = blockIdx.x, n_copy = n_copy_ctas;
  const int n_local = p.ag_batch * p.ag_tiles_per_rank;
  const int n_remote = m_tiles - n_local;
  const int row_bytes_i = p.K * EB;
  const int vec_per_row = row_bytes_i >> 4;
  const bool contiguous = p.ag_src_ld == p.K && row_bytes_i <= CP_CHUNK;   // whole rows per bulk chunk
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
    const int mt = ag_ordered_tile(p, n_local + idx);                   // rotated order: next rank's shard first
    int src_rank, src_row0;
    ag_tile_source(p, mt, src_rank, src_row0);
    const int rows = min(BM, p.M - mt * BM);
    if (contiguous) {
      // one thread drives a ring of bulk copies: peer memory -> shared -> local gather buffer
      if (threadIdx.x == 0) {
        const char* src = reinterpret_cast<const char*>(p.ag_src[src_rank] + (size_t)src_row0 * row_bytes_i);
        char* dst = reinterpret_cast<char*>(p.ag_dst + (size_t)mt * BM * row_bytes_i);
        const uint32_t row_bytes = (uint32_t)row_bytes_i;
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
      const uint4* src = reinterpret_cast<const uint4*>(p.ag_src[src_rank] + (size_t)src_row0 * p.ag_src_ld * EB);
      uint4* dst = reinterpret_cast<uint4*>(p.ag_dst + (size_t)mt * BM * row_bytes_i);
      const int total = rows * vec_per_row;
      const int src_ld8 = (p.ag_src_ld * EB) >> 4;
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
}

template <int B_MN, int EB>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA_local, const __grid_constant__ CUtensorMap tmA_gather,
               const __grid_constant__ CUtensorMap tmB, Params p) {
  extern __shared__ uint8_t smem_raw[];
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  constexpr int BKE = 128 / EB;                          // K elements per k-block (a shared-memory row is 128 bytes)
  constexpr int MNB = 128 / EB;                          // MN elements per 128-byte row of an MN-major box
  constexpr int MN_BOX_BYTES = BKE * 128;
  const int num_kb = (p.K + BKE - 1) / BKE;
  const bool ag = p.ag_world > 1;
  const int n_gemm = ag ? p.n_gemm_ctas : gridDim.x;
  const int n_copy_ctas = gridDim.x - n_gemm;            // copy CTAs take the lowest block indices: scheduled first
  const int gemm_id = (int)blockIdx.x - n_copy_ctas;

  if (ag && (int)blockIdx.x < n_copy_ctas) {
    tp_copy_cta<EB>(p, smem_raw, m_tiles, n_copy_ctas);
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
    mt = ag ? ag_ordered_tile(p, mr) : mr;
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = gemm_id; tile < num_tiles && ok; tile += n_gemm) {
        int mt, nt; coords(tile, mt, nt);
        const int n0 = nt * BN;
        int src_rank = 0, src_row0 = mt * BM;
        if (ag) ag_tile_source(p, mt, src_rank, src_row0);
        const bool local = !ag || src_rank == p.ag_me;
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
        const int m0 = (local && ag) ? src_row0 : mt * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES, b_dst = a_dst + A_STAGE;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const int k0 = kb * BKE;
          tma_load_2d(a_dst, tma, k0, m0, full_bar(stage));
          if (B_MN == 0) tma_load_2d(b_dst, &tmB, k0, n0, full_bar(stage));
          else {
#pragma unroll
            for (int j = 0; j < BN / MNB; ++j) tma_load_2d(b_dst + j * MN_BOX_BYTES, &tmB, n0 + MNB * j, k0, full_bar(stage));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { const unsigned long long t0 = globaltimer(); while (globaltimer() - t0 < 200000ull) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr int UK = 32 / EB;                       // K elements per MMA (32 bytes)
      const uint32_t idesc = EB == 2 ? umma_idesc_bf16(BM, BN, 0, B_MN) : umma_idesc_fp8(BM, BN, 0, B_MN, p.a_fmt, p.b_fmt);
      constexpr uint32_t b_lbo = B_MN ? (uint32_t)MN_BOX_BYTES : 16u, b_step = B_MN ? (UK * 128u) >> 4 : 2u;
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
          for (int k = 0; k < 4; ++k) {
            if (EB == 2) umma_bf16(d_tmem, adesc + k * 2, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_fp8(d_tmem, adesc + k * 2, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
          }
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
    const float alpha = (p.alpha ? p.alpha[0] : 1.f) * (p.alpha2 ? p.alpha2[0] : 1.f);
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
        const int row_w = mt * BM + q * 32;           // rows of one warp never straddle blocks (rows_per_block % 128 == 0)
        const int block = row_w / p.rs_rows_per_block, in_block = row_w - block * p.rs_rows_per_block;
        const int owner = block % p.rs_world, b = block / p.rs_world;
        const int ow = b < p.rs_batch ? owner : 0;
        const int lr = (b < p.rs_batch ? b : 0) * p.rs_rows_per_block + in_block;      // row in the owner's [batch * Ms, N] slot
        wbase = p.rs_dst[ow] + ((size_t)p.rs_me * p.rs_batch * p.rs_rows_per_block + lr) * p.N;
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
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]) * alpha, __uint_as_float(r[v * 8 + 2 * j + 1]) * alpha);
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
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]) * alpha;
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

// ------------------------------------------------------------------------------------ CTA-pair variant (cta_group::2)
// The same fused all-gather -> GEMM / GEMM -> reduce-scatter kernel on SM pairs: two CTAs of a cluster share one 256 x 256
// output tile (each stages 128 rows of A and 128 rows of B per k-block, six 32 KB stages; its TMEM holds the 128
// accumulator rows of its half), which removes a third of the shared-memory traffic per FLOP — the bound of the
// single-CTA kernel with one-byte operands.  Copy CTAs (an even number, lowest block indices) are unchanged and use no
// cluster feature; every GEMM CTA waits for the gather flag of its own 128-row half.  M % 256 == 0.
constexpr int TP_P_STAGES = 6, TP_P_STAGE_BYTES = 2 * 128 * 128;
constexpr int TP_P_SMEM_BYTES = TP_P_STAGES * TP_P_STAGE_BYTES + 1024 + 256 + EPI_BYTES;

template <int B_MN, int EB>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tp_pair_kernel(const __grid_constant__ CUtensorMap tmA_local, const __grid_constant__ CUtensorMap tmA_gather,
                    const __grid_constant__ CUtensorMap tmB, Params p) {
  extern __shared__ uint8_t smem_raw[];
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;      // m_tiles counts 128-row tiles
  const int m_tiles2 = m_tiles >> 1;
  const int num_tiles = m_tiles2 * n_tiles;
  constexpr int BKE = 128 / EB;
  constexpr int MNB = 128 / EB;
  constexpr int MN_BOX_BYTES = BKE * 128;
  const int num_kb = (p.K + BKE - 1) / BKE;
  const bool ag = p.ag_world > 1;
  const int n_gemm = ag ? p.n_gemm_ctas : gridDim.x;
  const int n_copy_ctas = gridDim.x - n_gemm;
  const int gemm_id = (int)blockIdx.x - n_copy_ctas;

  if (ag && (int)blockIdx.x < n_copy_ctas) {
    tp_copy_cta<EB>(p, smem_raw, m_tiles, n_copy_ctas);
    return;
  }

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + TP_P_STAGES * TP_P_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (TP_P_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * TP_P_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * TP_P_STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + TP_P_STAGES * TP_P_STAGE_BYTES + 8 * (2 * TP_P_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + TP_P_STAGES * TP_P_STAGE_BYTES + 8 * (2 * TP_P_STAGES + 4) + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = gemm_id >> 1, npairs = n_gemm >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_P_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA_local); prefetch_tmap(&tmA_gather); prefetch_tmap(&tmB);
  }
  if (warp == 1) { tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (this CTA's 128-row tile of the full row space, n tile): local shard first when A is being gathered
  auto coords = [&](int tile, int& mt, int& nt) {
    const int per_group = 8 * n_tiles;
    const int g = tile / per_group, first_m = g * 8;
    const int gsz = min(8, m_tiles2 - first_m);
    const int r = tile - g * per_group;
    const int mr2 = first_m + r % gsz;
    nt = r / gsz;
    const int idx = 2 * mr2 + (int)rank;
    mt = ag ? ag_ordered_tile(p, idx) : idx;
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        int mt, nt; coords(tile, mt, nt);
        const int n0 = nt * BN + (int)rank * 128;
        int src_rank = 0, src_row0 = mt * BM;
        if (ag) ag_tile_source(p, mt, src_rank, src_row0);
        const bool local = !ag || src_rank == p.ag_me;
        if (!local) {
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
        const int m0 = (local && ag) ? src_row0 : mt * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * TP_P_STAGE_BYTES, b_dst = a_dst + 128 * 128;
          const uint32_t bar = map_to_cta(full_bar(stage), 0);          // the even CTA counts both CTAs' bytes
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * TP_P_STAGE_BYTES);
          const int k0 = kb * BKE;
          tma_load_2d_pair(a_dst, tma, k0, m0, bar);
          if (B_MN == 0) tma_load_2d_pair(b_dst, &tmB, k0, n0, bar);
          else {
#pragma unroll
            for (int j = 0; j < 128 / MNB; ++j) tma_load_2d_pair(b_dst + j * MN_BOX_BYTES, &tmB, n0 + MNB * j, k0, bar);
          }
          if (++stage == TP_P_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { const unsigned long long t0 = globaltimer(); while (globaltimer() - t0 < 200000ull) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr int UK = 32 / EB;
      const uint32_t idesc = EB == 2 ? umma_idesc_bf16(256, BN, 0, B_MN) : umma_idesc_fp8(256, BN, 0, B_MN, p.a_fmt, p.b_fmt);
      constexpr uint32_t b_lbo = B_MN ? (uint32_t)MN_BOX_BYTES : 16u, b_step = B_MN ? (UK * 128u) >> 4 : 2u;
      int stage = 0; uint32_t phase = 0; uint32_t acc_phase[2] = {0u, 0u}; int local = 0; bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local) {
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        acc_phase[acc] ^= 1u;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * TP_P_STAGE_BYTES;
          const uint64_t adesc = umma_smem_desc(a_addr, 16u, 1024u);
          const uint64_t bdesc = umma_smem_desc(a_addr + 128 * 128, b_lbo, 1024u);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (EB == 2) umma_bf16_pair(d_tmem, adesc + k * 2, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_fp8_pair(d_tmem, adesc + k * 2, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));
          if (++stage == TP_P_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(acc));
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t acc_phase[2] = {0u, 0u}; int local = 0; bool ok = true;
    const bool rs = p.rs_world > 1;
    const float alpha = (p.alpha ? p.alpha[0] : 1.f) * (p.alpha2 ? p.alpha2[0] : 1.f);
    for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++local) {
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
      __nv_bfloat16* wbase = nullptr;
      if (rs) {
        const int row_w = mt * BM + q * 32;
        const int block = row_w / p.rs_rows_per_block, in_block = row_w - block * p.rs_rows_per_block;
        const int owner = block % p.rs_world, b = block / p.rs_world;
        const int ow = b < p.rs_batch ? owner : 0;
        const int lr = (b < p.rs_batch ? b : 0) * p.rs_rows_per_block + in_block;
        wbase = p.rs_dst[ow] + ((size_t)p.rs_me * p.rs_batch * p.rs_rows_per_block + lr) * p.N;
        crow = wbase + (size_t)lane * p.N;
        staged = ow != p.rs_me;
      } else {
        crow = p.C + (size_t)row * p.ldc;
      }
      __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem_gen + TP_P_STAGES * TP_P_STAGE_BYTES + 256) + q * 32 * EPI_LD;
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
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]) * alpha, __uint_as_float(r[v * 8 + 2 * j + 1]) * alpha);
            *reinterpret_cast<uint4*>(srow + v * 8) = out;
          }
          if (c & 1) {
            __syncwarp();
            const int cbase = n0 + (c - 1) * 32;
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
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]) * alpha;
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
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TMEM_COLS); }
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

// Plain peer gather (used where the gathered operand feeds a reduction dim: weight gradients): the full
// [batch, world, Ms, K] row space from the ranks' shards [batch * Ms, K]; `row16` = 16-byte vectors per row.
__global__ void gather_rows_kernel(Params p, int row16, int src_ld16) {
  const size_t total = (size_t)p.M * row16;
  const int rows_per_block = p.ag_tiles_per_rank * BM;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / row16; const int c = idx - r * row16;
    const int block = r / rows_per_block, in_block = r - (size_t)block * rows_per_block;
    const int src = block % p.ag_world, bb = block / p.ag_world;
    const size_t lr = (size_t)bb * rows_per_block + in_block;
    reinterpret_cast<uint4*>(p.ag_dst)[idx] = reinterpret_cast<const uint4*>(p.ag_src[src])[lr * src_ld16 + c];
  }
}

}  // namespace tp
}  // namespace sb

using namespace sb;
using namespace sb::tp;

// Fused projection.  A: own shard [batch * Ms, K] (leading dim lda) when ag_world > 1, else the full [M, K].  B: [N, K]
// (b_mn = 0) or [K, N] (b_mn = 1).  elem_bytes: 2 = bf16 operands, 1 = fp8 (a_fmt / b_fmt: 0 = e4m3, 1 = e5m2; the result
// is multiplied by alpha[0] * alpha2[0], device scalars, either may be null).  ag_src: `ag_world` shard base pointers
// (index = rank; entry `ag_me` = A); gather: local workspace [M, K]; flags: [ceil(M/128)] ints (any contents; `epoch` must
// differ from the previous call's on the same flags).  The full row space is [batch, world, Ms]: row block (b, r) is rank
// r's.  rs_dst: `rs_world` staging base pointers [rs_world, batch * M / (batch * rs_world), N]; with rs_world <= 1 the
// result goes to C (ldc) with optional bias.
static int g_tp_pair = 0;   // 1: run the CTA-pair variant where its shape conditions hold
extern "C" int sb_gemm_tp_set_pair(int on) { g_tp_pair = on ? 1 : 0; return 0; }

extern "C" int sb_gemm_tp(const void* A, int lda, const void* B, int ldb, int b_mn, void* C, int ldc, const void* bias,
                          int M, int N, int K, int batch, int elem_bytes, const float* alpha, const float* alpha2, int a_fmt,
                          int b_fmt, int ag_world, int ag_me, const void* const* ag_src, void* gather, int* flags, int epoch,
                          int n_copy_ctas, int rs_world, int rs_me, void* const* rs_dst, unsigned int* status,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int EBv = elem_bytes == 1 ? 1 : 2;
  const int al = 16 / EBv;                                  // elements per 16 bytes
  if ((N % 8) || (K % al) || (lda % al) || (ldb % al) || batch < 1 || (M % batch)) return -3;
  if (EBv == 1 && b_mn && (N % 16)) return -3;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias; p.status = status;
  p.alpha = alpha; p.alpha2 = alpha2; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  const bool ag = ag_world > 1, rs = rs_world > 1;
  const uint32_t bke = 128 / EBv;
  auto tmap = [&](CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t bi, uint32_t bo) {
    return EBv == 2 ? make_tmap_2d_bf16(out, base, inner, outer, ld, bi, bo) : make_tmap_2d_u8(out, base, inner, outer, ld, bi, bo);
  };
  CUtensorMap tmL, tmG, tmB;
  int rc;
  if (ag) {
    if (ag_world > MAXR || (M % (ag_world * batch)) || ((M / (ag_world * batch)) % BM)) return -7;
    const int Ms = M / (ag_world * batch);
    p.ag_world = ag_world; p.ag_me = ag_me; p.ag_tiles_per_rank = Ms / BM; p.ag_batch = batch; p.ag_epoch = epoch;
    p.ag_flags = flags;
    for (int r = 0; r < ag_world; ++r) p.ag_src[r] = (const uint8_t*)ag_src[r];
    p.ag_src_ld = lda; p.ag_dst = (uint8_t*)gather;
    if ((rc = tmap(&tmL, A, K, (uint64_t)Ms * batch, lda, bke, BM))) return rc;
    if ((rc = tmap(&tmG, gather, K, M, K, bke, BM))) return rc;
  } else {
    if ((rc = tmap(&tmL, A, K, M, lda, bke, BM))) return rc;
    tmG = tmL;
  }
  if (!b_mn) rc = tmap(&tmB, B, K, N, ldb, bke, BN);
  else       rc = tmap(&tmB, B, N, K, ldb, bke, bke);
  if (rc) return rc;
  if (rs) {
    if (rs_world > MAXR || (M % (rs_world * batch)) || ((M / (rs_world * batch)) % BM)) return -8;
    p.rs_world = rs_world; p.rs_me = rs_me; p.rs_rows_per_block = M / (rs_world * batch); p.rs_batch = batch;
    for (int r = 0; r < rs_world; ++r) p.rs_dst[r] = (__nv_bfloat16*)rs_dst[r];
  } else if (ldc % 8) return -3;
  const int sms = sb::num_sms();
  if (g_tp_pair && M % 256 == 0 && (!ag || (p.ag_tiles_per_rank % 2 == 0)) && (!rs || p.rs_rows_per_block % 256 == 0)) {
    // CTA pairs: B boxes of 128 rows per CTA, an even number of copy CTAs, clusters of two
    if (!b_mn && (rc = tmap(&tmB, B, K, N, ldb, bke, 128))) return rc;
    int n_copy = ag ? (n_copy_ctas > 0 ? n_copy_ctas : 16) : 0;
    n_copy += n_copy & 1;
    const int tiles2 = (M / 256) * ((N + BN - 1) / BN);
    int pairs = (sms - n_copy) / 2;
    if (tiles2 < pairs) pairs = tiles2;
    p.n_gemm_ctas = 2 * pairs;
    void (*kp)(const CUtensorMap, const CUtensorMap, const CUtensorMap, Params);
    if (EBv == 2) kp = b_mn ? gemm_tp_pair_kernel<1, 2> : gemm_tp_pair_kernel<0, 2>;
    else          kp = b_mn ? gemm_tp_pair_kernel<1, 1> : gemm_tp_pair_kernel<0, 1>;
    static bool pattr[4] = {false, false, false, false};
    const int pi = (EBv == 1 ? 2 : 0) + (b_mn ? 1 : 0);
    if (!pattr[pi]) {
      if (cudaFuncSetAttribute(kp, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_P_SMEM_BYTES) != cudaSuccess) return -5;
      pattr[pi] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs + n_copy);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = TP_P_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kp, tmL, tmG, tmB, p) == cudaSuccess ? 0 : -6;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int n_copy = ag ? (n_copy_ctas > 0 ? n_copy_ctas : 16) : 0;
  int n_gemm = sms - n_copy;
  if (tiles < n_gemm) n_gemm = tiles;
  p.n_gemm_ctas = n_gemm;
  void (*kern)(const CUtensorMap, const CUtensorMap, const CUtensorMap, Params);
  if (EBv == 2) kern = b_mn ? gemm_tp_kernel<1, 2> : gemm_tp_kernel<0, 2>;
  else          kern = b_mn ? gemm_tp_kernel<1, 1> : gemm_tp_kernel<0, 1>;
  static bool attr_set[4] = {false, false, false, false};
  const int ai = (EBv == 1 ? 2 : 0) + (b_mn ? 1 : 0);
  if (!attr_set[ai]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -5;
    attr_set[ai] = true;
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

// gather[M, K] <- the full [batch, world, Ms] row space from src[r] = rank r's shard [batch * Ms, K] (leading dim ld);
// elem_bytes = 2 (bf16) or 1 (fp8)
extern "C" int sb_gather_rows(const void* const* src, int world, void* gather, int M, int K, int ld, int batch, int elem_bytes,
                              cudaStream_t stream) {
  const int EBv = elem_bytes == 1 ? 1 : 2, al = 16 / EBv;
  if ((K % al) || (ld % al) || world > MAXR || batch < 1 || (M % (world * batch)) || ((M / (world * batch)) % BM)) return -1;
  Params p{};
  p.M = M; p.K = K; p.ag_world = world; p.ag_batch = batch; p.ag_tiles_per_rank = (M / (world * batch)) / BM;
  p.ag_dst = (uint8_t*)gather;
  for (int r = 0; r < world; ++r) p.ag_src[r] = (const uint8_t*)src[r];
  gather_rows_kernel<<<sb::num_sms() * 4, 512, 0, stream>>>(p, K * EBv / 16, ld * EBv / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
