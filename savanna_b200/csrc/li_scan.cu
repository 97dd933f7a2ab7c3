// Hyena-LI with the implicit modal filter, evaluated as what it is: an order-O diagonal linear recurrence.
//
//   h[d,t] = sum_o R[d,o] lam[d,o]^t          =>   s_o[t] = lam_o s_o[t-1] + u[t],   y[t] = sum_o R_o s_o[t] + bias u[t]
//   u = x2 * v,  z = x1 * y                        (features interleaved (x1,x2,v), channel-last bf16, fp32 state)
//
// The sequence is cut into chunks of TC steps that run in parallel (chunked scan):
//   1. local   : every chunk runs from a zero state and stores its end state          [B, NC, D, O]
//   2. prefix  : per (b, d, o) a serial pass over the NC chunk states turns them into the state ENTERING each chunk
//   3. apply   : every chunk reruns from its entering state and writes z
// so the cost is two streaming reads of the features and one write of z, instead of the size-2L fp32 FFTs the
// filter's materialised form needs.  The backward pass uses the same structure twice: a forward scan that
// carries the state s and its sensitivity w = ds/dlam (gradients of R, lam, bias and dx1), and a reverse scan of
// the adjoint a[t] = R dy[t] + lam a[t+1] (gradients of x2 and v).  `state_in` / `state_out` expose the recurrence
// state at the shard boundaries, which is all context parallelism needs to hand over.
//
// One thread owns one channel (its O states live in registers); a warp reads 32 channels x 3 features = 192
// contiguous bytes per time step.  O is padded to 16 (lam = 0, R = 0 beyond the real order).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {
typedef __nv_bfloat16 bf16;
constexpr int LO = 16;            // padded filter order
constexpr int LI_THREADS = 128;

__device__ __forceinline__ float b2f(const bf16 v) { return __bfloat162float(v); }

struct LiDims { int B, L, D, TC, NC; };

__device__ __forceinline__ void load_vec16(const float* p, float (&r)[LO]) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < LO / 4; ++i) { float4 t = q[i]; r[4 * i] = t.x; r[4 * i + 1] = t.y; r[4 * i + 2] = t.z; r[4 * i + 3] = t.w; }
}
__device__ __forceinline__ void store_vec16(float* p, const float (&r)[LO]) {
  float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
  for (int i = 0; i < LO / 4; ++i) q[i] = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
}

// ------------------------------------------------------------------------------------ forward
// pass 1: chunk-local end state from a zero state
__global__ void __launch_bounds__(LI_THREADS)
li_local_kernel(const bf16* __restrict__ feat, const float* __restrict__ loglam, float* __restrict__ Sloc, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = __expf(lam[o]); s[o] = 0.f; }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = feat + ((size_t)b * d.L + t0) * 3 * d.D + 3 * ch;
#pragma unroll 8
  for (int t = t0; t < t1; ++t, f += 3 * d.D) {
    const float u = b2f(f[1]) * b2f(f[2]);
#pragma unroll
    for (int o = 0; o < LO; ++o) s[o] = lam[o] * s[o] + u;
  }
  store_vec16(Sloc + (((size_t)b * d.NC + n) * d.D + ch) * LO, s);
}

// pass 2: exclusive prefix over chunks, in place: S[n] <- state entering chunk n.  One thread per (b, ch, o).
// Chunks are full (TC steps) except possibly the last one, whose end state only feeds state_out.
__global__ void li_prefix_kernel(float* __restrict__ S, const float* __restrict__ loglam, const float* __restrict__ state_in,
                                 float* __restrict__ state_out, LiDims d) {
  const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t per_b = (size_t)d.D * LO;
  if (idx >= (size_t)d.B * per_b) return;
  const int b = idx / per_b;
  const size_t r = idx - (size_t)b * per_b;               // ch * LO + o
  const float ll = loglam[r];
  const float step = __expf(ll * d.TC);
  float carry = state_in ? state_in[idx] : 0.f;
  float* p = S + (size_t)b * d.NC * per_b + r;
  // the chunk states are independent loads: fetch eight ahead, then run the serial carry over them
  for (int n0 = 0; n0 < d.NC; n0 += 8) {
    float loc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) loc[j] = n0 + j < d.NC ? p[(size_t)(n0 + j) * per_b] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j;
      if (n < d.NC) {
        p[(size_t)n * per_b] = carry;
        const int len = min(d.TC, d.L - n * d.TC);
        const float st = len == d.TC ? step : __expf(ll * len);
        carry = st * carry + loc[j];
      }
    }
  }
  if (state_out) state_out[idx] = carry;
}

// pass 3: rerun each chunk from its entering state and emit z
__global__ void __launch_bounds__(LI_THREADS)
li_apply_kernel(const bf16* __restrict__ feat, const float* __restrict__ loglam, const float* __restrict__ R,
                const float* __restrict__ bias, const float* __restrict__ Sin, bf16* __restrict__ z, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO], rr[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
  load_vec16(R + (size_t)ch * LO, rr);
  load_vec16(Sin + (((size_t)b * d.NC + n) * d.D + ch) * LO, s);
#pragma unroll
  for (int o = 0; o < LO; ++o) lam[o] = __expf(lam[o]);
  const float be = bias[ch];
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = feat + ((size_t)b * d.L + t0) * 3 * d.D + 3 * ch;
  bf16* zo = z + ((size_t)b * d.L + t0) * d.D + ch;
#pragma unroll 8
  for (int t = t0; t < t1; ++t, f += 3 * d.D, zo += d.D) {
    const float x1 = b2f(f[0]);
    const float u = b2f(f[1]) * b2f(f[2]);
    float y = be * u;
#pragma unroll
    for (int o = 0; o < LO; ++o) { s[o] = lam[o] * s[o] + u; y += rr[o] * s[o]; }
    *zo = __float2bfloat16_rn(x1 * y);
  }
}

// ------------------------------------------------------------------------------------ backward
// pass B1: chunk-local quantities from zero states:
//   Sloc  end state;  Wloc end sensitivity (w[t] = s[t-1] + lam w[t-1]);
//   Aloc  adjoint leaving the chunk on its left edge: sum_t lam^(t-t0) R dy[t], dy = dz * x1
__global__ void __launch_bounds__(LI_THREADS)
li_bwd_local_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ dz, const float* __restrict__ loglam,
                    const float* __restrict__ R, float* __restrict__ Sloc, float* __restrict__ Wloc,
                    float* __restrict__ Aloc, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO], w[LO], pw[LO], a[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = __expf(lam[o]); s[o] = 0.f; w[o] = 0.f; pw[o] = 1.f; a[o] = 0.f; }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = feat + ((size_t)b * d.L + t0) * 3 * d.D + 3 * ch;
  const bf16* g = dz + ((size_t)b * d.L + t0) * d.D + ch;
#pragma unroll 4
  for (int t = t0; t < t1; ++t, f += 3 * d.D, g += d.D) {
    const float u = b2f(f[1]) * b2f(f[2]);
    const float dy = b2f(*g) * b2f(f[0]);
#pragma unroll
    for (int o = 0; o < LO; ++o) {
      w[o] = s[o] + lam[o] * w[o];
      s[o] = lam[o] * s[o] + u;
      a[o] += pw[o] * dy;
      pw[o] *= lam[o];
    }
  }
  float rr[LO];
  load_vec16(R + (size_t)ch * LO, rr);
#pragma unroll
  for (int o = 0; o < LO; ++o) a[o] *= rr[o];
  const size_t off = (((size_t)b * d.NC + n) * d.D + ch) * LO;
  store_vec16(Sloc + off, s);
  store_vec16(Wloc + off, w);
  store_vec16(Aloc + off, a);
}

// pass B2: (S, W) exclusive prefix (forward), A exclusive suffix (reverse), in place.
//   S_in[n+1] = lam^len S_in[n] + Sloc[n]
//   W_in[n+1] = lam^len W_in[n] + len lam^(len-1) S_in[n] + Wloc[n]
//   A_in[n-1] = lam^len(n) A_in[n] + Aloc[n]          (A_in[n] = adjoint at the right edge of chunk n)
// Also: w_end (sensitivity of the final state), dstate_in = lam * (adjoint at t = 0).
__global__ void li_bwd_prefix_kernel(float* __restrict__ S, float* __restrict__ W, float* __restrict__ A,
                                     const float* __restrict__ loglam, const float* __restrict__ state_in,
                                     const float* __restrict__ dstate_out, float* __restrict__ w_end,
                                     float* __restrict__ dstate_in, LiDims d) {
  const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t per_b = (size_t)d.D * LO;
  if (idx >= (size_t)d.B * per_b) return;
  const int b = idx / per_b;
  const size_t r = idx - (size_t)b * per_b;
  const float ll = loglam[r];
  const size_t base = (size_t)b * d.NC * per_b + r;
  float cs = state_in ? state_in[idx] : 0.f, cw = 0.f;
  const float st_full = __expf(ll * d.TC), stm1_full = __expf(ll * (d.TC - 1));
  // independent loads of eight chunks ahead of the serial carries (forward for S and W, backward for A)
  for (int n0 = 0; n0 < d.NC; n0 += 8) {
    float ls[8], lw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const size_t o = base + (size_t)(n0 + j) * per_b;
      ls[j] = n0 + j < d.NC ? S[o] : 0.f;
      lw[j] = n0 + j < d.NC ? W[o] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j;
      if (n < d.NC) {
        const size_t o = base + (size_t)n * per_b;
        S[o] = cs; W[o] = cw;
        const int len = min(d.TC, d.L - n * d.TC);
        const float st = len == d.TC ? st_full : __expf(ll * len);
        const float stm1 = len == d.TC ? stm1_full : __expf(ll * (len - 1));
        cw = st * cw + len * stm1 * cs + lw[j];
        cs = st * cs + ls[j];
      }
    }
  }
  if (w_end) w_end[idx] = cw;
  // The gradient of the returned state, g = dL/ds[L-1], enters the adjoint at the LAST step without a factor lam
  // (a[L-1] = R dy[L-1] + g): the last chunk therefore starts from a zero adjoint, the reverse kernel adds g at its first
  // step, and the carry into the chunk before it picks up lam^(len-1) g.
  const float gout = dstate_out ? dstate_out[idx] : 0.f;
  float ca = 0.f;
  for (int n0 = d.NC - 1; n0 >= 0; n0 -= 8) {
    float la[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) la[j] = n0 - j >= 0 ? A[base + (size_t)(n0 - j) * per_b] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 - j;
      if (n >= 0) {
        A[base + (size_t)n * per_b] = ca;
        const int len = min(d.TC, d.L - n * d.TC);
        ca = (len == d.TC ? st_full : __expf(ll * len)) * ca + la[j];
        if (n == d.NC - 1 && gout != 0.f) ca += (len == d.TC ? stm1_full : __expf(ll * (len - 1))) * gout;
      }
    }
  }
  if (dstate_in) dstate_in[idx] = __expf(ll) * ca;
}

// pass B3 (forward direction): y, dx1 = dz*y (into tmp), and per-chunk partial sums of dR, dlam, dbias
__global__ void __launch_bounds__(LI_THREADS)
li_bwd_apply_fwd_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ dz, const float* __restrict__ loglam,
                        const float* __restrict__ R, const float* __restrict__ bias, const float* __restrict__ Sin,
                        const float* __restrict__ Win, bf16* __restrict__ dx1, float* __restrict__ dRp,
                        float* __restrict__ dLp, float* __restrict__ dBp, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO], w[LO], rr[LO], dr[LO], dl[LO];
  const size_t off = (((size_t)b * d.NC + n) * d.D + ch) * LO;
  load_vec16(loglam + (size_t)ch * LO, lam);
  load_vec16(R + (size_t)ch * LO, rr);
  load_vec16(Sin + off, s);
  load_vec16(Win + off, w);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = __expf(lam[o]); dr[o] = 0.f; dl[o] = 0.f; }
  const float be = bias[ch];
  float db = 0.f;
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = feat + ((size_t)b * d.L + t0) * 3 * d.D + 3 * ch;
  const bf16* g = dz + ((size_t)b * d.L + t0) * d.D + ch;
  bf16* o1 = dx1 + ((size_t)b * d.L + t0) * d.D + ch;
#pragma unroll 4
  for (int t = t0; t < t1; ++t, f += 3 * d.D, g += d.D, o1 += d.D) {
    const float x1 = b2f(f[0]);
    const float u = b2f(f[1]) * b2f(f[2]);
    const float gz = b2f(*g);
    const float dy = gz * x1;
    float y = be * u;
#pragma unroll
    for (int o = 0; o < LO; ++o) {
      w[o] = s[o] + lam[o] * w[o];
      s[o] = lam[o] * s[o] + u;
      y += rr[o] * s[o];
      dr[o] += dy * s[o];
      dl[o] += dy * w[o];
    }
    db += dy * u;
    *o1 = __float2bfloat16_rn(gz * y);
  }
#pragma unroll
  for (int o = 0; o < LO; ++o) dl[o] *= rr[o];
  store_vec16(dRp + off, dr);
  store_vec16(dLp + off, dl);
  dBp[((size_t)b * d.NC + n) * d.D + ch] = db;
}

// pass R3 (reverse direction): adjoint scan, writes the full interleaved gradient (dx1 from tmp)
__global__ void __launch_bounds__(LI_THREADS)
li_bwd_apply_rev_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ dz, const float* __restrict__ loglam,
                        const float* __restrict__ R, const float* __restrict__ bias, const float* __restrict__ Ain,
                        const bf16* __restrict__ dx1, bf16* __restrict__ dfeat, const float* __restrict__ dstate_out,
                        LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], a[LO], rr[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
  load_vec16(R + (size_t)ch * LO, rr);
  load_vec16(Ain + (((size_t)b * d.NC + n) * d.D + ch) * LO, a);
#pragma unroll
  for (int o = 0; o < LO; ++o) lam[o] = __expf(lam[o]);
  const float be = bias[ch];
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = feat + ((size_t)b * d.L + (t1 - 1)) * 3 * d.D + 3 * ch;
  const bf16* g = dz + ((size_t)b * d.L + (t1 - 1)) * d.D + ch;
  const bf16* i1 = dx1 + ((size_t)b * d.L + (t1 - 1)) * d.D + ch;
  bf16* df = dfeat + ((size_t)b * d.L + (t1 - 1)) * 3 * d.D + 3 * ch;
  const bool tail = dstate_out != nullptr && n == d.NC - 1;       // the chunk that ends the sequence: see li_bwd_prefix_kernel
  float gs[LO];
  if (tail) load_vec16(dstate_out + ((size_t)b * d.D + ch) * LO, gs);
#pragma unroll 8
  for (int t = t1 - 1; t >= t0; --t, f -= 3 * d.D, g -= d.D, i1 -= d.D, df -= 3 * d.D) {
    const float x1 = b2f(f[0]), x2 = b2f(f[1]), v = b2f(f[2]);
    const float dy = b2f(*g) * x1;
    float du = be * dy;
#pragma unroll
    for (int o = 0; o < LO; ++o) { a[o] = rr[o] * dy + lam[o] * a[o]; }
    if (tail && t == t1 - 1) {
#pragma unroll
      for (int o = 0; o < LO; ++o) a[o] += gs[o];
    }
#pragma unroll
    for (int o = 0; o < LO; ++o) du += a[o];
    df[0] = *i1;
    df[1] = __float2bfloat16_rn(du * v);
    df[2] = __float2bfloat16_rn(du * x2);
  }
}

// ------------------------------------------------------------------------------------ tiled kernels
// The kernels above walk the sequence with 2-byte loads at a stride of a whole row: a warp moves 192 useful bytes per
// step with 96 load instructions, and the time loop waits on them.  The tiled kernels below (D % 8 == 0) stage
// [rows x 128 channels] tiles of the interleaved features in shared memory with 16-byte asynchronous copies that are all
// in flight at once, run the recurrences out of shared memory, and store their outputs as 16-byte chunks.
//   forward   local / apply: sub-tiles of LT_ROWS steps, double buffered, any chunk length that is a multiple of LT_ROWS
//   backward  one kernel per chunk of LB_TC steps holds the chunk's features, dz and dx1 in shared memory: the forward
//             sweep (state, sensitivity: y, dx1, filter-gradient partials) and the reverse sweep (adjoint: du) run back
//             to back, so dx1 never goes through global memory and the chunk is read once.
constexpr int LT_ROWS = 16, LT_CH = 128;
constexpr int LB_TC = 64;

__device__ __forceinline__ void li_cp_async16(void* smem_dst, const void* src, int nbytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(nbytes) : "memory");
}
__device__ __forceinline__ void li_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void li_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Stage `rows` feature rows starting at time t_lo (rows beyond t_hi are zero-filled) for channels [c0, c0 + 128) into
// tile[rows][3 * 128]; chunks of 8 bf16.  `ncv` = number of valid 16-byte chunks per row (channels beyond D: zeros).
__device__ __forceinline__ void li_stage_feat(bf16 (*tile)[3 * LT_CH], const bf16* feat_b, int t_lo, int t_hi, int rows, int c0,
                                              int D, int tid, int nthreads) {
  constexpr int CHK = 3 * LT_CH / 8;                        // 48 chunks per row
  const int ncv = min(CHK, (3 * (D - c0)) / 8);
  for (int idx = tid; idx < rows * CHK; idx += nthreads) {
    const int r = idx / CHK, ch = idx - r * CHK, t = t_lo + r;
    const bool ok = t < t_hi && ch < ncv;
    const bf16* src = ok ? feat_b + (size_t)t * 3 * D + 3 * c0 + ch * 8 : feat_b;
    li_cp_async16(&tile[r][ch * 8], src, ok ? 16 : 0);
  }
}
__device__ __forceinline__ void li_stage_d(bf16 (*tile)[LT_CH], const bf16* g_b, int t_lo, int t_hi, int rows, int c0, int D,
                                           int tid, int nthreads) {
  constexpr int CHK = LT_CH / 8;                            // 16 chunks per row
  const int ncv = min(CHK, (D - c0) / 8);
  for (int idx = tid; idx < rows * CHK; idx += nthreads) {
    const int r = idx / CHK, ch = idx - r * CHK, t = t_lo + r;
    const bool ok = t < t_hi && ch < ncv;
    const bf16* src = ok ? g_b + (size_t)t * D + c0 + ch * 8 : g_b;
    li_cp_async16(&tile[r][ch * 8], src, ok ? 16 : 0);
  }
}

// pass 1 (tiled): chunk-local end state from a zero state
__global__ void __launch_bounds__(LT_CH)
li_local_tiled_kernel(const bf16* __restrict__ feat, const float* __restrict__ loglam, float* __restrict__ Sloc, LiDims d) {
  __shared__ __align__(16) bf16 fS[2][LT_ROWS][3 * LT_CH];
  const int tid = threadIdx.x, c0 = blockIdx.x * LT_CH, ch = c0 + tid;
  const int n = blockIdx.y, b = blockIdx.z;
  const bool live = ch < d.D;
  float lam[LO], s[LO];
  if (live) load_vec16(loglam + (size_t)ch * LO, lam);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = live ? __expf(lam[o]) : 0.f; s[o] = 0.f; }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* fb = feat + (size_t)b * d.L * 3 * d.D;
  const int ntile = (t1 - t0 + LT_ROWS - 1) / LT_ROWS;
  li_stage_feat(fS[0], fb, t0, t1, LT_ROWS, c0, d.D, tid, LT_CH);
  li_cp_commit();
  for (int k = 0; k < ntile; ++k) {
    if (k + 1 < ntile) li_stage_feat(fS[(k + 1) & 1], fb, t0 + (k + 1) * LT_ROWS, t1, LT_ROWS, c0, d.D, tid, LT_CH);
    li_cp_commit();
    li_cp_wait<1>();
    __syncthreads();
    const bf16 (*T)[3 * LT_CH] = fS[k & 1];
    const int rows = min(LT_ROWS, t1 - (t0 + k * LT_ROWS));
#pragma unroll 8
    for (int r = 0; r < rows; ++r) {
      const float u = b2f(T[r][3 * tid + 1]) * b2f(T[r][3 * tid + 2]);
#pragma unroll
      for (int o = 0; o < LO; ++o) s[o] = lam[o] * s[o] + u;
    }
    __syncthreads();                                        // the buffer is refilled two iterations from now
  }
  if (live) store_vec16(Sloc + (((size_t)b * d.NC + n) * d.D + ch) * LO, s);
}

// pass 3 (tiled): rerun each chunk from its entering state and emit z through a staged tile
__global__ void __launch_bounds__(LT_CH)
li_apply_tiled_kernel(const bf16* __restrict__ feat, const float* __restrict__ loglam, const float* __restrict__ R,
                      const float* __restrict__ bias, const float* __restrict__ Sin, bf16* __restrict__ z, LiDims d) {
  __shared__ __align__(16) bf16 fS[2][LT_ROWS][3 * LT_CH];
  __shared__ __align__(16) bf16 zS[LT_ROWS][LT_CH];
  const int tid = threadIdx.x, c0 = blockIdx.x * LT_CH, ch = c0 + tid;
  const int n = blockIdx.y, b = blockIdx.z;
  const bool live = ch < d.D;
  float lam[LO], s[LO], rr[LO];
  float be = 0.f;
  if (live) {
    load_vec16(loglam + (size_t)ch * LO, lam);
    load_vec16(R + (size_t)ch * LO, rr);
    load_vec16(Sin + (((size_t)b * d.NC + n) * d.D + ch) * LO, s);
    be = bias[ch];
  }
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = live ? __expf(lam[o]) : 0.f; if (!live) { s[o] = 0.f; rr[o] = 0.f; } }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* fb = feat + (size_t)b * d.L * 3 * d.D;
  bf16* zb = z + (size_t)b * d.L * d.D;
  const int ntile = (t1 - t0 + LT_ROWS - 1) / LT_ROWS;
  const int zcv = min(LT_CH / 8, (d.D - c0) / 8);
  li_stage_feat(fS[0], fb, t0, t1, LT_ROWS, c0, d.D, tid, LT_CH);
  li_cp_commit();
  for (int k = 0; k < ntile; ++k) {
    if (k + 1 < ntile) li_stage_feat(fS[(k + 1) & 1], fb, t0 + (k + 1) * LT_ROWS, t1, LT_ROWS, c0, d.D, tid, LT_CH);
    li_cp_commit();
    li_cp_wait<1>();
    __syncthreads();
    const bf16 (*T)[3 * LT_CH] = fS[k & 1];
    const int tt = t0 + k * LT_ROWS, rows = min(LT_ROWS, t1 - tt);
#pragma unroll 8
    for (int r = 0; r < rows; ++r) {
      const float x1 = b2f(T[r][3 * tid]);
      const float u = b2f(T[r][3 * tid + 1]) * b2f(T[r][3 * tid + 2]);
      float y = be * u;
#pragma unroll
      for (int o = 0; o < LO; ++o) { s[o] = lam[o] * s[o] + u; y += rr[o] * s[o]; }
      zS[r][tid] = __float2bfloat16_rn(x1 * y);
    }
    __syncthreads();
    for (int idx = tid; idx < rows * (LT_CH / 8); idx += LT_CH) {
      const int r = idx / (LT_CH / 8), cv = idx - r * (LT_CH / 8);
      if (cv < zcv) *reinterpret_cast<uint4*>(zb + (size_t)(tt + r) * d.D + c0 + cv * 8) = *reinterpret_cast<const uint4*>(&zS[r][cv * 8]);
    }
    __syncthreads();
  }
}

// backward pass B1 (tiled): Sloc, Wloc, Aloc of a chunk (see li_bwd_local_kernel)
__global__ void __launch_bounds__(LT_CH)
li_bwd_local_tiled_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ dz, const float* __restrict__ loglam,
                          const float* __restrict__ R, float* __restrict__ Sloc, float* __restrict__ Wloc,
                          float* __restrict__ Aloc, LiDims d) {
  __shared__ __align__(16) bf16 fS[2][LT_ROWS][3 * LT_CH];
  __shared__ __align__(16) bf16 gS[2][LT_ROWS][LT_CH];
  const int tid = threadIdx.x, c0 = blockIdx.x * LT_CH, ch = c0 + tid;
  const int n = blockIdx.y, b = blockIdx.z;
  const bool live = ch < d.D;
  float lam[LO], s[LO], w[LO], pw[LO], a[LO];
  if (live) load_vec16(loglam + (size_t)ch * LO, lam);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = live ? __expf(lam[o]) : 0.f; s[o] = 0.f; w[o] = 0.f; pw[o] = 1.f; a[o] = 0.f; }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* fb = feat + (size_t)b * d.L * 3 * d.D;
  const bf16* gb = dz + (size_t)b * d.L * d.D;
  const int ntile = (t1 - t0 + LT_ROWS - 1) / LT_ROWS;
  li_stage_feat(fS[0], fb, t0, t1, LT_ROWS, c0, d.D, tid, LT_CH);
  li_stage_d(gS[0], gb, t0, t1, LT_ROWS, c0, d.D, tid, LT_CH);
  li_cp_commit();
  for (int k = 0; k < ntile; ++k) {
    if (k + 1 < ntile) {
      li_stage_feat(fS[(k + 1) & 1], fb, t0 + (k + 1) * LT_ROWS, t1, LT_ROWS, c0, d.D, tid, LT_CH);
      li_stage_d(gS[(k + 1) & 1], gb, t0 + (k + 1) * LT_ROWS, t1, LT_ROWS, c0, d.D, tid, LT_CH);
    }
    li_cp_commit();
    li_cp_wait<1>();
    __syncthreads();
    const bf16 (*T)[3 * LT_CH] = fS[k & 1];
    const bf16 (*G)[LT_CH] = gS[k & 1];
    const int rows = min(LT_ROWS, t1 - (t0 + k * LT_ROWS));
#pragma unroll 4
    for (int r = 0; r < rows; ++r) {
      const float u = b2f(T[r][3 * tid + 1]) * b2f(T[r][3 * tid + 2]);
      const float dy = b2f(G[r][tid]) * b2f(T[r][3 * tid]);
#pragma unroll
      for (int o = 0; o < LO; ++o) {
        w[o] = s[o] + lam[o] * w[o];
        s[o] = lam[o] * s[o] + u;
        a[o] += pw[o] * dy;
        pw[o] *= lam[o];
      }
    }
    __syncthreads();
  }
  if (!live) return;
  float rr[LO];
  load_vec16(R + (size_t)ch * LO, rr);
#pragma unroll
  for (int o = 0; o < LO; ++o) a[o] *= rr[o];
  const size_t off = (((size_t)b * d.NC + n) * d.D + ch) * LO;
  store_vec16(Sloc + off, s);
  store_vec16(Wloc + off, w);
  store_vec16(Aloc + off, a);
}

// backward pass B3 + R3 in one kernel (chunk length LB_TC): the chunk's features and dz stay in shared memory between the
// forward sweep (y, dx1 = dz y into shared memory, partial sums of dR / dlam / dbias) and the reverse sweep (adjoint scan,
// du; the gradient tile overwrites the feature tile in place and leaves as 16-byte chunks).
constexpr int LB_SMEM = LB_TC * (3 * LT_CH + LT_CH + LT_CH) * 2;     // features + dz + dx1
__global__ void __launch_bounds__(LT_CH, 2)
li_bwd_apply_tiled_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ dz, const float* __restrict__ loglam,
                          const float* __restrict__ R, const float* __restrict__ bias, const float* __restrict__ Sin,
                          const float* __restrict__ Win, const float* __restrict__ Ain, bf16* __restrict__ dfeat,
                          float* __restrict__ dRp, float* __restrict__ dLp, float* __restrict__ dBp,
                          const float* __restrict__ dstate_out, LiDims d) {
  extern __shared__ __align__(16) uint8_t li_smem[];
  bf16 (*fS)[3 * LT_CH] = reinterpret_cast<bf16 (*)[3 * LT_CH]>(li_smem);
  bf16 (*gS)[LT_CH] = reinterpret_cast<bf16 (*)[LT_CH]>(li_smem + LB_TC * 3 * LT_CH * 2);
  bf16 (*xS)[LT_CH] = reinterpret_cast<bf16 (*)[LT_CH]>(li_smem + LB_TC * 4 * LT_CH * 2);
  const int tid = threadIdx.x, c0 = blockIdx.x * LT_CH, ch = c0 + tid;
  const int n = blockIdx.y, b = blockIdx.z;
  const bool live = ch < d.D;
  const int t0 = n * LB_TC, t1 = min(t0 + LB_TC, d.L), rows = t1 - t0;
  const bf16* fb = feat + (size_t)b * d.L * 3 * d.D;
  const bf16* gb = dz + (size_t)b * d.L * d.D;
  li_stage_feat(fS, fb, t0, t1, LB_TC, c0, d.D, tid, LT_CH);
  li_stage_d(gS, gb, t0, t1, LB_TC, c0, d.D, tid, LT_CH);
  li_cp_commit();
  float lam[LO], rr[LO];
  float be = 0.f;
  const size_t off = (((size_t)b * d.NC + n) * d.D + ch) * LO;
  if (live) { load_vec16(loglam + (size_t)ch * LO, lam); load_vec16(R + (size_t)ch * LO, rr); be = bias[ch]; }
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = live ? __expf(lam[o]) : 0.f; if (!live) rr[o] = 0.f; }
  li_cp_wait<0>();
  __syncthreads();
  {
    // ---- forward sweep
    float s[LO], w[LO], dr[LO], dl[LO];
    if (live) { load_vec16(Sin + off, s); load_vec16(Win + off, w); }
#pragma unroll
    for (int o = 0; o < LO; ++o) { dr[o] = 0.f; dl[o] = 0.f; if (!live) { s[o] = 0.f; w[o] = 0.f; } }
    float db = 0.f;
#pragma unroll 4
    for (int r = 0; r < rows; ++r) {
      const float x1 = b2f(fS[r][3 * tid]);
      const float u = b2f(fS[r][3 * tid + 1]) * b2f(fS[r][3 * tid + 2]);
      const float gz = b2f(gS[r][tid]);
      const float dy = gz * x1;
      float y = be * u;
#pragma unroll
      for (int o = 0; o < LO; ++o) {
        w[o] = s[o] + lam[o] * w[o];
        s[o] = lam[o] * s[o] + u;
        y += rr[o] * s[o];
        dr[o] += dy * s[o];
        dl[o] += dy * w[o];
      }
      db += dy * u;
      xS[r][tid] = __float2bfloat16_rn(gz * y);
    }
    if (live) {
#pragma unroll
      for (int o = 0; o < LO; ++o) dl[o] *= rr[o];
      store_vec16(dRp + off, dr);
      store_vec16(dLp + off, dl);
      dBp[((size_t)b * d.NC + n) * d.D + ch] = db;
    }
  }
  {
    // ---- reverse sweep (each thread touches only its own three tile entries: no barrier needed in between)
    float a[LO], gs[LO];
    if (live) load_vec16(Ain + off, a);
    const bool tail = dstate_out != nullptr && n == d.NC - 1 && live;
    if (tail) load_vec16(dstate_out + ((size_t)b * d.D + ch) * LO, gs);
#pragma unroll
    for (int o = 0; o < LO; ++o) { if (!live) a[o] = 0.f; if (!tail) gs[o] = 0.f; }
#pragma unroll 4
    for (int r = rows - 1; r >= 0; --r) {
      const float x1 = b2f(fS[r][3 * tid]), x2 = b2f(fS[r][3 * tid + 1]), v = b2f(fS[r][3 * tid + 2]);
      const float dy = b2f(gS[r][tid]) * x1;
      float du = be * dy;
#pragma unroll
      for (int o = 0; o < LO; ++o) a[o] = rr[o] * dy + lam[o] * a[o];
      if (tail && r == rows - 1) {
#pragma unroll
        for (int o = 0; o < LO; ++o) a[o] += gs[o];
      }
#pragma unroll
      for (int o = 0; o < LO; ++o) du += a[o];
      fS[r][3 * tid] = xS[r][tid];
      fS[r][3 * tid + 1] = __float2bfloat16_rn(du * v);
      fS[r][3 * tid + 2] = __float2bfloat16_rn(du * x2);
    }
  }
  __syncthreads();
  constexpr int CHK = 3 * LT_CH / 8;
  const int ncv = min(CHK, (3 * (d.D - c0)) / 8);
  bf16* db_ = dfeat + (size_t)b * d.L * 3 * d.D;
  for (int idx = tid; idx < rows * CHK; idx += LT_CH) {
    const int r = idx / CHK, cv = idx - r * CHK;
    if (cv < ncv) *reinterpret_cast<uint4*>(db_ + (size_t)(t0 + r) * 3 * d.D + 3 * c0 + cv * 8) = *reinterpret_cast<const uint4*>(&fS[r][cv * 8]);
  }
}

static int g_li_tiled = 1;

// ------------------------------------------------------------------------------------ context parallel: all-to-all inside the scan
// Sequence-sharded ranks (zigzag: rank r holds natural chunks r and 2cp-1-r of `chunk_len` rows, [B, l, Dtot] with
// l = 2 chunk_len) switch to a channel-sharded scan over the whole sequence (this rank: d = Dtot / cp channels) and back.
// Only the pre-gated signal u = x2 v travels: every rank writes u into a symmetric staging buffer, and after one
// stream-ordered barrier the scan's first pass reads its channel block of every chunk straight from the owner's
// staging buffer (plain peer loads), keeping a local copy for the second pass.  The second pass stores y straight into
// the owner's staging buffer (plain peer stores); after the second barrier the owner gates it with its own x1.  No
// tensor is permuted or copied by a separate kernel, and a third of the bytes of exchanging (x1, x2, v) and z cross
// NVLink.  `LiCpMap.base[j]`: row 0 of natural chunk j in its owner's staging buffer, already offset to this rank's
// channel block.  The scan chunk length TC must divide chunk_len, so a scan chunk never straddles two owners.
struct LiCpMap {
  void* base[32];
  long long batch_stride;   // elements between batches of a staging buffer (l * Dtot)
  int row_stride;           // elements between rows (Dtot)
  int chunk_len;
  int n_chunks;             // 2 cp
};

__device__ __forceinline__ bf16* cp_row(const LiCpMap& m, int b, int t) {
  const int j = t / m.chunk_len;
  return reinterpret_cast<bf16*>(m.base[j]) + (size_t)b * m.batch_stride + (size_t)(t - j * m.chunk_len) * m.row_stride;
}

// pass 1: pull u from the owners, keep a local copy [B, L, d], chunk-local end state from a zero state
__global__ void __launch_bounds__(LI_THREADS)
li_cp_local_kernel(const LiCpMap u_in, bf16* __restrict__ ufull, const float* __restrict__ loglam, float* __restrict__ Sloc,
                   LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = __expf(lam[o]); s[o] = 0.f; }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* src = cp_row(u_in, b, t0) + ch;
  bf16* dst = ufull + ((size_t)b * d.L + t0) * d.D + ch;
#pragma unroll 8
  for (int t = t0; t < t1; ++t, src += u_in.row_stride, dst += d.D) {
    const bf16 raw = *src;
    *dst = raw;
    const float u = b2f(raw);
#pragma unroll
    for (int o = 0; o < LO; ++o) s[o] = lam[o] * s[o] + u;
  }
  store_vec16(Sloc + (((size_t)b * d.NC + n) * d.D + ch) * LO, s);
}

// pass 3: rerun each chunk from its entering state; y goes to the owner of the rows
__global__ void __launch_bounds__(LI_THREADS)
li_cp_apply_kernel(const bf16* __restrict__ ufull, const float* __restrict__ loglam, const float* __restrict__ R,
                   const float* __restrict__ bias, const float* __restrict__ Sin, const LiCpMap y_out, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO], rr[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
  load_vec16(R + (size_t)ch * LO, rr);
  load_vec16(Sin + (((size_t)b * d.NC + n) * d.D + ch) * LO, s);
#pragma unroll
  for (int o = 0; o < LO; ++o) lam[o] = __expf(lam[o]);
  const float be = bias[ch];
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = ufull + ((size_t)b * d.L + t0) * d.D + ch;
  bf16* yo = cp_row(y_out, b, t0) + ch;
#pragma unroll 8
  for (int t = t0; t < t1; ++t, f += d.D, yo += y_out.row_stride) {
    const float u = b2f(*f);
    float y = be * u;
#pragma unroll
    for (int o = 0; o < LO; ++o) { s[o] = lam[o] * s[o] + u; y += rr[o] * s[o]; }
    *yo = __float2bfloat16_rn(y);
  }
}

// backward pass B1: pull dy = dz x1 from the owners (local copy [B, L, d]); Sloc, Wloc, Aloc as in li_bwd_local_kernel
__global__ void __launch_bounds__(LI_THREADS)
li_cp_bwd_local_kernel(const bf16* __restrict__ ufull, const LiCpMap dy_in, bf16* __restrict__ dyfull,
                       const float* __restrict__ loglam, const float* __restrict__ R, float* __restrict__ Sloc,
                       float* __restrict__ Wloc, float* __restrict__ Aloc, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO], w[LO], pw[LO], a[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = __expf(lam[o]); s[o] = 0.f; w[o] = 0.f; pw[o] = 1.f; a[o] = 0.f; }
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = ufull + ((size_t)b * d.L + t0) * d.D + ch;
  const bf16* g = cp_row(dy_in, b, t0) + ch;
  bf16* gd = dyfull + ((size_t)b * d.L + t0) * d.D + ch;
#pragma unroll 4
  for (int t = t0; t < t1; ++t, f += d.D, g += dy_in.row_stride, gd += d.D) {
    const float u = b2f(*f);
    const bf16 raw = *g;
    *gd = raw;
    const float dy = b2f(raw);
#pragma unroll
    for (int o = 0; o < LO; ++o) {
      w[o] = s[o] + lam[o] * w[o];
      s[o] = lam[o] * s[o] + u;
      a[o] += pw[o] * dy;
      pw[o] *= lam[o];
    }
  }
  float rr[LO];
  load_vec16(R + (size_t)ch * LO, rr);
#pragma unroll
  for (int o = 0; o < LO; ++o) a[o] *= rr[o];
  const size_t off = (((size_t)b * d.NC + n) * d.D + ch) * LO;
  store_vec16(Sloc + off, s);
  store_vec16(Wloc + off, w);
  store_vec16(Aloc + off, a);
}

// backward pass B3 (forward direction): y back to the owners (for dx1 = dz y), per-chunk partials of dR, dlam, dbias
__global__ void __launch_bounds__(LI_THREADS)
li_cp_bwd_apply_fwd_kernel(const bf16* __restrict__ ufull, const bf16* __restrict__ dyfull, const float* __restrict__ loglam,
                           const float* __restrict__ R, const float* __restrict__ bias, const float* __restrict__ Sin,
                           const float* __restrict__ Win, const LiCpMap y_out, float* __restrict__ dRp,
                           float* __restrict__ dLp, float* __restrict__ dBp, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], s[LO], w[LO], rr[LO], dr[LO], dl[LO];
  const size_t off = (((size_t)b * d.NC + n) * d.D + ch) * LO;
  load_vec16(loglam + (size_t)ch * LO, lam);
  load_vec16(R + (size_t)ch * LO, rr);
  load_vec16(Sin + off, s);
  load_vec16(Win + off, w);
#pragma unroll
  for (int o = 0; o < LO; ++o) { lam[o] = __expf(lam[o]); dr[o] = 0.f; dl[o] = 0.f; }
  const float be = bias[ch];
  float db = 0.f;
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* f = ufull + ((size_t)b * d.L + t0) * d.D + ch;
  const bf16* g = dyfull + ((size_t)b * d.L + t0) * d.D + ch;
  bf16* yo = cp_row(y_out, b, t0) + ch;
#pragma unroll 4
  for (int t = t0; t < t1; ++t, f += d.D, g += d.D, yo += y_out.row_stride) {
    const float u = b2f(*f);
    const float dy = b2f(*g);
    float y = be * u;
#pragma unroll
    for (int o = 0; o < LO; ++o) {
      w[o] = s[o] + lam[o] * w[o];
      s[o] = lam[o] * s[o] + u;
      y += rr[o] * s[o];
      dr[o] += dy * s[o];
      dl[o] += dy * w[o];
    }
    db += dy * u;
    *yo = __float2bfloat16_rn(y);
  }
#pragma unroll
  for (int o = 0; o < LO; ++o) dl[o] *= rr[o];
  store_vec16(dRp + off, dr);
  store_vec16(dLp + off, dl);
  dBp[((size_t)b * d.NC + n) * d.D + ch] = db;
}

// backward pass R3 (reverse direction): adjoint scan, du back to the owners (for dx2 = du v, dv = du x2)
__global__ void __launch_bounds__(LI_THREADS)
li_cp_bwd_apply_rev_kernel(const bf16* __restrict__ dyfull, const float* __restrict__ loglam, const float* __restrict__ R,
                           const float* __restrict__ bias, const float* __restrict__ Ain, const LiCpMap du_out, LiDims d) {
  const int ch = blockIdx.x * LI_THREADS + threadIdx.x;
  if (ch >= d.D) return;
  const int n = blockIdx.y, b = blockIdx.z;
  float lam[LO], a[LO], rr[LO];
  load_vec16(loglam + (size_t)ch * LO, lam);
  load_vec16(R + (size_t)ch * LO, rr);
  load_vec16(Ain + (((size_t)b * d.NC + n) * d.D + ch) * LO, a);
#pragma unroll
  for (int o = 0; o < LO; ++o) lam[o] = __expf(lam[o]);
  const float be = bias[ch];
  const int t0 = n * d.TC, t1 = min(t0 + d.TC, d.L);
  const bf16* g = dyfull + ((size_t)b * d.L + (t1 - 1)) * d.D + ch;
  bf16* uo = cp_row(du_out, b, t1 - 1) + ch;
#pragma unroll 8
  for (int t = t1 - 1; t >= t0; --t, g -= d.D, uo -= du_out.row_stride) {
    const float dy = b2f(*g);
    float du = be * dy;
#pragma unroll
    for (int o = 0; o < LO; ++o) { a[o] = rr[o] * dy + lam[o] * a[o]; du += a[o]; }
    *uo = __float2bfloat16_rn(du);
  }
}

// Local gate kernels around the exchange, 8 channels per thread (feat rows are 3D interleaved (x1, x2, v)).
// mode 0: out[n, D] = x2 v                     (u, staged before the forward scan)
// mode 1: out[n, D] = x1 a                     (z = x1 y after the forward scan;  dy = dz x1 before the backward scan)
__global__ void li_cp_gate_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ a, bf16* __restrict__ out,
                                  size_t n_vec, int mode) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4* fp = reinterpret_cast<const uint4*>(feat) + 3 * i;
    const uint4 q0 = fp[0], q1 = fp[1], q2 = fp[2];
    const uint32_t fw[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
    float all[24];
#pragma unroll
    for (int j = 0; j < 12; ++j) {
      const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&fw[j]));
      all[2 * j] = t.x; all[2 * j + 1] = t.y;
    }
    float r[8];
    if (mode == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = all[3 * j + 1] * all[3 * j + 2];
    } else {
      const uint4 av = reinterpret_cast<const uint4*>(a)[i];
      const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[j]));
        r[2 * j] = all[6 * j] * t.x; r[2 * j + 1] = all[6 * j + 3] * t.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// dfeat[n, 3D] = (dz y, du v, du x2) from the returned y and du
__global__ void li_cp_finalize_bwd_kernel(const bf16* __restrict__ feat, const bf16* __restrict__ dz, const bf16* __restrict__ y,
                                          const bf16* __restrict__ du, bf16* __restrict__ dfeat, size_t n_vec) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4* fp = reinterpret_cast<const uint4*>(feat) + 3 * i;
    const uint4 q0 = fp[0], q1 = fp[1], q2 = fp[2];
    const uint32_t fw[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
    float all[24], gz[8], yy[8], dd[8], o[24];
#pragma unroll
    for (int j = 0; j < 12; ++j) {
      const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&fw[j]));
      all[2 * j] = t.x; all[2 * j + 1] = t.y;
    }
    const uint4 a = reinterpret_cast<const uint4*>(dz)[i], bq = reinterpret_cast<const uint4*>(y)[i],
                c = reinterpret_cast<const uint4*>(du)[i];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {bq.x, bq.y, bq.z, bq.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[j])); gz[2 * j] = t.x; gz[2 * j + 1] = t.y;
      t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[j])); yy[2 * j] = t.x; yy[2 * j + 1] = t.y;
      t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cw[j])); dd[2 * j] = t.x; dd[2 * j + 1] = t.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[3 * j] = gz[j] * yy[j];
      o[3 * j + 1] = dd[j] * all[3 * j + 2];
      o[3 * j + 2] = dd[j] * all[3 * j + 1];
    }
    uint4 ov[3];
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(ov);
#pragma unroll
    for (int j = 0; j < 12; ++j) o2[j] = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
    uint4* dp = reinterpret_cast<uint4*>(dfeat) + 3 * i;
    dp[0] = ov[0]; dp[1] = ov[1]; dp[2] = ov[2];
  }
}

}  // namespace sb

using namespace sb;

static inline LiDims li_dims(int B, int L, int D, int TC) { return LiDims{B, L, D, TC, (L + TC - 1) / TC}; }

// Scratch sizes (floats): S = B*NC*D*16.  Callers allocate and pass them.
extern "C" int sb_li_num_chunks(int L, int TC) { return (L + TC - 1) / TC; }

extern "C" int sb_li_fwd(const void* feat, const float* loglam, const float* R, const float* bias, const float* state_in,
                         float* state_out, float* S_scratch, void* z, int B, int L, int D, int TC, cudaStream_t st) {
  if (B * L == 0) return 0;
  LiDims d = li_dims(B, L, D, TC);
  dim3 grid((D + LI_THREADS - 1) / LI_THREADS, d.NC, B);
  const size_t n = (size_t)B * D * LO;
  if (g_li_tiled && D % 8 == 0 && TC % LT_ROWS == 0) {
    li_local_tiled_kernel<<<grid, LT_CH, 0, st>>>((const bf16*)feat, loglam, S_scratch, d);
    li_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S_scratch, loglam, state_in, state_out, d);
    li_apply_tiled_kernel<<<grid, LT_CH, 0, st>>>((const bf16*)feat, loglam, R, bias, S_scratch, (bf16*)z, d);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  li_local_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, loglam, S_scratch, d);
  li_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S_scratch, loglam, state_in, state_out, d);
  li_apply_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, loglam, R, bias, S_scratch, (bf16*)z, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// 1 (default): shared-memory tiled scan kernels where the shape allows; 0: the per-thread streaming kernels
extern "C" int sb_li_set_variant(int tiled) { sb::g_li_tiled = tiled ? 1 : 0; return 0; }
// Chunk length the backward pass uses for a given forward choice: the tiled backward keeps a whole chunk in shared memory
// and therefore fixes its own chunk length; callers size the scratch arrays with the value returned here.
extern "C" int sb_li_bwd_chunk(int D, int TC) { return (sb::g_li_tiled && D % 8 == 0) ? sb::LB_TC : TC; }

// Scratch: S, W, A, dRp, dLp each B*NC*D*16 floats; dBp B*NC*D floats; dx1_tmp B*L*D bf16.
// Outputs: dfeat; per-chunk partials dRp/dLp/dBp (the caller sums over B and NC); w_end, dstate_in optional.
extern "C" int sb_li_bwd(const void* feat, const void* dz, const float* loglam, const float* R, const float* bias,
                         const float* state_in, const float* dstate_out, float* S, float* W, float* A, float* dRp,
                         float* dLp, float* dBp, void* dx1_tmp, void* dfeat, float* w_end, float* dstate_in, int B, int L,
                         int D, int TC, cudaStream_t st) {
  if (B * L == 0) return 0;
  LiDims d = li_dims(B, L, D, TC);
  dim3 grid((D + LI_THREADS - 1) / LI_THREADS, d.NC, B);
  const size_t n = (size_t)B * D * LO;
  if (g_li_tiled && D % 8 == 0 && TC == LB_TC) {
    static bool attr = false;
    if (!attr) {
      if (cudaFuncSetAttribute(li_bwd_apply_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LB_SMEM) != cudaSuccess) return -5;
      attr = true;
    }
    li_bwd_local_tiled_kernel<<<grid, LT_CH, 0, st>>>((const bf16*)feat, (const bf16*)dz, loglam, R, S, W, A, d);
    li_bwd_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S, W, A, loglam, state_in, dstate_out, w_end, dstate_in, d);
    li_bwd_apply_tiled_kernel<<<grid, LT_CH, LB_SMEM, st>>>((const bf16*)feat, (const bf16*)dz, loglam, R, bias, S, W, A,
                                                           (bf16*)dfeat, dRp, dLp, dBp, dstate_out, d);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  li_bwd_local_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, (const bf16*)dz, loglam, R, S, W, A, d);
  li_bwd_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S, W, A, loglam, state_in, dstate_out, w_end, dstate_in, d);
  li_bwd_apply_fwd_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, (const bf16*)dz, loglam, R, bias, S, W,
                                                      (bf16*)dx1_tmp, dRp, dLp, dBp, d);
  li_bwd_apply_rev_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, (const bf16*)dz, loglam, R, bias, A,
                                                      (const bf16*)dx1_tmp, (bf16*)dfeat, dstate_out, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static inline unsigned li_gate_grid(size_t n_vec) {
  size_t g = (n_vec + 255) / 256;
  const size_t cap = 2048;
  return (unsigned)(g > cap ? cap : (g < 1 ? 1 : g));
}

// out[n, D] = x2 v (mode 0) or x1 a (mode 1) for feat [n, 3D]; D % 8 == 0, 16-byte aligned rows.
extern "C" int sb_li_cp_gate(const void* feat, const void* a, void* out, long long n_rows, int D, int mode, cudaStream_t st) {
  if ((D % 8) || (mode == 1 && !a)) return -1;
  const size_t n_vec = (size_t)n_rows * (D / 8);
  if (n_vec == 0) return 0;
  li_cp_gate_kernel<<<li_gate_grid(n_vec), 256, 0, st>>>((const bf16*)feat, (const bf16*)a, (bf16*)out, n_vec, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_li_cp_finalize_bwd(const void* feat, const void* dz, const void* y, const void* du, void* dfeat,
                                     long long n_rows, int D, cudaStream_t st) {
  if (D % 8) return -1;
  const size_t n_vec = (size_t)n_rows * (D / 8);
  if (n_vec == 0) return 0;
  li_cp_finalize_bwd_kernel<<<li_gate_grid(n_vec), 256, 0, st>>>((const bf16*)feat, (const bf16*)dz, (const bf16*)y,
                                                                (const bf16*)du, (bf16*)dfeat, n_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static inline bool li_cp_map_ok(const LiCpMap* m, int L, int TC) {
  return m && m->n_chunks >= 1 && m->n_chunks <= 32 && m->chunk_len > 0 && (long long)m->chunk_len * m->n_chunks == L &&
         (m->chunk_len % TC) == 0;
}

// Channel-sharded forward scan of this rank (d channels, whole sequence L) with the exchange inside: u pulled from the
// owners' staging (u_in) into ufull [B, L, d], y stored into the owners' staging (y_out).  S: B*NC*d*16 floats.
extern "C" int sb_li_cp_fwd(const LiCpMap* u_in, const LiCpMap* y_out, const float* loglam, const float* R, const float* bias,
                            float* S, void* ufull, int B, int L, int d, int TC, cudaStream_t st) {
  if (B * L == 0) return 0;
  if (!li_cp_map_ok(u_in, L, TC) || !li_cp_map_ok(y_out, L, TC)) return -9;
  LiDims dm = li_dims(B, L, d, TC);
  dim3 grid((d + LI_THREADS - 1) / LI_THREADS, dm.NC, B);
  li_cp_local_kernel<<<grid, LI_THREADS, 0, st>>>(*u_in, (bf16*)ufull, loglam, S, dm);
  const size_t n = (size_t)B * d * LO;
  li_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S, loglam, nullptr, nullptr, dm);
  li_cp_apply_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)ufull, loglam, R, bias, S, *y_out, dm);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Backward of the above: dy pulled from the owners (dy_in) into dyfull, y and du stored into the owners' staging.
// Scratch S, W, A, dRp, dLp: B*NC*d*16 floats each; dBp: B*NC*d floats (the caller sums the partials over B and NC).
extern "C" int sb_li_cp_bwd(const LiCpMap* dy_in, const LiCpMap* y_out, const LiCpMap* du_out, const void* ufull, void* dyfull,
                            const float* loglam, const float* R, const float* bias, float* S, float* W, float* A, float* dRp,
                            float* dLp, float* dBp, int B, int L, int d, int TC, cudaStream_t st) {
  if (B * L == 0) return 0;
  if (!li_cp_map_ok(dy_in, L, TC) || !li_cp_map_ok(y_out, L, TC) || !li_cp_map_ok(du_out, L, TC)) return -9;
  LiDims dm = li_dims(B, L, d, TC);
  dim3 grid((d + LI_THREADS - 1) / LI_THREADS, dm.NC, B);
  li_cp_bwd_local_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)ufull, *dy_in, (bf16*)dyfull, loglam, R, S, W, A, dm);
  const size_t n = (size_t)B * d * LO;
  li_bwd_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S, W, A, loglam, nullptr, nullptr, nullptr, nullptr, dm);
  li_cp_bwd_apply_fwd_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)ufull, (const bf16*)dyfull, loglam, R, bias, S, W, *y_out,
                                                         dRp, dLp, dBp, dm);
  li_cp_bwd_apply_rev_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)dyfull, loglam, R, bias, A, *du_out, dm);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ------------------------------------------------------------------------------------ allocation-free variant
// See li_scan_noalloc.h for who needs this and for the contract.
#include <stdio.h>

#include "li_scan_noalloc.h"

// The chunk-state scratch of the forward scan, resident in the library's device image (one copy per GPU).
static __device__ __align__(256) float g_li_noalloc_scratch[SB_LI_NOALLOC_SCRATCH_BYTES / sizeof(float)];

// In host code the symbol above is only a handle; the kernels need its device address, looked up once per device.
static float* g_li_noalloc_ptr[64] = {nullptr};

extern "C" int sb_li_fwd_noalloc(const void* feat, const float* loglam, const float* R, const float* bias,
                                 const float* state_in, float* state_out, void* z, int B, int L, int D, int TC,
                                 cudaStream_t st) {
  if (B <= 0 || L <= 0 || D <= 0 || TC <= 0) return 0;
  LiDims d = li_dims(B, L, D, TC);
  const unsigned long long need = (unsigned long long)B * d.NC * D * LO * sizeof(float);
  if (need > SB_LI_NOALLOC_SCRATCH_BYTES) {
    fprintf(stderr,
            "sb_li_fwd_noalloc: B=%d L=%d D=%d TC=%d needs %llu bytes of chunk-state scratch, the built-in buffer holds "
            "%u; use sb_li_fwd with a caller-provided buffer\n", B, L, D, TC, need, SB_LI_NOALLOC_SCRATCH_BYTES);
    return SB_LI_NOALLOC_TOO_LARGE;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SB_LI_NOALLOC_SETUP_FAILED;
  if (g_li_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_li_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "sb_li_fwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return SB_LI_NOALLOC_SETUP_FAILED;
    }
    g_li_noalloc_ptr[dev] = p;
  }
  float* S = g_li_noalloc_ptr[dev];
  dim3 grid((D + LI_THREADS - 1) / LI_THREADS, d.NC, B);
  li_local_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, loglam, S, d);
  const size_t n = (size_t)B * D * LO;
  li_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(S, loglam, state_in, state_out, d);
  li_apply_kernel<<<grid, LI_THREADS, 0, st>>>((const bf16*)feat, loglam, R, bias, S, (bf16*)z, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
