// Varlen (cu_seqlens) flash attention for sm_100a, head_dim 64, non-causal, optional symmetric
// sliding window, on packed activations qkv[T][3][H][64] (bf16).
//
// Both kernels tile the FLAT token axis in blocks of 128, whatever the sequence boundaries are:
// a 128-token tile may hold several short sequences (or a slice of a long one). The key range
// it needs is [start of the first sequence in the tile, end of the last one), clipped by the
// window, and each row masks keys outside its own sequence / window. Short proteins therefore
// do not waste tensor-core tiles on padding.
//
//   forward : S = Q K^T (tcgen05, fp32 in TMEM) -> online softmax in registers (one thread per
//             row) -> P (bf16) to swizzled shared memory -> O_part = P V (tcgen05) -> registers.
//   backward: per 128-key tile, loop over query tiles: S^T = K Q^T, dP^T = V dO^T (TMEM) ->
//             P^T, dS^T (bf16, shared) -> dV += P^T dO, dK += dS^T Q (TMEM-resident across the
//             loop), dQ_part = dS K -> fp32 atomics into a dq accumulator.
//
// Replaces flash_attn_varlen_func as called by the reference
// (src/nanoplm/pretraining/models/modern_bert/modeling.py:331-366) with window (-1,-1) or
// (64,64); mask semantics match its SDPA route (modeling.py:142-156): |q - k| <= window.
//
// All operand tiles are [128 rows][64 bf16] = [128][128 B] with the 128-byte swizzle, loaded by
// one TMA box each; the same tile serves as a K-major operand (contraction over head_dim) and
// as an MN-major operand (contraction over tokens).
#include "common.cuh"

namespace nplm {

constexpr int FA_T = 128;          // tile of tokens (queries and keys)
constexpr int FA_D = 64;           // head dim
constexpr int FA_TILE_BYTES = FA_T * FA_D * 2;  // 16 KB
constexpr float LOG2E = 1.4426950408889634f;

// byte offset of 16-byte chunk `chunk` (0..7) of row `r` inside a [rows][128 B] swizzled tile
__device__ __forceinline__ uint32_t swz(int r, int chunk) {
  return static_cast<uint32_t>(r * 128 + ((chunk ^ (r & 7)) << 4));
}

// ---------------------------------------------------------------------------- seq bounds
// seq_start[t], seq_end[t] from cu_seqlens (n_seq + 1 entries, may contain empty sequences)
__global__ void seq_bounds_kernel(const int* __restrict__ cu, int n_seq, int* __restrict__ s_start,
                                  int* __restrict__ s_end, int T) {
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    // last i in [0, n_seq) with cu[i] <= t
    int lo = 0, hi = n_seq;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    int a = cu[lo], b = cu[lo + 1];
    if (t < a || t >= b) {  // token not covered by any sequence: attends to itself only
      a = t;
      b = t + 1;
    }
    s_start[t] = a;
    s_end[t] = b;
  }
}

// ---------------------------------------------------------------------------- forward
struct FaFwdArgs {
  __nv_bfloat16* out;   // [T][H*64]
  float* lse;           // [H][T] natural-log LSE of the scaled scores
  const int* seq_start;
  const int* seq_end;
  int T, H, window;     // window < 0: unlimited
  float scale;
  int* status;
};

constexpr int FA_FWD_SMEM = FA_TILE_BYTES * (1 + 2 + 2) + 2 * FA_TILE_BYTES + 256;

__global__ void __launch_bounds__(128, 2)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const FaFwdArgs args) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(args.status, ST_BAD_ARG);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = smem + FA_TILE_BYTES;       // 2 buffers
  uint8_t* sV = smem + 3 * FA_TILE_BYTES;   // 2 buffers
  uint8_t* sP = smem + 5 * FA_TILE_BYTES;   // [2 column blocks][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * FA_TILE_BYTES);
  uint64_t* bar_q = bars;
  uint64_t* bar_kv = bars + 1;  // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int T = args.T, H = args.H, w = args.window;
  const int t0 = blockIdx.x * FA_T;
  const int h = blockIdx.y;
  const int HD = H * FA_D;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQKV);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;        // 128 columns
  const uint32_t tO = tmem_base + 128;  // 64 columns

  const int row = t0 + tid;
  const bool row_ok = row < T;
  int lo = 0, hi = 0;  // this row attends to keys [lo, hi)
  if (row_ok) {
    lo = args.seq_start[row];
    hi = args.seq_end[row];
    if (w >= 0) {
      lo = max(lo, row - w);
      hi = min(hi, row + w + 1);
    }
  }
  const int last = min(t0 + FA_T - 1, T - 1);
  int kv_lo = args.seq_start[t0];
  int kv_hi = args.seq_end[last];
  if (w >= 0) {
    kv_lo = max(kv_lo, t0 - w);
    kv_hi = min(kv_hi, last + w + 1);
  }
  const int n_kv = kv_hi > kv_lo ? (kv_hi - kv_lo + FA_T - 1) / FA_T : 0;

  constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
  const int colQ = h * FA_D, colK = HD + h * FA_D, colV = 2 * HD + h * FA_D;

  auto issue_s = [&](int buf) {
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + buf * FA_TILE_BYTES);
#pragma unroll
    for (int k = 0; k < FA_D / 16; ++k)
      umma_bf16(tS, make_smem_desc(qa + k * 32, 16, 1024), make_smem_desc(ka + k * 32, 16, 1024),
                idesc_s, k > 0 ? 1u : 0u);
    umma_commit(bar_s);
  };

  if (tid == 0 && n_kv > 0) {
    mbar_arrive_expect_tx(bar_q, FA_TILE_BYTES);
    tma_load_2d(sQ, &tmQKV, bar_q, colQ, t0);
    mbar_arrive_expect_tx(&bar_kv[0], 2 * FA_TILE_BYTES);
    tma_load_2d(sK, &tmQKV, &bar_kv[0], colK, kv_lo);
    tma_load_2d(sV, &tmQKV, &bar_kv[0], colV, kv_lo);
    if (mbar_wait(bar_q, 0) && mbar_wait(&bar_kv[0], 0)) {
      tc_fence_after();
      issue_s(0);
    } else {
      atomicExch(args.status, ST_TIMEOUT_FULL);
      *abort_flag = 1;
    }
  }

  const float sl2 = args.scale * LOG2E;
  float m_run = -1e30f, l_run = 0.f;
  float o[FA_D];
#pragma unroll
  for (int e = 0; e < FA_D; ++e) o[e] = 0.f;

  bool alive = true;
  for (int j = 0; j < n_kv && alive; ++j) {
    const int buf = j & 1;
    const int kv0 = kv_lo + j * FA_T;
    if (tid == 0 && j + 1 < n_kv) {
      mbar_arrive_expect_tx(&bar_kv[buf ^ 1], 2 * FA_TILE_BYTES);
      tma_load_2d(sK + (buf ^ 1) * FA_TILE_BYTES, &tmQKV, &bar_kv[buf ^ 1], colK, kv0 + FA_T);
      tma_load_2d(sV + (buf ^ 1) * FA_TILE_BYTES, &tmQKV, &bar_kv[buf ^ 1], colV, kv0 + FA_T);
    }
    bool ok = mbar_wait(bar_s, j & 1);
    ok = __syncthreads_and(ok);
    if (!ok) {
      if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      alive = false;
      break;
    }
    tc_fence_after();
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;

    // pass 1: row maximum over the valid keys of this tile. A 32-column chunk that no row of this
    // warp can see is skipped by the whole warp (tcgen05.ld is warp-aligned, so the decision is
    // taken with a warp vote); a chunk that lies completely inside the row's key range takes the
    // compare-free path.
    float tmax = -1e30f;
#pragma unroll 1
    for (int c = 0; c < FA_T; c += 32) {
      const int c_lo = kv0 + c, c_hi = c_lo + 32;
      const bool none = c_hi <= lo || c_lo >= hi;
      if (__all_sync(0xffffffffu, none)) continue;
      // the fast path is taken by the whole warp or not at all: a per-lane split would run both
      const bool w_in = __all_sync(0xffffffffu, c_lo >= lo && c_hi <= hi);
      uint32_t r[32];
      tmem_ld32(tS + lane_addr + c, r);
      tmem_ld_wait();
      if (w_in) {
#pragma unroll
        for (int e = 0; e < 32; ++e) tmax = fmaxf(tmax, __uint_as_float(r[e]));
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int col = c_lo + e;
          if (col >= lo && col < hi) tmax = fmaxf(tmax, __uint_as_float(r[e]));
        }
      }
    }
    const float m_new = fmaxf(m_run, tmax);
    const float alpha = exp2f((m_run - m_new) * sl2);
    const float moff = m_new * sl2;
    float psum = 0.f;
    // pass 2: probabilities -> bf16 -> swizzled shared memory (A operand of P V)
#pragma unroll 1
    for (int c = 0; c < FA_T; c += 32) {
      const int c_lo = kv0 + c, c_hi = c_lo + 32;
      const bool none = c_hi <= lo || c_lo >= hi;
      const bool skip = __all_sync(0xffffffffu, none);
      uint32_t packed[16];
      if (!skip) {
        uint32_t r[32];
        tmem_ld32(tS + lane_addr + c, r);
        tmem_ld_wait();
        if (__all_sync(0xffffffffu, c_lo >= lo && c_hi <= hi)) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(r[e]), sl2, -moff));
            const float p1 = exp2f(fmaf(__uint_as_float(r[e + 1]), sl2, -moff));
            psum += p0 + p1;
            packed[e >> 1] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int col = c_lo + e;
            float p0 = 0.f, p1 = 0.f;
            if (col >= lo && col < hi) p0 = exp2f(fmaf(__uint_as_float(r[e]), sl2, -moff));
            if (col + 1 >= lo && col + 1 < hi) p1 = exp2f(fmaf(__uint_as_float(r[e + 1]), sl2, -moff));
            psum += p0 + p1;
            packed[e >> 1] = pack_bf16x2(p0, p1);
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) packed[e] = 0u;
      }
      uint8_t* blk = sP + (c >> 6) * FA_TILE_BYTES;
      const int chunk0 = ((c >> 5) & 1) * 4;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        *reinterpret_cast<uint4*>(blk + swz(tid, chunk0 + q)) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
    }
    l_run = l_run * alpha + psum;
    m_run = m_new;
#pragma unroll
    for (int e = 0; e < FA_D; ++e) o[e] *= alpha;

    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t pa = smem_u32(sP), va = smem_u32(sV + buf * FA_TILE_BYTES);
#pragma unroll
      for (int k = 0; k < FA_T / 16; ++k)
        umma_bf16(tO, make_smem_desc(pa + (k >> 2) * FA_TILE_BYTES + (k & 3) * 32, 16, 1024),
                  make_smem_desc(va + k * 2048, 8192, 1024), idesc_o, k > 0 ? 1u : 0u);
      umma_commit(bar_o);
      if (j + 1 < n_kv) {
        if (mbar_wait(&bar_kv[buf ^ 1], ((j + 1) >> 1) & 1)) {
          tc_fence_after();
          issue_s(buf ^ 1);
        } else {
          atomicExch(args.status, ST_TIMEOUT_FULL);
          *abort_flag = 1;
        }
      }
    }
    ok = mbar_wait(bar_o, j & 1);
    ok = __syncthreads_and(ok);
    if (!ok) {
      if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      alive = false;
      break;
    }
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < FA_D; c += 32) {
      uint32_t r[32];
      tmem_ld32(tO + lane_addr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) o[c + e] += __uint_as_float(r[e]);
    }
    tc_fence_before();
  }

  if (row_ok && alive) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* dst = args.out + static_cast<size_t>(row) * HD + h * FA_D;
#pragma unroll
    for (int e = 0; e < FA_D; e += 8) {
      uint4 u;
      uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) p[q] = pack_bf16x2(o[e + 2 * q] * inv, o[e + 2 * q + 1] * inv);
      *reinterpret_cast<uint4*>(dst + e) = u;
    }
    args.lse[static_cast<size_t>(h) * T + row] =
        l_run > 0.f ? m_run * args.scale + __logf(l_run) : 0.f;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 256);
  }
}

// Forward, second generation. Same tiling and interface as fa_fwd_kernel; the differences:
//   * the score tile is read from TMEM once (128 registers per thread); as soon as every warp has
//     its copy, S of the NEXT chunk is issued, so that MMA runs under this chunk's softmax;
//   * the running maximum is only raised when it grew by more than 2^8 (warp vote), probabilities
//     stay below 2^8 and the output accumulator lives in TMEM across chunks (PV accumulates in
//     place); it is read back, rescaled and stored only on those rare raises;
//   * max and sum run as four independent chains; masks are applied per 32-column group only
//     where a sequence / window boundary crosses it; a chunk no row of a warp can see is skipped
//     by that warp (it writes zero probabilities);
//   * K and V have separate barriers: K(j+2) is requested when S(j) has finished, V(j+1) when
//     PV(j-1) has.
__global__ void __launch_bounds__(128, 2)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQKV, const FaFwdArgs args) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(args.status, ST_BAD_ARG);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = smem + FA_TILE_BYTES;       // 2 buffers
  uint8_t* sV = smem + 3 * FA_TILE_BYTES;   // 2 buffers
  uint8_t* sP = smem + 5 * FA_TILE_BYTES;   // [2 column blocks][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * FA_TILE_BYTES);
  uint64_t* bar_q = bars;
  uint64_t* bar_k = bars + 1;  // [2]
  uint64_t* bar_v = bars + 3;  // [2]
  uint64_t* bar_s = bars + 5;
  uint64_t* bar_o = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int T = args.T, H = args.H, w = args.window;
  const int t0 = blockIdx.x * FA_T;
  const int h = blockIdx.y;
  const int HD = H * FA_D;

  if (tid == 0) {
    for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQKV);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;        // 128 columns
  const uint32_t tO = tmem_base + 128;  // 64 columns

  const int row = t0 + tid;
  const bool row_ok = row < T;
  int lo = 0, hi = 0;  // this row attends to keys [lo, hi)
  if (row_ok) {
    lo = args.seq_start[row];
    hi = args.seq_end[row];
    if (w >= 0) {
      lo = max(lo, row - w);
      hi = min(hi, row + w + 1);
    }
  }
  const int last = min(t0 + FA_T - 1, T - 1);
  int kv_lo = args.seq_start[t0];
  int kv_hi = args.seq_end[last];
  if (w >= 0) {
    kv_lo = max(kv_lo, t0 - w);
    kv_hi = min(kv_hi, last + w + 1);
  }
  const int n_kv = kv_hi > kv_lo ? (kv_hi - kv_lo + FA_T - 1) / FA_T : 0;

  constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
  const int colQ = h * FA_D, colK = HD + h * FA_D, colV = 2 * HD + h * FA_D;

  auto issue_s = [&](int buf) {
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + buf * FA_TILE_BYTES);
#pragma unroll
    for (int k = 0; k < FA_D / 16; ++k)
      umma_bf16(tS, make_smem_desc(qa + k * 32, 16, 1024), make_smem_desc(ka + k * 32, 16, 1024),
                idesc_s, k > 0 ? 1u : 0u);
    umma_commit(bar_s);
  };

  if (tid == 0 && n_kv > 0) {
    mbar_arrive_expect_tx(bar_q, FA_TILE_BYTES);
    tma_load_2d(sQ, &tmQKV, bar_q, colQ, t0);
    mbar_arrive_expect_tx(&bar_k[0], FA_TILE_BYTES);
    tma_load_2d(sK, &tmQKV, &bar_k[0], colK, kv_lo);
    mbar_arrive_expect_tx(&bar_v[0], FA_TILE_BYTES);
    tma_load_2d(sV, &tmQKV, &bar_v[0], colV, kv_lo);
    if (n_kv > 1) {
      mbar_arrive_expect_tx(&bar_k[1], FA_TILE_BYTES);
      tma_load_2d(sK + FA_TILE_BYTES, &tmQKV, &bar_k[1], colK, kv_lo + FA_T);
    }
    if (mbar_wait(bar_q, 0) && mbar_wait(&bar_k[0], 0)) {
      tc_fence_after();
      issue_s(0);
    } else {
      atomicExch(args.status, ST_TIMEOUT_FULL);
      *abort_flag = 1;
    }
  }
  __syncwarp();

  const float sl2 = args.scale * LOG2E;
  const uint32_t NEG_INF = 0xff800000u;
  float m_used = -1e30f, l_run = 0.f;
  const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
  bool alive = true;

  for (int j = 0; j < n_kv; ++j) {
    const int buf = j & 1;
    const int kv0 = kv_lo + j * FA_T;
    bool ok = mbar_wait(bar_s, j & 1);
    tc_fence_after();
    const bool none = (kv0 + FA_T <= lo) || (kv0 >= hi);
    const bool warp_none = __all_sync(0xffffffffu, none);
    uint32_t r[FA_T];
    if (!warp_none) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld32(tS + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_ld_wait();
    }
    tc_fence_before();
    ok = __syncthreads_and(ok && *abort_flag == 0);  // every warp holds its scores: tS is free
    if (!ok) {
      if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      alive = false;
      break;
    }
    if (tid == 0) {
      if (j + 1 < n_kv) {
        if (mbar_wait(&bar_k[buf ^ 1], ((j + 1) >> 1) & 1)) {
          tc_fence_after();
          issue_s(buf ^ 1);
        } else {
          atomicExch(args.status, ST_TIMEOUT_FULL);
          *abort_flag = 1;
        }
      }
      if (j + 2 < n_kv) {  // S(j) is complete, its K buffer can take K(j+2)
        mbar_arrive_expect_tx(&bar_k[buf], FA_TILE_BYTES);
        tma_load_2d(sK + buf * FA_TILE_BYTES, &tmQKV, &bar_k[buf], colK, kv0 + 2 * FA_T);
      }
    }
    __syncwarp();

    // masks (only where a boundary crosses a 32-column group) and the row maximum
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (!warp_none) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int c_lo = kv0 + c * 32, c_hi = c_lo + 32;
        if (!(c_lo >= lo && c_hi <= hi)) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c_lo + e;
            if (!(col >= lo && col < hi)) r[c * 32 + e] = NEG_INF;
          }
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(r[c * 32 + e]));
      }
    }
    const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
    const float m_new = fmaxf(m_used, tmax);
    const bool warp_need = __any_sync(0xffffffffu, (m_new - m_used) * sl2 > 8.f);
    float alpha = 1.f;
    if (warp_need) {
      alpha = exp2f((m_used - m_new) * sl2);
      m_used = m_new;
    }
    // PV(j-1) has finished: sP and the other V buffer are free, the accumulator may be rescaled
    if (j > 0) ok = mbar_wait(bar_o, (j - 1) & 1);
    if (tid == 0 && ok && j + 1 < n_kv) {
      mbar_arrive_expect_tx(&bar_v[buf ^ 1], FA_TILE_BYTES);
      tma_load_2d(sV + (buf ^ 1) * FA_TILE_BYTES, &tmQKV, &bar_v[buf ^ 1], colV, kv0 + FA_T);
    }
    __syncwarp();
    tc_fence_after();
    if (warp_need && j > 0) {
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t o[32];
        tmem_ld32(tO + lane_addr + hlf * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
        tmem_st32(tO + lane_addr + hlf * 32, o);
      }
      tmem_st_wait();
    }
    l_run *= alpha;

    const float moff = m_used * sl2;
    float ps[4] = {0.f, 0.f, 0.f, 0.f};
    if (!warp_none) {
#pragma unroll
      for (int c8 = 0; c8 < 16; ++c8) {
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float p0 = exp2f(fmaf(__uint_as_float(r[c8 * 8 + 2 * q]), sl2, -moff));
          const float p1 = exp2f(fmaf(__uint_as_float(r[c8 * 8 + 2 * q + 1]), sl2, -moff));
          ps[q] += p0 + p1;
          pk[q] = pack_bf16x2(p0, p1);
        }
        *reinterpret_cast<uint4*>(sP + (c8 >> 3) * FA_TILE_BYTES + swz(tid, c8 & 7)) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    } else {
#pragma unroll
      for (int c8 = 0; c8 < 16; ++c8)
        *reinterpret_cast<uint4*>(sP + (c8 >> 3) * FA_TILE_BYTES + swz(tid, c8 & 7)) = make_uint4(0u, 0u, 0u, 0u);
    }
    l_run += (ps[0] + ps[1]) + (ps[2] + ps[3]);

    fence_proxy_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok && *abort_flag == 0);
    if (!ok) {
      if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      alive = false;
      break;
    }
    if (tid == 0) {
      if (mbar_wait(&bar_v[buf], (j >> 1) & 1)) {
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + buf * FA_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < FA_T / 16; ++k)
          umma_bf16(tO, make_smem_desc(pa + (k >> 2) * FA_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    make_smem_desc(va + k * 2048, 8192, 1024), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar_o);
      } else {
        atomicExch(args.status, ST_TIMEOUT_FULL);
        *abort_flag = 1;
        umma_commit(bar_o);  // lets the other threads fall through to the abort check
      }
    }
    __syncwarp();
  }

  if (alive && n_kv > 0) {
    bool ok = mbar_wait(bar_o, (n_kv - 1) & 1);
    ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
    tc_fence_after();
    if (ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = args.out + static_cast<size_t>(row) * HD + h * FA_D;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t o[32];
        tmem_ld32(tO + lane_addr + hlf * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 u;
            uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              p[q] = pack_bf16x2(__uint_as_float(o[e + 2 * q]) * inv, __uint_as_float(o[e + 2 * q + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + hlf * 32 + e) = u;
          }
        }
      }
      if (row_ok)
        args.lse[static_cast<size_t>(h) * T + row] = l_run > 0.f ? m_used * args.scale + __logf(l_run) : 0.f;
    } else if (tid == 0) {
      atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
    }
  } else if (n_kv == 0 && row_ok) {
    __nv_bfloat16* dst = args.out + static_cast<size_t>(row) * HD + h * FA_D;
#pragma unroll
    for (int e = 0; e < FA_D; e += 8) *reinterpret_cast<uint4*>(dst + e) = make_uint4(0u, 0u, 0u, 0u);
    args.lse[static_cast<size_t>(h) * T + row] = 0.f;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------- backward
// delta[h][t] = sum_d dO[t,h,d] * O[t,h,d]; also clears nothing (dq accumulator is cleared by
// the host wrapper with a memset).
__global__ void __launch_bounds__(256)
fa_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                float* __restrict__ delta, int T, int H) {
  // 8 threads per (t, h): each handles 8 of the 64 channels
  const long long total = static_cast<long long>(T) * H * 8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int sub = static_cast<int>(idx & 7);
    const long long th = idx >> 3;
    const int h = static_cast<int>(th % H);
    const int t = static_cast<int>(th / H);
    const size_t off = (static_cast<size_t>(t) * H + h) * FA_D + sub * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(o + off);
    const uint4 b = *reinterpret_cast<const uint4*>(dout + off);
    const uint32_t* pa = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 x = unpack_bf16x2(pa[q]);
      const float2 y = unpack_bf16x2(pb[q]);
      s += x.x * y.x + x.y * y.y;
    }
    const uint32_t gmask = 0xffu << (threadIdx.x & 24);  // the 8 lanes that share this (t, h)
    s += __shfl_xor_sync(gmask, s, 1);
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 4);
    if (sub == 0) delta[static_cast<size_t>(h) * T + t] = s;
  }
}

struct FaBwdArgs {
  __nv_bfloat16* dqkv;   // [T][3][H][64]: the kernel writes the dK and dV parts
  float* dq_acc;         // [T][H*64] fp32, zero-initialised by the caller
  const float* lse;      // [H][T]
  const float* delta;    // [H][T]
  const int* seq_start;
  const int* seq_end;
  int T, H, window;
  float scale;
  int* status;
  // optional: q / k were rotated (RoPE) before the forward pass; when set, dQ and dK are
  // rotated back so the caller receives gradients of the un-rotated projections
  const int* rope_pos;
  const float* rope_cos;   // [max_pos][32]
  const float* rope_sin;
  int heads_per_cta;       // consecutive heads handled by one CTA (grid.y = ceil(H / heads_per_cta))
};

// smem: K, V, Q[2], dO[2] (16 KB each) + P^T (32 KB) + dS^T (32 KB) + lse/delta (2*2*128 fp32)
constexpr int FA_BWD_SMEM = 6 * FA_TILE_BYTES + 4 * FA_TILE_BYTES + 2048 + 256;

template <bool MULTI_HEAD>
__global__ void __launch_bounds__(256, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
              const FaBwdArgs args) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(args.status, ST_BAD_ARG);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = smem + FA_TILE_BYTES;
  uint8_t* sQ = smem + 2 * FA_TILE_BYTES;    // 2 buffers
  uint8_t* sdO = smem + 4 * FA_TILE_BYTES;   // 2 buffers
  uint8_t* sPT = smem + 6 * FA_TILE_BYTES;   // [2 q blocks][128 kv rows][128 B]
  uint8_t* sdST = smem + 8 * FA_TILE_BYTES;  // same layout
  float* s_lse = reinterpret_cast<float*>(smem + 10 * FA_TILE_BYTES);  // [2][128]
  float* s_delta = s_lse + 256;                                        // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 10 * FA_TILE_BYTES + 2048);
  uint64_t* bar_kv = bars;
  uint64_t* bar_q = bars + 1;  // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_g = bars + 4;
  uint64_t* bar_dq = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int quarter = warp & 3;
  const int half = warp >> 2;
  const int T = args.T, H = args.H, w = args.window;
  const int kv0 = blockIdx.x * FA_T;
  // One CTA handles a 128-key tile for heads_per_cta consecutive heads: barriers, TMEM and the
  // key / query ranges are set up once, and the operand loads of head h+1 are in flight while the
  // dK / dV tiles of head h leave TMEM.
  // (MULTI_HEAD = false: exactly one head per CTA, which lets the compiler drop the hand-over code.)
  const int h_first = MULTI_HEAD ? blockIdx.y * args.heads_per_cta : blockIdx.y;
  const int h_last = MULTI_HEAD ? min(H, h_first + args.heads_per_cta) : h_first + 1;
  const int HD = H * FA_D;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(&bar_q[0], 1);
    mbar_init(&bar_q[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_g, 1);
    mbar_init(bar_dq, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;         // S^T   [kv][q] 128 cols
  const uint32_t tdP = tmem_base + 128;  // dP^T  [kv][q] 128 cols
  const uint32_t tdQ = tmem_base + 256;  // dQ    [q][d]   64 cols
  const uint32_t tdK = tmem_base + 320;  // dK    [kv][d]  64 cols
  const uint32_t tdV = tmem_base + 384;  // dV    [kv][d]  64 cols

  const int krow_local = quarter * 32 + lane;
  const int krow = kv0 + krow_local;
  const bool krow_ok = krow < T;
  int lo = 0, hi = 0;  // this key is attended by queries [lo, hi)
  if (krow_ok) {
    lo = args.seq_start[krow];
    hi = args.seq_end[krow];
    if (w >= 0) {
      lo = max(lo, krow - w);
      hi = min(hi, krow + w + 1);
    }
  }
  const int last = min(kv0 + FA_T - 1, T - 1);
  int q_lo = args.seq_start[kv0];
  int q_hi = args.seq_end[last];
  if (w >= 0) {
    q_lo = max(q_lo, kv0 - w);
    q_hi = min(q_hi, last + w + 1);
  }
  const int n_q = q_hi > q_lo ? (q_hi - q_lo + FA_T - 1) / FA_T : 0;

  constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_kv = make_idesc_bf16(128, 64, 0, 1);  // A K-major, B MN-major
  constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, 1, 1);  // A MN-major, B MN-major
  const float sl2 = args.scale * LOG2E;

  auto load_kv = [&](int h) {
    mbar_arrive_expect_tx(bar_kv, 2 * FA_TILE_BYTES);
    tma_load_2d(sK, &tmQKV, bar_kv, HD + h * FA_D, kv0);
    tma_load_2d(sV, &tmQKV, bar_kv, 2 * HD + h * FA_D, kv0);
  };
  auto load_q_tile = [&](int buf, int q0, int h) {
    mbar_arrive_expect_tx(&bar_q[buf], 2 * FA_TILE_BYTES);
    tma_load_2d(sQ + buf * FA_TILE_BYTES, &tmQKV, &bar_q[buf], h * FA_D, q0);
    tma_load_2d(sdO + buf * FA_TILE_BYTES, &tmDO, &bar_q[buf], h * FA_D, q0);
  };
  auto issue_s = [&](int buf) {
    const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
    const uint32_t qa = smem_u32(sQ + buf * FA_TILE_BYTES), da = smem_u32(sdO + buf * FA_TILE_BYTES);
#pragma unroll
    for (int k = 0; k < FA_D / 16; ++k)
      umma_bf16(tS, make_smem_desc(ka + k * 32, 16, 1024), make_smem_desc(qa + k * 32, 16, 1024),
                idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
    for (int k = 0; k < FA_D / 16; ++k)
      umma_bf16(tdP, make_smem_desc(va + k * 32, 16, 1024), make_smem_desc(da + k * 32, 16, 1024),
                idesc_s, k > 0 ? 1u : 0u);
    umma_commit(bar_s);
  };
  // Row statistics of a query tile: threads 0-127 fetch lse (scaled to log2), 128-255 delta. The
  // global load and the shared-memory store are separate steps, so the value can travel while
  // the thread works on the current tile.
  auto fetch_stat = [&](int q0, int h) -> float {
    const bool first = tid < 128;
    const int q = q0 + (first ? tid : tid - 128);
    if (q >= T) return 0.f;
    return first ? __ldg(args.lse + static_cast<size_t>(h) * T + q) * LOG2E
                 : __ldg(args.delta + static_cast<size_t>(h) * T + q);
  };
  auto store_stat = [&](int buf, float v) {
    if (tid < 128) s_lse[buf * 128 + tid] = v;
    else s_delta[buf * 128 + tid - 128] = v;
  };

  // completions consumed so far on each barrier (the wait parity is the low bit)
  uint32_t c_kv = 0, c_q0 = 0, c_q1 = 0, c_s = 0, c_g = 0, c_dq = 0;
  auto wait_q = [&](int buf) -> bool {
    const bool r = buf == 0 ? mbar_wait(&bar_q[0], c_q0 & 1u) : mbar_wait(&bar_q[1], c_q1 & 1u);
    if (buf == 0) ++c_q0; else ++c_q1;
    return r;
  };

  if (n_q > 0 && h_first < h_last) {
    store_stat(0, fetch_stat(q_lo, h_first));
    if (tid == 0) {
      load_kv(h_first);
      load_q_tile(0, q_lo, h_first);
      const bool got_kv = mbar_wait(bar_kv, c_kv & 1u);
      const bool got_q = wait_q(0);
      if (got_kv && got_q) {
        tc_fence_after();
        issue_s(0);
      } else {
        atomicExch(args.status, ST_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
    ++c_kv;
  }

  bool alive = true;
  const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
  for (int h = h_first; h < h_last && alive; ++h) {
    for (int j = 0; j < n_q; ++j) {
      const int buf = j & 1;
      const int q0 = q_lo + j * FA_T;
      float next_stat = 0.f;
      if (j + 1 < n_q) {
        next_stat = fetch_stat(q0 + FA_T, h);   // stored to shared memory after this tile's softmax
        if (tid == 0) load_q_tile(buf ^ 1, q0 + FA_T, h);
      }
      __syncthreads();  // stats of tile j visible (written one iteration ahead, or before the loop)
      bool ok = mbar_wait(bar_s, c_s & 1u);
      ++c_s;
      ok = __syncthreads_and(ok && *abort_flag == 0);
      if (!ok) {
        if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
        alive = false;
        break;
      }
      tc_fence_after();
      // this thread: key row krow_local, query columns [half*64, half*64+64)
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        const int cbase = half * 64 + c;
        uint32_t rs[32], rp[32];
        tmem_ld32(tS + lane_addr + cbase, rs);
        tmem_ld32(tdP + lane_addr + cbase, rp);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
        const float4* lse4 = reinterpret_cast<const float4*>(s_lse + buf * 128 + cbase);
        const float4* del4 = reinterpret_cast<const float4*>(s_delta + buf * 128 + cbase);
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 l4 = lse4[e >> 2], d4 = del4[e >> 2];   // broadcast reads, 4 columns each
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
          float p[4], ds[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int q = q0 + cbase + e + u;
            float pv = 0.f;
            if (q >= lo && q < hi) pv = exp2f(fmaf(__uint_as_float(rs[e + u]), sl2, -ls[u]));
            p[u] = pv;
            ds[u] = pv * (__uint_as_float(rp[e + u]) - dl[u]);
          }
          pk[e >> 1] = pack_bf16x2(p[0], p[1]);
          pk[(e >> 1) + 1] = pack_bf16x2(p[2], p[3]);
          dk[e >> 1] = pack_bf16x2(ds[0], ds[1]);
          dk[(e >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
        }
        const int chunk0 = (c >> 5) * 4;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t off = half * FA_TILE_BYTES + swz(krow_local, chunk0 + q4);
          *reinterpret_cast<uint4*>(sPT + off) =
              make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(sdST + off) =
              make_uint4(dk[4 * q4], dk[4 * q4 + 1], dk[4 * q4 + 2], dk[4 * q4 + 3]);
        }
      }
      if (j + 1 < n_q) store_stat(buf ^ 1, next_stat);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        const uint32_t pa = smem_u32(sPT), sa = smem_u32(sdST);
        const uint32_t qa = smem_u32(sQ + buf * FA_TILE_BYTES), da = smem_u32(sdO + buf * FA_TILE_BYTES);
        const uint32_t ka = smem_u32(sK);
        // dQ first, with its own barrier: its read-out (TMEM -> fp32 atomics) then overlaps the
        // dV / dK MMAs that follow in the tensor pipe
#pragma unroll
        for (int k = 0; k < FA_T / 16; ++k) {  // dQ[q][d] = dS[q][kv] K[kv][d]
          umma_bf16(tdQ, make_smem_desc(sa + k * 2048, FA_TILE_BYTES, 1024),
                    make_smem_desc(ka + k * 2048, 8192, 1024), idesc_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_dq);
#pragma unroll
        for (int k = 0; k < FA_T / 16; ++k) {  // dV[kv][d] += P^T[kv][q] dO[q][d]
          umma_bf16(tdV, make_smem_desc(pa + (k >> 2) * FA_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    make_smem_desc(da + k * 2048, 8192, 1024), idesc_kv, (j > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < FA_T / 16; ++k) {  // dK[kv][d] += dS^T[kv][q] Q[q][d]
          umma_bf16(tdK, make_smem_desc(sa + (k >> 2) * FA_TILE_BYTES + (k & 3) * 32, 16, 1024),
                    make_smem_desc(qa + k * 2048, 8192, 1024), idesc_kv, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar_g);
        if (j + 1 < n_q) {
          if (wait_q(buf ^ 1)) {
            tc_fence_after();
            issue_s(buf ^ 1);
          } else {
            atomicExch(args.status, ST_TIMEOUT_FULL);
            *abort_flag = 1;
          }
        }
      }
      ok = mbar_wait(bar_dq, c_dq & 1u);
      ++c_dq;
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      if (ok) {
        // dQ tile: lane = query row, this thread adds channels [half*32, half*32+32)
        uint32_t r[32];
        tmem_ld32(tdQ + lane_addr + half * 32, r);
        tmem_ld_wait();
        const int q = q0 + krow_local;
        if (q < T && q < q_hi) {
          float* dst = args.dq_acc + static_cast<size_t>(q) * HD + h * FA_D + half * 32;
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            atomicAdd(reinterpret_cast<float4*>(dst + e),
                      make_float4(__uint_as_float(r[e]) * args.scale, __uint_as_float(r[e + 1]) * args.scale,
                                  __uint_as_float(r[e + 2]) * args.scale,
                                  __uint_as_float(r[e + 3]) * args.scale));
          }
        }
      }
      ok = mbar_wait(bar_g, c_g & 1u) && ok;   // dV / dK of this tile done: operand buffers are free
      ++c_g;
      tc_fence_before();   // the dQ columns may be overwritten by the next tile's MMA after this barrier
      ok = __syncthreads_and(ok && *abort_flag == 0);
      if (!ok) {
        if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
        alive = false;
        break;
      }
    }
    if (!alive) break;
    tc_fence_after();
    // Every MMA of this head has finished (bar_g of its last tile): K, V, Q and dO buffers are free.
    // Start the next head's loads before the dK / dV tiles are read out.
    const bool more = MULTI_HEAD && h + 1 < h_last && n_q > 0;
    if (more) {
      store_stat(0, fetch_stat(q_lo, h + 1));
      if (tid == 0) {
        load_kv(h + 1);
        load_q_tile(0, q_lo, h + 1);
      }
    }

    // tcgen05.ld is warp-aligned: every lane of the warp executes it, rows past T only skip the
    // global stores. Warps 0-3 (half 0) write dK, warps 4-7 (half 1) write dV; each thread owns
    // all 64 channels of its key row, which is what the inverse rotation of dK needs.
    float g[FA_D];
    if (n_q > 0) {
      const uint32_t src = (half == 0 ? tdK : tdV) + lane_addr;
#pragma unroll
      for (int c = 0; c < FA_D; c += 32) {
        uint32_t r[32];
        tmem_ld32(src + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) g[c + e] = __uint_as_float(r[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < FA_D; ++e) g[e] = 0.f;
    }
    if (more) {
      // all warps hold their dK / dV values: the accumulators may be overwritten by the next head
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        const bool got_kv = mbar_wait(bar_kv, c_kv & 1u);
        const bool got_q = wait_q(0);
        if (got_kv && got_q) {
          tc_fence_after();
          issue_s(0);
        } else {
          atomicExch(args.status, ST_TIMEOUT_FULL);
          *abort_flag = 1;
        }
      }
      ++c_kv;
    }
    if (krow_ok) {
      if (half == 0) {
#pragma unroll
        for (int e = 0; e < FA_D; ++e) g[e] *= args.scale;
        if (args.rope_pos != nullptr) {
          const int pos = args.rope_pos[krow];
          const float4* cp = reinterpret_cast<const float4*>(args.rope_cos + static_cast<size_t>(pos) * 32);
          const float4* sp = reinterpret_cast<const float4*>(args.rope_sin + static_cast<size_t>(pos) * 32);
          float4 c4[8], s4[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {   // 16 independent 16-byte loads, issued back to back
            c4[q] = __ldg(cp + q);
            s4[q] = __ldg(sp + q);
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float cc[4] = {c4[q].x, c4[q].y, c4[q].z, c4[q].w};
            const float ss[4] = {s4[q].x, s4[q].y, s4[q].z, s4[q].w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int e = q * 4 + u;
              const float a = g[e], b = g[e + 32];
              g[e] = a * cc[u] + b * ss[u];
              g[e + 32] = b * cc[u] - a * ss[u];
            }
          }
        }
      }
      __nv_bfloat16* dst = args.dqkv + (static_cast<size_t>(krow) * 3 + 1 + half) * HD + h * FA_D;
#pragma unroll
      for (int e = 0; e < FA_D; e += 8) {
        uint4 u;
        uint32_t* pk = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
        for (int q = 0; q < 4; ++q) pk[q] = pack_bf16x2(g[e + 2 * q], g[e + 2 * q + 1]);
        *reinterpret_cast<uint4*>(dst + e) = u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// dq (fp32 accumulator) -> bf16 into the q part of dqkv[T][3][H][64]; with rope_pos the gradient is
// rotated back first. One thread handles channels [8v, 8v+8) and [32+8v, 32+8v+8) of one head.
__global__ void __launch_bounds__(256)
fa_dq_store_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int T, int H,
                   const int* __restrict__ rope_pos, const float* __restrict__ rope_cos,
                   const float* __restrict__ rope_sin) {
  const int HD = H * FA_D;
  const long long total = static_cast<long long>(T) * H * 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i & 3);
    const long long th = i >> 2;
    const int h = static_cast<int>(th % H);
    const int t = static_cast<int>(th / H);
    const float* src = dq_acc + static_cast<size_t>(t) * HD + h * FA_D + v * 8;
    float a[8], b[8];
    *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(src);
    *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(src + 4);
    *reinterpret_cast<float4*>(b) = *reinterpret_cast<const float4*>(src + 32);
    *reinterpret_cast<float4*>(b + 4) = *reinterpret_cast<const float4*>(src + 36);
    if (rope_pos != nullptr) {
      const int pos = rope_pos[t];
      const float* cp = rope_cos + static_cast<size_t>(pos) * 32 + v * 8;
      const float* sp = rope_sin + static_cast<size_t>(pos) * 32 + v * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float c = cp[e], sn = sp[e], x1 = a[e], x2 = b[e];
        a[e] = x1 * c + x2 * sn;
        b[e] = x2 * c - x1 * sn;
      }
    }
    __nv_bfloat16* dst = dqkv + static_cast<size_t>(t) * 3 * HD + h * FA_D + v * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]),
                                                pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
    *reinterpret_cast<uint4*>(dst + 32) = make_uint4(pack_bf16x2(b[0], b[1]), pack_bf16x2(b[2], b[3]),
                                                     pack_bf16x2(b[4], b[5]), pack_bf16x2(b[6], b[7]));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rows = T, cols contiguous; box = [128 rows][64 cols]
static int fa_make_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows) {
  EncodeTiledFn fn = fa_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {FA_D, FA_T};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// cudaFuncSetAttribute applies to the current device only: one flag per device ordinal. Returns the
// slot of the current device (or a negative / CUDA error code).
constexpr int FA_MAX_DEVICES = 64;
static bool fa_fwd_configured[FA_MAX_DEVICES];
static bool fa_bwd_configured[FA_MAX_DEVICES];

static int fa_current_device(int* dev) {
  NPLM_CUDA_CHECK(cudaGetDevice(dev));
  if (*dev < 0 || *dev >= FA_MAX_DEVICES) return -4;
  return 0;
}

}  // namespace nplm

using namespace nplm;

extern "C" int nplm_seq_bounds(const int* cu_seqlens, int n_seq, int* seq_start, int* seq_end,
                               int T, cudaStream_t st) {
  if (T <= 0 || n_seq <= 0) return 0;
  seq_bounds_kernel<<<(T + 255) / 256, 256, 0, st>>>(cu_seqlens, n_seq, seq_start, seq_end, T);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_fa_fwd(const void* qkv, void* out, float* lse, const int* seq_start,
                           const int* seq_end, int T, int H, int D, int window, float scale,
                           int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D != FA_D) return -3;
  if (reinterpret_cast<uintptr_t>(qkv) & 15) return -3;
  CUtensorMap tm;
  int rc = fa_make_map(&tm, qkv, static_cast<uint64_t>(3) * H * D, T);
  if (rc) return rc;
  int dev = 0;
  rc = fa_current_device(&dev);
  if (rc) return rc;
  static int force = 0;  // NPLM_FA_FWD_KERNEL=1 / 2 pins one generation (benchmarks)
  if (!fa_fwd_configured[dev]) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FA_FWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FA_FWD_SMEM));
    const char* env = getenv("NPLM_FA_FWD_KERNEL");
    if (env != nullptr && (env[0] == '1' || env[0] == '2')) force = env[0] - '0';
    fa_fwd_configured[dev] = true;
  }
  FaFwdArgs a;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.seq_start = seq_start;
  a.seq_end = seq_end;
  a.T = T;
  a.H = H;
  a.window = window;
  a.scale = scale;
  a.status = status;
  dim3 grid((T + FA_T - 1) / FA_T, H);
  // measured on 65 536 packed tokens: the second generation is ahead on unlimited attention
  // (0.436 vs 0.449 ms), the first on the +-64 window (0.300 vs 0.307 ms)
  const bool second = force ? force == 2 : window < 0;
  if (second)
    fa_fwd2_kernel<<<grid, 128, FA_FWD_SMEM, st>>>(tm, a);
  else
    fa_fwd_kernel<<<grid, 128, FA_FWD_SMEM, st>>>(tm, a);
  return static_cast<int>(cudaGetLastError());
}

// dq_acc: caller-provided fp32 scratch [T][H*D]; it is cleared here. delta: fp32 scratch [H][T],
// computed here from out and dout unless out is null (then it must hold rowsum(dO * O) already).
extern "C" int nplm_fa_bwd_rope(const void* qkv, const void* out, const void* dout, const float* lse,
                                void* dqkv, float* dq_acc, float* delta, const int* seq_start,
                                const int* seq_end, int T, int H, int D, int window, float scale,
                                const int* rope_pos, const float* rope_cos, const float* rope_sin,
                                int* status, cudaStream_t st);

extern "C" int nplm_fa_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                           void* dqkv, float* dq_acc, float* delta, const int* seq_start,
                           const int* seq_end, int T, int H, int D, int window, float scale,
                           int* status, cudaStream_t st) {
  return nplm_fa_bwd_rope(qkv, out, dout, lse, dqkv, dq_acc, delta, seq_start, seq_end, T, H, D, window,
                          scale, nullptr, nullptr, nullptr, status, st);
}

// Same, for q / k that were rotated before the forward pass (rope_* may be null): dQ and dK are
// returned as gradients of the un-rotated projections.
extern "C" int nplm_fa_bwd_rope(const void* qkv, const void* out, const void* dout, const float* lse,
                                void* dqkv, float* dq_acc, float* delta, const int* seq_start,
                                const int* seq_end, int T, int H, int D, int window, float scale,
                                const int* rope_pos, const float* rope_cos, const float* rope_sin,
                                int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D != FA_D) return -3;
  CUtensorMap tmQKV, tmDO;
  int rc = fa_make_map(&tmQKV, qkv, static_cast<uint64_t>(3) * H * D, T);
  if (rc) return rc;
  rc = fa_make_map(&tmDO, dout, static_cast<uint64_t>(H) * D, T);
  if (rc) return rc;
  int dev = 0;
  rc = fa_current_device(&dev);
  if (rc) return rc;
  if (!fa_bwd_configured[dev]) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FA_BWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FA_BWD_SMEM));
    fa_bwd_configured[dev] = true;
  }
  const int HD = H * D;
  NPLM_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(T) * HD * sizeof(float), st));
  if (out != nullptr) {   // out == nullptr: the caller has filled delta already
    const long long total = static_cast<long long>(T) * H * 8;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fa_delta_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout),
        delta, T, H);
  }
  FaBwdArgs a;
  a.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  a.dq_acc = dq_acc;
  a.lse = lse;
  a.delta = delta;
  a.seq_start = seq_start;
  a.seq_end = seq_end;
  a.T = T;
  a.H = H;
  a.window = window;
  a.scale = scale;
  a.status = status;
  a.rope_pos = rope_pos;
  a.rope_cos = rope_cos;
  a.rope_sin = rope_sin;
  // several heads per CTA amortise the per-CTA set-up and overlap the next head's loads with the
  // dK / dV read-out, as long as the grid still fills the GPU a few times over
  static int hpc_env = -1;
  if (hpc_env < 0) {
    const char* e = getenv("NPLM_FA_BWD_HEADS_PER_CTA");
    hpc_env = (e != nullptr && e[0] >= '1' && e[0] <= '8') ? e[0] - '0' : 0;
  }
  // measured on 65 536 packed tokens, 16 heads: 4 heads per CTA help the +-64 window (few query
  // tiles per key tile, so the set-up weighs more): 0.818 vs 0.892 ms; unlimited attention is best
  // with one head per CTA (1.357 ms)
  const int n_tiles = (T + FA_T - 1) / FA_T;
  int hpc = hpc_env > 0 ? hpc_env : (window >= 0 ? 4 : 1);
  while (hpc > 1 && (static_cast<long long>(n_tiles) * ((H + hpc - 1) / hpc) < 148LL * 4)) hpc >>= 1;
  if (hpc > H) hpc = H;
  a.heads_per_cta = hpc;
  dim3 grid(n_tiles, (H + hpc - 1) / hpc);
  if (hpc > 1)
    fa_bwd_kernel<true><<<grid, 256, FA_BWD_SMEM, st>>>(tmQKV, tmDO, a);
  else
    fa_bwd_kernel<false><<<grid, 256, FA_BWD_SMEM, st>>>(tmQKV, tmDO, a);
  {
    const long long total = static_cast<long long>(T) * H * 4;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fa_dq_store_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        dq_acc, reinterpret_cast<__nv_bfloat16*>(dqkv), T, H, rope_pos, rope_cos, rope_sin);
  }
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------- no-allocation entry
#include "attention_noalloc.h"

// Scratch of the allocation-free entry point: [dq accumulator | per-row statistics]. File scope,
// so it exists once per device that loads this library and lives until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[NPLM_NOALLOC_MAX_DQ_FLOATS + NPLM_NOALLOC_MAX_STAT_FLOATS];

extern "C" const char* nplm_fa_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case NPLM_NOALLOC_TOO_LARGE:
      return "problem too large for the built-in scratch: need T*H*D <= 4 Mi and T*H <= 64 Ki floats";
    case NPLM_NOALLOC_SYMBOL_LOOKUP_FAILED:
      return "cudaGetSymbolAddress failed for the built-in scratch array";
    case -3: return "unsupported head dimension or misaligned pointer";
    default: return code > 0 ? "CUDA runtime error (cudaError_t)" : "rejected arguments";
  }
}

extern "C" int nplm_fa_bwd_noalloc(const void* qkv, const void* out, const void* dout, const float* lse,
                                   void* dqkv, const int* seq_start, const int* seq_end, int T, int H,
                                   int D, int window, float scale, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || D <= 0 || out == nullptr) return -3;   // this entry always computes delta itself
  const size_t need_dq = static_cast<size_t>(T) * H * D;
  const size_t need_stat = static_cast<size_t>(T) * H;
  if (need_dq > NPLM_NOALLOC_MAX_DQ_FLOATS || need_stat > NPLM_NOALLOC_MAX_STAT_FLOATS)
    return NPLM_NOALLOC_TOO_LARGE;
  // The array's name is only a host-side handle: the kernels need its device address, which
  // differs per device, so it is looked up once per device with that device current.
  constexpr int MAX_DEVICES = 64;
  static float* device_ptr[MAX_DEVICES] = {nullptr};
  int dev = 0;
  NPLM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return NPLM_NOALLOC_SYMBOL_LOOKUP_FAILED;
  if (device_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return NPLM_NOALLOC_SYMBOL_LOOKUP_FAILED;
    device_ptr[dev] = p;
  }
  float* dq_acc = device_ptr[dev];
  float* delta = device_ptr[dev] + NPLM_NOALLOC_MAX_DQ_FLOATS;
  // nplm_fa_bwd clears dq_acc on `stream` (cudaMemsetAsync) and overwrites delta before use.
  return nplm_fa_bwd(qkv, out, dout, lse, dqkv, dq_acc, delta, seq_start, seq_end, T, H, D, window,
                     scale, status, stream);
}
