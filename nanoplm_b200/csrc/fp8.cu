// FP8 (e4m3) training kernels for sm_100a: block-scaled quantisation and a tcgen05 GEMM with
// per-128-K-block scale promotion.
//
// The reference trains in bf16 only (src/nanoplm/pretraining/pure_pipeline.py:485-487 sets a bf16
// MixedPrecisionPolicy); this file serves the `pretraining.fp8` extension: activations scaled per
// 1 x 128 (row x K-block), weights per 128 x 128, e4m3 operands for forward, data gradient and
// weight gradient, fp32 accumulation.
//
// Scale layout. Every quantised operand is K-major (contraction axis contiguous) and carries
// fp32 scales stored K-block-major: scale[kb * rows + r] for row-scaled operands (1 x 128) and
// scale[kb * row_blocks + r / 128] for block-scaled ones (128 x 128). value = q * scale.
//
// GEMM. C[M,N] (+)= sum_kb (A_kb * sa[.,kb]) (B_kb * sb[.,kb])^T. One pipeline stage holds one
// 128-wide K block of A (128 rows) and B (128 rows) as 128-byte swizzled rows; the MMA warp issues
// four kind::f8f6f4 UMMAs (K = 32 each) per stage into one of four TMEM buffers and the eight
// epilogue warps read each partial product, multiply by the scales of that K block and add it to
// fp32 registers ("promotion"), so the scales never have to be folded into 8-bit data.
#include <cuda_fp8.h>

#include "common.cuh"

namespace nplm {

constexpr float E4M3_MAX = 448.f;

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// ------------------------------------------------------------------ quantise, no transpose
// x bf16 [R][K] (row stride ldx) -> q e4m3 [R][K], 1 x 128 scales [K/128][R]. 16 threads per
// (row, K block), 8 elements each.
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int R, int K, int ldx, uint8_t* __restrict__ q,
                  float* __restrict__ scale) {
  const int KB = K / 128;
  const long long groups = static_cast<long long>(R) * KB;
  const int sub = threadIdx.x & 15;
  const long long warp_global = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  // two groups per warp and iteration; the loop bound is warp-uniform (full-mask shuffles inside)
  for (long long gw = warp_global * 2; gw < groups; gw += warps_total * 2) {
    const long long g = gw + ((threadIdx.x >> 4) & 1);
    const bool valid = g < groups;
    const int r = valid ? static_cast<int>(g / KB) : 0, kb = valid ? static_cast<int>(g % KB) : 0;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ldx + kb * 128 + sub * 8);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = unpack_bf16x2(w[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
      amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fmaxf(amax, 1e-12f) / E4M3_MAX;
    const float inv = 1.f / s;
    if (valid) {
      uint2 o2;
      o2.x = pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
      o2.y = pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
      *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * K + kb * 128 + sub * 8) = o2;
      if (sub == 0) scale[static_cast<size_t>(kb) * R + r] = s;
    }
  }
}

// ------------------------------------------------------------------ 128 x 128 tile kernel
// One CTA per 128 x 128 tile of x bf16 [R][K] (R, K multiples of 128).
//   TRANSPOSE = false, BLOCK = true : q [R][K],  scale[(k/128) * (R/128) + r/128]   (weights)
//   TRANSPOSE = true,  BLOCK = true : q [K][R],  scale[(r/128) * (K/128) + k/128]   (weights^T)
//   TRANSPOSE = true,  BLOCK = false: q [K][R],  scale[(r/128) * K + k]  (1 x 128 along the old row
//                                     axis: operands of the weight-gradient GEMM)
template <bool TRANSPOSE, bool BLOCK>
__global__ void __launch_bounds__(256)
quant_tile_kernel(const __nv_bfloat16* __restrict__ x, int R, int K, int ldx, uint8_t* __restrict__ q,
                  float* __restrict__ scale) {
  __shared__ __nv_bfloat16 tile[128][130];
  __shared__ float s_red[128];
  const int r0 = blockIdx.y * 128, k0 = blockIdx.x * 128;
  const int tid = threadIdx.x;
  // load: 128 rows x 16 chunks of 8
  for (int i = tid; i < 128 * 16; i += 256) {
    const int r = i >> 4, c = (i & 15) * 8;
    float f[8];
    if (r0 + r < R) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0 + r) * ldx + k0 + c);
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack_bf16x2(w[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[r][c + j] = __float2bfloat16(f[j]);
  }
  __syncthreads();
  // amax: per column of the tile (1 x 128 along rows) or of the whole tile
  if (tid < 128) {
    float m = 0.f;
#pragma unroll 8
    for (int r = 0; r < 128; ++r) m = fmaxf(m, fabsf(__bfloat162float(tile[r][tid])));
    s_red[tid] = m;
  }
  __syncthreads();
  if (BLOCK) {
    if (tid < 32) {
      float m = fmaxf(fmaxf(s_red[tid], s_red[tid + 32]), fmaxf(s_red[tid + 64], s_red[tid + 96]));
      m = warp_max(m);
      if (tid == 0) s_red[0] = fmaxf(m, 1e-12f) / E4M3_MAX;
    }
    __syncthreads();
    const float s = s_red[0];
    if (tid == 0) {
      if (TRANSPOSE)
        scale[static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x] = s;
      else
        scale[static_cast<size_t>(blockIdx.x) * gridDim.y + blockIdx.y] = s;
    }
  } else {
    if (tid < 128) {
      const float s = fmaxf(s_red[tid], 1e-12f) / E4M3_MAX;
      s_red[tid] = s;
      scale[static_cast<size_t>(blockIdx.y) * K + k0 + tid] = s;
    }
    __syncthreads();
  }
  // store 128 output rows x 8 chunks of 16 bytes
  for (int i = tid; i < 128 * 8; i += 256) {
    const int orow = i >> 3, oc = (i & 7) * 16;
    uint32_t pk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = oc + 4 * j + e;
        const float val = __bfloat162float(TRANSPOSE ? tile[c][orow] : tile[orow][c]);
        const float s = BLOCK ? s_red[0] : s_red[TRANSPOSE ? orow : c];
        v[e] = val / s;
      }
      pk[j] = pack_e4m3x4(v[0], v[1], v[2], v[3]);
    }
    if (TRANSPOSE) {
      // output [K][R]: row k0 + orow, columns r0 + oc ..
      if (r0 + oc < R)
        *reinterpret_cast<uint4*>(q + static_cast<size_t>(k0 + orow) * R + r0 + oc) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
    } else {
      if (r0 + orow < R)
        *reinterpret_cast<uint4*>(q + static_cast<size_t>(r0 + orow) * K + k0 + oc) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
}

// ------------------------------------------------------------------ GEMM
constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;  // BK in elements = bytes
constexpr int F8_STAGES = 6;
constexpr int F8_ACC = 4;  // TMEM partial-product buffers (4 x 128 columns = all of TMEM)
constexpr int F8_STAGE_BYTES = (F8_BM + F8_BN) * F8_BK;  // 32 KB
constexpr int F8_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps (2 per TMEM lane quarter)
constexpr int F8_SMEM = F8_STAGES * F8_STAGE_BYTES + 256 + 1024;

struct Fp8Args {
  void* C;
  const float* sa;   // [KB][M]
  const float* sb;   // [KB][N] (b_block == 0) or [KB][ceil(N/128)] (b_block == 1)
  int M, N, K, ldc;
  int b_block;
  int out_mode;      // 0: bf16 store, 1: fp32 store, 2: fp32 atomic add
  int* status;
  // All-gather mode (ag_world > 1, block-scaled B only): B's rows and the matching scale columns
  // are sharded over the ranks. The epilogue warps of all CTAs first copy the other ranks' e4m3
  // rows (half the bytes of a bf16 gather) and scales out of peer memory into the local full-size
  // buffers, bump ag_flags[shard], and both the TMA producer and the epilogue wait (bounded) on a
  // shard's flag before touching it. Tiles are visited shard by shard, the local shard first.
  int ag_world, ag_rank, ag_rows;
  const uint8_t* ag_src[8];   // peer r's shard rows (ag_rows x K bytes)
  const float* ag_ssrc[8];    // peer r's full-size scale buffer [KB][N/128]
  uint8_t* ag_dst;            // local full B
  float* ag_sdst;             // local full scale buffer
  unsigned* ag_flags;         // [ag_world], zeroed before the launch
};

__device__ __forceinline__ bool f8_wait_shard(const Fp8Args& args, int shard, unsigned target) {
  const long long t0 = clock64();
  while (ld_acquire_gpu(args.ag_flags + shard) < target) {
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    __nanosleep(100);
  }
  return true;
}

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const Fp8Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F8_STAGES * F8_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + F8_STAGES;
  uint64_t* tfull_bar = bars + 2 * F8_STAGES;
  uint64_t* tempty_bar = bars + 2 * F8_STAGES + F8_ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F8_STAGES + 2 * F8_ACC);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = args.M, N = args.N;
  const int num_m = (M + F8_BM - 1) / F8_BM, num_n = (N + F8_BN - 1) / F8_BN;
  const int KB = args.K / F8_BK;
  const int total = num_m * num_n;
  // work item -> tile origin (all-gather mode: shard by shard, the local one first)
  auto tile_of = [&](int w, int& m0, int& n0) {
    if (args.ag_world > 1) {
      const int n_per = args.ag_rows / F8_BN;
      const int per_shard = num_m * n_per;
      const int shard = (args.ag_rank + w / per_shard) % args.ag_world;
      const int rem = w % per_shard;
      m0 = (rem / n_per) * F8_BM;
      n0 = shard * args.ag_rows + (rem % n_per) * F8_BN;
    } else {
      m0 = (w / num_n) * F8_BM;
      n0 = (w % num_n) * F8_BN;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < F8_ACC; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
    }
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, F8_ACC * F8_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t ag_seen = 0;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        int m0, n0;
        tile_of(w, m0, n0);
        if (args.ag_world > 1) {
          const int shard = n0 / args.ag_rows;
          if (shard != args.ag_rank && !((ag_seen >> shard) & 1u)) {
            if (!f8_wait_shard(args, shard, gridDim.x)) {
              atomicExch(args.status, ST_TIMEOUT_PEER);
              ok = false;
              break;
            }
            ag_seen |= 1u << shard;
            fence_proxy_async_global();
          }
        }
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicExch(args.status, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * F8_STAGE_BYTES;
          uint8_t* sb = sa + F8_BM * F8_BK;
          mbar_arrive_expect_tx(&full_bar[stage], F8_STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * F8_BK, m0);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * F8_BK, n0);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3(F8_BM, F8_BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1)) {
            atomicExch(args.status, ST_TIMEOUT_TMEM_EMPTY);
            ok = false;
            break;
          }
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicExch(args.status, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * F8_STAGE_BYTES);
          const uint32_t sb = sa + F8_BM * F8_BK;
          const uint32_t d_tmem = tmem_base + acc * F8_BN;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)
            umma_f8(d_tmem, make_smem_desc(sa + k * 32, 16, 1024), make_smem_desc(sb + k * 32, 16, 1024),
                    idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          umma_commit(&tfull_bar[acc]);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1;
          }
          if (++acc == F8_ACC) {
            acc = 0;
            acc_phase ^= 1;
          }
        }
      }
    }
  } else {
    // warp w owns TMEM lanes 32 * (w % 4) .. +31 (hardware rule) and the column half (w - 2) / 4
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HC = F8_BN / 2;  // 64 columns per thread
    uint32_t ag_seen = 0;
    if (args.ag_world > 1) {
      const int et = threadIdx.x - 64;  // 0..255 over the eight epilogue warps
      const long long shard_vecs = static_cast<long long>(args.ag_rows) * args.K / 16;
      const long long per_cta = (shard_vecs + gridDim.x - 1) / gridDim.x;
      const long long v0 = per_cta * blockIdx.x, v1 = min(shard_vecs, v0 + per_cta);
      const int nb_all = num_n, nb_shard = args.ag_rows / F8_BN;
      for (int d = 1; d < args.ag_world; ++d) {
        const int shard = (args.ag_rank + d) % args.ag_world;
        const uint4* src = reinterpret_cast<const uint4*>(args.ag_src[shard]);
        uint4* dst = reinterpret_cast<uint4*>(args.ag_dst + static_cast<size_t>(shard) * args.ag_rows * args.K);
        for (long long v = v0 + et; v < v1; v += 256) dst[v] = src[v];
        if (blockIdx.x == 0) {   // the scale columns of this shard, every K block
          for (int i = et; i < KB * nb_shard; i += 256) {
            const int idx = (i / nb_shard) * nb_all + shard * nb_shard + (i % nb_shard);
            args.ag_sdst[idx] = args.ag_ssrc[shard][idx];
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (et == 0) red_release_gpu_add(args.ag_flags + shard, 1u);
      }
    }
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      int m0, n0;
      tile_of(w, m0, n0);
      if (args.ag_world > 1) {
        const int shard = n0 / args.ag_rows;
        if (shard != args.ag_rank && !((ag_seen >> shard) & 1u)) {
          if (!f8_wait_shard(args, shard, gridDim.x)) {   // scales of this shard must have landed
            if (lane == 0) atomicExch(args.status, ST_TIMEOUT_PEER);
            ok = false;
            break;
          }
          ag_seen |= 1u << shard;
        }
      }
      n0 += half * HC;
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < M;
      float c[HC];
#pragma unroll
      for (int j = 0; j < HC; ++j) c[j] = 0.f;
      // scales of K block 0; those of block kb + 1 are fetched while block kb is being awaited
      float sa_n = row_ok ? args.sa[row] : 0.f;
      float sb_n = args.b_block ? __ldcg(args.sb + (n0 >> 7)) : 0.f;
      for (int kb = 0; kb < KB; ++kb) {
        const float sa = sa_n;
        const float sblk = sb_n * sa;
        if (kb + 1 < KB) {
          sa_n = row_ok ? args.sa[static_cast<size_t>(kb + 1) * M + row] : 0.f;
          if (args.b_block) sb_n = __ldcg(args.sb + static_cast<size_t>(kb + 1) * num_n + (n0 >> 7));
        }
        if (!mbar_wait(&tfull_bar[acc], acc_phase)) {
          if (lane == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * F8_BN + half * HC + (static_cast<uint32_t>(quarter * 32) << 16);
        uint32_t r0[32], r1[32];
        tmem_ld32(taddr, r0);
        tmem_ld32(taddr + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        if (args.b_block) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            c[e] = fmaf(__uint_as_float(r0[e]), sblk, c[e]);
            c[32 + e] = fmaf(__uint_as_float(r1[e]), sblk, c[32 + e]);
          }
        } else {
#pragma unroll
          const float4* sbp = reinterpret_cast<const float4*>(args.sb + static_cast<size_t>(kb) * N + n0);
#pragma unroll
          for (int e4 = 0; e4 < HC / 4; ++e4) {
            const float4 s4 = (n0 + e4 * 4 < N) ? __ldg(sbp + e4) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int e = e4 * 4 + u;
              const float p = __uint_as_float(e < 32 ? r0[e] : r1[e - 32]) * sa;
              c[e] = fmaf(p, ss[u], c[e]);
            }
          }
        }
        if (++acc == F8_ACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (!ok) break;
      if (row_ok) {
        if (args.out_mode == 0) {
          __nv_bfloat16* Cb = reinterpret_cast<__nv_bfloat16*>(args.C) + static_cast<size_t>(row) * args.ldc + n0;
#pragma unroll
          for (int j = 0; j < HC; j += 8) {
            if (n0 + j < N) {
              uint4 o;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) ow[e] = pack_bf16x2(c[j + 2 * e], c[j + 2 * e + 1]);
              *reinterpret_cast<uint4*>(Cb + j) = o;
            }
          }
        } else {
          float* Cf = reinterpret_cast<float*>(args.C) + static_cast<size_t>(row) * args.ldc + n0;
#pragma unroll
          for (int j = 0; j < HC; j += 4) {
            if (n0 + j < N) {
              const float4 v = make_float4(c[j], c[j + 1], c[j + 2], c[j + 3]);
              if (args.out_mode == 2)
                atomicAdd(reinterpret_cast<float4*>(Cf + j), v);
              else
                *reinterpret_cast<float4*>(Cf + j) = v;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, F8_ACC * F8_BN);
  }
}

typedef CUresult (*EncodeTiledFn8)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn8 f8_encode_fn() {
  static EncodeTiledFn8 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn8>(p);
  }
  return fn;
}

// uint8 [rows][K] row-major, box 128 bytes x 128 rows, 128-byte swizzle
static int f8_make_map(CUtensorMap* map, const void* base, uint64_t K, uint64_t rows) {
  EncodeTiledFn8 fn = f8_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int f8_grid(long long threads_needed, int block) {
  long long g = (threads_needed + block - 1) / block;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return static_cast<int>(g);
}

}  // namespace nplm

using namespace nplm;

// x bf16 [R][K] -> q e4m3 [R][K], scales fp32 [K/128][R]
extern "C" int nplm_fp8_quant_rows(const void* x, int R, int K, int ldx, void* q, float* scale,
                                   cudaStream_t stream) {
  if (R <= 0 || K <= 0) return 0;
  if ((K % 128) || (ldx % 8)) return -3;
  const long long threads = static_cast<long long>(R) * (K / 128) * 16;
  quant_rows_kernel<<<f8_grid(threads, 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), R, K, ldx, reinterpret_cast<uint8_t*>(q), scale);
  return static_cast<int>(cudaGetLastError());
}

// 128 x 128 tile quantisation of x bf16 [R][K]; see quant_tile_kernel for the three forms.
//   transpose = 0, block = 1: R, K multiples of 128
//   transpose = 1: K multiple of 128, R multiple of 16 (rows beyond R count as zeros)
extern "C" int nplm_fp8_quant_tile(const void* x, int R, int K, int ldx, int transpose, int block,
                                   void* q, float* scale, cudaStream_t stream) {
  if (R <= 0 || K <= 0) return 0;
  if ((K % 128) || (ldx % 8) || (R % 16)) return -3;
  if (!transpose && (!block || (R % 128))) return -3;
  dim3 grid(K / 128, (R + 127) / 128);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  uint8_t* qp = reinterpret_cast<uint8_t*>(q);
  if (!transpose)
    quant_tile_kernel<false, true><<<grid, 256, 0, stream>>>(xp, R, K, ldx, qp, scale);
  else if (block)
    quant_tile_kernel<true, true><<<grid, 256, 0, stream>>>(xp, R, K, ldx, qp, scale);
  else
    quant_tile_kernel<true, false><<<grid, 256, 0, stream>>>(xp, R, K, ldx, qp, scale);
  return static_cast<int>(cudaGetLastError());
}

// C[M][N] (+)= (A * sa) (B * sb)^T, A e4m3 [M][K], B e4m3 [N][K] (both K-major, K % 128 == 0).
// sa fp32 [K/128][M]; sb fp32 [K/128][N] (b_block = 0) or [K/128][ceil(N/128)] (b_block = 1).
// out_mode 0: bf16 C; 1: fp32 C; 2: fp32 C accumulated with atomics.
extern "C" int nplm_gemm_fp8(const void* A, const void* B, void* C, const float* sa, const float* sb,
                             int M, int N, int K, int ldc, int b_block, int out_mode, int* status,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 128) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (out_mode == 0 ? ((N % 8) || (ldc % 8)) : ((N % 4) || (ldc % 4))) return -5;
  if (!b_block && (N % 4)) return -5;
  CUtensorMap tmA, tmB;
  int rc = f8_make_map(&tmA, A, K, M);
  if (rc) return rc;
  rc = f8_make_map(&tmB, B, K, N);
  if (rc) return rc;
  static bool configured_on[nplm::MAX_DEVICES];
  const int dev_slot = nplm::current_device_slot();
  if (dev_slot < 0) return -4;
  bool& configured = configured_on[dev_slot];
  if (!configured) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM));
    configured = true;
  }
  Fp8Args args;
  args.C = C;
  args.sa = sa;
  args.sb = sb;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.b_block = b_block;
  args.out_mode = out_mode;
  args.status = status;
  args.ag_world = 0;
  args.ag_rank = 0;
  args.ag_rows = 0;
  args.ag_dst = nullptr;
  args.ag_sdst = nullptr;
  args.ag_flags = nullptr;
  for (int r = 0; r < 8; ++r) {
    args.ag_src[r] = nullptr;
    args.ag_ssrc[r] = nullptr;
  }
  const int total = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = total < sms ? total : sms;
  gemm_fp8_kernel<<<grid, F8_THREADS, F8_SMEM, stream>>>(tmA, tmB, args);
  return static_cast<int>(cudaGetLastError());
}

// All-gather fused into the fp8 GEMM. b_ptrs[r] / sb_ptrs[r]: rank r's full-size e4m3 weight buffer
// [N][K] and block-scale buffer [K/128][N/128] in peer-mapped memory; on entry only the rows (and
// scale columns) of shard r are valid in buffer r. N / world must be a multiple of 128. On return
// this rank's buffers hold the whole quantised weight. flags: 8 device words.
extern "C" int nplm_gemm_fp8_ag(const void* A, void* const* b_ptrs, void* C, const float* sa,
                                void* const* sb_ptrs, int M, int N, int K, int ldc, int out_mode,
                                int rank, int world, unsigned* flags, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 2 || world > 8 || rank < 0 || rank >= world || (N % world) || ((N / world) % F8_BN) ||
      (K % 128) || flags == nullptr)
    return -10;
  if (out_mode == 0 ? ((N % 8) || (ldc % 8)) : ((N % 4) || (ldc % 4))) return -5;
  CUtensorMap tmA, tmB;
  int rc = f8_make_map(&tmA, A, K, M);
  if (rc) return rc;
  rc = f8_make_map(&tmB, b_ptrs[rank], K, N);
  if (rc) return rc;
  static bool configured_on[nplm::MAX_DEVICES];
  const int dev_slot = nplm::current_device_slot();
  if (dev_slot < 0) return -4;
  bool& configured = configured_on[dev_slot];
  if (!configured) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM));
    configured = true;
  }
  Fp8Args args;
  args.C = C;
  args.sa = sa;
  args.sb = reinterpret_cast<const float*>(sb_ptrs[rank]);
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.b_block = 1;
  args.out_mode = out_mode;
  args.status = status;
  args.ag_world = world;
  args.ag_rank = rank;
  args.ag_rows = N / world;
  args.ag_dst = reinterpret_cast<uint8_t*>(b_ptrs[rank]);
  args.ag_sdst = reinterpret_cast<float*>(sb_ptrs[rank]);
  args.ag_flags = flags;
  for (int r = 0; r < 8; ++r) {
    args.ag_src[r] = r < world ? reinterpret_cast<const uint8_t*>(b_ptrs[r]) + static_cast<size_t>(r) * args.ag_rows * K
                               : nullptr;
    args.ag_ssrc[r] = r < world ? reinterpret_cast<const float*>(sb_ptrs[r]) : nullptr;
  }
  NPLM_CUDA_CHECK(cudaMemsetAsync(flags, 0, 8 * sizeof(unsigned), stream));
  const int total = ((M + F8_BM - 1) / F8_BM) * (N / F8_BN);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = total < sms ? total : sms;
  void* params[] = {&tmA, &tmB, &args};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(gemm_fp8_kernel), dim3(grid),
                                                      dim3(F8_THREADS), params, F8_SMEM, stream));
}
