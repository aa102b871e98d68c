// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA-fed shared-memory pipeline,
// tcgen05.mma with fp32 accumulators in TMEM (double-buffered so the epilogue of tile i
// overlaps the main loop of tile i+1), fused epilogues.
//
//   C[M,N] (+)= op(A) * op(B)^T
//     a_mn = 0 : A stored [M][K] row-major (K contiguous)   -> K-major operand
//     a_mn = 1 : A stored [K][M] row-major (M contiguous)   -> MN-major operand
//     b_mn = 0 : B stored [N][K] row-major                  -> K-major operand
//     b_mn = 1 : B stored [K][N] row-major                  -> MN-major operand
//   With these four forms forward (x W^T), dgrad (dY W) and wgrad (dY^T X) all run
//   without a transposed copy of any tensor.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference
// (src/nanoplm/pretraining/models/modern_bert/modeling.py:281-302,340,366,559).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (each owns the TMEM lane quarter warp_idx % 4).
#include "common.cuh"

namespace nplm {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

enum : int {
  EPI_STORE = 0,       // C(bf16) = acc
  EPI_ADD = 1,         // C(bf16) = acc + R(bf16)
  EPI_ATOMIC_F32 = 2,  // C(fp32) += acc   (split-K capable; used for weight gradients)
  EPI_GELU = 3,        // C(bf16) = act(acc), act = GELU (erf) or ReLU (GemmArgs::act_relu); also writes
                       // the pre-activation to R when R != null
  EPI_STORE_F32 = 4,   // C(fp32) = acc
  EPI_SWIGLU = 5,      // B tile = [value rows | gate rows]; C(bf16, N/2 wide) = silu(gate)*value,
                       // pre-activations (bf16, N wide) written to R
  EPI_RELU = 7,        // host-side alias: EPI_GELU with act_relu = 1
  EPI_ROPE = 6,        // C(bf16) = acc with rotary embedding applied to every 64-wide head whose
                       // first column is < rope_cols (the q and k parts of a fused QKV projection)
  EPI_STORE_DELTA = 9, // C(bf16) = acc, and delta[col / 64][row] = sum over each 64-column head of
                       // bf16(acc) * R (the attention backward's rowsum(dO * O), R = O)
  EPI_SWIGLU_BWD = 8,  // acc = gradient of the SwiGLU output h = silu(gate) * value, N wide;
                       // R = the pre-activations [value | gate] (bf16, 2N wide); C (bf16, 2N wide) =
                       // [acc * silu(gate) | acc * value * silu'(gate)], the gradient of R
};

// PAIR: two CTAs of a cluster (cta_group::2) share one 256 x BN tile; each holds its own 128 rows
// of A and half of B, which cuts the L2 -> shared-memory traffic per FLOP by a third.
// STAGED: the epilogue goes through shared memory (TMA stores); kernels that write straight from
// registers (fp32 outputs, the direct epilogue) spend that room on one more pipeline stage.
template <int BN, bool PAIR = false, bool STAGED = true>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? (STAGED ? 6 : 7) : ((BN == 256) ? 4 : (STAGED ? 6 : 7));
  static constexpr int BAR_BYTES = 256;
  // epilogue staging: 4 warps x 2 buffers x (32 rows x 128 B), written swizzled, read by TMA stores
  static constexpr int EPI_BYTES = STAGED ? 4 * 2 * 4096 : 0;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;  // + alignment slack
};

struct GemmArgs {
  void* C;
  const __nv_bfloat16* R;  // residual (EPI_ADD) or pre-activation output (EPI_GELU / EPI_SWIGLU)
  int M, N, K;
  int ldc, ldr;
  int splits;
  float* delta;     // EPI_STORE_DELTA: fp32 [N / 64][M]
  int swiglu_half;  // EPI_SWIGLU: row offset of the gate half inside B (= N/2)
  int* status;
  // EPI_ROPE: position of every output row, cos / sin tables [max_pos][32] (head_dim 64)
  const int* rope_pos;
  const float* rope_cos;
  const float* rope_sin;
  int rope_cols;
  int act_relu;        // EPI_GELU: 0 = GELU, 1 = ReLU
  // Grouped (mixture-of-experts) forms, one launch for all groups:
  //   group_mode 1: rows of A / C are partitioned into groups in units of 128-row tiles
  //                 (tile_group[m_tile] = group, or -1 for an unused tile); group g multiplies by
  //                 its own B, found b_group_rows * g rows further down the B tensor map.
  //   group_mode 2: weight gradients. A and B are MN-major over a common row axis; group g
  //                 contracts rows [group_off[g], group_off[g+1]) (multiples of 128) and adds the
  //                 M x N result into C + g * c_group_stride.
  int group_mode;
  int groups;
  const int* tile_group;
  // group_mode 1, optional: rows of A arrive from other GPUs. The producer loads the rows of tile t only
  // after row_arrive[t] (bumped once per landed row, system scope) has reached row_expect[t].
  const uint32_t* row_arrive;
  const int* row_expect;
  const int* group_off;
  int b_group_rows;
  long long c_group_stride;
  // All-gather mode (ag_world > 1): B [N][K] is row-sharded over ag_world ranks, ag_rows rows each.
  // The local B buffer holds this rank's rows only; at kernel start the epilogue warps of all CTAs
  // copy the other shards out of the peers' memory (plain P2P loads, each byte crosses NVLink
  // once), bump ag_flags[shard] when their slice of a shard has landed, and the TMA producer waits
  // (bounded) for a shard's flag before it loads the first tile of that shard. Tiles are visited
  // shard by shard, the local shard first, so the copies overlap the first waves of MMAs.
  int ag_world, ag_rank, ag_rows;
  const void* ag_src[8];   // peer r's shard: ag_rows x K, row stride ag_ld elements
  void* ag_dst;            // local full B (row stride ag_ld)
  int ag_ld;
  unsigned* ag_flags;      // [ag_world], zeroed before the launch
};

struct WorkItem {
  int m0, n0, kb0, kb1, b_row;
  long long c_off;
};

// Writes 32 rows x 64 bf16 columns held by one warp (lane = row, packed[0..31] = the 64 values of
// that row) through a swizzled shared-memory buffer with one TMA store. Two buffers per warp
// alternate; a buffer is reused once the store issued two calls earlier has read it. Rows and
// columns beyond the tensor are clipped by the TMA unit.
__device__ __forceinline__ void stage_store_bf16(uint8_t* stage, int& toggle, const CUtensorMap* tm,
                                                 const uint32_t (&packed)[32], int x, int y, int lane) {
  if (lane == 0) tma_store_wait_read<1>();
  __syncwarp();
  uint8_t* buf = stage + toggle * 4096;
  toggle ^= 1;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
        make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tm, buf, x, y);
    tma_store_commit();
  }
}

template <int BN, bool A_MN, bool B_MN, int EPI, bool TMA_EPI, bool PAIR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
                 const GemmArgs args) {
  using S = GemmSmem<BN, PAIR, TMA_EPI>;
  // CTA pair: rank 0 issues the MMAs, both CTAs load operands and run their own epilogue
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int work_first = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int work_stride = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int MT = PAIR ? 2 * BM : BM;   // rows of one work item
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_stage = smem + STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES + S::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* res_bar = bars + 2 * STAGES + 4;  // [4 warps][2 buffers], residual tiles (EPI_ADD)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int M = args.M, N = args.N, K = args.K;
  // For EPI_SWIGLU the logical tile covers BN/2 value columns and BN/2 gate columns.
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  const int n_extent = (EPI == EPI_SWIGLU) ? args.swiglu_half : N;
  const int num_m = (M + MT - 1) / MT;
  const int num_n = (n_extent + TILE_N - 1) / TILE_N;
  const int num_kb = (K + BK - 1) / BK;
  // splits == 0: stream-K. The tiles x k-blocks units are cut into one contiguous, equally long
  // range per worker (CTA or CTA pair); a worker's range covers the tail of one tile, whole tiles
  // and the head of another, and every piece is added to C atomically (EPI_ATOMIC_F32 only).
  const bool stream_k = args.splits == 0;
  const int splits = stream_k ? 1 : args.splits;
  const int kb_per = (num_kb + splits - 1) / splits;
  const long long sk_units = static_cast<long long>(num_m) * num_n * num_kb;
  const long long sk_lo = sk_units * work_first / work_stride;
  const long long sk_hi = sk_units * (work_first + 1) / work_stride;
  const int w_begin = stream_k ? 0 : work_first;
  const int w_step = stream_k ? 1 : work_stride;
  const int total_work = stream_k ? static_cast<int>((sk_hi + num_kb - 1) / num_kb - sk_lo / num_kb)
                                  : (args.group_mode == 2 ? args.groups : splits) * num_m * num_n;

  // work item -> tile coordinates and contraction range; false = nothing to do for this item
  auto decode = [&](int w, WorkItem& it) -> bool {
    it.b_row = 0;
    it.c_off = 0;
    if (args.group_mode == 2) {
      const int per = num_m * num_n;
      const int g = w / per, tile = w % per;
      it.m0 = (tile / num_n) * MT + static_cast<int>(rank) * BM;
      it.n0 = (tile % num_n) * TILE_N;
      it.kb0 = args.group_off[g] / BK;
      it.kb1 = args.group_off[g + 1] / BK;
      it.c_off = static_cast<long long>(g) * args.c_group_stride;
      return it.kb0 < it.kb1;
    }
    if (stream_k) {
      const long long tile = sk_lo / num_kb + w;
      const long long first = tile * num_kb;
      it.m0 = static_cast<int>(tile / num_n) * MT + static_cast<int>(rank) * BM;
      it.n0 = static_cast<int>(tile % num_n) * TILE_N;
      it.kb0 = w == 0 ? static_cast<int>(sk_lo - first) : 0;
      it.kb1 = static_cast<int>(min(sk_hi - first, static_cast<long long>(num_kb)));
      return it.kb0 < it.kb1;
    }
    // tiles run fastest: the CTAs of one wave then walk the same contraction range of different
    // tiles, so an operand panel fetched for one of them serves its whole tile row / column from L2
    const int num_tiles = num_m * num_n;
    const int split = w / num_tiles, tile = w % num_tiles;
    if (args.ag_world > 1) {
      // shard by shard starting with the local one; inside a shard n runs fastest. SwiGLU: output
      // columns [n0, n0 + TILE_N) read value rows n0.. and gate rows swiglu_half + n0.., which live
      // in two shards (v and n_shards + v); the tiles walk the value shards
      const int n_shards = (EPI == EPI_SWIGLU) ? args.swiglu_half / args.ag_rows : args.ag_world;
      const int n_per = args.ag_rows / TILE_N;
      const int per_shard = num_m * n_per;
      const int shard = (args.ag_rank + tile / per_shard) % n_shards;
      const int rem = tile % per_shard;
      it.m0 = (rem / n_per) * BM;
      it.n0 = shard * args.ag_rows + (rem % n_per) * TILE_N;
    } else {
      it.m0 = (tile / num_n) * MT + static_cast<int>(rank) * BM;
      it.n0 = (tile % num_n) * TILE_N;
    }
    it.kb0 = split * kb_per;
    it.kb1 = min(num_kb, it.kb0 + kb_per);
    if (args.group_mode == 1) {
      const int g = args.tile_group[it.m0 / BM];
      if (g < 0) return false;
      it.b_row = g * args.b_group_rows;
    }
    return it.kb0 < it.kb1;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], PAIR ? 8 : 4);   // epilogue warps of both CTAs release rank 0's accumulator
    }
    for (int i = 0; i < 8; ++i) mbar_init(&res_bar[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if constexpr (TMA_EPI) {
      tma_prefetch_desc(&tmC);
      tma_prefetch_desc(&tmR);
    }
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // hands accumulator `a` back to the MMA thread (of rank 0)
  auto release_acc = [&](int a) {
    if constexpr (PAIR) {
      if (rank == 0) mbar_arrive(&tempty_bar[a]);
      else mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[a]), 0));
    } else {
      mbar_arrive(&tempty_bar[a]);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t ag_seen = 0;
      for (int w = w_begin; w < total_work && ok; w += w_step) {
        WorkItem it;
        if (!decode(w, it)) continue;
        const int m0 = it.m0, n0 = it.n0, kb0 = it.kb0, kb1 = it.kb1;
        const int brow = it.b_row;
        if (args.group_mode == 1 && args.row_arrive != nullptr) {
          const int tile = m0 / BM;
          const uint32_t need = static_cast<uint32_t>(args.row_expect[tile]);
          const long long t0 = clock64();
          while (ld_acquire_sys_u32(args.row_arrive + tile) < need) {
            // the senders are other ranks' host threads away (their launch may lag): ten times the usual limit
            if (clock64() - t0 > 10 * WAIT_LIMIT_CYCLES) {
              atomicExch(args.status, ST_TIMEOUT_PEER);
              *abort_flag = 1;
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_global();    // the rows were written with generic stores, TMA reads them
        }
        if (args.ag_world > 1) {
          const int n_need = (EPI == EPI_SWIGLU) ? 2 : 1;
          for (int q = 0; q < n_need && ok; ++q) {
            const int shard = (q == 0 ? n0 : args.swiglu_half + n0) / args.ag_rows;
            if (shard != args.ag_rank && !((ag_seen >> shard) & 1u)) {
              const long long t0 = clock64();
              while (ld_acquire_gpu(args.ag_flags + shard) < gridDim.x) {
                if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                  atomicExch(args.status, ST_TIMEOUT_PEER);
                  *abort_flag = 1;
                  ok = false;
                  break;
                }
                __nanosleep(100);
              }
              if (!ok) break;
              ag_seen |= 1u << shard;
              fence_proxy_async_global();  // the shard was written with generic stores, TMA reads it
            }
          }
          if (!ok) break;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicExch(args.status, ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          const int k0 = kb * BK;
          if constexpr (PAIR) {
            // rank 0's barrier counts the bytes of both CTAs; every CTA loads its own 128 rows of A
            // (m0 already carries the rank offset) and its half of B
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
            if constexpr (!A_MN) {
              tma_load_2d_pair(sa, &tmA, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int g = 0; g < BM / 64; ++g)
                tma_load_2d_pair(sa + g * (BK * 128), &tmA, &full_bar[stage], m0 + g * 64, k0);
            }
            if constexpr (EPI == EPI_SWIGLU) {
              // rank 0 holds the value rows, rank 1 the gate rows of this tile
              tma_load_2d_pair(sb, &tmB, &full_bar[stage], k0,
                               (rank == 0 ? 0 : args.swiglu_half) + n0);
            } else if constexpr (!B_MN) {
              tma_load_2d_pair(sb, &tmB, &full_bar[stage], k0, n0 + static_cast<int>(rank) * (BN / 2));
            } else {
#pragma unroll
              for (int g = 0; g < BN / 128; ++g)
                tma_load_2d_pair(sb + g * (BK * 128), &tmB, &full_bar[stage],
                                 n0 + (static_cast<int>(rank) * (BN / 128) + g) * 64, k0);
            }
          } else {
          mbar_arrive_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g)
              tma_load_2d(sa + g * (BK * 128), &tmA, &full_bar[stage], m0 + g * 64, k0);
          }
          if constexpr (EPI == EPI_SWIGLU) {
            // value rows then gate rows, both K-major
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, brow + n0);
            tma_load_2d(sb + (BN / 2) * 128, &tmB, &full_bar[stage], k0, brow + args.swiglu_half + n0);
          } else if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, brow + n0);
          } else {
#pragma unroll
            for (int g = 0; g < BN / 64; ++g)
              tma_load_2d(sb + g * (BK * 128), &tmB, &full_bar[stage], n0 + g * 64, brow + k0);
          }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && (!PAIR || rank == 0)) {
      constexpr uint32_t idesc = make_idesc_bf16(PAIR ? 2 * BM : BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // arrive-on-completion of everything issued so far; in a pair both CTAs are notified
      auto commit = [&](uint64_t* bar) {
        if constexpr (PAIR) {
          const uint32_t a = smem_u32(bar);
          umma_commit_pair(a);
          umma_commit_pair(mapa_shared(a, 1));
        } else {
          umma_commit(bar);
        }
      };
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = w_begin; w < total_work && ok; w += w_step) {
        WorkItem it;
        if (!decode(w, it)) continue;
        const int kb0 = it.kb0, kb1 = it.kb1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1)) {
          atomicExch(args.status, ST_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicExch(args.status, ST_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024);
            if constexpr (PAIR)
              umma_bf16_pair(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else
              umma_bf16(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          commit(&empty_bar[stage]);  // frees the stage when these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        commit(&tfull_bar[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    if (args.ag_world > 1) {
      // all-gather: this CTA's slice of every remote shard, nearest shard (in visiting order) first
      const int et = threadIdx.x - 64;                       // 0..127 over the four epilogue warps
      const long long row_vecs = args.K / 8;                 // 16-byte vectors per row
      const long long shard_vecs = static_cast<long long>(args.ag_rows) * row_vecs;
      const long long per_cta = (shard_vecs + gridDim.x - 1) / gridDim.x;
      const long long v0 = per_cta * blockIdx.x;
      const long long v1 = min(shard_vecs, v0 + per_cta);
      for (int d = 1; d < args.ag_world; ++d) {
        const int shard = (args.ag_rank + d) % args.ag_world;
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(args.ag_src[shard]);
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(args.ag_dst) +
                             static_cast<size_t>(shard) * args.ag_rows * args.ag_ld;
        for (long long v = v0 + et; v < v1; v += 128) {
          const long long r = v / row_vecs, c = (v % row_vecs) * 8;
          const uint4 val = *reinterpret_cast<const uint4*>(src + r * args.ag_ld + c);
          *reinterpret_cast<uint4*>(dst + r * args.ag_ld + c) = val;
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps only
        if (et == 0) red_release_gpu_add(args.ag_flags + shard, 1u);
      }
    }
    int acc = 0;
    uint32_t acc_phase = 0;
    int stage_toggle = 0;       // which of this warp's two staging buffers is next
    uint32_t res_phase = 0;     // parity bits of this warp's two residual barriers
    for (int w = w_begin; w < total_work; w += w_step) {
      WorkItem it;
      if (!decode(w, it)) continue;
      const int m0 = it.m0, n0 = it.n0;
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) {
        if (lane == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);

      if constexpr (TMA_EPI) {
        // ---- shared-memory staged epilogue, 64 output columns per step, one TMA store each
        uint8_t* stage = epi_stage + quarter * 8192;
        const int y0 = m0 + quarter * 32;
        const bool rows_in = y0 < M;
        if constexpr (EPI == EPI_SWIGLU) {
          constexpr int NCH = BN / 2 / 64;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            uint32_t pv[32], pg[32], po[32];
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
              uint32_t v[32], g[32];
              tmem_ld32(taddr + c * 64 + hlf * 32, v);
              tmem_ld32(taddr + BN / 2 + c * 64 + hlf * 32, g);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const uint32_t a = pack_bf16x2(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
                const uint32_t b = pack_bf16x2(__uint_as_float(g[2 * e]), __uint_as_float(g[2 * e + 1]));
                const float2 vr = unpack_bf16x2(a);
                const float2 gr = unpack_bf16x2(b);
                pv[hlf * 16 + e] = a;
                pg[hlf * 16 + e] = b;
                po[hlf * 16 + e] = pack_bf16x2(gr.x / (1.0f + __expf(-gr.x)) * vr.x,
                                               gr.y / (1.0f + __expf(-gr.y)) * vr.y);
              }
            }
            if (c == NCH - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) release_acc(acc);
            }
            const int x = n0 + c * 64;
            if (rows_in && x < n_extent) {
              stage_store_bf16(stage, stage_toggle, &tmC, po, x, y0, lane);
              if (args.R != nullptr) {
                stage_store_bf16(stage, stage_toggle, &tmR, pv, x, y0, lane);
                stage_store_bf16(stage, stage_toggle, &tmR, pg, args.swiglu_half + x, y0, lane);
              }
            }
          }
        } else if constexpr (EPI == EPI_STORE_DELTA) {
          constexpr int NCH = BN / 64;
          const __nv_bfloat16* orow = args.R + static_cast<size_t>(row_ok ? row : 0) * args.ldr;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            const int x = n0 + c * 64;
            const bool active = rows_in && x < N;
            uint4 ov[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) ov[j] = make_uint4(0, 0, 0, 0);
            if (active && row_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j) ov[j] = __ldg(reinterpret_cast<const uint4*>(orow + x) + j);
            }
            uint32_t packed[32];
            float dot = 0.f;
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
              uint32_t d[32];
              tmem_ld32(taddr + c * 64 + hlf * 32, d);
              tmem_ld_wait();
              if (c == NCH - 1 && hlf == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) release_acc(acc);
              }
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int q = hlf * 16 + e;
                const uint32_t pk = pack_bf16x2(__uint_as_float(d[2 * e]), __uint_as_float(d[2 * e + 1]));
                packed[q] = pk;
                const float2 g2 = unpack_bf16x2(pk);
                const float2 o2 = unpack_bf16x2(reinterpret_cast<const uint32_t*>(&ov[q >> 2])[q & 3]);
                dot += g2.x * o2.x + g2.y * o2.y;
              }
            }
            if (active) {
              stage_store_bf16(stage, stage_toggle, &tmC, packed, x, y0, lane);
              if (row_ok) args.delta[static_cast<size_t>(x >> 6) * M + row] = dot;
            }
          }
        } else if constexpr (EPI == EPI_SWIGLU_BWD) {
          constexpr int NCH = BN / 64;
          const __nv_bfloat16* prow = args.R + static_cast<size_t>(row_ok ? row : 0) * args.ldr;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            const int x = n0 + c * 64;
            const bool active = rows_in && x < N;
            // this lane's 64 value and 64 gate pre-activations: in flight while the accumulator loads
            uint4 vv[8], gg[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              vv[j] = make_uint4(0, 0, 0, 0);
              gg[j] = make_uint4(0, 0, 0, 0);
            }
            if (active && row_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                vv[j] = __ldg(reinterpret_cast<const uint4*>(prow + x) + j);
                gg[j] = __ldg(reinterpret_cast<const uint4*>(prow + N + x) + j);
              }
            }
            uint32_t dvp[32], dgp[32];
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
              uint32_t d[32];
              tmem_ld32(taddr + c * 64 + hlf * 32, d);
              tmem_ld_wait();
              if (c == NCH - 1 && hlf == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) release_acc(acc);
              }
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int q = hlf * 16 + e;   // bf16 pair index inside the 64-column chunk
                const uint32_t vraw = reinterpret_cast<const uint32_t*>(&vv[q >> 2])[q & 3];
                const uint32_t graw = reinterpret_cast<const uint32_t*>(&gg[q >> 2])[q & 3];
                const float2 v2 = unpack_bf16x2(vraw), g2 = unpack_bf16x2(graw);
                const float d0 = __uint_as_float(d[2 * e]), d1 = __uint_as_float(d[2 * e + 1]);
                const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
                dvp[q] = pack_bf16x2(d0 * g2.x * s0, d1 * g2.y * s1);
                dgp[q] = pack_bf16x2(d0 * v2.x * s0 * (1.f + g2.x * (1.f - s0)),
                                     d1 * v2.y * s1 * (1.f + g2.y * (1.f - s1)));
              }
            }
            if (active) {
              stage_store_bf16(stage, stage_toggle, &tmC, dvp, x, y0, lane);
              stage_store_bf16(stage, stage_toggle, &tmC, dgp, N + x, y0, lane);
            }
          }
        } else {
          constexpr int NCH = BN / 64;
          if constexpr (EPI == EPI_ADD) {
            // residual tile of chunk 0 (issued before the accumulator wait would be even better;
            // the tile is already in L2 in the encoder, where the residual is the block input)
            if (lane == 0 && rows_in && n0 < N) {
              tma_store_wait_read<0>();
              mbar_arrive_expect_tx(&res_bar[quarter * 2 + stage_toggle], 4096);
              tma_load_2d(stage + stage_toggle * 4096, &tmR, &res_bar[quarter * 2 + stage_toggle], n0, y0);
            }
            __syncwarp();
          }
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            uint32_t packed[32];
            float f[64];
            {
              uint32_t r0[32], r1[32];
              tmem_ld32(taddr + c * 64, r0);
              tmem_ld32(taddr + c * 64 + 32, r1);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                f[e] = __uint_as_float(r0[e]);
                f[32 + e] = __uint_as_float(r1[e]);
              }
            }
            if (c == NCH - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) release_acc(acc);
            }
            const int x = n0 + c * 64;
            const bool active = rows_in && x < N;
            if constexpr (EPI == EPI_ADD) {
              const int buf = stage_toggle;
              // prefetch the residual of the next chunk into the other buffer
              if (lane == 0 && rows_in && c + 1 < NCH && x + 64 < N) {
                tma_store_wait_read<0>();
                mbar_arrive_expect_tx(&res_bar[quarter * 2 + (buf ^ 1)], 4096);
                tma_load_2d(stage + (buf ^ 1) * 4096, &tmR, &res_bar[quarter * 2 + (buf ^ 1)], x + 64, y0);
              }
              if (active) {
                const bool got = mbar_wait(&res_bar[quarter * 2 + buf], (res_phase >> buf) & 1u);
                res_phase ^= (1u << buf);
                if (!got) {
                  if (lane == 0) atomicExch(args.status, ST_TIMEOUT_MISC);
                } else {
                  uint8_t* rb = stage + buf * 4096;
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const uint4 rv = *reinterpret_cast<const uint4*>(rb + lane * 128 + ((j ^ (lane & 7)) << 4));
                    const uint32_t* rr = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 t = unpack_bf16x2(rr[e]);
                      f[j * 8 + 2 * e] += t.x;
                      f[j * 8 + 2 * e + 1] += t.y;
                    }
                  }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) packed[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
                // in-place: the buffer that held the residual now holds the result
                __syncwarp();
                uint8_t* ob = stage + buf * 4096;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  *reinterpret_cast<uint4*>(ob + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                      make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&tmC, ob, x, y0);
                  tma_store_commit();
                }
                stage_toggle ^= 1;
              }
            } else if constexpr (EPI == EPI_GELU) {
              if (active) {
                uint32_t pre[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  pre[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
                  const float2 t = unpack_bf16x2(pre[e]);
                  packed[e] = args.act_relu ? pack_bf16x2(fmaxf(t.x, 0.f), fmaxf(t.y, 0.f))
                                            : pack_bf16x2(gelu_erf(t.x), gelu_erf(t.y));
                }
                stage_store_bf16(stage, stage_toggle, &tmC, packed, x, y0, lane);
                if (args.R != nullptr) stage_store_bf16(stage, stage_toggle, &tmR, pre, x, y0, lane);
              }
            } else {
              if (active) {
                if constexpr (EPI == EPI_ROPE) {
                  if (x < args.rope_cols) {
                    // this thread holds one whole head (64 channels) of its row: rotate-half RoPE
                    const int rr = y0 + lane;
                    const int pos = rr < M ? args.rope_pos[rr] : 0;
                    const float4* cp = reinterpret_cast<const float4*>(args.rope_cos + static_cast<size_t>(pos) * 32);
                    const float4* sp = reinterpret_cast<const float4*>(args.rope_sin + static_cast<size_t>(pos) * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                      const float4 c4 = cp[q4], s4 = sp[q4];
                      const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                      for (int u = 0; u < 4; ++u) {
                        const int e = q4 * 4 + u;
                        const float a = f[e], b = f[e + 32];
                        f[e] = a * cc[u] - b * ss[u];
                        f[e + 32] = b * cc[u] + a * ss[u];
                      }
                    }
                  }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) packed[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
                stage_store_bf16(stage, stage_toggle, &tmC, packed, x, y0, lane);
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        __nv_bfloat16* Cb = reinterpret_cast<__nv_bfloat16*>(args.C);
        __nv_bfloat16* Pb = const_cast<__nv_bfloat16*>(args.R);
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t v[32], g[32];
          tmem_ld32(taddr + c, v);
          tmem_ld32(taddr + BN / 2 + c, g);
          tmem_ld_wait();
          if (c + 32 >= BN / 2) {
            // last read of this accumulator: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) release_acc(acc);
          }
          const int col = n0 + c;
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < n_extent) {
                uint4 ov, pv, pg;
                uint32_t* o = reinterpret_cast<uint32_t*>(&ov);
                uint32_t* p1 = reinterpret_cast<uint32_t*>(&pv);
                uint32_t* p2 = reinterpret_cast<uint32_t*>(&pg);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float v0 = __uint_as_float(v[j + 2 * e]), v1 = __uint_as_float(v[j + 2 * e + 1]);
                  const float g0 = __uint_as_float(g[j + 2 * e]), g1 = __uint_as_float(g[j + 2 * e + 1]);
                  p1[e] = pack_bf16x2(v0, v1);
                  p2[e] = pack_bf16x2(g0, g1);
                  // activation is computed from the bf16-rounded pre-activations so that the
                  // backward pass (which only sees the stored bf16 values) is consistent
                  const float2 vr = unpack_bf16x2(p1[e]);
                  const float2 gr = unpack_bf16x2(p2[e]);
                  const float s0 = gr.x / (1.0f + __expf(-gr.x));
                  const float s1 = gr.y / (1.0f + __expf(-gr.y));
                  o[e] = pack_bf16x2(s0 * vr.x, s1 * vr.y);
                }
                *reinterpret_cast<uint4*>(Cb + static_cast<size_t>(row) * args.ldc + col + j) = ov;
                if (Pb != nullptr) {
                  *reinterpret_cast<uint4*>(Pb + static_cast<size_t>(row) * args.ldr + col + j) = pv;
                  *reinterpret_cast<uint4*>(Pb + static_cast<size_t>(row) * args.ldr +
                                            args.swiglu_half + col + j) = pg;
                }
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c, r);
          tmem_ld_wait();
          if (c + 32 >= BN) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) release_acc(acc);
          }
          const int col = n0 + c;
          if (row_ok) {
            if constexpr (EPI == EPI_ATOMIC_F32 || EPI == EPI_STORE_F32) {
              float* Cf = reinterpret_cast<float*>(args.C) + it.c_off + static_cast<size_t>(row) * args.ldc;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                if (col + j < N) {
                  float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                         __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                  if constexpr (EPI == EPI_ATOMIC_F32) {
                    atomicAdd(reinterpret_cast<float4*>(Cf + col + j), v);
                  } else {
                    *reinterpret_cast<float4*>(Cf + col + j) = v;
                  }
                }
              }
            } else {
              __nv_bfloat16* Cb =
                  reinterpret_cast<__nv_bfloat16*>(args.C) + static_cast<size_t>(row) * args.ldc;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (col + j < N) {
                  uint4 ov;
                  uint32_t* o = reinterpret_cast<uint32_t*>(&ov);
                  if constexpr (EPI == EPI_ADD) {
                    const uint4 rv = *reinterpret_cast<const uint4*>(
                        args.R + static_cast<size_t>(row) * args.ldr + col + j);
                    const uint32_t* rr = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 f = unpack_bf16x2(rr[e]);
                      o[e] = pack_bf16x2(__uint_as_float(r[j + 2 * e]) + f.x,
                                         __uint_as_float(r[j + 2 * e + 1]) + f.y);
                    }
                  } else if constexpr (EPI == EPI_GELU) {
                    uint4 pv;
                    uint32_t* p = reinterpret_cast<uint32_t*>(&pv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      p[e] = pack_bf16x2(__uint_as_float(r[j + 2 * e]),
                                         __uint_as_float(r[j + 2 * e + 1]));
                      const float2 f = unpack_bf16x2(p[e]);
                      o[e] = args.act_relu ? pack_bf16x2(fmaxf(f.x, 0.f), fmaxf(f.y, 0.f))
                                           : pack_bf16x2(gelu_erf(f.x), gelu_erf(f.y));
                    }
                    if (args.R != nullptr) {
                      *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(args.R) +
                                                static_cast<size_t>(row) * args.ldr + col + j) = pv;
                    }
                  } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                      o[e] = pack_bf16x2(__uint_as_float(r[j + 2 * e]),
                                         __uint_as_float(r[j + 2 * e + 1]));
                  }
                  *reinterpret_cast<uint4*>(Cb + col + j) = ov;
                }
              }
            }
          }
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if constexpr (TMA_EPI) {
      if (lane == 0) tma_store_wait<0>();
      __syncwarp();
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // nobody leaves while the peer may still signal or use this CTA
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D bf16 tensor map, 128-byte swizzle. inner = contiguous extent, outer = rows.
static int make_map_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer,
                       int elem_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt =
      elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int g_num_sms = 0;

static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

struct GemmMaps {
  CUtensorMap A, B, C, R;
  bool tma_epi;
};

template <int BN, bool A_MN, bool B_MN, int EPI, bool TMA_EPI>
static int launch_impl(const GemmMaps& maps, const GemmArgs& args, int max_ctas, cudaStream_t stream) {
  const CUtensorMap& tmA = maps.A;
  const CUtensorMap& tmB = maps.B;
  using S = GemmSmem<BN, false, TMA_EPI>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, EPI, TMA_EPI>;
  static bool configured_on[nplm::MAX_DEVICES];
  const int dev_slot = nplm::current_device_slot();
  if (dev_slot < 0) return -4;
  bool& configured = configured_on[dev_slot];
  if (!configured) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured = true;
  }
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  const int n_extent = (EPI == EPI_SWIGLU) ? args.swiglu_half : args.N;
  const int num_m = (args.M + BM - 1) / BM;
  const int num_n = (n_extent + TILE_N - 1) / TILE_N;
  const long long total = args.splits == 0
                              ? static_cast<long long>(num_m) * num_n * ((args.K + BK - 1) / BK)
                              : static_cast<long long>(num_m) * num_n *
                                    (args.group_mode == 2 ? args.groups : args.splits);
  int grid = total < num_sms() ? static_cast<int>(total) : num_sms();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid <= 0) return 0;
  if (args.ag_world > 1) {
    // CTAs wait on one another's copies: they must all be resident, which a cooperative launch
    // guarantees (it fails instead of running a grid that does not fit)
    if (grid > num_sms()) grid = num_sms();
    void* params[] = {const_cast<CUtensorMap*>(&tmA), const_cast<CUtensorMap*>(&tmB),
                      const_cast<CUtensorMap*>(&maps.C), const_cast<CUtensorMap*>(&maps.R),
                      const_cast<GemmArgs*>(&args)};
    return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(grid),
                                                        dim3(GEMM_THREADS), params, S::TOTAL, stream));
  }
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, maps.C, maps.R, args);
  return static_cast<int>(cudaGetLastError());
}

// CTA-pair form (BN = 256 only): clusters of two CTAs, one 256 x 256 work item per cluster and step.
template <bool A_MN, bool B_MN, int EPI, bool TMA_EPI>
static int launch_pair_impl(const GemmMaps& maps, const GemmArgs& args, cudaStream_t stream) {
  using S = GemmSmem<256, true, TMA_EPI>;
  auto kern = gemm_bf16_kernel<256, A_MN, B_MN, EPI, TMA_EPI, true>;
  static bool configured_on[nplm::MAX_DEVICES];
  const int dev_slot = nplm::current_device_slot();
  if (dev_slot < 0) return -4;
  bool& configured = configured_on[dev_slot];
  if (!configured) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured = true;
  }
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? 128 : 256;
  const int n_extent = (EPI == EPI_SWIGLU) ? args.swiglu_half : args.N;
  const int num_m = (args.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (n_extent + TILE_N - 1) / TILE_N;
  const long long total = static_cast<long long>(num_m) * num_n *
                          (args.splits == 0 ? (args.K + BK - 1) / BK : args.splits);
  int pairs = num_sms() / 2;
  if (pairs > total) pairs = static_cast<int>(total);
  if (pairs <= 0) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, maps.A, maps.B, maps.C, maps.R, args));
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_pair(const GemmMaps& maps, const GemmArgs& args, cudaStream_t stream) {
  if constexpr (EPI == EPI_ROPE) {
    return launch_pair_impl<A_MN, B_MN, EPI, true>(maps, args, stream);
  } else {
    if constexpr (EPI == EPI_STORE || EPI == EPI_ADD || EPI == EPI_GELU || EPI == EPI_SWIGLU) {
      if (maps.tma_epi) return launch_pair_impl<A_MN, B_MN, EPI, true>(maps, args, stream);
    }
    return launch_pair_impl<A_MN, B_MN, EPI, false>(maps, args, stream);
  }
}

template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch(const GemmMaps& maps, const GemmArgs& args, int max_ctas, cudaStream_t stream) {
  if constexpr (EPI == EPI_ROPE || EPI == EPI_SWIGLU_BWD || EPI == EPI_STORE_DELTA) {
    return launch_impl<BN, A_MN, B_MN, EPI, true>(maps, args, max_ctas, stream);
  } else {
    if constexpr (EPI == EPI_STORE || EPI == EPI_ADD || EPI == EPI_GELU || EPI == EPI_SWIGLU) {
      if (maps.tma_epi) return launch_impl<BN, A_MN, B_MN, EPI, true>(maps, args, max_ctas, stream);
    }
    return launch_impl<BN, A_MN, B_MN, EPI, false>(maps, args, max_ctas, stream);
  }
}

}  // namespace nplm

using namespace nplm;

// C ABI entry point. Returns 0 on success, a cudaError_t (>0) or a negative code for bad
// arguments. `status` is a device int the kernel writes a non-zero code to if a bounded wait
// ran out. `max_ctas` (0 = all SMs) caps the grid so a concurrent communication kernel keeps
// some SMs.
struct GroupSpec {
  int mode = 0;
  int groups = 1;
  const int* tile_group = nullptr;
  const uint32_t* row_arrive = nullptr;   // mode 1: per-tile arrival counters and expected rows (optional)
  const int* row_expect = nullptr;
  const int* group_off = nullptr;
  int b_group_rows = 0;
  long long c_group_stride = 0;
  // CTA-pair (cta_group::2) kernel, BN = 256, plain (not grouped / all-gather) GEMMs only
  bool pair = false;
  // all-gather mode
  int ag_world = 0, ag_rank = 0;
  void* const* ag_ptrs = nullptr;  // every rank's full B buffer (this rank's one is B itself)
  unsigned* ag_flags = nullptr;
  float* delta = nullptr;          // EPI_STORE_DELTA side output
};

static int gemm_entry(const void* A, const void* B, void* C, const void* R, int M, int N,
                      int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn,
                      int epi, int splits, int bn, int max_ctas, int direct_epilogue,
                      const int* rope_pos, const float* rope_cos, const float* rope_sin,
                      int rope_cols, int* status, cudaStream_t stream, const GroupSpec& grp) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int act_relu = 0;
  if (epi == EPI_RELU) {
    epi = EPI_GELU;
    act_relu = 1;
  }
  if (grp.mode == 1 && (grp.tile_group == nullptr || grp.groups < 1 || (K % BK) || epi == EPI_ATOMIC_F32))
    return -9;
  if (grp.mode == 2 && (grp.group_off == nullptr || grp.groups < 1 || !a_mn || !b_mn ||
                        (epi != EPI_ATOMIC_F32 && epi != EPI_STORE_F32)))
    return -9;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return -3;
  if (a_mn && (M % 64)) return -4;
  if (b_mn && (N % 64)) return -4;
  if (epi == EPI_SWIGLU && (b_mn || (N % 2) || ((N / 2) % 8))) return -4;
  if ((epi == EPI_ATOMIC_F32 || epi == EPI_STORE_F32) ? (N % 4 || ldc % 4) : (N % 8 || ldc % 8))
    return -5;
  if (bn != 128 && bn != 256) return -6;
  if (epi == EPI_ROPE && (a_mn || b_mn || direct_epilogue || rope_pos == nullptr || rope_cos == nullptr ||
                          rope_sin == nullptr || (rope_cols % 64) || (N % 64)))
    return -7;
  if (epi == EPI_STORE_DELTA && (a_mn || direct_epilogue || R == nullptr || grp.delta == nullptr || (N % 64) ||
                                 (ldr % 8) || (reinterpret_cast<uintptr_t>(R) & 15) || grp.mode != 0 ||
                                 grp.ag_world > 1 || bn != 256))
    return -7;
  if (epi == EPI_SWIGLU_BWD && (a_mn || direct_epilogue || R == nullptr || (N % 64) || (ldr % 8) || (ldc % 8) ||
                                (reinterpret_cast<uintptr_t>(R) & 15) || grp.mode != 0 || grp.ag_world > 1))
    return -7;
  const int num_kb = (K + BK - 1) / BK;
  if (splits < 0) splits = 1;
  if (splits > num_kb) splits = num_kb;
  if (epi != EPI_ATOMIC_F32 || grp.mode != 0) splits = 1;   // splits == 0 (stream-K) adds atomically too
  if (splits == 0 && grp.ag_world > 1) splits = 1;
  // outer (row) extent of the B tensor map: all groups' operands stacked
  const uint64_t b_rows_kmajor = grp.mode == 1 ? static_cast<uint64_t>(grp.b_group_rows) * grp.groups : N;
  const uint64_t b_rows_mnmajor = grp.mode == 1 ? static_cast<uint64_t>(grp.b_group_rows) * grp.groups : K;

  const bool pair = grp.pair && bn == 256 && grp.mode == 0 && grp.ag_world <= 1 && max_ctas == 0 &&
                    !(a_mn && !b_mn) && epi != EPI_SWIGLU_BWD && epi != EPI_STORE_DELTA;
  GemmMaps maps;
  CUtensorMap& tmA = maps.A;
  CUtensorMap& tmB = maps.B;
  int rc;
  if (!a_mn)
    rc = make_map_2d(&tmA, A, K, M, lda, BK, BM, 2);
  else
    rc = make_map_2d(&tmA, A, M, K, lda, 64, BK, 2);
  if (rc) return rc;
  if (epi == EPI_SWIGLU)
    rc = make_map_2d(&tmB, B, K, b_rows_kmajor, ldb, BK, bn / 2, 2);
  else if (!b_mn)
    rc = make_map_2d(&tmB, B, K, b_rows_kmajor, ldb, BK, pair ? bn / 2 : bn, 2);   // a pair CTA loads half of the rows
  else
    rc = make_map_2d(&tmB, B, N, b_rows_mnmajor, ldb, 64, BK, 2);
  if (rc) return rc;
  // staged (TMA store) epilogue for the bf16 outputs; maps C / R describe [32 rows][64 cols] boxes
  maps.tma_epi = !direct_epilogue &&
                 (epi == EPI_STORE || epi == EPI_ADD || epi == EPI_GELU || epi == EPI_SWIGLU || epi == EPI_ROPE ||
                  epi == EPI_SWIGLU_BWD || epi == EPI_STORE_DELTA) &&
                 !(epi == EPI_ADD && (R == nullptr || (reinterpret_cast<uintptr_t>(R) & 15) || (ldr % 8)));
  maps.C = tmA;
  maps.R = tmA;
  if (maps.tma_epi) {
    const int out_cols = epi == EPI_SWIGLU ? N / 2 : (epi == EPI_SWIGLU_BWD ? 2 * N : N);
    rc = make_map_2d(&maps.C, C, out_cols, M, ldc, 64, 32, 2);
    if (rc) return rc;
    if (R != nullptr && epi != EPI_SWIGLU_BWD && epi != EPI_STORE_DELTA) {
      if ((reinterpret_cast<uintptr_t>(R) & 15) || (ldr % 8)) return -3;
      rc = make_map_2d(&maps.R, R, N, M, ldr, 64, 32, 2);
      if (rc) return rc;
    }
  }

  GemmArgs args;
  args.C = C;
  args.R = reinterpret_cast<const __nv_bfloat16*>(R);
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.ldr = ldr;
  args.splits = splits;
  args.delta = grp.delta;
  args.swiglu_half = N / 2;
  args.status = status;
  args.rope_pos = rope_pos;
  args.rope_cos = rope_cos;
  args.rope_sin = rope_sin;
  args.rope_cols = rope_cols;
  args.act_relu = act_relu;
  args.group_mode = grp.mode;
  args.groups = grp.groups;
  args.tile_group = grp.tile_group;
  args.row_arrive = grp.row_arrive;
  args.row_expect = grp.row_expect;
  args.group_off = grp.group_off;
  args.b_group_rows = grp.b_group_rows;
  args.c_group_stride = grp.c_group_stride;
  args.ag_world = grp.ag_world;
  args.ag_rank = grp.ag_rank;
  args.ag_rows = 0;
  args.ag_dst = const_cast<void*>(B);
  args.ag_ld = ldb;
  args.ag_flags = grp.ag_flags;
  for (int r = 0; r < 8; ++r) args.ag_src[r] = nullptr;
  if (grp.ag_world > 1) {
    if (grp.ag_world > 8 || a_mn || b_mn || grp.mode != 0 || epi == EPI_ATOMIC_F32 ||
        grp.ag_ptrs == nullptr || grp.ag_flags == nullptr || (N % grp.ag_world) || (K % 8))
      return -10;
    args.ag_rows = N / grp.ag_world;
    if (epi == EPI_SWIGLU) {
      // value rows and gate rows of a tile come from two different shards: the halves must be
      // whole numbers of shards, and a half-tile (bn / 2 rows) must not straddle two of them
      if ((grp.ag_world % 2) || ((N / 2) % args.ag_rows) || (args.ag_rows % (bn / 2))) return -10;
    } else if (args.ag_rows % bn) {
      return -10;   // a tile must not straddle two shards
    }
    for (int r = 0; r < grp.ag_world; ++r)
      args.ag_src[r] = reinterpret_cast<const __nv_bfloat16*>(grp.ag_ptrs[r]) +
                       static_cast<size_t>(r) * args.ag_rows * ldb;
    NPLM_CUDA_CHECK(cudaMemsetAsync(grp.ag_flags, 0, 8 * sizeof(unsigned), stream));
  }

#define NPLM_DISPATCH_EPI(BN_, AMN_, BMN_)                                                   \
  switch (epi) {                                                                             \
    case EPI_STORE: return launch<BN_, AMN_, BMN_, EPI_STORE>(maps, args, max_ctas, stream); \
    case EPI_ADD: return launch<BN_, AMN_, BMN_, EPI_ADD>(maps, args, max_ctas, stream);     \
    case EPI_ATOMIC_F32:                                                                     \
      return launch<BN_, AMN_, BMN_, EPI_ATOMIC_F32>(maps, args, max_ctas, stream);      \
    case EPI_STORE_F32:                                                                      \
      return launch<BN_, AMN_, BMN_, EPI_STORE_F32>(maps, args, max_ctas, stream);       \
    default: break;                                                                          \
  }

  if (pair) {
#define NPLM_DISPATCH_PAIR(AMN_, BMN_)                                                     \
  switch (epi) {                                                                           \
    case EPI_STORE: return launch_pair<AMN_, BMN_, EPI_STORE>(maps, args, stream);         \
    case EPI_ADD: return launch_pair<AMN_, BMN_, EPI_ADD>(maps, args, stream);             \
    case EPI_ATOMIC_F32: return launch_pair<AMN_, BMN_, EPI_ATOMIC_F32>(maps, args, stream); \
    case EPI_STORE_F32: return launch_pair<AMN_, BMN_, EPI_STORE_F32>(maps, args, stream); \
    default: break;                                                                        \
  }
    if (epi == EPI_GELU || epi == EPI_SWIGLU || epi == EPI_ROPE) {
      if (a_mn || b_mn) return -7;
      if (epi == EPI_GELU) return launch_pair<false, false, EPI_GELU>(maps, args, stream);
      if (epi == EPI_SWIGLU) return launch_pair<false, false, EPI_SWIGLU>(maps, args, stream);
      return launch_pair<false, false, EPI_ROPE>(maps, args, stream);
    }
    if (!a_mn && !b_mn) { NPLM_DISPATCH_PAIR(false, false) }
    else if (!a_mn && b_mn) { NPLM_DISPATCH_PAIR(false, true) }
    else { NPLM_DISPATCH_PAIR(true, true) }
#undef NPLM_DISPATCH_PAIR
    return -8;
  }
  if (epi == EPI_GELU) {
    if (a_mn || b_mn) return -7;
    if (bn == 256) return launch<256, false, false, EPI_GELU>(maps, args, max_ctas, stream);
    return launch<128, false, false, EPI_GELU>(maps, args, max_ctas, stream);
  }
  if (epi == EPI_SWIGLU) {
    if (a_mn || b_mn) return -7;
    if (bn == 256) return launch<256, false, false, EPI_SWIGLU>(maps, args, max_ctas, stream);
    return launch<128, false, false, EPI_SWIGLU>(maps, args, max_ctas, stream);
  }
  if (epi == EPI_ROPE) {
    if (bn == 256) return launch<256, false, false, EPI_ROPE>(maps, args, max_ctas, stream);
    return launch<128, false, false, EPI_ROPE>(maps, args, max_ctas, stream);
  }
  if (epi == EPI_STORE_DELTA) {
    if (b_mn) return launch<256, false, true, EPI_STORE_DELTA>(maps, args, max_ctas, stream);
    return launch<256, false, false, EPI_STORE_DELTA>(maps, args, max_ctas, stream);
  }
  if (epi == EPI_SWIGLU_BWD) {
    if (bn != 256) return -6;
    if (b_mn) return launch<256, false, true, EPI_SWIGLU_BWD>(maps, args, max_ctas, stream);
    return launch<256, false, false, EPI_SWIGLU_BWD>(maps, args, max_ctas, stream);
  }
  if (bn == 256) {
    if (!a_mn && !b_mn) { NPLM_DISPATCH_EPI(256, false, false) }
    else if (!a_mn && b_mn) { NPLM_DISPATCH_EPI(256, false, true) }
    else if (a_mn && b_mn) { NPLM_DISPATCH_EPI(256, true, true) }
    else { NPLM_DISPATCH_EPI(256, true, false) }
  } else {
    if (!a_mn && !b_mn) { NPLM_DISPATCH_EPI(128, false, false) }
    else if (!a_mn && b_mn) { NPLM_DISPATCH_EPI(128, false, true) }
    else if (a_mn && b_mn) { NPLM_DISPATCH_EPI(128, true, true) }
    else { NPLM_DISPATCH_EPI(128, true, false) }
  }
  return -8;
}

extern "C" int nplm_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N,
                              int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn,
                              int epi, int splits, int bn, int max_ctas, int direct_epilogue,
                              const int* rope_pos, const float* rope_cos, const float* rope_sin,
                              int rope_cols, int* status, cudaStream_t stream) {
  return gemm_entry(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, epi, splits, bn, max_ctas,
                    direct_epilogue, rope_pos, rope_cos, rope_sin, rope_cols, status, stream, GroupSpec());
}

// Same GEMM on CTA pairs (tcgen05 cta_group::2): two SMs share every 256 x 256 tile, each loading
// its own rows of A and half of B. bn is 256; unsupported forms fall back to the single-CTA kernel.
extern "C" int nplm_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N,
                                   int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn,
                                   int epi, int splits, int direct_epilogue, const int* rope_pos,
                                   const float* rope_cos, const float* rope_sin, int rope_cols,
                                   int* status, cudaStream_t stream) {
  GroupSpec g;
  g.pair = true;
  return gemm_entry(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, epi, splits, 256, 0,
                    direct_epilogue, rope_pos, rope_cos, rope_sin, rope_cols, status, stream, g);
}

// C = A B^T (b_mn = 0) or A B (b_mn = 1) in bf16, plus delta[h][row] = sum_{64 columns of head h}
// C[row] * R[row] (fp32 [N / 64][M]): the data gradient of the attention output projection and the
// rowsum(dO * O) term of the attention backward in one pass (R = the attention output O).
extern "C" int nplm_gemm_bf16_delta(const void* A, const void* B, void* C, const void* R, float* delta, int M,
                                    int N, int K, int lda, int ldb, int ldc, int ldr, int b_mn, int* status,
                                    cudaStream_t stream) {
  GroupSpec g;
  g.delta = delta;
  return gemm_entry(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, 0, b_mn, EPI_STORE_DELTA, 1, 256, 0, 0, nullptr,
                    nullptr, nullptr, 0, status, stream, g);
}

// Grouped GEMM over row groups (mixture-of-experts forward and data gradient).
//   A [M][K] (rows of all groups, every group padded to whole 128-row tiles), C [M][N] likewise;
//   B holds `groups` operands stacked along its row axis, b_group_rows apart (N rows per group
//   for a K-major B, K rows per group for an MN-major B); tile_group[M / 128] names the group of
//   every row tile (-1 = tile not in use, skipped). K must be a multiple of 64.
// row_arrive / row_expect (both or neither): [M / 128] counters in this GPU's memory that other GPUs
// bump once per row they have stored into A, and the number of rows each tile waits for; the tiles
// of a group start as soon as their own rows have landed (no barrier between the dispatch and
// this GEMM). The wait is bounded (ST_TIMEOUT_PEER).
extern "C" int nplm_gemm_bf16_grouped_gated(const void* A, const void* B, void* C, const void* R, int M,
                                            int N, int K, int lda, int ldb, int ldc, int ldr, int b_mn,
                                            int epi, int bn, int groups, const int* tile_group,
                                            int b_group_rows, const unsigned* row_arrive,
                                            const int* row_expect, int* status, cudaStream_t stream) {
  if ((row_arrive == nullptr) != (row_expect == nullptr)) return -3;
  GroupSpec g;
  g.mode = 1;
  g.groups = groups;
  g.tile_group = tile_group;
  g.b_group_rows = b_group_rows;
  g.row_arrive = row_arrive;
  g.row_expect = row_expect;
  return gemm_entry(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, 0, b_mn, epi, 1, bn, 0, 0, nullptr,
                    nullptr, nullptr, 0, status, stream, g);
}

extern "C" int nplm_gemm_bf16_grouped(const void* A, const void* B, void* C, const void* R, int M,
                                      int N, int K, int lda, int ldb, int ldc, int ldr, int b_mn,
                                      int epi, int bn, int groups, const int* tile_group,
                                      int b_group_rows, int* status, cudaStream_t stream) {
  return nplm_gemm_bf16_grouped_gated(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, b_mn, epi, bn, groups,
                                      tile_group, b_group_rows, nullptr, nullptr, status, stream);
}

// Grouped weight gradient: C_g[M][N] (fp32, += or =) = A[rows_g][M]^T * B[rows_g][N] with
// rows_g = [group_off[g], group_off[g+1]), offsets multiples of 128, `rows` rows in total.
extern "C" int nplm_gemm_bf16_grouped_wgrad(const void* A, const void* B, float* C, int M, int N,
                                            int rows, int lda, int ldb, int ldc, int accumulate,
                                            int bn, int groups, const int* group_off,
                                            long long c_group_stride, int* status,
                                            cudaStream_t stream) {
  GroupSpec g;
  g.mode = 2;
  g.groups = groups;
  g.group_off = group_off;
  g.c_group_stride = c_group_stride;
  return gemm_entry(A, B, C, nullptr, M, N, rows, lda, ldb, ldc, 0, 1, 1,
                    accumulate ? EPI_ATOMIC_F32 : EPI_STORE_F32, 1, bn, 0, 0, nullptr, nullptr,
                    nullptr, 0, status, stream, g);
}

// All-gather fused into the GEMM: C[M][N] = A[M][K] * B[N][K]^T where B is row-sharded over
// `world` ranks. b_ptrs[r] is rank r's full-size B buffer (peer-mapped); on entry only rows
// [r * N/world, (r+1) * N/world) of buffer r are valid. On return this rank's buffer holds all of
// B (the all-gather result, reusable by later GEMMs) and C is complete. flags: 8 device words.
// The caller orders this launch after the peers' writes of their shards (a barrier) and keeps the
// shards unchanged until every rank's launch has finished.
extern "C" int nplm_gemm_bf16_ag_rope(const void* A, void* const* b_ptrs, void* C, const void* R, int M,
                                      int N, int K, int lda, int ldb, int ldc, int ldr, int epi, int bn,
                                      int rank, int world, unsigned* flags, const int* rope_pos,
                                      const float* rope_cos, const float* rope_sin, int rope_cols,
                                      int* status, cudaStream_t stream) {
  GroupSpec g;
  g.ag_world = world;
  g.ag_rank = rank;
  g.ag_ptrs = b_ptrs;
  g.ag_flags = flags;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return -10;
  return gemm_entry(A, b_ptrs[rank], C, R, M, N, K, lda, ldb, ldc, ldr, 0, 0, epi, 1, bn, 0, 0, rope_pos,
                    rope_cos, rope_sin, rope_cols, status, stream, g);
}

extern "C" int nplm_gemm_bf16_ag(const void* A, void* const* b_ptrs, void* C, const void* R, int M, int N,
                                 int K, int lda, int ldb, int ldc, int ldr, int epi, int bn, int rank,
                                 int world, unsigned* flags, int* status, cudaStream_t stream) {
  return nplm_gemm_bf16_ag_rope(A, b_ptrs, C, R, M, N, K, lda, ldb, ldc, ldr, epi, bn, rank, world, flags,
                                nullptr, nullptr, nullptr, 0, status, stream);
}
