// Inference attention with an additive relative-position bias for the T5-style teacher
// (head_dim 64 or 128, non-causal, key-padding mask through per-token key ranges), sm_100a.
//
//   out[t, h, :] = softmax_k( scale * q_t . k_k + bias[h][k - t + S - 1] ) v_k,   k in [seq_start[t], seq_end[t])
//
// Replaces the eager attention of the HF T5 encoder the reference uses as its distillation teacher
// (src/nanoplm/distillation/models/teacher/prott5.py:24-52 loads T5EncoderModel; the bias is T5's
// bucketed relative_attention_bias, shared by all layers). bias is a per-head table indexed by
// the relative position (key - query), built once per forward on the host side of the model.
//
// Same tiling as the training forward in attention.cu: the flat token axis (batch x padded
// length) is cut into 128-token tiles; operands are [128 rows][64 bf16] swizzled tiles loaded by
// TMA (two per operand for head_dim 128), S = Q K^T and O_part = P V run on tcgen05 with fp32
// accumulators in TMEM, the online softmax runs one thread per query row.
//
// Keys are consumed KC at a time: 128 for head_dim 64; 64 for head_dim 128, which keeps a CTA at
// 112 KB of shared memory and 192 TMEM columns so that two CTAs share an SM (the kernel is bound
// by the latency of its MMA -> softmax -> MMA chain, so the second CTA nearly doubles throughput).
// The bias table is read through the read-only cache instead of shared memory for the same reason.
#include "common.cuh"

namespace nplm {

constexpr int AB_T = 128;
constexpr int AB_TILE = AB_T * 64 * 2;  // one [128][64] bf16 tile, 16 KB
constexpr float AB_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t ab_swz(int r, int chunk) {
  return static_cast<uint32_t>(r * 128 + ((chunk ^ (r & 7)) << 4));
}

struct AbArgs {
  __nv_bfloat16* out;    // [T][H*D]
  const int* seq_start;  // [T]
  const int* seq_end;    // [T]
  const float* bias;     // [H][2*S-1], index = key - query + S - 1
  int T, H, S;
  float scale;
  int* status;
};

template <int D, int KC>
constexpr int ab_smem_bytes() {
  // Q + 2 K + 2 V + P + barriers
  return (D / 64) * AB_TILE + 4 * (D / 64) * (KC * 128) + AB_T * KC * 2 + 256;
}

template <int D, int KC>
__global__ void __launch_bounds__(128, 2)
fa_bias_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmKV,
                   const AbArgs args) {
  constexpr int NA = D / 64;              // 64-column atoms per operand tile
  constexpr int QB = NA * AB_TILE;        // bytes of the Q tile (128 rows)
  constexpr int KA = KC * 128;            // bytes of one K / V atom (KC rows x 64 columns)
  constexpr int OP = NA * KA;             // bytes of one K / V tile
  constexpr int PB = AB_T * KC * 2;       // bytes of the P tile (KC / 64 atoms of [128][128 B])
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(args.status, ST_BAD_ARG);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = smem + QB;            // 2 buffers
  uint8_t* sV = smem + QB + 2 * OP;   // 2 buffers
  uint8_t* sP = smem + QB + 4 * OP;   // [KC / 64 key blocks][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + QB + 4 * OP + PB);
  uint64_t* bar_q = bars;
  uint64_t* bar_kv = bars + 1;  // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const float* g_bias = args.bias + static_cast<size_t>(blockIdx.y) * (2 * args.S - 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int T = args.T, H = args.H, S = args.S;
  const int t0 = blockIdx.x * AB_T;
  const int h = blockIdx.y;
  const int HD = H * D;

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
  const uint32_t tS = tmem_base;        // KC columns
  const uint32_t tO = tmem_base + 128;  // D columns

  const int row = t0 + tid;
  const bool row_ok = row < T;
  int lo = 0, hi = 0;
  if (row_ok) {
    lo = args.seq_start[row];
    hi = args.seq_end[row];
  }
  const int last = min(t0 + AB_T - 1, T - 1);
  // key range of the tile: union over its rows (rows of one padded sequence share a range; a tile
  // may span several sequences)
  int kv_lo = args.seq_start[t0], kv_hi = args.seq_end[last];
  {
    int* s_rng = reinterpret_cast<int*>(bars + 6);  // [lo, hi]
    if (tid == 0) {
      s_rng[0] = kv_lo;
      s_rng[1] = kv_hi;
    }
    __syncthreads();
    if (row_ok) {
      atomicMin(&s_rng[0], lo);
      atomicMax(&s_rng[1], hi);
    }
    __syncthreads();
    kv_lo = s_rng[0];
    kv_hi = s_rng[1];
  }
  const int n_kv = kv_hi > kv_lo ? (kv_hi - kv_lo + KC - 1) / KC : 0;

  constexpr uint32_t idesc_s = make_idesc_bf16(128, KC, 0, 0);
  constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
  const int colQ = h * D, colK = HD + h * D, colV = 2 * HD + h * D;

  auto load_q = [&](uint8_t* dst, uint64_t* bar, int col, int r0) {
#pragma unroll
    for (int a = 0; a < NA; ++a) tma_load_2d(dst + a * AB_TILE, &tmQKV, bar, col + a * 64, r0);
  };
  auto load_tile = [&](uint8_t* dst, uint64_t* bar, int col, int r0) {   // KC rows
#pragma unroll
    for (int a = 0; a < NA; ++a) tma_load_2d(dst + a * KA, &tmKV, bar, col + a * 64, r0);
  };
  auto issue_s = [&](int buf) {
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + buf * OP);
#pragma unroll
    for (int k = 0; k < D / 16; ++k)
      umma_bf16(tS, make_smem_desc(qa + (k >> 2) * AB_TILE + (k & 3) * 32, 16, 1024),
                make_smem_desc(ka + (k >> 2) * KA + (k & 3) * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
    umma_commit(bar_s);
  };

  if (tid == 0 && n_kv > 0) {
    mbar_arrive_expect_tx(bar_q, QB);
    load_q(sQ, bar_q, colQ, t0);
    mbar_arrive_expect_tx(&bar_kv[0], 2 * OP);
    load_tile(sK, &bar_kv[0], colK, kv_lo);
    load_tile(sV, &bar_kv[0], colV, kv_lo);
    if (mbar_wait(bar_q, 0) && mbar_wait(&bar_kv[0], 0)) {
      tc_fence_after();
      issue_s(0);
    } else {
      atomicExch(args.status, ST_TIMEOUT_FULL);
      *abort_flag = 1;
    }
  }
  __syncwarp();

  const float sl2 = args.scale * AB_LOG2E;
  const int boff = S - 1 - row;  // bias index = key + boff
  float m_run = -1e30f, l_run = 0.f;
  float o[D];
#pragma unroll
  for (int e = 0; e < D; ++e) o[e] = 0.f;
  const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;

  bool alive = true;
  for (int j = 0; j < n_kv && alive; ++j) {
    const int buf = j & 1;
    const int kv0 = kv_lo + j * KC;
    if (tid == 0 && j + 1 < n_kv) {
      mbar_arrive_expect_tx(&bar_kv[buf ^ 1], 2 * OP);
      load_tile(sK + (buf ^ 1) * OP, &bar_kv[buf ^ 1], colK, kv0 + KC);
      load_tile(sV + (buf ^ 1) * OP, &bar_kv[buf ^ 1], colV, kv0 + KC);
    }
    __syncwarp();
    bool ok = mbar_wait(bar_s, j & 1);
    ok = __syncthreads_and(ok && *abort_flag == 0);
    if (!ok) {
      if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      alive = false;
      break;
    }
    tc_fence_after();

    // pass 1: row maximum of scale * s + bias over the valid keys (log2 domain)
    float tmax = -1e30f;
#pragma unroll 1
    for (int c = 0; c < KC; c += 32) {
      uint32_t r[32];
      tmem_ld32(tS + lane_addr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int col = kv0 + c + e;
        if (col >= lo && col < hi)
          tmax = fmaxf(tmax, fmaf(__uint_as_float(r[e]), sl2, __ldg(g_bias + col + boff) * AB_LOG2E));
      }
    }
    const float m_new = fmaxf(m_run, tmax);
    const float alpha = exp2f(m_run - m_new);
    float psum = 0.f;
    // pass 2: probabilities -> bf16 -> swizzled shared memory
#pragma unroll 1
    for (int c = 0; c < KC; c += 32) {
      uint32_t r[32];
      tmem_ld32(tS + lane_addr + c, r);
      tmem_ld_wait();
      uint32_t packed[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float p[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int col = kv0 + c + e + u;
          p[u] = 0.f;
          if (col >= lo && col < hi)
            p[u] = exp2f(fmaf(__uint_as_float(r[e + u]), sl2, __ldg(g_bias + col + boff) * AB_LOG2E) - m_new);
        }
        psum += p[0] + p[1];
        packed[e >> 1] = pack_bf16x2(p[0], p[1]);
      }
      uint8_t* blk = sP + (c >> 6) * AB_TILE;
      const int chunk0 = ((c >> 5) & 1) * 4;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(blk + ab_swz(tid, chunk0 + q)) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
    }
    l_run = l_run * alpha + psum;
    m_run = m_new;
#pragma unroll
    for (int e = 0; e < D; ++e) o[e] *= alpha;

    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t pa = smem_u32(sP), va = smem_u32(sV + buf * OP);
#pragma unroll
      for (int k = 0; k < KC / 16; ++k)
        umma_bf16(tO, make_smem_desc(pa + (k >> 2) * AB_TILE + (k & 3) * 32, 16, 1024),
                  make_smem_desc(va + k * 2048, KA, 1024), idesc_o, k > 0 ? 1u : 0u);
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
    __syncwarp();
    ok = mbar_wait(bar_o, j & 1);
    ok = __syncthreads_and(ok && *abort_flag == 0);
    if (!ok) {
      if (tid == 0) atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      alive = false;
      break;
    }
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < D; c += 32) {
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
    __nv_bfloat16* dst = args.out + static_cast<size_t>(row) * HD + h * D;
#pragma unroll
    for (int e = 0; e < D; e += 8) {
      uint4 u;
      uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) p[q] = pack_bf16x2(o[e + 2 * q] * inv, o[e + 2 * q + 1] * inv);
      *reinterpret_cast<uint4*>(dst + e) = u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 256);
  }
}

typedef CUresult (*AbEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

static AbEncodeFn ab_encode_fn() {
  static AbEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AbEncodeFn>(p);
  }
  return fn;
}

template <int D, int KC>
static int ab_launch(const CUtensorMap& tmQ, const CUtensorMap& tmKV, const AbArgs& a, cudaStream_t st) {
  constexpr int smem = ab_smem_bytes<D, KC>();
  static bool configured_on[nplm::MAX_DEVICES];
  const int dev_slot = nplm::current_device_slot();
  if (dev_slot < 0) return -4;
  bool& configured = configured_on[dev_slot];
  if (!configured) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bias_fwd_kernel<D, KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  dim3 grid((a.T + AB_T - 1) / AB_T, a.H);
  fa_bias_fwd_kernel<D, KC><<<grid, 128, smem, st>>>(tmQ, tmKV, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace nplm

using namespace nplm;

// qkv bf16 [T][3][H][D]; out bf16 [T][H*D]; bias fp32 [H][2*S-1] with S >= the longest key range.
extern "C" int nplm_fa_bias_fwd(const void* qkv, void* out, const int* seq_start, const int* seq_end,
                                const float* bias, int T, int H, int D, int S, float scale, int* status,
                                cudaStream_t st) {
  if (T <= 0) return 0;
  if ((D != 64 && D != 128) || S < 1 || (reinterpret_cast<uintptr_t>(qkv) & 15)) return -3;
  AbEncodeFn fn = ab_encode_fn();
  if (fn == nullptr) return -1;
  CUtensorMap tmQ, tmKV;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(3) * H * D, static_cast<cuuint64_t>(T)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(3) * H * D * 2};
  cuuint32_t estr[2] = {1, 1};
  const cuuint32_t kc = D == 64 ? 128 : 64;     // key rows per K / V box
  cuuint32_t box_q[2] = {64, AB_T};
  cuuint32_t box_kv[2] = {64, kc};
  if (fn(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides, box_q, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -2;
  if (fn(&tmKV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides, box_kv, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -2;
  AbArgs a;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.seq_start = seq_start;
  a.seq_end = seq_end;
  a.bias = bias;
  a.T = T;
  a.H = H;
  a.S = S;
  a.scale = scale;
  a.status = status;
  return D == 64 ? ab_launch<64, 128>(tmQ, tmKV, a, st) : ab_launch<128, 64>(tmQ, tmKV, a, st);
}
