// Warp-specialised varlen (cu_seqlens) flash attention for sm_100a, head_dim 64, non-causal,
// optional symmetric sliding window, on packed activations qkv[T][3][H][64] (bf16).
//
// Same interface, tiling of the FLAT token axis and mask semantics as attention.cu (the kernels
// there stay available as the single-role form); what differs is how an SM is kept busy:
//
//   * persistent: one CTA per SM walks a static list of work items (256 query tokens x 1 head),
//     so barrier / TMEM set-up happens once and the loads of item i+1 are in flight while item i
//     is still in its softmax;
//   * roles: two softmax warpgroups own one 128-row query tile each; in a third warpgroup one warp
//     issues every TMA load and one every tcgen05.mma (that warpgroup gives most of its registers
//     to the softmax warpgroups with setmaxnreg). The two tiles share the K / V tiles of the
//     item, and their score / output accumulators (S0, S1, O0, O1) are all resident in TMEM, so
//     the tensor pipe works on one tile's QK^T or PV while the other tile is in its exponentials;
//   * a softmax warpgroup copies its score tile to registers, hands the TMEM tile straight back
//     (the next QK^T runs under this tile's exponentials), writes the bf16 probabilities back to
//     tensor memory (the A operand of the PV product) and only rescales its output accumulator when
//     the running maximum grew by more than 2^8;
//   * nothing on the path of a computing warp waits for global memory: results leave through
//     swizzled staging tiles in shared memory and TMA stores / reduce-adds issued by one thread,
//     and the small loads a warp needs (sequence bounds, row statistics, an item's geometry) are
//     issued one step or one item before their use. Inside these kernels a global load or store on
//     the critical path cost 1 000 - 4 500 cycles (measured with the in-kernel trace below).
//
// Replaces flash_attn_varlen_func as called by the reference
// (src/nanoplm/pretraining/models/modern_bert/modeling.py:331-366) with window (-1,-1) or (64,64).
#include "common.cuh"

namespace nplm {

constexpr int FA_T = 128;                       // tile of tokens (queries and keys)
constexpr int FA_D = 64;                        // head dim
constexpr int FA_TILE_BYTES = FA_T * FA_D * 2;  // 16 KB
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t swz(int r, int chunk) {
  return static_cast<uint32_t>(r * 128 + ((chunk ^ (r & 7)) << 4));
}

struct FaWsArgs {
  __nv_bfloat16* out;   // [T][H*64]
  float* lse;           // [H][T] natural-log LSE of the scaled scores
  const int* seq_start;
  const int* seq_end;
  int T, H, window;     // window < 0: unlimited
  float scale;
  int* status;
};

// Optional in-kernel trace for tuning (compiled in with -DNPLM_WS_TRACE only): when a buffer has been
// registered (nplm_fa_ws_set_trace), CTA 0 records (clock64 << 8 | event) per role: role 0 = MMA
// issuer, 1 / 2 = lane 0 of one warp of two compute warpgroups, 3 = loader. 1024 slots per role, in
// order; the host clears the buffer first and reads up to the first zero.
#ifdef NPLM_WS_TRACE
__device__ long long* g_ws_trace = nullptr;
#define WS_TRACE_INIT()                                                       \
  long long* const tr_base = (blockIdx.x == 0) ? g_ws_trace : nullptr;        \
  int tr_n = 0
#define WS_TRACE(cond, role, ev)                                                        \
  do {                                                                                  \
    if (tr_base != nullptr && (threadIdx.x & 31) == 0 && (cond) && tr_n < 1024)         \
      tr_base[(role) * 1024 + tr_n++] = (clock64() << 8) | (ev);                        \
  } while (0)
#else
#define WS_TRACE_INIT() do { } while (0)
#define WS_TRACE(cond, role, ev) do { } while (0)
#endif

constexpr int WS_KV_STAGES = 3;
constexpr int WS_THREADS = 384;   // 2 softmax warpgroups (warps 0-7), then loader warp 8, MMA warps 9 / 10, 1 idle warp
constexpr int WS_LOADER_WARP = 8, WS_MMA_WARP = 9;
// setmaxnreg: the loader / MMA warpgroup drops to WS_REGS_LIGHT registers per thread, the two
// compute warpgroups grow to WS_REGS_HEAVY. The increase BLOCKS until the CTA's register pool holds
// enough, and the pool is what the launch allocated (168 per thread at 384 threads, the most three
// warps per scheduler can get), not the whole register file: the sum must fit or the kernel hangs.
constexpr int WS_REGS_LAUNCH = 168, WS_REGS_LIGHT = 72, WS_REGS_HEAVY = 216;
static_assert(128 * WS_REGS_LIGHT + 256 * WS_REGS_HEAVY <= WS_THREADS * WS_REGS_LAUNCH,
              "setmaxnreg.inc would wait forever for registers the CTA does not own");
static_assert(WS_REGS_LIGHT % 8 == 0 && WS_REGS_HEAVY % 8 == 0, "setmaxnreg takes multiples of 8");
// Q: 2 buffers x 2 tiles; K, V: WS_KV_STAGES tiles each; P: 2 tiles x 2 column blocks
constexpr int WS_OFF_Q = 0;
constexpr int WS_OFF_K = WS_OFF_Q + 4 * FA_TILE_BYTES;
constexpr int WS_OFF_V = WS_OFF_K + WS_KV_STAGES * FA_TILE_BYTES;
constexpr int WS_OFF_P = WS_OFF_V + WS_KV_STAGES * FA_TILE_BYTES;
constexpr int WS_OFF_BAR = WS_OFF_P + 4 * FA_TILE_BYTES;
constexpr int WS_FWD_SMEM = WS_OFF_BAR + 512;

// Key-tile geometry of one work item: query tiles i = 0, 1 cover tokens [t0 + 128 i, +128); the
// item walks key tiles j = 0 .. n-1 starting at kv_lo, and tile i takes part in j in [a[i], b[i]).
// three-input maximum and packed two-lane fp32 arithmetic (sm_100): half the instructions of the
// scalar forms in the softmax loops
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)),
        "l"(*reinterpret_cast<uint64_t*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}

// Named barrier `id` over 128 threads (one warpgroup) with an AND over everybody's predicate: the
// warps of a warpgroup agree on going on before they meet at plain barriers (a warp that had left
// after a time-out would leave the others there for ever; a leaving warp calls this with false).
__device__ __forceinline__ bool wg_barrier_and(int id, bool p) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred q, o;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "bar.red.and.pred o, %1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, o;\n\t"
      "}"
      : "=r"(r)
      : "r"(id), "r"(static_cast<uint32_t>(p))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void wg_barrier(int id) {
  asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}

struct WsGeo {
  int t0, kv_lo, n;
  int a[2], b[2];
};

// The four loads of an item's geometry: issued by the softmax warpgroups one item ahead.
struct WsGeoRaw {
  int lo[2], hi[2];
};
__device__ __forceinline__ WsGeoRaw ws_geo_load(const FaWsArgs& args, int pair) {
  WsGeoRaw raw;
  const int T = args.T;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int first = pair * 2 * FA_T + i * FA_T;
    raw.lo[i] = raw.hi[i] = 0;
    if (first < T) {
      raw.lo[i] = __ldg(args.seq_start + first);
      raw.hi[i] = __ldg(args.seq_end + min(first + FA_T - 1, T - 1));
    }
  }
  return raw;
}

__device__ __forceinline__ WsGeo ws_geo_make(const FaWsArgs& args, int pair, const WsGeoRaw& raw) {
  WsGeo g;
  const int T = args.T, w = args.window;
  g.t0 = pair * 2 * FA_T;
  int lo[2] = {0, 0}, hi[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int first = g.t0 + i * FA_T;
    if (first < T) {
      const int last = min(first + FA_T - 1, T - 1);
      lo[i] = raw.lo[i];
      hi[i] = raw.hi[i];
      if (w >= 0) {
        lo[i] = max(lo[i], first - w);
        hi[i] = min(hi[i], last + w + 1);
      }
    }
  }
  g.kv_lo = lo[0];
  const int kv_hi = max(hi[0], hi[1]);
  g.n = kv_hi > g.kv_lo ? (kv_hi - g.kv_lo + FA_T - 1) / FA_T : 0;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (hi[i] > lo[i]) {
      g.a[i] = (lo[i] - g.kv_lo) / FA_T;
      g.b[i] = (hi[i] - g.kv_lo + FA_T - 1) / FA_T;
    } else {
      g.a[i] = g.b[i] = 0;
    }
  }
  return g;
}

__device__ __forceinline__ WsGeo ws_geometry(const FaWsArgs& args, int pair) {
  return ws_geo_make(args, pair, ws_geo_load(args, pair));
}

// PTMEM: the probabilities go back to tensor memory (bf16, 64 columns per tile) and the P V product
// reads its A operand from there. The tensor core fetches shared-memory operands at about 64 bytes
// per clock, so a 128 x 64 x 16 instruction with P in shared memory waits 3x longer for operands
// than it computes; with P in tensor memory only the V rows come from shared memory. Without PTMEM
// the probabilities go through a swizzled shared-memory tile (the form the single-role kernels use).
template <bool PTMEM>
__global__ void __launch_bounds__(WS_THREADS, 1)
fa_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmO,
                 const FaWsArgs args) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(args.status, ST_BAD_ARG);
    return;
  }
  uint8_t* sQ = smem + WS_OFF_Q;   // [buf][tile]
  uint8_t* sK = smem + WS_OFF_K;
  uint8_t* sV = smem + WS_OFF_V;
  uint8_t* sP = smem + WS_OFF_P;   // [tile][column block][128 rows][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WS_OFF_BAR);
  uint64_t* q_full = bars;                       // [2]
  uint64_t* q_empty = bars + 2;                  // [2]
  uint64_t* k_full = bars + 4;                   // [WS_KV_STAGES]
  uint64_t* k_empty = k_full + WS_KV_STAGES;
  uint64_t* v_full = k_empty + WS_KV_STAGES;
  uint64_t* v_empty = v_full + WS_KV_STAGES;
  uint64_t* s_full = v_empty + WS_KV_STAGES;     // [2] per query tile
  uint64_t* s_free = s_full + 2;
  uint64_t* p_ready = s_free + 2;
  uint64_t* pv_done = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int T = args.T, H = args.H;
  const int HD = H * FA_D;
  const int n_items = ((T + 2 * FA_T - 1) / (2 * FA_T)) * H;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 2);     // both MMA issuers
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);      // one lane of each softmax warp
      mbar_init(&p_ready[i], 4);     // one lane per softmax warp, after every lane's proxy fence
      mbar_init(&pv_done[i], 1);
    }
    for (int i = 0; i < WS_KV_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);     // both MMA issuers
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQKV);
  }
  if (warp == WS_MMA_WARP) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S0 [0,128), S1 [128,256), O0 [256,320), O1 [320,384), P0 [384,448), P1 [448,512)
  WS_TRACE_INIT();

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WS_REGS_LIGHT));
  if (warp == WS_LOADER_WARP) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      uint32_t qc = 0, kc = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const int h = item % H;
        const WsGeo g = ws_geometry(args, item / H);
        const int colQ = h * FA_D, colK = HD + h * FA_D, colV = 2 * HD + h * FA_D;
        const uint32_t qb = qc & 1u;
        if (!mbar_wait(&q_empty[qb], ((qc >> 1) & 1u) ^ 1u)) { ok = false; break; }
        const int nq = (g.b[0] > g.a[0] ? 1 : 0) + (g.b[1] > g.a[1] ? 1 : 0);
        mbar_arrive_expect_tx(&q_full[qb], nq * FA_TILE_BYTES);
        if (g.b[0] > g.a[0]) tma_load_2d(sQ + (qb * 2 + 0) * FA_TILE_BYTES, &tmQKV, &q_full[qb], colQ, g.t0);
        if (g.b[1] > g.a[1]) tma_load_2d(sQ + (qb * 2 + 1) * FA_TILE_BYTES, &tmQKV, &q_full[qb], colQ, g.t0 + FA_T);
        for (int j = 0; j < g.n; ++j, ++kc) {
          const uint32_t st = kc % WS_KV_STAGES, ph = (kc / WS_KV_STAGES) & 1u;
          const int kv0 = g.kv_lo + j * FA_T;
          if (!mbar_wait(&k_empty[st], ph ^ 1u)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[st], FA_TILE_BYTES);
          tma_load_2d(sK + st * FA_TILE_BYTES, &tmQKV, &k_full[st], colK, kv0);
          WS_TRACE(true, 3, 1);
          if (!mbar_wait(&v_empty[st], ph ^ 1u)) { ok = false; break; }
          mbar_arrive_expect_tx(&v_full[st], FA_TILE_BYTES);
          tma_load_2d(sV + st * FA_TILE_BYTES, &tmQKV, &v_full[st], colV, kv0);
        }
        ++qc;
        if (*abort_flag) ok = false;
      }
      if (!ok && *abort_flag == 0) {
        atomicExch(args.status, ST_TIMEOUT_EMPTY);
        *abort_flag = 1;
      }
    }
  } else if (warp == WS_MMA_WARP || warp == WS_MMA_WARP + 1) {
    // ------------------------------------------------------------------ MMA issuers
    // One issuing thread per query tile: the two tiles then advance independently (a tile whose
    // probabilities are late does not hold back the other tile's next score tile), and the issue
    // work of a step (12 instructions per tile) is spread over two schedulers. Descriptors of a
    // tile are formed once; a step inside a tile only adds to the 14-bit address field.
    if (lane == 0) {
      const int i = warp - WS_MMA_WARP;
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
      uint32_t qc = 0, kc = 0;
      uint32_t s_cnt = 0, p_cnt = 0;
      bool ok = true;
      int why = ST_TIMEOUT_FULL;
      const uint32_t tS = tmem_base + i * 128;
      const uint32_t tO = tmem_base + 256 + i * 64;
      const uint64_t dP0 = make_smem_desc(smem_u32(sP + i * 2 * FA_TILE_BYTES), 16, 1024);
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const WsGeo g = ws_geometry(args, item / H);
        const uint32_t qb = qc & 1u;
        if (!mbar_wait(&q_full[qb], (qc >> 1) & 1u)) { ok = false; break; }
        const uint64_t dQ0 = make_smem_desc(smem_u32(sQ + (qb * 2 + i) * FA_TILE_BYTES), 16, 1024);
        for (int j = 0; j <= g.n && ok; ++j) {
          if (j < g.n) {   // scores of key tile j
            const uint32_t st = (kc + j) % WS_KV_STAGES, ph = ((kc + j) / WS_KV_STAGES) & 1u;
            if (!mbar_wait(&k_full[st], ph)) { ok = false; break; }
            WS_TRACE(true, 0, 1);
            if (j >= (i ? g.a[1] : g.a[0]) && j < (i ? g.b[1] : g.b[0])) {
              // the warpgroup holds the previous score tile in registers
              if (!mbar_wait(&s_free[i], (s_cnt & 1u) ^ 1u)) { ok = false; why = ST_TIMEOUT_TMEM_EMPTY; break; }
              tc_fence_after();
              const uint64_t dK0 = make_smem_desc(smem_u32(sK + st * FA_TILE_BYTES), 16, 1024);
#pragma unroll
              for (int k = 0; k < FA_D / 16; ++k)   // 32 bytes along the row per 16 channels
                umma_bf16(tS, dQ0 + 2 * k, dK0 + 2 * k, idesc_s, k > 0 ? 1u : 0u);
              umma_commit(&s_full[i]);
              ++s_cnt;
              WS_TRACE(true, 0, 2);
            }
            // both issuers release the stage (a commit with nothing outstanding arrives at once)
            umma_commit(&k_empty[st]);
            if (j == g.n - 1) umma_commit(&q_empty[qb]);
          }
          if (j >= 1) {    // output update with key tile j - 1
            const int jj = j - 1;
            const uint32_t st = (kc + jj) % WS_KV_STAGES, ph = ((kc + jj) / WS_KV_STAGES) & 1u;
            if (!mbar_wait(&v_full[st], ph)) { ok = false; break; }
            if (jj >= (i ? g.a[1] : g.a[0]) && jj < (i ? g.b[1] : g.b[0])) {
              if (!mbar_wait(&p_ready[i], p_cnt & 1u)) { ok = false; why = ST_TIMEOUT_MISC; break; }
              WS_TRACE(true, 0, 3);
              tc_fence_after();
              const uint64_t dV0 = make_smem_desc(smem_u32(sV + st * FA_TILE_BYTES), 8192, 1024);
              if constexpr (PTMEM) {
#pragma unroll
                for (int k = 0; k < FA_T / 16; ++k)   // P: 8 columns per 16 keys; V: 16 key rows = 2048 bytes
                  umma_bf16_ts(tO, tmem_base + 384 + i * 64 + k * 8, dV0 + k * (2048 >> 4), idesc_o,
                               (jj > (i ? g.a[1] : g.a[0]) || k > 0) ? 1u : 0u);
              } else {
#pragma unroll
                for (int k = 0; k < FA_T / 16; ++k)   // P: 32 bytes per 16 keys, next column block after 4;
                                                      // V: 16 key rows = 2048 bytes
                  umma_bf16(tO, dP0 + ((k >> 2) * (FA_TILE_BYTES >> 4) + (k & 3) * 2), dV0 + k * (2048 >> 4),
                            idesc_o, (jj > (i ? g.a[1] : g.a[0]) || k > 0) ? 1u : 0u);
              }
              umma_commit(&pv_done[i]);
              ++p_cnt;
              WS_TRACE(true, 0, 4);
            }
            umma_commit(&v_empty[st]);
          }
        }
        kc += g.n;
        ++qc;
        if (*abort_flag) ok = false;
      }
      if (!ok && *abort_flag == 0) {
        atomicExch(args.status, why);
        *abort_flag = 1;
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WS_REGS_HEAVY));
    const int i = warp >> 2;                // query tile of this warpgroup
    const int quarter = warp & 3;           // TMEM lane quarter this warp may access
    const int row_local = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + i * 128 + lane_addr;
    const uint32_t tO = tmem_base + 256 + i * 64 + lane_addr;
    uint8_t* sPi = sP + i * 2 * FA_TILE_BYTES;
    const float sl2 = args.scale * LOG2E;
    const uint32_t NEG_INF = 0xff800000u;
    const int w = args.window;
    uint32_t s_cnt = 0, pv_cnt = 0;
    bool ok = true;
    const bool st_issuer = quarter == 0 && lane == 0;     // issues this warpgroup's output stores
    // geometry and key range of an item's rows are loaded one item ahead (a global load at an item
    // boundary cost 1 000 - 4 500 cycles inside this kernel)
    WsGeoRaw raw_n = ws_geo_load(args, blockIdx.x / H);
    int lo_n = 0, hi_n = 0;
    {
      const int row0 = (static_cast<int>(blockIdx.x) / H) * 2 * FA_T + i * FA_T + row_local;
      if (row0 < T) {
        lo_n = __ldg(args.seq_start + row0);
        hi_n = __ldg(args.seq_end + row0);
      }
    }
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int h = item % H;
      const WsGeo g = ws_geo_make(args, item / H, raw_n);
      const int row = g.t0 + i * FA_T + row_local;
      const bool row_ok = row < T;
      int lo = lo_n, hi = hi_n;  // this row attends to keys [lo, hi)
      if (row_ok && w >= 0) {
        lo = max(lo, row - w);
        hi = min(hi, row + w + 1);
      }
      if (item + static_cast<int>(gridDim.x) < n_items) {
        const int pair_n = (item + gridDim.x) / H;
        raw_n = ws_geo_load(args, pair_n);
        const int row_n = pair_n * 2 * FA_T + i * FA_T + row_local;
        lo_n = hi_n = 0;
        if (row_n < T) {
          lo_n = __ldg(args.seq_start + row_n);
          hi_n = __ldg(args.seq_end + row_n);
        }
      }
      if ((i ? g.b[1] : g.b[0]) <= (i ? g.a[1] : g.a[0])) continue;
      float m_used = -1e30f, l_run = 0.f;
      for (int j = (i ? g.a[1] : g.a[0]); j < (i ? g.b[1] : g.b[0]); ++j) {
        const int kv0 = g.kv_lo + j * FA_T;
        ok = mbar_wait(&s_full[i], s_cnt & 1u);
        ++s_cnt;
        ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
        if (!ok) break;
        WS_TRACE(quarter == 0, 1 + i, 1);
        tc_fence_after();
        const bool none = (kv0 + FA_T <= lo) || (kv0 >= hi);
        const bool warp_none = __all_sync(0xffffffffu, none);
        // 32-key chunks that no row of this warp can see (keys of other sequences, or outside the
        // window of all 32 rows): no mask, maximum or exponential, their probabilities are zero
        uint32_t dead = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int c_lo = kv0 + c * 32;
          if (__all_sync(0xffffffffu, c_lo >= hi || c_lo + 32 <= lo)) dead |= 1u << c;
        }
        uint32_t r[FA_T];
        if (!warp_none) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
          tmem_ld_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[i]);   // the score tile may be overwritten
        WS_TRACE(quarter == 0, 1 + i, 2);

        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (!warp_none) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if ((dead >> c) & 1u) continue;
            const int c_lo = kv0 + c * 32, c_hi = c_lo + 32;
            if (!(c_lo >= lo && c_hi <= hi)) {
              // bit e of `bits`: key c_lo + e lies inside the row's range [lo, hi). One mask word per
              // 32 keys instead of two comparisons per key.
              const int a = max(lo - c_lo, 0), b = min(hi - c_lo, 32);
              const uint32_t bits = b > a ? (0xffffffffu >> (32 - (b - a))) << a : 0u;
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (!(bits & (1u << e))) r[c * 32 + e] = NEG_INF;
            }
#pragma unroll
            for (int e = 0; e < 32; e += 2)
              mx[(e >> 1) & 3] = fmax3(mx[(e >> 1) & 3], __uint_as_float(r[c * 32 + e]),
                                       __uint_as_float(r[c * 32 + e + 1]));
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
        if (j > (i ? g.a[1] : g.a[0])) {
          // the previous output update has finished: the P tile is free and O may be rescaled
          ok = mbar_wait(&pv_done[i], pv_cnt & 1u);
          ++pv_cnt;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          WS_TRACE(quarter == 0, 1 + i, 4);
          tc_fence_after();
          if (warp_need) {
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
              uint32_t o[32];
              tmem_ld32(tO + hlf * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
              tmem_st32(tO + hlf * 32, o);
            }
            tmem_st_wait();
          }
        }
        l_run *= alpha;

        const float moff = m_used * sl2;
        float ps[4] = {0.f, 0.f, 0.f, 0.f};
        const float2 sl2v = make_float2(sl2, sl2), noffv = make_float2(-moff, -moff);
        float2 ps2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        if constexpr (PTMEM) {
          // probabilities packed in place: word c of r[] takes keys 2c, 2c + 1 (both already consumed)
          if (!warp_none) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if ((dead >> q) & 1u) {
#pragma unroll
                for (int c = q * 16; c < q * 16 + 16; ++c) r[c] = 0u;
              } else {
#pragma unroll
                for (int c = q * 16; c < q * 16 + 16; ++c) {
                  const float2 x = fma2(make_float2(__uint_as_float(r[2 * c]), __uint_as_float(r[2 * c + 1])),
                                        sl2v, noffv);
                  const float2 p = make_float2(exp2f(x.x), exp2f(x.y));
                  ps2[c & 1] = add2(ps2[c & 1], p);
                  r[c] = pack_bf16x2(p.x, p.y);
                }
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 64; ++c) r[c] = 0u;
          }
          const uint32_t tP = tmem_base + 384 + i * 64 + lane_addr;
          tmem_st32(tP, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_st32(tP + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_st_wait();
          l_run += ((ps2[0].x + ps2[0].y) + (ps2[1].x + ps2[1].y)) + ((ps[0] + ps[1]) + (ps[2] + ps[3]));
          tc_fence_before();
        } else {
          if (!warp_none) {
#pragma unroll
            for (int c8 = 0; c8 < 16; ++c8) {
              uint32_t pk[4] = {0u, 0u, 0u, 0u};
              if (!((dead >> (c8 >> 2)) & 1u)) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float p0 = exp2f(fmaf(__uint_as_float(r[c8 * 8 + 2 * q]), sl2, -moff));
                  const float p1 = exp2f(fmaf(__uint_as_float(r[c8 * 8 + 2 * q + 1]), sl2, -moff));
                  ps[q] += p0 + p1;
                  pk[q] = pack_bf16x2(p0, p1);
                }
              }
              *reinterpret_cast<uint4*>(sPi + (c8 >> 3) * FA_TILE_BYTES + swz(row_local, c8 & 7)) =
                  make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          } else {
#pragma unroll
            for (int c8 = 0; c8 < 16; ++c8)
              *reinterpret_cast<uint4*>(sPi + (c8 >> 3) * FA_TILE_BYTES + swz(row_local, c8 & 7)) =
                  make_uint4(0u, 0u, 0u, 0u);
          }
          l_run += (ps[0] + ps[1]) + (ps[2] + ps[3]);
          fence_proxy_async_smem();
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[i]);
        WS_TRACE(quarter == 0, 1 + i, 3);
      }
      if (ok) {
        // last output update of this item
        ok = mbar_wait(&pv_done[i], pv_cnt & 1u);
        ++pv_cnt;
        ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
      }
      if constexpr (PTMEM) {
        // The output tile leaves through this warpgroup's 16 KB of the (otherwise unused) P area and one
        // TMA store: the warpgroup goes on to its next item while the copy engine writes the rows.
        if (st_issuer && ok) tma_store_wait_read<0>();     // the previous item's store has read the tile
        ok = wg_barrier_and(1 + i, ok);                    // (a warp that gives up says so here)
        if (!ok) break;
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t o[32];
          tmem_ld32(tO + hlf * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 u;
            uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              p[q] = pack_bf16x2(__uint_as_float(o[e + 2 * q]) * inv, __uint_as_float(o[e + 2 * q + 1]) * inv);
            *reinterpret_cast<uint4*>(sPi + swz(row_local, hlf * 4 + (e >> 3))) = u;
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        wg_barrier(1 + i);
        if (st_issuer) {                                   // rows past the end of the batch are clipped
          tma_store_2d(&tmO, sPi, h * FA_D, g.t0 + i * FA_T);
          tma_store_commit();
        }
        if (row_ok)
          args.lse[static_cast<size_t>(h) * T + row] = l_run > 0.f ? m_used * args.scale + __logf(l_run) : 0.f;
        WS_TRACE(quarter == 0, 1 + i, 5);
        continue;
      }
      if (!ok) break;
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = args.out + static_cast<size_t>(row) * HD + h * FA_D;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t o[32];
        tmem_ld32(tO + hlf * 32, o);
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
      tc_fence_before();
      if (row_ok)
        args.lse[static_cast<size_t>(h) * T + row] = l_run > 0.f ? m_used * args.scale + __logf(l_run) : 0.f;
      WS_TRACE(quarter == 0, 1 + i, 5);
    }
    if (PTMEM && st_issuer) tma_store_wait<0>();   // the stores are complete before the CTA gives up its shared memory
    if (!ok && lane == 0 && *abort_flag == 0) {
      atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == WS_MMA_WARP) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------- backward
// One work item = one 128-key tile of one head; the item streams the query tiles that can see it.
// Every thread of the NWG compute warpgroups owns one query row of the current tile (row statistics
// lse / delta and the row's key range are plain registers); warpgroup g handles key columns
// [g 128 / NWG, +128 / NWG) of S = Q K^T and dP = dO V^T (TMEM, [query lanes][key columns]).
//   P = exp2(S * scale * log2e - lse * log2e) inside the row's key range, dS = P (dP - delta)
//   -> bf16 tiles [query rows][key columns] in shared memory, dS also as bf16 pairs in tensor memory ->
//   dV += P^T dO, dK += dS^T Q (TMEM-resident across the item), dQ = dS K (dS from tensor memory).
// The loader runs ahead by up to two query tiles and one key tile; S / dP of step j + 1 are
// issued as soon as the warpgroups hold step j in registers.
// With four compute warpgroups a further (drain) warpgroup takes every result out of tensor memory:
// each step's dQ tile goes through a staging tile in shared memory into the fp32 accumulator with TMA
// reduce-adds (issued as vector atomics from the SM instead, the adds filled the load / store path,
// and the row data of the next step, four small loads per thread, waited about 3 000 cycles behind
// them in every step), and at the end of an item dK / dV (the item's dQ in the query-stationary
// launch) go through the staging tiles and TMA stores into dqkv while the compute warpgroups are
// already on the next item. With two compute warpgroups (NPLM_FA_BWD_MODE=2) the compute warps add
// dQ with vector atomics and store dK / dV themselves.
struct FaWsBwdArgs {
  __nv_bfloat16* dqkv;   // [T][3][H][64]: the kernel writes the dK and dV parts
  float* dq_acc;         // [T][H*64] fp32, zero-initialised by the caller
  const float* lse;      // [H][T]
  const float* delta;    // [H][T]
  const int* seq_start;
  const int* seq_end;
  int T, H, window;
  float scale;
  int* status;
  const int* rope_pos;   // optional: q / k were rotated before the forward pass
  const float* rope_cos; // [max_pos][32]
  const float* rope_sin;
};

constexpr int WSB_Q_STAGES = 2;
constexpr int WSB_OFF_K = 0;                                   // [2]
constexpr int WSB_OFF_V = WSB_OFF_K + 2 * FA_TILE_BYTES;       // [2]
constexpr int WSB_OFF_Q = WSB_OFF_V + 2 * FA_TILE_BYTES;       // [WSB_Q_STAGES]
constexpr int WSB_OFF_DO = WSB_OFF_Q + WSB_Q_STAGES * FA_TILE_BYTES;
constexpr int WSB_OFF_P = WSB_OFF_DO + WSB_Q_STAGES * FA_TILE_BYTES;   // [2 key blocks][128 q rows][128 B]
constexpr int WSB_OFF_DS = WSB_OFF_P + 2 * FA_TILE_BYTES;
constexpr int WSB_OFF_DQ = WSB_OFF_DS + 2 * FA_TILE_BYTES;   // [2 channel halves][128 q rows][32 fp32] staging of a dQ tile
constexpr int WSB_OFF_BAR = WSB_OFF_DQ + 2 * FA_TILE_BYTES;
constexpr int WS_BWD_SMEM = WSB_OFF_BAR + 512;

struct WsBwdGeo {
  int kv0, q_lo, q_hi, n_q;
};

// The two loads of an item's geometry, and the arithmetic on them, apart: the compute warpgroups issue
// the loads of the NEXT item early and use them a few thousand cycles later (a global load on the
// critical path of an item boundary cost 1 000 - 4 500 cycles inside this kernel).
__device__ __forceinline__ void ws_bwd_geo_load(const FaWsBwdArgs& args, int kt, int& a, int& b) {
  const int kv0 = kt * FA_T;
  a = __ldg(args.seq_start + kv0);
  b = __ldg(args.seq_end + min(kv0 + FA_T - 1, args.T - 1));
}

__device__ __forceinline__ WsBwdGeo ws_bwd_geo_make(const FaWsBwdArgs& args, int kt, int a, int b) {
  WsBwdGeo g;
  const int T = args.T, w = args.window;
  g.kv0 = kt * FA_T;
  const int last = min(g.kv0 + FA_T - 1, T - 1);
  g.q_lo = a;
  g.q_hi = b;
  if (w >= 0) {
    g.q_lo = max(g.q_lo, g.kv0 - w);
    g.q_hi = min(g.q_hi, last + w + 1);
  }
  g.n_q = g.q_hi > g.q_lo ? (g.q_hi - g.q_lo + FA_T - 1) / FA_T : 0;
  return g;
}

__device__ __forceinline__ WsBwdGeo ws_bwd_geometry(const FaWsBwdArgs& args, int kt) {
  WsBwdGeo g;
  const int T = args.T, w = args.window;
  g.kv0 = kt * FA_T;
  const int last = min(g.kv0 + FA_T - 1, T - 1);
  g.q_lo = __ldg(args.seq_start + g.kv0);
  g.q_hi = __ldg(args.seq_end + last);
  if (w >= 0) {
    g.q_lo = max(g.q_lo, g.kv0 - w);
    g.q_hi = min(g.q_hi, last + w + 1);
  }
  g.n_q = g.q_hi > g.q_lo ? (g.q_hi - g.q_lo + FA_T - 1) / FA_T : 0;
  return g;
}

// NWG compute warpgroups share the key columns of a step: warpgroup g handles columns
// [g * 128 / NWG, +128 / NWG) of every query row. Four warpgroups put four compute warps on every
// scheduler (the per-element work has no cross-thread dependency, so the split is free) at 104
// registers per thread; two warpgroups run at 216.
// DQ: also form dQ = dS K per step and add it to the fp32 accumulator. Without it the kernel produces
// dK / dV only and dQ comes from the query-stationary launch (MODE 2 below: no atomics, no scratch,
// bitwise reproducible).
// With four compute warpgroups a further (drain) warpgroup does nothing but move results out of tensor
// memory: staging tiles in shared memory, then TMA reduce-adds (dQ tiles) or TMA stores (dK / dV, the
// item's dQ in the query-stationary launch) issued by one of its threads.
template <int NWG, bool DQ>
struct WsBwdCfg {
  static constexpr bool DRAIN_WG = NWG == 4;
  static constexpr int THREADS = (NWG + 1 + (DRAIN_WG ? 1 : 0)) * 128;
  static constexpr int LOADER_WARP = NWG * 4, MMA_WARP = NWG * 4 + 1, DRAIN_WARP = NWG * 4 + 4;
  static constexpr int CPT = FA_T / NWG;              // key columns per thread
  // registers per thread the launch allocates: the most a scheduler's share of the warps allows
  static constexpr int REGS_LAUNCH = NWG == 2 ? 168 : (DRAIN_WG ? 80 : 96);
  static constexpr int REGS_LIGHT = NWG == 2 ? 72 : (DRAIN_WG ? 48 : 56);   // loader / MMA issuers
  static constexpr int REGS_DRAIN = 48;                                     // dQ / dK / dV drain warpgroup
  static constexpr int REGS_HEAVY = NWG == 2 ? 216 : (DRAIN_WG ? 96 : 104);
  static_assert(128 * REGS_LIGHT + (DRAIN_WG ? 128 * REGS_DRAIN : 0) + NWG * 128 * REGS_HEAVY <= THREADS * REGS_LAUNCH,
                "setmaxnreg.inc would wait forever for registers the CTA does not own");
};

// MODE 0: key-stationary, dK / dV only. MODE 1: key-stationary, dK / dV and dQ through atomics.
// MODE 2: QUERY-stationary: an item is one 128-query tile, the key tiles that can see it stream by,
// and dQ accumulates in tensor memory over the whole item; at the end warpgroup 0 scales it, rotates
// it back and stores bf16 straight into dqkv. Same loads, same S / dP products and the same
// per-element code with the two sides swapped (the mask is symmetric); no dK / dV, no atomics, no
// scratch. MODE 0 + MODE 2 together are the bitwise-reproducible backward pass.
constexpr int BWD_KV = 0, BWD_KV_DQ = 1, BWD_Q = 2;

template <int NWG, int MODE>
__global__ void __launch_bounds__(WsBwdCfg<NWG, MODE == BWD_KV_DQ>::THREADS, 1)
fa_bwd_ws_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmOUT,
                 const FaWsBwdArgs args) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(args.status, ST_BAD_ARG);
    return;
  }
  uint8_t* sK = smem + WSB_OFF_K;
  uint8_t* sV = smem + WSB_OFF_V;
  uint8_t* sQ = smem + WSB_OFF_Q;
  uint8_t* sdO = smem + WSB_OFF_DO;
  uint8_t* sP = smem + WSB_OFF_P;
  uint8_t* sdS = smem + WSB_OFF_DS;
  uint8_t* sDQ = smem + WSB_OFF_DQ;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WSB_OFF_BAR);
  uint64_t* kv_full = bars;                        // [2]
  uint64_t* kv_empty = bars + 2;                   // [2]
  uint64_t* qdo_full = bars + 4;                   // [WSB_Q_STAGES]
  uint64_t* qdo_empty = qdo_full + WSB_Q_STAGES;
  uint64_t* sdp_full = qdo_empty + WSB_Q_STAGES;   // S and dP of a step are in TMEM
  uint64_t* sdp_free = sdp_full + 1;               // the warpgroups hold them in registers
  uint64_t* pds_ready = sdp_free + 1;              // P and dS of a step are in shared memory
  uint64_t* g_done = pds_ready + 1;                // dV, dK, dQ of a step have finished
  uint64_t* dq_free = g_done + 1;                  // the dQ tile has been read back
  uint64_t* acc_free = dq_free + 1;                // dK / dV of the previous item have been read back
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  constexpr bool DQ = MODE == BWD_KV_DQ, QST = MODE == BWD_Q;
  using Cfg = WsBwdCfg<NWG, DQ>;
  constexpr int CPT = Cfg::CPT;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int T = args.T, H = args.H;
  const int HD = H * FA_D;
  const int n_items = ((T + FA_T - 1) / FA_T) * H;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], DQ ? 2 : 1);   // issuer A, and C when it reads K from the item's buffer
    }
    for (int i = 0; i < WSB_Q_STAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 2);           // issuers A and B (query-stationary: A and C)
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, NWG * 4);   // one lane of each compute warp
    mbar_init(pds_ready, NWG * 4);     // one lane per compute warp, after every lane's proxy fence
    mbar_init(g_done, DQ ? 2 : 1);           // issuer B, and C when both run (query-stationary: C alone)
    mbar_init(dq_free, (Cfg::DRAIN_WG || QST) ? 4 : NWG * 4);   // the warps that read dQ back
    mbar_init(acc_free, Cfg::DRAIN_WG ? 4 : 8);   // the warps that read dK / dV back
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == Cfg::MMA_WARP) {
    __syncwarp();
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;          // S   [q][kv] 128 columns
  const uint32_t tdP = tmem_base + 128;   // dP  [q][kv] 128 columns
  const uint32_t tdQ = tmem_base + 256;   // dQ  [q][d]   64 columns
  const uint32_t tdK = tmem_base + 320;   // dK  [kv][d]  64 columns
  const uint32_t tdV = tmem_base + 384;   // dV  [kv][d]  64 columns
  const uint32_t tdS = tmem_base + 448;   // dS  [q][kv]  bf16, two keys per column: 64 columns (A operand of dQ)
  WS_TRACE_INIT();

  if (warp >= NWG * 4) {
  if (Cfg::DRAIN_WG && warp >= Cfg::DRAIN_WARP) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_DRAIN));
    // ------------------------------------------------------------------ dQ drain warpgroup
    // thread = query row of the step's tile: waits for the step's products, copies the row's 64 channels
    // out of tensor memory (scaled) into the staging tile and hands the tensor-memory tile back; one
    // thread then adds the staging tile into the fp32 accumulator with two TMA reduce-adds (32 channels
    // = one 128-byte swizzled row each). Rows the item's queries do not reach hold zeros (their
    // probabilities are masked), rows past the end of the batch are clipped by the tensor map.
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool issuer = warp == Cfg::DRAIN_WARP && lane == 0;
    uint32_t c_g = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int h = item % H;
      const WsBwdGeo g = ws_bwd_geometry(args, item / H);
      for (int j = 0; j < g.n_q; ++j) {
        ok = mbar_wait(g_done, c_g & 1u);
        ++c_g;
        // the previous tile's reduce-adds have finished reading the staging tile
        if (issuer) tma_store_wait_read<0>();
        // barrier over the warpgroup that also agrees on going on: all four warps leave together (a warp
        // that stayed behind would leave the others at the second barrier below for ever)
        ok = wg_barrier_and(1, ok && *abort_flag == 0);
        if (!ok) break;
        tc_fence_after();
        if constexpr (DQ) {
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {     // 32 channels at a time: this warpgroup runs on few registers
          uint32_t v[32];
          tmem_ld32(tdQ + lane_addr + hlf * 32, v);
          tmem_ld_wait();
          if (hlf == 1) {                       // both halves have left tensor memory
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_free);
          }
          uint8_t* row = sDQ + hlf * FA_TILE_BYTES + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(row + (((c ^ (r & 7))) << 4)) =
                make_float4(__uint_as_float(v[4 * c]) * args.scale, __uint_as_float(v[4 * c + 1]) * args.scale,
                            __uint_as_float(v[4 * c + 2]) * args.scale, __uint_as_float(v[4 * c + 3]) * args.scale);
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          const int q0 = g.q_lo + j * FA_T;
          tma_reduce_add_2d(&tmDQ, sDQ, h * FA_D, q0);
          tma_reduce_add_2d(&tmDQ, sDQ + FA_TILE_BYTES, h * FA_D + 32, q0);
          tma_store_commit();
        }
        }
      }
      if (!ok) break;
      // ---- the item's dK and dV: the last products have finished (the wait above covered them). This
      // warpgroup, not the compute warpgroups, moves them out: thread = key row kv0 + r, 16 + 16 channels
      // at a time (channel e and its rotation partner e + 32), scaled and rotated back (dK), packed to
      // bf16 into the two halves of the staging area laid out as TMA boxes, then two TMA stores into
      // dqkv. The compute warpgroups are already working on the next item meanwhile.
      if (issuer) tma_store_wait_read<0>();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      {
        const int krow = g.kv0 + r;
        const bool rot = args.rope_pos != nullptr && krow < T;
        const int pos = rot ? __ldg(args.rope_pos + krow) : 0;
        constexpr int N_OUT = QST ? 1 : 2;                 // query-stationary: the item's dQ instead
#pragma unroll
        for (int which = 0; which < N_OUT; ++which) {      // 0: dK (dQ when QST), 1: dV
          const uint32_t src = (QST ? tdQ : (which == 0 ? tdK : tdV)) + lane_addr;
          uint8_t* row = sDQ + which * FA_TILE_BYTES + r * 128;
#pragma unroll
          for (int grp = 0; grp < 4; ++grp) {              // channels [8 grp, +8) and their partners + 32
            uint32_t a[8], b[8];
            if (g.n_q > 0) {
              tmem_ld8(src + grp * 8, a);
              tmem_ld8(src + 32 + grp * 8, b);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) a[e] = b[e] = 0u;
            }
            if (which == N_OUT - 1 && grp == 3) {          // everything has left tensor memory
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(QST ? dq_free : acc_free);
            }
            float fa[8], fb[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              fa[e] = __uint_as_float(a[e]);
              fb[e] = __uint_as_float(b[e]);
            }
            if (which == 0) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                fa[e] *= args.scale;
                fb[e] *= args.scale;
              }
              if (rot) {
                const float4* cp = reinterpret_cast<const float4*>(args.rope_cos + static_cast<size_t>(pos) * 32) + grp * 2;
                const float4* sp = reinterpret_cast<const float4*>(args.rope_sin + static_cast<size_t>(pos) * 32) + grp * 2;
#pragma unroll
                for (int q4 = 0; q4 < 2; ++q4) {
                  const float4 c4 = __ldg(cp + q4), s4 = __ldg(sp + q4);
                  const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
                  const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const int e = q4 * 4 + u;
                    const float x = fa[e], y = fb[e];
                    fa[e] = x * cc[u] + y * ss[u];
                    fb[e] = y * cc[u] - x * ss[u];
                  }
                }
              }
            }
            // 8 channels = one 16-byte chunk of the row: chunk grp, and chunk 4 + grp for the partners
            *reinterpret_cast<uint4*>(row + ((grp ^ (r & 7)) << 4)) =
                make_uint4(pack_bf16x2(fa[0], fa[1]), pack_bf16x2(fa[2], fa[3]), pack_bf16x2(fa[4], fa[5]),
                           pack_bf16x2(fa[6], fa[7]));
            *reinterpret_cast<uint4*>(row + (((4 + grp) ^ (r & 7)) << 4)) =
                make_uint4(pack_bf16x2(fb[0], fb[1]), pack_bf16x2(fb[2], fb[3]), pack_bf16x2(fb[4], fb[5]),
                           pack_bf16x2(fb[6], fb[7]));
          }
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (issuer) {
        if constexpr (QST) {
          tma_store_2d(&tmOUT, sDQ, h * FA_D, g.kv0);
        } else {
          tma_store_2d(&tmOUT, sDQ, HD + h * FA_D, g.kv0);
          tma_store_2d(&tmOUT, sDQ + FA_TILE_BYTES, 2 * HD + h * FA_D, g.kv0);
        }
        tma_store_commit();
      }
    }
    if (issuer) tma_store_wait<0>();            // the adds are complete before the CTA gives up its shared memory
    if (!ok && lane == 0 && *abort_flag == 0) {
      atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      *abort_flag = 1;
    }
  } else {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_LIGHT));   // all four warps of the warpgroup
  if (warp == Cfg::LOADER_WARP) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      uint32_t ic = 0, qc = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
        const int h = item % H;
        const WsBwdGeo g = ws_bwd_geometry(args, item / H);
        const uint32_t kb = ic & 1u;
        if (!mbar_wait(&kv_empty[kb], ((ic >> 1) & 1u) ^ 1u)) { ok = false; break; }
        mbar_arrive_expect_tx(&kv_full[kb], 2 * FA_TILE_BYTES);
        // item buffer: the stationary pair (K, V of the key tile; query-stationary: Q, dO of the query tile)
        if constexpr (QST) {
          tma_load_2d(sK + kb * FA_TILE_BYTES, &tmQKV, &kv_full[kb], h * FA_D, g.kv0);
          tma_load_2d(sV + kb * FA_TILE_BYTES, &tmDO, &kv_full[kb], h * FA_D, g.kv0);
        } else {
          tma_load_2d(sK + kb * FA_TILE_BYTES, &tmQKV, &kv_full[kb], HD + h * FA_D, g.kv0);
          tma_load_2d(sV + kb * FA_TILE_BYTES, &tmQKV, &kv_full[kb], 2 * HD + h * FA_D, g.kv0);
        }
        for (int j = 0; j < g.n_q; ++j, ++qc) {
          const uint32_t st = qc % WSB_Q_STAGES, ph = (qc / WSB_Q_STAGES) & 1u;
          if (!mbar_wait(&qdo_empty[st], ph ^ 1u)) { ok = false; break; }
          mbar_arrive_expect_tx(&qdo_full[st], 2 * FA_TILE_BYTES);
          // ring: the streamed pair (Q, dO; query-stationary: K, V)
          if constexpr (QST) {
            tma_load_2d(sQ + st * FA_TILE_BYTES, &tmQKV, &qdo_full[st], HD + h * FA_D, g.q_lo + j * FA_T);
            tma_load_2d(sdO + st * FA_TILE_BYTES, &tmQKV, &qdo_full[st], 2 * HD + h * FA_D, g.q_lo + j * FA_T);
          } else {
            tma_load_2d(sQ + st * FA_TILE_BYTES, &tmQKV, &qdo_full[st], h * FA_D, g.q_lo + j * FA_T);
            tma_load_2d(sdO + st * FA_TILE_BYTES, &tmDO, &qdo_full[st], h * FA_D, g.q_lo + j * FA_T);
          }
        }
        if (*abort_flag) ok = false;
      }
      if (!ok && *abort_flag == 0) {
        atomicExch(args.status, ST_TIMEOUT_EMPTY);
        *abort_flag = 1;
      }
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------------ MMA issuers
    // Three issuing threads, one per kind of product, so that a step's 24 - 32 instructions do not
    // queue behind one thread: A issues S = Q K^T and dP = dO V^T of the NEXT step as soon as the
    // warpgroups hold the current one in registers; B issues dV += P^T dO and dK += dS^T Q; C issues
    // dQ = dS K (only with DQ). Descriptors are formed once per buffer; a step adds to the address
    // field. Buffers read by several issuers are released by all of them (barrier counts).
    const int role = warp - Cfg::MMA_WARP;            // 0 = A, 1 = B, 2 = C
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    constexpr uint32_t idesc_g = make_idesc_bf16(128, 64, 1, 1);   // A MN-major, B MN-major
    constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, 0, 1);  // A K-major, B MN-major
    uint32_t ic = 0, qc = 0;       // items, query steps started so far
    uint32_t c_sdp = 0, c_pds = 0, c_dq = 0;
    bool ok = true;
    int why = ST_TIMEOUT_FULL;
    if (role == 0) {
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
        const WsBwdGeo g = ws_bwd_geometry(args, item / H);
        const uint32_t kb = ic & 1u;
        if (!mbar_wait(&kv_full[kb], (ic >> 1) & 1u)) { ok = false; break; }
        const uint64_t dK0 = make_smem_desc(smem_u32(sK + kb * FA_TILE_BYTES), 16, 1024);
        const uint64_t dV0 = make_smem_desc(smem_u32(sV + kb * FA_TILE_BYTES), 16, 1024);
        for (int j = 0; j < g.n_q; ++j) {
          const uint32_t step = qc + j;
          const uint32_t st = step % WSB_Q_STAGES, ph = (step / WSB_Q_STAGES) & 1u;
          if (!mbar_wait(&qdo_full[st], ph)) { ok = false; break; }
          if (!mbar_wait(sdp_free, (c_sdp & 1u) ^ 1u)) { ok = false; why = ST_TIMEOUT_TMEM_EMPTY; break; }
          tc_fence_after();
          const uint64_t dQ0 = make_smem_desc(smem_u32(sQ + st * FA_TILE_BYTES), 16, 1024);
          const uint64_t dO0 = make_smem_desc(smem_u32(sdO + st * FA_TILE_BYTES), 16, 1024);
          // S[q][kv] = Q K^T, dP[q][kv] = dO V^T: the query side is the A operand. Key-stationary: the
          // ring holds (Q, dO), the item buffer (K, V); query-stationary: the other way round
#pragma unroll
          for (int k = 0; k < FA_D / 16; ++k)
            umma_bf16(tS, (QST ? dK0 : dQ0) + 2 * k, (QST ? dQ0 : dK0) + 2 * k, idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < FA_D / 16; ++k)
            umma_bf16(tdP, (QST ? dV0 : dO0) + 2 * k, (QST ? dO0 : dV0) + 2 * k, idesc_s, k > 0 ? 1u : 0u);
          umma_commit(sdp_full);
          ++c_sdp;
          umma_commit(&qdo_empty[st]);     // with issuer B
          WS_TRACE(true, 0, 1);
        }
        if (!ok) break;
        umma_commit(&kv_empty[kb]);        // with issuer C when dQ is formed here
        qc += g.n_q;
        if (*abort_flag) ok = false;
      }
    } else if (role == 1 && !QST) {
      const uint64_t dPT = make_smem_desc(smem_u32(sP), FA_TILE_BYTES, 1024);    // P^T / dS^T as MN-major A
      const uint64_t dST = make_smem_desc(smem_u32(sdS), FA_TILE_BYTES, 1024);
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
        const WsBwdGeo g = ws_bwd_geometry(args, item / H);
        for (int j = 0; j < g.n_q; ++j) {
          const uint32_t step = qc + j;
          const uint32_t st = step % WSB_Q_STAGES;
          if (!mbar_wait(pds_ready, c_pds & 1u)) { ok = false; why = ST_TIMEOUT_MISC; break; }
          ++c_pds;
          WS_TRACE(true, 3, 2);
          if (j == 0 && !mbar_wait(acc_free, (ic & 1u) ^ 1u)) { ok = false; why = ST_TIMEOUT_TMEM_EMPTY; break; }
          tc_fence_after();
          const uint64_t dQ0 = make_smem_desc(smem_u32(sQ + st * FA_TILE_BYTES), 8192, 1024);   // MN-major B
          const uint64_t dO0 = make_smem_desc(smem_u32(sdO + st * FA_TILE_BYTES), 8192, 1024);
#pragma unroll
          for (int k = 0; k < FA_T / 16; ++k)   // dV[kv][d] += P^T[kv][q] dO[q][d]; 16 query rows = 2048 bytes
            umma_bf16(tdV, dPT + k * 128, dO0 + k * 128, idesc_g, (j > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < FA_T / 16; ++k)   // dK[kv][d] += dS^T[kv][q] Q[q][d]
            umma_bf16(tdK, dST + k * 128, dQ0 + k * 128, idesc_g, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(g_done);                 // with issuer C when dQ is formed here
          umma_commit(&qdo_empty[st]);
          WS_TRACE(true, 3, 3);
        }
        if (!ok) break;
        qc += g.n_q;
        if (*abort_flag) ok = false;
      }
    } else if (role == 2 && DQ) {
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
        const WsBwdGeo g = ws_bwd_geometry(args, item / H);
        const uint32_t kb = ic & 1u;
        if (!mbar_wait(&kv_full[kb], (ic >> 1) & 1u)) { ok = false; break; }
        const uint64_t dK0 = make_smem_desc(smem_u32(sK + kb * FA_TILE_BYTES), 8192, 1024);     // MN-major B
        for (int j = 0; j < g.n_q; ++j) {
          if (!mbar_wait(pds_ready, c_pds & 1u)) { ok = false; why = ST_TIMEOUT_MISC; break; }
          ++c_pds;
          if (!mbar_wait(dq_free, (c_dq & 1u) ^ 1u)) { ok = false; why = ST_TIMEOUT_TMEM_EMPTY; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < FA_T / 16; ++k)   // dQ[q][d] = dS[q][kv] K[kv][d], dS read from tensor memory
            umma_bf16_ts(tdQ, tdS + k * 8, dK0 + k * 128, idesc_dq, k > 0 ? 1u : 0u);
          ++c_dq;
          umma_commit(g_done);
        }
        if (!ok) break;
        umma_commit(&kv_empty[kb]);
        if (*abort_flag) ok = false;
      }
    }
    else if (role == 2 && QST) {
      // dQ[q][d] += dS[q][kv] K[kv][d] over the item's key tiles (K = ring slot 0, read MN-major)
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
        const WsBwdGeo g = ws_bwd_geometry(args, item / H);
        for (int j = 0; j < g.n_q; ++j) {
          const uint32_t step = qc + j;
          const uint32_t st = step % WSB_Q_STAGES, ph = (step / WSB_Q_STAGES) & 1u;
          if (!mbar_wait(pds_ready, c_pds & 1u)) { ok = false; why = ST_TIMEOUT_MISC; break; }
          ++c_pds;
          if (!mbar_wait(&qdo_full[st], ph)) { ok = false; break; }
          // the previous item's dQ has been read back before this item's first product overwrites it
          if (j == 0 && !mbar_wait(dq_free, (ic & 1u) ^ 1u)) { ok = false; why = ST_TIMEOUT_TMEM_EMPTY; break; }
          tc_fence_after();
          const uint64_t dKr = make_smem_desc(smem_u32(sQ + st * FA_TILE_BYTES), 8192, 1024);
#pragma unroll
          for (int k = 0; k < FA_T / 16; ++k)
            umma_bf16_ts(tdQ, tdS + k * 8, dKr + k * 128, idesc_dq, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(g_done);
          umma_commit(&qdo_empty[st]);     // with issuer A
        }
        if (!ok) break;
        qc += g.n_q;
        if (*abort_flag) ok = false;
      }
    }
    if (!ok && *abort_flag == 0) {
      atomicExch(args.status, why);
      *abort_flag = 1;
    }
  }
  }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_HEAVY));
    const int gh = warp >> 2;               // key-column slice of this warpgroup
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;      // query row inside the tile (= key row for dK / dV)
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = args.scale * LOG2E;
    const int w = args.window;
    uint32_t c_sdp = 0, c_g = 0;
    bool ok = true;

    // row statistics and key range of query row q of head h (zeros / empty range past T)
    struct RowInfo { float lse2, delta; int klo, khi; };
    auto fetch_row = [&](int q, int h) -> RowInfo {
      RowInfo ri{0.f, 0.f, 0, 0};
      if (q < T) {
        ri.lse2 = __ldg(args.lse + static_cast<size_t>(h) * T + q) * LOG2E;
        ri.delta = __ldg(args.delta + static_cast<size_t>(h) * T + q);
        ri.klo = __ldg(args.seq_start + q);
        ri.khi = __ldg(args.seq_end + q);
        if (w >= 0) {
          ri.klo = max(ri.klo, q - w);
          ri.khi = min(ri.khi, q + w + 1);
        }
      }
      return ri;
    };
    // dQ tile of the step whose query rows start at q0: this thread adds its share of the channels of row q0 + r
    auto drain_dq = [&](int q0, int q_hi, int h) {
      if constexpr (DQ && !Cfg::DRAIN_WG) {
        constexpr int DQC = FA_D / NWG;       // dQ channels per thread
        uint32_t v[DQC];
        if constexpr (DQC == 32) tmem_ld32(tdQ + lane_addr + gh * DQC, v);
        else tmem_ld16(tdQ + lane_addr + gh * DQC, v);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_free);
        const int q = q0 + r;
        if (q < T && q < q_hi) {
          float* dst = args.dq_acc + static_cast<size_t>(q) * HD + h * FA_D + gh * DQC;
#pragma unroll
          for (int e = 0; e < DQC; e += 4)
            atomicAdd(reinterpret_cast<float4*>(dst + e),
                      make_float4(__uint_as_float(v[e]) * args.scale, __uint_as_float(v[e + 1]) * args.scale,
                                  __uint_as_float(v[e + 2]) * args.scale, __uint_as_float(v[e + 3]) * args.scale));
        }
      }
    };

    // Geometry and first row data of an item are fetched during the item before it.
    WsBwdGeo g_cur{0, 0, 0, 0};
    RowInfo first{0.f, 0.f, 0, 0};
    if (static_cast<int>(blockIdx.x) < n_items) {
      g_cur = ws_bwd_geometry(args, blockIdx.x / H);
      first = fetch_row((QST ? g_cur.kv0 : g_cur.q_lo) + r, blockIdx.x % H);
    }
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int h = item % H;
      const WsBwdGeo g = g_cur;
      const int item_n = item + gridDim.x;
      int gn_a = 0, gn_b = 0;
      if (item_n < n_items) ws_bwd_geo_load(args, item_n / H, gn_a, gn_b);   // used in the item's last step
      // key-stationary: the query row changes with every step; query-stationary: one row per item
      RowInfo nxt = first;
      for (int j = 0; j < g.n_q; ++j) {
        const int q0 = g.q_lo + j * FA_T;      // first row of the streamed tile (queries, or keys when QST)
        const RowInfo ri = nxt;
        if (!QST && j + 1 < g.n_q) nxt = fetch_row(q0 + FA_T + r, h);
        if (j == g.n_q - 1 && item_n < n_items) {
          g_cur = ws_bwd_geo_make(args, item_n / H, gn_a, gn_b);
          first = fetch_row((QST ? g_cur.kv0 : g_cur.q_lo) + r, item_n % H);
        }
        ok = mbar_wait(sdp_full, c_sdp & 1u);
        ++c_sdp;
        ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
        if (!ok) break;
        WS_TRACE(warp == 0 || warp == NWG * 4 - 1, warp == 0 ? 1 : 2, 1);
        tc_fence_after();
        uint32_t rs[CPT], rp[CPT];
#pragma unroll
        for (int c = 0; c < CPT; c += 32) {
          tmem_ld32(tS + lane_addr + gh * CPT + c, *reinterpret_cast<uint32_t(*)[32]>(&rs[c]));
          tmem_ld32(tdP + lane_addr + gh * CPT + c, *reinterpret_cast<uint32_t(*)[32]>(&rp[c]));
        }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_free);
        WS_TRACE(warp == 0 || warp == NWG * 4 - 1, warp == 0 ? 1 : 2, 2);
        if (j > 0) {
          // the previous step's dV / dK / dQ have finished: P / dS tiles are free, dQ can be read
          ok = mbar_wait(g_done, c_g & 1u);
          ++c_g;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          WS_TRACE(warp == 0 || warp == NWG * 4 - 1, warp == 0 ? 1 : 2, 4);
          tc_fence_after();
          drain_dq(q0 - FA_T, g.q_hi, h);
        }
        // keys of this thread's columns: [c0, c0 + CPT)
        const int c0 = (QST ? q0 : g.kv0) + gh * CPT;
        const bool inside = __all_sync(0xffffffffu, c0 >= ri.klo && c0 + CPT <= ri.khi);
        const bool outside = __all_sync(0xffffffffu, c0 >= ri.khi || c0 + CPT <= ri.klo);
        // first 16-byte chunk of this thread: column block (gh * CPT) / 64, chunk ((gh * CPT) % 64) / 8
        uint8_t* rowP = sP + ((gh * CPT) >> 6) * FA_TILE_BYTES + r * 128;
        uint8_t* rowS = sdS + ((gh * CPT) >> 6) * FA_TILE_BYTES + r * 128;
        const int chunk0 = ((gh * CPT) & 63) >> 3;
        const int rx = r & 7;
        uint32_t dsw[CPT / 2];
        if (outside) {
          // no query row of this warp sees any of these keys (they belong to other sequences):
          // zero tiles, no exponentials
#pragma unroll
          for (int c8 = 0; c8 < CPT / 8; ++c8) {
            const uint32_t off = static_cast<uint32_t>(((chunk0 + c8) ^ rx) << 4);
            if constexpr (!QST) {
              *reinterpret_cast<uint4*>(rowP + off) = make_uint4(0u, 0u, 0u, 0u);
              *reinterpret_cast<uint4*>(rowS + off) = make_uint4(0u, 0u, 0u, 0u);
            }
          }
          if constexpr (DQ || QST) {
#pragma unroll
            for (int c = 0; c < CPT / 2; ++c) dsw[c] = 0u;
          }
        } else {
          // bit e of kbits: key c0 + e lies inside the row's range (CPT <= 64 keys per thread)
          uint64_t kbits = ~0ull;
          if (!inside) {
            const int a = max(ri.klo - c0, 0), b = min(ri.khi - c0, CPT);
            kbits = b > a ? (~0ull >> (64 - (b - a))) << a : 0ull;
          }
#pragma unroll
          for (int c8 = 0; c8 < CPT / 8; ++c8) {
            uint32_t pk[4], dk[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int e = c8 * 8 + 2 * u;
              float p0 = exp2f(fmaf(__uint_as_float(rs[e]), sl2, -ri.lse2));
              float p1 = exp2f(fmaf(__uint_as_float(rs[e + 1]), sl2, -ri.lse2));
              if (!inside) {
                if (!(kbits & (1ull << e))) p0 = 0.f;
                if (!(kbits & (1ull << (e + 1)))) p1 = 0.f;
              }
              const float d0 = p0 * (__uint_as_float(rp[e]) - ri.delta);
              const float d1 = p1 * (__uint_as_float(rp[e + 1]) - ri.delta);
              pk[u] = pack_bf16x2(p0, p1);
              dk[u] = pack_bf16x2(d0, d1);
            }
            const uint32_t off = static_cast<uint32_t>(((chunk0 + c8) ^ rx) << 4);
            if constexpr (!QST) {    // the query-stationary pass forms dQ only: no P, and dS only in tensor memory
              *reinterpret_cast<uint4*>(rowP + off) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              *reinterpret_cast<uint4*>(rowS + off) = make_uint4(dk[0], dk[1], dk[2], dk[3]);
            }
            if constexpr (DQ || QST) {
#pragma unroll
              for (int u = 0; u < 4; ++u) dsw[c8 * 4 + u] = dk[u];
            }
          }
        }
        if constexpr (DQ || QST) {
          // dS of this thread's keys as the A operand of the dQ product: two keys per 32-bit column
          if constexpr (CPT == 64) tmem_st32(tdS + lane_addr + gh * (CPT / 2), dsw);
          else tmem_st16(tdS + lane_addr + gh * (CPT / 2), dsw);
          tmem_st_wait();
          tc_fence_before();
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_ready);
        WS_TRACE(warp == 0 || warp == NWG * 4 - 1, warp == 0 ? 1 : 2, 3);
      }
      if (!ok) break;
      if (g.n_q == 0 && item_n < n_items) {    // (an item without steps did not reach the prefetch above)
        g_cur = ws_bwd_geo_make(args, item_n / H, gn_a, gn_b);
        first = fetch_row((QST ? g_cur.kv0 : g_cur.q_lo) + r, item_n % H);
      }
      if (g.n_q > 0) {
        ok = mbar_wait(g_done, c_g & 1u);
        ++c_g;
        ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
        if (!ok) break;
        tc_fence_after();
        drain_dq(g.q_lo + (g.n_q - 1) * FA_T, g.q_hi, h);
      }
      WS_TRACE(warp == 0 || warp == NWG * 4 - 1, warp == 0 ? 1 : 2, 5);
      // dK (warpgroup 0) / dV (warpgroup 1): every thread owns the 64 channels of key row kv0 + r.
      // Query-stationary: warpgroup 0 alone reads the item's dQ (row kv0 + r of the query tile).
      if (Cfg::DRAIN_WG || gh >= (QST ? 1 : 2)) continue;   // (the drain warpgroup stores dK / dV when it exists)
      uint64_t* const read_back = QST ? dq_free : acc_free;
      float acc[FA_D];
      if (g.n_q > 0) {
        const uint32_t src = (QST ? tdQ : (gh == 0 ? tdK : tdV)) + lane_addr;
#pragma unroll
        for (int c = 0; c < FA_D; c += 32) {
          uint32_t v[32];
          tmem_ld32(src + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[c + e] = __uint_as_float(v[e]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(read_back);
      } else {
#pragma unroll
        for (int e = 0; e < FA_D; ++e) acc[e] = 0.f;
        __syncwarp();
        if (lane == 0) mbar_arrive(read_back);   // keeps the per-item phase count in step with the MMA warp
      }
      const int krow = g.kv0 + r;
      if (krow < T) {
        if (gh == 0) {
#pragma unroll
          for (int e = 0; e < FA_D; ++e) acc[e] *= args.scale;
          if (args.rope_pos != nullptr) {
            const int pos = __ldg(args.rope_pos + krow);
            const float4* cp = reinterpret_cast<const float4*>(args.rope_cos + static_cast<size_t>(pos) * 32);
            const float4* sp = reinterpret_cast<const float4*>(args.rope_sin + static_cast<size_t>(pos) * 32);
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              const float4 c4 = __ldg(cp + q4), s4 = __ldg(sp + q4);
              const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
              const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int e = q4 * 4 + u;
                const float a = acc[e], b = acc[e + 32];
                acc[e] = a * cc[u] + b * ss[u];
                acc[e + 32] = b * cc[u] - a * ss[u];
              }
            }
          }
        }
        __nv_bfloat16* dst = args.dqkv + (static_cast<size_t>(krow) * 3 + (QST ? 0 : 1 + gh)) * HD + h * FA_D;
#pragma unroll
        for (int e = 0; e < FA_D; e += 8) {
          uint4 u4;
          uint32_t* pk = reinterpret_cast<uint32_t*>(&u4);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) pk[q4] = pack_bf16x2(acc[e + 2 * q4], acc[e + 2 * q4 + 1]);
          *reinterpret_cast<uint4*>(dst + e) = u4;
        }
      }
    }
    if (!ok && lane == 0 && *abort_flag == 0) {
      atomicExch(args.status, ST_TIMEOUT_TMEM_FULL);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::MMA_WARP) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h][t] = sum_d dO[t,h,d] * O[t,h,d]
__global__ void __launch_bounds__(256)
ws_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                float* __restrict__ delta, int T, int H) {
  const long long total = static_cast<long long>(T) * H * 8;   // 8 threads per (t, h)
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
    const uint32_t gmask = 0xffu << (threadIdx.x & 24);
    s += __shfl_xor_sync(gmask, s, 1);
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 4);
    if (sub == 0) delta[static_cast<size_t>(h) * T + t] = s;
  }
}

// dq (fp32 accumulator) -> bf16 into the q part of dqkv[T][3][H][64]; with rope_pos the gradient is
// rotated back first. One thread handles channels [8v, 8v+8) and [32+8v, 32+8v+8) of one head.
__global__ void __launch_bounds__(256)
ws_dq_store_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int T, int H,
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

static EncodeTiledFn ws_encode_fn() {
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
// fp32 [rows][cols] accumulator, boxes of 128 rows x 32 columns (one 128-byte swizzled row each)
static int ws_make_map_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows) {
  EncodeTiledFn fn = ws_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 4};
  cuuint32_t box[2] = {32, FA_T};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int ws_make_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows) {
  EncodeTiledFn fn = ws_encode_fn();
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

// cudaFuncSetAttribute and the SM count are per device: one slot per device ordinal
constexpr int WS_MAX_DEVICES = 64;
struct WsDeviceInfo {
  bool configured;
  int sms;
};
static WsDeviceInfo ws_device[WS_MAX_DEVICES];

static int ws_configure(int* sms) {
  int dev = 0;
  NPLM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= WS_MAX_DEVICES) return -4;
  if (!ws_device[dev].configured) {
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_ws_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         WS_FWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_ws_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         WS_FWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_ws_kernel<2, BWD_KV_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         WS_BWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_ws_kernel<4, BWD_KV_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         WS_BWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_ws_kernel<4, BWD_KV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         WS_BWD_SMEM));
    NPLM_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_ws_kernel<4, BWD_Q>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         WS_BWD_SMEM));
    int n = 0;
    NPLM_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    ws_device[dev].sms = n;
    ws_device[dev].configured = true;
  }
  *sms = ws_device[dev].sms;
  return 0;
}

}  // namespace nplm

using namespace nplm;

// Forward. The current device must be the one that owns `st` and the tensors.
extern "C" int nplm_fa_fwd_ws(const void* qkv, void* out, float* lse, const int* seq_start,
                              const int* seq_end, int T, int H, int D, int window, float scale,
                              int max_ctas, int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D != FA_D || H <= 0) return -3;
  if (reinterpret_cast<uintptr_t>(qkv) & 15) return -3;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -3;
  CUtensorMap tm, tmO;
  int rc = ws_make_map(&tm, qkv, static_cast<uint64_t>(3) * H * D, T);
  if (rc) return rc;
  rc = ws_make_map(&tmO, out, static_cast<uint64_t>(H) * D, T);
  if (rc) return rc;
  int sms = 0;
  rc = ws_configure(&sms);
  if (rc) return rc;
  FaWsArgs a;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.seq_start = seq_start;
  a.seq_end = seq_end;
  a.T = T;
  a.H = H;
  a.window = window;
  a.scale = scale;
  a.status = status;
  const int n_items = ((T + 2 * FA_T - 1) / (2 * FA_T)) * H;
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > n_items) grid = n_items;
  static int p_smem = -1;   // NPLM_FA_FWD_P_SMEM=1: probabilities through shared memory (benchmarks)
  if (p_smem < 0) {
    const char* e = getenv("NPLM_FA_FWD_P_SMEM");
    p_smem = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  if (p_smem)
    fa_fwd_ws_kernel<false><<<grid, WS_THREADS, WS_FWD_SMEM, st>>>(tm, tmO, a);
  else
    fa_fwd_ws_kernel<true><<<grid, WS_THREADS, WS_FWD_SMEM, st>>>(tm, tmO, a);
  return static_cast<int>(cudaGetLastError());
}

// Backward. dq_acc: caller-provided fp32 scratch [T][H*D], cleared here. delta: fp32 scratch [H][T],
// computed here from out and dout unless out is null (then it must hold rowsum(dO * O) already).
// rope_* (may be null): q / k were rotated before the forward pass; dQ and dK are returned as
// gradients of the un-rotated projections.
// mode: 4 = four compute warpgroups, dQ through fp32 atomics (fastest); 2 = two compute warpgroups, same
// scheme; 0 = dK / dV only (timing experiments); 3 = bitwise reproducible: a key-stationary launch for
// dK / dV and a query-stationary launch for dQ, no atomics, dq_acc unused (may be null); -1 = the value
// of NPLM_FA_BWD_MODE ("2", "0", "det" / "3"), else 4.
static int ws_bwd_impl(const void* qkv, const void* out, const void* dout, const float* lse,
                       void* dqkv, float* dq_acc, float* delta, const int* seq_start,
                       const int* seq_end, int T, int H, int D, int window, float scale,
                       const int* rope_pos, const float* rope_cos, const float* rope_sin,
                       int max_ctas, int mode, int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D != FA_D || H <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(dout) & 15)) return -3;
  if (mode < 0) {
    static int env_mode = -1;
    if (env_mode < 0) {
      const char* e = getenv("NPLM_FA_BWD_MODE");
      env_mode = 4;
      if (e != nullptr && (e[0] == '2' || e[0] == '0' || e[0] == '3')) env_mode = e[0] - '0';
      if (e != nullptr && e[0] == 'd') env_mode = 3;
    }
    mode = env_mode;
  }
  if (mode != 0 && mode != 2 && mode != 3 && mode != 4) return -3;
  if (mode != 3 && dq_acc == nullptr) return -3;
  CUtensorMap tmQKV, tmDO;
  int rc = ws_make_map(&tmQKV, qkv, static_cast<uint64_t>(3) * H * D, T);
  if (rc) return rc;
  rc = ws_make_map(&tmDO, dout, static_cast<uint64_t>(H) * D, T);
  if (rc) return rc;
  CUtensorMap tmDQ = tmDO, tmOUT = tmDO;     // read by the drain warpgroup of the four-warpgroup kernels
  if (mode != 2) {
    if (reinterpret_cast<uintptr_t>(dqkv) & 15) return -3;
    rc = ws_make_map(&tmOUT, dqkv, static_cast<uint64_t>(3) * H * D, T);
    if (rc) return rc;
  }
  if (mode == 4) {
    if (reinterpret_cast<uintptr_t>(dq_acc) & 15) return -3;
    rc = ws_make_map_f32(&tmDQ, dq_acc, static_cast<uint64_t>(H) * D, T);
    if (rc) return rc;
  }
  int sms = 0;
  rc = ws_configure(&sms);
  if (rc) return rc;
  const int HD = H * D;
  if (mode != 3)
    NPLM_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(T) * HD * sizeof(float), st));
  if (out != nullptr) {
    const long long total = static_cast<long long>(T) * H * 8;
    long long blocks = (total + 255) / 256;
    if (blocks > sms * 16) blocks = sms * 16;
    ws_delta_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, T, H);
  }
  FaWsBwdArgs a;
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
  const int n_items = ((T + FA_T - 1) / FA_T) * H;
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > n_items) grid = n_items;
  if (mode == 2) {
    fa_bwd_ws_kernel<2, BWD_KV_DQ><<<grid, WsBwdCfg<2, true>::THREADS, WS_BWD_SMEM, st>>>(tmQKV, tmDO, tmDQ, tmOUT, a);
  } else if (mode == 0) {
    fa_bwd_ws_kernel<4, BWD_KV><<<grid, WsBwdCfg<4, false>::THREADS, WS_BWD_SMEM, st>>>(tmQKV, tmDO, tmDQ, tmOUT, a);
  } else if (mode == 3) {
    fa_bwd_ws_kernel<4, BWD_KV><<<grid, WsBwdCfg<4, false>::THREADS, WS_BWD_SMEM, st>>>(tmQKV, tmDO, tmDQ, tmOUT, a);
    fa_bwd_ws_kernel<4, BWD_Q><<<grid, WsBwdCfg<4, false>::THREADS, WS_BWD_SMEM, st>>>(tmQKV, tmDO, tmDQ, tmOUT, a);
    return static_cast<int>(cudaGetLastError());
  } else {
    fa_bwd_ws_kernel<4, BWD_KV_DQ><<<grid, WsBwdCfg<4, true>::THREADS, WS_BWD_SMEM, st>>>(tmQKV, tmDO, tmDQ, tmOUT, a);
  }
  {
    const long long total = static_cast<long long>(T) * H * 4;
    long long blocks = (total + 255) / 256;
    if (blocks > sms * 16) blocks = sms * 16;
    ws_dq_store_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        dq_acc, reinterpret_cast<__nv_bfloat16*>(dqkv), T, H, rope_pos, rope_cos, rope_sin);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_fa_bwd_ws(const void* qkv, const void* out, const void* dout, const float* lse,
                              void* dqkv, float* dq_acc, float* delta, const int* seq_start,
                              const int* seq_end, int T, int H, int D, int window, float scale,
                              const int* rope_pos, const float* rope_cos, const float* rope_sin,
                              int max_ctas, int* status, cudaStream_t st) {
  return ws_bwd_impl(qkv, out, dout, lse, dqkv, dq_acc, delta, seq_start, seq_end, T, H, D, window, scale,
                     rope_pos, rope_cos, rope_sin, max_ctas, -1, status, st);
}

// Same with the mode given by the caller (see ws_bwd_impl).
extern "C" int nplm_fa_bwd_ws_mode(const void* qkv, const void* out, const void* dout, const float* lse,
                                   void* dqkv, float* dq_acc, float* delta, const int* seq_start,
                                   const int* seq_end, int T, int H, int D, int window, float scale,
                                   const int* rope_pos, const float* rope_cos, const float* rope_sin,
                                   int max_ctas, int mode, int* status, cudaStream_t st) {
  return ws_bwd_impl(qkv, out, dout, lse, dqkv, dq_acc, delta, seq_start, seq_end, T, H, D, window, scale,
                     rope_pos, rope_cos, rope_sin, max_ctas, mode, status, st);
}

#ifdef NPLM_WS_TRACE
// Registers (or clears, with null) the trace buffer of 4 x 1024 int64 for the following launches on
// the current device; see WS_TRACE.
extern "C" int nplm_fa_ws_set_trace(long long* buf) {
  return static_cast<int>(cudaMemcpyToSymbol(g_ws_trace, &buf, sizeof(buf)));
}
#endif
