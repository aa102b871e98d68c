// Optimizer-step communication fused into the compute kernels, over NVLink peer memory.
//
// The reference leaves this to FSDP2 + NCCL + torch.optim: a reduce-scatter of fp32 gradients, a
// separate clip_grad_norm_ (foreach kernels + a scalar all-reduce + .item()), a foreach AdamW and,
// on the next micro-step, an all-gather of the updated parameters
// (src/nanoplm/pretraining/pure_pipeline.py:479-506, 755-764). Here every rank's gradient buffer,
// parameter buffer and a few flag words live in symmetric (peer-mapped) memory and three kernels
// do all of it with plain P2P loads and stores, no collective library call:
//
//   rs_sumsq_kernel   : slice owner PULLS the slice of every peer's fp32 gradient (rank order, so
//                       the sum is deterministic), writes the reduced slice locally and
//                       accumulates its sum of squares (reduce-scatter + norm in one pass).
//   adamw_push_kernel : global norm from the per-rank partial sums -> clip coefficient -> AdamW
//                       on the fp32 master slice -> the updated bf16 values are PUSHED into the
//                       parameter buffer of every rank (sharded update + all-gather in one pass).
//   push_kernel       : a range this rank computed in place in a symmetric buffer is stored into every
//                       peer's copy (Muon: the orthogonalised updates of the matrices a rank owns).
//   peer_barrier_kernel / publish_kernel : flag-based cross-GPU barrier and the exchange of the
//                       partial sums. Every wait on a peer flag is bounded and reports
//                       ST_TIMEOUT_PEER through the status word instead of hanging.
//
// No multimem / multicast instruction is used: only ld/st to peer-mapped addresses.
#include "common.cuh"

namespace nplm {

constexpr int MAX_PEERS = 8;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// flags.p[r] -> uint32[world] on rank r. Rank `rank` writes `epoch` into slot [rank] of every
// peer, then waits until every slot of its own array has reached `epoch`.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, uint32_t epoch,
                                    long long limit_cycles, int* status) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[p]) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + p;
    const long long t0 = clock64();
    // epochs only grow; the signed difference keeps the comparison valid across wrap-around
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > limit_cycles) {
        atomicExch(status, ST_TIMEOUT_PEER);
        break;
      }
      __nanosleep(200);
    }
  }
}

// shard[i] = sum_p grads.p[p][lo + i] (fixed rank order); sumsq += sum shard[i]^2
__global__ void __launch_bounds__(512)
rs_sumsq_kernel(PeerPtrs grads, int world, long long lo, long long n, float* __restrict__ shard,
                float* __restrict__ sumsq) {
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p) {
      if (p < world) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[p]) + lo + 4 * i);
        s.x += v.x;
        s.y += v.y;
        s.z += v.z;
        s.w += v.w;
      }
    }
    reinterpret_cast<float4*>(shard)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  __shared__ float ws[16];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += ws[i];
    atomicAdd(sumsq, t);
  }
}

// slots.p[r] -> float[world] on rank r; writes this rank's partial into slot [rank] everywhere
__global__ void publish_kernel(PeerPtrs slots, int rank, int world, const float* partial) {
  const int p = threadIdx.x;
  if (p < world) {
    reinterpret_cast<volatile float*>(slots.p[p])[rank] = *partial;
    __threadfence_system();
  }
}

// Packed statistics all-reduce (tokens, raw tokens, elapsed time, ... of a logging window): every
// rank stores its <= 16 doubles into its row of every peer's table, raises a flag there, waits
// (bounded) for the flags of all peers in its own table and reduces the rows in rank order:
// value i is summed, or maximised when bit i of max_mask is set. One launch of one block replaces
// the 2-3 small library all-reduces of the reference's logging path
// (src/nanoplm/pretraining/pure_pipeline.py:775-800). Per-rank area behind buf.p[r]:
//   double rows[2][MAX_PEERS][16]; uint32 flags[2][MAX_PEERS]     (2 = parity of the call counter:
// a rank can run at most one call ahead of a peer, so two alternating tables never collide).
constexpr int STATS_MAX = 16;
constexpr int STATS_FLAG_OFFSET = 2 * MAX_PEERS * STATS_MAX * 8;   // bytes

__global__ void __launch_bounds__(128)
stats_allreduce_kernel(PeerPtrs buf, int rank, int world, uint32_t epoch, const double* __restrict__ in,
                       double* __restrict__ out, int n, uint32_t max_mask, long long limit_cycles,
                       int* status) {
  __shared__ int failed;
  const int t = threadIdx.x;
  const int par = static_cast<int>(epoch & 1u);
  if (t == 0) failed = 0;
  {
    const int p = t / STATS_MAX, i = t % STATS_MAX;
    if (p < world && i < n) {
      volatile double* rows = reinterpret_cast<volatile double*>(buf.p[p]);
      rows[(par * MAX_PEERS + rank) * STATS_MAX + i] = in[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (t < world) {
    uint32_t* peer_flags = reinterpret_cast<uint32_t*>(static_cast<char*>(buf.p[t]) + STATS_FLAG_OFFSET);
    st_release_sys(peer_flags + par * MAX_PEERS + rank, epoch);
    const uint32_t* mine =
        reinterpret_cast<const uint32_t*>(static_cast<char*>(buf.p[rank]) + STATS_FLAG_OFFSET) + par * MAX_PEERS + t;
    const long long t0 = clock64();
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > limit_cycles) {
        atomicExch(status, ST_TIMEOUT_PEER);
        failed = 1;
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (t < n && !failed) {
    const volatile double* rows = reinterpret_cast<const volatile double*>(buf.p[rank]);
    double acc = rows[(par * MAX_PEERS + 0) * STATS_MAX + t];
    for (int p = 1; p < world; ++p) {
      const double v = rows[(par * MAX_PEERS + p) * STATS_MAX + t];
      acc = ((max_mask >> t) & 1u) ? fmax(acc, v) : acc + v;
    }
    out[t] = acc;
  }
}

// AdamW on the owned slice [lo, lo+n) + push of the bf16 result to every rank's parameter buffer.
// hyper: [lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale, max_norm].
// Elements with global index < decay_end use weight_decay, the rest none. n is a multiple of 8.
// `world` parameter buffers receive the result (1 = only this rank's own buffer: the other ranks
// fetch the rows later, inside the GEMM that consumes them); the norm sums n_slots partial sums.
__global__ void __launch_bounds__(512)
adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                  const float* __restrict__ g, PeerPtrs params, int world, long long lo, long long n,
                  long long decay_end, const float* __restrict__ hyper, const float* __restrict__ slots,
                  int n_slots, float* __restrict__ norm_out) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd0 = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], gs = hyper[7], max_norm = hyper[8];
  float total = 0.f;
  for (int p = 0; p < n_slots; ++p) total += slots[p];
  const float norm = sqrtf(total) * gs;
  float scale = gs;
  if (max_norm > 0.f) scale = gs * fminf(1.f, max_norm / (norm + 1e-6f));
  if (blockIdx.x == 0 && threadIdx.x == 0 && norm_out) *norm_out = norm;
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long base = 8 * i;
    float pv[8], mv[8], vv[8], gv[8];
    *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(master + base);
    *reinterpret_cast<float4*>(pv + 4) = *reinterpret_cast<const float4*>(master + base + 4);
    *reinterpret_cast<float4*>(mv) = *reinterpret_cast<const float4*>(m + base);
    *reinterpret_cast<float4*>(mv + 4) = *reinterpret_cast<const float4*>(m + base + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + base);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + base + 4);
    *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(g + base);
    *reinterpret_cast<float4*>(gv + 4) = *reinterpret_cast<const float4*>(g + base + 4);
    const float wd = (lo + base < decay_end) ? wd0 : 0.f;   // groups are 64-element aligned
    uint4 packed;
    uint32_t* pk = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gr = gv[e] * scale;
      float x = pv[e] * (1.f - lr * wd);
      mv[e] = b1 * mv[e] + (1.f - b1) * gr;
      vv[e] = b2 * vv[e] + (1.f - b2) * gr * gr;
      x -= step_size * mv[e] / (sqrtf(vv[e]) * inv_sqrt_bc2 + eps);
      pv[e] = x;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) pk[e] = pack_bf16x2(pv[2 * e], pv[2 * e + 1]);
    *reinterpret_cast<float4*>(master + base) = *reinterpret_cast<float4*>(pv);
    *reinterpret_cast<float4*>(master + base + 4) = *reinterpret_cast<float4*>(pv + 4);
    *reinterpret_cast<float4*>(m + base) = *reinterpret_cast<float4*>(mv);
    *reinterpret_cast<float4*>(m + base + 4) = *reinterpret_cast<float4*>(mv + 4);
    *reinterpret_cast<float4*>(v + base) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + base + 4) = *reinterpret_cast<float4*>(vv + 4);
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p) {
      if (p < world)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[p]) + lo + base) = packed;
    }
  }
}

// Copies n16 16-byte words at the same offset of a symmetric buffer from this rank's copy into
// every other rank's copy (the all-gather of a run that this rank has just computed in place).
__global__ void __launch_bounds__(512)
push_kernel(PeerPtrs bufs, int rank, int world, long long word0, long long n16) {
  const uint4* src = reinterpret_cast<const uint4*>(bufs.p[rank]) + word0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p) {
      if (p < world && p != rank) (reinterpret_cast<uint4*>(bufs.p[p]) + word0)[i] = v;
    }
  }
}

}  // namespace nplm

using namespace nplm;

static PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

extern "C" int nplm_peer_barrier(void* const* flag_ptrs, int rank, int world, unsigned epoch,
                                 double timeout_s, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS) return -3;
  const long long limit = static_cast<long long>(timeout_s * 1.8e9);
  peer_barrier_kernel<<<1, 32, 0, st>>>(to_peers(flag_ptrs, world), rank, world, epoch, limit, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_rs_sumsq(void* const* grad_ptrs, int world, long long lo, long long n, float* shard,
                             float* sumsq, cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || (n & 3) || (lo & 3)) return -3;
  if (n == 0) return 0;
  long long blocks = (n / 4 + 511) / 512;
  if (blocks > 148 * 4) blocks = 148 * 4;
  rs_sumsq_kernel<<<static_cast<int>(blocks), 512, 0, st>>>(to_peers(grad_ptrs, world), world, lo, n, shard, sumsq);
  return static_cast<int>(cudaGetLastError());
}

// buffer bytes per rank that nplm_stats_allreduce needs (zero-initialised symmetric memory)
extern "C" int nplm_stats_buffer_bytes() { return STATS_FLAG_OFFSET + 2 * MAX_PEERS * 4; }

extern "C" int nplm_stats_allreduce(void* const* buf_ptrs, int rank, int world, unsigned epoch, const double* in,
                                    double* out, int n, unsigned max_mask, double timeout_s, int* status,
                                    cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || n < 1 || n > STATS_MAX || epoch == 0) return -3;
  const long long limit = static_cast<long long>(timeout_s * 1.8e9);
  stats_allreduce_kernel<<<1, 128, 0, st>>>(to_peers(buf_ptrs, world), rank, world, epoch, in, out, n, max_mask,
                                            limit, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_publish(void* const* slot_ptrs, int rank, int world, const float* partial,
                            cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS) return -3;
  publish_kernel<<<1, 32, 0, st>>>(to_peers(slot_ptrs, world), rank, world, partial);
  return static_cast<int>(cudaGetLastError());
}

// Pushes to `world` buffers and sums `n_slots` partial sums of squares for the clipping norm.
extern "C" int nplm_adamw_push_ex(float* master, float* m, float* v, const float* g, void* const* param_ptrs,
                                  int world, long long lo, long long n, long long decay_end,
                                  const float* hyper, const float* slots, int n_slots, float* norm_out,
                                  cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || n_slots < 1 || n_slots > MAX_PEERS || (n & 7) || (lo & 7)) return -3;
  if (n == 0) return 0;
  long long blocks = (n / 8 + 511) / 512;
  if (blocks > 148 * 4) blocks = 148 * 4;
  adamw_push_kernel<<<static_cast<int>(blocks), 512, 0, st>>>(master, m, v, g, to_peers(param_ptrs, world), world,
                                                              lo, n, decay_end, hyper, slots, n_slots, norm_out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_adamw_push(float* master, float* m, float* v, const float* g, void* const* param_ptrs,
                               int world, long long lo, long long n, long long decay_end,
                               const float* hyper, const float* slots, float* norm_out, cudaStream_t st) {
  return nplm_adamw_push_ex(master, m, v, g, param_ptrs, world, lo, n, decay_end, hyper, slots, world, norm_out,
                            st);
}

// buf_ptrs[r]: rank r's copy of one symmetric buffer. Bytes [byte_offset, byte_offset + bytes) of this
// rank's copy are stored into every other rank's copy. Offsets and sizes are multiples of 16.
extern "C" int nplm_push(void* const* buf_ptrs, int rank, int world, long long byte_offset, long long bytes,
                         cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || (byte_offset & 15) || (bytes & 15)) return -3;
  if (bytes == 0 || world == 1) return 0;
  const long long n16 = bytes >> 4;
  long long blocks = (n16 + 511) / 512;
  if (blocks > 148 * 4) blocks = 148 * 4;
  push_kernel<<<static_cast<int>(blocks), 512, 0, st>>>(to_peers(buf_ptrs, world), rank, world, byte_offset >> 4, n16);
  return static_cast<int>(cudaGetLastError());
}
