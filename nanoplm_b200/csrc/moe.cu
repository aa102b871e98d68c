// Mixture-of-experts routing, dispatch and combine kernels for sm_100a.
//
// The reference has no MoE layers; these kernels serve the `model.moe` extension of the encoder
// (top-k softmax router, SwiGLU experts, Switch-style balance loss) and its expert-parallel form.
//
// Layout. Every (token, slot) assignment gets a row in an "expert-major" buffer: the rows of one
// expert are contiguous and every expert's segment is padded to a multiple of 128 rows (zero
// rows), so the grouped tcgen05 GEMM sees only whole row tiles and the grouped weight gradient
// can contract over a segment without masking. With expert parallelism expert e lives on rank
// e / experts_per_rank; its segment holds the rows of source rank 0 first, then rank 1, ...
// The order inside (expert, source rank) is the token order, so the layout is deterministic.
//
// All communication is token-side and goes through peer-mapped pointers (plain ld/st over
// NVLink): rows are PUSHED into the owner's buffer (dispatch, and the gradient of combine) and
// PULLED back from it (combine, and the gradient of dispatch). No multimem / multicast
// instruction is used.
#include "common.cuh"

namespace nplm {

constexpr int MOE_MAX_PEERS = 8;
constexpr int MOE_MAX_E = 256;   // experts (global)
constexpr int MOE_MAX_K = 8;     // top-k

struct MoePeers {
  void* p[MOE_MAX_PEERS];
};

// ------------------------------------------------------------------------------- router
// One warp per token: softmax over E logits (fp32), top-k by repeated arg-max (ties -> lower
// index), gates renormalised to sum 1. probs are kept for the backward pass; probsum[e]
// accumulates sum_t p[t,e] and counts[e] the assignments of expert e, for the balance loss.
__global__ void __launch_bounds__(256)
router_topk_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int k,
                   float* __restrict__ probs, float* __restrict__ gates, int* __restrict__ experts,
                   float* __restrict__ probsum, int* __restrict__ counts) {
  __shared__ float s_sum[MOE_MAX_E];
  __shared__ int s_cnt[MOE_MAX_E];
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    s_sum[i] = 0.f;
    s_cnt[i] = 0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  constexpr int PER = MOE_MAX_E / 32;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      v[j] = e < E ? __bfloat162float(logits[static_cast<size_t>(t) * E + e]) : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      v[j] = (j * 32 + lane) < E ? __expf(v[j] - mx) : 0.f;
      sum += v[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      v[j] *= inv;
      if (e < E) {
        probs[static_cast<size_t>(t) * E + e] = v[j];
        atomicAdd(&s_sum[e], v[j]);
      }
    }
    // top-k
    float gsel = 0.f;   // lane s holds the s-th selected probability
    int esel = 0;
    float gtot = 0.f;
    for (int s = 0; s < k; ++s) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int e = j * 32 + lane;
        if (e < E && v[j] > best) {
          best = v[j];
          bi = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) {
          best = ob;
          bi = oi;
        }
      }
      // remove the winner from further rounds
#pragma unroll
      for (int j = 0; j < PER; ++j)
        if (j * 32 + lane == bi) v[j] = -2.f;
      if (lane == s) {
        gsel = best;
        esel = bi;
      }
      gtot += best;
    }
    if (lane < k) {
      gates[static_cast<size_t>(t) * k + lane] = gsel / fmaxf(gtot, 1e-9f);
      experts[static_cast<size_t>(t) * k + lane] = esel;
      atomicAdd(&s_cnt[esel], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    atomicAdd(&probsum[i], s_sum[i]);
    if (s_cnt[i]) atomicAdd(&counts[i], s_cnt[i]);
  }
}

// dlogits from d_gates [T,k] and the balance-loss term d_aux * E * f_e / T added to dL/dp.
//   g_i = p_{e_i} / s,  s = sum_i p_{e_i}   =>   dL/dp_{e_j} += (dg_j - sum_i dg_i g_i) / s
//   dz = p * (dp - sum_e p_e dp_e)
__global__ void __launch_bounds__(256)
router_bwd_kernel(const float* __restrict__ probs, const float* __restrict__ gates,
                  const int* __restrict__ experts, const float* __restrict__ d_gates,
                  const float* __restrict__ aux_grad_per_expert,  // [E], already scaled, or null
                  int T, int E, int k, __nv_bfloat16* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  constexpr int PER = MOE_MAX_E / 32;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    float p[PER], dp[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      p[j] = e < E ? probs[static_cast<size_t>(t) * E + e] : 0.f;
      dp[j] = (e < E && aux_grad_per_expert != nullptr) ? aux_grad_per_expert[e] : 0.f;
    }
    float s = 0.f, dot = 0.f;
    for (int i = 0; i < k; ++i) {
      const int e = experts[static_cast<size_t>(t) * k + i];
      const float g = gates[static_cast<size_t>(t) * k + i];
      const float pe = probs[static_cast<size_t>(t) * E + e];
      s += pe;
      dot += d_gates[static_cast<size_t>(t) * k + i] * g;
    }
    const float inv_s = 1.f / fmaxf(s, 1e-9f);
    for (int i = 0; i < k; ++i) {
      const int e = experts[static_cast<size_t>(t) * k + i];
      const float add = (d_gates[static_cast<size_t>(t) * k + i] - dot) * inv_s;
#pragma unroll
      for (int j = 0; j < PER; ++j)
        if (j * 32 + lane == e) dp[j] += add;
    }
    float pd = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) pd += p[j] * dp[j];
    pd = warp_sum(pd);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      if (e < E) dlogits[static_cast<size_t>(t) * E + e] = __float2bfloat16(p[j] * (dp[j] - pd));
    }
  }
}

// ------------------------------------------------------------------------------- planning
// counts[e] = number of assignments routed to expert e; block e counts. The result is written to
// slot [rank][e] of the count table of every peer (world == 1: the local table).
__global__ void __launch_bounds__(1024)
moe_count_kernel(const int* __restrict__ experts, int n, int E, MoePeers tables, int rank, int world) {
  const int e = blockIdx.x;
  int c = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) c += (experts[i] == e);
  __shared__ int s_part[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if (lane == 0) s_part[warp] = c;
  __syncthreads();
  if (warp == 0) {
    c = lane < (blockDim.x >> 5) ? s_part[lane] : 0;
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (lane == 0) {
      for (int p = 0; p < world; ++p) reinterpret_cast<int*>(tables.p[p])[rank * E + e] = c;
    }
  }
}

// One block. From the count table [world][E]:
//   seg_off[e]   (E+1 entries per owner, local numbering): padded segment offsets on each owner,
//                stored for the LOCAL experts in group_off[0..El]
//   my_base[e]   row (in the owner's buffer) where this rank's first assignment of e goes
//   tile_group[] local expert of every 128-row tile of the local buffer, -1 beyond the end
//   pad_lo/pad_hi[el] the zero-padding rows of local expert el
//   tile_rows[]  (optional) number of real rows of every tile = the value its arrival counter reaches
//   overflow: when the local rows exceed the buffer capacity the rows past it are DROPPED (push,
//   pull and their backward kernels skip them, so those assignments contribute nothing) and counted
//   in *dropped; training goes on (a skewed router costs some tokens of the tail experts of a rank,
//   as with a capacity factor)
__global__ void __launch_bounds__(256)
moe_plan_kernel(const int* __restrict__ table, int world, int rank, int E, int capacity_rows,
                int* __restrict__ group_off, int* __restrict__ my_base, int* __restrict__ tile_group,
                int max_tiles, int* __restrict__ pad_lo, int* __restrict__ pad_hi, int* dropped,
                int* __restrict__ tile_rows) {
  __shared__ int s_total[MOE_MAX_E];   // assignments of expert e over all ranks
  __shared__ int s_before[MOE_MAX_E];  // ... from ranks below this one
  __shared__ int s_off[MOE_MAX_E + 1]; // padded offset of e inside its owner's buffer
  const int El = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int r = 0; r < world; ++r) {
      const int c = table[r * E + e];
      if (r < rank) before += c;
      tot += c;
    }
    s_total[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  if (threadIdx.x < world) {
    // owner `o` scans its El experts
    const int o = threadIdx.x;
    int off = 0;
    for (int el = 0; el < El; ++el) {
      const int e = o * El + el;
      s_off[e] = off;
      off += (s_total[e] + 127) & ~127;
    }
    if (o == rank) {
      group_off[El] = off;
      if (off > capacity_rows && dropped != nullptr) {
        int lost = 0;     // real (non-padding) rows that fall past the capacity
        for (int el = 0; el < El; ++el) {
          const int e = o * El + el;
          lost += max(0, s_off[e] + s_total[e] - max(capacity_rows, s_off[e]));
        }
        atomicAdd(dropped, lost);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) my_base[e] = s_off[e] + s_before[e];
  for (int el = threadIdx.x; el < El; el += blockDim.x) {
    const int e = rank * El + el;
    group_off[el] = s_off[e];
    pad_lo[el] = s_off[e] + s_total[e];
    pad_hi[el] = s_off[e] + ((s_total[e] + 127) & ~127);
  }
  __syncthreads();
  const int end = group_off[El];
  for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) {
    const int row = tile * 128;
    int g = -1;
    if (row < end && row < capacity_rows) {
      // last local expert whose offset is <= row
      int lo = 0, hi = El;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[rank * El + mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    tile_group[tile] = g;
    // real (pushed) rows of this tile: what its arrival counter has to reach
    if (tile_rows != nullptr)
      tile_rows[tile] = g < 0 ? 0 : min(128, max(0, min(pad_lo[g], capacity_rows) - row));
  }
}

// pos_of[i] = my_base[e] + (number of earlier assignments i' < i with the same expert). Block e
// walks the assignment list in order: deterministic, no atomics.
__global__ void __launch_bounds__(1024)
moe_assign_kernel(const int* __restrict__ experts, int n, const int* __restrict__ my_base,
                  int* __restrict__ pos_of) {
  const int e = blockIdx.x;
  __shared__ int s_warp[32];
  __shared__ int s_run, s_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) s_run = my_base[e];
  __syncthreads();
  for (int base = 0; base < n; base += 4 * blockDim.x) {
    const int i0 = base + 4 * threadIdx.x;
    int f[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) f[q] = (i0 + q < n) ? (experts[i0 + q] == e) : 0;
    const int mine = f[0] + f[1] + f[2] + f[3];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int w = lane < nwarps ? s_warp[lane] : 0;
      int wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += up;
      }
      s_warp[lane] = wi - w;  // exclusive prefix over the warps
      if (lane == 31) s_total = wi;
    }
    __syncthreads();
    int pos = s_run + s_warp[warp] + (incl - mine);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (f[q]) pos_of[i0 + q] = pos++;
    }
    __syncthreads();
    if (threadIdx.x == 0) s_run += s_total;
    __syncthreads();
  }
}

// zero rows [pad_lo[el], pad_hi[el]) of a [rows][C] bf16 buffer (C multiple of 8)
__global__ void __launch_bounds__(256)
moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, int C, const int* __restrict__ pad_lo,
                    const int* __restrict__ pad_hi, int capacity_rows) {
  const int el = blockIdx.x;
  const int lo = pad_lo[el], hi = min(pad_hi[el], capacity_rows);
  const int per_row = C / 8;
  const long long n = static_cast<long long>(max(hi - lo, 0)) * per_row;
  uint4* dst = reinterpret_cast<uint4*>(buf + static_cast<size_t>(lo) * C);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
}

// ------------------------------------------------------------------------------- rows in / out
// One warp per assignment i = t*k + s: dst_owner[pos_of[i]] = (scale ? scale[i] : 1) * src[t].
// With `arrive` (per-rank uint32 counters, one per 128-row tile of the owner's buffer) every landed row is
// counted, so the consumer can start a tile without a barrier over all ranks.
__global__ void __launch_bounds__(256)
moe_push_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ experts,
                     const int* __restrict__ pos_of, const float* __restrict__ scale, int n, int k,
                     int C, int experts_per_rank, int capacity_rows, MoePeers dst, MoePeers arrive) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n; i += gridDim.x * wpb) {
    const int pos = pos_of[i];
    if (pos < 0 || pos >= capacity_rows) continue;
    const int owner = experts[i] / experts_per_rank;
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(i / k) * C);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[owner]) +
                                        static_cast<size_t>(pos) * C);
    if (scale == nullptr) {
      for (int c = lane; c < C / 8; c += 32) d[c] = s[c];
    } else {
      const float g = scale[i];
      for (int c = lane; c < C / 8; c += 32) {
        uint4 v = s[c];
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16x2(w[q]);
          w[q] = pack_bf16x2(f.x * g, f.y * g);
        }
        d[c] = v;
      }
    }
    if (arrive.p[0] != nullptr) {
      // the row has landed: bump the arrival counter of its 128-row tile on the owner (release at system
      // scope after the warp's stores; the owner's grouped GEMM acquires it before loading the tile)
      __syncwarp();
      if (lane == 0) {
        __threadfence_system();
        red_release_sys_add(reinterpret_cast<uint32_t*>(arrive.p[owner]) + (pos >> 7), 1u);
      }
    }
  }
}

// One warp per token: out[t] = sum_s (gates ? gates[t,s] : 1) * src_owner[pos_of[t,s]]
__global__ void __launch_bounds__(256)
moe_pull_rows_kernel(MoePeers src, const int* __restrict__ experts, const int* __restrict__ pos_of,
                     const float* __restrict__ gates, int T, int k, int C, int experts_per_rank,
                     int capacity_rows, __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    for (int c = lane; c < C / 8; c += 32) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int s = 0; s < k; ++s) {
        const int i = t * k + s;
        const int pos = pos_of[i];
        if (pos < 0 || pos >= capacity_rows) continue;
        const int owner = experts[i] / experts_per_rank;
        const float g = gates != nullptr ? gates[i] : 1.f;
        const uint4 v = reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(src.p[owner]) + static_cast<size_t>(pos) * C)[c];
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16x2(w[q]);
          acc[2 * q] += g * f.x;
          acc[2 * q + 1] += g * f.y;
        }
      }
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) ow[q] = pack_bf16x2(acc[2 * q], acc[2 * q + 1]);
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * C)[c] = o;
    }
  }
}

// Gradient of combine, one warp per assignment: d_gates[i] = <dy[t], ys_owner[pos]> (pulled) and
// d_ys_owner[pos] = gates[i] * dy[t] (pushed; counted per tile in `arrive` when given, as in the
// forward push).
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, MoePeers ys, MoePeers d_ys,
                       const int* __restrict__ experts, const int* __restrict__ pos_of,
                       const float* __restrict__ gates, int n, int k, int C, int experts_per_rank,
                       int capacity_rows, float* __restrict__ d_gates, MoePeers arrive) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n; i += gridDim.x * wpb) {
    const int pos = pos_of[i];
    const bool ok = pos >= 0 && pos < capacity_rows;  // warp-uniform
    float dot = 0.f;
    if (ok) {
      const int owner = experts[i] / experts_per_rank;
      const float g = gates[i];
      const uint4* s = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(i / k) * C);
      const uint4* y = reinterpret_cast<const uint4*>(
          reinterpret_cast<const __nv_bfloat16*>(ys.p[owner]) + static_cast<size_t>(pos) * C);
      uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(d_ys.p[owner]) +
                                          static_cast<size_t>(pos) * C);
      for (int c = lane; c < C / 8; c += 32) {
        uint4 v = s[c];
        const uint4 yv = y[c];
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
        const uint32_t* yw = reinterpret_cast<const uint32_t*>(&yv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16x2(w[q]);
          const float2 yy = unpack_bf16x2(yw[q]);
          dot += f.x * yy.x + f.y * yy.y;
          w[q] = pack_bf16x2(f.x * g, f.y * g);
        }
        d[c] = v;
      }
      if (arrive.p[0] != nullptr) {     // the d_ys row has landed: count it for its tile on the owner
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          red_release_sys_add(reinterpret_cast<uint32_t*>(arrive.p[owner]) + (pos >> 7), 1u);
        }
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) d_gates[i] = ok ? dot : 0.f;
  }
}

static int grid_for(long long items, int per_block) {
  long long g = (items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > 148 * 8) g = 148 * 8;
  return static_cast<int>(g);
}

}  // namespace nplm

using namespace nplm;

extern "C" int nplm_router_topk(const void* logits, int T, int E, int k, float* probs, float* gates,
                                int* experts, float* probsum, int* counts, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > MOE_MAX_E || k < 1 || k > MOE_MAX_K || k > E) return -3;
  router_topk_kernel<<<grid_for(T, 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(logits), T, E, k, probs, gates, experts, probsum, counts);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_router_bwd(const float* probs, const float* gates, const int* experts,
                               const float* d_gates, const float* aux_grad, int T, int E, int k,
                               void* dlogits, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > MOE_MAX_E || k < 1 || k > MOE_MAX_K) return -3;
  router_bwd_kernel<<<grid_for(T, 8), 256, 0, stream>>>(probs, gates, experts, d_gates, aux_grad, T, E,
                                                        k, reinterpret_cast<__nv_bfloat16*>(dlogits));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_count(const int* experts, int n, int E, void* const* tables, int rank,
                              int world, cudaStream_t stream) {
  if (E < 1 || E > MOE_MAX_E || world < 1 || world > MOE_MAX_PEERS || rank < 0 || rank >= world) return -3;
  MoePeers t;
  for (int p = 0; p < MOE_MAX_PEERS; ++p) t.p[p] = p < world ? tables[p] : nullptr;
  moe_count_kernel<<<E, 1024, 0, stream>>>(experts, n, E, t, rank, world);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_plan(const int* table, int world, int rank, int E, int capacity_rows,
                             int* group_off, int* my_base, int* tile_group, int max_tiles,
                             int* pad_lo, int* pad_hi, int* dropped, int* tile_rows, cudaStream_t stream) {
  if (E < 1 || E > MOE_MAX_E || world < 1 || world > MOE_MAX_PEERS || (E % world)) return -3;
  moe_plan_kernel<<<1, 256, 0, stream>>>(table, world, rank, E, capacity_rows, group_off, my_base,
                                         tile_group, max_tiles, pad_lo, pad_hi, dropped, tile_rows);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_assign(const int* experts, int n, int E, const int* my_base, int* pos_of,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  moe_assign_kernel<<<E, 1024, 0, stream>>>(experts, n, my_base, pos_of);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_zero_pad(void* buf, int C, const int* pad_lo, const int* pad_hi,
                                 int local_experts, int capacity_rows, cudaStream_t stream) {
  if (C % 8) return -3;
  moe_zero_pad_kernel<<<local_experts, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(buf), C, pad_lo,
                                                         pad_hi, capacity_rows);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_push_rows(const void* src, const int* experts, const int* pos_of,
                                  const float* scale, int n, int k, int C, int experts_per_rank,
                                  int capacity_rows, void* const* dst, void* const* arrive, int world,
                                  cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((C % 8) || world < 1 || world > MOE_MAX_PEERS) return -3;
  MoePeers d, a;
  for (int p = 0; p < MOE_MAX_PEERS; ++p) {
    d.p[p] = p < world ? dst[p] : nullptr;
    a.p[p] = (arrive != nullptr && p < world) ? arrive[p] : nullptr;
  }
  moe_push_rows_kernel<<<grid_for(n, 8), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(src),
                                                           experts, pos_of, scale, n, k, C,
                                                           experts_per_rank, capacity_rows, d, a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_pull_rows(void* const* src, const int* experts, const int* pos_of,
                                  const float* gates, int T, int k, int C, int experts_per_rank,
                                  int capacity_rows, void* out, int world, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((C % 8) || world < 1 || world > MOE_MAX_PEERS) return -3;
  MoePeers s;
  for (int p = 0; p < MOE_MAX_PEERS; ++p) s.p[p] = p < world ? src[p] : nullptr;
  moe_pull_rows_kernel<<<grid_for(T, 8), 256, 0, stream>>>(s, experts, pos_of, gates, T, k, C,
                                                           experts_per_rank, capacity_rows,
                                                           reinterpret_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_moe_combine_bwd(const void* dy, void* const* ys, void* const* d_ys,
                                    const int* experts, const int* pos_of, const float* gates, int n,
                                    int k, int C, int experts_per_rank, int capacity_rows,
                                    float* d_gates, void* const* arrive, int world, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((C % 8) || world < 1 || world > MOE_MAX_PEERS) return -3;
  MoePeers a, b, cnt;
  for (int p = 0; p < MOE_MAX_PEERS; ++p) {
    a.p[p] = p < world ? ys[p] : nullptr;
    b.p[p] = p < world ? d_ys[p] : nullptr;
    cnt.p[p] = (arrive != nullptr && p < world) ? arrive[p] : nullptr;
  }
  moe_combine_bwd_kernel<<<grid_for(n, 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), a, b, experts, pos_of, gates, n, k, C,
      experts_per_rank, capacity_rows, d_gates, cnt);
  return static_cast<int>(cudaGetLastError());
}
