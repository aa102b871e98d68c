// Kernels for the optional encoder blocks: varlen depthwise convolution and hyper-connection
// (mHC) stream mixing. The reference has neither; semantics are defined here.
//
// Varlen depthwise conv (kernel size KS, odd, "same" centring): for packed tokens x[T][C],
//   y[t][c] = bias[c] + sum_{k} w[c][k] * x[t + k - KS/2][c]   over taps that stay inside the
// sequence of token t (seq_start[t] <= t + k - KS/2 < seq_end[t]); taps that would cross a
// sequence boundary contribute zero.
//   dx[t][c] = sum_k w[c][k] * dy[t - (k - KS/2)][c]            (same boundary rule, flipped taps)
//   dw[c][k] = sum_t dy[t][c] * x[t + k - KS/2][c],  dbias[c] = sum_t dy[t][c]
//
// mHC mixing on streams X[T][n][C] with per-token coefficients:
//   read : h[t][:]     = sum_i alpha[t][i] * X[t][i][:]
//   write: Xn[t][i][:] = sum_j R[t][i][j] * X[t][j][:] + beta[t][i] * y[t][:]
// plus the backward of both (gradients w.r.t. X, y and the coefficients).
#include "common.cuh"

namespace nplm {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = unpack_bf16x2(w[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}

__device__ __forceinline__ void unpack8x(const uint4& u, float (&f)[8]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = unpack_bf16x2(w[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}

__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) w[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

constexpr int MAX_KS = 9;

// flip = 0: forward (tap k reads t + k - r);  flip = 1: input gradient (tap k reads t - (k - r))
__global__ void __launch_bounds__(256)
dwconv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
              const __nv_bfloat16* __restrict__ bias, const int* __restrict__ s_start,
              const int* __restrict__ s_end, __nv_bfloat16* __restrict__ y, int T, int C, int KS, int flip) {
  const int vec = C >> 3;
  const int r = KS >> 1;
  const long long total = static_cast<long long>(T) * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec);
    const int c = static_cast<int>(idx % vec) * 8;
    const int a = s_start[t], b = s_end[t];
    float acc[8];
    if (bias != nullptr && !flip) {
      ld8(bias + c, acc);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    }
    for (int k = 0; k < KS; ++k) {
      const int src = flip ? t - (k - r) : t + (k - r);
      if (src < a || src >= b) continue;
      float xv[8];
      ld8(x + static_cast<size_t>(src) * C + c, xv);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += xv[e] * __bfloat162float(w[(c + e) * KS + k]);
    }
    st8(y + static_cast<size_t>(t) * C + c, acc);
  }
}

// Same convolution with the kernel size known at compile time: a thread owns 8 channels of
// DW_TT consecutive tokens, keeps its 8 x KS weights in registers and walks the DW_TT + KS - 1 input
// rows once (the general kernel above re-reads KS rows and 8 x KS scalar weights per output row).
constexpr int DW_TT = 8;

template <int KS>
__global__ void __launch_bounds__(256)
dwconv_tile_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ bias, const int* __restrict__ s_start,
                   const int* __restrict__ s_end, __nv_bfloat16* __restrict__ y, int T, int C, int flip) {
  constexpr int R = KS / 2;
  const int vec = C >> 3;
  const int n_tb = (T + DW_TT - 1) / DW_TT;
  const long long total = static_cast<long long>(n_tb) * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t0 = static_cast<int>(idx / vec) * DW_TT;
    const int c = static_cast<int>(idx % vec) * 8;
    // all loads of the thread are issued before the first use: DW_TT + KS - 1 input rows (16 bytes
    // each, zero outside the tensor) and the 8 x KS weights, which are contiguous in w[C][KS]
    uint4 xr[DW_TT + KS - 1];
#pragma unroll
    for (int j = 0; j < DW_TT + KS - 1; ++j) {
      const int src = t0 - R + j;
      xr[j] = (src >= 0 && src < T) ? __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(src) * C + c))
                                    : make_uint4(0u, 0u, 0u, 0u);
    }
    uint4 wr[KS];      // 8 channels x KS taps = 8 * KS bf16 = KS 16-byte words (c is a multiple of 8)
#pragma unroll
    for (int q = 0; q < KS; ++q) wr[q] = __ldg(reinterpret_cast<const uint4*>(w + static_cast<size_t>(c) * KS) + q);
    float wt[KS][8];   // wt[k][e]: weight of tap k (already flipped for the input gradient)
    {
      const __nv_bfloat16* wl = reinterpret_cast<const __nv_bfloat16*>(wr);
#pragma unroll
      for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int k = 0; k < KS; ++k) wt[k][e] = __bfloat162float(wl[e * KS + (flip ? KS - 1 - k : k)]);
    }
    float acc[DW_TT][8];
    int lo[DW_TT], hi[DW_TT];
    float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (bias != nullptr && !flip) ld8(bias + c, b8);
#pragma unroll
    for (int i = 0; i < DW_TT; ++i) {
      const int t = t0 + i;
      lo[i] = t < T ? s_start[t] : 0;
      hi[i] = t < T ? s_end[t] : 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] = b8[e];
    }
    // output t0 + i takes input row src with tap k = src - (t0 + i) + R (after the flip both
    // directions read "tap k at offset k - R"); rows outside [lo, hi) belong to another sequence
#pragma unroll
    for (int j = 0; j < DW_TT + KS - 1; ++j) {
      const int src = t0 - R + j;
      float xv[8];
      unpack8x(xr[j], xv);
#pragma unroll
      for (int i = 0; i < DW_TT; ++i) {
        const int k = j - i;   // = src - (t0 + i) + R
        if (k >= 0 && k < KS) {
          const float m = (src >= lo[i] && src < hi[i]) ? 1.f : 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i][e] += m * xv[e] * wt[k][e];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < DW_TT; ++i)
      if (t0 + i < T) st8(y + static_cast<size_t>(t0 + i) * C + c, acc[i]);
  }
}

// dw[c][k] += sum_t dy[t][c] x[t+k-r][c];  dbias[c] += sum_t dy[t][c]. One block handles a slab of
// tokens for 32 channels x 8 token lanes and reduces through shared memory before the atomics.
__global__ void __launch_bounds__(256)
dwconv_bwd_w_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                    const int* __restrict__ s_start, const int* __restrict__ s_end,
                    float* __restrict__ dw, float* __restrict__ dbias, int T, int C, int KS,
                    int tokens_per_block) {
  __shared__ float red[8][32][MAX_KS + 1];
  const int cl = threadIdx.x & 31;       // channel lane
  const int tl = threadIdx.x >> 5;       // token lane
  const int c = blockIdx.y * 32 + cl;
  const int r = KS >> 1;
  float acc[MAX_KS + 1];
#pragma unroll
  for (int k = 0; k <= MAX_KS; ++k) acc[k] = 0.f;
  const int t0 = blockIdx.x * tokens_per_block;
  const int t1 = min(T, t0 + tokens_per_block);
  if (c < C) {
    for (int t = t0 + tl; t < t1; t += 8) {
      const float g = __bfloat162float(dy[static_cast<size_t>(t) * C + c]);
      const int a = s_start[t], b = s_end[t];
      acc[MAX_KS] += g;
#pragma unroll
      for (int k = 0; k < MAX_KS; ++k) {
        if (k < KS) {
          const int src = t + k - r;
          if (src >= a && src < b) acc[k] += g * __bfloat162float(x[static_cast<size_t>(src) * C + c]);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k <= MAX_KS; ++k) red[tl][cl][k] = acc[k];
  __syncthreads();
  if (tl == 0 && c < C) {
    for (int k = 0; k <= MAX_KS; ++k) {
      float s = 0.f;
      for (int j = 0; j < 8; ++j) s += red[j][cl][k];
      if (k < KS) atomicAdd(&dw[c * KS + k], s);
      else if (k == MAX_KS && dbias != nullptr) atomicAdd(&dbias[c], s);
    }
  }
}

// Weight gradient with the kernel size known at compile time: same block shape, but a token lane
// walks one contiguous run of the slab and keeps the KS input values around the current token in
// registers, so a token costs one x and one dy load instead of KS + 1.
template <int KS>
__global__ void __launch_bounds__(256)
dwconv_bwd_w_tile_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                         const int* __restrict__ s_start, const int* __restrict__ s_end,
                         float* __restrict__ dw, float* __restrict__ dbias, int T, int C,
                         int tokens_per_block) {
  constexpr int R = KS / 2;
  __shared__ float red[8][32][KS + 1];
  const int cl = threadIdx.x & 31;       // channel lane
  const int tl = threadIdx.x >> 5;       // token lane
  const int c = blockIdx.y * 32 + cl;
  float acc[KS + 1];
#pragma unroll
  for (int k = 0; k <= KS; ++k) acc[k] = 0.f;
  const int run = (tokens_per_block + 7) / 8;
  const int ts = blockIdx.x * tokens_per_block + tl * run;
  const int te = min(min(T, ts + run), (static_cast<int>(blockIdx.x) + 1) * tokens_per_block);
  if (c < C && ts < te) {
    float win[KS];   // x[t - R .. t + R] of channel c
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      const int src = ts - R + k;
      win[k] = (src >= 0 && src < T) ? __bfloat162float(x[static_cast<size_t>(src) * C + c]) : 0.f;
    }
    for (int t = ts; t < te; ++t) {
      const float g = __bfloat162float(dy[static_cast<size_t>(t) * C + c]);
      const int a = s_start[t], b = s_end[t];
      const int nsrc = t + 1 + R;
      const float nx = nsrc < T ? __bfloat162float(x[static_cast<size_t>(nsrc) * C + c]) : 0.f;
      acc[KS] += g;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        const int src = t + k - R;
        if (src >= a && src < b) acc[k] += g * win[k];
      }
#pragma unroll
      for (int k = 0; k + 1 < KS; ++k) win[k] = win[k + 1];
      win[KS - 1] = nx;
    }
  }
#pragma unroll
  for (int k = 0; k <= KS; ++k) red[tl][cl][k] = acc[k];
  __syncthreads();
  if (tl == 0 && c < C) {
#pragma unroll
    for (int k = 0; k <= KS; ++k) {
      float sum = 0.f;
      for (int j = 0; j < 8; ++j) sum += red[j][cl][k];
      if (k < KS) atomicAdd(&dw[c * KS + k], sum);
      else if (dbias != nullptr) atomicAdd(&dbias[c], sum);
    }
  }
}

// ---------------------------------------------------------------------------- mHC
constexpr int MAX_STREAMS = 8;

// h[t][:] = sum_i alpha[t][i] X[t][i][:]
__global__ void __launch_bounds__(256)
mhc_read_kernel(const __nv_bfloat16* __restrict__ X, const float* __restrict__ alpha,
                __nv_bfloat16* __restrict__ h, int T, int n, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(T) * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec);
    const int c = static_cast<int>(idx % vec) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < n; ++i) {
      float xv[8];
      ld8(X + (static_cast<size_t>(t) * n + i) * C + c, xv);
      const float a = alpha[t * n + i];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += a * xv[e];
    }
    st8(h + static_cast<size_t>(t) * C + c, acc);
  }
}

// Xn[t][i][:] = sum_j R[t][i][j] X[t][j][:] + beta[t][i] y[t][:]
// N = number of streams (compile-time, so every per-stream array stays in registers).
template <int N>
__global__ void __launch_bounds__(256)
mhc_write_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ y,
                 const float* __restrict__ R, const float* __restrict__ beta,
                 __nv_bfloat16* __restrict__ Xn, int T, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(T) * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec);
    const int c = static_cast<int>(idx % vec) * 8;
    uint4 xr[N];
#pragma unroll
    for (int j = 0; j < N; ++j)
      xr[j] = __ldg(reinterpret_cast<const uint4*>(X + (static_cast<size_t>(t) * N + j) * C + c));
    float yv[8];
    ld8(y + static_cast<size_t>(t) * C + c, yv);
    float acc[N][8];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float bt = beta[t * N + i];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] = bt * yv[e];
    }
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float xv[8];
      unpack8x(xr[j], xv);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float rr = R[(t * N + i) * N + j];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] += rr * xv[e];
      }
    }
#pragma unroll
    for (int i = 0; i < N; ++i) st8(Xn + (static_cast<size_t>(t) * N + i) * C + c, acc[i]);
  }
}

// Sum of V <= 32 per-lane values over the warp: lane l (l < 32) returns the total of value l.
// Five exchange rounds that halve the number of live values (31 shuffles instead of 5 per value).
template <int V>
__device__ __forceinline__ float warp_transpose_sum(float (&v)[32], int lane) {
#pragma unroll
  for (int i = V; i < 32; ++i) v[i] = 0.f;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float keep = upper ? v[i + off] : v[i];
      const float send = upper ? v[i] : v[i + off];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

// Backward of read and / or write, one warp per token (dXn == null: read part only, dh == null:
// write part only; outputs of the missing part are not touched):
//   given dXn[t][i][:] (gradient of the written streams) and dh[t][:] (gradient of the read),
//   dX[t][j][:]  = sum_i R[t][i][j] dXn[t][i][:] + alpha[t][j] dh[t][:]
//   dy[t][:]     = sum_i beta[t][i] dXn[t][i][:]
//   dR[t][i][j]  = <dXn[t][i], X[t][j]>,  dbeta[t][i] = <dXn[t][i], y[t]>,  dalpha[t][j] = <dh[t], X[t][j]>
// All loads of a 256-channel slice are issued before the first use and kept packed in registers.
template <int N>
__global__ void __launch_bounds__(256, 2)
mhc_bwd_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ y,
               const float* __restrict__ R, const float* __restrict__ alpha, const float* __restrict__ beta,
               const __nv_bfloat16* __restrict__ dXn, const __nv_bfloat16* __restrict__ dh,
               __nv_bfloat16* __restrict__ dX, __nv_bfloat16* __restrict__ dy, float* __restrict__ dR,
               float* __restrict__ dalpha, float* __restrict__ dbeta, int T, int C) {
  static_assert(N * N + 2 * N <= 32, "too many streams for the warp-transpose reduction");
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const bool has_w = dXn != nullptr, has_r = dh != nullptr;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    // sums[i * N + j] = dR[i][j], sums[N*N + i] = dbeta[i], sums[N*N + N + j] = dalpha[j]
    float sums[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) sums[i] = 0.f;
    float rc[N][N], bt[N], al[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      bt[i] = has_w ? beta[t * N + i] : 0.f;
      al[i] = has_r ? alpha[t * N + i] : 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) rc[i][j] = has_w ? R[(t * N + i) * N + j] : 0.f;
    }
#pragma unroll 1
    for (int c = lane * 8; c < C; c += 256) {
      uint4 xr[N], gr[N], yr = make_uint4(0u, 0u, 0u, 0u), hr = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        xr[j] = __ldg(reinterpret_cast<const uint4*>(X + (static_cast<size_t>(t) * N + j) * C + c));
        gr[j] = has_w ? __ldg(reinterpret_cast<const uint4*>(dXn + (static_cast<size_t>(t) * N + j) * C + c))
                      : make_uint4(0u, 0u, 0u, 0u);
      }
      if (has_w) yr = __ldg(reinterpret_cast<const uint4*>(y + static_cast<size_t>(t) * C + c));
      if (has_r) hr = __ldg(reinterpret_cast<const uint4*>(dh + static_cast<size_t>(t) * C + c));
      float yv[8], hv[8];
      unpack8x(yr, yv);
      unpack8x(hr, hv);
      float dyv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float o[N][8];
#pragma unroll
      for (int j = 0; j < N; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) o[j][e] = al[j] * hv[e];
#pragma unroll
      for (int j = 0; j < N; ++j) {
        float xv[8];
        unpack8x(xr[j], xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) sums[N * N + N + j] += hv[e] * xv[e];
#pragma unroll
        for (int i = 0; i < N; ++i) {
          float gv[8];
          unpack8x(gr[i], gv);
#pragma unroll
          for (int e = 0; e < 8; ++e) sums[i * N + j] += gv[e] * xv[e];
        }
      }
#pragma unroll
      for (int i = 0; i < N; ++i) {
        float gv[8];
        unpack8x(gr[i], gv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dyv[e] += bt[i] * gv[e];
          sums[N * N + i] += gv[e] * yv[e];
        }
#pragma unroll
        for (int j = 0; j < N; ++j)
#pragma unroll
          for (int e = 0; e < 8; ++e) o[j][e] += rc[i][j] * gv[e];
      }
      if (has_w) st8(dy + static_cast<size_t>(t) * C + c, dyv);
#pragma unroll
      if (dX != nullptr) {
#pragma unroll
        for (int j = 0; j < N; ++j) st8(dX + (static_cast<size_t>(t) * N + j) * C + c, o[j]);
      }
    }
    // every lane takes part in the reduction; lane l ends up with the total of sums[l]
    const float total = warp_transpose_sum<N * N + 2 * N>(sums, lane);
    if (lane < N * N) {
      if (has_w) dR[t * N * N + lane] = total;
    } else if (lane < N * N + N) {
      if (has_w) dbeta[t * N + (lane - N * N)] = total;
    } else if (lane < N * N + 2 * N) {
      if (has_r) dalpha[t * N + (lane - N * N - N)] = total;
    }
  }
}

// z[t][:] = (1/n) sum_i X[t][i][:]   (what the coefficient network of a site sees)
__global__ void __launch_bounds__(256)
mhc_mean_kernel(const __nv_bfloat16* __restrict__ X, __nv_bfloat16* __restrict__ z, int T, int n, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(T) * vec;
  const float inv = 1.f / static_cast<float>(n);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec);
    const int c = static_cast<int>(idx % vec) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < n; ++i) {
      float xv[8];
      ld8(X + (static_cast<size_t>(t) * n + i) * C + c, xv);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += xv[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv;
    st8(z + static_cast<size_t>(t) * C + c, acc);
  }
}

// Gradient of the streams entering a site, all three consumers in one pass:
//   dX[t][j][:] = g[t][j][:] (from the write, may be null) + alpha[t][j] dh[t][:] (read, may be null)
//                 + dz[t][:] / n (stream mean, may be null)
__global__ void __launch_bounds__(256)
mhc_dx_combine_kernel(const __nv_bfloat16* __restrict__ g, const float* __restrict__ alpha,
                      const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ dz,
                      __nv_bfloat16* __restrict__ dX, int T, int n, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(T) * vec;
  const float inv = 1.f / static_cast<float>(n);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec);
    const int c = static_cast<int>(idx % vec) * 8;
    float hv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, zv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (dh != nullptr) ld8(dh + static_cast<size_t>(t) * C + c, hv);
    if (dz != nullptr) {
      ld8(dz + static_cast<size_t>(t) * C + c, zv);
#pragma unroll
      for (int e = 0; e < 8; ++e) zv[e] *= inv;
    }
    for (int j = 0; j < n; ++j) {
      float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (g != nullptr) ld8(g + (static_cast<size_t>(t) * n + j) * C + c, o);
      const float a = (dh != nullptr) ? alpha[t * n + j] : 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] += a * hv[e] + zv[e];
      st8(dX + (static_cast<size_t>(t) * n + j) * C + c, o);
    }
  }
}

static int grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  if (b > 148LL * 16) b = 148LL * 16;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace nplm

using namespace nplm;

extern "C" int nplm_dwconv(const void* x, const void* w, const void* bias, const int* s_start,
                           const int* s_end, void* y, int T, int C, int KS, int flip, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((C % 8) || KS < 1 || KS > MAX_KS || !(KS & 1)) return -3;
  const bool aligned = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
  if ((KS == 3 || KS == 5 || KS == 7 || KS == 9) && aligned) {   // the tile kernel loads 16-byte words of w
    const int grid = grid_for(static_cast<long long>((T + DW_TT - 1) / DW_TT) * (C / 8), 256);
#define NPLM_DWCONV(KS_)                                                                                   \
  dwconv_tile_kernel<KS_><<<grid, 256, 0, st>>>(                                                           \
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),                \
      reinterpret_cast<const __nv_bfloat16*>(bias), s_start, s_end, reinterpret_cast<__nv_bfloat16*>(y), T, C, flip)
    switch (KS) {
      case 3: NPLM_DWCONV(3); break;
      case 5: NPLM_DWCONV(5); break;
      case 7: NPLM_DWCONV(7); break;
      default: NPLM_DWCONV(9); break;
    }
#undef NPLM_DWCONV
    return static_cast<int>(cudaGetLastError());
  }
  dwconv_kernel<<<grid_for(static_cast<long long>(T) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<const __nv_bfloat16*>(bias), s_start, s_end, reinterpret_cast<__nv_bfloat16*>(y), T, C,
      KS, flip);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_dwconv_bwd_w(const void* x, const void* dy, const int* s_start, const int* s_end,
                                 float* dw, float* dbias, int T, int C, int KS, cudaStream_t st) {
  if (T <= 0) return 0;
  if (KS < 1 || KS > MAX_KS || !(KS & 1)) return -3;
  const int tokens_per_block = 512;
  dim3 grid((T + tokens_per_block - 1) / tokens_per_block, (C + 31) / 32);
  if (KS == 3 || KS == 5 || KS == 7 || KS == 9) {
#define NPLM_DWCONV_W(KS_)                                                                              \
  dwconv_bwd_w_tile_kernel<KS_><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x),          \
                                                      reinterpret_cast<const __nv_bfloat16*>(dy), s_start, \
                                                      s_end, dw, dbias, T, C, tokens_per_block)
    switch (KS) {
      case 3: NPLM_DWCONV_W(3); break;
      case 5: NPLM_DWCONV_W(5); break;
      case 7: NPLM_DWCONV_W(7); break;
      default: NPLM_DWCONV_W(9); break;
    }
#undef NPLM_DWCONV_W
    return static_cast<int>(cudaGetLastError());
  }
  dwconv_bwd_w_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                            reinterpret_cast<const __nv_bfloat16*>(dy), s_start, s_end, dw,
                                            dbias, T, C, KS, tokens_per_block);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_mhc_read(const void* X, const float* alpha, void* h, int T, int n, int C, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((C % 8) || n < 1 || n > MAX_STREAMS) return -3;
  mhc_read_kernel<<<grid_for(static_cast<long long>(T) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(X), alpha, reinterpret_cast<__nv_bfloat16*>(h), T, n, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_mhc_mean(const void* X, void* z, int T, int n, int C, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((C % 8) || n < 1 || n > MAX_STREAMS) return -3;
  mhc_mean_kernel<<<grid_for(static_cast<long long>(T) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(X), reinterpret_cast<__nv_bfloat16*>(z), T, n, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_mhc_dx_combine(const void* g, const float* alpha, const void* dh, const void* dz, void* dX,
                                   int T, int n, int C, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((C % 8) || n < 1 || n > MAX_STREAMS || (dh != nullptr && alpha == nullptr)) return -3;
  mhc_dx_combine_kernel<<<grid_for(static_cast<long long>(T) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(g), alpha, reinterpret_cast<const __nv_bfloat16*>(dh),
      reinterpret_cast<const __nv_bfloat16*>(dz), reinterpret_cast<__nv_bfloat16*>(dX), T, n, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_mhc_write(const void* X, const void* y, const float* R, const float* beta, void* Xn,
                              int T, int n, int C, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((C % 8) || n < 1 || n > 4) return -3;
  const int grid = grid_for(static_cast<long long>(T) * (C / 8), 256);
#define NPLM_MHC_WRITE(N_)                                                                              \
  mhc_write_kernel<N_><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(X),                  \
                                             reinterpret_cast<const __nv_bfloat16*>(y), R, beta,         \
                                             reinterpret_cast<__nv_bfloat16*>(Xn), T, C)
  switch (n) {
    case 1: NPLM_MHC_WRITE(1); break;
    case 2: NPLM_MHC_WRITE(2); break;
    case 3: NPLM_MHC_WRITE(3); break;
    default: NPLM_MHC_WRITE(4); break;
  }
#undef NPLM_MHC_WRITE
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_mhc_bwd(const void* X, const void* y, const float* R, const float* alpha,
                            const float* beta, const void* dXn, const void* dh, void* dX, void* dy,
                            float* dR, float* dalpha, float* dbeta, int T, int n, int C, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((C % 8) || n < 1 || n > 4) return -3;
  int blocks = (T + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
#define NPLM_MHC_BWD(N_)                                                                                  \
  mhc_bwd_kernel<N_><<<blocks, 256, 0, st>>>(                                                              \
      reinterpret_cast<const __nv_bfloat16*>(X), reinterpret_cast<const __nv_bfloat16*>(y), R, alpha, beta, \
      reinterpret_cast<const __nv_bfloat16*>(dXn), reinterpret_cast<const __nv_bfloat16*>(dh),              \
      reinterpret_cast<__nv_bfloat16*>(dX), reinterpret_cast<__nv_bfloat16*>(dy), dR, dalpha, dbeta, T, C)
  switch (n) {
    case 1: NPLM_MHC_BWD(1); break;
    case 2: NPLM_MHC_BWD(2); break;
    case 3: NPLM_MHC_BWD(3); break;
    default: NPLM_MHC_BWD(4); break;
  }
#undef NPLM_MHC_BWD
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------- device-side MLM masking
// Counter-based (Philox4x32-10) masking of packed token ids, the semantics of the host collator
// (src/nanoplm/pretraining/collator.py:333-382): a position is selected with probability p_sel
// unless its id is special (bit set in special_mask) or it lies at / beyond n_real; selected
// positions keep their id as label and become <mask> with probability p_mask, a random id from
// pool[0..pool_n) with probability p_rand, or stay unchanged. The stream depends only on
// (seed, step, position), so a batch is reproducible whatever the launch geometry.
#include <curand_kernel.h>

namespace nplm {

__global__ void __launch_bounds__(256)
mlm_mask_kernel(const long long* __restrict__ ids_in, long long* __restrict__ ids_out,
                long long* __restrict__ labels, int n, int n_real, unsigned long long special_mask,
                int mask_id, const int* __restrict__ pool, int pool_n, float p_sel, float p_mask,
                float p_rand, unsigned long long seed, unsigned long long step) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    curandStatePhilox4_32_10_t st;
    curand_init(seed, static_cast<unsigned long long>(i), step * 4ULL, &st);
    const float4 u = curand_uniform4(&st);
    const long long id = ids_in[i];
    const bool special = id < 0 || id >= 64 || ((special_mask >> id) & 1ULL) || i >= n_real;
    long long out = id, lab = -100;
    if (!special && u.x <= p_sel) {        // curand_uniform is (0, 1]
      lab = id;
      if (u.y <= p_mask) {
        out = mask_id;
      } else if (u.y <= p_mask + p_rand) {
        int k = static_cast<int>(u.z * pool_n);
        if (k >= pool_n) k = pool_n - 1;
        out = pool[k];
      }
    }
    ids_out[i] = out;
    labels[i] = lab;
  }
}

}  // namespace nplm

extern "C" int nplm_mlm_mask(const long long* ids_in, long long* ids_out, long long* labels, int n, int n_real,
                             unsigned long long special_mask, int mask_id, const int* pool, int pool_n,
                             float p_sel, float p_mask, float p_rand, unsigned long long seed,
                             unsigned long long step, cudaStream_t st) {
  if (n <= 0) return 0;
  if (pool_n <= 0) return -3;
  int blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  nplm::mlm_mask_kernel<<<blocks, 256, 0, st>>>(ids_in, ids_out, labels, n, n_real, special_mask, mask_id, pool,
                                                pool_n, p_sel, p_mask, p_rand, seed, step);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------- mHC coefficients
// One thread per token turns the raw outputs of the coefficient projection (before tanh) into the
// mixing coefficients of one hyper-connection site:
//   d      = tanh(pre[t, :])                                   [2N + N*N]
//   alpha  = softmax(a + s0 * d[0:N])
//   beta   = 2 * sigmoid(b + s1 * d[N:2N])
//   R      = exp(sinkhorn_log(r + s2 * d[2N:], iters))         (rows, then columns, `iters` times)
// The backward kernel recomputes the forward, keeps the value after every Sinkhorn half-step
// (for y = x - logsumexp(x): dx = dy - exp(y) * sum(dy)), and returns the gradient w.r.t. pre
// (bf16) plus block-reduced atomics for the static parameters a, b, r and the three scales.
// The reference has no hyper-connections.
namespace nplm {

constexpr int MHC_MAX_ITERS = 8;

template <int N>
__device__ __forceinline__ void mhc_coef_forward(const float (&d)[2 * N + N * N], const float* a, const float* b,
                                                 const float* r, const float* s, int iters,
                                                 float (&alpha)[N], float (&beta)[N], float (&x)[N * N],
                                                 float* hist) {
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    alpha[i] = a[i] + s[0] * d[i];
    mx = fmaxf(mx, alpha[i]);
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    alpha[i] = __expf(alpha[i] - mx);
    sum += alpha[i];
  }
#pragma unroll
  for (int i = 0; i < N; ++i) alpha[i] /= sum;
#pragma unroll
  for (int i = 0; i < N; ++i) beta[i] = 2.f / (1.f + __expf(-(b[i] + s[1] * d[N + i])));
#pragma unroll
  for (int i = 0; i < N * N; ++i) x[i] = r[i] + s[2] * d[2 * N + i];
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < N; ++i) {   // rows
      float m = -INFINITY, se = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) m = fmaxf(m, x[i * N + j]);
#pragma unroll
      for (int j = 0; j < N; ++j) se += __expf(x[i * N + j] - m);
      const float lse = m + __logf(se);
#pragma unroll
      for (int j = 0; j < N; ++j) x[i * N + j] -= lse;
    }
    if (hist != nullptr) {
#pragma unroll
      for (int i = 0; i < N * N; ++i) hist[(2 * it) * N * N + i] = x[i];
    }
#pragma unroll
    for (int j = 0; j < N; ++j) {   // columns
      float m = -INFINITY, se = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) m = fmaxf(m, x[i * N + j]);
#pragma unroll
      for (int i = 0; i < N; ++i) se += __expf(x[i * N + j] - m);
      const float lse = m + __logf(se);
#pragma unroll
      for (int i = 0; i < N; ++i) x[i * N + j] -= lse;
    }
    if (hist != nullptr) {
#pragma unroll
      for (int i = 0; i < N * N; ++i) hist[(2 * it + 1) * N * N + i] = x[i];
    }
  }
}

template <int N>
__global__ void __launch_bounds__(128)
mhc_coef_fwd_kernel(const __nv_bfloat16* __restrict__ pre, const float* __restrict__ a,
                    const float* __restrict__ b, const float* __restrict__ r, const float* __restrict__ s,
                    int iters, int T, float* __restrict__ alpha_out, float* __restrict__ beta_out,
                    float* __restrict__ R_out) {
  constexpr int M = 2 * N + N * N;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    float d[M];
#pragma unroll
    for (int i = 0; i < M; ++i) d[i] = tanhf(__bfloat162float(pre[static_cast<size_t>(t) * M + i]));
    float alpha[N], beta[N], x[N * N];
    mhc_coef_forward<N>(d, a, b, r, s, iters, alpha, beta, x, nullptr);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      alpha_out[t * N + i] = alpha[i];
      beta_out[t * N + i] = beta[i];
    }
#pragma unroll
    for (int i = 0; i < N * N; ++i) R_out[static_cast<size_t>(t) * N * N + i] = __expf(x[i]);
  }
}

template <int N>
__global__ void __launch_bounds__(128)
mhc_coef_bwd_kernel(const __nv_bfloat16* __restrict__ pre, const float* __restrict__ a,
                    const float* __restrict__ b, const float* __restrict__ r, const float* __restrict__ s,
                    int iters, int T, const float* __restrict__ dalpha, const float* __restrict__ dbeta,
                    const float* __restrict__ dR, __nv_bfloat16* __restrict__ dpre,
                    float* __restrict__ da, float* __restrict__ db, float* __restrict__ dr,
                    float* __restrict__ ds) {
  constexpr int M = 2 * N + N * N;
  static_assert(M + 3 <= 32, "parameter gradients are reduced with one value per lane");
  // per-thread sums of the parameter gradients: [da (N) | db (N) | dr (N*N) | ds (3)]
  float acc[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) acc[i] = 0.f;
  const int lane = threadIdx.x & 31;
  // every warp runs the same number of iterations (the reduction below is warp-wide)
  const int per_pass = gridDim.x * blockDim.x;
  for (int base = blockIdx.x * blockDim.x; base < T; base += per_pass) {
    const int t = base + threadIdx.x;
    if (t < T) {
      float d[M];
#pragma unroll
      for (int i = 0; i < M; ++i) d[i] = tanhf(__bfloat162float(pre[static_cast<size_t>(t) * M + i]));
      float alpha[N], beta[N], x[N * N];
      float hist[2 * MHC_MAX_ITERS * N * N];
      mhc_coef_forward<N>(d, a, b, r, s, iters, alpha, beta, x, hist);
      float gd[M];   // gradient w.r.t. d (tanh output)
      // alpha = softmax(u): du = alpha * (dalpha - sum alpha * dalpha)
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) dot += alpha[i] * dalpha[t * N + i];
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float du = alpha[i] * (dalpha[t * N + i] - dot);
        acc[i] += du;
        acc[2 * N + N * N] += du * d[i];
        gd[i] = du * s[0];
      }
      // beta = 2 sigmoid(v): dv = dbeta * beta * (1 - beta / 2)
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float dv = dbeta[t * N + i] * beta[i] * (1.f - 0.5f * beta[i]);
        acc[N + i] += dv;
        acc[2 * N + N * N + 1] += dv * d[N + i];
        gd[N + i] = dv * s[1];
      }
      // R = exp(x_final): dx = dR * R, then back through the half-steps
      float g[N * N];
#pragma unroll
      for (int i = 0; i < N * N; ++i) g[i] = dR[static_cast<size_t>(t) * N * N + i] * __expf(x[i]);
      for (int it = iters - 1; it >= 0; --it) {
        const float* yc = hist + (2 * it + 1) * N * N;   // after the column step
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float sg = 0.f;
#pragma unroll
          for (int i = 0; i < N; ++i) sg += g[i * N + j];
#pragma unroll
          for (int i = 0; i < N; ++i) g[i * N + j] -= __expf(yc[i * N + j]) * sg;
        }
        const float* yr = hist + (2 * it) * N * N;       // after the row step
#pragma unroll
        for (int i = 0; i < N; ++i) {
          float sg = 0.f;
#pragma unroll
          for (int j = 0; j < N; ++j) sg += g[i * N + j];
#pragma unroll
          for (int j = 0; j < N; ++j) g[i * N + j] -= __expf(yr[i * N + j]) * sg;
        }
      }
#pragma unroll
      for (int i = 0; i < N * N; ++i) {
        acc[2 * N + i] += g[i];
        acc[2 * N + N * N + 2] += g[i] * d[2 * N + i];
        gd[2 * N + i] = g[i] * s[2];
      }
#pragma unroll
      for (int i = 0; i < M; ++i)
        dpre[static_cast<size_t>(t) * M + i] = __float2bfloat16(gd[i] * (1.f - d[i] * d[i]));
    }
  }
  // warp-wide sums (lane l receives the total of acc[l]), one atomic per value and warp
  const float total = warp_transpose_sum<M + 3>(acc, lane);
  if (lane < N) atomicAdd(&da[lane], total);
  else if (lane < 2 * N) atomicAdd(&db[lane - N], total);
  else if (lane < 2 * N + N * N) atomicAdd(&dr[lane - 2 * N], total);
  else if (lane < M + 3) atomicAdd(&ds[lane - M], total);
}

}  // namespace nplm

extern "C" int nplm_mhc_coef_fwd(const void* pre, const float* a, const float* b, const float* r,
                                 const float* s, int iters, int T, int n, float* alpha, float* beta,
                                 float* R, cudaStream_t st) {
  if (T <= 0) return 0;
  if (n != 4 && n != 2) return -3;
  if (iters < 1 || iters > nplm::MHC_MAX_ITERS) return -3;
  int blocks = (T + 127) / 128;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(pre);
  if (n == 4)
    nplm::mhc_coef_fwd_kernel<4><<<blocks, 128, 0, st>>>(p, a, b, r, s, iters, T, alpha, beta, R);
  else
    nplm::mhc_coef_fwd_kernel<2><<<blocks, 128, 0, st>>>(p, a, b, r, s, iters, T, alpha, beta, R);
  return static_cast<int>(cudaGetLastError());
}

// da / db / dr / ds are accumulated (callers pass zeroed or running fp32 buffers)
extern "C" int nplm_mhc_coef_bwd(const void* pre, const float* a, const float* b, const float* r,
                                 const float* s, int iters, int T, int n, const float* dalpha,
                                 const float* dbeta, const float* dR, void* dpre, float* da, float* db,
                                 float* dr, float* ds, cudaStream_t st) {
  if (T <= 0) return 0;
  if (n != 4 && n != 2) return -3;
  if (iters < 1 || iters > nplm::MHC_MAX_ITERS) return -3;
  int blocks = (T + 127) / 128;
  if (blocks > 148 * 4) blocks = 148 * 4;
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(pre);
  __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(dpre);
  if (n == 4)
    nplm::mhc_coef_bwd_kernel<4><<<blocks, 128, 0, st>>>(p, a, b, r, s, iters, T, dalpha, dbeta, dR, dp, da, db,
                                                         dr, ds);
  else
    nplm::mhc_coef_bwd_kernel<2><<<blocks, 128, 0, st>>>(p, a, b, r, s, iters, T, dalpha, dbeta, dR, dp, da, db,
                                                         dr, ds);
  return static_cast<int>(cudaGetLastError());
}
