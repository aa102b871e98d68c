// Memory-bound kernels for the encoder: LayerNorm / RMSNorm (fwd, bwd), embedding gather +
// norm, RoPE, SwiGLU, GELU backward, fused MLM-head cross-entropy (V <= 32), row gather /
// scatter, fused AdamW with on-device gradient clipping, sum of squares.
//
// They replace the ATen / Inductor-generated kernels the reference gets from
// src/nanoplm/pretraining/models/modern_bert/modeling.py:112-131 (RoPE), :219-223 (embedding +
// LayerNorm), :300-302 (SwiGLU), :555-559 (head), :659-664 (decoder + cross entropy) and
// src/nanoplm/pretraining/pure_pipeline.py:755-764 (clip + AdamW).
//
// Activations are bf16, statistics and gradients of parameters are fp32. All kernels are
// plain grid-stride / warp-per-row kernels: none of them waits on anything.
#include <stdlib.h>

#include "common.cuh"

namespace nplm {

constexpr int MAX_CHUNKS = 16;  // a warp keeps a row of up to 16*256 = 4096 channels in registers

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = unpack_bf16x2(w[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = unpack_bf16x2(w[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) w[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------ norm forward
// One warp per row. ids != nullptr: the row is gathered from table[ids[row]] (embedding).
// rms = 0: LayerNorm without bias, rms = 1: RMSNorm. w == nullptr means weight 1.
template <int CHUNKS>
__global__ void __launch_bounds__(256)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int C, float eps,
                int rms) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < T;
       row += gridDim.x * warps_per_block) {
    const __nv_bfloat16* src =
        ids ? x + static_cast<size_t>(ids[row]) * C : x + static_cast<size_t>(row) * C;
    float v[CHUNKS][8];
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
        load8(src + i, v[c]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += v[c][e];
      }
    }
    float mean = 0.f;
    if (!rms) mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = v[c][e] - mean;
          q += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
        float wv[8];
        if (w) {
          load8(w + i, wv);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) wv[e] = 1.f;
        }
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (v[c][e] - mean) * rstd * wv[e];
        store8(y + static_cast<size_t>(row) * C + i, o);
      }
    }
  }
}

// ------------------------------------------------------------------ norm backward
// dx = [dres +] rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * w   (LayerNorm)
// dx = [dres +] rstd * (g - xhat * mean(g * xhat))                           (RMSNorm)
// dw (fp32) accumulates sum_rows dy * xhat: registers per warp -> shared per block -> atomics.
// ids != nullptr (embedding): x rows are gathered from the table, dx is not written, and the
// row gradient is accumulated into dtable[ids[row]] (fp32) instead.
template <int CHUNKS>
__global__ void __launch_bounds__(256, 2)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ dw, float* __restrict__ dtable, int T, int C, int rms) {
  extern __shared__ float sm_dw[];  // [C]
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < C; i += blockDim.x) sm_dw[i] = 0.f;
  __syncthreads();

  float acc[CHUNKS][8];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[c][e] = 0.f;

  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < T;
       row += gridDim.x * warps_per_block) {
    const __nv_bfloat16* src =
        ids ? x + static_cast<size_t>(ids[row]) * C : x + static_cast<size_t>(row) * C;
    // Every global load of the row (x, dy and the skip gradient) is issued before the first use and
    // kept packed (bf16) in registers, so a warp has 6 KB in flight; the second pass unpacks again.
    uint4 xr[CHUNKS], dr[CHUNKS], rr[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      xr[c] = dr[c] = rr[c] = make_uint4(0u, 0u, 0u, 0u);
      if (i < C) {
        xr[c] = __ldg(reinterpret_cast<const uint4*>(src + i));
        dr[c] = __ldg(reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * C + i));
        if (dres) rr[c] = __ldg(reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * C + i));
      }
    }
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
        float xv[8], dv[8], wv[8];
        unpack8(xr[c], xv);
        unpack8(dr[c], dv);
        if (w) {
          load8(w + i, wv);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) wv[e] = 1.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = (xv[e] - mean) * rstd;
          const float g = dv[e] * wv[e];
          sg += g;
          sgx += g * xh;
          acc[c][e] += dv[e] * xh;
        }
      }
    }
    sg = rms ? 0.f : warp_sum(sg) / C;
    sgx = warp_sum(sgx) / C;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
        float xv[8], dv[8], wv[8], o[8];
        unpack8(xr[c], xv);
        unpack8(dr[c], dv);
        if (w) {
          load8(w + i, wv);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) wv[e] = 1.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = (xv[e] - mean) * rstd;
          o[e] = rstd * (dv[e] * wv[e] - sg - xh * sgx);
        }
        if (ids) {
          float* dst = dtable + static_cast<size_t>(ids[row]) * C + i;
#pragma unroll
          for (int e = 0; e < 8; ++e) atomicAdd(dst + e, o[e]);
        } else {
          if (dres) {
            float r[8];
            unpack8(rr[c], r);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += r[e];
          }
          store8(dx + static_cast<size_t>(row) * C + i, o);
        }
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
#pragma unroll
        for (int e = 0; e < 8; ++e) atomicAdd(&sm_dw[i + e], acc[c][e]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < C; i += blockDim.x) atomicAdd(&dw[i], sm_dw[i]);
  }
}

// Norm backward with a thread block per group of ROWS rows (C/8 threads, each owning 8 channels
// of every row of the group). All loads of a group are issued before the first reduction, so a
// block keeps ROWS * 3 * C * 2 bytes in flight; the row reductions of the whole group share one
// __syncthreads. Registers per thread stay low enough for several blocks per SM.
//   ids == nullptr : dx[row] = [dres[row] +] norm-backward(dy[row]),  dw += sum dy * xhat
//   ids != nullptr : embedding mode. x rows are table[ids[row]]; the row gradients are summed per
//                    vocabulary entry in shared memory (each thread owns its channels, so no
//                    atomics inside the block) and flushed to dtable with one atomic per element.
template <int ROWS, int SUB>
__global__ void __launch_bounds__(512)
norm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                     const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                     float* __restrict__ dw, float* __restrict__ dtable, int T, int C, int V, int rms) {
  extern __shared__ float s_table[];   // [V][C] in embedding mode
  // SUB row groups run side by side in one block (blockDim.x / SUB threads each): they share the
  // table sums, which therefore take shared-memory atomics (two groups may hold the same token)
  __shared__ float red[2][SUB][ROWS][8][2];
  const int cthreads = blockDim.x / SUB;
  const int sub = threadIdx.x / cthreads, tid = threadIdx.x % cthreads;
  const int lane = tid & 31, warp = tid >> 5, nwarps = cthreads >> 5;
  const int i = tid * 8;
  const bool on = i < C;
  if (ids != nullptr) {
    for (int k = threadIdx.x; k < V * C; k += blockDim.x) s_table[k] = 0.f;
    __syncthreads();
  }
  float wv[8], acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    wv[e] = 1.f;
    acc[e] = 0.f;
  }
  if (on && w) load8(w + i, wv);
  int buf = 0;
  // every thread of the block runs the same number of iterations (the barrier below is block-wide)
  for (int base = blockIdx.x * ROWS * SUB; base < T; base += gridDim.x * ROWS * SUB, buf ^= 1) {
    const int row0 = base + sub * ROWS;
    float xh[ROWS][8], g[ROWS][8];
    float rstd[ROWS];
    int id[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = row0 + r;
      float sg = 0.f, sgx = 0.f;
      rstd[r] = 0.f;
      id[r] = 0;
      if (row < T) {
        const float mean = rms ? 0.f : mean_in[row];
        rstd[r] = rstd_in[row];
        if (ids != nullptr) id[r] = ids[row];
        if (on) {
          float xv[8], dv[8];
          const __nv_bfloat16* src = ids ? x + static_cast<size_t>(id[r]) * C : x + static_cast<size_t>(row) * C;
          load8(src + i, xv);
          load8(dy + static_cast<size_t>(row) * C + i, dv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            xh[r][e] = (xv[e] - mean) * rstd[r];
            g[r][e] = dv[e] * wv[e];
            sg += g[r][e];
            sgx += g[r][e] * xh[r][e];
            acc[e] += dv[e] * xh[r][e];
          }
        }
      }
      sg = warp_sum(sg);
      sgx = warp_sum(sgx);
      if (lane == 0) {
        red[buf][sub][r][warp][0] = sg;
        red[buf][sub][r][warp][1] = sgx;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = row0 + r;
      if (row < T && on) {
        float tg = 0.f, tgx = 0.f;
        for (int k = 0; k < nwarps; ++k) {
          tg += red[buf][sub][r][k][0];
          tgx += red[buf][sub][r][k][1];
        }
        tg = rms ? 0.f : tg / C;
        tgx /= C;
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd[r] * (g[r][e] - tg - xh[r][e] * tgx);
        if (ids != nullptr) {
          float* dst = s_table + static_cast<size_t>(id[r]) * C + i;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (SUB > 1) atomicAdd(&dst[e], o[e]);
            else dst[e] += o[e];
          }
        } else {
          if (dres) {
            float rr[8];
            load8(dres + static_cast<size_t>(row) * C + i, rr);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += rr[e];
          }
          store8(dx + static_cast<size_t>(row) * C + i, o);
        }
      }
    }
  }
  if (dw && on) {
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(&dw[i + e], acc[e]);
  }
  if (ids != nullptr) {
    __syncthreads();
    for (int k = threadIdx.x; k < V * C; k += blockDim.x) {
      const float v = s_table[k];
      if (v != 0.f) atomicAdd(&dtable[k], v);
    }
  }
}

// ------------------------------------------------------------------ RoPE (in place on packed qkv)
// qkv: [T][3][H][D] bf16. Rotates q and k: out = x*cos + rotate_half(x)*sin with
// cos/sin[pos][D/2] fp32 (the two halves of the reference table are identical). sign = -1
// applies the transpose (backward).
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int T, int H, int D,
            float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;  // 8 elements per thread from each half
  const long long total = static_cast<long long>(T) * 2 * H * vec_per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vv = static_cast<int>(idx % vec_per_head);
    long long r = idx / vec_per_head;
    const int h = static_cast<int>(r % H);
    r /= H;
    const int qk = static_cast<int>(r % 2);
    const int t = static_cast<int>(r / 2);
    __nv_bfloat16* base = qkv + ((static_cast<size_t>(t) * 3 + qk) * H + h) * D + vv * 8;
    const int p = pos[t];
    const float* cp = cos_t + static_cast<size_t>(p) * half + vv * 8;
    const float* sp = sin_t + static_cast<size_t>(p) * half + vv * 8;
    float x1[8], x2[8], o1[8], o2[8];
    load8(base, x1);
    load8(base + half, x2);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float c = cp[e], s = sign * sp[e];
      o1[e] = x1[e] * c - x2[e] * s;
      o2[e] = x2[e] * c + x1[e] * s;
    }
    store8(base, o1);
    store8(base + half, o2);
  }
}

// ------------------------------------------------------------------ SwiGLU
// pre: [T][2I] = [value | gate]; out[T][I] = silu(gate) * value
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ out,
                  long long T, int I) {
  const int vec = I >> 3;
  const long long total = T * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / vec;
    const int i = static_cast<int>(idx % vec) * 8;
    float v[8], g[8], o[8];
    load8(pre + t * 2 * I + i, v);
    load8(pre + t * 2 * I + I + i, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.f + __expf(-g[e])) * v[e];
    store8(out + t * I + i, o);
  }
}

// dpre[T][2I] from dout[T][I]: dvalue = dout*silu(g), dgate = dout*v*sig(g)*(1+g*(1-sig(g)))
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ pre, const __nv_bfloat16* __restrict__ dout,
                  __nv_bfloat16* __restrict__ dpre, long long T, int I) {
  const int vec = I >> 3;
  const long long total = T * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / vec;
    const int i = static_cast<int>(idx % vec) * 8;
    float v[8], g[8], d[8], dv[8], dg[8];
    load8(pre + t * 2 * I + i, v);
    load8(pre + t * 2 * I + I + i, g);
    load8(dout + t * I + i, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-g[e]));
      dv[e] = d[e] * g[e] * sg;
      dg[e] = d[e] * v[e] * sg * (1.f + g[e] * (1.f - sg));
    }
    store8(dpre + t * 2 * I + i, dv);
    store8(dpre + t * 2 * I + I + i, dg);
  }
}

// ------------------------------------------------------------------ activations
// act: 0 gelu(erf), 1 relu, 2 silu
__global__ void __launch_bounds__(256)
act_fwd_kernel(const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ out,
               long long n8, int act) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < n8;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p[8], o[8];
    load8(pre + idx * 8, p);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[e] = act == 0 ? gelu_erf(p[e]) : act == 1 ? fmaxf(p[e], 0.f) : p[e] / (1.f + __expf(-p[e]));
    }
    store8(out + idx * 8, o);
  }
}

__global__ void __launch_bounds__(256)
act_bwd_kernel(const __nv_bfloat16* __restrict__ pre, const __nv_bfloat16* __restrict__ dout,
               __nv_bfloat16* __restrict__ dpre, long long n8, int act) {
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < n8;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p[8], d[8], o[8];
    load8(pre + idx * 8, p);
    load8(dout + idx * 8, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float gr;
      if (act == 0) {
        gr = gelu_erf_grad(p[e]);
      } else if (act == 1) {
        gr = p[e] > 0.f ? 1.f : 0.f;
      } else {
        const float sg = 1.f / (1.f + __expf(-p[e]));
        gr = sg * (1.f + p[e] * (1.f - sg));
      }
      o[e] = d[e] * gr;
    }
    store8(dpre + idx * 8, o);
  }
}

// ------------------------------------------------------------------ row gather / scatter
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx,
                   __nv_bfloat16* __restrict__ dst, int n, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(n) * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec);
    const int c = static_cast<int>(i % vec) * 8;
    *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * C + c) =
        *reinterpret_cast<const uint4*>(src + static_cast<size_t>(idx[r]) * C + c);
  }
}

// dst[idx[r]] = src[r] (indices are unique); rows not named keep their contents.
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx,
                    __nv_bfloat16* __restrict__ dst, int n, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(n) * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec);
    const int c = static_cast<int>(i % vec) * 8;
    *reinterpret_cast<uint4*>(dst + static_cast<size_t>(idx[r]) * C + c) =
        *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * C + c);
  }
}

// ------------------------------------------------------------------ fused MLM-head cross entropy
// One warp per row. h: [n][C] bf16 (output of the head norm), W: [V][C] bf16 (tied decoder),
// bias: [V] bf16 or null, labels: [n] int (ignore_index = -100). V <= 32.
// Writes dlogits[n][32] fp32 = (softmax - onehot) * inv_count (0 for ignored rows), optional
// logits[n][V] fp32, and accumulates loss_sum += -log p[label] * inv_count.
// inv_count is read from device memory (1 / number of valid labels).
constexpr int CE_WARPS = 8;

template <int CHUNKS>
__global__ void __launch_bounds__(CE_WARPS * 32)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ W,
              const __nv_bfloat16* __restrict__ bias, const int* __restrict__ labels,
              const float* __restrict__ inv_count, float* __restrict__ dlogits,
              float* __restrict__ logits_out, float* __restrict__ loss_sum, int n, int C, int V) {
  extern __shared__ __nv_bfloat16 sW[];  // [V][C]
  for (int i = threadIdx.x * 8; i < V * C; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(sW + i) = *reinterpret_cast<const uint4*>(W + i);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const float invc = *inv_count;
  float block_loss = 0.f;
  for (int row = blockIdx.x * CE_WARPS + (threadIdx.x >> 5); row < n; row += gridDim.x * CE_WARPS) {
    float hv[CHUNKS][8];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) load8(h + static_cast<size_t>(row) * C + i, hv[c]);
    }
    float part[32];
#pragma unroll
    for (int v = 0; v < 32; ++v) {
      float s = 0.f;
      if (v < V) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          const int i = c * 256 + lane * 8;
          if (i < C) {
            float wv[8];
            load8(sW + v * C + i, wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) s += hv[c][e] * wv[e];
          }
        }
      }
      part[v] = s;
    }
    // transpose-reduce: after the 5 steps lane l holds the full sum for vocab entry l
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
      const bool upper = (lane & step) != 0;
#pragma unroll
      for (int j = 0; j < step; ++j) {
        const float send = upper ? part[j] : part[j + step];
        const float keep = upper ? part[j + step] : part[j];
        part[j] = keep + __shfl_xor_sync(0xffffffffu, send, step);
      }
    }
    float logit = part[0];
    if (lane < V) {
      if (bias) logit += __bfloat162float(bias[lane]);
    } else {
      logit = -INFINITY;
    }
    if (logits_out && lane < V) logits_out[static_cast<size_t>(row) * V + lane] = logit;
    const float mx = warp_max(logit);
    const float ex = lane < V ? __expf(logit - mx) : 0.f;
    const float se = warp_sum(ex);
    const int lab = labels[row];
    float dl = 0.f;
    if (lab >= 0) {
      const float p = ex / se;
      dl = (p - (lane == lab ? 1.f : 0.f)) * invc;
      const float lab_logit = __shfl_sync(0xffffffffu, logit, lab);
      if (lane == 0) block_loss += (mx + __logf(se) - lab_logit) * invc;
    }
    dlogits[static_cast<size_t>(row) * 32 + lane] = dl;
  }
  if (lane == 0 && block_loss != 0.f) atomicAdd(loss_sum, block_loss);
}

// Backward: dh[row] = g * sum_v dl[row][v] W[v];  dW[v] += g * sum_rows dl[row][v] h[row];
// dbias[v] += g * sum_rows dl[row][v].  g = *gscale (upstream gradient of the loss).
// dW is accumulated per block in shared memory ([V][C] fp32) and flushed with atomics.
template <int CHUNKS>
__global__ void __launch_bounds__(CE_WARPS * 32)
ce_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ W,
              const float* __restrict__ dlogits, const float* __restrict__ gscale,
              __nv_bfloat16* __restrict__ dh, float* __restrict__ dW, float* __restrict__ dbias,
              int n, int C, int V) {
  extern __shared__ float sdW[];  // [V][C] fp32, then [32] dbias
  float* sdb = sdW + V * C;
  for (int i = threadIdx.x; i < V * C + 32; i += blockDim.x) sdW[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const float g = *gscale;
  for (int row = blockIdx.x * CE_WARPS + (threadIdx.x >> 5); row < n; row += gridDim.x * CE_WARPS) {
    const float dl = dlogits[static_cast<size_t>(row) * 32 + lane] * g;
    if (__ballot_sync(0xffffffffu, dl != 0.f) == 0u) {
      // ignored row: zero gradient
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int i = c * 256 + lane * 8;
        if (i < C) *reinterpret_cast<uint4*>(dh + static_cast<size_t>(row) * C + i) = make_uint4(0, 0, 0, 0);
      }
      continue;
    }
    if (lane < V) atomicAdd(&sdb[lane], dl);
    // broadcast every dlogit to every lane first: the shuffles need the whole warp, the channel
    // loop below does not run on lanes whose channels lie beyond C
    float dv[32];
#pragma unroll
    for (int v = 0; v < 32; ++v) dv[v] = __shfl_sync(0xffffffffu, dl, v);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = c * 256 + lane * 8;
      if (i < C) {
        float hv[8], o[8];
        load8(h + static_cast<size_t>(row) * C + i, hv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = 0.f;
#pragma unroll
        for (int v = 0; v < 32; ++v) {
          if (v < V) {
            const float d = dv[v];
            float wv[8];
            load8(W + static_cast<size_t>(v) * C + i, wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              o[e] += d * wv[e];
              atomicAdd(&sdW[v * C + i + e], d * hv[e]);
            }
          }
        }
        store8(dh + static_cast<size_t>(row) * C + i, o);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V * C; i += blockDim.x) {
    const float v = sdW[i];
    if (v != 0.f) atomicAdd(&dW[i], v);
  }
  if (dbias && threadIdx.x < V) atomicAdd(&dbias[threadIdx.x], sdb[threadIdx.x]);
}

// Same backward for C <= 1024 (C % 4 == 0) as a tiled product: a block stages 32 rows of h (bf16)
// and their dlogits in shared memory next to W; thread t owns channels 4t .. 4t+3 and keeps
// dW[v][4t..4t+3] for all v in registers (4 V accumulators), so a row costs 8 V FMAs per thread and
// no atomics; the block's dW is flushed once at the end.
constexpr int CE_TILE_ROWS = 32;

__global__ void __launch_bounds__(256)
ce_bwd_tiled_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ W,
                    const float* __restrict__ dlogits, const float* __restrict__ gscale,
                    __nv_bfloat16* __restrict__ dh, float* __restrict__ dW, float* __restrict__ dbias,
                    int n, int C, int V) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __nv_bfloat16* sW = reinterpret_cast<__nv_bfloat16*>(ce_smem);            // [V][C]
  __nv_bfloat16* sH = sW + static_cast<size_t>(V) * C;                       // [32][C]
  float* sD = reinterpret_cast<float*>(sH + static_cast<size_t>(CE_TILE_ROWS) * C);  // [32][32]
  const int t = threadIdx.x;
  for (int i = t * 8; i < V * C; i += 256 * 8)
    *reinterpret_cast<uint4*>(sW + i) = *reinterpret_cast<const uint4*>(W + i);
  const float g = *gscale;
  const int ch = t * 4;
  const bool own = ch < C;
  float acc[32][4];
#pragma unroll
  for (int v = 0; v < 32; ++v)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[v][e] = 0.f;
  float db = 0.f;
  const int tiles = (n + CE_TILE_ROWS - 1) / CE_TILE_ROWS;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int r0 = tile * CE_TILE_ROWS;
    __syncthreads();   // previous tile fully consumed (and sW written, first time round)
    for (int i = t * 8; i < CE_TILE_ROWS * C; i += 256 * 8) {
      const int r = i / C;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r0 + r < n) val = *reinterpret_cast<const uint4*>(h + static_cast<size_t>(r0) * C + i);
      *reinterpret_cast<uint4*>(sH + i) = val;
    }
    for (int i = t; i < CE_TILE_ROWS * 32; i += 256) {
      const int r = i >> 5;
      sD[i] = (r0 + r < n) ? dlogits[static_cast<size_t>(r0) * 32 + i] * g : 0.f;
    }
    __syncthreads();
    if (t < V) {
#pragma unroll 8
      for (int r = 0; r < CE_TILE_ROWS; ++r) db += sD[r * 32 + t];
    }
    if (own) {
      const int rows = min(CE_TILE_ROWS, n - r0);
      for (int r = 0; r < rows; ++r) {
        const uint2 hp = *reinterpret_cast<const uint2*>(sH + static_cast<size_t>(r) * C + ch);
        const float2 h01 = unpack_bf16x2(hp.x), h23 = unpack_bf16x2(hp.y);
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int v = 0; v < 32; ++v) {
          if (v < V) {
            const float d = sD[r * 32 + v];
            const uint2 wp = *reinterpret_cast<const uint2*>(sW + static_cast<size_t>(v) * C + ch);
            const float2 w01 = unpack_bf16x2(wp.x), w23 = unpack_bf16x2(wp.y);
            o0 += d * w01.x; o1 += d * w01.y; o2 += d * w23.x; o3 += d * w23.y;
            acc[v][0] += d * h01.x; acc[v][1] += d * h01.y; acc[v][2] += d * h23.x; acc[v][3] += d * h23.y;
          }
        }
        uint2 op;
        op.x = pack_bf16x2(o0, o1);
        op.y = pack_bf16x2(o2, o3);
        *reinterpret_cast<uint2*>(dh + static_cast<size_t>(r0 + r) * C + ch) = op;
      }
    }
  }
  if (own) {
#pragma unroll
    for (int v = 0; v < 32; ++v) {
      if (v < V) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (acc[v][e] != 0.f) atomicAdd(&dW[static_cast<size_t>(v) * C + ch + e], acc[v][e]);
      }
    }
  }
  if (dbias && t < V && db != 0.f) atomicAdd(&dbias[t], db);
}

// ------------------------------------------------------------------ optimizer
// sum of squares of an fp32 buffer, accumulated into out[0]
__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n4 << 2; i < n; ++i) s += x[i] * x[i];
  s = warp_sum(s);
  __shared__ float ws[8];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += ws[i];
    atomicAdd(out, t);
  }
}

// AdamW on fp32 master weights with decoupled weight decay; the gradient is scaled by
// grad_scale * min(1, max_norm / (sqrt(*sumsq * grad_scale^2) + 1e-6)) (clip_grad_norm_
// semantics), read on the device so no host round trip is needed. Writes the bf16 compute copy
// and, when zero_grad != 0, clears the gradient for the next accumulation window.
// hyper: [lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale, max_norm]
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
             float* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16,
             const float* __restrict__ hyper, const float* __restrict__ sumsq, long long n,
             int zero_grad) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], gs = hyper[7], max_norm = hyper[8];
  float scale = gs;
  if (sumsq != nullptr && max_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * gs;
    scale = gs * fminf(1.f, max_norm / (norm + 1e-6f));
  }
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gr = g[i] * scale;
    float pv = p[i];
    pv *= (1.f - lr * wd);
    const float mv = b1 * m[i] + (1.f - b1) * gr;
    const float vv = b2 * v[i] + (1.f - b2) * gr * gr;
    const float denom = sqrtf(vv) * inv_sqrt_bc2 + eps;
    pv -= step_size * mv / denom;
    p[i] = pv;
    m[i] = mv;
    v[i] = vv;
    if (p_bf16) p_bf16[i] = __float2bfloat16(pv);
    if (zero_grad) g[i] = 0.f;
  }
}

// ---- Muon (matrices of one shape, addressed through a table of flat offsets) -----------------
// gradient scale shared by the optimizer kernels: grad_scale and clip_grad_norm_ by the global norm
__device__ __forceinline__ float clip_scale(const float* sumsq, float gs, float max_norm) {
  if (sumsq == nullptr || max_norm <= 0.f) return gs;
  return gs * fminf(1.f, max_norm / (sqrtf(*sumsq) * gs + 1e-6f));
}

// Momentum of matrix blockIdx.y (numel elements at flat offset off[y]) and the bf16 update that
// enters the Newton-Schulz iterations:  m <- mu m + g,  u = nesterov ? g + mu m : m,
// upd[y] = bf16(u),  usq[y] += sum of the rounded u^2 (its Frobenius norm normalises the iteration).
__global__ void __launch_bounds__(256)
muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ m,
                     const long long* __restrict__ off, long long numel,
                     __nv_bfloat16* __restrict__ upd, float* __restrict__ usq,
                     const float* __restrict__ sumsq, float gs, float max_norm, float mu, int nesterov) {
  const float scale = clip_scale(sumsq, gs, max_norm);
  const long long base = off[blockIdx.y];
  const float4* g4 = reinterpret_cast<const float4*>(g + base);
  float4* m4 = reinterpret_cast<float4*>(m + base);
  uint2* u4 = reinterpret_cast<uint2*>(upd + static_cast<long long>(blockIdx.y) * numel);
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < (numel >> 2);
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 gv = g4[i];
    float4 mv = m4[i];
    gv.x *= scale; gv.y *= scale; gv.z *= scale; gv.w *= scale;
    mv.x = mu * mv.x + gv.x; mv.y = mu * mv.y + gv.y; mv.z = mu * mv.z + gv.z; mv.w = mu * mv.w + gv.w;
    m4[i] = mv;
    float4 u = mv;
    if (nesterov) { u.x = gv.x + mu * mv.x; u.y = gv.y + mu * mv.y; u.z = gv.z + mu * mv.z; u.w = gv.w + mu * mv.w; }
    uint2 pk;
    pk.x = pack_bf16x2(u.x, u.y);
    pk.y = pack_bf16x2(u.z, u.w);
    u4[i] = pk;
    const float2 a = unpack_bf16x2(pk.x), b = unpack_bf16x2(pk.y);
    acc += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
  }
  acc = warp_sum(acc);
  __shared__ float ws[8];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += ws[i];
    atomicAdd(&usq[blockIdx.y], t);
  }
}

// Applies the orthogonalised update O[y] (bf16) to matrix y: decoupled weight decay (cautious:
// only where the update and the weight agree in sign), p <- p - lr O, and the bf16 compute copy.
__global__ void __launch_bounds__(256)
muon_apply_kernel(float* __restrict__ p, __nv_bfloat16* __restrict__ p16,
                  const long long* __restrict__ off, long long numel,
                  const __nv_bfloat16* __restrict__ O, float lr, float wd, int cautious) {
  const long long base = off[blockIdx.y];
  float4* p4 = reinterpret_cast<float4*>(p + base);
  uint2* q4 = p16 ? reinterpret_cast<uint2*>(p16 + base) : nullptr;
  const uint2* o4 = reinterpret_cast<const uint2*>(O + static_cast<long long>(blockIdx.y) * numel);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < (numel >> 2);
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pv = p4[i];
    const uint2 ov = o4[i];
    const float2 oa = unpack_bf16x2(ov.x), ob = unpack_bf16x2(ov.y);
    const float o[4] = {oa.x, oa.y, ob.x, ob.y};
    float* pe = reinterpret_cast<float*>(&pv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float x = pe[e];
      if (wd > 0.f) {
        if (cautious) x -= (o[e] * x > 0.f) ? lr * wd * x : 0.f;
        else x *= (1.f - lr * wd);
      }
      pe[e] = x - lr * o[e];
    }
    p4[i] = pv;
    if (q4) {
      uint2 pk;
      pk.x = pack_bf16x2(pv.x, pv.y);
      pk.y = pack_bf16x2(pv.z, pv.w);
      q4[i] = pk;
    }
  }
}

// AdamW over a table of parameter tensors of one flat buffer (tensor y: numel[y] elements at
// offset off[y], weight decay only where decay[y] != 0); same update as adamw_kernel.
__global__ void __launch_bounds__(256)
adamw_slots_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                   const float* __restrict__ g, __nv_bfloat16* __restrict__ p16,
                   const long long* __restrict__ off, const long long* __restrict__ numel,
                   const int* __restrict__ decay, const float* __restrict__ sumsq, float gs, float max_norm,
                   float lr, float b1, float b2, float eps, float wd, float bc1, float bc2) {
  const float scale = clip_scale(sumsq, gs, max_norm);
  const long long base = off[blockIdx.y], n = numel[blockIdx.y];
  const float decay_mul = decay[blockIdx.y] ? (1.f - lr * wd) : 1.f;
  const float step_size = lr / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long j = base + i;
    const float gr = g[j] * scale;
    float pv = p[j] * decay_mul;
    const float mv = b1 * m[j] + (1.f - b1) * gr;
    const float vv = b2 * v[j] + (1.f - b2) * gr * gr;
    pv -= step_size * mv / (sqrtf(vv) * inv_sqrt_bc2 + eps);
    p[j] = pv;
    m[j] = mv;
    v[j] = vv;
    if (p16) p16[j] = __float2bfloat16(pv);
  }
}

__global__ void __launch_bounds__(256)
cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                        long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

// masked MSE for embedding distillation: loss = sum_{valid tokens} sum_c (s-t)^2 / max(1, n_valid)
// (src/nanoplm/distillation/trainer.py:30-40). ds = 2 (s-t) * inv_count for valid rows, else 0.
__global__ void __launch_bounds__(256)
masked_mse_kernel(const __nv_bfloat16* __restrict__ s, const __nv_bfloat16* __restrict__ t,
                  const int* __restrict__ valid, const float* __restrict__ inv_count,
                  __nv_bfloat16* __restrict__ ds, float* __restrict__ loss_sum, int T, int C) {
  const int vec = C >> 3;
  const long long total = static_cast<long long>(T) * vec;
  const float invc = *inv_count;
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec);
    const int c = static_cast<int>(i % vec) * 8;
    float o[8];
    if (valid == nullptr || valid[r]) {
      float a[8], b[8];
      load8(s + static_cast<size_t>(r) * C + c, a);
      load8(t + static_cast<size_t>(r) * C + c, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = a[e] - b[e];
        acc += d * d;
        o[e] = 2.f * d * invc;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = 0.f;
    }
    if (ds) store8(ds + static_cast<size_t>(r) * C + c, o);
  }
  acc = warp_sum(acc);
  __shared__ float ws[8];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tsum = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) tsum += ws[i];
    atomicAdd(loss_sum, tsum * invc);
  }
}

static int grid_for(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace nplm

using namespace nplm;

#define NPLM_CHUNK_DISPATCH(C_, CALL)                      \
  do {                                                     \
    const int chunks_ = ((C_) + 255) / 256;                \
    if (chunks_ <= 1) { CALL(1); }                         \
    else if (chunks_ <= 2) { CALL(2); }                    \
    else if (chunks_ <= 3) { CALL(3); }                    \
    else if (chunks_ <= 4) { CALL(4); }                    \
    else if (chunks_ <= 8) { CALL(8); }                    \
    else if (chunks_ <= 16) { CALL(16); }                  \
    else return -3;                                        \
  } while (0)

extern "C" int nplm_norm_fwd(const void* x, const int* ids, const void* w, void* y, float* mean,
                             float* rstd, int T, int C, float eps, int rms, cudaStream_t st) {
  if (T <= 0) return 0;
  if (C % 8) return -3;
  const int blocks = (T + 7) / 8 < 148 * 8 ? (T + 7) / 8 : 148 * 8;
#define CALL(N_)                                                                               \
  norm_fwd_kernel<N_><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), ids,  \
                                              reinterpret_cast<const __nv_bfloat16*>(w),       \
                                              reinterpret_cast<__nv_bfloat16*>(y), mean, rstd, \
                                              T, C, eps, rms)
  NPLM_CHUNK_DISPATCH(C, CALL);
#undef CALL
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_norm_bwd(const void* dy, const void* x, const int* ids, const void* w,
                             const float* mean, const float* rstd, const void* dres, void* dx,
                             float* dw, float* dtable, int T, int C, int V, int rms, cudaStream_t st) {
  if (T <= 0) return 0;
  if (C % 8) return -3;
  if (C >= 256 && C <= 2048 && ids != nullptr && dtable != nullptr && V > 0) {
    // embedding gradient: row-group kernel, per-vocabulary-entry sums in shared memory
    // (C/8 threads, rounded up to whole warps)
    // the table sums fill the SM's shared memory (one block per SM), so the block itself keeps
    // ROWS * SUB rows in flight: 4 groups of C/8 threads up to C = 1024, 2 beyond (512 threads)
    constexpr int ROWS = 4;
    const int sub = C <= 1024 ? 4 : 2;
    const int threads = ((C / 8) + 31) / 32 * 32 * sub;
    const size_t smem = static_cast<size_t>(V) * C * sizeof(float);
    if (smem <= 200 * 1024) {
      const int groups = (T + ROWS * sub - 1) / (ROWS * sub);
      int blocks = 148;
      if (blocks > groups) blocks = groups;
#define CALL_ROWS(SUB_)                                                                                   \
  do {                                                                                                    \
    if (smem > 48 * 1024)                                                                                 \
      cudaFuncSetAttribute(norm_bwd_rows_kernel<ROWS, SUB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           static_cast<int>(smem));                                                       \
    norm_bwd_rows_kernel<ROWS, SUB_><<<blocks, threads, smem, st>>>(                                      \
        reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x), ids,       \
        reinterpret_cast<const __nv_bfloat16*>(w), mean, rstd, reinterpret_cast<const __nv_bfloat16*>(dres), \
        reinterpret_cast<__nv_bfloat16*>(dx), dw, dtable, T, C, V, rms);                                  \
  } while (0)
      if (sub == 4) CALL_ROWS(4);
      else CALL_ROWS(2);
#undef CALL_ROWS
      return static_cast<int>(cudaGetLastError());
    }
  }
  int blocks = (T + 7) / 8;
  if (blocks > 148 * 2) blocks = 148 * 2;   // more blocks only add contention on the dw atomics
#define CALL(N_)                                                                              \
  norm_bwd_kernel<N_><<<blocks, 256, C * sizeof(float), st>>>(                                \
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),  \
      ids, reinterpret_cast<const __nv_bfloat16*>(w), mean, rstd,                             \
      reinterpret_cast<const __nv_bfloat16*>(dres), reinterpret_cast<__nv_bfloat16*>(dx), dw, \
      dtable, T, C, rms)
  NPLM_CHUNK_DISPATCH(C, CALL);
#undef CALL
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_rope(void* qkv, const int* pos, const float* cos_t, const float* sin_t, int T,
                         int H, int D, int backward, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 16) return -3;
  const long long total = static_cast<long long>(T) * 2 * H * (D / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(qkv), pos,
                                                    cos_t, sin_t, T, H, D, backward ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_swiglu_fwd(const void* pre, void* out, long long T, int I, cudaStream_t st) {
  if (T <= 0) return 0;
  if (I % 8) return -3;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(pre), reinterpret_cast<__nv_bfloat16*>(out), T, I);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_swiglu_bwd(const void* pre, const void* dout, void* dpre, long long T, int I,
                               cudaStream_t st) {
  if (T <= 0) return 0;
  if (I % 8) return -3;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(pre), reinterpret_cast<const __nv_bfloat16*>(dout),
      reinterpret_cast<__nv_bfloat16*>(dpre), T, I);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_act_fwd(const void* pre, void* out, long long n, int act, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -3;
  act_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(pre), reinterpret_cast<__nv_bfloat16*>(out), n / 8, act);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_act_bwd(const void* pre, const void* dout, void* dpre, long long n, int act,
                            cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -3;
  act_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(pre), reinterpret_cast<const __nv_bfloat16*>(dout),
      reinterpret_cast<__nv_bfloat16*>(dpre), n / 8, act);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_gather_rows(const void* src, const int* idx, void* dst, int n, int C,
                                cudaStream_t st) {
  if (n <= 0) return 0;
  if (C % 8) return -3;
  gather_rows_kernel<<<grid_for(static_cast<long long>(n) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), idx, reinterpret_cast<__nv_bfloat16*>(dst), n, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_scatter_rows(const void* src, const int* idx, void* dst, int n, int C,
                                 cudaStream_t st) {
  if (n <= 0) return 0;
  if (C % 8) return -3;
  scatter_rows_kernel<<<grid_for(static_cast<long long>(n) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), idx, reinterpret_cast<__nv_bfloat16*>(dst), n, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_ce_fwd(const void* h, const void* W, const void* bias, const int* labels,
                           const float* inv_count, float* dlogits, float* logits, float* loss_sum,
                           int n, int C, int V, cudaStream_t st) {
  if (n <= 0) return 0;
  if (V > 32 || V < 1 || (C % 8)) return -3;
  const size_t smem = static_cast<size_t>(V) * C * 2;
  if (smem > 200 * 1024) return -4;
  int blocks = (n + CE_WARPS - 1) / CE_WARPS;
  if (blocks > 148 * 2) blocks = 148 * 2;
#define CALL(N_)                                                                                   \
  do {                                                                                             \
    cudaFuncSetAttribute(ce_fwd_kernel<N_>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                         static_cast<int>(smem));                                                  \
    ce_fwd_kernel<N_><<<blocks, CE_WARPS * 32, smem, st>>>(                                        \
        reinterpret_cast<const __nv_bfloat16*>(h), reinterpret_cast<const __nv_bfloat16*>(W),      \
        reinterpret_cast<const __nv_bfloat16*>(bias), labels, inv_count, dlogits, logits, loss_sum, \
        n, C, V);                                                                                  \
  } while (0)
  NPLM_CHUNK_DISPATCH(C, CALL);
#undef CALL
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_ce_bwd(const void* h, const void* W, const float* dlogits, const float* gscale,
                           void* dh, float* dW, float* dbias, int n, int C, int V,
                           cudaStream_t st) {
  if (n <= 0) return 0;
  if (V > 32 || V < 1 || (C % 8)) return -3;
  if (C <= 1024) {
    const size_t tsm = (static_cast<size_t>(V) * C + static_cast<size_t>(CE_TILE_ROWS) * C) * 2 +
                       CE_TILE_ROWS * 32 * 4;
    static bool configured_on[nplm::MAX_DEVICES];
    const int dev_slot = nplm::current_device_slot();
    if (dev_slot < 0) return -4;
    bool& configured = configured_on[dev_slot];
    if (!configured) {
      cudaFuncSetAttribute(ce_bwd_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      configured = true;
    }
    int tb = (n + CE_TILE_ROWS - 1) / CE_TILE_ROWS;
    if (tb > 148) tb = 148;
    ce_bwd_tiled_kernel<<<tb, 256, tsm, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(h), reinterpret_cast<const __nv_bfloat16*>(W), dlogits, gscale,
        reinterpret_cast<__nv_bfloat16*>(dh), dW, dbias, n, C, V);
    return static_cast<int>(cudaGetLastError());
  }
  const size_t smem = (static_cast<size_t>(V) * C + 32) * 4;
  if (smem > 220 * 1024) return -4;
  int blocks = (n + CE_WARPS - 1) / CE_WARPS;
  if (blocks > 148) blocks = 148;
#define CALL(N_)                                                                              \
  do {                                                                                        \
    cudaFuncSetAttribute(ce_bwd_kernel<N_>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                         static_cast<int>(smem));                                             \
    ce_bwd_kernel<N_><<<blocks, CE_WARPS * 32, smem, st>>>(                                   \
        reinterpret_cast<const __nv_bfloat16*>(h), reinterpret_cast<const __nv_bfloat16*>(W), \
        dlogits, gscale, reinterpret_cast<__nv_bfloat16*>(dh), dW, dbias, n, C, V);           \
  } while (0)
  NPLM_CHUNK_DISPATCH(C, CALL);
#undef CALL
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_sumsq(const float* x, long long n, float* out, cudaStream_t st) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(x) & 15) return -3;
  sumsq_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, st>>>(x, n, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_adamw(float* p, float* m, float* v, float* g, void* p_bf16, const float* hyper,
                          const float* sumsq, long long n, int zero_grad, cudaStream_t st) {
  if (n <= 0) return 0;
  adamw_kernel<<<grid_for(n, 256), 256, 0, st>>>(p, m, v, g, reinterpret_cast<__nv_bfloat16*>(p_bf16),
                                                 hyper, sumsq, n, zero_grad);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_muon_momentum(const float* g, float* m, const long long* off, int n_mat, long long numel,
                                  void* upd, float* usq, const float* sumsq, float gs, float max_norm,
                                  float mu, int nesterov, cudaStream_t st) {
  if (n_mat <= 0 || numel <= 0) return 0;
  if (numel & 3) return -3;
  int bx = grid_for(numel / 4, 256);
  if (bx > 592) bx = 592;
  muon_momentum_kernel<<<dim3(bx, n_mat), 256, 0, st>>>(g, m, off, numel, reinterpret_cast<__nv_bfloat16*>(upd),
                                                        usq, sumsq, gs, max_norm, mu, nesterov);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_muon_apply(float* p, void* p16, const long long* off, int n_mat, long long numel,
                               const void* O, float lr, float wd, int cautious, cudaStream_t st) {
  if (n_mat <= 0 || numel <= 0) return 0;
  if (numel & 3) return -3;
  int bx = grid_for(numel / 4, 256);
  if (bx > 592) bx = 592;
  muon_apply_kernel<<<dim3(bx, n_mat), 256, 0, st>>>(p, reinterpret_cast<__nv_bfloat16*>(p16), off, numel,
                                                     reinterpret_cast<const __nv_bfloat16*>(O), lr, wd, cautious);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_adamw_slots(float* p, float* m, float* v, const float* g, void* p16, const long long* off,
                                const long long* numel, const int* decay, int n_slots, long long max_numel,
                                const float* sumsq, float gs, float max_norm, float lr, float b1, float b2,
                                float eps, float wd, float bc1, float bc2, cudaStream_t st) {
  if (n_slots <= 0 || max_numel <= 0) return 0;
  int bx = grid_for(max_numel, 256);
  if (bx > 64) bx = 64;
  adamw_slots_kernel<<<dim3(bx, n_slots), 256, 0, st>>>(p, m, v, g, reinterpret_cast<__nv_bfloat16*>(p16), off,
                                                        numel, decay, sumsq, gs, max_norm, lr, b1, b2, eps, wd,
                                                        bc1, bc2);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, st>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int nplm_masked_mse(const void* s, const void* t, const int* valid,
                               const float* inv_count, void* ds, float* loss_sum, int T, int C,
                               cudaStream_t st) {
  if (T <= 0) return 0;
  if (C % 8) return -3;
  masked_mse_kernel<<<grid_for(static_cast<long long>(T) * (C / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(s), reinterpret_cast<const __nv_bfloat16*>(t), valid,
      inv_count, reinterpret_cast<__nv_bfloat16*>(ds), loss_sum, T, C);
  return static_cast<int>(cudaGetLastError());
}
