// Row kernels of decoders whose mixer reads the normalised residual through a short causal convolution over time:
//
//   pg_rmsnorm_conv     h = x / sqrt(mean(x^2) + eps) * g (g: one weight per channel, or ONE number for the whole row);
//                       out_h[t] = h[t] (what a feed-forward beside the mixer reads), out_conv[t] = h[t] + sum_j cw[j, :] h[t - taps + 1 + j]
//                       per channel, zeros before the sequence's start.  The last taps - 1 rows h of a sequence live in an fp32
//                       state slot, so a portion or a decoded token continues where the sequence stopped.
//   pg_polynorm         out = a N(z) + b N(z^2) + c N(z^3) + e with N(v) = v / sqrt(mean(v^2) + eps) over the row (powers element-wise)
//   pg_sigmoid_gate_mul y[t, c] *= sigmoid(gate[t, c])
//
// Statistics, h, the convolution and the state are fp32; only the written activations have the activation type.
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

#define PG_ST(s) reinterpret_cast<cudaStream_t>(s)
#define PG_RET()                                                    \
  do {                                                              \
    pg_count_launch(1);                                             \
    return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA; \
  } while (0)

namespace {

constexpr int MAX_K = 7;  // taps - 1 at most

__device__ __forceinline__ void st_a(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_a(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float ld_a(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld_a(const bf16* p, long long i) { return __bfloat162float(p[i]); }

// sum over the CTA's 256 threads; every thread gets the result.  `red` = 8 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();  // the previous use of `red` is over
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) s += red[w];
  return s;
}

__device__ __forceinline__ float row_rstd(const float* __restrict__ xr, int D, float eps, float* red) {
  float s = 0.f;
  if ((D & 3) == 0 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    for (int i = threadIdx.x; i < D / 4; i += 256) { const float4 v = x4[i]; s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s)))); }
  } else {
    for (int d = threadIdx.x; d < D; d += 256) { const float v = xr[d]; s = fmaf(v, v, s); }
  }
  return 1.0f / sqrtf(block_sum(s, red) / (float)D + eps);
}

// One CTA per row.  Rows K = taps - 1 or more tokens into their entry find every earlier row they need in this step and recompute
// its 1 / rms from x (just written by the layer before: L2).  The first K rows of an entry also need the state slot: ALL of them
// are produced by the CTA of the entry's first row, which alone reads the slot and alone writes it (the last K rows h of the
// sequence, recomputed here from x), so no other CTA of the launch touches the slot; the CTAs of rows 1 .. K-1 have nothing to do.
template <typename TO>
__global__ void __launch_bounds__(256) rmsnorm_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, int w_stride,
                                                           const float* __restrict__ cw, int taps, float* __restrict__ state,
                                                           TO* __restrict__ out_h, TO* __restrict__ out_conv, const int* __restrict__ row_entry,
                                                           const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                           const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int D, float eps,
                                                           int by_entry) {
  __shared__ float red[8];
  __shared__ float inv[2 * MAX_K + 1];
  const int K = cw != nullptr ? taps - 1 : 0;
  // by_entry: one CTA per entry, for its first rows and its slot only (the other rows belong to the row-chunk kernel)
  const long long t = by_entry ? entry_row0[blockIdx.x] : blockIdx.x;
  int i = 0, ne = 1, e = 0;
  if (K > 0) {
    e = by_entry ? (int)blockIdx.x : row_entry[t];
    i = (int)(t - entry_row0[e]);
    ne = entry_n[e];
    if (i > 0 && i < K) return;
  }
  if (i >= K) {
    for (int j = 0; j <= K; ++j) {
      const float r = row_rstd(x + (t - K + j) * D, D, eps, red);
      if (threadIdx.x == 0) inv[j] = r;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += 256) {
      const float g = w[(long long)d * w_stride];
      const float hv = x[t * D + d] * inv[K] * g;
      if (out_h != nullptr) st_a(out_h, t * D + d, hv);
      if (out_conv != nullptr) {
        float acc = hv;
        if (cw != nullptr) {
          acc = fmaf(cw[(long long)K * D + d], hv, acc);
          for (int j = 0; j < K; ++j) acc = fmaf(cw[(long long)j * D + d], x[(t - K + j) * D + d] * inv[j] * g, acc);
        }
        st_a(out_conv, t * D + d, acc);
      }
    }
    return;
  }
  // i == 0 < K: the entry's first m rows and the slot
  const int m = min(ne, K);
  for (int r = 0; r < m; ++r) {
    const float a = row_rstd(x + (t + r) * D, D, eps, red);
    const float b = ne - m + r < m ? 0.f : row_rstd(x + (t + ne - m + r) * D, D, eps, red);  // the entry's last m rows (the same rows when ne <= K)
    if (threadIdx.x == 0) { inv[r] = a; inv[MAX_K + r] = b; }
  }
  __syncthreads();
  const bool fresh = entry_ctx[e] == 0;  // nothing before this entry: zeros, whatever an earlier sequence left in the slot
  float* slot = state + (long long)entry_slot[e] * K * D;
  for (int d = threadIdx.x; d < D; d += 256) {
    const float g = w[(long long)d * w_stride];
    float old[MAX_K], hf[MAX_K];
#pragma unroll
    for (int k = 0; k < MAX_K; ++k) {
      old[k] = (k < K && !fresh) ? slot[(long long)k * D + d] : 0.f;  // h of position ctx - K + k
      hf[k] = k < m ? x[(t + k) * D + d] * inv[k] * g : 0.f;
    }
#pragma unroll
    for (int r = 0; r < MAX_K; ++r) {
      if (r < m) {
        if (out_h != nullptr) st_a(out_h, (t + r) * D + d, hf[r]);
        if (out_conv != nullptr) {
          float acc = hf[r];
#pragma unroll
          for (int j = 0; j <= MAX_K; ++j) {
            if (j <= K) {
              const int src = r - K + j;  // row of the entry, negative: before it
              float v = 0.f;
#pragma unroll
              for (int q = 0; q < MAX_K; ++q) {
                if (src == q) v = hf[q];
                if (K + src == q && src < 0) v = old[q];
              }
              acc = fmaf(cw[(long long)j * D + d], v, acc);
            }
          }
          st_a(out_conv, (t + r) * D + d, acc);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < MAX_K; ++k) {
      if (k < K) {
        const int idx = ne - K + k;  // row of the entry whose h becomes slot row k; negative: it stays an older one
        float v = 0.f;
        if (idx >= 0) {
          const int r = idx - (ne - m);  // index among the last m rows
          v = idx < m ? 0.f : x[(t + idx) * D + d] * inv[MAX_K + r] * g;
#pragma unroll
          for (int q = 0; q < MAX_K; ++q)
            if (idx == q && idx < m) v = hf[q];
        } else {
#pragma unroll
          for (int q = 0; q < MAX_K; ++q)
            if (K + idx == q) v = old[q];
        }
        slot[(long long)k * D + d] = v;
      }
    }
  }
}

// The same scheme with four channels per thread and 16-byte accesses (D a multiple of 4, 16-byte aligned rows), and with every
// register array indexed at compile time: the rows before an entry are held newest first (before[m] = h of the entry's row -1 - m),
// so that row r's m-th earlier row is hf[r - 1 - m] or before[m - r] whatever taps is; taps beyond the real ones carry zero weights.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 mul4(float4 a, float s, float4 g) { return make_float4(a.x * s * g.x, a.y * s * g.y, a.z * s * g.z, a.w * s * g.w); }
__device__ __forceinline__ void fma4(float4& acc, float4 a, float4 b) {
  acc.x = fmaf(a.x, b.x, acc.x); acc.y = fmaf(a.y, b.y, acc.y); acc.z = fmaf(a.z, b.z, acc.z); acc.w = fmaf(a.w, b.w, acc.w);
}
__device__ __forceinline__ void st_o4(float* p, long long i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void st_o4(bf16* p, long long i, float4 v) {
  uint2 u;
  u.x = pg::pack_bf16(v.x, v.y);
  u.y = pg::pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(p + i) = u;
}

template <typename TO>
__global__ void __launch_bounds__(256) rmsnorm_conv_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, int w_stride,
                                                               const float* __restrict__ cw, int taps, float* __restrict__ state,
                                                               TO* __restrict__ out_h, TO* __restrict__ out_conv, const int* __restrict__ row_entry,
                                                               const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                               const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int D, float eps,
                                                               int by_entry) {
  __shared__ float red[8];
  __shared__ float inv[2 * MAX_K + 1];
  const int K = cw != nullptr ? taps - 1 : 0;
  const long long t = by_entry ? entry_row0[blockIdx.x] : blockIdx.x;
  int i = 0, ne = 1, e = 0;
  if (K > 0) {
    e = by_entry ? (int)blockIdx.x : row_entry[t];
    i = (int)(t - entry_row0[e]);
    ne = entry_n[e];
    if (i > 0 && i < K) return;
  }
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i >= K) {
    if (by_entry) return;
    for (int j = 0; j <= K; ++j) {
      const float r = row_rstd(x + (t - K + j) * D, D, eps, red);
      if (threadIdx.x == 0) inv[j] = r;
    }
    __syncthreads();
    for (int c = 4 * threadIdx.x; c < D; c += 1024) {
      float4 g;
      if (w_stride) g = ld4(w + c);
      else g.x = g.y = g.z = g.w = w[0];
      float4 acc = zero, hv = zero;
#pragma unroll
      for (int j = 0; j <= MAX_K; ++j) {
        if (j <= K) {
          const float4 hj = mul4(ld4(x + (t - K + j) * D + c), inv[j], g);
          if (cw != nullptr) fma4(acc, ld4(cw + (long long)j * D + c), hj);
          if (j == K) hv = hj;
        }
      }
      if (out_h != nullptr) st_o4(out_h, t * D + c, hv);
      if (out_conv != nullptr) st_o4(out_conv, t * D + c, make_float4(hv.x + acc.x, hv.y + acc.y, hv.z + acc.z, hv.w + acc.w));
    }
    return;
  }
  // i == 0 < K: the entry's first m rows and the slot
  const int m = min(ne, K);
  for (int r = 0; r < m; ++r) {
    const float a = row_rstd(x + (t + r) * D, D, eps, red);
    if (threadIdx.x == 0) inv[r] = a;
  }
  for (int mm = 0; mm < m; ++mm) {  // the entry's last rows, newest first
    const int row = ne - 1 - mm;
    const float b = row < m ? 0.f : row_rstd(x + (t + row) * D, D, eps, red);
    if (threadIdx.x == 0 && row >= m) inv[MAX_K + mm] = b;
  }
  __syncthreads();
  if (threadIdx.x < m && ne - 1 - (int)threadIdx.x < m) inv[MAX_K + threadIdx.x] = inv[ne - 1 - threadIdx.x];
  __syncthreads();
  const bool fresh = entry_ctx[e] == 0;  // nothing before this entry: zeros, whatever an earlier sequence left in the slot
  float* slot = state + (long long)entry_slot[e] * K * D;
  for (int c = 4 * threadIdx.x; c < D; c += 1024) {
    float4 g;
    if (w_stride) g = ld4(w + c);
    else g.x = g.y = g.z = g.w = w[0];
    float4 before[MAX_K], cwr[MAX_K], hf[MAX_K];
    const float4 cwcur = ld4(cw + (long long)K * D + c);
#pragma unroll
    for (int mm = 0; mm < MAX_K; ++mm) {
      before[mm] = (mm < K && !fresh) ? ld4(slot + (long long)(K - 1 - mm) * D + c) : zero;
      cwr[mm] = mm < K ? ld4(cw + (long long)(K - 1 - mm) * D + c) : zero;
      hf[mm] = mm < m ? mul4(ld4(x + (t + mm) * D + c), inv[mm], g) : zero;
    }
#pragma unroll
    for (int r = 0; r < MAX_K; ++r) {
      if (r < m) {
        float4 acc = zero;
        fma4(acc, cwcur, hf[r]);
#pragma unroll
        for (int mm = 0; mm < MAX_K; ++mm) fma4(acc, cwr[mm], mm < r ? hf[r - 1 - mm] : before[mm - r]);
        if (out_h != nullptr) st_o4(out_h, (t + r) * D + c, hf[r]);
        if (out_conv != nullptr) st_o4(out_conv, (t + r) * D + c, make_float4(hf[r].x + acc.x, hf[r].y + acc.y, hf[r].z + acc.z, hf[r].w + acc.w));
      }
    }
    // the slot afterwards, oldest first: rows of before the entry move up by ne, the entry's last rows follow
#pragma unroll
    for (int mm = 0; mm < MAX_K; ++mm)
      if (mm < K && mm + ne < K) *reinterpret_cast<float4*>(slot + (long long)(K - 1 - mm - ne) * D + c) = before[mm];
#pragma unroll
    for (int mm = 0; mm < MAX_K; ++mm)
      if (mm < m) *reinterpret_cast<float4*>(slot + (long long)(K - 1 - mm) * D + c) = mul4(ld4(x + (t + ne - 1 - mm) * D + c), inv[MAX_K + mm], g);
  }
}

// Prompt portions: one CTA per chunk of RC consecutive rows.  Pass 1: a warp per row (the chunk and the taps - 1 rows before it) leaves
// 1 / rms in shared memory.  Pass 2: a thread owns four channels and walks down the chunk's rows; the earlier rows it needs are the
// ones it read in its last iterations (L1).  Rows less than taps - 1 tokens
// into their entry are left to the per-entry launch of the kernel above (they need the state slot).
__device__ __forceinline__ void st_a4(float* p, long long i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void st_a4(bf16* p, long long i, float4 v) {
  uint2 u;
  u.x = pg::pack_bf16(v.x, v.y);
  u.y = pg::pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(p + i) = u;
}

template <typename TO>
__global__ void __launch_bounds__(256) rmsnorm_conv_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, int w_stride,
                                                                const float* __restrict__ cw, int taps, TO* __restrict__ out_h,
                                                                TO* __restrict__ out_conv, const int* __restrict__ row_entry,
                                                                const int* __restrict__ entry_row0, int rows, int RC, int D, float eps) {
  __shared__ float inv[32 + MAX_K];
  __shared__ int into[32];  // rows into their entry
  const int K = taps - 1;
  const int r0 = blockIdx.x * RC, nr = min(RC, rows - r0);
  const int first = max(r0 - K, 0), nh = r0 - first, total = nh + nr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = threadIdx.x; r < nr; r += 256) into[r] = r0 + r - entry_row0[row_entry[r0 + r]];
  for (int rr = warp; rr < total; rr += 8) {
    const float4* x4 = reinterpret_cast<const float4*>(x + (long long)(first + rr) * D);
    float s = 0.f;
    for (int i = lane; i < D / 4; i += 32) { const float4 v = x4[i]; s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s)))); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) inv[rr] = 1.0f / sqrtf(s / (float)D + eps);
  }
  __syncthreads();
  for (int c4 = threadIdx.x; c4 < D / 4; c4 += 256) {
    const int c = 4 * c4;
    float4 g;
    if (w_stride) g = *reinterpret_cast<const float4*>(w + c);
    else g.x = g.y = g.z = g.w = w[0];
    for (int r = 0; r < nr; ++r) {
      if (into[r] < K) continue;  // needs the state slot
      const long long t = r0 + r;
      float4 hv, acc;
      for (int j = 0; j <= K; ++j) {
        const float4 xv = *reinterpret_cast<const float4*>(x + (t - K + j) * D + c);
        const float iv = inv[nh + r - K + j];
        const float4 cj = *reinterpret_cast<const float4*>(cw + (long long)j * D + c);
        const float4 hj = make_float4(xv.x * iv * g.x, xv.y * iv * g.y, xv.z * iv * g.z, xv.w * iv * g.w);
        if (j == 0) acc = make_float4(0.f, 0.f, 0.f, 0.f);
        acc.x = fmaf(cj.x, hj.x, acc.x); acc.y = fmaf(cj.y, hj.y, acc.y); acc.z = fmaf(cj.z, hj.z, acc.z); acc.w = fmaf(cj.w, hj.w, acc.w);
        if (j == K) hv = hj;
      }
      if (out_h != nullptr) st_a4(out_h, t * D + c, hv);
      st_a4(out_conv, t * D + c, make_float4(hv.x + acc.x, hv.y + acc.y, hv.z + acc.z, hv.w + acc.w));
    }
  }
}

// One CTA per row: the three mean powers in one pass, the polynomial in a second one over the same (cached) row.  out may be z.
template <typename TA>
__global__ void __launch_bounds__(256) polynorm_kernel(const TA* z, long long ldz, const float* __restrict__ coef, TA* out,
                                                       long long ldo, int F, float eps) {
  __shared__ float red[8];
  const long long t = blockIdx.x;
  const TA* zr = z + t * ldz;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int f = threadIdx.x; f < F; f += 256) {
    const float v = ld_a(zr, f), v2 = v * v, v4 = v2 * v2;
    s2 += v2;
    s4 += v4;
    s6 = fmaf(v4, v2, s6);
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float a = coef[0] / sqrtf(s2 / (float)F + eps), b = coef[1] / sqrtf(s4 / (float)F + eps), c = coef[2] / sqrtf(s6 / (float)F + eps);
  const float e = coef[3];
  for (int f = threadIdx.x; f < F; f += 256) {
    const float v = ld_a(zr, f);
    st_a(out, t * ldo + f, fmaf(v, fmaf(v, fmaf(v, c, b), a), e));
  }
}

// The same with 16-byte accesses, eight elements per thread and step (F and the pitches multiples of 8, 16-byte aligned rows).
__device__ __forceinline__ void ld8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8(const bf16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t q[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(q[i] << 16); v[2 * i + 1] = __uint_as_float(q[i] & 0xffff0000u); }
}
__device__ __forceinline__ void st8(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8(bf16* p, const float* v) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pg::pack_bf16(v[0], v[1]), pg::pack_bf16(v[2], v[3]), pg::pack_bf16(v[4], v[5]), pg::pack_bf16(v[6], v[7]));
}

template <typename TA>
__global__ void __launch_bounds__(256) polynorm_vec_kernel(const TA* z, long long ldz, const float* __restrict__ coef, TA* out, long long ldo, int F,
                                                           float eps) {
  __shared__ float red[8];
  const long long t = blockIdx.x;
  const TA* zr = z + t * ldz;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int f = 8 * threadIdx.x; f < F; f += 8 * 256) {
    float v[8];
    ld8(zr + f, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v2 = v[i] * v[i], v4 = v2 * v2;
      s2 += v2;
      s4 += v4;
      s6 = fmaf(v4, v2, s6);
    }
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float a = coef[0] / sqrtf(s2 / (float)F + eps), b = coef[1] / sqrtf(s4 / (float)F + eps), c = coef[2] / sqrtf(s6 / (float)F + eps);
  const float e = coef[3];
  for (int f = 8 * threadIdx.x; f < F; f += 8 * 256) {
    float v[8];
    ld8(zr + f, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = fmaf(v[i], fmaf(v[i], fmaf(v[i], c, b), a), e);
    st8(out + t * ldo + f, v);
  }
}

template <typename TA>
__global__ void sigmoid_gate_mul_kernel(TA* __restrict__ y, long long ldy, const TA* __restrict__ gate, long long ldg, int n, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / n;
    const int c = (int)(i % n);
    const float g = ld_a(gate, t * ldg + c);
    st_a(y, t * ldy + c, ld_a(y, t * ldy + c) / (1.0f + expf(-g)));
  }
}

}  // namespace

extern "C" int pg_rmsnorm_conv(const float* x, const float* w, int w_scalar, const float* conv_w, int taps, float* state, void* out_h, void* out_conv,
                               const int* row_entry, const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* entry_slot, int rows,
                               int entries, int D, float eps, int out_f32, void* stream) {
  if (rows <= 0 || D <= 0 || x == nullptr || w == nullptr || (out_h == nullptr && out_conv == nullptr)) return PG_ERR_ARG;
  if (conv_w != nullptr) {
    if (taps < 1 || taps - 1 > MAX_K || out_conv == nullptr) return PG_ERR_ARG;
    if (taps > 1 && (state == nullptr || row_entry == nullptr || entry_row0 == nullptr || entry_n == nullptr || entry_ctx == nullptr || entry_slot == nullptr))
      return PG_ERR_ARG;
  }
  cudaStream_t st = PG_ST(stream);
  const int ws = w_scalar ? 0 : 1;
  // prompt portions: chunks of consecutive rows, about two waves of four CTAs per SM; the entries' first rows and slots in a launch of their own
  const int RC = min(32, (rows + 8 * pg::num_sms() - 1) / (8 * pg::num_sms()));
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (conv_w != nullptr && taps > 1 && entries > 0 && RC >= 2 && D % 4 == 0 && al16(x) && (w_scalar || al16(w)) && al16(conv_w) && al16(state) && al16(out_h) && al16(out_conv)) {
    const int chunks = (rows + RC - 1) / RC;
    if (out_f32) {
      rmsnorm_conv_rows_kernel<float><<<chunks, 256, 0, st>>>(x, w, ws, conv_w, taps, static_cast<float*>(out_h), static_cast<float*>(out_conv), row_entry, entry_row0, rows, RC, D, eps);
      rmsnorm_conv_vec_kernel<float><<<entries, 256, 0, st>>>(x, w, ws, conv_w, taps, state, static_cast<float*>(out_h), static_cast<float*>(out_conv), row_entry,
                                                              entry_row0, entry_n, entry_ctx, entry_slot, D, eps, 1);
    } else {
      rmsnorm_conv_rows_kernel<bf16><<<chunks, 256, 0, st>>>(x, w, ws, conv_w, taps, static_cast<bf16*>(out_h), static_cast<bf16*>(out_conv), row_entry, entry_row0, rows, RC, D, eps);
      rmsnorm_conv_vec_kernel<bf16><<<entries, 256, 0, st>>>(x, w, ws, conv_w, taps, state, static_cast<bf16*>(out_h), static_cast<bf16*>(out_conv), row_entry,
                                                             entry_row0, entry_n, entry_ctx, entry_slot, D, eps, 1);
    }
    pg_count_launch(1);
    PG_RET();
  }
  const bool vec = D % 4 == 0 && al16(x) && (w_scalar || al16(w)) && al16(conv_w) && al16(state) && al16(out_h) && al16(out_conv);
#define PG_RC(KERN, TO, GRID, BY)                                                                                                                     \
  KERN<TO><<<GRID, 256, 0, st>>>(x, w, ws, conv_w, taps, state, static_cast<TO*>(out_h), static_cast<TO*>(out_conv), row_entry, entry_row0, entry_n, \
                                 entry_ctx, entry_slot, D, eps, BY)
  if (vec) {
    if (out_f32) PG_RC(rmsnorm_conv_vec_kernel, float, rows, 0);
    else PG_RC(rmsnorm_conv_vec_kernel, bf16, rows, 0);
  } else {
    if (out_f32) PG_RC(rmsnorm_conv_kernel, float, rows, 0);
    else PG_RC(rmsnorm_conv_kernel, bf16, rows, 0);
  }
  PG_RET();
}

extern "C" int pg_polynorm(const void* z, long long ldz, const float* coef, void* out, long long ldo, int rows, int F, float eps, int act_f32,
                           void* stream) {
  if (rows <= 0 || F <= 0 || z == nullptr || coef == nullptr || out == nullptr) return PG_ERR_ARG;
  if (F % 8 == 0 && ldz % 8 == 0 && ldo % 8 == 0 && ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    if (act_f32)
      polynorm_vec_kernel<float><<<rows, 256, 0, PG_ST(stream)>>>(static_cast<const float*>(z), ldz, coef, static_cast<float*>(out), ldo, F, eps);
    else
      polynorm_vec_kernel<bf16><<<rows, 256, 0, PG_ST(stream)>>>(static_cast<const bf16*>(z), ldz, coef, static_cast<bf16*>(out), ldo, F, eps);
    PG_RET();
  }
  if (act_f32)
    polynorm_kernel<float><<<rows, 256, 0, PG_ST(stream)>>>(static_cast<const float*>(z), ldz, coef, static_cast<float*>(out), ldo, F, eps);
  else
    polynorm_kernel<bf16><<<rows, 256, 0, PG_ST(stream)>>>(static_cast<const bf16*>(z), ldz, coef, static_cast<bf16*>(out), ldo, F, eps);
  PG_RET();
}

extern "C" int pg_sigmoid_gate_mul(void* y, long long ldy, const void* gate, long long ldg, int rows, int n, int act_f32, void* stream) {
  if (rows <= 0 || n <= 0 || y == nullptr || gate == nullptr) return PG_ERR_ARG;
  const long long total = (long long)rows * n;
  const int blocks = (int)((total + 255) / 256 < 8 * 148 ? (total + 255) / 256 : 8 * 148);
  if (act_f32)
    sigmoid_gate_mul_kernel<float><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<float*>(y), ldy, static_cast<const float*>(gate), ldg, n, total);
  else
    sigmoid_gate_mul_kernel<bf16><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<bf16*>(y), ldy, static_cast<const bf16*>(gate), ldg, n, total);
  PG_RET();
}
