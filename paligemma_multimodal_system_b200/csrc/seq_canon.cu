// Row kernels of decoders whose mixer reads the normalised residual through a short causal convolution over time:
//
//   pg_rmsnorm_conv     h = x / sqrt(mean(x^2) + eps) * g (g: one weight per channel, or ONE number for the whole row);
//                       out_h[t] = h[t] (what a feed-forward beside the mixer reads), out_conv[t] = h[t] + sum_j cw[:, j] h[t - taps + 1 + j]
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
                                                           const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int D, float eps) {
  __shared__ float red[8];
  __shared__ float inv[2 * MAX_K + 1];
  const long long t = blockIdx.x;
  const int K = cw != nullptr ? taps - 1 : 0;
  int i = 0, ne = 1, e = 0;
  if (K > 0) {
    e = row_entry[t];
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
          acc = fmaf(cw[(long long)d * taps + K], hv, acc);
          for (int j = 0; j < K; ++j) acc = fmaf(cw[(long long)d * taps + j], x[(t - K + j) * D + d] * inv[j] * g, acc);
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
              acc = fmaf(cw[(long long)d * taps + j], v, acc);
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
                               int D, float eps, int out_f32, void* stream) {
  if (rows <= 0 || D <= 0 || x == nullptr || w == nullptr || (out_h == nullptr && out_conv == nullptr)) return PG_ERR_ARG;
  if (conv_w != nullptr) {
    if (taps < 1 || taps - 1 > MAX_K || out_conv == nullptr) return PG_ERR_ARG;
    if (taps > 1 && (state == nullptr || row_entry == nullptr || entry_row0 == nullptr || entry_n == nullptr || entry_ctx == nullptr || entry_slot == nullptr))
      return PG_ERR_ARG;
  }
  cudaStream_t st = PG_ST(stream);
  const int ws = w_scalar ? 0 : 1;
  if (out_f32)
    rmsnorm_conv_kernel<float><<<rows, 256, 0, st>>>(x, w, ws, conv_w, taps, state, static_cast<float*>(out_h), static_cast<float*>(out_conv), row_entry,
                                                     entry_row0, entry_n, entry_ctx, entry_slot, D, eps);
  else
    rmsnorm_conv_kernel<bf16><<<rows, 256, 0, st>>>(x, w, ws, conv_w, taps, state, static_cast<bf16*>(out_h), static_cast<bf16*>(out_conv), row_entry,
                                                    entry_row0, entry_n, entry_ctx, entry_slot, D, eps);
  PG_RET();
}

extern "C" int pg_polynorm(const void* z, long long ldz, const float* coef, void* out, long long ldo, int rows, int F, float eps, int act_f32,
                           void* stream) {
  if (rows <= 0 || F <= 0 || z == nullptr || coef == nullptr || out == nullptr) return PG_ERR_ARG;
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
