// Kernels of the token-sequence decoders (ragged steps: every row is one token of some request) that are not
// contractions on the tensor cores: exact-precision GEMM (fp32, or bf16 operands of shapes the TMA kernels cannot take),
// embedding rows, grouped RMS norm folded into the residual add, gated RMS norm, GeGLU product, per-token side input.
//
// "act" tensors hold activations in the model's activation type: bf16 (is_f32 = 0) or fp32 (is_f32 = 1).  Norm
// statistics, the residual stream and every sum are fp32.
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

#define PG_ST(s) reinterpret_cast<cudaStream_t>(s)
#define PG_RET()                                                   \
  do {                                                             \
    pg_count_launch(1);                                            \
    return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA; \
  } while (0)

namespace {

template <typename T>
__device__ __forceinline__ float ld_f(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_f<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void st_f(T* p, long long i, float v);
template <>
__device__ __forceinline__ void st_f<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st_f<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide sum of one value per thread; `red` holds at least 32 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// ---------------------------------------------------------------------------------------------------------------------
// out[t, f] = sum_k x[t, k] * w[f, k]: 64 x 64 output tile per CTA, 16-wide k steps through shared memory, a 4 x 4
// register tile per thread, plain fp32 FMAs in k order (no reduced-precision tensor mode, no split accumulation).
// ---------------------------------------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TI* __restrict__ x, long long ldx, const TI* __restrict__ w, long long ldw,
                                                        TO* __restrict__ out, long long ldo, int T, int F, int K, long long bsx = 0,
                                                        long long bsw = 0, long long bso = 0, const float* __restrict__ bias = nullptr,
                                                        int accumulate = 0, float scale = 1.0f) {
  __shared__ float xs[16][64 + 4];
  __shared__ float ws[16][64 + 4];
  x += blockIdx.z * bsx;  // batched form: grid.z independent products with their own operand offsets
  w += blockIdx.z * bsw;
  out += blockIdx.z * bso;
  const int t0 = blockIdx.y * 64, f0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, k = i & 15;
      xs[k][r] = (t0 + r < T && k0 + k < K) ? ld_f(x, (long long)(t0 + r) * ldx + k0 + k) : 0.f;
      ws[k][r] = (f0 + r < F && k0 + k < K) ? ld_f(w, (long long)(f0 + r) * ldw + k0 + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + ty * 4 + i, f = f0 + tx * 4 + j;
      if (t < T && f < F) {
        float v = acc[i][j];
        if (bias != nullptr) v += bias[f];
        v *= scale;
        if (accumulate) v += ld_f(out, (long long)t * ldo + f);
        st_f(out, (long long)t * ldo + f, v);
      }
    }
}

// x[t, :] = table[token[t], col0 : col0 + D] * scale   (fp32 out)
template <typename TI>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const TI* __restrict__ table, long long ld, int col0, float* __restrict__ out,
                                  int D, float scale) {
  const int t = blockIdx.x;
  const long long row = tokens[t];
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(long long)t * D + d] = ld_f(table, row * ld + col0 + d) * scale;
}

// Grouped RMS norm of y (fp32) times w, optionally added to the fp32 residual row x (in place); the result (the new residual,
// or the bare norm when x == NULL) is also written in the activation type when out_act != NULL.  One CTA per row; the
// row is cut into `groups` equal consecutive parts with their own mean square.  The 8 warps share the groups (8 / groups warps
// per group when that divides, else warp w takes groups w, w + 8, ...), one block barrier, then one pass that re-reads y from L1.
// VEC: float4 accesses (group size a multiple of 4, 16-byte aligned rows).
__device__ __forceinline__ void st_act4(float* p, long long i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void st_act4(bf16* p, long long i, float4 v) {
  uint2 u;
  u.x = pg::pack_bf16(v.x, v.y);
  u.y = pg::pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(p + i) = u;
}

template <typename TO, bool VEC>
__global__ void __launch_bounds__(256) group_rmsnorm_add_kernel(const float* __restrict__ y, long long ldy, const float* __restrict__ w,
                                                                float* __restrict__ x, TO* __restrict__ out_act, int D, int groups, float eps) {
  extern __shared__ float sm[];  // 8 partial sums, then 1 / rms of every group
  float* red = sm;
  float* inv = sm + 8;
  const long long t = blockIdx.x;
  const float* yr = y + t * ldy;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gs = D / groups;
  const int wpg = (groups <= 8 && 8 % groups == 0) ? 8 / groups : 1;
  if (wpg > 1) {
    const int g = warp / wpg, part = warp % wpg;
    float s = 0.f;
    if (VEC) {
      const float4* y4 = reinterpret_cast<const float4*>(yr + (long long)g * gs);
      for (int i = part * 32 + lane; i < gs / 4; i += wpg * 32) { const float4 v = y4[i]; s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s)))); }
    } else {
      for (int i = part * 32 + lane; i < gs; i += wpg * 32) { const float v = yr[(long long)g * gs + i]; s = fmaf(v, v, s); }
    }
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (threadIdx.x < groups) {
      float tot = 0.f;
      for (int p = 0; p < wpg; ++p) tot += red[threadIdx.x * wpg + p];
      inv[threadIdx.x] = 1.0f / sqrtf(tot / (float)gs + eps);
    }
  } else {
    for (int g = warp; g < groups; g += 8) {
      float s = 0.f;
      for (int i = lane; i < gs; i += 32) { const float v = yr[(long long)g * gs + i]; s = fmaf(v, v, s); }
      s = warp_sum(s);
      if (lane == 0) inv[g] = 1.0f / sqrtf(s / (float)gs + eps);
    }
  }
  __syncthreads();
  if (VEC) {
    const float4* y4 = reinterpret_cast<const float4*>(yr);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (int i = threadIdx.x; i < D / 4; i += 256) {
      const float4 v = y4[i], ww = w4[i];
      const float iv = inv[(i * 4) / gs];
      float4 r = make_float4(v.x * iv * ww.x, v.y * iv * ww.y, v.z * iv * ww.z, v.w * iv * ww.w);
      if (x != nullptr) {
        float4* xp = reinterpret_cast<float4*>(x + t * D) + i;
        const float4 xv = *xp;
        r.x += xv.x; r.y += xv.y; r.z += xv.z; r.w += xv.w;
        *xp = r;
      }
      if (out_act != nullptr) st_act4(out_act, t * D + 4LL * i, r);
    }
  } else {
    for (int d = threadIdx.x; d < D; d += 256) {
      float v = yr[d] * inv[d / gs] * w[d];
      if (x != nullptr) { v += x[t * D + d]; x[t * D + d] = v; }
      if (out_act != nullptr) st_f(out_act, t * D + d, v);
    }
  }
}

// out[t, :] = rms(o[t, :]) * w * sigmoid(gate[t, :])   (o fp32 [T, D]; gate: activation-type column slice, pitch ldg)
// VEC: four elements per thread and access (D a multiple of 4, 16-byte aligned fp32 rows, 8-byte aligned bf16 rows).
__device__ __forceinline__ float4 ld_act4(const float* p, long long i) { return *reinterpret_cast<const float4*>(p + i); }
__device__ __forceinline__ float4 ld_act4(const bf16* p, long long i) {
  const uint2 u = *reinterpret_cast<const uint2*>(p + i);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}

template <typename TA, bool VEC>
__global__ void __launch_bounds__(256) rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const TA* __restrict__ gate,
                                                           long long ldg, TA* __restrict__ out, int D, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float s = 0.f;
  if (VEC) {
    const float4* o4 = reinterpret_cast<const float4*>(o + t * D);
    for (int i = threadIdx.x; i < D / 4; i += 256) { const float4 v = o4[i]; s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s)))); }
  } else {
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = o[t * D + d]; s = fmaf(v, v, s); }
  }
  s = block_sum(s, red);
  const float inv = 1.0f / sqrtf(s / (float)D + eps);
  if (VEC) {
    const float4* o4 = reinterpret_cast<const float4*>(o + t * D);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (int i = threadIdx.x; i < D / 4; i += 256) {
      const float4 v = o4[i], ww = w4[i], g = ld_act4(gate, t * ldg + 4LL * i);
      st_act4(out, t * D + 4LL * i, make_float4(v.x * inv * ww.x / (1.0f + expf(-g.x)), v.y * inv * ww.y / (1.0f + expf(-g.y)),
                                                v.z * inv * ww.z / (1.0f + expf(-g.z)), v.w * inv * ww.w / (1.0f + expf(-g.w))));
    }
  } else {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const float g = ld_f(gate, t * ldg + d);
      st_f(out, t * D + d, o[t * D + d] * inv * w[d] * (1.0f / (1.0f + expf(-g))));
    }
  }
}

// out[t, f] = gelu_tanh(gu[t, f]) * gu[t, F + f]    (unfused gate || up product: the exact-precision path)
template <typename TA>
__global__ void geglu_kernel(const TA* __restrict__ gu, long long ldgu, TA* __restrict__ out, long long ldo, int F, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / F;
  const int f = (int)(i % F);
  st_f(out, t * ldo + f, pg::gelu_tanh(ld_f(gu, t * ldgu + f)) * ld_f(gu, t * ldgu + F + f));
}

// x[t, f] <- relu(x[t, f])^2 in place (the unfused activation of the exact-precision path)
template <typename TA>
__global__ void relu2_kernel(TA* __restrict__ x, long long ld, int F, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / F;
  const int f = (int)(i % F);
  const float v = fmaxf(ld_f(x, t * ld + f), 0.f);
  st_f(x, t * ld + f, v * v);
}

// out[t, j] = gelu_tanh(z[t, j]) * table[token[t], col0 + j]  for j < n, zero for n <= j < n_pad   (z fp32)
template <typename TA>
__global__ void side_gate_kernel(const float* __restrict__ z, long long ldz, const int* __restrict__ tokens, const TA* __restrict__ table, long long ldt,
                                 int col0, TA* __restrict__ out, long long ldo, int n, int n_pad, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / n_pad;
  const int j = (int)(i % n_pad);
  float v = 0.f;
  if (j < n) v = pg::gelu_tanh(z[t * ldz + j]) * ld_f(table, (long long)tokens[t] * ldt + col0 + j);
  st_f(out, t * ldo + j, v);
}

}  // namespace

extern "C" int pg_gemm_simt(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int tokens, int features,
                            int K, int in_f32, int out_f32, void* stream) {
  if (tokens <= 0 || features <= 0 || K <= 0 || x == nullptr || w == nullptr || out == nullptr) return PG_ERR_ARG;
  dim3 grid((features + 63) / 64, (tokens + 63) / 64);
  if (grid.y > 65535) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  if (in_f32 && out_f32)
    gemm_simt_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ldx, static_cast<const float*>(w), ldw, static_cast<float*>(out), ldo, tokens, features, K);
  else if (!in_f32 && out_f32)
    gemm_simt_kernel<bf16, float><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), ldw, static_cast<float*>(out), ldo, tokens, features, K);
  else if (!in_f32 && !out_f32)
    gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), ldw, static_cast<bf16*>(out), ldo, tokens, features, K);
  else
    return PG_ERR_ARG;
  PG_RET();
}

extern "C" int pg_gemm_simt_bias(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, const float* bias,
                                 int accumulate, float scale, int tokens, int features, int K, int in_f32, int out_f32, void* stream) {
  if (tokens <= 0 || features <= 0 || K <= 0 || x == nullptr || w == nullptr || out == nullptr) return PG_ERR_ARG;
  dim3 grid((features + 63) / 64, (tokens + 63) / 64);
  if (grid.y > 65535) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  if (in_f32 && out_f32)
    gemm_simt_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ldx, static_cast<const float*>(w), ldw, static_cast<float*>(out), ldo, tokens, features, K, 0, 0, 0, bias, accumulate, scale);
  else if (!in_f32 && out_f32)
    gemm_simt_kernel<bf16, float><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), ldw, static_cast<float*>(out), ldo, tokens, features, K, 0, 0, 0, bias, accumulate, scale);
  else if (!in_f32 && !out_f32)
    gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), ldw, static_cast<bf16*>(out), ldo, tokens, features, K, 0, 0, 0, bias, accumulate, scale);
  else
    return PG_ERR_ARG;
  PG_RET();
}

extern "C" int pg_gemm_simt_batched(const void* x, long long ldx, long long batch_x, const void* w, long long ldw, long long batch_w, void* out,
                                    long long ldo, long long batch_out, int tokens, int features, int K, int batch, int in_f32, int out_f32,
                                    void* stream) {
  if (tokens <= 0 || features <= 0 || K <= 0 || batch <= 0 || batch > 65535 || x == nullptr || w == nullptr || out == nullptr) return PG_ERR_ARG;
  dim3 grid((features + 63) / 64, (tokens + 63) / 64, batch);
  if (grid.y > 65535) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  if (in_f32 && out_f32)
    gemm_simt_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ldx, static_cast<const float*>(w), ldw, static_cast<float*>(out), ldo, tokens, features, K, batch_x, batch_w, batch_out);
  else if (!in_f32 && out_f32)
    gemm_simt_kernel<bf16, float><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), ldw, static_cast<float*>(out), ldo, tokens, features, K, batch_x, batch_w, batch_out);
  else if (!in_f32 && !out_f32)
    gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), ldw, static_cast<bf16*>(out), ldo, tokens, features, K, batch_x, batch_w, batch_out);
  else
    return PG_ERR_ARG;
  PG_RET();
}

extern "C" int pg_embed_rows(const int* tokens, const void* table, long long ld, int col0, float* out, int rows, int D, float scale,
                             int table_f32, void* stream) {
  if (rows <= 0 || D <= 0) return PG_ERR_ARG;
  if (table_f32)
    embed_rows_kernel<float><<<rows, 128, 0, PG_ST(stream)>>>(tokens, static_cast<const float*>(table), ld, col0, out, D, scale);
  else
    embed_rows_kernel<bf16><<<rows, 128, 0, PG_ST(stream)>>>(tokens, static_cast<const bf16*>(table), ld, col0, out, D, scale);
  PG_RET();
}

extern "C" int pg_group_rmsnorm_add(const float* y, long long ldy, const float* w, float* x, void* out_act, int rows, int D, int groups,
                                    float eps, int out_f32, void* stream) {
  if (rows <= 0 || D <= 0 || groups <= 0 || (D % groups) != 0 || groups > 4096) return PG_ERR_ARG;
  const size_t smem = (8 + groups) * sizeof(float);
  cudaStream_t st = PG_ST(stream);
  const bool vec = ((D / groups) % 4 == 0) && (ldy % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out_act)) & 15) == 0;
  if (out_f32) {
    if (vec) group_rmsnorm_add_kernel<float, true><<<rows, 256, smem, st>>>(y, ldy, w, x, static_cast<float*>(out_act), D, groups, eps);
    else group_rmsnorm_add_kernel<float, false><<<rows, 256, smem, st>>>(y, ldy, w, x, static_cast<float*>(out_act), D, groups, eps);
  } else {
    if (vec) group_rmsnorm_add_kernel<bf16, true><<<rows, 256, smem, st>>>(y, ldy, w, x, static_cast<bf16*>(out_act), D, groups, eps);
    else group_rmsnorm_add_kernel<bf16, false><<<rows, 256, smem, st>>>(y, ldy, w, x, static_cast<bf16*>(out_act), D, groups, eps);
  }
  PG_RET();
}

extern "C" int pg_rmsnorm_gate(const float* o, const float* w, const void* gate, long long ldg, void* out, int rows, int D, float eps,
                               int act_f32, void* stream) {
  if (rows <= 0 || D <= 0) return PG_ERR_ARG;
  const uintptr_t act_mask = act_f32 ? 15 : 7;
  const bool vec = (D % 4 == 0) && (ldg % 4 == 0) && ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(out)) & act_mask) == 0;
  cudaStream_t st = PG_ST(stream);
  if (act_f32) {
    if (vec) rmsnorm_gate_kernel<float, true><<<rows, 256, 0, st>>>(o, w, static_cast<const float*>(gate), ldg, static_cast<float*>(out), D, eps);
    else rmsnorm_gate_kernel<float, false><<<rows, 256, 0, st>>>(o, w, static_cast<const float*>(gate), ldg, static_cast<float*>(out), D, eps);
  } else {
    if (vec) rmsnorm_gate_kernel<bf16, true><<<rows, 256, 0, st>>>(o, w, static_cast<const bf16*>(gate), ldg, static_cast<bf16*>(out), D, eps);
    else rmsnorm_gate_kernel<bf16, false><<<rows, 256, 0, st>>>(o, w, static_cast<const bf16*>(gate), ldg, static_cast<bf16*>(out), D, eps);
  }
  PG_RET();
}

extern "C" int pg_geglu(const void* gu, long long ldgu, void* out, long long ldo, int rows, int F, int act_f32, void* stream) {
  if (rows <= 0 || F <= 0) return PG_ERR_ARG;
  const long long total = (long long)rows * F;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act_f32)
    geglu_kernel<float><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<const float*>(gu), ldgu, static_cast<float*>(out), ldo, F, total);
  else
    geglu_kernel<bf16><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<const bf16*>(gu), ldgu, static_cast<bf16*>(out), ldo, F, total);
  PG_RET();
}

extern "C" int pg_relu2(void* x, long long ld, int rows, int F, int act_f32, void* stream) {
  if (rows <= 0 || F <= 0) return PG_ERR_ARG;
  const long long total = (long long)rows * F;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act_f32) relu2_kernel<float><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<float*>(x), ld, F, total);
  else relu2_kernel<bf16><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<bf16*>(x), ld, F, total);
  PG_RET();
}

extern "C" int pg_side_gate(const float* z, long long ldz, const int* tokens, const void* table, long long ldt, int col0, void* out,
                            long long ldo, int rows, int n, int n_pad, int act_f32, void* stream) {
  if (rows <= 0 || n <= 0 || n_pad < n) return PG_ERR_ARG;
  const long long total = (long long)rows * n_pad;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act_f32)
    side_gate_kernel<float><<<blocks, 256, 0, PG_ST(stream)>>>(z, ldz, tokens, static_cast<const float*>(table), ldt, col0,
                                                              static_cast<float*>(out), ldo, n, n_pad, total);
  else
    side_gate_kernel<bf16><<<blocks, 256, 0, PG_ST(stream)>>>(z, ldz, tokens, static_cast<const bf16*>(table), ldt, col0,
                                                             static_cast<bf16*>(out), ldo, n, n_pad, total);
  PG_RET();
}
