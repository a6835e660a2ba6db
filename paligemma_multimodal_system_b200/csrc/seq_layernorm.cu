// Row kernels of decoders whose layers read ONE residual through two layer norms at once (mixer and feed-forward side by
// side), with the mixer's input blended with the previous token's:
//
//   pg_layernorm_shift   a = LN(x; w1, b1), b = LN(x; w2, b2) from one mean / variance of the row;
//                        out1[t] = a[t] + (a[t-1] - a[t]) * shift   (a[-1] = 0; a of a sequence's last token is kept in an
//                        fp32 state slot, so a portion or a decoded token continues where the sequence stopped), out2[t] = b[t]
//   pg_glu               gated-unit activations on a [gate | up] product that the GEMM epilogue did not fuse
//
// LN(z) = (z - mean) / sqrt(mean((z - mean)^2) + eps) * w + b, statistics in fp32 from the fp32 residual.
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

template <typename T>
__device__ __forceinline__ void st_act(T* p, long long i, float v);
template <>
__device__ __forceinline__ void st_act<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st_act<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
template <typename T>
__device__ __forceinline__ float ld_act(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_act<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_act<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }

// sum over the 256 threads of the CTA; every thread gets the result.  `red` = 8 floats of shared memory.
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

// row -> shared memory, mean and 1 / sqrt(var + eps) (two passes over the staged row: the variance is the mean of the squared
// deviations, not a difference of large numbers)
__device__ __forceinline__ void stage_row(const float* __restrict__ src, float* buf, int D, float eps, float* red, float& mean, float& rstd) {
  float s = 0.f;
  for (int d = threadIdx.x; d < D; d += 256) {
    const float v = src[d];
    buf[d] = v;
    s += v;
  }
  mean = block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int d = threadIdx.x; d < D; d += 256) {  // each thread re-reads what it wrote
    const float c = buf[d] - mean;
    q = fmaf(c, c, q);
  }
  rstd = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
}

// One CTA per row.  Who owns the state slot of entry e: the CTA of the entry's FIRST row -- it reads the slot (the previous
// token's a) and it alone writes the slot (a of the entry's last row, recomputed here when that is another row), so no other
// CTA of the launch touches the slot.  Rows inside an entry recompute a of the row before them from x.
template <typename TO>
__global__ void __launch_bounds__(256) layernorm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ b1,
                                                              const float* __restrict__ shift, const float* __restrict__ w2,
                                                              const float* __restrict__ b2, TO* __restrict__ out1, TO* __restrict__ out2,
                                                              float* __restrict__ state, const int* __restrict__ pos,
                                                              const int* __restrict__ row_entry, const int* __restrict__ entry_row0,
                                                              const int* __restrict__ entry_n, const int* __restrict__ entry_slot, int D, float eps) {
  extern __shared__ float sm[];
  float* cur = sm;          // [D] this row
  float* oth = sm + D;      // [D] the row before / the entry's last row (only with a shift)
  __shared__ float red[8];
  const long long t = blockIdx.x;
  float mean, rstd;
  stage_row(x + t * D, cur, D, eps, red, mean, rstd);
  if (shift == nullptr) {
    for (int d = threadIdx.x; d < D; d += 256) {
      const float c = (cur[d] - mean) * rstd;
      st_act(out1, t * D + d, fmaf(c, w1[d], b1[d]));
      if (out2 != nullptr) st_act(out2, t * D + d, fmaf(c, w2[d], b2[d]));
    }
    return;
  }
  const int e = row_entry[t], p = pos[t];
  const int first = entry_row0[e], n = entry_n[e];
  const bool owner = t == first;
  float* slot = state + (long long)entry_slot[e] * D;
  float pm = 0.f, pr = 0.f;
  const int prev_kind = p == 0 ? 0 : owner ? 1 : 2;  // zeros / the state slot / the row before
  if (prev_kind == 2) stage_row(x + (t - 1) * D, oth, D, eps, red, pm, pr);
  for (int d = threadIdx.x; d < D; d += 256) {
    const float c = (cur[d] - mean) * rstd;
    const float a = fmaf(c, w1[d], b1[d]);
    float ap = 0.f;
    if (prev_kind == 1) ap = slot[d];
    else if (prev_kind == 2) ap = fmaf((oth[d] - pm) * pr, w1[d], b1[d]);
    st_act(out1, t * D + d, fmaf(ap - a, shift[d], a));
    if (out2 != nullptr) st_act(out2, t * D + d, fmaf(c, w2[d], b2[d]));
    if (owner && n == 1) slot[d] = a;  // the same thread read slot[d] above
  }
  if (owner && n > 1) {
    stage_row(x + (long long)(first + n - 1) * D, oth, D, eps, red, pm, pr);  // block_sum's barriers order this after the loop above
    for (int d = threadIdx.x; d < D; d += 256) slot[d] = fmaf((oth[d] - pm) * pr, w1[d], b1[d]);
  }
}

// The same for widths that are a multiple of 4 up to 8192: the row (and the row before) in registers as VT float4 per thread, every
// load of both rows in flight at once, and the two rows' statistics reduced TOGETHER (two block reductions for mean and variance
// of both rows).  Used whenever the pointers are 16-byte aligned; the kernel above is the fallback for other widths.
__device__ __forceinline__ void block_sum2(float& a, float& b, float (*red)[8]) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  __syncthreads();  // the previous use of `red` is over
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a; red[1][threadIdx.x >> 5] = b; }
  __syncthreads();
  a = 0.f; b = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
}

__device__ __forceinline__ float sum4(float4 v) { return (v.x + v.y) + (v.z + v.w); }
__device__ __forceinline__ float dev4(float4 v, float m) {
  const float a = v.x - m, b = v.y - m, c = v.z - m, d = v.w - m;
  return fmaf(a, a, fmaf(b, b, fmaf(c, c, d * d)));
}
__device__ __forceinline__ float4 ln4(float4 v, float mean, float rstd, float4 w, float4 b) {
  return make_float4(fmaf((v.x - mean) * rstd, w.x, b.x), fmaf((v.y - mean) * rstd, w.y, b.y), fmaf((v.z - mean) * rstd, w.z, b.z),
                     fmaf((v.w - mean) * rstd, w.w, b.w));
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TO, int VT>
__global__ void __launch_bounds__(256) layernorm_shift_vec_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ b1,
                                                                  const float* __restrict__ shift, const float* __restrict__ w2,
                                                                  const float* __restrict__ b2, TO* __restrict__ out1, TO* __restrict__ out2,
                                                                  float* __restrict__ state, const int* __restrict__ pos,
                                                                  const int* __restrict__ row_entry, const int* __restrict__ entry_row0,
                                                                  const int* __restrict__ entry_n, const int* __restrict__ entry_slot, int D, float eps) {
  __shared__ float red[2][8];
  const long long t = blockIdx.x;
  int e = 0, first = 0, n = 1, prev_kind = 0;
  if (shift != nullptr) {
    e = row_entry[t];
    first = entry_row0[e];
    n = entry_n[e];
    prev_kind = pos[t] == 0 ? 0 : t == first ? 1 : 2;  // zeros / the state slot / the row before
  }
  const bool owner = shift != nullptr && t == first;
  float* slot = shift != nullptr ? state + (long long)entry_slot[e] * D : nullptr;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[VT], u[VT];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < VT; ++i) {
    const int d = 4 * (threadIdx.x + 256 * i);
    v[i] = d < D ? ld4(x + t * D + d) : zero;
    u[i] = (prev_kind == 2 && d < D) ? ld4(x + (t - 1) * D + d) : (prev_kind == 1 && d < D) ? ld4(slot + d) : zero;
    s1 += sum4(v[i]);
    s2 += sum4(u[i]);
  }
  block_sum2(s1, s2, red);
  const float mean = s1 / (float)D, pm = s2 / (float)D;
  float q1 = 0.f, q2 = 0.f;
#pragma unroll
  for (int i = 0; i < VT; ++i)
    if (4 * (threadIdx.x + 256 * i) < D) {
      q1 += dev4(v[i], mean);
      q2 += dev4(u[i], pm);
    }
  block_sum2(q1, q2, red);
  const float rstd = 1.0f / sqrtf(q1 / (float)D + eps), pr = 1.0f / sqrtf(q2 / (float)D + eps);
#pragma unroll
  for (int i = 0; i < VT; ++i) {
    const int d = 4 * (threadIdx.x + 256 * i);
    if (d >= D) continue;
    const float4 w = ld4(w1 + d), b = ld4(b1 + d);
    const float4 a = ln4(v[i], mean, rstd, w, b);
    if (shift != nullptr) {
      const float4 ap = prev_kind == 2 ? ln4(u[i], pm, pr, w, b) : u[i];  // the slot already holds a; zeros at position 0
      const float4 sh = ld4(shift + d);
      st4(out1 + t * D + d, make_float4(fmaf(ap.x - a.x, sh.x, a.x), fmaf(ap.y - a.y, sh.y, a.y), fmaf(ap.z - a.z, sh.z, a.z), fmaf(ap.w - a.w, sh.w, a.w)));
      if (owner && n == 1) st4(slot + d, a);  // the same thread read slot[d .. d + 3] above
    } else {
      st4(out1 + t * D + d, a);
    }
    if (out2 != nullptr) st4(out2 + t * D + d, ln4(v[i], mean, rstd, ld4(w2 + d), ld4(b2 + d)));
  }
  if (owner && n > 1) {  // this CTA alone touches the slot: a of the entry's last row
    const float* xl = x + (long long)(first + n - 1) * D;
    float sl = 0.f, dummy = 0.f;
#pragma unroll
    for (int i = 0; i < VT; ++i) {
      const int d = 4 * (threadIdx.x + 256 * i);
      u[i] = d < D ? ld4(xl + d) : zero;
      sl += sum4(u[i]);
    }
    block_sum2(sl, dummy, red);
    const float lm = sl / (float)D;
    float ql = 0.f;
#pragma unroll
    for (int i = 0; i < VT; ++i)
      if (4 * (threadIdx.x + 256 * i) < D) ql += dev4(u[i], lm);
    block_sum2(ql, dummy, red);
    const float lr = 1.0f / sqrtf(ql / (float)D + eps);
#pragma unroll
    for (int i = 0; i < VT; ++i) {
      const int d = 4 * (threadIdx.x + 256 * i);
      if (d < D) st4(slot + d, ln4(u[i], lm, lr, ld4(w1 + d), ld4(b1 + d)));
    }
  }
}

// Many rows (prompt portions): a CTA walks R CONSECUTIVE rows.  The next row's loads are in flight while the current one is
// reduced and written, and a of the row just finished stays in registers as the next row's "previous token", so a row is read
// once; only a chunk's first row, when it continues an entry, rebuilds a of the row before it.  Slot ownership as above.
__device__ __forceinline__ float block_sum1(float a, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) s += red[w];
  return s;
}

template <int VT>
__device__ __forceinline__ void row_stats(const float4 (&v)[VT], int D, float eps, float* red, float& mean, float& rstd) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VT; ++i) s += sum4(v[i]);  // lanes past D hold zeros
  mean = block_sum1(s, red) / (float)D;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VT; ++i)
    if (4 * (threadIdx.x + 256 * i) < D) q += dev4(v[i], mean);
  rstd = 1.0f / sqrtf(block_sum1(q, red) / (float)D + eps);
}

template <int VT>
__device__ __forceinline__ void load_row(const float* __restrict__ src, int D, float4 (&v)[VT]) {
#pragma unroll
  for (int i = 0; i < VT; ++i) {
    const int d = 4 * (threadIdx.x + 256 * i);
    v[i] = d < D ? ld4(src + d) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <typename TO, int VT>
__global__ void __launch_bounds__(256) layernorm_shift_rows_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ b1,
                                                                   const float* __restrict__ shift, const float* __restrict__ w2,
                                                                   const float* __restrict__ b2, TO* __restrict__ out1, TO* __restrict__ out2,
                                                                   float* __restrict__ state, const int* __restrict__ pos,
                                                                   const int* __restrict__ row_entry, const int* __restrict__ entry_row0,
                                                                   const int* __restrict__ entry_n, const int* __restrict__ entry_slot, int rows, int R, int D,
                                                                   float eps) {
  __shared__ float red[8];
  const int t0 = blockIdx.x * R, t1 = min(rows, t0 + R);
  if (t0 >= rows) return;
  float4 v[VT], vn[VT], ap[VT];
  load_row<VT>(x + (long long)t0 * D, D, vn);
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int i = 0; i < VT; ++i) v[i] = vn[i];
    if (t + 1 < t1) load_row<VT>(x + (long long)(t + 1) * D, D, vn);  // in flight during this row's reductions
    float mean, rstd;
    row_stats<VT>(v, D, eps, red, mean, rstd);
    const int e = row_entry[t];
    const int first = entry_row0[e], n = entry_n[e];
    const bool owner = t == first;
    float* slot = state + (long long)entry_slot[e] * D;
    if (pos[t] == 0) {
#pragma unroll
      for (int i = 0; i < VT; ++i) ap[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else if (owner) {
      load_row<VT>(slot, D, ap);
    } else if (t == t0) {  // the chunk starts inside an entry: a of the row before, rebuilt from x
      float pm, pr;
      load_row<VT>(x + (long long)(t - 1) * D, D, ap);
      row_stats<VT>(ap, D, eps, red, pm, pr);
#pragma unroll
      for (int i = 0; i < VT; ++i) {
        const int d = 4 * (threadIdx.x + 256 * i);
        if (d < D) ap[i] = ln4(ap[i], pm, pr, ld4(w1 + d), ld4(b1 + d));
      }
    }  // else: ap holds a of row t - 1 of the same entry, left by the previous iteration
#pragma unroll
    for (int i = 0; i < VT; ++i) {
      const int d = 4 * (threadIdx.x + 256 * i);
      if (d >= D) continue;
      const float4 a = ln4(v[i], mean, rstd, ld4(w1 + d), ld4(b1 + d));
      const float4 sh = ld4(shift + d);
      st4(out1 + (long long)t * D + d, make_float4(fmaf(ap[i].x - a.x, sh.x, a.x), fmaf(ap[i].y - a.y, sh.y, a.y), fmaf(ap[i].z - a.z, sh.z, a.z),
                                                   fmaf(ap[i].w - a.w, sh.w, a.w)));
      if (out2 != nullptr) st4(out2 + (long long)t * D + d, ln4(v[i], mean, rstd, ld4(w2 + d), ld4(b2 + d)));
      if (owner && n == 1) st4(slot + d, a);  // the same thread read slot[d .. d + 3] above
      ap[i] = a;
    }
    if (owner && n > 1) {  // this CTA alone touches the slot: a of the entry's last row
      float4 u[VT];
      float lm, lr;
      load_row<VT>(x + (long long)(first + n - 1) * D, D, u);
      row_stats<VT>(u, D, eps, red, lm, lr);
#pragma unroll
      for (int i = 0; i < VT; ++i) {
        const int d = 4 * (threadIdx.x + 256 * i);
        if (d < D) st4(slot + d, ln4(u[i], lm, lr, ld4(w1 + d), ld4(b1 + d)));
      }
    }
  }
}

template <typename TO, int VT>
int launch_ln_rows(const float* x, const float* w1, const float* b1, const float* shift, const float* w2, const float* b2, void* out1, void* out2, float* state,
                   const int* pos, const int* row_entry, const int* entry_row0, const int* entry_n, const int* entry_slot, int rows, int R, int D, float eps,
                   cudaStream_t st) {
  layernorm_shift_rows_kernel<TO, VT><<<(rows + R - 1) / R, 256, 0, st>>>(x, w1, b1, shift, w2, b2, static_cast<TO*>(out1), static_cast<TO*>(out2), state, pos,
                                                                          row_entry, entry_row0, entry_n, entry_slot, rows, R, D, eps);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

template <typename TO, int VT>
int launch_ln_vec(const float* x, const float* w1, const float* b1, const float* shift, const float* w2, const float* b2, void* out1, void* out2, float* state,
                  const int* pos, const int* row_entry, const int* entry_row0, const int* entry_n, const int* entry_slot, int rows, int D, float eps,
                  cudaStream_t st) {
  layernorm_shift_vec_kernel<TO, VT><<<rows, 256, 0, st>>>(x, w1, b1, shift, w2, b2, static_cast<TO*>(out1), static_cast<TO*>(out2), state, pos, row_entry,
                                                           entry_row0, entry_n, entry_slot, D, eps);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

// kind 1: silu(g) * u;  kind 2: g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1)
template <typename TA>
__global__ void glu_kernel(const TA* __restrict__ gu, long long ldgu, TA* __restrict__ out, long long ldo, int F, long long total, int kind,
                           float limit, float alpha) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / F;
    const int f = (int)(i % F);
    float g = ld_act(gu, t * ldgu + f), u = ld_act(gu, t * ldgu + F + f), y;
    if (kind == 2) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      y = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    } else {
      y = g / (1.0f + expf(-g)) * u;
    }
    st_act(out, t * ldo + f, y);
  }
}

}  // namespace

extern "C" int pg_layernorm_shift(const float* x, const float* w1, const float* b1, const float* shift, const float* w2, const float* b2, void* out1,
                                  void* out2, float* state, const int* pos, const int* row_entry, const int* entry_row0, const int* entry_n,
                                  const int* entry_slot, int rows, int D, float eps, int out_f32, void* stream) {
  if (rows <= 0 || D <= 0 || x == nullptr || w1 == nullptr || b1 == nullptr || out1 == nullptr) return PG_ERR_ARG;
  if ((out2 != nullptr) && (w2 == nullptr || b2 == nullptr)) return PG_ERR_ARG;
  if (shift != nullptr && (state == nullptr || pos == nullptr || row_entry == nullptr || entry_row0 == nullptr || entry_n == nullptr || entry_slot == nullptr))
    return PG_ERR_ARG;
  const size_t smem = (size_t)(shift != nullptr ? 2 : 1) * D * sizeof(float);
  if (smem > 200 * 1024) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (D % 4 == 0 && D <= 8192 && al16(x) && al16(w1) && al16(b1) && al16(shift) && al16(w2) && al16(b2) && al16(out1) && al16(out2) && al16(state)) {
#define PG_LNV(VT)                                                                                                                                      \
  return out_f32 ? launch_ln_vec<float, VT>(x, w1, b1, shift, w2, b2, out1, out2, state, pos, row_entry, entry_row0, entry_n, entry_slot, rows, D, eps, st) \
                 : launch_ln_vec<bf16, VT>(x, w1, b1, shift, w2, b2, out1, out2, state, pos, row_entry, entry_row0, entry_n, entry_slot, rows, D, eps, st)
    // prompt portions: chunks of consecutive rows, about two waves of four CTAs per SM
    const int R = min(32, (rows + 8 * pg::num_sms() - 1) / (8 * pg::num_sms()));
    if (shift != nullptr && R >= 2) {
#define PG_LNR(VT)                                                                                                                                          \
  return out_f32 ? launch_ln_rows<float, VT>(x, w1, b1, shift, w2, b2, out1, out2, state, pos, row_entry, entry_row0, entry_n, entry_slot, rows, R, D, eps, st) \
                 : launch_ln_rows<bf16, VT>(x, w1, b1, shift, w2, b2, out1, out2, state, pos, row_entry, entry_row0, entry_n, entry_slot, rows, R, D, eps, st)
      if (D <= 1024) PG_LNR(1);
      if (D <= 2048) PG_LNR(2);
      if (D <= 4096) PG_LNR(4);
      PG_LNR(8);
#undef PG_LNR
    }
    if (D <= 1024) PG_LNV(1);
    if (D <= 2048) PG_LNV(2);
    if (D <= 4096) PG_LNV(4);
    PG_LNV(8);
#undef PG_LNV
  }
  if (out_f32) {
    auto kern = layernorm_shift_kernel<float>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
    kern<<<rows, 256, smem, st>>>(x, w1, b1, shift, w2, b2, static_cast<float*>(out1), static_cast<float*>(out2), state, pos, row_entry, entry_row0,
                                  entry_n, entry_slot, D, eps);
  } else {
    auto kern = layernorm_shift_kernel<bf16>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
    kern<<<rows, 256, smem, st>>>(x, w1, b1, shift, w2, b2, static_cast<bf16*>(out1), static_cast<bf16*>(out2), state, pos, row_entry, entry_row0,
                                  entry_n, entry_slot, D, eps);
  }
  PG_RET();
}

extern "C" int pg_glu(const void* gu, long long ldgu, void* out, long long ldo, int rows, int F, int kind, float limit, float alpha, int act_f32,
                      void* stream) {
  if (rows <= 0 || F <= 0 || (kind != 1 && kind != 2)) return PG_ERR_ARG;
  const long long total = (long long)rows * F;
  const int blocks = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
  if (act_f32)
    glu_kernel<float><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<const float*>(gu), ldgu, static_cast<float*>(out), ldo, F, total, kind, limit, alpha);
  else
    glu_kernel<bf16><<<blocks, 256, 0, PG_ST(stream)>>>(static_cast<const bf16*>(gu), ldgu, static_cast<bf16*>(out), ldo, F, total, kind, limit, alpha);
  PG_RET();
}
