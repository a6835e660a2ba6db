// Token mixers of the token-sequence decoders over a RAGGED step: the rows of a step are the new tokens of several
// requests ("entries"), each entry a run of n consecutive rows that continues a sequence whose first `ctx` tokens are
// already in the paged cache / the recurrent state.  A whole prompt, a portion of one and a single decoded token are
// the same case with different n and ctx, so the arithmetic of a position never depends on how its sequence was cut.
//
//   pg_attn_prepare        q/k RMS norm (shared per-head weight), interleaved partial rotation, weightless value norm;
//                          k and v rows go to their cache pages, q to a dense buffer
//   pg_attn_ragged         causal softmax attention of the new rows over the paged cache (grouped k/v heads, tanh soft cap,
//                          sigmoid output gate); scores, probabilities and the output accumulation in fp32
//   pg_linear_attn_scan    decayed outer-product recurrence S <- a S + k v^T, o = S^T q with the state in fp32,
//                          token by token (decode, short portions)
//   pg_linear_attn_chunked the same recurrence in blocks of 32 tokens (prompt portions)
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
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void stf(T* p, long long i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------------------------------
// One CTA per token row.  The cos / sin of the token's rot_dims/2 angles are computed once (angle = position * frequency
// in double, so that a position in the thousands loses nothing to the product's rounding) and shared by every head.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128) attn_prepare_kernel(const TA* __restrict__ qkv, long long ld, const int* __restrict__ pos,
                                                           const int* __restrict__ row_entry, const int* __restrict__ page_table, int max_pages,
                                                           int page, const double* __restrict__ freq, const float* __restrict__ qn,
                                                           const float* __restrict__ kn, TA* __restrict__ q_out, TA* __restrict__ k_pages,
                                                           TA* __restrict__ v_pages, int H, int G, int dim, int vdim, int rot, float eps,
                                                           int norm_qk, int norm_v, int v_from_k) {
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const long long t = blockIdx.x;
  const int p = pos[t];
  for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
    double s, c;
    sincos((double)p * freq[i], &s, &c);
    cs[i] = (float)c;
    cs[rot / 2 + i] = (float)s;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const long long pg_row = (long long)page_table[(long long)row_entry[t] * max_pages + p / page] * page + p % page;
  const TA* row = qkv + t * ld;
  const int nvec = k_pages != nullptr ? H + 2 * G : H;  // a layer that borrows another layer's keys / values prepares its queries only
  for (int vec = warp; vec < nvec; vec += nw) {
    const bool is_q = vec < H, is_k = !is_q && vec < H + G;
    const int n = (is_q || is_k) ? dim : vdim;
    // v_from_k: the row has no value columns; value head g is key head g as projected (vdim == dim), before norm and rotation
    const long long off = is_q ? (long long)vec * dim : is_k ? (long long)H * dim + (long long)(vec - H) * dim
                          : v_from_k ? (long long)H * dim + (long long)(vec - H - G) * dim
                                     : (long long)(H + G) * dim + (long long)(vec - H - G) * vdim;
    // lane <-> pairs (2i, 2i+1): a rotation never needs another lane's element; an odd last element is a pair with a zero
    float inv = 1.0f;
    if ((is_q || is_k) ? norm_qk : norm_v) {
      float ss = 0.f;
      for (int d = 2 * lane; d < n; d += 64) {
        const float a = ldf(row, off + d), b2 = d + 1 < n ? ldf(row, off + d + 1) : 0.f;
        ss = fmaf(a, a, fmaf(b2, b2, ss));
      }
      ss = wsum(ss);
      inv = 1.0f / sqrtf(ss / (float)n + eps);
    }
    const float* w = is_q ? qn : kn;  // NULL: a norm without a weight
    TA* dst = is_q   ? q_out + t * ((long long)H * dim) + (long long)vec * dim
              : is_k ? k_pages + pg_row * ((long long)G * dim) + (long long)(vec - H) * dim
                     : v_pages + pg_row * ((long long)G * vdim) + (long long)(vec - H - G) * vdim;
    for (int d = 2 * lane; d < n; d += 64) {
      const bool two = d + 1 < n;
      float a = ldf(row, off + d) * inv, b2 = two ? ldf(row, off + d + 1) * inv : 0.f;
      if (is_q || is_k) {
        if (w != nullptr) {
          a *= w[d];
          if (two) b2 *= w[d + 1];
        }
        if (d < rot) {  // rot is even: the pair is rotated as a whole
          const float c = cs[d >> 1], sn = cs[rot / 2 + (d >> 1)];
          const float ra = a * c - b2 * sn, rb = b2 * c + a * sn;
          a = ra; b2 = rb;
        }
      }
      stf(dst, d, a);
      if (two) stf(dst, d + 1, b2);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Causal attention of an entry's new rows over its paged keys / values.  CTA = 32 query rows (token x query head of one
// k/v head) of one entry; 8 warps x 4 rows.  Keys pass in tiles of 32 through shared memory (fp32); per tile lane j scores
// key j for the warp's 4 rows, the warp keeps a running max / sum per row and accumulates P V with lane <-> value columns.
// VC = ceil(vdim / 32) value columns per lane.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA, int VC>
__global__ void __launch_bounds__(256) attn_ragged_kernel(const TA* __restrict__ q, const TA* __restrict__ k_pages, const TA* __restrict__ v_pages,
                                                          const TA* __restrict__ gate, long long ldg, TA* __restrict__ out,
                                                          const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                          const int* __restrict__ entry_ctx, const int* __restrict__ page_table, int max_pages,
                                                          int page, int H, int G, int dim, int vdim, float scale, float softcap, int skip_single,
                                                          long long krow, long long vrow, int gate_per_head, int alias, PgAttnScore sx) {
  const int e = blockIdx.z, g = blockIdx.y, gsz = H / G;
  const int n = entry_n[e], ctx = entry_ctx[e], row0 = entry_row0[e];
  if (skip_single && n == 1) return;
  const int rows = n * gsz;
  const int r0 = blockIdx.x * 32;
  if (r0 >= rows) return;
  const int window = sx.window > 0 ? sx.window : 0x3fffffff, keep = sx.window > 0 ? max(sx.keep_first, 0) : 0;
  const int dimp = (dim + 3) & ~3, ks = dimp + 4;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                    // [32][dimp]
  float* Ks = Qs + 32 * dimp;        // [32][ks]
  float* Vs = alias ? Ks : Ks + 32 * ks;             // [32][vdim]; alias: the values are the first vdim columns of the key rows
  float* Ps = Ks + 32 * ks + (alias ? 0 : 32 * vdim);  // [8][4][32]
  const int vst = alias ? ks : vdim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // query rows: r -> token r / gsz, head g * gsz + r % gsz
  for (int i = threadIdx.x; i < 32 * dimp; i += 256) {
    const int r = i / dimp, d = i % dimp, rr = r0 + r;
    float v = 0.f;
    if (rr < rows && d < dim) v = ldf(q, (long long)(row0 + rr / gsz) * ((long long)H * dim) + (long long)(g * gsz + rr % gsz) * dim + d);
    Qs[i] = v;
  }
  float m[4], l[4], o[4][VC];
  int lim[4];  // last visible key of the row = the query's position (-1: row does not exist)
  float hsc[4], da[4], db[4];  // per-row head constants of the score
  int wlim = -1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) o[i][c] = 0.f;
    const int rr = r0 + warp * 4 + i;
    lim[i] = rr < rows ? ctx + rr / gsz : -1;
    wlim = max(wlim, lim[i]);
    const int head = g * gsz + (rr < rows ? rr % gsz : 0);
    hsc[i] = scale * (sx.head_scale != nullptr ? sx.head_scale[head] : 1.f);
    da[i] = sx.dist_a != nullptr ? sx.dist_a[head] : 0.f;
    db[i] = sx.dist_a != nullptr ? sx.dist_b[head] : 0.f;
  }
  const int last_row = min(rows, r0 + 32) - 1;
  const int kmax = ctx + last_row / gsz;  // last key any row of this CTA sees
  // first key inside the window of the CTA's / the warp's first row (later rows start later); tiles wholly between the kept first
  // keys and that key are skipped
  const int cta_lo = ctx + r0 / gsz - window + 1;
  const int warp_lo = ctx + min(r0 + warp * 4, rows - 1) / gsz - window + 1;
  const int* pt = page_table + (long long)e * max_pages;
  for (int k0 = 0; k0 <= kmax; k0 += 32) {
    if (k0 >= keep && k0 + 32 <= cta_lo) {
      k0 = (cta_lo / 32) * 32 - 32;  // uniform over the CTA
      continue;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * dimp; i += 256) {
      const int r = i / dimp, d = i % dimp, j = k0 + r;
      float v = 0.f;
      if (j <= kmax && d < dim) v = ldf(k_pages, ((long long)pt[j / page] * page + j % page) * krow + (long long)g * dim + d);
      Ks[r * ks + d] = v;
    }
    if (!alias)
      for (int i = threadIdx.x; i < 32 * vdim; i += 256) {
        const int r = i / vdim, d = i % vdim, j = k0 + r;
        float v = 0.f;
        if (j <= kmax) v = ldf(v_pages, ((long long)pt[j / page] * page + j % page) * vrow + (long long)g * vdim + d);
        Vs[i] = v;
      }
    __syncthreads();
    if (k0 > wlim || (k0 >= keep && k0 + 32 <= warp_lo)) continue;  // no row of this warp sees a key of the tile
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * ks;
    const float* qw = Qs + warp * 4 * dimp;
    for (int d = 0; d < dimp; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 qv = *reinterpret_cast<const float4*>(qw + i * dimp + d);
        s[i] = fmaf(qv.x, kv.x, s[i]); s[i] = fmaf(qv.y, kv.y, s[i]); s[i] = fmaf(qv.z, kv.z, s[i]); s[i] = fmaf(qv.w, kv.w, s[i]);
      }
    }
    float* pw = Ps + warp * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float sc = s[i] * hsc[i];
      if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      const int key = k0 + lane;
      const bool vis = key <= lim[i] && (lim[i] - key < window || key < keep);
      if (sx.dist_a != nullptr && vis) sc -= da[i] * log1pf(db[i] * (float)(lim[i] - key));
      sc = vis ? sc : -INFINITY;
      const float mn = fmaxf(m[i], wmax(sc));
      float pr = 0.f, corr = 1.f;
      if (mn > -INFINITY) {
        pr = vis ? expf(sc - mn) : 0.f;
        corr = expf(m[i] - mn);  // m = -inf on the first visible tile: exp(-inf) = 0
      }
      l[i] = l[i] * corr + wsum(pr);
      m[i] = mn;
#pragma unroll
      for (int c = 0; c < VC; ++c) o[i][c] *= corr;
      pw[i * 32 + lane] = pr;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      for (int j = 0; j < 32; j += 4) {
        const float4 p4 = *reinterpret_cast<const float4*>(pw + i * 32 + j);
        const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int c = 0; c < VC; ++c) {
            const int col = lane + 32 * c;
            if (col < vdim) o[i][c] = fmaf(pv[jj], Vs[(j + jj) * vst + col], o[i][c]);
          }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = r0 + warp * 4 + i;
    if (rr >= rows) continue;
    const long long t = row0 + rr / gsz;
    const int head = g * gsz + rr % gsz;
    float osc = 1.f;
    if (sx.sink != nullptr) {  // the sink joins the denominator once; the numerator has no term for it
      const float sk = sx.sink[head], mm = fmaxf(m[i], sk);
      osc = expf(m[i] - mm);
      l[i] = l[i] * osc + expf(sk - mm);
    }
    const float inv = osc / l[i];
#pragma unroll
    for (int c = 0; c < VC; ++c) {
      const int col = lane + 32 * c;
      if (col < vdim) {
        float v = o[i][c] * inv;
        if (gate != nullptr) v *= sigmoidf(ldf(gate, t * ldg + (gate_per_head ? (long long)head : (long long)head * vdim + col)));
        stf(out, t * ((long long)H * vdim) + (long long)head * vdim + col, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention of single new tokens (decode rows: entries with n == 1).  CTA = (key split, k/v head, entry), 8 warps; every
// warp walks its own 32-key tiles straight from the cache pages (lane <-> key for the scores, lane <-> value columns for
// P V), no block-wide barrier inside the loop.  The warps' (max, sum, accumulator) triples are merged through shared memory;
// with several key splits the CTA leaves its triple in `partial` and attn_decode_merge_kernel finishes the row.
// Up to 4 query heads of the group per pass (the keys are re-read for more).
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA>
__device__ __forceinline__ void ld8(const TA* p, float* v);
template <>
__device__ __forceinline__ void ld8<float>(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void ld8<bf16>(const bf16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// VC = ceil(vdim / 64).  VEC: 16-byte loads -- lane l reads key l's row for the scores; for P V the warp reads four keys per
// instruction (lane = key l / 8 of the four, value columns 8 (l % 8) .. + 8 of every 64) and the four key groups are summed
// by shuffles at the end.  All loads of a tile are independent, so a tile costs about one memory round trip.
template <typename TA, int VC, bool VEC>
__global__ void __launch_bounds__(256) attn_decode_kernel(const TA* __restrict__ q, const TA* __restrict__ k_pages, const TA* __restrict__ v_pages,
                                                          const TA* __restrict__ gate, long long ldg, TA* __restrict__ out, float* __restrict__ partial,
                                                          const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                          const int* __restrict__ entry_ctx, const int* __restrict__ page_table, int max_pages,
                                                          int page, int H, int G, int dim, int vdim, float scale, float softcap, long long krow,
                                                          long long vrow, int gate_per_head, PgAttnScore sx) {
  constexpr int NO = VEC ? 8 * VC : 2 * VC;  // accumulator columns per lane
  const int e = blockIdx.z, g = blockIdx.y, split = blockIdx.x, nsplit = gridDim.x, gsz = H / G;
  if (entry_n[e] != 1) return;
  const int ctx = entry_ctx[e];
  const long long t = entry_row0[e];
  const int dimp = (dim + 7) & ~7;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                       // [gsz][dimp]
  float* Pw = Qs + gsz * dimp;          // [8][4][32]
  float* Mg = Pw + 8 * 128;             // [8][4] max, [8][4] sum, then [8][4][vdim] accumulators
  float* Lg = Mg + 32;
  float* Og = Lg + 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kg = lane >> 3, l8 = lane & 7;
  for (int i = threadIdx.x; i < gsz * dimp; i += 256) {
    const int r = i / dimp, d = i % dimp;
    Qs[i] = d < dim ? ldf(q, t * ((long long)H * dim) + (long long)(g * gsz + r) * dim + d) : 0.f;
  }
  __syncthreads();
  const int* pt = page_table + (long long)e * max_pages;
  const int ntiles = ctx / 32 + 1;  // keys 0 .. ctx
  // with a window only the tiles of the kept first keys [0, nk) and of the window [t_lo, ntiles) are walked
  const int window = sx.window > 0 ? sx.window : 0x3fffffff, keep = sx.window > 0 ? max(sx.keep_first, 0) : 0;
  const int t_lo = max(0, ctx - window + 1) / 32;
  const int nkeep = min(min((keep + 31) / 32, ntiles), t_lo);
  const int nwalk = nkeep + ntiles - t_lo;
  for (int rb = 0; rb < gsz; rb += 4) {
    const int nr = min(4, gsz - rb);
    float m[4], l[4], o[4][NO];
    float hsc[4], da[4], db[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
      for (int c = 0; c < NO; ++c) o[i][c] = 0.f;
      const int head = g * gsz + min(rb + i, gsz - 1);
      hsc[i] = scale * (sx.head_scale != nullptr ? sx.head_scale[head] : 1.f);
      da[i] = sx.dist_a != nullptr ? sx.dist_a[head] : 0.f;
      db[i] = sx.dist_a != nullptr ? sx.dist_b[head] : 0.f;
    }
    for (int walk = split * 8 + warp; walk < nwalk; walk += nsplit * 8) {
      const int it = walk < nkeep ? walk : t_lo + (walk - nkeep);
      const int j = it * 32 + lane;
      const bool vis = j <= ctx && (ctx - j < window || j < keep);
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      if (vis) {
        const TA* kr = k_pages + ((long long)pt[j / page] * page + j % page) * krow + (long long)g * dim;
        if (VEC) {
#pragma unroll 4
          for (int d = 0; d < dim; d += 8) {
            float kv[8];
            ld8(kr + d, kv);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (i < nr) {
                const float4 qa = *reinterpret_cast<const float4*>(Qs + (rb + i) * dimp + d), qb = *reinterpret_cast<const float4*>(Qs + (rb + i) * dimp + d + 4);
                s[i] = fmaf(qa.x, kv[0], s[i]); s[i] = fmaf(qa.y, kv[1], s[i]); s[i] = fmaf(qa.z, kv[2], s[i]); s[i] = fmaf(qa.w, kv[3], s[i]);
                s[i] = fmaf(qb.x, kv[4], s[i]); s[i] = fmaf(qb.y, kv[5], s[i]); s[i] = fmaf(qb.z, kv[6], s[i]); s[i] = fmaf(qb.w, kv[7], s[i]);
              }
          }
        } else {
          for (int d = 0; d < dim; ++d) {
            const float kv = ldf(kr, d);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (i < nr) s[i] = fmaf(Qs[(rb + i) * dimp + d], kv, s[i]);
          }
        }
      }
      float* pw = Pw + warp * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float sc = s[i] * hsc[i];
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
        if (sx.dist_a != nullptr && vis) sc -= da[i] * log1pf(db[i] * (float)(ctx - j));
        sc = vis ? sc : -INFINITY;
        const float mn = fmaxf(m[i], wmax(sc));  // every walked tile holds a visible key: mn is finite
        const float pr = vis ? expf(sc - mn) : 0.f;
        const float corr = expf(m[i] - mn);
        l[i] = l[i] * corr + wsum(pr);
        m[i] = mn;
#pragma unroll
        for (int c = 0; c < NO; ++c) o[i][c] *= corr;
        pw[i * 32 + lane] = pr;
      }
      __syncwarp();
      if (VEC) {
        // a 32-key tile never straddles a page (the page size is a multiple of 32)
        const TA* vt = v_pages + ((long long)pt[(it * 32) / page] * page + (it * 32) % page) * vrow + (long long)g * vdim;
#pragma unroll
        for (int jj0 = 0; jj0 < 32; jj0 += 4) {
          const int jj = jj0 + kg;
          if (it * 32 + jj <= ctx) {
            float vv[8 * VC];
#pragma unroll
            for (int c = 0; c < VC; ++c) {
              const int col = 8 * l8 + 64 * c;
              if (col < vdim) ld8(vt + (long long)jj * vrow + col, vv + 8 * c);
              else {
#pragma unroll
                for (int x = 0; x < 8; ++x) vv[8 * c + x] = 0.f;
              }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float pj = pw[i * 32 + jj];
#pragma unroll
              for (int c = 0; c < 8 * VC; ++c) o[i][c] = fmaf(pj, vv[c], o[i][c]);
            }
          }
        }
      } else {
        const int nk = min(32, ctx + 1 - it * 32);
        for (int jj = 0; jj < nk; ++jj) {
          const int key = it * 32 + jj;
          const TA* vr = v_pages + ((long long)pt[key / page] * page + key % page) * vrow + (long long)g * vdim;
          float vv[2 * VC];
#pragma unroll
          for (int c = 0; c < VC; ++c) {
            const int col = 2 * lane + 64 * c;
            vv[2 * c] = col < vdim ? ldf(vr, col) : 0.f;
            vv[2 * c + 1] = col + 1 < vdim ? ldf(vr, col + 1) : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float pj = pw[i * 32 + jj];
#pragma unroll
            for (int c = 0; c < 2 * VC; ++c) o[i][c] = fmaf(pj, vv[c], o[i][c]);
          }
        }
      }
      __syncwarp();
    }
    if (VEC) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < NO; ++c) {
          o[i][c] += __shfl_xor_sync(0xffffffffu, o[i][c], 8);
          o[i][c] += __shfl_xor_sync(0xffffffffu, o[i][c], 16);
        }
    }
    // merge the 8 warps
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (lane == 0) { Mg[warp * 4 + i] = m[i]; Lg[warp * 4 + i] = l[i]; }
      if (VEC) {
        if (kg == 0) {
#pragma unroll
          for (int c = 0; c < NO; ++c) {
            const int col = 8 * l8 + 64 * (c / 8) + (c % 8);
            if (col < vdim) Og[(warp * 4 + i) * vdim + col] = o[i][c];
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < NO; ++c) {
          const int col = 2 * lane + 64 * (c / 2) + (c % 2);
          if (col < vdim) Og[(warp * 4 + i) * vdim + col] = o[i][c];
        }
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nr * vdim; idx += 256) {
      const int i = idx / vdim, col = idx % vdim;
      float M = -INFINITY;
      for (int w = 0; w < 8; ++w) M = fmaxf(M, Mg[w * 4 + i]);
      float acc = 0.f, ls = 0.f;
      if (M > -INFINITY)
        for (int w = 0; w < 8; ++w) {
          const float f = expf(Mg[w * 4 + i] - M);
          acc = fmaf(f, Og[(w * 4 + i) * vdim + col], acc);
          ls = fmaf(f, Lg[w * 4 + i], ls);
        }
      const int head = g * gsz + rb + i;
      if (nsplit == 1) {
        if (sx.sink != nullptr) {
          const float sk = sx.sink[head], mm = fmaxf(M, sk), f = expf(M - mm);
          acc *= f;
          ls = ls * f + expf(sk - mm);
        }
        float v = acc / ls;
        if (gate != nullptr) v *= sigmoidf(ldf(gate, t * ldg + (gate_per_head ? (long long)head : (long long)head * vdim + col)));
        stf(out, t * ((long long)H * vdim) + (long long)head * vdim + col, v);
      } else {
        float* pp = partial + (((long long)e * H + head) * nsplit + split) * (vdim + 2);
        pp[2 + col] = acc;
        if (col == 0) { pp[0] = M; pp[1] = ls; }
      }
    }
  }
}

// one value column per thread up to 256 columns: the loop over the splits is a chain of dependent loads per column
static inline int merge_threads(int vdim) { return vdim <= 64 ? 64 : vdim <= 128 ? 128 : 256; }

template <typename TA>
__global__ void attn_decode_merge_kernel(const float* __restrict__ partial, const TA* __restrict__ gate, long long ldg, TA* __restrict__ out,
                                         const int* __restrict__ entry_row0, const int* __restrict__ entry_n, int H, int vdim, int nsplit,
                                         int gate_per_head, const float* __restrict__ sink) {
  const int e = blockIdx.y, head = blockIdx.x;
  if (entry_n[e] != 1) return;
  const long long t = entry_row0[e];
  const float* pp = partial + ((long long)e * H + head) * nsplit * (vdim + 2);
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, pp[s * (vdim + 2)]);
  for (int col = threadIdx.x; col < vdim; col += blockDim.x) {
    float acc = 0.f, ls = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = pp[s * (vdim + 2)];
      if (ms > -INFINITY) {
        const float f = expf(ms - M);
        acc = fmaf(f, pp[s * (vdim + 2) + 2 + col], acc);
        ls = fmaf(f, pp[s * (vdim + 2) + 1], ls);
      }
    }
    if (sink != nullptr) {
      const float sk = sink[head], mm = fmaxf(M, sk), f = expf(M - mm);
      acc *= f;
      ls = ls * f + expf(sk - mm);
    }
    float v = acc / ls;
    if (gate != nullptr) v *= sigmoidf(ldf(gate, t * ldg + (gate_per_head ? (long long)head : (long long)head * vdim + col)));
    stf(out, t * ((long long)H * vdim) + (long long)head * vdim + col, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Decayed linear attention, token by token.  CTA = (value-column block of VB columns, head, entry); thread = one value
// column x one slice of DC key dimensions, its part of the state in registers.  q, k, v = silu(projection) are formed
// in fp32 from the activation-type projections; state, decay and output are fp32.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA, int DCMAX>
__global__ void __launch_bounds__(256) linear_attn_scan_kernel(const TA* __restrict__ qkv, long long ld, float* __restrict__ state,
                                                               const float* __restrict__ decay, float* __restrict__ out,
                                                               const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                               const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int H,
                                                               int dim, int vdim, int VB) {
  const int e = blockIdx.z, h = blockIdx.y, vb = blockIdx.x;
  const int n = entry_n[e], row0 = entry_row0[e];
  const int nchunk = 256 / VB, DC = (dim + nchunk - 1) / nchunk;
  const int vl = threadIdx.x % VB, chunk = threadIdx.x / VB;
  const int v = vb * VB + vl;
  const bool v_ok = v < vdim;
  extern __shared__ float sm[];
  float* qs = sm;              // [dim]
  float* ksm = qs + dim;       // [dim]
  float* red = ksm + dim;      // [nchunk][VB]
  float S[DCMAX];
  float* st = state + (((long long)entry_slot[e] * H + h) * dim) * vdim;
  const bool fresh = entry_ctx[e] == 0;
#pragma unroll
  for (int i = 0; i < DCMAX; ++i) {
    const int d = chunk * DC + i;
    S[i] = (!fresh && i < DC && d < dim && v_ok) ? st[(long long)d * vdim + v] : 0.f;
  }
  const float a = decay[h];
  const long long qo = (long long)h * dim, ko = (long long)H * dim + (long long)h * dim, vo = 2LL * H * dim + (long long)h * vdim;
  for (int t = 0; t < n; ++t) {
    const TA* row = qkv + (long long)(row0 + t) * ld;
    for (int d = threadIdx.x; d < dim; d += 256) {
      qs[d] = silu(ldf(row, qo + d));
      ksm[d] = silu(ldf(row, ko + d));
    }
    const float vv = v_ok ? silu(ldf(row, vo + v)) : 0.f;
    __syncthreads();
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < DCMAX; ++i) {
      const int d = chunk * DC + i;
      if (i < DC && d < dim) {
        S[i] = fmaf(a, S[i], ksm[d] * vv);
        part = fmaf(S[i], qs[d], part);
      }
    }
    red[chunk * VB + vl] = part;
    __syncthreads();
    if (chunk == 0 && v_ok) {
      float o = 0.f;
      for (int c = 0; c < nchunk; ++c) o += red[c * VB + vl];
      out[(long long)(row0 + t) * ((long long)H * vdim) + (long long)h * vdim + v] = o;
    }
  }
#pragma unroll
  for (int i = 0; i < DCMAX; ++i) {
    const int d = chunk * DC + i;
    if (i < DC && d < dim && v_ok) st[(long long)d * vdim + v] = S[i];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same recurrence advanced 32 tokens at a time.  With a = decay, block rows i, j = 0 .. c-1 and S the state before the block:
//   o_i = sum_{j <= i} a^(i-j) (q_i . k_j) v_j  +  a^(i+1) S^T q_i        S' = a^c S + sum_j a^(c-1-j) k_j v_j^T
// CTA = (value-column block, head, entry); the state block [dim][VB] lives in shared memory for the whole entry.
// Thread = value column x row group for the outputs, value column x key-dimension slice for the state update.
// ---------------------------------------------------------------------------------------------------------------------
// VEC: the block's q / k / v rows are fetched with 16-byte loads ONE BLOCK AHEAD into registers (<= 2 + 2 + 1 loads per thread:
// dim <= 128), so the memory round trip of block b + 1 hides behind the arithmetic of block b.
template <typename TA, bool VEC, int VB>
__global__ void __launch_bounds__(256, 2) linear_attn_chunked_kernel(const TA* __restrict__ qkv, long long ld, float* __restrict__ state,
                                                                  const float* __restrict__ decay, float* __restrict__ out,
                                                                  const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                                  const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int H,
                                                                  int dim, int vdim) {
  constexpr int C = 32;
  const int e = blockIdx.z, h = blockIdx.y, vb = blockIdx.x;
  const int n = entry_n[e], row0 = entry_row0[e];
  constexpr int ngrp = 256 / VB, rpt = C / ngrp;  // row groups; rows per thread (8 for 64 value columns per CTA)
  const int vl = threadIdx.x % VB, grp = threadIdx.x / VB;  // a warp lies inside one group: its row / key operands are broadcasts
  const int v = vb * VB + vl;
  const bool v_ok = v < vdim;
  const int dim4 = (dim + 3) & ~3, kd = dim4 + 4;  // padded key dimensions are zeros; rows stay 16-byte aligned
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                 // [C][kd]
  float* Ks = Qs + C * kd;        // [C][kd]
  float* Vs = Ks + C * kd;        // [C][VB]
  float* As = Vs + C * VB;        // [C][C]
  float* Ss = As + C * C;         // [dim4][VB]
  float* ap = Ss + dim4 * VB;     // a^0 .. a^C
  float* st = state + (((long long)entry_slot[e] * H + h) * dim) * vdim;
  const bool fresh = entry_ctx[e] == 0;
  for (int i = threadIdx.x; i < dim4 * VB; i += 256) {
    const int d = i / VB, c = vb * VB + i % VB;
    Ss[i] = (!fresh && d < dim && c < vdim) ? st[(long long)d * vdim + c] : 0.f;
  }
  const double a = (double)decay[h];
  for (int i = threadIdx.x; i <= C; i += 256) ap[i] = (float)pow(a, (double)i);
  const long long qo = (long long)h * dim, ko = (long long)H * dim + (long long)h * dim, vo = 2LL * H * dim + (long long)h * vdim;
  // bf16 projections carry 8 mantissa bits: their silu may use the hardware exponential and reciprocal
  auto act = [](float z) { return sizeof(TA) == 2 ? z * __frcp_rn(1.0f + __expf(-z)) : silu(z); };
  float pq[2][8], pk[2][8], pv[8];
  auto fetch = [&](int t0) {
    const int cn = min(C, n - t0), d8 = dim / 8, v8 = VB / 8;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int idx = threadIdx.x + 256 * k, r = idx / d8, c = (idx % d8) * 8;
      if (idx < C * d8 && r < cn) {
        const TA* row = qkv + (long long)(row0 + t0 + r) * ld;
        ld8(row + qo + c, pq[k]);
        ld8(row + ko + c, pk[k]);
      } else {
#pragma unroll
        for (int x = 0; x < 8; ++x) pq[k][x] = pk[k][x] = 0.f;
      }
    }
    const int r = threadIdx.x / v8, c = vb * VB + (threadIdx.x % v8) * 8;
    if (threadIdx.x < C * v8 && r < cn && c < vdim) ld8(qkv + (long long)(row0 + t0 + r) * ld + vo + c, pv);
    else {
#pragma unroll
      for (int x = 0; x < 8; ++x) pv[x] = 0.f;
    }
  };
  if (VEC) fetch(0);
  for (int t0 = 0; t0 < n; t0 += C) {
    const int cn = min(C, n - t0);
    __syncthreads();
    if (VEC) {
      const int d8 = dim / 8, v8 = VB / 8;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int idx = threadIdx.x + 256 * k, r = idx / d8, c = (idx % d8) * 8;
        if (idx < C * d8) {
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            Qs[r * kd + c + x] = act(pq[k][x]);
            Ks[r * kd + c + x] = act(pk[k][x]);
          }
        }
      }
      if (threadIdx.x < C * v8) {
        const int r = threadIdx.x / v8, c = (threadIdx.x % v8) * 8;
#pragma unroll
        for (int x = 0; x < 8; ++x) Vs[r * VB + c + x] = act(pv[x]);
      }
      if (t0 + C < n) fetch(t0 + C);
    } else {
      for (int i = threadIdx.x; i < C * dim4; i += 256) {
        const int r = i / dim4, d = i % dim4;
        float qv = 0.f, kv = 0.f;
        if (r < cn && d < dim) {
          const TA* row = qkv + (long long)(row0 + t0 + r) * ld;
          qv = silu(ldf(row, qo + d));
          kv = silu(ldf(row, ko + d));
        }
        Qs[r * kd + d] = qv;
        Ks[r * kd + d] = kv;
      }
      for (int i = threadIdx.x; i < C * VB; i += 256) {
        const int r = i / VB, c = vb * VB + i % VB;
        Vs[i] = (r < cn && c < vdim) ? silu(ldf(qkv + (long long)(row0 + t0 + r) * ld, vo + c)) : 0.f;
      }
    }
    __syncthreads();
    {  // A[i][j] = a^(i-j) q_i . k_j  (j <= i): a 2 x 2 block per thread, float4 along the key dimension
      const int i0 = 2 * (threadIdx.x / 16), j0 = 2 * (threadIdx.x % 16);
      float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;
      if (j0 <= i0 + 1) {
        const float4* qa = reinterpret_cast<const float4*>(Qs + i0 * kd);
        const float4* qb = reinterpret_cast<const float4*>(Qs + (i0 + 1) * kd);
        const float4* ka = reinterpret_cast<const float4*>(Ks + j0 * kd);
        const float4* kb = reinterpret_cast<const float4*>(Ks + (j0 + 1) * kd);
        for (int d = 0; d < dim4 / 4; ++d) {
          const float4 q0 = qa[d], q1 = qb[d], k0 = ka[d], k1 = kb[d];
          s00 = fmaf(q0.x, k0.x, fmaf(q0.y, k0.y, fmaf(q0.z, k0.z, fmaf(q0.w, k0.w, s00))));
          s01 = fmaf(q0.x, k1.x, fmaf(q0.y, k1.y, fmaf(q0.z, k1.z, fmaf(q0.w, k1.w, s01))));
          s10 = fmaf(q1.x, k0.x, fmaf(q1.y, k0.y, fmaf(q1.z, k0.z, fmaf(q1.w, k0.w, s10))));
          s11 = fmaf(q1.x, k1.x, fmaf(q1.y, k1.y, fmaf(q1.z, k1.z, fmaf(q1.w, k1.w, s11))));
        }
      }
      As[i0 * C + j0] = j0 <= i0 ? s00 * ap[i0 - j0] : 0.f;
      As[i0 * C + j0 + 1] = j0 + 1 <= i0 ? s01 * ap[i0 - j0 - 1] : 0.f;
      As[(i0 + 1) * C + j0] = j0 <= i0 + 1 ? s10 * ap[i0 + 1 - j0] : 0.f;
      As[(i0 + 1) * C + j0 + 1] = j0 + 1 <= i0 + 1 ? s11 * ap[i0 - j0] : 0.f;
    }
    __syncthreads();
    // outputs of the thread's rows i = grp * rpt + r: a^(i+1) q_i . S[:, v]  +  sum_j A[i][j] v_j
    float acc[rpt];
#pragma unroll
    for (int r = 0; r < rpt; ++r) acc[r] = 0.f;
    for (int d = 0; d < dim4; d += 4) {
      const float s0 = Ss[d * VB + vl], s1 = Ss[(d + 1) * VB + vl], s2 = Ss[(d + 2) * VB + vl], s3 = Ss[(d + 3) * VB + vl];
#pragma unroll
      for (int r = 0; r < rpt; ++r) {
          const float4 q4 = *reinterpret_cast<const float4*>(Qs + (grp * rpt + r) * kd + d);
          acc[r] = fmaf(q4.x, s0, fmaf(q4.y, s1, fmaf(q4.z, s2, fmaf(q4.w, s3, acc[r]))));
        }
    }
#pragma unroll
    for (int r = 0; r < rpt; ++r) acc[r] *= ap[grp * rpt + r + 1];
    for (int j = 0; j < C; j += 4) {
      const float v0 = Vs[j * VB + vl], v1 = Vs[(j + 1) * VB + vl], v2 = Vs[(j + 2) * VB + vl], v3 = Vs[(j + 3) * VB + vl];
#pragma unroll
      for (int r = 0; r < rpt; ++r) {
          const float4 a4 = *reinterpret_cast<const float4*>(As + (grp * rpt + r) * C + j);
          acc[r] = fmaf(a4.x, v0, fmaf(a4.y, v1, fmaf(a4.z, v2, fmaf(a4.w, v3, acc[r]))));
        }
    }
#pragma unroll
    for (int r = 0; r < rpt; ++r) {
      const int i = grp * rpt + r;
      if (i < cn && v_ok) out[(long long)(row0 + t0 + i) * ((long long)H * vdim) + (long long)h * vdim + v] = acc[r];
    }
    __syncthreads();  // every read of the old state is done
    // state: thread = value column x key dimensions 4 (grp + ngrp k) .. + 4
    float vw[C];
#pragma unroll
    for (int j = 0; j < C; ++j) vw[j] = j < cn ? Vs[j * VB + vl] * ap[cn - 1 - j] : 0.f;
    const float ac = ap[cn];
    for (int d = 4 * grp; d < dim4; d += 4 * ngrp) {
      float s0 = ac * Ss[d * VB + vl], s1 = ac * Ss[(d + 1) * VB + vl], s2 = ac * Ss[(d + 2) * VB + vl], s3 = ac * Ss[(d + 3) * VB + vl];
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(Ks + j * kd + d);
        s0 = fmaf(k4.x, vw[j], s0); s1 = fmaf(k4.y, vw[j], s1); s2 = fmaf(k4.z, vw[j], s2); s3 = fmaf(k4.w, vw[j], s3);
      }
      Ss[d * VB + vl] = s0; Ss[(d + 1) * VB + vl] = s1; Ss[(d + 2) * VB + vl] = s2; Ss[(d + 3) * VB + vl] = s3;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim * VB; i += 256) {
    const int d = i / VB, c = vb * VB + i % VB;
    if (c < vdim) st[(long long)d * vdim + c] = Ss[i];
  }
}

}  // namespace

extern "C" int pg_attn_prepare(const void* qkv, long long ld, const int* pos, const int* row_entry, const int* page_table, int max_pages,
                               int page, const double* freq, const float* q_norm, const float* k_norm, void* q_out, void* k_pages,
                               void* v_pages, int rows, int H, int G, int dim, int vdim, int rot_dims, float eps, int norm_qk, int norm_v,
                               int v_from_k, int act_f32, void* stream) {
  if (rows <= 0 || H <= 0 || G <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || page <= 0) return PG_ERR_ARG;
  if (v_from_k && vdim != dim) return PG_ERR_ARG;
  if ((k_pages == nullptr) != (v_pages == nullptr)) return PG_ERR_ARG;
  const size_t smem = (size_t)(rot_dims + 2) * sizeof(float);
  if (act_f32)
    attn_prepare_kernel<float><<<rows, 128, smem, PG_ST(stream)>>>(static_cast<const float*>(qkv), ld, pos, row_entry, page_table, max_pages, page, freq,
                                                                  q_norm, k_norm, static_cast<float*>(q_out), static_cast<float*>(k_pages),
                                                                  static_cast<float*>(v_pages), H, G, dim, vdim, rot_dims, eps, norm_qk, norm_v, v_from_k);
  else
    attn_prepare_kernel<bf16><<<rows, 128, smem, PG_ST(stream)>>>(static_cast<const bf16*>(qkv), ld, pos, row_entry, page_table, max_pages, page, freq,
                                                                 q_norm, k_norm, static_cast<bf16*>(q_out), static_cast<bf16*>(k_pages),
                                                                 static_cast<bf16*>(v_pages), H, G, dim, vdim, rot_dims, eps, norm_qk, norm_v, v_from_k);
  PG_RET();
}

template <typename TA, int VC>
static int launch_attn_ragged(const void* q, const void* kp, const void* vp, const void* gate, long long ldg, void* out, const int* row0,
                              const int* n, const int* ctx, const int* pt, int max_pages, int page, int entries, int max_n, int H, int G,
                              int dim, int vdim, float scale, float softcap, int skip_single, long long krow, long long vrow, int gate_per_head,
                              const PgAttnScore& sx, cudaStream_t st) {
  const int dimp = (dim + 3) & ~3;
  // one latent row serves as key and value (one k/v head, values = leading key columns): the tile is staged once
  const int alias = (kp == vp && G == 1 && krow == vrow && vdim <= dim) ? 1 : 0;
  const size_t smem = ((size_t)32 * dimp + 32 * (dimp + 4) + (alias ? 0 : 32 * vdim) + 8 * 128) * sizeof(float);
  if (smem > 220 * 1024) return PG_ERR_ARG;
  auto kern = attn_ragged_kernel<TA, VC>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  dim3 grid((max_n * (H / G) + 31) / 32, G, entries);
  kern<<<grid, 256, smem, st>>>(static_cast<const TA*>(q), static_cast<const TA*>(kp), static_cast<const TA*>(vp), static_cast<const TA*>(gate), ldg,
                                static_cast<TA*>(out), row0, n, ctx, pt, max_pages, page, H, G, dim, vdim, scale, softcap, skip_single, krow, vrow,
                                gate_per_head, alias, sx);
  PG_RET();
}

extern "C" int pg_attn_ragged(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out,
                              const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                              int entries, int max_n, int H, int G, int dim, int vdim, float scale, float softcap, int skip_single, int act_f32,
                              long long krow, long long vrow, int gate_per_head, const PgAttnScore* score, void* stream) {
  if (entries <= 0 || max_n <= 0 || H <= 0 || G <= 0 || (H % G) != 0 || dim <= 0 || vdim <= 0 || vdim > 512 || entries > 65535 || G > 65535)
    return PG_ERR_ARG;
  if (score != nullptr && ((score->dist_a == nullptr) != (score->dist_b == nullptr))) return PG_ERR_ARG;
  const PgAttnScore sx = score != nullptr ? *score : PgAttnScore{};
  if (krow <= 0) krow = (long long)G * dim;
  if (vrow <= 0) vrow = (long long)G * vdim;
  cudaStream_t st = PG_ST(stream);
#define PG_ATTN(TA, VC) \
  return launch_attn_ragged<TA, VC>(q, k_pages, v_pages, gate, ldg, out, entry_row0, entry_n, entry_ctx, page_table, max_pages, page, entries, max_n, \
                                    H, G, dim, vdim, scale, softcap, skip_single, krow, vrow, gate_per_head, sx, st)
  if (act_f32) {
    if (vdim <= 64) PG_ATTN(float, 2);
    if (vdim <= 128) PG_ATTN(float, 4);
    if (vdim <= 256) PG_ATTN(float, 8);
    PG_ATTN(float, 16);
  }
  if (vdim <= 64) PG_ATTN(bf16, 2);
  if (vdim <= 128) PG_ATTN(bf16, 4);
  if (vdim <= 256) PG_ATTN(bf16, 8);
  PG_ATTN(bf16, 16);
#undef PG_ATTN
}

template <typename TA, int DCMAX>
static int launch_scan(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* row0, const int* n, const int* ctx,
                       const int* slot, int entries, int H, int dim, int vdim, int VB, cudaStream_t st) {
  const int nchunk = 256 / VB;
  const size_t smem = ((size_t)2 * dim + (size_t)nchunk * VB) * sizeof(float);
  dim3 grid((vdim + VB - 1) / VB, H, entries);
  linear_attn_scan_kernel<TA, DCMAX><<<grid, 256, smem, st>>>(static_cast<const TA*>(qkv), ld, state, decay, out, row0, n, ctx, slot, H, dim, vdim, VB);
  PG_RET();
}

extern "C" int pg_linear_attn_scan(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* entry_row0,
                                   const int* entry_n, const int* entry_ctx, const int* entry_slot, int entries, int H, int dim, int vdim,
                                   int act_f32, void* stream) {
  if (entries <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || dim > 1024 || entries > 65535 || H > 65535) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  // VB value columns per CTA (a power of two <= 64); the 256 / VB thread groups split the key dimensions
  int VB = 64;
  while (VB > 8 && VB / 2 >= vdim) VB /= 2;
  const int DC = (dim + 256 / VB - 1) / (256 / VB);
#define PG_SCAN(TA, DCM) return launch_scan<TA, DCM>(qkv, ld, state, decay, out, entry_row0, entry_n, entry_ctx, entry_slot, entries, H, dim, vdim, VB, st)
  if (act_f32) {
    if (DC <= 16) PG_SCAN(float, 16);
    if (DC <= 64) PG_SCAN(float, 64);
    PG_SCAN(float, 256);
  }
  if (DC <= 16) PG_SCAN(bf16, 16);
  if (DC <= 64) PG_SCAN(bf16, 64);
  PG_SCAN(bf16, 256);
#undef PG_SCAN
}

template <typename TA, bool VEC, int VB>
static int launch_chunked(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* row0, const int* n, const int* ctx,
                          const int* slot, int entries, int H, int dim, int vdim, size_t smem, cudaStream_t st) {
  auto kern = linear_attn_chunked_kernel<TA, VEC, VB>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  kern<<<dim3((vdim + VB - 1) / VB, H, entries), 256, smem, st>>>(static_cast<const TA*>(qkv), ld, state, decay, out, row0, n, ctx, slot, H, dim, vdim);
  PG_RET();
}

extern "C" int pg_linear_attn_chunked(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* entry_row0,
                                      const int* entry_n, const int* entry_ctx, const int* entry_slot, int entries, int H, int dim, int vdim,
                                      int act_f32, void* stream) {
  if (entries <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || entries > 65535 || H > 65535) return PG_ERR_ARG;
  int VB = 64;
  while (VB > 8 && VB / 2 >= vdim) VB /= 2;
  // narrower value blocks (the scores are recomputed per block) only while the grid does not even fill the SMs once
  while (VB > 16 && (long long)((vdim + VB - 1) / VB) * H * entries < (long long)pg::num_sms()) VB /= 2;
  const int dim4 = (dim + 3) & ~3;
  auto bytes = [&](int vb) { return ((size_t)2 * 32 * (dim4 + 4) + 32 * vb + 32 * 32 + (size_t)dim4 * vb + 36) * sizeof(float); };
  while (VB > 8 && bytes(VB) > 200 * 1024) VB /= 2;
  const size_t smem = bytes(VB);
  if (smem > 200 * 1024) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  // 16-byte fetches: every head's q / k / v slice of a row starts on an 8-element boundary
  const bool vec = dim % 8 == 0 && vdim % 8 == 0 && dim <= 128 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0;
#define PG_CHUNK(TA, VEC, VBV) \
  return launch_chunked<TA, VEC, VBV>(qkv, ld, state, decay, out, entry_row0, entry_n, entry_ctx, entry_slot, entries, H, dim, vdim, smem, st)
#define PG_CHUNK_VB(TA, VEC)          \
  do {                                \
    if (VB == 64) PG_CHUNK(TA, VEC, 64); \
    if (VB == 32) PG_CHUNK(TA, VEC, 32); \
    if (VB == 16) PG_CHUNK(TA, VEC, 16); \
    PG_CHUNK(TA, VEC, 8);             \
  } while (0)
  if (act_f32) {
    if (vec) PG_CHUNK_VB(float, true);
    PG_CHUNK_VB(float, false);
  }
  if (vec) PG_CHUNK_VB(bf16, true);
  PG_CHUNK_VB(bf16, false);
#undef PG_CHUNK_VB
#undef PG_CHUNK
}

template <typename TA, int VC, bool VEC>
static int launch_attn_decode(const void* q, const void* kp, const void* vp, const void* gate, long long ldg, void* out, float* partial,
                              const int* row0, const int* n, const int* ctx, const int* pt, int max_pages, int page, int entries, int nsplit, int H,
                              int G, int dim, int vdim, float scale, float softcap, long long krow, long long vrow, int gate_per_head,
                              const PgAttnScore& sx, cudaStream_t st) {
  const int gsz = H / G, dimp = (dim + 7) & ~7;
  const size_t smem = ((size_t)gsz * dimp + 8 * 128 + 64 + (size_t)32 * vdim) * sizeof(float);
  if (smem > 200 * 1024) return PG_ERR_ARG;
  auto kern = attn_decode_kernel<TA, VC, VEC>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  kern<<<dim3(nsplit, G, entries), 256, smem, st>>>(static_cast<const TA*>(q), static_cast<const TA*>(kp), static_cast<const TA*>(vp),
                                                     static_cast<const TA*>(gate), ldg, static_cast<TA*>(out), partial, row0, n, ctx, pt, max_pages, page,
                                                     H, G, dim, vdim, scale, softcap, krow, vrow, gate_per_head, sx);
  pg_count_launch(1);
  if (nsplit > 1) {
    attn_decode_merge_kernel<TA><<<dim3(H, entries), merge_threads(vdim), 0, st>>>(partial, static_cast<const TA*>(gate), ldg, static_cast<TA*>(out), row0, n, H, vdim, nsplit,
                                                                  gate_per_head, sx.sink);
    pg_count_launch(1);
  }
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

extern "C" int pg_attn_decode_merge(const float* partial, const void* gate, long long ldg, void* out, const int* entry_row0, const int* entry_n,
                                    int entries, int nsplit, int H, int vdim, int gate_per_head, int act_f32, const PgAttnScore* score, void* stream) {
  if (entries <= 0 || entries > 65535 || nsplit <= 0 || H <= 0 || vdim <= 0 || partial == nullptr) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  const float* sink = score != nullptr ? score->sink : nullptr;
  if (act_f32)
    attn_decode_merge_kernel<float><<<dim3(H, entries), merge_threads(vdim), 0, st>>>(partial, static_cast<const float*>(gate), ldg, static_cast<float*>(out), entry_row0, entry_n,
                                                                     H, vdim, nsplit, gate_per_head, sink);
  else
    attn_decode_merge_kernel<bf16><<<dim3(H, entries), merge_threads(vdim), 0, st>>>(partial, static_cast<const bf16*>(gate), ldg, static_cast<bf16*>(out), entry_row0, entry_n, H,
                                                                    vdim, nsplit, gate_per_head, sink);
  PG_RET();
}

extern "C" int pg_attn_decode(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out, float* partial,
                              const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                              int entries, int nsplit, int H, int G, int dim, int vdim, float scale, float softcap, int act_f32, long long krow,
                              long long vrow, int gate_per_head, const PgAttnScore* score, void* stream) {
  if (entries <= 0 || nsplit <= 0 || nsplit > 64 || H <= 0 || G <= 0 || (H % G) != 0 || dim <= 0 || vdim <= 0 || vdim > 512 || entries > 65535 ||
      G > 65535 || (nsplit > 1 && partial == nullptr))
    return PG_ERR_ARG;
  if (score != nullptr && ((score->dist_a == nullptr) != (score->dist_b == nullptr))) return PG_ERR_ARG;
  const PgAttnScore sx = score != nullptr ? *score : PgAttnScore{};
  if (krow <= 0) krow = (long long)G * dim;
  if (vrow <= 0) vrow = (long long)G * vdim;
  cudaStream_t st = PG_ST(stream);
  // 16-byte loads need every head's key / value row to start on an 8-element boundary and tiles that stay inside a page
  const bool vec = (dim % 8 == 0) && (vdim % 8 == 0) && (krow % 8 == 0) && (vrow % 8 == 0) && (page % 32 == 0) && vdim <= 128 &&
                   ((reinterpret_cast<uintptr_t>(k_pages) & 15) == 0) && ((reinterpret_cast<uintptr_t>(v_pages) & 15) == 0);
#define PG_ATTD(TA, VC, VEC) \
  return launch_attn_decode<TA, VC, VEC>(q, k_pages, v_pages, gate, ldg, out, partial, entry_row0, entry_n, entry_ctx, page_table, max_pages, page, \
                                         entries, nsplit, H, G, dim, vdim, scale, softcap, krow, vrow, gate_per_head, sx, st)
  if (act_f32) {
    if (vec && vdim <= 64) PG_ATTD(float, 1, true);
    if (vec) PG_ATTD(float, 2, true);
    if (vdim <= 64) PG_ATTD(float, 1, false);
    if (vdim <= 128) PG_ATTD(float, 2, false);
    if (vdim <= 256) PG_ATTD(float, 4, false);
    PG_ATTD(float, 8, false);
  }
  if (vec && vdim <= 64) PG_ATTD(bf16, 1, true);
  if (vec) PG_ATTD(bf16, 2, true);
  if (vdim <= 64) PG_ATTD(bf16, 1, false);
  if (vdim <= 128) PG_ATTD(bf16, 2, false);
  if (vdim <= 256) PG_ATTD(bf16, 4, false);
  PG_ATTD(bf16, 8, false);
#undef PG_ATTD
}
